"""Python face of the native block manager + iteration-level scheduler."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import _native
from ..api.errors import SessionError
from .request import RequestState

PLAN_NONE, PLAN_PREFILL, PLAN_DECODE = 0, 1, 2


@dataclass
class StepBatch:
    kind: int
    n_items: int
    n_tokens: int
    req_ids: np.ndarray


class HostBatchBuffers:
    """Pinned host staging for one step.  One int32 region so a single copy carries it to the device:
    [token_ids | positions | slot_mapping | token_item | ctx_per_token | q_start | seq_lens | sample_index | block_tables]."""

    def __init__(self, max_tokens: int, max_items: int, max_blocks: int, pin: bool):
        self.max_tokens, self.max_items, self.max_blocks = max_tokens, max_items, max_blocks
        sizes = [("token_ids", max_tokens), ("positions", max_tokens), ("slot_mapping", max_tokens),
                 ("token_item", max_tokens), ("ctx_per_token", max_tokens), ("q_start", max_items + 1),
                 ("seq_lens", max_items), ("sample_index", max_items), ("block_tables", max_items * max_blocks)]
        self.offsets = {}
        off = 0
        for name, n in sizes:
            off = (off + 3) // 4 * 4            # 16-byte aligned fields
            self.offsets[name] = (off, n)
            off += n
        self.total = off
        self.host = torch.zeros(self.total, dtype=torch.int32)
        if pin and torch.cuda.is_available():
            self.host = self.host.pin_memory()
        self.req_ids = np.zeros(max_items, dtype=np.int64)
        self.np = self.host.numpy()

    def field(self, name: str) -> np.ndarray:
        off, n = self.offsets[name]
        return self.np[off:off + n]

    def field_ptr(self, name: str) -> int:
        off, _ = self.offsets[name]
        return self.host.data_ptr() + off * 4


class Scheduler:
    def __init__(self, block_size: int, num_blocks: int, max_num_seqs: int, max_batch_tokens: int,
                 prefill_chunk: int = 0, policy: str = "fcfs", enable_prefix_cache: bool = False,
                 max_blocks_per_seq: int = 64):
        self._lib = _native.host()
        self._h = self._lib.ronn_sched_new(block_size, num_blocks, max_num_seqs, max_batch_tokens, prefill_chunk,
                                           1 if policy == "priority" else 0, 1 if enable_prefix_cache else 0,
                                           max_blocks_per_seq)
        if not self._h:
            raise SessionError("invalid scheduler configuration")
        self.block_size, self.num_blocks = block_size, num_blocks
        self.max_blocks_per_seq = max_blocks_per_seq

    def __del__(self):
        try:
            if self._h:
                self._lib.ronn_sched_free(self._h)
                self._h = None
        except Exception:
            pass

    _PREEMPT_MODES = {"recompute": 0, "swap": 1, "auto": 2}

    def set_preemption(self, mode: str, num_cpu_blocks: int, auto_min_tokens: int = 64) -> None:
        """How a preempted sequence keeps its KV cache: ``recompute`` (drop it), ``swap`` (copy its blocks to a host
        pool of ``num_cpu_blocks`` blocks and back on resume) or ``auto`` (swap sequences with at least
        ``auto_min_tokens`` cached tokens).  Before any request is added."""
        if mode not in self._PREEMPT_MODES:
            raise SessionError(f"unknown preemption mode '{mode}'")
        if self._lib.ronn_sched_set_swap(self._h, self._PREEMPT_MODES[mode], int(num_cpu_blocks), int(auto_min_tokens)):
            raise SessionError("preemption mode must be set on an empty scheduler with a non-negative host pool")

    def swaps(self):
        """Block copies to run before this step's forward pass: (out_src, out_dst, in_src, in_dst) int32 arrays;
        device block -> host block first, then host block -> device block."""
        cnt = np.zeros(2, dtype=np.int32)
        self._lib.ronn_sched_swap_counts(self._h, cnt.ctypes.data_as(_native.c_i32p))
        arrs = [np.zeros(max(int(cnt[0]), 1), dtype=np.int32), np.zeros(max(int(cnt[0]), 1), dtype=np.int32),
                np.zeros(max(int(cnt[1]), 1), dtype=np.int32), np.zeros(max(int(cnt[1]), 1), dtype=np.int32)]
        if cnt[0] or cnt[1]:
            self._lib.ronn_sched_get_swaps(self._h, *[a.ctypes.data_as(_native.c_i32p) for a in arrs])
        return arrs[0][:cnt[0]], arrs[1][:cnt[0]], arrs[2][:cnt[1]], arrs[3][:cnt[1]]

    def swap_stats(self) -> dict:
        out = np.zeros(4, dtype=np.int64)
        self._lib.ronn_sched_swap_stats(self._h, out.ctypes.data_as(_native.c_i64p))
        return {"swap_preemptions": int(out[0]), "swapped_out_blocks": int(out[1]), "swapped_in_blocks": int(out[2]),
                "free_cpu_blocks": int(out[3])}

    def add(self, req_id: int, prompt: List[int], max_new_tokens: int, priority: int = 2) -> None:
        arr = np.ascontiguousarray(prompt, dtype=np.int32)
        rc = self._lib.ronn_sched_add(self._h, req_id, arr.ctypes.data_as(_native.c_i32p), len(arr), max_new_tokens,
                                      int(priority))
        if rc == -1:
            raise SessionError(f"request id {req_id} already exists")
        if rc == -2:
            raise SessionError(f"request {req_id} (prompt {len(arr)} + {max_new_tokens} new tokens) can never fit "
                               f"the KV cache or the batch budget")

    def cancel(self, req_id: int) -> bool:
        return self._lib.ronn_sched_cancel(self._h, req_id) == 0

    def schedule(self) -> int:
        return self._lib.ronn_sched_schedule(self._h)

    def plan_size(self) -> int:
        return self._lib.ronn_sched_plan_size(self._h)

    def plan_tokens(self) -> int:
        return self._lib.ronn_sched_plan_tokens(self._h)

    def fill(self, buf: HostBatchBuffers, kind: int) -> StepBatch:
        n_items = self.plan_size()
        n_tok = self._lib.ronn_sched_fill(
            self._h, buf.req_ids.ctypes.data, buf.field_ptr("q_start"), buf.field_ptr("seq_lens"),
            buf.field_ptr("sample_index"), buf.field_ptr("token_ids"), buf.field_ptr("positions"),
            buf.field_ptr("slot_mapping"), buf.field_ptr("token_item"), buf.field_ptr("block_tables"), buf.max_blocks)
        if n_tok < 0:
            raise SessionError("block table stride too small for a scheduled sequence")
        return StepBatch(kind, n_items, n_tok, buf.req_ids[:n_items])

    def commit(self, sampled: np.ndarray, eos_token: int = -1) -> np.ndarray:
        n = self.plan_size()
        fin = np.zeros(max(n, 1), dtype=np.int32)
        s = np.ascontiguousarray(sampled, dtype=np.int32)
        self._lib.ronn_sched_commit(self._h, s.ctypes.data, eos_token, fin.ctypes.data)
        return fin[:n]

    def abort_step(self) -> None:
        self._lib.ronn_sched_abort_step(self._h)

    def state(self, req_id: int) -> Optional[RequestState]:
        s = self._lib.ronn_sched_state(self._h, req_id)
        return None if s < 0 else RequestState(s)

    def num_tokens(self, req_id: int) -> int:
        """Prompt plus generated tokens of a live request (-1 when unknown)."""
        return self._lib.ronn_sched_num_tokens(self._h, req_id)

    def tokens(self, req_id: int) -> List[int]:
        n = self._lib.ronn_sched_num_tokens(self._h, req_id)
        if n < 0:
            raise SessionError(f"unknown request {req_id}")
        out = np.empty(max(n, 1), dtype=np.int32)
        self._lib.ronn_sched_get_tokens(self._h, req_id, out.ctypes.data_as(_native.c_i32p), n)
        return out[:n].tolist()

    def prompt_len(self, req_id: int) -> int:
        return self._lib.ronn_sched_prompt_len(self._h, req_id)

    def blocks(self, req_id: int) -> List[int]:
        out = np.empty(self.max_blocks_per_seq, dtype=np.int32)
        n = self._lib.ronn_sched_get_blocks(self._h, req_id, out.ctypes.data_as(_native.c_i32p), len(out))
        return out[:max(n, 0)].tolist()

    def cpu_blocks(self, req_id: int) -> List[int]:
        """Host-pool blocks that hold the request's cache while it is swapped out."""
        out = np.empty(self.max_blocks_per_seq, dtype=np.int32)
        n = self._lib.ronn_sched_get_cpu_blocks(self._h, req_id, out.ctypes.data_as(_native.c_i32p), len(out))
        return out[:max(n, 0)].tolist()

    def num_computed(self, req_id: int) -> int:
        return self._lib.ronn_sched_num_computed(self._h, req_id)

    def preemptions(self, req_id: int) -> int:
        return self._lib.ronn_sched_preemptions(self._h, req_id)

    def forget(self, req_id: int) -> None:
        self._lib.ronn_sched_forget(self._h, req_id)

    @property
    def num_waiting(self) -> int:
        return self._lib.ronn_sched_num_waiting(self._h)

    @property
    def num_running(self) -> int:
        return self._lib.ronn_sched_num_running(self._h)

    @property
    def num_free_blocks(self) -> int:
        return self._lib.ronn_sched_num_free_blocks(self._h)

    def block_ref(self, block: int) -> int:
        return self._lib.ronn_sched_block_ref(self._h, block)

    def stats(self) -> Dict[str, int]:
        out = (C.c_int64 * 8)()
        self._lib.ronn_sched_stats(self._h, out)
        keys = ["steps", "prefill_steps", "decode_steps", "preemptions", "prefix_hit_blocks", "finished",
                "cancelled", "scheduled_tokens"]
        return dict(zip(keys, [int(x) for x in out]))
