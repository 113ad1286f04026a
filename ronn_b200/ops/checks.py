"""Index checks at the kernel boundary, switched on with ``RONN_KERNEL_CHECKS=1``.

The kernels that take indices from data (cache block tables, cache slots, sequence offsets, token ids) trust them:
a block table entry past the cache is an out-of-bounds read on the device.  ``compute-sanitizer`` is not available
where this runs, so the debug mode checks those indices on the host before the launch (one device-to-host copy per
call, which also serialises the stream: a debugging aid, not a production setting) and raises ``KernelError`` naming
the first offending value; nothing is launched for a call that fails its check.  The reference validates shapes in its
operator wrappers and has no device-side checks (crates/ronn-core/src/ops/*.rs).

Every function works on tensors of any device, which is how the CPU suite tests them.
"""
from __future__ import annotations

import os
from typing import Optional

import torch


class IndexCheckError(ValueError):
    pass


def enabled() -> bool:
    """On when the switch is set, except while the current stream is being captured into a CUDA graph: the checks
    read device tensors on the host, which a capture does not allow (check the eager warm-up run instead)."""
    if os.environ.get("RONN_KERNEL_CHECKS", "0") != "1":
        return False
    try:
        return not (torch.cuda.is_available() and torch.cuda.is_current_stream_capturing())
    except Exception:
        return True


def _first_bad(t: torch.Tensor, bad: torch.Tensor):
    idx = torch.nonzero(bad.reshape(-1), as_tuple=False)
    i = int(idx[0]) if idx.numel() else -1
    return i, (int(t.reshape(-1)[i]) if i >= 0 else None)


def _in_range(name: str, t: Optional[torch.Tensor], lo: int, hi: int, what: str, mask: Optional[torch.Tensor] = None):
    """Every (selected) value of t in [lo, hi)."""
    if t is None or t.numel() == 0:
        return
    v = t.long()
    bad = (v < lo) | (v >= hi)
    if mask is not None:
        bad = bad & mask
    if bool(bad.any()):
        i, val = _first_bad(t, bad)
        raise IndexCheckError(f"{name}[{i}] = {val} is outside [{lo}, {hi}) ({what})")


def paged_attention(q, kcache, block_tables, ctx_len, heads: int, head_dim: int, max_ctx: int,
                    bt_row=None, append_slots=None, positions=None) -> None:
    rows = q.shape[0]
    n_blocks, block = kcache.shape[0], kcache.shape[2]
    if q.shape[1] < heads * head_dim:
        raise IndexCheckError(f"q has {q.shape[1]} columns, {heads} heads of {head_dim} need {heads * head_dim}")
    if ctx_len.numel() < rows:
        raise IndexCheckError(f"ctx_len has {ctx_len.numel()} entries for {rows} rows")
    cap = min(int(max_ctx), block_tables.shape[1] * block)
    _in_range("ctx_len", ctx_len[:rows], 0, cap + 1, "keys a row may attend to: max_ctx and the width of its table row")
    _in_range("bt_row", None if bt_row is None else bt_row[:rows], 0, block_tables.shape[0], "rows of block_tables")
    tables = block_tables if bt_row is None else block_tables.index_select(0, bt_row[:rows].long().clamp(0, block_tables.shape[0] - 1))
    tables = tables[:rows]
    used = torch.arange(block_tables.shape[1], device=tables.device)[None, :] * block < ctx_len[:rows].long()[:, None]
    _in_range("block_tables", tables, 0, n_blocks, "cache blocks", used)
    if append_slots is not None:
        _in_range("append_slots", append_slots[:rows], -1, n_blocks * block, "cache slots (-1: no append)")
    if positions is not None:
        _in_range("positions", positions[:rows], 0, 1 << 30, "token positions")


def kv_append(qkv, slots, kcache, positions=None) -> None:
    tokens = qkv.shape[0]
    if slots.numel() < tokens:
        raise IndexCheckError(f"slots has {slots.numel()} entries for {tokens} tokens")
    _in_range("slots", slots[:tokens], -1, kcache.shape[0] * kcache.shape[2], "cache slots (-1: skip)")
    if positions is not None:
        _in_range("positions", positions[:tokens], 0, 1 << 30, "token positions")


def embedding(ids, table, positions=None, pos_table=None) -> None:
    _in_range("ids", ids, 0, table.shape[0], "rows of the embedding table")
    if positions is not None and pos_table is not None:
        _in_range("positions", positions, 0, pos_table.shape[0], "rows of the position table")


def sequences(tokens: int, seq_start, q_len, kv_len, contiguous_kv: bool, table_keys: Optional[int] = None) -> None:
    """Sequence index tensors of the tensor-core attention kernels: query rows inside the buffer; keys inside the
    buffer (contiguous form) or inside a table row (paged form)."""
    _in_range("seq_start", seq_start, 0, max(tokens, 1), "rows of the token buffer")
    _in_range("q_len", q_len, 0, tokens + 1, "rows of the token buffer")
    end = seq_start.long() + q_len.long()
    if bool((end > tokens).any()):
        i, _ = _first_bad(end, end > tokens)
        raise IndexCheckError(f"sequence {i}: rows {int(seq_start[i])}..{int(end[i])} pass the {tokens} rows of the buffer")
    if contiguous_kv:
        kend = seq_start.long() + kv_len.long()
        if bool((kend > tokens).any()):
            i, _ = _first_bad(kend, kend > tokens)
            raise IndexCheckError(f"sequence {i}: keys {int(seq_start[i])}..{int(kend[i])} pass the {tokens} rows of the buffer")
    else:
        _in_range("kv_len", kv_len, 0, int(table_keys) + 1, "keys a table row can list")
        short = kv_len.long() < q_len.long()
        if bool(short.any()):
            i, _ = _first_bad(kv_len, short)
            raise IndexCheckError(f"sequence {i}: {int(q_len[i])} queries but only {int(kv_len[i])} keys")
