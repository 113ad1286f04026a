"""Read-only view of the paged KV cache in the vocabulary of the KV-cache design
(docs/new/RONN-KV-Cache-Compression-Branch-Prompt.md:125-195): ``PageTable`` maps (sequence, logical block) to a physical
block, ``BlockMetadata`` carries reference count, location, precision and token count of a block, ``BlockManager`` reports
the device pool, the host pool and the memory budget.

The state itself lives in the native scheduler (``csrc/serving/scheduler.cc``: block pool, reference counts, page tables,
host-pool assignments of swapped-out sequences) and in the engine (the cache tensors); nothing is duplicated here.
Blocks hold 16 tokens.  Cache precision is the engine's compute dtype: the quantised cache precisions of the design are
listed for parity of the vocabulary, and asking for one raises.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch

from ..api.errors import SessionError


class BlockLocation(enum.Enum):
    GPU = "gpu"
    CPU = "cpu"                 # swapped out to the host pool
    UNIFIED = "unified"         # a CPU engine: cache tensors live in host memory that the compute reads directly


class CachePrecision(enum.Enum):
    FP32 = "fp32"
    FP16 = "fp16"
    BF16 = "bf16"
    INT8 = "int8"
    INT4 = "int4"
    INT2 = "int2"
    INT1 = "int1"

    @staticmethod
    def of(dtype: torch.dtype) -> "CachePrecision":
        table = {torch.float32: CachePrecision.FP32, torch.float16: CachePrecision.FP16,
                 torch.bfloat16: CachePrecision.BF16}
        if dtype not in table:
            raise SessionError(f"no cache precision for {dtype}")
        return table[dtype]

    def require_supported(self) -> "CachePrecision":
        if self in (CachePrecision.INT8, CachePrecision.INT4, CachePrecision.INT2, CachePrecision.INT1):
            raise SessionError(f"KV cache precision {self.value} is not implemented (quantised caches are out of scope)")
        return self


@dataclass(frozen=True)
class BlockMetadata:
    ref_count: int
    location: BlockLocation
    precision: CachePrecision
    num_tokens: int


class PageTable:
    """(sequence id, logical block) -> (location, physical block) of the live sequences."""

    def __init__(self, engine):
        self._e = engine

    def blocks(self, seq_id: int) -> List[Tuple[BlockLocation, int]]:
        s = self._e.sched
        dev = BlockLocation.GPU if self._e.device.type == "cuda" else BlockLocation.UNIFIED
        swapped = s.cpu_blocks(seq_id)
        if swapped:
            return [(BlockLocation.CPU, b) for b in swapped]
        return [(dev, b) for b in s.blocks(seq_id)]

    def lookup(self, seq_id: int, logical_block: int) -> Tuple[BlockLocation, int]:
        blocks = self.blocks(seq_id)
        if not 0 <= logical_block < len(blocks):
            raise KeyError((seq_id, logical_block))
        return blocks[logical_block]

    def as_dict(self) -> Dict[Tuple[int, int], Tuple[BlockLocation, int]]:
        out = {}
        for rid in self._e.requests:
            if self._e.sched.state(rid) is None:
                continue
            for lb, entry in enumerate(self.blocks(rid)):
                out[(rid, lb)] = entry
        return out


class BlockManager:
    def __init__(self, engine):
        self._e = engine
        self.page_table = PageTable(engine)
        self.block_size = engine.cfg.block_size
        self.precision = CachePrecision.of(engine.runner.kcache[0].dtype).require_supported()

    @property
    def block_bytes(self) -> int:
        """Bytes of one block over all layers, keys and values."""
        k = self._e.runner.kcache[0]
        return 2 * len(self._e.runner.kcache) * k[0].numel() * k.element_size()

    @property
    def gpu_pool(self) -> Dict[str, int]:
        total = self._e.runner.num_blocks
        return {"total_blocks": total, "free_blocks": self._e.sched.num_free_blocks}

    @property
    def cpu_pool(self) -> Dict[str, int]:
        total = 0 if self._e._cpu_k is None else self._e._cpu_k[0].shape[0]
        return {"total_blocks": total, "free_blocks": self._e.sched.swap_stats()["free_cpu_blocks"]}

    @property
    def vram_budget(self) -> int:
        """Bytes the device block pool occupies."""
        return self._e.runner.num_blocks * self.block_bytes

    def metadata(self, seq_id: int, logical_block: int) -> BlockMetadata:
        loc, phys = self.page_table.lookup(seq_id, logical_block)
        cached = max(self._e.sched.num_computed(seq_id), 0)
        tokens = max(0, min(self.block_size, cached - logical_block * self.block_size))
        ref = 1 if loc == BlockLocation.CPU else self._e.sched.block_ref(phys)
        return BlockMetadata(ref, loc, self.precision, tokens)

    def utilization(self) -> float:
        pool = self.gpu_pool
        return 1.0 - pool["free_blocks"] / pool["total_blocks"] if pool["total_blocks"] else 0.0
