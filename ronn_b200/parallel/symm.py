"""Fused compute + collective communicator over NVLink peer memory.

One symmetric allocation per rank (``torch.distributed._symmetric_memory``: every rank maps every
peer's copy) holds the partial-product slots (two parities) and the flag words of the fused
row-parallel GEMM.  ``FusedComm.gemm_allreduce`` / ``gemm_reduce_scatter`` launch ONE kernel that
computes this rank's partial GEMM on the tensor cores, publishes it, waits for the peers with a
bounded spin, and reduces straight from peer memory (see ``csrc/kernels/comm_gemm.cu``).  NCCL is
only used for the rendezvous and for the tiny (max, index) gather of the sharded argmax.

Four exchange protocols share the class (``RONN_TP_PROTO`` or the ``proto`` argument):

* ``ll`` (default, results up to ``RONN_LL_ELEMS`` elements with N % 32 == 0): ``csrc/kernels/gemm_ll.cu``.  Partial
  rows travel to their owner rank and finished rows to every rank as {data, sequence} words; readers poll their own
  memory, so no fence, flag or atomic lies between the ranks and a call costs two one-way NVLink trips.  Larger
  results fall through to ``pull`` / the library all-reduce.
* ``two_shot``: ``csrc/kernels/gemm_fuse.cu``.  Every output row has one owner rank; the owner sums the
  fp32 partials of all ranks (``multimem.ld_reduce`` through the NVSwitch when the allocation has a multicast
  address, peer loads otherwise), applies bias / residual / norm once and stores the finished rows into every
  rank's output (``multimem.st`` or peer stores).  Each rank moves 1/W of the result.
* ``pull`` / ``push``: the one-shot protocols of ``csrc/kernels/comm_gemm.cu`` (every rank reads or receives every
  peer's whole partial result and reduces redundantly).

A device-side wait that runs out leaves ``STATUS_WAIT_PEER`` in the status word; ``check()``
turns it into ``CommTimeoutError`` on the host; ``reset()`` (collective) clears the counters afterwards.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native
from ..api.errors import ProviderError
from ..ops import kernels as K
from .group import TPComm

MAX_RANKS = 8
_FLAG_INTS = 2 * MAX_RANKS


class FusedComm(TPComm):
    """Tensor-parallel communicator whose row-parallel collectives are fused into the GEMM kernel."""
    fused = True

    def __init__(self, device: torch.device, max_rows: int = 8192, max_cols: int = 8192, group=None,
                 wait_seconds: Optional[float] = None, proto: Optional[str] = None, nvls: Optional[bool] = None):
        super().__init__(group)
        self._ctor = dict(max_rows=max_rows, max_cols=max_cols, group=group, wait_seconds=wait_seconds, proto=proto,
                          nvls=nvls)
        if self.world > MAX_RANKS:
            raise ProviderError(f"fused collectives support at most {MAX_RANKS} ranks")
        import torch.distributed._symmetric_memory as symm
        self.device = torch.device(device)
        self.max_elems = max_rows * max_cols
        self.part_stride = self.max_elems * 2                       # bytes of one parity slot (16-bit elements)
        flag_bytes = 512                                            # reduce flags [2][8] ints, gather flags [8] ints
        self.shard_bytes = (max_rows // max(self.world, 1) + 128) * max_cols * 2
        # receive area of the push variant: [2 parities][world sources][push_elems] values, 4 bytes each (16-bit data
        # paired with the call's sequence number)
        self.push_elems = int(os.environ.get("RONN_PUSH_ELEMS", 1 << 20)) if self.world > 1 else 0
        self.recv_src_stride = self.push_elems * 4
        self.recv_parity_stride = self.recv_src_stride * self.world
        recv_bytes = 2 * self.recv_parity_stride
        # exchange area of the sharded argmax: [2 parities][world sources][max_argmax_rows] records of 16 bytes
        self.max_argmax_rows = 4096
        argmax_bytes = 2 * self.world * self.max_argmax_rows * 16
        total = 2 * self.part_stride + flag_bytes + self.shard_bytes + recv_bytes + argmax_bytes
        self._buf = symm.empty(total, dtype=torch.uint8, device=self.device)
        self._buf.zero_()
        torch.cuda.synchronize(self.device)
        pg = group if group is not None else dist.group.WORLD
        self._hdl = symm.rendezvous(self._buf, pg.group_name if hasattr(pg, "group_name") else pg)
        ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        self._part_ptrs = (C.c_void_p * MAX_RANKS)(*[ptrs[p] if p < self.world else None for p in range(MAX_RANKS)])
        self._flag_ptrs = (C.c_void_p * MAX_RANKS)(*[(ptrs[p] + 2 * self.part_stride) if p < self.world else None
                                                    for p in range(MAX_RANKS)])
        self._ag_flag_ptrs = (C.c_void_p * MAX_RANKS)(*[(ptrs[p] + 2 * self.part_stride + 256) if p < self.world else None
                                                       for p in range(MAX_RANKS)])
        shard_off = 2 * self.part_stride + flag_bytes
        self._shard_ptrs = (C.c_void_p * MAX_RANKS)(*[(ptrs[p] + shard_off) if p < self.world else None
                                                     for p in range(MAX_RANKS)])
        self._shard_local = self._buf[shard_off: shard_off + self.shard_bytes]
        recv_off = shard_off + self.shard_bytes
        self._recv_ptrs = (C.c_void_p * MAX_RANKS)(*[(ptrs[p] + recv_off) if p < self.world else None
                                                    for p in range(MAX_RANKS)])
        argmax_off = recv_off + recv_bytes
        self._argmax_ptrs = (C.c_void_p * MAX_RANKS)(*[(ptrs[p] + argmax_off) if p < self.world else None
                                                      for p in range(MAX_RANKS)])
        self._argmax_state = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._ag_flags_local = ptrs[self.rank] + 2 * self.part_stride + 256
        self._ag_state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._state = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.wait_seconds = float(os.environ.get("RONN_PEER_WAIT_S", wait_seconds if wait_seconds is not None else 2.0))
        self.proto = proto or os.environ.get("RONN_TP_PROTO", "ll")
        if self.proto not in ("ll", "two_shot", "pull", "push"):
            raise ProviderError(f"unknown tensor-parallel protocol '{self.proto}'")
        self._init_two_shot(symm, pg, nvls)
        self.fused_calls = 0
        self.bitlinear_ll = os.environ.get("RONN_BITLINEAR_LL", "1") != "0"      # one-launch row-parallel BitLinear
        self.one_shot_elems = int(os.environ.get("RONN_ONE_SHOT_ELEMS", 2 << 20))
        self.argmax_exchange = self.world > 1 and os.environ.get("RONN_ARGMAX_EXCHANGE", "1") != "0"
        # Push pays when there is one peer (measured, GPT-2 medium decode: TP=2 85-88K tokens/s against 80K with the pull
        # protocol).  With more peers every rank stores world copies of its partials as 16-byte NVLink writes at twice
        # the data volume, and the pull protocol wins (TP=4 103K against 92K, TP=8 102K against 71K).
        env = os.environ.get("RONN_TP_PUSH")
        self.push = self.world > 1 and (env == "1" if env is not None else self.world == 2)
        if self.proto == "push":
            self.push = self.world > 1
        elif self.proto == "pull":
            self.push = False
        dist.barrier(group=group)                                     # flags and counters are zero everywhere

    def clone(self, max_rows: Optional[int] = None) -> "FusedComm":
        """A second communicator with its own symmetric buffers, flags and call counter, for launches that run
        concurrently with this one's on another stream.  Collective: every rank calls it in the same order."""
        kw = dict(self._ctor)
        if max_rows is not None:
            kw["max_rows"] = max_rows
        return FusedComm(self.device, **kw)

    # ------------------------------------------------------------------ two-shot protocol (gemm_fuse.cu)
    def _init_two_shot(self, symm, pg, nvls: Optional[bool]) -> None:
        """Second symmetric allocation: counters, fp32 partial slots (two parities) and two alternating pairs of output
        slots (residual stream X, normalised H).  Outputs must be symmetric because the owner of a row stores it into
        every rank's copy."""
        from ..ops import fuse as F
        lib = F._lib()
        self._flag_ints = lib.ronn_gemm_fuse_flag_ints()
        self._flag_bytes = (self._flag_ints * 4 + 1023) // 1024 * 1024
        self.parity_floats = min(self.max_elems, int(os.environ.get("RONN_TWO_SHOT_ELEMS", 8 << 20)))
        self._out_bytes = self.parity_floats * 2
        # areas of the low-latency protocol: [2 parities][world sources][owner rows * N] and [2 parities][M * N]
        # values of 4 bytes (a 16-bit value and its half of the sequence word)
        self.ll_elems = min(int(os.environ.get("RONN_LL_ELEMS", 1 << 20)), self.max_elems)
        self._ll_cols = 8192
        self._ll_scatter_stride = (self.ll_elems * max(1, MAX_RANKS // max(self.world, 1)) + MAX_RANKS * self._ll_cols) * 4
        self._ll_result_stride = self.ll_elems * 4
        self._ll_off = self._flag_bytes + 2 * self.parity_floats * 4 + 4 * self._out_bytes
        total = self._ll_off + 2 * self._ll_scatter_stride + 2 * self._ll_result_stride
        self._buf2 = symm.empty(total, dtype=torch.uint8, device=self.device)
        self._buf2.zero_()
        torch.cuda.synchronize(self.device)
        self._hdl2 = symm.rendezvous(self._buf2, pg.group_name if hasattr(pg, "group_name") else pg)
        self._ptrs2 = [int(p) for p in self._hdl2.buffer_ptrs]
        mc = int(getattr(self._hdl2, "multicast_ptr", 0) or 0)
        want = nvls if nvls is not None else os.environ.get("RONN_NVLS", "1") != "0"
        self.nvls_available = bool(mc) and self.world > 1
        self.nvls = bool(want and self.nvls_available)              # may be switched off (not on) later
        self._mc2 = mc
        self._state2 = torch.zeros(lib.ronn_gemm_fuse_state_ints(), dtype=torch.int32, device=self.device)
        self._slot = 0
        self._ll_state = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.trace = None                                           # set to a uint64 tensor [ctas, 8] to record timestamps

    def _slot_views(self, slot: int, M: int, N: int, dtype):
        off_x = self._flag_bytes + 2 * self.parity_floats * 4 + (2 * slot) * self._out_bytes
        off_h = off_x + self._out_bytes
        n = M * N * 2
        x = self._buf2[off_x: off_x + n].view(dtype).view(M, N)
        h = self._buf2[off_h: off_h + n].view(dtype).view(M, N)
        return off_x, off_h, x, h

    def reset(self) -> None:
        """Collective: clear every counter after an abandoned wait (the ranks' counters no longer agree)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self._buf2[: self._flag_bytes].zero_()
        self._buf2[self._ll_off:].zero_()
        self._state2.zero_()
        self._ll_state.zero_()
        self._buf[2 * self.part_stride: 2 * self.part_stride + 512].zero_()
        self._state.zero_()
        self._ag_state.zero_()
        self._argmax_state.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def _gemm_two_shot(self, a, w_nk, bias, residual, norm, scatter: bool, splitk: int = 0, bn: int = 0):
        from ..ops import fuse as F
        M, Kd = a.shape
        N = w_nk.shape[0]
        S = splitk if splitk > 0 else F.pick_splitk(M, N, Kd)
        while S > 1 and S * M * N > self.parity_floats:
            S //= 2
        if S * M * N > self.parity_floats:
            raise ProviderError(f"fused GEMM of {M}x{N} exceeds the symmetric buffer of the two-shot protocol")
        if bias is not None and bias.dtype != a.dtype:
            bias = bias.to(a.dtype)
        per = -(-M // self.world)
        p = F.FuseParams()
        p.A, p.W = a.data_ptr(), w_nk.data_ptr()
        p.M, p.N, p.K, p.lda, p.ldw = M, N, Kd, a.stride(0), w_nk.stride(0)
        p.splitk, p.bn, p.dtype = S, bn, 0 if a.dtype == torch.bfloat16 else 1
        part_off = self._flag_bytes
        for r in range(self.world):
            p.part[r] = self._ptrs2[r] + part_off
            p.flags[r] = self._ptrs2[r]
        p.parity_stride = self.parity_floats
        p.state = self._state2.data_ptr()
        use_mc = self.nvls and self.nvls_available
        p.rank, p.world, p.nvls, p.scatter = self.rank, self.world, 1 if use_mc else 0, 1 if scatter else 0
        if use_mc:
            p.part_mc, p.flags_mc = self._mc2 + part_off, self._mc2
        normed = None
        if scatter:
            rows = max(min(per, M - self.rank * per), 0)
            out = torch.empty((rows, N), dtype=a.dtype, device=a.device)
            p.out[self.rank] = out.data_ptr()
            for r in range(self.world):
                if r != self.rank:
                    p.out[r] = out.data_ptr()                     # never dereferenced in this mode
            if norm is not None:
                normed = torch.empty_like(out)
                for r in range(self.world):
                    p.norm_out[r] = normed.data_ptr()
        else:
            self._slot ^= 1
            off_x, off_h, out, h = self._slot_views(self._slot, M, N, a.dtype)
            for r in range(self.world):
                p.out[r] = self._ptrs2[r] + off_x
                p.norm_out[r] = self._ptrs2[r] + off_h
            if use_mc:
                p.out_mc, p.norm_mc = self._mc2 + off_x, self._mc2 + off_h
            if norm is not None:
                normed = h
        p.ld_out = N
        if residual is not None:
            if residual.stride(1) != 1 or residual.shape != out.shape:
                residual = residual.reshape(out.shape).contiguous()
            p.residual, p.ld_res = residual.data_ptr(), residual.stride(0)
        p.bias = None if bias is None else bias.data_ptr()
        if norm is not None:
            kind, gamma, beta, eps = norm
            p.norm_mode, p.eps = (1 if kind == "layernorm" else 2), float(eps)
            p.gamma = None if gamma is None else gamma.data_ptr()
            p.beta = None if beta is None else beta.data_ptr()
        p.wait_seconds = self.wait_seconds
        p.trace = None if self.trace is None else self.trace.data_ptr()
        rc = F._lib().ronn_gemm_fuse(C.byref(p), K.status_word(a.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise K.KernelError(f"gemm_fuse (world {self.world}) failed with code {rc}")
        self.fused_calls += 1
        return out if norm is None else (out, normed)

    # ------------------------------------------------------------------ low-latency protocol (gemm_ll.cu)
    def _ll_ok(self, M: int, N: int) -> bool:
        return (self.world > 1 and M * N <= self.ll_elems and N % 32 == 0 and N <= self._ll_cols
                and -(-M // self.world) * self.world * N * 4 <= self._ll_scatter_stride)

    def _ll_splitk(self, M: int, N: int, Kd: int) -> int:
        """K slices per rank: at least eight 64-wide K blocks per slice, at most 8 (rank, slice) sources in all."""
        env = os.environ.get("RONN_LL_SPLITK")
        s = int(env) if env else max(1, min(MAX_RANKS // self.world, ((Kd + 63) // 64) // 8))
        while s > 1 and -(-M // self.world) * self.world * s * N * 4 > self._ll_scatter_stride:
            s -= 1
        return s

    def _ll_fill_areas(self, p) -> None:
        """Areas, epoch word, rank / world and the NVLS choice of a low-latency call (``LLParams``)."""
        res_off = self._ll_off + 2 * self._ll_scatter_stride
        for r in range(self.world):
            p.scatter_area[r] = self._ptrs2[r] + self._ll_off
            p.result_area[r] = self._ptrs2[r] + res_off
        use_mc = self.nvls and self.nvls_available
        p.result_mc = (self._mc2 + res_off) if use_mc else None
        p.scatter_parity_stride, p.result_parity_stride = self._ll_scatter_stride, self._ll_result_stride
        p.state = self._ll_state.data_ptr()
        p.rank, p.world, p.nvls = self.rank, self.world, 1 if use_mc else 0
        p.wait_seconds = self.wait_seconds
        p.trace = None if self.trace is None else self.trace.data_ptr()

    def _bitlinear_ll(self, q, x_scale, w_packed, w_scale: float, n: int, k: int, out_dtype, residual, norm_quant=None):
        """Row-parallel BitLinear + cross-rank sum + residual in ONE launch (low-latency protocol).  Returns None when
        the launcher says the shape does not fit (grid larger than the SMs): the caller takes the two-launch path.
        ``norm_quant=(gamma, eps)``: the unpack pass also applies RMSNorm * gamma and the per-token int8 quantisation
        the next BitLinear layer needs; the result is then (out, q, scale)."""
        from ..ops import fuse as F
        M = q.shape[0]
        out = torch.empty((M, n), dtype=out_dtype, device=q.device)
        if residual is not None and (residual.stride(1) != 1 or residual.shape != out.shape):
            residual = residual.reshape(M, n).contiguous()
        bp = F.BitLinearLLParams()
        bp.xq, bp.w_packed, bp.x_scale = q.data_ptr(), w_packed.data_ptr(), x_scale.data_ptr()
        bp.w_scale, bp.ldx = float(w_scale), q.stride(0)
        p = bp.ll
        p.M, p.N, p.K, p.dtype = M, n, k, 0 if out_dtype == torch.bfloat16 else 1
        self._ll_fill_areas(p)
        p.out, p.ld_out = out.data_ptr(), out.stride(0)
        if residual is not None:
            p.residual, p.ld_res = residual.data_ptr(), residual.stride(0)
        nq = ns = None
        if norm_quant is not None:
            gamma, eps = norm_quant
            nq = torch.empty((M, n), dtype=torch.int8, device=q.device)
            ns = torch.empty(M, dtype=torch.float32, device=q.device)
            p.norm_mode, p.gamma, p.eps = 3, gamma.data_ptr(), float(eps)
            p.quant_out, p.quant_scale = nq.data_ptr(), ns.data_ptr()
        rc = F._lib().ronn_bitlinear_ll(C.byref(bp), K.status_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
        if rc == -12:
            return None
        if rc != 0:
            raise K.KernelError(f"bitlinear_ll (world {self.world}) failed with code {rc}")
        self.fused_calls += 1
        return out if norm_quant is None else (out, nq, ns)

    def _gemm_ll(self, a, w_nk, bias, residual, norm, bn: int = 0):
        from ..ops import fuse as F
        M, Kd = a.shape
        N = w_nk.shape[0]
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
        if bias is not None and bias.dtype != a.dtype:
            bias = bias.to(a.dtype)
        if residual is not None and (residual.stride(1) != 1 or residual.shape != out.shape):
            residual = residual.reshape(M, N).contiguous()
        p = F.LLParams()
        p.A, p.W = a.data_ptr(), w_nk.data_ptr()
        p.M, p.N, p.K, p.lda, p.ldw = M, N, Kd, a.stride(0), w_nk.stride(0)
        p.bn, p.dtype, p.splitk = bn, 0 if a.dtype == torch.bfloat16 else 1, self._ll_splitk(M, N, Kd)
        self._ll_fill_areas(p)
        p.out, p.ld_out = out.data_ptr(), out.stride(0)
        p.bias = None if bias is None else bias.data_ptr()
        if residual is not None:
            p.residual, p.ld_res = residual.data_ptr(), residual.stride(0)
        normed = None
        if norm is not None:
            kind, gamma, beta, eps = norm
            normed = torch.empty_like(out)
            p.norm_out, p.norm_mode, p.eps = normed.data_ptr(), (1 if kind == "layernorm" else 2), float(eps)
            p.gamma = None if gamma is None else gamma.data_ptr()
            p.beta = None if beta is None else beta.data_ptr()
        p.wait_seconds = self.wait_seconds
        p.trace = None if self.trace is None else self.trace.data_ptr()
        rc = F._lib().ronn_gemm_ll(C.byref(p), K.status_word(a.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise K.KernelError(f"gemm_ll (world {self.world}) failed with code {rc}")
        self.fused_calls += 1
        return out if norm is None else (out, normed)

    # ------------------------------------------------------------------ fused row-parallel GEMM
    def _gemm_reduce(self, a, w_nk, bias, residual, row_begin, row_end, bn=0, norm=None):
        M, Kd = a.shape
        N = w_nk.shape[0]
        if M * N > self.max_elems:
            raise ProviderError(f"fused GEMM of {M}x{N} exceeds the symmetric buffer ({self.max_elems} elements)")
        rows = row_end - row_begin
        out = torch.empty((rows, N), dtype=a.dtype, device=a.device)
        if residual is not None and (residual.stride(1) != 1 or residual.shape != out.shape):
            residual = residual.reshape(rows, N).contiguous()
        if bias is not None and bias.dtype != a.dtype:
            bias = bias.to(a.dtype)
        normed, gamma, beta, eps, mode = None, None, None, 0.0, 0
        if norm is not None:
            kind, gamma, beta, eps = norm
            mode = 1 if kind == "layernorm" else 2
            normed = torch.empty_like(out)
        args = (a.data_ptr(), w_nk.data_ptr(), M, N, Kd, a.stride(0), w_nk.stride(0), self._part_ptrs, self._flag_ptrs,
                self.part_stride, self._state.data_ptr(), self.rank, self.world, row_begin, row_end, out.data_ptr(),
                out.stride(0), None if bias is None else bias.data_ptr(),
                None if residual is None else residual.data_ptr(), residual.stride(0) if residual is not None else 0,
                self.wait_seconds, 0 if a.dtype == torch.bfloat16 else 1, bn,
                None if normed is None else normed.data_ptr(), None if gamma is None else gamma.data_ptr(),
                None if beta is None else beta.data_ptr(), float(eps), mode)
        tail = (K.status_word(a.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
        if self.push and 0 < M * N <= self.push_elems and N % 32 == 0 and N <= 1024:
            # small result (decode): partial tiles are stored into every rank's receive slots by the GEMM epilogue
            rc = _native.cuda().ronn_gemm_reduce_push(*args, self._recv_ptrs, self.recv_parity_stride,
                                                      self.recv_src_stride, *tail)
        else:
            rc = _native.cuda().ronn_gemm_reduce(*args, *tail)
        if rc != 0:
            raise K.KernelError(f"gemm_reduce failed with code {rc}")
        self.fused_calls += 1
        return out if norm is None else (out, normed)

    def gemm_allreduce(self, a, w_nk, bias=None, residual=None, bn=0, norm=None):
        """sum over ranks of (a @ w_nk^T) + bias + residual, full result on every rank (bit-identical).
        ``norm=(kind, gamma, beta, eps)`` (hidden size <= 1024) also returns the normalised rows: the reduction
        pass holds whole rows in registers, so the next block's LayerNorm / RMSNorm costs no extra kernel.

        The one-shot exchange (every rank reads every peer's whole partial result) is a latency design: measured
        1.3-1.6x faster than GEMM + NCCL all-reduce + norm for decode-sized results, but 0.7x at 8192 x 1024 where
        moving (world - 1) full copies per rank costs more than a ring.  Results above ``one_shot_elems`` therefore
        take the GEMM kernel + library all-reduce + the fused bias/residual/norm kernel."""
        M, N = a.shape[0], w_nk.shape[0]
        if self.proto == "ll" and self._ll_ok(M, N):
            return self._gemm_ll(a, w_nk, bias, residual, norm, bn=bn)
        if self.proto == "two_shot" and M <= 8192 and M * N <= self.parity_floats:
            return self._gemm_two_shot(a, w_nk, bias, residual, norm, scatter=False, bn=bn)
        if self.world > 1 and M * N > self.one_shot_elems:
            y = K.gemm(a, w_nk)
            dist.all_reduce(y, group=self.group)
            self.calls += 1
            if bias is not None:
                y += bias
            if norm is None:
                return y + residual if residual is not None else y
            kind, gamma, beta, eps = norm
            if kind == "layernorm":
                normed, total = K.layernorm(y, gamma, beta, eps, residual=residual, return_sum=True)
            else:
                normed, total = K.rmsnorm(y, gamma, eps, residual=residual, return_sum=True)
            return total, normed
        return self._gemm_reduce(a, w_nk, bias, residual, 0, a.shape[0], bn, norm)

    def argmax_combine(self, idx: torch.Tensor, mx: torch.Tensor) -> torch.Tensor:
        """Greedy token per row over the vocabulary shards: every rank's (index, max) pairs are exchanged through
        symmetric memory by one small kernel (sequence-numbered words, no library collective); largest value wins,
        lowest index on ties, the same on every rank."""
        rows = idx.shape[0]
        if not self.argmax_exchange or rows > self.max_argmax_rows:
            vals = self.all_gather_small(mx)
            idxs = self.all_gather_small(idx)
            return K.argmax_combine(vals.contiguous(), idxs.contiguous())
        idx = idx.contiguous()
        mx = mx.float().contiguous()
        tokens = torch.empty(rows, dtype=torch.int32, device=idx.device)
        rc = _native.cuda().ronn_argmax_exchange(idx.data_ptr(), mx.data_ptr(), tokens.data_ptr(), rows, self._argmax_ptrs,
                                                 self.max_argmax_rows, self._argmax_state.data_ptr(), self.rank,
                                                 self.world, self.wait_seconds, K.status_word(idx.device).data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise K.KernelError(f"argmax_exchange failed with code {rc}")
        return tokens

    # ------------------------------------------------------------------ BitLinear partials + cross-rank reduction
    def bitlinear_allreduce(self, q, x_scale, w_packed, w_scale: float, n: int, k: int, out_dtype, residual=None,
                            norm_quant=None):
        """Row-parallel BitLinear + cross-rank sum + residual, bit-identical on every rank, no library collective.
        Under the low-latency protocol ONE launch: the BitLinear kernel's epilogue scatters its scaled rows to their
        owner ranks as {data, sequence} words and goes on to reduce, broadcast and unpack (``ronn_bitlinear_ll``;
        ``RONN_BITLINEAR_LL=0`` turns it off).  Otherwise two launches: the kernel writes this rank's [M, n] partial
        straight into the current slot of the symmetric partial buffer (slot chosen on the device) and the reduction
        kernel sums the ranks' partials over NVLink peer memory in rank order."""
        from ..ops.bitnet import _check as _bcheck
        M = q.shape[0]
        if (self.proto == "ll" and self.bitlinear_ll and self._ll_ok(M, n) and k % 64 == 0
                and w_packed.data_ptr() % 16 == 0):
            y = self._bitlinear_ll(q, x_scale, w_packed, w_scale, n, k, out_dtype, residual,
                                   norm_quant if (norm_quant is not None and n % 8 == 0 and n <= 8192
                                                  and norm_quant[0].dtype == out_dtype) else None)
            if y is not None:
                return y
        if M * n > self.max_elems:
            raise ProviderError(f"fused BitLinear of {M}x{n} exceeds the symmetric buffer ({self.max_elems} elements)")
        lib = _native.cuda()
        dt = 0 if out_dtype == torch.bfloat16 else 1
        stream = torch.cuda.current_stream().cuda_stream
        status = K.status_word(q.device).data_ptr()
        from ..ops.bitnet import slice_workspace
        ws = slice_workspace(M, n, k, q.device)
        _bcheck(lib.ronn_bitlinear_to_slot(q.data_ptr(), w_packed.data_ptr(), x_scale.data_ptr(), float(w_scale),
                                           self._part_ptrs[self.rank], self._state.data_ptr(), self.part_stride,
                                           None if ws is None else ws.data_ptr(), M, n, k,
                                           q.stride(0), dt, status, stream), "bitlinear_to_slot")
        out = torch.empty((M, n), dtype=out_dtype, device=q.device)
        if residual is not None and (residual.stride(1) != 1 or residual.shape != out.shape):
            residual = residual.reshape(M, n).contiguous()
        rc = lib.ronn_peer_reduce(M, n, self._part_ptrs, self._flag_ptrs, self.part_stride, self._state.data_ptr(),
                                  self.rank, self.world, 0, M, out.data_ptr(), out.stride(0), None,
                                  None if residual is None else residual.data_ptr(),
                                  residual.stride(0) if residual is not None else 0, self.wait_seconds, dt, None, None,
                                  None, 0.0, 0, status, stream)
        if rc != 0:
            raise K.KernelError(f"peer_reduce failed with code {rc}")
        self.fused_calls += 1
        return out

    def gemm_reduce_scatter(self, a, w_nk, bias=None, residual_shard=None, bn=0):
        """Same sum, but each rank keeps only its contiguous shard of the rows (M must divide by the world size)."""
        M = a.shape[0]
        if M % self.world:
            raise ProviderError("reduce-scatter needs the row count to divide by the world size")
        per = M // self.world
        if self.proto == "two_shot" and M <= 8192 and M * w_nk.shape[0] <= self.parity_floats:
            return self._gemm_two_shot(a, w_nk, bias, residual_shard, None, scatter=True, bn=bn)
        return self._gemm_reduce(a, w_nk, bias, residual_shard, self.rank * per, (self.rank + 1) * per, bn)

    # ------------------------------------------------------------------ fused all-gather -> column-parallel GEMM
    def shard_buffer(self, rows: int, cols: int, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """This rank's [rows, cols] activation shard inside the symmetric allocation: write the shard here (e.g. as the
        output of the norm kernel), call ``signal_shard_ready()``, then ``ag_gemm``."""
        nbytes = rows * cols * 2
        if nbytes > self.shard_bytes:
            raise ProviderError(f"shard of {rows}x{cols} exceeds the symmetric shard buffer")
        return self._shard_local[:nbytes].view(dtype).view(rows, cols)

    def signal_shard_ready(self) -> None:
        rc = _native.cuda().ronn_signal_peers(self._ag_flag_ptrs, self.rank, self.world,
                                              torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise K.KernelError(f"signal_peers failed with code {rc}")

    def ag_gemm(self, rows_per_rank: int, k: int, w_nk: torch.Tensor, bias=None, activation: str = "", bn: int = 0):
        """concat over ranks of the [rows_per_rank, k] shards (read tile by tile from peer memory) @ w_nk^T.
        rows_per_rank must be a multiple of 128; a fused row-parallel GEMM must separate two gathers."""
        N = w_nk.shape[0]
        out = torch.empty((rows_per_rank * self.world, N), dtype=w_nk.dtype, device=w_nk.device)
        if bias is not None and bias.dtype != w_nk.dtype:
            bias = bias.to(w_nk.dtype)
        rc = _native.cuda().ronn_ag_gemm(self._shard_ptrs, k, w_nk.data_ptr(), w_nk.stride(0), out.data_ptr(), out.stride(0),
                                         None if bias is None else bias.data_ptr(), rows_per_rank, N, k, self.rank, self.world,
                                         self._ag_flags_local, self._ag_state.data_ptr(), K._ACT[activation],
                                         self.wait_seconds, 0 if w_nk.dtype == torch.bfloat16 else 1, bn,
                                         K.status_word(w_nk.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise K.KernelError(f"ag_gemm failed with code {rc}")
        self.fused_calls += 1
        return out

    def check(self) -> None:
        K.check_status(self.device)
