"""BitNet execution provider (crates/ronn-providers/src/bitnet/provider.rs:25-386).

Declares the reference's twelve operators and its speed-up constants.  MatMul / Gemm / FusedGemm nodes whose weight
is an initializer are compiled to PACKED low-bit weights (quantised and packed once at compile time - the reference
re-quantises both operands on every call, bitnet/kernels.rs:265-278) and executed by the low-bit kernels:

* on a GPU, the tcgen05 ``kind::i8`` BitLinear kernel (``csrc/kernels/bitnet.cu``): 2-bit packed weights expanded in
  shared memory, int8 activations, int32 accumulation in TMEM;
* on the host, the exact-integer kernel of ``csrc/cpu/bitnet_cpu.cc``.

Ternary (threshold or absmean) weights use the codes {-1, 0, +1}; binary weights {-1, +1} are the same format
without zeros.  Activations are quantised per token to int8 (absmax), or, with ``binarize_activations`` (the
reference's XNOR-popcount semantics, bitnet/kernels.rs:74-131), to sign bits with the scale mean|x|: a +-1 int8
operand through the same integer kernel gives exactly the XNOR-popcount result.  ``com.ronn::BitLinear`` nodes run
the same kernel; everything else uses the full-precision operator table.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ...core.types import (DataType, MemoryType, PerformanceProfile, ProviderCapability, ProviderConfig, ProviderType)
from ...graph.ir import ModelGraph
from ...onnx.registry import default_registry
from ..allocator import BitNetAllocator
from ..base import CompiledKernel, ExecutionProvider, build_kernel
from .quantization import QuantizationMethod, pack_ternary_rows, quantize_binary, quantize_ternary

BITNET_OPS = ["MatMul", "Gemm", "Conv", "Add", "Sub", "Mul", "And", "Or", "Xor", "BatchNormalization", "Relu", "Sigmoid"]


@dataclass
class BitNetProviderConfig:
    quantization_method: QuantizationMethod = QuantizationMethod.BINARY
    enable_kernel_caching: bool = True
    max_cache_size: int = 64 * 1024 * 1024
    enable_mixed_precision: bool = True
    memory_optimization_level: int = 2
    enable_simd: bool = True
    binarize_activations: bool = False      # True: sign-bit activations (XNOR-popcount arithmetic); False: per-token int8


class BitNetExecutionProvider(ExecutionProvider):
    provider_id = ProviderType.BITNET
    name = "BitNetExecutionProvider"

    def __init__(self, config: BitNetProviderConfig = None):
        self.config = config or BitNetProviderConfig()
        self.allocator = BitNetAllocator()

    def estimate_speedup(self, op_type: str) -> float:
        m = self.config.quantization_method
        table = {"MatMul": {QuantizationMethod.BINARY: 64.0, QuantizationMethod.TERNARY: 32.0, QuantizationMethod.ASYMMETRIC: 48.0},
                 "Gemm": {QuantizationMethod.BINARY: 64.0, QuantizationMethod.TERNARY: 32.0, QuantizationMethod.ASYMMETRIC: 48.0},
                 "Conv": {QuantizationMethod.BINARY: 32.0, QuantizationMethod.TERNARY: 24.0, QuantizationMethod.ASYMMETRIC: 28.0}}
        if op_type in table:
            return table[op_type][m]
        if op_type in ("And", "Or", "Xor"):
            return 128.0
        if op_type in ("Add", "Sub", "Mul", "Relu", "Sigmoid"):
            return 16.0
        return 1.0

    def get_capability(self) -> ProviderCapability:
        return ProviderCapability(
            supported_ops=set(default_registry().supported_ops()),
            data_types=[DataType.F32, DataType.BF16, DataType.F16, DataType.I8, DataType.U8, DataType.BOOL],
            memory_types=[MemoryType.SYSTEM, MemoryType.DEVICE],
            performance_profile=PerformanceProfile.MEMORY_OPTIMIZED,
            features={"quantization": self.config.quantization_method.value, "native_ops": list(BITNET_OPS)})

    def configure(self, config: ProviderConfig) -> None:
        opts = config.custom_options
        if "quantization_method" in opts:
            self.config.quantization_method = QuantizationMethod(opts["quantization_method"].lower())
        if "enable_simd" in opts:
            self.config.enable_simd = opts["enable_simd"].lower() in ("1", "true", "yes")

    def get_allocator(self):
        return self.allocator

    def compile_graph(self, graph: ModelGraph, profiler=None) -> CompiledKernel:
        reg = default_registry()
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        packed_cache = {}
        self.packed_weights = packed_cache         # name -> PackedLinear (inspection, tests, memory accounting)

        def pack_weight(name, transposed: bool):
            key = (name, transposed)
            if key not in packed_cache:
                w = graph.initializers[name].float()
                w_nk = w if transposed else w.t()                      # [N, K]: one packed row per output feature
                packed_cache[key] = PackedLinear.from_dense(w_nk.contiguous(), self.config.quantization_method, dev)
            return packed_cache[key]

        def resolve(node, g):
            if node.op_type in ("MatMul", "Gemm", "FusedGemm") and len(node.inputs) > 1 \
                    and node.inputs[1] in g.initializers and g.initializers[node.inputs[1]].dim() == 2 \
                    and g.initializers[node.inputs[1]].is_floating_point() \
                    and not (node.op_type == "Gemm" and int(node.attr("transA", 0))):
                transposed = bool(int(node.attr("transB", 0))) if node.op_type in ("Gemm", "FusedGemm") else False
                pl = pack_weight(node.inputs[1], transposed)
                if pl is not None:
                    return _low_bit_linear(node, pl, self.config.binarize_activations)
            return reg.get(node.op_type).fn

        # pack first, so that place() knows which initializers are only ever read in packed form
        for n in graph.nodes:
            resolve(n, graph)
        packed_names = {name for (name, _) in packed_cache}

        def place(name, t, users):
            only_packed = name in packed_names and users and all(
                u.op_type in ("MatMul", "Gemm", "FusedGemm") and len(u.inputs) > 1 and u.inputs[1] == name
                and name not in (list(u.inputs[:1]) + list(u.inputs[2:])) for u in users)
            if only_packed and name not in graph.output_names():
                return torch.empty(0, device=dev)          # no dense copy of a weight that only the packed kernel reads
            return t.to(dev)

        return build_kernel(graph, dev, resolve, place, self, profiler)


class PackedLinear:
    """A [N, K] weight in the BitLinear format: 2-bit codes, four per byte, one row per output feature, one fp32
    scale.  K is padded to a multiple of 64 with zero codes (they contribute nothing)."""
    __slots__ = ("packed", "scale", "n", "k", "k_padded", "n_padded", "method", "dense_bytes")

    def __init__(self, packed, scale, n, k, k_padded, n_padded, method, dense_bytes):
        self.packed, self.scale, self.n, self.k, self.k_padded, self.n_padded = packed, scale, n, k, k_padded, n_padded
        self.method, self.dense_bytes = method, dense_bytes

    @staticmethod
    def from_dense(w_nk: torch.Tensor, method: QuantizationMethod, device) -> "PackedLinear":
        n, k = w_nk.shape
        if method == QuantizationMethod.BINARY:
            scale = float(w_nk.abs().mean())
            vals = torch.where(w_nk >= 0, torch.ones((), dtype=torch.int8), -torch.ones((), dtype=torch.int8)).to(torch.int8)
        else:
            q = quantize_ternary(w_nk, "absmean" if method == QuantizationMethod.ASYMMETRIC else "threshold")
            scale, vals = q.scale, q.values().reshape(n, k)
        kp = -(-k // 64) * 64
        if kp != k:
            vals = torch.cat([vals, torch.zeros(n, kp - k, dtype=torch.int8)], dim=1)
        npad = -(-n // 8) * 8                                  # whole 16-byte output vectors; the extra rows are zero codes
        if npad != n:
            vals = torch.cat([vals, torch.zeros(npad - n, kp, dtype=torch.int8)], dim=0)
        packed = pack_ternary_rows(vals.contiguous()).contiguous().to(device)
        return PackedLinear(packed, float(scale), n, k, kp, npad, method, n * k * 4)

    def compression_ratio(self) -> float:
        return self.dense_bytes / max(self.packed.numel(), 1)


def _quantize_rows(x2: torch.Tensor, binarize: bool, k: int):
    """[rows, K padded] float activations (the first k columns are real) -> (int8 [rows, K], fp32 scale per row)."""
    if binarize:
        s = x2[:, :k].float().abs().mean().clamp_min(1e-12).expand(x2.shape[0]).contiguous()   # one scale per tensor
        q = torch.where(x2 >= 0, 1, -1).to(torch.int8)
        return q, s
    if x2.is_cuda and x2.dtype in (torch.bfloat16, torch.float16) and x2.shape[1] % 16 == 0:
        from ...ops import bitnet as KB
        return KB.act_quant_int8(x2)
    xf = x2.float()
    s = xf.abs().amax(-1).clamp_min(1e-5) / 127.0
    q = torch.round(xf / s[:, None]).clamp(-127, 127).to(torch.int8)
    return q, s.contiguous()


def _low_bit_linear(node, pl: PackedLinear, binarize: bool):
    """Operator function of a MatMul / Gemm / FusedGemm node whose weight is packed: quantise the activations, run the
    integer kernel (device or host), then the node's own epilogue (alpha / beta, bias, activation, residual)."""
    op = node.op_type
    alpha = float(node.attr("alpha", 1.0)) if op in ("Gemm", "FusedGemm") else 1.0
    beta = float(node.attr("beta", 1.0)) if op in ("Gemm", "FusedGemm") else 1.0
    act = node.attr("activation", "") if op == "FusedGemm" else ""

    def run(inputs, attrs, ctx):
        x = inputs[0]
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if pl.k_padded != pl.k:
            x2 = torch.nn.functional.pad(x2, (0, pl.k_padded - pl.k))
        q, s = _quantize_rows(x2, binarize, pl.k)
        if x2.is_cuda:
            from ...ops import bitnet as KB
            odt = x.dtype if x.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
            y = KB.bitlinear_q(q.contiguous(), s.float().contiguous(), pl.packed, pl.scale, None, pl.n_padded, pl.k_padded, odt)
            y = y[:, :pl.n].to(x.dtype)
        else:
            import ctypes as C
            import numpy as np
            from ... import _native
            qa = np.ascontiguousarray(q.numpy())
            sa = np.ascontiguousarray(s.float().numpy())
            wp = pl.packed.numpy()
            out = np.empty((qa.shape[0], pl.n_padded), dtype=np.float32)
            _native.host().ronn_bitnet_ternary_int8_matmul(qa.ctypes.data, sa.ctypes.data, wp.ctypes.data, C.c_float(pl.scale),
                                                           out.ctypes.data, None, qa.shape[0], pl.n_padded, pl.k_padded)
            y = torch.from_numpy(out[:, :pl.n].copy()).to(x.dtype)
        y = y.reshape(*lead, pl.n)
        if alpha != 1.0:
            y = y * alpha
        if len(inputs) > 2 and inputs[2] is not None:
            y = y + (inputs[2] if beta == 1.0 else inputs[2] * beta)
        if act:
            a = act.lower()
            if a == "relu":
                y = torch.relu(y)
            elif a == "gelu":
                y = torch.nn.functional.gelu(y.float(), approximate="tanh").to(y.dtype)
            elif a in ("sigmoid",):
                y = torch.sigmoid(y)
            elif a == "tanh":
                y = torch.tanh(y)
        if op == "FusedGemm" and len(inputs) > 3 and inputs[3] is not None:
            y = y + inputs[3]
        return [y]

    return run
