"""Execution providers and the factories that assemble a registry
(crates/ronn-providers/src/lib.rs:104-236)."""
from __future__ import annotations

import torch

from .base import CompiledKernel, ExecutionProvider, TensorAllocator
from .cpu import CpuExecutionProvider, create_cpu_provider
from .registry import ProviderRegistry


def create_gpu_provider(**kw):
    from .gpu import GpuExecutionProvider
    return GpuExecutionProvider(**kw)


def create_bitnet_provider(**kw):
    from .bitnet.provider import BitNetExecutionProvider
    return BitNetExecutionProvider(**kw)


def create_cpu_only_system() -> ProviderRegistry:
    reg = ProviderRegistry()
    reg.register_provider(create_cpu_provider())
    return reg


def create_provider_system() -> ProviderRegistry:
    """CPU always, GPU when a CUDA device exists, BitNet always (device kernels on a GPU box, the
    exact integer host kernels otherwise)."""
    reg = create_cpu_only_system()
    if torch.cuda.is_available():
        reg.register_provider(create_gpu_provider())
    reg.register_provider(create_bitnet_provider())
    return reg


def create_comprehensive_provider_system() -> ProviderRegistry:
    """Adds the WebAssembly-target provider and an NPU-style custom provider (host-emulated device) to the system."""
    from .custom.targets import NpuProvider, WasmProvider
    reg = create_provider_system()
    reg.register_provider(WasmProvider())
    reg.register_provider(NpuProvider())
    return reg


def create_custom_provider_registry(plugin_paths=None):
    """Registry of vendor plugins (``providers/custom/registry.py``)."""
    from .custom.registry import CustomProviderRegistry
    return CustomProviderRegistry(plugin_paths)
