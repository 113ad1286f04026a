"""Provider registry, allocators, CPU provider, kernel compiler, BitNet, topology (host-side logic)."""
import threading

import numpy as np
import pytest
import torch

from ronn_b200.api.errors import ProviderError
from ronn_b200.core.types import (DataType, OperatorSpec, PerformanceProfile, ProviderCapability, ProviderConfig,
                                  ProviderType, MemoryType)
from ronn_b200.graph.ir import GraphBuilder
from ronn_b200.providers import create_comprehensive_provider_system, create_cpu_only_system, create_provider_system
from ronn_b200.providers.allocator import (AlignedMemoryAllocator, BitNetAllocator, MemoryPool, PoolConfig,
                                           PooledMemoryAllocator, SystemMemoryAllocator, calculate_tensor_size)
from ronn_b200.providers.base import ExecutionProvider
from ronn_b200.providers.compiler import FusionType, KernelCompiler
from ronn_b200.providers.cpu import CpuExecutionProvider
from ronn_b200.providers.registry import ProviderRegistry


class MockProvider(ExecutionProvider):
    def __init__(self, pid, ops, profile):
        self.provider_id, self.ops, self.profile, self.down = pid, set(ops), profile, False
        self.name = f"Mock{pid.name}"

    def get_capability(self):
        return ProviderCapability(self.ops, [DataType.F32], [MemoryType.SYSTEM], self.profile)

    def compile_graph(self, graph, profiler=None):
        return "kernel-" + self.provider_id.name

    def compile_subgraph(self, sg, initializers=None):
        return "kernel-" + self.provider_id.name

    def shutdown(self):
        self.down = True


def specs(*ops):
    return [OperatorSpec(o) for o in ops]


def test_registry_selection_and_fallback():
    reg = ProviderRegistry()
    cpu = MockProvider(ProviderType.CPU, ["Add", "MatMul", "Relu"], PerformanceProfile.CPU)
    gpu = MockProvider(ProviderType.GPU, ["MatMul", "Conv"], PerformanceProfile.GPU)
    reg.register_provider(cpu)
    reg.register_provider(gpu)
    assert reg.get_preference_order() == [ProviderType.GPU, ProviderType.CPU]
    with pytest.raises(ProviderError, match="already registered"):
        reg.register_provider(MockProvider(ProviderType.CPU, [], PerformanceProfile.CPU))
    assert reg.select_provider(specs("MatMul")) == ProviderType.GPU
    assert reg.select_provider(specs("MatMul", "Add")) == ProviderType.CPU
    assert reg.select_provider(specs("MatMul", "Softmax")) is None
    chain = reg.get_fallback_chain(specs("Conv", "Add", "Softmax"))
    assert [p for _, p in chain] == [ProviderType.GPU, ProviderType.CPU, None]
    reg.set_preference_order([ProviderType.CPU])
    assert reg.select_provider(specs("MatMul")) == ProviderType.CPU
    with pytest.raises(ProviderError):
        reg.set_preference_order([ProviderType.BITNET])
    with pytest.raises(ProviderError):
        reg.unregister_provider(ProviderType.WASM)
    sg = GraphBuilder().add_op("MatMul", ["a", "b"], ["c"]).graph.extract_subgraph([0])
    assert reg.compile_subgraph(sg) == (ProviderType.CPU, "kernel-CPU")
    assert reg.get_statistics().provider_count == 2
    reg.shutdown()
    assert reg.provider_count() == 0 and cpu.down and gpu.down


def test_registry_thread_safety():
    reg = create_cpu_only_system()
    errs = []

    def q():
        try:
            for _ in range(200):
                reg.select_provider(specs("Add", "Relu"))
                reg.get_fallback_chain(specs("Conv"))
        except Exception as e:
            errs.append(e)
    ts = [threading.Thread(target=q) for _ in range(8)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errs


def test_provider_systems():
    reg = create_provider_system()
    ids = reg.get_provider_ids()
    assert ProviderType.CPU in ids and ProviderType.BITNET in ids
    assert (ProviderType.GPU in ids) == torch.cuda.is_available()
    full = create_comprehensive_provider_system()
    wasm = full.get_provider(ProviderType.WASM)
    assert wasm is not None and wasm.can_handle(specs("Add", "LSTM")) == [True, False]
    assert full.get_provider(ProviderType.CUSTOM).name == "NpuProvider"
    from ronn_b200.providers.custom.targets import NpuConfig, NpuProvider, TpuConfig, TpuProvider
    assert NpuProvider().config.device_id == "npu0" and TpuProvider().config.core_count == 8
    assert "AllReduce" in TpuProvider().ops


def test_allocators():
    for alloc in (SystemMemoryAllocator(), AlignedMemoryAllocator(64), PooledMemoryAllocator(), MemoryPool()):
        with pytest.raises(ProviderError, match="zero"):
            alloc.allocate([0], DataType.F32)
        base = alloc.stats().allocated_bytes
        b = alloc.allocate([10, 10], DataType.F32)
        assert b.size == 400 and b.ptr % 16 == 0
        alloc.as_numpy(b, np.float32)[:] = 3.0
        alloc.deallocate(b)
        assert alloc.stats().allocated_bytes == base
        with pytest.raises(ProviderError):
            alloc.deallocate(b)                                            # double free is reported, not fatal
    a = AlignedMemoryAllocator(64)
    assert all(a.allocate([n], DataType.I8).ptr % 64 == 0 for n in (1, 7, 100, 4097))
    with pytest.raises(ProviderError):
        AlignedMemoryAllocator(48)
    p = PooledMemoryAllocator(PoolConfig(max_buffers_per_bucket=2, max_pool_size=1 << 20, bucket_granularity=64))
    assert p.bucket_size(100) == 128
    bufs = [p.allocate([100], DataType.U8) for _ in range(4)]
    for b in bufs:
        p.deallocate(b)
    st = p.stats()
    assert st.pooled_buffers == 2 and st.misses == 4
    again = p.allocate([120], DataType.U8)
    assert p.stats().hits == 1 and 0 < p.hit_rate() < 1
    p.deallocate(again)
    p.clear_pools()
    assert p.stats().pooled_buffers == 0
    mp = MemoryPool()
    assert mp.bucket_size(1000) == 1024 and mp.bucket_size(64) == 64
    assert calculate_tensor_size([2, 3], DataType.BF16) == 12
    assert BitNetAllocator.packed_size([1000], DataType.BOOL) == 125 and BitNetAllocator.packed_size([1000], DataType.U8) == 250
    # concurrent use
    errs = []

    def work():
        try:
            for _ in range(200):
                b = p.allocate([256], DataType.F32)
                p.deallocate(b)
        except Exception as e:
            errs.append(e)
    ts = [threading.Thread(target=work) for _ in range(8)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errs and p.stats().allocated_bytes == 0


def test_cpu_provider_config_and_kernels():
    p = CpuExecutionProvider(thread_count=3, numa_node=0)
    cap = p.get_capability()
    assert cap.performance_profile == PerformanceProfile.CPU and "MatMul" in cap.supported_ops
    assert cap.features["threads"] == 3 and DataType.F32 in cap.data_types
    p.configure(ProviderConfig(thread_count=5, custom_options={"enable_simd": "false", "numa_node": "1"}))
    assert p.thread_count == 5 and p.simd_features == [] and p.numa_node == 1
    with pytest.raises(ProviderError):
        p.configure(ProviderConfig(custom_options={"numa_node": "abc"}))
    with pytest.raises(ProviderError):
        p.configure(ProviderConfig(thread_count=-2))
    g = GraphBuilder().add_input("a", [4]).add_input("b", [4]).add_output("c", [4])
    g.add_op("Add", ["a", "b"], ["c"])
    k = p.compile_graph(g.build())
    out = k.execute({"a": torch.ones(4), "b": torch.ones(4)})
    assert out["c"].tolist() == [2.0] * 4 and k.get_performance_stats().execution_count == 1
    sg = GraphBuilder().add_op("NoSuchOp", ["a"], ["b"]).graph.extract_subgraph([0])
    with pytest.raises(ProviderError, match="does not support"):
        p.compile_subgraph(sg)
    with pytest.raises(ProviderError, match="empty"):
        from ronn_b200.graph.ir import SubGraph
        p.compile_subgraph(SubGraph([], [], [], []))


def test_native_simd_kernels_match_torch():
    from ronn_b200 import _native
    lib = _native.host()
    a, b = torch.randn(1000), torch.randn(1000)
    for lvl in (0, 1, 2):
        lib.ronn_cpu_force_level(lvl)
        assert abs(lib.ronn_cpu_dot_f32(a.data_ptr(), b.data_ptr(), 1000) - float(a @ b)) < 1e-2
        o = torch.empty(1000)
        lib.ronn_cpu_binary_f32(a.data_ptr(), b.data_ptr(), o.data_ptr(), 1000, 0, 1)
        torch.testing.assert_close(o, torch.relu(a + b))
        for (M, N, K) in ((1, 128, 784), (5, 10, 128), (7, 37, 19)):
            A, B, bias = torch.randn(M, K), torch.randn(K, N), torch.randn(N)
            C = torch.empty(M, N)
            lib.ronn_cpu_gemm_f32(A.data_ptr(), B.data_ptr(), bias.data_ptr(), C.data_ptr(), M, N, K, 1)
            torch.testing.assert_close(C, torch.relu(A @ B + bias), atol=1e-3, rtol=1e-4)
    lib.ronn_cpu_force_level(-1)
    x = torch.randn(4, 33)
    y = torch.empty_like(x)
    lib.ronn_cpu_softmax_f32(x.data_ptr(), y.data_ptr(), 4, 33)
    torch.testing.assert_close(y, torch.softmax(x, -1))


def test_kernel_compiler_groups_and_memory_plan():
    b = GraphBuilder().add_input("x", [1, 3, 8, 8]).add_output("o", [1, 4, 8, 8])
    for n in ("w", "g", "be", "m", "v", "w2", "bias"):
        b.add_initializer(n, torch.zeros(1))
    b.add_op("Conv", ["x", "w"], ["c"]).add_op("BatchNormalization", ["c", "g", "be", "m", "v"], ["bn"]).add_op("Relu", ["bn"], ["r"])
    b.add_op("MatMul", ["r", "w2"], ["mm"]).add_op("Add", ["mm", "bias"], ["a"]).add_op("Softmax", ["a"], ["o"])
    plan = KernelCompiler.performance_preset().analyze(b.build(validate=False))
    kinds = [g.fusion_type for g in plan.groups]
    assert kinds == [FusionType.CONV_BN_RELU, FusionType.MATMUL_BIAS, FusionType.NONE]
    assert plan.groups[0].op_types == ["Conv", "BatchNormalization", "Relu"]
    assert plan.total_cost < 105 + 51 + 8 and plan.buffers < 6 and plan.peak_bytes > 0
    mem = KernelCompiler.memory_preset()
    assert mem.fusion.max_fusion_depth == 3 and not mem.can_fuse("Conv", "BatchNormalization")


def test_topology_and_placement_on_described_box():
    from ronn_b200.parallel.topology import (CommunicationType, GpuDeviceInfo, GpuTopologyManager, LinkType,
                                             LoadBalancing, MultiGpuManager, Workload)
    devs = [GpuDeviceInfo(i, "B200", 180 << 30, (180 - 10 * i) << 30, (10, 0), 148) for i in range(8)]
    peers = [[a != b for b in range(8)] for a in range(8)]
    topo = GpuTopologyManager(devices=devs, peer_matrix=peers)
    assert topo.link(0, 7).link_type == LinkType.NVSWITCH and topo.link(0, 7).bandwidth_gbps == 900.0
    w = Workload(num_devices=4, memory_bytes=40 << 30, bytes_exchanged=1 << 20, communication=CommunicationType.ALL_REDUCE)
    plan = topo.place_locality_aware(w)
    assert len(plan.device_ids) == 4 and plan.device_ids[0] == 0 and plan.estimated_comm_time_us > 1.0
    assert len(topo.place_bandwidth_optimized(w).device_ids) == 4 and len(topo.place_power_efficient(w).device_ids) == 4
    mgr = MultiGpuManager([0, 1, 2], LoadBalancing.ROUND_ROBIN)
    assert [mgr.select_device() for _ in range(4)] == [0, 1, 2, 0]
    mgr.strategy = LoadBalancing.MEMORY_BASED
    mgr.record_execution(0, 1.0, memory_bytes=1 << 30)
    assert mgr.select_device() == 1
    mgr.strategy = LoadBalancing.COST_MODEL
    mgr.record_execution(1, 50.0)
    assert mgr.select_device() == 2
    from ronn_b200.parallel.memory_manager import MultiGpuMemoryManager, P2PConnectivityMatrix
    mm = MultiGpuMemoryManager([0, 1], connectivity=P2PConnectivityMatrix(2, [[False, True], [True, False]]))
    if not torch.cuda.is_available():
        t = mm.allocate(0, [4, 4])
        moved = mm.transfer_between_devices(t, 0, 1)
        assert moved.shape == t.shape and mm.events[-1].nbytes == 64 and mm.global_stats()["transfers"] == 1
        with pytest.raises(ProviderError):
            mm.allocate(0, [0])
