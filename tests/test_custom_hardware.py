"""Custom-hardware plugin layer on CPU: contracts, the host-emulated device, the plugin registry, and the NPU / TPU /
WebAssembly-target providers built on them (reference behaviour: crates/ronn-providers/src/custom/traits.rs:14-330,
custom/registry.rs:18-410, wasm/allocator.rs:15-247)."""
import json
import textwrap

import pytest
import torch

from ronn_b200 import Model, SessionOptions
from ronn_b200.api.errors import ProviderError
from ronn_b200.core.types import ProviderType
from ronn_b200.graph.ir import GraphBuilder
from ronn_b200.providers.custom.host_device import (ArenaMemory, HostEmulatedProvider, StaticDiscovery, npu_capability,
                                                    tpu_capability)
from ronn_b200.providers.custom.interface import (ABI_VERSION, CompilationOptions, CustomProviderAdapter, DeviceStatus,
                                                  HardwareDevice, PluginMetadata, WallClockProfiler)
from ronn_b200.providers.custom.registry import CustomProviderRegistry
from ronn_b200.providers.custom.targets import (NpuConfig, NpuProvider, TpuProvider, WasmMemory, WasmModelCache,
                                                WasmProvider, WasmProviderConfig, WASM_PAGE)


def mlp_graph(seed=0):
    g = torch.Generator().manual_seed(seed)
    b = GraphBuilder().add_input("x", [2, 16]).add_output("y", [2, 4])
    b.add_initializer("w1", torch.randn(16, 32, generator=g) * 0.3).add_initializer("b1", torch.randn(32, generator=g) * 0.1)
    b.add_initializer("w2", torch.randn(32, 4, generator=g) * 0.3)
    b.add_op("MatMul", ["x", "w1"], ["h0"]).add_op("Add", ["h0", "b1"], ["h1"]).add_op("Relu", ["h1"], ["h2"])
    b.add_op("MatMul", ["h2", "w2"], ["h3"]).add_op("Softmax", ["h3"], ["y"], axis=-1)
    return b.build()


def test_arena_memory_alignment_limits_and_bounds():
    m = ArenaMemory(1 << 20, device_id=3)
    a = m.allocate(1000, 256)
    b = m.allocate(10, 64)
    assert a.handle % 256 == 0 and b.handle % 64 == 0 and a.device_id == 3
    m.copy_to_device(b"abcdef", b)
    assert m.copy_from_device(b, 6) == b"abcdef"
    with pytest.raises(ProviderError, match="exceeds"):
        m.copy_to_device(b"x" * 11, b)
    with pytest.raises(ProviderError, match="power of two"):
        m.allocate(8, 48)
    with pytest.raises(ProviderError, match="out of device memory"):
        m.allocate(2 << 20)
    info = m.get_memory_info()
    assert info.allocated_bytes == 1010 and info.total_bytes == 1 << 20
    m.deallocate(a)
    with pytest.raises(ProviderError, match="not allocated"):
        m.deallocate(a)
    big = m.allocate((1 << 20) - 4096, 64)          # freed space coalesces: nearly the whole arena fits again
    m.deallocate(big)
    m.deallocate(b)
    assert m.get_memory_info().allocated_bytes == 0 and m.peak >= 1010
    other = ArenaMemory(1 << 10, device_id=4)
    assert not m.can_access(m.allocate(8), other.allocate(8))


def test_host_emulated_provider_compiles_and_runs_with_its_numeric_personality():
    graph = mlp_graph()
    x = torch.randn(2, 16)
    ref = Model.from_graph(graph).create_session(SessionOptions().with_provider("cpu")).run({"x": x})["y"]
    for prov, tol in ((NpuProvider(NpuConfig(memory_pool_size=1 << 20)), 3e-2), (TpuProvider(), 3e-2),
                      (NpuProvider(NpuConfig(memory_pool_size=1 << 20, enable_quantization=False)), 1e-6)):
        kern = prov.compile_graph(graph)
        out = kern.execute({"x": x})["y"]
        torch.testing.assert_close(out, ref, atol=tol, rtol=tol)
        hw = prov.provider
        assert hw.get_performance_stats().total_operations == 1
        assert hw.get_device_memory().get_memory_info().allocated_bytes > 0
        info = kern.kernel.get_kernel_info()
        assert info.operations == ["MatMul", "Add", "Relu", "MatMul", "Softmax"] and info.estimated_memory_bytes > 0
        assert hw.profiler.get_profiling_summary().total_operations == 1
        prov.shutdown()
        assert hw.get_device_memory().get_memory_info().allocated_bytes == 0
    # int8 weights take a quarter of the fp32 bytes on the device
    q, f = NpuProvider(NpuConfig(memory_pool_size=1 << 20)), NpuProvider(NpuConfig(memory_pool_size=1 << 20, enable_quantization=False))
    q.compile_graph(graph), f.compile_graph(graph)
    assert q.provider.memory.get_memory_info().allocated_bytes < f.provider.memory.get_memory_info().allocated_bytes / 2
    # a model that does not fit the device is refused and leaves nothing allocated
    tiny = NpuProvider(NpuConfig(memory_pool_size=256))
    with pytest.raises(ProviderError, match="out of device memory"):
        tiny.compile_graph(graph)
    assert tiny.provider.memory.get_memory_info().allocated_bytes == 0
    # unsupported operators are named
    b = GraphBuilder().add_input("x", [1, 4]).add_output("y", [1, 4])
    b.add_op("LSTM", ["x"], ["y"])
    with pytest.raises(ProviderError, match="LSTM"):
        NpuProvider().compile_graph(b.build())


def test_session_runs_on_a_custom_provider_instance():
    graph = mlp_graph(1)
    x = torch.randn(2, 16)
    model = Model.from_graph(graph)
    ref = model.create_session(SessionOptions().with_provider("cpu")).run({"x": x})["y"]
    tpu = TpuProvider()
    out = model.create_session(SessionOptions().with_provider(tpu)).run({"x": x})["y"]
    assert out.dtype == torch.float32
    torch.testing.assert_close(out, ref, atol=3e-2, rtol=3e-2)


PLUGIN_SRC = '''
from ronn_b200.providers.custom.host_device import HostEmulatedProvider, npu_capability
from ronn_b200.providers.custom.interface import PluginMetadata, ProviderPlugin

class Plugin(ProviderPlugin):
    def get_metadata(self):
        return PluginMetadata(name="{name}", version="1.2.3", author="vendor", supported_hardware=["mock-npu"],
                              min_ronn_version="{minver}")
    def create_provider(self, config=None):
        return HostEmulatedProvider("{name}", npu_capability(1 << 20), (config or {{}}).get("memory", 1 << 20))
    def is_hardware_available(self):
        return {available}
    def get_abi_version(self):
        return {abi}

def ronn_plugin():
    return Plugin()
'''


def _write_plugin(d, fname, **kw):
    args = dict(name=fname, minver="0.1.0", available=True, abi=ABI_VERSION)
    args.update(kw)
    (d / f"{fname}.py").write_text(textwrap.dedent(PLUGIN_SRC.format(**args)))
    return str(d / f"{fname}.py")


def test_plugin_registry_discovers_validates_loads_and_shuts_down(tmp_path):
    good = _write_plugin(tmp_path, "mocknpu")
    _write_plugin(tmp_path, "oldabi", abi=ABI_VERSION + 1)
    _write_plugin(tmp_path, "toonew", minver="99.0.0")
    _write_plugin(tmp_path, "nohw", available=False)
    (tmp_path / "broken.py").write_text("raise RuntimeError('driver missing')\n")
    (tmp_path / "mocknpu.plugin.json").write_text(json.dumps({"description": "from the side file", "license": "MIT"}))
    reg = CustomProviderRegistry([str(tmp_path)])
    found = {m.name: m for m in reg.discover_plugins()}
    assert found["mocknpu"].status == "loaded" and found["mocknpu"].description == "from the side file"
    assert found["oldabi"].status == "incompatible" and found["toonew"].status == "incompatible"
    assert found["nohw"].status == "disabled" and found["broken"].status.startswith("load_error:")
    st = reg.get_statistics()
    assert (st.total_plugins, st.loaded_plugins, st.failed_plugins, st.total_providers) == (5, 1, 3, 0)
    name = reg.load_plugin_from_file(good, {"memory": 1 << 19})
    assert name == "mocknpu" and reg.list_providers() == ["mocknpu"]
    assert reg.get_provider("mocknpu").get_device_memory().get_memory_info().total_bytes == 1 << 19
    with pytest.raises(ProviderError, match="already registered"):
        reg.load_plugin_from_file(good)
    with pytest.raises(ProviderError, match="ABI version"):
        reg.load_plugin_from_file(str(tmp_path / "oldabi.py"))
    with pytest.raises(ProviderError, match="not available"):
        reg.load_plugin_from_file(str(tmp_path / "nohw.py"))
    # the registered provider runs a session
    graph = mlp_graph(2)
    x = torch.randn(2, 16)
    ep = reg.as_execution_provider("mocknpu")
    assert ep.provider_id == ProviderType.CUSTOM
    out = Model.from_graph(graph).create_session(SessionOptions().with_provider(ep)).run({"x": x})["y"]
    ref = Model.from_graph(graph).create_session(SessionOptions().with_provider("cpu")).run({"x": x})["y"]
    torch.testing.assert_close(out, ref, atol=1e-5, rtol=1e-5)
    reg.unregister_provider("mocknpu")
    with pytest.raises(ProviderError, match="not registered"):
        reg.unregister_provider("mocknpu")
    reg.register_provider("again", HostEmulatedProvider("again", tpu_capability(1 << 20), 1 << 20))
    reg.shutdown()
    assert reg.list_providers() == []


def test_hardware_discovery_and_profiler():
    dev = HardwareDevice("npu0", "mock", "vendor", "npu", npu_capability(1 << 20))
    disc = StaticDiscovery([dev])
    reg = CustomProviderRegistry(discovery=disc)
    assert [d.device_id for d in reg.discover_hardware()] == ["npu0"] and disc.is_device_available("npu0")
    disc.set_status("npu0", DeviceStatus.ERROR, "overheated")
    assert not disc.is_device_available("npu0") and disc.get_device_info("npu0").error == "overheated"
    assert disc.get_device_info("npu9") is None and CustomProviderRegistry().discover_hardware() == []
    prof = WallClockProfiler(power_watts=10.0)
    s = prof.start_profiling("matmul")
    r = prof.stop_profiling(s, memory_usage_bytes=4096, hardware_utilization=0.5, cache_hits=3)
    assert r.operation_name == "matmul" and r.execution_time_us >= 0 and r.custom_metrics == {"cache_hits": 3.0}
    with pytest.raises(ProviderError, match="not open"):
        prof.stop_profiling(s)
    summ = prof.get_profiling_summary()
    assert summ.total_operations == 1 and summ.peak_memory_bytes == 4096 and summ.top_operations_by_time[0][0] == "matmul"
    prof.reset_profiling()
    assert prof.get_profiling_summary().total_operations == 0


def test_wasm_linear_memory_grows_in_pages_up_to_its_limit():
    m = WasmMemory(limit_bytes=4 * WASM_PAGE, initial_pages=1)
    a = m.allocate(100)
    assert a % 16 == 0 and m.stats()["pages"] == 1
    b = m.allocate(WASM_PAGE)                        # does not fit the first page: memory grows
    assert m.stats()["pages"] >= 2 and m.stats()["grow_count"] >= 1
    with pytest.raises(ProviderError, match="memory limit"):
        m.allocate(4 * WASM_PAGE)
    m.free(a)
    m.free(b)
    with pytest.raises(ProviderError, match="not allocated"):
        m.free(b)
    assert m.stats()["allocated_bytes"] == 0
    c = m.allocate(2 * WASM_PAGE)                    # freed ranges coalesced
    assert m.stats()["allocated_bytes"] == 2 * WASM_PAGE and c % 16 == 0


def test_wasm_model_cache_lru_size_and_expiry():
    now = [0.0]
    c = WasmModelCache(max_bytes=100, expiry_hours=1.0, clock=lambda: now[0])
    assert c.put("a", "A", 40) and c.put("b", "B", 40)
    assert c.get("a") == "A"                          # a is now the most recently used
    assert c.put("c", "C", 40)                        # evicts b
    assert c.get("b") is None and c.get("a") == "A" and c.get("c") == "C" and c.evictions == 1
    assert not c.put("huge", "H", 101)
    now[0] = 3601.0
    assert c.get("a") is None and len(c) == 1        # expired entries disappear when they are looked up
    assert c.hits == 3 and c.misses == 2


def test_wasm_provider_runs_graphs_within_its_operator_set_and_memory_limit():
    graph = mlp_graph(3)
    x = torch.randn(2, 16)
    ref = Model.from_graph(graph).create_session(SessionOptions().with_provider("cpu")).run({"x": x})["y"]
    p = WasmProvider()
    k1 = p.compile_graph(graph)
    torch.testing.assert_close(k1.execute({"x": x})["y"], ref, atol=1e-6, rtol=1e-6)
    assert p.memory.stats()["allocated_bytes"] >= (16 * 32 + 32 + 32 * 4) * 4
    assert p.compile_graph(graph) is k1 and p.model_cache.hits == 1          # same graph: served from the model cache
    p.release(k1)
    assert p.memory.stats()["allocated_bytes"] == 0
    small = WasmProvider(WasmProviderConfig(memory_limit_bytes=WASM_PAGE // 64))
    b = GraphBuilder().add_input("x", [1, 512]).add_output("y", [1, 512])
    b.add_initializer("w", torch.randn(512, 512))
    b.add_op("MatMul", ["x", "w"], ["y"])
    with pytest.raises(ProviderError, match="memory limit"):
        small.compile_graph(b.build())
    b2 = GraphBuilder().add_input("x", [1, 4]).add_output("y", [1, 4])
    b2.add_op("Erf", ["x"], ["y"])
    with pytest.raises(ProviderError, match="Erf"):
        p.compile_graph(b2.build())
