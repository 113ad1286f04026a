"""Custom-hardware providers: run one model on the CPU provider, on the example NPU and TPU providers (host-emulated
devices behind the CustomHardwareProvider contracts) and on the WASM-style provider, and compare.

    python examples/custom_hardware.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ronn_b200 import Model, SessionOptions  # noqa: E402
from ronn_b200.graph.ir import GraphBuilder  # noqa: E402
from ronn_b200.providers.custom.targets import NpuConfig, NpuProvider, TpuProvider, WasmProvider  # noqa: E402


def build_mlp(seed=0):
    g = torch.Generator().manual_seed(seed)
    b = GraphBuilder().add_input("x", [4, 64]).add_output("y", [4, 10])
    b.add_initializer("w1", torch.randn(64, 128, generator=g) * 0.2).add_initializer("b1", torch.randn(128, generator=g) * 0.1)
    b.add_initializer("w2", torch.randn(128, 10, generator=g) * 0.2)
    b.add_op("MatMul", ["x", "w1"], ["h0"]).add_op("Add", ["h0", "b1"], ["h1"]).add_op("Relu", ["h1"], ["h2"])
    b.add_op("MatMul", ["h2", "w2"], ["h3"]).add_op("Softmax", ["h3"], ["y"], axis=-1)
    return b.build()


def main():
    model = Model.from_graph(build_mlp())
    x = torch.randn(4, 64)
    want = model.create_session(SessionOptions().with_provider("cpu")).run({"x": x})["y"]
    for name, provider in (("npu (int8 weights)", NpuProvider(NpuConfig(memory_pool_size=1 << 20))),
                           ("npu (fp32)", NpuProvider(NpuConfig(memory_pool_size=1 << 20, enable_quantization=False))),
                           ("tpu (bf16)", TpuProvider()), ("wasm", WasmProvider())):
        sess = model.create_session(SessionOptions().with_provider(provider))
        got = sess.run({"x": x})["y"]
        hw = getattr(provider, "provider", None)
        mem = hw.get_device_memory().get_memory_info().allocated_bytes if hw is not None else 0
        print(f"{name:20s} max |diff| vs cpu = {float((got - want).abs().max()):.2e}   device memory in use = {mem} bytes")
        provider.shutdown()


if __name__ == "__main__":
    main()
