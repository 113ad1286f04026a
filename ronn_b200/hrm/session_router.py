"""Wires the HRM router into a session: System 1 = the same model on the BitNet provider, System 2 =
the session's own (full-precision) kernel.  The reference documents ``enable_hrm=True`` and a
``ComplexityRouter`` in its README (README.md:105-106,192-205, crates/ronn-python/README.md:46-60) but
never connects the module to the API."""
from __future__ import annotations

from typing import Dict

import torch

from ..core.types import ProviderType
from .module import HierarchicalReasoningModule
from .router import RoutingStrategy


class SessionRouter:
    def __init__(self, session, strategy: RoutingStrategy = RoutingStrategy.ADAPTIVE_HYBRID):
        from ..api.session import SessionBuilder
        self.session = session
        fast_opts = session.options().with_provider(ProviderType.BITNET).with_hrm(False)
        self.fast = SessionBuilder(session._model).with_options(fast_opts).build()
        self.hrm = HierarchicalReasoningModule(strategy, system1=self._run_fast, system2=self._run_precise)
        self.last = None

    def _run_fast(self, feed):
        dev = self.fast._kernel.device
        return self.fast._kernel.execute({k: v.to(dev) for k, v in feed.items()})

    def _run_precise(self, feed):
        return self.session._kernel.execute(feed)

    def run(self, feed: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        probe = next((v for v in feed.values() if v.is_floating_point()), next(iter(feed.values())))
        res = self.hrm.process(probe, payload=feed)
        self.last = res
        dev = self.session._kernel.device
        return {k: v.to(dev) for k, v in res.output.items()}


def attach_router(session, strategy: RoutingStrategy = RoutingStrategy.ADAPTIVE_HYBRID) -> SessionRouter:
    r = SessionRouter(session, strategy)
    session._router = r
    return r
