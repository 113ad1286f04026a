"""GPU topology, placement strategies and device selection.

Data model of the reference (crates/ronn-providers/src/gpu/topology.rs:15-1209): ``GpuDeviceInfo``,
``InterconnectLink{link_type, bandwidth, latency, quality}``, ``Workload`` with a communication
pattern, three placement strategies returning a ``PlacementPlan``; and the per-sub-graph device
selectors of ``MultiGpuManager`` (crates/ronn-providers/src/gpu/provider.rs:77-366: round robin,
memory based, utilisation based, operation based, cost model with EMA execution-time stats).
Discovery here is real: devices, memory and peer access come from the CUDA runtime; on an NVSwitch
box every pair is an NVLink 5 link at 900 GB/s per direction.  Without GPUs an explicit description
can be supplied (used by the CPU tests).  Under tensor parallelism placement is static, so these
strategies only serve replica / sub-graph placement.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


class LinkType(enum.Enum):
    NVLINK = "nvlink"
    NVSWITCH = "nvswitch"
    PCIE = "pcie"
    SYSTEM_MEMORY = "system_memory"
    INFINITY_FABRIC = "infinity_fabric"


class CommunicationType(enum.Enum):
    P2P = "p2p"
    ALL_TO_ALL = "all_to_all"
    ALL_REDUCE = "all_reduce"
    BROADCAST = "broadcast"
    SCATTER = "scatter"
    GATHER = "gather"


@dataclass
class GpuDeviceInfo:
    device_id: int
    name: str
    total_memory: int
    free_memory: int
    compute_capability: Tuple[int, int]
    sm_count: int
    numa_node: int = 0
    utilization: float = 0.0
    power_watts: float = 0.0


@dataclass
class InterconnectLink:
    src: int
    dst: int
    link_type: LinkType
    bandwidth_gbps: float
    latency_us: float

    @property
    def quality(self) -> float:
        return self.bandwidth_gbps / max(self.latency_us, 1e-3)


@dataclass
class Workload:
    name: str = "workload"
    compute_flops: float = 0.0
    memory_bytes: int = 0
    communication: CommunicationType = CommunicationType.ALL_REDUCE
    bytes_exchanged: int = 0
    num_devices: int = 1
    fault_tolerance: bool = False


@dataclass
class PlacementPlan:
    device_ids: List[int]
    estimated_comm_time_us: float
    estimated_memory_per_device: int
    strategy: str


@dataclass
class TopologyConfig:
    nvlink_gbps: float = 900.0          # per direction per GPU through NVSwitch
    nvlink_latency_us: float = 1.0
    pcie_gbps: float = 64.0
    pcie_latency_us: float = 5.0
    cache_topology: bool = True


class GpuTopologyManager:
    def __init__(self, config: TopologyConfig = None, devices: Optional[List[GpuDeviceInfo]] = None,
                 peer_matrix: Optional[List[List[bool]]] = None):
        self.config = config or TopologyConfig()
        self.devices: List[GpuDeviceInfo] = devices if devices is not None else self._discover()
        self.links: Dict[Tuple[int, int], InterconnectLink] = {}
        self._build_links(peer_matrix)

    @staticmethod
    def _discover() -> List[GpuDeviceInfo]:
        out = []
        if not torch.cuda.is_available():
            return out
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            try:
                free, total = torch.cuda.mem_get_info(i)
            except Exception:
                free, total = p.total_memory, p.total_memory
            out.append(GpuDeviceInfo(i, p.name, total, free, (p.major, p.minor), p.multi_processor_count))
        return out

    def _build_links(self, peer_matrix) -> None:
        c = self.config
        n = len(self.devices)
        for a in range(n):
            for b in range(n):
                if a == b:
                    continue
                if peer_matrix is not None:
                    peer = peer_matrix[a][b]
                elif torch.cuda.is_available():
                    try:
                        peer = torch.cuda.can_device_access_peer(a, b)
                    except Exception:
                        peer = False
                else:
                    peer = False
                if peer:
                    self.links[(a, b)] = InterconnectLink(a, b, LinkType.NVSWITCH, c.nvlink_gbps, c.nvlink_latency_us)
                else:
                    self.links[(a, b)] = InterconnectLink(a, b, LinkType.PCIE, c.pcie_gbps, c.pcie_latency_us)

    def link(self, a: int, b: int) -> Optional[InterconnectLink]:
        return self.links.get((a, b))

    def device_count(self) -> int:
        return len(self.devices)

    def estimate_collective_us(self, kind: CommunicationType, nbytes: int, ids: List[int]) -> float:
        n = len(ids)
        if n <= 1 or nbytes == 0:
            return 0.0
        bw = min((self.links[(a, b)].bandwidth_gbps for a in ids for b in ids if a != b), default=1.0)
        lat = max((self.links[(a, b)].latency_us for a in ids for b in ids if a != b), default=0.0)
        factor = {CommunicationType.ALL_REDUCE: 2.0 * (n - 1) / n, CommunicationType.ALL_TO_ALL: (n - 1) / n,
                  CommunicationType.GATHER: (n - 1) / n, CommunicationType.SCATTER: (n - 1) / n,
                  CommunicationType.BROADCAST: 1.0, CommunicationType.P2P: 1.0}[kind]
        return lat + factor * nbytes / (bw * 1e3)

    # ---- placement strategies
    def place_locality_aware(self, w: Workload) -> PlacementPlan:
        ids = [d.device_id for d in self.devices]
        if not ids:
            raise RuntimeError("no devices to place on")
        chosen = [max(ids, key=lambda i: self.devices[i].free_memory)]
        while len(chosen) < min(w.num_devices, len(ids)):
            rest = [i for i in ids if i not in chosen]
            chosen.append(max(rest, key=lambda i: sum(self.links[(i, c)].quality for c in chosen)))
        return self._plan(w, chosen, "locality_aware")

    def place_bandwidth_optimized(self, w: Workload) -> PlacementPlan:
        ids = [d.device_id for d in self.devices]
        best = sorted(ids, key=lambda i: -sum(l.bandwidth_gbps for (a, _), l in self.links.items() if a == i))
        return self._plan(w, best[: max(1, min(w.num_devices, len(ids)))], "bandwidth_optimized")

    def place_power_efficient(self, w: Workload) -> PlacementPlan:
        ids = sorted((d.device_id for d in self.devices), key=lambda i: (self.devices[i].power_watts, self.devices[i].utilization))
        need = max(1, min(w.num_devices, len(ids)))
        per = w.memory_bytes // need if need else w.memory_bytes
        fit = [i for i in ids if self.devices[i].free_memory >= per]
        return self._plan(w, (fit or ids)[:need], "power_efficient")

    def _plan(self, w: Workload, ids: List[int], name: str) -> PlacementPlan:
        return PlacementPlan(ids, self.estimate_collective_us(w.communication, w.bytes_exchanged, ids),
                             w.memory_bytes // max(len(ids), 1), name)


class LoadBalancing(enum.Enum):
    ROUND_ROBIN = "round_robin"
    MEMORY_BASED = "memory_based"
    UTILIZATION_BASED = "utilization_based"
    OPERATION_BASED = "operation_based"
    COST_MODEL = "cost_model"


@dataclass
class DeviceStats:
    memory_used: int = 0
    utilization: float = 0.0
    avg_exec_ms: float = 0.0
    executions: int = 0


class MultiGpuManager:
    def __init__(self, device_ids: List[int], strategy: LoadBalancing = LoadBalancing.ROUND_ROBIN):
        if not device_ids:
            raise ValueError("at least one device is required")
        self.device_ids = list(device_ids)
        self.strategy = strategy
        self.stats: Dict[int, DeviceStats] = {d: DeviceStats() for d in device_ids}
        self._rr = 0

    def select_device(self, op_type: str = "", memory_bytes: int = 0) -> int:
        s = self.strategy
        if s == LoadBalancing.ROUND_ROBIN:
            d = self.device_ids[self._rr % len(self.device_ids)]
            self._rr += 1
            return d
        if s == LoadBalancing.MEMORY_BASED:
            return min(self.device_ids, key=lambda d: self.stats[d].memory_used)
        if s == LoadBalancing.UTILIZATION_BASED:
            return min(self.device_ids, key=lambda d: self.stats[d].utilization)
        if s == LoadBalancing.OPERATION_BASED:
            heavy = op_type in ("Conv", "MatMul", "Gemm", "Attention")
            key = (lambda d: self.stats[d].utilization) if heavy else (lambda d: self.stats[d].memory_used)
            return min(self.device_ids, key=key)
        return min(self.device_ids, key=lambda d: self.stats[d].memory_used / 2 ** 30 + 2.0 * self.stats[d].utilization
                   + self.stats[d].avg_exec_ms)

    def record_execution(self, device: int, ms: float, memory_bytes: int = 0, utilization: Optional[float] = None):
        st = self.stats[device]
        st.avg_exec_ms = ms if st.executions == 0 else 0.9 * st.avg_exec_ms + 0.1 * ms
        st.executions += 1
        st.memory_used += memory_bytes
        if utilization is not None:
            st.utilization = utilization
