"""System topology sensors: CPU / NUMA / memory from the OS, GPU properties from the CUDA runtime (through
PyTorch) and NVML when present, folded into the constraints the planners read.

Reference parity: ``SystemTopology{cpu, numa, gpu, constraints}`` (src/sensors/mod.rs:20-272),
``MemoryNetworkSensors`` (:94), ``GpuTopology`` / ``GpuPlatform`` (src/sensors/gpu.rs:24-107),
``CompilerConstraints{simd_width_bits, l2_cache_size, TileBits, GpuSmPartition}`` (src/jit/compiler_constraints.rs);
memory pressure readers (src/compat/memory.rs:8-172). Nothing here changes a device setting: all reads.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class CpuTopology:
    logical_cores: int = 1
    model: str = ""
    flags: List[str] = field(default_factory=list)

    @property
    def simd_width_bits(self) -> int:
        f = set(self.flags)
        return 512 if "avx512f" in f else 256 if "avx2" in f else 128


@dataclass
class NumaTopology:
    nodes: int = 1
    cpus_per_node: Dict[int, List[int]] = field(default_factory=dict)


@dataclass
class GpuInfo:
    present: bool = False
    name: str = ""
    count: int = 0
    sm_count: int = 0
    cc_major: int = 0
    cc_minor: int = 0
    total_memory: int = 0
    l2_bytes: int = 0
    nvlink_peers: List[int] = field(default_factory=list)

    @property
    def is_blackwell(self) -> bool:
        return self.cc_major == 10


@dataclass
class SmPartition:
    compute_sms: int
    comm_sms: int


@dataclass
class PlannerConstraints:
    simd_width_bits: int
    l2_cache_size: int
    tile_m: int
    tile_n: int
    sm_partition: SmPartition


@dataclass
class SystemTopology:
    cpu: CpuTopology
    numa: NumaTopology
    gpu: GpuInfo
    constraints: PlannerConstraints


def read_meminfo(path: str = "/proc/meminfo") -> Dict[str, int]:
    out = {}
    try:
        with open(path) as f:
            for line in f:
                k, _, rest = line.partition(":")
                parts = rest.split()
                if parts:
                    out[k.strip()] = int(parts[0]) * (1024 if len(parts) > 1 and parts[1] == "kB" else 1)
    except OSError:
        pass
    return out


def host_memory_pressure(meminfo: Optional[Dict[str, int]] = None) -> float:
    m = meminfo if meminfo is not None else read_meminfo()
    total, avail = m.get("MemTotal", 0), m.get("MemAvailable", m.get("MemFree", 0))
    return 0.0 if total == 0 else 1.0 - avail / total


def probe_cpu(cpuinfo_path: str = "/proc/cpuinfo") -> CpuTopology:
    t = CpuTopology(logical_cores=os.cpu_count() or 1)
    try:
        with open(cpuinfo_path) as f:
            for line in f:
                if line.startswith("model name") and not t.model:
                    t.model = line.split(":", 1)[1].strip()
                elif line.startswith("flags") and not t.flags:
                    t.flags = line.split(":", 1)[1].split()
    except OSError:
        pass
    return t


def probe_numa(root: str = "/sys/devices/system/node") -> NumaTopology:
    n = NumaTopology()
    try:
        nodes = sorted(d for d in os.listdir(root) if d.startswith("node") and d[4:].isdigit())
        n.nodes = max(1, len(nodes))
        for d in nodes:
            try:
                with open(os.path.join(root, d, "cpulist")) as f:
                    cpus = []
                    for part in f.read().strip().split(","):
                        a, _, b = part.partition("-")
                        cpus.extend(range(int(a), int(b or a) + 1))
                    n.cpus_per_node[int(d[4:])] = cpus
            except (OSError, ValueError):
                pass
    except OSError:
        pass
    return n


def probe_gpu() -> GpuInfo:
    import torch
    g = GpuInfo()
    if not torch.cuda.is_available():
        return g
    p = torch.cuda.get_device_properties(0)
    g.present, g.name, g.count = True, p.name, torch.cuda.device_count()
    g.sm_count, g.cc_major, g.cc_minor, g.total_memory = p.multi_processor_count, p.major, p.minor, p.total_memory
    g.l2_bytes = getattr(p, "L2_cache_size", 0)
    for peer in range(1, g.count):
        try:
            if torch.cuda.can_device_access_peer(0, peer):
                g.nvlink_peers.append(peer)
        except Exception:
            pass
    return g


def derive_constraints(cpu: CpuTopology, gpu: GpuInfo, comm_sm_ratio: float = 0.0) -> PlannerConstraints:
    sms = gpu.sm_count or 1
    comm = int(round(sms * comm_sm_ratio))
    tile_m, tile_n = (128, 256) if gpu.is_blackwell else (128, 128)
    return PlannerConstraints(cpu.simd_width_bits, gpu.l2_bytes or (32 << 20), tile_m, tile_n, SmPartition(sms - comm, comm))


def probe_system(comm_sm_ratio: float = 0.0) -> SystemTopology:
    cpu, numa, gpu = probe_cpu(), probe_numa(), probe_gpu()
    return SystemTopology(cpu, numa, gpu, derive_constraints(cpu, gpu, comm_sm_ratio))
