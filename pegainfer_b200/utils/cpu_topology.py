"""NUMA-aware CPU placement for per-GPU worker processes.

Reads the GPU's NUMA node from sysfs and pins the calling process to that node's CPUs
(split evenly between the ranks that share the node), so pinned-memory staging and
launch threads stay local to their GPU.

Reference parity: pegainfer-core/src/cpu_topology.rs:13-329,
pegainfer-kimi-k2/src/runner/affinity.rs.
"""
from __future__ import annotations

import os
from typing import Optional


def parse_cpulist(text: str) -> list:
    out = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            out.extend(range(int(a), int(b) + 1))
        else:
            out.append(int(part))
    return out


def gpu_numa_node(pci_bus_id: str, sys_root: str = "/sys") -> Optional[int]:
    p = os.path.join(sys_root, "bus/pci/devices", pci_bus_id.lower(), "numa_node")
    try:
        with open(p) as f:
            n = int(f.read().strip())
        return n if n >= 0 else None
    except (OSError, ValueError):
        return None


def node_cpus(node: int, sys_root: str = "/sys") -> list:
    try:
        with open(os.path.join(sys_root, f"devices/system/node/node{node}/cpulist")) as f:
            return parse_cpulist(f.read())
    except OSError:
        return []


def plan_affinity(cpus: list, local_rank_on_node: int, ranks_on_node: int) -> list:
    """Even contiguous split of a node's CPUs between the ranks living on it."""
    if not cpus or ranks_on_node <= 0:
        return []
    per = max(1, len(cpus) // ranks_on_node)
    lo = min(local_rank_on_node * per, len(cpus) - per)
    return cpus[lo : lo + per]


def pin_to_gpu(device_index: int, local_rank_on_node: int = 0, ranks_on_node: int = 1) -> list:
    """Pin this process near ``cuda:device_index``; returns the CPU set used ([] = unchanged)."""
    try:
        import torch

        bus = torch.cuda.get_device_properties(device_index).pci_bus_id  # type: ignore[attr-defined]
        bus_id = f"0000:{bus:02x}:00.0" if isinstance(bus, int) else str(bus)
    except Exception:
        return []
    node = gpu_numa_node(bus_id)
    if node is None:
        return []
    cpus = plan_affinity(node_cpus(node), local_rank_on_node, ranks_on_node)
    if cpus:
        try:
            os.sched_setaffinity(0, cpus)
        except OSError:
            return []
    return cpus
