"""Topology discovery: which ranks share a node, an NVLink fabric domain, or only a network.

Every rank probes its own GPU (name, PCI bus id, UUID, NUMA node, NVLink fabric cluster UUID and
clique id, NVLink peers) through ``pynvml`` when present, else through what torch and sysfs can
tell; the records are exchanged as JSON over ``torch.distributed`` and folded into a
``TopologyMap`` that answers ``get_interconnect_level(rank_a, rank_b)`` and plans how a symmetric
heap has to be shared (IPC/VMM handles inside a node, fabric handles inside an NVLink rack domain,
RDMA beyond). Same model and class names as the reference
(iris/host/distributed/topology.py:21-1396); a B200 has 18 NVLink 5 links.
"""
from __future__ import annotations

import json
import os
import socket
from dataclasses import asdict, dataclass, field
from enum import IntEnum

MAX_NVLINK_LINKS = 18  # NVLink 5 on B200


class InterconnectLevel(IntEnum):
    SAME_DEVICE = 0
    INTRA_NODE = 1          # NVLink / NVSwitch or PCIe inside one host: IPC or POSIX-fd VMM handles
    INTRA_RACK_FABRIC = 2   # multi-node NVLink domain (same cluster UUID and clique): fabric handles
    INTER_NODE_RDMA = 3     # only the network


@dataclass
class GPUInfo:
    rank: int = -1
    hostname: str = ""
    local_id: int = 0
    name: str = ""
    pci_bus_id: str = ""
    uuid: str = ""
    numa_node: int = -1
    cluster_uuid: str = ""
    clique_id: int = -1
    nvlink_peer_pci: list = field(default_factory=list)
    has_infiniband: bool = False


def normalize_pci_bus_id(bus_id) -> str:
    """``00000000:1B:00.0`` / ``0000:1b:00.0`` / bytes -> ``0000:1b:00.0``."""
    if isinstance(bus_id, bytes):
        bus_id = bus_id.decode()
    bus_id = bus_id.strip().lower()
    parts = bus_id.split(":")
    if len(parts) == 3:
        parts[0] = parts[0][-4:].rjust(4, "0")
        return ":".join(parts)
    if len(parts) == 2:
        return "0000:" + bus_id
    return bus_id


def visible_device_to_physical(local_id: int) -> int:
    """Index inside ``CUDA_VISIBLE_DEVICES`` -> physical index (NVML enumerates physical devices)."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if not vis:
        return local_id
    ids = [v.strip() for v in vis.split(",") if v.strip()]
    if local_id < len(ids) and ids[local_id].isdigit():
        return int(ids[local_id])
    return local_id


def detect_infiniband(sys_root: str = "/sys/class/infiniband") -> bool:
    try:
        return os.path.isdir(sys_root) and len(os.listdir(sys_root)) > 0
    except OSError:
        return False


class TopologyDiscovery:
    """Probe the local GPU and gather everybody's record."""

    def __init__(self, rank: int, local_id: int, nvml=None):
        self.rank, self.local_id = rank, local_id
        self._nvml = nvml

    def _load_nvml(self):
        if self._nvml is not None:
            return self._nvml
        try:
            import pynvml

            return pynvml
        except Exception:
            return None

    def probe(self) -> GPUInfo:
        info = GPUInfo(rank=self.rank, hostname=socket.gethostname(), local_id=self.local_id,
                       has_infiniband=detect_infiniband())
        nvml = self._load_nvml()
        if nvml is not None:
            try:
                nvml.nvmlInit()
                h = nvml.nvmlDeviceGetHandleByIndex(visible_device_to_physical(self.local_id))
                name = nvml.nvmlDeviceGetName(h)
                info.name = name.decode() if isinstance(name, bytes) else str(name)
                info.pci_bus_id = normalize_pci_bus_id(nvml.nvmlDeviceGetPciInfo(h).busId)
                uuid = nvml.nvmlDeviceGetUUID(h)
                info.uuid = uuid.decode() if isinstance(uuid, bytes) else str(uuid)
                try:
                    info.numa_node = int(nvml.nvmlDeviceGetNumaNodeId(h))
                except Exception:
                    info.numa_node = _numa_from_sysfs(info.pci_bus_id)
                try:
                    fab = nvml.nvmlDeviceGetGpuFabricInfo(h)
                    cu = getattr(fab, "clusterUuid", b"")
                    info.cluster_uuid = bytes(cu).hex() if not isinstance(cu, str) else cu
                    info.clique_id = int(getattr(fab, "cliqueId", -1))
                except Exception:
                    pass
                peers = []
                for link in range(MAX_NVLINK_LINKS):
                    try:
                        if nvml.nvmlDeviceGetNvLinkState(h, link):
                            peers.append(normalize_pci_bus_id(nvml.nvmlDeviceGetNvLinkRemotePciInfo(h, link).busId))
                    except Exception:
                        break
                info.nvlink_peer_pci = sorted(set(peers))
                return info
            except Exception:
                pass
        try:
            import torch

            if torch.cuda.is_available():
                p = torch.cuda.get_device_properties(self.local_id)
                info.name = p.name
                info.uuid = str(getattr(p, "uuid", ""))
                info.pci_bus_id = normalize_pci_bus_id(f"{getattr(p, 'pci_domain_id', 0):04x}:{getattr(p, 'pci_bus_id', 0):02x}:{getattr(p, 'pci_device_id', 0):02x}.0")
        except Exception:
            pass
        return info

    def discover(self, group=None) -> "TopologyMap":
        import torch.distributed as dist

        mine = json.dumps(asdict(self.probe()))
        world = dist.get_world_size(group)
        gathered = [None] * world
        dist.all_gather_object(gathered, mine, group=group)
        return TopologyMap([GPUInfo(**json.loads(s)) for s in gathered])


def _numa_from_sysfs(pci_bus_id: str) -> int:
    try:
        with open(f"/sys/bus/pci/devices/{pci_bus_id}/numa_node") as f:
            return int(f.read().strip())
    except Exception:
        return -1


class TopologyMap:
    def __init__(self, gpus: list):
        self.gpus = sorted(gpus, key=lambda g: g.rank)
        self.by_rank = {g.rank: g for g in self.gpus}

    @property
    def world_size(self) -> int:
        return len(self.gpus)

    def get_interconnect_level(self, a: int, b: int) -> InterconnectLevel:
        ga, gb = self.by_rank[a], self.by_rank[b]
        if a == b:
            return InterconnectLevel.SAME_DEVICE
        if ga.hostname == gb.hostname:
            return InterconnectLevel.INTRA_NODE
        if ga.cluster_uuid and ga.cluster_uuid == gb.cluster_uuid and ga.clique_id >= 0 and ga.clique_id == gb.clique_id \
                and set(ga.cluster_uuid) != {"0"}:
            return InterconnectLevel.INTRA_RACK_FABRIC
        return InterconnectLevel.INTER_NODE_RDMA

    def nvlink_connected(self, a: int, b: int) -> bool:
        """Direct NVLink between two GPUs of one node (through NVSwitch every pair counts as linked:
        the remote end of each link is the switch, so the peer list is empty and the node level decides)."""
        ga, gb = self.by_rank[a], self.by_rank[b]
        return gb.pci_bus_id in ga.nvlink_peer_pci or ga.pci_bus_id in gb.nvlink_peer_pci

    def node_groups(self) -> list:
        groups: dict[str, list] = {}
        for g in self.gpus:
            groups.setdefault(g.hostname, []).append(g.rank)
        return [sorted(v) for _, v in sorted(groups.items())]

    def fabric_groups(self) -> list:
        groups: dict[tuple, list] = {}
        for g in self.gpus:
            key = (g.cluster_uuid, g.clique_id) if g.cluster_uuid and g.clique_id >= 0 and set(g.cluster_uuid) != {"0"} else ("host", g.hostname)
            groups.setdefault(key, []).append(g.rank)
        return [sorted(v) for _, v in sorted(groups.items(), key=lambda kv: kv[1][0])]

    def heap_distribution_plan(self, rank: int) -> dict:
        """How ``rank`` reaches every other rank's heap: ipc (same node), fabric, or rdma."""
        plan = {"ipc": [], "fabric": [], "rdma": []}
        for g in self.gpus:
            if g.rank == rank:
                continue
            lvl = self.get_interconnect_level(rank, g.rank)
            plan["ipc" if lvl == InterconnectLevel.INTRA_NODE else "fabric" if lvl == InterconnectLevel.INTRA_RACK_FABRIC else "rdma"].append(g.rank)
        return plan

    def single_nvlink_domain(self) -> bool:
        """True when one symmetric heap can span all ranks with loads/stores (no RDMA leg)."""
        return all(not self.heap_distribution_plan(g.rank)["rdma"] for g in self.gpus)

    def to_json(self) -> str:
        return json.dumps([asdict(g) for g in self.gpus])
