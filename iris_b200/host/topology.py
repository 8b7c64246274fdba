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


class IntraNodeLinkType(IntEnum):
    """How two GPUs of one host are connected (the columns of ``nvidia-smi topo -m``)."""

    SELF = -1
    NVLINK = 0              # direct NVLink between the two GPUs
    NVSWITCH = 1            # NVLink through an NVSwitch (every pair at full bandwidth)
    PCIE_SWITCH = 2         # PIX / PXB
    PCIE_HOST_BRIDGE = 3    # PHB
    PCIE_NUMA = 4           # NODE
    PCIE_SYSTEM = 5         # SYS
    UNKNOWN = 99

    def __str__(self) -> str:
        return self.name


@dataclass
class FabricInfo:
    """Where a GPU sits in a multi-node NVLink fabric: two GPUs with the same ``domain_key`` reach each
    other by loads and stores (NVML ``clusterUuid`` + ``cliqueId``). Empty = no fabric information."""

    cluster_uuid: str = ""
    clique_id: int = 0

    @property
    def is_valid(self) -> bool:
        return bool(self.cluster_uuid) and set(self.cluster_uuid) != {"0"}

    @property
    def domain_key(self) -> str:
        return f"{self.cluster_uuid}:{self.clique_id}" if self.is_valid else ""

    def to_dict(self) -> dict:
        return {"cluster_uuid": self.cluster_uuid, "clique_id": self.clique_id}

    @classmethod
    def from_dict(cls, d: dict) -> "FabricInfo":
        return cls(cluster_uuid=d.get("cluster_uuid", ""), clique_id=d.get("clique_id", 0))


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
    nvlink_active_links: int = 0
    total_memory_mb: int = 0
    ib_devices: list = field(default_factory=list)

    @property
    def fabric_info(self) -> FabricInfo:
        return FabricInfo(self.cluster_uuid, self.clique_id) if self.clique_id >= 0 else FabricInfo()

    # names used by the reference's GPUInfo
    @property
    def gpu_id(self) -> int:
        return self.local_id

    @property
    def local_rank(self) -> int:
        return self.local_id

    @property
    def device_name(self) -> str:
        return self.name

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: dict) -> "GPUInfo":
        known = {k: v for k, v in d.items() if k in cls.__dataclass_fields__}
        return cls(**known)


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


def list_infiniband_devices(sys_root: str = "/sys/class/infiniband") -> list:
    try:
        return sorted(os.listdir(sys_root)) if os.path.isdir(sys_root) else []
    except OSError:
        return []


def detect_infiniband(sys_root: str = "/sys/class/infiniband") -> bool:
    return len(list_infiniband_devices(sys_root)) > 0


_TOPO_TOKENS = {"X": IntraNodeLinkType.SELF, "PIX": IntraNodeLinkType.PCIE_SWITCH, "PXB": IntraNodeLinkType.PCIE_SWITCH,
                "PHB": IntraNodeLinkType.PCIE_HOST_BRIDGE, "NODE": IntraNodeLinkType.PCIE_NUMA, "SYS": IntraNodeLinkType.PCIE_SYSTEM}


def parse_topo_matrix(text: str) -> list:
    """The GPU x GPU block of ``nvidia-smi topo -m`` as a matrix of ``IntraNodeLinkType`` values.

    ``NV<n>`` entries become ``NVLINK``; when EVERY pair of GPUs is NVLink-connected with the same
    link count (what an NVSwitch system shows: ``NV18`` everywhere on B200) they become ``NVSWITCH``.
    Rows that are not GPUs (NICs, legend) are ignored. Returns ``[]`` when no matrix is found."""
    rows = {}
    n_cols = 0
    for line in text.splitlines():
        cells = line.replace("\t", " ").split()
        if not cells:
            continue
        if cells[0].startswith("GPU0") and not rows and all(c.startswith(("GPU", "NIC", "CPU", "NUMA", "mlx", "Affinity", "ID")) for c in cells):
            n_cols = sum(1 for c in cells if c.startswith("GPU") and c[3:].isdigit())
            continue
        if cells[0].startswith("GPU") and cells[0][3:].isdigit() and n_cols and len(cells) > n_cols:
            rows[int(cells[0][3:])] = cells[1:1 + n_cols]
    if not rows or sorted(rows) != list(range(len(rows))) or len(rows) != n_cols:
        return []
    n = len(rows)
    counts = set()
    mat = [[int(IntraNodeLinkType.UNKNOWN)] * n for _ in range(n)]
    for i in range(n):
        for j, tok in enumerate(rows[i]):
            if tok.startswith("NV") and tok[2:].isdigit():
                mat[i][j] = int(IntraNodeLinkType.NVLINK)
                counts.add(tok)
            else:
                mat[i][j] = int(_TOPO_TOKENS.get(tok, IntraNodeLinkType.UNKNOWN))
    all_nv = all(mat[i][j] == IntraNodeLinkType.NVLINK for i in range(n) for j in range(n) if i != j)
    if n > 2 and all_nv and len(counts) == 1:
        for i in range(n):
            for j in range(n):
                if i != j:
                    mat[i][j] = int(IntraNodeLinkType.NVSWITCH)
    return mat


class TopologyDiscovery:
    """Probe the local GPU and gather everybody's record."""

    def __init__(self, rank: int, local_id: int, nvml=None):
        self.rank, self.local_id = rank, local_id
        self._nvml = nvml
        self._topology = None

    @property
    def topology(self):
        """The map built by the last ``discover()`` (``None`` before)."""
        return self._topology

    def get_communication_groups(self) -> dict:
        """``{level: [[ranks], ...]}``: one group per host, one per fabric domain (hosts outside any
        domain stand alone there), and everybody for the network level."""
        if self._topology is None:
            raise RuntimeError("Must call discover() before get_communication_groups()")
        return self._topology.communication_groups()

    def get_heap_distribution_plan(self) -> dict:
        """``{rank: {"ipc_peers", "fabric_peers", "rdma_peers", "node", "local_rank", "gpu_id", "fabric_domain"}}``."""
        if self._topology is None:
            raise RuntimeError("Must call discover() before get_heap_distribution_plan()")
        return self._topology.full_heap_distribution_plan()

    def _load_nvml(self):
        if self._nvml is not None:
            return self._nvml
        try:
            import pynvml

            return pynvml
        except Exception:
            return None

    def probe(self) -> GPUInfo:
        ib = list_infiniband_devices()
        info = GPUInfo(rank=self.rank, hostname=socket.gethostname(), local_id=self.local_id,
                       has_infiniband=bool(ib), ib_devices=ib)
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
                try:
                    info.total_memory_mb = int(nvml.nvmlDeviceGetMemoryInfo(h).total) >> 20
                except Exception:
                    pass
                peers, active = [], 0
                for link in range(MAX_NVLINK_LINKS):
                    try:
                        if nvml.nvmlDeviceGetNvLinkState(h, link):
                            active += 1
                            peers.append(normalize_pci_bus_id(nvml.nvmlDeviceGetNvLinkRemotePciInfo(h, link).busId))
                    except Exception:
                        break
                info.nvlink_peer_pci = sorted(set(peers))
                info.nvlink_active_links = active
                return info
            except Exception:
                pass
        try:
            import torch

            if torch.cuda.is_available():
                p = torch.cuda.get_device_properties(self.local_id)
                info.name = p.name
                info.total_memory_mb = int(p.total_memory) >> 20
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
        self._topology = TopologyMap([GPUInfo.from_dict(json.loads(s)) for s in gathered])
        return self._topology


def _numa_from_sysfs(pci_bus_id: str) -> int:
    try:
        with open(f"/sys/bus/pci/devices/{pci_bus_id}/numa_node") as f:
            return int(f.read().strip())
    except Exception:
        return -1


@dataclass
class NodeInfo:
    """One host: its ranks, its physical GPUs and how they are linked."""

    hostname: str = ""
    ranks: list = field(default_factory=list)
    gpu_ids: list = field(default_factory=list)          # device index per rank (ranks may share a GPU)
    unique_gpu_ids: list = field(default_factory=list)
    unique_pci_ids: list = field(default_factory=list)
    num_gpus: int = 0                                    # physical GPUs, not ranks
    num_ranks: int = 0
    has_infiniband: bool = False
    ib_devices: list = field(default_factory=list)
    link_types: list | None = None                       # [gpu_i][gpu_j] of IntraNodeLinkType values, by device index
    p2p_access: list | None = None
    fabric_domain_key: str = ""
    fabric_domain_keys: list = field(default_factory=list)

    def get_link_type(self, gpu_id_a: int, gpu_id_b: int) -> IntraNodeLinkType:
        if self.link_types is None:
            return IntraNodeLinkType.UNKNOWN
        if gpu_id_a == gpu_id_b:
            return IntraNodeLinkType.SELF
        if not (0 <= gpu_id_a < len(self.link_types) and 0 <= gpu_id_b < len(self.link_types[0])):
            return IntraNodeLinkType.UNKNOWN          # more ranks than GPUs, or a device the matrix does not cover
        return IntraNodeLinkType(self.link_types[gpu_id_a][gpu_id_b])

    def can_p2p_access(self, gpu_id_a: int, gpu_id_b: int) -> bool:
        if gpu_id_a == gpu_id_b:
            return True
        if self.p2p_access is None:
            return False
        if not (0 <= gpu_id_a < len(self.p2p_access) and 0 <= gpu_id_b < len(self.p2p_access[0])):
            return False
        return bool(self.p2p_access[gpu_id_a][gpu_id_b])


def _link_matrix(gpus: list) -> tuple:
    """Link types and peer access between the devices of one host, from what each rank probed:
    a direct NVLink when the peer's PCI id is at the far end of one of my links, NVSwitch when both
    have active links whose far ends are not GPUs of this host, else PCIe classified by NUMA node."""
    by_dev = {}
    for g in gpus:
        by_dev.setdefault(g.local_id, g)
    n = max(by_dev) + 1 if by_dev else 0
    types = [[int(IntraNodeLinkType.UNKNOWN)] * n for _ in range(n)]
    p2p = [[False] * n for _ in range(n)]
    for a in range(n):
        for b in range(n):
            if a == b:
                types[a][b], p2p[a][b] = int(IntraNodeLinkType.SELF), True
                continue
            ga, gb = by_dev.get(a), by_dev.get(b)
            if ga is None or gb is None:
                continue
            if gb.pci_bus_id and (gb.pci_bus_id in ga.nvlink_peer_pci or ga.pci_bus_id in gb.nvlink_peer_pci):
                t = IntraNodeLinkType.NVLINK
            elif ga.nvlink_active_links > 0 and gb.nvlink_active_links > 0:
                t = IntraNodeLinkType.NVSWITCH
            elif ga.numa_node >= 0 and gb.numa_node >= 0:
                t = IntraNodeLinkType.PCIE_HOST_BRIDGE if ga.numa_node == gb.numa_node else IntraNodeLinkType.PCIE_SYSTEM
            else:
                t = IntraNodeLinkType.UNKNOWN
            types[a][b] = int(t)
            p2p[a][b] = t in (IntraNodeLinkType.NVLINK, IntraNodeLinkType.NVSWITCH, IntraNodeLinkType.PCIE_SWITCH,
                              IntraNodeLinkType.PCIE_HOST_BRIDGE)
    return types, p2p


class TopologyMap:
    def __init__(self, gpus: list):
        self.gpus = sorted(gpus, key=lambda g: g.rank)
        self.by_rank = {g.rank: g for g in self.gpus}
        self.gpu_info = self.by_rank                     # the reference's name for the same table
        self.nodes: dict = {}
        for g in self.gpus:
            self.nodes.setdefault(g.hostname, []).append(g)
        self.nodes = {h: self._node_info(h, gs) for h, gs in self.nodes.items()}
        self.fabric_domains: dict = {}                   # domain key -> hostnames
        for g in self.gpus:
            key = g.fabric_info.domain_key
            if key and g.hostname not in self.fabric_domains.setdefault(key, []):
                self.fabric_domains[key].append(g.hostname)

    @staticmethod
    def _node_info(hostname: str, gs: list) -> NodeInfo:
        types, p2p = _link_matrix(gs)
        keys = sorted({g.fabric_info.domain_key for g in gs if g.fabric_info.domain_key})
        pci = sorted({g.pci_bus_id for g in gs if g.pci_bus_id})
        devs = sorted({g.local_id for g in gs})
        return NodeInfo(hostname=hostname, ranks=sorted(g.rank for g in gs), gpu_ids=[g.local_id for g in sorted(gs, key=lambda g: g.rank)],
                        unique_gpu_ids=devs, unique_pci_ids=pci, num_gpus=len(pci) if pci else len(devs), num_ranks=len(gs),
                        has_infiniband=any(g.has_infiniband for g in gs), ib_devices=sorted({d for g in gs for d in g.ib_devices}),
                        link_types=types, p2p_access=p2p, fabric_domain_key=keys[0] if keys else "", fabric_domain_keys=keys)

    @property
    def world_size(self) -> int:
        return len(self.gpus)

    @property
    def num_nodes(self) -> int:
        return len(self.nodes)

    def get_interconnect_level(self, a: int, b: int) -> InterconnectLevel:
        ga, gb = self.by_rank[a], self.by_rank[b]
        if a == b:
            return InterconnectLevel.SAME_DEVICE
        if ga.hostname == gb.hostname:
            return InterconnectLevel.INTRA_NODE
        ka, kb = ga.fabric_info.domain_key, gb.fabric_info.domain_key
        if ka and ka == kb:
            return InterconnectLevel.INTRA_RACK_FABRIC
        return InterconnectLevel.INTER_NODE_RDMA

    # ---- peers of one rank
    def get_node_peers(self, rank: int) -> set:
        """Other ranks on the same host."""
        return {r for r in self.nodes[self.by_rank[rank].hostname].ranks if r != rank}

    def get_fabric_domain_peers(self, rank: int) -> set:
        """Other ranks in the same NVLink fabric domain (same host included)."""
        key = self.by_rank[rank].fabric_info.domain_key
        if not key:
            return set()
        return {g.rank for g in self.gpus if g.rank != rank and g.fabric_info.domain_key == key}

    def get_rdma_peers(self, rank: int) -> set:
        """Ranks reachable only over the network."""
        near = self.get_node_peers(rank) | self.get_fabric_domain_peers(rank) | {rank}
        return {g.rank for g in self.gpus} - near

    def get_ranks_for_node(self, hostname: str) -> list:
        return list(self.nodes[hostname].ranks) if hostname in self.nodes else []

    def get_ranks_for_fabric_domain(self, domain_key: str) -> list:
        return sorted(g.rank for g in self.gpus if domain_key and g.fabric_info.domain_key == domain_key)

    def nvlink_connected(self, a: int, b: int) -> bool:
        """Direct NVLink between two GPUs of one node (through NVSwitch every pair counts as linked:
        the remote end of each link is the switch, so the peer list is empty and the node level decides)."""
        ga, gb = self.by_rank[a], self.by_rank[b]
        return gb.pci_bus_id in ga.nvlink_peer_pci or ga.pci_bus_id in gb.nvlink_peer_pci

    def get_link_type(self, a: int, b: int) -> IntraNodeLinkType:
        """Link between the GPUs of two ranks of one host (``UNKNOWN`` across hosts)."""
        ga, gb = self.by_rank[a], self.by_rank[b]
        if ga.hostname != gb.hostname:
            return IntraNodeLinkType.UNKNOWN
        return self.nodes[ga.hostname].get_link_type(ga.local_id, gb.local_id)

    # ---- groups
    def node_groups(self) -> list:
        return [list(n.ranks) for _, n in sorted(self.nodes.items())]

    def fabric_groups(self) -> list:
        groups: dict[tuple, list] = {}
        for g in self.gpus:
            key = ("fabric", g.fabric_info.domain_key) if g.fabric_info.domain_key else ("host", g.hostname)
            groups.setdefault(key, []).append(g.rank)
        return [sorted(v) for _, v in sorted(groups.items(), key=lambda kv: kv[1][0])]

    def communication_groups(self) -> dict:
        fabric = []
        if self.fabric_domains:
            fabric = [self.get_ranks_for_fabric_domain(k) for k in sorted(self.fabric_domains)]
            inside = {h for hs in self.fabric_domains.values() for h in hs}
            fabric += [list(n.ranks) for h, n in sorted(self.nodes.items()) if h not in inside]
        return {InterconnectLevel.INTRA_NODE: self.node_groups(), InterconnectLevel.INTRA_RACK_FABRIC: fabric,
                InterconnectLevel.INTER_NODE_RDMA: [sorted(self.by_rank)]}

    # ---- heap sharing
    def heap_distribution_plan(self, rank: int) -> dict:
        """How ``rank`` reaches every other rank's heap: ipc (same node), fabric, or rdma."""
        plan = {"ipc": [], "fabric": [], "rdma": []}
        for g in self.gpus:
            if g.rank == rank:
                continue
            lvl = self.get_interconnect_level(rank, g.rank)
            plan["ipc" if lvl == InterconnectLevel.INTRA_NODE else "fabric" if lvl == InterconnectLevel.INTRA_RACK_FABRIC else "rdma"].append(g.rank)
        return plan

    def full_heap_distribution_plan(self) -> dict:
        out = {}
        for g in self.gpus:
            p = self.heap_distribution_plan(g.rank)
            out[g.rank] = {"ipc_peers": p["ipc"], "fabric_peers": p["fabric"], "rdma_peers": p["rdma"], "node": g.hostname,
                           "local_rank": g.local_rank, "gpu_id": g.gpu_id, "fabric_domain": g.fabric_info.domain_key}
        return out

    def single_nvlink_domain(self) -> bool:
        """True when one symmetric heap can span all ranks with loads/stores (no RDMA leg)."""
        return all(not self.heap_distribution_plan(g.rank)["rdma"] for g in self.gpus)

    def summary(self) -> str:
        lines = ["=== Iris Cluster Topology ===",
                 f"World size: {self.world_size}  |  Nodes: {self.num_nodes}  |  Fabric domains: {len(self.fabric_domains)}", ""]
        for hostname, node in sorted(self.nodes.items()):
            ib = f"IB: {', '.join(node.ib_devices)}" if node.ib_devices else ("IB: present" if node.has_infiniband else "IB: none")
            fabric = f" fabric: {node.fabric_domain_key}" if node.fabric_domain_key else ""
            over = f" [oversubscribed: {node.num_ranks} ranks on {node.num_gpus} GPUs]" if node.num_ranks > node.num_gpus else ""
            lines.append(f"  Node '{hostname}': {node.num_gpus} GPUs, ranks {node.ranks}, {ib}{fabric}{over}")
            for r in node.ranks:
                g = self.by_rank[r]
                lines.append(f"    rank {r}: GPU{g.gpu_id} ({g.device_name}, {g.total_memory_mb}MB) PCI={g.pci_bus_id} NUMA={g.numa_node}")
        if self.fabric_domains:
            lines += ["", "Fabric Domains:"]
            for key, hosts in sorted(self.fabric_domains.items()):
                total = sum(self.nodes[h].num_gpus for h in hosts)
                lines.append(f"  {key}: {len(hosts)} nodes, {total} GPUs, hosts={hosts}")
        return "\n".join(lines)

    def __str__(self) -> str:
        return self.summary()

    def to_json(self) -> str:
        return json.dumps([asdict(g) for g in self.gpus])
