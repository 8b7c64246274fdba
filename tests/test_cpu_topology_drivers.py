"""Topology map and fabric-driver logic against fakes (no GPU, no NVML): the approach of the
reference's tests/unittests/test_topology.py and test_drivers.py."""
import types

import pytest

from iris_b200.host.topology import (GPUInfo, InterconnectLevel, TopologyDiscovery, TopologyMap, normalize_pci_bus_id,
                                     visible_device_to_physical)


def _fake_nvml(cluster=b"\x11" * 16, clique=3, links=2):
    m = types.SimpleNamespace()
    m.nvmlInit = lambda: None
    m.nvmlDeviceGetHandleByIndex = lambda i: ("h", i)
    m.nvmlDeviceGetName = lambda h: b"NVIDIA B200"
    m.nvmlDeviceGetPciInfo = lambda h: types.SimpleNamespace(busId=b"00000000:1B:00.0")
    m.nvmlDeviceGetUUID = lambda h: b"GPU-abc"
    m.nvmlDeviceGetNumaNodeId = lambda h: 1
    m.nvmlDeviceGetGpuFabricInfo = lambda h: types.SimpleNamespace(clusterUuid=cluster, cliqueId=clique)

    def state(h, link):
        if link >= links:
            raise RuntimeError("no such link")
        return 1

    m.nvmlDeviceGetNvLinkState = state
    m.nvmlDeviceGetNvLinkRemotePciInfo = lambda h, link: types.SimpleNamespace(busId=f"0000:{0x20 + link:02X}:00.0")
    return m


def test_pci_normalisation_and_visible_devices(monkeypatch):
    assert normalize_pci_bus_id("00000000:1B:00.0") == "0000:1b:00.0"
    assert normalize_pci_bus_id(b"0000:AF:00.0") == "0000:af:00.0"
    assert normalize_pci_bus_id("1b:00.0") == "0000:1b:00.0"
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "4,6")
    assert visible_device_to_physical(1) == 6 and visible_device_to_physical(5) == 5
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES")
    assert visible_device_to_physical(3) == 3


def test_probe_with_fake_nvml():
    info = TopologyDiscovery(rank=2, local_id=0, nvml=_fake_nvml()).probe()
    assert info.rank == 2 and info.name == "NVIDIA B200" and info.pci_bus_id == "0000:1b:00.0"
    assert info.uuid == "GPU-abc" and info.numa_node == 1 and info.clique_id == 3
    assert info.cluster_uuid == "11" * 16 and info.nvlink_peer_pci == ["0000:20:00.0", "0000:21:00.0"]


def test_interconnect_levels_and_plan():
    gpus = [GPUInfo(rank=0, hostname="a", cluster_uuid="aa", clique_id=1), GPUInfo(rank=1, hostname="a", cluster_uuid="aa", clique_id=1),
            GPUInfo(rank=2, hostname="b", cluster_uuid="aa", clique_id=1), GPUInfo(rank=3, hostname="c", cluster_uuid="", clique_id=-1)]
    tm = TopologyMap(gpus)
    assert tm.get_interconnect_level(0, 0) == InterconnectLevel.SAME_DEVICE
    assert tm.get_interconnect_level(0, 1) == InterconnectLevel.INTRA_NODE
    assert tm.get_interconnect_level(0, 2) == InterconnectLevel.INTRA_RACK_FABRIC
    assert tm.get_interconnect_level(0, 3) == InterconnectLevel.INTER_NODE_RDMA
    assert tm.node_groups() == [[0, 1], [2], [3]]
    assert tm.fabric_groups() == [[0, 1, 2], [3]]
    assert tm.heap_distribution_plan(0) == {"ipc": [1], "fabric": [2], "rdma": [3]}
    assert not tm.single_nvlink_domain()
    assert TopologyMap(gpus[:3]).single_nvlink_domain()
    assert "hostname" in tm.to_json()


class FakeRuntime:
    """Stands in for the native runtime: records calls, can be told to fail a step."""

    def __init__(self, fail=None, cuda=True):
        self.calls, self.fail, self.cuda, self.next = [], fail or set(), cuda, 0x1000

    def iris_rt_cuda_ok(self, err, n):
        return 1 if self.cuda else 0

    def iris_rt_set_device(self, d):
        return 0

    def iris_heap_create(self, size, dev, rank, world, kind, fabric, err, n):
        self.calls.append(("create", size, kind, fabric))
        if "create" in self.fail:
            return None
        self.next += 0x1000
        return self.next

    def iris_heap_base(self, h):
        return h * 16

    def iris_heap_mapped_size(self, h):
        return 1 << 21

    def iris_heap_export_blob(self, h, blob, err, n):
        self.calls.append(("export", h))
        return -1 if "export" in self.fail else 0

    def iris_heap_import_blob(self, h, slot, data, err, n):
        self.calls.append(("import", h, slot, len(data)))
        return -1 if "import" in self.fail else 0

    def iris_heap_peer_base(self, h, slot):
        return h * 16 + slot

    def iris_heap_destroy(self, h):
        self.calls.append(("destroy", h))
        return 2 if "destroy" in self.fail else 0


def test_fabric_driver_lifecycle_with_fake_runtime():
    from iris_b200.drivers import (AmdFabricDriver, DriverNotInitialized, DriverNotSupported, DriverStack, NvidiaFabricDriver,
                                   fabric_handle_bytes_to_tensor)

    rt = FakeRuntime()
    drv = NvidiaFabricDriver(runtime=rt)
    with pytest.raises(DriverNotInitialized):
        drv.allocate_exportable(1 << 20)
    drv.initialize(0)
    alloc = drv.allocate_exportable(1 << 20)
    assert ("create", 1 << 20, 0, 1) in rt.calls                 # VMM heap with fabric handles
    handle = drv.export_handle(alloc)
    assert len(handle) == 64 and fabric_handle_bytes_to_tensor(handle).numel() == 64
    with pytest.raises(ValueError):
        drv.import_and_map(b"short", 1 << 20)
    m = drv.import_and_map(handle, 1 << 20)
    assert m.slot == 1 and m.va == m.owner * 16 + 1
    assert drv.cleanup_local(alloc) == 0 and drv.close() == 0
    assert [c[0] for c in rt.calls].count("destroy") == 2
    # failures are reported, and cleanup still runs and reports how many steps failed
    bad = NvidiaFabricDriver(runtime=FakeRuntime(fail={"export", "destroy"}))
    bad.initialize(0)
    a = bad.allocate_exportable(1 << 20)
    with pytest.raises(RuntimeError):
        bad.export_handle(a)
    assert bad.cleanup_local(a) == 2
    with pytest.raises(DriverNotSupported):
        NvidiaFabricDriver(runtime=FakeRuntime(cuda=False)).initialize(0)
    with pytest.raises(DriverNotSupported):
        AmdFabricDriver().initialize(0)
    assert isinstance(DriverStack("nvidia", runtime=rt).fabric, NvidiaFabricDriver)
    assert isinstance(DriverStack("amd").fabric, AmdFabricDriver)


TOPO_NVSWITCH = """\
\tGPU0\tGPU1\tGPU2\tGPU3\tNIC0\tCPU Affinity\tNUMA Affinity\tGPU NUMA ID
GPU0\t X \tNV18\tNV18\tNV18\tPIX\t0-55\t0\t\tN/A
GPU1\tNV18\t X \tNV18\tNV18\tNODE\t0-55\t0\t\tN/A
GPU2\tNV18\tNV18\t X \tNV18\tSYS\t56-111\t1\t\tN/A
GPU3\tNV18\tNV18\tNV18\t X \tSYS\t56-111\t1\t\tN/A
NIC0\tPIX\tNODE\tSYS\tSYS\t X

Legend:

  X    = Self
  SYS  = Connection traversing PCIe as well as the SMP interconnect between NUMA nodes
  NV#  = Connection traversing a bonded set of # NVLinks
"""

TOPO_MIXED = """\
        GPU0    GPU1    GPU2    GPU3    CPU Affinity
GPU0     X      NV2     PIX     SYS     0-31
GPU1    NV2      X      PHB     SYS     0-31
GPU2    PIX     PHB      X      NODE    0-31
GPU3    SYS     SYS     NODE     X      32-63
"""


def test_topo_matrix_parser():
    from iris_b200.host.topology import IntraNodeLinkType as L
    from iris_b200.host.topology import parse_topo_matrix

    m = parse_topo_matrix(TOPO_NVSWITCH)
    assert len(m) == 4 and all(len(r) == 4 for r in m)
    assert all(m[i][i] == L.SELF for i in range(4))
    assert all(m[i][j] == L.NVSWITCH for i in range(4) for j in range(4) if i != j)       # NV18 everywhere: a switch
    m = parse_topo_matrix(TOPO_MIXED)
    assert m[0][1] == L.NVLINK and m[1][0] == L.NVLINK                                    # a bridge between two GPUs
    assert m[0][2] == L.PCIE_SWITCH and m[1][2] == L.PCIE_HOST_BRIDGE and m[2][3] == L.PCIE_NUMA and m[0][3] == L.PCIE_SYSTEM
    assert parse_topo_matrix("no matrix here") == [] and parse_topo_matrix("") == []
    assert str(L.NVSWITCH) == "NVSWITCH" and L(99) == L.UNKNOWN


def test_fabric_info_and_gpu_info_round_trip():
    from iris_b200.host.topology import FabricInfo

    f = FabricInfo("ab" * 16, 7)
    assert f.is_valid and f.domain_key == "ab" * 16 + ":7"
    assert FabricInfo.from_dict(f.to_dict()) == f
    assert not FabricInfo().is_valid and FabricInfo().domain_key == "" and not FabricInfo("00" * 16, 1).is_valid
    g = GPUInfo(rank=3, hostname="n1", local_id=2, name="NVIDIA B200", pci_bus_id="0000:1b:00.0", cluster_uuid="cd" * 16, clique_id=4,
                total_memory_mb=183359, ib_devices=["mlx5_0"], has_infiniband=True)
    d = g.to_dict()
    d["field_from_a_newer_version"] = 1                       # unknown keys are dropped, not fatal
    g2 = GPUInfo.from_dict(d)
    assert g2 == g and g2.fabric_info.domain_key == "cd" * 16 + ":4"
    assert (g2.gpu_id, g2.local_rank, g2.device_name) == (2, 2, "NVIDIA B200")
    assert GPUInfo(cluster_uuid="cd" * 16, clique_id=-1).fabric_info.domain_key == ""


def _cluster():
    """Two 2-GPU hosts in one NVLink fabric domain, a third host with PCIe-only GPUs and two ranks
    sharing one GPU, a fourth host alone."""
    fab = dict(cluster_uuid="aa" * 16, clique_id=1)
    return [
        GPUInfo(rank=0, hostname="n0", local_id=0, name="B200", pci_bus_id="0000:1b:00.0", nvlink_active_links=18, numa_node=0, **fab),
        GPUInfo(rank=1, hostname="n0", local_id=1, name="B200", pci_bus_id="0000:2b:00.0", nvlink_active_links=18, numa_node=1, **fab),
        GPUInfo(rank=2, hostname="n1", local_id=0, name="B200", pci_bus_id="0000:1b:00.0", nvlink_active_links=18, **fab),
        GPUInfo(rank=3, hostname="n1", local_id=1, name="B200", pci_bus_id="0000:2b:00.0", nvlink_active_links=18, **fab),
        GPUInfo(rank=4, hostname="n2", local_id=0, name="L4", pci_bus_id="0000:3b:00.0", numa_node=0, has_infiniband=True, ib_devices=["mlx5_0"]),
        GPUInfo(rank=5, hostname="n2", local_id=1, name="L4", pci_bus_id="0000:5e:00.0", numa_node=1, has_infiniband=True, ib_devices=["mlx5_0"]),
        GPUInfo(rank=6, hostname="n2", local_id=1, name="L4", pci_bus_id="0000:5e:00.0", numa_node=1, has_infiniband=True, ib_devices=["mlx5_0"]),
        GPUInfo(rank=7, hostname="n3", local_id=0, name="B200", pci_bus_id="0000:1b:00.0",
                nvlink_peer_pci=["0000:99:00.0"], nvlink_active_links=2),
    ]


def test_nodes_peers_groups_and_plans():
    from iris_b200.host.topology import IntraNodeLinkType as L

    tm = TopologyMap(_cluster())
    assert tm.world_size == 8 and tm.num_nodes == 4 and sorted(tm.nodes) == ["n0", "n1", "n2", "n3"]
    key = "aa" * 16 + ":1"
    assert tm.fabric_domains == {key: ["n0", "n1"]}
    n0, n2 = tm.nodes["n0"], tm.nodes["n2"]
    assert n0.ranks == [0, 1] and n0.num_gpus == 2 and n0.num_ranks == 2 and n0.fabric_domain_key == key and not n0.has_infiniband
    assert n2.ranks == [4, 5, 6] and n2.gpu_ids == [0, 1, 1] and n2.unique_gpu_ids == [0, 1] and n2.num_gpus == 2 and n2.num_ranks == 3
    assert n2.has_infiniband and n2.ib_devices == ["mlx5_0"] and n2.fabric_domain_keys == []
    # link types inside a host
    assert n0.get_link_type(0, 1) == L.NVSWITCH and n0.get_link_type(1, 1) == L.SELF and n0.can_p2p_access(0, 1)
    assert n2.get_link_type(0, 1) == L.PCIE_SYSTEM and not n2.can_p2p_access(0, 1) and n2.can_p2p_access(1, 1)
    assert n0.get_link_type(0, 5) == L.UNKNOWN and not n0.can_p2p_access(0, 5)           # outside the matrix: no IndexError
    assert tm.get_link_type(0, 1) == L.NVSWITCH and tm.get_link_type(5, 6) == L.SELF and tm.get_link_type(0, 2) == L.UNKNOWN
    direct = TopologyMap([GPUInfo(rank=0, hostname="h", local_id=0, pci_bus_id="0000:01:00.0", nvlink_peer_pci=["0000:02:00.0"], nvlink_active_links=4),
                          GPUInfo(rank=1, hostname="h", local_id=1, pci_bus_id="0000:02:00.0", nvlink_peer_pci=["0000:01:00.0"], nvlink_active_links=4)])
    assert direct.get_link_type(0, 1) == L.NVLINK and direct.nvlink_connected(0, 1)
    # peers of a rank
    assert tm.get_node_peers(0) == {1} and tm.get_fabric_domain_peers(0) == {1, 2, 3} and tm.get_rdma_peers(0) == {4, 5, 6, 7}
    assert tm.get_node_peers(5) == {4, 6} and tm.get_fabric_domain_peers(5) == set() and tm.get_rdma_peers(5) == {0, 1, 2, 3, 7}
    assert tm.get_ranks_for_node("n1") == [2, 3] and tm.get_ranks_for_node("nowhere") == []
    assert tm.get_ranks_for_fabric_domain(key) == [0, 1, 2, 3] and tm.get_ranks_for_fabric_domain("") == []
    # levels
    assert tm.get_interconnect_level(0, 3) == InterconnectLevel.INTRA_RACK_FABRIC
    assert tm.get_interconnect_level(0, 7) == InterconnectLevel.INTER_NODE_RDMA
    # groups per level
    groups = tm.communication_groups()
    assert groups[InterconnectLevel.INTRA_NODE] == [[0, 1], [2, 3], [4, 5, 6], [7]]
    assert groups[InterconnectLevel.INTRA_RACK_FABRIC] == [[0, 1, 2, 3], [4, 5, 6], [7]]     # hosts outside a domain stand alone
    assert groups[InterconnectLevel.INTER_NODE_RDMA] == [list(range(8))]
    assert TopologyMap(_cluster()[4:7]).communication_groups()[InterconnectLevel.INTRA_RACK_FABRIC] == []   # no fabric anywhere
    # heap plan for everybody
    plan = tm.full_heap_distribution_plan()
    assert plan[0] == {"ipc_peers": [1], "fabric_peers": [2, 3], "rdma_peers": [4, 5, 6, 7], "node": "n0", "local_rank": 0, "gpu_id": 0,
                       "fabric_domain": key}
    assert plan[6]["ipc_peers"] == [4, 5] and plan[6]["fabric_peers"] == [] and plan[6]["fabric_domain"] == ""
    for r, p in plan.items():
        assert sorted(p["ipc_peers"] + p["fabric_peers"] + p["rdma_peers"] + [r]) == list(range(8))
    # summary
    text = str(tm)
    assert text.startswith("=== Iris Cluster Topology ===") and "World size: 8  |  Nodes: 4  |  Fabric domains: 1" in text
    assert "oversubscribed: 3 ranks on 2 GPUs" in text and "IB: mlx5_0" in text and "IB: none" in text
    assert f"{key}: 2 nodes, 4 GPUs, hosts=['n0', 'n1']" in text and "rank 7: GPU0 (B200, 0MB) PCI=0000:1b:00.0" in text


def test_discovery_needs_discover_first_and_lists_ib(tmp_path):
    from iris_b200.host.topology import detect_infiniband, list_infiniband_devices

    d = TopologyDiscovery(rank=0, local_id=0, nvml=_fake_nvml())
    assert d.topology is None
    with pytest.raises(RuntimeError):
        d.get_communication_groups()
    with pytest.raises(RuntimeError):
        d.get_heap_distribution_plan()
    info = d.probe()
    assert info.nvlink_active_links == 2
    root = tmp_path / "infiniband"
    assert list_infiniband_devices(str(root)) == [] and not detect_infiniband(str(root))
    root.mkdir()
    assert not detect_infiniband(str(root))
    (root / "mlx5_1").mkdir()
    (root / "mlx5_0").mkdir()
    assert list_infiniband_devices(str(root)) == ["mlx5_0", "mlx5_1"] and detect_infiniband(str(root))


def _discover(rank, world):
    from iris_b200.host.topology import TopologyDiscovery as TD

    d = TD(rank=rank, local_id=rank, nvml=_fake_nvml(links=0))
    tm = d.discover()
    assert d.topology is tm and tm.world_size == world and tm.num_nodes == 1
    groups = d.get_communication_groups()
    assert groups[InterconnectLevel.INTRA_NODE] == [list(range(world))]
    plan = d.get_heap_distribution_plan()
    assert plan[rank]["ipc_peers"] == [r for r in range(world) if r != rank] and plan[rank]["rdma_peers"] == []
    assert tm.single_nvlink_domain()


def test_discovery_over_gloo_ranks():
    from helpers import run_ranks

    run_ranks(_discover, 3)


def test_fabric_driver_through_the_native_runtime_on_the_host_memory_driver():
    """The same life cycle as above, but with nothing faked in Python: the native runtime creates
    the exportable allocation, produces the 64-byte handle, imports it and maps it, on the host-memory
    stand-in for the driver (whose fabric handles are valid inside the exporting process)."""
    import torch

    import iris_b200 as iris
    from iris_b200 import hip
    from iris_b200.drivers import DriverNotSupported, NvidiaFabricDriver

    if hip.count_devices() == 0:
        with pytest.raises(DriverNotSupported):
            NvidiaFabricDriver().initialize(0)                  # no driver on this machine
    assert hip.install_fake_driver(2) == 2
    try:
        drv = NvidiaFabricDriver()
        drv.initialize(1)
        alloc = drv.allocate_exportable(3 << 20)
        assert alloc.size >= 3 << 20 and alloc.size % hip.get_allocation_granularity(1) == 0      # rounded up to the granularity
        handle = drv.export_handle(alloc)
        assert len(handle) == 64 and any(handle)
        mapping = drv.import_and_map(handle, alloc.size)
        assert mapping.va not in (0, alloc.va)
        mine = iris.tensor_from_ptr(alloc.va, 1024, torch.int32, "cpu")
        theirs = iris.tensor_from_ptr(mapping.va, 1024, torch.int32, "cpu")
        mine.copy_(torch.arange(1024, dtype=torch.int32))
        assert torch.equal(theirs, mine)                        # two mappings of one allocation
        theirs[5] = 99
        assert int(mine[5]) == 99
        with pytest.raises(RuntimeError):
            drv.import_and_map(bytes(64), alloc.size)           # not a handle of this driver
        del mine, theirs
        drv.cleanup_import(mapping)
        assert drv.close() == 0 and drv.cleanup_local(alloc) == 0
    finally:
        hip.install_fake_driver(0)
