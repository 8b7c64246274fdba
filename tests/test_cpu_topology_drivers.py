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
