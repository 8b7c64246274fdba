"""Runtime bindings, distributed helpers, timing loops and raw-pointer tensors without a GPU.

The reference covers these in tests/unittests/test_hip_apis.py, test_get_num_xcc.py,
test_iris_helpers.py, test_broadcast.py, test_logging.py and test_is_symmetric.py, all on GPUs. The
parts that need no device are checked here; the device queries themselves are in the GPU suite.
"""
import ctypes
import logging
import os

import numpy as np
import pytest
import torch

from helpers import run_ranks


def test_runtime_bindings_without_a_device(monkeypatch):
    import iris_b200 as iris
    from iris_b200 import hip

    # the names the reference exposes under iris.hip
    for name in ("count_devices", "set_device", "get_device_id", "get_cu_count", "get_wall_clock_rate", "get_arch_string",
                 "get_num_xcc", "get_ipc_handle", "open_ipc_handle", "get_address_range"):
        assert callable(getattr(hip, name)), name
    assert hip.get_num_xcc() == 1 and hip.get_num_xcc(3) == 1           # no chiplets to spread tiles over
    assert hip.get_wall_clock_rate() == 1_000_000                        # kHz of a nanosecond counter
    if not torch.cuda.is_available():
        assert hip.count_devices() == 0 and hip.get_device_id() == -1
        with pytest.raises(RuntimeError):
            hip.get_address_range(0x1000)
    monkeypatch.delenv("LOCAL_RANK", raising=False)
    assert [iris.get_device_id_for_rank(r, 4) for r in range(6)] == [0, 1, 2, 3, 0, 1]
    monkeypatch.setenv("LOCAL_RANK", "5")
    assert iris.get_device_id_for_rank(0, 4) == 1 and iris.get_device_id_for_rank(9, 8) == 5
    monkeypatch.setenv("IRIS_SIMULATION", "1")
    assert iris.is_simulation_env()
    monkeypatch.setenv("IRIS_SIMULATION", "0")
    assert not iris.is_simulation_env()


def test_do_bench_protocol_and_return_modes():
    import iris_b200 as iris

    log = []
    out = iris.do_bench(lambda: log.append("fn"), barrier_fn=lambda: log.append("b"), preamble_fn=lambda: log.append("p"),
                        n_warmup=2, n_repeat=3, return_mode="all")
    assert isinstance(out, list) and len(out) == 3 and all(t >= 0 for t in out)
    # one untimed call, the warm-ups, the timed calls; each wrapped as barrier, preamble, barrier, fn
    assert log == ["b", "p", "b", "fn"] * (1 + 2 + 3)
    for mode in ("mean", "min", "max", "median"):
        assert isinstance(iris.do_bench(lambda: None, n_warmup=0, n_repeat=4, return_mode=mode), float)
    q = iris.do_bench(lambda: None, n_warmup=0, n_repeat=8, quantiles=[0.2, 0.5, 0.8])
    assert len(q) == 3 and q[0] <= q[1] <= q[2]
    assert isinstance(iris.do_bench(lambda: None, n_warmup=0, n_repeat=4, quantiles=[0.5]), float)
    with pytest.raises(ValueError):
        iris.do_bench(lambda: None, return_mode="p99")


def test_tensor_from_raw_pointer():
    import iris_b200 as iris

    for dt in (torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int16, torch.int32,
               torch.int64, torch.bool):
        n = 24
        esize = torch.empty((), dtype=dt).element_size()
        backing = (ctypes.c_uint8 * (n * esize))()
        t = iris.tensor_from_ptr(ctypes.addressof(backing), n, dt, "cpu", keepalive=backing)
        assert t.dtype == dt and t.shape == (n,) and t.data_ptr() == ctypes.addressof(backing)
        t.fill_(1)
        assert any(bytes(backing))                               # writes go to the wrapped memory, not to a copy
        ctypes.memset(backing, 0, n * esize)
        assert not t.any()
    assert iris.tensor_from_ptr(0, 0, torch.float32, "cpu").shape == (0,)
    cai = iris.CUDAArrayInterface(0x7000_0000_0000, (4, 2), "<f4")
    assert cai.__cuda_array_interface__ == {"shape": (4, 2), "typestr": "<f4", "data": (0x7000_0000_0000, False), "version": 3,
                                            "strides": None}


def test_logger_levels(capsys):
    import iris_b200 as iris

    assert iris.logger.name == "iris"
    iris.set_logger_level(iris.DEBUG)
    assert iris.logger.level == logging.DEBUG
    iris.set_logger_level(iris.ERROR)
    assert iris.logger.level == logging.ERROR and not iris.logger.isEnabledFor(iris.WARNING)
    iris.set_logger_level(iris.WARNING)
    assert (iris.DEBUG, iris.INFO, iris.WARNING, iris.ERROR) == (logging.DEBUG, logging.INFO, logging.WARNING, logging.ERROR)


def test_context_needs_a_process_group():
    import torch.distributed as dist

    import iris_b200 as iris

    assert not dist.is_initialized()
    with pytest.raises(RuntimeError, match="init_process_group"):
        iris.iris(1 << 20)


def _helpers(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.host import distributed as D
    from iris_b200.utils import time_max_over_ranks

    assert D.init_distributed() == (None, rank, world)
    for dt in (np.int32, np.int64, np.uint64, np.float32, np.float64, np.uint8, np.bool_):
        got = D.distributed_allgather(np.array([rank + 1, 7], dtype=dt))
        assert got.shape == (world, 2) and got.dtype == dt
        assert got[:, 0].tolist() == [dt(r + 1) for r in range(world)] and all(got[:, 1] == dt(7))
    big = D.distributed_allgather(np.array([2**63 + rank], dtype=np.uint64))        # above the int64 range
    assert [int(v) for v in big[:, 0]] == [2**63 + r for r in range(world)]
    md = D.distributed_allgather_multidim(np.full((2, 3), rank, dtype=np.int64))
    assert md.shape == (world, 2, 3) and all((md[r] == r).all() for r in range(world))
    objs = D.distributed_allgather_object({"rank": rank, "name": f"r{rank}"})
    assert objs == [{"rank": r, "name": f"r{r}"} for r in range(world)]
    src = world - 1
    for value in (7, 2.5, True, "heap", None, (1, "a"), np.float32(1.5)):
        assert D.distributed_broadcast_scalar(value if rank == src else "junk", src) == value
    t = D.distributed_broadcast_tensor(torch.arange(6).view(2, 3) * (rank + 1), src)
    assert torch.equal(torch.as_tensor(t), torch.arange(6).view(2, 3) * (src + 1))
    a = D.distributed_broadcast_tensor(np.arange(4, dtype=np.float32) + rank, 0)
    assert isinstance(a, np.ndarray) and a.dtype == np.float32 and a.tolist() == [0, 1, 2, 3]
    for dt in (torch.float16, torch.bfloat16, torch.int8, torch.float64):
        got = D.distributed_broadcast_tensor(torch.full((3,), rank + 2, dtype=dt), 0)
        assert got.dtype == dt and torch.all(got == 2)
    D.distributed_barrier()

    ctx = iris.iris(1 << 22)
    # Iris.broadcast: scalars come back as scalars, arrays as arrays, whatever the non-source ranks pass
    assert ctx.broadcast(3.25 if rank == 0 else None, src=0) == 3.25
    assert ctx.broadcast(rank, src=src) == src
    got = ctx.broadcast(torch.ones(4) * (rank + 1) if rank == src else None, src=src)
    assert torch.all(torch.as_tensor(got) == src + 1)
    got = ctx.broadcast(np.array([rank, rank]), src=0)
    assert np.asarray(got).tolist() == [0, 0]
    # rank-prefixed logging helpers
    for fn in (ctx.debug, ctx.info, ctx.warning, ctx.error):
        fn("message")
    # the slowest rank sets the reported time
    import time

    res = time_max_over_ranks(lambda: time.sleep(0.002 * (rank + 1)), ctx, n_warmup=0, n_repeat=3)
    assert res["n_warmup"] == 3 and res["n_repeat"] == 3
    assert res["ms"] >= 2.0 * world * 0.9 and res["ms_min_over_ranks"] <= res["ms_this_rank"] <= res["ms"] + 1e-9
    all_ms = D.distributed_allgather(np.array([res["ms"]]))
    assert len(set(all_ms.flatten().tolist())) == 1                 # every rank reports the same maximum
    dist.barrier()
    ctx.barrier()


def test_distributed_helpers_and_broadcast_world2():
    run_ranks(_helpers, 2, timeout=120.0)


def test_distributed_helpers_and_broadcast_world3():
    run_ranks(_helpers, 3, timeout=120.0)


@pytest.fixture
def fake_driver():
    from iris_b200 import hip

    assert hip.install_fake_driver(2) == 2
    try:
        yield hip
    finally:
        hip.install_fake_driver(0)


def test_vmm_primitives_against_a_host_memory_driver(fake_driver):
    """Reserve, create, map, grant access, write; export the allocation as a file descriptor, import
    it, map it a second time and see the same bytes; take everything down again. The sequence of the
    reference's tests/unittests/test_hip_vmem_primitives.py and test_vmem_peer_exchange.py, on a
    stand-in for the driver that keeps allocations in memfd files (no GPU)."""
    import iris_b200 as iris

    hip = fake_driver
    assert hip.count_devices() == 2 and hip.get_cu_count(0) == 148 and hip.get_arch_string(1) == "sm_100"
    assert hip.get_driver_version() >= 12000 and hip.get_rocm_version() == (12, 9) and hip.get_ipc_handle_size() == 64
    assert hip.can_access_peer(0, 1) and not hip.can_access_peer(1, 1)
    gran = hip.get_allocation_granularity(0)
    assert gran == hip.get_allocation_granularity(1, recommended=False) and gran % 4096 == 0
    size = 2 * gran
    va = hip.mem_address_reserve(2 * size)                      # room for two allocations side by side
    h1, h2 = hip.mem_create(size, 0), hip.mem_create(size, 1)
    hip.mem_map(va, size, 0, h1)
    hip.mem_map(va + size, size, 0, h2)
    hip.mem_set_access(va, 2 * size, [0, 1])                    # cumulative access over both mappings
    t = iris.tensor_from_ptr(va, 2 * size // 4, torch.int32, "cpu")
    t.copy_(torch.arange(t.numel(), dtype=torch.int32))
    assert hip.get_address_range(va + size + 64) == (va + size, size)
    # a second mapping of the first allocation, through an exported descriptor
    fd = hip.mem_export_to_shareable_handle(h1)
    assert fd > 2
    h1b, va2 = hip.import_dmabuf_handle(fd, size, device_ids=[0])
    os.close(fd)
    peer = iris.tensor_from_ptr(va2, size // 4, torch.int32, "cpu")
    assert torch.equal(peer, torch.arange(size // 4, dtype=torch.int32))
    peer[7] = -5                                                # one allocation, two windows
    assert int(t[7]) == -5
    # the descriptor of whatever is mapped at an address
    fd2 = hip.export_dmabuf_handle(va + size + 128)
    h2b = hip.mem_import_from_shareable_handle(fd2)
    os.close(fd2)
    va3 = hip.mem_address_reserve(size)
    hip.mem_map(va3, size, 0, h2b)
    hip.mem_set_access(va3, size, 1)
    assert int(iris.tensor_from_ptr(va3, 4, torch.int32, "cpu")[3]) == size // 4 + 3
    # misuse is refused with the driver's error, nothing crashes
    for bad in (lambda: hip.mem_create(size + 1, 0), lambda: hip.mem_create(size, 5), lambda: hip.mem_map(va, size, 0, h1),
                lambda: hip.mem_set_access(va, size, [9]), lambda: hip.mem_address_free(va, 2 * size),      # still mapped
                lambda: hip.mem_unmap(va + 4096, size), lambda: hip.mem_release(123456)):
        with pytest.raises(hip.DriverError):
            bad()
    # orderly teardown; released allocations stay readable through live mappings until unmapped
    hip.mem_release(h1)
    assert int(t[7]) == -5
    del t, peer
    hip.destroy_external_memory(h1b, va2, size)
    hip.destroy_external_memory(h2b, va3, size)
    hip.mem_unmap(va, size)
    hip.mem_unmap(va + size, size)
    hip.mem_address_free(va, 2 * size)
    hip.mem_release(h2)
    with pytest.raises(RuntimeError):
        hip.get_address_range(va)
    # plain allocations
    p = hip.hip_malloc(1 << 16, 0)
    buf = iris.tensor_from_ptr(p, 1 << 16, torch.uint8, "cpu")
    buf.fill_(3)
    assert hip.get_address_range(p + 100)[0] == p and hip.malloc_fine_grained is hip.hip_malloc
    del buf
    hip.hip_free(p)
    with pytest.raises(hip.DriverError):
        hip.hip_free(p)


def test_vmm_primitives_without_a_driver_raise():
    from iris_b200 import hip

    if hip.count_devices() == 0:
        for call in (lambda: hip.mem_create(1 << 21), lambda: hip.mem_address_reserve(1 << 21), lambda: hip.hip_malloc(16),
                     lambda: hip.get_allocation_granularity(), lambda: hip.get_driver_version()):
            with pytest.raises(hip.DriverError) as ei:
                call()
            assert ei.value.code == 1000 and "no CUDA driver" in str(ei.value)
    hip.gpu_try(0)
    with pytest.raises(hip.DriverError):
        hip.gpu_try(-1, "something")


def _vmm_heap(rank, world):
    """The symmetric heap's VMM backend end to end on the host-memory driver: every rank creates its
    region, exports it as a file descriptor over the UNIX-socket mesh, imports and maps the others'."""
    import torch.distributed as dist

    from iris_b200.host.heap import KIND_VMM, SymmetricHeap

    heap = SymmetricHeap(8 << 20, 0, rank, world, allocator_type="vmem", enable_multicast=False)
    assert heap.kind == KIND_VMM and heap.device.type == "cpu" and heap.mc_base == 0
    bases = [int(b) for b in heap.bases_host()]
    assert bases[rank] == heap.base and len(set(bases)) == world            # one mapping per rank's region, in this process
    a = heap.allocate(1000, torch.float32)
    b = heap.allocate(7, torch.int64)
    assert heap.is_symmetric(a) and heap.offset_of(a) == 0 and heap.offset_of(b) % 1024 == 0
    a.fill_(float(rank + 1))
    b.copy_(torch.arange(7) + 100 * rank)
    dist.barrier()
    for r in range(world):                                                 # every peer's copy, through this rank's mapping of it
        assert torch.all(heap.peer_view(a, r) == r + 1)
        assert torch.equal(heap.peer_view(b, r), torch.arange(7) + 100 * r)
    dist.barrier()
    heap.peer_view(a, (rank + 1) % world)[0] = -1.0                       # a remote write lands in the peer's memory
    dist.barrier()
    assert float(a[0]) == -1.0 and float(a[1]) == rank + 1
    with pytest.raises(MemoryError):
        heap.allocate(9 << 20, torch.uint8)
    mark = heap.get_offset()
    heap.allocate(4096, torch.uint8)
    heap.set_offset(mark)
    assert heap.get_offset() == mark
    dist.barrier()
    del a, b
    heap.close()


def test_symmetric_heap_vmm_backend_on_the_host_memory_driver_world2():
    run_ranks(_vmm_heap, 2, env={"IRIS_FAKE_DRIVER_DEVICES": "2"}, timeout=120.0)


def test_symmetric_heap_vmm_backend_on_the_host_memory_driver_world3():
    run_ranks(_vmm_heap, 3, env={"IRIS_FAKE_DRIVER_DEVICES": "2"}, timeout=120.0)


def _context_on_vmm_heap(rank, world):
    """A whole context on top of the VMM heap of the host-memory driver: one-sided operations,
    barriers and collectives work on it exactly as on the shared-memory heap."""
    import iris_b200 as iris
    from iris_b200.host.heap import KIND_VMM

    ctx = iris.iris(1 << 24)
    assert ctx.heap.kind == KIND_VMM and ctx.is_cpu
    peer = (rank + 1) % world
    buf = ctx.zeros(256, dtype=torch.float32)
    cnt = ctx.zeros(1, dtype=torch.int32)
    ctx.barrier()
    ctx.rma.store(buf, float(rank + 1), to_rank=peer)
    for r in range(world):
        ctx.rma.atomic_add(cnt, 1, to_rank=r)
    ctx.device_barrier()
    assert torch.all(buf == (rank - 1) % world + 1) and int(cnt.item()) == world
    inp, out = ctx.full((8, 4 * world), float(rank + 1)), ctx.zeros((8, 4 * world))
    ctx.ccl.all_reduce(out, inp)
    assert torch.all(out == sum(range(1, world + 1)))
    ag = ctx.zeros((8 * world, 4 * world))
    ctx.ccl.all_gather(ag, inp)
    assert all(torch.all(ag[8 * r:8 * (r + 1)] == r + 1) for r in range(world))
    ctx.verify_symmetry()
    ctx.check()
    ctx.barrier()


def test_context_on_the_vmm_heap_of_the_host_memory_driver():
    run_ranks(_context_on_vmm_heap, 3, env={"IRIS_FAKE_DRIVER_DEVICES": "4"}, timeout=120.0)


def _vmm_growth(rank, world):
    """A growable heap (allocator_type="vmem"): address space for the whole heap, physical memory mapped on
    demand, every rank's new segment mapped at the same offset of its window in every peer; and an external
    allocation taken into the heap without a copy. Reference: tests/unittests/test_vmem_allocator.py,
    test_vmem_segmented_export_import.py, test_vmem_imported_tensor_rma.py (on GPUs there)."""
    import torch.distributed as dist

    from iris_b200.host import platform as hip
    from iris_b200.host.heap import SymmetricHeap, _rt
    from iris_b200.host.tensor_utils import tensor_from_ptr

    heap = SymmetricHeap(32 << 20, 0, rank, world, allocator_type="vmem")
    rt = _rt()
    assert heap.reserve == 32 << 20 and heap.mc_base == 0
    first = rt.iris_heap_mapped_size(heap._handle)
    assert first <= 4 << 20                                                    # IRIS_VMEM_INITIAL, rounded to the granularity
    a = heap.allocate(256 << 10, torch.float32)                               # 1 MB: inside the first segment
    assert rt.iris_heap_num_segments(heap._handle) == 0
    b = heap.allocate(2 << 20, torch.float32)                                 # 8 MB: needs more than is mapped
    assert rt.iris_heap_num_segments(heap._handle) >= 1 and rt.iris_heap_mapped_size(heap._handle) > first
    assert heap.is_symmetric(b) and heap.offset_of(b) >= heap.offset_of(a) + a.numel() * 4
    a.fill_(float(rank + 1))
    b.fill_(float(10 * (rank + 1)))
    dist.barrier()
    for r in range(world):                                                     # both segments of every peer, through this rank's windows
        assert float(heap.peer_view(a, r)[-1]) == r + 1 and float(heap.peer_view(b, r)[-1]) == 10 * (r + 1)
    dist.barrier()
    # an allocation made outside the heap with the driver's virtual-memory API ...
    gran = hip.get_allocation_granularity(0)
    h = hip.mem_create(gran, 0)
    va = hip.mem_address_reserve(gran)
    hip.mem_map(va, gran, 0, h)
    hip.mem_set_access(va, gran, 0)
    ext = tensor_from_ptr(va, 1024, torch.int32, heap.device)
    ext.copy_(torch.arange(1024, dtype=torch.int32) + 1000 * rank)
    # ... becomes part of the heap without a copy: same memory, second address
    sym = heap.as_symmetric(ext)
    assert heap.is_symmetric(sym) and sym.data_ptr() != ext.data_ptr()
    assert torch.equal(sym, ext)
    ext[0] = -7
    assert int(sym[0]) == -7                                                   # aliases, not copies
    dist.barrier()
    nxt = (rank + 1) % world
    assert int(heap.peer_view(sym, nxt)[1]) == 1 + 1000 * nxt and int(heap.peer_view(sym, nxt)[0]) == -7
    c = heap.allocate(16, torch.float32)                                       # later allocations come after the imported segment
    assert heap.offset_of(c) >= heap.offset_of(sym) + sym.numel() * 4
    with pytest.raises(MemoryError):
        heap.allocate(40 << 20, torch.uint8)                                   # beyond the reserved address space
    dist.barrier()
    del a, b, c, sym, ext
    heap.close()
    hip.mem_unmap(va, gran)
    hip.mem_address_free(va, gran)
    hip.mem_release(h)


def test_growable_vmm_heap_and_zero_copy_import_on_the_host_memory_driver():
    run_ranks(_vmm_growth, 2, env={"IRIS_FAKE_DRIVER_DEVICES": "2", "IRIS_VMEM_INITIAL": str(2 << 20), "IRIS_VMEM_CHUNK": str(4 << 20)},
              timeout=120.0)
