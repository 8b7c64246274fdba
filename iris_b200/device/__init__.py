"""Python handles of the device API.

The device-side API of this framework is the CUDA C++ header library ``include/iris/iris.cuh``;
user kernels are written in CUDA C++ and compiled with ``iris_b200.jit``. The names the reference
exports at top level for use inside Triton kernels (``iris.load``, ``iris.store``,
``iris.DeviceContext`` ...; iris/__init__.py:55-69) are kept here as descriptors that say which
header symbol implements them, so that ``iris.load.__doc__`` and ``iris.load.cuda`` answer the
question "where did this go"; calling one from Python raises with that pointer. One-sided
operations from the host are ``ctx.rma.load/store/...``.
"""
from __future__ import annotations


class DeviceSymbol:
    """A device-library symbol: ``name`` in namespace ``iris`` of ``header``."""

    def __init__(self, name: str, header: str, signature: str):
        self.name, self.header, self.signature = name, header, signature
        self.cuda = f"iris::{name}"
        self.__doc__ = f"Device function {self.cuda} ({header}): {signature}"

    def __call__(self, *a, **k):
        raise RuntimeError(
            f"{self.cuda} is device code ({self.header}); call it from a CUDA C++ kernel compiled with iris_b200.jit, "
            f"or use ctx.rma.{self.name} for a one-sided operation issued from the host"
        )

    def __repr__(self):
        return f"<device symbol {self.cuda}: {self.signature}>"


_RMA = "include/iris/rma.cuh"
load = DeviceSymbol("load", _RMA, "T load(const T* ptr, int to_rank, int from_rank, const uint64_t* heap_bases, bool pred, T other)")
store = DeviceSymbol("store", _RMA, "void store(T* ptr, T value, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
copy = DeviceSymbol("copy", _RMA, "void copy(const T* src, T* dst, int from_rank, int to_rank, int cur_rank, const uint64_t* heap_bases, bool pred)")
get = DeviceSymbol("get", _RMA, "void get(const T* from_ptr, T* to_ptr, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
put = DeviceSymbol("put", _RMA, "void put(const T* from_ptr, T* to_ptr, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
atomic_add = DeviceSymbol("atomic_add", _RMA, "T atomic_add<Sem, Scope>(T* ptr, T val, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
atomic_sub = DeviceSymbol("atomic_sub", _RMA, "T atomic_sub<Sem, Scope>(T* ptr, T val, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
atomic_cas = DeviceSymbol("atomic_cas", _RMA, "T atomic_cas<Sem, Scope>(T* ptr, T cmp, T val, int from_rank, int to_rank, const uint64_t* heap_bases)")
atomic_xchg = DeviceSymbol("atomic_xchg", _RMA, "T atomic_xchg<Sem, Scope>(T* ptr, T val, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
atomic_xor = DeviceSymbol("atomic_xor", _RMA, "T atomic_xor<Sem, Scope>(T* ptr, T val, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
atomic_or = DeviceSymbol("atomic_or", _RMA, "T atomic_or<Sem, Scope>(T* ptr, T val, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
atomic_and = DeviceSymbol("atomic_and", _RMA, "T atomic_and<Sem, Scope>(T* ptr, T val, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
atomic_min = DeviceSymbol("atomic_min", _RMA, "T atomic_min<Sem, Scope>(T* ptr, T val, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
atomic_max = DeviceSymbol("atomic_max", _RMA, "T atomic_max<Sem, Scope>(T* ptr, T val, int from_rank, int to_rank, const uint64_t* heap_bases, bool pred)")
DeviceContext = DeviceSymbol("DeviceContext", "include/iris/context.cuh", "struct DeviceContext { static DeviceContext initialize(const int64_t* ctx, bool tracing); translate/remote/mc ... }")
Context = DeviceSymbol("Ctx", "include/iris/iris.cuh", "struct Ctx { load/store/get/put/copy/atomic_* with the caller's rank implied }")
Tile = DeviceSymbol("TileView", "include/iris/types.cuh", "struct TileView { pid_m, pid_n, block_m, block_n } (a tile's data lives in registers / TMEM)")
TileView = DeviceSymbol("TileView", "include/iris/types.cuh", "struct TileView { pid_m, pid_n, block_m, block_n }")
TensorView = DeviceSymbol("TensorView", "include/iris/types.cuh", "template <class T> struct TensorView { ptr, M, N, stride_m, stride_n }")
AllReduceConfig = DeviceSymbol("AllReduceConfig", "include/iris/types.cuh", "struct AllReduceConfig { variant_code, locks_ptr }")
make_tensor_view = DeviceSymbol("make_tensor_view", "include/iris/types.cuh", "TensorView<T> make_tensor_view(T* ptr, int M, int N, int64_t stride_m, int64_t stride_n)")

# Device-side tracing aggregate and intrinsics (reference: iris/mem/triton/tracing.py:19-186, iris/mem/utils.py:25-92).
Tracing = DeviceSymbol("Tracing", "include/iris/tracing.cuh", "struct Tracing { int record_event_start(event_id, target_rank, address, pid_m, pid_n, payload_bytes); void record_event_end(int handle); }")
read_realtime = DeviceSymbol("read_realtime", "include/iris/iris.cuh", "uint64_t read_realtime()  // nanoseconds of %globaltimer")
get_cu_id = DeviceSymbol("get_cu_id", "include/iris/iris.cuh", "uint32_t get_cu_id()  // %smid")
get_xcc_id = DeviceSymbol("get_xcc_id", "include/iris/iris.cuh", "uint32_t get_xcc_id()  // always 0: a B200 exposes no chiplet partition")
# Flag helpers every kernel of this library waits with (no counterpart in the reference, which spins on atomic_cas).
wait_flag_ge = DeviceSymbol("wait_flag_ge", "include/iris/sync.cuh", "bool wait_flag_ge(const DeviceContext& ctx, const int32_t* flag, int32_t target)  // bounded by ctx.timeout_ns")
