"""``iris.mem`` of the reference (device-side memory API, iris/mem/{triton,gluon}/*.py and
iris/mem/utils.py): the same symbols as ``iris_b200.device``, under the reference's module path."""
from ..device import (AllReduceConfig, Context, DeviceContext, DeviceSymbol, TensorView, Tile, TileView, Tracing, atomic_add,  # noqa: F401
                      atomic_and, atomic_cas, atomic_max, atomic_min, atomic_or, atomic_sub, atomic_xchg, atomic_xor, copy, get,
                      get_cu_id, get_xcc_id, load, make_tensor_view, put, read_realtime, store, wait_flag_ge)
