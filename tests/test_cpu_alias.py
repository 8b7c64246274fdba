"""``import iris`` resolves to this framework (the reference's package name, iris/__init__.py:45-136)."""
import importlib


def test_iris_alias_exposes_the_reference_names():
    import iris
    import iris_b200

    assert iris.iris is iris_b200.iris and iris.Iris is iris_b200.Iris
    for sub in ("ccl", "ops", "bench", "experimental", "gluon", "hip", "tensor_creation"):
        assert importlib.import_module("iris." + sub) is getattr(iris_b200, sub)
    from iris.ccl import Config, ReduceOp  # noqa: F401
    from iris.gluon import IrisDeviceCtx  # noqa: F401
    for name in ("DeviceContext", "Context", "TraceEvent", "Tile", "TileView", "TensorView", "AllReduceConfig", "make_tensor_view",
                 "load", "store", "copy", "get", "put", "atomic_add", "atomic_cas", "atomic_xchg", "atomic_xor", "atomic_or",
                 "atomic_and", "atomic_min", "atomic_max", "do_bench", "get_device_id_for_rank", "is_simulation_env",
                 "CUDAArrayInterface", "tensor_from_ptr", "set_logger_level", "logger", "DEBUG", "INFO", "WARNING", "ERROR"):
        assert getattr(iris, name) is getattr(iris_b200, name), name
