"""Build hook: compiles the native libraries in-tree (nvcc for sm_100a, g++ for the runtime) before
the Python package is assembled. `pip install -e .` and `python setup.py build_ext --inplace` both
end up calling `iris_b200._build.build_all`; the headers under `include/` and the sources under
`csrc/` must be present (source checkout). The reference is pure setuptools (pyproject.toml:4-6)."""
import importlib.util
import os

from setuptools import setup
from setuptools.command.build_ext import build_ext
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _build_native():
    spec = importlib.util.spec_from_file_location("_iris_b200_build", os.path.join(HERE, "iris_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build_all(verbose=True)


class BuildNative(build_ext):
    def run(self):
        _build_native()


class BuildPy(build_py):
    def run(self):
        _build_native()
        super().run()


setup(cmdclass={"build_ext": BuildNative, "build_py": BuildPy})
