#!/usr/bin/env python3
"""Writes docs/api_reference.md from the docstrings of the public host API (no GPU needed)."""
import importlib
import inspect
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

MODULES = [
    "iris_b200.host.iris", "iris_b200.host.heap", "iris_b200.host.rma", "iris_b200.host.tracing", "iris_b200.host.topology",
    "iris_b200.host.platform", "iris_b200.host.artifacts", "iris_b200.ccl", "iris_b200.ccl.config", "iris_b200.ops",
    "iris_b200.ops.config", "iris_b200.ops.gemm", "iris_b200.ops.gemm_fp8", "iris_b200.ops.workspace",
    "iris_b200.models.flash_decode", "iris_b200.models.moe", "iris_b200.models.ring_attention", "iris_b200.models.tp_mlp", "iris_b200.bench._core",
    "iris_b200.bench._runner", "iris_b200.jit", "iris_b200.drivers",
    "iris_b200.parallel.layout", "iris_b200.parallel.tensor_parallel", "iris_b200.parallel.data_parallel",
    "iris_b200.parallel.sequence_parallel", "iris_b200.parallel.expert_parallel", "iris_b200.parallel.p2p", "iris_b200.host.watchdog",
    "iris_b200.utils.validation",
    "iris_b200.utils.records", "iris_b200.utils.roofline", "iris_b200.utils.timing",
]


def first(doc):
    return inspect.cleandoc(doc).split("\n\n")[0].replace("\n", " ") if doc else ""


def sig(fn):
    try:
        return str(inspect.signature(fn))
    except (TypeError, ValueError):
        return "(...)"


def main():
    out = ["# API reference (generated from the docstrings: `python docs/gen_api_reference.py`)\n",
           "Signatures of the public host API. The device API (`include/iris/iris.cuh`) is described in `programming_model.md`.\n"]
    for name in MODULES:
        m = importlib.import_module(name)
        out.append(f"\n## `{name}`\n\n{first(m.__doc__)}\n")
        names = getattr(m, "__all__", None) or [n for n, o in vars(m).items()
                                                 if not n.startswith("_") and getattr(o, "__module__", None) == name]
        for n in names:
            o = getattr(m, n, None)
            if inspect.isclass(o):
                out.append(f"\n### class `{n}`\n\n{first(o.__doc__)}\n")
                for k, v in vars(o).items():
                    if inspect.isfunction(v) and not k.startswith("_"):
                        out.append(f"* `{k}{sig(v)}` - {first(v.__doc__)}")
            elif inspect.isfunction(o):
                out.append(f"\n### `{n}{sig(o)}`\n\n{first(o.__doc__)}\n")
    with open(os.path.join(ROOT, "docs", "api_reference.md"), "w") as f:
        f.write("\n".join(out) + "\n")


if __name__ == "__main__":
    main()
