"""Every example script runs to completion on the CPU backend (two gloo ranks, shared-memory heap):
the scripts validate their own results, so exit code 0 is the assertion."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXAMPLES = ["rma_basics", "tp_mlp_training_step", "ccl_collectives", "ops_fused", "gemm_patterns", "all_reduce_variants", "flash_decode", "moe",
            "ring_attention", "tracing", "parallel_layouts"]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("name", EXAMPLES)
def test_example_runs_on_the_cpu_backend(name):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "examples", name + ".py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
