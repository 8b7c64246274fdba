#!/usr/bin/env bash
# Runs the test suites the way CI does.
#   tests/run_tests.sh cpu     build + every test that needs no GPU (gloo ranks, fakes), then the RMA and
#                              collective tests once more on the VMM heap of the host-memory driver stand-in
#   tests/run_tests.sh gpu     every GPU test on the visible B200s (multi-GPU tests use up to 4)
#   tests/run_tests.sh all     both
set -euo pipefail
cd "$(dirname "$0")/.."
what="${1:-cpu}"
python -m iris_b200._build
if [ "$what" = "cpu" ] || [ "$what" = "all" ]; then
  python -m pytest tests -x -q -m "not gpu"
  IRIS_FAKE_DRIVER_DEVICES=8 python -m pytest tests/test_cpu_rma.py tests/test_cpu_rma_sweep.py tests/test_cpu_process_groups.py -x -q
fi
if [ "$what" = "gpu" ] || [ "$what" = "all" ]; then
  IRIS_TIMEOUT_MS="${IRIS_TIMEOUT_MS:-3000}" python -m pytest tests -x -q -m gpu
fi
