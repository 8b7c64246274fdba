#!/usr/bin/env bash
# Runs the test suites the way CI does.
#   tests/run_tests.sh cpu     build + every test that needs no GPU (gloo ranks, fakes)
#   tests/run_tests.sh gpu     every GPU test on the visible B200s (multi-GPU tests use up to 4)
#   tests/run_tests.sh all     both
set -euo pipefail
cd "$(dirname "$0")/.."
what="${1:-cpu}"
python -m iris_b200._build
if [ "$what" = "cpu" ] || [ "$what" = "all" ]; then
  python -m pytest tests -x -q -m "not gpu"
fi
if [ "$what" = "gpu" ] || [ "$what" = "all" ]; then
  IRIS_TIMEOUT_MS="${IRIS_TIMEOUT_MS:-3000}" python -m pytest tests -x -q -m gpu
fi
