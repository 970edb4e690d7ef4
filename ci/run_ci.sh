#!/usr/bin/env bash
# Continuous-integration entry: build the native libraries, run the CPU suite everywhere and the GPU suite when a
# CUDA device is visible.  Mirrors the role of the reference's ci/run_ci.sh.
set -euo pipefail
cd "$(dirname "$0")/.."
python -m mindspeed_b200.ops.build
python -m pytest tests -q -m "not gpu" "$@"
if python -c 'import torch,sys; sys.exit(0 if torch.cuda.is_available() else 1)'; then
  python -m pytest tests -q -m gpu "$@"
fi
