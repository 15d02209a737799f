#!/bin/bash
# Builds the CUDA kernels in-tree for sm_100a and checks the Python dependencies. No package index is contacted:
# everything this framework needs beyond PyTorch is optional and is checked when the feature is used.
set -euo pipefail
cd "$(dirname "$0")"
python - <<'PY'
from maxdiffusion_b200.dependency_versions_check import check_required
check_required()
from maxdiffusion_b200 import build
print("kernels built:", build.build(verbose=True))
PY
