#!/usr/bin/env bash
# CPU tests first, then the GPU tests if a GPU is present.  Multi-GPU cases start their own ranks.
set -euo pipefail
cd "$(dirname "$0")/.."
python -m multimodal_training_b200.csrc.build
python -m pytest tests -q -m "not gpu"
if python -c "import torch, sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
    python -m pytest tests -q -m gpu
else
    echo "no GPU visible: skipped the GPU tests"
fi
