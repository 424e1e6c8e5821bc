#!/usr/bin/env bash
# In-tree build for B200 (sm_100a) only.  Successor of the reference's build.sh:1-7, which
# exports include paths and TORCH_CUDA_ARCH_LIST="9.0a" before `pip install ./kernels`.
set -euo pipefail
cd "$(dirname "$0")"
export TORCH_CUDA_ARCH_LIST="10.0a"
python build_native.py "$@"
