#!/usr/bin/env bash
# Installs the package from this checkout into the active Python environment and compiles the sm_100a kernel library
# and the host runtime in place.  Needs nvcc (CUDA 12.8 or newer) and a PyTorch build with CUDA already installed;
# nothing is fetched from a package index.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)"
command -v nvcc >/dev/null || { echo "nvcc not found: put CUDA 12.8+ on PATH or set NVCC" >&2; exit 1; }
python -c 'import torch, sys; sys.exit(0 if torch.version.cuda else 1)' || { echo "PyTorch with CUDA support is required" >&2; exit 1; }
python -m pip install --no-deps --no-build-isolation --no-index -e "$here"
python -m aspec_b200.build
python -m aspec_b200.cli doctor
