#!/usr/bin/env bash
# Builds the REFERENCE's own CUDA extension (csrc/btp/_bindings.cu, which #includes both kernel files)
# for sm_100, straight from the reference checkout, into oracle/_ref/_btp.so.  Test infrastructure: it
# is the GPU yardstick ("kernel to beat" and "the reference kernel's own error") that
# oracle/compare_reference_kernel.py runs next to this repository's kernels.  Nothing is copied into the
# repository; oracle/_ref/ is git-ignored.  Needs: nvcc, torch headers, CUTLASS headers (the image ships
# them inside the flashinfer wheel).  One translation unit, about four minutes.
#
#   oracle/build_reference_kernel.sh /path/to/reference      (or set SPEAR_REFERENCE)
set -euo pipefail
REF="${1:-${SPEAR_REFERENCE:?give the path of the reference checkout}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
mkdir -p "$OUT"
PY="${PYTHON:-python}"
TORCH_INC=$($PY - <<'PYEOF'
from torch.utils.cpp_extension import include_paths
print(" ".join("-I" + p for p in include_paths()))
PYEOF
)
TORCH_LIB=$($PY -c "import torch, os; print(os.path.join(os.path.dirname(torch.__file__), 'lib'))")
PY_INC=$($PY -c "import sysconfig; print(sysconfig.get_paths()['include'])")
CXX11=$($PY -c "import torch; print(int(torch._C._GLIBCXX_USE_CXX11_ABI))")
CUTLASS_INC="${CUTLASS_INCLUDE_PATH:-$($PY -c "import flashinfer, os; print(os.path.join(os.path.dirname(flashinfer.__file__), 'data', 'cutlass', 'include'))")}"
nvcc -O3 --use_fast_math -std=c++17 -gencode arch=compute_100,code=sm_100 --expt-relaxed-constexpr \
  $TORCH_INC -I"$PY_INC" -I"$CUTLASS_INC" -I"$REF/csrc" \
  -DTORCH_EXTENSION_NAME=_btp -DTORCH_API_INCLUDE_EXTENSION_H=1 -D_GLIBCXX_USE_CXX11_ABI=$CXX11 \
  -Xcompiler -fPIC -shared "$REF/csrc/btp/_bindings.cu" -o "$OUT/_btp.so" \
  -L"$TORCH_LIB" -ltorch -ltorch_cpu -ltorch_cuda -lc10 -lc10_cuda -ltorch_python --threads 4 \
  -Xlinker -rpath -Xlinker "$TORCH_LIB"
echo "built $OUT/_btp.so"
