#!/usr/bin/env bash
# Builds the UNMODIFIED reference extension (its two shipped translation units)
# for sm_100a from the sources where they lie, into oracle/_ref/ only.
# The result, oracle/_ref/mor_ref_C.so, registers the reference's own
# torch.ops.mor.* operators (CUDA dispatch key only).  It is test infrastructure:
# only tests/golden/make_gpu_golden.py loads it, in a process of its own, to record
# the reference's outputs on a GPU.  Nothing in the product imports it.
#
# usage: oracle/build_ref.sh [reference_root]
#        (default: $MOR_REFERENCE_ROOT, else the folder "reference" beside this repository)
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${1:-${MOR_REFERENCE_ROOT:-$(dirname "$(dirname "$HERE")")/reference}}"
OUT="$HERE/_ref"
mkdir -p "$OUT"
TI="$(python -c 'import torch,os;print(os.path.dirname(torch.__file__))')"
PYINC="$(python -c 'import sysconfig;print(sysconfig.get_paths()["include"])')"
INC=(-I"$TI/include" -I"$TI/include/torch/csrc/api/include" -I/usr/local/cuda/include -I"$PYINC")
DEFS=(-DTORCH_EXTENSION_NAME=mor_ref_C -DTORCH_API_INCLUDE_EXTENSION_H)
# -O3 only, no fast-math, asserts left on: the flags of the reference's setup.py.
nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a --expt-relaxed-constexpr \
     -Xcompiler -fPIC "${DEFS[@]}" "${INC[@]}" \
     -c "$REF/mor/csrc/cuda/fake_quantize.cu" -o "$OUT/fq_cuda.o"
g++ -O2 -std=c++17 -fPIC "${DEFS[@]}" "${INC[@]}" \
     -c "$REF/mor/csrc/fake_quantize.cpp" -o "$OUT/fq_cpp.o"
g++ -shared "$OUT/fq_cuda.o" "$OUT/fq_cpp.o" -L"$TI/lib" -L/usr/local/cuda/lib64 \
     -Wl,-rpath,"$TI/lib" -lc10 -lc10_cuda -ltorch -ltorch_cpu -ltorch_cuda -ltorch_python -lcudart \
     -o "$OUT/mor_ref_C.so"
rm -f "$OUT/fq_cuda.o" "$OUT/fq_cpp.o"
echo "built $OUT/mor_ref_C.so"
