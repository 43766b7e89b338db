#!/bin/bash
# Builds the reference's own GPU GEMM runtime -- its tessera_nvidia_gemm.cpp, unmodified, read where it
# lies in the reference checkout given as the first argument -- into baseline/_ref/ (git-ignored).
# The reference's CMake step that turns aot/tessera_nvidia_mma_f16_sm120_v1.cu into a header with the
# source text and its SHA-256 (runtime/cuda/CMakeLists.txt:30-35) is reproduced by the few lines of
# Python below; nothing of the reference is copied into this repository.
set -euo pipefail
REF=${1:?usage: build_ref_gemm.sh <reference checkout>}
SRC="$REF/src/compiler/codegen/tessera_gpu_backend_NVIDIA/runtime/cuda"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
CUDA=${CUDA_HOME:-/usr/local/cuda}
mkdir -p "$OUT/gen"
python3 - "$SRC/aot/tessera_nvidia_mma_f16_sm120_v1.cu" "$OUT/gen/tessera_nvidia_mma_f16_sm120_v1_source.h" <<'PY'
import hashlib, sys
src, dst = sys.argv[1], sys.argv[2]
data = open(src, "rb").read()
with open(dst, "w") as f:
    f.write("// Generated from tessera_nvidia_mma_f16_sm120_v1.cu.\n")
    f.write('inline constexpr char kSrcF16Aot[] = R"TESSERA_AOT(\n' + data.decode() + '\n)TESSERA_AOT";\n')
    f.write('inline constexpr char kSm120F16AotSourceSha256[] = "' + hashlib.sha256(data).hexdigest() + '";\n')
PY
g++ -std=c++17 -O2 -shared -fPIC -I"$OUT/gen" -I"$CUDA/include" "$SRC/tessera_nvidia_gemm.cpp" \
    -o "$OUT/libtessera_nvidia_gemm.so" -L"$CUDA/lib64" -L"$CUDA/lib64/stubs" -lcuda -lnvrtc -ldl
echo "built $OUT/libtessera_nvidia_gemm.so"
