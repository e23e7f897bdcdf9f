#!/bin/sh
# Builds the unmodified reference (CMake, Release, AVX2) from a scratch copy and installs its static libraries plus the
# config-1 timing harness into baseline/_ref/ (git-ignored).
# Usage: baseline/build_reference.sh <reference tree>      (or TFB_REFERENCE_SRC=<reference tree>)
set -e
here="$(cd "$(dirname "$0")" && pwd)"
src="${1:-$TFB_REFERENCE_SRC}"
if [ -z "$src" ] || [ ! -d "$src" ]; then
  echo "usage: $0 <path of the reference source tree>" >&2
  exit 2
fi
work="$(mktemp -d /tmp/tfb_ref_build.XXXXXX)"
cp -r "$src" "$work/src"
cmake -S "$work/src" -B "$work/build" -DCMAKE_BUILD_TYPE=Release -DQUANT_AVX2=ON -DQUANT_BUILD_TESTS=OFF \
      -DQUANT_BUILD_BENCHMARKS=OFF -DQUANT_BUILD_TOOLS=OFF > "$work/cmake.log" 2>&1
cmake --build "$work/build" -j 8 --target quant_inference quant_model quant_kernel quant_math quant_format quant_core \
      quant_tokenizer > "$work/build.log" 2>&1
mkdir -p "$here/_ref/lib" "$here/_ref/bin"
find "$work/build" -name 'libquant_*.a' -exec cp {} "$here/_ref/lib/" \;
L="$here/_ref/lib"
g++ -O2 -std=c++20 -mavx2 -mfma -I "$work/src/include" -I "$work/build" "$here/ref_gpt2_cpu.cpp" -o "$here/_ref/bin/ref_gpt2_cpu" \
    -Wl,--start-group "$L"/libquant_*.a -Wl,--end-group -pthread
echo "installed: $here/_ref/bin/ref_gpt2_cpu"
