#!/bin/sh
# Builds the reference arm of bench.py: dynalm-project/dynalm's CPU engine (no ggml, no server, nothing fetched from
# a network) and baseline/ref_bench.cpp against its two static libraries, into baseline/_ref/.
#   sh baseline/build_reference.sh /path/to/dynalm [build-folder]
set -e
REF=$(cd "$1" && pwd)
HERE=$(cd "$(dirname "$0")" && pwd)
BUILD=${2:-$HERE/_ref/build}
mkdir -p "$HERE/_ref"
cmake -S "$REF" -B "$BUILD" -G Ninja -DCMAKE_BUILD_TYPE=Release -DDYNALM_NATIVE_ONLY=ON -DENABLE_SERVER=OFF \
      -DENABLE_BENCHMARKS=OFF > "$HERE/_ref/cmake.log"
ninja -C "$BUILD" dynalm > "$HERE/_ref/ninja.log"
g++ -std=c++20 -O2 -I"$REF/dynalm/src" -I"$REF/dynacore/include" -I"$BUILD/dynalm/src/generated" \
    "$HERE/ref_bench.cpp" "$BUILD/dynalm/src/libdynalm.a" "$BUILD/dynacore/libdynacore.a" -lpthread \
    -o "$HERE/_ref/ref_bench"
echo "built $HERE/_ref/ref_bench"
