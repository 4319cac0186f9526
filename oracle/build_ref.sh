#!/usr/bin/env bash
# Test infrastructure only -- not part of the shipped library.
#
# Builds the reference's OWN CPU implementation of the hot path (lazy Array /
# op:: expression -> canonical() -> JIT -> run, plus op::dot) from the sources
# where they lie in the reference checkout, into oracle/_ref/ :
#
#   oracle/_ref/libdali_ref.so   the reference's dali/array + dali/utils, CPU only
#   oracle/_ref/ref_driver       oracle/ref_driver.cpp linked against it
#   oracle/_ref/include/         the five headers the reference's run-time JIT
#                                #includes when it shells out to g++
#   oracle/_ref/cache/           the reference's JIT module cache (pre-warmed by
#                                oracle/warm_ref_cache.sh so that a machine
#                                without the checkout can still run the driver)
#
# Nothing of the reference is written anywhere else; oracle/_ref/ is
# git-ignored.  The reference's CMake build is NOT used (it needs GoogleTest,
# a system BLAS and two un-vendored submodules); this script repeats by hand
# what its virtual source tree does (CMakeLists.txt:295-343: *.cu.cpp -> *.cpp
# for a CPU build, *.cu skipped) on a throw-away copy under $TMPDIR, with:
#   * dali/config.h written by hand from dali/config.h.in (CUDA off, 0 GPUs);
#   * oracle/shims/ for libcuckoo, cblas.h, the dangling "uniform.h" include
#     and a force-included fixups.h;
#   * three behaviour-neutral edits of the throw-away copy: U+00A0 bytes in
#     jit/scalar_view.cpp and op/softmax.cpp become spaces, and the JIT's
#     "cmd &> log" (bash-only; /bin/sh backgrounds it and the dlopen retry
#     loop then spins) becomes "cmd > log 2>&1" in utils/compiler.cpp.
set -euo pipefail

HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${DALI_REFERENCE_DIR:-/root/reference}"
OUT="$HERE/_ref"
JOBS="${JOBS:-$(nproc)}"
CXX="${CXX:-g++}"

if [ ! -d "$REF/dali/array" ]; then
    echo "build_ref: no reference checkout at $REF -- keeping whatever is in $OUT" >&2
    exit 0
fi
if [ -x "$OUT/ref_driver" ] && [ "$OUT/ref_driver" -nt "$HERE/ref_driver.cpp" ] \
   && [ "$OUT/libdali_ref.so" -nt "$HERE/build_ref.sh" ] && [ -z "${FORCE:-}" ]; then
    echo "build_ref: $OUT is up to date"
    exit 0
fi

STAGE="$(mktemp -d "${TMPDIR:-/tmp}/dali_ref_stage.XXXXXX")"
trap 'rm -rf "$STAGE"' EXIT
mkdir -p "$OUT/include/dali/array/jit" "$OUT/cache" "$STAGE/obj"

# 1. throw-away mirror of dali/ (headers + CPU sources, tests left out)
(cd "$REF" && find dali -type f \( -name '*.h' -o -name '*.cpp' \) \
    ! -name '*tests*' ! -name 'tests_main.cpp' ! -path '*/tests/*' -print0) |
while IFS= read -r -d '' f; do
    dst="$STAGE/${f%.cu.cpp}"
    case "$f" in *.cu.cpp) dst="$dst.cpp";; *) dst="$STAGE/$f";; esac
    mkdir -p "$(dirname "$dst")"
    cp "$REF/$f" "$dst"
done

# 2. config.h by hand
cat > "$STAGE/dali/config.h" <<EOF
#ifndef DALI_CONFIG_H
#define DALI_CONFIG_H
#define DALI_DATA_DIR $REF/data
#define DALI_MAX_GPU_DEVICES 0
#define WITH_PRETTY_STACKTRACES 0
#define DALI_APPLE_STACKTRACES 0
#define DALI_COMPILE_DIRECTORY $OUT/include
#define DALI_CXX_COMPILER $(command -v "$CXX")
#define DALI_CUDA_CXX_COMPILER compiled_without_cuda
#define DALI_CXX_COMPILER_ID gnu
#define DALI_BLAS_INCLUDE_DIRECTORY $OUT/include
#define DALI_CUDA_VERSION 0
#define EXISTS_AND_TRUE(VAR) 7-VAR-7 == -1
#endif
EOF

# 3. behaviour-neutral edits of the throw-away copy
sed -i 's/\xc2\xa0/ /g' "$STAGE/dali/array/jit/scalar_view.cpp" "$STAGE/dali/array/op/softmax.cpp"
sed -i 's/" -O3 &> ", logfile/" -O3 > ", logfile, " 2>\&1"/g' "$STAGE/dali/utils/compiler.cpp"
grep -q '2>&1' "$STAGE/dali/utils/compiler.cpp"

# 4. headers the run-time JIT needs (git-ignored output)
for h in dali/array/jit/array_view.h dali/array/jit/reducer_kernels.h dali/array/functor.h dali/macros.h dali/config.h; do
    mkdir -p "$OUT/include/$(dirname "$h")"
    cp "$STAGE/$h" "$OUT/include/$h"
done

# 5. compile dali/array + dali/utils + runtime_config (CPU only)
CXXFLAGS="-std=c++11 -O1 -w -fPIC -include $HERE/shims/fixups.h -I$STAGE -I$HERE/shims -DDALI_CACHE_DIR=$OUT/cache/"
(cd "$STAGE" && { find dali/array dali/utils -name '*.cpp'; echo dali/runtime_config.cpp; }) > "$STAGE/srcs.txt"
compile_one() {
    src="$1"; obj="$STAGE/obj/$(echo "$src" | tr '/' '_').o"
    $CXX $CXXFLAGS -c "$STAGE/$src" -o "$obj" 2> "$obj.log" || { echo "FAILED $src"; cat "$obj.log"; exit 1; }
}
export -f compile_one; export CXX CXXFLAGS STAGE
xargs -a "$STAGE/srcs.txt" -P "$JOBS" -I{} bash -c 'compile_one {}'

# 6. BLAS: an LP64 OpenBLAS exporting plain cblas_sgemm if one is around, else mini_cblas.c
BLAS_ARGS=""
CANDS="$(python -c 'import glob, site
for sp in site.getsitepackages():
    for p in sorted(glob.glob(sp + "/opencv_python_headless.libs/libopenblas*.so")):
        print(p)' 2>/dev/null || true)"
for cand in $CANDS; do
    SYMS="$(nm -D "$cand" 2>/dev/null || true)"
    if grep -q ' T cblas_sgemm$' <<< "$SYMS"; then
        BLAS_ARGS="$cand -Wl,--disable-new-dtags -Wl,-rpath,$(dirname "$cand")"; echo "build_ref: BLAS = $cand"; break
    fi
done
if [ -z "$BLAS_ARGS" ]; then
    echo "build_ref: no OpenBLAS found, using oracle/shims/mini_cblas.c"
    gcc -O3 -fPIC -I"$HERE/shims" -c "$HERE/shims/mini_cblas.c" -o "$STAGE/mini_cblas.o"
    BLAS_ARGS="$STAGE/mini_cblas.o"
fi
echo "$BLAS_ARGS" | awk '{print $1}' > "$OUT/blas.txt"

$CXX -shared -o "$OUT/libdali_ref.so" "$STAGE"/obj/*.o $BLAS_ARGS -lz -ldl -lpthread

# 7. the driver (our code, written against the reference's public API)
$CXX -std=c++11 -O2 -w -include "$HERE/shims/fixups.h" -I"$STAGE" -I"$HERE/shims" \
    "$HERE/ref_driver.cpp" -o "$OUT/ref_driver" \
    -L"$OUT" -ldali_ref -Wl,-rpath,'$ORIGIN' $BLAS_ARGS -lz -ldl -lpthread
echo "build_ref: built $OUT/libdali_ref.so and $OUT/ref_driver"
