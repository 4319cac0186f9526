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
#   oracle/_ref/libdali_ref_bound.so, ref_driver_bound
#                                the same library and driver with the reference-side binding compiled in
#                                (oracle/ref_binding/): a JITRunner and a MatMul of the reference's own graph
#                                are computed by dali_b200/lib/libdali_b200.so.  Built only when that library
#                                exists; libdali_ref.so itself stays the unmodified reference
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
B200_LIB="$HERE/../dali_b200/lib/libdali_b200.so"
bound_current() {
    [ ! -f "$B200_LIB" ] && return 0          # nothing to bind to yet
    [ -x "$OUT/ref_driver_bound" ] || return 1
    for f in "$HERE"/ref_binding/* "$HERE/ref_driver.cpp" "$HERE/build_ref.sh" "$HERE/../include/dali_b200.h"; do
        [ "$OUT/libdali_ref_bound.so" -nt "$f" ] || return 1
    done
    return 0
}
if [ -x "$OUT/ref_driver" ] && [ "$OUT/ref_driver" -nt "$HERE/ref_driver.cpp" ] \
   && [ "$OUT/libdali_ref.so" -nt "$HERE/build_ref.sh" ] && bound_current && [ -z "${FORCE:-}" ]; then
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

# 8. the same library with the reference-side binding compiled in (oracle/ref_binding/README in the files' headers):
#    patched copies of the two translation units that register the implementations of JITRunner and MatMul
if [ -f "$B200_LIB" ]; then
    mkdir -p "$STAGE/bound/dali/array/jit" "$STAGE/bound/dali/array/gemm" "$STAGE/obj_bound"
    JIT="$STAGE/bound/dali/array/jit/jit.cpp"; GEMM="$STAGE/bound/dali/array/gemm/cpu_gemm.cpp"
    cp "$STAGE/dali/array/jit/jit.cpp" "$JIT"; cp "$STAGE/dali/array/gemm/cpu_gemm.cpp" "$GEMM"
    grep -q '^int registered_jit_runner_impl = register_implementation_default<JITRunner, JITRunnerImpl>();$' "$JIT"
    grep -q '^int cpu_gemm_impl = register_implementation($' "$GEMM"
    # the registration of JITRunnerImpl becomes the binding (which registers itself and keeps JITRunnerImpl as the path for
    # what it does not take); the other places that create a JITRunnerImpl directly create the binding's class too
    sed -i 's|^int registered_jit_runner_impl = register_implementation_default<JITRunner, JITRunnerImpl>();$|#include "jit_b200_binding.inc"|' "$JIT"
    sed -i 's|std::make_shared<JITRunnerImpl>(|std::make_shared<b200_binding::B200RunnerImpl>(|g' "$JIT"
    sed -i 's|^int cpu_gemm_impl = register_implementation($|#include "gemm_b200_binding.inc"\nint cpu_gemm_impl = register_implementation(|' "$GEMM"
    sed -i '1i #include "binding_includes.h"' "$JIT" "$GEMM"
    BFLAGS="$CXXFLAGS -I$HERE/ref_binding -I$HERE/../include"
    $CXX $BFLAGS -I"$STAGE/dali/array/jit" -c "$JIT" -o "$STAGE/obj_bound/jit.o"
    $CXX $BFLAGS -I"$STAGE/dali/array/gemm" -c "$GEMM" -o "$STAGE/obj_bound/cpu_gemm.o"
    OBJS="$(ls "$STAGE"/obj/*.o | grep -v -e 'dali_array_jit_jit.cpp.o$' -e 'dali_array_gemm_cpu_gemm.cpp.o$')"
    B200_DIR="$(cd "$(dirname "$B200_LIB")" && pwd)"
    $CXX -shared -o "$OUT/libdali_ref_bound.so" $OBJS "$STAGE/obj_bound/jit.o" "$STAGE/obj_bound/cpu_gemm.o" $BLAS_ARGS \
        -L"$B200_DIR" -ldali_b200 -Wl,-rpath,'$ORIGIN/../../dali_b200/lib' -lz -ldl -lpthread
    $CXX -std=c++11 -O2 -w -include "$HERE/shims/fixups.h" -I"$STAGE" -I"$HERE/shims" -DREF_DRIVER_BOUND=1 \
        "$HERE/ref_driver.cpp" -o "$OUT/ref_driver_bound" \
        -L"$OUT" -ldali_ref_bound -L"$B200_DIR" -ldali_b200 -Wl,-rpath,'$ORIGIN' -Wl,-rpath,'$ORIGIN/../../dali_b200/lib' $BLAS_ARGS -lz -ldl -lpthread
    echo "build_ref: built $OUT/libdali_ref_bound.so and $OUT/ref_driver_bound"
fi
