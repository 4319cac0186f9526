#!/usr/bin/env bash
# Test infrastructure only -- not part of the shipped library.
#
# Builds the reference's OWN autodiff layer (dali/tensor: Tensor, the tape and
# the tensor_ops that are alive in the reference) from the sources where they
# lie in the reference checkout, UNCHANGED, against the B200 front end's headers
# (dali_b200/host/include) instead of the reference's dali/array, and links it
# with libdali_b200.so.  What comes out shows that code written against the
# reference's Array API -- here the reference's own caller of the hot path --
# compiles and runs on the new back end:
#
#   oracle/_ref/libdali_tensor_on_b200.so   the reference's dali/tensor objects
#   oracle/_ref/tensor_layer_smoke          tests/cpp/tensor_layer_smoke.cpp linked
#                                           against it (run by the GPU tests)
#
# Nothing of the reference is written anywhere but oracle/_ref/ (git-ignored).
# Left out: op/cost.cpp (does not compile against the reference's own headers
# either: op::eltmax, three-argument op::softmax and Array::insert_broadcast_axis
# do not exist there) and op/spatial.cpp (convolution / pooling: cuDNN side of the
# reference).
set -euo pipefail

HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(cd "$HERE/../.." && pwd)"
REF="${DALI_REFERENCE_DIR:-/root/reference}"
OUT="$ROOT/oracle/_ref"
CXX="${CXX:-g++}"
LIBDIR="$ROOT/dali_b200/lib"
SMOKE_SRC="$ROOT/tests/cpp/tensor_layer_smoke.cpp"

if [ ! -d "$REF/dali/tensor" ]; then
    echo "build_tensor_layer: no reference checkout at $REF -- keeping whatever is in $OUT" >&2
    exit 0
fi
if [ ! -f "$LIBDIR/libdali_b200.so" ]; then
    echo "build_tensor_layer: build the library first (python -m dali_b200.build)" >&2
    exit 1
fi
if [ -x "$OUT/tensor_layer_smoke" ] && [ "$OUT/tensor_layer_smoke" -nt "$SMOKE_SRC" ] \
   && [ "$OUT/tensor_layer_smoke" -nt "$LIBDIR/libdali_b200.so" ] \
   && [ "$OUT/libdali_tensor_on_b200.so" -nt "$HERE/build_tensor_layer.sh" ] \
   && [ "$OUT/libdali_tensor_on_b200.so" -nt "$HERE/shims.cpp" ] && [ -z "${FORCE:-}" ]; then
    echo "build_tensor_layer: $OUT is up to date"
    exit 0
fi

STAGE="$(mktemp -d "${TMPDIR:-/tmp}/dali_tensor_stage.XXXXXX")"
trap 'rm -rf "$STAGE"' EXIT
mkdir -p "$OUT" "$STAGE/obj" "$STAGE/inc/dali/array/gemm" "$STAGE/inc/dali/array/op"

# include tree: dali/tensor and two header-only pieces of dali/array come from the reference (links, no copies);
# everything else under dali/array and dali/utils resolves to the B200 front end's headers
ln -s "$REF/dali/tensor" "$STAGE/inc/dali/tensor"
ln -s "$REF/dali/array/gemm/tensordot_as_dot.h" "$STAGE/inc/dali/array/gemm/tensordot_as_dot.h"
ln -s "$REF/dali/array/op/spatial_enums.h" "$STAGE/inc/dali/array/op/spatial_enums.h"
# force-included standard headers: dali/tensor/tape.h names size_t, solver.cpp std::transform and
# solver_updates/adam.cpp std::pow / sqrt without including <cstddef>, <algorithm>, <cmath>
INC="-include cstddef -include algorithm -include cmath -I$ROOT/dali_b200/host/include -I$HERE/include -I$STAGE/inc"

SRCS="dali/tensor/tape.cpp dali/tensor/tensor.cpp dali/tensor/op/unary.cpp dali/tensor/op/binary.cpp
      dali/tensor/op/reducers.cpp dali/tensor/op/dot.cpp dali/tensor/op/reshape.cpp dali/tensor/op/composite.cpp
      dali/tensor/op/other.cpp dali/tensor/op/dropout.cpp dali/array/gemm/tensordot_as_dot.cpp
      dali/tensor/solver.cpp dali/tensor/op/solver_updates/sgd.cpp dali/tensor/op/solver_updates/adagrad.cpp
      dali/tensor/op/solver_updates/rmsprop.cpp dali/tensor/op/solver_updates/adadelta.cpp
      dali/tensor/op/solver_updates/adam.cpp dali/tensor/op/solver_updates/clip_and_regularize.cpp"
pids=""
for src in $SRCS; do
    obj="$STAGE/obj/$(echo "$src" | tr '/' '_').o"
    ( $CXX -std=c++14 -O1 -w -fPIC $INC -c "$REF/$src" -o "$obj" 2> "$obj.log" || { echo "FAILED $src"; cat "$obj.log"; exit 1; } ) &
    pids="$pids $!"
done
for p in $pids; do wait "$p"; done
$CXX -std=c++14 -O1 -w -fPIC $INC -c "$HERE/shims.cpp" -o "$STAGE/obj/shims.o"

$CXX -shared -o "$OUT/libdali_tensor_on_b200.so" "$STAGE"/obj/*.o -L"$LIBDIR" -ldali_b200 \
    -Wl,--no-undefined -Wl,-rpath,'$ORIGIN/../../dali_b200/lib'

$CXX -std=c++14 -O1 -w $INC "$SMOKE_SRC" -o "$OUT/tensor_layer_smoke" \
    -L"$OUT" -ldali_tensor_on_b200 -L"$LIBDIR" -ldali_b200 \
    -Wl,-rpath,'$ORIGIN' -Wl,-rpath,'$ORIGIN/../../dali_b200/lib'
echo "build_tensor_layer: built $OUT/libdali_tensor_on_b200.so and $OUT/tensor_layer_smoke"

