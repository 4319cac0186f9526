#!/usr/bin/env bash
# Test infrastructure only -- not part of the shipped library.
#
# Fills the reference's JIT module cache (oracle/_ref/cache/) by running the reference driver once over every kind of
# case the tests and the benchmark's CPU legs use, on small seeded inputs.  The reference compiles one module per
# expression STRUCTURE (rank, dtypes, node types), not per size, so a machine that only receives oracle/_ref/ -- no
# reference checkout -- then loads these modules instead of compiling (it still can: the compiler line and the five
# headers the modules include are part of oracle/_ref/).
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="$HERE/_ref"
[ -x "$REF/ref_driver" ] || { echo "warm_ref_cache: no $REF/ref_driver, nothing to do"; exit 0; }
if [ -n "$(ls -A "$REF/cache" 2>/dev/null | head -1)" ] && [ "$REF/cache" -nt "$REF/libdali_ref.so" ] && [ -z "${FORCE:-}" ]; then
    echo "warm_ref_cache: $REF/cache is warm"
    exit 0
fi
TMP="$(mktemp -d "${TMPDIR:-/tmp}/dali_ref_warm.XXXXXX")"
trap 'rm -rf "$TMP"' EXIT
python - "$TMP" <<'PY'
import sys, os
import numpy as np
tmp = sys.argv[1]
rng = np.random.default_rng(1)
def save(name, a): np.save(os.path.join(tmp, name + ".npy"), a)
save("a", rng.standard_normal((24, 40)).astype(np.float32))
save("x", rng.standard_normal(4096).astype(np.float32))
save("b", rng.standard_normal((40, 16)).astype(np.float32))
save("bias", rng.standard_normal(16).astype(np.float32))
B, H = 8, 16
for k in ("lx", "lh", "lc"): save(k, rng.standard_normal((B, H)).astype(np.float32))
for k in ("Wx", "Wh"): save(k, (rng.standard_normal((H, 4 * H)) * 0.1).astype(np.float32))
save("lb", np.zeros((1, 4 * H), np.float32))
save("src", rng.standard_normal((50, 16)).astype(np.float32))
save("idx", rng.integers(0, 50, (20,)).astype(np.int32))
save("idxr", rng.integers(0, 16, (50,)).astype(np.int32))
save("v", rng.standard_normal(12).astype(np.float32))
save("w", rng.standard_normal(7).astype(np.float32))
PY
run() { (cd "$TMP" && "$REF/ref_driver" "$REF/cache" "$@" > /dev/null 2>&1) || echo "warm_ref_cache: case '$*' failed (ignored)"; }
run unary tanh a.npy o.npy
run unary sigmoid a.npy o.npy
run binary add a.npy a.npy o.npy
run binary eltmul a.npy a.npy o.npy
for op in sum max min argmax argmin mean l2 prod; do for ax in -1 0 all; do run reduce $op $ax a.npy o.npy; done; done
run softmax a.npy o.npy
run softmax_naive a.npy o.npy
run lstm lx.npy lh.npy lc.npy Wx.npy Wh.npy lb.npy co.npy ho.npy
run gemm_tanh a.npy b.npy bias.npy o.npy
run dot a.npy b.npy o.npy
run chain x.npy 0.5 0.1 o.npy
run gather src.npy idx.npy o.npy
run gather_rows src.npy idxr.npy o.npy
run scatter_add src.npy idx.npy o.npy
run outer v.npy w.npy o.npy
run one_hot idx.npy 50 1.0 0.0 o.npy
run unary_t tanh a.npy o.npy
run scan sum 1 a.npy o.npy
run scan sum 0 a.npy o.npy
touch "$REF/cache"
echo "warm_ref_cache: $(ls "$REF/cache" | grep -c '\.so$') modules in $REF/cache"
