// Launch planning: from run-time shapes/strides to a kernel variant + geometry.
//
// Takes over what JITRunnerImpl::run does before it calls the compiled module
// (dali/array/jit/jit.cpp:1146-1164: rank collapse via min_computation_rank /
// jit_right_fit_ndim, :1227-1251) and what the emitted host code does to size
// the grid (:716-772), with 64-bit extents.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <sstream>

#include "runtime.h"

namespace dalib {

namespace {

const int kSMs = 148;   // B200

struct Dim {
    long long extent;
    std::vector<long long> stride;   // per arg
};

// drop extent-1 dims, then merge neighbours that every arg walks contiguously
void collapse(std::vector<Dim>* dims) {
    std::vector<Dim> out;
    for (const Dim& d : *dims)
        if (d.extent != 1) out.push_back(d);
    bool merged = true;
    while (merged && out.size() > 1) {
        merged = false;
        for (size_t i = 0; i + 1 < out.size(); ++i) {
            bool ok = true;
            for (size_t a = 0; a < out[i].stride.size(); ++a)
                ok = ok && out[i].stride[a] == out[i + 1].stride[a] * out[i + 1].extent;
            if (ok) {
                out[i + 1].extent *= out[i].extent;
                out.erase(out.begin() + i);
                merged = true;
                break;
            }
        }
    }
    *dims = out;
}

int pow2_ceil(long long x) {
    int p = 1;
    while (p < x && p < (1 << 30)) p <<= 1;
    return p;
}

// tuning overrides for experiments: DALI_B200_<NAME>=<int>
int env_int(const char* name, int fallback) {
    const char* e = std::getenv(name);
    return e && *e ? std::atoi(e) : fallback;
}

int ilog2(int x) {
    int l = 0;
    while ((1 << l) < x) ++l;
    return l;
}

}  // namespace

std::string LaunchPlan::describe() const {
    std::ostringstream s;
    s << variant.key() << " grid=" << grid_x << "x" << grid_y << " R=" << (words.size() > 0 ? words[0] : 0)
      << " C=" << (words.size() > 1 ? words[1] : 0);
    return s.str();
}

bool plan_launch(const Program& p, const int64_t* space, int rank,
                 void* const* array_data, const int64_t* offsets,
                 const int64_t* const* strides, int n_arrays,
                 const void* const* scalars, int n_scalars,
                 LaunchPlan* plan, std::string* err) {
    if (p.has_acc) { *err = "launch: this program reads a GEMM accumulator; run it through dalib200_gemm_fused"; return false; }
    for (const Stmt& st_ : p.stmts)
        if (st_.kind == S_STX && p.args[st_.arg].dtype == BF16) { *err = "launch: no scatter into a bf16 array (there is no 16-bit atomic path)"; return false; }
    if (rank != p.rank) { *err = "launch: space rank differs from the program's"; return false; }
    if (n_arrays != (int)p.args.size()) { *err = "launch: wrong number of arrays"; return false; }
    if (n_scalars != (int)p.scalars.size()) { *err = "launch: wrong number of scalars"; return false; }
    const int nargs = n_arrays;
    long long total = 1;
    for (int d = 0; d < rank; ++d) {
        if (space[d] < 0) { *err = "launch: negative extent"; return false; }
        total *= space[d];
    }
    LaunchPlan out;
    if (total == 0) {
        if (p.nreduce > 0) { *err = "launch: reduction over an empty space"; return false; }
        out.empty = true;
        *plan = out;
        return true;
    }

    // per-arg strides in space coordinates
    std::vector<std::vector<long long>> st(nargs, std::vector<long long>(rank, 0));
    const int n_outer_dims = rank - p.nreduce;
    for (int a = 0; a < nargs; ++a) {
        const bool elem = p.nreduce == 0 ? true : p.args[a].elem_level;
        const int used = elem ? rank : n_outer_dims;
        if (strides && strides[a]) {
            for (int d = 0; d < used; ++d) st[a][d] = strides[a][d];
        } else {
            long long s = 1;
            for (int d = used - 1; d >= 0; --d) { st[a][d] = s; s *= space[d]; }
        }
        for (int d = 0; d < rank; ++d) if (space[d] == 1) st[a][d] = 0;
    }

    // split into outer / inner groups and collapse each
    std::vector<Dim> outer, inner;
    for (int d = 0; d < rank; ++d) {
        Dim dim;
        dim.extent = space[d];
        for (int a = 0; a < nargs; ++a) dim.stride.push_back(st[a][d]);
        if (p.nreduce == 0 || d < n_outer_dims) outer.push_back(dim);
        else inner.push_back(dim);
    }
    collapse(&outer);
    collapse(&inner);
    if (p.nreduce == 0) {
        // map: the innermost collapsed dim becomes the inner group
        if (!outer.empty()) { inner.push_back(outer.back()); outer.pop_back(); }
    }
    if (inner.empty()) {
        Dim one;
        one.extent = 1;
        one.stride.assign(nargs, 0);
        inner.push_back(one);
    }
    if (outer.size() > 8 || inner.size() > 8) { *err = "launch: more than 8 non-collapsible dims"; return false; }

    Variant v;
    v.nout = (int)outer.size();
    v.nin = (int)inner.size();
    long long R = 1, C = 1;
    for (const Dim& d : outer) R *= d.extent;
    for (const Dim& d : inner) C *= d.extent;

    // stride classes along the (single) inner dim / (single) outer dim
    std::vector<char*> ptr(nargs);
    for (int a = 0; a < nargs; ++a)
        ptr[a] = (char*)array_data[a] + (offsets ? offsets[a] : 0) * dtype_size(p.args[a].dtype);
    v.cls.assign(nargs, 's');
    v.ocls.assign(nargs, 's');
    for (int a = 0; a < nargs; ++a) {
        if (v.nin == 1) {
            long long s = inner[0].stride[a];
            v.cls[a] = (s == 1 || C == 1) ? 'u' : (s == 0 ? 'z' : 's');
            if (C == 1 && s == 0) v.cls[a] = 'z';
        }
        if (v.nout == 1) {
            long long s = outer[0].stride[a];
            v.ocls[a] = s == 1 ? 'u' : (s == 0 ? 'z' : 's');
        }
    }

    auto arg_elem = [&](int a) { return p.nreduce == 0 ? true : p.args[a].elem_level; };
    int max_item = 4;
    int n_elem_args = 0;   // element-level args that are read (their rows may be kept in registers)
    for (int a = 0; a < nargs; ++a)
        if (arg_elem(a) && !p.args[a].indirect) {
            max_item = std::max(max_item, dtype_size(p.args[a].dtype));
            if (p.args[a].read) ++n_elem_args;
        }

    // ---------------------------------------------------------------- skeleton choice
    bool elem_stores = false;
    for (const Stmt& s : p.stmts)
        if ((s.kind == S_ST || s.kind == S_STX) && s.elem) elem_stores = true;
    bool col_ok = p.nreduce > 0 && v.nout == 1 && v.nin == 1 && p.max_stage <= 1 && !elem_stores &&
                  !p.has_indirect && p.n_reductions > 0;
    if (col_ok) {
        // threads should run along the outer dim when that is the contiguous one
        bool any_unit_outer = false, all_fit = true;
        for (int a = 0; a < nargs; ++a) {
            if (!arg_elem(a) || !p.args[a].read) continue;
            if (v.ocls[a] == 'u' && v.cls[a] != 'u') any_unit_outer = true;
            else if (v.ocls[a] == 'z' || (v.ocls[a] == 'u' && C == 1)) {}
            else all_fit = false;
        }
        col_ok = any_unit_outer && all_fit;
        // element work must not read row-level loads (they would vary per lane)
        for (const Stmt& s : p.stmts) {
            if (!s.elem) continue;
            for (int in : s.in) {
                const Stmt& src = p.stmts[p.value_stmt[in]];
                if (!src.elem && src.kind != S_SC && src.kind != S_CONST) col_ok = false;
            }
        }
    }
    bool all_ok = p.nreduce == p.rank && p.nreduce > 0 && p.max_stage <= 1 && !elem_stores && p.n_reductions > 0;

    if (p.has_xrank && !all_ok) { *err = "launch: reductions across ranks run in the all-axis skeleton only (one level of reductions, no element stores)"; return false; }
    v.xrank = p.has_xrank;
    if (p.nreduce == 0) v.kind = K_MAP;
    else if (all_ok) v.kind = K_ALL;
    else if (col_ok) v.kind = K_COL;
    else v.kind = K_ROW;

    // ---------------------------------------------------------------- vector width
    auto aligned = [&](int a, int vec, bool along_outer) {
        const int bytes = dtype_size(p.args[a].dtype) * vec;
        if (!p.args[a].iota && ((uintptr_t)ptr[a]) % bytes != 0) return false;
        const std::vector<Dim>& other = along_outer ? inner : outer;
        for (const Dim& d : other)
            if (d.stride[a] % vec != 0) return false;
        return true;
    };
    int vec = 16 / max_item;
    if (v.kind == K_COL) {
        if (R % vec != 0) vec = 1;
        for (int a = 0; a < nargs && vec > 1; ++a) {
            if (!arg_elem(a)) continue;
            if (v.ocls[a] == 'z') continue;
            if (v.ocls[a] != 'u' || !aligned(a, vec, true)) vec = 1;
        }
    } else {
        if (v.nin != 1 || C % vec != 0) vec = 1;
        for (int a = 0; a < nargs && vec > 1; ++a) {
            if (!arg_elem(a)) continue;
            if (p.args[a].indirect) continue;   // scalar access through the index
            if (v.cls[a] == 'z') continue;
            if (v.cls[a] != 'u' || !aligned(a, vec, false)) vec = 1;
        }
    }
    v.vec = vec;
    // indirectly read args (gather sources) whose indexed rows can be fetched with full-width vector loads
    v.xv.assign(nargs, '0');
    v.unchecked = false;     // decided with the grid below
    v.stream_out = v.kind == K_MAP && p.has_indirect && env_int("DALI_B200_GATHER_STREAM", 0);
    // (opt-in: on 2^20 rows of 1 KiB gathered from a 64 MiB table the kernel is bound by the 1 GiB it writes -- 292 us with
    // scalar gathers and plain stores, 326 us with 128-bit gathers, 314-320 us with streaming stores, DALI_B200_GATHER_STREAM;
    // L2 eviction hints through createpolicy -- evict_last on the table's loads, evict_first on the stores -- measured
    // 333 us, 324 us and 318 us for loads only, stores only and both, and are not in the tree)
    if (vec > 1 && v.kind != K_COL && v.nin == 1 && env_int("DALI_B200_GATHER_VEC", 0))
        for (int a = 0; a < nargs; ++a) {
            if (!p.args[a].indirect || p.args[a].written || p.args[a].iota || !arg_elem(a)) continue;
            const long long xs = strides && strides[a] ? strides[a][rank] : 1;
            if (v.cls[a] == 'u' && xs % vec == 0 && aligned(a, vec, false) && dtype_size(p.args[a].dtype) * vec >= 8) v.xv[a] = '1';
        }

    // ---------------------------------------------------------------- geometry
    long long aux0 = 0, aux1 = 0;
    const long long groups = (C + vec - 1) / vec;
    // MAP with a transposed operand: read-only, unit stride along the (single) outer dim, strided along the inner one
    bool map_tiled = false;
    if (v.kind == K_MAP && v.nout == 1 && v.nin == 1 && !p.has_indirect && R >= 32 && C >= 32 && env_int("DALI_B200_MAP_TILE", 1)) {
        bool others_fit = true;
        for (int a = 0; a < nargs; ++a) {
            if (p.args[a].iota) continue;
            const bool transposed = v.cls[a] == 's' && v.ocls[a] == 'u' && !p.args[a].written;
            if (transposed) map_tiled = true;
            else if (v.cls[a] == 's') others_fit = false;      // strided some other way: the tile would not help it
        }
        map_tiled = map_tiled && others_fit;
    }
    if (map_tiled) {
        for (int a = 0; a < nargs; ++a)
            if (!p.args[a].iota && v.cls[a] == 's' && v.ocls[a] == 'u' && !p.args[a].written) v.cls[a] = 't';
        // 32 x 32 tiles; 64 x 64 (DALI_B200_MAP_TILE=64) measured no faster on a transposed copy of [8192, 8192]
        // (4138 against 4062 GB/s) and slower with a second operand (more shared memory, fewer CTAs per SM)
        size_t tile_bytes = 0;
        for (int a = 0; a < nargs; ++a)
            if (v.cls[a] == 't') tile_bytes += 64 * 65 * dtype_size(p.args[a].dtype);
        int ts = 32;
        if (env_int("DALI_B200_MAP_TILE", 1) == 64 && tile_bytes <= 40 * 1024) ts = 64;
        // 4 x 4 register blocks when every operand is 4 bytes wide and 16-byte aligned along its contiguous direction
        bool micro = R % 4 == 0 && C % 4 == 0 && env_int("DALI_B200_MAP_TILE", 1) == 1;
        for (int a = 0; a < nargs && micro; ++a) {
            if (p.args[a].iota) continue;
            if (dtype_size(p.args[a].dtype) != 4) micro = false;
            else if (v.cls[a] == 't') micro = ((uintptr_t)ptr[a]) % 16 == 0 && inner[0].stride[a] % 4 == 0;
            else if (v.cls[a] == 'u') micro = aligned(a, 4, false);
            else if (v.cls[a] != 'z') micro = false;
        }
        v.threads = 256;
        v.unroll = 1;
        if (micro) {
            v.tile = 4;
            v.vec = 4;
            out.grid_x = (unsigned)((C + 127) / 128);
            out.grid_y = (unsigned)std::min<long long>((R + 31) / 32, 65535);
        } else {
            v.tile = ts;
            v.vec = 1;
            out.grid_x = (unsigned)((C + ts - 1) / ts);
            out.grid_y = (unsigned)std::min<long long>((R + ts - 1) / ts, 65535);
        }
        if ((C + 31) / 32 > 2147483647LL) { *err = "launch: inner extent too large"; return false; }
        v.T = 0; v.vpt = 0; v.tx = 0; v.ty = 0;
    } else if (v.kind == K_MAP) {
        v.threads = 256;
        v.unroll = groups >= 1024 ? 4 : 1;
        int TX = (int)std::min<long long>(256, pow2_ceil((groups + v.unroll - 1) / v.unroll));
        int TY = 256 / TX;
        aux0 = ilog2(TX);
        long long gx = (groups + (long long)TX * v.unroll - 1) / ((long long)TX * v.unroll);
        long long gy = std::min<long long>((R + TY - 1) / TY, 65535);
        if (gx > 2147483647LL) { *err = "launch: inner extent too large"; return false; }
        out.grid_x = (unsigned)gx;
        out.grid_y = (unsigned)gy;
        v.T = 0; v.vpt = 0; v.tx = 0; v.ty = 0;
    } else if (v.kind == K_ROW) {
        if (C > 2147483647LL) { *err = "launch: reduced extent too large for the row skeleton"; return false; }
        // Threads per row.  A warp per row (no shared memory, no barrier, 8 vector loads in
        // flight per thread) while the row fits 8 vector groups per lane and there are enough
        // rows to fill the machine; wider otherwise.
        // Measured on [4096,1024] softmax: 4 vector groups per lane (T = 64) beats 8 (T = 32) and
        // 2 (T = 128); single-pass reductions ([8192,8192] sums) run best with 8.
        // Rows that are transformed and written back (a softmax) and fit eight vector groups per lane: one warp per row,
        // rows staged through shared memory by bulk asynchronous copies, a ring of `stage` rows per warp (see codegen).
        // Needs every element-level operand that is read to be a plain row of memory: unit stride, rows that start on
        // 16-byte boundaries.  Opt-in (DALI_B200_ROW_STAGE = ring depth): at [4096,1024] the staged kernel measured 7.5-8.5 us
        // per launch against 7.1 us for the plain one (rows straight into registers, 2048 CTAs) -- what a 5 us kernel
        // loses in one in-order stream is the hand-over from one launch to the next, not load latency inside it.
        int stage = env_int("DALI_B200_ROW_STAGE", 0);
        {
            bool ok = stage > 0 && elem_stores && v.nin == 1 && vec > 1 && groups <= 8 * 32 && groups > 32 && !p.has_indirect &&
                      R >= (long long)kSMs * 16 && (long long)8 * vec * (n_elem_args + p.n_reductions) <= 96 && n_elem_args >= 1;
            for (int a = 0; a < nargs && ok; ++a) {
                if (!arg_elem(a) || !p.args[a].read) continue;
                if (p.args[a].iota || v.cls[a] != 'u' || !aligned(a, 16 / dtype_size(p.args[a].dtype), false) ||
                    (C * dtype_size(p.args[a].dtype)) % 16 != 0)
                    ok = false;
            }
            if (!ok) stage = 0;
        }
        const int max_vpt = (p.max_stage <= 1 && !elem_stores) || stage ? 8 : 4;
        int T = 32;
        while (T < 1024 && (groups + T - 1) / T > max_vpt) T <<= 1;
        while (T > 1 && groups <= T / 2) T >>= 1;                       // short rows: sub-warp groups
        while (T < 1024 && (groups + T - 1) / T > 1 && R * T < (long long)kSMs * 512) T <<= 1;  // few rows
        T = env_int("DALI_B200_ROW_T", T);
        int vpt = (int)((groups + T - 1) / T);
        int n_cached = n_elem_args + p.n_reductions;  // leaf arrays + value caches (upper bound)
        bool cached = v.nin == 1 && (long long)vpt * vec * n_cached <= 96;
        v.T = T;
        v.vpt = cached ? vpt : 0;
        v.threads = T > 128 ? T : 128;
        v.threads = env_int("DALI_B200_ROW_THREADS", v.threads);
        // few rows: smaller CTAs spread them over more SMs
        while (v.threads > T && v.threads > 64 && R * T / v.threads < 2 * kSMs) v.threads >>= 1;
        if (v.threads < 32) v.threads = 32;
        if (v.threads < T) v.threads = T;
        int rpc = v.threads / T;
        long long gx = (R + rpc - 1) / rpc;
        out.grid_x = (unsigned)std::min<long long>(gx, (long long)kSMs * env_int("DALI_B200_ROW_CTAS_PER_SM", 32));
        // (compiling the [4096,1024] softmax for more CTAs per SM so that all its rows are resident at once -- 12, 14, 16
        // of 128 threads -- spills: 7.6, 10.7, 10.7 us against 7.2 us; 0 = no bound)
        v.minb = env_int("DALI_B200_ROW_MINB", 0);
        // Few rows, each far too long for one CTA's registers: a thread-block cluster shares every row (see codegen).
        // As many rows are in flight as fit L2 together (a softmax reads its row three times: the second and third
        // pass then come from L2), and the cluster is made as wide as it takes to put those rows on every SM.
        // Measured (softmax, fp32): [9,1M] 185 -> 35 us, [32,2M] 558 -> 277 us, [64,1M] 312 -> 207 us, [150,256K] 115 -> 104 us;
        // with as many rows as SMs one CTA per row is as good ([300,128K]) or better ([1000,64K]).
        if (!cached && v.nin == 1 && T >= 512 && !p.has_indirect && 2 * R <= 3 * kSMs && env_int("DALI_B200_ROW_CLUSTER", 1)) {
            long long row_bytes = 0;
            for (int a = 0; a < nargs; ++a)
                if (arg_elem(a)) row_bytes += C * dtype_size(p.args[a].dtype);
            long long in_flight = std::max<long long>(1, std::min<long long>(R, ((long long)env_int("DALI_B200_ROW_CLUSTER_L2_MB", 32) << 20) / std::max<long long>(1, row_bytes)));
            in_flight = std::max<long long>(in_flight, std::min<long long>(R, (kSMs + 15) / 16));   // rows beyond L2's reach: fill the machine at least
            int cl = 1;
            while (cl < 16 && in_flight * cl * 2 <= 2 * kSMs) cl <<= 1;
            cl = env_int("DALI_B200_ROW_CLUSTER_SIZE", cl);
            if (cl >= 2 && C >= (long long)cl * 4096) {
                v.cluster = cl;
                v.T = T = 512;
                v.threads = 512;
                rpc = 1;
                out.cluster = (unsigned)cl;
                out.grid_x = (unsigned)(in_flight * cl);
            }
        }
        if (stage && cached && T == 32) {
            // 8 warps per CTA; the rings of a CTA: operands x 8 warps x stage x one padded row
            v.threads = env_int("DALI_B200_ROW_THREADS", 256);
            rpc = v.threads / 32;
            long long slot = 0;
            for (int a = 0; a < nargs; ++a)
                if (arg_elem(a) && p.args[a].read) slot = std::max<long long>(slot, (C * dtype_size(p.args[a].dtype) + 127) / 128 * 128);
            long long smem = slot * stage * rpc * n_elem_args;
            while (smem > 200 * 1024 && stage > 1) { --stage; smem = slot * stage * rpc * n_elem_args; }
            if (smem <= 200 * 1024) {
                v.stage = stage;
                aux0 = slot;
                out.smem_bytes = (unsigned)smem;
                const long long per_sm = std::max<long long>(1, std::min<long long>(200 * 1024 / smem, 2048 / v.threads));
                gx = (R + rpc - 1) / rpc;
                out.grid_x = (unsigned)std::min<long long>(gx, (long long)kSMs * env_int("DALI_B200_ROW_STAGE_CTAS", (int)per_sm));
            }
        }
        // (streamed rows: hoisting the loads of 2-8 groups ahead of their use -- DALI_B200_ROW_UNROLL -- measured slower
        // than the plain loop on [64,1M] and [150,256K] softmaxes, 0.25 and 0.20 ms against 0.21 and 0.115 ms)
        v.unroll = (!cached && v.nin == 1) ? env_int("DALI_B200_ROW_UNROLL", 1) : 1;
        v.tx = 0; v.ty = 0;
    } else if (v.kind == K_ALL) {
        v.threads = env_int("DALI_B200_ALL_THREADS", 256);
        v.unroll = env_int("DALI_B200_ALL_UNROLL", 4);
        long long chunk = (long long)v.threads * vec * v.unroll;
        long long gx = (C + chunk - 1) / chunk;
        // One resident wave (148 x 8 CTAs) for small inputs; beyond that more, shorter CTAs, which the
        // hardware hands to whichever SM frees up first: the fused chain over 2^31 elements takes 1.62 ms as one
        // wave (CTAs of one SM progress unevenly and the last ones run with too few warps to hide the loads) and 1.50 ms
        // as 16 waves; a 2^26-element sum takes 50 / 53 / 59 us as 4 / 8 / 14 waves.  The work of a CTA depends on the
        // grid only, so results stay bit-equal from run to run.
        // (whole waves only, a CTA of about 8 chunks: 2^26 elements run as two waves -- sum 46.1 us against 46.7-47.4 us as
        // one, argmax 45.9 against 48.3 us -- and the second wave evens out the SMs' finishing times, which is what the
        // other ranks of a fused exchange wait for)
        const long long wave = (long long)kSMs * env_int("DALI_B200_ALL_CTAS_PER_SM", 8);
        const long long per_cta = env_int("DALI_B200_ALL_CHUNKS_PER_CTA", 8);
        long long waves = (gx + per_cta * wave / 2) / (per_cta * wave);
        waves = std::max<long long>(1, std::min<long long>(waves, env_int("DALI_B200_ALL_MAX_WAVES", 16)));
        const long long ctas = std::min(gx, wave * waves);
        out.grid_x = (unsigned)ctas;
        // full chunks without per-vector bounds checks: the loop body exists twice then, which pays when a CTA runs it
        // often (2^31-element chain, 28 chunks per CTA: 1.504 -> 1.483 ms) and costs when it does not (2^26-element sum,
        // 7 chunks per CTA: 54.9 -> 60.4 us)
        v.unchecked = env_int("DALI_B200_ALL_UNCHECKED", gx >= 16 * ctas ? 1 : 0) != 0;
        out.scratch_bytes = (size_t)out.grid_x * 16 * std::max(1, p.n_reductions);
        out.counters = 1;
        v.T = 0; v.vpt = 0; v.tx = 0; v.ty = 0;
    } else {  // K_COL
        // 64 threads along the contiguous outer dim x 4 along the reduced one; a thin outer dim ([N, 4] summed over
        // axis 0) turns the idle outer threads into more rows in flight: [16M, 4] 2780 -> 69 us at tx = 1, ty = 256
        int tx = 64;
        while (tx > 1 && (long long)(tx / 2) * vec >= R) tx >>= 1;
        v.tx = env_int("DALI_B200_COL_TX", tx);
        v.ty = env_int("DALI_B200_COL_TY", 256 / v.tx);
        v.threads = v.tx * v.ty;
        bool has_arg = false;
        for (const Stmt& st_ : p.stmts) has_arg = has_arg || st_.kind == S_ARGRED;
        // (arg-reductions park the rows in flight before they fold them: 4 rows and 4 CTAs per SM, 52.5 us on [8192,8192];
        // 8 rows need 3 CTAs per SM, 56 us; more CTAs per SM spill -- 5: 62 us, 8: 102 us)
        v.unroll = env_int("DALI_B200_COL_UNROLL", has_arg ? 4 : 8);
        long long tiles = (R + (long long)v.tx * vec - 1) / ((long long)v.tx * vec);
        // The grid is one wave: every SM holds `per_sm` CTAs for the whole launch.  A plain reduction is compiled to fit 8
        // per SM (32 registers; without the bound max took 40 and its 1184 CTAs ran as a wave of 888 and a tail); an
        // arg-reduction carries (value, 64-bit position) pairs and the parked rows, and is sized for 4 per SM.
        int per_sm = env_int("DALI_B200_COL_CTAS_PER_SM", has_arg ? 4 : 8);
        if (v.threads == 256 && p.stmts.size() <= 6) v.minb = per_sm;
        long long S = has_arg ? std::max<long long>(1, (long long)kSMs * per_sm / tiles)
                              : ((long long)kSMs * per_sm + tiles - 1) / tiles;
        long long maxS = std::max<long long>(1, C / (v.ty * 8));
        S = std::max<long long>(1, std::min<long long>(std::min<long long>(S, maxS), 256));
        long long per = (C + S - 1) / S;
        S = (C + per - 1) / per;
        aux0 = per;
        if (tiles > 2147483647LL) { *err = "launch: outer extent too large"; return false; }
        out.grid_x = (unsigned)tiles;
        out.grid_y = (unsigned)S;
        if (S > 1) {
            out.scratch_bytes = (size_t)std::max(1, p.n_reductions) * (size_t)S * (size_t)tiles * v.tx * vec * 16;
            out.counters = (size_t)tiles;
        }
        v.T = 0; v.vpt = 0;
    }

    // ---------------------------------------------------------------- parameter words
    ParamLayout L(p, v);
    out.words.assign(L.total, 0);
    out.words[L.w_R] = R;
    out.words[L.w_C] = C;
    out.words[L.w_aux0] = aux0;
    out.words[L.w_aux1] = aux1;
    for (int k = 0; k < v.nout; ++k) out.words[L.w_oshape + k] = outer[k].extent;
    for (int k = 0; k < v.nin; ++k) out.words[L.w_ishape + k] = inner[k].extent;
    for (int a = 0; a < nargs; ++a) {
        // an iota arg has no memory: its "pointer" word is the base value (the element offset)
        out.words[L.arg_ptr(a)] = p.args[a].iota ? (long long)(offsets ? offsets[a] : 0) : (long long)(uintptr_t)ptr[a];
        // lead stride of an indirectly addressed arg travels as one extra stride
        // entry after the `rank` space strides
        long long xs = 0;
        if (p.args[a].indirect) {
            if (!strides || !strides[a]) { *err = "launch: indirect arg needs explicit strides (rank + 1 entries)"; return false; }
            xs = strides[a][rank];
        }
        out.words[L.arg_xs(a)] = xs;
        for (int k = 0; k < v.nout; ++k) out.words[L.arg_rs(a, k)] = outer[k].stride[a];
        for (int k = 0; k < v.nin; ++k) out.words[L.arg_cs(a, k, v.nout)] = inner[k].stride[a];
    }
    for (int j = 0; j < n_scalars; ++j) {
        long long w = 0;
        if (!scalars || !scalars[j]) { *err = "launch: null scalar"; return false; }
        std::memcpy(&w, scalars[j], dtype_size(p.scalars[j]));
        out.words[L.w_scalars + j] = w;
    }
    out.variant = v;
    *plan = out;
    return true;
}

}  // namespace dalib
