// Host side of the tcgen05 GEMM: epilogue splicing, tile choice, TMA tensor
// maps, 3xTF32 operand split, launch.  Kernel: gemm_sm100.cuh.
//
// Replaces CublasGemmImpl::run (dali/array/gemm/cublas_gemm.cu:110-186) for
// the large aligned products, together with the elementwise kernel that the
// reference launches afterwards on the product (dali/array/jit/jit.cpp:1080-
// 1142 keeps MatMul out of every fused kernel, dali/array/op/dot.h:7).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <sstream>

#include "../../include/dali_b200.h"
#include "runtime.h"

namespace dalib {

static const char* kGemmSkeleton =
#include "gemm_embed.inc"
    ;

cudaError_t split_tf32(cudaStream_t stream, const float* x, long long rows, long long cols, long long ld, bool transpose,
                       float* hi, float* lo);
cudaError_t split_tf32_pair(cudaStream_t stream, const float* x0, const float* x1, long long rows, long long cols, long long ld0,
                            long long ld1, float* hi0, float* lo0, float* hi1, float* lo1);

namespace {

struct GemmVariant {
    int esize;      // 2 bf16, 4 tf32
    int split;      // 3xTF32
    int bm, bn, bk, stages;
    int ksplit = 0; // a cluster of two CTAs per tile, one operand pair each, partial sums exchanged through DSMEM
    int slices = 1; // the epilogue reads this many column slices of the product per output element
    int pair = 0;   // two CTAs (cta_group::2) share a 2*bm x bn tile, each staging half of the B tile
    int kpair = 0;  // with ksplit: clusters of four, a cta_group::2 pair per operand pair on a tile of 2*bm rows
    bool b_kmajor() const { return split != 0; }   // the fp32 path transposes B while splitting it
    bool ncat() const { return split != 0 && (bn <= 64 || ksplit) && !kpair; }   // b_hi | b_lo read as one operand of 2 * bn columns
    unsigned idesc(int n_cols = 0) const {
        if (!n_cols) n_cols = bn;
        unsigned fmt = esize == 2 ? 1u : 2u;       // kind::f16: 1 = bf16; kind::tf32: 2 = tf32
        unsigned d = 0;
        d |= 1u << 4;                              // accumulate in fp32
        d |= fmt << 7;                             // A format
        d |= fmt << 10;                            // B format
        d |= 0u << 15;                             // A is K-major
        d |= (b_kmajor() ? 0u : 1u) << 16;         // B: K-major ([N,K]) or MN-major ([K,N])
        d |= (unsigned)(n_cols >> 3) << 17;
        d |= (unsigned)((((pair || kpair) ? 2 : 1) * bm) >> 4) << 24;
        return d;
    }
    size_t stage_bytes() const {
        return (size_t)(split ? 2 : 1) * ((size_t)bm * bk * esize + (size_t)(bn / ((pair || kpair) ? 2 : 1)) * bk * esize);
    }
    size_t xchg_bytes() const { return ksplit ? (size_t)bm * (bn / 2) * 4 : 0; }     // half a tile of fp32 partial sums
    size_t smem_bytes() const { return stages * stage_bytes() + xchg_bytes() + 1024; }
    std::string key() const {
        std::ostringstream o;
        o << "gemm.e" << esize << ".s" << split << ".m" << bm << ".n" << bn << ".k" << bk << ".st" << stages;
        if (pair) o << ".pair";
        if (ncat()) o << ".ncat";
        if (slices > 1) o << ".sl" << slices;
        if (ksplit) o << ".ksplit";
        if (kpair) o << ".kpair";
        return o.str();
    }
};

const char* red_c(DType t) { return dtype_c_name(t); }

// EPILOGUE_CHUNK(row, col0, acc, nvalid): thread-local slab of GEMM_CHUNK columns of one output row; `acc`
// holds the accumulator of slice q in acc[q * GEMM_CHUNK ..]
bool epilogue_macro(const Program& p, std::string* out, std::string* err) {
    if (!p.has_acc || p.nreduce != 0 || p.rank != 2) { *err = "epilogue program must be 'space 2 0' and read 'acc'"; return false; }
    if (p.has_indirect || p.n_reductions || p.has_iota) { *err = "epilogue program may not gather, reduce or use iota args"; return false; }
    const int nargs = (int)p.args.size();
    std::ostringstream o;
    auto W = [&](int w) { return "p.w[" + std::to_string(w) + "]"; };
    auto argT = [&](int a) -> std::string { return p.args[a].dtype == BF16 ? "unsigned short" : dtype_c_name(p.args[a].dtype); };
    o << "#define EPILOGUE_CHUNK(row, col0, acc, nvalid) { \\\n";
    for (int a = 0; a < nargs; ++a) {
        bool ro = !p.args[a].written;
        o << "  " << (ro ? "const " : "") << argT(a) << "* const a" << a << " = reinterpret_cast<" << (ro ? "const " : "")
          << argT(a) << "*>(" << W(3 * a) << ") + (row) * " << W(3 * a + 1) << "; \\\n";
    }
    // loads
    std::vector<bool> loaded(nargs, false);
    for (const Stmt& s : p.stmts) {
        int a = -1;
        if (s.kind == S_LD) a = s.arg;
        if (s.kind == S_ST && s.aop != A_ASSIGN) a = s.arg;
        if (a < 0 || loaded[a]) continue;
        loaded[a] = true;
        o << "  float in" << a << "[GEMM_CHUNK]; gemm_io::load_chunk(a" << a << ", (col0), " << W(3 * a + 2) << ", in" << a << ", (nvalid)); \\\n";
    }
    for (const Stmt& s : p.stmts)
        if (s.kind == S_ST) o << "  float out" << s.arg << "[GEMM_CHUNK]; \\\n";
    for (const Stmt& s : p.stmts) {
        if (s.kind == S_SC)
            o << "  const " << red_c(s.dtype) << " v" << s.id << " = *reinterpret_cast<const " << red_c(s.dtype) << "*>(&"
              << W(3 * nargs + s.arg) << "); \\\n";
        if (s.kind == S_CONST) {
            std::string lit = s.literal;
            if (s.dtype != I32 && lit.find_first_of(".eEn") == std::string::npos) lit += ".0";
            o << "  const " << red_c(s.dtype) << " v" << s.id << " = (" << red_c(s.dtype) << ")(" << lit << "); \\\n";
        }
    }
    o << "  _Pragma(\"unroll\") for (int j = 0; j < GEMM_CHUNK; ++j) { \\\n";
    for (const Stmt& s : p.stmts) {
        const std::string T = red_c(s.dtype);
        switch (s.kind) {
            case S_ACC: o << "    const float v" << s.id << " = acc[" << s.arg << " * GEMM_CHUNK + j]; \\\n"; break;
            case S_LD: o << "    const " << T << " v" << s.id << " = (" << T << ")in" << s.arg << "[j]; \\\n"; break;
            case S_CAST: o << "    const " << T << " v" << s.id << " = (" << T << ")v" << s.in[0] << "; \\\n"; break;
            case S_OP: {
                o << "    const " << T << " v" << s.id << " = ";
                if (s.name == "round" || s.name == "ceiling") o << "f_" << s.name << "<" << T << ">(v" << s.in[0] << ")";
                else if (s.name == "rng_uniform" || s.name == "rng_normal")
                    o << "f_" << s.name << "<" << T << ">(v" << s.in[0] << ", v" << s.in[1] << ")";
                else {
                    o << "f_" << s.name << "(v" << s.in[0];
                    if (s.in.size() > 1) o << ", v" << s.in[1];
                    o << ")";
                }
                o << "; \\\n";
                break;
            }
            case S_ST: {
                std::string v = "(float)v" + std::to_string(s.in[0]);
                std::string old = "in" + std::to_string(s.arg) + "[j]";
                switch (s.aop) {
                    case A_ASSIGN: break;
                    case A_ADD: v = old + " + " + v; break;
                    case A_SUB: v = old + " - " + v; break;
                    case A_MUL: v = old + " * " + v; break;
                    case A_DIV: v = old + " / " + v; break;
                }
                o << "    out" << s.arg << "[j] = " << v << "; \\\n";
                break;
            }
            default: break;
        }
    }
    o << "  } \\\n";
    for (const Stmt& s : p.stmts)
        if (s.kind == S_ST)
            o << "  gemm_io::store_chunk(a" << s.arg << ", (col0), " << W(3 * s.arg + 2) << ", out" << s.arg << ", (nvalid)); \\\n";
    o << "}\n";
    *out = o.str();
    return true;
}

// chunk I/O helpers used by the epilogue macro
const char* kGemmIo = R"IO(
namespace gemm_io {
DEV bool aligned16(const void* p) { return (reinterpret_cast<unsigned long long>(p) & 15ull) == 0; }
// GEMM_CHUNK consecutive columns of one row, element stride cs, as fp32
DEV void load_chunk(const float* p, long long col0, long long cs, float* dst, int nvalid) {
    if (cs == 1 && nvalid == GEMM_CHUNK && aligned16(p + col0)) {
        const float4* q = reinterpret_cast<const float4*>(p + col0);
#pragma unroll
        for (int i = 0; i < GEMM_CHUNK / 4; ++i) { float4 t = q[i]; dst[4 * i] = t.x; dst[4 * i + 1] = t.y; dst[4 * i + 2] = t.z; dst[4 * i + 3] = t.w; }
    } else if (cs == 0) {
        const float t = p[0];
#pragma unroll
        for (int i = 0; i < GEMM_CHUNK; ++i) dst[i] = t;
    } else {
#pragma unroll
        for (int i = 0; i < GEMM_CHUNK; ++i) dst[i] = i < nvalid ? p[(col0 + i) * cs] : 0.0f;
    }
}
DEV void load_chunk(const unsigned short* p, long long col0, long long cs, float* dst, int nvalid) {
    if (cs == 1 && nvalid == GEMM_CHUNK && aligned16(p + col0)) {
        const uint4* q = reinterpret_cast<const uint4*>(p + col0);
#pragma unroll
        for (int i = 0; i < GEMM_CHUNK / 8; ++i) {
            uint4 t = q[i];
            unsigned w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) { dst[8 * i + 2 * k] = __uint_as_float(w[k] << 16); dst[8 * i + 2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u); }
        }
    } else {
#pragma unroll
        for (int i = 0; i < GEMM_CHUNK; ++i) dst[i] = i < nvalid ? gemm::bf16_to_f32(p[cs == 0 ? 0 : (col0 + i) * cs]) : 0.0f;
    }
}
template <typename T> DEV void load_chunk(const T* p, long long col0, long long cs, float* dst, int nvalid) {
#pragma unroll
    for (int i = 0; i < GEMM_CHUNK; ++i) dst[i] = i < nvalid ? (float)p[cs == 0 ? 0 : (col0 + i) * cs] : 0.0f;
}
DEV void store_chunk(float* p, long long col0, long long cs, const float* src, int nvalid) {
    if (cs == 1 && nvalid == GEMM_CHUNK && aligned16(p + col0)) {
        float4* q = reinterpret_cast<float4*>(p + col0);
#pragma unroll
        for (int i = 0; i < GEMM_CHUNK / 4; ++i) q[i] = make_float4(src[4 * i], src[4 * i + 1], src[4 * i + 2], src[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < GEMM_CHUNK; ++i) if (i < nvalid) p[(col0 + i) * cs] = src[i];
    }
}
DEV void store_chunk(unsigned short* p, long long col0, long long cs, const float* src, int nvalid) {
    if (cs == 1 && nvalid == GEMM_CHUNK && aligned16(p + col0)) {
        uint4* q = reinterpret_cast<uint4*>(p + col0);
#pragma unroll
        for (int i = 0; i < GEMM_CHUNK / 8; ++i)
            q[i] = make_uint4(gemm::pack_bf16x2(src[8 * i], src[8 * i + 1]), gemm::pack_bf16x2(src[8 * i + 2], src[8 * i + 3]),
                              gemm::pack_bf16x2(src[8 * i + 4], src[8 * i + 5]), gemm::pack_bf16x2(src[8 * i + 6], src[8 * i + 7]));
    } else {
#pragma unroll
        for (int i = 0; i < GEMM_CHUNK; ++i)
            if (i < nvalid) p[(col0 + i) * cs] = (unsigned short)(gemm::pack_bf16x2(src[i], 0.0f) & 0xffffu);
    }
}
template <typename T> DEV void store_chunk(T* p, long long col0, long long cs, const float* src, int nvalid) {
#pragma unroll
    for (int i = 0; i < GEMM_CHUNK; ++i) if (i < nvalid) p[(col0 + i) * cs] = (T)src[i];
}
}  // namespace gemm_io
)IO";

struct GemmSourceCtx { const Program* p; GemmVariant v; };

bool gemm_source(void* ctx, std::string* src, std::string* err) {
    GemmSourceCtx* c = static_cast<GemmSourceCtx*>(ctx);
    std::string macro;
    if (!epilogue_macro(*c->p, &macro, err)) return false;
    std::ostringstream o;
    o << device_prelude() << "\n";
    o << "#define GEMM_BM " << c->v.bm << "\n#define GEMM_BN " << c->v.bn << "\n#define GEMM_BK " << c->v.bk << "\n";
    o << "#define GEMM_STAGES " << c->v.stages << "\n#define GEMM_ESIZE " << c->v.esize << "\n#define GEMM_SPLIT " << c->v.split << "\n";
    o << "#define GEMM_IDESC " << c->v.idesc() << "u\n";
    o << "#define GEMM_SLICES " << c->v.slices << "\n#define GEMM_KSPLIT " << c->v.ksplit << "\n";
    o << "#define GEMM_NCAT " << (c->v.ncat() ? 1 : 0) << "\n#define GEMM_IDESC_WIDE " << c->v.idesc(2 * c->v.bn) << "u\n";
    o << "#define GEMM_B_KMAJOR " << (c->v.b_kmajor() ? 1 : 0) << "\n#define GEMM_PAIR " << c->v.pair << "\n";
    o << "#define GEMM_KPAIR " << c->v.kpair << "\n";
    int words = 3 * (int)c->p->args.size() + (int)c->p->scalars.size();
    o << "#define GEMM_EPI_WORDS " << (words < 1 ? 1 : words) << "\n";
    // the io helpers need gemm:: conversions, which the skeleton defines: split the skeleton at its kernel
    std::string skel(kGemmSkeleton);
    size_t cut = skel.find("//@EPILOGUE@");
    o << skel.substr(0, cut) << kGemmIo << macro << skel.substr(cut);
    *src = o.str();
    return true;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool make_map(CUtensorMap* map, bool bf16, const void* base, uint64_t inner, uint64_t outer, uint64_t ld_elems, uint32_t box_inner,
              uint32_t box_outer, std::string* err) {
    static EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(driver_entry("cuTensorMapEncodeTiled"));
    if (!encode) { *err = "cuTensorMapEncodeTiled unavailable"; return false; }
    const uint64_t esize = bf16 ? 2 : 4;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {ld_elems * esize};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base),
                        dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r); return false; }
    return true;
}

// fp32 [slices][cols][k] view of a transposed operand (row pitch ld_elems): box = all slices x box_cols x box_k
bool make_map_sliced(CUtensorMap* map, const void* base, uint64_t k, uint64_t cols, uint64_t slices, uint64_t ld_elems,
                     uint32_t box_k, uint32_t box_cols, uint32_t box_slices, std::string* err) {
    static EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(driver_entry("cuTensorMapEncodeTiled"));
    if (!encode) { *err = "cuTensorMapEncodeTiled unavailable"; return false; }
    cuuint64_t dims[3] = {k, cols, slices};
    cuuint64_t strides[2] = {ld_elems * 4, cols * ld_elems * 4};
    cuuint32_t box[3] = {box_k, box_cols, box_slices};       // a CTA pair stages half of the slices each
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled (3-D) failed with CUresult " + std::to_string((int)r); return false; }
    return true;
}

GemmVariant choose_variant(bool bf16, int64_t m, int64_t n) {
    GemmVariant v;
    v.esize = bf16 ? 2 : 4;
    v.split = bf16 ? 0 : 1;
    v.bm = 128;
    v.bk = 128 / v.esize;
    const int64_t mt = (m + 127) / 128;
    auto tiles = [&](int bn) { return mt * ((n + bn - 1) / bn); };
    const int max_bn = bf16 ? 256 : 128;
    v.bn = 64;
    for (int bn = max_bn; bn >= 64; bn >>= 1)
        if (n >= bn && tiles(bn) >= 120) { v.bn = bn; break; }
    if (n < 64) v.bn = 64;
    // bf16 with enough 256 x 256 tiles to fill the SM pairs: CTA-pair MMA
    const char* pair_env = std::getenv("DALI_B200_GEMM_PAIR");
    const bool want_pair = pair_env && pair_env[0] ? pair_env[0] == '1'      // 1 / 0 force it on / off (tests)
                                                   : (m >= 256 && n >= 256 && ((m + 255) / 256) * ((n + 255) / 256) >= 64);
    if (bf16 && want_pair) {
        v.pair = 1;
        v.bn = 256;
    }
    const size_t budget = 200 * 1024;
    v.stages = (int)(budget / v.stage_bytes());
    if (v.stages > 8) v.stages = 8;
    if (v.stages < 2) v.stages = 2;
    return v;
}

struct GemmP {
    long long M, N, K, K2;
    unsigned tiles_m, tiles_n;
    int* err;
    long long w[64];
};

thread_local std::string tl_gemm_variant;

}  // namespace

const std::string& last_gemm_variant() { return tl_gemm_variant; }

// One operand pair of acc = sum_p A_p . B_p.  a / b: device pointers; lda / ldb in elements.  For
// fp32 these are the already split operands (hi parts in a / b, lo parts in a_lo / b_lo, B transposed).
struct GemmPair {
    int64_t k;
    const void *a, *a_lo, *b, *b_lo;
    int64_t lda, ldb;
};

int gemm_fused_launch(int device, void* stream, bool bf16, int64_t m, int64_t n, const GemmPair* pairs_in, int n_pairs,
                      uint64_t epilogue_hash, void* const* array_data, const int64_t* offsets, const int64_t* const* strides,
                      int n_arrays, const void* const* scalars, int n_scalars, bool compile_only) {
    // One pre-split fp32 product with few output tiles (small M): its K range becomes two operand pairs, so that the
    // cluster form below applies -- the two halves of K on the two CTAs of a pair.  (Row-major K-major operands: the
    // second half is the same matrix 16-byte aligned further along its rows.)
    GemmPair halves[2];
    const GemmPair* pairs = pairs_in;
    {
        const char* ks = std::getenv("DALI_B200_GEMM_KSPLIT");
        const int64_t k = pairs_in[0].k;
        const int64_t tiles128 = ((m + 127) / 128) * ((n + 127) / 128);
        if (!bf16 && n_pairs == 1 && pairs_in[0].a_lo && pairs_in[0].b_lo && k >= 256 && k % 64 == 0 && n >= 128 &&
            tiles128 < 120 && !(ks && ks[0] == '0')) {
            const int64_t k1 = k / 2;
            halves[0] = pairs_in[0];
            halves[0].k = k1;
            halves[1] = pairs_in[0];
            halves[1].k = k - k1;
            halves[1].a = (const float*)pairs_in[0].a + k1;
            halves[1].a_lo = (const float*)pairs_in[0].a_lo + k1;
            halves[1].b = (const float*)pairs_in[0].b + k1;
            halves[1].b_lo = (const float*)pairs_in[0].b_lo + k1;
            pairs = halves;
            n_pairs = 2;
        }
    }
    Program prog;
    if (!find_program(epilogue_hash, &prog)) { set_error("unknown epilogue hash"); return DALIB200_ERR_NOT_FOUND; }
    if (n_arrays != (int)prog.args.size() || n_scalars != (int)prog.scalars.size()) {
        set_error("gemm_fused: wrong number of epilogue arrays / scalars");
        return DALIB200_ERR_INVALID;
    }
    if (3 * n_arrays + n_scalars > 64) { set_error("gemm_fused: too many epilogue operands"); return DALIB200_ERR_TOO_LARGE; }
    const int slices = prog.acc_slices;
    if (slices > 1 && (bf16 || (slices != 2 && slices != 4))) {
        set_error("gemm_fused: an epilogue over column slices of the product needs fp32 operands and 2 or 4 slices");
        return DALIB200_ERR_UNSUPPORTED;
    }
    GemmSourceCtx ctx{&prog, choose_variant(bf16, m, slices > 1 ? (int64_t)n * slices : n)};
    if (slices > 1) {
        // 64 accumulator columns = 64 / slices output columns x slices; row blocks of 16 or 32 keep the swizzle groups whole
        ctx.v.bn = 64;
        ctx.v.slices = slices;
        const size_t budget = 200 * 1024;
        ctx.v.stages = (int)(budget / ctx.v.stage_bytes());
        if (ctx.v.stages > 8) ctx.v.stages = 8;
    }
    // Two pre-split fp32 operand pairs (the sum of two products: an LSTM's x.Wx + h.Wh), plain or with four slices:
    // one CTA per pair on a 128-column tile, the halves meet through distributed shared memory -- each CTA pulls
    // 2/3 of the operand bytes of the single-CTA form, and operand delivery is what bounds these products.
    {
        const char* ks = std::getenv("DALI_B200_GEMM_KSPLIT");
        const int64_t b_total = (int64_t)n * slices;
        if (!bf16 && n_pairs == 2 && (slices == 4 || slices == 1) && pairs[0].a_lo && b_total >= 128 && !(ks && ks[0] == '0')) {
            ctx.v.ksplit = 1;
            ctx.v.slices = slices;
            ctx.v.bn = 128;
            ctx.v.stages = 3;
            // CTA pairs inside the K split (clusters of four on tiles of 256 rows): opt-in, measured slower (see the skeleton)
            const char* kp = std::getenv("DALI_B200_GEMM_KPAIR");
            if (kp && kp[0] == '1' && m > 128) {
                ctx.v.kpair = 1;
                ctx.v.stages = 4;
            }
        }
    }
    const GemmVariant& v = ctx.v;
    const uint64_t b_cols = (uint64_t)n * (uint64_t)slices;      // columns of the product (rows of the transposed B)
    // (the skeleton and the prelude are hashed once: tens of kilobytes of source, ~100 us per launch otherwise)
    static const std::string source_tag =
        std::string("|sm_100a|gemm|") +
#include "source_hash.inc"
        + "|" + std::to_string(fnv1a(kGemmSkeleton)) + "|" + std::to_string(fnv1a(device_prelude())) + "|" + nvrtc_defines_text();
    std::ostringstream key;
    key << std::hex << epilogue_hash << "_" << fnv1a(v.key() + source_tag);
    tl_gemm_variant = std::string(bf16 ? "tcgen05.bf16 " : "tcgen05.tf32x3 ") + v.key() + (n_pairs > 1 ? " x2" : "");
    note_gemm_kernel(tl_gemm_variant);
    void* fn = nullptr;
    int rc = acquire_kernel(compile_only ? -1 : device, key.str(), "dali_gemm_kernel", gemm_source, &ctx, &fn, nullptr);
    if (rc != DALIB200_OK || compile_only) return rc;

    std::string err;
    CUtensorMap tm[8];
    const uint32_t sw = 128 / v.esize;
    for (int pi = 0; pi < 2; ++pi) {
        const GemmPair& g = pairs[pi < n_pairs ? pi : 0];     // an unused second set just repeats the first
        const uint64_t k = (uint64_t)g.k;
        bool ok = make_map(&tm[4 * pi + 0], bf16, g.a, k, (uint64_t)m, (uint64_t)g.lda, (uint32_t)v.bk, (uint32_t)v.bm, &err) &&
                  make_map(&tm[4 * pi + 2], bf16, g.a_lo ? g.a_lo : g.a, k, (uint64_t)m, (uint64_t)g.lda, (uint32_t)v.bk, (uint32_t)v.bm, &err);
        if (ok && v.b_kmajor() && slices > 1)
            ok = make_map_sliced(&tm[4 * pi + 1], g.b, k, (uint64_t)n, (uint64_t)slices, (uint64_t)g.ldb, (uint32_t)v.bk,
                                 (uint32_t)(v.bn / slices), (uint32_t)(slices / (v.kpair ? 2 : 1)), &err) &&
                 make_map_sliced(&tm[4 * pi + 3], g.b_lo ? g.b_lo : g.b, k, (uint64_t)n, (uint64_t)slices, (uint64_t)g.ldb,
                                 (uint32_t)v.bk, (uint32_t)(v.bn / slices), (uint32_t)(slices / (v.kpair ? 2 : 1)), &err);
        else if (ok && v.b_kmajor())
            ok = make_map(&tm[4 * pi + 1], bf16, g.b, k, b_cols, (uint64_t)g.ldb, (uint32_t)v.bk,
                          (uint32_t)(v.bn / slices / (v.kpair ? 2 : 1)), &err) &&
                 make_map(&tm[4 * pi + 3], bf16, g.b_lo ? g.b_lo : g.b, k, b_cols, (uint64_t)g.ldb, (uint32_t)v.bk,
                          (uint32_t)(v.bn / slices / (v.kpair ? 2 : 1)), &err);
        else if (ok)
            ok = make_map(&tm[4 * pi + 1], bf16, g.b, (uint64_t)n, k, (uint64_t)g.ldb, sw, (uint32_t)v.bk, &err) &&
                 make_map(&tm[4 * pi + 3], bf16, g.b_lo ? g.b_lo : g.b, (uint64_t)n, k, (uint64_t)g.ldb, sw, (uint32_t)v.bk, &err);
        if (!ok) { set_error("gemm_fused: " + err); return DALIB200_ERR_CUDA; }
    }
    GemmP p;
    std::memset(&p, 0, sizeof p);
    p.M = m; p.N = n; p.K = pairs[0].k; p.K2 = n_pairs > 1 ? pairs[1].k : 0;
    p.err = gemm_error_word(device);
    if (!p.err) { set_error("gemm_fused: cannot allocate the error word"); return DALIB200_ERR_CUDA; }
    for (int i = 0; i < n_arrays; ++i) {
        const int es = dtype_size(prog.args[i].dtype);
        p.w[3 * i] = (long long)(uintptr_t)((char*)array_data[i] + (offsets ? offsets[i] : 0) * es);
        p.w[3 * i + 1] = strides && strides[i] ? strides[i][0] : n;
        p.w[3 * i + 2] = strides && strides[i] ? strides[i][1] : 1;
    }
    for (int j = 0; j < n_scalars; ++j) {
        long long w = 0;
        std::memcpy(&w, scalars[j], dtype_size(prog.scalars[j]));
        p.w[3 * n_arrays + j] = w;
    }
    // the kernel's GemmP has exactly GEMM_EPI_WORDS words; ours is a superset with the same prefix
    void* params[] = {&tm[0], &tm[1], &tm[2], &tm[3], &tm[4], &tm[5], &tm[6], &tm[7], &p};
    // persistent CTAs (CTA pairs), at most one per SM (SM pair); they take the tiles round robin
    const int64_t rows_per_tile = (int64_t)v.bm * ((v.pair || v.kpair) ? 2 : 1);
    p.tiles_m = (unsigned)((m + rows_per_tile - 1) / rows_per_tile);
    p.tiles_n = (unsigned)((n + v.bn / slices - 1) / (v.bn / slices));
    const uint64_t total_tiles = (uint64_t)p.tiles_m * p.tiles_n;
    if (total_tiles > 0x7fffffffull) { set_error("gemm_fused: too many output tiles"); return DALIB200_ERR_TOO_LARGE; }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_ordinal(device)) != cudaSuccess || sms < 2) sms = 148;
    const int per_worker = v.kpair ? 4 : (v.pair || v.ksplit) ? 2 : 1;       // CTAs of a cluster
    uint64_t workers = (uint64_t)(sms / per_worker);
    if (workers > total_tiles) workers = total_tiles;
    const unsigned gx = (unsigned)(workers * per_worker), gy = 1;
    // the kernel waits for its predecessor (griddepcontrol.wait) after its own set-up: barriers, tensor memory
    return launch_function(device, fn, gx, gy, 192, (unsigned)v.smem_bytes(), stream, params, /*dependent=*/true);
}

}  // namespace dalib

using namespace dalib;

extern "C" {

int dalib200_gemm_fused_sum(int device, void* stream, int ab_dtype, int n_pairs, int64_t m, int64_t n, const int64_t* k,
                            const void* const* a, const int64_t* lda, const void* const* b, const int64_t* ldb,
                            const void* const* a_lo, const void* const* b_lo, uint64_t epilogue_hash,
                            void* const* array_data, const int64_t* offsets, const int64_t* const* strides, int n_arrays,
                            const void* const* scalars, int n_scalars) {
    DeviceRestore restore_device;
    if (ab_dtype != DALIB200_BF16 && ab_dtype != DALIB200_F32) {
        set_error("dalib200_gemm_fused: operands must be bf16 or f32");
        return DALIB200_ERR_INVALID;
    }
    if (n_pairs < 1 || n_pairs > 2 || m < 0 || n < 0 || !k || !a || !b || !lda || !ldb) {
        set_error("dalib200_gemm_fused: bad argument (one or two operand pairs)");
        return DALIB200_ERR_INVALID;
    }
    if (m == 0 || n == 0) return DALIB200_OK;
    const bool bf16 = ab_dtype == DALIB200_BF16;
    const int es = bf16 ? 2 : 4;
    const bool compile_only = device < 0;
    // an epilogue that reads S column slices per output element: n is the width of one slice, B has S * n columns
    int64_t n_total = n;
    {
        Program prog;
        if (!find_program(epilogue_hash, &prog)) { set_error("unknown epilogue hash"); return DALIB200_ERR_NOT_FOUND; }
        n_total = n * prog.acc_slices;
    }
    bool presplit = !bf16 && a_lo && b_lo && a_lo[0] && b_lo[0];
    GemmPair pairs[2];
    for (int p = 0; p < n_pairs; ++p) {
        const bool lo_a = a_lo && a_lo[p], lo_b = b_lo && b_lo[p];
        if (!bf16 && (lo_a != lo_b || (lo_a && lo_b) != presplit)) {
            set_error("dalib200_gemm_fused: pass the split parts of every operand or of none");
            return DALIB200_ERR_INVALID;
        }
        if (!a[p] || !b[p] || k[p] < 0) { set_error("dalib200_gemm_fused: bad operand pair"); return DALIB200_ERR_INVALID; }
        // what TMA needs: 16-byte aligned bases and row pitches
        if (((uintptr_t)a[p] & 15) || ((uintptr_t)b[p] & 15) || (lda[p] * es) % 16 || (ldb[p] * es) % 16 || lda[p] < k[p] ||
            ldb[p] < (presplit ? k[p] : n_total) || (lo_a && ((uintptr_t)a_lo[p] & 15)) || (lo_b && ((uintptr_t)b_lo[p] & 15)) ||
            m > 2147483647LL || n > 2147483647LL || k[p] > 2147483647LL) {
            set_error("dalib200_gemm_fused: operands must be row-major with 16-byte aligned base and row pitch");
            return DALIB200_ERR_UNSUPPORTED;
        }
        pairs[p] = GemmPair{k[p], a[p], lo_a ? a_lo[p] : nullptr, b[p], lo_b ? b_lo[p] : nullptr, lda[p], ldb[p]};
    }
    if (bf16 || compile_only || presplit)
        return gemm_fused_launch(device, stream, bf16, m, n, pairs, n_pairs, epilogue_hash, array_data, offsets, strides,
                                 n_arrays, scalars, n_scalars, compile_only);
    // fp32 without pre-split operands: split here into pool temporaries (recycled in stream order)
    int ord = device_ordinal(device);
    if (ord < 0) { set_error("device index out of range"); return DALIB200_ERR_INVALID; }
    cudaSetDevice(ord);
    void* tmp[8] = {nullptr};
    size_t bytes[8] = {0};
    int rc = DALIB200_OK;
    for (int p = 0; p < n_pairs && rc == DALIB200_OK; ++p) {
        if (k[p] % 4 || n_total % 4) { set_error("dalib200_gemm_fused: fp32 operands need k and n to be multiples of 4"); rc = DALIB200_ERR_UNSUPPORTED; break; }
        bytes[4 * p] = bytes[4 * p + 1] = (size_t)m * k[p] * 4;
        bytes[4 * p + 2] = bytes[4 * p + 3] = (size_t)k[p] * n_total * 4;
        for (int j = 0; j < 4 && rc == DALIB200_OK; ++j) rc = dalib200_alloc(device, bytes[4 * p + j], &tmp[4 * p + j]);
        if (rc != DALIB200_OK) break;
        if (split_tf32((cudaStream_t)stream, (const float*)a[p], m, k[p], lda[p], false, (float*)tmp[4 * p], (float*)tmp[4 * p + 1]) != cudaSuccess ||
            split_tf32((cudaStream_t)stream, (const float*)b[p], k[p], n_total, ldb[p], true, (float*)tmp[4 * p + 2], (float*)tmp[4 * p + 3]) != cudaSuccess) {
            set_error("split_tf32 launch failed");
            rc = DALIB200_ERR_CUDA;
        }
        pairs[p] = GemmPair{k[p], tmp[4 * p], tmp[4 * p + 1], tmp[4 * p + 2], tmp[4 * p + 3], k[p], k[p]};
    }
    if (rc == DALIB200_OK)
        rc = gemm_fused_launch(device, stream, false, m, n, pairs, n_pairs, epilogue_hash, array_data, offsets, strides, n_arrays,
                               scalars, n_scalars, false);
    for (int j = 0; j < 8; ++j)
        if (tmp[j]) dalib200_free(device, tmp[j], bytes[j]);
    return rc;
}

int dalib200_gemm_fused(int device, void* stream, int ab_dtype, int64_t m, int64_t n, int64_t k, const void* a, int64_t lda,
                        const void* b, int64_t ldb, const void* a_lo, const void* b_lo, uint64_t epilogue_hash,
                        void* const* array_data, const int64_t* offsets, const int64_t* const* strides, int n_arrays,
                        const void* const* scalars, int n_scalars) {
    if (ab_dtype == DALIB200_F32 && ((a_lo != nullptr) != (b_lo != nullptr))) {
        set_error("dalib200_gemm_fused: pass both split operands or neither");
        return DALIB200_ERR_INVALID;
    }
    if (!a || !b) { set_error("dalib200_gemm_fused: bad argument"); return DALIB200_ERR_INVALID; }
    return dalib200_gemm_fused_sum(device, stream, ab_dtype, 1, m, n, &k, &a, &lda, &b, &ldb, a_lo ? &a_lo : nullptr,
                                   b_lo ? &b_lo : nullptr, epilogue_hash, array_data, offsets, strides, n_arrays, scalars,
                                   n_scalars);
}

int dalib200_gemm_split_tf32(int device, void* stream, const float* x, int64_t rows, int64_t cols, int64_t ld, int transpose,
                             float* hi, float* lo) {
    DeviceRestore restore_device;
    int ord = device_ordinal(device);
    if (ord < 0) { set_error("device index out of range"); return dalib200_device_count() ? DALIB200_ERR_INVALID : DALIB200_ERR_NO_DEVICE; }
    if (!x || !hi || !lo || cols % 4 || ld % 4 || ((uintptr_t)x & 15) || ((uintptr_t)hi & 15) || ((uintptr_t)lo & 15)) {
        set_error("dalib200_gemm_split_tf32: needs 16-byte aligned pointers and cols, ld multiples of 4");
        return DALIB200_ERR_INVALID;
    }
    cudaSetDevice(ord);
    if (transpose && rows % 4) { set_error("dalib200_gemm_split_tf32: transposed output needs rows % 4 == 0"); return DALIB200_ERR_INVALID; }
    if (split_tf32((cudaStream_t)stream, x, rows, cols, ld, transpose != 0, hi, lo) != cudaSuccess) {
        set_error("split_tf32 launch failed");
        return DALIB200_ERR_CUDA;
    }
    return DALIB200_OK;
}

int dalib200_gemm_split_tf32_pair(int device, void* stream, const float* x0, const float* x1, int64_t rows, int64_t cols,
                                  int64_t ld0, int64_t ld1, float* hi0, float* lo0, float* hi1, float* lo1) {
    DeviceRestore restore_device;
    int ord = device_ordinal(device);
    if (ord < 0) { set_error("device index out of range"); return dalib200_device_count() ? DALIB200_ERR_INVALID : DALIB200_ERR_NO_DEVICE; }
    const void* ptrs[6] = {x0, x1, hi0, lo0, hi1, lo1};
    bool ok = cols % 4 == 0 && ld0 % 4 == 0 && ld1 % 4 == 0 && rows >= 0 && cols >= 0;
    for (const void* q : ptrs) ok = ok && q && ((uintptr_t)q & 15) == 0;
    if (!ok) { set_error("dalib200_gemm_split_tf32_pair: needs 16-byte aligned pointers and cols, ld multiples of 4"); return DALIB200_ERR_INVALID; }
    cudaSetDevice(ord);
    if (split_tf32_pair((cudaStream_t)stream, x0, x1, rows, cols, ld0, ld1, hi0, lo0, hi1, lo1) != cudaSuccess) {
        set_error("split_tf32_pair launch failed");
        return DALIB200_ERR_CUDA;
    }
    return DALIB200_OK;
}

int dalib200_gemm_error_flag(int device, int* flag) {
    DeviceRestore restore_device;
    int ord = device_ordinal(device);
    if (ord < 0) { set_error("device index out of range"); return DALIB200_ERR_INVALID; }
    int* w = gemm_error_word(device);
    if (!w) { set_error("no error word"); return DALIB200_ERR_CUDA; }
    cudaSetDevice(ord);
    cudaError_t e = cudaMemcpy(flag, w, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { set_error(std::string("cudaMemcpy: ") + cudaGetErrorString(e)); return DALIB200_ERR_CUDA; }
    if (*flag) cudaMemset(w, 0, sizeof(int));
    return DALIB200_OK;
}

}  // extern "C"
