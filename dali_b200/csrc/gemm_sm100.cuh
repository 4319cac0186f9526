// tcgen05 / TMEM GEMM skeleton for sm_100a with a spliced elementwise epilogue.
// Compiled at run time by NVRTC behind dalib200_gemm_fused; the host side
// (gemm_sm100.cc) prepends the device prelude, a block of #defines
//   GEMM_BM GEMM_BN GEMM_BK GEMM_STAGES   tile and pipeline depth
//   GEMM_ESIZE        operand element bytes: 2 (bf16, kind::f16) or 4 (tf32)
//   GEMM_SPLIT        1: 3xTF32 (operands come with their low parts), else 0
//   GEMM_B_KMAJOR     1: B is given transposed, [N,K] row-major (K-major, like A);
//                     0: B is [K,N] row-major (MN-major).  bf16 takes B as it lies in
//                     memory; the fp32 path gets B transposed for free by the pass that
//                     splits it into high and low parts
//   GEMM_PAIR         1: two CTAs on neighbouring SMs (a cluster of 2, tcgen05 cta_group::2) share one
//                     256 x GEMM_BN tile: each loads its own 128 rows of A and HALF of the B tile,
//                     the leader CTA issues one MMA that runs on both tensor cores and reads both
//                     halves of B, each CTA ends up with its 128 rows of the accumulator in its own
//                     tensor memory.  Halves the shared-memory traffic per flop, which is what
//                     bounds the single-CTA 128 x 256 bf16 tile
//   GEMM_NCAT         1 (with GEMM_SPLIT, GEMM_B_KMAJOR, GEMM_BN <= 128): the B hi and lo tiles lie one after
//                     the other in a stage and are read as ONE operand of 2*GEMM_BN columns, so a K step
//                     issues a_hi.[b_hi | b_lo] (GEMM_IDESC_WIDE) and a_lo.b_hi: two instructions and one
//                     read of a_hi instead of three and two.  Each round-robin accumulator then has its own
//                     correction accumulator in the columns next to it.
//   GEMM_SLICES       S > 1 (fp32 K-major path): the epilogue's space is [M, N] and it reads S values per output
//                     element, the product's columns q*N + col for q < S (the four gates of an LSTM unit).  A tile
//                     then covers GEMM_BN / S output columns; its B tile is one 3-D TMA copy of the
//                     (transposed) operand seen as [slice][column][k], so accumulator column q * (GEMM_BN / S) + j is slice q of output j
//   GEMM_KSPLIT       1 (with GEMM_SPLIT, GEMM_NCAT, GEMM_BN = 128, GEMM_SLICES = 1 or 4, two operand pairs): a cluster of two CTAs
//                     shares an output tile; CTA r accumulates operand pair r (x.Wx or h.Wh) over the whole
//                     tile, the halves meet through distributed shared memory and each CTA finishes half of
//                     the tile's columns.  Per CTA this halves the operand bytes pulled from L2, which is what
//                     bounds the M = 256 products (separate kernel body: dali_gemm_kernel below)
//   GEMM_KPAIR        1 (with GEMM_KSPLIT, GEMM_NCAT = 0): the K split over CTA PAIRS -- a cluster of four CTAs shares a tile of
//                     256 rows: CTAs 2p and 2p + 1 form a cta_group::2 pair that accumulates operand pair p over the whole
//                     tile (each stages its own 128 rows of A and HALF of the B tile, the even CTA issues one MMA for both
//                     tensor cores), CTA 2p + h then exchanges partial sums with CTA 2(1 - p) + h, which holds the same
//                     128 rows of the other operand pair.  Per CTA and K block 48 KB arrive by TMA instead of 64 KB and the
//                     tensor core reads 72 KB instead of 80 KB from this SM's shared memory.  Opt-in (DALI_B200_GEMM_KPAIR=1):
//                     correct, and slower than the plain K split on the LSTM cell (32.0 against 29.1 us): three 128-column
//                     instructions per K step instead of a 256- and a 128-column one, and each costs 4.5 us over the 128
//                     K steps -- the 32 KB it reads from shared memory at 128 B per clock, which is what bounds these
//                     TF32 products (23.0 / 27.4 / 32.0 us with one / two / three of the instructions issued)
//   GEMM_IDESC        tcgen05 instruction descriptor
// and a macro EPILOGUE_CHUNK(row, col0, acc, nvalid) generated from the
// expression that consumes the product.
//
// Replaces cublasSgemm + a separate elementwise kernel that re-reads C
// (dali/array/gemm/cublas_gemm.cu:157-178 followed by the JIT kernel of the
// surrounding expression): one kernel, the accumulator goes from tensor memory
// through the epilogue straight to its destination.
//
// Layout of the work:
//   persistent CTAs (one per SM, or one pair per two SMs) take output tiles round robin; 192 threads:
//     warps 0-3  epilogue: warp w owns TMEM lanes 32w..32w+31 (= tile rows)
//     warp 4     TMA producer (one elected lane)
//     warp 5     allocates TMEM, issues tcgen05.mma (one elected lane)
//   A is K-major (row-major [M,K]), B is MN-major (row-major [K,N]); both are
//   staged by TMA with 128-byte swizzle into a GEMM_STAGES-deep ring guarded
//   by full / empty mbarriers; tcgen05.commit releases a stage when the MMAs
//   that read it have finished.  Tensor memory holds the accumulators of two
//   tiles when they fit, so the epilogue of a tile runs while the tensor core
//   works on the next one.  No multicast loads.
//
// Every wait is bounded (about a second of polling): on expiry the waiting
// thread records a code in *p.err, raises a CTA-wide abort flag and all roles
// drain; TMEM is always released before the CTA exits.

struct alignas(64) TensorMap { unsigned long long opaque[16]; };

struct GemmP {
    long long M, N, K;        // K: reduction length of the first (or only) operand pair
    long long K2;             // of the second pair (0 = none): acc = A.B + A2.B2 in one accumulator
    unsigned tiles_m, tiles_n;   // output tiles (of a CTA pair: 2*GEMM_BM rows) in each direction
    int* err;                 // device int, 0 = fine
    long long w[GEMM_EPI_WORDS];
};

#define GEMM_THREADS 192
#ifndef GEMM_SLICES
#define GEMM_SLICES 1
#endif
#define GEMM_TILE_N (GEMM_BN / GEMM_SLICES)                  /* output columns of a tile */
#ifndef GEMM_KSPLIT
#define GEMM_KSPLIT 0
#endif
/* output columns an epilogue call handles (with a K split each CTA of the pair finishes half of the tile's columns) */
#define GEMM_CHUNK (GEMM_KSPLIT && GEMM_SLICES > 1 ? GEMM_TILE_N / 2 : GEMM_SLICES > 1 ? GEMM_TILE_N : 32)
#define GEMM_RASTER 8u
#ifndef GEMM_PAIR
#define GEMM_PAIR 0
#endif
#ifndef GEMM_KPAIR
#define GEMM_KPAIR 0
#endif
#define GEMM_CLUSTER (GEMM_PAIR || GEMM_KSPLIT)      /* the kernel runs as clusters of two (GEMM_KPAIR: four) CTAs */
#if GEMM_PAIR || GEMM_KPAIR
#define GEMM_CG "2"
#define GEMM_BN_LOCAL (GEMM_BN / 2)                          /* columns of B this CTA stages */
#else
#define GEMM_CG "1"
#define GEMM_BN_LOCAL GEMM_BN
#endif
#define GEMM_SWIZZLE_ELEMS (128 / GEMM_ESIZE)               /* elements per 128-byte swizzle row */
#define GEMM_UMMA_K (32 / GEMM_ESIZE)                        /* K per tcgen05.mma: 32 bytes */
#define GEMM_A_TILE_BYTES (GEMM_BM * GEMM_BK * GEMM_ESIZE)
#define GEMM_B_ATOMS (GEMM_BN_LOCAL / GEMM_SWIZZLE_ELEMS)          /* 128-byte wide column panels of the B tile */
#define GEMM_B_ATOM_BYTES (GEMM_BK * 128)
#define GEMM_B_TILE_BYTES (GEMM_B_ATOMS * GEMM_B_ATOM_BYTES)
#define GEMM_OPERAND_SETS (GEMM_SPLIT ? 2 : 1)
#define GEMM_STAGE_BYTES (GEMM_OPERAND_SETS * (GEMM_A_TILE_BYTES + GEMM_B_TILE_BYTES))
// Accumulators in tensor memory.  The tensor core adds into its fp32 accumulator with
// truncation, a bias of about half an ulp of the accumulator per tcgen05.mma (measured:
// 1.5e-5 absolute on O(1) sums after the 384 instructions of a K = 1024 3xTF32 product).
// For fp32 parity the split path therefore keeps the small correction products
// (a_lo.b_hi, a_hi.b_lo) in an accumulator of their own and deals the main products round
// robin over GEMM_NACC accumulators, which the epilogue adds up in fp32 on the CUDA cores.
#ifndef GEMM_NCAT
#define GEMM_NCAT 0
#endif
#if GEMM_SPLIT && GEMM_NCAT && GEMM_KSPLIT
#define GEMM_NACC 2                          /* 2 x (128 main + 128 correction columns) fill tensor memory */
#define GEMM_ACC_SETS (2 * GEMM_NACC)
#elif GEMM_SPLIT && GEMM_NCAT
#define GEMM_NACC 3
#define GEMM_ACC_SETS (2 * GEMM_NACC)        /* (main, correction) pairs side by side */
#elif GEMM_SPLIT
#define GEMM_NACC 3
#define GEMM_ACC_SETS (GEMM_NACC + 1)
#else
#define GEMM_NACC 1
#define GEMM_ACC_SETS 1
#endif
#define GEMM_ACC_COLS (GEMM_ACC_SETS * GEMM_BN)                 /* tensor-memory columns of one tile's accumulators */
#define GEMM_ACC_STAGES (2 * GEMM_ACC_COLS <= 512 ? 2 : 1)      /* two tiles' worth when they fit: the epilogue of one tile overlaps the next main loop */
#define GEMM_TMEM_NEED (GEMM_ACC_STAGES * GEMM_ACC_COLS)
#define GEMM_TMEM_COLS (GEMM_TMEM_NEED <= 32 ? 32 : GEMM_TMEM_NEED <= 64 ? 64 : GEMM_TMEM_NEED <= 128 ? 128 : GEMM_TMEM_NEED <= 256 ? 256 : 512)

namespace gemm {

DEV unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

DEV void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
DEV void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
DEV bool mbar_test(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false after ~1 s (or as soon as another role aborted)
DEV bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_test(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > 2000000000LL) return false;
    }
}

#if GEMM_KSPLIT
// the same with cluster scope: what the peer CTA wrote into this CTA's shared memory before it arrived is visible
DEV bool mbar_test_cluster(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
DEV bool mbar_wait_cluster(unsigned long long* bar, unsigned parity, volatile int* abort_flag) {
    if (mbar_test_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_test_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > 2000000000LL) return false;
    }
}
#endif

DEV void tma_load_2d(void* dst, const TensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
DEV void tma_load_3d(void* dst, const TensorMap* map, unsigned long long* bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
#if GEMM_PAIR || GEMM_KPAIR
// the copy lands in THIS CTA's shared memory and reports its bytes to the barrier at shared::cluster
// address bar_cluster (the leader CTA's), as a CTA-pair MMA expects
DEV void tma_load_2d_pair(void* dst, const TensorMap* map, unsigned bar_cluster, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
DEV void tma_load_3d_pair(void* dst, const TensorMap* map, unsigned bar_cluster, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster), "r"(x), "r"(y), "r"(z) : "memory");
}
// arrives on the barrier at the same address in every CTA of the cluster whose bit is set in `mask` when every
// tcgen05.mma issued so far by this thread has completed
DEV void umma_commit_mask(unsigned long long* bar, unsigned short mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
#endif
#if GEMM_CLUSTER
DEV unsigned cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same variable in CTA `rank` of this cluster
DEV unsigned map_to_cta(const void* p, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
DEV void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
#endif

// one arrival on `bar` of the leader CTA (of this CTA when there is no pair)
DEV void arrive_at_leader(unsigned long long* bar) {
#if GEMM_PAIR
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(map_to_cta(bar, 0)) : "memory");
#else
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
#endif
}

DEV void tmem_alloc(unsigned* slot, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::" GEMM_CG ".sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::" GEMM_CG ".sync.aligned;" ::: "memory");
}
DEV void tmem_dealloc(unsigned taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::" GEMM_CG ".sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
DEV void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DEV void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

DEV void umma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
#if GEMM_ESIZE == 2
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::" GEMM_CG ".kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
#else
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::" GEMM_CG ".kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
#endif
}
// arrives on `bar` when every tcgen05.mma issued so far by this thread has completed
DEV void umma_commit(unsigned long long* bar) {
#if GEMM_PAIR
    // the same barrier in both CTAs of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
#else
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
#endif
}

// shared-memory matrix descriptor: 128-byte swizzle, 1024-byte groups of 8 rows
//   K-major operand (A):  rows = M, a row holds GEMM_BK elements (128 bytes); SBO = 1024 between 8-row groups
//   MN-major operand (B): rows = K, a row holds 128 bytes of N; SBO = 1024 between 8-row K groups,
//                         LBO = bytes between 128-byte-wide N panels
DEV unsigned long long smem_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;          // descriptor version of this architecture
    d |= 2ull << 61;          // SWIZZLE_128B
    return d;
}

DEV void tmem_ld32(unsigned taddr, float* v) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// two fp32 -> packed bf16x2, round to nearest even (lo in the low half)
DEV unsigned pack_bf16x2(float lo, float hi) {
    unsigned r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
DEV float bf16_to_f32(unsigned short b) { return __uint_as_float(((unsigned)b) << 16); }

}  // namespace gemm

//@EPILOGUE@  (the host side puts the chunk I/O helpers and the EPILOGUE_CHUNK macro here)

#if GEMM_KSPLIT
// ---------------------------------------------------------------------------------------------------
// K split over a cluster of two CTAs (see GEMM_KSPLIT above).  Tile = GEMM_BM rows x GEMM_TILE_N output
// columns x GEMM_SLICES slices; accumulator column q * GEMM_TILE_N + j is slice q of output column j.
// CTA r finishes output columns [r * GEMM_FIN, (r + 1) * GEMM_FIN) of the tile (of every slice): it keeps its own
// partial sums for them, receives the peer's through `xchg` and sends the peer the partial sums of the other half.
// xchg[i][t] is the i-th float4 of row t: conflict-free on both sides.  GEMM_BN is 128 here: with four slices a
// 32-column accumulator group is one slice (16 columns each way), without slices two groups go each way.
#define GEMM_FIN (GEMM_TILE_N / 2)                              /* output columns per slice this CTA finishes */
#define GEMM_XCHG_VEC (GEMM_BN / 2 / 4)                         /* float4 per row and direction */
#define GEMM_XCHG_BYTES (GEMM_XCHG_VEC * GEMM_BM * 16)

extern "C" __global__ void __launch_bounds__(GEMM_THREADS, 1) __cluster_dims__(GEMM_KPAIR ? 4 : 2, 1, 1)
dali_gemm_kernel(const __grid_constant__ TensorMap tmA, const __grid_constant__ TensorMap tmB,
                 const __grid_constant__ TensorMap tmAlo, const __grid_constant__ TensorMap tmBlo,
                 const __grid_constant__ TensorMap tmA2, const __grid_constant__ TensorMap tmB2,
                 const __grid_constant__ TensorMap tmA2lo, const __grid_constant__ TensorMap tmB2lo,
                 const __grid_constant__ GemmP p) {
    using namespace gemm;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<unsigned long long>(smem_raw) + 1023) & ~1023ull);
    float4* xchg = reinterpret_cast<float4*>(tiles + (size_t)GEMM_STAGES * GEMM_STAGE_BYTES);
    __shared__ __align__(8) unsigned long long full_bar[GEMM_STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[GEMM_STAGES];
    __shared__ __align__(8) unsigned long long acc_full;      // MMA -> epilogue: this CTA's partial sums are complete
    __shared__ __align__(8) unsigned long long acc_empty;     // epilogue -> MMA: they have been read
    __shared__ __align__(8) unsigned long long xchg_full;     // the peer has written its half into this CTA's xchg
    __shared__ __align__(8) unsigned long long xchg_free;     // the peer has read what this CTA wrote into the peer's xchg
    __shared__ unsigned tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#if GEMM_KPAIR
    // cluster rank = 2 * (operand pair) + (row half); the MMA pair is (2p, 2p + 1), the exchange partner has the same rows
    const unsigned crank = cluster_ctarank();
    const unsigned cta_rank = crank >> 1, half = crank & 1u, peer = crank ^ 2u, lead = crank & ~1u;
    const unsigned worker = blockIdx.x >> 2, n_workers = gridDim.x >> 2;
    const unsigned short pair_mask = (unsigned short)(3u << lead);
#else
    const unsigned cta_rank = cluster_ctarank(), peer = cta_rank ^ 1u;
    const unsigned worker = blockIdx.x >> 1, n_workers = gridDim.x >> 1;
#endif
    const unsigned total_tiles = p.tiles_m * p.tiles_n;
    // CTA r (GEMM_KPAIR: CTA pair r) works on operand pair r over the whole tile
    const TensorMap* mA = cta_rank ? &tmA2 : &tmA;
    const TensorMap* mB = cta_rank ? &tmB2 : &tmB;
    const TensorMap* mAlo = cta_rank ? &tmA2lo : &tmAlo;
    const TensorMap* mBlo = cta_rank ? &tmB2lo : &tmBlo;
    const int num_kb = (int)(((cta_rank ? p.K2 : p.K) + GEMM_BK - 1) / GEMM_BK);

    auto tile_origin = [&](unsigned lin, long long* m0, long long* n0) {
        const unsigned band = lin / (GEMM_RASTER * p.tiles_m);
        const unsigned band_n0 = band * GEMM_RASTER;
        const unsigned band_w = p.tiles_n - band_n0 < GEMM_RASTER ? p.tiles_n - band_n0 : GEMM_RASTER;
        const unsigned in_band = lin - band * GEMM_RASTER * p.tiles_m;
#if GEMM_KPAIR
        *m0 = ((long long)(in_band / band_w) * 2 + half) * GEMM_BM;        // this CTA's 128 of the tile's 256 rows
#else
        *m0 = (long long)(in_band / band_w) * GEMM_BM;
#endif
        *n0 = (long long)(band_n0 + in_band % band_w) * GEMM_TILE_N;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, GEMM_KPAIR ? 8 : 4);      // GEMM_KPAIR: the epilogue warps of both CTAs report to the even one
        mbar_init(&xchg_full, 128);      // every epilogue thread of the peer arrives after its stores
        mbar_init(&xchg_free, 128);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) tmem_alloc(&tmem_slot, GEMM_TMEM_COLS);
    fence_before_sync();
    __syncthreads();
    cluster_sync();      // the peer's barriers exist before anything is sent to them
    fence_after_sync();
    const unsigned tmem_base = tmem_slot;
    // Launched as a programmatic dependent, everything above overlapped the tail of the kernel before this one in
    // the stream; nothing below may run before that kernel has completed and its writes are visible.  The kernel
    // after this one may begin its own set-up from here on (it waits the same way before it touches memory).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 4 && lane == 0) {
        // ------------------------------------------------------------ TMA producer: a_hi, [b_hi | b_lo], a_lo
        unsigned it = 0;
        bool ok = true;
        for (unsigned t = worker; t < total_tiles && ok; t += n_workers) {
            long long m0, n0;
            tile_origin(t, &m0, &n0);
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const unsigned s = it % GEMM_STAGES;
                if (!mbar_wait(&empty_bar[s], ((it / GEMM_STAGES) & 1u) ^ 1u, &abort_flag)) { atomicExch(p.err, 1); abort_flag = 1; ok = false; break; }
                unsigned char* st = tiles + (size_t)s * GEMM_STAGE_BYTES;
                const int kx = kb * GEMM_BK;
#if GEMM_KPAIR
                // stage = a_hi, b_hi, a_lo, b_lo with this CTA's HALF of the B tile's columns (slices 2 * half, 2 * half + 1 of
                // a sliced tile); both CTAs' copies report to the even CTA's barrier, which it arms for both
                if (half == 0) mbar_expect_tx(&full_bar[s], 2 * GEMM_STAGE_BYTES);
                const unsigned bar = map_to_cta(&full_bar[s], lead);
                unsigned char* bt = st + GEMM_A_TILE_BYTES;
                unsigned char* alo = bt + GEMM_B_TILE_BYTES;
                unsigned char* blo = alo + GEMM_A_TILE_BYTES;
                tma_load_2d_pair(st, mA, bar, kx, (int)m0);
                tma_load_2d_pair(alo, mAlo, bar, kx, (int)m0);
#if GEMM_SLICES > 1
                tma_load_3d_pair(bt, mB, bar, kx, (int)n0, (int)(half * (GEMM_SLICES / 2)));
                tma_load_3d_pair(blo, mBlo, bar, kx, (int)n0, (int)(half * (GEMM_SLICES / 2)));
#else
                tma_load_2d_pair(bt, mB, bar, kx, (int)(n0 + half * GEMM_BN_LOCAL));
                tma_load_2d_pair(blo, mBlo, bar, kx, (int)(n0 + half * GEMM_BN_LOCAL));
#endif
#else
                mbar_expect_tx(&full_bar[s], GEMM_STAGE_BYTES);
                tma_load_2d(st, mA, &full_bar[s], kx, (int)m0);
#if GEMM_SLICES > 1
                tma_load_3d(st + GEMM_A_TILE_BYTES, mB, &full_bar[s], kx, (int)n0, 0);
                tma_load_3d(st + GEMM_A_TILE_BYTES + GEMM_B_TILE_BYTES, mBlo, &full_bar[s], kx, (int)n0, 0);
#else
                tma_load_2d(st + GEMM_A_TILE_BYTES, mB, &full_bar[s], kx, (int)n0);
                tma_load_2d(st + GEMM_A_TILE_BYTES + GEMM_B_TILE_BYTES, mBlo, &full_bar[s], kx, (int)n0);
#endif
                tma_load_2d(st + GEMM_A_TILE_BYTES + 2 * GEMM_B_TILE_BYTES, mAlo, &full_bar[s], kx, (int)m0);
#endif
            }
        }
#if GEMM_KPAIR
    } else if (warp == 5 && lane == 0 && half == 0) {
        // ------------------------------------------------------------ MMA issuer of a CTA pair (the even CTA): every
        // instruction runs on both tensor cores, reads the A rows of each CTA from that CTA's shared memory and the two
        // halves of the B tile from both, and leaves each CTA's 128 rows of the product in its own tensor memory.
        // Accumulators: the main products round robin over GEMM_NACC sets, the two correction products in one more.
        unsigned it = 0, done = 0;
        bool ok = true;
        for (unsigned t = worker; t < total_tiles && ok && num_kb > 0; t += n_workers, ++done) {
            if (!mbar_wait_cluster(&acc_empty, (done & 1u) ^ 1u, &abort_flag)) { atomicExch(p.err, 5); abort_flag = 1; ok = false; break; }
            fence_after_sync();
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const unsigned s = it % GEMM_STAGES;
                if (!mbar_wait(&full_bar[s], (it / GEMM_STAGES) & 1u, &abort_flag)) { atomicExch(p.err, 2); abort_flag = 1; ok = false; break; }
                fence_after_sync();
                const unsigned a_addr = smem_u32(tiles + (size_t)s * GEMM_STAGE_BYTES);
                const unsigned b_addr = a_addr + GEMM_A_TILE_BYTES;
                const unsigned alo_addr = b_addr + GEMM_B_TILE_BYTES;
                const unsigned blo_addr = alo_addr + GEMM_A_TILE_BYTES;
                const unsigned corr = tmem_base + (unsigned)(GEMM_NACC * GEMM_BN);
#pragma unroll
                for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
                    const unsigned long long ad = smem_desc(a_addr + k * 32, 0, 1024);
                    const unsigned long long bd = smem_desc(b_addr + k * 32, 0, 1024);
                    const unsigned long long ald = smem_desc(alo_addr + k * 32, 0, 1024);
                    const unsigned long long bld = smem_desc(blo_addr + k * 32, 0, 1024);
                    umma(tmem_base + (unsigned)((kb % GEMM_NACC) * GEMM_BN), ad, bd, GEMM_IDESC, (kb >= GEMM_NACC || k > 0) ? 1u : 0u);
                    umma(corr, ald, bd, GEMM_IDESC, (kb > 0 || k > 0) ? 1u : 0u);     // a_lo . b_hi
                    umma(corr, ad, bld, GEMM_IDESC, 1u);                              // a_hi . b_lo
                }
                umma_commit_mask(&empty_bar[s], pair_mask);      // the stage is free in both CTAs
            }
            if (ok) umma_commit_mask(&acc_full, pair_mask);      // both CTAs' epilogues may read their rows
        }
#else
    } else if (warp == 5 && lane == 0) {
        // ------------------------------------------------------------ MMA issuer (one per CTA, its own tensor core)
        unsigned it = 0, done = 0;
        bool ok = true;
        for (unsigned t = worker; t < total_tiles && ok && num_kb > 0; t += n_workers, ++done) {
            if (!mbar_wait(&acc_empty, (done & 1u) ^ 1u, &abort_flag)) { atomicExch(p.err, 5); abort_flag = 1; ok = false; break; }
            fence_after_sync();
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const unsigned s = it % GEMM_STAGES;
                if (!mbar_wait(&full_bar[s], (it / GEMM_STAGES) & 1u, &abort_flag)) { atomicExch(p.err, 2); abort_flag = 1; ok = false; break; }
                fence_after_sync();
                const unsigned a_addr = smem_u32(tiles + (size_t)s * GEMM_STAGE_BYTES);
                const unsigned b_addr = a_addr + GEMM_A_TILE_BYTES;
                const unsigned alo_addr = b_addr + 2 * GEMM_B_TILE_BYTES;
#pragma unroll
                for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
                    const unsigned long long ad = smem_desc(a_addr + k * 32, 0, 1024);
                    const unsigned long long bd = smem_desc(b_addr + k * 32, 0, 1024);
                    const unsigned long long ald = smem_desc(alo_addr + k * 32, 0, 1024);
                    const unsigned pair0 = tmem_base + (unsigned)((kb % GEMM_NACC) * 2 * GEMM_BN);
                    umma(pair0, ad, bd, GEMM_IDESC_WIDE, (kb >= GEMM_NACC || k > 0) ? 1u : 0u);     // a_hi.[b_hi | b_lo]
                    umma(pair0 + GEMM_BN, ald, bd, GEMM_IDESC, 1u);                                 // a_lo.b_hi
                }
                umma_commit(&empty_bar[s]);
            }
            if (ok) umma_commit(&acc_full);
        }
#endif
    } else if (warp < 4) {
        // ------------------------------------------------------------ exchange + epilogue
        const int trow = warp * 32 + lane;                        // row of the tile = TMEM lane
        const unsigned peer_xchg = map_to_cta(xchg, peer);
        const unsigned peer_full = map_to_cta(&xchg_full, peer), peer_free = map_to_cta(&xchg_free, peer);
        unsigned done = 0;
        bool ok = true;
        for (unsigned t = worker; t < total_tiles && ok; t += n_workers, ++done) {
            long long m0, n0;
            tile_origin(t, &m0, &n0);
            if (num_kb > 0 && !mbar_wait(&acc_full, done & 1u, &abort_flag)) { if (lane == 0) atomicExch(p.err, 3); abort_flag = 1; ok = false; break; }
            // the peer must have read what the previous tile left in its xchg
            if (!mbar_wait_cluster(&xchg_free, (done & 1u) ^ 1u, &abort_flag)) { if (lane == 0) atomicExch(p.err, 6); abort_flag = 1; ok = false; break; }
            fence_after_sync();
            float mine[GEMM_BN / 2];                              // [slice][column of this CTA's half]
#pragma unroll
            for (int q = 0; q < GEMM_BN / 32; ++q) {
                // accumulator columns 32 q .. 32 q + 31, summed over the accumulator sets
                float v[32];
                if (num_kb > 0) {
                    const unsigned lane_base = tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)(q * 32);
                    tmem_ld32(lane_base, v);
                    const int used = num_kb < GEMM_NACC ? num_kb : GEMM_NACC;
                    float part[32];
#if GEMM_KPAIR
                    for (int a = 1; a < used; ++a) {                                      // main sets
                        tmem_ld32(lane_base + (unsigned)(a * GEMM_BN), part);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] += part[i];
                    }
                    tmem_ld32(lane_base + (unsigned)(GEMM_NACC * GEMM_BN), part);         // corrections
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] += part[i];
#else
                    for (int a = 1; a < 2 * used; ++a) {
                        tmem_ld32(lane_base + (unsigned)(a * GEMM_BN), part);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] += part[i];
                    }
#endif
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.0f;
                }
#if GEMM_SLICES > 1
                // the group is slice q (GEMM_TILE_N = 32): keep this CTA's 16 columns, send the other 16
#pragma unroll
                for (int j = 0; j < GEMM_FIN; ++j) mine[q * GEMM_FIN + j] = cta_rank ? v[GEMM_FIN + j] : v[j];
#pragma unroll
                for (int g4 = 0; g4 < GEMM_FIN / 4; ++g4) {
                    const int src = (cta_rank ? 0 : GEMM_FIN) + 4 * g4;
                    const unsigned dst = peer_xchg + (unsigned)(((q * (GEMM_FIN / 4) + g4) * GEMM_BM + trow) * 16);
                    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};"
                                 ::"r"(dst), "f"(v[src]), "f"(v[src + 1]), "f"(v[src + 2]), "f"(v[src + 3]) : "memory");
                }
#else
                // no slices: groups 0, 1 are CTA 0's columns, groups 2, 3 CTA 1's -- a group is kept or sent whole
                if ((unsigned)(q >> 1) == cta_rank) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) mine[(q & 1) * 32 + j] = v[j];
                } else {
#pragma unroll
                    for (int g4 = 0; g4 < 8; ++g4) {
                        const unsigned dst = peer_xchg + (unsigned)((((q & 1) * 8 + g4) * GEMM_BM + trow) * 16);
                        asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(dst), "f"(v[4 * g4]), "f"(v[4 * g4 + 1]), "f"(v[4 * g4 + 2]), "f"(v[4 * g4 + 3]) : "memory");
                    }
                }
#endif
            }
            if (num_kb > 0) {
                // this warp has read its part of tensor memory: the MMA issuer may start the next tile
                fence_before_sync();
                __syncwarp();
#if GEMM_KPAIR
                if (lane == 0) asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(map_to_cta(&acc_empty, lead)) : "memory");
#else
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty)) : "memory");
#endif
            }
            // tell the peer its xchg holds this thread's share, then wait for the peer's share in ours
            asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(peer_full) : "memory");
            if (!mbar_wait_cluster(&xchg_full, done & 1u, &abort_flag)) { if (lane == 0) atomicExch(p.err, 7); abort_flag = 1; ok = false; break; }
#pragma unroll
            for (int i = 0; i < GEMM_XCHG_VEC; ++i) {
                const float4 r = xchg[i * GEMM_BM + trow];
                mine[4 * i] += r.x; mine[4 * i + 1] += r.y; mine[4 * i + 2] += r.z; mine[4 * i + 3] += r.w;
            }
            // our xchg may be overwritten for the next tile
            asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(peer_free) : "memory");
            const long long row = m0 + trow;
#pragma unroll 1
            for (int sub = 0; sub < GEMM_FIN / GEMM_CHUNK; ++sub) {       // one call with slices, two 32-column calls without
                const long long col0 = n0 + (long long)cta_rank * GEMM_FIN + sub * GEMM_CHUNK;
                if (row < p.M && col0 < p.N) {
                    const int nvalid = (p.N - col0) < GEMM_CHUNK ? (int)(p.N - col0) : GEMM_CHUNK;
                    const float* acc_sub = mine + sub * GEMM_CHUNK;
                    EPILOGUE_CHUNK(row, col0, acc_sub, nvalid)
                }
            }
        }
    }
    // ---------------------------------------------------------------- teardown
    fence_before_sync();
    __syncthreads();
    if (abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
        __syncthreads();
    }
    cluster_sync();      // the peer may still be storing into this CTA's xchg or arriving on its barriers
    if (warp == 5) {
        fence_after_sync();
        tmem_dealloc(tmem_base, GEMM_TMEM_COLS);
    }
}
#else   // !GEMM_KSPLIT

extern "C" __global__ void __launch_bounds__(GEMM_THREADS, 1)
#if GEMM_PAIR
__cluster_dims__(2, 1, 1)
#endif
dali_gemm_kernel(const __grid_constant__ TensorMap tmA, const __grid_constant__ TensorMap tmB,
                 const __grid_constant__ TensorMap tmAlo, const __grid_constant__ TensorMap tmBlo,
                 const __grid_constant__ TensorMap tmA2, const __grid_constant__ TensorMap tmB2,
                 const __grid_constant__ TensorMap tmA2lo, const __grid_constant__ TensorMap tmB2lo,
                 const __grid_constant__ GemmP p) {
    using namespace gemm;
    extern __shared__ unsigned char smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle pattern
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<unsigned long long>(smem_raw) + 1023) & ~1023ull);
    __shared__ __align__(8) unsigned long long full_bar[GEMM_STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[GEMM_STAGES];
    __shared__ __align__(8) unsigned long long acc_full[GEMM_ACC_STAGES];     // MMA -> epilogue: the tile's accumulators are complete
    __shared__ __align__(8) unsigned long long acc_empty[GEMM_ACC_STAGES];    // epilogue -> MMA: they have been read
    __shared__ unsigned tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#if GEMM_PAIR
    const unsigned cta_rank = cluster_ctarank();     // the two CTAs of a pair are neighbours in x
    const unsigned worker = blockIdx.x >> 1, n_workers = gridDim.x >> 1;
#else
    const unsigned cta_rank = 0;
    const unsigned worker = blockIdx.x, n_workers = gridDim.x;
#endif
    const bool leader = cta_rank == 0;
    const unsigned total_tiles = p.tiles_m * p.tiles_n;
    const int num_kb1 = (int)((p.K + GEMM_BK - 1) / GEMM_BK);
    const int num_kb = num_kb1 + (int)((p.K2 + GEMM_BK - 1) / GEMM_BK);

    // Tiles are numbered in bands of GEMM_RASTER column tiles, rows fastest inside a band, so that the
    // operands of the tiles in flight at any time (consecutive numbers) stay inside L2.
    auto tile_origin = [&](unsigned lin, long long* m0, long long* n0) {
        const unsigned band = lin / (GEMM_RASTER * p.tiles_m);
        const unsigned band_n0 = band * GEMM_RASTER;
        const unsigned band_w = p.tiles_n - band_n0 < GEMM_RASTER ? p.tiles_n - band_n0 : GEMM_RASTER;
        const unsigned in_band = lin - band * GEMM_RASTER * p.tiles_m;
        *m0 = ((long long)(in_band / band_w) * (GEMM_PAIR ? 2 : 1) + cta_rank) * GEMM_BM;     // this CTA's rows
        *n0 = (long long)(band_n0 + in_band % band_w) * GEMM_TILE_N;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        // every epilogue warp (of both CTAs of a pair) reports to the leader's barrier
        for (int s = 0; s < GEMM_ACC_STAGES; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 4 * (GEMM_PAIR ? 2 : 1)); }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) tmem_alloc(&tmem_slot, GEMM_TMEM_COLS);
    fence_before_sync();
    __syncthreads();
#if GEMM_PAIR
    cluster_sync();      // the peer's barriers exist before anything is sent to them
#endif
    fence_after_sync();
    const unsigned tmem_base = tmem_slot;
    // Launched as a programmatic dependent, everything above overlapped the tail of the kernel before this one in
    // the stream; nothing below may run before that kernel has completed and its writes are visible.  The kernel
    // after this one may begin its own set-up from here on (it waits the same way before it touches memory).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 4 && lane == 0) {
        // ------------------------------------------------------------ TMA producer
        unsigned it = 0;      // K blocks issued so far, over all tiles: position in the stage ring
        bool ok = true;
        for (unsigned t = worker; t < total_tiles && ok; t += n_workers) {
            long long m0, n0;
            tile_origin(t, &m0, &n0);
            const long long n_load = n0 + (long long)cta_rank * GEMM_BN_LOCAL;      // the part of the B tile this CTA stages
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const unsigned s = it % GEMM_STAGES;
                const unsigned parity = (it / GEMM_STAGES) & 1u;
                if (!mbar_wait(&empty_bar[s], parity ^ 1u, &abort_flag)) { atomicExch(p.err, 1); abort_flag = 1; ok = false; break; }
                unsigned char* st = tiles + (size_t)s * GEMM_STAGE_BYTES;
                // K blocks of the second operand pair follow those of the first
                const bool second = kb >= num_kb1;
                const int kx = (second ? kb - num_kb1 : kb) * GEMM_BK;
                const TensorMap* mA = second ? &tmA2 : &tmA;
                const TensorMap* mB = second ? &tmB2 : &tmB;
                unsigned char* bt = st + GEMM_A_TILE_BYTES;
#if GEMM_PAIR
                // both CTAs' copies report to the leader's barrier, which the leader arms for both
                if (leader) mbar_expect_tx(&full_bar[s], 2 * GEMM_STAGE_BYTES);
                const unsigned bar = map_to_cta(&full_bar[s], 0);
                tma_load_2d_pair(st, mA, bar, kx, (int)m0);
#pragma unroll
                for (int j = 0; j < GEMM_B_ATOMS; ++j)
                    tma_load_2d_pair(bt + j * GEMM_B_ATOM_BYTES, mB, bar, (int)n_load + j * GEMM_SWIZZLE_ELEMS, kx);
#else
                mbar_expect_tx(&full_bar[s], GEMM_STAGE_BYTES);
                tma_load_2d(st, mA, &full_bar[s], kx, (int)m0);
#if GEMM_B_KMAJOR && GEMM_SLICES > 1
                // the transposed operand as [slice][column][k]: one copy brings the GEMM_TILE_N rows of every slice
                tma_load_3d(bt, mB, &full_bar[s], kx, (int)n0, 0);
#elif GEMM_B_KMAJOR
                tma_load_2d(bt, mB, &full_bar[s], kx, (int)n0);
#else
#pragma unroll
                for (int j = 0; j < GEMM_B_ATOMS; ++j)
                    tma_load_2d(bt + j * GEMM_B_ATOM_BYTES, mB, &full_bar[s], (int)n_load + j * GEMM_SWIZZLE_ELEMS, kx);
#endif
#if GEMM_SPLIT
                const TensorMap* mAlo = second ? &tmA2lo : &tmAlo;
                const TensorMap* mBlo = second ? &tmB2lo : &tmBlo;
#if GEMM_NCAT
                unsigned char* blo = bt + GEMM_B_TILE_BYTES;            // stage = a_hi, b_hi, b_lo, a_lo
                unsigned char* alo = blo + GEMM_B_TILE_BYTES;
#else
                unsigned char* alo = bt + GEMM_B_TILE_BYTES;            // stage = a_hi, b_hi, a_lo, b_lo
                unsigned char* blo = alo + GEMM_A_TILE_BYTES;
#endif
                tma_load_2d(alo, mAlo, &full_bar[s], kx, (int)m0);
#if GEMM_B_KMAJOR && GEMM_SLICES > 1
                tma_load_3d(blo, mBlo, &full_bar[s], kx, (int)n0, 0);
#elif GEMM_B_KMAJOR
                tma_load_2d(blo, mBlo, &full_bar[s], kx, (int)n0);
#else
#pragma unroll
                for (int j = 0; j < GEMM_B_ATOMS; ++j)
                    tma_load_2d(blo + j * GEMM_B_ATOM_BYTES, mBlo, &full_bar[s], (int)n0 + j * GEMM_SWIZZLE_ELEMS, kx);
#endif
#endif
#endif      // GEMM_PAIR
            }
        }
    } else if (warp == 5 && lane == 0 && leader) {
        // ------------------------------------------------------------ MMA issuer (of a pair: the leader CTA)
        unsigned it = 0, done = 0;     // K blocks consumed; tiles finished
        bool ok = true;
        for (unsigned t = worker; t < total_tiles && ok && num_kb > 0; t += n_workers, ++done) {
            const unsigned as = done % GEMM_ACC_STAGES;
            // the epilogue must have read what this accumulator stage held two tiles ago
            if (!mbar_wait(&acc_empty[as], ((done / GEMM_ACC_STAGES) & 1u) ^ 1u, &abort_flag)) { atomicExch(p.err, 5); abort_flag = 1; ok = false; break; }
            fence_after_sync();
            const unsigned acc0 = tmem_base + as * GEMM_ACC_COLS;
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const unsigned s = it % GEMM_STAGES;
                const unsigned parity = (it / GEMM_STAGES) & 1u;
                if (!mbar_wait(&full_bar[s], parity, &abort_flag)) { atomicExch(p.err, 2); abort_flag = 1; ok = false; break; }
                fence_after_sync();
                const unsigned a_addr = smem_u32(tiles + (size_t)s * GEMM_STAGE_BYTES);
                const unsigned b_addr = a_addr + GEMM_A_TILE_BYTES;
#pragma unroll
                for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
                    // A: 32 bytes further along its 128-byte rows; B: GEMM_UMMA_K rows (128 bytes each) further down
                    const unsigned long long ad = smem_desc(a_addr + k * 32, 0, 1024);
#if GEMM_B_KMAJOR
                    const unsigned long long bd = smem_desc(b_addr + k * 32, 0, 1024);
#else
                    const unsigned long long bd = smem_desc(b_addr + k * GEMM_UMMA_K * 128, GEMM_B_ATOM_BYTES, 1024);
#endif
#if GEMM_SPLIT && GEMM_NCAT
                    // [main | correction] pair kb % GEMM_NACC: a_hi.[b_hi | b_lo] writes both halves (the first
                    // use overwrites), a_lo.b_hi adds into the correction half
                    const unsigned pair0 = acc0 + (unsigned)((kb % GEMM_NACC) * 2 * GEMM_BN);
                    const unsigned alo_addr = b_addr + 2 * GEMM_B_TILE_BYTES;
                    const unsigned long long ald = smem_desc(alo_addr + k * 32, 0, 1024);
                    umma(pair0, ad, bd, GEMM_IDESC_WIDE, (kb >= GEMM_NACC || k > 0) ? 1u : 0u);
                    umma(pair0 + GEMM_BN, ald, bd, GEMM_IDESC, 1u);
#elif GEMM_SPLIT
                    // main products: accumulator kb % GEMM_NACC (its first use overwrites)
                    umma(acc0 + (unsigned)((kb % GEMM_NACC) * GEMM_BN), ad, bd, GEMM_IDESC, (kb >= GEMM_NACC || k > 0) ? 1u : 0u);
                    const unsigned alo_addr = b_addr + GEMM_B_TILE_BYTES;
                    const unsigned blo_addr = alo_addr + GEMM_A_TILE_BYTES;
                    const unsigned long long ald = smem_desc(alo_addr + k * 32, 0, 1024);
#if GEMM_B_KMAJOR
                    const unsigned long long bld = smem_desc(blo_addr + k * 32, 0, 1024);
#else
                    const unsigned long long bld = smem_desc(blo_addr + k * GEMM_UMMA_K * 128, GEMM_B_ATOM_BYTES, 1024);
#endif
                    const unsigned corr = acc0 + (unsigned)(GEMM_NACC * GEMM_BN);
                    umma(corr, ald, bd, GEMM_IDESC, (kb > 0 || k > 0) ? 1u : 0u);   // a_lo * b_hi
                    umma(corr, ad, bld, GEMM_IDESC, 1u);                            // a_hi * b_lo
#else
                    umma(acc0, ad, bd, GEMM_IDESC, (kb > 0 || k > 0) ? 1u : 0u);
#endif
                }
                umma_commit(&empty_bar[s]);       // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(&acc_full[as]);   // the tile's accumulators are complete
        }
    } else if (warp < 4) {
        // ------------------------------------------------------------ epilogue
        unsigned done = 0;
        bool ok = true;
        for (unsigned t = worker; t < total_tiles && ok; t += n_workers, ++done) {
            long long m0, n0;
            tile_origin(t, &m0, &n0);
            const unsigned as = done % GEMM_ACC_STAGES;
            if (num_kb > 0 && !mbar_wait(&acc_full[as], (done / GEMM_ACC_STAGES) & 1u, &abort_flag)) {
                if (lane == 0) atomicExch(p.err, 3);
                abort_flag = 1;
                ok = false;
                break;
            }
            fence_after_sync();
            const long long row = m0 + warp * 32 + lane;
#if GEMM_SLICES > 1
            {
                // all GEMM_BN accumulator columns of this row: slice q of output column j sits at q * GEMM_TILE_N + j
                float acc[GEMM_BN];
#pragma unroll
                for (int c = 0; c < GEMM_BN; c += 32) {
                    if (num_kb > 0) {
                        const unsigned lane_base = tmem_base + as * GEMM_ACC_COLS + ((unsigned)(warp * 32) << 16) + (unsigned)c;
                        tmem_ld32(lane_base, acc + c);
                        const int used = num_kb < GEMM_NACC ? num_kb : GEMM_NACC;
                        float part[32];
                        for (int a = 1; a < (GEMM_NCAT ? 2 * used : used); ++a) {
                            tmem_ld32(lane_base + (unsigned)(a * GEMM_BN), part);
#pragma unroll
                            for (int i = 0; i < 32; ++i) acc[c + i] += part[i];
                        }
#if !GEMM_NCAT
                        tmem_ld32(lane_base + (unsigned)(GEMM_NACC * GEMM_BN), part);
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[c + i] += part[i];
#endif
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[c + i] = 0.0f;
                    }
                }
                const long long col0 = n0;
                if (row < p.M && col0 < p.N) {
                    const int nvalid = (p.N - col0) < GEMM_CHUNK ? (int)(p.N - col0) : GEMM_CHUNK;
                    EPILOGUE_CHUNK(row, col0, acc, nvalid)
                }
            }
#else
#pragma unroll 1
            for (int c = 0; c < GEMM_BN; c += 32) {
                float acc[32];
                if (num_kb > 0) {
                    const unsigned lane_base = tmem_base + as * GEMM_ACC_COLS + ((unsigned)(warp * 32) << 16) + (unsigned)c;
                    tmem_ld32(lane_base, acc);
#if GEMM_SPLIT && GEMM_NCAT
                    const int used = num_kb < GEMM_NACC ? num_kb : GEMM_NACC;
                    float part[32];
                    for (int a = 1; a < 2 * used; ++a) {          // main_0 (+) corr_0 (+) main_1 (+) corr_1 ...
                        tmem_ld32(lane_base + (unsigned)(a * GEMM_BN), part);
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[i] += part[i];
                    }
#elif GEMM_SPLIT
                    const int used = num_kb < GEMM_NACC ? num_kb : GEMM_NACC;
                    float part[32];
                    for (int a = 1; a < used; ++a) {
                        tmem_ld32(lane_base + (unsigned)(a * GEMM_BN), part);
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[i] += part[i];
                    }
                    tmem_ld32(lane_base + (unsigned)(GEMM_NACC * GEMM_BN), part);
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[i] += part[i];
#endif
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
                }
                const long long col0 = n0 + c;
                if (row < p.M && col0 < p.N) {
                    const int nvalid = (p.N - col0) < 32 ? (int)(p.N - col0) : 32;
                    EPILOGUE_CHUNK(row, col0, acc, nvalid)
                }
            }
#endif      // GEMM_SLICES
            if (num_kb > 0) {
                // this warp has read its part of the accumulator stage: hand it back to the MMA issuer
                fence_before_sync();
                __syncwarp();
                if (lane == 0) arrive_at_leader(&acc_empty[as]);
            }
        }
    }
    // ---------------------------------------------------------------- teardown
    fence_before_sync();
    __syncthreads();
    if (abort_flag) {
        // let copies that were already issued land before the shared memory goes away
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
        __syncthreads();
    }
#if GEMM_PAIR
    // neither CTA may free tensor memory or leave (the leader's MMAs read the peer's shared memory,
    // the peer's copies and epilogue report to the leader's barriers) before both are done
    cluster_sync();
#endif
    if (warp == 5) {
        fence_after_sync();
        tmem_dealloc(tmem_base, GEMM_TMEM_COLS);
    }
}
#endif  // GEMM_KSPLIT
