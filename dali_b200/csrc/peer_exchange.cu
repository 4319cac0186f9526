// One-shot collectives over peer memory (see peer.h for the protocol): all-reduce of small
// payloads and the (value, index) combine of sharded arg-reductions.
//
// The reference has no collective of any kind (its cross-GPU copy asserts,
// dali/array/memory/memory_ops.cu.cpp:120-125); these kernels are what stands behind
// dalib200_allreduce / dalib200_arg_allreduce when every rank's exchange block is mapped
// into every other rank (comm.cc).  A CTA owns one 4 KiB chunk of the payload end to end:
// it stores the chunk into its rank's slot on every GPU (128-bit stores over NVLink),
// raises the chunk's flag everywhere, waits -- bounded -- for the same chunk of every rank
// to arrive in its own block and folds them in rank order.  CTAs never wait on one another.
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/dali_b200.h"
#include "peer.h"
#include "peer_device.cuh"
#include "runtime.h"

namespace {

constexpr int kThreads = 256;
enum { OP_SUM = 0, OP_PROD = 1, OP_MAX = 2, OP_MIN = 3 };

template <int OP, typename T> __device__ __forceinline__ T fold(T a, T b) {
    if (OP == OP_SUM) return a + b;
    if (OP == OP_PROD) return a * b;
    if (OP == OP_MAX) return b > a ? b : a;
    return b < a ? b : a;
}
template <int OP, typename T> __device__ __forceinline__ bool better(T v, T than) { return OP == OP_MAX ? v > than : v < than; }

// One rank's part of the exchange for chunk `chunk`.  ARG: `idx` travels with the values in the upper half of
// the slot and the fold keeps, per element, the extreme value and the lowest index among equal values.
template <typename T, int OP, bool ARG>
__device__ __forceinline__ void exchange_chunk(const DaliPeerTable& t, T* buf, int* idx, long long n, int chunk, int n_chunks) {
    constexpr int EPT = 16 / (int)sizeof(T);                 // elements per thread (one 128-bit store)
    constexpr int EPC = DALI_PEER_CHUNK_BYTES / (int)sizeof(T);
    constexpr int IDX_OFF = DALI_PEER_SLOT_BYTES / 2;
    __shared__ unsigned long long s_epoch;
    const int tid = threadIdx.x;
    if (tid == 0) s_epoch = *t.epoch + 1;
    __syncthreads();
    const unsigned long long epoch = s_epoch;
    const int parity = (int)(epoch & 1);
    const long long e0 = (long long)chunk * EPC + (long long)tid * EPT;

    // ---- my contribution, into my slot on every rank (my own included)
    struct alignas(16) Pack { T x[EPT]; };
    Pack mine;
#pragma unroll
    for (int j = 0; j < EPT; ++j) mine.x[j] = e0 + j < n ? buf[e0 + j] : (T)0;
    int mine_i[EPT];
    if (ARG) {
#pragma unroll
        for (int j = 0; j < EPT; ++j) mine_i[j] = e0 + j < n ? idx[e0 + j] : 0;
    }
    for (int r = 0; r < t.world; ++r) {
        char* slot = dali_peer_slot(t.block[r], parity, t.rank);
        *reinterpret_cast<Pack*>(slot + (size_t)chunk * DALI_PEER_CHUNK_BYTES + (size_t)tid * 16) = mine;
        if (ARG) {
            int* dst = reinterpret_cast<int*>(slot + IDX_OFF) + e0;
#pragma unroll
            for (int j = 0; j < EPT; ++j) dst[j] = mine_i[j];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (tid < t.world) dali_peer_flag_release(dali_peer_flag(t.block[tid], parity, t.rank, chunk), epoch);

    // ---- everyone's contribution to this chunk, out of my own block
    char* const my_block = t.block[t.rank];
    // (a wait that gives up has raised *t.error: the fold below then runs on whatever the block holds and the
    // host learns of it from the error word)
    if (tid < t.world) dali_peer_wait(dali_peer_flag(my_block, parity, tid, chunk), epoch, t.wait_ns, t.error);
    __syncthreads();
    {
        Pack acc;
        int acc_i[EPT];
        for (int r = 0; r < t.world; ++r) {
            const char* slot = dali_peer_slot(my_block, parity, r);
            const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(slot + (size_t)chunk * DALI_PEER_CHUNK_BYTES + (size_t)tid * 16));
            Pack in;
            *reinterpret_cast<uint4*>(&in) = raw;
            int in_i[EPT];
            if (ARG) {
                const int* src = reinterpret_cast<const int*>(slot + IDX_OFF) + e0;
#pragma unroll
                for (int j = 0; j < EPT; ++j) in_i[j] = __ldcg(src + j);
            }
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                if (r == 0) {
                    acc.x[j] = in.x[j];
                    if (ARG) acc_i[j] = in_i[j];
                } else if (ARG) {
                    if (better<OP>(in.x[j], acc.x[j]) || (in.x[j] == acc.x[j] && in_i[j] < acc_i[j])) { acc.x[j] = in.x[j]; acc_i[j] = in_i[j]; }
                } else {
                    acc.x[j] = fold<OP>(acc.x[j], in.x[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (e0 + j < n) {
                buf[e0 + j] = acc.x[j];
                if (ARG) idx[e0 + j] = acc_i[j];
            }
    }
    // ---- the last chunk to finish advances the rank's epoch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicInc(t.ticket, (unsigned)n_chunks - 1) == (unsigned)n_chunks - 1) {
            *t.epoch = epoch;
            __threadfence();
        }
    }
}

template <typename T, int OP, bool ARG>
__global__ void __launch_bounds__(kThreads) peer_exchange_kernel(const DaliPeerTable* table, T* buf, int* idx, long long n) {
    exchange_chunk<T, OP, ARG>(*table, buf, idx, n, (int)blockIdx.x, (int)gridDim.x);
}

// `world` virtual ranks in ONE cooperative launch on one GPU (blockIdx.y = rank): the protocol, fold order and
// epoch handling of the kernel above on a box with fewer GPUs than ranks.  Separate launches on one GPU must
// never wait on one another, hence one grid whose CTAs are all resident.
template <typename T, int OP, bool ARG>
__global__ void __launch_bounds__(kThreads) peer_exchange_emulated_kernel(const DaliPeerTable* tables, T* const* bufs, int* const* idxs, long long n) {
    const int r = (int)blockIdx.y;
    exchange_chunk<T, OP, ARG>(tables[r], bufs[r], ARG ? idxs[r] : nullptr, n, (int)blockIdx.x, (int)gridDim.x);
}

template <typename T, bool ARG>
cudaError_t launch_op(int op, bool emulated, dim3 grid, cudaStream_t s, const void* table, void* buf, void* idx, long long n) {
    void* args[] = {(void*)&table, (void*)&buf, (void*)&idx, (void*)&n};
    const void* fn = nullptr;
#define DALI_PICK(OPC)                                                                                    \
    fn = emulated ? (const void*)peer_exchange_emulated_kernel<T, OPC, ARG> : (const void*)peer_exchange_kernel<T, OPC, ARG>
    switch (op) {
        case OP_SUM: if (ARG) return cudaErrorInvalidValue; DALI_PICK(OP_SUM); break;
        case OP_PROD: if (ARG) return cudaErrorInvalidValue; DALI_PICK(OP_PROD); break;
        case OP_MAX: DALI_PICK(OP_MAX); break;
        case OP_MIN: DALI_PICK(OP_MIN); break;
        default: return cudaErrorInvalidValue;
    }
#undef DALI_PICK
    if (emulated) return cudaLaunchCooperativeKernel(fn, grid, dim3(kThreads), args, 0, s);
    return cudaLaunchKernel(fn, grid, dim3(kThreads), args, 0, s);
}

// all_values / all_indices: [world, n] as gathered by NCCL; the extreme per element, lowest index among equals
template <typename T, int OP>
__global__ void arg_pick_kernel(const T* all_values, const int* all_indices, int world, long long n, T* values, int* indices) {
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
        T bv = all_values[e];
        int bi = all_indices[e];
        for (int r = 1; r < world; ++r) {
            const T x = all_values[(long long)r * n + e];
            const int xi = all_indices[(long long)r * n + e];
            if (better<OP>(x, bv) || (x == bv && xi < bi)) { bv = x; bi = xi; }
        }
        values[e] = bv;
        indices[e] = bi;
    }
}

template <typename T>
cudaError_t launch_pick(cudaStream_t s, int op, const void* av, const int* ai, int world, long long n, void* v, int* i) {
    const unsigned grid = (unsigned)((n + kThreads - 1) / kThreads < 1184 ? (n + kThreads - 1) / kThreads : 1184);
    if (op == OP_MAX) arg_pick_kernel<T, OP_MAX><<<grid, kThreads, 0, s>>>((const T*)av, ai, world, n, (T*)v, i);
    else arg_pick_kernel<T, OP_MIN><<<grid, kThreads, 0, s>>>((const T*)av, ai, world, n, (T*)v, i);
    return cudaGetLastError();
}

}  // namespace

namespace dalib {

cudaError_t arg_pick_launch(cudaStream_t stream, int dtype, int op, const void* all_values, const int* all_indices, int world,
                            long long n, void* values, int* indices) {
    if (n <= 0) return cudaSuccess;
    if (op != OP_MAX && op != OP_MIN) return cudaErrorInvalidValue;
    switch (dtype) {
        case DALIB200_F32: return launch_pick<float>(stream, op, all_values, all_indices, world, n, values, indices);
        case DALIB200_F64: return launch_pick<double>(stream, op, all_values, all_indices, world, n, values, indices);
        case DALIB200_I32: return launch_pick<int>(stream, op, all_values, all_indices, world, n, values, indices);
        default: return cudaErrorInvalidValue;
    }
}

// Launches the exchange on `stream` of the current device.  table: device address of the rank's DaliPeerTable
// (emulated: of `world` tables, buf / idx then being device arrays of per-rank pointers).
cudaError_t peer_exchange_launch(cudaStream_t stream, const void* table, int dtype, int op, bool arg, void* buf, void* idx,
                                 long long n, int emulated_world) {
    const int item = dtype == DALIB200_F64 ? 8 : 4;
    const long long bytes = n * item;
    if (n <= 0 || bytes > (arg ? DALI_PEER_SLOT_BYTES / 2 : DALI_PEER_SLOT_BYTES)) return cudaErrorInvalidValue;
    const unsigned chunks = (unsigned)((bytes + DALI_PEER_CHUNK_BYTES - 1) / DALI_PEER_CHUNK_BYTES);
    dim3 grid(chunks, emulated_world > 0 ? (unsigned)emulated_world : 1u);
    const bool emu = emulated_world > 0;
    switch (dtype) {
        case DALIB200_F32: return arg ? launch_op<float, true>(op, emu, grid, stream, table, buf, idx, n)
                                      : launch_op<float, false>(op, emu, grid, stream, table, buf, idx, n);
        case DALIB200_F64: return arg ? launch_op<double, true>(op, emu, grid, stream, table, buf, idx, n)
                                      : launch_op<double, false>(op, emu, grid, stream, table, buf, idx, n);
        case DALIB200_I32: return arg ? launch_op<int, true>(op, emu, grid, stream, table, buf, idx, n)
                                      : launch_op<int, false>(op, emu, grid, stream, table, buf, idx, n);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace dalib
