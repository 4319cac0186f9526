// Ranks and collectives: the GPUs of one box as the shards of one computation.
//
// The reference keeps a slot per GPU in every buffer (dali/array/memory/synchronized_memory.h:46-49) but has
// no way to move data between GPUs (memory_ops.cu.cpp:120-125 asserts) and picks a device per node by a
// heuristic (dali/array/jit/jit.cpp:367-385).  Here one process drives one GPU and holds one shard; this file
// is what the shards meet through, and only reductions that cross the sharded dimension ever call it:
//
//   transport "nccl+peer"  payloads up to 256 KiB per rank go through the one-shot exchange over peer memory
//                          (peer.h, peer_exchange.cu, and inside generated all-axis kernels); larger ones
//                          through NCCL (ring / tree / in-switch reduction over NVLink)
//   transport "nccl"       everything through NCCL (peer mapping unavailable, more than 8 ranks, or
//                          DALI_B200_PEER=0)
//   transport "host"       caller-supplied functions on host buffers (any fabric torch.distributed, MPI ... offers;
//                          device buffers are staged through page-locked memory) -- what the CPU tests run on
//   transport "single"     world == 1: nothing to exchange
//
// NCCL is loaded with dlopen at the first use (the copy a host program such as PyTorch has already loaded is
// shared), so the library itself links against nothing but the CUDA runtime and NVRTC.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/dali_b200.h"
#include "peer.h"
#include "runtime.h"

namespace dalib {
cudaError_t peer_exchange_launch(cudaStream_t stream, const void* table, int dtype, int op, bool arg, void* buf, void* idx,
                                 long long n, int emulated_world);
cudaError_t arg_pick_launch(cudaStream_t stream, int dtype, int op, const void* all_values, const int* all_indices, int world,
                            long long n, void* values, int* indices);
}

using namespace dalib;

namespace {

#define CUDA_OK(call)                                                                       \
    do {                                                                                    \
        cudaError_t e_ = (call);                                                            \
        if (e_ != cudaSuccess) {                                                            \
            set_error(std::string(#call) + ": " + cudaGetErrorString(e_));                  \
            return DALIB200_ERR_CUDA;                                                       \
        }                                                                                   \
    } while (0)

// ------------------------------------------------------------------ NCCL, by name
struct Nccl {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    std::string why;
};

Nccl& nccl() {
    static Nccl n;
    return n;
}

bool load_nccl() {
    Nccl& n = nccl();
    if (n.handle) return true;
    std::vector<std::string> names;
    if (const char* e = std::getenv("DALI_B200_NCCL_LIB")) names.push_back(e);
    names.push_back("libnccl.so.2");
    names.push_back("libnccl.so");
    for (const std::string& name : names) {
        n.handle = dlopen(name.c_str(), RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);     // the copy already in the process, if any
        if (!n.handle) n.handle = dlopen(name.c_str(), RTLD_NOW | RTLD_GLOBAL);
        if (n.handle) break;
    }
    if (!n.handle) { n.why = std::string("libnccl.so.2 not found (set DALI_B200_NCCL_LIB): ") + (dlerror() ? dlerror() : ""); return false; }
    bool ok = true;
    auto sym = [&](const char* name) { void* p = dlsym(n.handle, name); if (!p) { ok = false; n.why = std::string("NCCL symbol missing: ") + name; } return p; };
    n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(sym("ncclGetUniqueId"));
    n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(sym("ncclCommInitRank"));
    n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(sym("ncclCommDestroy"));
    n.AllReduce = reinterpret_cast<decltype(n.AllReduce)>(sym("ncclAllReduce"));
    n.AllGather = reinterpret_cast<decltype(n.AllGather)>(sym("ncclAllGather"));
    n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(sym("ncclGetErrorString"));
    if (!ok) { dlclose(n.handle); n.handle = nullptr; }
    return ok;
}

#define NCCL_OK(call)                                                                       \
    do {                                                                                    \
        ncclResult_t r_ = (call);                                                           \
        if (r_ != ncclSuccess) {                                                            \
            set_error(std::string(#call) + ": " + nccl().GetErrorString(r_));               \
            return DALIB200_ERR_CUDA;                                                       \
        }                                                                                   \
    } while (0)

// ------------------------------------------------------------------ the process's communicator
enum Transport { T_NONE, T_SINGLE, T_NCCL, T_NCCL_PEER, T_HOST };

struct Comm {
    Transport transport = T_NONE;
    int world = 0, rank = 0, device = -1;
    ncclComm_t nccl = nullptr;
    // peer exchange (T_NCCL_PEER, and T_SINGLE for the generated kernels' table)
    char* block = nullptr;
    char* mapped[DALI_PEER_MAX_WORLD] = {nullptr};
    DaliPeerTable* table = nullptr;      // device
    void* words = nullptr;               // device: epochs, error, ticket
    std::string note;                    // why the peer transport is off, if it is
    // host transport
    dalib200_host_allreduce_fn host_allreduce = nullptr;
    dalib200_host_allgather_fn host_allgather = nullptr;
    void* host_ctx = nullptr;
    void* staging = nullptr;             // page-locked
    size_t staging_bytes = 0;
};

std::mutex g_mu;
Comm g_comm;
// what launches read without taking g_mu (a launch holds the runtime's own lock, collectives take g_mu first)
std::atomic<const void*> g_table_published{nullptr};
std::atomic<int> g_table_device{-1};
void publish_table(const Comm& c) {
    const bool has = (c.transport == T_NCCL_PEER || c.transport == T_SINGLE) && c.table;
    g_table_device.store(has ? c.device : -1);
    g_table_published.store(has ? c.table : nullptr);
}

unsigned long long wait_ns_setting() {
    const char* e = std::getenv("DALI_B200_PEER_WAIT_MS");
    const double ms = e && *e ? std::atof(e) : 10000.0;
    return (unsigned long long)(std::max(1.0, ms) * 1e6);
}

int dtype_bytes(int dtype) { return dtype == DALIB200_F64 ? 8 : 4; }

// Allocates the rank's exchange block and the words its kernels need; fills the table for a world of one.
int make_local_block(Comm& c) {
    CUDA_OK(cudaMalloc((void**)&c.block, DALI_PEER_BYTES));
    CUDA_OK(cudaMemset(c.block, 0, DALI_PEER_BYTES));
    CUDA_OK(cudaMalloc(&c.words, 256));
    CUDA_OK(cudaMemset(c.words, 0, 256));
    CUDA_OK(cudaMalloc((void**)&c.table, sizeof(DaliPeerTable)));
    return DALIB200_OK;
}

int upload_table(Comm& c) {
    DaliPeerTable t;
    std::memset(&t, 0, sizeof t);
    t.world = c.world;
    t.rank = c.rank;
    t.wait_ns = wait_ns_setting();
    t.epoch = reinterpret_cast<unsigned long long*>(c.words);                      // [0], [1]
    t.error = reinterpret_cast<int*>(reinterpret_cast<char*>(c.words) + 64);
    t.ticket = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(c.words) + 128);
    for (int r = 0; r < c.world; ++r) t.block[r] = r == c.rank ? c.block : c.mapped[r];
    CUDA_OK(cudaMemcpy(c.table, &t, sizeof t, cudaMemcpyHostToDevice));
    CUDA_OK(cudaDeviceSynchronize());
    return DALIB200_OK;
}

void release_peer(Comm& c) {
    for (int r = 0; r < DALI_PEER_MAX_WORLD; ++r)
        if (c.mapped[r]) { cudaIpcCloseMemHandle(c.mapped[r]); c.mapped[r] = nullptr; }
    if (c.table) { cudaFree(c.table); c.table = nullptr; }
    if (c.words) { cudaFree(c.words); c.words = nullptr; }
    if (c.block) { cudaFree(c.block); c.block = nullptr; }
}

struct Hello {            // what every rank tells every other rank at set-up
    cudaIpcMemHandle_t handle;
    int ordinal;
    int pad[15];
};

// Maps every rank's exchange block into this process.  All ranks end up with the same answer (a rank that
// fails makes every rank fall back to NCCL): the outcome is itself all-reduced.
int setup_peer(Comm& c, int ordinal) {
    const char* off = std::getenv("DALI_B200_PEER");
    bool want = !(off && off[0] == '0') && c.world <= DALI_PEER_MAX_WORLD;
    if (!want) c.note = c.world > DALI_PEER_MAX_WORLD ? "more than 8 ranks" : "DALI_B200_PEER=0";
    int rc = make_local_block(c);
    if (rc != DALIB200_OK) return rc;
    Hello mine;
    std::memset(&mine, 0, sizeof mine);
    mine.ordinal = ordinal;
    int ok = want ? 1 : 0;
    if (ok && cudaIpcGetMemHandle(&mine.handle, c.block) != cudaSuccess) {
        c.note = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(cudaGetLastError());
        ok = 0;
    }
    Hello* d_all = nullptr;
    CUDA_OK(cudaMalloc((void**)&d_all, sizeof(Hello) * (c.world + 1)));
    CUDA_OK(cudaMemcpy(d_all + c.world, &mine, sizeof mine, cudaMemcpyHostToDevice));
    NCCL_OK(nccl().AllGather(d_all + c.world, d_all, sizeof(Hello), ncclChar, c.nccl, nullptr));
    CUDA_OK(cudaStreamSynchronize(nullptr));
    std::vector<Hello> all(c.world);
    CUDA_OK(cudaMemcpy(all.data(), d_all, sizeof(Hello) * c.world, cudaMemcpyDeviceToHost));
    for (int r = 0; r < c.world && ok; ++r) {
        if (r == c.rank) continue;
        int can = 0;
        if (cudaDeviceCanAccessPeer(&can, ordinal, all[r].ordinal) != cudaSuccess || !can) {
            cudaGetLastError();
            c.note = "GPU " + std::to_string(ordinal) + " cannot address GPU " + std::to_string(all[r].ordinal);
            ok = 0;
            break;
        }
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, all[r].handle, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            c.note = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e);
            ok = 0;
            break;
        }
        c.mapped[r] = static_cast<char*>(p);
    }
    // agree
    int* d_ok = reinterpret_cast<int*>(d_all);
    CUDA_OK(cudaMemcpy(d_ok, &ok, sizeof ok, cudaMemcpyHostToDevice));
    NCCL_OK(nccl().AllReduce(d_ok, d_ok, 1, ncclInt32, ncclMin, c.nccl, nullptr));
    CUDA_OK(cudaStreamSynchronize(nullptr));
    int all_ok = 0;
    CUDA_OK(cudaMemcpy(&all_ok, d_ok, sizeof all_ok, cudaMemcpyDeviceToHost));
    cudaFree(d_all);
    if (!all_ok) {
        if (ok) c.note = "another rank could not map its peers";
        for (int r = 0; r < DALI_PEER_MAX_WORLD; ++r)
            if (c.mapped[r]) { cudaIpcCloseMemHandle(c.mapped[r]); c.mapped[r] = nullptr; }
        c.transport = T_NCCL;
        return DALIB200_OK;
    }
    c.transport = T_NCCL_PEER;
    return upload_table(c);
}

ncclDataType_t nccl_dtype(int dtype) { return dtype == DALIB200_F64 ? ncclFloat64 : (dtype == DALIB200_I32 ? ncclInt32 : ncclFloat32); }
ncclRedOp_t nccl_op(int op) {
    switch (op) {
        case DALIB200_OP_PROD: return ncclProd;
        case DALIB200_OP_MAX: return ncclMax;
        case DALIB200_OP_MIN: return ncclMin;
        default: return ncclSum;
    }
}

int ensure_staging(Comm& c, size_t bytes) {
    if (c.staging_bytes >= bytes) return DALIB200_OK;
    if (c.staging) cudaFreeHost(c.staging);
    c.staging = nullptr;
    c.staging_bytes = 0;
    size_t want = std::max<size_t>(bytes, 1 << 20);
    CUDA_OK(cudaHostAlloc(&c.staging, want, cudaHostAllocPortable));
    c.staging_bytes = want;
    return DALIB200_OK;
}

template <typename T> void host_arg_pick(int op, const T* all_v, const int* all_i, int world, int64_t n, T* v, int* i) {
    for (int64_t e = 0; e < n; ++e) {
        T bv = all_v[e];
        int bi = all_i[e];
        for (int r = 1; r < world; ++r) {
            const T x = all_v[(int64_t)r * n + e];
            const int xi = all_i[(int64_t)r * n + e];
            const bool better = op == DALIB200_OP_MAX ? x > bv : x < bv;
            if (better || (x == bv && xi < bi)) { bv = x; bi = xi; }
        }
        v[e] = bv;
        i[e] = bi;
    }
}

int check_args(const Comm& c, int dtype, int op, int64_t n, const void* buf, bool arg) {
    if (c.transport == T_NONE) { set_error("no communicator: call dalib200_comm_init_rank (or _init_host) first"); return DALIB200_ERR_INVALID; }
    if (dtype != DALIB200_F32 && dtype != DALIB200_F64 && dtype != DALIB200_I32) { set_error("collective: dtype must be f32, f64 or i32"); return DALIB200_ERR_INVALID; }
    if (op < DALIB200_OP_SUM || op > DALIB200_OP_MIN) { set_error("collective: unknown reduction"); return DALIB200_ERR_INVALID; }
    if (arg && op != DALIB200_OP_MAX && op != DALIB200_OP_MIN) { set_error("arg collective: max or min only"); return DALIB200_ERR_INVALID; }
    if (n < 0 || (n > 0 && !buf)) { set_error("collective: bad buffer"); return DALIB200_ERR_INVALID; }
    return DALIB200_OK;
}

}  // namespace

namespace dalib {
// Device address of the rank's peer table for generated kernels that reduce across ranks; nullptr when the
// transport has none (the front end then finishes such a reduction with dalib200_allreduce instead).
const void* comm_peer_table(int device) {
    return g_table_device.load() == device ? g_table_published.load() : nullptr;
}
}  // namespace dalib

extern "C" {

int dalib200_shard_range(int64_t n, int rank, int world, int64_t* lo, int64_t* hi) {
    if (n < 0 || world < 1 || rank < 0 || rank >= world || !lo || !hi) { set_error("dalib200_shard_range: bad argument"); return DALIB200_ERR_INVALID; }
    const int64_t base = n / world, extra = n % world;
    *lo = rank * base + std::min<int64_t>(rank, extra);
    *hi = *lo + base + (rank < extra ? 1 : 0);
    return DALIB200_OK;
}

int dalib200_comm_unique_id(void* id) {
    if (!id) { set_error("null id"); return DALIB200_ERR_INVALID; }
    if (!load_nccl()) { set_error(nccl().why); return DALIB200_ERR_UNSUPPORTED; }
    static_assert(sizeof(ncclUniqueId) == DALIB200_COMM_ID_BYTES, "NCCL unique id size");
    ncclUniqueId u;
    NCCL_OK(nccl().GetUniqueId(&u));
    std::memcpy(id, &u, sizeof u);
    return DALIB200_OK;
}

int dalib200_comm_init_rank(int device, int world, int rank, const void* id) {
    DeviceRestore restore_device;
    std::lock_guard<std::mutex> g(g_mu);
    Comm& c = g_comm;
    if (c.transport != T_NONE) { set_error("a communicator exists already (dalib200_comm_destroy first)"); return DALIB200_ERR_INVALID; }
    if (world < 1 || rank < 0 || rank >= world) { set_error("dalib200_comm_init_rank: bad world / rank"); return DALIB200_ERR_INVALID; }
    const int ordinal = device_ordinal(device);
    if (ordinal < 0) { set_error("dalib200_comm_init_rank: device not bound (dalib200_init first)"); return dalib200_device_count() ? DALIB200_ERR_INVALID : DALIB200_ERR_NO_DEVICE; }
    CUDA_OK(cudaSetDevice(ordinal));
    c = Comm();
    c.world = world; c.rank = rank; c.device = device;
    if (world == 1) {
        int rc = make_local_block(c);
        if (rc == DALIB200_OK) rc = upload_table(c);
        if (rc != DALIB200_OK) { release_peer(c); c = Comm(); return rc; }
        c.transport = T_SINGLE;
        publish_table(c);
        return DALIB200_OK;
    }
    if (!id) { set_error("dalib200_comm_init_rank: null id"); return DALIB200_ERR_INVALID; }
    if (!load_nccl()) { set_error(nccl().why); return DALIB200_ERR_UNSUPPORTED; }
    ncclUniqueId u;
    std::memcpy(&u, id, sizeof u);
    NCCL_OK(nccl().CommInitRank(&c.nccl, world, u, rank));
    c.transport = T_NCCL;
    int rc = setup_peer(c, ordinal);
    if (rc != DALIB200_OK) {
        release_peer(c);
        nccl().CommDestroy(c.nccl);
        c = Comm();
        return rc;
    }
    if (c.transport == T_NCCL) release_peer(c);
    publish_table(c);
    return DALIB200_OK;
}

int dalib200_comm_init_host(int world, int rank, dalib200_host_allreduce_fn allreduce, dalib200_host_allgather_fn allgather, void* ctx) {
    std::lock_guard<std::mutex> g(g_mu);
    Comm& c = g_comm;
    if (c.transport != T_NONE) { set_error("a communicator exists already (dalib200_comm_destroy first)"); return DALIB200_ERR_INVALID; }
    if (world < 1 || rank < 0 || rank >= world || !allreduce || !allgather) { set_error("dalib200_comm_init_host: bad argument"); return DALIB200_ERR_INVALID; }
    c = Comm();
    c.world = world; c.rank = rank; c.device = -1;
    c.host_allreduce = allreduce; c.host_allgather = allgather; c.host_ctx = ctx;
    c.transport = T_HOST;
    return DALIB200_OK;
}

int dalib200_comm_world(void) { std::lock_guard<std::mutex> g(g_mu); return g_comm.transport == T_NONE ? 0 : g_comm.world; }
int dalib200_comm_rank(void) { std::lock_guard<std::mutex> g(g_mu); return g_comm.transport == T_NONE ? -1 : g_comm.rank; }

size_t dalib200_comm_transport(char* buffer, size_t capacity) {
    std::lock_guard<std::mutex> g(g_mu);
    std::string s;
    switch (g_comm.transport) {
        case T_NONE: s = "none"; break;
        case T_SINGLE: s = "single"; break;
        case T_NCCL: s = "nccl (" + g_comm.note + ")"; break;
        case T_NCCL_PEER: s = "nccl+peer"; break;
        case T_HOST: s = "host"; break;
    }
    if (buffer && capacity) {
        size_t n = std::min(s.size(), capacity - 1);
        std::memcpy(buffer, s.data(), n);
        buffer[n] = '\0';
    }
    return s.size();
}

int dalib200_comm_destroy(void) {
    DeviceRestore restore_device;
    std::lock_guard<std::mutex> g(g_mu);
    Comm& c = g_comm;
    if (c.transport == T_NONE) return DALIB200_OK;
    if (c.device >= 0) {
        const int ordinal = device_ordinal(c.device);
        if (ordinal >= 0) { cudaSetDevice(ordinal); cudaDeviceSynchronize(); }
    }
    g_table_published.store(nullptr);
    g_table_device.store(-1);
    release_peer(c);
    if (c.nccl) nccl().CommDestroy(c.nccl);
    if (c.staging) cudaFreeHost(c.staging);
    c = Comm();
    return DALIB200_OK;
}

int dalib200_comm_error_flag(int* flag) {
    DeviceRestore restore_device;
    std::lock_guard<std::mutex> g(g_mu);
    Comm& c = g_comm;
    if (!flag) { set_error("null flag"); return DALIB200_ERR_INVALID; }
    *flag = 0;
    if (!c.words) return DALIB200_OK;
    CUDA_OK(cudaSetDevice(device_ordinal(c.device)));
    CUDA_OK(cudaDeviceSynchronize());
    CUDA_OK(cudaMemcpy(flag, reinterpret_cast<char*>(c.words) + 64, sizeof(int), cudaMemcpyDeviceToHost));
    if (*flag) CUDA_OK(cudaMemset(reinterpret_cast<char*>(c.words) + 64, 0, sizeof(int)));
    return DALIB200_OK;
}

int dalib200_allreduce(int device, void* stream, void* buf, int64_t n, int dtype, int op) {
    DeviceRestore restore_device;
    std::lock_guard<std::mutex> g(g_mu);
    Comm& c = g_comm;
    int rc = check_args(c, dtype, op, n, buf, false);
    if (rc != DALIB200_OK) return rc;
    if (n == 0 || c.transport == T_SINGLE || c.world == 1) return DALIB200_OK;
    const size_t bytes = (size_t)n * dtype_bytes(dtype);
    if (c.transport == T_HOST) {
        if (device < 0) {
            if (c.host_allreduce(c.host_ctx, buf, n, dtype, op) != 0) { set_error("host all-reduce callback failed"); return DALIB200_ERR_CUDA; }
            return DALIB200_OK;
        }
        const int ordinal = device_ordinal(device);
        if (ordinal < 0) { set_error("collective: device not bound"); return DALIB200_ERR_INVALID; }
        CUDA_OK(cudaSetDevice(ordinal));
        rc = ensure_staging(c, bytes);
        if (rc != DALIB200_OK) return rc;
        CUDA_OK(cudaMemcpyAsync(c.staging, buf, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
        CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
        if (c.host_allreduce(c.host_ctx, c.staging, n, dtype, op) != 0) { set_error("host all-reduce callback failed"); return DALIB200_ERR_CUDA; }
        CUDA_OK(cudaMemcpyAsync(buf, c.staging, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
        CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));      // the staging buffer is reused by the next call
        return DALIB200_OK;
    }
    if (device != c.device) { set_error("collective: the communicator was created on another device"); return DALIB200_ERR_INVALID; }
    CUDA_OK(cudaSetDevice(device_ordinal(device)));
    const char* force = std::getenv("DALI_B200_ALLREDUCE");
    const bool peer = c.transport == T_NCCL_PEER && bytes <= DALI_PEER_SLOT_BYTES && !(force && std::string(force) == "nccl");
    if (peer) {
        CUDA_OK(peer_exchange_launch((cudaStream_t)stream, c.table, dtype, op, false, buf, nullptr, n, 0));
        count_launch();
        return DALIB200_OK;
    }
    NCCL_OK(nccl().AllReduce(buf, buf, (size_t)n, nccl_dtype(dtype), nccl_op(op), c.nccl, (cudaStream_t)stream));
    return DALIB200_OK;
}

int dalib200_arg_allreduce(int device, void* stream, void* values, int32_t* indices, int64_t n, int dtype, int op) {
    DeviceRestore restore_device;
    std::lock_guard<std::mutex> g(g_mu);
    Comm& c = g_comm;
    int rc = check_args(c, dtype, op, n, values, true);
    if (rc != DALIB200_OK) return rc;
    if (n > 0 && !indices) { set_error("arg collective: null indices"); return DALIB200_ERR_INVALID; }
    if (n == 0 || c.transport == T_SINGLE || c.world == 1) return DALIB200_OK;
    const int item = dtype_bytes(dtype);
    const size_t vbytes = (size_t)n * item, ibytes = (size_t)n * 4;
    if (c.transport == T_HOST) {
        std::vector<char> all_v(vbytes * c.world);
        std::vector<int> all_i((size_t)n * c.world);
        void* hv = values;
        int* hi = indices;
        cudaStream_t s = (cudaStream_t)stream;
        if (device >= 0) {
            const int ordinal = device_ordinal(device);
            if (ordinal < 0) { set_error("collective: device not bound"); return DALIB200_ERR_INVALID; }
            CUDA_OK(cudaSetDevice(ordinal));
            rc = ensure_staging(c, vbytes + ibytes);
            if (rc != DALIB200_OK) return rc;
            hv = c.staging;
            hi = reinterpret_cast<int*>(static_cast<char*>(c.staging) + vbytes);
            CUDA_OK(cudaMemcpyAsync(hv, values, vbytes, cudaMemcpyDeviceToHost, s));
            CUDA_OK(cudaMemcpyAsync(hi, indices, ibytes, cudaMemcpyDeviceToHost, s));
            CUDA_OK(cudaStreamSynchronize(s));
        }
        if (c.host_allgather(c.host_ctx, hv, all_v.data(), (int64_t)vbytes) != 0 ||
            c.host_allgather(c.host_ctx, hi, all_i.data(), (int64_t)ibytes) != 0) {
            set_error("host all-gather callback failed");
            return DALIB200_ERR_CUDA;
        }
        if (dtype == DALIB200_F32) host_arg_pick(op, reinterpret_cast<const float*>(all_v.data()), all_i.data(), c.world, n, static_cast<float*>(hv), hi);
        else if (dtype == DALIB200_F64) host_arg_pick(op, reinterpret_cast<const double*>(all_v.data()), all_i.data(), c.world, n, static_cast<double*>(hv), hi);
        else host_arg_pick(op, reinterpret_cast<const int*>(all_v.data()), all_i.data(), c.world, n, static_cast<int*>(hv), hi);
        if (device >= 0) {
            CUDA_OK(cudaMemcpyAsync(values, hv, vbytes, cudaMemcpyHostToDevice, s));
            CUDA_OK(cudaMemcpyAsync(indices, hi, ibytes, cudaMemcpyHostToDevice, s));
            CUDA_OK(cudaStreamSynchronize(s));
        }
        return DALIB200_OK;
    }
    if (device != c.device) { set_error("collective: the communicator was created on another device"); return DALIB200_ERR_INVALID; }
    CUDA_OK(cudaSetDevice(device_ordinal(device)));
    const char* force = std::getenv("DALI_B200_ALLREDUCE");
    const bool peer = c.transport == T_NCCL_PEER && (size_t)n * 8 <= DALI_PEER_SLOT_BYTES / 2 && !(force && std::string(force) == "nccl");
    if (peer) {
        CUDA_OK(peer_exchange_launch((cudaStream_t)stream, c.table, dtype, op, true, values, indices, n, 0));
        count_launch();
        return DALIB200_OK;
    }
    // NCCL has no arg-reduction: gather every rank's (value, index) pairs and pick locally, lowest index among equals
    void* all = nullptr;
    rc = scratch_space(device, stream, (vbytes + ibytes) * c.world + 256, &all);
    if (rc != DALIB200_OK) return rc;
    char* all_v = static_cast<char*>(all);
    int* all_i = reinterpret_cast<int*>(all_v + ((vbytes * c.world + 255) / 256) * 256);
    NCCL_OK(nccl().AllGather(values, all_v, vbytes, ncclChar, c.nccl, (cudaStream_t)stream));
    NCCL_OK(nccl().AllGather(indices, all_i, ibytes, ncclChar, c.nccl, (cudaStream_t)stream));
    CUDA_OK(arg_pick_launch((cudaStream_t)stream, dtype, op, all_v, all_i, c.world, n, values, indices));
    count_launch();
    return DALIB200_OK;
}

int dalib200_peer_emulate(int device, void* stream, int world, int dtype, int op, int arg, void* const* bufs,
                          int32_t* const* indices, int64_t n, int repeats, int* error_flag) {
    DeviceRestore restore_device;
    const int ordinal = device_ordinal(device);
    if (ordinal < 0) { set_error("dalib200_peer_emulate: device not bound (dalib200_init first)"); return dalib200_device_count() ? DALIB200_ERR_INVALID : DALIB200_ERR_NO_DEVICE; }
    if (world < 1 || world > DALI_PEER_MAX_WORLD || !bufs || n <= 0 || repeats < 1 || (arg && !indices)) { set_error("dalib200_peer_emulate: bad argument"); return DALIB200_ERR_INVALID; }
    if (n * dtype_bytes(dtype) > (arg ? DALI_PEER_SLOT_BYTES / 2 : DALI_PEER_SLOT_BYTES)) { set_error("dalib200_peer_emulate: payload larger than a slot"); return DALIB200_ERR_TOO_LARGE; }
    CUDA_OK(cudaSetDevice(ordinal));
    // every virtual rank's CTAs must be resident at once
    const long long chunks = (n * dtype_bytes(dtype) + DALI_PEER_CHUNK_BYTES - 1) / DALI_PEER_CHUNK_BYTES;
    int sms = 0;
    CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal));
    if (chunks * world > sms) { set_error("dalib200_peer_emulate: more CTAs than SMs; use a smaller payload"); return DALIB200_ERR_TOO_LARGE; }
    char* blocks = nullptr;
    char* words = nullptr;
    DaliPeerTable* tables = nullptr;
    void** d_bufs = nullptr;
    CUDA_OK(cudaMalloc((void**)&blocks, DALI_PEER_BYTES * world));
    CUDA_OK(cudaMemset(blocks, 0, DALI_PEER_BYTES * world));
    CUDA_OK(cudaMalloc((void**)&words, 256 * world));
    CUDA_OK(cudaMemset(words, 0, 256 * world));
    CUDA_OK(cudaMalloc((void**)&tables, sizeof(DaliPeerTable) * world));
    CUDA_OK(cudaMalloc((void**)&d_bufs, sizeof(void*) * 2 * world));
    std::vector<DaliPeerTable> t(world);
    for (int r = 0; r < world; ++r) {
        std::memset(&t[r], 0, sizeof(DaliPeerTable));
        t[r].world = world; t[r].rank = r; t[r].wait_ns = 2000000000ull;
        t[r].epoch = reinterpret_cast<unsigned long long*>(words + 256 * r);
        t[r].error = reinterpret_cast<int*>(words + 256 * r + 64);
        t[r].ticket = reinterpret_cast<unsigned int*>(words + 256 * r + 128);
        for (int q = 0; q < world; ++q) t[r].block[q] = blocks + DALI_PEER_BYTES * q;
    }
    std::vector<void*> ptrs(2 * world, nullptr);
    for (int r = 0; r < world; ++r) { ptrs[r] = bufs[r]; ptrs[world + r] = arg ? (void*)indices[r] : nullptr; }
    CUDA_OK(cudaMemcpy(tables, t.data(), sizeof(DaliPeerTable) * world, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_bufs, ptrs.data(), sizeof(void*) * 2 * world, cudaMemcpyHostToDevice));
    cudaError_t e = cudaSuccess;
    for (int k = 0; k < repeats && e == cudaSuccess; ++k)
        e = peer_exchange_launch((cudaStream_t)stream, tables, dtype, op, arg != 0, d_bufs, d_bufs + world, n, world);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    int flag = 0;
    for (int r = 0; r < world && e == cudaSuccess; ++r) {
        int f = 0;
        e = cudaMemcpy(&f, words + 256 * r + 64, sizeof f, cudaMemcpyDeviceToHost);
        flag |= f;
    }
    cudaFree(d_bufs); cudaFree(tables); cudaFree(words); cudaFree(blocks);
    if (e != cudaSuccess) { set_error(std::string("dalib200_peer_emulate: ") + cudaGetErrorString(e)); return DALIB200_ERR_CUDA; }
    if (error_flag) *error_flag = flag;
    return DALIB200_OK;
}

}  // extern "C"
