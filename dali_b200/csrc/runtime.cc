// C ABI implementation: registry, NVRTC compile cache, launch, memory pool.
//
// Replaces dali/utils/compiler.cpp (source -> system("nvcc ...") -> dlopen ->
// function pointer map) with NVRTC -> cubin -> cuModuleLoadData, and
// dali/array/memory/{memory_bank,memory_ops} with a 64-bit pooled allocator.
#include <cuda.h>
#include <cuda_runtime.h>
#include <nvrtc.h>

#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <unordered_map>

#include "../../include/dali_b200.h"
#include "runtime.h"

namespace dalib {

static const char* kPrelude =
#include "prelude_embed.inc"
    ;
// Hash (made by the build) of the sources that decide the text of a generated kernel and the layout of its parameter
// block -- code generator, launch planner, IR, GEMM skeleton and its host side, device prelude.  It is part of every
// cache key: a cubin on disk is only ever loaded by a library built from the same sources as the one that wrote it.
static const char* kCodegenVersion = "dali_b200-"
#include "source_hash.inc"
    ;

// ------------------------------------------------------------------ errors
static thread_local std::string tl_error;
static thread_local std::string tl_variant;
void set_error(const std::string& msg) { tl_error = msg; }
const std::string& get_error() { return tl_error; }

DeviceRestore::DeviceRestore() : prev(-1) {
    if (cudaGetDevice(&prev) != cudaSuccess) { prev = -1; cudaGetLastError(); }
}
DeviceRestore::~DeviceRestore() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
}

uint64_t fnv1a(const std::string& s, uint64_t h) {
    for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
    return h;
}

// ------------------------------------------------------------------ NVRTC
// DALI_B200_DEFINES="A,B=2": macros handed to every generated kernel (tuning switches of the device prelude).  The text
// is part of the kernel cache key.
std::string nvrtc_defines_text() {
    const char* e = std::getenv("DALI_B200_DEFINES");
    return e ? std::string(e) : std::string();
}
static std::vector<std::string> nvrtc_defines() {
    std::vector<std::string> out;
    std::string text = nvrtc_defines_text(), cur;
    for (size_t i = 0; i <= text.size(); ++i) {
        if (i == text.size() || text[i] == ',') {
            if (!cur.empty()) out.push_back("-D" + cur);
            cur.clear();
        } else if (text[i] != ' ') {
            cur.push_back(text[i]);
        }
    }
    return out;
}

bool nvrtc_compile(const std::string& source, const std::string& name,
                   std::vector<char>* cubin, std::string* log) {
    nvrtcProgram prog;
    nvrtcResult r = nvrtcCreateProgram(&prog, source.c_str(), name.c_str(), 0, nullptr, nullptr);
    if (r != NVRTC_SUCCESS) { *log = std::string("nvrtcCreateProgram: ") + nvrtcGetErrorString(r); return false; }
    const char* arch = std::getenv("DALI_B200_ARCH");
    std::string arch_opt = std::string("--gpu-architecture=") + (arch && *arch ? arch : "sm_100a");
    std::vector<std::string> defines = nvrtc_defines();
    std::vector<const char*> opts = {arch_opt.c_str(), "--std=c++17", "-lineinfo", "--extra-device-vectorization"};
    for (const std::string& d : defines) opts.push_back(d.c_str());
    r = nvrtcCompileProgram(prog, (int)opts.size(), opts.data());
    size_t log_size = 0;
    nvrtcGetProgramLogSize(prog, &log_size);
    if (log_size > 1) {
        log->resize(log_size);
        nvrtcGetProgramLog(prog, &(*log)[0]);
    }
    if (r != NVRTC_SUCCESS) {
        *log = std::string("nvrtcCompileProgram: ") + nvrtcGetErrorString(r) + "\n" + *log;
        nvrtcDestroyProgram(&prog);
        return false;
    }
    size_t size = 0;
    r = nvrtcGetCUBINSize(prog, &size);
    if (r != NVRTC_SUCCESS || size == 0) {
        *log += "\nnvrtcGetCUBINSize failed";
        nvrtcDestroyProgram(&prog);
        return false;
    }
    cubin->resize(size);
    nvrtcGetCUBIN(prog, cubin->data());
    nvrtcDestroyProgram(&prog);
    return true;
}

// ------------------------------------------------------------------ driver entry points
struct Driver {
    bool ready = false;
    CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                             unsigned, CUstream, void**, void**) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
};
static Driver g_drv;

template <typename F>
static bool load_entry(const char* name, F* out) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || fn == nullptr) return false;
    *out = reinterpret_cast<F>(fn);
    return true;
}

static std::string cu_err(CUresult r) {
    const char* s = nullptr;
    if (g_drv.GetErrorString) g_drv.GetErrorString(r, &s);
    return s ? s : ("CUresult " + std::to_string((int)r));
}

// ------------------------------------------------------------------ global state
struct Scratch {
    void* buf = nullptr;
    size_t bytes = 0;
    unsigned* counters = nullptr;
    size_t n_counters = 0;
};

struct DeviceState {
    int ordinal = 0;
    std::map<void*, Scratch> scratch;                    // per stream
    std::vector<void*> retired;                          // outgrown scratch, freed at pool_clear
    std::unordered_map<size_t, std::vector<void*>> pool; // rounded size -> free blocks
    std::unordered_map<std::string, CUfunction> functions;  // kernel key -> loaded function
    std::vector<CUmodule> modules;
};

struct KernelImage {
    std::vector<char> cubin;
};

struct State {
    std::mutex mu;
    std::vector<DeviceState> devices;
    std::unordered_map<uint64_t, Program> programs;
    std::unordered_map<std::string, KernelImage> images;   // kernel key -> cubin
    std::string cache_dir;
    bool recompile_checked = false;
    bool always_recompile = false;
    std::unordered_map<std::string, bool> recompiled_once;
    uint64_t n_compiles = 0, n_disk_hits = 0, n_launches = 0;
};
static State& S() {
    static State* s = new State();   // never destroyed: device memory outlives static teardown order
    return *s;
}

static std::string default_cache_dir() {
    const char* e = std::getenv("DALI_CACHE_DIR");
    if (e && *e) return e;
    const char* home = std::getenv("HOME");
    return std::string(home && *home ? home : "/tmp") + "/.dali_b200/cache";
}

static void make_dirs(const std::string& path) {
    std::string cur;
    for (size_t i = 0; i <= path.size(); ++i) {
        if (i == path.size() || path[i] == '/') {
            if (!cur.empty()) mkdir(cur.c_str(), 0755);
        }
        if (i < path.size()) cur += path[i];
    }
}

static const std::string& cache_dir_locked() {
    State& s = S();
    if (s.cache_dir.empty()) s.cache_dir = default_cache_dir();
    return s.cache_dir;
}

static bool always_recompile_locked() {
    State& s = S();
    if (!s.recompile_checked) {
        const char* e = std::getenv("DALI_JIT_ALWAYS_RECOMPILE");
        s.always_recompile = e && (std::string(e) == "true" || std::string(e) == "1");
        s.recompile_checked = true;
    }
    return s.always_recompile;
}

static std::string kernel_key(uint64_t hash, const Variant& v) {
    std::ostringstream k;
    // the device prelude is part of every kernel: its text is part of the key
    static const uint64_t prelude_hash = fnv1a(kPrelude);
    k << std::hex << hash << "_" << fnv1a(v.key() + "|sm_100a|" + kCodegenVersion + "|abi" +
                                            std::to_string(DALIB200_ABI_VERSION) + "|" + std::to_string(prelude_hash) + "|" + nvrtc_defines_text());
    return k.str();
}

// Returns the cubin for `key`: memory -> disk -> NVRTC (source from `make_source`).
static bool get_image(const std::string& key, const std::string& what, SourceFn make_source, void* ctx,
                      const KernelImage** out) {
    State& s = S();
    bool force = always_recompile_locked() && !s.recompiled_once[key];
    auto it = s.images.find(key);
    if (it != s.images.end() && !force) { *out = &it->second; return true; }
    const std::string dir = cache_dir_locked();
    const std::string base = dir + "/" + key;
    KernelImage img;
    if (!force) {
        std::ifstream f(base + ".cubin", std::ios::binary);
        if (f.good()) {
            img.cubin.assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
            if (img.cubin.size() > 64 && std::memcmp(img.cubin.data(), "\x7f" "ELF", 4) == 0) {
                ++s.n_disk_hits;
                s.images[key] = img;
                *out = &s.images[key];
                return true;
            }
            img.cubin.clear();   // truncated / corrupt file: fall through and rebuild it
        }
    }
    std::string src, err;
    if (!make_source(ctx, &src, &err)) { set_error("codegen: " + err); return false; }
    std::string log;
    make_dirs(dir);
    { std::ofstream f(base + ".cu"); f << src; }
    bool ok = nvrtc_compile(src, key + ".cu", &img.cubin, &log);
    { std::ofstream f(base + ".log"); f << log; }
    ++s.n_compiles;
    if (!ok) {
        set_error("NVRTC failed for kernel " + key + " (" + what + "), source " + base + ".cu:\n" + log);
        return false;
    }
    {
        const std::string tmp = base + ".cubin.tmp" + std::to_string((long)getpid());
        std::ofstream f(tmp, std::ios::binary);
        f.write(img.cubin.data(), (std::streamsize)img.cubin.size());
        f.close();
        std::rename(tmp.c_str(), (base + ".cubin").c_str());
    }
    s.recompiled_once[key] = true;
    s.images[key] = img;
    *out = &s.images[key];
    return true;
}

struct ExprSourceCtx { const Program* p; const Variant* v; };
static bool expr_source(void* ctx, std::string* src, std::string* err) {
    ExprSourceCtx* c = static_cast<ExprSourceCtx*>(ctx);
    std::string body;
    if (!generate_kernel(*c->p, *c->v, &body, err)) return false;
    *src = std::string(kPrelude) + "\n" + body;
    return true;
}

static int check_device(int device) {
    State& s = S();
    if (s.devices.empty()) { set_error("dalib200_init has not bound any CUDA device"); return DALIB200_ERR_NO_DEVICE; }
    if (device < 0 || device >= (int)s.devices.size()) { set_error("device index out of range"); return DALIB200_ERR_INVALID; }
    return DALIB200_OK;
}

#define CUDA_OK(call)                                                                       \
    do {                                                                                    \
        cudaError_t e_ = (call);                                                            \
        if (e_ != cudaSuccess) {                                                            \
            set_error(std::string(#call) + ": " + cudaGetErrorString(e_));                  \
            return DALIB200_ERR_CUDA;                                                       \
        }                                                                                   \
    } while (0)

static size_t round_size(size_t bytes) {
    if (bytes == 0) bytes = 1;
    return (bytes + 511) / 512 * 512;
}

static int pool_alloc_locked(int device, size_t bytes, void** out) {
    DeviceState& d = S().devices[device];
    size_t r = round_size(bytes);
    auto it = d.pool.find(r);
    if (it != d.pool.end() && !it->second.empty()) {
        *out = it->second.back();
        it->second.pop_back();
        return DALIB200_OK;
    }
    CUDA_OK(cudaSetDevice(d.ordinal));
    cudaError_t e = cudaMalloc(out, r);
    if (e != cudaSuccess) {
        // give pooled blocks back to the driver and retry once
        for (auto& kv : d.pool) { for (void* p : kv.second) cudaFree(p); kv.second.clear(); }
        e = cudaMalloc(out, r);
    }
    if (e != cudaSuccess) { set_error(std::string("cudaMalloc: ") + cudaGetErrorString(e)); return DALIB200_ERR_CUDA; }
    return DALIB200_OK;
}

static int get_scratch_locked(int device, void* stream, size_t bytes, size_t counters, Scratch* out) {
    DeviceState& d = S().devices[device];
    Scratch& sc = d.scratch[stream];
    CUDA_OK(cudaSetDevice(d.ordinal));
    if (sc.bytes < bytes) {
        size_t want = std::max<size_t>(bytes, 4u << 20);
        if (sc.buf) d.retired.push_back(sc.buf);   // may still be read by kernels in flight
        CUDA_OK(cudaMalloc(&sc.buf, want));
        sc.bytes = want;
    }
    if (sc.n_counters < counters) {
        size_t want = std::max<size_t>(counters, 4096);
        if (sc.counters) d.retired.push_back(sc.counters);
        CUDA_OK(cudaMalloc((void**)&sc.counters, want * sizeof(unsigned)));
        // tickets wrap back to zero by themselves (atomicInc), so this is the only clear
        CUDA_OK(cudaMemset(sc.counters, 0, want * sizeof(unsigned)));
        CUDA_OK(cudaDeviceSynchronize());
        sc.n_counters = want;
    }
    *out = sc;
    return DALIB200_OK;
}

int scratch_space(int device, void* stream, size_t bytes, void** out) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    int rc = check_device(device);
    if (rc != DALIB200_OK) return rc;
    Scratch sc;
    rc = get_scratch_locked(device, stream, bytes, 0, &sc);
    if (rc != DALIB200_OK) return rc;
    *out = sc.buf;
    return DALIB200_OK;
}

static int get_function_locked(int device, const std::string& key, const KernelImage& img, CUfunction* fn,
                               const char* entry = "dali_kernel") {
    DeviceState& d = S().devices[device];
    auto it = d.functions.find(key);
    if (it != d.functions.end()) { *fn = it->second; return DALIB200_OK; }
    CUDA_OK(cudaSetDevice(d.ordinal));
    CUmodule mod;
    CUresult r = g_drv.ModuleLoadData(&mod, img.cubin.data());
    if (r != CUDA_SUCCESS) { set_error("cuModuleLoadData(" + key + "): " + cu_err(r)); return DALIB200_ERR_CUDA; }
    r = g_drv.ModuleGetFunction(fn, mod, entry);
    if (r != CUDA_SUCCESS) { set_error("cuModuleGetFunction: " + cu_err(r)); return DALIB200_ERR_CUDA; }
    d.modules.push_back(mod);
    d.functions[key] = *fn;
    return DALIB200_OK;
}

static int do_launch(uint64_t hash, int device, void* stream, const int64_t* space, int rank,
                     void* const* array_data, const int64_t* offsets, const int64_t* const* strides,
                     int n_arrays, const void* const* scalars, int n_scalars, bool compile_only,
                     size_t* cubin_size) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    auto pit = s.programs.find(hash);
    if (pit == s.programs.end()) { set_error("unknown kernel hash"); return DALIB200_ERR_NOT_FOUND; }
    const Program& p = pit->second;
    LaunchPlan plan;
    std::string err;
    std::vector<const void*> fake_scalars;
    long long zero = 0;
    if (compile_only && !scalars) {
        fake_scalars.assign(p.scalars.size(), &zero);
        scalars = fake_scalars.data();
        n_scalars = (int)fake_scalars.size();
    }
    if (!plan_launch(p, space, rank, array_data, offsets, strides, n_arrays, scalars, n_scalars, &plan, &err)) {
        set_error(err);
        return DALIB200_ERR_INVALID;
    }
    if (plan.empty) { tl_variant = "empty"; return DALIB200_OK; }
    tl_variant = plan.describe();
    const std::string key = kernel_key(hash, plan.variant);
    const KernelImage* img = nullptr;
    ExprSourceCtx ctx{&p, &plan.variant};
    if (!get_image(key, plan.variant.key(), expr_source, &ctx, &img)) return DALIB200_ERR_COMPILE;
    if (cubin_size) *cubin_size = img->cubin.size();
    if (compile_only) return DALIB200_OK;

    int rc = check_device(device);
    if (rc != DALIB200_OK) return rc;
    CUfunction fn;
    rc = get_function_locked(device, key, *img, &fn);
    if (rc != DALIB200_OK) return rc;
    ParamLayout L(p, plan.variant);
    if (plan.scratch_bytes || plan.counters) {
        Scratch sc;
        rc = get_scratch_locked(device, stream, plan.scratch_bytes, plan.counters, &sc);
        if (rc != DALIB200_OK) return rc;
        plan.words[L.w_scratch] = (long long)(uintptr_t)sc.buf;
        plan.words[L.w_counter] = (long long)(uintptr_t)sc.counters;
    }
    if (plan.variant.xrank) {
        const void* table = comm_peer_table(device);
        if (!table) {
            set_error("this program combines a reduction across ranks inside the kernel: it needs a communicator whose ranks "
                      "can address one another's memory (dalib200_comm_init_rank, transport \"nccl+peer\" or \"single\")");
            return DALIB200_ERR_UNSUPPORTED;
        }
        plan.words[L.w_aux0] = (long long)(uintptr_t)table;
    }
    CUDA_OK(cudaSetDevice(s.devices[device].ordinal));
    void* params[] = {plan.words.data()};
    typedef CUresult (*LaunchExFn)(const CUlaunchConfig*, CUfunction, void**, void**);
    static LaunchExFn launch_ex = reinterpret_cast<LaunchExFn>(driver_entry("cuLaunchKernelEx"));
    CUresult r;
    if (plan.smem_bytes > 32 * 1024) {      // (the kernel's static shared memory counts towards the 48 KiB default limit too)
        static CUresult (*set_attr)(CUfunction, CUfunction_attribute, int) =
            reinterpret_cast<CUresult (*)(CUfunction, CUfunction_attribute, int)>(driver_entry("cuFuncSetAttribute"));
        if (!set_attr) { set_error("cuFuncSetAttribute unavailable"); return DALIB200_ERR_CUDA; }
        r = set_attr(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)plan.smem_bytes);
        if (r != CUDA_SUCCESS) { set_error("cuFuncSetAttribute(max dynamic smem): " + cu_err(r)); return DALIB200_ERR_CUDA; }
    }
    if (plan.cluster > 8) {
        static CUresult (*set_attr2)(CUfunction, CUfunction_attribute, int) =
            reinterpret_cast<CUresult (*)(CUfunction, CUfunction_attribute, int)>(driver_entry("cuFuncSetAttribute"));
        if (!set_attr2 || set_attr2(fn, CU_FUNC_ATTRIBUTE_NON_PORTABLE_CLUSTER_SIZE_ALLOWED, 1) != CUDA_SUCCESS) {
            set_error("clusters of more than 8 CTAs are not available on this device");
            return DALIB200_ERR_CUDA;
        }
    }
    if (plan.cluster > 1 && !launch_ex) { set_error("cuLaunchKernelEx unavailable: cannot launch a thread-block cluster"); return DALIB200_ERR_CUDA; }
    if (launch_ex && (dependent_launch_enabled() || plan.cluster > 1)) {
        // programmatic dependent launch: every generated kernel begins with griddepcontrol.wait (prelude: kernel_entry)
        CUlaunchAttribute attrs[2];
        std::memset(attrs, 0, sizeof attrs);
        unsigned n_attrs = 0;
        if (dependent_launch_enabled()) {
            attrs[n_attrs].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
            attrs[n_attrs].value.programmaticStreamSerializationAllowed = 1;
            ++n_attrs;
        }
        if (plan.cluster > 1) {
            attrs[n_attrs].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
            attrs[n_attrs].value.clusterDim.x = plan.cluster;
            attrs[n_attrs].value.clusterDim.y = 1;
            attrs[n_attrs].value.clusterDim.z = 1;
            ++n_attrs;
        }
        CUlaunchConfig cfg;
        std::memset(&cfg, 0, sizeof cfg);
        cfg.gridDimX = plan.grid_x; cfg.gridDimY = plan.grid_y; cfg.gridDimZ = 1;
        cfg.blockDimX = (unsigned)plan.variant.threads; cfg.blockDimY = 1; cfg.blockDimZ = 1;
        cfg.sharedMemBytes = plan.smem_bytes;
        cfg.hStream = (CUstream)stream;
        cfg.attrs = attrs;
        cfg.numAttrs = n_attrs;
        r = launch_ex(&cfg, fn, params, nullptr);
    } else {
        r = g_drv.LaunchKernel(fn, plan.grid_x, plan.grid_y, 1, (unsigned)plan.variant.threads, 1, 1, plan.smem_bytes, (CUstream)stream,
                               params, nullptr);
    }
    if (r != CUDA_SUCCESS) { set_error("cuLaunchKernel(" + tl_variant + "): " + cu_err(r)); return DALIB200_ERR_CUDA; }
    ++s.n_launches;
    return DALIB200_OK;
}

bool find_program(uint64_t hash, Program* out) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    auto it = s.programs.find(hash);
    if (it == s.programs.end()) return false;
    *out = it->second;
    return true;
}

const char* device_prelude() { return kPrelude; }

int acquire_kernel(int device, const std::string& key, const char* entry_name, SourceFn make_source, void* ctx,
                   void** function, size_t* cubin_size) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    const KernelImage* img = nullptr;
    if (!get_image(key, entry_name, make_source, ctx, &img)) return DALIB200_ERR_COMPILE;
    if (cubin_size) *cubin_size = img->cubin.size();
    if (device < 0) return DALIB200_OK;
    int rc = check_device(device);
    if (rc != DALIB200_OK) return rc;
    CUfunction fn;
    rc = get_function_locked(device, key, *img, &fn, entry_name);
    if (rc != DALIB200_OK) return rc;
    *function = (void*)fn;
    return DALIB200_OK;
}

void* driver_entry(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    return fn;
}

int device_ordinal(int device) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    if (device < 0 || device >= (int)s.devices.size()) return -1;
    return s.devices[device].ordinal;
}

void count_launch() {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    ++s.n_launches;
}

bool dependent_launch_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("DALI_B200_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

int launch_function(int device, void* function, unsigned gx, unsigned gy, unsigned threads, unsigned smem_bytes,
                    void* stream, void** params, bool dependent) {
    int ord = device_ordinal(device);
    if (ord < 0) { set_error("device index out of range"); return DALIB200_ERR_INVALID; }
    CUDA_OK(cudaSetDevice(ord));
    static CUresult (*set_attr)(CUfunction, CUfunction_attribute, int) = nullptr;
    if (!set_attr) set_attr = reinterpret_cast<CUresult (*)(CUfunction, CUfunction_attribute, int)>(driver_entry("cuFuncSetAttribute"));
    if (smem_bytes > 48 * 1024) {
        if (!set_attr) { set_error("cuFuncSetAttribute unavailable"); return DALIB200_ERR_CUDA; }
        CUresult r = set_attr((CUfunction)function, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)smem_bytes);
        if (r != CUDA_SUCCESS) { set_error("cuFuncSetAttribute(max dynamic smem): " + cu_err(r)); return DALIB200_ERR_CUDA; }
    }
    typedef CUresult (*LaunchExFn)(const CUlaunchConfig*, CUfunction, void**, void**);
    static LaunchExFn launch_ex = reinterpret_cast<LaunchExFn>(driver_entry("cuLaunchKernelEx"));
    CUresult r;
    if (dependent && launch_ex && dependent_launch_enabled()) {
        CUlaunchAttribute attr;
        std::memset(&attr, 0, sizeof attr);
        attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr.value.programmaticStreamSerializationAllowed = 1;
        CUlaunchConfig cfg;
        std::memset(&cfg, 0, sizeof cfg);
        cfg.gridDimX = gx; cfg.gridDimY = gy; cfg.gridDimZ = 1;
        cfg.blockDimX = threads; cfg.blockDimY = 1; cfg.blockDimZ = 1;
        cfg.sharedMemBytes = smem_bytes;
        cfg.hStream = (CUstream)stream;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        r = launch_ex(&cfg, (CUfunction)function, params, nullptr);
    } else {
        r = g_drv.LaunchKernel((CUfunction)function, gx, gy, 1, threads, 1, 1, smem_bytes, (CUstream)stream, params, nullptr);
    }
    if (r != CUDA_SUCCESS) { set_error("cuLaunchKernel: " + cu_err(r)); return DALIB200_ERR_CUDA; }
    count_launch();
    return DALIB200_OK;
}

int* gemm_error_word(int device) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    static int* words[64] = {nullptr};
    if (device < 0 || device >= (int)s.devices.size() || device >= 64) return nullptr;
    if (!words[device]) {
        cudaSetDevice(s.devices[device].ordinal);
        if (cudaMalloc((void**)&words[device], 256) != cudaSuccess) return nullptr;
        cudaMemset(words[device], 0, 256);
        cudaDeviceSynchronize();
    }
    return words[device];
}

}  // namespace dalib

namespace dalib {
cudaError_t gemm_simt(cudaStream_t stream, int dtype, int64_t m, int64_t n, int64_t k, const void* a, int64_t ars,
                      int64_t acs, const void* b, int64_t brs, int64_t bcs, void* c, int64_t crs, int64_t ccs,
                      double alpha, double beta);
static thread_local std::string tl_gemm_kernel;
void note_gemm_kernel(const std::string& name) { tl_gemm_kernel = name; }
}  // namespace dalib

using namespace dalib;

// =========================================================================== C ABI
extern "C" {

size_t dalib200_last_error(char* buffer, size_t capacity) {
    const std::string& e = get_error();
    if (buffer && capacity) {
        size_t n = e.size() < capacity - 1 ? e.size() : capacity - 1;
        std::memcpy(buffer, e.data(), n);
        buffer[n] = '\0';
    }
    return e.size();
}

int dalib200_abi_version(void) { return DALIB200_ABI_VERSION; }

int dalib200_init(int n_gpus) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        set_error(std::string("no CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0"));
        return DALIB200_ERR_NO_DEVICE;
    }
    int want = (n_gpus <= 0 || n_gpus > count) ? count : n_gpus;
    if (!g_drv.ready) {
        bool ok = load_entry("cuModuleLoadData", &g_drv.ModuleLoadData) &&
                  load_entry("cuModuleUnload", &g_drv.ModuleUnload) &&
                  load_entry("cuModuleGetFunction", &g_drv.ModuleGetFunction) &&
                  load_entry("cuLaunchKernel", &g_drv.LaunchKernel) &&
                  load_entry("cuGetErrorString", &g_drv.GetErrorString);
        if (!ok) { set_error("CUDA driver entry points unavailable"); return DALIB200_ERR_NO_DEVICE; }
        g_drv.ready = true;
    }
    int prev = 0;
    cudaGetDevice(&prev);
    for (int d = (int)s.devices.size(); d < want; ++d) {
        CUDA_OK(cudaSetDevice(d));
        CUDA_OK(cudaFree(0));   // creates / retains the primary context
        DeviceState ds;
        ds.ordinal = d;
        s.devices.push_back(std::move(ds));
    }
    cudaSetDevice(prev);
    return DALIB200_OK;
}

int dalib200_device_count(void) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    return (int)s.devices.size();
}

int dalib200_compile(uint64_t hash, const char* ir, size_t ir_len) {
    if (!ir) { set_error("null IR"); return DALIB200_ERR_INVALID; }
    std::string text(ir, ir_len);
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    auto it = s.programs.find(hash);
    if (it != s.programs.end()) {
        if (it->second.text == text) return DALIB200_OK;
        set_error("hash collision: a different program is registered under this hash");
        return DALIB200_ERR_INVALID;
    }
    Program p;
    std::string err;
    if (!parse_program(text, &p, &err)) { set_error(err); return DALIB200_ERR_INVALID; }
    s.programs[hash] = p;
    return DALIB200_OK;
}

int dalib200_is_loaded(uint64_t hash) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    return s.programs.count(hash) ? 1 : 0;
}

int dalib200_precompile(uint64_t hash, const int64_t* space, int space_rank, void* const* array_data,
                        const int64_t* offsets, const int64_t* const* strides, int n_arrays, size_t* cubin_size) {
    DeviceRestore restore_device;
    return do_launch(hash, 0, nullptr, space, space_rank, array_data, offsets, strides, n_arrays, nullptr, 0, true,
                     cubin_size);
}

int dalib200_cache_set_dir(const char* dir) {
    if (!dir || !*dir) { set_error("empty cache dir"); return DALIB200_ERR_INVALID; }
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    s.cache_dir = dir;
    while (s.cache_dir.size() > 1 && s.cache_dir.back() == '/') s.cache_dir.pop_back();
    return DALIB200_OK;
}

size_t dalib200_cache_get_dir(char* buffer, size_t capacity) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    const std::string& d = cache_dir_locked();
    if (buffer && capacity) {
        size_t n = d.size() < capacity - 1 ? d.size() : capacity - 1;
        std::memcpy(buffer, d.data(), n);
        buffer[n] = '\0';
    }
    return d.size();
}

int dalib200_cache_clear(int remove_files) {
    DeviceRestore restore_device;
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    if (remove_files) {
        const std::string dir = cache_dir_locked();
        for (auto& kv : s.images) {
            for (const char* ext : {".cubin", ".cu", ".log"}) std::remove((dir + "/" + kv.first + ext).c_str());
        }
    }
    for (DeviceState& d : s.devices) {
        cudaSetDevice(d.ordinal);
        cudaDeviceSynchronize();
        for (CUmodule m : d.modules) g_drv.ModuleUnload(m);
        d.modules.clear();
        d.functions.clear();
    }
    s.images.clear();
    return DALIB200_OK;
}

int dalib200_cache_stats(uint64_t stats[5]) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    stats[0] = s.programs.size();
    stats[1] = s.images.size();
    stats[2] = s.n_compiles;
    stats[3] = s.n_disk_hits;
    stats[4] = s.n_launches;
    return DALIB200_OK;
}

int dalib200_launch(uint64_t hash, int device, void* stream, const int64_t* space, int space_rank,
                    void* const* array_data, const int64_t* offsets, const int64_t* const* strides, int n_arrays,
                    const void* const* scalars, int n_scalars) {
    DeviceRestore restore_device;
    {
        State& s = S();
        std::lock_guard<std::mutex> g(s.mu);
        int rc = check_device(device);
        if (rc != DALIB200_OK) return rc;
    }
    return do_launch(hash, device, stream, space, space_rank, array_data, offsets, strides, n_arrays, scalars,
                     n_scalars, false, nullptr);
}

int dalib200_launch_host(uint64_t hash, int device, const int64_t* space, int space_rank, void* const* host_data,
                         const int64_t* extents, const int64_t* offsets, const int64_t* const* strides, int n_arrays,
                         const void* const* scalars, int n_scalars) {
    DeviceRestore restore_device;
    State& s = S();
    std::vector<DType> dts;
    std::vector<bool> rd, wr, iota;
    {
        std::lock_guard<std::mutex> g(s.mu);
        int rc = check_device(device);
        if (rc != DALIB200_OK) return rc;
        auto pit = s.programs.find(hash);
        if (pit == s.programs.end()) { set_error("unknown kernel hash"); return DALIB200_ERR_NOT_FOUND; }
        if (n_arrays != (int)pit->second.args.size()) { set_error("launch: wrong number of arrays"); return DALIB200_ERR_INVALID; }
        for (const ArgDecl& a : pit->second.args) {
            dts.push_back(a.dtype); rd.push_back(a.read); wr.push_back(a.written); iota.push_back(a.iota);
        }
    }
    std::vector<void*> dev(n_arrays, nullptr);
    int rc = DALIB200_OK;
    for (int a = 0; a < n_arrays && rc == DALIB200_OK; ++a) {
        if (iota[a]) continue;      // nothing behind it
        size_t bytes = (size_t)extents[a] * dtype_size(dts[a]);
        rc = dalib200_alloc(device, bytes, &dev[a]);
        // partially written views keep their untouched elements: upload written args too
        if (rc == DALIB200_OK) rc = dalib200_memcpy_h2d(device, dev[a], host_data[a], bytes, nullptr);
    }
    if (rc == DALIB200_OK)
        rc = dalib200_launch(hash, device, nullptr, space, space_rank, dev.data(), offsets, strides, n_arrays, scalars,
                             n_scalars);
    for (int a = 0; a < n_arrays && rc == DALIB200_OK; ++a)
        if (wr[a]) rc = dalib200_memcpy_d2h(device, host_data[a], dev[a], (size_t)extents[a] * dtype_size(dts[a]), nullptr);
    if (rc == DALIB200_OK) rc = dalib200_sync(device, nullptr);
    for (int a = 0; a < n_arrays; ++a)
        if (dev[a]) dalib200_free(device, dev[a], (size_t)extents[a] * dtype_size(dts[a]));
    (void)rd;
    return rc;
}

size_t dalib200_last_variant(char* buffer, size_t capacity) {
    if (buffer && capacity) {
        size_t n = tl_variant.size() < capacity - 1 ? tl_variant.size() : capacity - 1;
        std::memcpy(buffer, tl_variant.data(), n);
        buffer[n] = '\0';
    }
    return tl_variant.size();
}

int dalib200_gemm(int device, void* stream, int dtype, int64_t m, int64_t n, int64_t k, const void* a, int64_t ars,
                  int64_t acs, const void* b, int64_t brs, int64_t bcs, void* c, int64_t crs, int64_t ccs, double alpha,
                  double beta) {
    DeviceRestore restore_device;
    {
        State& s = S();
        std::lock_guard<std::mutex> g(s.mu);
        int rc = check_device(device);
        if (rc != DALIB200_OK) return rc;
        CUDA_OK(cudaSetDevice(s.devices[device].ordinal));
    }
    if (dtype != DALIB200_F32 && dtype != DALIB200_F64 && dtype != DALIB200_I32) {
        set_error("dalib200_gemm: dtype must be f32, f64 or i32");
        return DALIB200_ERR_INVALID;
    }
    if (m < 0 || n < 0 || k < 0 || !a || !b || !c) { set_error("dalib200_gemm: bad argument"); return DALIB200_ERR_INVALID; }
    if (m == 0 || n == 0) return DALIB200_OK;
    tl_gemm_kernel = "simt";
    CUDA_OK(gemm_simt((cudaStream_t)stream, dtype, m, n, k, a, ars, acs, b, brs, bcs, c, crs, ccs, alpha, beta));
    return DALIB200_OK;
}

size_t dalib200_last_gemm_kernel(char* buffer, size_t capacity) {
    if (buffer && capacity) {
        size_t n = tl_gemm_kernel.size() < capacity - 1 ? tl_gemm_kernel.size() : capacity - 1;
        std::memcpy(buffer, tl_gemm_kernel.data(), n);
        buffer[n] = '\0';
    }
    return tl_gemm_kernel.size();
}

int dalib200_alloc(int device, size_t bytes, void** out) {
    DeviceRestore restore_device;
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    int rc = check_device(device);
    if (rc != DALIB200_OK) return rc;
    if (!out) { set_error("null out pointer"); return DALIB200_ERR_INVALID; }
    return pool_alloc_locked(device, bytes, out);
}

int dalib200_free(int device, void* ptr, size_t bytes) {
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    int rc = check_device(device);
    if (rc != DALIB200_OK) return rc;
    if (!ptr) return DALIB200_OK;
    s.devices[device].pool[round_size(bytes)].push_back(ptr);
    return DALIB200_OK;
}

int dalib200_host_alloc(size_t bytes, void** out) {
    if (!out) { set_error("null out pointer"); return DALIB200_ERR_INVALID; }
    if (dalib200_device_count() <= 0) { set_error("page-locked memory needs a bound CUDA device"); return DALIB200_ERR_NO_DEVICE; }
    void* p = nullptr;
    CUDA_OK(cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocPortable));
    *out = p;
    return DALIB200_OK;
}

int dalib200_host_free(void* ptr) {
    if (!ptr) return DALIB200_OK;
    CUDA_OK(cudaFreeHost(ptr));
    return DALIB200_OK;
}

int dalib200_pool_clear(int device) {
    DeviceRestore restore_device;
    State& s = S();
    std::lock_guard<std::mutex> g(s.mu);
    int rc = check_device(device);
    if (rc != DALIB200_OK) return rc;
    DeviceState& d = s.devices[device];
    CUDA_OK(cudaSetDevice(d.ordinal));
    CUDA_OK(cudaDeviceSynchronize());
    for (auto& kv : d.pool) { for (void* p : kv.second) cudaFree(p); kv.second.clear(); }
    for (void* p : d.retired) cudaFree(p);
    d.retired.clear();
    return DALIB200_OK;
}

static int copy_common(int device, void* dst, const void* src, size_t bytes, void* stream, cudaMemcpyKind kind) {
    DeviceRestore restore_device;
    {
        State& s = S();
        std::lock_guard<std::mutex> g(s.mu);
        int rc = check_device(device);
        if (rc != DALIB200_OK) return rc;
        CUDA_OK(cudaSetDevice(s.devices[device].ordinal));
    }
    if (bytes == 0) return DALIB200_OK;
    CUDA_OK(cudaMemcpyAsync(dst, src, bytes, kind, (cudaStream_t)stream));
    return DALIB200_OK;
}

int dalib200_memcpy_h2d(int device, void* dst, const void* src, size_t bytes, void* stream) {
    return copy_common(device, dst, src, bytes, stream, cudaMemcpyHostToDevice);
}
int dalib200_memcpy_d2h(int device, void* dst, const void* src, size_t bytes, void* stream) {
    return copy_common(device, dst, src, bytes, stream, cudaMemcpyDeviceToHost);
}
int dalib200_memcpy_d2d(int device, void* dst, const void* src, size_t bytes, void* stream) {
    return copy_common(device, dst, src, bytes, stream, cudaMemcpyDeviceToDevice);
}

int dalib200_memset(int device, void* dst, int byte, size_t bytes, void* stream) {
    DeviceRestore restore_device;
    {
        State& s = S();
        std::lock_guard<std::mutex> g(s.mu);
        int rc = check_device(device);
        if (rc != DALIB200_OK) return rc;
        CUDA_OK(cudaSetDevice(s.devices[device].ordinal));
    }
    if (bytes == 0) return DALIB200_OK;
    CUDA_OK(cudaMemsetAsync(dst, byte, bytes, (cudaStream_t)stream));
    return DALIB200_OK;
}

int dalib200_sync(int device, void* stream) {
    DeviceRestore restore_device;
    {
        State& s = S();
        std::lock_guard<std::mutex> g(s.mu);
        int rc = check_device(device);
        if (rc != DALIB200_OK) return rc;
        CUDA_OK(cudaSetDevice(s.devices[device].ordinal));
    }
    if (stream == (void*)-1) CUDA_OK(cudaDeviceSynchronize());
    else CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
    return DALIB200_OK;
}

}  // extern "C"
