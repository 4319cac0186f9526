// extern "C" binding of the Array / op:: front end (include/dali_b200_array.h).
#include <cstdlib>
#include <cstring>
#include <functional>
#include <map>
#include <memory>

#include "../../../include/dali_b200.h"
#include "../../../include/dali_b200_array.h"
#include "../runtime.h"
#include "dali/array/op.h"
#include "dali/array/expression/expression.h"
#include "dali/utils/random.h"
#include "dali/utils/scope.h"

struct dali_array_s { Array a; };

namespace {

int guard(const std::function<void()>& f) {
    try {
        f();
        return DALIB200_OK;
    } catch (const std::exception& e) {
        dalib::set_error(e.what());
        return DALIB200_ERR_INVALID;
    }
}

std::vector<int> to_shape(const int64_t* shape, int ndim) {
    std::vector<int> s(ndim);
    for (int d = 0; d < ndim; ++d) s[d] = (int)shape[d];
    return s;
}

DType to_dtype(int dtype) {
    DALI_ASSERT(dtype >= 0 && dtype <= 3, "dtype must be 0 (float), 1 (double), 2 (int32) or 3 (bf16, a storage type)");
    return (DType)dtype;
}

size_t copy_out(const std::string& s, char* buffer, size_t capacity) {
    if (buffer && capacity) {
        size_t n = s.size() < capacity - 1 ? s.size() : capacity - 1;
        std::memcpy(buffer, s.data(), n);
        buffer[n] = '\0';
    }
    return s.size();
}

dali_array_t wrap(const Array& a) {
    dali_array_s* h = new dali_array_s();
    h->a = a;
    return h;
}

}  // namespace

extern "C" {

int dali_array_from_host(const void* data, const int64_t* shape, int ndim, int dtype, dali_array_t* out) {
    return guard([&]() {
        DType dt = to_dtype(dtype);
        std::vector<int> s = to_shape(shape, ndim);
        int64_t n = 1;
        for (int d : s) n *= d;
        size_t bytes = (size_t)n * size_of_dtype(dt);
        void* buf = std::malloc(bytes ? bytes : 1);
        DALI_ASSERT(buf, "out of host memory");
        std::memcpy(buf, data, bytes);
        *out = wrap(Array::adopt_buffer(buf, s, dt, memory::Device::cpu()));
    });
}

int dali_array_borrow_host(void* data, const int64_t* shape, int ndim, int dtype, dali_array_t* out) {
    return guard([&]() { *out = wrap(Array::borrow_host(data, to_shape(shape, ndim), to_dtype(dtype))); });
}

int dali_array_eval_together(const dali_array_t* arrays, int n, int wait) {
    return guard([&]() {
        std::vector<Array> v;
        for (int i = 0; i < n; ++i) v.push_back(arrays[i]->a);
        Array::eval_together(v, wait != 0);
    });
}

int dali_array_load(const char* path, dali_array_t* out) {
    return guard([&]() { *out = wrap(Array::load(std::string(path))); });
}
int dali_array_save(const char* path, dali_array_t a) {
    return guard([&]() { Array::save(std::string(path), a->a); });
}

int dali_array_from_device(void* device_ptr, const int64_t* shape, int ndim, int dtype, int gpu, dali_array_t* out) {
    return guard([&]() {
        DType dt = to_dtype(dtype);
        std::vector<int> s = to_shape(shape, ndim);
        int64_t n = 1;
        for (int d : s) n *= d;
        auto mem = std::make_shared<memory::SynchronizedMemory>((size_t)n * size_of_dtype(dt), s.empty() ? 1 : s.back(),
                                                                memory::Device::gpu(gpu));
        mem->borrow_buffer(memory::Device::gpu(gpu), device_ptr);
        *out = wrap(Array(s, mem, 0, std::vector<int>(), dt));
    });
}

int dali_array_empty(const int64_t* shape, int ndim, int dtype, dali_array_t* out) {
    return guard([&]() { *out = wrap(Array(to_shape(shape, ndim), to_dtype(dtype))); });
}
int dali_array_zeros(const int64_t* shape, int ndim, int dtype, dali_array_t* out) {
    return guard([&]() { *out = wrap(Array::zeros(to_shape(shape, ndim), to_dtype(dtype))); });
}
int dali_array_scalar(double value, int dtype, dali_array_t* out) {
    return guard([&]() { *out = wrap(Array(value, to_dtype(dtype))); });
}
int dali_array_arange(int start, int stop, int step, dali_array_t* out) {
    return guard([&]() { *out = wrap(op::arange(start, stop, step)); });
}
int dali_array_free(dali_array_t a) {
    delete a;
    return DALIB200_OK;
}

int dali_array_ndim(dali_array_t a) { return a->a.ndim(); }
int dali_array_dtype(dali_array_t a) { return a->a.is_stateless() ? -1 : (int)a->a.dtype(); }
int dali_array_shape(dali_array_t a, int64_t* shape_out) {
    return guard([&]() { for (int d = 0; d < a->a.ndim(); ++d) shape_out[d] = a->a.shape()[d]; });
}
int dali_array_is_buffer(dali_array_t a) { return a->a.is_buffer() ? 1 : 0; }
size_t dali_array_expression_name(dali_array_t a, char* buffer, size_t capacity) {
    return copy_out(a->a.full_expression_name(), buffer, capacity);
}

int dali_array_eval(dali_array_t a, int wait) {
    return guard([&]() { a->a.eval(wait != 0); });
}

int dali_array_to_host(dali_array_t a, void* out, size_t capacity) {
    return guard([&]() {
        size_t bytes = (size_t)a->a.numel() * size_of_dtype(a->a.dtype());
        DALI_ASSERT(capacity >= bytes, "dali_array_to_host: output buffer too small");
        a->a.to_host(out);
    });
}

int dali_array_item(dali_array_t a, double* out) {
    return guard([&]() { *out = (double)a->a; });
}

int dali_array_device_ptr(dali_array_t a, int gpu, void** out) {
    return guard([&]() {
        a->a.eval();
        DALI_ASSERT(a->a.contiguous_memory(), "dali_array_device_ptr needs a contiguous Array");
        BufferView* b = as<BufferView>(a->a);
        *out = (char*)const_cast<void*>(b->memory_->readonly_data(memory::Device::gpu(gpu))) + b->offset_ * size_of_dtype(b->dtype_);
    });
}

int dali_array_index(dali_array_t a, int axis, int idx, dali_array_t* out) {
    return guard([&]() { *out = wrap(a->a.pluck_axis(axis, idx)); });
}
int dali_array_slice(dali_array_t a, int axis, int start, int stop, int step, dali_array_t* out) {
    return guard([&]() { *out = wrap(a->a.pluck_axis(axis, Slice(start, stop, step))); });
}
int dali_array_expand_dims(dali_array_t a, int axis, dali_array_t* out) {
    return guard([&]() { *out = wrap(a->a.expand_dims(axis)); });
}
int dali_array_squeeze(dali_array_t a, int axis, dali_array_t* out) {
    return guard([&]() { *out = wrap(a->a.squeeze(axis)); });
}
int dali_array_transpose(dali_array_t a, const int* axes, int n_axes, dali_array_t* out) {
    return guard([&]() {
        *out = wrap(n_axes == 0 ? a->a.transpose() : a->a.transpose(std::vector<int>(axes, axes + n_axes)));
    });
}
int dali_array_broadcast_to(dali_array_t a, const int64_t* shape, int ndim, dali_array_t* out) {
    return guard([&]() { *out = wrap(a->a.broadcast_to_shape(to_shape(shape, ndim))); });
}
int dali_array_reshape(dali_array_t a, const int64_t* shape, int ndim, dali_array_t* out) {
    return guard([&]() { *out = wrap(a->a.reshape(to_shape(shape, ndim))); });
}
int dali_array_astype(dali_array_t a, int dtype, dali_array_t* out) {
    return guard([&]() { *out = wrap(a->a.astype(to_dtype(dtype))); });
}

int dali_op_unary(const char* name, dali_array_t a, dali_array_t* out) {
    return guard([&]() {
        static const std::map<std::string, Array (*)(Array)> table = {
            {"identity", op::identity}, {"sqrt", op::sqrt}, {"square", op::square}, {"abs", op::abs},
            {"sigmoid", op::sigmoid}, {"dsigmoid", op::dsigmoid}, {"tanh", op::tanh}, {"dtanh", op::dtanh},
            {"relu", op::relu}, {"relu_backward", op::relu_backward}, {"eltinv", op::eltinv}, {"exp", op::exp},
            {"log", op::log}, {"log_or_zero", op::log_or_zero}, {"sign", op::sign}, {"softplus", op::softplus},
            {"softplus_backward", op::softplus_backward}, {"cube", op::cube}, {"rsqrt", op::rsqrt},
            {"isnan", op::isnan}, {"isinf", op::isinf}, {"inverse_tanh", op::inverse_tanh},
            {"round", op::round}, {"ceil", op::ceil}};
        if (std::string(name) == "negate") { *out = wrap(-a->a); return; }
        auto it = table.find(name);
        DALI_ASSERT(it != table.end(), std::string("unknown unary op '") + name + "'");
        *out = wrap(it->second(a->a));
    });
}

int dali_op_binary(const char* name, dali_array_t a, dali_array_t b, dali_array_t* out) {
    return guard([&]() {
        static const std::map<std::string, Array (*)(Array, Array)> table = {
            {"add", op::add}, {"subtract", op::subtract}, {"eltmul", op::eltmul}, {"eltdiv", op::eltdiv},
            {"equals", op::equals}, {"pow", op::pow}, {"steep_sigmoid", op::steep_sigmoid},
            {"steep_sigmoid_backward", op::steep_sigmoid_backward}, {"clipped_relu", op::clipped_relu},
            {"clipped_relu_backward", op::clipped_relu_backward}, {"prelu", op::prelu},
            {"prelu_backward_weights", op::prelu_backward_weights}, {"prelu_backward_inputs", op::prelu_backward_inputs},
            {"lessthanequal", op::lessthanequal}, {"greaterthanequal", op::greaterthanequal},
            {"maximum", op::maximum}, {"minimum", op::minimum}, {"clip", op::clip},
            {"binary_cross_entropy", op::binary_cross_entropy},
            {"binary_cross_entropy_grad", op::binary_cross_entropy_grad}, {"all_equals", op::all_equals}};
        auto it = table.find(name);
        DALI_ASSERT(it != table.end(), std::string("unknown binary op '") + name + "'");
        *out = wrap(it->second(a->a, b->a));
    });
}

int dali_op_reduce(const char* name, dali_array_t a, const int* axes, int n_axes, int keepdims, dali_array_t* out) {
    return guard([&]() {
        std::string n(name);
        const Array& x = a->a;
        bool all = n_axes < 0;
        std::vector<int> ax;
        if (!all) ax.assign(axes, axes + n_axes);
        Array r;
        if (n == "sum") r = all ? op::sum(x) : op::sum(x, ax, keepdims != 0);
        else if (n == "prod") r = all ? op::prod(x) : op::prod(x, ax, keepdims != 0);
        else if (n == "max") r = all ? op::max(x) : op::max(x, ax, keepdims != 0);
        else if (n == "min") r = all ? op::min(x) : op::min(x, ax, keepdims != 0);
        else if (n == "mean") r = all ? op::mean(x) : op::mean(x, ax, keepdims != 0);
        else if (n == "L2_norm") r = all ? op::L2_norm(x) : op::L2_norm(x, ax, keepdims != 0);
        else throw std::runtime_error("unknown reducer '" + n + "'");
        *out = wrap(r);
    });
}

int dali_op_argreduce(const char* name, dali_array_t a, int axis, int all_axes, dali_array_t* out) {
    return guard([&]() {
        std::string n(name);
        DALI_ASSERT(n == "argmax" || n == "argmin", "unknown arg-reducer '" + n + "'");
        if (n == "argmax") *out = wrap(all_axes ? op::argmax(a->a) : op::argmax(a->a, axis));
        else *out = wrap(all_axes ? op::argmin(a->a) : op::argmin(a->a, axis));
    });
}

int dali_op_gather(dali_array_t source, dali_array_t indices, dali_array_t* out) {
    return guard([&]() { *out = wrap(op::gather(source->a, indices->a)); });
}
int dali_op_gather_from_rows(dali_array_t source, dali_array_t indices, dali_array_t* out) {
    return guard([&]() { *out = wrap(op::gather_from_rows(source->a, indices->a)); });
}
int dali_op_diag(dali_array_t diag, int rows, int cols, dali_array_t* out) {
    return guard([&]() { *out = wrap(op::diag(diag->a, rows, cols)); });
}
int dali_op_one_hot(dali_array_t indices, int depth, dali_array_t on_value, dali_array_t off_value, dali_array_t* out) {
    return guard([&]() { *out = wrap(op::one_hot(indices->a, depth, on_value->a, off_value->a)); });
}
int dali_op_outer(dali_array_t a, dali_array_t b, dali_array_t* out) {
    return guard([&]() { *out = wrap(op::outer(a->a, b->a)); });
}
int dali_op_concatenate(const dali_array_t* arrays, int n, int axis, dali_array_t* out) {
    return guard([&]() {
        std::vector<Array> v;
        for (int i = 0; i < n; ++i) v.push_back(arrays[i]->a);
        *out = wrap(op::concatenate(v, axis));
    });
}
int dali_op_scan(dali_array_t a, const char* reducer, int inclusive, dali_array_t* out) {
    return guard([&]() { *out = wrap(op::axis_scan(a->a, reducer, inclusive != 0)); });
}
int dali_op_arange(dali_array_t start, dali_array_t stop, dali_array_t step, dali_array_t* out) {
    return guard([&]() { *out = wrap(op::arange(start->a, stop->a, step->a)); });
}
int dali_op_random(const char* kind, dali_array_t a, dali_array_t b, const int64_t* shape, int ndim, dali_array_t* out) {
    return guard([&]() {
        const std::string k(kind);
        std::vector<int> s = to_shape(shape, ndim);
        if (k == "uniform") *out = wrap(op::uniform(a->a, b->a, s));
        else if (k == "normal") *out = wrap(op::normal(a->a, b->a, s));
        else if (k == "bernoulli") *out = wrap(op::bernoulli(a->a, s));
        else if (k == "bernoulli_normalized") *out = wrap(op::bernoulli_normalized(a->a, s));
        else throw std::runtime_error("dali_op_random: unknown kind " + k);
    });
}
int dali_random_set_seed(int seed) {
    return guard([&]() { utils::random::set_seed(seed); });
}
int dali_op_softmax(dali_array_t logits, int axis, dali_array_t* out) {
    return guard([&]() { *out = wrap(op::softmax(logits->a, axis)); });
}
int dali_op_dot(dali_array_t a, dali_array_t b, dali_array_t* out) {
    return guard([&]() { *out = wrap(op::dot(a->a, b->a)); });
}

int dali_array_assign(dali_array_t dest, int op_code, dali_array_t value) {
    return guard([&]() {
        switch (op_code) {
            case 0: dest->a.assign(value->a); break;
            case 1: dest->a += Array(value->a); break;      // (a handle says nothing about being named: fused like a temporary)
            case 2: dest->a -= Array(value->a); break;
            case 3: dest->a *= Array(value->a); break;
            case 4: dest->a /= Array(value->a); break;
            case 5: dest->a <<= Array(value->a); break;
            default: throw std::runtime_error("unknown assignment operator code");
        }
    });
}

int dali_set_default_device(int gpu) {
    return guard([&]() {
        DALI_ASSERT(gpu >= 0, "dali_set_default_device: gpu index must be non-negative");
        memory::default_preferred_device = memory::Device::gpu(gpu);
    });
}

int dali_lazy_set_dry_run(int on) {
    lazy::set_dry_run(on != 0);
    return DALIB200_OK;
}

int dali_lazy_stats(int64_t counts[3]) {
    counts[0] = lazy::stats().kernels;
    counts[1] = lazy::stats().gemms;
    counts[2] = lazy::stats().temporaries;
    return DALIB200_OK;
}
int dali_array_set_shard(dali_array_t a, int axis, int64_t lo, int64_t total) {
    return guard([&]() { a->a.set_shard(axis, lo, total); });
}
int dali_array_get_shard(dali_array_t a, int* axis, int64_t* lo, int64_t* total) {
    return guard([&]() {
        const Shard s = a->a.shard();
        *axis = s.axis; *lo = s.lo; *total = s.total;
    });
}
int dali_array_scatter_rows(const void* data, const int64_t* global_shape, int ndim, int dtype, dali_array_t* out) {
    return guard([&]() { *out = wrap(Array::scatter_rows(data, to_shape(global_shape, ndim), to_dtype(dtype))); });
}
size_t dali_lazy_collectives(int64_t* count, char* buffer, size_t capacity) {
    if (count) *count = lazy::stats().collectives;
    return copy_out(lazy::stats().last_collective, buffer, capacity);
}
// names of the trace scopes left since dali_scope_trace_start, one per line
static std::unique_ptr<ScopeObserver> g_trace_observer;
static std::string g_trace;
int dali_scope_trace_start(void) {
    g_trace.clear();
    g_trace_observer.reset(new ScopeObserver(nullptr, [](const ScopeObserver::State& state) {
        if (!state.trace.empty()) g_trace += *state.trace.back() + "\n";
    }));
    return DALIB200_OK;
}
size_t dali_scope_trace_stop(char* buffer, size_t capacity) {
    g_trace_observer.reset();
    return copy_out(g_trace, buffer, capacity);
}
size_t dali_lazy_last_ir(char* buffer, size_t capacity) { return copy_out(lazy::stats().last_ir, buffer, capacity); }
size_t dali_lazy_last_variant(char* buffer, size_t capacity) { return copy_out(lazy::stats().last_variant, buffer, capacity); }

}  // extern "C"
