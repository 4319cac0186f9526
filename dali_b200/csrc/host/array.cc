// class Array: handle to a lazily evaluated expression (reference:
// dali/array/array.cpp).  View algebra on evaluated buffers follows
// dali/array/expression/buffer.cpp:113-286; on lazy nodes it composes View
// index maps instead of inserting reshape nodes.
#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <unordered_set>

#include "../../../include/dali_b200.h"
#include "dali/array/op.h"
#include "dali/array/expression/computation.h"
#include "dali/array/expression/expression.h"
#include "dali/array/expression/optimization.h"

// ------------------------------------------------------------------ dtype helpers
int size_of_dtype(DType dtype) { return dtype == DTYPE_DOUBLE ? 8 : (dtype == DTYPE_BF16 ? 2 : 4); }
static float bf16_bits_to_float(unsigned short bits) {
    unsigned u = (unsigned)bits << 16;
    float f;
    std::memcpy(&f, &u, sizeof f);
    return f;
}
std::string dtype_to_name(DType dtype) {
    switch (dtype) {
        case DTYPE_FLOAT: return "float";
        case DTYPE_DOUBLE: return "double";
        case DTYPE_INT32: return "int32";
        case DTYPE_BF16: return "bfloat16";
    }
    return "unknown";
}
std::ostream& operator<<(std::ostream& os, const DType& d) { return os << dtype_to_name(d); }
template <> DType template_to_dtype<float>() { return DTYPE_FLOAT; }
template <> DType template_to_dtype<double>() { return DTYPE_DOUBLE; }
template <> DType template_to_dtype<int>() { return DTYPE_INT32; }

static std::string shape_str(const std::vector<int>& s) {
    std::ostringstream o;
    o << "[";
    for (size_t i = 0; i < s.size(); ++i) o << (i ? ", " : "") << s[i];
    o << "]";
    return o.str();
}

// ------------------------------------------------------------------ Slice
Slice Slice::normalize_and_check(const Slice& s, int dim) {
    DALI_ASSERT(s.step != 0, "slice step cannot be zero");
    Slice r;
    r.step = s.step;
    r.has_start = r.has_end = true;
    if (s.step > 0) {
        r.start = s.has_start ? s.start : 0;
        r.end = s.has_end ? s.end : dim;
    } else {
        // a negative step walks [start, end) backwards, as the reference's Slice does
        r.start = s.has_start ? s.start : 0;
        r.end = s.has_end ? s.end : dim;
    }
    if (r.start < 0) r.start += dim;
    if (r.end < 0) r.end += dim;
    DALI_ASSERT(r.start >= 0 && r.start <= dim && r.end >= 0 && r.end <= dim && r.start <= r.end,
                "slice [" + std::to_string(s.start) + ":" + std::to_string(s.end) + "] out of range for dimension of size " +
                    std::to_string(dim));
    return r;
}
Slice::Slice(int start_, int end_, int step_) : has_start(true), has_end(true), start(start_), end(end_), step(step_) {
    if ((start >= 0 && end >= 0) || (start < 0 && end < 0))
        DALI_ASSERT(start < end, "Slice start (" + std::to_string(start) + ") must be less than end (" + std::to_string(end) + ")");
    DALI_ASSERT(step != 0, "slice step cannot be zero");
}

bool Slice::contains(int index) const {
    DALI_ASSERT(has_end, "can only compute size of slice if end index is specified.");
    DALI_ASSERT(start >= 0 && end >= 0, "slice length can only be use with positive indexing.");
    const bool in_range = start <= index && index < end;
    const bool good_jump = step > 0 ? (index - start) % step == 0 : (end - 1 - index) % (-step) == 0;
    return in_range && good_jump;
}

int Slice::size() const {
    DALI_ASSERT(has_end, "can only compute size of slice if end index is specified.");
    int span = end - start;
    int st = step > 0 ? step : -step;
    return (span + st - 1) / st;
}

// ------------------------------------------------------------------ Expression helpers
std::string Expression::full_name() const {
    std::string s = name();
    if (!arguments_.empty()) {
        s += "(";
        for (size_t i = 0; i < arguments_.size(); ++i) s += (i ? ", " : "") + arguments_[i].full_expression_name();
        s += ")";
    }
    return s;
}

BufferView::BufferView(std::shared_ptr<memory::SynchronizedMemory> memory, const std::vector<int>& shape, DType dtype,
                       int64_t offset, const std::vector<int>& strides)
    : Expression(N_BUFFER, shape, dtype, {}), memory_(memory), offset_(offset), strides_(strides) {
    DALI_ASSERT(strides.empty() || strides.size() == shape.size(), "strides must be empty or match the shape's rank");
    for (int s : shape) DALI_ASSERT(s >= 0, "negative dimension in shape " + shape_str(shape));
    if (contiguous()) strides_.clear();
}

std::shared_ptr<BufferView> BufferView::create(const std::vector<int>& shape, DType dtype, memory::Device device) {
    int64_t n = 1;
    for (int s : shape) {
        DALI_ASSERT(s >= 0, "negative dimension in shape " + shape_str(shape));
        n *= s;
    }
    auto mem = std::make_shared<memory::SynchronizedMemory>((size_t)n * size_of_dtype(dtype),
                                                            shape.empty() ? 1 : shape.back(), device);
    return std::make_shared<BufferView>(mem, shape, dtype, 0, std::vector<int>());
}

std::vector<int> BufferView::normalized_strides() const {
    if (!strides_.empty()) return strides_;
    std::vector<int> st(shape_.size());
    int64_t s = 1;
    for (int d = (int)shape_.size() - 1; d >= 0; --d) { st[d] = (int)s; s *= shape_[d]; }
    return st;
}

bool BufferView::contiguous() const {
    if (strides_.empty()) return true;
    int64_t s = 1;
    for (int d = (int)shape_.size() - 1; d >= 0; --d) {
        if (shape_[d] != 1 && strides_[d] != s) return false;
        s *= shape_[d];
    }
    return true;
}


static std::vector<int> scan_shape(const Array& a, bool inclusive) {
    std::vector<int> s = a.shape();
    if (!inclusive) s.back() += 1;
    return s;
}
Scan::Scan(const Array& a, const std::string& reducer, bool inclusive)
    : Expression(N_SCAN, scan_shape(a, inclusive), a.dtype(), {a}), reducer_(reducer), inclusive_(inclusive) {
    DALI_ASSERT(shard_.axis != ndim() - 1, "a running reduction along the sharded axis is not supported (each rank holds only its part of every row)");
}

bool Iota::linear(int64_t* step) const {
    // walk from the innermost dim: stride[k] must equal step * (product of the extents after k)
    int64_t s = 0, expect = 0;
    bool have = false;
    for (int k = ndim() - 1; k >= 0; --k) {
        if (shape_[k] == 1) continue;
        if (!have) { s = strides_[k]; expect = s * shape_[k]; have = true; continue; }
        if (strides_[k] != expect) return false;
        expect *= shape_[k];
    }
    *step = have ? s : 0;
    return true;
}

static std::vector<int> gather_shape(const Array& source, const Array& indices) {
    std::vector<int> s = indices.shape();
    s.insert(s.end(), source.shape().begin() + 1, source.shape().end());
    return s;
}
Gather::Gather(const Array& source, const Array& indices)
    : Expression(N_GATHER, gather_shape(source, indices), value_dtype(source.dtype()), {source, indices}) {
    DALI_ASSERT(!source.shard().sharded(), "gather from a sharded source is not supported (the indices would name other ranks' rows)");
    shard_ = indices.shard();          // out dims = the indices' dims, then the source's trailing dims
}

static std::vector<int> gather_rows_shape(const Array& source, const Array& indices) {
    std::vector<int> s = indices.shape();
    s.insert(s.end(), source.shape().begin() + 2, source.shape().end());
    return s;
}
GatherFromRows::GatherFromRows(const Array& source, const Array& indices)
    : Expression(N_GATHER_ROWS, gather_rows_shape(source, indices), value_dtype(source.dtype()), {source, indices}) {
    const Shard s = source.shard(), i = indices.shard();
    DALI_ASSERT(s.axis <= 0 && i.axis <= 0, "gather_from_rows: only the row dimension may be sharded");
    DALI_ASSERT(!(s.sharded() && i.sharded()) || s == i, "gather_from_rows: source and indices are sharded differently");
    shard_ = s.sharded() ? s : i;
}

MatMul::MatMul(const Array& left, const Array& right)
    : Expression(N_MATMUL, {left.shape()[0], right.shape()[1]}, value_dtype(left.dtype()), {left, right}) {
    const Shard l = left.shard(), r = right.shard();
    if (l.axis == 1 || r.axis == 0) {
        DALI_ASSERT(l.axis == 1 && r.axis == 0 && l.lo == r.lo && l.total == r.total,
                    "dot: the contracted dimension must be sharded the same way on both operands");
        partial_ = true;                // every rank ends up with the whole product
    } else if (l.axis == 0) {
        DALI_ASSERT(!r.sharded(), "dot: sharding along two dimensions of the product is not supported");
        shard_ = l;
    } else if (r.axis == 1) {
        shard_ = r;
    }
}

// ------------------------------------------------------------------ construction
Array::Array() {}
Array::Array(expression_ptr e) : state_(std::make_shared<ArrayState>(e)) {}
Array::Array(const std::vector<int>& shape, DType dtype, memory::Device dev)
    : state_(std::make_shared<ArrayState>(BufferView::create(shape, dtype, dev))) {}
Array::Array(std::initializer_list<int> shape, DType dtype, memory::Device dev)
    : Array(std::vector<int>(shape), dtype, dev) {}
Array::Array(const std::vector<int>& shape, std::shared_ptr<memory::SynchronizedMemory> mem, const int& offset,
             const std::vector<int>& strides, DType dtype)
    : state_(std::make_shared<ArrayState>(std::make_shared<BufferView>(mem, shape, dtype, offset, strides))) {}
Array::Array(const Array& other, bool copy_memory) {
    if (copy_memory && !other.is_stateless()) {
        Array fresh(other.shape(), other.dtype(), other.preferred_device());
        fresh.expression()->shard_ = other.shard();
        fresh.assign(other);
        fresh.eval();
        state_ = fresh.state_;
    } else {
        state_ = other.state_;
    }
}
Array::Array(const int& v) : Array(std::make_shared<ScalarValue>((double)v, DTYPE_INT32)) {}
Array::Array(const double& v) : Array(std::make_shared<ScalarValue>(v, DTYPE_DOUBLE)) {}
Array::Array(const float& v) : Array(std::make_shared<ScalarValue>((double)v, DTYPE_FLOAT)) {}
Array::Array(const int& v, DType d) : Array(std::make_shared<ScalarValue>((double)v, d)) {}
Array::Array(const double& v, DType d) : Array(std::make_shared<ScalarValue>(v, d)) {}
Array::Array(const float& v, DType d) : Array(std::make_shared<ScalarValue>((double)v, d)) {}

Array Array::zeros(const std::vector<int>& shape, DType dtype, memory::Device dev) {
    Array out(shape, dtype, dev);
    as<BufferView>(out)->memory_->clear();   // zero on first touch
    return out;
}
Array Array::zeros_like(const Array& o) { Array r = zeros(o.shape(), o.dtype(), o.preferred_device()); r.expression()->shard_ = o.shard(); return r; }
Array Array::empty_like(const Array& o) { Array r(o.shape(), o.dtype(), o.preferred_device()); r.expression()->shard_ = o.shard(); return r; }
Array Array::ones(const std::vector<int>& shape, DType dtype, memory::Device dev) {
    Array out(shape, dtype, dev);
    out = 1;
    return out;
}
Array Array::ones_like(const Array& o) { Array r = ones(o.shape(), o.dtype(), o.preferred_device()); r.expression()->shard_ = o.shard(); return r; }

Array Array::adopt_buffer(void* buffer, const std::vector<int>& shape, DType dtype, memory::Device loc,
                          const std::vector<int>& strides) {
    int64_t span = 1;   // elements the view can reach
    if (strides.empty()) {
        for (int s : shape) span *= s;
    } else {
        span = 1;
        for (size_t d = 0; d < shape.size(); ++d) span += (int64_t)(shape[d] - 1) * std::abs(strides[d]);
    }
    auto mem = std::make_shared<memory::SynchronizedMemory>((size_t)span * size_of_dtype(dtype),
                                                            shape.empty() ? 1 : shape.back(),
                                                            loc.is_gpu() ? loc : memory::default_preferred_device);
    mem->adopt_buffer(loc, buffer);
    return Array(shape, mem, 0, strides, dtype);
}
void Array::disown_buffer(memory::Device loc) { memory()->disown_buffer(loc); }

// ------------------------------------------------------------------ state
Array::ArrayState::ArrayState(expression_ptr e) : expression_(e) {
    if (e) shape_ = e->shape_;
}
expression_ptr Array::expression() const { return state_ ? state_->expression_ : nullptr; }
void Array::set_expression(expression_ptr e) const {
    if (!state_) { state_ = std::make_shared<ArrayState>(e); return; }
    state_->expression_ = e;
    if (e && state_->shape_ != e->shape_) state_->shape_ = e->shape_;   // untouched (references stay valid) when equal
}
std::string Array::expression_name() const { return is_stateless() ? "" : expression()->name(); }
std::string Array::full_expression_name() const { return is_stateless() ? "" : expression()->full_name(); }
bool Array::is_stateless() const { return !state_ || !state_->expression_; }
bool Array::is_scalar() const { return ndim() == 0; }
bool Array::is_vector() const { return ndim() == 1; }
bool Array::is_matrix() const { return ndim() == 2; }
bool Array::is_buffer() const { return !is_stateless() && expression()->kind_ == N_BUFFER; }
bool Array::is_assignment() const { return !is_stateless() && expression()->kind_ == N_ASSIGN; }
bool Array::is_assignable() const {
    if (is_stateless()) return false;
    NodeKind k = expression()->kind_;
    if (k == N_BUFFER || k == N_ASSIGN) return true;
    if (k == N_GATHER || k == N_GATHER_ROWS) return expression()->arguments_[0].is_assignable();
    return false;
}

static void require_state(const Array& a, const char* what) {
    DALI_ASSERT(!a.is_stateless(), std::string(what) + " called on a stateless Array");
}
const std::vector<int>& Array::shape() const { require_state(*this, "shape()"); return state_->shape_; }
DType Array::dtype() const { require_state(*this, "dtype()"); return expression()->dtype_; }
int Array::ndim() const { return is_stateless() ? 0 : expression()->ndim(); }
int64_t Array::numel() const { return is_stateless() ? 0 : expression()->numel(); }
int Array::number_of_elements() const {
    int64_t n = numel();
    DALI_ASSERT(n <= INT_MAX, "number_of_elements() overflows int; use numel()");
    return (int)n;
}
std::vector<int> Array::subshape() const {
    if (ndim() == 0) return {};
    return std::vector<int>(shape().begin() + 1, shape().end());
}

void Array::eval(bool wait) const {
    require_state(*this, "eval()");
    if (expression()->kind_ == N_BUFFER) return;
    // optimize -> lower -> run (reference: array.cpp:232-245): the value becomes an assignment, the assignment a list
    // of computations (user-registered implementations first, the fused-kernel lowering otherwise), and every
    // computation replaces its assignment by the buffer it wrote
    Array root = canonical(*this);
    for (const std::shared_ptr<Computation>& step : convert_to_ops(root)) step->run_and_cleanup();
    if (wait && !lazy::dry_run()) {
        memory::Device d = preferred_device();
        if (d.is_gpu()) lazy::check(dalib200_sync(lazy::device_index(d), nullptr), "dalib200_sync");
    }
}

Array Array::borrow_host(void* buffer, const std::vector<int>& shape, DType dtype) {
    int64_t n = 1;
    for (int d : shape) n *= d;
    auto mem = std::make_shared<memory::SynchronizedMemory>((size_t)n * size_of_dtype(dtype), shape.empty() ? 1 : shape.back());
    mem->borrow_buffer(memory::Device::cpu(), buffer);
    return Array(shape, mem, 0, std::vector<int>(), dtype);
}

void Array::to_host(void* out, bool wait) const {
    Array c = ascontiguousarray();
    c.eval(false);      // the copy below is ordered behind the kernels on the device's stream
    const size_t bytes = (size_t)c.numel() * size_of_dtype(c.dtype());
    BufferView* b = as<BufferView>(c);
    const size_t skip = (size_t)b->offset_ * size_of_dtype(b->dtype_);
    if (!b->memory_->is_fresh(memory::Device::cpu())) {
        const int g = b->memory_->fresh_gpu();
        if (g >= 0) {
            const char* src = (const char*)b->memory_->readonly_data(memory::Device::gpu(g)) + skip;
            lazy::check(dalib200_memcpy_d2h(g, out, src, bytes, nullptr), "dalib200_memcpy_d2h");
            if (wait) lazy::check(dalib200_sync(g, nullptr), "dalib200_sync");
            return;
        }
    }
    std::memcpy(out, (const char*)b->memory_->readonly_data(memory::Device::cpu()) + skip, bytes);
}

void Array::eval_together(const std::vector<Array>& arrays, bool wait) {
    lazy::eval_together(arrays);
    if (wait && !arrays.empty() && !lazy::dry_run()) {
        memory::Device d = arrays[0].preferred_device();
        if (d.is_gpu()) lazy::check(dalib200_sync(lazy::device_index(d), nullptr), "dalib200_sync");
    }
}

std::shared_ptr<memory::SynchronizedMemory> Array::memory() const {
    require_state(*this, "memory()");
    if (!is_buffer()) eval();
    DALI_ASSERT(is_buffer(), "memory(): expression did not evaluate to a buffer");
    return as<BufferView>(*this)->memory_;
}
int Array::offset() const { memory(); return (int)as<BufferView>(*this)->offset_; }
const std::vector<int>& Array::strides() const { memory(); return as<BufferView>(*this)->strides_; }
std::vector<int> Array::normalized_strides() const { memory(); return as<BufferView>(*this)->normalized_strides(); }
bool Array::contiguous_memory() const { memory(); return as<BufferView>(*this)->contiguous(); }
bool Array::spans_entire_memory() const {
    memory();
    BufferView* b = as<BufferView>(*this);
    return b->contiguous() && b->offset_ == 0 && (size_t)b->numel() * size_of_dtype(b->dtype_) == b->memory_->total_memory;
}
bool Array::is_transpose() const {
    if (!is_buffer() || ndim() <= 1) return ndim() <= 1;
    BufferView* b = as<BufferView>(*this);
    if (b->strides_.empty()) return false;
    std::vector<int> rs(b->shape_.rbegin(), b->shape_.rend());
    int64_t s = 1;
    for (int d = 0; d < ndim(); ++d) {   // strides ascending: contiguous in reversed dim order
        if (b->shape_[d] != 1 && b->strides_[d] != s) return false;
        s *= b->shape_[d];
    }
    return true;
}

static memory::Device device_of(const expression_ptr& e) {
    if (!e) return memory::default_preferred_device;
    if (e->kind_ == N_BUFFER) return static_cast<BufferView*>(e.get())->memory_->preferred_device;
    for (const Array& a : e->arguments_) {
        if (a.is_stateless()) continue;
        if (a.expression()->kind_ == N_SCALAR || a.expression()->kind_ == N_IOTA) continue;
        return device_of(a.expression());
    }
    return memory::default_preferred_device;
}
memory::Device Array::preferred_device() const {
    memory::Device d = device_of(expression());
    // computing happens on a GPU; the host is only a staging place
    return d.is_gpu() ? d : (memory::default_preferred_device.is_gpu() ? memory::default_preferred_device : memory::Device::gpu(0));
}
void Array::to_device(memory::Device device) const { memory()->to_device(device); }

DType type_promotion(const Array& a, const Array& b) {
    if (a.dtype() == b.dtype()) return value_dtype(a.dtype());      // (two bf16 operands compute in float)
    if (a.dtype() == DTYPE_DOUBLE || b.dtype() == DTYPE_DOUBLE) return DTYPE_DOUBLE;
    return DTYPE_FLOAT;
}
memory::Device device_promotion(const Array& a, const Array& b) {
    memory::Device da = a.preferred_device(), db = b.preferred_device();
    return da == db ? da : memory::default_preferred_device;
}

// ------------------------------------------------------------------ views
// result[i...] = a[off_k + step_k * i_{src_k}] with the given output shape
static Array make_view(const Array& a, const std::vector<int>& shape, const std::vector<ViewDim>& dims);

// A view of a lazy value that is being written to: the value is evaluated into a buffer first -- its handle, and
// every handle that shares its state, now names that buffer -- and the view is taken of the buffer (reference:
// expression.cpp:48-56 turns the owner of any view into an assignment to a fresh buffer).
Array lazy::writable_view(const Array& dest) {
    if (dest.is_stateless() || dest.expression()->kind_ != N_VIEW) return dest;
    View* v = static_cast<View*>(dest.expression().get());
    Array base = v->arguments_[0];
    base.eval(false);
    return make_view(base, v->shape_, v->dims_);
}

static Array make_view(const Array& a, const std::vector<int>& shape, const std::vector<ViewDim>& dims) {
    require_state(a, "view");
    DALI_ASSERT((int)dims.size() == a.ndim(), "internal: view map rank mismatch");
    expression_ptr e = a.expression();
    if (e->kind_ == N_ASSIGN) { a.eval(); e = a.expression(); }
    if (e->kind_ == N_BUFFER) {
        BufferView* b = static_cast<BufferView*>(e.get());
        std::vector<int> st = b->normalized_strides();
        int64_t off = b->offset_;
        std::vector<int> nst(shape.size(), 0);
        for (size_t k = 0; k < dims.size(); ++k) {
            off += dims[k].off * st[k];
            if (dims[k].src >= 0) nst[dims[k].src] += (int)(dims[k].step * st[k]);
        }
        // (the constructor drops the strides again when they are the contiguous ones)
        auto view = std::make_shared<BufferView>(b->memory_, shape, b->dtype_, off, nst);
        view->shard_ = lazy::shard_through_view(b->shard_, b->shape_, dims, shape);
        return Array(view);
    }
    if (e->kind_ == N_SCALAR) {
        return a;   // a scalar broadcasts by itself wherever it is used
    }
    if (e->kind_ == N_VIEW) {
        View* v = static_cast<View*>(e.get());
        std::vector<ViewDim> composed(v->dims_.size());
        for (size_t k = 0; k < v->dims_.size(); ++k) {
            const ViewDim& inner = v->dims_[k];        // arg dim k <- v's out dim inner.src
            if (inner.src < 0) { composed[k] = inner; continue; }
            const ViewDim& outer = dims[inner.src];    // v's out dim <- new out dim
            composed[k].off = inner.off + inner.step * outer.off;
            composed[k].step = inner.step * outer.step;
            composed[k].src = outer.src;
            if (outer.src < 0) composed[k].step = 0;
        }
        return Array(std::make_shared<View>(v->arguments_[0], shape, composed));
    }
    return Array(std::make_shared<View>(a, shape, dims));
}

static std::vector<ViewDim> identity_map(int n) {
    std::vector<ViewDim> d(n);
    for (int k = 0; k < n; ++k) d[k] = ViewDim{k, 0, 1};
    return d;
}

Array Array::pluck_axis(int axis, const Slice& slice_unnormalized) const {
    const int n = ndim();
    if (axis < 0) axis += n;
    DALI_ASSERT(axis >= 0 && axis < n, "pluck_axis dimension (" + std::to_string(axis) + ") must be less than the dimensionality of plucked array (" + std::to_string(n) + ").");
    Slice s = Slice::normalize_and_check(slice_unnormalized, shape()[axis]);
    std::vector<int> nshape = shape();
    nshape[axis] = s.size();
    std::vector<ViewDim> dims = identity_map(n);
    if (s.step > 0) dims[axis] = ViewDim{axis, s.start, s.step};
    else dims[axis] = ViewDim{axis, s.end - 1, s.step};
    return make_view(*this, nshape, dims);
}

Array Array::pluck_axis(const int& axis_, const int& idx_) const {
    const int n = ndim();
    int axis = axis_ < 0 ? axis_ + n : axis_;
    DALI_ASSERT(axis >= 0 && axis < n, "pluck_axis dimension (" + std::to_string(axis) + ") must be less than the dimensionality of plucked array (" + std::to_string(n) + ").");
    int idx = idx_ < 0 ? idx_ + shape()[axis] : idx_;
    DALI_ASSERT(idx >= 0 && idx < shape()[axis], "index " + std::to_string(idx_) + " out of range for dimension " + std::to_string(axis) + " of size " + std::to_string(shape()[axis]));
    std::vector<int> nshape;
    std::vector<ViewDim> dims(n);
    for (int k = 0; k < n; ++k) {
        if (k == axis) { dims[k] = ViewDim{-1, idx, 0}; continue; }
        dims[k] = ViewDim{(int)nshape.size(), 0, 1};
        nshape.push_back(shape()[k]);
    }
    return make_view(*this, nshape, dims);
}

Array Array::operator[](const int& idx) const {
    DALI_ASSERT(ndim() > 0, "Slicing a scalar array is not allowed.");
    return pluck_axis(0, idx);
}
Array Array::operator[](const Array& indices) const { return op::gather(*this, indices); }
Array Array::gather_from_rows(const Array& indices) const { return op::gather_from_rows(*this, indices); }
SlicingInProgress<Array> Array::operator[](const Slice& s) const { return SlicingInProgress<Array>(*this)[s]; }
SlicingInProgress<Array> Array::operator[](const Broadcast& b) const { return SlicingInProgress<Array>(*this)[b]; }

Array Array::operator()(int idx) const {
    int64_t n = numel();
    DALI_ASSERT(idx >= 0 && idx < n, "Index " + std::to_string(idx) + " must be in [0," + std::to_string(n) + "].");
    std::vector<ViewDim> dims(ndim());
    int64_t rem = idx;
    for (int d = ndim() - 1; d >= 0; --d) {
        dims[d] = ViewDim{-1, rem % shape()[d], 0};
        rem /= shape()[d];
    }
    return make_view(*this, {}, dims);
}

Array Array::expand_dims(int new_axis) const {
    const int n = ndim();
    if (new_axis < 0) new_axis += n + 1;
    DALI_ASSERT(new_axis >= 0 && new_axis <= n, "expand_dims new_axis argument must be strictly positive and at most the dimensionality of the array (got new_axis = " + std::to_string(new_axis) + ", ndim = " + std::to_string(n) + ").");
    std::vector<int> nshape = shape();
    nshape.insert(nshape.begin() + new_axis, 1);
    std::vector<ViewDim> dims(n);
    for (int k = 0; k < n; ++k) dims[k] = ViewDim{k < new_axis ? k : k + 1, 0, 1};
    return make_view(*this, nshape, dims);
}

Array Array::squeeze(int axis) const {
    const int n = ndim();
    if (axis < 0) axis += n;
    DALI_ASSERT(axis >= 0 && axis < n, "squeeze dimension (" + std::to_string(axis) + ") must be less the dimensionality of compacted tensor (" + std::to_string(n) + ").");
    DALI_ASSERT(shape()[axis] == 1, "cannot select an axis to squeeze out which has size not equal to one (got axis = " + std::to_string(axis) + ", shape[" + std::to_string(axis) + "] = " + std::to_string(shape()[axis]) + ").");
    return pluck_axis(axis, 0);
}

Array Array::broadcast_scalar_to_ndim(const int& target) const {
    DALI_ASSERT(target >= 0, "broadcast_scalar_to_ndim expected a non-negative integer (got " + std::to_string(target) + ").");
    if (!is_scalar()) return *this;
    Array res = *this;
    for (int i = 0; i < target; ++i) res = res.expand_dims(0);
    return res;
}

Array Array::right_fit_ndim(int target) const {
    Array res = *this;
    while (res.ndim() < target) res = res.expand_dims(0);
    return res;
}

Array Array::dimshuffle(const std::vector<int>& pattern) const {
    const int n = ndim();
    DALI_ASSERT((int)pattern.size() == n, "number of dimensions in dimshuffle does not correspond to the dimensionality of the array (got pattern of length " + std::to_string(pattern.size()) + " and ndim = " + std::to_string(n) + ").");
    std::vector<bool> seen(n, false);
    std::vector<int> nshape(n);
    std::vector<ViewDim> dims(n);
    for (int d = 0; d < n; ++d) {
        int p = pattern[d] < 0 ? pattern[d] + n : pattern[d];
        DALI_ASSERT(p >= 0 && p < n && !seen[p], "dimshuffle pattern must be a permutation of the axes (got " + shape_str(pattern) + ").");
        seen[p] = true;
        nshape[d] = shape()[p];
        dims[p] = ViewDim{d, 0, 1};
    }
    return make_view(*this, nshape, dims);
}
Array Array::transpose() const {
    std::vector<int> p(ndim());
    for (int d = 0; d < ndim(); ++d) p[d] = ndim() - 1 - d;
    return dimshuffle(p);
}
Array Array::transpose(const std::vector<int>& axes) const { return dimshuffle(axes); }
Array Array::swapaxes(int a1, int a2) const {
    const int n = ndim();
    if (a1 < 0) a1 += n;
    if (a2 < 0) a2 += n;
    DALI_ASSERT(a1 >= 0 && a1 < n && a2 >= 0 && a2 < n, "swapaxes axes must be less than ndim (got " + std::to_string(a1) + ", " + std::to_string(a2) + ", ndim = " + std::to_string(n) + ").");
    std::vector<int> p(n);
    for (int d = 0; d < n; ++d) p[d] = d;
    std::swap(p[a1], p[a2]);
    return dimshuffle(p);
}

Array Array::broadcast_to_shape(const std::vector<int>& target) const {
    const int n = ndim();
    DALI_ASSERT((int)target.size() == n, "broadcast_to_shape must receive a shape (" + shape_str(target) + ") with the same dimensionality as the array (current shape = " + shape_str(shape()) + ").");
    std::vector<ViewDim> dims(n);
    bool changed = false;
    for (int d = 0; d < n; ++d) {
        if (shape()[d] == target[d]) { dims[d] = ViewDim{d, 0, 1}; continue; }
        DALI_ASSERT(shape()[d] == 1, "broadcast_to_shape cannot reshape broadcasted dimension " + std::to_string(d) + " from current size " + std::to_string(shape()[d]) + " to " + std::to_string(target[d]) + " (current shape = " + shape_str(shape()) + ", new shape = " + shape_str(target) + ").");
        dims[d] = ViewDim{-1, 0, 0};
        changed = true;
    }
    if (!changed) return *this;
    return make_view(*this, target, dims);
}

Array Array::reshape(const std::vector<int>& new_shape_) const {
    std::vector<int> ns = new_shape_;
    int64_t known = 1;
    int unknown = -1;
    for (size_t d = 0; d < ns.size(); ++d) {
        if (ns[d] < 0) {
            DALI_ASSERT(unknown < 0, "can only specify one unknown dimension (-1) for reshape.");
            unknown = (int)d;
        } else {
            known *= ns[d];
        }
    }
    if (unknown >= 0) {
        DALI_ASSERT(known > 0 && numel() % known == 0, "cannot deduce unknown dimension (" + shape_str(ns) + ") for array with " + std::to_string(numel()) + " elements.");
        ns[unknown] = (int)(numel() / known);
        known *= ns[unknown];
    }
    DALI_ASSERT(known == numel(), "New shape (" + shape_str(ns) + ") must have the same number of elements as previous shape (" + shape_str(shape()) + ")");
    if (ns == shape()) return *this;
    const Shard reshaped = lazy::shard_through_reshape(shard(), shape(), ns);
    if (Iota* io = as<Iota>(*this)) {
        int64_t step;
        if (io->linear(&step)) {      // offset + step * linear index, whatever the shape
            std::vector<int64_t> st(ns.size(), 0);
            int64_t acc = step;
            for (int d = (int)ns.size() - 1; d >= 0; --d) { st[d] = acc; acc *= ns[d]; }
            return Array(std::make_shared<Iota>(ns, io->offset_, st));
        }
    }
    Array src = *this;
    if (!src.is_buffer()) src.eval(false);
    if (!src.contiguous_memory()) src = src.ascontiguousarray();
    BufferView* b = as<BufferView>(src);
    auto out = std::make_shared<BufferView>(b->memory_, ns, b->dtype_, b->offset_, std::vector<int>());
    out->shard_ = reshaped;
    return Array(out);
}
Array Array::ravel() const { return reshape({-1}); }

Array Array::ascontiguousarray() const {
    if (is_buffer() && as<BufferView>(*this)->contiguous()) return *this;
    Array out(shape(), dtype(), preferred_device());
    out.expression()->shard_ = shard();
    lazy::run_assignment(out, OPERATOR_T_EQL, *this);
    return out;
}

void Array::initialize(const std::vector<int>& shape, DType dtype, memory::Device dev) {
    set_expression(BufferView::create(shape, dtype, dev));
}
Array& Array::reset() { state_.reset(); return *this; }

Array Array::astype(DType d) const { return op::astype(*this, d); }

// ------------------------------------------------------------------ member shortcuts
Array Array::sum() const { return op::sum(*this); }
Array Array::mean() const { return op::mean(*this); }
Array Array::min() const { return op::min(*this); }
Array Array::max() const { return op::max(*this); }
Array Array::L2_norm() const { return op::L2_norm(*this); }
Array Array::abs() const { return op::abs(*this); }
Array Array::exp() const { return op::exp(*this); }
Array Array::tanh() const { return op::tanh(*this); }
Array Array::sigmoid() const { return op::sigmoid(*this); }
Array Array::sum(const std::vector<int>& axes, bool k) const { return op::sum(*this, axes, k); }
Array Array::mean(const std::vector<int>& axes, bool k) const { return op::mean(*this, axes, k); }
Array Array::min(const std::vector<int>& axes, bool k) const { return op::min(*this, axes, k); }
Array Array::max(const std::vector<int>& axes, bool k) const { return op::max(*this, axes, k); }
Array Array::L2_norm(const std::vector<int>& axes, bool k) const { return op::L2_norm(*this, axes, k); }
Array Array::argmin(const int& axis) const { return op::argmin(*this, axis); }
Array Array::argmin() const { return op::argmin(*this); }
Array Array::argmax(const int& axis) const { return op::argmax(*this, axis); }
Array Array::argmax() const { return op::argmax(*this); }
Array Array::dot(const Array& other) const { return op::dot(*this, other); }
Array Array::operator-() const { return op::elementwise(*this, "negate"); }
bool Array::any_isnan() const { return (int)Array(op::any_isnan(*this)) != 0; }
bool Array::any_isinf() const { return (int)Array(op::any_isinf(*this)) != 0; }

// ------------------------------------------------------------------ host access
template <typename T>
T Array::scalar_value() const {
    DALI_ASSERT(numel() == 1, "Scalar cast must only be called on an Array with a single element (got shape = " + shape_str(shape()) + ").");
    Array src = *this;
    src.eval();
    BufferView* b = as<BufferView>(src);
    const char* base = (const char*)b->memory_->readonly_data(memory::Device::cpu());
    base += b->offset_ * size_of_dtype(b->dtype_);
    switch (b->dtype_) {
        case DTYPE_FLOAT: return (T)(*(const float*)base);
        case DTYPE_DOUBLE: return (T)(*(const double*)base);
        case DTYPE_INT32: return (T)(*(const int*)base);
        case DTYPE_BF16: return (T)bf16_bits_to_float(*(const unsigned short*)base);
    }
    return T();
}
Array::operator float() const { return scalar_value<float>(); }
Array::operator double() const { return scalar_value<double>(); }
Array::operator int() const { return scalar_value<int>(); }

// ------------------------------------------------------------------ assignment
// Does the value `a` read, through any handle in its tree (pending assignments included), the state `s`?  Handles
// share their state, so once a new pending expression is installed in `s` every such handle names IT: a value that
// reads the array it is assigned to (w -= step * dw with dw += w * ... still pending) would then read itself.
static bool reaches_state(const Array& a, const Array::ArrayState* s, std::unordered_set<const Expression*>& seen, int depth = 0) {
    if (a.is_stateless() || depth > 256) return false;
    if (a.state().get() == s) return true;
    const Expression* e = a.expression().get();
    if (!seen.insert(e).second) return false;
    for (const Array& arg : e->arguments_)
        if (reaches_state(arg, s, seen, depth + 1)) return true;
    return false;
}
static bool reads_itself(const Array& left, const Array& right) {
    std::unordered_set<const Expression*> seen;
    return reaches_state(right, left.state().get(), seen);
}

Array& Array::assign(const Array& other) {
    require_state(other, "assign");
    if (is_stateless()) {
        Array fresh(other.shape(), other.dtype(), other.preferred_device());
        state_ = fresh.state_;
    }
    // runs now, for the reasons given at inplace() below.  A view of a lazy value is a place once that value has been
    // evaluated into a buffer (the handles on its state then name the buffer, lower.cc:writable_view)
    if (expression()->kind_ == N_VIEW) set_expression(lazy::writable_view(*this).expression());
    if (expression()->kind_ != N_BUFFER && expression()->kind_ != N_GATHER && expression()->kind_ != N_GATHER_ROWS) eval(false);
    lazy::evaluate_shared_values(other);
    Array update(std::make_shared<Assignment>(Array(expression()), OPERATOR_T_EQL, other));
    update.eval(false);
    return *this;
}
void Array::copy_from(const Array& other) { assign(other); eval(false); }
Array& Array::operator=(const int& v) { return assign(Array(v)); }
Array& Array::operator=(const float& v) { return assign(Array(v)); }
Array& Array::operator=(const double& v) { return assign(Array(v)); }
void Array::clear() {
    if (is_buffer() && spans_entire_memory()) as<BufferView>(*this)->memory_->clear();
    else assign(Array(0.0));
}

// left (op)= right.  An update of a PLACE (a buffer, a view of one, a gather of one) runs when the statement is
// written, not when the array is next read: the arrays the right-hand side reads may be overwritten by the
// statements that follow (a solver clears the gradient right after the update that read it), and handles share
// their state, so a pending update would read what they hold later.  The reference leaves such updates pending
// (dali/array/array.cpp:722-726) and its own solvers then read cleared gradients.  With the update run the lazy
// values below it that other handles name too (a solver's running averages) and, when the right-hand side is a
// named lazy value (`named`: passed as an lvalue), that value itself are evaluated in place: they read the same arrays.
// A lazy left-hand side is not a place: the operator is folded into its expression, as in the reference
// (dali/array/jit/jit.cpp:1052-1078).
static Array& inplace(Array& left, OPERATOR_T op, const Array& right, bool named = false) {
    DALI_ASSERT(!left.is_stateless(), "in-place operation on a stateless Array");
    if (left.expression()->kind_ == N_VIEW) left.set_expression(lazy::writable_view(left).expression());
    if (!left.is_assignable() && !reads_itself(left, right)) {
        if (op == OPERATOR_T_LSE) {
            Array r = op::autoreduce_assign(left, right);
            left.set_expression(r.expression());
            return left;
        }
        Array cur(left.expression());
        Array res;
        switch (op) {
            case OPERATOR_T_ADD: res = op::add(cur, right); break;
            case OPERATOR_T_SUB: res = op::subtract(cur, right); break;
            case OPERATOR_T_MUL: res = op::eltmul(cur, right); break;
            case OPERATOR_T_DIV: res = op::eltdiv(cur, right); break;
            default: res = right;
        }
        left.set_expression(res.expression());
        return left;
    }
    if (left.expression()->kind_ != N_BUFFER && left.expression()->kind_ != N_GATHER && left.expression()->kind_ != N_GATHER_ROWS)
        left.eval(false);                      // a pending assignment, or a lazy value that reads itself below
    if (!right.is_stateless()) {
        lazy::evaluate_shared_values(right);
        if (named && !right.is_buffer() && right.expression()->kind_ != N_SCALAR) right.eval(false);
    }
    Array update = op == OPERATOR_T_LSE ? op::autoreduce_assign(left, right)
                                        : Array(std::make_shared<Assignment>(Array(left.expression()), op, right));
    update.eval(false);
    return left;
}
#define DALI_DEFINE_INPLACE(SYMBOL, OP)                                                             \
    Array& operator SYMBOL(Array& left, const Array& right) { return inplace(left, OP, right, true); }    \
    Array& operator SYMBOL(Array& left, Array&& right) { return inplace(left, OP, right, false); }         \
    void operator SYMBOL(Array&& left, const Array& right) { Array l(left); inplace(l, OP, right, true); l.eval(false); }  \
    void operator SYMBOL(Array&& left, Array&& right) { Array l(left); inplace(l, OP, right, false); l.eval(false); }
DALI_DEFINE_INPLACE(+=, OPERATOR_T_ADD)
DALI_DEFINE_INPLACE(-=, OPERATOR_T_SUB)
DALI_DEFINE_INPLACE(*=, OPERATOR_T_MUL)
DALI_DEFINE_INPLACE(/=, OPERATOR_T_DIV)
DALI_DEFINE_INPLACE(<<=, OPERATOR_T_LSE)

#define DALI_DEFINE_INTERACTION(SYMBOL, FN)                                                         \
    Array operator SYMBOL(const Array& l, const Array& r) { return op::FN(l, r); }                  \
    Array operator SYMBOL(const Array& l, double r) { return op::FN(l, Array(r)); }                 \
    Array operator SYMBOL(const Array& l, float r) { return op::FN(l, Array(r)); }                  \
    Array operator SYMBOL(const Array& l, int r) { return op::FN(l, Array(r)); }                    \
    Array operator SYMBOL(double l, const Array& r) { return op::FN(Array(l), r); }                 \
    Array operator SYMBOL(float l, const Array& r) { return op::FN(Array(l), r); }                  \
    Array operator SYMBOL(int l, const Array& r) { return op::FN(Array(l), r); }
DALI_DEFINE_INTERACTION(+, add)
DALI_DEFINE_INTERACTION(-, subtract)
DALI_DEFINE_INTERACTION(*, eltmul)
DALI_DEFINE_INTERACTION(/, eltdiv)

// ------------------------------------------------------------------ comparison, printing, IO
bool Array::equals(const Array& l, const Array& r) {
    if (l.is_stateless() && r.is_stateless()) return true;
    if (l.is_stateless() || r.is_stateless()) return false;
    if (l.shape() != r.shape()) return false;
    return (int)Array(op::all_equals(l, r)) != 0;
}
bool Array::allclose(const Array& l, const Array& r, const double& atol) {
    if (l.is_stateless() && r.is_stateless()) return true;
    if (l.is_stateless() || r.is_stateless()) return false;
    if (l.shape() != r.shape()) return false;
    return (int)Array(op::all_close(l, r, Array(atol))) != 0;
}
bool operator==(const Array& l, const Array& r) { return Array::equals(l, r); }

void Array::print(std::basic_ostream<char>& stream, const int& indent, const bool& add_newlines, const bool& print_comma) const {
    Array c = ascontiguousarray();
    c.eval();
    BufferView* b = as<BufferView>(c);
    const char* base = (const char*)b->memory_->readonly_data(memory::Device::cpu()) + b->offset_ * size_of_dtype(b->dtype_);
    auto at = [&](int64_t i) -> double {
        switch (b->dtype_) {
            case DTYPE_FLOAT: return ((const float*)base)[i];
            case DTYPE_DOUBLE: return ((const double*)base)[i];
            case DTYPE_BF16: return bf16_bits_to_float(((const unsigned short*)base)[i]);
            default: return ((const int*)base)[i];
        }
    };
    std::string pad(indent, ' ');
    if (ndim() == 0) {
        stream << pad << at(0);
    } else if (ndim() == 1) {
        stream << pad << "[";
        for (int i = 0; i < shape()[0]; ++i) stream << (i ? " " : "") << at(i);
        stream << "]";
    } else {
        stream << pad << "[\n";
        for (int i = 0; i < shape()[0]; ++i) (*this)[i].print(stream, indent + 4, true, i + 1 < shape()[0]);
        stream << pad << "]";
    }
    if (print_comma) stream << ",";
    if (add_newlines) stream << "\n";
}

// minimal .npy (format 1.0) reader / writer for <f4 <f8 <i4
namespace {
// the .npy reader over any byte source: read(dst, n) returns the bytes it delivered
template <typename Read>
Array load_npy(Read read, const std::string& what) {
    char magic[10];
    DALI_ASSERT(read(magic, 10) == 10 && std::memcmp(magic, "\x93NUMPY", 6) == 0, "npy_load: " + what + " is not a .npy file");
    size_t hlen = (unsigned char)magic[8] | ((unsigned char)magic[9] << 8);
    if (magic[6] >= 2) {
        char extra[2];
        DALI_ASSERT(read(extra, 2) == 2, "npy_load: truncated header in " + what);
        hlen |= ((size_t)(unsigned char)extra[0] << 16) | ((size_t)(unsigned char)extra[1] << 24);
    }
    std::string header(hlen, ' ');
    DALI_ASSERT(read(&header[0], hlen) == hlen, "npy_load: truncated header in " + what);
    auto find_val = [&](const std::string& key) {
        size_t p = header.find(key);
        DALI_ASSERT(p != std::string::npos, "npy_load: malformed header in " + what);
        return header.substr(header.find(':', p) + 1);
    };
    std::string descr = find_val("'descr'");
    DType dtype;
    if (descr.find("f4") != std::string::npos) dtype = DTYPE_FLOAT;
    else if (descr.find("f8") != std::string::npos) dtype = DTYPE_DOUBLE;
    else if (descr.find("i4") != std::string::npos) dtype = DTYPE_INT32;
    else throw std::runtime_error("can only load numpy arrays with dtype float, double or int32 (" + what + ")");
    bool fortran = find_val("'fortran_order'").find("True") < 8;
    std::string shp = find_val("'shape'");
    shp = shp.substr(shp.find('(') + 1, shp.find(')') - shp.find('(') - 1);
    std::vector<int> shape;
    std::istringstream ss(shp);
    std::string tok;
    while (std::getline(ss, tok, ',')) {
        bool digits = false;
        for (char c : tok) digits = digits || (c >= '0' && c <= '9');
        if (digits) shape.push_back(std::atoi(tok.c_str()));
    }
    int64_t n = 1;
    for (int s : shape) n *= s;
    const size_t bytes = (size_t)n * size_of_dtype(dtype);
    void* buf = std::malloc(bytes + 1);
    if (read((char*)buf, bytes) != bytes) {
        std::free(buf);
        throw std::runtime_error("npy_load: truncated file " + what);
    }
    if (fortran) {
        std::vector<int> rs(shape.rbegin(), shape.rend());
        return Array::adopt_buffer(buf, rs, dtype).transpose();
    }
    return Array::adopt_buffer(buf, shape, dtype);
}
}  // namespace

Array Array::load(const std::string& fname) {
    std::ifstream f(fname, std::ios::binary);
    DALI_ASSERT(f.good(), "npy_load: Error! Unable to open file " + fname);
    return load_npy([&](char* dst, size_t n) { f.read(dst, (std::streamsize)n); return (size_t)f.gcount(); }, fname);
}

// reads one array from the current position of an open file (several arrays can follow one another)
Array Array::load(FILE* fp) {
    DALI_ASSERT(fp != nullptr, "npy_load: null FILE*");
    return load_npy([&](char* dst, size_t n) { return std::fread(dst, 1, n, fp); }, "<FILE*>");
}

void Array::save(const std::string& fname, const Array& arr, const std::ios_base::openmode& mode) {
    std::ofstream f(fname, std::ios::binary | mode);
    DALI_ASSERT(f.good(), "cannot open " + fname + " for writing");
    Array::save(f, arr);
}

void Array::save(std::basic_ostream<char>& f, const Array& arr) {
    // (NumPy has no bf16: such an array is written as the float32 values it holds, exactly)
    Array c = arr.dtype() == DTYPE_BF16 ? arr.astype(DTYPE_FLOAT).ascontiguousarray() : arr.ascontiguousarray();
    c.eval();
    BufferView* b = as<BufferView>(c);
    const char* base = (const char*)b->memory_->readonly_data(memory::Device::cpu()) + b->offset_ * size_of_dtype(b->dtype_);
    std::string descr = b->dtype_ == DTYPE_FLOAT ? "<f4" : (b->dtype_ == DTYPE_DOUBLE ? "<f8" : "<i4");
    std::ostringstream h;
    h << "{'descr': '" << descr << "', 'fortran_order': False, 'shape': (";
    for (int d = 0; d < c.ndim(); ++d) h << c.shape()[d] << (c.ndim() == 1 || d + 1 < c.ndim() ? "," : "") << (d + 1 < c.ndim() ? " " : "");
    h << "), }";
    std::string header = h.str();
    while ((10 + header.size() + 1) % 64 != 0) header += ' ';
    header += '\n';
    f.write("\x93NUMPY\x01\x00", 8);
    unsigned short len = (unsigned short)header.size();
    f.write((const char*)&len, 2);
    f.write(header.data(), (std::streamsize)header.size());
    f.write(base, (std::streamsize)(c.numel() * size_of_dtype(b->dtype_)));
}
