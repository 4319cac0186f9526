// Dali's lazy Array front end over the B200 back end.
//
// Source-compatible with the part of the reference API that lies on the
// expression -> optimize -> compile -> cache -> run path
// (dali/array/array.h:18-260, slice.h:13-60, dtype.h:6-10,
// memory/device.h:13-57, memory/synchronized_memory.h:35-140,
// runtime_config.h:9-22): same class names, method names, argument meaning
// and error behaviour (std::runtime_error for shape / rank / dtype
// violations), so code written against the reference compiles and runs
// unchanged.  What lies underneath is new: expression trees are lowered to
// the fused-expression IR of the C ABI (include/dali_b200.h) and run as
// generated sm_100a kernels; there is no CPU compute path.
#ifndef DALI_ARRAY_ARRAY_H
#define DALI_ARRAY_ARRAY_H

#include <cstdint>
#include <cstdio>
#include <initializer_list>
#include <iostream>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "dali/utils/assert2.h"
#include "dali/utils/make_message.h"
#include "dali/utils/print_utils.h"

// ------------------------------------------------------------------ dtype
// DTYPE_BF16 is not in the reference (dali/array/dtype.h:6-10 has the first three): a 16-bit STORAGE type.  Views of a
// bf16 Array stay bf16; every computation on one runs in fp32 and yields a float Array (x.astype(DTYPE_BF16) or an
// assignment into a bf16 Array round the result back, to nearest even); op::dot of two bf16 matrices is the bf16
// tensor-core product with fp32 accumulation.
enum DType { DTYPE_FLOAT = 0, DTYPE_DOUBLE = 1, DTYPE_INT32 = 2, DTYPE_BF16 = 3 };
// the type arithmetic on `dtype` happens in (float for bf16, the type itself otherwise)
inline DType value_dtype(DType dtype) { return dtype == DTYPE_BF16 ? DTYPE_FLOAT : dtype; }
int size_of_dtype(DType dtype);
std::string dtype_to_name(DType dtype);
std::ostream& operator<<(std::ostream&, const DType&);
template <typename T> DType template_to_dtype();
template <> DType template_to_dtype<float>();
template <> DType template_to_dtype<double>();
template <> DType template_to_dtype<int>();

// assignment operators (dali/array/expression/operator.h)
enum OPERATOR_T {
    OPERATOR_T_EQL = 0, OPERATOR_T_ADD = 1, OPERATOR_T_SUB = 2, OPERATOR_T_MUL = 3, OPERATOR_T_DIV = 4,
    OPERATOR_T_LSE = 5
};

// ------------------------------------------------------------------ memory
namespace memory {
enum DeviceT { DEVICE_T_ERROR = 0, DEVICE_T_FAKE = 1, DEVICE_T_CPU = 2, DEVICE_T_GPU = 3 };
enum AM { AM_READONLY = 0, AM_MUTABLE = 1, AM_OVERWRITE = 2 };

class Device {
    DeviceT type_;
    int number_;
  public:
    Device(DeviceT type = DEVICE_T_ERROR, int number = -1) : type_(type), number_(number) {}
    DeviceT type() const { return type_; }
    int number() const { return number_; }
    bool is_cpu() const { return type_ == DEVICE_T_CPU; }
    bool is_gpu() const { return type_ == DEVICE_T_GPU; }
    bool is_error() const { return type_ == DEVICE_T_ERROR; }
    static Device cpu() { return Device(DEVICE_T_CPU, -1); }
    static Device gpu(int number) { return Device(DEVICE_T_GPU, number); }
    static int num_gpus();
    static std::vector<Device> installed_devices();
    bool operator==(const Device& o) const { return type_ == o.type_ && number_ == o.number_; }
    bool operator!=(const Device& o) const { return !(*this == o); }
};
std::ostream& operator<<(std::ostream&, const Device&);

// Where newly created Arrays compute.  gpu(0) as in a CUDA build of the
// reference (dali/runtime_config.cpp:12-18).  memory::Device::cpu() remains
// a place to stage host data, never a place to compute.
extern Device default_preferred_device;
class WithDevicePreference {
    const Device old_value;
    WithDevicePreference(const WithDevicePreference&) = delete;
    WithDevicePreference& operator=(const WithDevicePreference&) = delete;
  public:
    explicit WithDevicePreference(Device device);
    ~WithDevicePreference();
};

// One logical buffer with a host copy and a copy on each GPU, each with a
// freshness flag; data(device, mode) makes the requested copy fresh (copying
// from a fresh one if needed) and, for writable modes, marks the others stale.
// Byte counts are 64-bit (the reference's are int).
class SynchronizedMemory {
  public:
    const size_t total_memory;
    const int inner_dimension;
    Device preferred_device;
    SynchronizedMemory(size_t total_memory, int inner_dimension = 1, Device preferred_device = default_preferred_device,
                       bool clear_on_allocation = false);
    ~SynchronizedMemory();
    SynchronizedMemory(const SynchronizedMemory&) = delete;

    void* data(const Device& device, AM access_mode = AM_MUTABLE);
    const void* readonly_data(const Device& device);
    void* mutable_data(const Device& device);
    void* overwrite_data(const Device& device);
    bool is_fresh(const Device& device) const;
    bool is_allocated(const Device& device) const;
    bool is_any_fresh() const;
    int fresh_gpu() const;                               // a GPU that holds a fresh copy, -1 if none does
    void clear();                                        // zero everything, lazily
    void to_device(const Device& device);
    // takes ownership of a caller buffer (host: freed with free(); device: returned to the pool)
    void adopt_buffer(const Device& device, void* buffer);
    // uses a caller buffer WITHOUT taking ownership: it is never freed here
    void borrow_buffer(const Device& device, void* buffer);
    void disown_buffer(const Device& device);
    // Counts writable accesses; lets derived data (e.g. the TF32 split of a weight matrix)
    // be kept next to the buffer and dropped when the buffer changes.
    uint64_t version() const;
    std::shared_ptr<void>& derived_data();
    uint64_t& derived_version();
  private:
    struct Impl;
    Impl* impl_;
};
}  // namespace memory

// ------------------------------------------------------------------ slicing
struct Broadcast {};

struct Slice {
    bool has_start, has_end;
    int start, end, step;
    Slice() : has_start(false), has_end(false), start(0), end(0), step(1) {}
    Slice(int end_) : has_start(false), has_end(true), start(0), end(end_), step(1) {}
    // start and end of one sign must be ordered, the step cannot be zero (dali/array/slice.cpp:25-38)
    Slice(int start_, int end_, int step_ = 1);
    // resolves negative / missing bounds against a dimension size and checks the range
    static Slice normalize_and_check(const Slice&, int dim_size);
    int size() const;
    // whether walking the slice visits `index` (a negative step walks [start, end) backwards; slice.cpp:79-92)
    bool contains(int index) const;
};

// ------------------------------------------------------------------ sharding (not in the reference)
// How an Array relates to the other ranks of the communicator (one process per GPU, include/dali_b200.h):
// the local part of a logical array cut along `axis`, holding indices [lo, lo + local extent) of `total`.
// axis < 0: every rank holds the whole array.  Replaces the reference's per-node device heuristic
// (dali/array/jit/jit.cpp:367-385): placement is explicit, and ranks exchange data only where a reduction or a
// product contracts the sharded dimension.
struct Shard {
    int axis;
    int64_t lo, total;
    Shard() : axis(-1), lo(0), total(0) {}
    Shard(int axis_, int64_t lo_, int64_t total_) : axis(axis_), lo(lo_), total(total_) {}
    bool sharded() const { return axis >= 0; }
    bool operator==(const Shard& o) const { return axis == o.axis && (axis < 0 || (lo == o.lo && total == o.total)); }
};

class Expression;
typedef std::shared_ptr<Expression> expression_ptr;
template <typename Container> struct SlicingInProgress;

// ------------------------------------------------------------------ Array
class Array {
  public:
    // shape_ is the state's own copy of the expression's shape: shape() hands out a reference to it, which stays
    // valid when the expression is replaced by its evaluated buffer (callers of the reference hold such references
    // across calls that evaluate the array, e.g. dali/array/gemm/tensordot_as_dot.h:82-103)
    struct ArrayState {
        mutable expression_ptr expression_;
        mutable std::vector<int> shape_;
        explicit ArrayState(expression_ptr e);
    };
  private:
    mutable std::shared_ptr<ArrayState> state_;
    template <typename T> T scalar_value() const;
  public:
    expression_ptr expression() const;
    void set_expression(expression_ptr) const;
    std::shared_ptr<ArrayState> state() const { return state_; }
    long handle_count() const { return state_.use_count(); }     // Arrays (user variables, node arguments) that share this state
    std::string expression_name() const;
    std::string full_expression_name() const;

    Array();
    Array(expression_ptr);
    Array(const std::vector<int>& shape, DType dtype = DTYPE_FLOAT, memory::Device preferred_device = memory::default_preferred_device);
    Array(std::initializer_list<int> shape, DType dtype = DTYPE_FLOAT, memory::Device preferred_device = memory::default_preferred_device);
    Array(const std::vector<int>& shape, std::shared_ptr<memory::SynchronizedMemory>, const int& offset,
          const std::vector<int>& strides, DType dtype = DTYPE_FLOAT);
    Array(const Array& other, bool copy_memory = false);
    Array(const int& value);
    Array(const double& value);
    Array(const float& value);
    Array(const int& value, DType dtype);
    Array(const double& value, DType dtype);
    Array(const float& value, DType dtype);

    static Array zeros(const std::vector<int>& shape, DType dtype = DTYPE_FLOAT, memory::Device preferred_device = memory::default_preferred_device);
    static Array zeros_like(const Array& other);
    static Array empty_like(const Array& other);
    static Array ones(const std::vector<int>& shape, DType dtype = DTYPE_FLOAT, memory::Device preferred_device = memory::default_preferred_device);
    static Array ones_like(const Array& other);
    // takes ownership of `buffer` (host memory from malloc, or device memory from dalib200_alloc)
    static Array adopt_buffer(void* buffer, const std::vector<int>& shape, DType dtype,
                              memory::Device buffer_location = memory::Device::cpu(), const std::vector<int>& strides = {});
    void disown_buffer(memory::Device buffer_location = memory::Device::cpu());
    // Not in the reference.  Wraps HOST memory the caller keeps owning (never copied, never freed here; page-locked
    // memory reaches the GPU by DMA); it must stay alive and unchanged until what reads it has been evaluated.
    static Array borrow_host(void* buffer, const std::vector<int>& shape, DType dtype);
    // Not in the reference.  Evaluates and copies the value, C-contiguous, into caller memory; a value that lives
    // on a GPU only goes straight there (no intermediate host copy).  wait = false leaves a copy into page-locked
    // memory in flight on the device's stream (several results, one synchronisation at the end).
    void to_host(void* out, bool wait = true) const;
    // Not in the reference.  Evaluates several lazy arrays of one shape in ONE kernel where their trees allow it
    // (what they share is computed once; an LSTM cell's c' and h' become one GEMM launch whose epilogue is the
    // gating), one after the other otherwise.
    static void eval_together(const std::vector<Array>& arrays, bool wait = true);
    // Not in the reference.  Declares this (evaluated) Array to be the rows [lo, lo + shape()[axis]) of a logical array
    // of `total` rows along `axis` that is spread over the ranks of the communicator.  Elementwise work, views that
    // leave the axis whole, reductions over other axes and dot(x, W) with a whole W stay local and keep the mark;
    // a reduction over the axis (sum / prod / max / min / argmax / argmin, also all-axis) or a product that contracts it
    // computes the local part and combines the parts of all ranks (dalib200_allreduce), giving every rank the whole
    // result; argmax / argmin return indices of the logical array.  Indexing or slicing the axis, and gathering
    // from a sharded source, throw: a rank only holds its own rows.
    Array& set_shard(int axis, int64_t lo, int64_t total);
    Shard shard() const;
    // This rank's rows (dalib200_shard_range of the communicator's world and rank) of a C-contiguous host array of
    // shape `global_shape`, marked as a shard along axis 0.
    static Array scatter_rows(const void* host_data, const std::vector<int>& global_shape, DType dtype);

    // Optimise, lower and launch whatever this Array lazily stands for; afterwards it is a
    // plain buffer.  wait = true also synchronises the device.
    void eval(bool wait = true) const;

    static Array load(const std::string& fname);                 // .npy
    static Array load(FILE* fp);                                 // one array from the file's current position
    static void save(const std::string& fname, const Array& arr, const std::ios_base::openmode& mode = std::ios_base::out);
    static void save(std::basic_ostream<char>& stream, const Array& arr);

    static bool equals(const Array& left, const Array& right);
    static bool allclose(const Array& left, const Array& right, const double& atolerance);

    bool any_isnan() const;
    bool any_isinf() const;
    bool is_stateless() const;
    bool is_scalar() const;
    bool is_vector() const;
    bool is_matrix() const;
    Array ascontiguousarray() const;
    void initialize(const std::vector<int>& shape, DType dtype = DTYPE_FLOAT, memory::Device preferred_device = memory::default_preferred_device);
    Array& reset();

    const std::vector<int>& shape() const;
    std::shared_ptr<memory::SynchronizedMemory> memory() const;   // forces evaluation
    int offset() const;
    const std::vector<int>& strides() const;                       // empty = contiguous
    std::vector<int> normalized_strides() const;
    DType dtype() const;
    Array astype(DType dtype_) const;
    memory::Device preferred_device() const;
    void to_device(memory::Device device) const;

    int ndim() const;
    int number_of_elements() const;                                // throws above INT_MAX
    int64_t numel() const;                                         // 64-bit element count
    std::vector<int> subshape() const;
    bool contiguous_memory() const;
    bool spans_entire_memory() const;
    bool is_assignable() const;
    bool is_buffer() const;
    bool is_assignment() const;
    bool is_transpose() const;

    Array operator[](const int& idx) const;
    Array operator[](const Array& indices) const;
    SlicingInProgress<Array> operator[](const Slice& s) const;
    SlicingInProgress<Array> operator[](const Broadcast& b) const;
    Array gather_from_rows(const Array& indices) const;
    Array operator()(int idx) const;
    Array transpose() const;
    Array transpose(const std::vector<int>& axes) const;
    Array swapaxes(int axis1, int axis2) const;
    Array dimshuffle(const std::vector<int>& pattern) const;
    Array ravel() const;
    Array reshape(const std::vector<int>& shape) const;
    Array broadcast_to_shape(const std::vector<int>& shape) const;
    Array pluck_axis(int axis, const Slice& slice) const;
    Array pluck_axis(const int& axis, const int& idx) const;
    Array squeeze(int axis) const;
    Array expand_dims(int new_axis) const;
    Array broadcast_scalar_to_ndim(const int& ndim) const;
    Array right_fit_ndim(int dimensionality) const;

    Array sum() const;
    Array mean() const;
    Array min() const;
    Array max() const;
    Array L2_norm() const;
    Array abs() const;
    Array exp() const;
    Array tanh() const;
    Array sigmoid() const;
    Array sum(const std::vector<int>& axes, bool keepdims = false) const;
    Array mean(const std::vector<int>& axes, bool keepdims = false) const;
    Array min(const std::vector<int>& axes, bool keepdims = false) const;
    Array max(const std::vector<int>& axes, bool keepdims = false) const;
    Array L2_norm(const std::vector<int>& axes, bool keepdims = false) const;
    Array argmin(const int& axis) const;
    Array argmin() const;
    Array argmax(const int& axis) const;
    Array argmax() const;

    operator float() const;
    operator double() const;
    operator int() const;

    void copy_from(const Array& other);
    Array& operator=(const int& other);
    Array& operator=(const float& other);
    Array& operator=(const double& other);
    Array& assign(const Array& other);

    void print(std::basic_ostream<char>& stream = std::cout, const int& indent = 0, const bool& add_newlines = true,
               const bool& print_comma = false) const;
    void clear();
    Array dot(const Array& other) const;
    Array operator-() const;
};
bool operator==(const Array& left, const Array& right);

// (the Array&& forms take a right-hand side that is a temporary: an unnamed expression is fused into the update,
// a named lazy value is evaluated in place first -- see array.cc:inplace)
#define DALI_DECLARE_ARRAY_INTERACTION_INPLACE(SYMBOL) \
    Array& operator SYMBOL(Array& left, const Array& right); \
    Array& operator SYMBOL(Array& left, Array&& right); \
    void operator SYMBOL(Array&& left, const Array& right); \
    void operator SYMBOL(Array&& left, Array&& right);
DALI_DECLARE_ARRAY_INTERACTION_INPLACE(+=)
DALI_DECLARE_ARRAY_INTERACTION_INPLACE(-=)
DALI_DECLARE_ARRAY_INTERACTION_INPLACE(*=)
DALI_DECLARE_ARRAY_INTERACTION_INPLACE(/=)
DALI_DECLARE_ARRAY_INTERACTION_INPLACE(<<=)

#define DALI_DECLARE_ARRAY_INTERACTION(SYMBOL) \
    Array operator SYMBOL(const Array& left, const Array& right); \
    Array operator SYMBOL(const Array& left, double right); \
    Array operator SYMBOL(const Array& left, float right); \
    Array operator SYMBOL(const Array& left, int right); \
    Array operator SYMBOL(double left, const Array& right); \
    Array operator SYMBOL(float left, const Array& right); \
    Array operator SYMBOL(int left, const Array& right);
DALI_DECLARE_ARRAY_INTERACTION(+)
DALI_DECLARE_ARRAY_INTERACTION(-)
DALI_DECLARE_ARRAY_INTERACTION(*)
DALI_DECLARE_ARRAY_INTERACTION(/)

DType type_promotion(const Array& a, const Array& b);
memory::Device device_promotion(const Array& a, const Array& b);

// a[Slice(..)][Broadcast()][3] collects its steps and applies them when converted back
template <typename Container>
struct SlicingInProgress {
  private:
    enum SliceAction { SLICE_RANGE, SLICE_IDX, BROADCAST };
    int consumed_dims;
    std::vector<Slice> slice;
    std::vector<SliceAction> action;
    Container input;
  public:
    SlicingInProgress() : consumed_dims(0) {}
    SlicingInProgress(const Container& input_) : consumed_dims(0), input(input_) {}
    SlicingInProgress<Container> operator[](const Slice& s) const {
        if (consumed_dims >= input.ndim()) throw std::runtime_error("Slicing a scalar container is not allowed.");
        SlicingInProgress<Container> res(*this);
        res.slice.push_back(s);
        res.action.push_back(SLICE_RANGE);
        res.consumed_dims += 1;
        return res;
    }
    SlicingInProgress<Container> operator[](const Broadcast&) const {
        SlicingInProgress<Container> res(*this);
        res.action.push_back(BROADCAST);
        return res;
    }
    SlicingInProgress<Container> operator[](const int& idx) const {
        if (consumed_dims >= input.ndim()) throw std::runtime_error("Slicing a scalar container is not allowed.");
        SlicingInProgress<Container> res(*this);
        res.slice.push_back(Slice(idx, idx + 1));
        res.action.push_back(SLICE_IDX);
        res.consumed_dims += 1;
        return res;
    }
    operator Container() const {
        Container out = input;
        int slice_pos = 0, dim = 0;
        for (size_t i = 0; i < action.size(); ++i) {
            if (action[i] == SLICE_RANGE) {
                out = out.pluck_axis(dim, slice[slice_pos++]);
                dim += 1;
            } else if (action[i] == SLICE_IDX) {
                out = out.pluck_axis(dim, slice[slice_pos++].start);
            } else {
                out = out.expand_dims(dim);
                dim += 1;
            }
        }
        return out;
    }
    Container assign(const Container& other) { Container c = *this; return c.assign(other); }
};

#endif
