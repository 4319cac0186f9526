// Expression graph behind the lazy Array front end.
//
// Plays the part of dali/array/expression/{expression,buffer,assignment}.h and
// of the JITNode family (dali/array/jit/jit.h:88-176) in the reference, with a
// different design: nodes carry no code generators.  A tree of these nodes is
// lowered as a whole (lower.cc) into one fused-expression IR program per
// kernel, where the reference asks every node for a C++ template snippet.
//
// Views of evaluated buffers are resolved at once into stride / offset algebra
// (as dali/array/expression/buffer.cpp:113-286 does); views of lazy nodes
// become a View node -- one affine index map that stands for the reference's
// ExpandDims / BroadcastedReshape / Squeeze / dimshuffle nodes
// (dali/array/jit/reshape.cpp:11-280) and folds into leaf strides at lowering,
// so a broadcast never forces a temporary.
#ifndef DALI_ARRAY_EXPRESSION_EXPRESSION_H
#define DALI_ARRAY_EXPRESSION_EXPRESSION_H

#include <memory>
#include <string>
#include <vector>

#include "dali/array/array.h"

enum NodeKind { N_BUFFER, N_SCALAR, N_ELEMENTWISE, N_REDUCE, N_VIEW, N_GATHER, N_GATHER_ROWS, N_MATMUL, N_ASSIGN, N_IOTA, N_SCAN };

class Expression {
  public:
    NodeKind kind_;
    std::vector<int> shape_;
    DType dtype_;
    std::vector<Array> arguments_;
    Shard shard_;          // which part of a logical array spread over the ranks this value is (shard.cc)

    Expression(NodeKind kind, const std::vector<int>& shape, DType dtype, const std::vector<Array>& arguments);
    virtual ~Expression() {}
    int ndim() const { return (int)shape_.size(); }
    int64_t numel() const {
        int64_t n = 1;
        for (int s : shape_) n *= s;
        return n;
    }
    virtual std::string name() const = 0;
    std::string full_name() const;
};

// A strided window into a SynchronizedMemory (strides empty = row-major contiguous).
struct BufferView : public Expression {
    std::shared_ptr<memory::SynchronizedMemory> memory_;
    int64_t offset_;
    std::vector<int> strides_;
    BufferView(std::shared_ptr<memory::SynchronizedMemory> memory, const std::vector<int>& shape, DType dtype,
               int64_t offset = 0, const std::vector<int>& strides = {});
    // freshly allocated, contiguous
    static std::shared_ptr<BufferView> create(const std::vector<int>& shape, DType dtype, memory::Device device);
    std::string name() const override { return "Buffer"; }
    std::vector<int> normalized_strides() const;
    bool contiguous() const;
};

// A scalar known on the host; becomes a run-time kernel argument, so its value
// is not part of the compiled kernel's key (dali/array/jit/scalar_view.cpp:15-71).
struct ScalarValue : public Expression {
    double value_;
    ScalarValue(double value, DType dtype) : Expression(N_SCALAR, {}, dtype, {}), value_(value) {}
    std::string name() const override { return "Scalar"; }
};

// value[i_0 .. i_{n-1}] = offset + sum_k i_k * strides[k], int32, no memory behind it.  One node
// stands for the reference's Arange (dali/array/op/arange.cpp:12-52) and for the index
// `query[k]` that its OneHot and Diag kernels compare against (one_hot.cpp:41-46,
// eye.cpp:33-38); being affine, it slices, transposes, broadcasts and reshapes for free.
struct Iota : public Expression {
    int64_t offset_;
    std::vector<int64_t> strides_;
    Iota(const std::vector<int>& shape, int64_t offset, const std::vector<int64_t>& strides)
        : Expression(N_IOTA, shape, DTYPE_INT32, {}), offset_(offset), strides_(strides) {}
    std::string name() const override { return "Iota"; }
    // offset + s * (row-major linear index)?  Then any reshape is again an Iota.
    bool linear(int64_t* step) const;
};

// Running reduction along the last dim (dali/array/op/scan.cpp:19-180): inclusive keeps the
// shape; exclusive starts with the reducer's neutral element and is one longer.
struct Scan : public Expression {
    std::string reducer_;   // sum | prod | max | min
    bool inclusive_;
    Scan(const Array& a, const std::string& reducer, bool inclusive);
    std::string name() const override { return std::string(inclusive_ ? "inclusive_" : "exclusive_") + "scan_" + reducer_; }
};

// functor(arg0[, arg1]); rank-0 arguments broadcast implicitly.
struct Elementwise : public Expression {
    std::string functor_;   // name without the "functor::" prefix
    Elementwise(const std::string& functor, const std::vector<Array>& args, const std::vector<int>& shape, DType dtype)
        : Expression(N_ELEMENTWISE, shape, dtype, args), functor_(functor) {}
    std::string name() const override { return functor_; }
};

// Folds the innermost `nreduce` dims of its argument (all of them for an
// all-axis reduction).  arg_ = true yields the int32 position of the extreme.
struct Reduce : public Expression {
    std::string reducer_;   // sum | prod | max | min
    int nreduce_;
    bool arg_;
    // the folded dims include the sharded one: the local result is a partial one and the ranks' partials are combined
    // (all_reduce; for arg_ the (value, index) pairs, xrank_offset_ being what makes a local flat index a global one)
    bool xrank_ = false;
    int64_t xrank_offset_ = 0;
    Reduce(const std::string& reducer, const Array& a, int nreduce, bool arg, DType dtype);
    std::string name() const override { return (arg_ ? "arg" : "") + reducer_; }
};

// out[i_0 .. i_{n-1}] = arg[ off_k + step_k * i_{src_k} ]  (src_k = -1: constant off_k)
struct ViewDim { int src; int64_t off; int64_t step; };
struct View : public Expression {
    std::vector<ViewDim> dims_;    // one per dim of the argument
    View(const Array& a, const std::vector<int>& shape, const std::vector<ViewDim>& dims);
    std::string name() const override { return "View"; }
};

// out[i..., j...] = source[indices[i...], j...]
struct Gather : public Expression {
    Gather(const Array& source, const Array& indices);
    std::string name() const override { return "Gather"; }
};
// out[i, j...] = source[i, indices[i], j...]
struct GatherFromRows : public Expression {
    GatherFromRows(const Array& source, const Array& indices);
    std::string name() const override { return "GatherFromRows"; }
};

struct MatMul : public Expression {
    // the contracted dim is the sharded one (left cut along its columns, right along its rows): the local product is
    // a partial sum and the ranks' partial products are added (the "GEMM reduce")
    bool partial_ = false;
    MatMul(const Array& left, const Array& right);
    std::string name() const override { return "MatMul"; }
};

// dest <op>= value; dest is a buffer view or a Gather / GatherFromRows of one (scatter).
struct Assignment : public Expression {
    OPERATOR_T operator_t_;
    Assignment(const Array& dest, OPERATOR_T op, const Array& value);
    std::string name() const override { return "Assignment"; }
};

template <typename T> inline T* as(const Array& a) { return dynamic_cast<T*>(a.expression().get()); }

// ---- evaluation (lower.cc) ---------------------------------------------------------
namespace lazy {
// Runs dest <op>= value as one or more fused kernels (temporaries only where a
// subtree cannot share the root's iteration space) on dest's device.
void run_assignment(const Array& dest, OPERATOR_T op, const Array& value);
// dest when it is a buffer (or a scatter); for a view of a lazy value: that value evaluated into a buffer (all
// handles that share its state see the buffer from now on) and the same view of the buffer (array.cc)
Array writable_view(const Array& dest);
// evaluates, in place, every lazy value below `value` that a second handle names
void evaluate_shared_values(const Array& value);
// Evaluates several lazy arrays of one shape in one kernel where their trees allow it (an extension: the
// reference evaluates one Array per kernel); otherwise one after the other.  Does not synchronise.
void eval_together(const std::vector<Array>& arrays);
// Number of kernels / GEMMs launched by this thread's evaluations so far, and the
// description of the last fused kernel (for tests, in the spirit of the scope
// counting in dali/array/tests/dot_tests.cpp:17-35).
struct Stats { long long kernels = 0, gemms = 0, temporaries = 0, collectives = 0; std::string last_ir, last_variant, last_collective; };
Stats& stats();
// Dry run (per thread): expressions are lowered, registered and compiled through NVRTC,
// but nothing is allocated, copied or launched and results are undefined.  For
// inspecting what fuses on a machine without a GPU.
void set_dry_run(bool on);
bool dry_run();
void ensure_backend();    // dalib200_init once; throws std::runtime_error without a GPU
int device_index(const memory::Device& d);
void check(int status, const char* what);
// ---- sharding rules (shard.cc)
Shard shard_of_same_rank(const std::vector<Array>& arguments, int ndim, const std::string& what);
Shard shard_through_view(const Shard& s, const std::vector<int>& arg_shape, const std::vector<ViewDim>& dims,
                         const std::vector<int>& out_shape);
Shard shard_through_reshape(const Shard& s, const std::vector<int>& from, const std::vector<int>& to);
// number of elements of the logical array `a` is a part of
int64_t global_numel(const Array& a);
}  // namespace lazy

#define DALI_ASSERT(cond, msg)                                                   \
    do {                                                                         \
        if (!(cond)) throw std::runtime_error(std::string(msg));                 \
    } while (0)

#endif
