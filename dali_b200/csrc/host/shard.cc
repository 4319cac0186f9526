// Sharding rules of the lazy front end: which part of a logical array, spread over the ranks of the
// communicator (include/dali_b200.h, "ranks and collectives"), every value is.
//
// The reference decides per node where it runs from where its arguments happen to live
// (dali/array/jit/jit.cpp:367-385, array.cpp:867-872 device_promotion) and cannot combine data of two GPUs
// (dali/array/memory/memory_ops.cu.cpp:120-125).  Here a buffer is declared a shard along one axis
// (Array::set_shard) and the mark travels with every value derived from it; only a reduction over that axis or
// a product that contracts it needs the other ranks, and lower.cc appends the combine there.
#include <algorithm>
#include <cstring>

#include "../../../include/dali_b200.h"
#include "dali/array/expression/expression.h"

Expression::Expression(NodeKind kind, const std::vector<int>& shape, DType dtype, const std::vector<Array>& arguments)
    : kind_(kind), shape_(shape), dtype_(dtype), arguments_(arguments) {
    // same-rank operands of an elementwise node (and the operand of a running reduction) hand their mark on;
    // every other kind states its own rule in its constructor
    if (kind == N_ELEMENTWISE || kind == N_SCAN) shard_ = lazy::shard_of_same_rank(arguments, (int)shape.size(), "operation");
}

View::View(const Array& a, const std::vector<int>& shape, const std::vector<ViewDim>& dims)
    : Expression(N_VIEW, shape, a.dtype(), {a}), dims_(dims) {
    shard_ = lazy::shard_through_view(a.shard(), a.shape(), dims, shape);
}

Assignment::Assignment(const Array& dest, OPERATOR_T op, const Array& value)
    : Expression(N_ASSIGN, dest.shape(), dest.dtype(), {dest, value}), operator_t_(op) {
    shard_ = dest.shard();
}

Reduce::Reduce(const std::string& reducer, const Array& a, int nreduce, bool arg, DType dtype)
    : Expression(N_REDUCE, std::vector<int>(a.shape().begin(), a.shape().end() - nreduce), dtype, {a}),
      reducer_(reducer), nreduce_(nreduce), arg_(arg) {
    const Shard s = a.shard();
    if (!s.sharded()) return;
    const int lead = a.ndim() - nreduce;
    if (s.axis < lead) { shard_ = s; return; }       // a kept dim: every rank reduces its own rows
    xrank_ = true;
    // position in the flattened reduced dims of the logical array = local position + lo * (extent of the dims after the axis)
    xrank_offset_ = s.lo;
    for (int d = s.axis + 1; d < a.ndim(); ++d) xrank_offset_ *= a.shape()[d];
}

namespace lazy {

Shard shard_of_same_rank(const std::vector<Array>& arguments, int ndim, const std::string& what) {
    Shard out;
    for (const Array& a : arguments) {
        if (a.is_stateless() || a.ndim() != ndim) continue;
        const Shard s = a.shard();
        if (!s.sharded()) continue;
        if (!out.sharded()) { out = s; continue; }
        DALI_ASSERT(out == s, what + ": operands are sharded differently (axis " + std::to_string(out.axis) + " from " +
                                  std::to_string(out.lo) + " of " + std::to_string(out.total) + " against axis " +
                                  std::to_string(s.axis) + " from " + std::to_string(s.lo) + " of " + std::to_string(s.total) + ")");
    }
    return out;
}

Shard shard_through_view(const Shard& s, const std::vector<int>& arg_shape, const std::vector<ViewDim>& dims,
                         const std::vector<int>& out_shape) {
    if (!s.sharded()) return Shard();
    const ViewDim& d = dims[s.axis];
    DALI_ASSERT(d.src >= 0, "cannot index into the sharded axis: a rank holds only its own part of it");
    DALI_ASSERT(d.step == 1 && d.off == 0 && out_shape[d.src] == arg_shape[s.axis],
                "cannot slice the sharded axis: a rank holds only its own part of it");
    return Shard(d.src, s.lo, s.total);
}

Shard shard_through_reshape(const Shard& s, const std::vector<int>& from, const std::vector<int>& to) {
    if (!s.sharded()) return Shard();
    // the dims in front of the axis and the axis itself are kept ...
    int64_t before = 1;
    for (int d = 0; d < s.axis; ++d) before *= from[d];
    int64_t acc = 1;
    for (int j = 0; j < (int)to.size(); ++j) {
        if (acc == before && to[j] == from[s.axis]) return Shard(j, s.lo, s.total);
        acc *= to[j];
        if (acc > before) break;
    }
    // ... or the leading (sharded) dim absorbs the dims that follow it: [rows, cols] -> [rows * cols]
    if (s.axis == 0 && !to.empty() && from[0] > 0 && to[0] % from[0] == 0) {
        const int64_t f = to[0] / from[0];
        return Shard(0, s.lo * f, s.total * f);
    }
    throw std::runtime_error("reshape would split or move the sharded axis");
}

int64_t global_numel(const Array& a) {
    const Shard s = a.shard();
    int64_t n = a.numel();
    if (s.sharded() && a.shape()[s.axis] > 0) n = n / a.shape()[s.axis] * s.total;
    return n;
}

}  // namespace lazy

Shard Array::shard() const {
    if (is_stateless()) return Shard();
    return expression()->shard_;
}

Array& Array::set_shard(int axis, int64_t lo, int64_t total) {
    DALI_ASSERT(!is_stateless(), "set_shard on a stateless Array");
    if (!is_buffer()) eval(false);
    if (axis < 0) { expression()->shard_ = Shard(); return *this; }
    DALI_ASSERT(axis < ndim(), "set_shard: axis " + std::to_string(axis) + " out of range for an array of rank " + std::to_string(ndim()));
    DALI_ASSERT(lo >= 0 && lo + shape()[axis] <= total,
                "set_shard: rows [" + std::to_string(lo) + ", " + std::to_string(lo + shape()[axis]) + ") do not lie inside [0, " + std::to_string(total) + ")");
    expression()->shard_ = Shard(axis, lo, total);
    return *this;
}

Array Array::scatter_rows(const void* host_data, const std::vector<int>& global_shape, DType dtype) {
    DALI_ASSERT(!global_shape.empty(), "scatter_rows needs an array of rank >= 1");
    const int world = std::max(1, dalib200_comm_world());
    const int rank = std::max(0, dalib200_comm_rank());
    int64_t lo = 0, hi = 0;
    lazy::check(dalib200_shard_range(global_shape[0], rank, world, &lo, &hi), "dalib200_shard_range");
    std::vector<int> local = global_shape;
    local[0] = (int)(hi - lo);
    int64_t row = size_of_dtype(dtype);
    for (size_t d = 1; d < global_shape.size(); ++d) row *= global_shape[d];
    Array out(local, dtype);
    if (hi > lo) {
        void* dst = out.memory()->data(memory::Device::cpu(), memory::AM_OVERWRITE);
        std::memcpy(dst, static_cast<const char*>(host_data) + lo * row, (size_t)((hi - lo) * row));
    }
    out.set_shard(0, lo, global_shape[0]);
    return out;
}
