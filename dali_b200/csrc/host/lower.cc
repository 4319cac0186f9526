// Lowering of lazy expression trees to fused kernels.
//
// Stands where canonical() + jit_merge + JITRunnerImpl::run stand in the
// reference (dali/array/expression/optimization.cpp:151-158,
// dali/array/jit/jit.cpp:1080-1142 and :1144-1225): it decides what fuses into
// one kernel, numbers the distinct buffers and scalars in first-visit order,
// derives the structural key, compiles on first use and launches.  Differences
// by design:
//   * a whole assignment -- elementwise work, broadcasts, reductions over the
//     trailing dims and the elementwise work after them -- becomes ONE
//     fused-expression IR program (dali_b200/csrc/ir.h); the reference splits
//     the same tree into one loop nest per reduction / broadcast with a
//     temporary between them (dali/array/jit/reshape.cpp:100-102);
//   * views of lazy nodes are affine index maps that fold into leaf strides;
//   * temporaries appear only where a subtree cannot share the root's
//     iteration space (a reduction over other dims, a MatMul, a gather from a
//     lazy source): that subtree is evaluated first, by the same machinery.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <unordered_map>
#include <set>
#include <sstream>

#include "../../../include/dali_b200.h"
#include "../runtime.h"
#include "dali/array/op.h"
#include "dali/array/expression/expression.h"
#include "dali/utils/scope.h"

namespace lazy {

static thread_local Stats tl_stats;
static thread_local bool tl_dry_run = false;
Stats& stats() { return tl_stats; }
void set_dry_run(bool on) { tl_dry_run = on; }
bool dry_run() { return tl_dry_run; }

void check(int status, const char* what) {
    if (status == DALIB200_OK) return;
    char buf[8192];
    dalib200_last_error(buf, sizeof buf);
    throw std::runtime_error(std::string(what) + " failed (status " + std::to_string(status) + "): " + buf);
}

void ensure_backend() {
    static bool ready = false;
    if (ready) return;
    check(dalib200_init(0), "dalib200_init");
    ready = true;
}

int device_index(const memory::Device& d) {
    DALI_ASSERT(d.is_gpu(), "computation needs a GPU device (there is no CPU compute path)");
    ensure_backend();
    DALI_ASSERT(d.number() >= 0 && d.number() < dalib200_device_count(), "GPU " + std::to_string(d.number()) + " is not available");
    return d.number();
}

}  // namespace lazy

namespace dalib { const void* comm_peer_table(int device); }

namespace lazy {
namespace {

// The node whose cross-rank combine the caller appends itself (a sharded reduction or a product over the sharded
// dimension at the root of an assignment): it is lowered like a local one.
thread_local const Expression* tl_local_only = nullptr;

bool needs_combine(const Expression* e) {
    if (!e || e == tl_local_only) return false;
    if (e->kind_ == N_REDUCE) return static_cast<const Reduce*>(e)->xrank_;
    if (e->kind_ == N_MATMUL) return static_cast<const MatMul*>(e)->partial_;
    return false;
}

bool contains_reduce(const Array& a, int depth = 0) {
    if (a.is_stateless() || depth > 64) return false;
    const Expression* e = a.expression().get();
    if (e->kind_ == N_REDUCE) return true;
    if (e->kind_ == N_BUFFER || e->kind_ == N_SCALAR || e->kind_ == N_IOTA) return false;
    for (const Array& arg : e->arguments_) if (contains_reduce(arg, depth + 1)) return true;
    return false;
}

// Can the partial results of this sharded reduction meet INSIDE the kernel that computes them?  Yes for an
// all-axis reduction of purely elementwise work when the ranks' exchange blocks are mapped into one another
// (transport "nccl+peer", or a world of one): the kernel's last CTA stores its partial into every rank's block,
// waits -- bounded -- for theirs and folds them in rank order.  Otherwise the local kernel is followed by
// dalib200_allreduce on its result.
bool xrank_fusable(const Reduce* r, const memory::Device& device) {
    if (r->nreduce_ != r->arguments_[0].ndim() || contains_reduce(r->arguments_[0])) return false;
    const char* off = std::getenv("DALI_B200_XRANK_FUSE");
    if (off && off[0] == '0') return false;
    if (tl_dry_run) { const char* e = std::getenv("DALI_B200_DRYRUN_PEER"); return e && e[0] == '1'; }
    return device.is_gpu() && dalib::comm_peer_table(device.number()) != nullptr;
}

const char* reducer_name_of(int op) { return op == DALIB200_OP_SUM ? "sum" : op == DALIB200_OP_PROD ? "prod" : op == DALIB200_OP_MAX ? "max" : "min"; }
int reducer_op(const std::string& r) { return r == "sum" ? DALIB200_OP_SUM : r == "prod" ? DALIB200_OP_PROD : r == "max" ? DALIB200_OP_MAX : DALIB200_OP_MIN; }

void note_collective(const std::string& what) {
    ++tl_stats.collectives;
    tl_stats.last_collective = what;
}

// IR type names: of VALUES (bf16 is a storage type: a value read from a bf16 array is an f32) and of ARGS
const char* ir_dtype(DType d) { return d == DTYPE_FLOAT || d == DTYPE_BF16 ? "f32" : (d == DTYPE_DOUBLE ? "f64" : "i32"); }
const char* ir_arg_dtype(DType d) { return d == DTYPE_BF16 ? "bf16" : ir_dtype(d); }
const char* ir_assign(OPERATOR_T op) {
    switch (op) {
        case OPERATOR_T_ADD: return "add";
        case OPERATOR_T_SUB: return "sub";
        case OPERATOR_T_MUL: return "mul";
        case OPERATOR_T_DIV: return "div";
        default: return "assign";
    }
}

// node dim j = off + mult * space[src]   (src = -1: the constant `off`)
struct DimMap { int src; int64_t mult; int64_t off; };
typedef std::vector<DimMap> IndexMap;

IndexMap identity_map(int n) {
    IndexMap m(n);
    for (int j = 0; j < n; ++j) m[j] = DimMap{j, 1, 0};
    return m;
}

std::string map_key(const IndexMap& m) {
    std::ostringstream o;
    for (const DimMap& d : m) o << d.src << ":" << d.mult << ":" << d.off << ",";
    return o.str();
}

struct Leaf {
    std::shared_ptr<memory::SynchronizedMemory> memory;
    DType dtype;
    int64_t offset;                   // elements
    std::vector<int64_t> strides;     // `rank` space strides (+ 1 lead stride when indirect)
    bool elem_level, written, read, indirect;
    bool iota = false;                // no memory: the value is offset + sum(index * stride)
};

struct Lowerer {
    std::vector<int64_t> space;
    int rank, nreduce, n_outer;
    memory::Device device;
    std::vector<std::string> body;
    std::vector<DType> types;            // per value
    std::vector<bool> elem;              // per value: varies over the reduced dims?
    std::vector<Leaf> leaves;
    std::vector<std::pair<DType, double>> scalars;
    // keyed by node address: every node that has an entry is kept alive in `memo_nodes`, or a node created
    // later (a temporary's buffer) could reuse the address of one that died during lowering and hit its entry
    std::map<std::pair<const Expression*, std::string>, int> memo;
    std::vector<expression_ptr> memo_nodes;
    std::map<const Expression*, int> scalar_slot;
    std::vector<Array> keep_alive;
    // the node whose value is the GEMM accumulator (epilogue programs): a MatMul, or the sum of two of them
    const Expression* acc_node = nullptr;
    // > 0: the program's space is [m, slice_width] and the accumulator node, seen through a column slice that
    // starts at q * slice_width, is the value `acc q` (gating over the four gate blocks of an LSTM product)
    int64_t slice_width = 0;
    std::set<int> slices_seen;
    bool slice_fail = false;

    Lowerer(const std::vector<int64_t>& space_, int nreduce_, memory::Device dev)
        : space(space_), rank((int)space_.size()), nreduce(nreduce_), n_outer(rank - nreduce_), device(dev) {}

    int new_value(DType t, bool is_elem, const std::string& text) {
        int id = (int)types.size();
        t = value_dtype(t);
        types.push_back(t);
        elem.push_back(is_elem);
        body.push_back("v" + std::to_string(id) + " " + ir_dtype(t) + " " + text);
        return id;
    }

    // leaf strides of a buffer seen through map m
    int leaf_for(BufferView* b, const IndexMap& m, bool written, bool indirect, int64_t lead_stride, int skip_dims_from,
                 int skip_count) {
        std::vector<int> st = b->normalized_strides();
        Leaf L;
        L.memory = b->memory_;
        L.dtype = b->dtype_;
        L.offset = b->offset_;
        L.strides.assign(rank, 0);
        L.indirect = indirect;
        int mj = 0;
        for (int k = 0; k < (int)st.size(); ++k) {
            if (k >= skip_dims_from && k < skip_dims_from + skip_count) continue;   // dim addressed through the index
            const DimMap& d = m[mj++];
            L.offset += d.off * st[k];
            if (d.src >= 0) L.strides[d.src] += d.mult * st[k];
        }
        for (int d = 0; d < rank; ++d) if (space[d] == 1) L.strides[d] = 0;
        L.elem_level = nreduce == 0;
        for (int d = n_outer; d < rank; ++d) if (L.strides[d] != 0) L.elem_level = true;
        if (indirect) L.strides.push_back(lead_stride);
        L.written = written;
        L.read = !written;
        for (size_t i = 0; i < leaves.size(); ++i) {
            Leaf& o = leaves[i];
            if (o.memory == L.memory && o.dtype == L.dtype && o.offset == L.offset && o.strides == L.strides &&
                o.indirect == L.indirect && o.elem_level == L.elem_level) {
                o.written = o.written || written;
                o.read = o.read || !written;
                return (int)i;
            }
        }
        leaves.push_back(L);
        return (int)leaves.size() - 1;
    }

    static bool contains_matmul(const Array& a) {
        if (a.is_stateless()) return false;
        Expression* e = a.expression().get();
        if (e->kind_ == N_MATMUL) return true;
        if (e->kind_ != N_ELEMENTWISE) return false;
        for (const Array& arg : e->arguments_) if (contains_matmul(arg)) return true;
        return false;
    }

    Array materialize(const Array& a) {
        Array t(a.expression());
        t.eval(false);
        ++tl_stats.temporaries;
        // remember the result in the node's own handle too, so a second visit reuses it
        a.set_expression(t.expression());
        keep_alive.push_back(t);
        return t;
    }

    bool reduce_fits(const Reduce* r, const IndexMap& m) const {
        if (nreduce == 0 || r->nreduce_ != nreduce) return false;
        if (r->ndim() != n_outer) return false;
        for (int j = 0; j < r->ndim(); ++j)
            if (m[j].src != j || m[j].mult != 1 || m[j].off != 0) return false;
        const std::vector<int>& as_ = r->arguments_[0].shape();
        for (int k = 0; k < nreduce; ++k)
            if (as_[r->ndim() + k] != space[n_outer + k]) return false;
        for (int j = 0; j < n_outer; ++j)
            if (as_[j] != space[j]) return false;
        return true;
    }

    int visit(const Array& a, const IndexMap& m) {
        DALI_ASSERT(!a.is_stateless(), "expression refers to a stateless Array");
        expression_ptr e = a.expression();
        if (e->kind_ == N_ASSIGN) { a.eval(false); e = a.expression(); }
        DALI_ASSERT((int)m.size() == e->ndim(), "internal: index map rank mismatch at " + e->name());
        auto key = std::make_pair((const Expression*)e.get(), map_key(m));
        auto it = memo.find(key);
        if (it != memo.end()) return it->second;
        int id = -1;
        switch (e->kind_) {
            case N_BUFFER: {
                BufferView* b = static_cast<BufferView*>(e.get());
                int leaf = leaf_for(b, m, false, false, 0, 0, 0);
                keep_alive.push_back(a);
                id = new_value(b->dtype_, leaves[leaf].elem_level, "ld " + std::to_string(leaf));
                break;
            }
            case N_SCALAR: {
                ScalarValue* s = static_cast<ScalarValue*>(e.get());
                auto sit = scalar_slot.find(s);
                int slot;
                if (sit == scalar_slot.end()) {
                    slot = (int)scalars.size();
                    scalars.push_back(std::make_pair(s->dtype_, s->value_));
                    scalar_slot[s] = slot;
                    keep_alive.push_back(a);      // the slot map is keyed by the node's address too
                } else {
                    slot = sit->second;
                }
                id = new_value(s->dtype_, false, "sc " + std::to_string(slot));
                break;
            }
            case N_ELEMENTWISE: {
                Elementwise* w = static_cast<Elementwise*>(e.get());
                if (e.get() == acc_node) {
                    const std::string t = acc_text(m);
                    if (!t.empty()) { id = new_value(DTYPE_FLOAT, true, t); break; }
                }
                std::vector<int> in;
                bool is_elem = false;
                for (const Array& arg : w->arguments_) {
                    int v = arg.ndim() == 0 ? visit(arg, IndexMap()) : visit(arg, m);
                    in.push_back(v);
                    is_elem = is_elem || elem[v];
                }
                if (w->functor_ == "cast") {
                    id = new_value(w->dtype_, is_elem, "cast v" + std::to_string(in[0]));
                } else {
                    // operands are promoted to the node's type, except for the converting functors
                    bool converts = w->functor_ == "round" || w->functor_ == "ceiling" || w->functor_ == "rng_uniform" ||
                                    w->functor_ == "rng_normal";
                    std::string text = "op " + w->functor_;
                    for (int v : in) {
                        if (!converts && types[v] != value_dtype(w->dtype_)) v = new_value(w->dtype_, elem[v], "cast v" + std::to_string(v));
                        text += " v" + std::to_string(v);
                    }
                    id = new_value(w->dtype_, is_elem, text);
                }
                break;
            }
            case N_VIEW: {
                View* v = static_cast<View*>(e.get());
                const Array& arg = v->arguments_[0];
                // a slice / broadcast of something that contains a product: evaluate that something
                // once (GEMM with its elementwise surroundings as epilogue) and view the result
                // (unless the product is this program's accumulator and the view one of its column slices)
                if (contains_matmul(arg) && !(slice_width > 0 && acc_node && contains_node(arg, acc_node))) materialize(arg);
                IndexMap am(v->dims_.size());
                for (size_t k = 0; k < v->dims_.size(); ++k) {
                    const ViewDim& d = v->dims_[k];
                    if (d.src < 0) { am[k] = DimMap{-1, 0, d.off}; continue; }
                    const DimMap& o = m[d.src];
                    am[k] = DimMap{o.src, d.step * o.mult, d.off + d.step * o.off};
                    if (o.src < 0) am[k].mult = 0;
                }
                id = visit(arg, am);
                break;
            }
            case N_REDUCE: {
                Reduce* r = static_cast<Reduce*>(e.get());
                if (!reduce_fits(r, m)) {
                    id = visit(materialize(a), m);
                    break;
                }
                // a reduction over the sharded dimension: the ranks' partial results meet inside this kernel where
                // that is possible (see xrank_fusable), else it is evaluated on its own and combined after its kernel
                const bool combine = needs_combine(r);
                if (combine && !xrank_fusable(r, device)) {
                    id = visit(materialize(a), m);
                    break;
                }
                int v = visit(r->arguments_[0], identity_map(rank));
                std::string x = combine ? " xrank" : "";
                if (combine && r->arg_) {
                    // the local position becomes a position in the logical array before the pairs are exchanged
                    const int slot = (int)scalars.size();
                    scalars.push_back(std::make_pair(DTYPE_INT32, (double)r->xrank_offset_));
                    x += " v" + std::to_string(new_value(DTYPE_INT32, false, "sc " + std::to_string(slot)));
                }
                if (combine) note_collective(std::string("in-kernel ") + (r->arg_ ? "arg" : "") + r->reducer_);
                if (r->arg_) id = new_value(DTYPE_INT32, false, "argred " + r->reducer_ + " v" + std::to_string(v) + x);
                else id = new_value(r->dtype_, false, "red " + r->reducer_ + " v" + std::to_string(v) + x);
                break;
            }
            case N_GATHER:
            case N_GATHER_ROWS: {
                const bool rows = e->kind_ == N_GATHER_ROWS;
                Array source = e->arguments_[0];
                const Array& indices = e->arguments_[1];
                if (!source.is_buffer()) source = materialize(source);
                BufferView* sb = as<BufferView>(source);
                keep_alive.push_back(source);
                const int ri = indices.ndim();
                IndexMap im(m.begin(), m.begin() + ri);
                int vi = visit(indices, im);
                std::vector<int> sst = sb->normalized_strides();
                // map for the source dims that are NOT addressed through the index
                IndexMap sm;
                if (rows) {
                    sm.push_back(m[0]);                                     // source dim 0 <- out dim 0
                    for (int t = 1; t < (int)m.size(); ++t) sm.push_back(m[t]);   // source dims 2.. <- out dims 1..
                } else {
                    for (int t = ri; t < (int)m.size(); ++t) sm.push_back(m[t]);  // source dims 1.. <- out dims ri..
                }
                int leaf = leaf_for(sb, sm, false, true, sst[rows ? 1 : 0], rows ? 1 : 0, 1);
                bool is_elem = elem[vi] || leaves[leaf].elem_level;
                id = new_value(sb->dtype_, is_elem, "ldx " + std::to_string(leaf) + " v" + std::to_string(vi));
                break;
            }
            case N_IOTA: {
                Iota* io = static_cast<Iota*>(e.get());
                Leaf L;
                L.dtype = DTYPE_INT32;
                L.offset = io->offset_;
                L.strides.assign(rank, 0);
                L.indirect = L.written = false;
                L.read = true;
                L.iota = true;
                for (int k = 0; k < io->ndim(); ++k) {
                    L.offset += m[k].off * io->strides_[k];
                    if (m[k].src >= 0) L.strides[m[k].src] += m[k].mult * io->strides_[k];
                }
                for (int d = 0; d < rank; ++d) if (space[d] == 1) L.strides[d] = 0;
                L.elem_level = nreduce == 0;
                for (int d = n_outer; d < rank; ++d) if (L.strides[d] != 0) L.elem_level = true;
                int leaf = -1;
                for (size_t i = 0; i < leaves.size() && leaf < 0; ++i)
                    if (leaves[i].iota && leaves[i].offset == L.offset && leaves[i].strides == L.strides) leaf = (int)i;
                if (leaf < 0) { leaves.push_back(L); leaf = (int)leaves.size() - 1; }
                id = new_value(DTYPE_INT32, leaves[leaf].elem_level, "ld " + std::to_string(leaf));
                break;
            }
            case N_SCAN:
                // never fused with what consumes it (dali/array/op/scan.cpp:37-39: chainable() is false)
                id = visit(materialize(a), m);
                break;
            case N_MATMUL: {
                const std::string t = e.get() == acc_node ? acc_text(m) : std::string();
                if (!t.empty()) id = new_value(DTYPE_FLOAT, true, t);
                else id = visit(materialize(a), m);
                break;
            }
            default:
                throw std::runtime_error("cannot lower expression node " + e->name());
        }
        memo[key] = id;
        memo_nodes.push_back(e);
        return id;
    }

    // the accumulator node reached through map m: "acc" / "acc q", or "" when m is not one the GEMM epilogue can serve
    std::string acc_text(const IndexMap& m) {
        if (is_identity(m) && slice_width == 0) return "acc";
        if (slice_width > 0 && (int)m.size() == 2 && m[0].src == 0 && m[0].mult == 1 && m[0].off == 0 && m[1].src == 1 &&
            m[1].mult == 1 && m[1].off >= 0 && m[1].off % slice_width == 0) {
            const int q = (int)(m[1].off / slice_width);
            slices_seen.insert(q);
            return q == 0 ? "acc" : "acc " + std::to_string(q);
        }
        if (slice_width > 0) slice_fail = true;
        return "";
    }

    static bool contains_node(const Array& a, const Expression* node) {
        if (a.is_stateless()) return false;
        Expression* e = a.expression().get();
        if (e == node) return true;
        if (e->kind_ != N_ELEMENTWISE) return false;
        for (const Array& arg : e->arguments_) if (contains_node(arg, node)) return true;
        return false;
    }

    static bool is_identity(const IndexMap& m) {
        return (int)m.size() == 2 && m[0].src == 0 && m[1].src == 1 && m[0].mult == 1 && m[1].mult == 1 && m[0].off == 0 &&
               m[1].off == 0;
    }

    std::string ir_text() const {
        std::ostringstream o;
        o << "dali-ir 1\nspace " << rank << " " << nreduce << "\n";
        for (size_t i = 0; i < leaves.size(); ++i)
            o << "arg " << i << " " << ir_arg_dtype(leaves[i].dtype) << " " << (leaves[i].elem_level || nreduce == 0 ? "E" : "R")
              << (leaves[i].iota ? " iota" : "") << "\n";
        for (size_t j = 0; j < scalars.size(); ++j) o << "scalar " << j << " " << ir_dtype(scalars[j].first) << "\n";
        for (const std::string& line : body) o << line << "\n";
        o << "end\n";
        return o.str();
    }

    void launch() {
        const std::string text = ir_text();
        const uint64_t hash = dalib::fnv1a(text);
        {
            DALI_SCOPE("get_function");        // as the reference's compile-or-load step (dali/array/jit/jit.cpp:1015)
            if (!dalib200_is_loaded(hash)) check(dalib200_compile(hash, text.c_str(), text.size()), "dalib200_compile");
        }
        const int n = (int)leaves.size();
        if (tl_dry_run) {
            // lower + compile only: aligned stand-in pointers, nothing touches a device
            std::vector<void*> fake(n);
            std::vector<int64_t> offs(n);
            std::vector<const int64_t*> st(n);
            for (int i = 0; i < n; ++i) { fake[i] = (void*)(uintptr_t)4096; offs[i] = leaves[i].offset; st[i] = leaves[i].strides.data(); }
            check(dalib200_precompile(hash, space.data(), rank, fake.data(), offs.data(), st.data(), n, nullptr), "dalib200_precompile");
            ++tl_stats.kernels;
            tl_stats.last_ir = text;
            char vbuf[512];
            dalib200_last_variant(vbuf, sizeof vbuf);
            tl_stats.last_variant = vbuf;
            return;
        }
        const int dev = device_index(device);
        std::vector<void*> ptrs(n);
        std::vector<int64_t> offsets(n);
        std::vector<const int64_t*> strides(n);
        // readers first, writers last, so the freshness flags end up describing the result
        for (int pass = 0; pass < 2; ++pass)
            for (int i = 0; i < n; ++i) {
                if ((pass == 1) != leaves[i].written) continue;
                ptrs[i] = leaves[i].iota ? nullptr
                                         : leaves[i].memory->data(device, leaves[i].written ? memory::AM_MUTABLE : memory::AM_READONLY);
                offsets[i] = leaves[i].offset;
                strides[i] = leaves[i].strides.data();
            }
        std::vector<double> sd(scalars.size());
        std::vector<float> sf(scalars.size());
        std::vector<int> si(scalars.size());
        std::vector<const void*> sp(scalars.size());
        for (size_t j = 0; j < scalars.size(); ++j) {
            sd[j] = scalars[j].second;
            sf[j] = (float)scalars[j].second;
            si[j] = (int)scalars[j].second;
            sp[j] = scalars[j].first == DTYPE_DOUBLE ? (const void*)&sd[j]
                                                    : (scalars[j].first == DTYPE_FLOAT ? (const void*)&sf[j] : (const void*)&si[j]);
        }
        check(dalib200_launch(hash, dev, nullptr, space.data(), rank, ptrs.data(), offsets.data(), strides.data(), n,
                              sp.data(), (int)sp.size()),
              "dalib200_launch");
        ++tl_stats.kernels;
        tl_stats.last_ir = text;
        char buf[512];
        dalib200_last_variant(buf, sizeof buf);
        tl_stats.last_variant = buf;
    }
};

// last MatMul reachable from `a` through elementwise nodes only
void find_matmul(const Array& a, const Expression** out) {
    if (a.is_stateless()) return;
    Expression* e = a.expression().get();
    if (e->kind_ == N_MATMUL) { *out = e; return; }
    if (e->kind_ != N_ELEMENTWISE) return;
    for (const Array& arg : e->arguments_) find_matmul(arg, out);
}

// add(MatMul, MatMul) of fp32 products reachable the same way: both accumulate in one GEMM launch
void find_matmul_sum(const Array& a, const Expression** out) {
    if (*out || a.is_stateless()) return;
    Expression* e = a.expression().get();
    if (e->kind_ != N_ELEMENTWISE) return;
    Elementwise* w = static_cast<Elementwise*>(e);
    if (w->functor_ == "add" && w->arguments_.size() == 2 && w->dtype_ == DTYPE_FLOAT) {
        const Array &l = w->arguments_[0], &r = w->arguments_[1];
        if (!l.is_stateless() && !r.is_stateless() && l.expression()->kind_ == N_MATMUL && r.expression()->kind_ == N_MATMUL &&
            l.dtype() == DTYPE_FLOAT && r.dtype() == DTYPE_FLOAT && l.shape() == r.shape() && l.shape() == w->shape_) {
            *out = e;
            return;
        }
    }
    for (const Array& arg : e->arguments_) find_matmul_sum(arg, out);
}

// TF32 split parts of an fp32 matrix, kept next to the buffer until it is written again
struct SplitParts {
    int device = 0;
    size_t bytes = 0;
    int64_t offset = 0, rows = 0, cols = 0, ld = 0;
    bool transposed = false;
    void *hi = nullptr, *lo = nullptr;
    std::shared_ptr<SplitParts> older;      // the split kept before this one: a weight matrix is read as W going forward and
                                            // as W^T going backward, and both splits stay valid while W does not change
    ~SplitParts() {
        if (hi) dalib200_free(device, hi, bytes);
        if (lo) dalib200_free(device, lo, bytes);
    }
};

// A split that has its (hi, lo) buffers but has not been launched yet: two of one shape go out as one launch.
struct PendingSplit { std::shared_ptr<SplitParts> parts; const float* x = nullptr; };

// returns the (hi, lo) parts of an fp32 matrix view as the GEMM wants them (row-major for a left operand, transposed
// for a right one); nullptr if the layout cannot be split in place.  The view is either row-contiguous or the pure
// transpose of a row-contiguous matrix (x.transpose() in a backward pass): the latter is split from the matrix
// underneath with the transposition flipped, so W^T as a right operand needs no transposition at all.
// With `pending` the split kernel of an operand that was not cached is left to the caller (launch_pending).
std::shared_ptr<SplitParts> split_operand(BufferView* b, bool transpose, memory::Device device, int dev,
                                          std::vector<PendingSplit>* pending = nullptr) {
    std::vector<int> st = b->normalized_strides();
    int64_t rows = b->shape_[0], cols = b->shape_[1], ld = st[0];
    if (st[1] != 1 && cols != 1) {
        if (st[0] != 1 && rows != 1) return nullptr;
        std::swap(rows, cols);          // the matrix underneath: [cols, rows] of the view, row pitch st[1]
        ld = st[1];
        transpose = !transpose;
    }
    if (ld < cols) return nullptr;      // (a broadcast row or column)
    if (cols % 4 || ld % 4 || (transpose && rows % 4) || (b->offset_ % 4)) return nullptr;
    auto& slot = b->memory_->derived_data();
    std::shared_ptr<SplitParts> previous;
    if (slot && b->memory_->derived_version() == b->memory_->version()) {
        previous = std::static_pointer_cast<SplitParts>(slot);
        for (std::shared_ptr<SplitParts> cached = previous; cached; cached = cached->older)
            if (cached->offset == b->offset_ && cached->rows == rows && cached->cols == cols && cached->ld == ld &&
                cached->transposed == transpose && cached->device == dev)
                return cached;
        previous->older.reset();            // two generations at most
    }
    const float* x = (const float*)b->memory_->data(device, memory::AM_READONLY) + b->offset_;
    if (((uintptr_t)x) & 15) return nullptr;
    auto parts = std::make_shared<SplitParts>();
    parts->device = dev;
    parts->bytes = (size_t)rows * cols * 4;
    parts->offset = b->offset_; parts->rows = rows; parts->cols = cols; parts->ld = ld; parts->transposed = transpose;
    check(dalib200_alloc(dev, parts->bytes, &parts->hi), "dalib200_alloc");
    check(dalib200_alloc(dev, parts->bytes, &parts->lo), "dalib200_alloc");
    if (pending && !transpose) {
        PendingSplit ps;
        ps.parts = parts;
        ps.x = x;
        pending->push_back(ps);
    } else {
        check(dalib200_gemm_split_tf32(dev, nullptr, x, rows, cols, ld, transpose ? 1 : 0, (float*)parts->hi, (float*)parts->lo),
              "dalib200_gemm_split_tf32");
    }
    parts->older = previous;                // (empty when the matrix has changed since)
    slot = parts;
    b->memory_->derived_version() = b->memory_->version();
    return parts;
}

void launch_pending(const std::vector<PendingSplit>& pending, int dev) {
    size_t i = 0;
    if (pending.size() == 2 && pending[0].parts->rows == pending[1].parts->rows && pending[0].parts->cols == pending[1].parts->cols) {
        const SplitParts &a = *pending[0].parts, &b = *pending[1].parts;
        check(dalib200_gemm_split_tf32_pair(dev, nullptr, pending[0].x, pending[1].x, a.rows, a.cols, a.ld, b.ld, (float*)a.hi,
                                            (float*)a.lo, (float*)b.hi, (float*)b.lo),
              "dalib200_gemm_split_tf32_pair");
        i = 2;
    }
    for (; i < pending.size(); ++i) {
        const SplitParts& a = *pending[i].parts;
        check(dalib200_gemm_split_tf32(dev, nullptr, pending[i].x, a.rows, a.cols, a.ld, 0, (float*)a.hi, (float*)a.lo),
              "dalib200_gemm_split_tf32");
    }
}

// a product (or one of the two of a sum) whose partial results still have to be added over the ranks: it cannot be
// the accumulator of a fused epilogue (the epilogue would run on a partial sum)
bool pending_partial(const Expression* acc) {
    if (!acc) return false;
    if (acc->kind_ == N_MATMUL) return needs_combine(acc);
    for (const Array& arg : acc->arguments_)
        if (!arg.is_stateless() && needs_combine(arg.expression().get())) return true;
    return false;
}

// first reduction reachable from `a` through elementwise nodes and views
struct FoundReduce { const Reduce* node = nullptr; bool through_view = false; };
void find_reduce(const Array& a, bool through_view, FoundReduce* out) {
    if (out->node || a.is_stateless()) return;
    Expression* e = a.expression().get();
    switch (e->kind_) {
        case N_REDUCE:
            out->node = static_cast<Reduce*>(e);
            out->through_view = through_view;
            return;
        case N_ELEMENTWISE:
            for (const Array& arg : e->arguments_) find_reduce(arg, through_view, out);
            return;
        case N_VIEW:
            find_reduce(e->arguments_[0], true, out);
            return;
        default:
            return;
    }
}

// nothing but elementwise nodes, views and leaves below `a`
bool only_elementwise(const Array& a) {
    if (a.is_stateless()) return true;
    Expression* e = a.expression().get();
    switch (e->kind_) {
        case N_BUFFER: case N_SCALAR: case N_IOTA: return true;
        case N_ELEMENTWISE: case N_VIEW:
            for (const Array& arg : e->arguments_) if (!only_elementwise(arg)) return false;
            return true;
        default: return false;
    }
}

// [first, last] element of the buffer that a view touches
static void view_span(const BufferView* b, int64_t* lo, int64_t* hi) {
    std::vector<int> st = b->normalized_strides();
    *lo = *hi = b->offset_;
    for (size_t d = 0; d < b->shape_.size(); ++d) {
        if (b->shape_[d] <= 0) { *hi = *lo - 1; return; }       // empty view
        const int64_t reach = (int64_t)(b->shape_[d] - 1) * st[d];
        if (reach < 0) *lo += reach; else *hi += reach;
    }
}
// Two views of one buffer whose element ranges intersect (a conservative test: interleaved views count as overlapping).
static bool views_may_overlap(const BufferView* x, const BufferView* y) {
    if (x->memory_ != y->memory_) return false;
    int64_t xl, xh, yl, yh;
    view_span(x, &xl, &xh);
    view_span(y, &yl, &yh);
    return xl <= yh && yl <= xh;
}
// Does a product below `a` (through elementwise nodes and views) read a buffer that `dest` is about to overwrite?
// A GEMM reads every operand element many times while other CTAs already store results: dest = dot(dest, w) must go
// through a temporary (the reference does not guard against it either; a numpy-like statement is well defined).
static bool product_reads_destination(const Array& a, const BufferView* dest) {
    if (a.is_stateless()) return false;
    Expression* e = a.expression().get();
    if (e->kind_ == N_MATMUL) {
        for (const Array& operand : e->arguments_) {
            if (BufferView* b = as<BufferView>(operand)) { if (views_may_overlap(b, dest)) return true; }
            else if (product_reads_destination(operand, dest)) return true;
        }
        return false;
    }
    if (e->kind_ != N_ELEMENTWISE && e->kind_ != N_VIEW) return false;
    for (const Array& arg : e->arguments_) if (product_reads_destination(arg, dest)) return true;
    return false;
}

// dest (op)= left . right through the GEMM entry point of the C ABI (reference:
// CublasGemmImpl::run, dali/array/gemm/cublas_gemm.cu:112-185, which ignores the
// operator and always overwrites; here += and -= accumulate as
// MatMul::supports_operator advertises, dali/array/op/dot.cpp:41-45).
void run_matmul(const Array& dest, OPERATOR_T op, MatMul* mm) {
    Array left = mm->arguments_[0], right = mm->arguments_[1];
    if (!left.is_buffer()) left.eval(false);
    if (!right.is_buffer()) right.eval(false);
    if (op == OPERATOR_T_MUL || op == OPERATOR_T_DIV) {
        Array tmp(dest.shape(), dest.dtype(), dest.preferred_device());
        run_matmul(tmp, OPERATOR_T_EQL, mm);
        run_assignment(dest, op, tmp);
        return;
    }
    DALI_ASSERT(left.dtype() != DTYPE_BF16 && right.dtype() != DTYPE_BF16 && dest.dtype() != DTYPE_BF16,
                "a bf16 product runs on the tensor cores only: both operands bf16, row-major with 16-byte aligned rows (no transposed or strided views)");
    DALI_ASSERT(dest.dtype() == left.dtype() && dest.dtype() == right.dtype(), "matmul operands and destination must share a dtype");
    BufferView* a = as<BufferView>(left);
    BufferView* b = as<BufferView>(right);
    BufferView* c = as<BufferView>(dest);
    if (views_may_overlap(a, c) || views_may_overlap(b, c)) {
        // the destination is one of the operands: product into a temporary, then the assignment
        Array tmp(dest.shape(), dest.dtype(), dest.preferred_device());
        Array product(std::make_shared<MatMul>(left, right));
        run_assignment(tmp, OPERATOR_T_EQL, product);
        run_assignment(dest, op, tmp);
        return;
    }
    const int64_t m = a->shape_[0], k = a->shape_[1], n = b->shape_[1];
    DALI_ASSERT(c->shape_.size() == 2 && c->shape_[0] == m && c->shape_[1] == n, "matmul destination has the wrong shape");
    if (m == 0 || n == 0) return;
    if (tl_dry_run) { ++tl_stats.gemms; return; }
    memory::Device device = dest.preferred_device();
    const int dev = device_index(device);
    std::vector<int> as_ = a->normalized_strides(), bs = b->normalized_strides(), cs = c->normalized_strides();
    const int item = size_of_dtype(dest.dtype());
    const char* pa = (const char*)a->memory_->data(device, memory::AM_READONLY) + a->offset_ * item;
    const char* pb = (const char*)b->memory_->data(device, memory::AM_READONLY) + b->offset_ * item;
    char* pc = (char*)c->memory_->data(device, memory::AM_MUTABLE) + c->offset_ * item;
    double alpha = op == OPERATOR_T_SUB ? -1.0 : 1.0;
    double beta = op == OPERATOR_T_EQL ? 0.0 : 1.0;
    check(dalib200_gemm(dev, nullptr, (int)dest.dtype(), m, n, k, pa, as_[0], as_[1], pb, bs[0], bs[1], pc, cs[0], cs[1],
                        alpha, beta),
          "dalib200_gemm");
    ++tl_stats.gemms;
}

// dest (op)= running reduction of the rows of the argument (reference: AxisScan, dali/array/op/scan.cpp:19-180).
void run_scan(const Array& dest, OPERATOR_T op, Scan* sc) {
    if (op != OPERATOR_T_EQL || !as<BufferView>(dest)->contiguous()) {
        Array tmp(dest.shape(), dest.dtype(), dest.preferred_device());
        run_scan(tmp, OPERATOR_T_EQL, sc);
        run_assignment(dest, op, tmp);
        return;
    }
    Array in = sc->arguments_[0];
    if (!in.is_buffer()) in.eval(false);
    if (!as<BufferView>(in)->contiguous()) in = in.ascontiguousarray();
    BufferView* a = as<BufferView>(in);
    BufferView* d = as<BufferView>(dest);
    const int64_t cols = a->shape_.back();
    const int64_t rows = cols ? a->numel() / cols : 0;
    const int64_t out_cols = cols + (sc->inclusive_ ? 0 : 1);
    if (tl_dry_run) { ++tl_stats.kernels; tl_stats.last_variant = "scan." + sc->name(); return; }
    memory::Device device = dest.preferred_device();
    const int dev = device_index(device);
    const int item = size_of_dtype(dest.dtype());
    const char* pin = (const char*)a->memory_->data(device, memory::AM_READONLY) + a->offset_ * item;
    char* pout = (char*)d->memory_->data(device, memory::AM_MUTABLE) + d->offset_ * item;
    const int opcode = sc->reducer_ == "sum" ? DALIB200_SCAN_SUM : sc->reducer_ == "prod" ? DALIB200_SCAN_PROD
                       : sc->reducer_ == "max" ? DALIB200_SCAN_MAX : DALIB200_SCAN_MIN;
    check(dalib200_scan(dev, nullptr, (int)dest.dtype(), opcode, sc->inclusive_ ? 1 : 0, rows, cols, pin, cols, pout, out_cols),
          "dalib200_scan");
    ++tl_stats.kernels;
    tl_stats.last_variant = "scan." + sc->name();
}

// dest (op)= tree(acc, other operands) with acc a product or the sum of two products: one
// tcgen05 GEMM whose epilogue is the tree.  false = this layout is not one the tensor-core path
// takes (the caller goes on with the general path); operands of the products have then already
// been evaluated, which is harmless.
// the operand buffers of the product(s) behind an accumulator node
struct GemmOperands {
    int np = 0;
    BufferView *a[2] = {nullptr, nullptr}, *b[2] = {nullptr, nullptr};
    std::vector<Array> keep;
    int64_t m = 0, n = 0, k[2] = {0, 0};
};
bool gemm_operands(const Expression* acc, GemmOperands* g) {
    std::vector<const Expression*> products;
    if (acc->kind_ == N_MATMUL) products.push_back(acc);
    else for (const Array& arg : acc->arguments_) products.push_back(arg.expression().get());
    g->np = (int)products.size();
    for (int p = 0; p < g->np; ++p) {
        Array left = products[p]->arguments_[0], right = products[p]->arguments_[1];
        if (!left.is_buffer()) left.eval(false);
        if (!right.is_buffer()) right.eval(false);
        g->a[p] = as<BufferView>(left);
        g->b[p] = as<BufferView>(right);
        if (!g->a[p] || !g->b[p]) return false;
        g->keep.push_back(left);
        g->keep.push_back(right);
        g->m = g->a[p]->shape_[0]; g->k[p] = g->a[p]->shape_[1]; g->n = g->b[p]->shape_[1];
        if (g->m == 0 || g->n == 0 || g->k[p] == 0) return false;
    }
    return true;
}

bool launch_gemm_program(Lowerer& L, const GemmOperands& g, int64_t m, int64_t n);

bool try_fused_gemm(const Array& dest, OPERATOR_T op, const Array& value, const Expression* acc) {
    GemmOperands g;
    if (!gemm_operands(acc, &g)) return false;
    const int64_t m = g.m, n = g.n;
    memory::Device device = dest.preferred_device();

    Lowerer L({m, n}, 0, device);
    L.acc_node = acc;
    int v = L.visit(value, identity_map(2));
    if (L.types[v] != DTYPE_FLOAT) return false;
    for (const Leaf& leaf : L.leaves)
        if (leaf.iota) return false;      // epilogue programs read memory operands only
    BufferView* db = as<BufferView>(dest);
    int leaf = L.leaf_for(db, identity_map(2), true, false, 0, 0, 0);
    if (op != OPERATOR_T_EQL) L.leaves[leaf].read = true;
    L.keep_alive.push_back(dest);
    L.body.push_back("st " + std::to_string(leaf) + " " + ir_assign(op) + " v" + std::to_string(v));
    return launch_gemm_program(L, g, m, n);
}

// Registers the epilogue program L holds, splits the operands and launches the GEMM over the [m, n] space
// (n = the width of one column slice when the program reads several).
bool launch_gemm_program(Lowerer& L, const GemmOperands& g, int64_t m, int64_t n) {
    const int np = g.np;
    BufferView* const* a = g.a;
    BufferView* const* b = g.b;
    const int64_t* k = g.k;
    const memory::Device device = L.device;
    const std::string text = L.ir_text();
    const uint64_t hash = dalib::fnv1a(text);
    if (!dalib200_is_loaded(hash)) check(dalib200_compile(hash, text.c_str(), text.size()), "dalib200_compile");
    tl_stats.last_ir = text;
    const void *pa_hi[2], *pa_lo[2], *pb_hi[2], *pb_lo[2];
    int64_t ld[2];
    // bf16 operands (both of every pair): one bf16 tensor-core pass straight from the arrays -- A [m,k] and B [k,n]
    // row-major with pitches TMA can address; nothing is split
    int n_bf16 = 0;
    for (int p = 0; p < np; ++p) n_bf16 += (a[p]->dtype_ == DTYPE_BF16) + (b[p]->dtype_ == DTYPE_BF16);
    if (n_bf16 != 0 && n_bf16 != 2 * np) return false;
    if (n_bf16) {
        int64_t lda[2], ldb[2];
        for (int p = 0; p < np; ++p) {
            std::vector<int> as_ = a[p]->normalized_strides(), bs = b[p]->normalized_strides();
            if ((as_[1] != 1 && k[p] != 1) || (bs[1] != 1 && g.n != 1)) return false;
            lda[p] = as_[0]; ldb[p] = bs[0];
            if (lda[p] % 8 || ldb[p] % 8 || a[p]->offset_ % 8 || b[p]->offset_ % 8 || lda[p] < k[p] || ldb[p] < g.n) return false;
        }
        const int na = (int)L.leaves.size();
        std::vector<void*> ptrs(na, (void*)(uintptr_t)4096);
        std::vector<int64_t> offsets(na, 0);
        std::vector<const int64_t*> strides(na, nullptr);
        std::vector<double> sd(L.scalars.size());
        std::vector<float> sf(L.scalars.size());
        std::vector<int> si(L.scalars.size());
        std::vector<const void*> sp(L.scalars.size());
        for (size_t j = 0; j < L.scalars.size(); ++j) {
            sd[j] = L.scalars[j].second; sf[j] = (float)sd[j]; si[j] = (int)sd[j];
            sp[j] = L.scalars[j].first == DTYPE_DOUBLE ? (const void*)&sd[j] : (L.scalars[j].first == DTYPE_FLOAT ? (const void*)&sf[j] : (const void*)&si[j]);
        }
        int dev = -1;
        if (!tl_dry_run) {
            dev = device_index(device);
            for (int p = 0; p < np; ++p) {
                pa_hi[p] = (const char*)a[p]->memory_->data(device, memory::AM_READONLY) + a[p]->offset_ * 2;
                pb_hi[p] = (const char*)b[p]->memory_->data(device, memory::AM_READONLY) + b[p]->offset_ * 2;
            }
            for (int pass = 0; pass < 2; ++pass)
                for (int i = 0; i < na; ++i) {
                    if ((pass == 1) != L.leaves[i].written) continue;
                    ptrs[i] = L.leaves[i].memory->data(device, L.leaves[i].written ? memory::AM_MUTABLE : memory::AM_READONLY);
                }
        } else {
            for (int p = 0; p < np; ++p) pa_hi[p] = pb_hi[p] = (void*)(uintptr_t)4096;
        }
        for (int i = 0; i < na; ++i) { offsets[i] = L.leaves[i].offset; strides[i] = L.leaves[i].strides.data(); }
        int rc = dalib200_gemm_fused_sum(dev, nullptr, DALIB200_BF16, np, m, n, k, pa_hi, lda, pb_hi, ldb, nullptr, nullptr, hash,
                                         ptrs.data(), offsets.data(), strides.data(), na, sp.data(), (int)sp.size());
        if (rc == DALIB200_ERR_UNSUPPORTED) return false;
        check(rc, "dalib200_gemm_fused_sum (bf16)");
        ++tl_stats.gemms;
        char buf[256];
        dalib200_last_gemm_kernel(buf, sizeof buf);
        tl_stats.last_variant = buf;
        return true;
    }
    if (tl_dry_run) {
        void* fake[16];
        for (auto& p : fake) p = (void*)(uintptr_t)4096;
        if (L.leaves.size() > 16 || n % 4) return false;     // (a multiple of 4 per slice is one for the whole product too)
        for (int p = 0; p < np; ++p) {
            if (k[p] % 4) return false;
            pa_hi[p] = pa_lo[p] = pb_hi[p] = pb_lo[p] = fake[0];
            ld[p] = k[p];
        }
        int rc = dalib200_gemm_fused_sum(-1, nullptr, DALIB200_F32, np, m, n, k, pa_hi, ld, pb_hi, ld, pa_lo, pb_lo, hash, fake,
                                         nullptr, nullptr, (int)L.leaves.size(), nullptr, 0);
        if (rc == DALIB200_ERR_UNSUPPORTED) return false;
        check(rc, "dalib200_gemm_fused_sum (compile only)");
        ++tl_stats.gemms;   // one launch, whatever the number of products
        tl_stats.last_variant = np > 1 ? "tcgen05.tf32x3 x2" : "tcgen05.tf32x3";
        return true;
    }
    const int dev = device_index(device);
    std::shared_ptr<SplitParts> parts[4];
    std::vector<PendingSplit> pending;       // left operands not split yet: x and h of a cell go out as one launch
    bool splittable = true;
    for (int p = 0; p < np && splittable; ++p) {
        parts[2 * p] = split_operand(a[p], false, device, dev, &pending);
        parts[2 * p + 1] = split_operand(b[p], true, device, dev);
        splittable = parts[2 * p] && parts[2 * p + 1];
    }
    launch_pending(pending, dev);             // also when giving up: the cached parts must hold what they promise
    if (!splittable) return false;
    for (int p = 0; p < np; ++p) {
        pa_hi[p] = parts[2 * p]->hi; pa_lo[p] = parts[2 * p]->lo;
        pb_hi[p] = parts[2 * p + 1]->hi; pb_lo[p] = parts[2 * p + 1]->lo;
        ld[p] = k[p];
    }
    const int na = (int)L.leaves.size();
    std::vector<void*> ptrs(na);
    std::vector<int64_t> offsets(na);
    std::vector<const int64_t*> strides(na);
    for (int pass = 0; pass < 2; ++pass)
        for (int i = 0; i < na; ++i) {
            if ((pass == 1) != L.leaves[i].written) continue;
            ptrs[i] = L.leaves[i].memory->data(device, L.leaves[i].written ? memory::AM_MUTABLE : memory::AM_READONLY);
            offsets[i] = L.leaves[i].offset;
            strides[i] = L.leaves[i].strides.data();
        }
    std::vector<double> sd(L.scalars.size());
    std::vector<float> sf(L.scalars.size());
    std::vector<int> si(L.scalars.size());
    std::vector<const void*> sp(L.scalars.size());
    for (size_t j = 0; j < L.scalars.size(); ++j) {
        sd[j] = L.scalars[j].second; sf[j] = (float)sd[j]; si[j] = (int)sd[j];
        sp[j] = L.scalars[j].first == DTYPE_DOUBLE ? (const void*)&sd[j] : (L.scalars[j].first == DTYPE_FLOAT ? (const void*)&sf[j] : (const void*)&si[j]);
    }
    int rc = dalib200_gemm_fused_sum(dev, nullptr, DALIB200_F32, np, m, n, k, pa_hi, ld, pb_hi, ld, pa_lo, pb_lo, hash,
                                     ptrs.data(), offsets.data(), strides.data(), na, sp.data(), (int)sp.size());
    if (rc == DALIB200_ERR_UNSUPPORTED) return false;
    check(rc, "dalib200_gemm_fused_sum");
    ++tl_stats.gemms;   // one launch, whatever the number of products
    char buf[256];
    dalib200_last_gemm_kernel(buf, sizeof buf);
    tl_stats.last_variant = buf;
    return true;
}

// A reduction over the trailing dims of few, very long rows.  The `row` skeleton gives a row to one CTA, which
// leaves most of the machine idle when there are fewer rows than SMs; the `all` skeleton spreads ONE reduction
// over every SM.  Such a reduction therefore runs as one all-axis reduction per row, and a tree around it (a
// softmax over [4, 16M]) is evaluated reduction by reduction with an elementwise kernel at the end.
// (not when the rows are read through a view or with a stride: a reduction over axis 0 arrives here as the last
// axis of a transposed view, and the `col` skeleton reads that layout with 128-bit loads)
bool reads_rows_contiguously(const Array& a, int depth = 0) {
    if (a.is_stateless() || depth > 64) return false;
    Expression* e = a.expression().get();
    switch (e->kind_) {
        case N_SCALAR: case N_IOTA: return true;
        case N_BUFFER: {
            BufferView* b = static_cast<BufferView*>(e);
            return b->ndim() == 0 || b->shape_.back() == 1 || b->normalized_strides().back() == 1;
        }
        case N_ELEMENTWISE:
            for (const Array& arg : e->arguments_) if (!reads_rows_contiguously(arg, depth + 1)) return false;
            return true;
        case N_VIEW: {
            // which dim of the argument runs along the view's last dim?  none: a broadcast along the rows (a keepdims
            // result), harmless; the argument's own last dim with step 1: look further down; anything else: strided
            View* v = static_cast<View*>(e);
            const int last = v->ndim() - 1;
            int from = -1;
            for (size_t k = 0; k < v->dims_.size(); ++k)
                if (v->dims_[k].src == last && v->arguments_[0].shape()[k] != 1) from = (int)k;
            if (from < 0) return true;
            if (from != (int)v->dims_.size() - 1 || v->dims_[from].step != 1) return false;
            return reads_rows_contiguously(v->arguments_[0], depth + 1);
        }
        default: return false;
    }
}

bool few_long_rows(const Reduce* r) {
    const Array& arg = r->arguments_[0];
    const int lead = arg.ndim() - r->nreduce_;
    if (lead < 1 || r->xrank_ || !reads_rows_contiguously(arg)) return false;    // (a sharded reduction is combined once, as a whole)
    int64_t rows = 1, cols = 1;
    for (int d = 0; d < arg.ndim(); ++d) (d < lead ? rows : cols) *= arg.shape()[d];
    return rows >= 1 && ((rows <= 8 && cols >= (1 << 18)) || (rows <= 32 && cols >= (1 << 22)));
}

// evaluates, bottom up and in place (the handle then names the buffer), every such reduction below `a`
void split_few_long_row_reductions(const Array& a, int depth = 0) {
    if (a.is_stateless() || depth > 64) return;
    Expression* e = a.expression().get();
    if (e->kind_ != N_ELEMENTWISE && e->kind_ != N_VIEW && e->kind_ != N_REDUCE) return;
    for (const Array& arg : e->arguments_) split_few_long_row_reductions(arg, depth + 1);
    if (e->kind_ == N_REDUCE && few_long_rows(static_cast<Reduce*>(e))) {
        a.eval(false);
        ++tl_stats.temporaries;
    }
}

// A lazy value that several handles name and whose tree has grown large is evaluated once, in place, instead of being
// re-derived inside every kernel that reads it.  What this bounds: state that is carried from step to step as a lazy
// expression of its own previous value (m = b1 * m + (1 - b1) * g in the reference's solvers,
// dali/tensor/op/solver_updates/adam.cpp:31-34, never evaluated by the caller) would otherwise make every step's
// program longer than the last one's, each a new kernel to compile.  Small shared values (the exp of a softmax, the
// c' of an LSTM cell) stay fused.
// "Large" is measured as depth (the longest chain of nodes): history makes a tree deeper with every step, while the
// wide trees that should stay fused (an LSTM cell's gating: depth 9) do not get deep.
// When one shared value has grown past the limit, every shared value of the tree that is more than a couple of nodes
// deep is evaluated with it: the carried states of a solver then all restart from buffers in the same step, and the
// steps that follow repeat a handful of program shapes instead of walking through every combination of phases.
constexpr int kSharedDepthLimit = 16, kSharedDepthFloor = 4;
int shared_depth(const Array& a, std::unordered_map<const Expression*, int>& depth_of, bool* over, int level = 0) {
    if (a.is_stateless() || level > 256) return 0;
    Expression* e = a.expression().get();
    if (e->kind_ == N_BUFFER || e->kind_ == N_SCALAR || e->kind_ == N_IOTA || e->kind_ == N_ASSIGN) return 0;
    auto it = depth_of.find(e);
    if (it != depth_of.end()) return it->second;
    int d = 0;
    for (const Array& arg : e->arguments_) d = std::max(d, shared_depth(arg, depth_of, over, level + 1));
    d += 1;
    if (level > 0 && d >= kSharedDepthLimit && a.handle_count() > 1) *over = true;
    depth_of[e] = d;
    return d;
}
void evaluate_shared(const Array& a, const std::unordered_map<const Expression*, int>& depth_of, int floor, int level = 0) {
    if (a.is_stateless() || level > 256) return;
    Expression* e = a.expression().get();
    auto it = depth_of.find(e);
    if (it == depth_of.end()) return;                      // a leaf, or evaluated on the way here
    const int d = it->second;
    for (const Array& arg : e->arguments_) evaluate_shared(arg, depth_of, floor, level + 1);
    if (level > 0 && d >= floor && a.handle_count() > 1 && !a.is_buffer()) {
        a.eval(false);
        ++tl_stats.temporaries;
    }
}
void trim_shared_history(const Array& value) {
    std::unordered_map<const Expression*, int> depth_of;
    bool over = false;
    shared_depth(value, depth_of, &over);
    if (over) evaluate_shared(value, depth_of, kSharedDepthFloor);
}

// Starts the host -> device copies of the buffers a tree reads before the tree is lowered: the copies (asynchronous
// from page-locked memory) then run while the host builds the program.  A gather's or scatter's source is copied as
// a whole too, as the launch would.
void prefetch_inputs(const Array& a, const memory::Device& device, int depth = 0) {
    if (a.is_stateless() || depth > 64 || !device.is_gpu()) return;
    Expression* e = a.expression().get();
    if (e->kind_ == N_BUFFER) {
        BufferView* b = static_cast<BufferView*>(e);
        if (!b->memory_->is_fresh(device) && b->memory_->is_fresh(memory::Device::cpu())) b->memory_->data(device, memory::AM_READONLY);
        return;
    }
    if (e->kind_ == N_ASSIGN) return;      // evaluated on its own, with its own prefetch
    for (const Array& arg : e->arguments_) prefetch_inputs(arg, device, depth + 1);
}

}  // namespace

// Every lazy value inside `value` that another handle also names is evaluated in place (see array.cc: an update that
// reads its own destination runs at once, and the values it is built from -- a solver's running averages, rebound
// every step to an expression of the gradient -- must be computed while the arrays they read still hold what they held
// when the statements were written).
void evaluate_shared_values(const Array& value) {
    std::unordered_map<const Expression*, int> depth_of;
    bool over = false;
    shared_depth(value, depth_of, &over);
    evaluate_shared(value, depth_of, 1);
}

namespace {
// dest (op)= value, where value is a reduction over the sharded dimension or a product that contracts it.
void run_with_combine(const Array& dest, OPERATOR_T op, const Array& value) {
    Expression* e = value.expression().get();
    const bool direct = op == OPERATOR_T_EQL && dest.is_buffer() && as<BufferView>(dest)->contiguous();
    if (!direct) {
        Array tmp(value.shape(), value.dtype(), dest.preferred_device());
        run_with_combine(tmp, OPERATOR_T_EQL, value);
        ++tl_stats.temporaries;
        run_assignment(dest, op, tmp);
        return;
    }
    const memory::Device device = dest.preferred_device();
    BufferView* db = as<BufferView>(dest);
    const int64_t n = db->numel();
    struct Restore { const Expression* prev; ~Restore() { tl_local_only = prev; } } restore{tl_local_only};
    tl_local_only = e;
    if (e->kind_ == N_MATMUL) {
        run_assignment(dest, OPERATOR_T_EQL, value);                    // the local product
        note_collective("allreduce sum " + std::to_string(n) + " " + ir_dtype(dest.dtype()) + " (product over the sharded dimension)");
        if (tl_dry_run || n == 0) return;
        const int dev = device_index(device);
        char* p = (char*)db->memory_->data(device, memory::AM_MUTABLE) + db->offset_ * size_of_dtype(dest.dtype());
        check(dalib200_allreduce(dev, nullptr, p, n, (int)dest.dtype(), DALIB200_OP_SUM), "dalib200_allreduce");
        return;
    }
    Reduce* r = static_cast<Reduce*>(e);
    const int opcode = reducer_op(r->reducer_);
    if (!r->arg_) {
        run_assignment(dest, OPERATOR_T_EQL, value);                    // the rank's partial results
        note_collective("allreduce " + r->reducer_ + " " + std::to_string(n) + " " + ir_dtype(dest.dtype()));
        if (tl_dry_run || n == 0) return;
        const int dev = device_index(device);
        char* p = (char*)db->memory_->data(device, memory::AM_MUTABLE) + db->offset_ * size_of_dtype(dest.dtype());
        check(dalib200_allreduce(dev, nullptr, p, n, (int)dest.dtype(), opcode), "dalib200_allreduce");
        return;
    }
    // argmax / argmin: ONE local kernel yields the extreme value and its position in the logical array (local
    // position + the shard's offset); the ranks' (value, position) pairs are then combined, lowest position among equals
    const Array& arg = r->arguments_[0];
    std::vector<int64_t> space;
    for (int d : arg.shape()) space.push_back(d);
    const int rank = (int)space.size();
    Lowerer L(space, r->nreduce_, device);
    const int v = L.visit(arg, identity_map(rank));
    const DType vt = L.types[v];
    const int best = L.new_value(vt, false, "red " + r->reducer_ + " v" + std::to_string(v));
    const int pos = L.new_value(DTYPE_INT32, false, "argred " + r->reducer_ + " v" + std::to_string(v));
    const int slot = (int)L.scalars.size();
    L.scalars.push_back(std::make_pair(DTYPE_INT32, (double)r->xrank_offset_));
    const int off = L.new_value(DTYPE_INT32, false, "sc " + std::to_string(slot));
    const int global = L.new_value(DTYPE_INT32, false, "op add v" + std::to_string(pos) + " v" + std::to_string(off));
    Array values(dest.shape(), vt, device);
    const IndexMap out_map = identity_map(rank - r->nreduce_);
    const int leaf_v = L.leaf_for(as<BufferView>(values), out_map, true, false, 0, 0, 0);
    const int leaf_i = L.leaf_for(db, out_map, true, false, 0, 0, 0);
    L.keep_alive.push_back(values);
    L.keep_alive.push_back(dest);
    L.body.push_back("st " + std::to_string(leaf_v) + " assign v" + std::to_string(best));
    L.body.push_back("st " + std::to_string(leaf_i) + " assign v" + std::to_string(global));
    L.launch();
    ++tl_stats.temporaries;
    note_collective("arg_allreduce " + r->reducer_ + " " + std::to_string(n) + " " + ir_dtype(vt));
    if (tl_dry_run || n == 0) return;
    const int dev = device_index(device);
    void* pv = as<BufferView>(values)->memory_->data(device, memory::AM_MUTABLE);
    int32_t* pi = (int32_t*)db->memory_->data(device, memory::AM_MUTABLE) + db->offset_;
    check(dalib200_arg_allreduce(dev, nullptr, pv, pi, n, (int)vt, opcode), "dalib200_arg_allreduce");
}
}  // namespace

void run_assignment(const Array& dest_in, OPERATOR_T op, const Array& value_in) {
    DALI_ASSERT(!dest_in.is_stateless() && !value_in.is_stateless(), "assignment with a stateless Array");
    DALI_ASSERT(op != OPERATOR_T_LSE, "internal: <<= must be rewritten before it runs");
    Array dest = dest_in;
    Array value = value_in;
    if (dest.is_assignment()) dest.eval(false);
    if (value.is_assignment()) value.eval(false);
    if (dest.expression()->kind_ == N_VIEW) dest = writable_view(dest);
    if (!tl_dry_run) prefetch_inputs(value, dest.preferred_device());

    // ---- the root needs the other ranks: a reduction over the sharded dimension that cannot finish inside its own
    // kernel, or a product that contracts the sharded dimension.  The local part is computed into a contiguous
    // buffer, the parts are combined there (every rank ends up with the same bits), then the operator is applied.
    if (needs_combine(value.expression().get()) &&
        !(value.expression()->kind_ == N_REDUCE && xrank_fusable(static_cast<Reduce*>(value.expression().get()), dest.preferred_device()))) {
        run_with_combine(dest, op, value);
        return;
    }

    // ---- peel pure re-indexing views off the root: dest = view(x)  ->  inverse_view(dest) = x
    // (x keeps its own iteration space, which its reductions / products need).  A tree of nothing but elementwise
    // nodes and views is left alone: the view folds into its leaves' strides, the destination is written in its
    // own order and transposed leaves are read through shared-memory tiles.
    while (value.expression()->kind_ == N_VIEW && dest.is_buffer() && !only_elementwise(value.expression()->arguments_[0])) {
        View* v = static_cast<View*>(value.expression().get());
        bool pure = true;
        std::vector<int> used(v->ndim(), -1);
        const std::vector<int>& arg_shape = v->arguments_[0].shape();
        for (size_t k = 0; k < v->dims_.size(); ++k) {
            const ViewDim& d = v->dims_[k];
            // a permutation / squeeze only: a slice that starts at 0 with step 1 but stops early is not one
            if (d.src < 0 || d.off != 0 || d.step != 1 || used[d.src] >= 0 || v->shape_[d.src] != arg_shape[k]) { pure = false; break; }
            used[d.src] = (int)k;
        }
        for (int d = 0; pure && d < v->ndim(); ++d)
            if (used[d] < 0 && v->shape_[d] != 1) pure = false;
        if (!pure || dest.shape() != v->shape_) break;
        // dest'[arg dims] : arg dim k reads dest dim v->dims_[k].src; dims not covered are size 1
        Array d2 = dest;
        std::vector<int> perm;   // build through pluck (size-1 dims) + dimshuffle
        for (int d = v->ndim() - 1; d >= 0; --d)
            if (used[d] < 0) d2 = d2.pluck_axis(d, 0);
        // remaining dest dims, in order, correspond to arg dims sorted by src
        std::vector<std::pair<int, int>> order;   // (src, arg dim)
        for (size_t k = 0; k < v->dims_.size(); ++k) order.push_back(std::make_pair(v->dims_[k].src, (int)k));
        std::sort(order.begin(), order.end());
        std::vector<int> pos_of_arg(v->dims_.size());
        for (size_t i = 0; i < order.size(); ++i) pos_of_arg[order[i].second] = (int)i;
        std::vector<int> pattern(v->dims_.size());
        for (size_t k = 0; k < v->dims_.size(); ++k) pattern[k] = pos_of_arg[k];
        if (!pattern.empty()) d2 = d2.dimshuffle(pattern);
        dest = d2;
        value = v->arguments_[0];
        if (value.is_assignment()) value.eval(false);
    }

    // ---- an elementwise tree around a product: tensor-core GEMM with the tree as its epilogue
    if (dest.is_buffer() && product_reads_destination(value, as<BufferView>(dest))) {
        Array tmp(dest.shape(), value_dtype(dest.dtype()), dest.preferred_device());
        run_assignment(tmp, OPERATOR_T_EQL, value);
        run_assignment(dest, op, tmp);
        return;
    }
    if (dest.is_buffer() && dest.ndim() == 2 && value_dtype(dest.dtype()) == DTYPE_FLOAT && value.shape() == dest.shape()) {
        const Expression* acc = nullptr;
        find_matmul_sum(value, &acc);
        if (!acc) find_matmul(value, &acc);
        if (acc && acc->dtype_ == DTYPE_FLOAT && !pending_partial(acc) && try_fused_gemm(dest, op, value, acc)) return;
    }

    // ---- reductions over few, very long rows: one all-axis reduction per row (see few_long_rows)
    if (value.expression()->kind_ == N_REDUCE && dest.is_buffer() && few_long_rows(static_cast<Reduce*>(value.expression().get()))) {
        Reduce* rd = static_cast<Reduce*>(value.expression().get());
        const Array& arg = rd->arguments_[0];
        split_few_long_row_reductions(arg);
        const int lead = arg.ndim() - rd->nreduce_;
        int64_t rows = 1;
        for (int d = 0; d < lead; ++d) rows *= arg.shape()[d];
        for (int64_t r = 0; r < rows; ++r) {
            Array a_r = arg, d_r = dest;
            int64_t rem = r, div = rows;
            for (int d = 0; d < lead; ++d) {
                div /= arg.shape()[d];
                const int idx = (int)(rem / div);
                rem %= div;
                a_r = a_r.pluck_axis(0, idx);
                d_r = d_r.pluck_axis(0, idx);
            }
            Array v_r(std::make_shared<Reduce>(rd->reducer_, a_r, rd->nreduce_, rd->arg_, rd->dtype_));
            run_assignment(d_r, op, v_r);
        }
        return;
    }
    split_few_long_row_reductions(value);
    trim_shared_history(value);

    // ---- a running reduction at the root has its own kernel
    if (value.expression()->kind_ == N_SCAN && dest.is_buffer()) {
        run_scan(dest, op, static_cast<Scan*>(value.expression().get()));
        return;
    }

    // ---- MatMul at the root goes to the general GEMM entry point
    if (value.expression()->kind_ == N_MATMUL && dest.is_buffer()) {
        run_matmul(dest, op, static_cast<MatMul*>(value.expression().get()));
        return;
    }

    // ---- destination: a buffer view, or a gather of one (scatter)
    const bool scatter = !dest.is_buffer();
    if (scatter) {
        DALI_ASSERT(dest.expression()->kind_ == N_GATHER || dest.expression()->kind_ == N_GATHER_ROWS,
                    "assignment destination must be a buffer or a gather of one (got " + dest.expression_name() + ")");
        DALI_ASSERT(dest.expression()->arguments_[0].is_assignable(), "cannot scatter into a value that is not stored anywhere");
    }
    if (ScalarValue* sv = as<ScalarValue>(value)) {
        // a host scalar takes the destination's type before it becomes a kernel argument
        if (sv->dtype_ != value_dtype(dest.dtype())) {
            double x = sv->value_;
            if (dest.dtype() == DTYPE_INT32) x = std::floor(x + 0.5);
            value = Array(std::make_shared<ScalarValue>(x, value_dtype(dest.dtype())));
        }
    }
    if (value.ndim() != 0 && value.shape() != dest.shape()) {
        DALI_ASSERT(value.ndim() == dest.ndim(), "cannot assign an array of shape rank " + std::to_string(value.ndim()) +
                                                     " to a destination of rank " + std::to_string(dest.ndim()));
        value = value.broadcast_to_shape(dest.shape());
    }
    if (dest.numel() == 0) return;
    memory::Device device = dest.preferred_device();

    // ---- iteration space
    FoundReduce fr;
    find_reduce(value, false, &fr);
    std::vector<int64_t> space;
    int nreduce = 0;
    bool row_level_root = false;
    if (fr.node && !fr.through_view && !scatter) {
        // the root lives at reduction-result level: iterate over the reduction's operand
        for (int s : fr.node->arguments_[0].shape()) space.push_back(s);
        nreduce = fr.node->nreduce_;
        row_level_root = true;
        if ((int)space.size() - nreduce != dest.ndim()) {   // shapes disagree (should not happen): no fusion
            space.clear();
            nreduce = 0;
            row_level_root = false;
        }
    }
    if (space.empty()) {
        for (int s : dest.shape()) space.push_back(s);
        if (fr.node && fr.through_view) {
            const int k = fr.node->nreduce_;
            const std::vector<int>& as_ = fr.node->arguments_[0].shape();
            bool fits = k < (int)space.size() && (int)as_.size() == (int)space.size();
            for (int d = 0; fits && d < (int)space.size(); ++d) fits = as_[d] == space[d];
            if (fits) nreduce = k;    // reductions over the trailing dims fuse with the elementwise root
        }
        if (space.empty()) space.push_back(1);   // rank-0 destination
    }
    const int rank = (int)space.size();
    const bool rank0_dest = dest.ndim() == 0 && !row_level_root;

    Lowerer L(space, nreduce, device);
    // ---- value
    IndexMap root_map = rank0_dest ? IndexMap() : identity_map(row_level_root ? rank - nreduce : (int)dest.shape().size());
    int v = value.ndim() == 0 ? L.visit(value, IndexMap()) : L.visit(value, root_map);
    if (L.types[v] != value_dtype(dest.dtype())) {
        // assignment converts; towards int32 it rounds, as op::astype does (towards bf16 the store itself rounds)
        if (dest.dtype() == DTYPE_INT32) v = L.new_value(DTYPE_INT32, L.elem[v], "op round v" + std::to_string(v));
        else v = L.new_value(dest.dtype(), L.elem[v], "cast v" + std::to_string(v));
    }
    // ---- store
    if (!scatter) {
        BufferView* db = as<BufferView>(dest);
        int leaf = L.leaf_for(db, root_map, true, false, 0, 0, 0);
        if (nreduce > 0 && !row_level_root) L.leaves[leaf].elem_level = true;
        if (op != OPERATOR_T_EQL) L.leaves[leaf].read = true;
        // The destination's buffer is also read through a DIFFERENT index map (a.assign(a.transpose()), a[1:] = a[:-1],
        // a[0] = sum(a, 0)): other threads would overwrite elements this one still has to read.  The value goes to a
        // temporary first.  (The same map is fine: every element is read and written by the same thread.)
        {
            const Leaf& w = L.leaves[leaf];
            auto span = [&](const Leaf& l, int64_t* lo, int64_t* hi) {
                *lo = *hi = l.offset;
                for (int d = 0; d < rank; ++d) {
                    const int64_t reach = (space[d] - 1) * l.strides[d];
                    if (reach < 0) *lo += reach; else *hi += reach;
                }
            };
            int64_t wl, wh;
            span(w, &wl, &wh);
            for (size_t i = 0; i < L.leaves.size(); ++i) {
                const Leaf& r = L.leaves[i];
                if ((int)i == leaf || r.iota || r.memory != w.memory) continue;
                int64_t rl, rh;
                span(r, &rl, &rh);
                if (r.indirect || (rl <= wh && wl <= rh)) {
                    Array tmp(dest.shape(), value_dtype(dest.dtype()), dest.preferred_device());
                    run_assignment(tmp, OPERATOR_T_EQL, value);
                    run_assignment(dest, op, tmp);
                    return;
                }
            }
        }
        L.keep_alive.push_back(dest);
        L.body.push_back("st " + std::to_string(leaf) + " " + ir_assign(op) + " v" + std::to_string(v));
    } else {
        Expression* g = dest.expression().get();
        const bool rows = g->kind_ == N_GATHER_ROWS;
        Array source = g->arguments_[0];
        if (!source.is_buffer()) source.eval(false);
        DALI_ASSERT(source.is_buffer(), "scatter destination must evaluate to a buffer");
        BufferView* sb = as<BufferView>(source);
        const Array& indices = g->arguments_[1];
        const int ri = indices.ndim();
        IndexMap im(root_map.begin(), root_map.begin() + ri);
        int vi = L.visit(indices, im);
        IndexMap sm;
        if (rows) {
            sm.push_back(root_map[0]);
            for (int t = 1; t < (int)root_map.size(); ++t) sm.push_back(root_map[t]);
        } else {
            for (int t = ri; t < (int)root_map.size(); ++t) sm.push_back(root_map[t]);
        }
        std::vector<int> sst = sb->normalized_strides();
        int leaf = L.leaf_for(sb, sm, true, true, sst[rows ? 1 : 0], rows ? 1 : 0, 1);
        L.leaves[leaf].elem_level = true;
        L.keep_alive.push_back(source);
        L.body.push_back("stx " + std::to_string(leaf) + " " + ir_assign(op) + " v" + std::to_string(vi) + " v" + std::to_string(v));
    }
    L.launch();
}

namespace {
// a product (or a sum of two) reachable from `a` through elementwise nodes AND views
void find_acc_through_views(const Array& a, const Expression** out) {
    if (*out || a.is_stateless()) return;
    Expression* e = a.expression().get();
    if (e->kind_ == N_MATMUL) { *out = e; return; }
    if (e->kind_ == N_ELEMENTWISE) {
        find_matmul_sum(a, out);
        if (*out) return;
    }
    if (e->kind_ != N_ELEMENTWISE && e->kind_ != N_VIEW) return;
    for (const Array& arg : e->arguments_) find_acc_through_views(arg, out);
}

// Elementwise roots of shape [m, n] that read a product of S * n columns only through its S column blocks
// (i, f, o, g of an LSTM cell): ONE GEMM launch whose epilogue computes and stores every root; the product
// itself is never written.  false = not that pattern (the caller goes on with the general path).
bool try_sliced_gemm(const std::vector<const Array*>& roots) {
    const Expression* acc = nullptr;
    for (const Array* r : roots) find_acc_through_views(*r, &acc);
    if (!acc || acc->dtype_ != DTYPE_FLOAT || roots[0]->ndim() != 2 || pending_partial(acc)) return false;
    GemmOperands g;
    if (!gemm_operands(acc, &g)) return false;
    const int64_t m = g.m, n = roots[0]->shape()[1];
    if (roots[0]->shape()[0] != m || n <= 0 || g.n % n != 0) return false;
    const int64_t slices = g.n / n;
    if (slices != 2 && slices != 4) return false;
    for (const Array* r : roots)
        if (r->dtype() != DTYPE_FLOAT) return false;
    const memory::Device device = roots[0]->preferred_device();
    Lowerer L({m, n}, 0, device);
    L.acc_node = acc;
    L.slice_width = n;
    std::vector<Array> dests;
    for (const Array* r : roots) {
        Array value(r->expression());
        int v = L.visit(value, identity_map(2));
        if (L.slice_fail || L.types[v] != DTYPE_FLOAT) return false;
        Array dest(value.shape(), DTYPE_FLOAT, device);
        int leaf = L.leaf_for(as<BufferView>(dest), identity_map(2), true, false, 0, 0, 0);
        L.keep_alive.push_back(dest);
        L.body.push_back("st " + std::to_string(leaf) + " assign v" + std::to_string(v));
        dests.push_back(dest);
    }
    if ((int64_t)L.slices_seen.size() != slices) return false;       // every block of the product is used
    for (const Leaf& leaf : L.leaves)
        if (leaf.iota) return false;
    if (!launch_gemm_program(L, g, m, n)) return false;
    for (size_t i = 0; i < roots.size(); ++i) roots[i]->set_expression(dests[i].expression());
    return true;
}
}  // namespace

// Several lazy arrays of one shape in ONE kernel: what their trees share (the c' that h' = o * tanh(c')
// is built from) is computed once and every root is stored.  The reference has no such call -- there each
// eval() is a kernel of its own; anything this cannot fuse (reductions, products or scans at a root, differing
// shapes) is evaluated one by one exactly as Array::eval would.
void eval_together(const std::vector<Array>& arrays) {
    if (!tl_dry_run)
        for (const Array& a : arrays)
            if (!a.is_stateless() && !a.is_buffer()) prefetch_inputs(a, a.preferred_device());
    std::vector<const Array*> roots;
    for (const Array& a : arrays) {
        DALI_ASSERT(!a.is_stateless(), "eval_together on a stateless Array");
        if (a.is_buffer()) continue;
        roots.push_back(&a);
    }
    bool fusable = roots.size() > 1;
    for (const Array* a : roots) {
        const Expression* e = a->expression().get();
        FoundReduce fr;
        find_reduce(*a, false, &fr);
        fusable = fusable && e->kind_ == N_ELEMENTWISE && !fr.node && e->ndim() > 0 && e->shape_ == roots[0]->expression()->shape_ &&
                  e->numel() > 0;
    }
    if (!fusable) {
        for (const Array* a : roots) a->eval(false);
        return;
    }
    if (try_sliced_gemm(roots)) return;
    const memory::Device device = roots[0]->preferred_device();
    std::vector<int64_t> space;
    for (int d : roots[0]->shape()) space.push_back(d);
    const int rank = (int)space.size();
    Lowerer L(space, 0, device);
    std::vector<Array> dests;
    for (const Array* a : roots) {
        Array value(a->expression());
        int v = L.visit(value, identity_map(rank));
        Array dest(value.shape(), value.dtype(), device);
        int leaf = L.leaf_for(as<BufferView>(dest), identity_map(rank), true, false, 0, 0, 0);
        L.keep_alive.push_back(dest);
        L.body.push_back("st " + std::to_string(leaf) + " assign v" + std::to_string(v));
        dests.push_back(dest);
    }
    L.launch();
    for (size_t i = 0; i < roots.size(); ++i) roots[i]->set_expression(dests[i].expression());
}

}  // namespace lazy
