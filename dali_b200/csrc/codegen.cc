// Kernel skeletons + expression splicing (see codegen.h).
#include "codegen.h"

#include <algorithm>
#include <map>
#include <set>
#include <sstream>

namespace dalib {

const char* Variant::kind_name() const {
    switch (kind) {
        case K_MAP: return "map";
        case K_ROW: return "row";
        case K_COL: return "col";
        case K_ALL: return "all";
    }
    return "?";
}

std::string Variant::key() const {
    std::ostringstream s;
    s << kind_name() << ".o" << nout << ".i" << nin << ".v" << vec << ".nt" << threads << ".T" << T
      << ".p" << vpt << ".u" << unroll << ".x" << tx << ".y" << ty << "." << cls << "." << ocls;
    if (tile) s << ".tile" << tile;
    if (xrank) s << ".xrank";
    if (stage) s << ".stage" << stage;
    if (cluster > 1) s << ".cl" << cluster;
    if (minb) s << ".mb" << minb;
    if (xv.find('1') != std::string::npos) s << ".xv" << xv;
    if (stream_out) s << ".cs";
    if (unchecked) s << ".nc";
    return s.str();
}

ParamLayout::ParamLayout(const Program& p, const Variant& v) {
    w_ishape = w_oshape + v.nout;
    w_args = w_ishape + v.nin;
    arg_words = 2 + v.nout + v.nin;
    w_scalars = w_args + (int)p.args.size() * arg_words;
    total = w_scalars + (int)p.scalars.size();
    if (total < 8) total = 8;
}

int scratch_slot_bytes(const Program& p) {
    // widest partial: ArgPair<double> = 16 bytes; plain values <= 8.
    int b = 4;
    for (const Stmt& s : p.stmts) {
        if (s.kind == S_ARGRED) b = 16;
        else if (s.kind == S_RED && dtype_size(s.dtype) > b && b < 16) b = dtype_size(s.dtype);
    }
    return b;
}

namespace {

const char* red_struct(const std::string& n) {
    if (n == "sum") return "RSum";
    if (n == "prod") return "RProd";
    if (n == "max") return "RMax";
    return "RMin";
}

struct Gen {
    const Program& p;
    const Variant& v;
    ParamLayout L;
    std::ostringstream o;
    std::set<int> need_inv;          // R-level f32 values whose reciprocal is precomputed
    std::vector<int> reds;           // stmt indices of reductions, program order
    std::vector<int> red_slot;       // per stmt index -> position in `reds`, or -1
    std::map<int, int> red_from_arg; // col / all: a max (min) whose operand an argmax (argmin) of the same program also
                                     // reduces -> that arg-reduction's stmt index.  Its running value IS the max, so the
                                     // element loop accumulates nothing for it; the value is copied over after the loop
                                     // (the pair programs of sharded arg-reductions: one reduction's work instead of two)

    Gen(const Program& p_, const Variant& v_) : p(p_), v(v_), L(p_, v_) {
        red_slot.assign(p.stmts.size(), -1);
        for (size_t i = 0; i < p.stmts.size(); ++i) {
            const Stmt& s = p.stmts[i];
            if (s.kind == S_RED || s.kind == S_ARGRED) {
                red_slot[i] = (int)reds.size();
                reds.push_back((int)i);
            }
            if (s.kind == S_OP && s.name == "eltdiv" && s.dtype == F32 && s.elem) {
                const Stmt& d = val(s.in[1]);
                if (!d.elem) need_inv.insert(d.id);
            }
        }
        if (v.kind == K_COL || v.kind == K_ALL)
            for (int r : reds) {
                const Stmt& s = p.stmts[r];
                if (s.kind != S_RED || (s.name != "max" && s.name != "min")) continue;
                for (int a : reds) {
                    const Stmt& t = p.stmts[a];
                    if (t.kind == S_ARGRED && t.name == s.name && t.in[0] == s.in[0] && t.stage == s.stage) { red_from_arg[r] = a; break; }
                }
            }
    }

    const Stmt& val(int id) const { return p.stmts[p.value_stmt[id]]; }
    std::string W(int w) const { return "p.w[" + std::to_string(w) + "]"; }
    std::string ct(DType t) const { return dtype_c_name(t); }
    std::string vn(int id) const { return std::string(val(id).elem ? "e" : "r") + std::to_string(id); }
    std::string argT(int a) const { return ct(p.args[a].dtype); }
    bool arg_elem(int a) const { return p.nreduce == 0 ? true : p.args[a].elem_level; }

    std::string literal(const Stmt& s) const {
        const std::string t = ct(s.dtype);
        if (s.literal == "inf") return "(" + t + ")__longlong_as_double(0x7ff0000000000000LL)";
        if (s.literal == "-inf") return "(" + t + ")__longlong_as_double(0xfff0000000000000LL)";
        if (s.literal == "nan") return "(" + t + ")__longlong_as_double(0x7ff8000000000000LL)";
        std::string lit = s.literal;
        if (s.dtype != I32 && lit.find_first_of(".eEn") == std::string::npos) lit += ".0";
        return "(" + t + ")(" + lit + ")";
    }

    // expression for a non-load, non-reduction value; lane_blocks: inside the lane loop of emit_group, where every
    // random node has an RngBlock rb<id> that its lanes share
    std::string expr(const Stmt& s, bool lane_blocks = false) const {
        switch (s.kind) {
            case S_CONST: return literal(s);
            case S_SC: return "*reinterpret_cast<const " + ct(s.dtype) + "*>(&" + W(L.w_scalars + s.arg) + ")";
            case S_CAST: return "(" + ct(s.dtype) + ")(" + vn(s.in[0]) + ")";
            case S_OP: {
                if (s.name == "round" || s.name == "ceiling")
                    return "f_" + s.name + "<" + ct(s.dtype) + ">(" + vn(s.in[0]) + ")";
                if (s.name == "rng_uniform" || s.name == "rng_normal")
                    return "f_" + s.name + "<" + ct(s.dtype) + ">(" + vn(s.in[0]) + ", " + vn(s.in[1]) +
                           (lane_blocks ? ", rb" + std::to_string(s.id) : std::string()) + ")";
                if (s.name == "eltdiv" && s.in.size() == 2 && need_inv.count(s.in[1]) && s.elem && s.dtype == F32)
                    return vn(s.in[0]) + " * rinv" + std::to_string(s.in[1]);
                std::string e = "f_" + s.name + "(" + vn(s.in[0]);
                if (s.in.size() > 1) e += ", " + vn(s.in[1]);
                return e + ")";
            }
            default: return "/*?*/";
        }
    }

    std::string assign_rhs(AssignOp op, const std::string& old, const std::string& val_) const {
        switch (op) {
            case A_ASSIGN: return val_;
            case A_ADD: return old + " + " + val_;
            case A_SUB: return old + " - " + val_;
            case A_MUL: return old + " * " + val_;
            case A_DIV: return old + " / " + val_;
        }
        return val_;
    }

    // ---- common kernel prologue
    void header() {
        o << "// dali_b200 generated kernel: " << v.key() << "\n";
        o << "struct P { long long w[" << L.total << "]; };\n";
        o << "#define NT " << v.threads << "\n#define VEC " << v.vec << "\n#define UNROLL " << v.unroll << "\n";
        if (v.minb) o << "extern \"C\" __global__ void __launch_bounds__(NT, " << v.minb << ") dali_kernel(const __grid_constant__ P p) {\n";
        else o << "extern \"C\" __global__ void __launch_bounds__(NT) dali_kernel(const __grid_constant__ P p) {\n";
        o << "  kernel_entry();\n";
        o << "  const i64 R = " << W(L.w_R) << "; const i64 C = " << W(L.w_C) << ";\n";
        o << "  const int tid = threadIdx.x;\n";
        for (size_t a = 0; a < p.args.size(); ++a) {
            bool ro = !p.args[a].written;
            if (p.args[a].iota) {
                o << "  const IotaPtr a" << a << "{" << W(L.arg_ptr((int)a)) << "};   // base value instead of a pointer\n";
                continue;
            }
            o << "  " << (ro ? "const " : "") << argT((int)a) << "* const a" << a << " = reinterpret_cast<"
              << (ro ? "const " : "") << argT((int)a) << "*>(" << W(L.arg_ptr((int)a)) << ");\n";
        }
        // uniform values: scalars and constants (and functors of only those at stage 0 are
        // left to the row scope; they are cheap)
        for (const Stmt& s : p.stmts) {
            if (s.kind == S_SC || s.kind == S_CONST) {
                o << "  const " << ct(s.dtype) << " " << vn(s.id) << " = " << expr(s) << ";\n";
                if (need_inv.count(s.id)) o << "  const float rinv" << s.id << " = 1.0f / " << vn(s.id) << ";\n";
            }
        }
    }

    // ---- outer (row) offsets: defines i64 ro<a> for every arg, given row index expr `r`
    void row_offsets(const std::string& ind, const std::string& r, const std::string& ro = "ro") {
        if (v.nout == 0) {
            for (size_t a = 0; a < p.args.size(); ++a) o << ind << "const i64 " << ro << a << " = 0;\n";
            return;
        }
        if (v.nout == 1) {
            for (size_t a = 0; a < p.args.size(); ++a)
                o << ind << "const i64 " << ro << a << " = " << r << " * " << W(L.arg_rs((int)a, 0)) << ";\n";
            return;
        }
        for (size_t a = 0; a < p.args.size(); ++a) o << ind << "i64 " << ro << a << " = 0;\n";
        o << ind << "{ i64 t_ = " << r << ";\n";
        for (int k = v.nout - 1; k >= 0; --k) {
            o << ind << "  { const i64 q_ = t_ / " << W(L.w_oshape + k) << "; const i64 i_ = t_ - q_ * "
              << W(L.w_oshape + k) << "; t_ = q_;\n";
            for (size_t a = 0; a < p.args.size(); ++a)
                o << ind << "    " << ro << a << " += i_ * " << W(L.arg_rs((int)a, k)) << ";\n";
            o << ind << "  }\n";
        }
        o << ind << "}\n";
    }

    // inner offset expression of arg a at inner index `c` (+ lane j); for nin > 1 the
    // caller has emitted col_decompose() which defines co<a>.
    std::string col_off(int a, const std::string& c) const {
        if (v.nin > 1) return "co" + std::to_string(a);
        char k = v.cls[a];
        if (k == 'u') return "(" + c + ")";
        if (k == 'z') return "0";
        return "(" + c + ") * " + W(L.arg_cs(a, 0, v.nout));
    }
    void col_decompose(const std::string& ind, const std::string& c) {
        if (v.nin <= 1) return;
        for (size_t a = 0; a < p.args.size(); ++a) o << ind << "i64 co" << a << " = 0;\n";
        o << ind << "{ i64 t_ = " << c << ";\n";
        for (int k = v.nin - 1; k >= 0; --k) {
            o << ind << "  { const i64 q_ = t_ / " << W(L.w_ishape + k) << "; const i64 i_ = t_ - q_ * "
              << W(L.w_ishape + k) << "; t_ = q_;\n";
            for (size_t a = 0; a < p.args.size(); ++a)
                o << ind << "    co" << a << " += i_ * " << W(L.arg_cs((int)a, k, v.nout)) << ";\n";
            o << ind << "  }\n";
        }
        o << ind << "}\n";
    }

    // ---- pass analysis ------------------------------------------------------
    // number of element passes: reductions of result stage q+1 fold in pass q,
    // element-level stores of stage q happen in pass q.
    int n_passes() const {
        int n = 0;
        for (const Stmt& s : p.stmts) {
            if ((s.kind == S_RED || s.kind == S_ARGRED)) n = std::max(n, s.stage);
            if ((s.kind == S_ST || s.kind == S_STX) && s.elem) n = std::max(n, s.stage + 1);
        }
        return n;
    }

    // stmt indices that are sinks of element pass q
    std::vector<int> pass_sinks(int q) const {
        std::vector<int> out;
        for (size_t i = 0; i < p.stmts.size(); ++i) {
            const Stmt& s = p.stmts[i];
            if ((s.kind == S_RED || s.kind == S_ARGRED) && s.stage == q + 1) out.push_back((int)i);
            if ((s.kind == S_ST || s.kind == S_STX) && s.elem && s.stage == q) out.push_back((int)i);
        }
        return out;
    }

    // element-level value ids needed in pass q.  With `cut` true, traversal stops at
    // element values of an earlier stage (they come from register caches); those are
    // returned in *cuts.
    std::set<int> pass_needed(int q, bool cut, std::set<int>* cuts) const {
        std::set<int> need;
        std::vector<int> stack;
        for (int si : pass_sinks(q))
            for (int in : p.stmts[si].in) stack.push_back(in);
        while (!stack.empty()) {
            int id = stack.back();
            stack.pop_back();
            const Stmt& s = val(id);
            if (!s.elem) continue;
            if (cut && s.stage < q && s.kind != S_LD) {
                if (cuts) cuts->insert(id);
                continue;
            }
            if (!need.insert(id).second) continue;
            for (int in : s.in) stack.push_back(in);
        }
        return need;
    }

    // ---- one vector group of element work ----------------------------------------
    // Emits: loads of the element-level args used, the lane loop computing `need`
    // values in program order, reduction accumulation and element stores of pass q.
    //   c        name of the inner index variable of lane 0 (int or i64)
    //   slot     text appended to cached-array names ("[i]") or "" when nothing is cached
    //   cached   element loads come from / go to register arrays LQ<a>slot
    //   loaded   args whose LQ<a> arrays already hold data (updated)
    //   cuts_rd  value caches to read, cuts_wr value caches to write (CV<id>[i*VEC+j])
    struct GroupCtx {
        std::string ind, c, slot;
        bool cached = false;
        std::set<int>* loaded = nullptr;
        std::set<int> cuts_rd, cuts_wr;
        std::string acc_suffix;    // "" or "[j]" (col kind keeps VEC accumulators)
        std::string argred_index;  // expression of the reduced-dim index of lane j
        std::string argred_defer;  // non-empty: arg-reductions only park their operand in av<si><argred_defer>[j]; the caller
                                   // folds a whole group of parked values at once (fold_deferred_args)
        bool skip_loads = false;   // loads were hoisted by the caller (map / all unrolling)
        std::string hoist_idx;     // "[u]" when loads were hoisted into arrays
    };

    std::set<int> args_loaded_in(const std::set<int>& need, int q) const {
        std::set<int> as;
        for (int id : need) if (val(id).kind == S_LD) as.insert(val(id).arg);
        for (int si : pass_sinks(q)) {
            const Stmt& s = p.stmts[si];
            if (s.kind == S_ST && s.aop != A_ASSIGN) as.insert(s.arg);
        }
        return as;
    }

    // load of the vector group of arg a into variable `dst`
    void emit_arg_load(const std::string& ind, int a, const std::string& dst, const std::string& c, bool declare,
                       const std::string& ro = "ro") {
        const std::string T = argT(a);
        char k = v.nin > 1 ? 's' : v.cls[a];
        if (declare) o << ind << "Vec<" << T << ", VEC> " << dst << ";\n";
        if (v.vec > 1 && k == 'u') {
            o << ind << dst << " = vload<" << T << ", VEC>(a" << a << " + " << ro << a << " + " << c << ");\n";
        } else if (k == 'z' && v.nin == 1) {
            o << ind << "{ const " << T << " t_ = a" << a << "[" << ro << a << "];\n" << ind
              << "  _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) " << dst << ".x[j] = t_; }\n";
        } else if (v.nin > 1) {
            o << ind << dst << ".x[0] = a" << a << "[" << ro << a << " + co" << a << "];\n";
        } else {
            o << ind << "_Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) " << dst << ".x[j] = a" << a << "[" << ro << a
              << " + " << col_off(a, c + " + j") << "];\n";
        }
    }

    void emit_arg_store(const std::string& ind, int a, const std::string& src, const std::string& c) {
        const std::string T = argT(a);
        char k = v.nin > 1 ? 's' : v.cls[a];
        if (v.vec > 1 && k == 'u') {
            // (stream_out: stores that do not displace a gather's table from L2 -- opt-in, see plan.cc)
            o << ind << (v.stream_out ? "vstore_stream<" : "vstore<") << T << ", VEC>(a" << a << " + ro" << a << " + " << c << ", " << src << ");\n";
        } else if (v.nin > 1) {
            o << ind << "a" << a << "[ro" << a << " + co" << a << "] = " << src << ".x[0];\n";
        } else if (k == 'z') {
            // every lane targets the same element; the last lane wins, as a serial loop would
            o << ind << "a" << a << "[ro" << a << "] = " << src << ".x[VEC - 1];\n";
        } else {
            o << ind << "_Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) a" << a << "[ro" << a << " + "
              << col_off(a, c + " + j") << "] = " << src << ".x[j];\n";
        }
    }

    void emit_group(int q, const std::set<int>& need, GroupCtx& g) {
        const std::string& ind = g.ind;
        std::set<int> largs = args_loaded_in(need, q);
        if (v.nin > 1) col_decompose(ind, g.c);
        // loads
        for (int a : largs) {
            const std::string name = g.cached ? "LQ" + std::to_string(a) + g.slot
                                              : (g.skip_loads ? "q" + std::to_string(a) + g.hoist_idx
                                                              : "q" + std::to_string(a));
            if (g.skip_loads) continue;
            if (g.cached) {
                // an arg that is also stored in this pass with an operator must be re-read
                if (g.loaded->count(a)) continue;
                emit_arg_load(ind, a, name, g.c, false);
                g.loaded->insert(a);
            } else {
                emit_arg_load(ind, a, name, g.c, true);
            }
        }
        auto argvec = [&](int a) {
            return g.cached ? "LQ" + std::to_string(a) + g.slot
                            : "q" + std::to_string(a) + (g.skip_loads ? g.hoist_idx : "");
        };
        // output staging
        std::vector<int> sinks = pass_sinks(q);
        for (int si : sinks) {
            const Stmt& s = p.stmts[si];
            if (s.kind == S_ST) o << ind << "Vec<" << argT(s.arg) << ", VEC> out" << si << ";\n";
        }
        for (const Stmt& s : p.stmts)
            if (s.id >= 0 && need.count(s.id) && s.kind == S_OP && (s.name == "rng_uniform" || s.name == "rng_normal"))
                o << ind << "RngBlock rb" << s.id << " = {0u, {0u, 0u, 0u, 0u}, 0};\n";
        // A gathered row read with full-width loads: every lane of the vector group uses the same index (the index
        // operand does not vary along the inner dim) and the row is aligned, so the group is one 128-bit load of the
        // indexed row instead of VEC scalar ones (dali/array/op/gather.cpp:45-65 reads element by element).
        std::set<int> vector_gathers;
        if (v.vec > 1 && v.nin == 1 && !g.cached)
            for (const Stmt& s : p.stmts) {
                if (s.id < 0 || !need.count(s.id) || s.kind != S_LDX) continue;
                const Stmt& ix = val(s.in[0]);
                if ((int)v.xv.size() <= s.arg || v.xv[s.arg] != '1' || ix.kind != S_LD || !arg_elem(s.arg) || !arg_elem(ix.arg) ||
                    v.cls[ix.arg] != 'z' || !largs.count(ix.arg))
                    continue;
                o << ind << "const Vec<" << argT(s.arg) << ", VEC> gx" << s.id << " = vload<" << argT(s.arg) << ", VEC>(a" << s.arg << " + ro"
                  << s.arg << " + " << col_off(s.arg, g.c) << " + (i64)" << argvec(ix.arg) << ".x[0] * " << W(L.arg_xs(s.arg)) << ");\n";
                vector_gathers.insert(s.id);
            }
        o << ind << "_Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) {\n";
        const std::string in2 = ind + "  ";
        for (int id : g.cuts_rd) {
            const Stmt& s = val(id);
            o << in2 << "const " << ct(s.dtype) << " " << vn(id) << " = CV" << id << g.slot.substr(0, g.slot.size() ? g.slot.size() - 1 : 0)
              << (g.slot.empty() ? "[j]" : " * VEC + j]") << ";\n";
        }
        for (const Stmt& s : p.stmts) {
            if (s.id < 0 || !need.count(s.id)) continue;
            if (s.kind == S_LD) {
                o << in2 << "const " << ct(s.dtype) << " " << vn(s.id) << " = " << argvec(s.arg) << ".x[j];\n";
            } else if (s.kind == S_LDX && vector_gathers.count(s.id)) {
                o << in2 << "const " << ct(s.dtype) << " " << vn(s.id) << " = gx" << s.id << ".x[j];\n";
            } else if (s.kind == S_LDX) {
                o << in2 << "const " << ct(s.dtype) << " " << vn(s.id) << " = a" << s.arg << "[ro" << s.arg << " + "
                  << (arg_elem(s.arg) ? col_off(s.arg, g.c + " + j") : std::string("0")) << " + (i64)" << vn(s.in[0])
                  << " * " << W(L.arg_xs(s.arg)) << "];\n";
            } else {
                o << in2 << "const " << ct(s.dtype) << " " << vn(s.id) << " = " << expr(s, true) << ";\n";
            }
            if (g.cuts_wr.count(s.id))
                o << in2 << "CV" << s.id << g.slot.substr(0, g.slot.size() ? g.slot.size() - 1 : 0)
                  << (g.slot.empty() ? "[j]" : " * VEC + j]") << " = " << vn(s.id) << ";\n";
        }
        for (int si : sinks) {
            const Stmt& s = p.stmts[si];
            if (s.kind == S_RED && red_from_arg.count(si)) {
                // nothing here: the value is taken from the arg-reduction's pair after the loop
            } else if (s.kind == S_RED) {
                o << in2 << "acc" << si << g.acc_suffix << " = " << red_struct(s.name) << "::apply(acc" << si
                  << g.acc_suffix << ", " << vn(s.in[0]) << ");\n";
            } else if (s.kind == S_ARGRED) {
                const Stmt& src = val(s.in[0]);
                if (!g.argred_defer.empty())
                    o << in2 << "av" << si << g.argred_defer << "[j] = " << vn(s.in[0]) << ";\n";
                else
                    o << in2 << "arg_take<" << red_struct(s.name) << ", " << ct(src.dtype) << ">(acc" << si << g.acc_suffix
                      << ", " << vn(s.in[0]) << ", (i64)(" << g.argred_index << "));\n";
            } else if (s.kind == S_ST) {
                std::string old = argvec(s.arg) + ".x[j]";
                o << in2 << "out" << si << ".x[j] = (" << argT(s.arg) << ")(" << assign_rhs(s.aop, old, vn(s.in[0])) << ");\n";
            } else if (s.kind == S_STX) {
                const std::string addr = "&a" + std::to_string(s.arg) + "[ro" + std::to_string(s.arg) + " + " +
                                         col_off(s.arg, g.c + " + j") + " + (i64)" + vn(s.in[0]) + " * " +
                                         W(L.arg_xs(s.arg)) + "]";
                const std::string val_ = vn(s.in[1]);
                switch (s.aop) {
                    case A_ASSIGN: o << in2 << "atomic_exch(" << addr << ", " << val_ << ");\n"; break;
                    case A_ADD: o << in2 << "atomic_add(" << addr << ", " << val_ << ");\n"; break;
                    case A_SUB: o << in2 << "atomic_add(" << addr << ", -" << val_ << ");\n"; break;
                    case A_MUL: o << in2 << "atomic_exch(" << addr << ", *" << addr << " * " << val_ << ");\n"; break;
                    case A_DIV: o << in2 << "atomic_exch(" << addr << ", *" << addr << " / " << val_ << ");\n"; break;
                }
            }
        }
        o << ind << "}\n";
        for (int si : sinks) {
            const Stmt& s = p.stmts[si];
            if (s.kind == S_ST) emit_arg_store(ind, s.arg, "out" + std::to_string(si), g.c);
        }
    }

    // ---- row-level statements of stage q (loads of R args, functors, stores) ----
    // `valid` guards memory accesses; `oidx` is appended to nothing (row kinds keep
    // scalars).  Reduction results must already be in r<id>.
    void emit_row_values(const std::string& ind, int q, const std::string& valid, bool leader_only_stores,
                         const std::string& leader) {
        for (size_t i = 0; i < p.stmts.size(); ++i) {
            const Stmt& s = p.stmts[i];
            if (s.elem || s.stage != q) continue;
            if (s.kind == S_LD) {
                o << ind << "const " << ct(s.dtype) << " " << vn(s.id) << " = " << valid << " ? (" << ct(s.dtype) << ")a" << s.arg << "[ro"
                  << s.arg << "] : (" << ct(s.dtype) << ")0;\n";
            } else if (s.kind == S_LDX) {
                o << ind << "const " << ct(s.dtype) << " " << vn(s.id) << " = " << valid << " ? (" << ct(s.dtype) << ")a" << s.arg << "[ro"
                  << s.arg << " + (i64)" << vn(s.in[0]) << " * " << W(L.arg_xs(s.arg)) << "] : (" << ct(s.dtype)
                  << ")0;\n";
            } else if (s.kind == S_OP || s.kind == S_CAST) {
                o << ind << "const " << ct(s.dtype) << " " << vn(s.id) << " = " << expr(s) << ";\n";
            } else if (s.kind == S_ST) {
                const std::string dst = "a" + std::to_string(s.arg) + "[ro" + std::to_string(s.arg) + "]";
                o << ind << "if (" << valid << (leader_only_stores ? " && " + leader : "") << ") " << dst << " = ("
                  << argT(s.arg) << ")(" << assign_rhs(s.aop, dst, vn(s.in[0])) << ");\n";
                continue;
            } else if (s.kind == S_STX) {
                const std::string addr = "&a" + std::to_string(s.arg) + "[ro" + std::to_string(s.arg) + " + (i64)" +
                                         vn(s.in[0]) + " * " + W(L.arg_xs(s.arg)) + "]";
                o << ind << "if (" << valid << (leader_only_stores ? " && " + leader : "") << ") ";
                switch (s.aop) {
                    case A_ASSIGN: o << "atomic_exch(" << addr << ", " << vn(s.in[1]) << ");\n"; break;
                    case A_ADD: o << "atomic_add(" << addr << ", " << vn(s.in[1]) << ");\n"; break;
                    case A_SUB: o << "atomic_add(" << addr << ", -" << vn(s.in[1]) << ");\n"; break;
                    case A_MUL: o << "atomic_exch(" << addr << ", *" << addr << " * " << vn(s.in[1]) << ");\n"; break;
                    case A_DIV: o << "atomic_exch(" << addr << ", *" << addr << " / " << vn(s.in[1]) << ");\n"; break;
                }
                continue;
            } else {
                continue;  // SC / CONST emitted in header, reductions by the caller
            }
            if (need_inv.count(s.id)) o << ind << "const float rinv" << s.id << " = 1.0f / " << vn(s.id) << ";\n";
        }
    }

    std::string acc_type(const Stmt& s) const {
        if (s.kind == S_ARGRED) return "ArgPair<" + ct(val(s.in[0]).dtype) + ">";
        return ct(s.dtype);
    }
    std::string acc_init(const Stmt& s) const {
        if (s.kind == S_ARGRED)
            return "arg_init<" + std::string(red_struct(s.name)) + ", " + ct(val(s.in[0]).dtype) + ">()";
        return std::string(red_struct(s.name)) + "::init<" + ct(s.dtype) + ">()";
    }
    std::string acc_merge(const Stmt& s, const std::string& a, const std::string& b) const {
        if (s.kind == S_ARGRED)
            return "arg_merge<" + std::string(red_struct(s.name)) + ", " + ct(val(s.in[0]).dtype) + ">(" + a + ", " + b + ")";
        return std::string(red_struct(s.name)) + "::apply(" + a + ", " + b + ")";
    }
    // final value of a reduction from its accumulator
    std::string acc_result(const Stmt& s, const std::string& a) const {
        if (s.kind == S_ARGRED) return "(int)" + a + ".i";
        return a;
    }

    // ======================================================================= MAP
    // MAP over TS x TS tiles (TS = 32 or 64) for trees that read a transposed operand (class 't': its unit stride runs along the
    // outer dim).  The reference reads such views element by element with a stride (dali/array/jit/array_view.h
    // strided views); here the tile of every transposed operand is read along ITS contiguous direction into shared
    // memory and handed to the threads transposed, so both the reads and the writes are coalesced.
    // The same trees when everything is 4 bytes wide and 16-byte aligned (tile = 4): no shared memory.  A thread owns a
    // 4 x 4 block: four 128-bit loads of a transposed operand along ITS contiguous direction, the transpose happens
    // in registers, four 128-bit stores along the destination's.  A warp is 8 threads along the rows x 4 along the
    // columns, so it reads four full 128-byte lines per load and writes eight 64-byte segments per store.
    bool gen_map_micro(std::string* err) {
        header();
        std::set<int> need = pass_needed(0, false, nullptr);
        std::set<int> largs = args_loaded_in(need, 0);
        o << "  const int lane = tid & 31, warp = tid >> 5;\n";
        o << "  const i64 c = ((i64)blockIdx.x * 32 + warp * 4 + (lane >> 3)) * 4;     // 128 columns per CTA\n";
        o << "  for (i64 rb = ((i64)blockIdx.y * 8 + (lane & 7)) * 4; rb < R; rb += (i64)gridDim.y * 32) {\n";
        o << "    if (c < C) {\n";
        for (int a : largs) {
            if (v.cls[a] != 't') continue;
            o << "      Vec<" << argT(a) << ", 4> t" << a << "_[4];\n";
            o << "      _Pragma(\"unroll\") for (int j = 0; j < 4; ++j) t" << a << "_[j] = vload<" << argT(a) << ", 4>(a" << a
              << " + rb * " << W(L.arg_rs(a, 0)) << " + (c + j) * " << W(L.arg_cs(a, 0, v.nout)) << ");\n";
        }
        o << "      _Pragma(\"unroll\") for (int i = 0; i < 4; ++i) {\n";
        o << "        const i64 r = rb + i;\n";
        row_offsets("        ", "r");
        for (int a : largs) {
            o << "        Vec<" << argT(a) << ", VEC> q" << a << ";\n";
            if (v.cls[a] == 't')
                o << "        _Pragma(\"unroll\") for (int j = 0; j < 4; ++j) q" << a << ".x[j] = t" << a << "_[j].x[i];\n";
            else emit_arg_load("        ", a, "q" + std::to_string(a), "c", false);
        }
        GroupCtx g;
        g.ind = "        ";
        g.c = "c";
        g.skip_loads = true;
        g.hoist_idx = "";
        emit_group(0, need, g);
        o << "      }\n    }\n  }\n}\n";
        (void)err;
        return true;
    }

    bool gen_map_tiled(std::string* err) {
        if (v.tile == 4) return gen_map_micro(err);
        header();
        std::set<int> need = pass_needed(0, false, nullptr);
        std::set<int> largs = args_loaded_in(need, 0);
        o << "#define TS " << v.tile << "\n";
        for (int a : largs)
            if (v.cls[a] == 't') o << "  __shared__ " << argT(a) << " tile" << a << "[TS][TS + 1];\n";
        o << "  const int tx = tid & 31, ty = tid >> 5;      // 32 x 8 threads, TS * TS / 256 elements of the tile each\n";
        o << "  const i64 c0 = (i64)blockIdx.x * TS;\n";
        o << "  for (i64 r0 = (i64)blockIdx.y * TS; r0 < R; r0 += (i64)gridDim.y * TS) {\n";
        for (int a : largs) {
            if (v.cls[a] != 't') continue;
            o << "    _Pragma(\"unroll\") for (int k = 0; k < TS / 8; ++k)\n";
            o << "      _Pragma(\"unroll\") for (int j = 0; j < TS / 32; ++j) {\n";
            o << "        const i64 sc = c0 + ty + 8 * k, sr = r0 + tx + 32 * j;     // consecutive threads walk the outer dim\n";
            o << "        tile" << a << "[ty + 8 * k][tx + 32 * j] = (sc < C && sr < R) ? a" << a << "[sr * " << W(L.arg_rs(a, 0)) << " + sc * "
              << W(L.arg_cs(a, 0, v.nout)) << "] : (" << argT(a) << ")0;\n";
            o << "      }\n";
        }
        o << "    __syncthreads();\n";
        o << "    _Pragma(\"unroll\") for (int k = 0; k < TS / 8; ++k) {\n";
        o << "      const i64 r = r0 + ty + 8 * k;\n";
        o << "      if (r < R) {\n";
        row_offsets("        ", "r");
        o << "        _Pragma(\"unroll\") for (int j = 0; j < TS / 32; ++j) {\n";
        o << "          const i64 c = c0 + tx + 32 * j;\n";
        o << "          if (c < C) {\n";
        for (int a : largs) {
            o << "            Vec<" << argT(a) << ", VEC> q" << a << ";\n";
            if (v.cls[a] == 't') o << "            q" << a << ".x[0] = tile" << a << "[tx + 32 * j][ty + 8 * k];\n";
            else emit_arg_load("            ", a, "q" + std::to_string(a), "c", false);
        }
        GroupCtx g;
        g.ind = "            ";
        g.c = "c";
        g.skip_loads = true;
        g.hoist_idx = "";
        emit_group(0, need, g);
        o << "          }\n        }\n      }\n    }\n    __syncthreads();\n  }\n}\n";
        (void)err;
        return true;
    }

    bool gen_map(std::string* err) {
        if (p.nreduce != 0) { *err = "map skeleton needs nreduce = 0"; return false; }
        if (v.tile) return gen_map_tiled(err);
        header();
        std::set<int> need = pass_needed(0, false, nullptr);
        std::set<int> largs = args_loaded_in(need, 0);
        o << "  const int txl = (int)" << W(L.w_aux0) << ";\n";
        o << "  const int TX = 1 << txl, TY = NT >> txl;\n";
        o << "  const int tx = tid & (TX - 1), ty = tid >> txl;\n";
        o << "  const i64 cbase = ((i64)blockIdx.x * UNROLL * TX + tx) * VEC;\n";
        o << "  const i64 cstep = (i64)TX * VEC;\n";
        o << "  for (i64 r = (i64)blockIdx.y * TY + ty; r < R; r += (i64)gridDim.y * TY) {\n";
        row_offsets("    ", "r");
        bool hoist = v.nin == 1 && v.unroll > 1;
        if (hoist) {
            for (int a : largs) o << "    Vec<" << argT(a) << ", VEC> q" << a << "[UNROLL];\n";
            o << "    _Pragma(\"unroll\") for (int u = 0; u < UNROLL; ++u) {\n";
            o << "      const i64 c = cbase + u * cstep;\n      if (c < C) {\n";
            for (int a : largs) emit_arg_load("        ", a, "q" + std::to_string(a) + "[u]", "c", false);
            o << "      }\n    }\n";
        }
        o << "    _Pragma(\"unroll\") for (int u = 0; u < UNROLL; ++u) {\n";
        o << "      const i64 c = cbase + u * cstep;\n      if (c < C) {\n";
        GroupCtx g;
        g.ind = "        ";
        g.c = "c";
        g.skip_loads = hoist;
        g.hoist_idx = "[u]";
        emit_group(0, need, g);
        o << "      }\n    }\n  }\n}\n";
        return true;
    }

    // ======================================================================= ROW
    bool gen_row(std::string* err) {
        if (p.nreduce == 0) { *err = "row skeleton needs nreduce > 0"; return false; }
        const int T = v.T;
        const bool cached = v.vpt > 0;
        header();
        o << "#define TROW " << T << "\n#define RPC (NT / TROW)\n#define VPT " << std::max(v.vpt, 1) << "\n";
        o << "  const int lane = tid % TROW;\n  const int sub = tid / TROW;\n";
        const int npass = n_passes();
        // shared buffers: one per reduction, double-buffered by row-iteration parity
        for (int si : reds) {
            const Stmt& s = p.stmts[si];
            if (T > 32) o << "  __shared__ " << acc_type(s) << " sm" << si << "[2][NT / 32];\n";
        }
        const bool clustered = v.cluster > 1;
        if (clustered) {
            if (cached || v.threads != T || v.nin != 1) { *err = "cluster rows: one streaming CTA per row slice"; return false; }
            o << "#define CL " << v.cluster << "\n";
            o << "  const unsigned cl_rank = cluster_rank();\n";
            o << "  const i64 cl_per = ((C + (i64)CL * VEC - 1) / ((i64)CL * VEC)) * VEC;     // columns per CTA of the cluster\n";
            o << "  const i64 cl_lo = (i64)cl_rank * cl_per;\n";
            o << "  const i64 cl_hi = cl_lo + cl_per < C ? cl_lo + cl_per : C;\n";
            for (int si : reds) o << "  __shared__ " << acc_type(p.stmts[si]) << " cx" << si << "[2][CL];\n";
        }
        // cut analysis for the cached variant
        std::vector<std::set<int>> cuts(npass + 1);
        std::set<int> all_cuts;
        if (cached)
            for (int q = 0; q < npass; ++q) {
                pass_needed(q, true, &cuts[q]);
                all_cuts.insert(cuts[q].begin(), cuts[q].end());
            }
        std::set<int> eargs;
        if (cached) {
            for (const Stmt& s : p.stmts)
                if (s.kind == S_LD && s.elem) eargs.insert(s.arg);
            for (const Stmt& s : p.stmts)
                if (s.kind == S_ST && s.elem && s.aop != A_ASSIGN) eargs.insert(s.arg);
        }
        // Staging: every warp owns a ring of STAGES rows (per operand) in shared memory.  Lane 0 issues one bulk
        // asynchronous copy per row and operand (cp.async.bulk, completion counted in bytes on the slot's mbarrier),
        // STAGES rows ahead of the row the warp works on; the warp waits on the slot, moves the row into registers and
        // hands the slot straight back to the copy engine.  Warps never synchronise with one another, so loads, the
        // reduction chain and the stores of different rows overlap for the whole launch.
        const bool staged = cached && v.stage > 0;
        if (staged) {
            if (T != 32 || v.nin != 1) { *err = "staged rows need one warp per row"; return false; }
            o << "#define STAGES " << v.stage << "\n";
            o << "  extern __shared__ __align__(128) unsigned char st_ring[];\n";
            o << "  __shared__ unsigned long long st_bar[RPC][STAGES];\n";
            o << "  const i64 st_slot = " << W(L.w_aux0) << ";        // bytes between two slots of the ring (a row, padded to 128 bytes)\n";
            o << "  const i64 st_step = (i64)gridDim.x * RPC;        // rows between two consecutive rows of a warp\n";
            int k = 0;
            for (int a : eargs) {
                o << "  unsigned char* const st_base" << a << " = st_ring + ((i64)" << k++ << " * RPC + sub) * STAGES * st_slot;\n";
                o << "  const unsigned st_bytes" << a << " = (unsigned)(C * sizeof(" << argT(a) << "));\n";
            }
            o << "  unsigned st_total = 0;\n";
            for (int a : eargs) o << "  st_total += st_bytes" << a << ";\n";
            o << "  if (lane == 0) { _Pragma(\"unroll\") for (int d = 0; d < STAGES; ++d) stage_bar_init(&st_bar[sub][d]); }\n";
            o << "  stage_fence_init();\n  __syncwarp();\n";
            // (kernel_entry(), the wait on the kernel before this one in the stream, has run: global memory may be read)
            o << "  if (lane == 0) {\n    _Pragma(\"unroll\") for (int d = 0; d < STAGES; ++d) {\n";
            o << "      const i64 pf_r = (i64)blockIdx.x * RPC + sub + d * st_step;\n      if (pf_r < R) {\n";
            row_offsets("        ", "pf_r", "rn");
            o << "        stage_expect(&st_bar[sub][d], st_total);\n";
            for (int a : eargs)
                o << "        stage_copy(st_base" << a << " + d * st_slot, a" << a << " + rn" << a << ", st_bytes" << a << ", &st_bar[sub][d]);\n";
            o << "      }\n    }\n  }\n";
            o << "  int st_it = 0;\n";
        }
        o << "  int parity = 0;\n";
        if (clustered)
            o << "  for (i64 rbase = (i64)(blockIdx.x / CL); rbase < R; rbase += (i64)(gridDim.x / CL), parity ^= 1) {\n";
        else
        o << "  for (i64 rbase = (i64)blockIdx.x * RPC; rbase < R; rbase += (i64)gridDim.x * RPC, parity ^= 1) {\n";
        o << "    const i64 r = rbase + sub;\n    const bool rv = r < R;\n";
        o << "    const i64 rr = rv ? r : 0;\n";
        row_offsets("    ", "rr");
        if (cached) {
            for (int a : eargs) o << "    Vec<" << argT(a) << ", VEC> LQ" << a << "[VPT];\n";
            for (int id : all_cuts) o << "    " << ct(val(id).dtype) << " CV" << id << "[VPT * VEC];\n";
        }
        std::set<int> loaded;
        if (staged) {
            o << "    const int st_d = st_it % STAGES;\n    const unsigned st_par = (unsigned)((st_it / STAGES) & 1);\n    ++st_it;\n";
            o << "    if (rv) stage_wait(&st_bar[sub][st_d], st_par);\n";
            o << "    _Pragma(\"unroll\") for (int i = 0; i < VPT; ++i) {\n";
            o << "      const int c = (i * TROW + lane) * VEC;\n      if (rv && c < (int)C) {\n";
            for (int a : eargs) {
                o << "        LQ" << a << "[i] = *reinterpret_cast<const Vec<" << argT(a) << ", VEC>*>(st_base" << a
                  << " + st_d * st_slot + (i64)c * sizeof(" << argT(a) << "));\n";
                loaded.insert(a);
            }
            o << "      }\n    }\n";
            o << "    __syncwarp();\n";
            o << "    if (lane == 0) {\n      const i64 pf_r = r + STAGES * st_step;\n      if (pf_r < R) {\n";
            row_offsets("        ", "pf_r", "rn");
            o << "        stage_fence_reuse();\n";
            o << "        stage_expect(&st_bar[sub][st_d], st_total);\n";
            for (int a : eargs)
                o << "        stage_copy(st_base" << a << " + st_d * st_slot, a" << a << " + rn" << a << ", st_bytes" << a << ", &st_bar[sub][st_d]);\n";
            o << "      }\n    }\n";
        }
        for (int q = 0; q <= npass; ++q) {
            o << "    // ---- stage " << q << "\n";
            emit_row_values("    ", q, "rv", true, clustered ? "lane == 0 && cl_rank == 0" : "lane == 0");
            if (q == npass) break;
            std::vector<int> sinks = pass_sinks(q);
            if (sinks.empty()) continue;
            for (int si : sinks) {
                const Stmt& s = p.stmts[si];
                if (s.kind == S_RED || s.kind == S_ARGRED)
                    o << "    " << acc_type(s) << " acc" << si << " = " << acc_init(s) << ";\n";
            }
            std::set<int> need = pass_needed(q, cached, nullptr);
            // values of this stage that later passes read from the cache must be computed here
            std::set<int> wr;
            if (cached) {
                for (int id : all_cuts)
                    if (val(id).stage == q) {
                        wr.insert(id);
                        // make sure it (and what it needs) is computed in this pass
                        std::vector<int> stack(1, id);
                        while (!stack.empty()) {
                            int x = stack.back();
                            stack.pop_back();
                            const Stmt& s = val(x);
                            if (!s.elem) continue;
                            if (s.stage < q && s.kind != S_LD) { cuts[q].insert(x); continue; }
                            if (!need.insert(x).second) continue;
                            for (int in : s.in) stack.push_back(in);
                        }
                    }
            }
            GroupCtx g;
            g.argred_index = "c + j";
            if (cached) {
                o << "    _Pragma(\"unroll\") for (int i = 0; i < VPT; ++i) {\n";
                o << "      const int c = (i * TROW + lane) * VEC;\n      if (rv && c < (int)C) {\n";
                g.ind = "        ";
                g.c = "c";
                g.slot = "[i]";
                g.cached = true;
                g.loaded = &loaded;
                g.cuts_rd = cuts[q];
                g.cuts_wr = wr;
                // an arg cached by an earlier pass is not reloaded; emit_group consults `loaded`
                std::set<int> before = loaded;
                emit_group(q, need, g);
                o << "      }\n    }\n";
            } else {
                const std::string lo = clustered ? "(int)cl_lo" : "0", hi = clustered ? "(int)cl_hi" : "(int)C";
                if (v.nin == 1 && v.unroll > 1) {
                    // UNROLL vector groups per thread and step, their loads issued before any of them is used: a
                    // streamed row keeps enough bytes in flight per thread to cover the memory latency
                    std::set<int> largs = args_loaded_in(need, q);
                    o << "    if (rv) for (int cb = " << lo << " + lane * VEC; cb < " << hi << "; cb += TROW * VEC * UNROLL) {\n";
                    for (int a : largs) o << "      Vec<" << argT(a) << ", VEC> q" << a << "[UNROLL];\n";
                    o << "      _Pragma(\"unroll\") for (int u = 0; u < UNROLL; ++u) {\n";
                    o << "        const int c = cb + u * TROW * VEC;\n        if (c < " << hi << ") {\n";
                    for (int a : largs) emit_arg_load("          ", a, "q" + std::to_string(a) + "[u]", "c", false);
                    o << "        }\n      }\n";
                    o << "      _Pragma(\"unroll\") for (int u = 0; u < UNROLL; ++u) {\n";
                    o << "        const int c = cb + u * TROW * VEC;\n        if (c < " << hi << ") {\n";
                    g.ind = "          ";
                    g.c = "c";
                    g.skip_loads = true;
                    g.hoist_idx = "[u]";
                    emit_group(q, need, g);
                    o << "        }\n      }\n    }\n";
                } else {
                    o << "    if (rv) for (int c = " << lo << " + lane * VEC; c < " << hi << "; c += TROW * VEC) {\n";
                    g.ind = "      ";
                    g.c = "c";
                    emit_group(q, need, g);
                    o << "    }\n";
                }
            }
            // combine across the T threads of the row
            for (int si : sinks) {
                const Stmt& s = p.stmts[si];
                if (s.kind != S_RED && s.kind != S_ARGRED) continue;
                const std::string buf = T > 32 ? "sm" + std::to_string(si) + "[parity]" : "nullptr";
                const std::string bufT = T > 32 ? buf : "(" + acc_type(s) + "*)nullptr";
                if (clustered) {
                    // the CTA's slice first, then the slices of the cluster's CTAs in rank order
                    const std::string slots = "cx" + std::to_string(si) + "[parity]";
                    if (s.kind == S_RED)
                        o << "    const " << ct(s.dtype) << " " << vn(s.id) << " = cluster_fold<" << red_struct(s.name) << ", CL>(row_reduce<"
                          << red_struct(s.name) << ", TROW>(acc" << si << ", " << bufT << "), " << slots << ", cl_rank);\n";
                    else
                        o << "    const int " << vn(s.id) << " = (int)cluster_arg_fold<" << red_struct(s.name) << ", CL>(row_arg_reduce<"
                          << red_struct(s.name) << ", TROW>(acc" << si << ", " << bufT << "), " << slots << ", cl_rank).i;\n";
                } else if (s.kind == S_RED)
                    o << "    const " << ct(s.dtype) << " " << vn(s.id) << " = row_reduce<" << red_struct(s.name)
                      << ", TROW>(acc" << si << ", " << bufT << ");\n";
                else
                    o << "    const int " << vn(s.id) << " = (int)row_arg_reduce<" << red_struct(s.name) << ", TROW>(acc"
                      << si << ", " << bufT << ").i;\n";
                if (need_inv.count(s.id)) o << "    const float rinv" << s.id << " = 1.0f / " << vn(s.id) << ";\n";
            }
        }
        o << "  }\n}\n";
        (void)err;
        return true;
    }

    // ======================================================================= ALL
    bool gen_all(std::string* err) {
        if (p.nreduce != p.rank) { *err = "all skeleton needs nreduce = rank"; return false; }
        if (p.max_stage > 1) { *err = "all skeleton handles one level of reductions"; return false; }
        for (const Stmt& s : p.stmts)
            if ((s.kind == S_ST || s.kind == S_STX) && s.elem) { *err = "all skeleton has no element stores"; return false; }
        header();
        for (size_t a = 0; a < p.args.size(); ++a) o << "  const i64 ro" << a << " = 0;\n";
        for (int si : reds) {
            const Stmt& s = p.stmts[si];
            o << "  __shared__ " << acc_type(s) << " sm" << si << "[NT / 32];\n";
            o << "  " << acc_type(s) << " acc" << si << " = " << acc_init(s) << ";\n";
        }
        // row-level values of stage 0 that feed the element work (loads of R args, functors)
        std::set<int> need = pass_needed(0, false, nullptr);
        std::set<int> largs = args_loaded_in(need, 0);
        // stage-0 row values are needed both before (operands) and after; emit those without
        // side effects now, stores later
        for (const Stmt& s : p.stmts) {
            if (s.elem || s.stage != 0) continue;
            if (s.kind == S_LD)
                o << "  const " << ct(s.dtype) << " " << vn(s.id) << " = a" << s.arg << "[0];\n";
            else if (s.kind == S_OP || s.kind == S_CAST)
                o << "  const " << ct(s.dtype) << " " << vn(s.id) << " = " << expr(s) << ";\n";
            else continue;
            if (need_inv.count(s.id)) o << "  const float rinv" << s.id << " = 1.0f / " << vn(s.id) << ";\n";
        }
        o << "  const i64 chunk = (i64)NT * VEC * UNROLL;\n";
        o << "  for (i64 cb = (i64)blockIdx.x * chunk; cb < C; cb += (i64)gridDim.x * chunk) {\n";
        bool hoist = v.nin == 1 && v.unroll > 1;
        // (v.unchecked: a chunk that lies wholly inside the data -- all but the last of the launch -- runs without the
        // per-vector bounds checks, 8 % fewer instructions on the fused chain, which is bound by instruction issue and the
        // power cap: 1.483 against 1.504 ms over 2^31 elements, three alternating runs each)
        // Arg-reductions: taking every element into the (value, position) pair costs a compare and three selects plus the
        // 64-bit position per element.  Instead the chunk's candidates are parked, one maximum (minimum) over all of
        // them decides whether any beats the running value -- after the first chunks almost none does -- and only then
        // are they taken one by one, in order, which keeps the first occurrence.
        std::vector<int> argreds;
        for (int si : reds) if (p.stmts[si].kind == S_ARGRED) argreds.push_back(si);
        auto emit_chunk = [&](bool checked) {
            const std::string guard = checked ? "if (c < C) {\n" : "{\n";
            for (int si : argreds) {
                const Stmt& s = p.stmts[si];
                const std::string T = ct(val(s.in[0]).dtype);
                o << "      " << T << " av" << si << "[UNROLL][VEC];\n";
                o << "      _Pragma(\"unroll\") for (int u = 0; u < UNROLL; ++u) _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) av" << si
                  << "[u][j] = " << red_struct(s.name) << "::init<" << T << ">();\n";
            }
            if (hoist) {
                for (int a : largs) o << "      Vec<" << argT(a) << ", VEC> q" << a << "[UNROLL];\n";
                o << "      _Pragma(\"unroll\") for (int u = 0; u < UNROLL; ++u) {\n";
                o << "        const i64 c = cb + ((i64)u * NT + tid) * VEC;\n        " << guard;
                for (int a : largs) emit_arg_load("          ", a, "q" + std::to_string(a) + "[u]", "c", false);
                o << "        }\n      }\n";
            }
            o << "      _Pragma(\"unroll\") for (int u = 0; u < UNROLL; ++u) {\n";
            o << "        const i64 c = cb + ((i64)u * NT + tid) * VEC;\n        " << guard;
            GroupCtx g;
            g.ind = "          ";
            g.c = "c";
            g.skip_loads = hoist;
            g.hoist_idx = "[u]";
            g.argred_index = "c + j";
            if (!argreds.empty()) g.argred_defer = "[u]";
            emit_group(0, need, g);
            o << "        }\n      }\n";
            for (int si : argreds) {
                const Stmt& s = p.stmts[si];
                const std::string T = ct(val(s.in[0]).dtype), R = red_struct(s.name);
                o << "      {\n        " << T << " m_ = av" << si << "[0][0];\n";
                o << "        _Pragma(\"unroll\") for (int u = 0; u < UNROLL; ++u) _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) m_ = "
                  << R << "::pick(m_, av" << si << "[u][j]);\n";
                o << "        if (" << R << "::better(m_, acc" << si << ".v)) {\n";
                o << "          _Pragma(\"unroll\") for (int u = 0; u < UNROLL; ++u) {\n";
                o << "            const i64 c = cb + ((i64)u * NT + tid) * VEC;\n";
                o << "            _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) arg_take<" << R << ", " << T << ">(acc" << si << ", av"
                  << si << "[u][j], c + j);\n";
                o << "          }\n        }\n      }\n";
            }
        };
        if (v.unchecked) {
            o << "    if (cb + chunk <= C) {\n";
            emit_chunk(false);
            o << "    } else {\n";
            emit_chunk(true);
            o << "    }\n  }\n";
        } else {
            o << "    {\n";
            emit_chunk(true);
            o << "    }\n  }\n";
        }
        for (const auto& ra : red_from_arg) o << "  acc" << ra.first << " = acc" << ra.second << ".v;\n";
        // CTA partials
        for (int si : reds) {
            const Stmt& s = p.stmts[si];
            if (s.kind == S_RED)
                o << "  acc" << si << " = block_reduce<" << red_struct(s.name) << ", NT>(acc" << si << ", sm" << si << ");\n";
            else
                o << "  acc" << si << " = block_arg_reduce<" << red_struct(s.name) << ", NT>(acc" << si << ", sm" << si << ");\n";
        }
        // cross-CTA exchange through scratch; the last CTA to arrive finishes
        o << "  if (gridDim.x > 1) {\n";
        o << "    __shared__ bool is_last;\n";
        o << "    char* const scratch = reinterpret_cast<char*>(" << W(L.w_scratch) << ");\n";
        o << "    u32* const counter = reinterpret_cast<u32*>(" << W(L.w_counter) << ");\n";
        size_t off = 0;
        std::vector<size_t> offs;
        for (int si : reds) {
            offs.push_back(off);
            off += 16;   // one 16-byte slot per reduction per CTA
        }
        o << "    const i64 stride = " << off << ";\n";
        o << "    if (tid == 0) {\n";
        for (size_t k = 0; k < reds.size(); ++k) {
            const Stmt& s = p.stmts[reds[k]];
            o << "      *reinterpret_cast<" << acc_type(s) << "*>(scratch + blockIdx.x * stride + " << offs[k]
              << ") = acc" << reds[k] << ";\n";
        }
        o << "      __threadfence();\n";
        o << "      const u32 t = atomicInc(counter, gridDim.x - 1);\n";
        o << "      is_last = (t == gridDim.x - 1);\n    }\n";
        o << "    __syncthreads();\n    if (!is_last) return;\n    __threadfence();\n";
        for (size_t k = 0; k < reds.size(); ++k) {
            const Stmt& s = p.stmts[reds[k]];
            int si = reds[k];
            o << "    acc" << si << " = " << acc_init(s) << ";\n";
            o << "    for (u32 b = tid; b < gridDim.x; b += NT) acc" << si << " = "
              << acc_merge(s, "acc" + std::to_string(si),
                           "ld_cg(reinterpret_cast<const " + acc_type(s) + "*>(scratch + b * stride + " +
                               std::to_string(offs[k]) + "))")
              << ";\n";
            o << "    __syncthreads();\n";
            if (s.kind == S_RED)
                o << "    acc" << si << " = block_reduce<" << red_struct(s.name) << ", NT>(acc" << si << ", sm" << si << ");\n";
            else
                o << "    acc" << si << " = block_arg_reduce<" << red_struct(s.name) << ", NT>(acc" << si << ", sm" << si << ");\n";
        }
        o << "  }\n";
        if (p.has_xrank) {
            // One CTA of the launch reaches this point holding the rank's results.  Thread r stores them into this
            // rank's slot on rank r (plain stores into peer memory over NVLink), raises the slot's flag there to this
            // call's epoch and waits -- bounded -- until rank r's results have arrived in this GPU's own block; then
            // every thread folds the slots of the own block in rank order, the same order on every rank.
            int k = 0;
            for (int si : reds) if (p.stmts[si].xrank) ++k;
            if (k * 16 > 256) { *err = "more than 16 cross-rank reductions in one kernel"; return false; }
            o << "  {\n";
            o << "    const DaliPeerTable* const pt = reinterpret_cast<const DaliPeerTable*>(" << W(L.w_aux0) << ");\n";
            o << "    __shared__ unsigned long long xr_epoch;\n";
            o << "    if (tid == 0) xr_epoch = pt->epoch[1] + 1;\n";
            o << "    __syncthreads();\n";
            o << "    const unsigned long long epoch = xr_epoch;\n";
            o << "    const int parity = (int)(epoch & 1);\n";
            for (int si : reds) {
                const Stmt& s = p.stmts[si];
                if (s.xrank && s.kind == S_ARGRED && s.xrank_offset >= 0)
                    o << "    acc" << si << ".i += (i64)" << vn(s.xrank_offset) << ";\n";
            }
            o << "    if (tid < pt->world) {\n";
            o << "      char* const slot = dali_peer_fused_slot(pt->block[tid], parity, pt->rank);\n";
            k = 0;
            for (int si : reds) {
                const Stmt& s = p.stmts[si];
                if (!s.xrank) continue;
                o << "      *reinterpret_cast<" << acc_type(s) << "*>(slot + " << 16 * k++ << ") = acc" << si << ";\n";
            }
            o << "      __threadfence_system();\n";
            o << "      dali_peer_flag_release(dali_peer_fused_flag(pt->block[tid], parity, pt->rank), epoch);\n";
            o << "      dali_peer_wait(dali_peer_fused_flag(pt->block[pt->rank], parity, tid), epoch, pt->wait_ns, pt->error);\n";
            o << "    }\n";
            o << "    __syncthreads();\n";
            k = 0;
            for (int si : reds) {
                const Stmt& s = p.stmts[si];
                if (!s.xrank) continue;
                const std::string at = "reinterpret_cast<const " + acc_type(s) + "*>(dali_peer_fused_slot(pt->block[pt->rank], parity, r_) + " +
                                       std::to_string(16 * k++) + ")";
                o << "    { int r_ = 0; acc" << si << " = ld_cg(" << at << ");\n";
                o << "      for (r_ = 1; r_ < pt->world; ++r_) acc" << si << " = " << acc_merge(s, "acc" + std::to_string(si), "ld_cg(" + at + ")") << "; }\n";
            }
            o << "    __syncthreads();\n";
            o << "    if (tid == 0) pt->epoch[1] = epoch;\n";
            o << "  }\n";
        }
        for (int si : reds) {
            const Stmt& s = p.stmts[si];
            o << "  const " << ct(s.dtype) << " " << vn(s.id) << " = " << acc_result(s, "acc" + std::to_string(si)) << ";\n";
            if (need_inv.count(s.id)) o << "  const float rinv" << s.id << " = 1.0f / " << vn(s.id) << ";\n";
        }
        // stage-0 stores (rare) and stage-1 row values + stores
        for (const Stmt& s : p.stmts) {
            if (s.elem || s.stage != 0 || (s.kind != S_ST && s.kind != S_STX)) continue;
            const std::string dst = "a" + std::to_string(s.arg) + "[0]";
            if (s.kind == S_ST) o << "  if (tid == 0) " << dst << " = (" << argT(s.arg) << ")(" << assign_rhs(s.aop, dst, vn(s.in[0])) << ");\n";
        }
        emit_row_values("  ", 1, "true", true, "tid == 0");
        o << "}\n";
        return true;
    }

    // ======================================================================= COL
    bool gen_col(std::string* err) {
        if (p.nreduce == 0 || v.nout != 1 || v.nin != 1) { *err = "col skeleton needs one outer and one reduced dim"; return false; }
        if (p.max_stage > 1) { *err = "col skeleton handles one level of reductions"; return false; }
        if (p.has_indirect) { *err = "col skeleton has no indirect access"; return false; }
        for (const Stmt& s : p.stmts)
            if ((s.kind == S_ST || s.kind == S_STX) && s.elem) { *err = "col skeleton has no element stores"; return false; }
        header();
        o << "#define TXO " << v.tx << "\n#define TYI " << v.ty << "\n";
        o << "  const int tx = tid % TXO, ty = tid / TXO;\n";
        o << "  const i64 o0 = ((i64)blockIdx.x * TXO + tx) * VEC;\n";
        o << "  const bool ov = o0 < R;\n";
        o << "  const i64 per = " << W(L.w_aux0) << ";\n";
        o << "  const i64 c0 = (i64)blockIdx.y * per;\n";
        o << "  const i64 c1 = (c0 + per < C) ? c0 + per : C;\n";
        for (int si : reds) {
            const Stmt& s = p.stmts[si];
            o << "  __shared__ " << acc_type(s) << " sm" << si << "[TYI][TXO * VEC];\n";
            o << "  " << acc_type(s) << " acc" << si << "[VEC];\n";
            o << "  _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) acc" << si << "[j] = " << acc_init(s) << ";\n";
        }
        // per-arg base along the outer dim: ro<a> points at outer index o0
        for (size_t a = 0; a < p.args.size(); ++a)
            o << "  const i64 ro" << a << " = (ov ? o0 : 0) * " << W(L.arg_rs((int)a, 0)) << ";\n";
        std::set<int> need = pass_needed(0, false, nullptr);
        std::set<int> largs = args_loaded_in(need, 0);
        // row-level stage-0 values used inside the loop must not vary with the outer
        // index here unless they come from R args; those are loaded per lane below
        std::set<int> r0_in_loop;
        for (int id : need)
            for (int in : val(id).in)
                if (!val(in).elem && val(in).kind != S_SC && val(in).kind != S_CONST) r0_in_loop.insert(in);
        if (!r0_in_loop.empty()) { *err = "col skeleton: element work may not use row-level loads"; return false; }
        // arg-reductions: the rows in flight are parked and one maximum (minimum) per column decides whether any of them
        // beats the column's running value (see the all-axis skeleton); the running sums / extremes of plain
        // reductions in the same program go on as before
        std::vector<int> argreds;
        for (int si : reds) if (p.stmts[si].kind == S_ARGRED) argreds.push_back(si);
        const bool defer = !argreds.empty();
        o << "  if (ov) {\n";
        if (defer) {
            o << "    for (i64 cb = c0 + ty; cb < c1; cb += (i64)TYI * " << v.unroll << ") {\n";
            for (int si : argreds) {
                const Stmt& s = p.stmts[si];
                const std::string T = ct(val(s.in[0]).dtype);
                o << "    " << T << " av" << si << "[" << v.unroll << "][VEC];\n";
                o << "    _Pragma(\"unroll\") for (int u = 0; u < " << v.unroll << "; ++u) _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) av"
                  << si << "[u][j] = " << red_struct(s.name) << "::init<" << T << ">();\n";
            }
            o << "    _Pragma(\"unroll\") for (int u = 0; u < " << v.unroll << "; ++u) {\n";
            o << "    const i64 c = cb + (i64)u * TYI;\n";
            o << "    if (c < c1) {\n";
        } else {
            o << "    _Pragma(\"unroll " << v.unroll << "\") for (i64 c = c0 + ty; c < c1; c += TYI) {\n";
        }
        for (int a : largs) {
            const std::string T = argT(a);
            char oc = v.ocls[a];
            const std::string coff = v.cls[a] == 'z' ? "0" : (v.cls[a] == 'u' ? "c" : "c * " + W(L.arg_cs(a, 0, v.nout)));
            o << "      Vec<" << T << ", VEC> q" << a << ";\n";
            if (v.vec > 1 && oc == 'u')
                o << "      q" << a << " = vload<" << T << ", VEC>(a" << a << " + ro" << a << " + " << coff << ");\n";
            else if (oc == 'z')
                o << "      { const " << T << " t_ = a" << a << "[" << coff << "]; _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) q"
                  << a << ".x[j] = t_; }\n";
            else
                o << "      _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) q" << a << ".x[j] = a" << a << "[ro" << a
                  << " + j * " << W(L.arg_rs(a, 0)) << " + " << coff << "];\n";
        }
        {
            GroupCtx g;
            g.ind = "      ";
            g.c = "c";
            g.skip_loads = true;
            g.hoist_idx = "";
            g.acc_suffix = "[j]";
            g.argred_index = "c";
            if (defer) g.argred_defer = "[u]";
            // emit_group's lane loop walks j over the OUTER lanes here
            emit_group(0, need, g);
        }
        if (defer) {
            o << "    }\n    }\n";      // if (c < c1), for u
            for (int si : argreds) {
                const Stmt& s = p.stmts[si];
                const std::string T = ct(val(s.in[0]).dtype), R = red_struct(s.name);
                o << "    _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) {\n";
                o << "      " << T << " m_ = av" << si << "[0][j];\n";
                o << "      _Pragma(\"unroll\") for (int u = 1; u < " << v.unroll << "; ++u) m_ = " << R << "::pick(m_, av" << si << "[u][j]);\n";
                o << "      if (" << R << "::better(m_, acc" << si << "[j].v)) {\n";
                o << "        _Pragma(\"unroll\") for (int u = 0; u < " << v.unroll << "; ++u) arg_take<" << R << ", " << T << ">(acc" << si
                  << "[j], av" << si << "[u][j], cb + (i64)u * TYI);\n";
                o << "      }\n    }\n";
            }
        }
        o << "    }\n  }\n";
        for (const auto& ra : red_from_arg)
            o << "  _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) acc" << ra.first << "[j] = acc" << ra.second << "[j].v;\n";
        // fold the TYI slices of the CTA
        for (int si : reds) {
            const Stmt& s = p.stmts[si];
            o << "  _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) sm" << si << "[ty][tx * VEC + j] = acc" << si << "[j];\n";
            (void)s;
        }
        o << "  __syncthreads();\n";
        o << "  if (ty == 0) {\n";
        for (int si : reds) {
            const Stmt& s = p.stmts[si];
            o << "    _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) {\n      " << acc_type(s) << " t_ = sm" << si
              << "[0][tx * VEC + j];\n      for (int k = 1; k < TYI; ++k) t_ = "
              << acc_merge(s, "t_", "sm" + std::to_string(si) + "[k][tx * VEC + j]") << ";\n      acc" << si
              << "[j] = t_;\n    }\n";
        }
        o << "  }\n";
        // cross-CTA: slices of the reduced dim meet in scratch, last CTA of the tile finishes
        o << "  if (gridDim.y > 1) {\n";
        o << "    __shared__ bool is_last;\n";
        o << "    char* const scratch = reinterpret_cast<char*>(" << W(L.w_scratch) << ");\n";
        o << "    u32* const counter = reinterpret_cast<u32*>(" << W(L.w_counter) << ");\n";
        o << "    const i64 Rpad = (i64)gridDim.x * TXO * VEC;\n";
        for (size_t k = 0; k < reds.size(); ++k) {
            const Stmt& s = p.stmts[reds[k]];
            o << "    " << acc_type(s) << "* const part" << reds[k] << " = reinterpret_cast<" << acc_type(s)
              << "*>(scratch + " << k << " * (i64)gridDim.y * Rpad * 16);\n";
        }
        o << "    if (ty == 0) {\n";
        for (int si : reds)
            o << "      _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) part" << si << "[(i64)blockIdx.y * Rpad + o0 + j] = acc" << si
              << "[j];\n";
        o << "    }\n";
        o << "    __threadfence();\n    __syncthreads();\n";
        o << "    if (tid == 0) { const u32 t = atomicInc(counter + blockIdx.x, gridDim.y - 1); is_last = (t == gridDim.y - 1); }\n";
        o << "    __syncthreads();\n    if (!is_last) return;\n    __threadfence();\n";
        // every thread folds the slices sl = ty, ty + TYI, ... of its outer lanes (independent
        // loads in flight instead of one serial chain), then the TYI partial folds meet in
        // shared memory in slice order
        for (int si : reds) {
            const Stmt& s = p.stmts[si];
            o << "    _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) {\n      " << acc_type(s) << " t_ = "
              << acc_init(s) << ";\n      if (ov) { _Pragma(\"unroll 4\") for (u32 sl = ty; sl < gridDim.y; sl += TYI) t_ = "
              << acc_merge(s, "t_", "ld_cg(&part" + std::to_string(si) + "[(i64)sl * Rpad + o0 + j])")
              << "; }\n      sm" << si << "[ty][tx * VEC + j] = t_;\n    }\n";
        }
        o << "    __syncthreads();\n";
        o << "    if (ty == 0) {\n";
        for (int si : reds) {
            const Stmt& s = p.stmts[si];
            o << "      _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) {\n        " << acc_type(s) << " t_ = sm" << si
              << "[0][tx * VEC + j];\n        for (int k = 1; k < TYI; ++k) t_ = "
              << acc_merge(s, "t_", "sm" + std::to_string(si) + "[k][tx * VEC + j]") << ";\n        acc" << si
              << "[j] = t_;\n      }\n";
        }
        o << "    }\n  }\n";
        // finish: row-level values and stores per outer index
        o << "  if (ty == 0 && ov) {\n";
        o << "    _Pragma(\"unroll\") for (int j = 0; j < VEC; ++j) {\n";
        for (size_t a = 0; a < p.args.size(); ++a)
            o << "      const i64 fo" << a << " = (o0 + j) * " << W(L.arg_rs((int)a, 0)) << ";\n";
        // shadow ro<a> with the per-lane offsets for emit_row_values
        o << "      {\n";
        for (size_t a = 0; a < p.args.size(); ++a) o << "        const i64 ro" << a << " = fo" << a << ";\n";
        for (int si : reds) {
            const Stmt& s = p.stmts[si];
            o << "        const " << ct(s.dtype) << " " << vn(s.id) << " = "
              << acc_result(s, "acc" + std::to_string(si) + "[j]") << ";\n";
            if (need_inv.count(s.id)) o << "        const float rinv" << s.id << " = 1.0f / " << vn(s.id) << ";\n";
        }
        emit_row_values("        ", 0, "true", false, "");
        emit_row_values("        ", 1, "true", false, "");
        o << "      }\n    }\n  }\n}\n";
        return true;
    }
};

}  // namespace

bool generate_kernel(const Program& p, const Variant& v, std::string* src, std::string* err) {
    if ((int)v.cls.size() != (int)p.args.size()) { *err = "variant: one inner-stride class per arg expected"; return false; }
    if (v.kind == K_COL && v.ocls.size() != p.args.size()) { *err = "variant: one outer-stride class per arg expected"; return false; }
    Gen g(p, v);
    bool ok = false;
    switch (v.kind) {
        case K_MAP: ok = g.gen_map(err); break;
        case K_ROW: ok = g.gen_row(err); break;
        case K_ALL: ok = g.gen_all(err); break;
        case K_COL: ok = g.gen_col(err); break;
    }
    if (ok) *src = g.o.str();
    return ok;
}

}  // namespace dalib
