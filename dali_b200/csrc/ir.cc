// Parser and static analysis of the fused-expression IR (see ir.h).
#include "ir.h"

#include <cstdlib>
#include <set>
#include <sstream>

namespace dalib {

const char* dtype_ir_name(DType t) {
    switch (t) {
        case F32: return "f32";
        case F64: return "f64";
        case I32: return "i32";
        case BF16: return "bf16";
    }
    return "?";
}

const char* dtype_c_name(DType t) {
    switch (t) {
        case F32: return "float";
        case F64: return "double";
        case I32: return "int";
        case BF16: return "bf16_t";
    }
    return "?";
}

int dtype_size(DType t) {
    switch (t) {
        case F32: return 4;
        case F64: return 8;
        case I32: return 4;
        case BF16: return 2;
    }
    return 0;
}

namespace {

bool parse_dtype(const std::string& s, DType* out) {
    if (s == "f32") { *out = F32; return true; }
    if (s == "f64") { *out = F64; return true; }
    if (s == "i32") { *out = I32; return true; }
    return false;   // bf16 is a storage type of args only, never an IR value type
}

bool parse_arg_dtype(const std::string& s, DType* out) {
    if (s == "bf16") { *out = BF16; return true; }
    return parse_dtype(s, out);
}

bool parse_value_ref(const std::string& s, int* out) {
    if (s.size() < 2 || s[0] != 'v') return false;
    for (size_t i = 1; i < s.size(); ++i) if (s[i] < '0' || s[i] > '9') return false;
    *out = std::atoi(s.c_str() + 1);
    return true;
}

bool parse_int(const std::string& s, int* out) {
    if (s.empty()) return false;
    size_t i = 0;
    if (s[0] == '-') i = 1;
    if (i == s.size()) return false;
    for (; i < s.size(); ++i) if (s[i] < '0' || s[i] > '9') return false;
    *out = std::atoi(s.c_str());
    return true;
}

bool parse_assign_op(const std::string& s, AssignOp* out) {
    if (s == "assign") { *out = A_ASSIGN; return true; }
    if (s == "add") { *out = A_ADD; return true; }
    if (s == "sub") { *out = A_SUB; return true; }
    if (s == "mul") { *out = A_MUL; return true; }
    if (s == "div") { *out = A_DIV; return true; }
    return false;
}

// functor name -> arity; the names are those of dali/array/functor.h:27-495
// without the "functor::" prefix ("ceiling" is what op::ceil asks for,
// dali/array/op/elementwise_operation.cpp:159).
int functor_arity(const std::string& n) {
    static const char* unary[] = {
        "identity", "square", "cube", "sqrt_f", "rsqrt", "inv", "sigmoid", "dsigmoid", "tanh",
        "dtanh", "inverse_tanh", "exp", "log", "negative_log", "safe_entropy_log", "log_or_zero",
        "abs", "sign", "relu", "relu_backward", "softplus", "softplus_backward", "isnotanumber",
        "isinfinity", "round", "ceiling", "negate",
        "bf16_round",      // not a reference functor: the float a bf16 store would keep (astype(bf16) inside an expression)
        "tf32_hi", "tf32_lo",   // not reference functors: the two parts a 3xTF32 product takes of an fp32 operand, so that
                                // the kernel that produces the operand can leave it split (a recurrent cell's next h)
        nullptr};
    static const char* binary[] = {
        "add", "subtract", "eltmul", "eltdiv", "equals", "power", "fill", "div_grad", "threshold",
        "max_scalar", "min_scalar", "steep_sigmoid", "steep_sigmoid_backward", "clipped_relu",
        "clipped_relu_backward", "clip", "lessthanequal", "greaterthanequal",
        "binary_cross_entropy", "binary_cross_entropy_grad", "prelu", "prelu_backward_weights",
        "prelu_backward_inputs",
        "rng_uniform", "rng_normal",   // (element index i32, seed i32) -> f32 / f64: Philox4x32-10, see the device prelude
        "where_nonzero",   // not a reference functor: a != 0 ? b : 0, the select of its Diag kernel (op/eye.cpp:37)
        nullptr};
    for (int i = 0; unary[i]; ++i) if (n == unary[i]) return 1;
    for (int i = 0; binary[i]; ++i) if (n == binary[i]) return 2;
    return 0;
}

std::vector<std::string> split_ws(const std::string& line) {
    std::vector<std::string> out;
    std::istringstream ss(line);
    std::string tok;
    while (ss >> tok) out.push_back(tok);
    return out;
}

}  // namespace

bool parse_program(const std::string& text, Program* out, std::string* err) {
    Program p;
    std::istringstream in(text);
    std::string line;
    int lineno = 0;
    bool seen_header = false, seen_space = false, seen_end = false;
    auto fail = [&](const std::string& msg) {
        *err = "IR line " + std::to_string(lineno) + ": " + msg + " [" + line + "]";
        return false;
    };
    auto value_ok = [&](int v) { return v >= 0 && v < (int)p.value_stmt.size(); };

    while (std::getline(in, line)) {
        ++lineno;
        size_t hash_pos = line.find('#');
        if (hash_pos != std::string::npos) line = line.substr(0, hash_pos);
        std::vector<std::string> t = split_ws(line);
        if (t.empty()) continue;
        if (seen_end) return fail("statement after 'end'");
        if (!seen_header) {
            if (t.size() != 2 || t[0] != "dali-ir" || t[1] != "1") return fail("expected 'dali-ir 1'");
            seen_header = true;
            continue;
        }
        if (t[0] == "space") {
            if (seen_space) return fail("duplicate 'space'");
            if (t.size() != 3 || !parse_int(t[1], &p.rank) || !parse_int(t[2], &p.nreduce))
                return fail("expected 'space <rank> <nreduce>'");
            if (p.rank < 1 || p.rank > 8) return fail("rank must be in [1, 8]");
            if (p.nreduce < 0 || p.nreduce > p.rank) return fail("nreduce must be in [0, rank]");
            seen_space = true;
            continue;
        }
        if (!seen_space) return fail("'space' must come first");
        if (t[0] == "arg") {
            int idx;
            ArgDecl a;
            if ((t.size() != 4 && t.size() != 5) || !parse_int(t[1], &idx) || !parse_arg_dtype(t[2], &a.dtype) ||
                (t[3] != "E" && t[3] != "R") || (t.size() == 5 && t[4] != "iota"))
                return fail("expected 'arg <i> <dtype> <E|R> [iota]'");
            if (t.size() == 5) {
                if (a.dtype != I32) return fail("an iota arg is int32");
                a.iota = true;
                p.has_iota = true;
            }
            if (idx != (int)p.args.size()) return fail("args must be declared densely in order");
            if (!p.stmts.empty()) return fail("args must precede statements");
            a.elem_level = t[3] == "E";
            if (a.dtype == BF16) p.has_bf16 = true;
            p.args.push_back(a);
            continue;
        }
        if (t[0] == "scalar") {
            int idx;
            DType d;
            if (t.size() != 3 || !parse_int(t[1], &idx) || !parse_dtype(t[2], &d))
                return fail("expected 'scalar <j> <dtype>'");
            if (idx != (int)p.scalars.size()) return fail("scalars must be declared densely in order");
            if (!p.stmts.empty()) return fail("scalars must precede statements");
            p.scalars.push_back(d);
            continue;
        }
        if (t[0] == "end") { seen_end = true; continue; }

        Stmt s;
        if (t[0] == "st" || t[0] == "stx") {
            bool x = t[0] == "stx";
            if ((int)t.size() != (x ? 5 : 4)) return fail("malformed store");
            if (!parse_int(t[1], &s.arg) || s.arg < 0 || s.arg >= (int)p.args.size())
                return fail("store to unknown arg");
            if (!parse_assign_op(t[2], &s.aop)) return fail("unknown assignment operator");
            int v;
            if (x) {
                int vi;
                if (!parse_value_ref(t[3], &vi) || !value_ok(vi)) return fail("bad index value");
                if (p.stmts[p.value_stmt[vi]].dtype != I32) return fail("scatter index must be i32");
                s.in.push_back(vi);
                if (!parse_value_ref(t[4], &v) || !value_ok(v)) return fail("bad stored value");
            } else {
                if (!parse_value_ref(t[3], &v) || !value_ok(v)) return fail("bad stored value");
            }
            s.in.push_back(v);
            s.kind = x ? S_STX : S_ST;
            s.dtype = p.args[s.arg].dtype;
            if (p.stmts[p.value_stmt[v]].dtype != (s.dtype == BF16 ? F32 : s.dtype))
                return fail("stored value type differs from the arg's type (insert a cast)");
            if (p.args[s.arg].iota) return fail("an iota arg cannot be stored to");
            p.args[s.arg].written = true;
            if (s.aop != A_ASSIGN) p.args[s.arg].read = true;
            if (x) p.args[s.arg].indirect = true;
            p.stmts.push_back(s);
            continue;
        }

        // value definition: v<k> <dtype> <kind> ...
        if (t.size() < 3 || !parse_value_ref(t[0], &s.id)) return fail("unknown statement");
        if (s.id != (int)p.value_stmt.size()) return fail("values must be numbered densely in order");
        if (!parse_dtype(t[1], &s.dtype)) return fail("unknown dtype");
        const std::string& k = t[2];
        if (k == "ld" || k == "ldx") {
            bool x = k == "ldx";
            if ((int)t.size() != (x ? 5 : 4)) return fail("malformed load");
            if (!parse_int(t[3], &s.arg) || s.arg < 0 || s.arg >= (int)p.args.size())
                return fail("load from unknown arg");
            if ((p.args[s.arg].dtype == BF16 ? F32 : p.args[s.arg].dtype) != s.dtype)
                return fail("load type differs from the arg's type");
            p.args[s.arg].read = true;
            if (x) {
                int vi;
                if (!parse_value_ref(t[4], &vi) || !value_ok(vi)) return fail("bad index value");
                if (p.stmts[p.value_stmt[vi]].dtype != I32) return fail("gather index must be i32");
                s.in.push_back(vi);
                if (p.args[s.arg].iota) return fail("an iota arg cannot be gathered from");
                p.args[s.arg].indirect = true;
                p.has_indirect = true;
            }
            s.kind = x ? S_LDX : S_LD;
        } else if (k == "acc") {
            if ((t.size() != 3 && t.size() != 4) || s.dtype != F32) return fail("expected 'v<k> f32 acc [slice]'");
            if (p.nreduce != 0 || p.rank != 2) return fail("'acc' needs 'space 2 0'");
            s.arg = 0;     // which column slice of the product (see Program::acc_slices)
            if (t.size() == 4 && (!parse_int(t[3], &s.arg) || s.arg < 0 || s.arg > 7)) return fail("bad accumulator slice");
            if (s.arg + 1 > p.acc_slices) p.acc_slices = s.arg + 1;
            s.kind = S_ACC;
            p.has_acc = true;
        } else if (k == "sc") {
            if (t.size() != 4 || !parse_int(t[3], &s.arg) || s.arg < 0 || s.arg >= (int)p.scalars.size())
                return fail("unknown scalar");
            if (p.scalars[s.arg] != s.dtype) return fail("scalar type mismatch");
            s.kind = S_SC;
        } else if (k == "const") {
            if (t.size() != 4) return fail("malformed const");
            char* endp = nullptr;
            std::strtod(t[3].c_str(), &endp);
            bool special = t[3] == "inf" || t[3] == "-inf" || t[3] == "nan";
            if (!special && (endp == nullptr || *endp != '\0')) return fail("bad literal");
            s.literal = t[3];
            s.kind = S_CONST;
        } else if (k == "op") {
            if (t.size() < 5) return fail("malformed op");
            s.name = t[3];
            int ar = functor_arity(s.name);
            if (ar == 0) return fail("unknown functor '" + s.name + "'");
            if ((int)t.size() != 4 + ar) return fail("wrong operand count for '" + s.name + "'");
            for (int i = 0; i < ar; ++i) {
                int v;
                if (!parse_value_ref(t[4 + i], &v) || !value_ok(v)) return fail("bad operand");
                const bool rng = s.name == "rng_uniform" || s.name == "rng_normal";
                bool converts = s.name == "round" || s.name == "ceiling" || rng;
                if (!converts && p.stmts[p.value_stmt[v]].dtype != s.dtype)
                    return fail("operand type differs from result type (insert a cast)");
                if (rng && (p.stmts[p.value_stmt[v]].dtype != I32 || s.dtype == I32))
                    return fail("rng functors take (i32 index, i32 seed) and yield f32 or f64");
                s.in.push_back(v);
            }
            s.kind = S_OP;
        } else if (k == "cast") {
            int v;
            if (t.size() != 4 || !parse_value_ref(t[3], &v) || !value_ok(v)) return fail("malformed cast");
            s.in.push_back(v);
            s.kind = S_CAST;
        } else if (k == "red" || k == "argred") {
            bool a = k == "argred";
            int v;
            if (t.size() < 5 || t.size() > (a ? 7u : 6u) || !parse_value_ref(t[4], &v) || !value_ok(v)) return fail("malformed reduction");
            if (t.size() > 5) {
                // 'xrank': the partial results of the ranks (dalib200_comm_init_rank) meet inside the kernel
                if (t[5] != "xrank") return fail("expected 'xrank' after the reduced value");
                if (p.nreduce != p.rank) return fail("a cross-rank reduction folds every dim of the space");
                s.xrank = true;
                p.has_xrank = true;
                if (t.size() == 7) {
                    int off;
                    if (!parse_value_ref(t[6], &off) || !value_ok(off)) return fail("bad index offset");
                    const Stmt& os = p.stmts[p.value_stmt[off]];
                    if (os.dtype != I32 || (os.kind != S_SC && os.kind != S_CONST)) return fail("the index offset is an i32 scalar or constant");
                    s.xrank_offset = off;
                }
            }
            s.name = t[3];
            if (a) {
                if (s.name != "max" && s.name != "min") return fail("argred takes max|min");
                if (s.dtype != I32) return fail("argred yields i32");
            } else {
                if (s.name != "sum" && s.name != "prod" && s.name != "max" && s.name != "min")
                    return fail("red takes sum|prod|max|min");
                if (p.stmts[p.value_stmt[v]].dtype != s.dtype) return fail("reduction changes type");
            }
            if (p.nreduce == 0) return fail("reduction in a program with nreduce = 0");
            s.in.push_back(v);
            s.kind = a ? S_ARGRED : S_RED;
            ++p.n_reductions;
        } else {
            return fail("unknown statement kind '" + k + "'");
        }
        p.value_stmt.push_back((int)p.stmts.size());
        p.stmts.push_back(s);
    }
    lineno = 0; line = "";
    if (!seen_header) return fail("empty program");
    if (!seen_end) return fail("missing 'end'");
    bool any_store = false;
    for (const Stmt& s : p.stmts) any_store = any_store || s.kind == S_ST || s.kind == S_STX;
    if (!any_store) return fail("program stores nothing");

    // levels and stages
    for (Stmt& s : p.stmts) {
        auto src = [&](int i) -> const Stmt& { return p.stmts[p.value_stmt[s.in[i]]]; };
        switch (s.kind) {
            case S_LD:
                s.elem = p.nreduce == 0 ? true : p.args[s.arg].elem_level;
                s.stage = 0;
                break;
            case S_LDX:
                s.elem = (p.nreduce == 0 ? true : p.args[s.arg].elem_level) || src(0).elem;
                s.stage = src(0).stage;
                break;
            case S_ACC:
                s.elem = true;
                s.stage = 0;
                break;
            case S_SC:
            case S_CONST:
                s.elem = false;
                s.stage = 0;
                break;
            case S_OP:
            case S_CAST:
                // without reductions there is no row scope: everything but scalars and
                // constants is computed per element
                s.elem = p.nreduce == 0;
                s.stage = 0;
                for (size_t i = 0; i < s.in.size(); ++i) {
                    s.elem = s.elem || src(i).elem;
                    if (src(i).stage > s.stage) s.stage = src(i).stage;
                }
                break;
            case S_RED:
            case S_ARGRED:
                s.elem = false;
                s.stage = src(0).stage + 1;
                break;
            case S_ST:
            case S_STX: {
                const Stmt& v = src(s.in.size() - 1);
                s.stage = v.stage;
                if (s.kind == S_STX && src(0).stage > s.stage) s.stage = src(0).stage;
                bool arg_elem = p.nreduce == 0 ? true : p.args[s.arg].elem_level;
                if (!arg_elem && (v.elem || (s.kind == S_STX && src(0).elem))) {
                    *err = "IR: element-level value stored to a row-level arg " + std::to_string(s.arg);
                    return false;
                }
                s.elem = arg_elem;
                break;
            }
        }
        if (s.stage > p.max_stage) p.max_stage = s.stage;
    }
    for (size_t i = 0; i < p.args.size(); ++i) {
        if (!p.args[i].read && !p.args[i].written) {
            *err = "IR: arg " + std::to_string(i) + " is never used";
            return false;
        }
    }
    p.text = text;
    *out = p;
    return true;
}

}  // namespace dalib
