// Fused-expression IR accepted by dalib200_compile().
//
// The reference turns a fused expression tree into C++/CUDA text made of
// nested view templates (dali/array/jit/jit.cpp:921-1009); this back end takes
// the same tree flattened into a small SSA program and splices it into
// hand-written sm_100a kernel skeletons.  Text format, one statement per line:
//
//   dali-ir 1
//   space <rank> <nreduce>      iteration space; reductions fold the innermost
//                               <nreduce> dims (0 = pure elementwise map)
//   arg <i> <f32|f64|i32|bf16> <E|R>  (bf16: a storage type -- loads yield f32, stores take f32 and round to
//                               nearest even; no indirect stores)
//                               i-th buffer.  E: indexed by the whole space,
//                               R: indexed by the outer (non-reduced) dims only
//   scalar <j> <dtype>          j-th run-time scalar (value read at launch)
//   v<k> <dtype> ld <arg>                   load at the current index
//   v<k> <dtype> ldx <arg> v<i>             indirect load: adds v<i> * lead-stride
//   v<k> <dtype> sc <j>                     scalar argument
//   v<k> <dtype> const <literal>
//   v<k> f32     acc                        the GEMM accumulator at (row, col); only in
//                                           epilogue programs run by dalib200_gemm_fused
//   v<k> <dtype> op <functor> v<a> [v<b>]   functor names as dali/array/functor.h
//   v<k> <dtype> cast v<a>                  static_cast (functor::cast)
//   v<k> <dtype> red <sum|prod|max|min> v<a> [xrank]
//   v<k> i32     argred <max|min> v<a> [xrank [v<o>]]   first occurrence wins
//                                           xrank (all-axis programs only): this rank's result is a partial one; the
//                                           kernel exchanges the partials of all ranks through peer memory and every
//                                           rank continues with the combined value.  v<o>: i32 scalar added to the
//                                           local position first, so that positions are those of the logical array
//   st <arg> <assign|add|sub|mul|div> v<k>
//   stx <arg> <assign|add|sub|mul|div> v<i> v<k>   scatter through index v<i>
//   end
//
// Values are numbered densely in program order.  A value is "row level" (R)
// when it does not vary over the reduced dims: scalars, constants, loads of
// R args, reduction results and functors of those; anything else is element
// level (E).  A store of an R value goes to an R arg.
#ifndef DALI_B200_CSRC_IR_H
#define DALI_B200_CSRC_IR_H

#include <cstdint>
#include <string>
#include <vector>

namespace dalib {

enum DType { F32 = 0, F64 = 1, I32 = 2, BF16 = 3 };
const char* dtype_ir_name(DType t);
const char* dtype_c_name(DType t);
int dtype_size(DType t);

enum StmtKind { S_LD, S_LDX, S_SC, S_CONST, S_OP, S_CAST, S_RED, S_ARGRED, S_ST, S_STX, S_ACC };
enum AssignOp { A_ASSIGN, A_ADD, A_SUB, A_MUL, A_DIV };

struct ArgDecl {
    DType dtype = F32;
    bool elem_level = true;   // E or R
    bool read = false;
    bool written = false;
    bool indirect = false;    // addressed through ldx / stx
    bool iota = false;        // no memory behind it: the value IS the element offset (base + sum of index * stride), int32
};

struct Stmt {
    StmtKind kind = S_OP;
    DType dtype = F32;
    int id = -1;                 // value number (-1 for stores)
    std::string name;            // functor / reducer name
    std::vector<int> in;         // operand value numbers
    int arg = -1;                // arg or scalar index
    std::string literal;         // const
    AssignOp aop = A_ASSIGN;
    bool xrank = false;          // red / argred: combined over the ranks inside the kernel
    int xrank_offset = -1;       // argred xrank: value number of the i32 scalar added to the local position, or -1
    // derived by analyse():
    bool elem = false;           // element level?
    int stage = 0;               // number of reductions on the longest path below
};

struct Program {
    int rank = 0;
    int nreduce = 0;
    std::vector<ArgDecl> args;
    std::vector<DType> scalars;
    std::vector<Stmt> stmts;
    std::vector<int> value_stmt;   // value number -> index in stmts
    int max_stage = 0;             // deepest reduction nesting
    int n_reductions = 0;
    bool has_indirect = false;
    bool has_iota = false;
    bool has_acc = false;          // reads the GEMM accumulator: an epilogue program
    int acc_slices = 1;            // 'acc q': the space is [m, n] and slice q is the product's columns q*n .. q*n + n - 1
    bool has_bf16 = false;
    bool has_xrank = false;        // some reduction is combined over the ranks inside the kernel
    std::string text;              // canonical source text (for collision checks)
};

// Parses and analyses `text`.  On failure returns false and fills `err`.
bool parse_program(const std::string& text, Program* out, std::string* err);

}  // namespace dalib
#endif
