// Kernel skeletons for fused expressions: turns an IR Program plus a concrete
// layout Variant into CUDA C++ for sm_100a.
//
// Replaces the reference's code emission (get_code_template,
// dali/array/jit/jit.cpp:921-1009; GPU kernel + launch text :426-539,716-772;
// reducer bodies dali/array/jit/all_reduce_kernel_utils.cpp:105-271).  Where
// the reference emits one view-template expression evaluated per element with
// `int` index arithmetic, one block per row and temporaries for every
// broadcast, the skeletons here are:
//
//   map  elementwise; 2-D thread tile, 128-bit loads/stores along the inner dim
//   row  reductions over the inner dims fused with the elementwise work around
//        them; T threads share a row, the row lives in registers between
//        stages (or is re-streamed when it does not fit), shuffle + shared
//        memory combine
//   col  same maths when the REDUCED dim is the strided one (axis-0 reductions):
//        threads run along the contiguous outer dim, the reduced dim is split
//        across CTAs, partials meet in scratch memory, last CTA finishes
//   all  all-axis reduction: grid-stride partials, scratch, last CTA finishes
#ifndef DALI_B200_CSRC_CODEGEN_H
#define DALI_B200_CSRC_CODEGEN_H

#include <string>
#include <vector>

#include "ir.h"

namespace dalib {

enum Kind { K_MAP, K_ROW, K_COL, K_ALL };

// Everything about a launch that is compiled into the kernel.  Shapes, stride
// values, pointers and scalars stay run-time parameters, as in the reference
// (dali/array/jit/jit.cpp:1017-1021: only structure is part of the key).
struct Variant {
    Kind kind = K_MAP;
    int nout = 0;            // outer (non-reduced) dims after collapsing, 0..8
    int nin = 1;             // inner dims after collapsing, >= 1
    int vec = 1;             // elements per 128-bit access (1 = scalar path)
    int threads = 256;       // CTA size
    int T = 256;             // row: threads sharing a row
    int vpt = 0;             // row: vector groups per thread kept in registers (0 = streaming)
    int unroll = 4;          // map / all / col: independent groups in flight per thread
    int tx = 32, ty = 8;     // col: threads along outer / along the reduced dim
    int stage = 0;           // row, T = 32: every warp keeps a ring of `stage` rows in flight, copied into shared memory by
                             // bulk asynchronous copies (cp.async.bulk + mbarrier) ahead of the rows it works on
    int minb = 0;            // col: CTAs per SM the grid was sized for; the kernel is compiled to fit that many (__launch_bounds__)
    int cluster = 0;         // row, streaming: a thread-block cluster of this many CTAs shares every row (each a slice of the
                             // columns), partial results meet through distributed shared memory
    bool xrank = false;      // all: partial results are exchanged with the other ranks before the kernel finishes
    int tile = 0;            // map with operands of class 't': 32 / 64 = edge of the shared-memory tiles they are read through, 4 = 4 x 4 register blocks (128-bit accesses), 0 = none
    std::string cls;         // per arg inner-stride class: u(nit) z(ero) s(trided) t(ransposed: unit stride along the OUTER dim)
    bool unchecked = false;  // all: chunks that lie wholly inside the data run without per-vector bounds checks
    bool stream_out = false; // map with a gather: element stores are streaming stores (evict-first in L2)
    std::string xv;          // per arg: '1' = an indirectly read arg whose rows can be fetched with full-width vector loads
    std::string ocls;        // col: per arg outer-stride class
    std::string key() const; // text folded into the cache key
    const char* kind_name() const;
};

// Layout of the kernel parameter block: 8-byte words.
struct ParamLayout {
    int w_R = 0, w_C = 1, w_scratch = 2, w_counter = 3, w_aux0 = 4, w_aux1 = 5;
    int w_oshape = 6;        // nout words
    int w_ishape = 0;        // nin words
    int w_args = 0;          // per arg: ptr, lead stride, nout outer strides, nin inner strides
    int arg_words = 0;
    int w_scalars = 0;
    int total = 0;
    ParamLayout(const Program& p, const Variant& v);
    int arg_ptr(int a) const { return w_args + a * arg_words; }
    int arg_xs(int a) const { return w_args + a * arg_words + 1; }
    int arg_rs(int a, int k) const { return w_args + a * arg_words + 2 + k; }
    int arg_cs(int a, int k, int nout) const { return w_args + a * arg_words + 2 + nout + k; }
};

// Bytes of scratch one reduction result occupies in the cross-CTA exchange.
int scratch_slot_bytes(const Program& p);

// Generates the translation unit (prelude excluded).  The kernel is
// `extern "C" __global__ void dali_kernel(const P p)`.
bool generate_kernel(const Program& p, const Variant& v, std::string* src, std::string* err);

}  // namespace dalib
#endif
