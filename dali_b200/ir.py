"""Tiny builder for the fused-expression IR text (dali_b200/csrc/ir.h).

Harness-side convenience for tests and benchmarks that drive the C ABI
directly; the C++ Array / op:: layer emits the same text from expression
graphs."""


class IRBuilder:
    def __init__(self, rank, nreduce=0):
        self.rank, self.nreduce = rank, nreduce
        self.args, self.scalars, self.body = [], [], []
        self.types = []

    def arg(self, dtype="f32", level="E", iota=False):
        """iota=True: no memory behind the arg; its element at offset i IS the int32 value (launch offset + i)."""
        self.args.append((dtype, level + (" iota" if iota else "")))
        return len(self.args) - 1

    def scalar(self, dtype="f32"):
        self.scalars.append(dtype)
        return len(self.scalars) - 1

    def _val(self, dtype, text):
        k = len(self.types)
        self.types.append(dtype)
        self.body.append("v%d %s %s" % (k, dtype, text))
        return k

    def ld(self, arg):
        dt = self.args[arg][0]
        return self._val("f32" if dt == "bf16" else dt, "ld %d" % arg)

    def ldx(self, arg, index):
        return self._val(self.args[arg][0], "ldx %d v%d" % (arg, index))

    def sc(self, j):
        return self._val(self.scalars[j], "sc %d" % j)

    def acc(self, slice_=0):
        """The GEMM accumulator at (row, col) -- epilogue programs only.  With slices, `acc q` is the product's
        column q * n + col (n = the width of the program's space)."""
        return self._val("f32", "acc" if slice_ == 0 else "acc %d" % slice_)

    def const(self, dtype, literal):
        return self._val(dtype, "const %s" % literal)

    def op(self, name, *vals, dtype=None):
        return self._val(dtype or self.types[vals[0]], "op %s %s" % (name, " ".join("v%d" % v for v in vals)))

    def cast(self, dtype, v):
        return self._val(dtype, "cast v%d" % v)

    def red(self, kind, v, xrank=False):
        """xrank (all-axis programs): the ranks' partial results are combined inside the kernel."""
        return self._val(self.types[v], "red %s v%d%s" % (kind, v, " xrank" if xrank else ""))

    def argred(self, kind, v, xrank=False, offset=None):
        """xrank: as red; offset = an i32 scalar value added to the local position before the pairs are exchanged."""
        tail = (" xrank" + (" v%d" % offset if offset is not None else "")) if xrank else ""
        return self._val("i32", "argred %s v%d%s" % (kind, v, tail))

    def st(self, arg, v, op="assign"):
        self.body.append("st %d %s v%d" % (arg, op, v))

    def stx(self, arg, index, v, op="assign"):
        self.body.append("stx %d %s v%d v%d" % (arg, op, index, v))

    def text(self):
        lines = ["dali-ir 1", "space %d %d" % (self.rank, self.nreduce)]
        lines += ["arg %d %s %s" % (i, d, l) for i, (d, l) in enumerate(self.args)]
        lines += ["scalar %d %s" % (j, d) for j, d in enumerate(self.scalars)]
        return "\n".join(lines + self.body + ["end"]) + "\n"


# ---- the fused expressions of the benchmark configurations ---------------------------
def softmax_ir():
    """exp(a - max(a,{-1},true)) / sum(exped,{-1},true) over [rows, cols]: args (out, a)."""
    b = IRBuilder(2, 1)
    out, a = b.arg("f32"), b.arg("f32")
    x = b.ld(a)
    m = b.red("max", x)
    e = b.op("exp", b.op("subtract", x, m))
    s = b.red("sum", e)
    b.st(out, b.op("eltdiv", e, s))
    return b.text()


def chain_sum_ir(xrank=False):
    """sum(sigmoid(x*w+b) * exp(-x*x)) over all elements: args (out scalar, x), scalars (w, b).  xrank: x is one
    rank's shard and the partial sums of the ranks meet inside the kernel."""
    b = IRBuilder(1, 1)
    out, x = b.arg("f32", "R"), b.arg("f32")
    w, bb = b.scalar("f32"), b.scalar("f32")
    v = b.ld(x)
    sig = b.op("sigmoid", b.op("add", b.op("eltmul", v, b.sc(w)), b.sc(bb)))
    ex = b.op("exp", b.op("eltmul", b.op("negate", v), v))
    b.st(out, b.red("sum", b.op("eltmul", sig, ex), xrank))
    return b.text()


def reduce_ir(kind, dtype="f32", rank=2, nreduce=1, arg=False, xrank=False):
    """out = reduce(x) over the innermost `nreduce` dims: args (out, x).  xrank (nreduce == rank): combined over the
    ranks inside the kernel; an arg-reduction then takes one i32 scalar, the offset of the rank's shard."""
    b = IRBuilder(rank, nreduce)
    out, x = b.arg("i32" if arg else dtype, "R"), b.arg(dtype)
    v = b.ld(x)
    if arg and xrank:
        b.st(out, b.argred(kind, v, True, b.sc(b.scalar("i32"))))
    else:
        b.st(out, b.argred(kind, v) if arg else b.red(kind, v, xrank))
    return b.text()


def arg_pair_ir(kind, dtype="f32", rank=2, nreduce=1):
    """(extreme value, its position + offset) over the innermost `nreduce` dims in one kernel: args (values, positions,
    x), scalar (offset i32) -- what a sharded argmax / argmin computes locally before dalib200_arg_allreduce."""
    b = IRBuilder(rank, nreduce)
    vals, pos, x = b.arg(dtype, "R"), b.arg("i32", "R"), b.arg(dtype)
    v = b.ld(x)
    b.st(vals, b.red(kind, v))
    b.st(pos, b.op("add", b.argred(kind, v), b.sc(b.scalar("i32"))))
    return b.text()


def lstm_gating_ir():
    """c' = sigmoid(f)*c + sigmoid(i)*tanh(g); h' = sigmoid(o)*tanh(c') over [B, H]:
    args (c_new, h_new, i, f, o, g, c) -- the four gate operands are column slices
    of one [B, 4H] buffer."""
    b = IRBuilder(2, 0)
    cn, hn = b.arg("f32"), b.arg("f32")
    gi, gf, go, gg, c = (b.arg("f32") for _ in range(5))
    i, f, o = (b.op("sigmoid", b.ld(a)) for a in (gi, gf, go))
    g = b.op("tanh", b.ld(gg))
    cnew = b.op("add", b.op("eltmul", f, b.ld(c)), b.op("eltmul", i, g))
    b.st(cn, cnew)
    b.st(hn, b.op("eltmul", o, b.op("tanh", cnew)))
    return b.text()


def gemm_bias_tanh_ir(out_dtype="bf16"):
    """tanh(acc + bias[col]) as a GEMM epilogue: args (out [m,n], bias broadcast over rows)."""
    b = IRBuilder(2, 0)
    out, bias = b.arg(out_dtype), b.arg("f32")
    b.st(out, b.op("tanh", b.op("add", b.acc(), b.ld(bias))))
    return b.text()


def gemm_store_ir(out_dtype="f32", op="assign"):
    """Plain product: args (out [m,n])."""
    b = IRBuilder(2, 0)
    out = b.arg(out_dtype)
    b.st(out, b.acc(), op)
    return b.text()


def lstm_cell_epilogue_ir(split_h=False):
    """The whole LSTM gating as the epilogue of gates = x.Wx + h.Wh: per output (row, unit) the four accumulator
    slices i, f, o, g plus their biases, c' = sigmoid(f)*c + sigmoid(i)*tanh(g), h' = sigmoid(o)*tanh(c').
    args (c_new, h_new, b_i, b_f, b_o, b_g, c); the gates matrix is never written.  With split_h the args end with
    (h_hi, h_lo): h' is also left as the two parts the next step's 3xTF32 product h'.Wh reads, so that a recurrent loop
    needs no separate split of h."""
    b = IRBuilder(2, 0)
    cn, hn = b.arg("f32"), b.arg("f32")
    bias = [b.arg("f32") for _ in range(4)]
    c = b.arg("f32")
    pre = [b.op("add", b.acc(q), b.ld(bias[q])) for q in range(4)]
    i, f, o = (b.op("sigmoid", pre[q]) for q in range(3))
    g = b.op("tanh", pre[3])
    cnew = b.op("add", b.op("eltmul", f, b.ld(c)), b.op("eltmul", i, g))
    b.st(cn, cnew)
    hnew = b.op("eltmul", o, b.op("tanh", cnew))
    b.st(hn, hnew)
    if split_h:
        hi, lo = b.arg("f32"), b.arg("f32")
        b.st(hi, b.op("tf32_hi", hnew))
        b.st(lo, b.op("tf32_lo", hnew))
    return b.text()
