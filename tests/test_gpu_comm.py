"""Ranks and collectives on ONE GPU: the peer-exchange protocol with 2 / 4 / 8 virtual ranks inside one cooperative
kernel (dalib200_peer_emulate), and a communicator of world size 1, through which a sharded Array's all-axis
reductions run in the kernel variant that exchanges partial results in-kernel (with itself)."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

F32, F64, I32 = 0, 1, 2
TORCH = {F32: torch.float32, F64: torch.float64, I32: torch.int32}


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [F32, F64, I32])
@pytest.mark.parametrize("n", [1, 1000, 4099])
def test_emulated_allreduce(lib, world, dtype, n):
    rng = np.random.default_rng(100 * world + 10 * dtype + n)
    parts = [rng.integers(-50, 50, n).astype(np.float64) for _ in range(world)]       # small integers: sums are exact
    for op, fold in (("sum", np.add), ("max", np.maximum), ("min", np.minimum)):
        bufs = [torch.from_numpy(p).to(TORCH[dtype]).cuda() for p in parts]
        repeats = 3                                   # both parities of the double-buffered slots, and one reuse
        assert lib.peer_emulate(bufs, n, dtype, op, repeats=repeats) == 0
        want = parts[0]
        for p in parts[1:]:
            want = fold(want, p)
        if op == "sum":
            want = want * world ** (repeats - 1)       # every repeat reduces the previous results again
        for b in bufs:
            np.testing.assert_array_equal(b.cpu().numpy().astype(np.float64), want)


def test_emulated_allreduce_float_order(lib):
    """Contributions are folded in rank order on every rank: bit-identical results, equal to the serial fold."""
    world, n = 8, 3000
    rng = np.random.default_rng(5)
    parts = [rng.standard_normal(n).astype(np.float32) for _ in range(world)]
    bufs = [torch.from_numpy(p).cuda() for p in parts]
    assert lib.peer_emulate(bufs, n, F32, "sum") == 0
    want = parts[0].copy()
    for p in parts[1:]:
        want = want + p
    for b in bufs:
        np.testing.assert_array_equal(b.cpu().numpy(), want)
    prod = [torch.from_numpy((1 + 0.01 * p).astype(np.float32)).cuda() for p in parts]
    assert lib.peer_emulate(prod, n, F32, "prod") == 0
    want = (1 + 0.01 * parts[0]).astype(np.float32)
    for p in parts[1:]:
        want = want * (1 + 0.01 * p).astype(np.float32)
    np.testing.assert_array_equal(prod[3].cpu().numpy(), want)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("dtype", [F32, F64, I32])
def test_emulated_arg_allreduce(lib, world, dtype):
    """(value, index) pairs: the extreme value wins, among equal values the lowest index -- whatever rank holds it."""
    n = 1500
    rng = np.random.default_rng(world + dtype)
    vals = [rng.integers(-5, 5, n).astype(np.float64) for _ in range(world)]          # many ties
    idxs = [rng.permutation(world * n)[:n].astype(np.int32) for _ in range(world)]
    for op in ("max", "min"):
        bv = [torch.from_numpy(v).to(TORCH[dtype]).cuda() for v in vals]
        bi = [torch.from_numpy(i).cuda() for i in idxs]
        assert lib.peer_emulate(bv, n, dtype, op, indices=bi, repeats=2) == 0
        V, I = np.stack(vals), np.stack(idxs)
        best = V.max(0) if op == "max" else V.min(0)
        pick = np.where(V == best, I, np.iinfo(np.int32).max).min(0)
        for r in range(world):
            np.testing.assert_array_equal(bv[r].cpu().numpy().astype(np.float64), best)
            np.testing.assert_array_equal(bi[r].cpu().numpy(), pick)


def test_emulate_refuses_oversized_payloads(lib):
    from dali_b200.capi import DaliB200Error
    bufs = [torch.zeros(70000, device="cuda") for _ in range(2)]
    with pytest.raises(DaliB200Error):
        lib.peer_emulate(bufs, 70000, F32, "sum")            # 280 KB > one 256 KiB slot
    with pytest.raises(DaliB200Error):
        lib.peer_emulate([torch.zeros(60000, device="cuda") for _ in range(8)], 60000, F32, "sum")   # more CTAs than SMs


@pytest.fixture
def single_rank(lib):
    lib.comm_init_rank(0, 1, 0, None)
    assert lib.comm_transport() == "single" and lib.comm_world() == 1
    yield lib
    assert lib.comm_error_flag() == 0
    lib.comm_destroy()


def test_world_of_one_fused_reductions(single_rank):
    """A shard that is the whole array: sum / mean / max / argmax over all axes run in the kernel variant that
    exchanges its partial results through the rank's peer block before finishing."""
    import dali_oracle as oracle
    from dali_b200.array import Array, collectives, last_ir, last_variant, op
    rng = np.random.default_rng(3)
    x = (rng.random((700, 333)) * 2 - 1).astype(np.float32)
    x[5, 7] = x[600, 2] = 0.99999994
    xs = Array.scatter_rows(x)
    assert xs.shard == (0, 0, 700)
    before = collectives()[0]
    chain = op.sum(op.sigmoid(xs * np.float32(0.5) + np.float32(0.1)) * op.exp(-xs * xs))
    got = float(chain.numpy())
    assert "red sum" in last_ir() and "xrank" in last_ir() and ".xrank" in last_variant()
    s32, s64, sabs = oracle.chain_sum(x, 0.5, 0.1)
    assert abs(got - s64) <= 1e-5 * sabs
    for k in range(5):                                         # epochs advance, slots alternate
        assert float(op.sum(xs).numpy()) == pytest.approx(float(x.astype(np.float64).sum()), abs=1e-5 * np.abs(x).sum())
    assert float(op.max(xs).numpy()) == x.max()
    assert int(op.argmax(xs).numpy()) == int(oracle.argreduce("max", x)) == 5 * 333 + 7
    assert int(op.argmin(xs).numpy()) == int(oracle.argreduce("min", x))
    m = float(op.mean(xs).numpy())
    assert abs(m - x.astype(np.float64).mean()) <= 1e-5 * np.abs(x).mean()
    assert collectives()[0] - before >= 10 and collectives()[1].startswith("in-kernel")
    # reductions that keep the sharded axis stay local; over it they end in a (trivial) all-reduce
    np.testing.assert_array_equal(op.max(xs, [0]).numpy(), x.max(0))
    np.testing.assert_array_equal(op.argmax(xs, 0).numpy(), oracle.argreduce("max", x, 0))
    assert op.sum(xs, [1]).shard == (0, 0, 700)


def test_cross_rank_program_through_the_c_abi(single_rank):
    lib = single_rank
    from dali_b200.ir import IRBuilder
    x = torch.arange(1 << 20, dtype=torch.float32, device="cuda") % 7
    out = torch.zeros(2, device="cuda")
    text = "\n".join(["dali-ir 1", "space 1 1", "arg 0 f32 R", "arg 1 f32 R", "arg 2 f32 E", "v0 f32 ld 2", "v1 f32 red sum v0 xrank",
                      "v2 f32 red max v0 xrank", "st 0 assign v1", "st 1 assign v2", "end", ""])
    h = lib.compile(text)
    for _ in range(3):
        lib.launch(h, (x.numel(),), [out[0:1], out[1:2], x])
    torch.cuda.synchronize()
    assert ".xrank" in lib.last_variant()
    assert out.tolist() == [float(x.sum().item()), 6.0]


def test_cross_rank_program_needs_a_communicator(lib):
    from dali_b200.capi import DaliB200Error
    assert lib.comm_transport() == "none"
    x = torch.ones(4096, device="cuda")
    out = torch.zeros(1, device="cuda")
    h = lib.compile("\n".join(["dali-ir 1", "space 1 1", "arg 0 f32 R", "arg 1 f32 E", "v0 f32 ld 1", "v1 f32 red sum v0 xrank",
                               "st 0 assign v1", "end", ""]))
    with pytest.raises(DaliB200Error, match="communicator"):
        lib.launch(h, (4096,), [out, x])
    bad = "\n".join(["dali-ir 1", "space 2 1", "arg 0 f32 R", "arg 1 f32 E", "v0 f32 ld 1", "v1 f32 red sum v0 xrank", "st 0 assign v1", "end", ""])
    with pytest.raises(DaliB200Error, match="every dim"):
        lib.compile(bad)
