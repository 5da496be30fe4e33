"""Several decode linears in one launch (mt_qgemm_chain / LinearChain) against the same linears issued one by one and
against the oracle, through the C ABI.  The chain runs the stream-K GEMV body per entry with the same split of the
work, so its outputs are bit-identical to single calls that take the stream-K schedule (flag variant 2)."""
import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import assert_close, oracle_out, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
STREAM_K = 2 << 24        # tuning bits of the flags: always the stream-K schedule of the decode GEMV


@pytest.fixture(scope="module")
def M(lib_built):
    import minit_b200
    return minit_b200


def lin(k, n, m, bits=4, dtype=torch.float16, seed=0, group_size=128):
    c = O.make_gptq_case(k, n, m, bits=bits, dtype=dtype, seed=seed, group_size=group_size)
    return c, to_dev(c, DEV)


def control_words(dev=DEV):
    from minit_b200 import _lib
    torch.cuda.synchronize()
    return [int(ws[_lib.COUNTER_BYTES - 12:_lib.COUNTER_BYTES].view(torch.int32).abs().sum().item()) for ws in _lib._workspaces.values()]


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("bits,dtype", [(4, torch.float16), (4, torch.bfloat16), (8, torch.float16)])
def test_independent_entries_match_single_calls(M, bits, dtype, m):
    from minit_b200.chain import ChainEntry, LinearChain
    shapes = [(1024, 1280), (1024, 8192), (8192, 7168), (3584, 1024), (128, 128)]
    cases = [lin(k, n, m, bits, dtype, seed=i + 10 * m) for i, (k, n) in enumerate(shapes)]
    outs = [torch.full((m, n), float("nan"), dtype=dtype, device=DEV) for _, n in shapes]
    chain = LinearChain([ChainEntry(d["x"], d["qweight"], d["qzeros"], d["scales"], o) for (_, d), o in zip(cases, outs)], bits=bits)
    chain()
    torch.cuda.synchronize()
    assert chain.single_launch is True
    for (c, d), o, (k, n) in zip(cases, outs, shapes):
        assert_close(o.cpu(), oracle_out(c, False), f"chain entry {k}x{n} bits={bits} {dtype} M={m}")
        single = M.quantized_matrix_multiply(d["x"], d["qweight"], d["qzeros"], d["scales"], None, bits=bits, flags=STREAM_K)
        assert torch.equal(o, single), f"chain entry {k}x{n} differs from the single call"
    assert control_words() and not any(control_words())


def layer_chain(M, m, dtype, fill):
    """o-projection (+ residual) -> gate/up with SwiGLU -> down (+ residual): every entry reads the one before."""
    from minit_b200.chain import ChainEntry
    h, ffn = 1024, 1536
    _, o_d = lin(h, h, m, 4, dtype, seed=1)
    _, g_d = lin(h, ffn, m, 4, dtype, seed=2)
    _, u_d = lin(h, ffn, m, 4, dtype, seed=3)
    _, d_d = lin(ffn, h, m, 4, dtype, seed=4)
    gu = M.interleave_gate_up((g_d["qweight"], g_d["qzeros"], g_d["scales"], None), (u_d["qweight"], u_d["qzeros"], u_d["scales"], None), bits=4)
    attn = o_d["x"]
    hidden = (torch.randn((m, h), generator=torch.Generator().manual_seed(5)) * 0.5).to(dtype).to(DEV)
    h1 = torch.full((m, h), fill, dtype=dtype, device=DEV)
    act = torch.full((m, ffn), fill, dtype=dtype, device=DEV)
    h2 = torch.full((m, h), fill, dtype=dtype, device=DEV)
    entries = [ChainEntry(attn, o_d["qweight"], o_d["qzeros"], o_d["scales"], h1, residual=hidden),
               ChainEntry(h1, gu[0], gu[1], gu[2], act, epilogue="swiglu"),
               ChainEntry(act, d_d["qweight"], d_d["qzeros"], d_d["scales"], h2, residual=h1)]
    return entries, (h1, act, h2)


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dependent_entries_match_the_sequence_of_single_calls(M, dtype, m):
    from minit_b200.chain import LinearChain
    entries, bufs = layer_chain(M, m, dtype, float("nan"))
    chain = LinearChain(entries, bits=4)
    ref_chain = LinearChain(entries, bits=4, flags=STREAM_K)
    ref_chain._one_by_one()                                   # the same linears, one launch each, in stream order
    torch.cuda.synchronize()
    want = [b.clone() for b in bufs]
    assert all(torch.isfinite(w.float()).all() for w in want)
    for rep in range(25):                                     # a race between an entry and its reader would not repeat 25 times
        for b in bufs:
            b.fill_(float("nan"))
        chain()
        torch.cuda.synchronize()
        assert chain.single_launch is True
        for b, w, name in zip(bufs, want, ("o + residual", "swiglu", "down + residual")):
            assert torch.equal(b, w), f"rep {rep}: {name} differs from the one-by-one sequence"
    assert not any(control_words())


def test_graph_replay_and_rotation(M):
    """The launch leaves its control words at zero, so a captured chain can be replayed; two chains alternate."""
    from minit_b200.chain import LinearChain
    e1, b1 = layer_chain(M, 1, torch.float16, 0.0)
    c1 = LinearChain(e1, bits=4)
    c1(); torch.cuda.synchronize()
    want = [b.clone() for b in b1]
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        c1(); c1(); c1()
    for _ in range(4):
        for b in b1:
            b.zero_()
        g.replay()
        torch.cuda.synchronize()
        for b, w in zip(b1, want):
            assert torch.equal(b, w)
    assert not any(control_words())


def test_list_that_does_not_fit_falls_back_to_single_launches(M):
    from minit_b200.chain import ChainEntry, LinearChain
    from minit_b200 import _lib
    c, d = lin(512, 256, 1, seed=9)
    outs = [torch.empty((1, 256), dtype=torch.float16, device=DEV) for _ in range(_lib.CHAIN_MAX + 1)]
    chain = LinearChain([ChainEntry(d["x"], d["qweight"], d["qzeros"], d["scales"], o) for o in outs], bits=4)
    chain(); torch.cuda.synchronize()
    assert chain.single_launch is False
    for o in outs:
        assert_close(o.cpu(), oracle_out(c, False), "17 entries")
    # group sizes 32 and 128 in one list: the folds differ in length, so no single kernel walks both
    c2, d2 = lin(512, 256, 1, seed=10, group_size=32)
    o1, o2 = (torch.empty((1, 256), dtype=torch.float16, device=DEV) for _ in range(2))
    mixed = LinearChain([ChainEntry(d["x"], d["qweight"], d["qzeros"], d["scales"], o1),
                         ChainEntry(d2["x"], d2["qweight"], d2["qzeros"], d2["scales"], o2)], bits=4)
    mixed(); torch.cuda.synchronize()
    assert mixed.single_launch is False
    assert_close(o1.cpu(), oracle_out(c, False), "mixed 0")
    assert_close(o2.cpu(), oracle_out(c2, False), "mixed 1")


def test_validation(M):
    from minit_b200.chain import ChainEntry, LinearChain
    _, d = lin(512, 256, 1, seed=11)
    good = torch.empty((1, 256), dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError):
        LinearChain([], bits=4)
    with pytest.raises(ValueError):
        LinearChain([ChainEntry(d["x"], d["qweight"], d["qzeros"], d["scales"], good[:, :128])], bits=4)
    with pytest.raises(ValueError):
        LinearChain([ChainEntry(d["x"], d["qweight"], d["qzeros"], d["scales"], good, residual=good[:, :128])], bits=4)
    with pytest.raises(ValueError):
        ChainEntry(d["x"], d["qweight"], d["qzeros"], d["scales"], good, epilogue="gelu")
    # three rows: not a decode GEMV request, so the library declines and the wrapper issues single launches
    c3, d3 = lin(512, 256, 3, seed=12)
    o3 = torch.empty((3, 256), dtype=torch.float16, device=DEV)
    ch = LinearChain([ChainEntry(d3["x"], d3["qweight"], d3["qzeros"], d3["scales"], o3)], bits=4)
    ch(); torch.cuda.synchronize()
    assert ch.single_launch is False
    assert_close(o3.cpu(), oracle_out(c3, False), "three rows")
