"""Parity of the CUDA library (called through its C ABI by the flash_bla operators)
against the CPU oracle and the golden fixtures.  All tests here need a GPU."""
import pytest
import torch

from oracle import bla_oracle as O
from helpers import check, golden_scale, load_golden, make_inputs, run_op

pytestmark = pytest.mark.gpu

from flash_bla.ops import _passes as P
from flash_bla.ops.linear_attn.decoupled import decoupled_la
from flash_bla.ops.linear_attn.fused import linear_attention
from flash_bla.ops.linear_attn.varlen import varlen_linear_attention
from flash_bla.ops.simple_la.fused import simple_la

DTYPES = [torch.float32, torch.bfloat16, torch.float16]


# ---------------------------------------------------------------------------------------
# golden fixtures (values computed by the reference itself), fp32
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["linear_attn_a", "linear_attn_b", "linear_attn_c"])
def test_golden_linear_attn(name):
    g = load_golden(name)
    o, dq, dk, dv = run_op(lambda q, k, v: linear_attention(q, k, v, golden_scale(g), g["eps"]),
                           [g["q"], g["k"], g["v"]], g["do"])
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        check(got, g[key], torch.float32, f"{name}.{key}")


@pytest.mark.parametrize("name", ["decoupled_a", "decoupled_b"])
def test_golden_decoupled(name):
    g = load_golden(name)
    outs = run_op(lambda *a: decoupled_la(*a, golden_scale(g), g["eps"]),
                  [g["q"], g["k"], g["q_rope"], g["k_rope"], g["v"]], g["do"])
    for got, key in zip(outs, ("o", "dq", "dk", "dq_rope", "dk_rope", "dv")):
        check(got, g[key], torch.float32, f"{name}.{key}")


@pytest.mark.parametrize("name", ["simple_la_a", "simple_la_b"])
def test_golden_simple_la(name):
    g = load_golden(name)
    outs = run_op(lambda q, k, v: simple_la(q, k, v, golden_scale(g)), [g["q"], g["k"], g["v"]], g["do"])
    for got, key in zip(outs, ("o", "dq", "dk", "dv")):
        check(got, g[key], torch.float32, f"{name}.{key}")


@pytest.mark.parametrize("name", ["varlen_a", "varlen_b", "varlen_c"])
def test_golden_varlen(name):
    g = load_golden(name)
    cu = g["cu_seqlens"].cuda()
    max_len = int((g["cu_seqlens"][1:] - g["cu_seqlens"][:-1]).max())
    outs = run_op(lambda q, k, v: varlen_linear_attention(q, k, v, cu, max_len, golden_scale(g), g["eps"]),
                  [g["q"], g["k"], g["v"]], g["do"])
    for got, key in zip(outs, ("o", "dq", "dk", "dv")):
        check(got, g[key], torch.float32, f"{name}.{key}")


# ---------------------------------------------------------------------------------------
# oracle parity on seeded inputs: dtypes, ragged lengths, DK != DV, both kernel paths
# ---------------------------------------------------------------------------------------
LINEAR_SHAPES = [
    (2, 4, 1024, 64, 64),     # the fp32 acceptance configuration
    (1, 2, 1, 64, 64),
    (1, 2, 31, 16, 16),
    (1, 3, 129, 64, 64),
    (2, 2, 383, 128, 128),
    (1, 2, 640, 128, 32),     # DK = 2*d, DV = d/2 as PolaFormer calls it
    (1, 1, 200, 40, 40),
    (1, 2, 2048, 64, 64),
    (1, 3, 19000, 64, 128),   # DK != DV on the tensor-core kernels, units spread over many CTAs
    (1, 3, 19000, 128, 64),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", LINEAR_SHAPES)
@pytest.mark.parametrize("generic", [False, True])
def test_linear_attn(shape, dtype, generic):
    B, H, T, DK, DV = shape
    q, k, v, do = make_inputs(0, (B, H, T, DK), (B, H, T, DV), dtype)
    if generic:
        with P.generic_kernels():
            outs = run_op(lambda *a: linear_attention(*a), [q, k, v], do)
    else:
        outs = run_op(lambda *a: linear_attention(*a), [q, k, v], do)
    ref = [O.linear_attn_fwd(q, k, v)] + list(O.linear_attn_bwd(q, k, v, do))
    # with a single token o barely depends on q: dq is the difference of two terms that
    # cancel to ~1e-9 of their size, so its error is measured against one of the terms
    # (the same holds for dk: with one token o depends on k only through eps)
    terms = {}
    if T == 1:
        parts = O.decoupled_la_bwd(q, k, q, k, v, do)
        terms = {"dq": parts[2], "dk": parts[3]}
    for got, r, key in zip(outs, ref, ("o", "dq", "dk", "dv")):
        assert got.dtype == dtype and got.is_contiguous()
        check(got, r, dtype, f"linear_attn{shape}.{key}", magnitude=terms.get(key))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 2, 300, 64, 64), (2, 2, 257, 128, 128), (1, 2, 100, 24, 8),
                                   (1, 2, 5000, 64, 128), (1, 2, 5000, 128, 64)])
@pytest.mark.parametrize("scale,eps", [(None, 1e-6), (0.02, 1e-4)])
def test_linear_attn_scale_eps(shape, dtype, scale, eps):
    B, H, T, DK, DV = shape
    q, k, v, do = make_inputs(3, (B, H, T, DK), (B, H, T, DV), dtype)
    outs = run_op(lambda *a: linear_attention(*a, scale=scale, eps=eps), [q, k, v], do)
    ref = [O.linear_attn_fwd(q, k, v, scale, eps)] + list(O.linear_attn_bwd(q, k, v, do, scale, eps))
    for got, r, key in zip(outs, ref, ("o", "dq", "dk", "dv")):
        check(got, r, dtype, f"linear_attn{shape}.{key}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(2, 2, 515, 64, 64), (1, 2, 256, 128, 128), (1, 2, 77, 32, 48)])
def test_decoupled(shape, dtype):
    B, H, T, DK, DV = shape
    q, k, qr, kr, v, do = make_inputs(1, (B, H, T, DK), (B, H, T, DV), dtype, n_qk=4)
    outs = run_op(lambda *a: decoupled_la(*a), [q, k, qr, kr, v], do)
    ref = [O.decoupled_la_fwd(q, k, qr, kr, v)] + list(O.decoupled_la_bwd(q, k, qr, kr, v, do))
    for got, r, key in zip(outs, ref, ("o", "dq", "dk", "dq_rope", "dk_rope", "dv")):
        check(got, r, dtype, f"decoupled{shape}.{key}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(2, 2, 1000, 128, 128), (1, 2, 333, 64, 64), (1, 1, 50, 20, 36),
                                   (1, 3, 19000, 64, 128), (1, 3, 19000, 128, 64)])
def test_simple_la(shape, dtype):
    B, H, T, DK, DV = shape
    q, k, v, do = make_inputs(2, (B, H, T, DK), (B, H, T, DV), dtype, positive=False)
    outs = run_op(lambda *a: simple_la(*a), [q, k, v], do)
    ref = [O.simple_la_fwd(q, k, v)] + list(O.simple_la_bwd(q, k, v, do))
    for got, r, key in zip(outs, ref, ("o", "dq", "dk", "dv")):
        check(got, r, dtype, f"simple_la{shape}.{key}")


VARLEN_CASES = [
    ([8, 17, 32], 1, 8, 8), ([8, 17, 32], 8, 17, 13), ([8, 17, 32], 8, 64, 48), ([8, 17, 32], 1, 128, 128),
    ([300, 1, 129, 640], 4, 64, 64), ([1000, 24], 2, 128, 128),
    ([300, 1, 129, 640], 4, 32, 32), ([700, 130], 3, 16, 96),      # 16-bit: head dims below the tensor-core tiles
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", VARLEN_CASES)
@pytest.mark.parametrize("scale", [None, 0.02])
def test_varlen(case, dtype, scale):
    lengths, H, DK, DV = case
    tot = sum(lengths)
    q, k, v, do = make_inputs(42, (tot, H, DK), (tot, H, DV), dtype)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    cud = cu.cuda()
    outs = run_op(lambda *a: varlen_linear_attention(*a, cud, max(lengths), scale=scale), [q, k, v], do)
    ref = [O.varlen_linear_attn_fwd(q, k, v, cu, scale)] + list(O.varlen_linear_attn_bwd(q, k, v, do, cu, scale))
    # sequences of different lengths have outputs of different magnitude (scale 1/len):
    # each sequence is judged against its own RMS
    # a one-token sequence has dq, dk that are differences of two cancelling terms (see
    # test_linear_attn): those are judged against the size of one term
    for got, r, key in zip(outs, ref, ("o", "dq", "dk", "dv")):
        for lo, hi in zip(cu[:-1].tolist(), cu[1:].tolist()):
            mag = None
            if hi - lo == 1 and key in ("dq", "dk"):
                qs, ks, vs, ds = (x[lo:hi].transpose(0, 1) for x in (q, k, v, do))
                sc = 1.0 if scale is None else scale
                parts = O.decoupled_la_bwd(qs, ks, qs, ks, vs, ds, scale=sc)
                mag = (parts[2] if key == "dq" else parts[3]).transpose(0, 1)
            check(got[lo:hi], r[lo:hi], dtype, f"varlen{case}.{key}[{lo}:{hi}]", magnitude=mag)


def test_varlen_oversized_max_seqlen_and_no_leakage():
    lengths = [7, 11, 140]
    tot = sum(lengths)
    q, k, v, do = make_inputs(7, (tot, 2, 16), (tot, 2, 16), torch.float32)
    cu = torch.tensor([0, 7, 18, tot], dtype=torch.int32).cuda()
    exact = varlen_linear_attention(q.cuda(), k.cuda(), v.cuda(), cu, max(lengths))
    over = varlen_linear_attention(q.cuda(), k.cuda(), v.cuda(), cu, tot)
    assert torch.equal(exact, over)
    # changing one sequence leaves the outputs of the others bit-identical
    k2, v2 = k.clone(), v.clone()
    k2[7:18] += 1.0
    v2[7:18] -= 3.0
    other = varlen_linear_attention(q.cuda(), k2.cuda(), v2.cuda(), cu, max(lengths))
    assert torch.equal(other[:7], exact[:7]) and torch.equal(other[18:], exact[18:])
    assert not torch.equal(other[7:18], exact[7:18])


def test_varlen_argument_contract():
    q = torch.rand(10, 2, 16, device="cuda")
    cu = torch.tensor([0, 4, 10], dtype=torch.int32, device="cuda")
    ok = dict(q=q, k=q.clone(), v=q.clone(), cu_seqlens=cu, max_seqlen=6)
    varlen_linear_attention(**ok)
    bad = [
        (dict(ok, q=q[0]), ValueError), (dict(ok, k=q[:, :1]), ValueError),
        (dict(ok, v=torch.rand(9, 2, 16, device="cuda")), ValueError),
        (dict(ok, v=q.double()), ValueError), (dict(ok, q=q.cpu(), k=q.cpu(), v=q.cpu()), ValueError),
        (dict(ok, q=q.double(), k=q.double(), v=q.double()), TypeError),
        (dict(ok, q=torch.rand(10, 2, 129, device="cuda"), k=torch.rand(10, 2, 129, device="cuda")), ValueError),
        (dict(ok, cu_seqlens=cu.long()), ValueError), (dict(ok, cu_seqlens=cu.cpu()), ValueError),
        (dict(ok, cu_seqlens=cu[:1]), ValueError), (dict(ok, max_seqlen=0), ValueError),
        (dict(ok, max_seqlen=6.0), ValueError),
    ]
    for kwargs, exc in bad:
        with pytest.raises(exc):
            varlen_linear_attention(**kwargs)


# ---------------------------------------------------------------------------------------
# size-independent properties at the benchmark's full size
# ---------------------------------------------------------------------------------------
def test_full_size_properties_bf16():
    B, H, T, D = 8, 16, 32768, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.nn.functional.elu(torch.randn(B, H, T, D, device="cuda", generator=g)).add_(1).bfloat16()
    k = torch.nn.functional.elu(torch.randn(B, H, T, D, device="cuda", generator=g)).add_(1).bfloat16()
    v = torch.randn(B, H, T, D, device="cuda", generator=g).bfloat16()
    do = torch.randn(B, H, T, D, device="cuda", generator=g).bfloat16()
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = linear_attention(q, k, v)
    o.backward(do)
    # (1) spot-check two (b, h) slices against the CPU oracle
    for b, h in ((0, 0), (7, 15)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        qq, kk, vv, dd = (x[sl].detach().cpu() for x in (q, k, v, do))
        check(o[sl], O.linear_attn_fwd(qq, kk, vv), torch.bfloat16, "o")
        for got, r, key in zip((q.grad[sl], k.grad[sl], v.grad[sl]), O.linear_attn_bwd(qq, kk, vv, dd),
                               ("dq", "dk", "dv")):
            check(got, r, torch.bfloat16, key)
    # (2) (b, h) units are independent: rewriting the keys and values of one unit changes that
    # unit's output and leaves every other unit bit-identical
    k_mod, v_mod = k.detach().clone(), v.detach().clone()
    k_mod[3, 5] += 0.5
    v_mod[3, 5] *= -1.0
    o_mod = linear_attention(q.detach(), k_mod, v_mod)
    same = (o_mod == o.detach()).flatten(2).all(dim=-1)          # per (b, h)
    assert not same[3, 5]
    same[3, 5] = True
    assert same.all()
    # (3) the operator is linear in v: doubling v doubles o exactly (power-of-two scaling)
    o2 = linear_attention(q.detach(), k.detach(), (v.detach() * 2))
    assert torch.equal(o2, o.detach() * 2)
    # (4) run-to-run determinism of forward and backward
    q2, k2, v2 = (x.detach().clone().requires_grad_() for x in (q, k, v))
    o_again = linear_attention(q2, k2, v2)
    o_again.backward(do)
    assert torch.equal(o_again, o) and torch.equal(q2.grad, q.grad)
    assert torch.equal(k2.grad, k.grad) and torch.equal(v2.grad, v.grad)


def test_full_size_simple_la_bf16():
    """simple_la at B4-H32-D128, T = 262144 on one GPU (8.6 GB per tensor): two (b, h) slices against the CPU
    oracle, linearity in v, run-to-run determinism."""
    B, H, T, D = 4, 32, 262144, 128
    if torch.cuda.mem_get_info()[0] < 100 * 2 ** 30:
        pytest.skip("needs about 100 GB of free device memory")
    g = torch.Generator(device="cuda").manual_seed(0)
    q, k, v, do = (torch.randn(B, H, T, D, device="cuda", generator=g, dtype=torch.bfloat16) for _ in range(4))
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = simple_la(q, k, v)
    o.backward(do)
    for b, h in ((0, 0), (3, 31)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        qq, kk, vv, dd = (x[sl].detach().cpu() for x in (q, k, v, do))
        check(o[sl], O.simple_la_fwd(qq, kk, vv), torch.bfloat16, "cfg3.o")
        for got, r, key in zip((q.grad[sl], k.grad[sl], v.grad[sl]), O.simple_la_bwd(qq, kk, vv, dd), ("dq", "dk", "dv")):
            check(got, r, torch.bfloat16, "cfg3." + key)
    dq, dk, dv = q.grad, k.grad, v.grad
    q.grad = k.grad = v.grad = None
    o_again = simple_la(q, k, v)
    o_again.backward(do)
    assert torch.equal(o_again, o) and torch.equal(q.grad, dq) and torch.equal(k.grad, dk) and torch.equal(v.grad, dv)
    del o_again, dq, dk, dv
    q.grad = k.grad = v.grad = None
    with torch.no_grad():
        v.mul_(2)
        o2 = simple_la(q, k, v)
        assert torch.equal(o2, o * 2)


def test_full_size_varlen_bf16():
    """The packed configuration: 32 sequences with lengths drawn from [256, 16384] (seeded), H = 16, D = 64,
    bf16.  The shortest, the longest and the two sequences around the middle boundary against the CPU
    oracle; rewriting one sequence leaves every other sequence bit-identical."""
    H, D = 16, 64
    lengths = torch.randint(256, 16385, (32,), generator=torch.Generator().manual_seed(0))
    cu = torch.cat([torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)]).to(torch.int32)
    tot = int(cu[-1])
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.nn.functional.elu(torch.randn(tot, H, D, device="cuda", generator=g)).add_(1).bfloat16()
    k = torch.nn.functional.elu(torch.randn(tot, H, D, device="cuda", generator=g)).add_(1).bfloat16()
    v = torch.randn(tot, H, D, device="cuda", generator=g).bfloat16()
    do = torch.randn(tot, H, D, device="cuda", generator=g).bfloat16()
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    cud = cu.cuda()
    o = varlen_linear_attention(q, k, v, cud, int(lengths.max()))
    o.backward(do)
    picks = sorted({int(lengths.argmin()), int(lengths.argmax()), 15, 16})
    for s in picks:
        lo, hi = int(cu[s]), int(cu[s + 1])
        qq, kk, vv, dd = (x[lo:hi].detach().cpu().transpose(0, 1) for x in (q, k, v, do))     # (H, len, D)
        check(o[lo:hi].transpose(0, 1), O.linear_attn_fwd(qq, kk, vv), torch.bfloat16, f"cfg4.o[{s}]")
        for got, r, key in zip((q.grad, k.grad, v.grad), O.linear_attn_bwd(qq, kk, vv, dd), ("dq", "dk", "dv")):
            check(got[lo:hi].transpose(0, 1), r, torch.bfloat16, f"cfg4.{key}[{s}]")
    # no state leaks across the boundaries: change sequence 16 only
    lo, hi = int(cu[16]), int(cu[17])
    k2, v2 = k.detach().clone(), v.detach().clone()
    k2[lo:hi] += 0.5
    v2[lo:hi] *= -1.0
    o2 = varlen_linear_attention(q.detach(), k2, v2, cud, int(lengths.max()))
    assert torch.equal(o2[:lo], o.detach()[:lo]) and torch.equal(o2[hi:], o.detach()[hi:])
    assert not torch.equal(o2[lo:hi], o.detach()[lo:hi])


@pytest.mark.parametrize("D", [64, 32])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_tensors_at_an_odd_storage_offset(dtype, D):
    """Contiguous views whose storage does not start on a 16-byte boundary (a slice of a larger buffer) are
    accepted, as the reference accepts them: the CUDA-core kernels serve them (D = 64), or the narrow route
    works on aligned copies (D = 32, 16-bit)."""
    B, H, T = 1, 2, 300
    q, k, v, do = make_inputs(71, (B, H, T, D), (B, H, T, D), dtype)
    ref = [O.linear_attn_fwd(q, k, v)] + list(O.linear_attn_bwd(q, k, v, do))

    def shifted(x):                     # same values, storage offset of one element
        buf = torch.empty(x.numel() + 1, dtype=x.dtype, device="cuda")
        buf[1:].copy_(x.reshape(-1))
        out = buf[1:].view(x.shape)
        assert out.is_contiguous() and out.data_ptr() % 16 != 0
        return out
    xs = [shifted(x).requires_grad_() for x in (q, k, v)]
    o = linear_attention(*xs)
    o.backward(shifted(do))
    for got, r, key in zip((o, xs[0].grad, xs[1].grad, xs[2].grad), ref, ("o", "dq", "dk", "dv")):
        check(got, r, dtype, f"offset.{key}")


def test_empty_and_errors():
    # no tokens: nothing to compute (the default scale 1/L is undefined, as in the reference)
    q = torch.rand(1, 2, 0, 16, device="cuda", requires_grad=True)
    o = linear_attention(q, q, q, scale=1.0)
    assert o.shape == q.shape
    o.sum().backward()
    assert q.grad.shape == q.shape
    with pytest.raises(ZeroDivisionError):
        linear_attention(q, q, q)
    with pytest.raises(RuntimeError):
        linear_attention(torch.rand(1, 1, 4, 300, device="cuda"), torch.rand(1, 1, 4, 300, device="cuda"),
                         torch.rand(1, 1, 4, 8, device="cuda"))
    with pytest.raises(RuntimeError):
        linear_attention(torch.rand(1, 1, 4, 8), torch.rand(1, 1, 4, 8), torch.rand(1, 1, 4, 8))


def test_first_call_from_a_fresh_thread():
    """A thread that has made no CUDA call of its own (an autograd worker) may be the first caller.

    The tensor-map encoder is a driver call and needs a context bound to the thread; every buffer is
    allocated here so that the worker's only CUDA work is the library's.
    """
    import threading
    B, H, T, D = 2, 16, 1024, 64
    q, k, v, d_o = (x.cuda() for x in make_inputs(21, (B, H, T, D), (B, H, T, D), torch.bfloat16))
    prob = P.make_problem(q, batch=B, heads=H, seq_len=T, dk=D, dv=D, normalize=True, scale=D ** -0.5, eps=1e-6)
    o, state = P.forward(prob, q, k, v)
    ref = [x.cpu() for x in (o,) + tuple(P.backward(prob, q, k, v, d_o, state))]
    del o, state        # their blocks go back to the caching allocator: the worker allocates nothing new
    torch.cuda.synchronize()
    out, err = [], []

    def worker():
        try:
            o, state = P.forward(prob, q, k, v)
            out.append((o,) + tuple(P.backward(prob, q, k, v, d_o, state)))
            torch.cuda.synchronize()
        except Exception as e:      # surfaced in the main thread below
            err.append(e)

    th = threading.Thread(target=worker)
    th.start()
    th.join()
    assert not err, err
    for got, want in zip(out[0], ref):
        assert torch.equal(got.cpu(), want)


def test_cuda_graph_replay_matches_eager():
    """Forward + backward captured in a CUDA graph (after a warm-up on a side stream) and replayed on new
    input values gives the eager results bit for bit."""
    B, H, T, D = 2, 4, 1024, 64
    q, k, v, d_o = (x.cuda() for x in make_inputs(31, (B, H, T, D), (B, H, T, D), torch.bfloat16))
    sq, sk, sv = (torch.zeros_like(x).requires_grad_() for x in (q, k, v))

    def once():
        o = linear_attention(sq, sk, sv)
        o.backward(d_o)
        return o

    with torch.no_grad():
        for s_, x in ((sq, q), (sk, k), (sv, v)):
            s_.copy_(x)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            once()
    torch.cuda.current_stream().wait_stream(side)
    for s_ in (sq, sk, sv):
        s_.grad = None
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        o_static = once()
    # new values in the static inputs, then replay
    q2, k2, v2, _ = (x.cuda() for x in make_inputs(32, (B, H, T, D), (B, H, T, D), torch.bfloat16))
    with torch.no_grad():
        for s_, x in ((sq, q2), (sk, k2), (sv, v2)):
            s_.copy_(x)
    g.replay()
    torch.cuda.synchronize()
    got = [o_static.clone(), sq.grad.clone(), sk.grad.clone(), sv.grad.clone()]
    eq, ek, ev = (x.clone().requires_grad_() for x in (q2, k2, v2))
    o = linear_attention(eq, ek, ev)
    o.backward(d_o)
    for a, b in zip(got, (o, eq.grad, ek.grad, ev.grad)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("shape", [(8, 16, 1024, 64, 64), (2, 4, 4096, 128, 64), (1, 3, 700, 64, 128), (2, 2, 33000, 128, 128)])
@pytest.mark.parametrize("op", ["linear_attn", "simple_la"])
def test_unreduced_state_route_gives_the_same_bits(shape, op):
    """The one-call entry points may leave the state in per-segment pieces that the consuming pass adds
    itself; both routes add in the same order, so outputs and gradients are bit-identical."""
    B, H, T, K, V = shape
    q, k, v, d_o = (x.cuda() for x in make_inputs(41, (B, H, T, K), (B, H, T, V), torch.bfloat16))
    fn = linear_attention if op == "linear_attn" else simple_la
    res = []
    saved = P._want_unreduced
    try:
        for want in (True, False):
            P._want_unreduced = want
            xs = [x.clone().requires_grad_() for x in (q, k, v)]
            o = fn(*xs)
            o.backward(d_o)
            res.append([o] + [x.grad for x in xs])
    finally:
        P._want_unreduced = saved
    for a, b in zip(*res):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 1000, 4, 64, 64), (3, 257, 2, 32, 48), (1, 4096, 16, 64, 128)])
def test_linear_attention_blhd_layout(shape, dtype):
    """layout="blhd" takes (B, L, H, D) tensors as they are; results match the oracle on the permuted tensors."""
    B, L, H, K, V = shape
    q, k, v, d_o = make_inputs(51, (B, H, L, K), (B, H, L, V), dtype)
    rq, rk, rv = (x.double() for x in (q, k, v))
    ro = O.linear_attn_fwd(rq, rk, rv, None, 1e-6)
    rdq, rdk, rdv = O.linear_attn_bwd(rq, rk, rv, d_o.double(), None, 1e-6)
    xs = [x.cuda().permute(0, 2, 1, 3).contiguous().requires_grad_() for x in (q, k, v)]
    o = linear_attention(*xs, layout="blhd")
    assert o.shape == (B, L, H, V) and o.is_contiguous()
    o.backward(d_o.cuda().permute(0, 2, 1, 3).contiguous())
    for got, ref, name in ((o, ro, "o"), (xs[0].grad, rdq, "dq"), (xs[1].grad, rdk, "dk"), (xs[2].grad, rdv, "dv")):
        check(got.permute(0, 2, 1, 3), ref, dtype, f"blhd{shape}.{name}")


@pytest.mark.skipif(__import__("os").environ.get("FBLA_PAD_SMALL_DIMS", "1") == "0"
                    or __import__("os").environ.get("FBLA_NARROW_DIMS", "1") == "0",
                    reason="the narrow / padded routes are switched off")
@pytest.mark.parametrize("shape", [(2, 8, 8192, 32, 32), (1, 16, 8192, 48, 24), (1, 16, 8192, 96, 32), (4, 4, 196, 32, 32),
                                   (1, 3, 3136, 16, 112), (1, 2, 700, 80, 48)])
def test_small_head_dims_take_the_tensor_core_kernels(shape):
    """16-bit inputs whose head dims are not 64 / 128 (the reference's layers use 32): multiples of 16 are read and
    written at their own width by the 64- / 128-wide tensor-core kernels (TMA boxes zero-fill / clip the missing
    features), at any size; other dims of streaming size are zero-padded first.  Outputs and gradients keep the
    caller's shapes and match the oracle."""
    B, H, T, K, V = shape
    dtype = torch.bfloat16
    q, k, v, d_o = make_inputs(61, (B, H, T, K), (B, H, T, V), dtype)
    prob = P.make_problem(q, batch=B, heads=H, seq_len=T, dk=K, dv=V, normalize=True)
    if K % 16 == 0 and V % 16 == 0:
        assert P.narrow_route(prob) and P.padded_dims(q.cuda(), v.cuda()) is None
        from flash_bla import _C
        prob.flags |= _C.FLAG_NARROW
        assert P.kernel_path(prob) == 1
    else:
        assert not P.narrow_route(prob) and P.padded_dims(q.cuda(), v.cuda()) is not None
    rq, rk, rv = (x.double() for x in (q, k, v))
    refs = (O.linear_attn_fwd(rq, rk, rv, None, 1e-6),) + tuple(O.linear_attn_bwd(rq, rk, rv, d_o.double(), None, 1e-6))
    xs = [x.cuda().requires_grad_() for x in (q, k, v)]
    o = linear_attention(*xs)
    o.backward(d_o.cuda())
    assert o.shape == (B, H, T, V) and all(x.grad.shape == x.shape for x in xs)
    for got, ref, name in zip((o, xs[0].grad, xs[1].grad, xs[2].grad), refs, ("o", "dq", "dk", "dv")):
        check(got, ref, dtype, f"padded{shape}.{name}")
    # simple_la: default scale from the caller's key dim, not the padded one
    ref_o = O.simple_la_fwd(rq, rk, rv, None)
    check(simple_la(q.cuda(), k.cuda(), v.cuda()), ref_o, dtype, f"padded{shape}.simple_la")
