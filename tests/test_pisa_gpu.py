"""piecewise_sparse_attention on the GPU against the golden fixtures (produced by the
reference's own Triton kernels) and the CPU oracle."""
import os

import pytest
import torch

from oracle import bla_oracle as O
from helpers import check, load_golden

pytestmark = pytest.mark.gpu

from flash_bla.ops.piecewise_attn.kernel import (attention_forward, block_statistics, first_order_state,
                                                 fused_chunk_reduce, piecewise_sparse_attention, select_blocks)


@pytest.mark.parametrize("name", ["pisa_a", "pisa_b"])
def test_golden(name):
    g = load_golden(name)
    bs = int(g["block_size"])
    q, k, v = (g[x].cuda() for x in ("q", "k", "v"))
    qc, kc, vc = block_statistics(q, k, v, bs)
    h = first_order_state(k, v, kc, vc, bs)
    for got, key in ((qc, "qc"), (kc, "kc"), (vc, "vc")):
        check(got, g[key], torch.float32, f"{name}.{key}")
    assert O.rel_l2(h.cpu(), g["h"]) < 1e-4
    idx = select_blocks(qc, kc, g["scale"], g["density"], torch.float32)
    assert torch.equal(idx.long().sort(-1).values.cpu(), g["indices"].sort(-1).values)
    o = attention_forward(q, k, v, kc, vc, h, g["indices"].cuda(), bs, g["scale"])
    assert O.rel_l2(o.cpu(), g["o"]) < 1e-4
    # the whole operator picks the same blocks here, so it must give the same output
    o2 = piecewise_sparse_attention(q, k, v, density=g["density"], block_size=bs, scale=g["scale"])
    assert O.rel_l2(o2.cpu(), g["o"]) < 1e-4


def test_golden_with_bias():
    """use_bias=True against the reference-generated fixture: block norms, biased selection, output."""
    from flash_bla.ops.piecewise_attn.kernel import block_state_norms
    g = load_golden("pisa_c")
    bs = int(g["block_size"])
    q, k, v = (g[x].cuda() for x in ("q", "k", "v"))
    qc, kc, vc = block_statistics(q, k, v, bs)
    hn = block_state_norms(k, v, kc, bs)
    assert O.rel_l2(hn.cpu(), g["h_norm"]) < 1e-5
    for p_ in (1, 3):
        assert O.rel_l2(block_state_norms(k, v, kc, bs, p_).cpu(), O.pisa_block_hnorm(g["k"], g["v"], bs, p_)) < 1e-4
    idx = select_blocks(qc, kc, g["scale"], g["density"], torch.float32, hn[..., None, :])
    assert torch.equal(idx.long().sort(-1).values.cpu(), g["indices"].sort(-1).values)
    o = piecewise_sparse_attention(q, k, v, density=g["density"], block_size=bs, scale=g["scale"], use_bias=True)
    assert O.rel_l2(o.cpu(), g["o"]) < 1e-4
    # and it differs from the unbiased operator on this fixture
    o0 = piecewise_sparse_attention(q, k, v, density=g["density"], block_size=bs, scale=g["scale"])
    assert O.rel_l2(o0.cpu(), g["o"]) > 1e-3


def test_golden_dit_layer_pair_on_the_tensor_core_kernels():
    """One (batch, head) pair of the DiT-layer configuration, bf16, against the output of the reference's
    own kernel (GROUP_SIZE = 128, one group) on the same bf16-rounded inputs."""
    import numpy as np
    import os
    from helpers import GOLDEN, bf16_from_bits
    z = np.load(os.path.join(GOLDEN, "pisa_d.npz"))
    q, k, v = (bf16_from_bits(z[n]).bfloat16().cuda() for n in ("q_bf16", "k_bf16", "v_bf16"))
    bs, scale, density = int(z["block_size"]), float(z["scale"]), float(z["density"])
    qc, kc, vc = block_statistics(q, k, v, bs)
    assert O.rel_l2(kc.cpu(), torch.from_numpy(z["kc"])) < 1e-5 and O.rel_l2(vc.cpu(), torch.from_numpy(z["vc"])) < 1e-5
    h = first_order_state(k, v, kc, vc, bs)
    assert O.rel_l2(h.cpu(), torch.from_numpy(z["h"])) < 2e-3
    rows = torch.from_numpy(z["o_rows"])
    want = torch.from_numpy(z["o"])
    o = attention_forward(q, k, v, kc, vc, h, torch.from_numpy(z["indices"]).cuda(), bs, scale)
    check(o[:, :, rows.cuda()], want, torch.bfloat16, "pisa_d.o")
    # the whole operator: its own selection (bf16 scores) may differ in a few near-ties from the fp32
    # selection of the fixture, so most rows must agree, not all
    o2 = piecewise_sparse_attention(q, k, v, density=density, block_size=bs, scale=scale)
    err = (o2[:, :, rows.cuda()].float().cpu() - want).abs().amax(-1) / want.pow(2).mean().sqrt()
    assert (err <= 2e-2).float().mean().item() > 0.9


def test_more_blocks_than_one_group_follows_the_formula():
    """NT = 40 > the reference's GROUP_SIZE = 32: the fixture holds the reference kernel's
    order-dependent result (pinned by the oracle's restatement of that order in the CPU tests); this
    library rescales g as well, i.e. computes the formula, and so differs from the fixture there."""
    g = load_golden("pisa_e")
    bs = int(g["block_size"])
    q, k, v = (g[x].cuda() for x in ("q", "k", "v"))
    qc, kc, vc = block_statistics(q, k, v, bs)
    h = first_order_state(k, v, kc, vc, bs)
    o = attention_forward(q, k, v, kc, vc, h, g["indices"].cuda(), bs, g["scale"]).cpu()
    args = (g["q"], g["k"], g["v"], g["kc"], g["vc"], g["h"], g["indices"], bs, g["scale"])
    assert O.rel_l2(o, O.pisa_fwd_given(*args)) < 1e-4
    assert O.rel_l2(O.pisa_fwd_given(*args, reference_group_size=32), g["o"]) < 1e-5
    assert O.rel_l2(o, g["o"]) > 1e-2


CASES = [
    (1, 2, 300, 64, 64, 64, 0.2),
    (2, 2, 1000, 128, 128, 64, 0.1),
    (1, 3, 257, 32, 48, 32, 0.3),
    (1, 1, 130, 16, 16, 128, 0.5),
    (1, 2, 4608, 128, 128, 64, 0.1),     # one (b, h) pair of the DiT-layer configuration
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES)
def test_forward_matches_oracle(case, dtype):
    B, H, T, K, V, bs, density = case
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(B, H, T, d, generator=g).to(dtype) for d in (K, K, V))
    scale = K ** -0.5
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    qc, kc, vc = block_statistics(qd, kd, vd, bs)
    h = first_order_state(kd, vd, kc, vc, bs)
    idx = select_blocks(qc, kc, scale, density, dtype)
    o, stats = attention_forward(qd, kd, vd, kc, vc, h, idx, bs, scale, want_stats=True)
    rqc, rkc, rvc, rh = O.pisa_block_stats(q, k, v, bs)
    assert O.rel_l2(qc.cpu(), rqc) < 1e-5 and O.rel_l2(kc.cpu(), rkc) < 1e-5 and O.rel_l2(vc.cpu(), rvc) < 1e-5
    assert O.rel_l2(h.cpu(), rh) < (1e-4 if dtype == torch.float32 else 2e-3)
    ref, _ = O.pisa_fwd(q, k, v, density, bs, scale, indices=idx.cpu())
    if dtype == torch.float32:
        assert O.rel_l2(o.cpu(), ref) < 2e-5
    else:
        check(o, ref, dtype, f"pisa{case}.o")
    assert torch.isfinite(stats).all() and (stats[..., 1] > 0).all()


BWD_CASES = [
    (1, 2, 96, 16, 16, 16, 0.34),
    (1, 2, 150, 32, 24, 32, 0.25),     # ragged last block, dk != dv
    (2, 1, 320, 64, 64, 64, 0.2),
    (1, 1, 640, 128, 128, 64, 0.1),
    (1, 2, 300, 64, 64, 64, 0.2),      # tensor-core shapes with a ragged last block
    (1, 2, 1000, 128, 128, 64, 0.1),
    (1, 1, 4608, 128, 128, 64, 0.1),   # more than 64 blocks: two chunks of block statistics
    (1, 1, 4500, 64, 64, 64, 0.05),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", BWD_CASES)
def test_backward_matches_oracle(case, dtype):
    from flash_bla.ops.piecewise_attn.kernel import attention_backward
    B, H, T, K, V, bs, density = case
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(B, H, T, d, generator=g).to(dtype) for d in (K, K, V))
    do = torch.randn(B, H, T, V, generator=g).to(dtype)
    scale = K ** -0.5
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    qc, kc, vc = block_statistics(qd, kd, vd, bs)
    h = first_order_state(kd, vd, kc, vc, bs)
    idx = select_blocks(qc, kc, scale, density, dtype)
    o, stats = attention_forward(qd, kd, vd, kc, vc, h, idx, bs, scale, want_stats=True)
    dq, dk, dv = attention_backward(qd, kd, vd, o, do.cuda(), kc, vc, h, idx, stats, bs, scale)
    rq, rk, rv = O.pisa_bwd(q, k, v, do, idx.cpu(), bs, scale)
    for got, ref, name in ((dq, rq, "dq"), (dk, rk, "dk"), (dv, rv, "dv")):
        if dtype == torch.float32:
            err = O.rel_l2(got.cpu(), ref)
            assert err < 5e-5, f"pisa{case}.{name}: {err:.3e}"
        else:
            check(got, ref, dtype, f"pisa{case}.{name}")


def test_full_size_dit_layer_bf16():
    """The DiT-layer configuration at its full size (B2-H24, T = 4608, D = 128, block 64, density 0.1, bf16):
    two (b, h) pairs of forward and backward against the CPU oracle (with the selection the library made),
    (b, h) pairs independent of one another, forward bit-reproducible."""
    B, H, T, D, bs, density = 2, 24, 4608, 128, 64, 0.1
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v, do = (torch.randn(B, H, T, D, device="cuda", generator=g).bfloat16() for _ in range(4))
    scale = D ** -0.5
    qc, kc, vc = block_statistics(q, k, v, bs)
    idx = select_blocks(qc, kc, scale, density, torch.bfloat16)
    assert idx.shape == (B, H, T // bs, 7)
    xs = [x.clone().requires_grad_() for x in (q, k, v)]
    o = piecewise_sparse_attention(*xs, density=density, block_size=bs)
    o.backward(do)
    for b, h in ((0, 0), (1, 23)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        qq, kk, vv, dd = (x[sl].cpu() for x in (q, k, v, do))
        ref, _ = O.pisa_fwd(qq, kk, vv, density, bs, scale, indices=idx[sl].cpu())
        check(o[sl], ref, torch.bfloat16, "cfg5.o")
        for got, r, key in zip((x.grad[sl] for x in xs), O.pisa_bwd(qq, kk, vv, dd, idx[sl].cpu(), bs, scale),
                               ("dq", "dk", "dv")):
            check(got, r, torch.bfloat16, "cfg5." + key)
    o_again = piecewise_sparse_attention(q, k, v, density=density, block_size=bs)
    assert torch.equal(o_again, o.detach())
    k2, v2 = k.clone(), v.clone()
    k2[1, 5] += 0.25
    v2[1, 5] *= -1.0
    o2 = piecewise_sparse_attention(q, k2, v2, density=density, block_size=bs)
    same = (o2 == o.detach()).flatten(2).all(dim=-1)
    assert not same[1, 5]
    same[1, 5] = True
    assert same.all()


@pytest.mark.parametrize("dtype,case", [(torch.float32, (1, 2, 192, 32, 32, 32)), (torch.bfloat16, (1, 2, 384, 64, 64, 64))])
def test_out_of_range_block_indices_select_nothing(dtype, case):
    """Indices come from the caller through the C ABI: -1 and NT must not be dereferenced.  A bad index
    selects nothing, on the CUDA-core kernels (fp32) and on the tensor-core kernels (bf16) alike, so
    the result equals the one with that entry replaced by a duplicate of a good one... which counts the
    block once: compare the two kernel families with each other and require finite outputs."""
    from flash_bla.ops.piecewise_attn.kernel import attention_backward
    B, H, T, K, V, bs = case
    g = torch.Generator().manual_seed(2)
    q, k, v, do = (torch.randn(B, H, T, K, generator=g).to(dtype).cuda() for _ in range(4))
    nt = T // bs
    qc, kc, vc = block_statistics(q, k, v, bs)
    h = first_order_state(k, v, kc, vc, bs)
    idx = torch.empty(B, H, nt, 3, dtype=torch.int32, device="cuda")
    idx[..., 0] = torch.arange(nt, device="cuda")          # the query block's own key block
    idx[..., 1] = -1
    idx[..., 2] = nt
    scale = K ** -0.5
    o, stats = attention_forward(q, k, v, kc, vc, h, idx, bs, scale, want_stats=True)
    dq, dk, dv = attention_backward(q, k, v, o, do, kc, vc, h, idx, stats, bs, scale)
    for t in (o, dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    # the same selection without the bad entries, on the oracle
    good = idx[..., :1].cpu().long()
    ref, _ = O.pisa_fwd(q.cpu(), k.cpu(), v.cpu(), 0.0, bs, scale, indices=good)
    if dtype == torch.float32:
        assert O.rel_l2(o.cpu(), ref) < 2e-5
    else:
        check(o, ref, dtype, "bad-index.o")
    rq, rk, rv = O.pisa_bwd(q.cpu(), k.cpu(), v.cpu(), do.cpu(), good, bs, scale)
    for got, r, name in ((dq, rq, "dq"), (dk, rk, "dk"), (dv, rv, "dv")):
        if dtype == torch.float32:
            assert O.rel_l2(got.cpu(), r) < 5e-5, name
        else:
            check(got, r, dtype, "bad-index." + name)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,density,bias", [((2, 3, 72, 128), 0.1, False), ((1, 2, 40, 16), 0.3, True),
                                                ((1, 1, 1000, 64), 0.05, False), ((1, 2, 1, 8), 0.5, False)])
def test_block_selection_kernel(shape, density, bias, dtype):
    """The selection kernel against the reference's einsum / softmax / topk (the torch path of the same
    function): same scores means the same blocks wherever the k-th score is not tied with the next one."""
    B, H, NT, K = shape
    g = torch.Generator().manual_seed(9)
    qc = torch.randn(B, H, NT, K, generator=g).cuda()
    kc = torch.randn(B, H, NT, K, generator=g).cuda()
    hn = (torch.rand(B, H, 1, NT, generator=g) + 0.05).cuda() if bias else None
    scale = K ** -0.5
    got = select_blocks(qc, kc, scale, density, dtype, hn)
    want = select_blocks(qc, kc, scale, density, dtype, hn, use_torch=True)
    ns = max(1, int(density * NT))
    assert got.dtype == torch.int32 and got.shape == (B, H, NT, ns) and want.shape == got.shape
    assert int(got.min()) >= 0 and int(got.max()) < NT
    # no block twice
    assert (got.long().sort(-1).values.diff(dim=-1) > 0).all() or ns == 1
    # scores as the reference forms them
    score = torch.einsum('bhid,bhjd->bhij', qc.to(dtype), (kc * scale).to(dtype)).float()
    if bias:
        score = score + torch.log(hn.to(dtype) + 1e-5).float()
    picked = torch.gather(score, -1, got.long())
    # descending order, and nothing left out that beats the weakest pick (16-bit scores and the biased
    # form are rounded a little differently here and in torch: allow for that)
    tol = 1e-6 * score.abs().max().item() if dtype == torch.float32 and not bias else 2e-2 * score.abs().max().item()
    assert (picked.diff(dim=-1) <= tol).all() or ns == 1
    kth = torch.gather(score, -1, want.long()).min(-1).values
    assert (picked.min(-1).values >= kth - tol).all()
    if dtype == torch.float32 and not bias:
        assert torch.equal(got.long().sort(-1).values, want.sort(-1).values)


def test_autograd_end_to_end():
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 2, 256, 32, device="cuda", requires_grad=True) for _ in range(3))
    o = piecewise_sparse_attention(q, k, v, density=0.25, block_size=32)
    o.square().sum().backward()
    assert all(x.grad is not None and torch.isfinite(x.grad).all() for x in (q, k, v))
    # directional finite difference in fp32 (selection is piecewise constant around this point)
    with torch.no_grad():
        d = torch.randn_like(v) * 1e-3
        f = lambda vv: piecewise_sparse_attention(q, k, vv, density=0.25, block_size=32).square().sum()
        fd = (f(v + d) - f(v - d)).item() / 2
        an = (v.grad * d).sum().item()
    assert abs(fd - an) <= 2e-2 * abs(an) + 1e-4


def test_reference_surface():
    q = torch.randn(1, 2, 128, 32, device="cuda")
    qc, kc, vc, h, bias = fused_chunk_reduce(q, q, q, 32)
    assert qc.shape == (1, 2, 4, 32) and h.shape == (1, 2, 32, 32) and bias is None and qc.dtype == q.dtype
    *_, bias = fused_chunk_reduce(q, q, q, 32, use_bias=True)
    assert bias.shape == (1, 2, 1, 4) and bias.dtype == q.dtype
    with pytest.raises(RuntimeError):
        piecewise_sparse_attention(q.cpu(), q.cpu(), q.cpu())


_CHILD = r"""
import sys, torch
sys.path.insert(0, sys.argv[1])
from flash_bla.ops.piecewise_attn.kernel import piecewise_sparse_attention
g = torch.Generator(device="cuda").manual_seed(11)
q, k, v, do = (torch.randn(1, 2, 1000, 128, device="cuda", generator=g).bfloat16() for _ in range(4))
xs = [x.clone().requires_grad_() for x in (q, k, v)]
o = piecewise_sparse_attention(*xs, density=0.2, block_size=64)
o.backward(do)
torch.save([o.detach().cpu()] + [x.grad.cpu() for x in xs], sys.argv[2])
"""


def test_mma_sync_kernels_agree_with_the_tcgen05_kernels(tmp_path):
    """The mma.sync attention kernels stay in the library (FBLA_PISA_TC=0; the key side of very long sequences):
    the same seeded forward + backward (ragged last block, bf16, D = 128) through both kernel families, each in
    its own process because the switch is read once."""
    import subprocess
    import sys
    pkg = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "flash-bidirectional-linear-attention_b200")
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    outs = []
    for flag in ("1", "0"):
        out = tmp_path / f"out{flag}.pt"
        env = dict(os.environ, FBLA_PISA_TC=flag)
        r = subprocess.run([sys.executable, str(script), pkg, str(out)], env=env, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(torch.load(out))
    for name, a, b in zip(("o", "dq", "dk", "dv"), *outs):
        # two results rounded to bf16 independently: within 2e-2 of the RMS, or neighbours on the bf16 grid
        a, b = a.double(), b.double()
        rms = b.square().mean().sqrt().item()
        diff = (a - b).abs()
        ulp = torch.exp2(torch.floor(torch.log2(torch.maximum(a.abs(), b.abs()).clamp_min(1e-30))) - 7)
        bad = (diff > 2e-2 * rms) & (diff > ulp)
        assert not bad.any(), f"{name}: tcgen05 vs mma.sync differ by {(diff / rms).max().item():.3e} of the RMS"
