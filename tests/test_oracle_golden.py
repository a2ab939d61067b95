"""The CPU oracle against the fixtures produced by the reference itself
(tests/golden/make_golden.py).  Pins the oracle; needs no GPU."""
import os

import numpy as np
import pytest
import torch

from oracle import bla_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for k in z.files:
        a = z[k]
        out[k] = torch.from_numpy(a) if a.ndim else a.item()
    return out


def scale_of(g):
    return None if g["scale"] < 0 else float(g["scale"])


# The golden values were produced in fp32 by torch; the oracle runs in fp64.
TOL = 2e-5


def close(got, ref):
    assert O.rel_l2(got, ref) < TOL, O.rel_l2(got, ref)


@pytest.mark.parametrize("name", ["linear_attn_a", "linear_attn_b", "linear_attn_c"])
def test_linear_attn(name):
    g = load(name)
    sc = scale_of(g)
    close(O.linear_attn_fwd(g["q"], g["k"], g["v"], sc, g["eps"]), g["o"])
    dq, dk, dv = O.linear_attn_bwd(g["q"], g["k"], g["v"], g["do"], sc, g["eps"])
    close(dq, g["dq"]), close(dk, g["dk"]), close(dv, g["dv"])


@pytest.mark.parametrize("name", ["decoupled_a", "decoupled_b"])
def test_decoupled(name):
    g = load(name)
    sc = scale_of(g)
    args = (g["q"], g["k"], g["q_rope"], g["k_rope"], g["v"])
    close(O.decoupled_la_fwd(*args, sc, g["eps"]), g["o"])
    dq, dk, dqr, dkr, dv = O.decoupled_la_bwd(*args, g["do"], sc, g["eps"])
    close(dq, g["dq"]), close(dk, g["dk"]), close(dqr, g["dq_rope"])
    close(dkr, g["dk_rope"]), close(dv, g["dv"])


@pytest.mark.parametrize("name", ["simple_la_a", "simple_la_b"])
def test_simple_la(name):
    g = load(name)
    sc = scale_of(g)
    close(O.simple_la_fwd(g["q"], g["k"], g["v"], sc), g["o"])
    dq, dk, dv = O.simple_la_bwd(g["q"], g["k"], g["v"], g["do"], sc)
    close(dq, g["dq"]), close(dk, g["dk"]), close(dv, g["dv"])


@pytest.mark.parametrize("name", ["varlen_a", "varlen_b", "varlen_c"])
def test_varlen(name):
    g = load(name)
    sc = scale_of(g)
    close(O.varlen_linear_attn_fwd(g["q"], g["k"], g["v"], g["cu_seqlens"], sc, g["eps"]), g["o"])
    dq, dk, dv = O.varlen_linear_attn_bwd(g["q"], g["k"], g["v"], g["do"], g["cu_seqlens"], sc, g["eps"])
    close(dq, g["dq"]), close(dk, g["dk"]), close(dv, g["dv"])


@pytest.mark.parametrize("name", ["pisa_a", "pisa_b"])
def test_pisa_forward(name):
    g = load(name)
    bs = int(g["block_size"])
    qc, kc, vc, h = O.pisa_block_stats(g["q"], g["k"], g["v"], bs)
    close(qc, g["qc"]), close(kc, g["kc"]), close(vc, g["vc"])
    assert O.rel_l2(h, g["h"]) < 1e-4
    # the selection: same set of blocks per query block
    idx = O.pisa_select(qc, kc, g["scale"], g["density"])
    assert torch.equal(idx.sort(-1).values, g["indices"].sort(-1).values)
    o, _ = O.pisa_fwd(g["q"], g["k"], g["v"], g["density"], bs, g["scale"], indices=g["indices"])
    assert O.rel_l2(o, g["o"]) < 1e-4


def test_pisa_forward_with_bias():
    """use_bias=True: the selection ranks softmax(score + log(norm of each block's first-order state))."""
    g = load("pisa_c")
    bs = int(g["block_size"])
    qc, kc, vc, h = O.pisa_block_stats(g["q"], g["k"], g["v"], bs)
    h_norm = O.pisa_block_hnorm(g["k"], g["v"], bs)
    assert O.rel_l2(h_norm, g["h_norm"]) < 1e-4
    assert O.rel_l2(O.pisa_scores(qc, kc, g["scale"], h_norm), g["score"]) < 1e-4
    idx = O.pisa_select(qc, kc, g["scale"], g["density"], h_norm)
    assert torch.equal(idx.sort(-1).values, g["indices"].sort(-1).values)
    # the bias changes the selection on this fixture, i.e. the case does exercise it
    assert not torch.equal(O.pisa_select(qc, kc, g["scale"], g["density"]).sort(-1).values, g["indices"].sort(-1).values)
    o, _ = O.pisa_fwd(g["q"], g["k"], g["v"], g["density"], bs, g["scale"], indices=g["indices"])
    assert O.rel_l2(o, g["o"]) < 1e-4


def test_pisa_dit_layer_pair_with_one_group():
    """One (batch, head) pair of the DiT-layer configuration (T = 4608, D = 128, 72 blocks, 7 selected),
    reference kernel run with GROUP_SIZE = 128: one group covers all blocks, the formula must hold."""
    import numpy as np
    from helpers import GOLDEN, bf16_from_bits
    z = np.load(os.path.join(GOLDEN, "pisa_d.npz"))
    q, k, v = (bf16_from_bits(z[n]) for n in ("q_bf16", "k_bf16", "v_bf16"))
    bs, scale = int(z["block_size"]), float(z["scale"])
    qc, kc, vc, h = O.pisa_block_stats(q, k, v, bs)
    assert O.rel_l2(kc, torch.from_numpy(z["kc"])) < 1e-5 and O.rel_l2(vc, torch.from_numpy(z["vc"])) < 1e-5
    assert O.rel_l2(h, torch.from_numpy(z["h"])) < 1e-5
    idx = O.pisa_select(qc, kc, scale, float(z["density"]))
    assert idx.shape[-1] == 7
    assert torch.equal(idx.sort(-1).values, torch.from_numpy(z["indices"]).sort(-1).values)
    o, _ = O.pisa_fwd(q, k, v, float(z["density"]), bs, scale, indices=torch.from_numpy(z["indices"]))
    assert O.rel_l2(o[:, :, torch.from_numpy(z["o_rows"])], torch.from_numpy(z["o"])) < 1e-5


def test_pisa_more_blocks_than_one_group_pins_the_reference_order():
    """NT = 40 > GROUP_SIZE = 32: the reference kernel does not rescale the g of earlier groups when
    the running maximum grows, so its output depends on GROUP_SIZE.  The oracle's restatement of that
    order reproduces the fixture; the formula (what this library computes, and what the kernel gives
    with one group) does not."""
    g = load("pisa_e")
    bs = int(g["block_size"])
    args = (g["q"], g["k"], g["v"], g["kc"], g["vc"], g["h"], g["indices"], bs, g["scale"])
    assert int(g["group_size"]) == 32 and g["kc"].shape[-2] == 40
    assert O.rel_l2(O.pisa_fwd_given(*args, reference_group_size=32), g["o"]) < 1e-5
    assert O.rel_l2(O.pisa_fwd_given(*args), g["o"]) > 1e-2
    # one group covering everything is the formula again
    assert O.rel_l2(O.pisa_fwd_given(*args, reference_group_size=64), O.pisa_fwd_given(*args)) < 1e-12


def test_pisa_backward_matches_finite_differences():
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 1, 40, 8, dtype=torch.float64) for _ in range(3))
    do = torch.randn(1, 1, 40, 8, dtype=torch.float64)
    _, idx = O.pisa_fwd(q, k, v, 0.4, 8)
    dq, dk, dv = O.pisa_bwd(q, k, v, do, idx, 8)

    def loss(q_, k_, v_):
        return (O.pisa_fwd(q_, k_, v_, 0.4, 8, indices=idx)[0] * do).sum().item()
    h = 1e-6
    for x, gx, name in ((q, dq, "q"), (k, dk, "k"), (v, dv, "v")):
        for pos in [(0, 0, 3, 2), (0, 0, 39, 7), (0, 0, 17, 0)]:
            xp, xm = x.clone(), x.clone()
            xp[pos] += h
            xm[pos] -= h
            args_p = {"q": q, "k": k, "v": v}
            args_m = dict(args_p)
            args_p[name], args_m[name] = xp, xm
            fd = (loss(args_p["q"], args_p["k"], args_p["v"]) - loss(args_m["q"], args_m["k"], args_m["v"])) / (2 * h)
            assert abs(fd - gx[pos].item()) < 1e-5 * max(1.0, abs(fd)), (name, pos, fd, gx[pos].item())
