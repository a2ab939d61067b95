"""CPU oracle for the bidirectional linear-attention operators.

TEST INFRASTRUCTURE ONLY.  This module restates, on the CPU with dense torch
tensors, what the reference operators compute.  It is the checker the parity
tests compare the CUDA library against, and the CPU baseline the benchmark
times beside the GPU run.  Nothing in the shipped package imports it.

Parity pin: every function below is checked against outputs of the reference's
own torch path (``flash_bla/ops/linear_attn/naive.py``,
``flash_bla/ops/simple_la/naive.py``, with gradients from torch autograd) and,
for the piecewise operator, against the reference Triton kernels executed by
the Triton CPU interpreter.  Those outputs are stored as fixtures under
``tests/golden/`` together with the script that produced them.
The backward of the piecewise operator has no counterpart in the reference:
its parity is unpinned; the oracle differentiates the forward restatement with
the block selection held constant.

All functions take and return CPU tensors.  ``acc`` selects the arithmetic
type (``torch.float64`` for the tightest check, ``torch.float32`` to mirror the
reference's own precision).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch


def _f(x: torch.Tensor, acc: torch.dtype) -> torch.Tensor:
    return x.detach().to(acc)


# ---------------------------------------------------------------------------
# linear_attn (normalised) -- flash_bla/ops/linear_attn/naive.py:6-14 (forward),
# flash_bla/ops/linear_attn/fused.py:238-242,327-328 (backward identities).
# ---------------------------------------------------------------------------

def linear_attn_state(k, v, t_norm: Optional[int] = None, acc=torch.float64):
    """Raw per-(batch, head) state: ``S = K^T V`` and the key sum.

    Follows flash_bla/ops/linear_attn/fused.py:66-75 without the scale (applied
    when the state is used) and without the division by L (``t_norm``)."""
    k_, v_ = _f(k, acc), _f(v, acc)
    s = k_.transpose(-2, -1) @ v_
    ksum = k_.sum(dim=-2)
    return s, ksum


def linear_attn_fwd(q, k, v, scale: Optional[float] = None, eps: float = 1e-6,
                    acc=torch.float64):
    """``O = Q (K^T (V*scale)) / (Q . mean_t K + eps)``;
    flash_bla/ops/linear_attn/naive.py:6-14, default scale 1/L
    (flash_bla/ops/linear_attn/fused.py:477-478)."""
    L = k.shape[-2]
    if scale is None:
        scale = 1.0 / L
    q_ = _f(q, acc)
    s, ksum = linear_attn_state(k, v, acc=acc)
    km = ksum / L
    z = (q_ * km[..., None, :]).sum(-1, keepdim=True) + eps
    return (q_ @ (s * scale)) / z


def linear_attn_bwd(q, k, v, do, scale: Optional[float] = None, eps: float = 1e-6,
                    acc=torch.float64):
    """Closed-form gradients (dq, dk, dv).

    Identities from flash_bla/ops/linear_attn/fused.py:238-242 (dS, dz, dq,
    dk-mean term) and :327-328 (dk, dv).  ``dz`` is written through
    ``o = qS/z`` so the saved output is not needed."""
    L = k.shape[-2]
    if scale is None:
        scale = 1.0 / L
    q_, k_, v_, do_ = (_f(x, acc) for x in (q, k, v, do))
    s = (k_.transpose(-2, -1) @ v_) * scale          # [.., DK, DV]
    km = k_.mean(dim=-2)                               # [.., DK]
    z = (q_ * km[..., None, :]).sum(-1, keepdim=True) + eps
    t = do_ @ s.transpose(-2, -1)                      # dO S^T  [.., L, DK]
    dz = -(q_ * t).sum(-1, keepdim=True) / (z * z)     # = -sum(o*dO)/z
    dq = t / z + dz * km[..., None, :]
    ds = (q_ / z).transpose(-2, -1) @ do_              # [.., DK, DV]
    dkm = (dz * q_).sum(dim=-2) / L                    # [.., DK]
    dk = (v_ * scale) @ ds.transpose(-2, -1) + dkm[..., None, :]
    dv = (k_ @ ds) * scale
    return dq, dk, dv


# ---------------------------------------------------------------------------
# decoupled_la -- flash_bla/ops/linear_attn/naive.py:17-26 (forward),
# flash_bla/ops/linear_attn/decoupled.py:277-281,377-380 (backward identities).
# ---------------------------------------------------------------------------

def decoupled_la_fwd(q, k, q_rope, k_rope, v, scale: Optional[float] = None,
                     eps: float = 1e-6, acc=torch.float64):
    L = k.shape[-2]
    if scale is None:
        scale = 1.0 / L
    q_, k_, qr_, kr_, v_ = (_f(x, acc) for x in (q, k, q_rope, k_rope, v))
    km = k_.mean(dim=-2)
    z = (q_ * km[..., None, :]).sum(-1, keepdim=True) + eps
    s = (kr_.transpose(-2, -1) @ v_) * scale
    return (qr_ @ s) / z


def decoupled_la_bwd(q, k, q_rope, k_rope, v, do, scale: Optional[float] = None,
                     eps: float = 1e-6, acc=torch.float64):
    """(dq, dk, dq_rope, dk_rope, dv); decoupled.py:277-281 and :377-380."""
    L = k.shape[-2]
    if scale is None:
        scale = 1.0 / L
    q_, k_, qr_, kr_, v_, do_ = (_f(x, acc) for x in (q, k, q_rope, k_rope, v, do))
    km = k_.mean(dim=-2)
    z = (q_ * km[..., None, :]).sum(-1, keepdim=True) + eps
    s = (kr_.transpose(-2, -1) @ v_) * scale
    t = do_ @ s.transpose(-2, -1)
    dz = -(qr_ * t).sum(-1, keepdim=True) / (z * z)
    dq_rope = t / z
    dq = dz * km[..., None, :]
    ds = (qr_ / z).transpose(-2, -1) @ do_
    dkm = (dz * q_).sum(dim=-2) / L
    dk = dkm[..., None, :].expand_as(k_).clone()
    dk_rope = (v_ * scale) @ ds.transpose(-2, -1)
    dv = (kr_ @ ds) * scale
    return dq, dk, dq_rope, dk_rope, dv


# ---------------------------------------------------------------------------
# simple_la -- flash_bla/ops/simple_la/naive.py:8-20 (forward),
# flash_bla/ops/simple_la/fused.py:198,395-397 (backward identities).
# ---------------------------------------------------------------------------

def simple_la_fwd(q, k, v, scale: Optional[float] = None, acc=torch.float64):
    if scale is None:
        scale = q.shape[-1] ** -0.5                    # simple_la/fused.py:648-649
    q_, k_, v_ = (_f(x, acc) for x in (q, k, v))
    return q_ @ ((k_.transpose(-2, -1) @ v_) * scale)


def simple_la_bwd(q, k, v, do, scale: Optional[float] = None, acc=torch.float64):
    if scale is None:
        scale = q.shape[-1] ** -0.5
    q_, k_, v_, do_ = (_f(x, acc) for x in (q, k, v, do))
    s = (k_.transpose(-2, -1) @ v_) * scale
    ds = q_.transpose(-2, -1) @ do_                    # simple_la/fused.py:198
    dq = do_ @ s.transpose(-2, -1)                     # :395
    dk = (v_ * scale) @ ds.transpose(-2, -1)           # :396
    dv = (k_ @ ds) * scale                             # :397
    return dq, dk, dv


# ---------------------------------------------------------------------------
# varlen_linear_attention -- flash_bla/ops/linear_attn/naive.py:29-43 (forward),
# flash_bla/ops/linear_attn/varlen.py:217-219,312-314 (backward identities).
# Packed layout (total_tokens, heads, dim); int32 cu_seqlens.
# ---------------------------------------------------------------------------

def _segments(cu_seqlens) -> Sequence[Tuple[int, int]]:
    cu = [int(x) for x in cu_seqlens.tolist()]
    return [(cu[i], cu[i + 1]) for i in range(len(cu) - 1)]


def varlen_linear_attn_fwd(q, k, v, cu_seqlens, scale: Optional[float] = None,
                           eps: float = 1e-6, acc=torch.float64):
    out = torch.zeros(q.shape[0], q.shape[1], v.shape[-1], dtype=acc)
    for bos, eos in _segments(cu_seqlens):
        if eos <= bos:
            continue
        # per-sequence default scale 1/length: varlen.py:66
        sc = (1.0 / (eos - bos)) if scale is None else scale
        o = linear_attn_fwd(q[bos:eos].transpose(0, 1), k[bos:eos].transpose(0, 1),
                            v[bos:eos].transpose(0, 1), scale=sc, eps=eps, acc=acc)
        out[bos:eos] = o.transpose(0, 1)
    return out


def varlen_linear_attn_bwd(q, k, v, do, cu_seqlens, scale: Optional[float] = None,
                           eps: float = 1e-6, acc=torch.float64):
    dq = torch.zeros(q.shape, dtype=acc)
    dk = torch.zeros(k.shape, dtype=acc)
    dv = torch.zeros(v.shape, dtype=acc)
    for bos, eos in _segments(cu_seqlens):
        if eos <= bos:
            continue
        sc = (1.0 / (eos - bos)) if scale is None else scale
        a, b, c = linear_attn_bwd(q[bos:eos].transpose(0, 1), k[bos:eos].transpose(0, 1),
                                  v[bos:eos].transpose(0, 1), do[bos:eos].transpose(0, 1),
                                  scale=sc, eps=eps, acc=acc)
        dq[bos:eos] = a.transpose(0, 1)
        dk[bos:eos] = b.transpose(0, 1)
        dv[bos:eos] = c.transpose(0, 1)
    return dq, dk, dv


# ---------------------------------------------------------------------------
# piecewise_sparse_attention (PISA) --
# flash_bla/ops/piecewise_attn/kernel.py:89-128 (block statistics),
# :152-176 (h = sum of per-block centred k^T v), :305-318 (scale, block score,
# top-k selection), :216-292 (exact / zeroth-order / first-order phases).
# ---------------------------------------------------------------------------

def pisa_block_stats(q, k, v, block_size: int, acc=torch.float64):
    """qc, kc = per-block means (divided by the true tail length), vc = per-block
    sums, h = sum over blocks of (k - kc)^T v.  kernel.py:105-118,174-176."""
    q_, k_, v_ = (_f(x, acc) for x in (q, k, v))
    T = k_.shape[-2]
    nt = (T + block_size - 1) // block_size
    qc, kc, vc = [], [], []
    h = torch.zeros(*k_.shape[:-2], k_.shape[-1], v_.shape[-1], dtype=acc)
    for c in range(nt):
        lo, hi = c * block_size, min(T, (c + 1) * block_size)
        qb, kb, vb = q_[..., lo:hi, :], k_[..., lo:hi, :], v_[..., lo:hi, :]
        qc.append(qb.mean(dim=-2))
        kcm = kb.mean(dim=-2)
        kc.append(kcm)
        vc.append(vb.sum(dim=-2))
        h = h + (kb - kcm[..., None, :]).transpose(-2, -1) @ vb
    return torch.stack(qc, -2), torch.stack(kc, -2), torch.stack(vc, -2), h


def pisa_block_hnorm(k, v, block_size: int, p: float = 2, acc=torch.float64):
    """p-norm of every block's first-order state ``hc_c = (K_c - kc_c)^T V_c`` taken over
    its dk*dv entries: the selection bias of ``use_bias=True``; kernel.py:118 (hc),
    :172-173 (norm).  Shape (..., NT)."""
    k_, v_ = _f(k, acc), _f(v, acc)
    T = k_.shape[-2]
    nt = (T + block_size - 1) // block_size
    out = []
    for c in range(nt):
        lo, hi = c * block_size, min(T, (c + 1) * block_size)
        kb, vb = k_[..., lo:hi, :], v_[..., lo:hi, :]
        hc = (kb - kb.mean(dim=-2, keepdim=True)).transpose(-2, -1) @ vb
        out.append(torch.norm(hc.flatten(-2, -1), p=p, dim=-1))
    return torch.stack(out, -1)


def pisa_scores(qc, kc, scale: float, h_norm=None):
    """Block scores the selection ranks; with the bias of ``use_bias=True`` they are
    ``softmax(score + log(h_norm + 1e-5))`` over the key blocks.  kernel.py:313-315."""
    score = torch.einsum('...id,...jd->...ij', qc, kc * scale)
    if h_norm is not None:
        score = torch.softmax(score + torch.log(h_norm[..., None, :] + 1e-5), dim=-1)
    return score


def pisa_select(qc, kc, scale: float, density: float, h_norm=None):
    """Indices of the top-scoring key blocks per query block; kernel.py:313-318."""
    nt = kc.shape[-2]
    top_k = max(1, int(density * nt))
    return torch.topk(pisa_scores(qc, kc, scale, h_norm), k=top_k, dim=-1).indices


def pisa_fwd_given(q, k, v, kc, vc, h, indices, block_size: int, scale: float,
                   acc=torch.float64, differentiable: bool = False,
                   reference_group_size: Optional[int] = None):
    """Forward with block statistics and the selection given.

    ``reference_group_size``: restate the reference kernel's evaluation order instead
    of the formula below.  The kernel visits the unselected blocks in groups of
    GROUP_SIZE (an autotuned constant, 32 or 128), and each time the running
    maximum grows it rescales the numerator and ``l`` but NOT the ``g`` gathered
    from earlier groups (kernel.py:262-276), so with more blocks than one group
    its result depends on GROUP_SIZE and differs from the formula.  With one
    group (NT <= GROUP_SIZE) both agree.

    Per query row: running max ``m`` over exact logits of the selected blocks
    and block-mean logits of the unselected blocks; ``p_ex = exp(s - m)`` on
    selected blocks; ``p_ap = exp(q.kc_c*scale - m)`` on unselected blocks c;
    ``g = sum_c p_ap*len_c``;
    ``O = (p_ex V + p_ap vc + (q h) g scale / T) / (sum p_ex + g)``.
    kernel.py:216-292."""
    cast = (lambda x: x.to(acc)) if differentiable else (lambda x: _f(x, acc))
    q_, k_, v_, kc_, vc_, h_ = (cast(x) for x in (q, k, v, kc, vc, h))
    indices = indices.long()
    T = k_.shape[-2]
    nt = kc_.shape[-2]
    lead = q_.shape[:-2]
    outs = []
    lens = torch.full((nt,), float(block_size), dtype=acc)
    lens[-1] = T - (nt - 1) * block_size
    for i in range(nt):
        lo, hi = i * block_size, min(T, (i + 1) * block_size)
        qb = q_[..., lo:hi, :]                                       # [.., bt, K]
        idx = indices[..., i, :]                                     # [.., NS]
        # token positions of the selected blocks, clipped at T
        pos = idx[..., :, None] * block_size + torch.arange(block_size)   # [.., NS, bs]
        valid = pos < T
        posc = pos.clamp(max=T - 1).flatten(-2)                      # [.., NS*bs]
        kk = torch.gather(k_, -2, posc[..., None].expand(*lead, posc.shape[-1], k_.shape[-1]))
        vv = torch.gather(v_, -2, posc[..., None].expand(*lead, posc.shape[-1], v_.shape[-1]))
        s_ex = (qb @ kk.transpose(-2, -1)) * scale
        s_ex = s_ex.masked_fill(~valid.flatten(-2)[..., None, :], float('-inf'))
        s_ap = (qb @ kc_.transpose(-2, -1)) * scale                  # [.., bt, nt]
        sel = torch.zeros(*lead, nt, dtype=torch.bool)
        sel.scatter_(-1, idx, True)
        s_ap = s_ap.masked_fill(sel[..., None, :], float('-inf'))
        if reference_group_size is None:
            m = torch.maximum(s_ex.max(-1).values, s_ap.max(-1).values)[..., None]
            p_ex = torch.exp(s_ex - m)
            p_ap = torch.exp(s_ap - m)
            g = (p_ap * lens).sum(-1, keepdim=True)
            num = p_ex @ vv + p_ap @ vc_ + (qb @ h_) * (g * scale / T)
            outs.append(num / (p_ex.sum(-1, keepdim=True) + g))
            continue
        # the reference kernel's order: exact phase, then groups of unselected blocks
        m = s_ex.max(-1, keepdim=True).values
        p_ex = torch.exp(s_ex - m)
        l = p_ex.sum(-1, keepdim=True)
        num = p_ex @ vv
        g = torch.zeros_like(l)
        for c0 in range(0, nt, reference_group_size):
            c1 = min(nt, c0 + reference_group_size)
            s_grp = s_ap[..., c0:c1]
            new_m = torch.maximum(m, s_grp.max(-1, keepdim=True).values)
            alpha = torch.exp(m - new_m)
            num, l, m = num * alpha, l * alpha, new_m               # kernel.py:264-267: g is left as it is
            p_grp = torch.exp(s_grp - m)
            num = num + p_grp @ vc_[..., c0:c1, :]
            g = g + (p_grp * lens[c0:c1]).sum(-1, keepdim=True)
        num = num + (qb @ h_) * (g * scale / T)
        outs.append(num / (l + g))
    return torch.cat(outs, dim=-2)


def pisa_fwd(q, k, v, density: float = 0.1, block_size: int = 64,
             scale: Optional[float] = None, indices=None, acc=torch.float64):
    """Whole operator; kernel.py:295-333 with ``use_bias=False``.  Returns
    (o, indices).  Pass ``indices`` to pin the selection."""
    K = k.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    qc, kc, vc, h = pisa_block_stats(q, k, v, block_size, acc=acc)
    if indices is None:
        indices = pisa_select(qc, kc, scale, density)
    o = pisa_fwd_given(q, k, v, kc, vc, h, indices, block_size, scale, acc=acc)
    return o, indices


def pisa_bwd(q, k, v, do, indices, block_size: int = 64, scale: Optional[float] = None,
             acc=torch.float64):
    """Gradients of the forward restatement by autograd with ``indices`` held
    constant (gradients flow through the block statistics kc, vc, h as well).
    No reference counterpart: parity unpinned."""
    K = k.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    q_, k_, v_ = (x.detach().to(acc).requires_grad_() for x in (q, k, v))
    T = k_.shape[-2]
    nt = (T + block_size - 1) // block_size
    kc, vc = [], []
    h = 0
    for c in range(nt):
        lo, hi = c * block_size, min(T, (c + 1) * block_size)
        kb, vb = k_[..., lo:hi, :], v_[..., lo:hi, :]
        kcm = kb.mean(dim=-2)
        kc.append(kcm)
        vc.append(vb.sum(dim=-2))
        h = h + (kb - kcm[..., None, :]).transpose(-2, -1) @ vb
    o = pisa_fwd_given(q_, k_, v_, torch.stack(kc, -2), torch.stack(vc, -2), h, indices,
                       block_size, scale, acc=acc, differentiable=True)
    o.backward(do.detach().to(acc))
    return q_.grad, k_.grad, v_.grad


# ---------------------------------------------------------------------------
# Metrics used by the parity tests.
# ---------------------------------------------------------------------------

def max_abs_over_rms(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max|got-ref| / rms(ref): the bf16 acceptance metric (<= 2e-2)."""
    ref64 = ref.detach().double()
    rms = ref64.square().mean().sqrt().item()
    return (got.detach().double() - ref64).abs().max().item() / (rms + 1e-30)


def rel_l2(got: torch.Tensor, ref: torch.Tensor) -> float:
    """||got-ref||_2 / ||ref||_2: the fp32 acceptance metric (<= 1e-5);
    the same ratio as flash_bla/utils.py:49-52."""
    ref64 = ref.detach().double()
    return ((got.detach().double() - ref64).norm() / (ref64.norm() + 1e-30)).item()


# ---------------------------------------------------------------------------
# The reference's CPU execution model, for timing: the dense torch forward in
# the tensors' own dtype and torch autograd for the backward, exactly how
# benchmarks/ops/benchmark_linear_attn.py:49-58 drives naive_linear_attn.
# ---------------------------------------------------------------------------

def linear_attn_torch_fwd_bwd(q, k, v, do, scale: Optional[float] = None, eps: float = 1e-6):
    """One forward + autograd backward of the dense torch statement
    (flash_bla/ops/linear_attn/naive.py:6-14) in the dtype of the inputs.
    Returns (o, dq, dk, dv)."""
    q_, k_, v_ = (x.detach().clone().requires_grad_() for x in (q, k, v))
    if scale is None:
        scale = 1.0 / k_.shape[-2]
    z = q_ @ k_.mean(dim=-2, keepdim=True).transpose(-2, -1)
    s = k_.transpose(-2, -1) @ (v_ * scale)
    o = q_ @ s / (z + eps)
    o.backward(do)
    return o.detach(), q_.grad, k_.grad, v_.grad
