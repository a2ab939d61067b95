"""Generate the golden fixtures in this directory from the reference itself.

Run once, in a container that holds the reference checkout:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference [fixture names]

For the four linear-attention operators the expected values come from the
reference's own dense torch path (``flash_bla/ops/linear_attn/naive.py``,
``flash_bla/ops/simple_la/naive.py``) on CPU tensors, gradients from torch
autograd.  For the piecewise operator the reference has no torch path, so the
expected values come from the reference's Triton kernels
(``flash_bla/ops/piecewise_attn/kernel.py``) executed by Triton's CPU
interpreter with explicit meta-parameters (the autotuner needs a GPU driver).

The files hold the seeded inputs and the expected outputs both, so the tests
never need the reference at run time.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


ONLY = set()      # fixture names given on the command line (empty: all)


def _save(name, _compressed=False, **arrays):
    if ONLY and name not in ONLY:
        return
    (np.savez_compressed if _compressed else np.savez)(os.path.join(HERE, name + ".npz"), **arrays)
    print("wrote", name)


def _np(x):
    return x.detach().to(torch.float32).numpy()


def _inputs(seed, shape_qk, shape_v, positive=True, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(shape_qk, generator=g)
    k = torch.randn(shape_qk, generator=g)
    v = torch.randn(shape_v, generator=g)
    do = torch.randn(shape_v, generator=g)
    if positive:
        q, k = F.elu(q) + 1, F.elu(k) + 1
    return [x.to(dtype) for x in (q, k, v, do)]


def main(ref_root):
    sys.path.insert(0, ref_root)
    from flash_bla.ops.linear_attn.naive import (naive_linear_attn, naive_decoupled_la,
                                                 naive_varlen_linear_attn)
    from flash_bla.ops.simple_la.naive import naive_simple_la

    # ---- linear_attn: default scale and explicit scale, DK != DV -------------
    for name, (B, H, T, DK, DV), scale in [
        ("linear_attn_a", (2, 3, 80, 16, 16), None),
        ("linear_attn_b", (1, 2, 131, 32, 24), 0.05),
        ("linear_attn_c", (1, 1, 160, 64, 64), None),
    ]:
        q, k, v, do = _inputs(1, (B, H, T, DK), (B, H, T, DV))
        q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
        o = naive_linear_attn(q, k, v, scale)
        o.backward(do)
        _save(name, q=_np(q), k=_np(k), v=_np(v), do=_np(do),
                 o=_np(o), dq=_np(q.grad), dk=_np(k.grad), dv=_np(v.grad),
                 scale=np.float64(-1.0 if scale is None else scale), eps=np.float64(1e-6))

    # ---- decoupled_la --------------------------------------------------------
    for name, (B, H, T, DK, DV), scale in [
        ("decoupled_a", (2, 2, 96, 16, 16), None),
        ("decoupled_b", (1, 1, 150, 64, 32), 0.01),
    ]:
        q, k, v, do = _inputs(2, (B, H, T, DK), (B, H, T, DV))
        g = torch.Generator().manual_seed(22)
        qr = torch.randn(B, H, T, DK, generator=g)
        kr = torch.randn(B, H, T, DK, generator=g)
        for x in (q, k, qr, kr, v):
            x.requires_grad_()
        o = naive_decoupled_la(q, k, qr, kr, v, scale)
        o.backward(do)
        _save(name, q=_np(q), k=_np(k), q_rope=_np(qr),
                 k_rope=_np(kr), v=_np(v), do=_np(do), o=_np(o), dq=_np(q.grad), dk=_np(k.grad),
                 dq_rope=_np(qr.grad), dk_rope=_np(kr.grad), dv=_np(v.grad),
                 scale=np.float64(-1.0 if scale is None else scale), eps=np.float64(1e-6))

    # ---- simple_la -----------------------------------------------------------
    for name, (B, H, T, DK, DV), scale in [
        ("simple_la_a", (1, 2, 100, 32, 32), None),
        ("simple_la_b", (1, 1, 72, 128, 128), 0.25),
    ]:
        q, k, v, do = _inputs(3, (B, H, T, DK), (B, H, T, DV), positive=False)
        q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
        o = naive_simple_la(q, k, v, scale)
        o.backward(do)
        _save(name, q=_np(q), k=_np(k), v=_np(v), do=_np(do),
                 o=_np(o), dq=_np(q.grad), dk=_np(k.grad), dv=_np(v.grad),
                 scale=np.float64(-1.0 if scale is None else scale))

    # ---- varlen: the reference test's lengths [8, 17, 32], its odd dims ------
    for name, lengths, (H, DK, DV), scale in [
        ("varlen_a", [8, 17, 32], (2, 17, 13), None),
        ("varlen_b", [8, 17, 32], (1, 64, 48), 0.02),
        ("varlen_c", [130, 1, 77], (2, 32, 32), None),
    ]:
        tot = sum(lengths)
        q, k, v, do = _inputs(42, (tot, H, DK), (tot, H, DV))
        cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32)
        q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
        o = naive_varlen_linear_attn(q, k, v, cu, scale=scale)
        o.backward(do)
        _save(name, q=_np(q), k=_np(k), v=_np(v), do=_np(do),
                 cu_seqlens=cu.numpy(), o=_np(o), dq=_np(q.grad), dk=_np(k.grad),
                 dv=_np(v.grad), scale=np.float64(-1.0 if scale is None else scale),
                 eps=np.float64(1e-6))

    # ---- piecewise_sparse_attention: reference Triton kernels, interpreted ---
    import triton
    from flash_bla.ops.piecewise_attn import kernel as pk

    def alloc_fn(size, alignment, stream):
        return torch.empty(size, dtype=torch.int8)
    triton.set_allocator(alloc_fn)

    for name, (B, H, T, K, V), bs, density in [
        ("pisa_a", (1, 2, 160, 16, 16), 16, 0.3),     # T multiple of the block
        ("pisa_b", (1, 1, 150, 32, 32), 32, 0.25),    # ragged last block
        ("pisa_c", (1, 2, 200, 16, 32), 32, 0.3),     # use_bias=True (selection biased by the block norms of hc)
    ]:
        use_bias = name == "pisa_c"
        g = torch.Generator().manual_seed(5)
        q = torch.randn(B, H, T, K, generator=g)
        k = torch.randn(B, H, T, K, generator=g)
        v = torch.randn(B, H, T, V, generator=g)
        scale = K ** -0.5
        NT = triton.cdiv(T, bs)
        qc = torch.empty(B, H, NT, K)
        kc = torch.empty(B, H, NT, K)
        vc = torch.empty(B, H, NT, V)
        hc = torch.empty(B, H, NT, K, V)
        pk.fused_chunk_reduce_kernel.fn[(1, NT, B * H)](
            q, k, v, qc, kc, vc, hc, T, N=NT, K=K, V=V, BT=bs, BK=K, BV=V)
        h = hc.sum(dim=2)
        score = torch.einsum('bhid,bhjd->bhij', qc, kc * scale)
        extra = {}
        if use_bias:       # kernel.py:172-173 and :314-315
            h_norm = torch.norm(hc.flatten(-2, -1), p=2, dim=-1)
            score = torch.softmax(score + torch.log(h_norm[..., None, :] + 1e-5), dim=-1)
            extra = dict(h_norm=_np(h_norm), score=_np(score))
        top_k = max(1, int(density * NT))
        indices = torch.topk(score, k=top_k, dim=-1).indices
        o = torch.empty_like(v)
        pk.piecewise_sparse_attention_fwd_kernel.fn[(1, NT, B * H)](
            q, k, v, kc, vc, h, o, indices, scale, T, K=K, V=V, BT=bs, BK=K, BV=V,
            NT=NT, NS=top_k, GROUP_SIZE=32)
        _save(name, q=_np(q), k=_np(k), v=_np(v), qc=_np(qc),
                 kc=_np(kc), vc=_np(vc), h=_np(h), indices=indices.numpy(), o=_np(o),
                 block_size=np.int64(bs), density=np.float64(density), scale=np.float64(scale), **extra)
    # ---- more blocks than one GROUP_SIZE: the kernel's result depends on its evaluation order ----
    # pisa_e: NT = 40 > GROUP_SIZE = 32 (two groups; the running maximum may grow between them)
    # pisa_d: one (batch, head) pair of the DiT-layer configuration (T = 4608 = 72 blocks of 64,
    #         D = 128, 7 selected blocks) with GROUP_SIZE = 128, i.e. one group.  Inputs are
    #         bf16-representable and stored as bf16 bit patterns; of the output only eight query
    #         blocks are kept (the first two, the last two, four in between).
    def bf16_bits(x):
        return (x.bfloat16().view(torch.int16).numpy().astype(np.uint16))

    for name, (B, H, T, K, V), bs, density, group in [
        ("pisa_e", (1, 2, 640, 16, 16), 16, 0.1, 32),
        ("pisa_d", (1, 1, 4608, 128, 128), 64, 0.1, 128),
    ]:
        g = torch.Generator().manual_seed(17)
        q = torch.randn(B, H, T, K, generator=g).bfloat16().float()
        k = torch.randn(B, H, T, K, generator=g).bfloat16().float()
        v = torch.randn(B, H, T, V, generator=g).bfloat16().float()
        if name == "pisa_e":
            # make later blocks score higher, so that the running maximum grows in the second group
            ramp = torch.linspace(0.0, 3.0, T)[None, None, :, None]
            k = (k + ramp * q.mean(dim=-2, keepdim=True).sign()).bfloat16().float()
            q = (q * 2).bfloat16().float()
        scale = K ** -0.5
        NT = triton.cdiv(T, bs)
        qc = torch.empty(B, H, NT, K)
        kc = torch.empty(B, H, NT, K)
        vc = torch.empty(B, H, NT, V)
        hc = torch.empty(B, H, NT, K, V)
        pk.fused_chunk_reduce_kernel.fn[(1, NT, B * H)](
            q, k, v, qc, kc, vc, hc, T, N=NT, K=K, V=V, BT=bs, BK=K, BV=V)
        h = hc.sum(dim=2)
        score = torch.einsum('bhid,bhjd->bhij', qc, kc * scale)
        top_k = max(1, int(density * NT))
        indices = torch.topk(score, k=top_k, dim=-1).indices
        o = torch.empty_like(v)
        pk.piecewise_sparse_attention_fwd_kernel.fn[(1, NT, B * H)](
            q, k, v, kc, vc, h, o, indices, scale, T, K=K, V=V, BT=bs, BK=K, BV=V,
            NT=NT, NS=top_k, GROUP_SIZE=group)
        if name == "pisa_d":
            keep = [0, 1, 17, 35, 36, 53, 70, 71]
            rows = np.concatenate([np.arange(b * bs, (b + 1) * bs) for b in keep])
            _save(name, _compressed=True, q_bf16=bf16_bits(q), k_bf16=bf16_bits(k),
                                v_bf16=bf16_bits(v), kc=_np(kc), vc=_np(vc), h=_np(h), indices=indices.numpy(),
                                o_rows=rows, o=_np(o[:, :, rows]), block_size=np.int64(bs),
                                density=np.float64(density), scale=np.float64(scale), group_size=np.int64(group))
        else:
            _save(name, q=_np(q), k=_np(k), v=_np(v), qc=_np(qc),
                     kc=_np(kc), vc=_np(vc), h=_np(h), indices=indices.numpy(), o=_np(o),
                     block_size=np.int64(bs), density=np.float64(density), scale=np.float64(scale),
                     group_size=np.int64(group))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: TRITON_INTERPRET=1 python make_golden.py <path to a checkout of the reference> [fixture ...]")
    ONLY.update(sys.argv[2:])
    main(sys.argv[1])
