"""Dense torch statements of the linear-attention operators (any device).  Same
names and signatures as the reference's ``flash_bla/ops/linear_attn/naive.py``
(:6-14, :17-26, :29-43); handy as a readable specification and for user-side checks.
The CUDA operators never call these."""
import torch


def _default_scale(k, scale):
    return 1.0 / k.shape[-2] if scale is None else scale


def naive_linear_attn(q, k, v, scale=None):
    kv = torch.matmul(k.transpose(-1, -2), v * _default_scale(k, scale))
    norm = torch.matmul(q, k.mean(dim=-2).unsqueeze(-1))
    return torch.matmul(q, kv) / (norm + 1e-6)


def naive_decoupled_la(q, k, q_rope, k_rope, v, scale=None):
    kv = torch.matmul(k_rope.transpose(-1, -2), v * _default_scale(k, scale))
    norm = torch.matmul(q, k.mean(dim=-2).unsqueeze(-1))
    return torch.matmul(q_rope, kv) / (norm + 1e-6)


def naive_varlen_linear_attn(q, k, v, cu_seqlens, scale=None, eps=1e-6):
    bounds = cu_seqlens.tolist()
    out = q.new_empty(q.shape[0], q.shape[1], v.shape[-1])
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        qs, ks, vs = (x[lo:hi].permute(1, 0, 2) for x in (q, k, v))      # (H, len, D)
        sc = 1.0 / (hi - lo) if scale is None else scale
        kv = torch.matmul(ks.transpose(-1, -2), vs * sc)
        norm = torch.matmul(qs, ks.mean(dim=1).unsqueeze(-1))
        out[lo:hi] = (torch.matmul(qs, kv) / (norm + eps)).permute(1, 0, 2)
    return out
