"""Dense torch statement of ``simple_la`` (any device); same name and signature as
the reference's ``flash_bla/ops/simple_la/naive.py:8-20``."""
import torch


def naive_simple_la(q, k, v, scale=None):
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return torch.matmul(q, torch.matmul(k.transpose(-1, -2), v * scale))
