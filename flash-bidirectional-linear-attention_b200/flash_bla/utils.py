"""Helpers shared by the operators; same names as the reference's
``flash_bla/utils.py`` (``contiguous`` :9-15, ``get_abs_err`` :45-46,
``get_err_ratio`` :49-52, ``assert_close`` :55-67)."""
import functools
import os
import warnings

import torch


def _as_contiguous(x):
    return x.contiguous() if isinstance(x, torch.Tensor) else x


def contiguous(fn):
    """Decorator for ``autograd.Function`` methods: every tensor argument is made
    contiguous before the call."""
    @functools.wraps(fn)
    def wrapper(ctx, *args, **kwargs):
        return fn(ctx, *map(_as_contiguous, args), **{n: _as_contiguous(a) for n, a in kwargs.items()})
    return wrapper


def checkpoint(func):
    def wrapper(*args, **kwargs):
        return torch.utils.checkpoint.checkpoint(func, *args, **kwargs)
    return wrapper


autocast_custom_fwd = functools.partial(torch.amp.custom_fwd, device_type="cuda")
autocast_custom_bwd = functools.partial(torch.amp.custom_bwd, device_type="cuda")


def get_abs_err(x, y):
    return (x.detach() - y.detach()).abs().max().item()


def get_err_ratio(x, y):
    """RMS of the difference over RMS of ``x``."""
    diff_rms = (x.detach() - y.detach()).float().pow(2).mean().sqrt().item()
    base_rms = x.detach().float().pow(2).mean().sqrt().item()
    return diff_rms / (base_rms + 1e-8)


def assert_close(prefix, ref, tri, ratio, warning=False, err_atol=1e-6):
    abs_err = get_abs_err(ref, tri)
    if abs_err <= err_atol:
        return abs_err
    err_ratio = get_err_ratio(ref, tri)
    msg = f"{prefix:>8} diff: {abs_err:.6f} ratio: {err_ratio:.6f}"
    if os.environ.get("FLASH_BLA_PRINT_ERR") == "1":     # lets a harness read the measured error
        print(msg, flush=True)
    if warning or err_ratio < 0.01 or abs_err <= 0.3:
        if err_ratio > ratio:
            warnings.warn(msg)
        return err_ratio
    assert err_ratio < ratio, msg
    return err_ratio
