"""ctypes binding of libflash_bla_sm100.so (the C ABI in include/flash_bla_sm100.h).

There is no fallback: if the shared library has not been built, or a call fails,
an exception is raised.
"""
import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FLASH_BLA_LIB") or os.path.join(_HERE, "lib", "libflash_bla_sm100.so")

F32, BF16, F16 = 0, 1, 2
FLAG_GENERIC = 1
FLAG_UNREDUCED = 2
FLAG_NARROW = 4

_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


class Problem(ctypes.Structure):
    """Mirror of ``struct fbla_problem``."""
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("dk", ctypes.c_int32),
        ("dv", ctypes.c_int32),
        ("seq_len", ctypes.c_int64),
        ("norm_len", ctypes.c_int64),
        ("cu_seqlens", ctypes.c_void_p),
        ("num_seqs", ctypes.c_int32),
        ("max_seqlen", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("scale_per_seq", ctypes.c_int32),
        ("eps", ctypes.c_float),
        ("normalize", ctypes.c_int32),
        ("flags", ctypes.c_int32),
    ]


class PisaProblem(ctypes.Structure):
    """Mirror of ``struct fbla_pisa_problem``."""
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("dk", ctypes.c_int32),
        ("dv", ctypes.c_int32),
        ("block_size", ctypes.c_int32),
        ("num_selected", ctypes.c_int32),
        ("seq_len", ctypes.c_int64),
        ("scale", ctypes.c_float),
    ]


class PeerGroup(ctypes.Structure):
    """Mirror of ``struct fbla_peer_group``."""
    _fields_ = [
        ("world", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("epoch", ctypes.c_uint32),
        ("reserved", ctypes.c_int32),
        ("parts", ctypes.POINTER(ctypes.c_void_p)),
        ("full", ctypes.POINTER(ctypes.c_void_p)),
        ("flags", ctypes.POINTER(ctypes.c_void_p)),
    ]


_P = ctypes.POINTER(Problem)
_vp = ctypes.c_void_p
_sz = ctypes.c_size_t

# name -> argument types after the leading ``const fbla_problem*``
_SIGNATURES = {
    "fwd_state": [_vp, _vp, _vp, _vp, _sz, _vp],                 # k, v, state, ws, ws_bytes, stream
    "fwd_out": [_vp, _vp, _vp, _vp],                             # q, state, o, stream
    "bwd_state": [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp],       # q, d_o, state, dq, dstate, ws, n, stream
    "bwd_in": [_vp, _vp, _vp, _vp, _vp, _vp],                    # k, v, dstate, dk, dv, stream
}
_DECOUPLED_SIGNATURES = {
    "fwd_state": [_vp, _vp, _vp, _vp, _vp, _sz, _vp],            # k, k_rope, v, state, ws, n, stream
    "fwd_out": [_vp, _vp, _vp, _vp, _vp],                        # q, q_rope, state, o, stream
    "bwd_state": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp],
    "bwd_in": [_vp, _vp, _vp, _vp, _vp, _vp, _vp],               # k_rope, v, dstate, dk, dk_rope, dv, stream
}
OPS = ("linear_attn", "simple_la", "decoupled_la", "varlen_linear_attn")

_lib = None
_lock = threading.Lock()


def exported_symbols():
    """Every symbol include/flash_bla_sm100.h declares."""
    names = ["fbla_version", "fbla_last_error", "fbla_launch_count", "fbla_state_floats",
             "fbla_workspace_bytes", "fbla_kernel_path"]
    for op in OPS:
        names += [f"fbla_{op}_{p}" for p in ("fwd_state", "fwd_out", "bwd_state", "bwd_in")]
    names += ["fbla_linear_attn_fwd", "fbla_linear_attn_bwd"]
    names += ["fbla_linear_attn_fwd_state_noalloc", "fbla_noalloc_status"]
    names += ["fbla_pisa_block_stats", "fbla_pisa_block_hnorm", "fbla_pisa_first_order_state", "fbla_pisa_select_blocks", "fbla_pisa_fwd", "fbla_pisa_fwd_ws", "fbla_pisa_fwd_scratch_bytes", "fbla_pisa_bwd",
              "fbla_pisa_bwd_scratch_floats"]
    names += ["fbla_peer_state_sum", "fbla_seq_sharded_supported", "fbla_seq_sharded_part_floats",
              "fbla_seq_sharded_fwd_state", "fbla_seq_sharded_bwd_state", "fbla_seq_sharded_exchange",
              "fbla_device_status", "fbla_clear_device_status", "fbla_unreduced_state"]
    return names


def lib():
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python build.py` in the package root "
                "(flash_bla has no CPU or Triton fallback)")
        L = ctypes.CDLL(LIB_PATH)
        L.fbla_version.restype = ctypes.c_int
        L.fbla_last_error.restype = ctypes.c_char_p
        L.fbla_launch_count.restype = ctypes.c_uint64
        for n in ("fbla_state_floats", "fbla_workspace_bytes"):
            getattr(L, n).restype = ctypes.c_int64
            getattr(L, n).argtypes = [_P]
        L.fbla_kernel_path.restype = ctypes.c_int
        L.fbla_kernel_path.argtypes = [_P]
        L.fbla_unreduced_state.restype = ctypes.c_int
        L.fbla_unreduced_state.argtypes = [_P]
        for op in OPS:
            sigs = _DECOUPLED_SIGNATURES if op == "decoupled_la" else _SIGNATURES
            for name, args in sigs.items():
                f = getattr(L, f"fbla_{op}_{name}")
                f.restype = ctypes.c_int
                f.argtypes = [_P] + args
        L.fbla_linear_attn_fwd.restype = ctypes.c_int
        L.fbla_linear_attn_fwd.argtypes = [_P, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]
        L.fbla_linear_attn_bwd.restype = ctypes.c_int
        L.fbla_linear_attn_bwd.argtypes = [_P] + [_vp] * 10 + [_sz, _vp]
        L.fbla_linear_attn_fwd_state_noalloc.restype = ctypes.c_int
        L.fbla_linear_attn_fwd_state_noalloc.argtypes = [_P, _vp, _vp, _vp, _vp]   # k, v, state, stream
        L.fbla_noalloc_status.restype = ctypes.c_int
        L.fbla_noalloc_status.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_int]
        _PP = ctypes.POINTER(PisaProblem)
        for name, n_ptr in (("fbla_pisa_block_stats", 7), ("fbla_pisa_first_order_state", 5), ("fbla_pisa_fwd", 10)):
            f = getattr(L, name)
            f.restype = ctypes.c_int
            f.argtypes = [_PP] + [_vp] * n_ptr          # tensor pointers, then the stream
        L.fbla_pisa_fwd_scratch_bytes.restype = ctypes.c_int64
        L.fbla_pisa_fwd_scratch_bytes.argtypes = [_PP]
        L.fbla_pisa_fwd_ws.restype = ctypes.c_int
        L.fbla_pisa_fwd_ws.argtypes = [_PP] + [_vp] * 10 + [_sz, _vp]      # 9 tensors, scratch, its size, stream
        _PG = ctypes.POINTER(PeerGroup)
        L.fbla_seq_sharded_supported.restype = ctypes.c_int
        L.fbla_seq_sharded_supported.argtypes = [_P]
        L.fbla_seq_sharded_part_floats.restype = ctypes.c_int64
        L.fbla_seq_sharded_part_floats.argtypes = [_P]
        for name, args in (("fwd_state", [_vp, _vp, _vp, _PG, _vp]),                 # k, k_rope, v, group, stream
                           ("bwd_state", [_vp, _vp, _vp, _vp, _PG, _vp, _vp, _vp]),  # q, q_rope, d_o, state, group, dq, dq_rope, stream
                           ("exchange", [_PG, _vp, _vp])):                           # group, state_out, stream
            f = getattr(L, "fbla_seq_sharded_" + name)
            f.restype = ctypes.c_int
            f.argtypes = [_P] + args
        L.fbla_device_status.restype = ctypes.c_int
        L.fbla_device_status.argtypes = []
        L.fbla_clear_device_status.restype = None
        L.fbla_clear_device_status.argtypes = []
        L.fbla_pisa_block_hnorm.restype = ctypes.c_int
        L.fbla_pisa_block_hnorm.argtypes = [_PP, _vp, _vp, _vp, ctypes.c_float, _vp, _vp]   # k, v, kc, p, hnorm, stream
        L.fbla_peer_state_sum.restype = ctypes.c_int
        L.fbla_peer_state_sum.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                          ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64, ctypes.c_uint32, _vp, _vp]
        L.fbla_pisa_select_blocks.restype = ctypes.c_int
        L.fbla_pisa_select_blocks.argtypes = [_PP, _vp, _vp, _vp, _vp, _vp]      # qc, kc, hnorm, indices, stream
        L.fbla_pisa_bwd_scratch_floats.restype = ctypes.c_int64
        L.fbla_pisa_bwd_scratch_floats.argtypes = [_PP]
        L.fbla_pisa_bwd.restype = ctypes.c_int
        L.fbla_pisa_bwd.argtypes = [_PP] + [_vp] * 14 + [_sz, _vp]   # 14 tensors, scratch size, stream
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        raise RuntimeError(f"flash_bla_sm100 error {rc}: {lib().fbla_last_error().decode()}")


def dtype_code(dtype):
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"dtype {dtype} is not supported (float16, bfloat16, float32)") from None


def ptr(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_of(t):
    """cudaStream_t (as an int) of torch's current stream on the tensor's device."""
    if _raw_stream is not None:
        return _raw_stream(t.device.index)
    return torch.cuda.current_stream(t.device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_no_guard = _NoGuard()


def device_guard(t):
    """Context that makes the tensor's device current; free when it already is."""
    if t.device.index == torch.cuda.current_device():
        return _no_guard
    return torch.cuda.device_of(t)
