"""ctypes binding of libhils_b200.so (the C ABI declared in include/hils_b200.h).

The library is built in-tree by ``python -m hils_attention_b200.build``; there is no CPU or
PyTorch fallback: if the shared library is missing, or a call is made without a CUDA device,
an error is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhils_b200.so")

F32, BF16 = 0, 1
_P, _I, _F, _I64, _SZ = C.c_void_p, C.c_int, C.c_float, C.c_int64, C.c_size_t

# name -> (restype, argtypes); mirrors include/hils_b200.h one to one
SIGNATURES = {
    "hils_version": (_I, []),
    "hils_last_error": (C.c_char_p, []),
    "hils_take_device_status": (_I, []),
    "hils_pool_fwd": (_I, [_P] * 4 + [_I] * 6 + [_I64, _F, _I, _I, _P]),
    "hils_pool_bwd": (_I, [_P] * 6 + [_I] * 6 + [_I64, _F, _I, _I, _P]),
    "hils_meanpool_fwd": (_I, [_P, _P] + [_I] * 5 + [_I64, _I, _P]),
    "hils_meanpool_bwd": (_I, [_P, _P] + [_I] * 6 + [_P]),
    "hils_topk_fwd": (_I, [_P] * 10 + [_I] * 12 + [_F, _I, _I, _P, _SZ, _P]),
    "hils_topk_fwd_workspace_bytes": (_SZ, [_I] * 7),
    "hils_topk_bwd": (_I, [_P] * 7 + [_I] * 8 + [_F, _I, _P]),
    "hils_topk_bwd_noalloc": (_I, [_P] * 6 + [_I] * 8 + [_F, _I, _P]),
    "hils_topk_bwd_noalloc_max_elems": (_SZ, []),
    "hils_sparse_attn_fwd": (_I, [_P] * 7 + [_I] * 10 + [_F, _I, _I, _P, _SZ, _P]),
    "hils_sparse_attn_fwd_workspace_bytes": (_SZ, [_I] * 10),
    "hils_sparse_attn_bwd": (_I, [_P] * 11 + [_I] * 10 + [_F, _I, _I, _P, _SZ, _P]),
    "hils_sparse_attn_bwd_workspace_bytes": (_SZ, [_I] * 10),
    "hils_sparse_attn_index_bytes": (_SZ, [_I] * 10),
    "hils_sparse_attn_bwd_with_index": (_I, [_P] * 11 + [_I] * 10 + [_F, _I, _I, _P, _SZ, _P, _SZ, _P]),
    "hils_chunk_logz_fwd": (_I, [_P] * 3 + [_I] * 7 + [_F, _I, _I, _P]),
    "hils_chunk_logz_bwd": (_I, [_P] * 6 + [_I] * 7 + [_F, _I, _P]),
    "hils_swa_fwd": (_I, [_P] * 5 + [_I] * 11 + [_F, _I, _I, _P]),
    "hils_swa_bwd": (_I, [_P] * 10 + [_I] * 10 + [_F, _I, _P, _SZ, _P]),
    "hils_swa_bwd_workspace_bytes": (_SZ, [_I] * 8),
    "hils_chunk_weights_fwd": (_I, [_P] * 5 + [_I] * 8 + [_P]),
    "hils_chunk_weights_bwd": (_I, [_P] * 6 + [_I] * 8 + [_P]),
    "hils_combine_fwd": (_I, [_P] * 4 + [_I] * 7 + [_P]),
    "hils_combine_bwd": (_I, [_P] * 5 + [_I] * 7 + [_P]),
    "hils_decode_step": (_I, [_P] * 6 + [_I] + [_P] * 2 + [_I] + [_P] * 2 + [_I] * 8 + [_F, _I, _P, _SZ, _P]),
    "hils_decode_step_workspace_bytes": (_SZ, [_I] * 8),
    "hils_decode_step_paged": (_I, [_P] * 7 + [_I] * 2 + [_P, _I] + [_P] * 2 + [_I] + [_P] * 2 + [_I] * 9 + [_F, _I, _P, _SZ, _P]),
    "hils_decode_step_paged_workspace_bytes": (_SZ, [_I] * 9),
    "hils_norm_rope_fwd": (_I, [_P] * 6 + [_I] * 5 + [_F, _I, _I, _P]),
    "hils_norm_rope_bwd": (_I, [_P] * 8 + [_I] * 7 + [_P]),
}

# kernels each entry point launches (memsets excluded); used to report launch counts
KERNELS_PER_CALL = {
    "hils_pool_fwd": 1, "hils_pool_bwd": 1, "hils_meanpool_fwd": 1, "hils_meanpool_bwd": 1,
    "hils_topk_fwd": 1, "hils_topk_bwd": 2, "hils_topk_bwd_noalloc": 2, "hils_sparse_attn_fwd": 6, "hils_sparse_attn_bwd": 6, "hils_sparse_attn_bwd_with_index": 6,
    "hils_chunk_logz_fwd": 1, "hils_chunk_logz_bwd": 2, "hils_swa_fwd": 1, "hils_swa_bwd": 2,
    "hils_chunk_weights_fwd": 1, "hils_chunk_weights_bwd": 1, "hils_combine_fwd": 1, "hils_combine_bwd": 1,
    "hils_norm_rope_fwd": 1, "hils_norm_rope_bwd": 1,
    "hils_decode_step_paged": 5,   # append, then as below
    "hils_decode_step": 4,   # window, key stream, selection + inter-chunk softmax, sparse + combine (the 2 copies not counted)
}
_launches = 0
# HILS_B200_CHECK_STATUS=1: read the device status word after every call (synchronises; for debugging)
_CHECK_STATUS = os.environ.get("HILS_B200_CHECK_STATUS", "0") not in ("", "0")

_lib: Optional[C.CDLL] = None


class HilsError(RuntimeError):
    """Raised when a C-ABI call returns a non-zero status."""


def load() -> C.CDLL:
    """Load the shared library (once) and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m hils_attention_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the .so lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float32:
        return F32
    raise TypeError(f"hils_b200 kernels take bfloat16 or float32 tensors, got {t.dtype}")


# Devices of the tensors whose pointers were taken for the call being assembled (per host thread: the
# autograd engine runs backward functions on its own threads).  ptr() records, stream() and call() check.
_tls = threading.local()


def _pending() -> list:
    devs = getattr(_tls, "devs", None)
    if devs is None:
        devs = _tls.devs = []
    return devs


def _call_device() -> Optional[torch.device]:
    """The one device all tensors of the pending call live on; raises if they disagree."""
    devs = _pending()
    if not devs:
        return None
    first = devs[0]
    for d in devs[1:]:
        if d != first:
            devs.clear()
            raise RuntimeError(f"hils_b200: tensors of one call live on different devices ({first} and {d}); "
                               "nothing was launched")
    return first


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        _pending().clear()
        raise RuntimeError("hils_b200 kernels need CUDA tensors (no CPU fallback exists)")
    # The kernels read rows with 8- and 16-byte vector loads and through TMA descriptors: a tensor that starts inside
    # a 16-byte word (an odd slice of a larger buffer) would fault on the device, so it is refused here.
    if t.data_ptr() % 16 != 0 and t.numel() * t.element_size() >= 16:
        _pending().clear()
        raise ValueError(f"hils_b200: tensor of shape {tuple(t.shape)} starts at an address that is not 16-byte aligned "
                         "(a view into the middle of a buffer?); copy it with .clone() first. Nothing was launched")
    _pending().append(t.device)
    return t.data_ptr()


def stream() -> int:
    """Current torch stream of the device the pending call's tensors live on (the kernels follow their
    tensors, like the reference's ops, not the process-wide current device)."""
    dev = _call_device()
    return torch.cuda.current_stream(dev).cuda_stream


def call(name: str, *args):
    """Invoke a status-returning entry point and raise HilsError on failure.  The call runs with the
    tensors' device current (tensor maps, symbol addresses and launches bind to the current context)."""
    global _launches
    lib = load()
    dev = _call_device()
    _pending().clear()
    if dev is not None and torch.cuda.current_device() != dev.index:
        with torch.cuda.device(dev):
            rc = getattr(lib, name)(*args)
    else:
        rc = getattr(lib, name)(*args)
    _launches += KERNELS_PER_CALL.get(name, 1)
    if rc != 0:
        msg = lib.hils_last_error().decode("utf-8", "replace")
        raise HilsError(f"{name} failed with status {rc}: {msg}")
    if _CHECK_STATUS:
        st = int(lib.hils_take_device_status())
        if st != 0:
            raise HilsError(f"{name}: a bounded device-side wait expired (status {st}); the output is incomplete")


def query(name: str, *args) -> int:
    return int(getattr(load(), name)(*args))


def launch_count() -> int:
    """Kernels of this library launched so far by this process."""
    return _launches
