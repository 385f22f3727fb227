"""ctypes binding of libmhc_b200.so, the C-ABI library of sm_100a kernels.

There is no fallback: if the shared object is missing or a tensor is not on a CUDA
device, the call raises.  Build the library with ``python mhc-triton_b200/build.py``.
"""

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# MHC_B200_LIB overrides the location of the shared object (e.g. a build with other tuning macros).
LIB_PATH = os.environ.get("MHC_B200_LIB") or os.path.join(_HERE, "libmhc_b200.so")

MHC_F32, MHC_BF16, MHC_F16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: MHC_F32, torch.bfloat16: MHC_BF16, torch.float16: MHC_F16}

(OP_ADD_RESIDUAL_BWD, OP_STREAM_MIX_BWD, OP_MEANPOOL_FWD, OP_DYNAMIC_WEIGHTS_FWD, OP_DYNAMIC_WEIGHTS_BWD,
 OP_HC_MIX_FWD, OP_HC_MIX_BWD) = range(7)

ABS0_ZERO, ABS0_PLUS_ONE = 0, 1

_P, _I, _L, _F = c_void_p, c_int, c_int64, c_float

# name -> argument types (every function returns int except where noted below)
_PROTOTYPES = {
    "mhc_sinkhorn_fwd": [_P, _P, _L, _I, _I, _F, _P],
    "mhc_sinkhorn_bwd": [_P, _P, _P, _L, _I, _I, _F, _I, _P],
    "mhc_stream_mix_fwd": [_P, _P, _P, _P, _P, _L, _L, _L, _I, _P],
    "mhc_stream_mix_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _P],
    "mhc_stream_mix_bwd_reduce": [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _P],
    "mhc_stream_mix_bwd_apply": [_P, _P, _P, _P, _P, _F, _P, _L, _L, _L, _I, _P],
    "mhc_add_residual_fwd": [_P, _P, _P, _P, _L, _L, _L, _I, _P],
    "mhc_add_residual_bwd": [_P, _P, _P, _P, _P, _P, _L, _P, _L, _L, _L, _I, _P],
    "mhc_meanpool_fwd": [_P, _P, _P, _L, _L, _L, _L, _I, _P],
    "mhc_dynamic_weights_fwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _I, _F, _P],
    "mhc_dynamic_weights_bwd": [_P] * 15 + [_L, _L, _L, _I, _F, _I, _I, _P],
    "mhc_add_residual_bwd_noalloc": [_P, _P, _P, _P, _P, _L, _L, _L, _I, _P],
    "mhc_hc_mix_fwd": [_P] * 16 + [_L, _P, _L, _P, _L, _L, _L, _I, _I, _F, _P],
    "mhc_add_residual_pool_fwd": [_P, _P, _P, _P, _P, _L, _L, _L, _I, _P],
    "mhc_add_residual_mix_fwd": [_P, _P, _P, _P, _P, _P, _L, _L, _L, _I, _P],
    "mhc_hc_mix_bwd": [_P] * 23 + [_L, _P, _P, _L, _L, _L, _I, _I, _F, _I, _I, _P],
}

EXPORTS = sorted(list(_PROTOTYPES) + ["mhc_version", "mhc_last_error_string", "mhc_status_name", "mhc_scratch_bytes",
                                          "mhc_launch_count", "mhc_profile_enable", "mhc_profile_count",
                                          "mhc_profile_get", "mhc_profile_select",
                                          "mhc_add_residual_bwd_noalloc_max_bytes", "mhc_add_residual_pool_chunks"])

_lib = None


class MhcError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def load():
    """Load (once) and return the ctypes handle; raises if the library has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: the mhc CUDA library is not built "
            "(run `python mhc-triton_b200/build.py`); there is no CPU or PyTorch fallback")
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in _PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.mhc_version.argtypes = []
    lib.mhc_version.restype = c_int
    lib.mhc_last_error_string.argtypes = []
    lib.mhc_last_error_string.restype = c_char_p
    lib.mhc_status_name.argtypes = [c_int]
    lib.mhc_status_name.restype = c_char_p
    lib.mhc_profile_enable.argtypes = [c_int]
    lib.mhc_profile_enable.restype = c_int
    lib.mhc_add_residual_bwd_noalloc_max_bytes.argtypes = []
    lib.mhc_add_residual_bwd_noalloc_max_bytes.restype = c_int64
    lib.mhc_add_residual_pool_chunks.argtypes = [c_int64, c_int64]
    lib.mhc_add_residual_pool_chunks.restype = c_int64
    lib.mhc_profile_select.argtypes = [c_char_p]
    lib.mhc_profile_select.restype = c_int
    lib.mhc_profile_count.argtypes = []
    lib.mhc_profile_count.restype = c_int64
    lib.mhc_profile_get.argtypes = [c_int64, ctypes.POINTER(c_char_p), ctypes.POINTER(c_float)]
    lib.mhc_profile_get.restype = c_int
    lib.mhc_launch_count.argtypes = []
    lib.mhc_launch_count.restype = c_int64
    lib.mhc_scratch_bytes.argtypes = [c_int, c_int64, c_int64, c_int64, c_int]
    lib.mhc_scratch_bytes.restype = c_int64
    _lib = lib
    return lib


def call(name, stream, *args):
    """Invoke an entry point (the stream is its last argument) and raise on a non-zero status."""
    return check(getattr(load(), name)(*args, stream))


def profile_start(only=None):
    """Start per-kernel timing inside the library (CUDA events around every kernel launch, or
    around the launches of the kernel named `only`)."""
    check(load().mhc_profile_select(only.encode() if only else None))
    check(load().mhc_profile_enable(1))


def profile_stop():
    """Stop timing and return {kernel name: (launches, total milliseconds)}.  Synchronises the device."""
    lib = load()
    check(lib.mhc_profile_enable(0))
    torch.cuda.synchronize()
    out = {}
    name, ms = c_char_p(), c_float()
    for i in range(lib.mhc_profile_count()):
        check(lib.mhc_profile_get(i, ctypes.byref(name), ctypes.byref(ms)))
        n, t = out.get(name.value.decode(), (0, 0.0))
        out[name.value.decode()] = (n + 1, t + ms.value)
    return out


def check(status):
    if status != 0:
        lib = load()
        raise MhcError(f"{lib.mhc_status_name(status).decode()}: {lib.mhc_last_error_string().decode()}")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise TypeError(f"mhc: unsupported dtype {t.dtype} (float32, bfloat16, float16 only)") from None


def require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("mhc: tensors must live on a CUDA device (this build has no CPU path)")


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor):
    """Raw cudaStream_t of torch's current stream on t's device."""
    return torch._C._cuda_getCurrentRawStream(t.device.index if t.device.index is not None
                                              else torch.cuda.current_device())


def scratch(op, B, S, D, like: torch.Tensor):
    """Caller-owned scratch for `op`, taken from torch's caching allocator."""
    n = load().mhc_scratch_bytes(op, B, S, D, _DTYPE_CODE.get(like.dtype, MHC_F32))
    if n < 0:
        raise MhcError("mhc_scratch_bytes: bad arguments")
    return torch.empty(max(n, 4) // 4, device=like.device, dtype=torch.float32), n


_tickets = {}
_tickets_on = os.environ.get("MHC_TICKETS", "1") != "0"


def set_ticket_finish(enabled: bool) -> None:
    """Finish the deterministic sums inside the producing kernels (default; MHC_TICKETS=0 in the
    environment turns it off) or with the separate finish kernels.  Results are bit-identical."""
    global _tickets_on
    _tickets_on = bool(enabled)


def tickets(like: torch.Tensor, n: int):
    """Device pointer of at least `n` zeroed int32 ticket counters for calls on `like`'s device and
    torch's current stream there.  The kernels leave the counters zero, so the buffer is zeroed only
    when it is created; it is kept per (device, stream) because calls that can overlap on the GPU
    must not share counters.  Created outside of stream capture on first use (warm up before
    capturing a CUDA graph, as torch requires anyway)."""
    if not _tickets_on:
        return None
    dev = like.device.index if like.device.index is not None else torch.cuda.current_device()
    key = (dev, stream_of(like))
    buf = _tickets.get(key)
    if buf is None or buf.numel() < n:
        if torch.cuda.is_current_stream_capturing():
            return None          # never allocate the persistent counters from a graph's private pool
        buf = torch.zeros(max(1024, 2 * n), device=like.device, dtype=torch.int32)
        _tickets[key] = buf
    return buf.data_ptr()


def f32c(t: torch.Tensor) -> torch.Tensor:
    """fp32, contiguous view or copy."""
    if t.dtype != torch.float32:
        t = t.float()
    return t.contiguous()
