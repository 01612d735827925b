"""ctypes binding of libfmta_b200.so (the C ABI declared in include/fmta_b200.h).

There is no CPU or PyTorch fallback: if the library is missing this module raises at
import, and every op requires CUDA tensors.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfmta_b200.so")

FMTA_DTYPE_F32 = 0
FMTA_DTYPE_BF16 = 1
FMTA_OP_BWD_DQ = 1
FMTA_OP_MIX_EXCHANGE = 5
FMTA_OP_FWD_TC = 2
FMTA_OP_BWD_TC = 3
FMTA_OP_BWD_TC_STREAM = 4

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "fmta_b200: %s is missing. Build it with `python flash-multi-token-attention_b200/build.py` "
        "(needs nvcc); there is no fallback path." % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

_vp, _fp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

lib.fmta_version.restype = _i
lib.fmta_strerror.restype = ctypes.c_char_p
lib.fmta_strerror.argtypes = [_i]
lib.fmta_last_cuda_error.restype = _i
lib.fmta_workspace_bytes.restype = _sz
lib.fmta_workspace_bytes.argtypes = [_i] * 8
lib.fmta_fwd.restype = _i
lib.fmta_fwd.argtypes = [_vp, _vp, _vp, _fp, _fp, _vp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i,
                         _vp, _sz, _vp]
lib.fmta_bwd_prep_D.restype = _i
lib.fmta_bwd_prep_D.argtypes = [_vp, _vp, _i, _fp, _sz, _i, _vp]
lib.fmta_bwd_dq_dw.restype = _i
lib.fmta_bwd_dq_dw.argtypes = [_vp, _vp, _vp, _vp, _fp, _fp, _fp, _fp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _i,
                               _f, _i, _vp, _sz, _vp]
lib.fmta_bwd_dq_dw_static.restype = _i
lib.fmta_bwd_dq_dw_static.argtypes = [_vp, _vp, _vp, _vp, _fp, _fp, _fp, _fp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i,
                                      _i, _f, _i, _vp]
lib.fmta_bwd.restype = _i
lib.fmta_bwd.argtypes = [_vp, _vp, _vp, _vp, _fp, _fp, _fp, _fp, _fp, _fp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _i, _f,
                         _i, _i, _vp, _sz, _vp]
lib.fmta_fwd_keep_ktilde.restype = _i
lib.fmta_fwd_keep_ktilde.argtypes = [_vp, _vp, _vp, _fp, _vp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _sz,
                                     _vp, _vp]
lib.fmta_bwd_with_ktilde.restype = _i
lib.fmta_bwd_with_ktilde.argtypes = [_vp, _vp, _vp, _vp, _fp, _fp, _fp, _fp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _f, _i,
                                     _vp, _sz, _vp, _vp]
lib.fmta_fwd_window.restype = _i
lib.fmta_fwd_window.argtypes = [_vp, _vp, _vp, _fp, _vp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _vp, _vp,
                                _sz, _vp]
lib.fmta_stacked_keys.restype = _i
lib.fmta_stacked_keys.argtypes = [_vp, _fp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp]
lib.fmta_bwd_window.restype = _i
lib.fmta_bwd_window.argtypes = [_vp, _vp, _vp, _vp, _fp, _fp, _fp, _fp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i,
                                _vp, _vp, _sz, _vp]
lib.fmta_profile_kernel.restype = _i
lib.fmta_profile_kernel.argtypes = [_i, _vp, _vp]
lib.fmta_set_path.restype = _i
lib.fmta_set_path.argtypes = [_i]
lib.fmta_bwd_dkdv.restype = _i
lib.fmta_bwd_dkdv.argtypes = [_vp, _vp, _vp, _vp, _fp, _fp, _fp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _i, _f, _i,
                              _vp]
lib.fmta_decode.restype = _i
lib.fmta_decode.argtypes = [_vp, _vp, _vp, _fp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp]
lib.fmta_decode_offset_causal.restype = _i
lib.fmta_decode_offset_causal.argtypes = lib.fmta_decode.argtypes
lib.fmta_decode_paged.restype = _i
lib.fmta_decode_paged.argtypes = [_vp, _vp, _vp, _vp, _vp, _fp, _fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _vp]
lib.fmta_kv_append_paged.restype = _i
lib.fmta_kv_append_paged.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]

lib.fmta_set_status_word.restype = _i
lib.fmta_set_status_word.argtypes = [_vp]
lib.fmta_selftest_expire_next.restype = _i
lib.fmta_selftest_expire_next.argtypes = [_i]

EXPORTS = ["fmta_set_status_word", "fmta_selftest_expire_next", "fmta_version", "fmta_strerror", "fmta_last_cuda_error", "fmta_workspace_bytes", "fmta_fwd",
           "fmta_bwd_prep_D", "fmta_bwd", "fmta_fwd_keep_ktilde", "fmta_bwd_with_ktilde", "fmta_fwd_window", "fmta_bwd_window", "fmta_stacked_keys", "fmta_set_path", "fmta_profile_kernel", "fmta_bwd_dq_dw", "fmta_bwd_dq_dw_static", "fmta_bwd_dkdv", "fmta_decode", "fmta_decode_offset_causal", "fmta_decode_paged", "fmta_kv_append_paged"]


def check(status, what):
    """Raise RuntimeError (what TORCH_CHECK raises in the reference wrappers) on a non-zero status."""
    if status != 0:
        msg = lib.fmta_strerror(status).decode()
        extra = ""
        if status == -6:
            extra = " (cudaError %d)" % lib.fmta_last_cuda_error()
        raise RuntimeError("%s: %s%s" % (what, msg, extra))


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr():
    """torch's current stream on the current device, as the `cudaStream_t` the C ABI takes."""
    if _raw_stream is not None:     # same handle as current_stream().cuda_stream, without building a Stream object
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def require_cuda_bf16(t, name):
    """CHECK_INPUT + dtype check of the reference wrappers (fwd_wrapper.cu:25-33)."""
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)
    if t.dtype != torch.bfloat16:
        raise RuntimeError("%s must be bfloat16" % name)


def as_f32(t):
    return t if (t.dtype == torch.float32 and t.is_contiguous()) else t.to(torch.float32).contiguous()


def require_on(ref, t, name, shape=None):
    """Every tensor whose address goes to a kernel must live on the device of ``ref`` (a CPU
    tensor would hand the kernel a host pointer) and, where given, have exactly ``shape``."""
    if not t.is_cuda or t.device != ref.device:
        raise RuntimeError("%s must be a CUDA tensor on %s (got %s)" % (name, ref.device, t.device))
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise RuntimeError("%s must have shape %s (got %s)" % (name, tuple(shape), tuple(t.shape)))


# ---- failure detection: one int32 status word per device, registered with the library ----
_status_words = {}


def _status_word(device):
    """The status word of ``device`` (created, zeroed and registered on first use)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        with torch.cuda.device(idx):
            w = torch.zeros(1, dtype=torch.int32, device="cuda:%d" % idx)
            check(lib.fmta_set_status_word(ctypes.c_void_p(w.data_ptr())), "fmta_set_status_word")
        _status_words[idx] = w
    return w


def arm_status(device):
    """Called by the op wrappers before they launch: makes sure the library folds the status of its
    tensor-core kernels into this device's status word."""
    _status_word(device)


def check_device_status(device=None):
    """Synchronises ``device`` and raises RuntimeError if a bounded wait inside one of the
    tensor-core kernels ran out since the last check (the outputs of that call are invalid).
    The word is cleared, so the next check reports only newer failures."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    w = _status_word(torch.device(device))
    v = int(w.item())          # synchronises
    if v != 0:
        w.zero_()
        check(-8, "fmta_b200 device status")
