"""ctypes binding of the C ABI declared in include/tpx_b200.h.

There is no fallback: if the CUDA library has not been built, importing a compute entry point
raises. Device pointers are taken from torch tensors (`data_ptr()`), the stream is torch's
current CUDA stream."""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.environ.get("TPX_LIBRARY") or os.path.join(_HERE, "libtpx_b200.so")  # TPX_LIBRARY: another build of the library (experiments)
_lib = None

c_i64, c_int, c_f32, c_vp, c_sz = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t

_SIGS = {
    "tpx_version": (c_int, []),
    "tpx_last_error": (ctypes.c_char_p, []),
    "tpx_sm_count": (c_int, []),
    "tpx_e2m1_pair_table": (c_int, [c_vp, c_vp]),
    "tpx_reload_options": (None, []),
    "tpx_remap_and_quantize_mxfp4": (c_int, [c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "tpx_remap_and_quantize_qint8": (c_int, [c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_i64, ctypes.POINTER(c_i64), c_vp]),
    "tpx_dequantize_mxfp4": (c_int, [c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp]),
    "tpx_dequantize_qint8": (c_int, [c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp]),
    "tpx_packed_bytes": (c_int, [c_int, c_i64, c_i64, c_i64, ctypes.POINTER(c_sz), ctypes.POINTER(c_sz)]),
    "tpx_repack_mxfp4": (c_int, [c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "tpx_repack_qint8": (c_int, [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "tpx_qlinear_scratch_bytes": (c_sz, [c_int, c_i64, c_i64, c_i64, c_i64, c_int]),
    "tpx_tc_packed_bytes": (c_int, [c_i64, c_i64, c_int, ctypes.POINTER(c_sz), ctypes.POINTER(c_sz)]),
    "tpx_repack_mxfp4_tc": (c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "tpx_qlinear_mxfp4_tc_scratch_bytes": (c_sz, [c_i64, c_i64, c_i64, c_int]),
    "tpx_qlinear_mxfp4_tc": (c_int, [c_vp, c_vp, c_int, c_vp, c_i64, c_i64, c_i64, c_vp, c_int, c_vp, c_vp, c_f32, c_vp,
                                     c_vp, c_sz, c_vp]),
    "tpx_rmsnorm_qlinear_mxfp4_tc": (c_int, [c_vp, c_vp, c_int, c_vp, c_vp, c_int, c_f32, c_i64, c_i64, c_i64, c_vp, c_int, c_vp, c_vp,
                                             c_f32, c_vp, c_vp, c_sz, c_vp]),
    "tpx_tc_packed_bytes_qint8": (c_int, [c_i64, c_i64, c_i64, c_vp, c_vp]),
    "tpx_repack_qint8_tc": (c_int, [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "tpx_unpack_qint8_tc_bf16": (c_int, [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp]),
    "tpx_qlinear_qint8_tc_scratch_bytes": (c_sz, [c_i64, c_i64, c_i64, c_i64]),
    "tpx_qlinear_qint8_tc": (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_f32, c_i64, c_i64, c_i64, c_i64, c_int, c_vp, c_int, c_vp, c_vp, c_f32,
                                     c_vp, c_vp, c_sz, c_vp]),
    "tpx_linear_bf16_tc_scratch_bytes": (c_sz, [c_i64, c_i64, c_i64]),
    "tpx_linear_bf16_tc": (c_int, [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_int, c_vp, c_vp, c_f32, c_vp, c_vp, c_sz, c_vp]),
    "tpx_allreduce_flag_bytes": (c_sz, []),
    "tpx_allreduce_bf16": (c_int, [c_vp, c_i64, c_int, c_int, c_vp, c_vp, c_vp, c_i64, c_vp]),
    "tpx_launch_count": (ctypes.c_ulonglong, []),
    "tpx_debug_tc_timeline": (None, [c_vp]),  # exported only by a -DTPX_DEBUG build
    "tpx_qlinear_mxfp4_tc_static_status": (c_int, [c_vp, ctypes.POINTER(ctypes.c_uint)]),
    "tpx_qlinear_mxfp4_tc_static_max_bytes": (c_sz, []),
    "tpx_qlinear_mxfp4_tc_static": (c_int, [c_vp, c_vp, c_int, c_vp, c_i64, c_i64, c_i64, c_vp, c_int, c_vp, c_vp, c_f32, c_vp, c_vp]),
    "tpx_rmsnorm": (c_int, [c_vp, c_vp, c_int, c_f32, c_i64, c_i64, c_vp, c_vp]),
    "tpx_layernorm": (c_int, [c_vp, c_vp, c_vp, c_int, c_f32, c_i64, c_i64, c_vp, c_vp]),
    "tpx_fp8_tc_packed_bytes": (c_int, [c_i64, c_i64, c_int, ctypes.POINTER(c_sz), ctypes.POINTER(c_sz)]),
    "tpx_repack_fp8_tc": (c_int, [c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "tpx_qlinear_fp8_tc_scratch_bytes": (c_sz, [c_i64, c_i64, c_i64, c_int]),
    "tpx_qlinear_fp8_tc": (c_int, [c_vp, c_vp, c_int, c_int, c_vp, c_vp, c_int, c_f32, c_i64, c_i64, c_i64, c_vp, c_int, c_vp, c_vp, c_f32,
                                   c_vp, c_vp, c_sz, c_vp]),
    "tpx_llama_layer_attention": (c_int, [c_vp, c_vp, c_vp]),
    "tpx_llama_layer_mlp": (c_int, [c_vp, c_vp, c_vp]),
    "tpx_rope_kv_update_gptj": (c_int, [c_vp, c_vp, c_vp] + [c_i64] * 10 + [c_vp] * 6 + [c_vp]),
    "tpx_argmax_bf16": (c_int, [c_vp, c_i64, c_i64, c_vp, c_vp]),
    "tpx_rope_kv_update": (c_int, [c_vp, c_vp, c_vp] + [c_i64] * 10 + [c_vp, c_vp, c_vp, c_vp, c_vp]),
    "tpx_rope_kv_update_paged": (c_int, [c_vp, c_vp, c_vp] + [c_i64] * 10 + [c_vp, c_vp, c_vp, c_vp, c_vp]),
    "tpx_attention_paged": (c_int, [c_vp, c_vp, c_vp, c_vp] + [c_i64] * 7 + [c_int, c_int, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "tpx_attention_scratch_bytes": (c_sz, [c_i64] * 6),
    "tpx_attention": (c_int, [c_vp, c_vp, c_vp, c_vp] + [c_i64] * 7 + [c_int, c_int, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "tpx_attention_tc_status": (c_int, [c_vp, ctypes.POINTER(ctypes.c_uint)]),
    "tpx_align_and_invert_mask": (c_int, [c_vp, c_i64, c_i64, c_i64, ctypes.c_uint16, c_vp, c_vp]),
    "tpx_qlinear": (c_int, [c_int, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_i64, c_i64, c_i64, c_vp, c_int, c_vp, c_vp,
                            c_f32, c_vp, c_vp, c_sz, c_vp]),
}


class TpxError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            raise TpxError(
                f"{_SO} is missing: build it with `python -m tpp_pytorch_extension_b200._build` "
                "(there is no CPU or eager fallback)")
        L = ctypes.CDLL(_SO)
        for name, (res, args) in _SIGS.items():
            if hasattr(L, name):
                fn = getattr(L, name)
                fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


class LlamaLayerStruct(ctypes.Structure):
    """TpxLlamaLayer of include/tpx_b200.h."""
    _fields_ = [(n, ctypes.c_int64) for n in ("D", "Nq", "Nkv", "H", "FF", "MP", "HR")] + \
               [("eps", ctypes.c_float), ("res_scale", ctypes.c_float), ("gamma_is_f32", ctypes.c_int)] + \
               [(n, ctypes.c_void_p) for n in ("gamma1", "gamma2", "bias_qkv", "ep", "wqkv", "sfa_qkv", "wo", "sfa_o", "wgu", "sfa_gu",
                                                 "wd", "sfa_d")]


class LlamaLayerIOStruct(ctypes.Structure):
    """TpxLlamaLayerIO of include/tpx_b200.h."""
    _fields_ = [(n, ctypes.c_int64) for n in ("B", "S", "Bpos", "Spad", "offset", "capacity")] + \
               [(n, ctypes.c_void_p) for n in ("x", "pos", "mask", "dev_len", "kc", "vc", "k_pages", "v_pages", "qkv", "q", "ctx", "so",
                                                 "inter", "out", "scratch")] + \
               [("scratch_bytes", ctypes.c_size_t), ("attn_scratch", ctypes.c_void_p), ("attn_scratch_bytes", ctypes.c_size_t),
                ("handoff", ctypes.c_void_p), ("handoff_bytes", ctypes.c_size_t)]


def check(rc):
    if rc != 0:
        raise TpxError(f"tpx error {rc}: {lib().tpx_last_error().decode()}")


def ptr(t):
    """Device pointer of a tensor, or NULL for None / empty (the reference's 'absent' tensor)."""
    if t is None or t.numel() == 0:
        return None
    return t.data_ptr()


def stream():
    """Raw handle of the current CUDA stream of the current device (the fast accessors: torch.cuda.current_stream() builds
    a Python Stream object, 3 us per call, which counted on every launch)."""
    try:
        return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())
    except AttributeError:  # other torch builds
        return torch.cuda.current_stream().cuda_stream


def current_device():
    try:
        return torch._C._cuda_getDevice()
    except AttributeError:
        return torch.cuda.current_device()


def require_cuda(t, name):
    if not t.is_cuda:
        raise TpxError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise TpxError(f"{name} must be contiguous")


def reload_options():
    """Re-read the TPX_* kernel-selection switches (the library and the Python side read them once)."""
    from ._C import _fused_llm_infer
    _fused_llm_infer._OPTS.clear()
    _fused_llm_infer._SCRATCH_BYTES.clear()  # sizes depend on the kernel family the switches select
    if _lib is not None:
        _lib.tpx_reload_options()


def assert_no_kernel_error(sync=True):
    """Raises if a kernel gave up on one of its bounded waits since the buffers were created: such a kernel leaves a
    code in the error word of its scratch and finishes early with a wrong result."""
    if sync:
        torch.cuda.synchronize()
    for (dev, _), buf in list(_scratch.items()):
        code = int(buf[65532:65536].view(torch.int32).item())
        if code:
            raise TpxError(f"a linear kernel on device {dev} gave up on a bounded wait (code {code})")
    from . import _peer_allreduce
    for inst in list(_peer_allreduce._instances.values()):
        code = inst.error_code()
        if code:
            raise TpxError(f"the peer-memory all-reduce gave up waiting for rank {code - 1}")
    if _lib is not None and torch.cuda.is_available():
        st = ctypes.c_uint(0)
        check(_lib.tpx_attention_tc_status(stream(), ctypes.byref(st)))
        if st.value:
            raise TpxError(f"the prefill attention kernel gave up on a bounded wait (code {st.value})")


_scratch = {}


def scratch(nbytes, device):
    """Per-device, per-stream zero-initialised scratch for split-K partial sums, grown on demand."""
    key = (device.index, stream())
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


_dense = {}


def dense_scratch(nbytes, device):
    """Transient buffer for a weight unpacked to bf16 for one call (int8 weights with many tokens); no initial state."""
    key = (device.index, stream())
    buf = _dense.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _dense[key] = buf
    return buf


_layer_ws = {}


def layer_workspace(nbytes, device):
    """Temporaries of one decoder layer (q/k/v, rotated q, attention output, the two MLP inputs): reused by every layer."""
    key = (device.index, stream())
    buf = _layer_ws.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _layer_ws[key] = buf
    return buf


_handoff = {}


def handoff_buffer(nbytes, device):
    """The buffer through which the gate/up kernel hands its output to the down projection as activation terms (decode
    shapes): zero-initialised, written by those kernels only."""
    key = (device.index, stream())
    buf = _handoff.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=device)
        _handoff[key] = buf
    off = (-buf.data_ptr()) % 1024
    return buf[off:off + nbytes]


_aux = {}


def aux_scratch(nbytes, device):
    """Attention scratch (arrival counters of the KV splits, zero before first use and left zero by the kernel, then
    the splits' partials), separate from the linear's."""
    key = (device.index, stream())
    buf = _aux.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _aux[key] = buf
    return buf
