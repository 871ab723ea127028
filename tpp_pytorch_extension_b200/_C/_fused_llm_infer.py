"""Mirror of the reference's `_C._fused_llm_infer` submodule / `torch.ops.tpp_llm`
(src/csrc/llm/fused_llm_infer.cpp:1568-1611) for the quantized-linear part of the path."""
import torch

from .. import _lib
from ._qtype import QTensor

ACT = {None: 0, "none": 0, "gelu": 1, "silu": 2, "relu": 3}
_SCRATCH_BYTES = {}


def mxfp4_path():
    """Kernel family for MXFP4 weights: "tc" = tcgen05 tensor-core kernel (default), "stream" = the
    mma.sync weight-streaming kernel. Read from TPX_MXFP4_PATH on every call so tests can flip it."""
    import os
    return os.environ.get("TPX_MXFP4_PATH", "tc")


def _qlinear(x, w, w2, bias, act, mul_in, res, res_scale):
    if not isinstance(w, QTensor):
        raise _lib.TpxError("fc_plain: weight must be a quantized tensor from remap_and_quantize_*")
    _lib.require_cuda(x, "input")
    if x.dtype != torch.bfloat16:
        raise _lib.TpxError("fc_plain: input must be bfloat16")
    N, K = w.out_features, w.in_features
    if x.shape[-1] != K:
        raise _lib.TpxError(f"fc_plain: input features {x.shape[-1]} do not match weight in-features {K}")
    M = x.numel() // K
    y = torch.empty(x.shape[:-1] + (N,), dtype=torch.bfloat16, device=x.device)
    L = _lib.lib()
    if x.device.index != torch.cuda.current_device():
        raise _lib.TpxError("fc_plain: input lives on a device other than the current one")
    for name, t in (("bias", bias), ("mul_in", mul_in), ("res", res)):
        if t is not None and t.numel() > 0:
            _lib.require_cuda(t, name)
            if t.dtype != torch.bfloat16:
                raise _lib.TpxError(f"fc_plain: {name} must be bfloat16")
    if w.kind == 1 and mxfp4_path() == "tc":
        if w2 is not None and (w2.out_features, w2.in_features, w2.kind) != (N, K, w.kind):
            raise _lib.TpxError("gate/up weights must have the same shape and quantization")
        wq, sfa = w.packed_tc(w2)
        key = ("tc", M, N, K, w2 is not None)
        nb = _SCRATCH_BYTES.get(key)
        if nb is None:
            nb = _SCRATCH_BYTES[key] = L.tpx_qlinear_mxfp4_tc_scratch_bytes(M, N, K, int(w2 is not None))
        sc = _lib.scratch(nb, x.device)
        rc = L.tpx_qlinear_mxfp4_tc(wq.data_ptr(), sfa.data_ptr(), int(w2 is not None), x.data_ptr(), M, N, K,
                                    _lib.ptr(bias), ACT[act], _lib.ptr(mul_in), _lib.ptr(res), float(res_scale),
                                    y.data_ptr(), sc.data_ptr(), sc.numel(), _lib.stream())
        if rc:
            _lib.check(rc)
        return y
    pc, ps = w.packed()
    pc2 = ps2 = None
    if w2 is not None:
        if (w2.out_features, w2.in_features, w2.kind, w2.block_size) != (N, K, w.kind, w.block_size):
            raise _lib.TpxError("gate/up weights must have the same shape and quantization")
        pc2, ps2 = w2.packed()
    key = (w.kind, min(M, 32), N, K, w.block_size, w2 is not None)
    nb = _SCRATCH_BYTES.get(key)
    if nb is None:
        nb = _SCRATCH_BYTES[key] = L.tpx_qlinear_scratch_bytes(w.kind, M, N, K, w.block_size, int(w2 is not None))
    sc = _lib.scratch(nb, x.device)
    rc = L.tpx_qlinear(w.kind, pc.data_ptr(), ps.data_ptr(), _lib.ptr(pc2), _lib.ptr(ps2), w.block_size,
                       x.data_ptr(), M, N, K, _lib.ptr(bias), ACT[act], _lib.ptr(mul_in), _lib.ptr(res),
                       float(res_scale), y.data_ptr(), sc.data_ptr(), sc.numel(), _lib.stream())
    if rc:
        _lib.check(rc)
    return y


def fc_plain(input, weight, bias=None, parallel_dim=-1, split_sizes=()):
    """torch.ops.tpp_llm.fc_plain (src/csrc/llm/fused_llm_infer.cpp:1514-1566), single-rank form."""
    if parallel_dim != -1:
        from ..llm import llm_common
        return llm_common.fc_plain_parallel(input, weight, bias, parallel_dim, list(split_sizes))
    return _qlinear(input, weight, None, bias, None, None, None, 1.0)


def fc_plain_act(input, weight, bias=None, act=None, mul_in=None, res=None, res_scale=1.0):
    """Linear with the reference's post-ops (src/csrc/fused_gemm.h:1343-1458), which the reference only
    reaches from inside its decoder blocks: act in {None, "gelu", "silu", "relu"}, then `* mul_in`
    (MulPostOp), then `+ res * res_scale` (AddScalePostOp)."""
    return _qlinear(input, weight, None, bias, act, mul_in, res, res_scale)


def fc_gate_up(input, w_gate, w_up, act="silu"):
    """act(x.Wg^T) * (x.Wu^T) in one pass over both weights (src/csrc/llm/fused_llm_infer.cpp:1271-1272)."""
    return _qlinear(input, w_gate, w_up, None, act, None, None, 1.0)
