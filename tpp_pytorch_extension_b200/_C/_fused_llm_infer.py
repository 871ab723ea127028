"""Mirror of the reference's `_C._fused_llm_infer` submodule / `torch.ops.tpp_llm`
(src/csrc/llm/fused_llm_infer.cpp:1568-1611) for the quantized-linear part of the path."""
import ctypes

import torch

from .. import _lib
from .. import _timers
from ._qtype import QTensor

import os

ACT = {None: 0, "none": 0, "gelu": 1, "silu": 2, "relu": 3}
_SCRATCH_BYTES = {}
_OPTS = {}  # TPX_* switches, read from the environment once; _lib.reload_options() empties it


def _opt(name, default):
    v = _OPTS.get(name)
    if v is None:
        v = _OPTS[name] = os.environ.get(name, default)
    return v


def mxfp4_path():
    """Kernel family for MXFP4 weights: "tc" = tcgen05 tensor-core kernel (default), "stream" = the
    mma.sync weight-streaming kernel (TPX_MXFP4_PATH)."""
    return _opt("TPX_MXFP4_PATH", "tc")


def int8_path():
    """Kernel family for int8 weights: "tc" (default) = tcgen05 kind::i8 kernel with the reference's
    activation-quantised arithmetic, "stream" = the mma.sync weight-only streaming kernel (TPX_INT8_PATH)."""
    return _opt("TPX_INT8_PATH", "tc")


INT8_DENSE_MIN_TOKENS = 128  # above this the int8 weight is unpacked to bf16 per call (256 tokens: 68 against 160 us)


def _int8_tc(x, y, w, w2, bias, act, mul_in, res, res_scale, norm=None):
    """int8 weights: up to 128 tokens through tpx_qlinear_qint8_tc (the reference's activation-quantised arithmetic); a
    gate/up pair runs as two calls, the second multiplying by the activated first. More tokens: weight-only arithmetic
    on the bf16 tensor-core kernel (TPX_INT8_DENSE=0 keeps the int8 kernel for every token count)."""
    L = _lib.lib()
    N, K = w.out_features, w.in_features
    M = x.numel() // K

    if M > INT8_DENSE_MIN_TOKENS and _opt("TPX_INT8_DENSE", "1") != "0":
        # many tokens: the weight unpacked to bf16 for this call, then the bf16 tensor-core kernel (weight-only
        # arithmetic; see tpx_unpack_qint8_tc_bf16)
        if norm is not None:
            x = rms_norm(x, norm[0], norm[1])

        def dense(wt):
            wq, sw = wt.packed_i8tc()
            buf = _lib.dense_scratch(N * K * 2, x.device)[: N * K * 2].view(torch.bfloat16).view(N, K)
            _lib.check(L.tpx_unpack_qint8_tc_bf16(wq.data_ptr(), sw.data_ptr(), N, K, wt.block_size, buf.data_ptr(), _lib.stream()))
            return buf

        if w2 is None:
            return _bf16_linear(x, dense(w), bias, act, mul_in, res, res_scale)
        h = _bf16_linear(x, dense(w), bias, act, None, None, 1.0)
        return _bf16_linear(x, dense(w2), None, None, h, None, 1.0)

    gam, eps = (norm[0], float(norm[1])) if norm is not None else (None, 0.0)

    def run(wt, out, b, a, m, r, rs, reuse=0):
        wq, sw = wt.packed_i8tc()
        key = ("i8tc", M, N, K, wt.block_size)
        nb = _SCRATCH_BYTES.get(key)
        if nb is None:
            nb = _SCRATCH_BYTES[key] = L.tpx_qlinear_qint8_tc_scratch_bytes(M, N, K, wt.block_size)
        sc = _lib.scratch(nb, x.device)
        rc = L.tpx_qlinear_qint8_tc(wq.data_ptr(), sw.data_ptr(), x.data_ptr(), _lib.ptr(gam), int(gam is not None and gam.dtype == torch.float32),
                                    eps, M, N, K, wt.block_size, reuse, _lib.ptr(b), ACT[a], _lib.ptr(m),
                                    _lib.ptr(r), float(rs), out.data_ptr(), sc.data_ptr(), sc.numel(), _lib.stream())
        if rc:
            _lib.check(rc)

    if w2 is None:
        run(w, y, bias, act, mul_in, res, res_scale)
        return y
    h = torch.empty_like(y)
    run(w, h, bias, act, None, None, 1.0)
    run(w2, y, None, None, h, None, 1.0, reuse=1)  # same x: the quantised activations are still in the scratch
    return y


def _bf16_linear(x, w, bias, act, mul_in, res, res_scale):
    """Unquantized bf16 weight, plain [N, K] (nn.Linear.weight) or blocked 5-D [N/bk, K/bc, bc/2, bk, 2]
    (BlockedParameter.block(), un-blocked once and cached on the tensor): tpx_linear_bf16_tc."""
    _lib.require_cuda(x, "input")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise _lib.TpxError("fc_plain: bf16 input and bf16 weight expected")
    if w.dim() == 5:
        plain = getattr(w, "_tpx_plain", None)
        if plain is None:
            from ..utils.blocked_layout import unblock_weight
            plain = unblock_weight(w)
            try:
                w._tpx_plain = plain
            except Exception:
                pass
        w = plain
    if w.dim() != 2 or not w.is_contiguous():
        raise _lib.TpxError("fc_plain: the bf16 weight must be a contiguous [out_features, in_features] matrix")
    N, K = w.shape
    if x.shape[-1] != K:
        raise _lib.TpxError(f"fc_plain: input features {x.shape[-1]} do not match weight in-features {K}")
    if not x.is_contiguous():
        x = x.contiguous()
    M = x.numel() // K
    y = torch.empty(x.shape[:-1] + (N,), dtype=torch.bfloat16, device=x.device)
    for name, t in (("bias", bias), ("mul_in", mul_in), ("res", res)):
        if t is not None and t.numel() > 0:
            _lib.require_cuda(t, name)
            if t.dtype != torch.bfloat16:
                raise _lib.TpxError(f"fc_plain: {name} must be bfloat16")
    sc = _lib.scratch(1 << 16, x.device)
    _lib.check(_lib.lib().tpx_linear_bf16_tc(w.data_ptr(), x.data_ptr(), M, N, K, _lib.ptr(bias), ACT[act], _lib.ptr(mul_in),
                                             _lib.ptr(res), float(res_scale), y.data_ptr(), sc.data_ptr(), sc.numel(), _lib.stream()))
    return y


_FP8 = (torch.float8_e4m3fn, torch.float8_e5m2)


def _wrap_fp8(w):
    """A plain [N, K] tensor of an 8-bit floating-point dtype -> its Fp8Weight (kept on the tensor)."""
    if isinstance(w, torch.Tensor) and w.dtype in _FP8:
        hit = getattr(w, "_tpx_fp8", None)
        if hit is None:
            from ._qtype import Fp8Weight
            hit = Fp8Weight(w)
            try:
                w._tpx_fp8 = hit
            except Exception:
                pass
        return hit
    return w


def _qlinear(x, w, w2, bias, act, mul_in, res, res_scale, norm=None, out=None):
    w, w2 = _wrap_fp8(w), _wrap_fp8(w2)
    if isinstance(w, torch.Tensor) and w2 is None:
        if out is not None:
            raise _lib.TpxError("fc_plain: out= is served for quantized weights only")
        if norm is not None:
            x = rms_norm(x, norm[0], norm[1])
        return _bf16_linear(x, w, bias, act, mul_in, res, res_scale)
    if not isinstance(w, QTensor):
        raise _lib.TpxError("fc_plain: weight must be a quantized tensor from remap_and_quantize_* or a bf16 tensor")
    # Host buffers: a PINNED host tensor may stand in for the input and for out= on the MXFP4 tensor-core path. Pinned
    # memory is addressable from the device, so the activation-split kernel reads x across the bus and the epilogue
    # writes y there: no separate copies, which on decode-sized tensors cost more stream time than the linear itself.
    host_in = not x.is_cuda
    if host_in:
        if not (x.is_pinned() and x.is_contiguous() and w.kind == 1 and mxfp4_path() == "tc" and norm is None):
            raise _lib.TpxError("input must be a CUDA tensor (a pinned, contiguous host tensor is accepted by the MXFP4 tensor-core path)")
        dev = torch.device("cuda", _lib.current_device())
    else:
        _lib.require_cuda(x, "input")
        dev = x.device
    if x.dtype != torch.bfloat16:
        raise _lib.TpxError("fc_plain: input must be bfloat16")
    N, K = w.out_features, w.in_features
    if x.shape[-1] != K:
        raise _lib.TpxError(f"fc_plain: input features {x.shape[-1]} do not match weight in-features {K}")
    M = x.numel() // K
    if out is not None:
        if (tuple(out.shape) != tuple(x.shape[:-1]) + (N,) or out.dtype != torch.bfloat16 or not out.is_contiguous()
                or not (out.is_cuda or (out.is_pinned() and w.kind == 1 and mxfp4_path() == "tc"))):
            raise _lib.TpxError("fc_plain: out= must be a contiguous bfloat16 tensor of the result's shape on the device (or pinned host memory, MXFP4 tensor-core path)")
        y = out
    else:
        y = torch.empty(x.shape[:-1] + (N,), dtype=torch.bfloat16, device=dev)
    L = _lib.lib()
    if dev.index != _lib.current_device():
        raise _lib.TpxError("fc_plain: input lives on a device other than the current one")
    for name, t in (("bias", bias), ("mul_in", mul_in), ("res", res)):
        if t is not None and t.numel() > 0:
            _lib.require_cuda(t, name)
            if t.dtype != torch.bfloat16:
                raise _lib.TpxError(f"fc_plain: {name} must be bfloat16")
    if w.kind == 3:  # 8-bit floating-point weight (bfloat8 / hfloat8): the 128-row tensor-core kernel reads the bytes as they are
        wq, sfa = w.packed_tc(w2)
        key = ("fp8", M, N, K, w2 is not None)
        nb = _SCRATCH_BYTES.get(key)
        if nb is None:
            nb = _SCRATCH_BYTES[key] = L.tpx_qlinear_fp8_tc_scratch_bytes(M, N, K, int(w2 is not None))
        sc = _lib.scratch(nb, dev)
        gamma = eps = None
        if norm is not None and K <= 8192 and _opt("TPX_FUSED_NORM", "1") != "0":
            gamma, eps = norm
        elif norm is not None:
            x = rms_norm(x, norm[0], norm[1])
        if not x.is_contiguous():
            x = x.contiguous()
        rc = L.tpx_qlinear_fp8_tc(wq.data_ptr(), sfa.data_ptr(), w.fmt, int(w2 is not None), x.data_ptr(), _lib.ptr(gamma),
                                  int(gamma is not None and gamma.dtype == torch.float32), float(eps or 0.0), M, N, K, _lib.ptr(bias),
                                  ACT[act], _lib.ptr(mul_in), _lib.ptr(res), float(res_scale), y.data_ptr(), sc.data_ptr(), sc.numel(),
                                  _lib.stream())
        if rc:
            _lib.check(rc)
        return y
    if w.kind == 1 and mxfp4_path() == "tc":
        if w2 is not None and (w2.out_features, w2.in_features, w2.kind) != (N, K, w.kind):
            raise _lib.TpxError("gate/up weights must have the same shape and quantization")
        wq, sfa = w.packed_tc(w2)
        key = ("tc", M, N, K, w2 is not None, _opt("TPX_TC_WIDE", "auto"), _opt("TPX_TC_F4", "auto"))
        nb = _SCRATCH_BYTES.get(key)
        if nb is None:
            nb = _SCRATCH_BYTES[key] = L.tpx_qlinear_mxfp4_tc_scratch_bytes(M, N, K, int(w2 is not None))
        sc = _lib.scratch(nb, dev)
        if norm is not None and K <= 8192 and _opt("TPX_FUSED_NORM", "1") != "0":
            gamma, eps = norm
            rc = L.tpx_rmsnorm_qlinear_mxfp4_tc(wq.data_ptr(), sfa.data_ptr(), int(w2 is not None), x.data_ptr(), gamma.data_ptr(),
                                                int(gamma.dtype == torch.float32), float(eps), M, N, K, _lib.ptr(bias), ACT[act],
                                                _lib.ptr(mul_in), _lib.ptr(res), float(res_scale), y.data_ptr(), sc.data_ptr(),
                                                sc.numel(), _lib.stream())
            if rc:
                _lib.check(rc)
            return y
        if norm is not None:
            x = rms_norm(x, norm[0], norm[1])
        rc = L.tpx_qlinear_mxfp4_tc(wq.data_ptr(), sfa.data_ptr(), int(w2 is not None), x.data_ptr(), M, N, K,
                                    _lib.ptr(bias), ACT[act], _lib.ptr(mul_in), _lib.ptr(res), float(res_scale),
                                    y.data_ptr(), sc.data_ptr(), sc.numel(), _lib.stream())
        if rc:
            _lib.check(rc)
        return y
    if w.kind != 1 and M > 0 and int8_path() == "tc" and w.block_size in (64, 128, 256, 512):
        if w2 is not None and (w2.out_features, w2.in_features, w2.kind, w2.block_size) != (N, K, w.kind, w.block_size):
            raise _lib.TpxError("gate/up weights must have the same shape and quantization")
        if norm is not None and not (K <= 8192 and w.block_size <= 256):
            x, norm = rms_norm(x, norm[0], norm[1]), None
        return _int8_tc(x, y, w, w2, bias, act, mul_in, res, res_scale, norm)
    if norm is not None:
        x = rms_norm(x, norm[0], norm[1])
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
    sc = _lib.scratch(nb, dev)
    rc = L.tpx_qlinear(w.kind, pc.data_ptr(), ps.data_ptr(), _lib.ptr(pc2), _lib.ptr(ps2), w.block_size,
                       x.data_ptr(), M, N, K, _lib.ptr(bias), ACT[act], _lib.ptr(mul_in), _lib.ptr(res),
                       float(res_scale), y.data_ptr(), sc.data_ptr(), sc.numel(), _lib.stream())
    if rc:
        _lib.check(rc)
    return y


def fc_plain(input, weight, bias=None, parallel_dim=-1, split_sizes=(), out=None):
    """torch.ops.tpp_llm.fc_plain (src/csrc/llm/fused_llm_infer.cpp:1514-1566), single-rank form. Extension: out= (a
    device tensor or, for MXFP4 weights, pinned host memory) receives the result; the input may be pinned host memory."""
    if parallel_dim != -1:
        from ..llm import llm_common
        return llm_common.fc_plain_parallel(input, weight, bias, parallel_dim, list(split_sizes))
    return _qlinear(input, weight, None, bias, None, None, None, 1.0, out=out)


def fc_plain_act(input, weight, bias=None, act=None, mul_in=None, res=None, res_scale=1.0):
    """Linear with the reference's post-ops (src/csrc/fused_gemm.h:1343-1458), which the reference only
    reaches from inside its decoder blocks: act in {None, "gelu", "silu", "relu"}, then `* mul_in`
    (MulPostOp), then `+ res * res_scale` (AddScalePostOp)."""
    return _qlinear(input, weight, None, bias, act, mul_in, res, res_scale)


def fc_gate_up(input, w_gate, w_up, act="silu", norm=None):
    """act(x.Wg^T) * (x.Wu^T) in one pass over both weights (src/csrc/llm/fused_llm_infer.cpp:1271-1272).
    norm = (gamma, eps): RMSNorm of the input first, fused into the linear where the kernel family supports it."""
    if isinstance(w_gate, torch.Tensor) and w_gate.dtype not in _FP8:  # bf16 weights: two passes, the second multiplying by the activated first
        if norm is not None:
            input = rms_norm(input, norm[0], norm[1])
        g = _bf16_linear(input, w_gate, None, act, None, None, 1.0)
        return _bf16_linear(input, w_up, None, None, g, None, 1.0)
    return _qlinear(input, w_gate, w_up, None, act, None, None, 1.0, norm)


def fc_plain_norm(input, gamma, eps, weight, bias=None):
    """llama_rms_norm followed by fc_plain (src/csrc/llm/fused_llm_infer.cpp:1204-1215) as one call."""
    if gamma.dtype not in (torch.bfloat16, torch.float32):
        raise _lib.TpxError("llama_rms_norm: unsupported gamma dtype")
    return _qlinear(input, weight, None, bias, None, None, None, 1.0, (gamma, eps))


# --------------------------------------------------------------------------- decoder-layer pieces
def layer_norm(x, gamma, beta, eps):
    """lyr_norm (src/csrc/llm/fused_llm_infer.cpp:256-306): LayerNorm over the last dimension, bf16 in and out, gamma and
    beta both bf16 or both fp32."""
    _lib.require_cuda(x, "input")
    if x.dtype != torch.bfloat16:
        raise _lib.TpxError("lyr_norm: input must be bfloat16")
    if gamma.dtype != beta.dtype or gamma.dtype not in (torch.bfloat16, torch.float32):
        raise _lib.TpxError("lyr_norm: unsupported gamma dtype")
    x = x.contiguous()
    y = torch.empty_like(x)
    D = x.shape[-1]
    _lib.check(_lib.lib().tpx_layernorm(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), int(gamma.dtype == torch.float32), float(eps),
                                        x.numel() // D if D else 0, D, y.data_ptr(), _lib.stream()))
    return y


def rms_norm(x, gamma, eps):
    """llama_rms_norm (src/csrc/llm/fused_llm_infer.cpp:336-363)."""
    _lib.require_cuda(x, "input")
    y = torch.empty_like(x)
    D = x.shape[-1]
    if gamma.dtype not in (torch.bfloat16, torch.float32):
        raise _lib.TpxError("llama_rms_norm: unsupported gamma dtype")
    _lib.check(_lib.lib().tpx_rmsnorm(x.data_ptr(), gamma.data_ptr(), int(gamma.dtype == torch.float32), float(eps),
                                      x.numel() // D, D, y.data_ptr(), _lib.stream()))
    return y


def argmax_rows(x):
    """Greedy pick over the last dimension of bf16 logits [..., n] -> int64 [...], torch.argmax semantics (first of
    equal maxima). One launch of a row-per-CTA kernel instead of the library's generic reduction."""
    _lib.require_cuda(x, "logits")
    if x.dtype != torch.bfloat16:
        raise _lib.TpxError("argmax_rows: bf16 logits expected")
    x = x.contiguous()
    n = x.shape[-1]
    out = torch.empty(x.shape[:-1], dtype=torch.int64, device=x.device)
    _lib.check(_lib.lib().tpx_argmax_bf16(x.data_ptr(), x.numel() // n if n else 0, n, out.data_ptr(), _lib.stream()))
    return out


_pg = None


def set_pg(pg):
    """tpp_llm.set_pg (src/csrc/llm/fused_llm_infer.cpp:66-99): the process group of the tensor-parallel ranks."""
    global _pg
    _pg = pg


def get_pg_size():
    import torch.distributed as dist
    return dist.get_world_size(_pg) if (_pg is not None and dist.is_initialized()) else 1


def allreduce(t):
    """tpp_llm.allreduce (src/csrc/llm/fused_llm_infer.cpp:101-119): in-place SUM over the tensor-parallel ranks
    (small bf16 tensors: this library's own kernel over peer memory, csrc/tpx_allreduce.cu; anything else: NCCL. The
    reference likewise has a shared-memory all-reduce beside the c10d backend)."""
    import torch.distributed as dist
    if _pg is None or not dist.is_initialized():
        raise _lib.TpxError("Missing process group when using model parallel, use set_pg()")
    if t.is_cuda:
        from .. import _peer_allreduce
        peer = _peer_allreduce.get(_pg)
        if peer is not None and peer.serves(t):
            return peer(t)
    dist.all_reduce(t, group=_pg)
    return t


def _cat_q(ws):
    """Concatenate quantized weights along the output features (the fused q/k/v loop nest of the reference,
    src/csrc/llm/fused_llm_infer.cpp:422-505): blocks are per output row, so stacking the storage is exact."""
    from ._qtype import QTensor
    w0 = ws[0]
    if w0.kind == 3:
        from ._qtype import Fp8Weight
        if any(w.kind != 3 or w.fmt != w0.fmt or w.shape[1] != w0.shape[1] for w in ws):
            raise _lib.TpxError("fused q/k/v: weights must share format and in-features")
        return Fp8Weight(torch.cat([w.codes for w in ws], 0).view(w0.dtype))
    from ._qtype import QInt2Tensor
    if isinstance(w0, QInt2Tensor):
        if any(not isinstance(w, QInt2Tensor) or (w.block_size, w.shape[1:]) != (w0.block_size, w0.shape[1:]) for w in ws):
            raise _lib.TpxError("fused q/k/v: weights must share quantization and in-features")
        codes = torch.cat([w.codes for w in ws], 0)
        return QInt2Tensor(codes, torch.cat([w.scales for w in ws], 0), (codes.shape[0],) + tuple(w0.shape[1:]), w0.block_size)
    for w in ws[1:]:
        if (w.kind, w.block_size, w.shape[1:]) != (w0.kind, w0.block_size, w0.shape[1:]):
            raise _lib.TpxError("fused q/k/v: weights must share quantization and in-features")
    codes = torch.cat([w.codes for w in ws], 0)
    scales = torch.cat([w.scales for w in ws], 0)
    return QTensor(codes, scales, (codes.shape[0],) + tuple(w0.shape[1:]), w0.qscheme(), w0.block_size)


class LlamaDecoderLayer:
    """torch.classes.tpp_llm.LlamaDecoderLayer (src/csrc/llm/fused_llm_infer.cpp:1071-1287).

    params: [input_ln_gamma, q, k, v, o, post_attention_ln_gamma, gate, up, down, embed_positions] in the
    reference's order (:1096-1110). The linear weights are quantized tensors from remap_and_quantize_*; blocked
    bf16 weights are quantized here when USE_MXFP4 / USE_QINT8 is set, as the reference's constructor does
    (:1122-1161)."""

    def __init__(self, params, layer_idx, eps, H, max_positions, rotary_dim):
        import os
        from . import _qtype
        if len(params) != 10:
            raise _lib.TpxError("LlamaDecoderLayer expects 10 parameters")
        self.Gi, Wq, Wk, Wv, Wp, self.Gpa, Wg, Wu, Wd, self.EP = params
        ws = [Wq, Wk, Wv, Wp, Wg, Wu, Wd]
        if not all(isinstance(w, _qtype.QTensor) for w in ws):
            if os.environ.get("USE_MXFP4", "0") == "1":
                ws = [w if isinstance(w, _qtype.QTensor) else _qtype.remap_and_quantize_mxfp4(w) for w in ws]
            elif os.environ.get("USE_QINT8", "0") == "1":
                ws = [w if isinstance(w, _qtype.QTensor) else _qtype.remap_and_quantize_qint8(w) for w in ws]
            elif all(isinstance(w, torch.Tensor) and w.dtype == torch.bfloat16 for w in ws):
                # unquantized bf16 weights (the reference's default): plain [N, K] matrices for the bf16 kernel
                from ..utils.blocked_layout import unblock_weight
                ws = [unblock_weight(w) if w.dim() == 5 else w.contiguous() for w in ws]
            else:
                raise _lib.TpxError("LlamaDecoderLayer: weights must be all quantized tensors or all bf16 tensors")
        Wq, Wk, Wv, self.Wp, self.Wg, self.Wu, self.Wd = ws
        self.layer_idx, self.eps, self.H = int(layer_idx), float(eps), int(H)
        self.max_positions, self.rotary_dim = int(max_positions), int(rotary_dim)
        self.bf16 = isinstance(Wq, torch.Tensor)
        self.Nq = (Wq.shape[0] if self.bf16 else Wq.out_features) // self.H
        self.Nkv = (Wk.shape[0] if self.bf16 else Wk.out_features) // self.H
        self.Wqkv = torch.cat([Wq, Wk, Wv], 0).contiguous() if self.bf16 else _cat_q([Wq, Wk, Wv])
        self.Bqkv = None  # Qwen2DecoderLayer sets the fused q/k/v bias
        if self.EP.dtype != torch.float32 or tuple(self.EP.shape[:1]) != (2,):
            raise _lib.TpxError("embed_positions must be fp32 [2, max_positions, rotary_dim]")
        self.EP = self.EP.contiguous()
        if not self.bf16:
            for w in (self.Wqkv, self.Wp, self.Wd):
                w.prepare()
            self.Wg.prepare(pair_with=self.Wu)

    def forward(self, inp, cache, use_cache=True, dev_len=None):
        """inp = [hidden_states [B,S,D] bf16, additive mask [B,Spad], position_ids int64 [1 or B, S]]
        (LLMBlock::forward_common / _forward, :531-561, :1195-1286). dev_len: int32 device scalar holding the number
        of cached tokens; when given, kernels read lengths from it (nothing in the call depends on host-side
        lengths, so the step can be recorded in a CUDA graph) and the cache must already have room."""
        from ._tpp_attn import attention
        hs, am, pos = inp[0], inp[1], inp[2]
        _lib.require_cuda(hs, "hidden_states")
        if self._c_level_ok():
            return self._forward_c(hs, am, pos, cache, use_cache, dev_len)
        B, S, D = hs.shape
        ws = get_pg_size()
        scale = 1.0 / ws
        L = _lib.lib()
        res = hs.reshape(B * S, D)
        T = B * S
        sc = _timers.scope

        def wbytes(w):  # bytes a linear has to read for its weight (packed codes + scales, or bf16)
            return w.numel() * 2 if isinstance(w, torch.Tensor) else (w.numel() * 17 // 32 if w.kind == 1 else w.numel() if w.kind == 3 else w.numel() + 4 * w.numel() // w.block_size)

        def nk(w):
            return tuple(w.shape) if isinstance(w, torch.Tensor) else (w.out_features, w.in_features)

        with sc("fqkv_gemm", 2 * T * nk(self.Wqkv)[0] * D, wbytes(self.Wqkv) + 2 * T * (D + nk(self.Wqkv)[0])):
            qkv = fc_plain_norm(res, self.Gi, self.eps, self.Wqkv, self.Bqkv)
        lc = cache.layer(self.layer_idx)
        if dev_len is None:
            lc.ensure(B, self.Nkv, self.H, S, hs.dtype, hs.device)
        R = self.Nq // self.Nkv
        q = torch.empty((B, self.Nkv, S, R, self.H), dtype=hs.dtype, device=hs.device)
        if pos.dtype != torch.int64 or not pos.is_contiguous():
            pos = pos.to(torch.int64).contiguous()
        paged = not lc.contiguous()  # several arenas: the kernels follow the page tables
        kc, vc = (None, None) if paged else lc.arenas[0]
        with sc("rotary", 0, 4 * T * (self.Nq + 2 * self.Nkv) * self.H):
            if paged:
                _lib.check(L.tpx_rope_kv_update_paged(qkv.data_ptr(), self.EP.data_ptr(), pos.data_ptr(), B, S, self.Nq, self.Nkv, self.H,
                                                      self.EP.shape[1], self.EP.shape[2], pos.shape[0], lc.offset, lc.capacity(),
                                                      _lib.ptr(dev_len), q.data_ptr(), lc.k_ptrs.data_ptr(), lc.v_ptrs.data_ptr(), _lib.stream()))
            else:
                _lib.check(L.tpx_rope_kv_update(qkv.data_ptr(), self.EP.data_ptr(), pos.data_ptr(), B, S, self.Nq, self.Nkv, self.H,
                                                self.EP.shape[1], self.EP.shape[2], pos.shape[0], lc.offset, lc.capacity(),
                                                _lib.ptr(dev_len), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), _lib.stream()))
        if dev_len is None:
            lc.offset += S
            key_len = lc.offset
        else:
            key_len = lc.capacity()  # planning maximum; the kernels read the real length from dev_len
        with sc("mha", 4 * T * self.Nq * self.H * key_len // (2 if S > 1 else 1), 4 * B * self.Nkv * self.H * key_len + 4 * T * self.Nq * self.H):
            ctx = attention(q, kc, vc, am, key_len, causal=True, out_bsnrh=True, dev_len=dev_len,
                            pages=(lc.k_ptrs, lc.v_ptrs) if paged else None).view(B * S, self.Nq * self.H)
        with sc("proj_gemm", 2 * T * D * nk(self.Wp)[1], wbytes(self.Wp) + 2 * T * (2 * D + nk(self.Wp)[1])):
            so = fc_plain_act(ctx, self.Wp, res=res, res_scale=scale)
        if ws > 1:
            with sc("allred", 0, 2 * T * D):
                allreduce(so)
        FF = nk(self.Wg)[0]
        with sc("i_gemm", 4 * T * FF * D, wbytes(self.Wg) + wbytes(self.Wu) + 2 * T * (D + FF)):
            inter = fc_gate_up(so, self.Wg, self.Wu, "silu", norm=(self.Gpa, self.eps))
        with sc("o_gemm", 2 * T * FF * D, wbytes(self.Wd) + 2 * T * (2 * D + FF)):
            out = fc_plain_act(inter, self.Wd, res=so, res_scale=scale)
        if ws > 1:
            with sc("allred", 0, 2 * T * D):
                allreduce(out)
        out = out.view(B, S, D)
        if use_cache:  # the cache tensors while they are one arena, else the list of arenas (TppCache.get gathers them)
            if paged:
                return [out, [a[0] for a in lc.arenas], [a[1] for a in lc.arenas]]
            return [out, kc, vc]
        return [out]


    # ----- the same forward as two C calls (tpx_llama_layer_attention / tpx_llama_layer_mlp): one foreign call per half
    # of the layer instead of one per kernel
    def _c_level_ok(self):
        if self.bf16 or _timers.enabled() or _opt("TPX_LAYER_C", "1") == "0" or mxfp4_path() != "tc" or _opt("TPX_FUSED_NORM", "1") == "0":
            return False
        return all(w.kind == 1 for w in (self.Wqkv, self.Wp, self.Wg, self.Wu, self.Wd)) and self.Wqkv.in_features <= 8192

    def _c_struct(self):
        st = getattr(self, "_cstruct", None)
        if st is None:
            L = _lib.LlamaLayerStruct()
            L.D, L.Nq, L.Nkv, L.H = self.Wqkv.in_features, self.Nq, self.Nkv, self.H
            L.FF, L.MP, L.HR = self.Wg.out_features, self.EP.shape[1], self.EP.shape[2]
            L.eps, L.gamma_is_f32 = self.eps, int(self.Gi.dtype == torch.float32)
            if self.Gi.dtype != self.Gpa.dtype:
                raise _lib.TpxError("LlamaDecoderLayer: the two norm weights must share a dtype")
            keep = [self.Wqkv.packed_tc(), self.Wp.packed_tc(), self.Wg.packed_tc(self.Wu), self.Wd.packed_tc()]
            (L.wqkv, L.sfa_qkv), (L.wo, L.sfa_o), (L.wgu, L.sfa_gu), (L.wd, L.sfa_d) = [(a.data_ptr(), b.data_ptr()) for a, b in keep]
            L.gamma1, L.gamma2, L.ep = self.Gi.data_ptr(), self.Gpa.data_ptr(), self.EP.data_ptr()
            L.bias_qkv = self.Bqkv.data_ptr() if self.Bqkv is not None else None
            st = self._cstruct = (L, keep)
        st[0].res_scale = 1.0 / get_pg_size()
        return st[0]

    def _forward_c(self, hs, am, pos, cache, use_cache, dev_len):
        B, S, D = hs.shape
        T = B * S
        L = self._c_struct()
        lib = _lib.lib()
        dev = hs.device
        if not hs.is_contiguous():
            hs = hs.contiguous()
        lc = cache.layer(self.layer_idx)
        if dev_len is None:
            lc.ensure(B, self.Nkv, self.H, S, hs.dtype, dev)
        if pos.dtype != torch.int64 or not pos.is_contiguous():
            pos = pos.to(torch.int64).contiguous()
        H, Nq, Nkv, FF = self.H, self.Nq, self.Nkv, L.FF
        nqkv = (Nq + 2 * Nkv) * H
        # temporaries of one layer live in one cached workspace (layers run one after the other on the stream)
        sizes = [T * nqkv, T * Nq * H, T * Nq * H, T * D, T * FF]
        ws = _lib.layer_workspace(sum(sizes) * 2 + 5 * 256, dev)
        views, o = [], 0
        for n in sizes:
            views.append(ws[o:o + n * 2])
            o += (n * 2 + 255) // 256 * 256
        key = ("layer_c", T, D, nqkv, FF, Nq * H)
        nb = _SCRATCH_BYTES.get(key)
        if nb is None:
            f = lib.tpx_qlinear_mxfp4_tc_scratch_bytes
            nb = _SCRATCH_BYTES[key] = max(f(T, nqkv, D, 0), f(T, D, Nq * H, 0), f(T, FF, D, 1), f(T, D, FF, 0))
        sc = _lib.scratch(nb, dev)
        key_len = lc.capacity() if dev_len is not None else lc.offset + S
        na = lib.tpx_attention_scratch_bytes(B, Nkv, S, Nq // Nkv, H, key_len)
        asc = _lib.aux_scratch(na, dev) if na else None
        out = torch.empty((B, S, D), dtype=hs.dtype, device=dev)
        io = _lib.LlamaLayerIOStruct()
        io.B, io.S, io.Bpos, io.Spad = B, S, pos.shape[0], (am.shape[1] if am is not None else 0)
        io.offset, io.capacity = lc.offset, lc.capacity()
        io.x, io.pos, io.mask, io.dev_len = hs.data_ptr(), pos.data_ptr(), _lib.ptr(am), _lib.ptr(dev_len)
        paged = not lc.contiguous()
        if paged:
            io.k_pages, io.v_pages = lc.k_ptrs.data_ptr(), lc.v_ptrs.data_ptr()
            kc = vc = None
        else:
            kc, vc = lc.arenas[0]
            io.kc, io.vc = kc.data_ptr(), vc.data_ptr()
        io.qkv, io.q, io.ctx, io.so, io.inter = [v.data_ptr() for v in views]
        io.out = out.data_ptr()
        io.scratch, io.scratch_bytes = sc.data_ptr(), sc.numel()
        io.attn_scratch, io.attn_scratch_bytes = _lib.ptr(asc), (asc.numel() if asc is not None else 0)
        if T <= 64 and _opt("TPX_HANDOFF", "1") != "0":  # gate/up hands its output to down as activation terms
            hb = _lib.handoff_buffer(2 * 64 * FF + 4 * FF + 2048, dev)
            io.handoff, io.handoff_bytes = hb.data_ptr(), hb.numel()
        st = _lib.stream()
        world = get_pg_size()
        rc = lib.tpx_llama_layer_attention(ctypes.byref(L), ctypes.byref(io), st)
        if rc:
            _lib.check(rc)
        if dev_len is None:
            lc.offset += S
        if world > 1:
            allreduce(views[3].view(torch.bfloat16).view(T, D))
        rc = lib.tpx_llama_layer_mlp(ctypes.byref(L), ctypes.byref(io), st)
        if rc:
            _lib.check(rc)
        if world > 1:
            allreduce(out)
        if use_cache:
            if paged:
                return [out, [a[0] for a in lc.arenas], [a[1] for a in lc.arenas]]
            return [out, kc, vc]
        return [out]


class Qwen2DecoderLayer(LlamaDecoderLayer):
    """torch.classes.tpp_llm.Qwen2DecoderLayer (src/csrc/llm/fused_llm_infer.cpp:1289-1510): the Llama block with
    biases on the q, k and v projections. params: [input_ln_gamma, q, k, v, o, post_attention_ln_gamma, gate, up,
    down, q_bias, k_bias, v_bias, embed_positions] (:1317-1333)."""

    def __init__(self, params, layer_idx, eps, H, max_positions, rotary_dim):
        if len(params) != 13:
            raise _lib.TpxError("Qwen2DecoderLayer expects 13 parameters")
        bq, bk, bv = params[9:12]
        super().__init__(list(params[:9]) + [params[12]], layer_idx, eps, H, max_positions, rotary_dim)
        for b, n in ((bq, self.Nq * self.H), (bk, self.Nkv * self.H), (bv, self.Nkv * self.H)):
            if b.numel() != n:
                raise _lib.TpxError("Qwen2DecoderLayer: bias length does not match its projection")
        self.Bqkv = torch.cat([bq.reshape(-1), bk.reshape(-1), bv.reshape(-1)]).to(self.EP.device, torch.bfloat16).contiguous()


class OPTDecoderLayer:
    """torch.classes.tpp_llm.OPTDecoderLayer (src/csrc/llm/fused_llm_infer.cpp:850-1069).

    params, in the reference's order (:877-898): [ln1_gamma, ln1_beta, ln2_gamma, ln2_beta, q, q_bias, k, k_bias, v,
    v_bias, out_proj, out_bias, fc1, fc1_bias, fc2, fc2_bias]; the linear weights are quantized tensors (or blocked bf16
    with USE_MXFP4 / USE_QINT8 set, or all plain bf16). No rotary embedding: positions enter through the model's
    learned position embedding before the first layer."""

    def __init__(self, params, layer_idx, eps1, eps2, H, do_layer_norm_before):
        import os
        from . import _qtype
        if len(params) != 16:
            raise _lib.TpxError("OPTDecoderLayer expects 16 parameters")
        (self.G1, self.B1, self.G2, self.B2, Wq, Bq, Wk, Bk, Wv, Bv, Wp, self.Bp, Wi, self.Bi, Wo, self.Bo) = params
        ws = [Wq, Wk, Wv, Wp, Wi, Wo]
        if not all(isinstance(w, _qtype.QTensor) for w in ws):
            if os.environ.get("USE_MXFP4", "0") == "1":
                ws = [w if isinstance(w, _qtype.QTensor) else _qtype.remap_and_quantize_mxfp4(w) for w in ws]
            elif os.environ.get("USE_QINT8", "0") == "1":
                ws = [w if isinstance(w, _qtype.QTensor) else _qtype.remap_and_quantize_qint8(w) for w in ws]
            elif all(isinstance(w, torch.Tensor) and w.dtype == torch.bfloat16 for w in ws):
                from ..utils.blocked_layout import unblock_weight
                ws = [unblock_weight(w) if w.dim() == 5 else w.contiguous() for w in ws]
            else:
                raise _lib.TpxError("OPTDecoderLayer: weights must be all quantized tensors or all bf16 tensors")
        Wq, Wk, Wv, self.Wp, self.Wi, self.Wo = ws
        self.layer_idx, self.eps1, self.eps2, self.H = int(layer_idx), float(eps1), float(eps2), int(H)
        self.do_layer_norm_before = bool(do_layer_norm_before)
        self.bf16 = isinstance(Wq, torch.Tensor)
        self.Nq = self.Nkv = (Wq.shape[0] if self.bf16 else Wq.out_features) // self.H
        self.Wqkv = torch.cat([Wq, Wk, Wv], 0).contiguous() if self.bf16 else _cat_q([Wq, Wk, Wv])
        dev = self.G1.device
        self.Bqkv = torch.cat([Bq.reshape(-1), Bk.reshape(-1), Bv.reshape(-1)]).to(dev, torch.bfloat16).contiguous()
        self.Bp, self.Bi, self.Bo = (b.to(dev, torch.bfloat16).contiguous() for b in (self.Bp, self.Bi, self.Bo))
        # the rotary kernel also appends k and v to the cache and lays q out for attention; with an empty table
        # (max_positions 0) it rotates nothing
        self._no_rope = torch.zeros((2, 1, self.H), dtype=torch.float32, device=dev)
        if not self.bf16:
            for w in (self.Wqkv, self.Wp, self.Wi, self.Wo):
                w.prepare()

    def forward(self, inp, cache, use_cache=True, dev_len=None):
        """inp = [hidden_states [B,S,D] bf16, additive mask [B,Spad]] (OPTDecoderLayer::_forward, :978-1068); a third
        element (position ids), if present, is ignored."""
        from ._tpp_attn import attention
        hs, am = inp[0], inp[1]
        _lib.require_cuda(hs, "hidden_states")
        B, S, D = hs.shape
        ws = get_pg_size()
        scale = 1.0 / ws
        L = _lib.lib()
        res = hs.reshape(B * S, D)
        sc = _timers.scope
        x = layer_norm(res, self.G1, self.B1, self.eps1) if self.do_layer_norm_before else res
        with sc("qkv_gemm", 0, 0):
            qkv = fc_plain(x, self.Wqkv, self.Bqkv)
        lc = cache.layer(self.layer_idx)
        if dev_len is None:
            lc.ensure(B, self.Nkv, self.H, S, hs.dtype, hs.device)
        q = torch.empty((B, self.Nkv, S, 1, self.H), dtype=hs.dtype, device=hs.device)
        pos = torch.zeros((1, S), dtype=torch.int64, device=hs.device)
        paged = not lc.contiguous()
        kc, vc = (None, None) if paged else lc.arenas[0]
        if paged:
            _lib.check(L.tpx_rope_kv_update_paged(qkv.data_ptr(), self._no_rope.data_ptr(), pos.data_ptr(), B, S, self.Nq, self.Nkv, self.H,
                                                  0, self.H, 1, lc.offset, lc.capacity(), _lib.ptr(dev_len), q.data_ptr(),
                                                  lc.k_ptrs.data_ptr(), lc.v_ptrs.data_ptr(), _lib.stream()))
        else:
            _lib.check(L.tpx_rope_kv_update(qkv.data_ptr(), self._no_rope.data_ptr(), pos.data_ptr(), B, S, self.Nq, self.Nkv, self.H,
                                            0, self.H, 1, lc.offset, lc.capacity(), _lib.ptr(dev_len), q.data_ptr(), kc.data_ptr(),
                                            vc.data_ptr(), _lib.stream()))
        if dev_len is None:
            lc.offset += S
            key_len = lc.offset
        else:
            key_len = lc.capacity()
        with sc("mha", 0, 0):
            ctx = attention(q, kc, vc, am, key_len, causal=True, out_bsnrh=True, dev_len=dev_len,
                            pages=(lc.k_ptrs, lc.v_ptrs) if paged else None).view(B * S, self.Nq * self.H)
        with sc("proj_gemm", 0, 0):
            so = fc_plain_act(ctx, self.Wp, self.Bp, res=res, res_scale=scale)
        if ws > 1:
            allreduce(so)
        if not self.do_layer_norm_before:
            so = layer_norm(so, self.G1, self.B1, self.eps1)
        x = layer_norm(so, self.G2, self.B2, self.eps2) if self.do_layer_norm_before else so
        with sc("i_gemm", 0, 0):
            inter = fc_plain_act(x, self.Wi, self.Bi, "relu")
        with sc("o_gemm", 0, 0):
            out = fc_plain_act(inter, self.Wo, self.Bo, res=so, res_scale=scale)
        if ws > 1:
            allreduce(out)
        if not self.do_layer_norm_before:
            out = layer_norm(out, self.G2, self.B2, self.eps2)
        out = out.view(B, S, D)
        if use_cache:
            if paged:
                return [out, [a[0] for a in lc.arenas], [a[1] for a in lc.arenas]]
            return [out, kc, vc]
        return [out]


class GPTJBlock:
    """torch.classes.tpp_llm.GPTJBlock (src/csrc/llm/fused_llm_infer.cpp:607-848).

    params, in the reference's order (:636-652): [ln_gamma, ln_beta, q, k, v, out_proj, fc_in, fc_in_bias, fc_out,
    fc_out_bias, embed_positions]; embed_positions is fp32 [max_positions, rotary_dim] (sines, then cosines). One
    LayerNorm feeds the attention and the MLP, which run side by side; the block's output is
    fc_out(gelu(fc_in(x))) + out_proj(attention) + residual / world, followed by ONE all-reduce."""

    def __init__(self, params, layer_idx, eps, H, max_positions, rotary_dim):
        import os
        from . import _qtype
        if len(params) != 11:
            raise _lib.TpxError("GPTJBlock expects 11 parameters")
        self.G, self.B, Wq, Wk, Wv, Wp, Wi, Bi, Wo, Bo, self.EP = params
        ws = [Wq, Wk, Wv, Wp, Wi, Wo]
        if not all(isinstance(w, _qtype.QTensor) for w in ws):
            if os.environ.get("USE_MXFP4", "0") == "1":
                ws = [w if isinstance(w, _qtype.QTensor) else _qtype.remap_and_quantize_mxfp4(w) for w in ws]
            elif os.environ.get("USE_QINT8", "0") == "1":
                ws = [w if isinstance(w, _qtype.QTensor) else _qtype.remap_and_quantize_qint8(w) for w in ws]
            elif all(isinstance(w, torch.Tensor) and w.dtype == torch.bfloat16 for w in ws):
                from ..utils.blocked_layout import unblock_weight
                ws = [unblock_weight(w) if w.dim() == 5 else w.contiguous() for w in ws]
            else:
                raise _lib.TpxError("GPTJBlock: weights must be all quantized tensors or all bf16 tensors")
        Wq, Wk, Wv, self.Wp, self.Wi, self.Wo = ws
        self.layer_idx, self.eps, self.H = int(layer_idx), float(eps), int(H)
        self.max_positions, self.rotary_dim = int(max_positions), int(rotary_dim)
        self.bf16 = isinstance(Wq, torch.Tensor)
        self.Nq = self.Nkv = (Wq.shape[0] if self.bf16 else Wq.out_features) // self.H
        self.Wqkv = torch.cat([Wq, Wk, Wv], 0).contiguous() if self.bf16 else _cat_q([Wq, Wk, Wv])
        dev = self.G.device
        self.Bi, self.Bo = Bi.to(dev, torch.bfloat16).contiguous(), Bo.to(dev, torch.bfloat16).contiguous()
        if self.EP.dtype != torch.float32 or self.EP.dim() != 2 or self.EP.shape[1] != self.rotary_dim:
            raise _lib.TpxError("embed_positions must be fp32 [max_positions, rotary_dim]")
        self.EP = self.EP.contiguous()
        if not self.bf16:
            for w in (self.Wqkv, self.Wp, self.Wi, self.Wo):
                w.prepare()

    def forward(self, inp, cache, use_cache=True, dev_len=None):
        """inp = [hidden_states [B,S,D] bf16, additive mask [B,Spad], position_ids int64 [1 or B, S]]."""
        from ._tpp_attn import attention
        hs, am, pos = inp[0], inp[1], inp[2]
        _lib.require_cuda(hs, "hidden_states")
        B, S, D = hs.shape
        ws = get_pg_size()
        L = _lib.lib()
        res = hs.reshape(B * S, D)
        x = layer_norm(res, self.G, self.B, self.eps)
        qkv = fc_plain(x, self.Wqkv)
        inter = fc_plain_act(x, self.Wi, self.Bi, "gelu")
        lc = cache.layer(self.layer_idx)
        if dev_len is None:
            lc.ensure(B, self.Nkv, self.H, S, hs.dtype, hs.device)
        q = torch.empty((B, self.Nkv, S, 1, self.H), dtype=hs.dtype, device=hs.device)
        if pos.dtype != torch.int64 or not pos.is_contiguous():
            pos = pos.to(torch.int64).contiguous()
        paged = not lc.contiguous()
        kc, vc = (None, None) if paged else lc.arenas[0]
        _lib.check(L.tpx_rope_kv_update_gptj(qkv.data_ptr(), self.EP.data_ptr(), pos.data_ptr(), B, S, self.Nq, self.Nkv, self.H,
                                             self.EP.shape[0], self.rotary_dim, pos.shape[0], lc.offset, lc.capacity(), _lib.ptr(dev_len),
                                             q.data_ptr(), _lib.ptr(kc), _lib.ptr(vc),
                                             lc.k_ptrs.data_ptr() if paged else None, lc.v_ptrs.data_ptr() if paged else None, _lib.stream()))
        if dev_len is None:
            lc.offset += S
            key_len = lc.offset
        else:
            key_len = lc.capacity()
        ctx = attention(q, kc, vc, am, key_len, causal=True, out_bsnrh=True, dev_len=dev_len,
                        pages=(lc.k_ptrs, lc.v_ptrs) if paged else None).view(B * S, self.Nq * self.H)
        so = fc_plain_act(ctx, self.Wp, res=res, res_scale=1.0 / ws)   # out_proj + residual / world
        out = fc_plain_act(inter, self.Wo, self.Bo, res=so, res_scale=1.0)  # fc_out + bias + (attention + residual)
        if ws > 1:
            allreduce(out)
        out = out.view(B, S, D)
        if use_cache:
            if paged:
                return [out, [a[0] for a in lc.arenas], [a[1] for a in lc.arenas]]
            return [out, kc, vc]
        return [out]
