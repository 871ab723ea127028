"""Mirror of the reference's `_C._qtype` submodule (src/csrc/qtypes.cpp:1075-1093) on CUDA.

The reference returns torch quantized tensors carried by a custom `at::Quantizer`
(src/csrc/qtypes.h:30-410). Those carriers cannot live on a CUDA device without the reference's
C++ classes, so the same information travels in a small Python object, `QTensor`: the code bytes
and the per-block scales in exactly the reference's storage layout, plus the quantizer's
attributes (`qscheme`, `block_size`, `axis`, `pack_size`). `QTensor.packed()` lazily re-lays the
weight into the streaming layout the kernels read."""
import ctypes

import torch

from .. import _lib

W_MXFP4, W_INT8, W_FP8 = 1, 2, 3
kPerBlockMxFP = "per_block_mxfp"      # at::kPerBlockMxFP, src/csrc/qtypes.h:12
kPerBlockAffine = "per_block_affine"  # at::kPerBlockAffine, src/csrc/qtypes.h:11


class QTensor:
    is_quantized = True

    def __init__(self, codes, scales, shape, qscheme, block_size, axis=2, is_vnni=True):
        self.codes = codes      # uint8 [K1,C1,C2,K2] (mxfp4, two codes per byte) or int8 [K1,C1,C2,K2,4]
        self.scales = scales    # uint8 [K1,C1,C2/16,K2] or fp32 [K1,C1,1,K2]
        self.shape = tuple(shape)  # logical 5-D shape, as Tensor.sizes() of the reference tensor
        self._qscheme = qscheme
        self.block_size = int(block_size)
        self.axis = axis
        self.is_vnni = is_vnni
        self._packed = None
        self._packed_tc = None

    # --- the attributes the reference's dispatch reads (src/csrc/fused_gemm.h:1517-1540)
    def qscheme(self):
        return self._qscheme

    @property
    def dtype(self):
        return torch.quint4x2 if self._qscheme == kPerBlockMxFP else torch.qint8

    @property
    def device(self):
        return self.codes.device

    def size(self, dim=None):
        return self.shape if dim is None else self.shape[dim]

    def dim(self):
        return len(self.shape)

    def numel(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def kind(self):
        return W_MXFP4 if self._qscheme == kPerBlockMxFP else W_INT8

    @property
    def out_features(self):
        return self.shape[0] * self.shape[3]

    @property
    def in_features(self):
        return self.shape[1] * self.shape[2] * self.shape[4]

    def dequantize(self):
        """fp32 tensor of the same 5-D shape (Tensor.dequantize(), src/csrc/qtypes.cpp:438-445, :521-529)."""
        K1, C1, C2, K2, _ = self.shape
        out = torch.empty(self.shape, dtype=torch.float32, device=self.codes.device)
        L = _lib.lib()
        with torch.cuda.device(self.codes.device):
            if self.kind == W_MXFP4:
                _lib.check(L.tpx_dequantize_mxfp4(self.codes.data_ptr(), self.scales.data_ptr(), K1, C1, C2, K2,
                                                  out.data_ptr(), _lib.stream()))
            else:
                _lib.check(L.tpx_dequantize_qint8(self.codes.data_ptr(), self.scales.data_ptr(), K1, C1, C2, K2,
                                                  out.data_ptr(), _lib.stream()))
        return out

    def packed(self, drop_interchange=False):
        """(codes, scales) in the streaming layout; built once and cached."""
        if self._packed is None:
            L = _lib.lib()
            N, K = self.out_features, self.in_features
            cb, sb = ctypes.c_size_t(), ctypes.c_size_t()
            _lib.check(L.tpx_packed_bytes(self.kind, N, K, self.block_size, ctypes.byref(cb), ctypes.byref(sb)))
            dev = self.codes.device
            pc = torch.empty(cb.value, dtype=torch.uint8, device=dev)
            with torch.cuda.device(dev):
                if self.kind == W_MXFP4:
                    if self.shape[2] * self.shape[4] != 64 or self.shape[3] != 32:
                        raise _lib.TpxError("MXFP4 repack expects the [N/32, K/64, 32, 32, 2] layout of remap_and_quantize_mxfp4")
                    ps = torch.empty(0, dtype=torch.uint8, device=dev)  # the scales ride inside the tiles
                    _lib.check(L.tpx_repack_mxfp4(self.codes.data_ptr(), self.scales.data_ptr(), N, K, pc.data_ptr(),
                                                  None, _lib.stream()))
                else:
                    if self.shape[3] != 16:
                        raise _lib.TpxError("int8 repack expects K2 == 16")
                    ps = torch.empty(sb.value // 4, dtype=torch.float32, device=dev)
                    _lib.check(L.tpx_repack_qint8(self.codes.data_ptr(), self.scales.data_ptr(), N, K, self.block_size,
                                                  pc.data_ptr(), ps.data_ptr(), _lib.stream()))
            self._packed = (pc, ps)
        if drop_interchange:
            self.codes = self.codes.new_empty(0)
        return self._packed


def _packed_i8tc(self):
    """(wq, swT) of an int8 weight for the tensor-core int8 linear: the plain int8 matrix padded to 128 x 128 tiles and
    feature-contiguous scales; built once and cached."""
    if self.kind == W_MXFP4:
        raise _lib.TpxError("the int8 tensor-core path takes int8 weights")
    hit = getattr(self, "_i8tc", None)
    if hit is not None:
        return hit
    if self.codes.numel() == 0:
        raise _lib.TpxError("the interchange tensors of this weight were dropped before it was packed for this use")
    L = _lib.lib()
    N, K = self.out_features, self.in_features
    wb, sb = ctypes.c_size_t(), ctypes.c_size_t()
    _lib.check(L.tpx_tc_packed_bytes_qint8(N, K, self.block_size, ctypes.byref(wb), ctypes.byref(sb)))
    dev = self.codes.device
    wq = torch.empty(wb.value, dtype=torch.int8, device=dev)
    sw = torch.empty(sb.value // 4, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(L.tpx_repack_qint8_tc(self.codes.data_ptr(), self.scales.data_ptr(), N, K, self.block_size, wq.data_ptr(),
                                         sw.data_ptr(), _lib.stream()))
    self._i8tc = (wq, sw)
    return self._i8tc


def _packed_tc(self, other=None):
    """(wq, sfa) in the tensor-core layout (MXFP4 only), built once and cached. With `other` (the up
    projection of a SwiGLU pair, `self` being the gate) the two weights are packed tile by tile side by
    side, which lets the kernel fetch a gate/up pair of tiles with one copy request."""
    if self.kind != W_MXFP4 or self.shape[2] * self.shape[4] != 64 or self.shape[3] != 32:
        raise _lib.TpxError("the tensor-core path takes MXFP4 weights in the [N/32, K/64, 32, 32, 2] layout")
    if other is None:
        if self._packed_tc is not None:
            return self._packed_tc
    else:
        hit = getattr(self, "_pair_tc", None)
        if hit is not None and hit[0] is other:
            return hit[1]
    if self.codes.numel() == 0 or (other is not None and other.codes.numel() == 0):
        raise _lib.TpxError("the interchange tensors of this weight were dropped before it was packed for this use")
    L = _lib.lib()
    N, K = self.out_features, self.in_features
    wb, sb = ctypes.c_size_t(), ctypes.c_size_t()
    _lib.check(L.tpx_tc_packed_bytes(N, K, int(other is not None), ctypes.byref(wb), ctypes.byref(sb)))
    dev = self.codes.device
    wq = torch.empty(wb.value, dtype=torch.uint8, device=dev)
    sfa = torch.empty(sb.value, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(L.tpx_repack_mxfp4_tc(self.codes.data_ptr(), self.scales.data_ptr(),
                                         other.codes.data_ptr() if other is not None else None,
                                         other.scales.data_ptr() if other is not None else None,
                                         N, K, wq.data_ptr(), sfa.data_ptr(), _lib.stream()))
    if other is None:
        self._packed_tc = (wq, sfa)
    else:
        self._pair_tc = (other, (wq, sfa))
    return (wq, sfa)


QTensor.packed_tc = _packed_tc
QTensor.packed_i8tc = _packed_i8tc


def _state(self):
    """Everything needed to use this weight again without quantizing or repacking: the quantizer's attributes, the
    interchange tensors (possibly already dropped) and every kernel layout built so far, on the CPU. What
    BlockedParameter's state-dict hooks do for blocked weights in the reference
    (src/tpp_pytorch_extension/utils/blocked_layout.py:309-364), for quantized and packed ones."""
    cpu = lambda t: None if t is None else t.detach().cpu()
    pair = getattr(self, "_pair_tc", None)
    i8 = getattr(self, "_i8tc", None)
    return {"shape": self.shape, "qscheme": self._qscheme, "block_size": self.block_size, "axis": self.axis, "is_vnni": self.is_vnni,
            "codes": cpu(self.codes), "scales": cpu(self.scales),
            "packed": None if self._packed is None else tuple(cpu(t) for t in self._packed),
            "packed_tc": None if self._packed_tc is None else tuple(cpu(t) for t in self._packed_tc),
            "pair_tc": None if pair is None else tuple(cpu(t) for t in pair[1]),
            "i8tc": None if i8 is None else tuple(cpu(t) for t in i8)}


def _from_state(st, device, pair_with=None):
    """Inverse of QTensor.state(). `pair_with`: the up-projection object this gate weight was packed with (the pair
    layout is looked up by that object's identity)."""
    dev = lambda t: None if t is None else t.to(device)
    if st.get("fp8"):
        q = Fp8Weight.__new__(Fp8Weight)
        QTensor.__init__(q, dev(st["codes"]), dev(st["scales"]), st["shape"], st["qscheme"], 0, st["axis"], st["is_vnni"])
        q.fmt = st["fp8"]
    else:
        q = QTensor(dev(st["codes"]), dev(st["scales"]), st["shape"], st["qscheme"], st["block_size"], st["axis"], st["is_vnni"])
    if st["packed"] is not None:
        q._packed = tuple(dev(t) for t in st["packed"])
    if st["packed_tc"] is not None:
        q._packed_tc = tuple(dev(t) for t in st["packed_tc"])
    if st["i8tc"] is not None:
        q._i8tc = tuple(dev(t) for t in st["i8tc"])
    if st["pair_tc"] is not None:
        if pair_with is None:
            raise _lib.TpxError("this weight was packed as the gate of a gate/up pair: pass the up projection")
        q._pair_tc = (pair_with, tuple(dev(t) for t in st["pair_tc"]))
    return q


QTensor.state = _state
QTensor.from_state = staticmethod(_from_state)


FP8_E4M3, FP8_E5M2 = 1, 2  # TPX_FP8_E4M3 / TPX_FP8_E5M2 of the C interface
FP8_DTYPES = {"hfloat8": torch.float8_e4m3fn, "bfloat8": torch.float8_e5m2,
              "float8_e4m3fn": torch.float8_e4m3fn, "float8_e5m2": torch.float8_e5m2}


class Fp8Weight(QTensor):
    """A linear weight held as 8-bit floating point, plain [N, K]: what `weight.data.to(bfloat8 | hfloat8)` leaves behind
    in the reference (src/tpp_pytorch_extension/llm/llm_common.py:519-522; the dtypes come from the reference's own
    PyTorch build). bfloat8 is E5M2 (torch.float8_e5m2), hfloat8 is E4M3 (torch.float8_e4m3fn); the cast rounds to
    nearest even and there are no scales. `codes` holds the bytes; the tensor-core layout is built by packed_tc()."""
    is_quantized = False

    def __init__(self, data):
        if data.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2) or data.dim() != 2:
            raise _lib.TpxError("Fp8Weight: a [N, K] tensor of torch.float8_e4m3fn or torch.float8_e5m2 expected")
        N, K = data.shape
        if N % 32 or K % 64:
            raise _lib.TpxError("8-bit floating-point weights need out-features % 32 == 0 and in-features % 64 == 0")
        self.fmt = FP8_E4M3 if data.dtype == torch.float8_e4m3fn else FP8_E5M2
        codes = data.contiguous().view(torch.uint8)
        super().__init__(codes, codes.new_empty(0), (N, K), "fp8_e4m3" if self.fmt == FP8_E4M3 else "fp8_e5m2", 0, axis=1, is_vnni=False)

    kind = W_FP8

    @property
    def dtype(self):
        return torch.float8_e4m3fn if self.fmt == FP8_E4M3 else torch.float8_e5m2

    @property
    def out_features(self):
        return self.shape[0]

    @property
    def in_features(self):
        return self.shape[1]

    def dequantize(self):
        return self.codes.view(self.dtype).float()

    def packed(self, drop_interchange=False):
        raise _lib.TpxError("8-bit floating-point weights run on the tensor-core path only")

    def packed_i8tc(self):
        raise _lib.TpxError("the int8 tensor-core path takes int8 weights")

    def packed_tc(self, other=None):
        """(wq, sfa) of tpx_repack_fp8_tc, built once and cached; `other`: the up projection of a gate/up pair."""
        if other is None:
            if self._packed_tc is not None:
                return self._packed_tc
        else:
            hit = getattr(self, "_pair_tc", None)
            if hit is not None and hit[0] is other:
                return hit[1]
            if not isinstance(other, Fp8Weight) or other.fmt != self.fmt or other.shape != self.shape:
                raise _lib.TpxError("gate/up weights must have the same shape and format")
        if self.codes.numel() == 0 or (other is not None and other.codes.numel() == 0):
            raise _lib.TpxError("the bytes of this weight were dropped before it was packed for this use")
        L = _lib.lib()
        N, K = self.shape
        wb, sb = ctypes.c_size_t(), ctypes.c_size_t()
        _lib.check(L.tpx_fp8_tc_packed_bytes(N, K, int(other is not None), ctypes.byref(wb), ctypes.byref(sb)))
        dev = self.codes.device
        wq = torch.empty(wb.value, dtype=torch.uint8, device=dev)
        sfa = torch.empty(sb.value, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(L.tpx_repack_fp8_tc(self.codes.data_ptr(), other.codes.data_ptr() if other is not None else None, N, K,
                                           wq.data_ptr(), sfa.data_ptr(), _lib.stream()))
        if other is None:
            self._packed_tc = (wq, sfa)
        else:
            self._pair_tc = (other, (wq, sfa))
        return (wq, sfa)

    def prepare(self, drop_interchange=False, pair_with=None):
        self.packed_tc(pair_with)
        if drop_interchange:
            self.codes = self.codes.new_empty(0)
            if pair_with is not None:
                pair_with.codes = pair_with.codes.new_empty(0)
        return self

    def state(self):
        st = _state(self)
        st["fp8"] = self.fmt
        return st


def to_fp8_weight(w, weight_dtype):
    """[N, K] weight (any floating dtype, or already 8-bit) -> Fp8Weight in the named format ("bfloat8" | "hfloat8" or a
    torch float8 dtype). The values pass through bf16 first, as the reference's do (the layer dtype)."""
    dt = FP8_DTYPES.get(weight_dtype, weight_dtype) if isinstance(weight_dtype, str) else weight_dtype
    if dt not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise _lib.TpxError(f"unknown 8-bit floating-point format {weight_dtype}")
    _lib.require_cuda(w, "weight")
    if w.dtype != dt:
        w = w.to(torch.bfloat16).to(dt)
    return Fp8Weight(w)


def _prepare(self, drop_interchange=False, pair_with=None):
    """Build the device layout of the kernel family in use now (`pair_with`: this weight is the gate of a
    gate/up pair and is only used that way); optionally free the interchange copy (dequantize() and the
    other layouts are then no longer available)."""
    from ._fused_llm_infer import mxfp4_path
    if self.kind == W_MXFP4 and mxfp4_path() == "tc":
        self.packed_tc(pair_with)
    else:
        self.packed()
        if pair_with is not None:
            pair_with.packed()
        if self.kind != W_MXFP4:  # int8: the decode kernel of the tensor-core family reads its own layout
            from ._fused_llm_infer import int8_path
            if int8_path() == "tc":
                self.packed_i8tc()
                if pair_with is not None:
                    pair_with.packed_i8tc()
    if drop_interchange:
        self.codes = self.codes.new_empty(0)
        if pair_with is not None:
            pair_with.codes = pair_with.codes.new_empty(0)
    return self


QTensor.prepare = _prepare


def _as_blocked_bf16(t):
    _lib.require_cuda(t, "weight")
    if t.dim() != 5:
        raise _lib.TpxError("expected a 5-D blocked weight [K1, C1, C2, K2, C3] (BlockedParameter.block())")
    if t.dtype != torch.bfloat16:
        raise _lib.TpxError("Unsupported input type for quantization: expected bfloat16")
    return t


def remap_and_quantize_mxfp4(t):
    """src/csrc/qtypes.cpp:783-864. `t`: blocked bf16 weight [K1, C1, C2, K2, 2] on a CUDA device."""
    t = _as_blocked_bf16(t)
    K1, C1, C2, K2, C3 = t.shape
    if not ((K2 <= 32 and 32 % K2 == 0 and K1 % (32 // K2) == 0) or (K2 > 32 and K2 % 32 == 0)):
        raise _lib.TpxError("Shape not compatible for MXFP4")
    K1o = K1 * K2 // 32
    codes = torch.empty((K1o, C1, C2, 32), dtype=torch.uint8, device=t.device)
    scales = torch.empty((K1o, C1, C2 * C3 // 32, 32), dtype=torch.uint8, device=t.device)
    with torch.cuda.device(t.device):
        _lib.check(_lib.lib().tpx_remap_and_quantize_mxfp4(t.data_ptr(), K1, C1, C2, K2, C3, codes.data_ptr(),
                                                           scales.data_ptr(), _lib.stream()))
    return QTensor(codes, scales, (K1o, C1, C2, 32, C3), kPerBlockMxFP, 32)


def qint8_block_size_used(C, own_block, block_size):
    """The block size remap_and_quantize_qint8 ends up with (src/csrc/qtypes.cpp:878-889): the requested one if it
    divides the in-features C; else the largest power of two from 4096 down to 64 that is smaller than the request and
    divides C; else the blocked tensor's own inner block C2*C3."""
    if block_size < 4 or block_size % 4:
        raise _lib.TpxError(f"remap_and_quantize_qint8: block size {block_size} must be a positive multiple of 4")
    if C % block_size == 0:
        return block_size
    qbs = 4096
    while qbs >= 64:
        if block_size > qbs and C % qbs == 0:
            return qbs
        qbs //= 2
    return own_block


def remap_and_quantize_qint8(t, block_size=None):
    """src/csrc/qtypes.cpp:866-932. `block_size` defaults to the QINT8_BLOCK_SIZE environment
    variable (256 if unset), as in the reference (:28)."""
    import os
    t = _as_blocked_bf16(t)
    if block_size is None:
        block_size = int(os.environ.get("QINT8_BLOCK_SIZE", "256"))
    K1, C1, C2, K2, C3 = t.shape
    C = C1 * C2 * C3
    B = qint8_block_size_used(C, C2 * C3, int(block_size))
    used = ctypes.c_int64(0)
    q = torch.empty(K1 * C * K2, dtype=torch.int8, device=t.device)
    scales = torch.empty(K1 * (C // B) * K2, dtype=torch.float32, device=t.device)
    with torch.cuda.device(t.device):
        _lib.check(_lib.lib().tpx_remap_and_quantize_qint8(t.data_ptr(), K1, C1, C2, K2, C3, block_size, q.data_ptr(),
                                                           scales.data_ptr(), scales.numel(), ctypes.byref(used), _lib.stream()))
    if used.value != B:
        raise _lib.TpxError(f"remap_and_quantize_qint8: the library used block size {used.value}, the host computed {B}")
    q = q.view(K1, C // B, B // 4, K2, 4)
    scales = scales[: K1 * (C // B) * K2].view(K1, C // B, 1, K2)
    return QTensor(q, scales, (K1, C // B, B // 4, K2, 4), kPerBlockAffine, B)


class QInt2Tensor(QTensor):
    """Carrier of remap_and_quantize_qint2_intlv (src/csrc/qtypes.cpp:1004-1073): ternary codes (0, +1, and 2 for -1), four
    to a byte, with one fp32 scale per output row and block of in-features. `codes` is uint8 [K1, C1, C2, K2, 4]: the
    byte at (k1, c1, c2, k2, c3) holds, in bit pairs 2*k3, the codes of rows 32*k1 + 8*k3 + k2 (K2 = 8, four row groups
    interleaved) at column c1*B + 4*c2 + c3; `scales` is fp32 [K1, C1, 32, 1]; the logical shape is [K1, C1, C2, 32, 4].
    The reference multiplies such weights through the same int8 GEMM class as qint8 (TppBlockedQInt8LinearW,
    src/csrc/fused_gemm.h:1531-1535): here the codes are expanded once to the int8 carrier (values -1, 0, +1, same scales and
    block size) and run on the int8 kernels, so the weight streams at one byte per element."""

    def __init__(self, codes, scales, shape, block_size):
        super().__init__(codes, scales, shape, kPerBlockAffine, block_size)
        self._twin = None

    @property
    def dtype(self):
        return torch.quint2x4

    def plain_codes(self):
        """int8 [N, K] with values -1, 0, +1."""
        K1, C1, C2, R, C3 = self.shape
        K2 = R // 4
        c = self.codes.view(K1, C1, C2, K2, C3)
        parts = [((c >> (2 * k3)) & 3) for k3 in range(4)]          # each [K1, C1, C2, K2, C3]
        q = torch.stack(parts, 3).to(torch.int8)                     # [K1, C1, C2, K3, K2, C3]
        q = torch.where(q == 2, torch.full_like(q, -1), q)
        return q.permute(0, 3, 4, 1, 2, 5).reshape(K1 * R, C1 * C2 * C3).contiguous()

    def plain_scales(self):
        """fp32 [N, K / block_size]."""
        K1, C1, C2, R, C3 = self.shape
        return self.scales.view(K1, C1, R).permute(0, 2, 1).reshape(K1 * R, C1).contiguous()

    def dequantize(self):
        """fp32 [N, K] (plain, not blocked)."""
        B = self.block_size
        return (self.plain_codes().float().view(self.out_features, -1, B) * self.plain_scales().unsqueeze(-1)).view(self.out_features, -1)

    def as_int8(self):
        """The same weight in the int8 carrier of remap_and_quantize_qint8 (16 rows per group), built once."""
        if self._twin is None:
            if self.codes.numel() == 0:
                raise _lib.TpxError("the interchange tensors of this weight were dropped before it was expanded")
            N, K, B = self.out_features, self.in_features, self.block_size
            q = self.plain_codes().view(N // 16, 16, K // B, B // 4, 4).permute(0, 2, 3, 1, 4).contiguous()
            sc = self.plain_scales().view(N // 16, 16, K // B).permute(0, 2, 1).contiguous().view(N // 16, K // B, 1, 16)
            self._twin = QTensor(q, sc, (N // 16, K // B, B // 4, 16, 4), kPerBlockAffine, B)
        return self._twin

    def packed(self, drop_interchange=False):
        return self.as_int8().packed(drop_interchange)

    def packed_i8tc(self):
        return self.as_int8().packed_i8tc()

    def packed_tc(self, other=None):
        raise _lib.TpxError("the MXFP4 tensor-core path takes MXFP4 weights")

    def prepare(self, drop_interchange=False, pair_with=None):
        self.as_int8().prepare(drop_interchange, pair_with.as_int8() if pair_with is not None else None)
        if drop_interchange:
            self.codes = self.codes.new_empty(0)
            if pair_with is not None:
                pair_with.codes = pair_with.codes.new_empty(0)
        return self

    def state(self):
        raise _lib.TpxError("packed checkpoints of qint2 weights are not supported")


def qint2_block_size_used(C, own_block, block_size):
    """Block size remap_and_quantize_qint2_intlv ends up with (src/csrc/qtypes.cpp:1033-1044): the requested one if it
    divides the in-features; else the largest power of two from 4096 down to 64 below the request that does; else the
    blocked tensor's own inner block."""
    if C % block_size == 0:
        return block_size
    qbs = 4096
    while qbs >= 64:
        if block_size > qbs and C % qbs == 0:
            return qbs
        qbs //= 2
    return own_block


def remap_and_quantize_qint2_intlv(t, block_size=None):
    """src/csrc/qtypes.cpp:1004-1073 for a blocked bf16 weight [K1, C1, C2, K2, 2] on a CUDA device whose out-features
    are a multiple of 32 (the K2 = 8, K3 = 4 case of the reference). `block_size` defaults to QINT2_BLOCK_SIZE (256).
    The same sequence of tensor operations as the reference: per (row, block) scale = max |w| (at least 1e-8), code =
    round(w / scale) clamped to [-1, 1], -1 stored as 2, four row groups interleaved into one byte."""
    import os
    t = _as_blocked_bf16(t)
    if block_size is None:
        block_size = int(os.environ.get("QINT2_BLOCK_SIZE", "256"))
    k1, c1, c2, k2, c3 = t.shape
    N = k1 * k2
    if N % 32:
        raise _lib.TpxError("remap_and_quantize_qint2_intlv: out-features must be a multiple of 32")
    w = t.permute(0, 3, 1, 2, 4).contiguous().view(N, -1)
    C = w.shape[1]
    if C % 4:
        raise _lib.TpxError("remap_and_quantize_qint2_intlv: in-features must be a multiple of 4")
    B = qint2_block_size_used(C, c2 * c3, int(block_size))
    if B not in (64, 128, 256, 512):
        raise _lib.TpxError(f"remap_and_quantize_qint2_intlv: block size {B} is not served by the int8 kernels (64, 128, 256, 512)")
    K1, K2, K3, C1, C2, C3 = N // 32, 8, 4, C // B, B // 4, 4
    wb = w.view(K1, K2 * K3, C1, B).permute(0, 2, 1, 3).contiguous()         # [K1, C1, 32, B]
    scales = wb.abs().amax(-1, keepdim=True).to(torch.float32).clamp_min_(1.0e-8)
    q = torch.round(wb / scales).clamp_(-1.0, 1.0).to(torch.int8)
    q = torch.where(q < 0, torch.full_like(q, 2), q).to(torch.uint8)
    q = q.view(K1, C1, K3, K2, C2, C3).permute(2, 0, 1, 4, 3, 5).contiguous()  # [K3, K1, C1, C2, K2, C3]
    packed = q[0] | (q[1] << 2) | (q[2] << 4) | (q[3] << 6)
    return QInt2Tensor(packed.contiguous(), scales.contiguous(), (K1, C1, C2, K2 * K3, C3), B)


def q_per_block_scales(q):
    return q.scales


def q_per_block_block_size(q):
    return q.block_size


def q_per_block_axis(q):
    return q.axis


def q_per_block_pack_size(q):
    return 2 if q.kind == W_MXFP4 else 1


def remap_and_quantize_qint4(t):
    """Imported by the reference's qtypes.py:19 although its C++ no longer registers it
    (src/csrc/qtypes.cpp:1090 is commented out); kept as an explicit refusal so imports succeed."""
    raise _lib.TpxError("remap_and_quantize_qint4 is not provided by the reference at this revision")
