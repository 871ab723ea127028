"""CPU oracle (numpy + the C file beside it) for the quantized-linear / attention hot path.

TEST INFRASTRUCTURE: imported only by tests/, the smoke test and the benchmark's CPU-baseline
legs. The product package never imports it.

bf16 tensors are carried as numpy uint16 arrays holding the bf16 bit patterns, so that every
rounding is explicit. Layout functions restate, step by step, the tensor views/permutes of the
reference (file:line cited per function, paths relative to the reference root).

Pinned against the reference: the MXFP4 element / scale / block quantizer and the dequantization table (its own
test vectors and, where the shim builds, its compiled conversion functions). Pinned against stock PyTorch: the 8-bit
floating-point casts, LayerNorm. Parity unpinned (restatements with no reference vector or runnable reference code
to hold them to): the int8 and the ternary quantizers, the blocked layouts (checked by address arithmetic), and the
GEMM / attention / layer math (cross-checked against Hugging Face's forward in the GPU tests instead).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

ACT_NONE, ACT_GELU, ACT_SILU, ACT_RELU = 0, 1, 2, 3


def build(force=False):
    """Compile the C oracle (and the reference shim when the reference tree is present)."""
    so = os.path.join(_HERE, "libtpx_oracle.so")
    src = os.path.join(_HERE, "tpx_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "--no-print-directory", "REF=" + reference_root()], stdout=subprocess.DEVNULL)
    return so


def reference_root():
    """Root of the reference's source tree: TPX_REFERENCE_ROOT, else a `reference` directory beside this repository;
    "" when neither holds the MX header (the prebuilt shim under oracle/_ref is then kept as it is)."""
    for cand in (os.environ.get("TPX_REFERENCE_ROOT", ""), os.path.join(_HERE, "..", "..", "reference")):
        if cand and os.path.exists(os.path.join(cand, "src", "csrc", "mxfp_quant.h")):
            return os.path.abspath(cand)
    return ""


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.orc_mx_scale_byte.restype = ctypes.c_uint8
        _LIB.orc_mx_scale_byte.argtypes = [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
        _LIB.orc_e2m1_code.restype = ctypes.c_uint8
        _LIB.orc_e2m1_code.argtypes = [ctypes.c_float]
        _LIB.orc_mxfp4_dequant_elem.restype = ctypes.c_float
        _LIB.orc_mxfp4_dequant_elem.argtypes = [ctypes.c_uint8, ctypes.c_uint8]
        _LIB.orc_num_threads.restype = ctypes.c_int
        _LIB.orc_set_num_threads.argtypes = [ctypes.c_int]
    return _LIB


def ref_lib():
    """The shim over the reference's own mxfp_quant.h (oracle/_ref); None if it was never built."""
    so = os.path.join(_HERE, "_ref", "libtpx_mxref.so")
    if not os.path.exists(so):
        return None
    L = ctypes.CDLL(so)
    L.ref_mx_scale_byte.restype = ctypes.c_uint8
    L.ref_mx_scale_byte.argtypes = [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    L.ref_e2m1_round.restype = ctypes.c_float
    L.ref_e2m1_round.argtypes = [ctypes.c_float]
    L.ref_fp_scale.restype = ctypes.c_float
    L.ref_fp_scale.argtypes = [ctypes.c_int]
    return L


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# --------------------------------------------------------------------------- bf16 helpers
def f32_to_bf16(x):
    """fp32 -> bf16 bit patterns, round to nearest even (what at::BFloat16 does)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_to_f32(h):
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def randn_bf16(rng, shape, std=1.0):
    return f32_to_bf16((rng.standard_normal(shape) * std).astype(np.float32))


# --------------------------------------------------------------------------- layouts
def block_weight(w, bk=16, bc=64, vnni=2):
    """W[N,K] -> blocked [N/bk, K/bc, bc/vnni, bk, vnni].

    BlockingManager.block (src/tpp_pytorch_extension/utils/blocked_layout.py:28-91) with the
    blocking FixLinear attaches for low-precision weights: factors [bk, [bc/vnni, vnni]],
    permute [0,2,3,1,4] (src/tpp_pytorch_extension/llm/llm_common.py:468-490)."""
    N, K = w.shape
    assert N % bk == 0 and K % bc == 0
    v = w.reshape(N // bk, bk, K // bc, bc // vnni, vnni)
    return np.ascontiguousarray(v.transpose(0, 2, 3, 1, 4))


def unblock_weight(wb):
    """Inverse of block_weight (BlockingManager.unblock, blocked_layout.py:80-91)."""
    K1, C1, C2, K2, C3 = wb.shape
    return np.ascontiguousarray(wb.transpose(0, 3, 1, 2, 4)).reshape(K1 * K2, C1 * C2 * C3)


def remap_mxfp4(wb):
    """5-D blocked weight -> K2 = 32 (src/csrc/qtypes.cpp:792-812)."""
    K1, C1, C2, K2, C3 = wb.shape
    want = 32
    if K2 < want and want % K2 == 0:
        R = want // K2
        assert K1 % R == 0, "Shape not compatible for MXFP4"
        t = wb.reshape(K1 // R, R, C1, C2, K2, C3).transpose(0, 2, 3, 1, 4, 5)
        return np.ascontiguousarray(t).reshape(K1 // R, C1, C2, R * K2, C3)
    if K2 > want and K2 % want == 0:
        R = K2 // want
        t = wb.reshape(K1, C1, C2, R, want, C3).transpose(0, 3, 1, 2, 4, 5)
        return np.ascontiguousarray(t).reshape(K1 * R, C1, C2, want, C3)
    return wb


def remap_qint8(wb, block_size=256):
    """5-D blocked weight -> [K1, C/B, B/4, K2, 4] (src/csrc/qtypes.cpp:870-898)."""
    K1, C1, C2, K2, C3 = wb.shape
    C = C1 * C2 * C3
    B = block_size
    if C % B != 0:
        for q in (4096, 2048, 1024, 512, 256, 128, 64):
            if block_size > q and C % q == 0:
                B = q
                break
    C2n, C1n = B // C3, C // B
    t = wb
    if C3 != 4:
        R = 4 // C3
        assert C2n % R == 0, "Shape not compatible for VNNI4"
        t = wb.reshape(K1, C1n, C2n // R, R, K2, C3).transpose(0, 1, 2, 4, 3, 5)
        t = np.ascontiguousarray(t).reshape(K1, C1n, C2n // R, K2, R * C3)
    else:
        t = wb.reshape(K1, C1n, C2n, K2, C3)
    return t, C2n * C3


# --------------------------------------------------------------------------- quantisers
def _block_dims(shape5, block_size):
    """pre/bs/post/vnni of PerBlockQuantizer for axis=2, is_vnni (src/csrc/qtypes.h:30-68)."""
    K1, C1, C2, K2, V = shape5
    bsi = block_size // V
    assert C2 % bsi == 0
    return K1 * C1 * (C2 // bsi), bsi, K2, V, (K1, C1, C2 // bsi, K2)


def quantize_mxfp4(t5):
    """quantize_mxfp4(t, 32, 2, True) (src/csrc/qtypes.cpp:602-611 -> qtypes.h:133-193).
    Returns codes uint8 [K1,C1,C2,K2] (two E2M1 codes per byte, low nibble = even lane) and
    UE8M0 scales uint8 [K1,C1,C2/16,K2]."""
    t5 = _c(t5, np.uint16)
    pre, bs, post, v, sshape = _block_dims(t5.shape, 32)
    codes = np.empty(t5.shape[:4], dtype=np.uint8)
    scales = np.empty(sshape, dtype=np.uint8)
    lib().orc_quantize_mxfp4_blocks(_p(t5), ctypes.c_long(pre), ctypes.c_long(bs), ctypes.c_long(post),
                                    ctypes.c_long(v), _p(codes), _p(scales))
    return codes, scales


def dequantize_mxfp4(codes, scales):
    """PerBlockMxFPQuantizer::dequantize -> fp32 [K1,C1,C2,K2,2] (src/csrc/qtypes.cpp:438-445)."""
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint8)
    shape5 = tuple(codes.shape) + (2,)
    pre, bs, post, v, _ = _block_dims(shape5, 32)
    out = np.empty(shape5, dtype=np.float32)
    lib().orc_dequantize_mxfp4_blocks(_p(codes), _p(scales), ctypes.c_long(pre), ctypes.c_long(bs),
                                      ctypes.c_long(post), ctypes.c_long(v), _p(out))
    return out


def quantize_int8(t5, block_size):
    """quantize_int8sym(t, block, 2, True) (src/csrc/qtypes.cpp:613-624). Returns int8
    [K1,C1,B/4,K2,4] and fp32 scales [K1,C1,1,K2]."""
    t5 = _c(t5, np.uint16)
    pre, bs, post, v, sshape = _block_dims(t5.shape, block_size)
    q = np.empty(t5.shape, dtype=np.int8)
    scales = np.empty(sshape, dtype=np.float32)
    lib().orc_quantize_int8_blocks(_p(t5), ctypes.c_long(pre), ctypes.c_long(bs), ctypes.c_long(post),
                                   ctypes.c_long(v), _p(q), _p(scales))
    return q, scales


def dequantize_int8(q, scales, block_size):
    q, scales = _c(q, np.int8), _c(scales, np.float32)
    pre, bs, post, v, _ = _block_dims(q.shape, block_size)
    out = np.empty(q.shape, dtype=np.float32)
    lib().orc_dequantize_int8_blocks(_p(q), _p(scales), ctypes.c_long(pre), ctypes.c_long(bs),
                                     ctypes.c_long(post), ctypes.c_long(v), _p(out))
    return out


def quantize_act_int8(x_bf16, block_size):
    """Activation quantisation of the reference int8 linear (src/csrc/fused_gemm.h:1249)."""
    x = _c(x_bf16, np.uint16)
    rows, K = x.shape
    q = np.empty((rows, K), dtype=np.int8)
    s = np.empty((rows, K // block_size), dtype=np.float32)
    lib().orc_quantize_act_int8(_p(x), ctypes.c_long(rows), ctypes.c_long(K), ctypes.c_long(block_size), _p(q), _p(s))
    return q, s


def remap_and_quantize_mxfp4(w_bf16, bk=16, bc=64):
    """Plain bf16 W[N,K] -> (codes, scales) exactly as FixLinear(weight_dtype="mxfp4") produces
    them (llm_common.py:495-499 -> src/csrc/qtypes.cpp:783-864)."""
    return quantize_mxfp4(remap_mxfp4(block_weight(w_bf16, bk, bc, 2)))


def remap_and_quantize_qint8(w_bf16, block_size=256, bk=16, bc=64):
    t, bs = remap_qint8(block_weight(w_bf16, bk, bc, 2), block_size)
    q, s = quantize_int8(t, bs)
    return q, s, bs


def plain_from_blocked5(t5):
    """[K1,C1,C2,K2,V] (element = W[K2*k1+k2, (C2*V)*c1 + V*c2 + v]) -> plain [N,K]."""
    K1, C1, C2, K2, V = t5.shape
    return np.ascontiguousarray(t5.transpose(0, 3, 1, 2, 4)).reshape(K1 * K2, C1 * C2 * V)


def mxfp4_dequant_plain(codes, scales):
    """Dequantised weight as plain fp32 [N,K]."""
    return plain_from_blocked5(dequantize_mxfp4(codes, scales))


def int8_dequant_plain(q, scales, block_size):
    return plain_from_blocked5(dequantize_int8(q, scales, block_size))


def int8_plain(q, scales):
    """Plain int8 [N,K] and scales [N, K/B] from the blocked tensors."""
    K1, C1, C2, K2, V = q.shape
    qp = plain_from_blocked5(q)
    sp = np.ascontiguousarray(scales.reshape(K1, C1, K2).transpose(0, 2, 1)).reshape(K1 * K2, C1)
    return qp, sp


# --------------------------------------------------------------------------- 8-bit floating-point weights
# The reference keeps a weight as bfloat8 / hfloat8 by a plain cast of the blocked bf16 tensor
# (src/tpp_pytorch_extension/llm/llm_common.py:519-522) and converts it up inside TppBlockedLinearW<Tin, bfloat8 | hfloat8>
# (src/csrc/fused_gemm.h:1558-1565). Those dtypes exist only in the reference's own PyTorch build; the formats are the
# published ones: bfloat8 = E5M2 (bias 15, infinities), hfloat8 = E4M3 (bias 7, largest finite value 448, no infinity).
# Round to nearest even; out-of-range values become infinity (E5M2) or NaN (E4M3). Pinned against the float8 casts of
# stock PyTorch on the CPU (tests/test_oracle.py).
FP8_E4M3, FP8_E5M2 = 1, 2
_FP8_PARAMS = {FP8_E4M3: (4, 3, 7, 448.0), FP8_E5M2: (5, 2, 15, 57344.0)}


def fp8_to_f32_table(fmt):
    ebits, mbits, bias, _ = _FP8_PARAMS[fmt]
    out = np.zeros(256, dtype=np.float32)
    for c in range(256):
        sign = -1.0 if c & 0x80 else 1.0
        e = (c >> mbits) & ((1 << ebits) - 1)
        m = c & ((1 << mbits) - 1)
        if fmt == FP8_E5M2 and e == 31:
            v = np.inf if m == 0 else np.nan
        elif fmt == FP8_E4M3 and e == 15 and m == 7:
            v = np.nan
        elif e == 0:
            v = m * 2.0 ** (1 - bias - mbits)
        else:
            v = (1.0 + m / (1 << mbits)) * 2.0 ** (e - bias)
        out[c] = sign * v
    return out


def f32_to_fp8(x, fmt):
    """fp32 array -> uint8 codes of the format, round to nearest even."""
    ebits, mbits, bias, vmax = _FP8_PARAMS[fmt]
    x = np.asarray(x, dtype=np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        return _f32_to_fp8(x, fmt, ebits, mbits, bias, vmax)


def _f32_to_fp8(x, fmt, ebits, mbits, bias, vmax):
    finite = np.isfinite(x)
    a = np.abs(np.where(finite, x, 0.0)).astype(np.float64)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    _, ex = np.frexp(a)                       # a = f * 2^ex, f in [0.5, 1)
    e = np.maximum(ex - 1, 1 - bias)          # exponent of the binade, clamped to the subnormal one
    step = np.ldexp(1.0, e - mbits)
    q = np.rint(a / step)                     # numpy rounds half to even; a / step is exact (power-of-two divisor)
    over = q * step > vmax
    e2 = np.where(q >= (2 << mbits), e + 1, e)  # the rounding carried into the next binade
    q2 = np.where(q >= (2 << mbits), q / 2, q)
    normal = q2 >= (1 << mbits)
    code = np.where(normal, ((e2 + bias).astype(np.int64) << mbits) | (q2.astype(np.int64) - (1 << mbits)), q2.astype(np.int64))
    if fmt == FP8_E5M2:
        code = np.where(over | np.isinf(x), 0x7c, code)
        code = np.where(np.isnan(x), 0x7f, code)
    else:
        code = np.where(over | ~finite, 0x7f, code)
    return (code.astype(np.uint8) | sign).astype(np.uint8)


def fp8_dequant(codes, fmt):
    return fp8_to_f32_table(fmt)[np.asarray(codes, dtype=np.uint8)]


# --------------------------------------------------------------------------- ternary ("qint2") weights
def remap_and_quantize_qint2(w_bf16, block_size=256):
    """remap_and_quantize_qint2_intlv (src/csrc/qtypes.cpp:1004-1073) on a plain bf16 weight [N, K] (bits), N a multiple
    of 32 (the reference's K2 = 8, K3 = 4 case): per (row, block) scale = max |w| in fp32 (at least 1e-8), code =
    round-half-even(w / scale) clamped to [-1, 1] with -1 stored as 2; four row groups of eight rows share a byte.
    Returns (packed uint8 [N/32, K/B, B/4, 8, 4], scales fp32 [N/32, K/B, 32, 1], B). Parity unpinned: the reference holds
    no vectors for this quantizer and cannot be built here; the restatement follows its tensor operations one by one."""
    w = bf16_to_f32(np.asarray(w_bf16, dtype=np.uint16))
    N, K = w.shape
    assert N % 32 == 0 and K % 4 == 0
    B = block_size
    if K % B:
        B = next((q for q in (4096, 2048, 1024, 512, 256, 128, 64) if block_size > q and K % q == 0), 64)
    K1, C1 = N // 32, K // B
    wb = w.reshape(K1, 32, C1, B).transpose(0, 2, 1, 3)                      # [K1, C1, 32, B]
    scales = np.maximum(np.abs(wb).max(-1, keepdims=True).astype(np.float32), np.float32(1e-8))
    q = np.clip(np.rint((wb / scales).astype(np.float32)), -1.0, 1.0).astype(np.int8)
    codes = np.where(q < 0, 2, q).astype(np.uint8)
    c = codes.reshape(K1, C1, 4, 8, B // 4, 4).transpose(2, 0, 1, 4, 3, 5)   # [K3, K1, C1, C2, K2, C3]
    packed = c[0] | (c[1] << 2) | (c[2] << 4) | (c[3] << 6)
    return np.ascontiguousarray(packed), np.ascontiguousarray(scales), B


def qint2_dequant_plain(packed, scales, block_size):
    """fp32 [N, K] from the carrier of remap_and_quantize_qint2."""
    K1, C1, C2, K2, C3 = packed.shape
    parts = np.stack([(packed >> (2 * k3)) & 3 for k3 in range(4)], 0).astype(np.int8)  # [K3, K1, C1, C2, K2, C3]
    q = np.where(parts == 2, -1, parts).astype(np.float32)
    q = q.transpose(1, 0, 4, 2, 3, 5).reshape(K1, 32, C1, C2 * C3)                       # [K1, (K3 K2), C1, B]
    w = q * scales.reshape(K1, C1, 32).transpose(0, 2, 1)[..., None]
    return np.ascontiguousarray(w.reshape(K1 * 32, C1 * block_size).astype(np.float32))


# --------------------------------------------------------------------------- linear
def qlinear(x_bf16, wd, bias=None, mul_in=None, res=None, res_scale=1.0, act=ACT_NONE, ref_rounding=False):
    x = _c(x_bf16, np.uint16)
    wd = _c(wd, np.float32)
    M, K = x.shape
    N = wd.shape[0]
    y = np.empty((M, N), dtype=np.uint16)
    b = _c(bias, np.uint16) if bias is not None else None
    mi = _c(mul_in, np.uint16) if mul_in is not None else None
    r = _c(res, np.uint16) if res is not None else None
    lib().orc_qlinear_f32w(_p(x), _p(wd), _p(b), _p(mi), _p(r), ctypes.c_float(res_scale), ctypes.c_int(act),
                           ctypes.c_int(int(ref_rounding)), ctypes.c_long(M), ctypes.c_long(N), ctypes.c_long(K), _p(y))
    return y


def gate_up(x_bf16, wg, wu, act=ACT_SILU, ref_rounding=False):
    x = _c(x_bf16, np.uint16)
    wg, wu = _c(wg, np.float32), _c(wu, np.float32)
    M, K = x.shape
    N = wg.shape[0]
    y = np.empty((M, N), dtype=np.uint16)
    lib().orc_gate_up_f32w(_p(x), _p(wg), _p(wu), ctypes.c_int(act), ctypes.c_int(int(ref_rounding)),
                           ctypes.c_long(M), ctypes.c_long(N), ctypes.c_long(K), _p(y))
    return y


def qlinear_mxfp4_packed(x_bf16, codes, scales, codes2=None, scales2=None, act=ACT_NONE):
    """Linear straight from the packed reference-layout MXFP4 tensors (timed CPU baseline)."""
    x = _c(x_bf16, np.uint16)
    M, K = x.shape
    N = codes.shape[0] * 32
    y = np.empty((M, N), dtype=np.uint16)
    lib().orc_qlinear_mxfp4_packed(_p(x), _p(_c(codes, np.uint8)), _p(_c(scales, np.uint8)),
                                   _p(_c(codes2, np.uint8)) if codes2 is not None else None,
                                   _p(_c(scales2, np.uint8)) if scales2 is not None else None,
                                   ctypes.c_int(act), ctypes.c_long(M), ctypes.c_long(N), ctypes.c_long(K), _p(y))
    return y


def qlinear_int8_dynact(x_bf16, q, scales, block_size, bias=None, act=ACT_NONE):
    """The reference's own int8 arithmetic (activations quantised on the fly, bf16 running output)."""
    xq, xs = quantize_act_int8(x_bf16, block_size)
    qp, sp = int8_plain(q, scales)
    M, K = xq.shape
    N = qp.shape[0]
    y = np.empty((M, N), dtype=np.uint16)
    b = _c(bias, np.uint16) if bias is not None else None
    lib().orc_qlinear_int8_dynact(_p(xq), _p(xs), _p(_c(qp, np.int8)), _p(_c(sp, np.float32)), _p(b),
                                  ctypes.c_int(act), ctypes.c_long(M), ctypes.c_long(N), ctypes.c_long(K),
                                  ctypes.c_long(block_size), _p(y))
    return y


# --------------------------------------------------------------------------- norm / rope / cache / attention
def rmsnorm(x_bf16, g_bf16, eps):
    x = _c(x_bf16, np.uint16)
    D = x.shape[-1]
    rows = x.size // D
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(_c(g_bf16, np.uint16)), ctypes.c_float(eps), ctypes.c_long(rows), ctypes.c_long(D), _p(y))
    return y


def layernorm(x_bf16, g_bf16, b_bf16, eps):
    """lyr_norm (src/csrc/llm/fused_llm_infer.cpp:256-306, LayerNormFwdTPP): fp32 mean and variance around the mean,
    y = (x - mean) * rsqrt(var + eps) * gamma + beta, rounded to bf16."""
    x = bf16_to_f32(_c(x_bf16, np.uint16)).astype(np.float32)
    g = bf16_to_f32(_c(g_bf16, np.uint16)).astype(np.float32)
    b = bf16_to_f32(_c(b_bf16, np.uint16)).astype(np.float32)
    mean = x.mean(-1, keepdims=True, dtype=np.float32)
    var = ((x - mean) ** 2).mean(-1, keepdims=True, dtype=np.float32)
    return f32_to_bf16(((x - mean) / np.sqrt(var + np.float32(eps))) * g + b)


def rope_table(max_pos, head_dim, theta):
    """cat(cos, sin).view(2, MP, head_dim) fp32 as built in OptimizeModelForLlama
    (src/tpp_pytorch_extension/llm/fused_llama_infer.py:186-204); HF's default rotary embedding:
    inv_freq = theta^(-2i/d), emb = cat(freqs, freqs)."""
    inv = 1.0 / (theta ** (np.arange(0, head_dim, 2, dtype=np.float32) / np.float32(head_dim)))
    inv = inv.astype(np.float32)
    t = np.arange(max_pos, dtype=np.float32)
    fr = np.outer(t, inv).astype(np.float32)
    emb = np.concatenate([fr, fr], axis=-1)
    return np.stack([np.cos(emb), np.sin(emb)]).astype(np.float32)


def rope_llama(x_bf16, ep, pos, n_heads, head_dim):
    """In-place-style RoPE on [B,S,N*H]; returns a new array."""
    x = _c(x_bf16, np.uint16).copy()
    B, S = x.shape[0], x.shape[1]
    pos = _c(pos, np.int64)
    lib().orc_rope_llama(_p(x), _p(_c(ep, np.float32)), _p(pos), ctypes.c_long(B), ctypes.c_long(S),
                         ctypes.c_long(n_heads), ctypes.c_long(head_dim), ctypes.c_long(ep.shape[1]),
                         ctypes.c_long(ep.shape[2]), ctypes.c_long(pos.shape[0]))
    return x


class KVCache:
    """LayerCache / KVLayout_BNSH (src/csrc/llm/attn.h:144-226, src/csrc/llm/attn.cpp:383-463):
    per layer K and V tensors [S1, B, Nkv, 32, H]; token t lives at (t // 32, t % 32); capacity
    grows to offset + S + 128 rounded up to 32 by allocating zeros and copying."""

    S2 = 32
    INC = 128

    def __init__(self):
        self.layers = {}

    def update(self, k, v, layer):
        """k, v: [B, S, Nkv, H] bf16 bit patterns (the reference passes [B,Nkv,S,H] views)."""
        B, S, Nkv, H = k.shape
        st = self.layers.get(layer)
        if st is None:
            st = {"off": 0, "k": np.zeros((0, B, Nkv, 32, H), np.uint16), "v": np.zeros((0, B, Nkv, 32, H), np.uint16)}
            self.layers[layer] = st
        need = st["off"] + S
        if need > st["k"].shape[0] * 32:
            cap = (need + self.INC + 31) // 32
            for key in ("k", "v"):
                n = np.zeros((cap, B, Nkv, 32, H), np.uint16)
                n[: st[key].shape[0]] = st[key]
                st[key] = n
        for s in range(S):
            t = st["off"] + s
            st["k"][t // 32, :, :, t % 32, :] = k[:, s]
            st["v"][t // 32, :, :, t % 32, :] = v[:, s]
        st["off"] = need
        return st["k"], st["v"]

    def get_seq_length(self, layer=0):
        return self.layers[layer]["off"] if layer in self.layers else 0


def align_and_invert_mask(mask01, dtype_min=-3.3895313892515355e38):
    """TppCache::align_and_invert_mask (src/csrc/llm/attn.h:310-322): pad the key axis to a
    multiple of 32; 1 -> 0, 0 -> finfo(bf16).min; the padding is masked. Returns bf16 patterns."""
    B, S = mask01.shape
    Sp = (S + 31) // 32 * 32
    out = np.full((B, Sp), dtype_min, dtype=np.float32)
    out[:, :S] = np.where(mask01 > 0, 0.0, dtype_min)
    return f32_to_bf16(out)


def attention(q, kc, vc, am, key_len, causal=True):
    """q [B,Nkv,Sq,R,H]; kc/vc [S1,B,Nkv,32,H]; am [B,Spad] or None."""
    q = _c(q, np.uint16)
    B, Nkv, Sq, R, H = q.shape
    out = np.empty_like(q)
    amc = _c(am, np.uint16) if am is not None else None
    lib().orc_attention(_p(q), _p(_c(kc, np.uint16)), _p(_c(vc, np.uint16)), _p(amc), ctypes.c_long(B),
                        ctypes.c_long(Nkv), ctypes.c_long(Sq), ctypes.c_long(R), ctypes.c_long(H),
                        ctypes.c_long(key_len), ctypes.c_long(amc.shape[1] if amc is not None else 0),
                        ctypes.c_int(int(causal)), _p(out))
    return out


def llama_layer(hs, mask, pos, W, cache, layer_idx, n_q, n_kv, head_dim, eps, ep, world=1, allreduce=None):
    """LlamaDecoderLayer::_forward (src/csrc/llm/fused_llm_infer.cpp:1195-1286).

    hs [B,S,D] bf16 patterns; W: dict of dequantised plain fp32 weights q,k,v,o,gate,up,down and
    bf16 norm weights ln1, ln2. `allreduce` is called on the fp32 view of the row-parallel outputs
    when world > 1 (the residual is pre-scaled by 1/world, :1206,1261,1273). Optional bf16 biases bq, bk, bv in W
    give Qwen2DecoderLayer::_forward (:1440-1510), which differs only in them."""
    B, S, D = hs.shape
    scale = 1.0 / world
    res = hs.reshape(B * S, D)
    x = rmsnorm(res, W["ln1"], eps)
    q = qlinear(x, W["q"], bias=W.get("bq")).reshape(B, S, n_q * head_dim)
    k = qlinear(x, W["k"], bias=W.get("bk")).reshape(B, S, n_kv * head_dim)
    v = qlinear(x, W["v"], bias=W.get("bv")).reshape(B, S, n_kv, head_dim)
    q = rope_llama(q, ep, pos, n_q, head_dim)
    k = rope_llama(k, ep, pos, n_kv, head_dim).reshape(B, S, n_kv, head_dim)
    kc, vc = cache.update(k, v, layer_idx)
    key_len = cache.get_seq_length(layer_idx)
    R = n_q // n_kv
    q5 = np.ascontiguousarray(q.reshape(B, S, n_kv, R, head_dim).transpose(0, 2, 1, 3, 4))
    ctx = attention(q5, kc, vc, mask, key_len, causal=True)
    ctx = np.ascontiguousarray(ctx.transpose(0, 2, 1, 3, 4)).reshape(B * S, n_q * head_dim)
    so = qlinear(ctx, W["o"], res=res, res_scale=scale)
    if world > 1:
        so = allreduce(so)
    x2 = rmsnorm(so, W["ln2"], eps)
    inter = gate_up(x2, W["gate"], W["up"], ACT_SILU)
    out = qlinear(inter, W["down"], res=so, res_scale=scale)
    if world > 1:
        out = allreduce(out)
    return out.reshape(B, S, D)


def opt_layer(hs, mask, W, cache, layer_idx, n_heads, head_dim, eps1, eps2, do_layer_norm_before=True, world=1, allreduce=None):
    """OPTDecoderLayer::_forward (src/csrc/llm/fused_llm_infer.cpp:978-1068): LayerNorm before (or after) each half,
    q/k/v with biases, attention without rotary embedding, out_proj + residual, fc1 + ReLU, fc2 + residual.
    W: plain fp32 weights q,k,v,o,fc1,fc2, bf16 biases bq,bk,bv,bo,b1,b2 and LayerNorm parameters g1,b_ln1,g2,b_ln2."""
    B, S, D = hs.shape
    scale = 1.0 / world
    res = hs.reshape(B * S, D)
    x = layernorm(res, W["g1"], W["b_ln1"], eps1) if do_layer_norm_before else res
    q = qlinear(x, W["q"], bias=W["bq"]).reshape(B, S, n_heads, head_dim)
    k = qlinear(x, W["k"], bias=W["bk"]).reshape(B, S, n_heads, head_dim)
    v = qlinear(x, W["v"], bias=W["bv"]).reshape(B, S, n_heads, head_dim)
    kc, vc = cache.update(k, v, layer_idx)
    key_len = cache.get_seq_length(layer_idx)
    q5 = np.ascontiguousarray(q.reshape(B, S, n_heads, 1, head_dim).transpose(0, 2, 1, 3, 4))
    ctx = attention(q5, kc, vc, mask, key_len, causal=True)
    ctx = np.ascontiguousarray(ctx.transpose(0, 2, 1, 3, 4)).reshape(B * S, n_heads * head_dim)
    so = qlinear(ctx, W["o"], bias=W["bo"], res=res, res_scale=scale)
    if world > 1:
        so = allreduce(so)
    if not do_layer_norm_before:
        so = layernorm(so, W["g1"], W["b_ln1"], eps1)
    x = layernorm(so, W["g2"], W["b_ln2"], eps2) if do_layer_norm_before else so
    inter = qlinear(x, W["fc1"], bias=W["b1"], act=ACT_RELU)
    out = qlinear(inter, W["fc2"], bias=W["b2"], res=so, res_scale=scale)
    if world > 1:
        out = allreduce(out)
    if not do_layer_norm_before:
        out = layernorm(out, W["g2"], W["b_ln2"], eps2)
    return out.reshape(B, S, D)


def rope_gptj(x_bf16, emb_pos, pos, n_heads, head_dim):
    """apply_rotary_pos_emb_gptj (src/csrc/llm/fused_llm_infer.cpp:150-204) on [B,S,N*H]: the first HR values of every head
    rotate in adjacent pairs (2i, 2i+1); emb_pos fp32 [MP, HR] holds HR/2 sines, then HR/2 cosines; positions beyond the
    table leave the row untouched. Products are rounded separately (no fused multiply-add), the result to bf16."""
    x = bf16_to_f32(_c(x_bf16, np.uint16)).astype(np.float32)
    B, S = x.shape[0], x.shape[1]
    MP, HR = emb_pos.shape
    x = x.reshape(B, S, n_heads, head_dim).copy()
    pos = np.asarray(pos, np.int64)
    for b in range(B):
        for s in range(S):
            p = int(pos[0 if pos.shape[0] == 1 else b, s])
            if p >= MP:
                continue
            sn, cs = emb_pos[p, :HR // 2].astype(np.float32), emb_pos[p, HR // 2:].astype(np.float32)
            x0, x1 = x[b, s, :, 0:HR:2].copy(), x[b, s, :, 1:HR:2].copy()
            x[b, s, :, 0:HR:2] = x0 * cs - x1 * sn
            x[b, s, :, 1:HR:2] = x1 * cs + x0 * sn
    return f32_to_bf16(x.reshape(B, S, n_heads * head_dim))


def gptj_layer(hs, mask, pos, W, cache, layer_idx, n_heads, head_dim, eps, emb_pos, world=1, allreduce=None):
    """GPTJBlock::_forward (src/csrc/llm/fused_llm_infer.cpp:735-848): one LayerNorm feeds attention (q, k, v without
    bias, GPT-J rotary, out_proj) and the MLP (fc_in + GELU, fc_out) side by side; out = fc_out(...) + attention output
    + residual / world (Add2ScalePostOp). W: plain fp32 weights q,k,v,o,fc_in,fc_out, bf16 b_in, b_out, g, b_ln."""
    B, S, D = hs.shape
    scale = 1.0 / world
    res = hs.reshape(B * S, D)
    x = layernorm(res, W["g"], W["b_ln"], eps)
    q = qlinear(x, W["q"]).reshape(B, S, n_heads * head_dim)
    k = qlinear(x, W["k"]).reshape(B, S, n_heads * head_dim)
    v = qlinear(x, W["v"]).reshape(B, S, n_heads, head_dim)
    q = rope_gptj(q, emb_pos, pos, n_heads, head_dim)
    k = rope_gptj(k, emb_pos, pos, n_heads, head_dim).reshape(B, S, n_heads, head_dim)
    kc, vc = cache.update(k, v, layer_idx)
    key_len = cache.get_seq_length(layer_idx)
    q5 = np.ascontiguousarray(q.reshape(B, S, n_heads, 1, head_dim).transpose(0, 2, 1, 3, 4))
    ctx = attention(q5, kc, vc, mask, key_len, causal=True)
    ctx = np.ascontiguousarray(ctx.transpose(0, 2, 1, 3, 4)).reshape(B * S, n_heads * head_dim)
    so = qlinear(ctx, W["o"], res=res, res_scale=scale)
    inter = qlinear(x, W["fc_in"], bias=W["b_in"], act=ACT_GELU)
    out = qlinear(inter, W["fc_out"], bias=W["b_out"], res=so, res_scale=1.0)
    if world > 1:
        out = allreduce(out)
    return out.reshape(B, S, D)


def rel_err(y_bf16, ref_bf16):
    """max |y - ref| / max |ref|: the normalised max error the parity tests bound by 2e-2."""
    a, b = bf16_to_f32(y_bf16).astype(np.float64), bf16_to_f32(ref_bf16).astype(np.float64)
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))
