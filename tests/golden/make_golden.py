"""Generates tests/golden/mxfp4_golden.npz from the REFERENCE's own MX helper code.

Run in a container that has the reference tree (oracle/Makefile builds oracle/_ref/libtpx_mxref.so
from the reference's src/csrc/mxfp_quant.h where it lies):

    make -C oracle && python tests/golden/make_golden.py

The element-level vectors are outputs of the reference functions themselves. The block-level
vectors compose those same reference functions in plain Python loops that follow
PerBlockQuantizer::quantize_symetric (src/csrc/qtypes.h:133-193) and MxFP4Quant
(src/csrc/qtypes.cpp:69-135) line by line, independently of the C oracle they later check.
The int8 vectors have no compilable reference counterpart (Int8SymQuant sits in a translation
unit that needs libxsmm) and are produced by a numpy restatement of src/csrc/qtypes.cpp:163-181.
"""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402  (only its bf16 helpers and layout views are used here)

LUT = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def code_of(r):
    """The if-chain of MxFP4Quant::quantize (src/csrc/qtypes.cpp:99-131)."""
    if r == 0.0:
        return 0
    if np.isnan(r):
        return 0
    return LUT.index(abs(r)) + (8 if r < 0 else 0)


def main():
    R = O.ref_lib()
    assert R is not None, "build oracle/_ref first (make -C oracle)"
    rng = np.random.default_rng(1234)
    # ---- element KAT
    xs = []
    for v in LUT:
        xs += [v, -v]
    ties = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    for t in ties:
        f = np.float32(t)
        xs += [f, -f, np.nextafter(f, np.float32(10)), np.nextafter(f, np.float32(0)), -np.nextafter(f, np.float32(10))]
    xs += [6.5, 7.0, 100.0, 1e30, -1e30, 0.1, 0.124, 0.125, 0.126, 1e-30, 1e-40, -1e-40, 0.2499999, 5.9999, 6.0000005]
    xs += list((rng.standard_normal(4096) * 3).astype(np.float32))
    xs += list(O.bf16_to_f32(rng.integers(0, 65536, 4096).astype(np.uint16)))
    xs = np.array([x for x in np.array(xs, dtype=np.float32) if np.isfinite(x)], dtype=np.float32)
    elem_round = np.array([R.ref_e2m1_round(float(x)) for x in xs], dtype=np.float32)
    elem_code = np.array([code_of(r) for r in elem_round], dtype=np.uint8)
    # ---- scale KAT
    ms = [0.0, 1e-45, 1e-39, 2.0 ** -126, 2.0 ** -125, 2.0 ** -124, 1.0, 1.5, 1.9999999, 5.9, 6.0, 6.1, 0.02, 0.07,
          3e38, float("inf")]
    ms += [2.0 ** e for e in range(-126, 128, 7)]
    ms += list(np.abs(rng.standard_normal(512) * 0.05).astype(np.float32))
    ms = np.array(ms, dtype=np.float32)
    sb, fl, sf = [], [], []
    for m in ms:
        f, s = ctypes.c_int(), ctypes.c_float()
        sb.append(R.ref_mx_scale_byte(float(m), ctypes.byref(f), ctypes.byref(s)))
        fl.append(f.value)
        sf.append(np.float32(s.value).view(np.uint32))
    fp_scale_bits = np.array([np.float32(R.ref_fp_scale(b)).view(np.uint32) for b in range(256)], dtype=np.uint32)
    # ---- block-level: plain bf16 W[64,128] -> blocked -> remap -> quantize, composed from reference element functions
    w = O.randn_bf16(rng, (64, 128), 0.02)
    w[3, :32] = 0  # an all-zero block (flushed, scale byte from e = 0)
    w[5, 64:96] = O.f32_to_bf16(np.full(32, 1e-39, np.float32))  # subnormal block
    w[7, 0] = O.f32_to_bf16(np.array([10.0], np.float32))[0]  # an outlier
    t5 = O.remap_mxfp4(O.block_weight(w, 16, 64, 2))  # [2, 2, 32, 32, 2]
    K1, C1, C2, K2, V = t5.shape
    bs, post = 16, K2
    tf = O.bf16_to_f32(t5).reshape(K1 * C1 * (C2 // bs), bs, post, V)
    codes = np.zeros((K1 * C1 * (C2 // bs), bs, post), np.uint8)
    scales = np.zeros((K1 * C1 * (C2 // bs), post), np.uint8)
    for i in range(tf.shape[0]):
        for j in range(post):
            mx = float(np.max(np.abs(tf[i, :, j, :])))
            f, s = ctypes.c_int(), ctypes.c_float()
            scales[i, j] = R.ref_mx_scale_byte(mx, ctypes.byref(f), ctypes.byref(s))
            for k in range(bs):
                packed = 0
                for v in range(2):
                    xin = 0.0 if f.value else float(np.float32(tf[i, k, j, v]) / np.float32(s.value))
                    packed |= code_of(R.ref_e2m1_round(xin)) << (4 * v)
                codes[i, k, j] = packed
    blk_codes = codes.reshape(K1, C1, C2, K2)
    blk_scales = scales.reshape(K1, C1, C2 // bs, K2)
    deq = np.zeros((K1, C1, C2, K2, 2), np.float32)
    sgn = [1, 1, 1, 1, 1, 1, 1, 1, -1, -1, -1, -1, -1, -1, -1, -1]
    for idx in np.ndindex(K1, C1, C2, K2):
        s = np.uint32(fp_scale_bits[blk_scales[idx[0], idx[1], idx[2] // bs, idx[3]]]).view(np.float32)
        p = int(blk_codes[idx])
        for v in range(2):
            c = (p >> (4 * v)) & 15
            deq[idx + (v,)] = np.float32(sgn[c] * LUT[c & 7]) * s
    # ---- int8 (numpy restatement of src/csrc/qtypes.cpp:163-181; no compilable reference)
    w8 = O.randn_bf16(rng, (32, 128), 0.02)
    w8[2, :64] = 0
    t8, B = O.remap_qint8(O.block_weight(w8, 16, 64, 2), 64)  # [2, 2, 16, 16, 4]
    f8 = O.bf16_to_f32(t8)
    mx8 = np.abs(f8).max(axis=(2, 4), keepdims=True)
    sc8 = (mx8.astype(np.float64) / 127.0).astype(np.float32)
    isc8 = np.where(sc8 != 0, np.float32(1.0) / np.where(sc8 != 0, sc8, np.float32(1)), np.float32(0)).astype(np.float32)
    q8 = np.clip(np.rint((f8 * isc8).astype(np.float32)), -127, 127).astype(np.int8)
    np.savez_compressed(
        os.path.join(os.path.dirname(os.path.abspath(__file__)), "mxfp4_golden.npz"),
        elem_x=xs, elem_round=elem_round, elem_code=elem_code,
        scale_absmax=ms, scale_byte=np.array(sb, np.uint8), scale_flush=np.array(fl, np.uint8),
        scale_fp_bits=np.array(sf, np.uint32), fp_scale_bits=fp_scale_bits,
        blk_w=w, blk_codes=blk_codes, blk_scales=blk_scales, blk_deq=deq,
        i8_w=w8, i8_q=q8, i8_scales=sc8.reshape(2, 2, 1, 16))
    print("wrote mxfp4_golden.npz:", len(xs), "element vectors,", len(ms), "scale vectors")


if __name__ == "__main__":
    main()
