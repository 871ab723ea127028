"""CPU tests: the oracle against the golden vectors produced from the reference's own MX helpers,
and the layout facts the CUDA kernels rely on."""
import ctypes

import numpy as np
import pytest

from oracle import oracle as O


def test_e2m1_element_matches_reference_vectors(golden):
    L = O.lib()
    got = np.array([L.orc_e2m1_code(float(x)) for x in golden["elem_x"]], dtype=np.uint8)
    assert np.array_equal(got, golden["elem_code"])


def test_scale_byte_matches_reference_vectors(golden):
    L = O.lib()
    for m, b, f, sbits in zip(golden["scale_absmax"], golden["scale_byte"], golden["scale_flush"], golden["scale_fp_bits"]):
        fl, sf = ctypes.c_int(), ctypes.c_float()
        got = L.orc_mx_scale_byte(float(m), ctypes.byref(fl), ctypes.byref(sf))
        assert (got, fl.value) == (int(b), int(f)), float(m)
        assert np.float32(sf.value).view(np.uint32) == sbits


def test_dequant_scale_table(golden):
    L = O.lib()
    for b in range(256):
        got = np.float32(L.orc_mxfp4_dequant_elem(2, b)).view(np.uint32)  # code 2 = 1.0
        assert got == golden["fp_scale_bits"][b]
    assert L.orc_mxfp4_dequant_elem(7, 0) == 0.0  # scale byte 0 dequantises to 0, not 2^-127


def test_live_reference_shim_if_present():
    """When oracle/_ref was built here, sweep every bf16 value through reference and oracle."""
    R = O.ref_lib()
    if R is None:
        import pytest
        pytest.skip("oracle/_ref not built in this checkout")
    L = O.lib()
    xs = (np.arange(0, 65536, 3, dtype=np.uint32) << 16).view(np.float32)
    lut = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for x in xs:
        if not np.isfinite(x):
            continue
        r = R.ref_e2m1_round(float(x))
        want = 0 if r == 0 else lut.index(abs(r)) + (8 if r < 0 else 0)
        assert L.orc_e2m1_code(float(x)) == want, x


def test_block_quantizer_matches_golden(golden):
    codes, scales = O.remap_and_quantize_mxfp4(golden["blk_w"])
    assert np.array_equal(codes, golden["blk_codes"])
    assert np.array_equal(scales, golden["blk_scales"])
    assert np.array_equal(O.dequantize_mxfp4(codes, scales).view(np.uint32), golden["blk_deq"].view(np.uint32))


def test_int8_quantizer_matches_golden(golden):
    q, s, bs = O.remap_and_quantize_qint8(golden["i8_w"], 64)
    assert bs == 64
    assert np.array_equal(q, golden["i8_q"])
    assert np.array_equal(s.view(np.uint32), golden["i8_scales"].view(np.uint32))


def test_mxfp4_layout_addresses():
    """Byte (k1,c1,r,k2) of the quantised tensor holds W[32k1+k2][64c1+2r+{0,1}], low nibble first;
    scale (k1,c1,b,k2) covers W[32k1+k2][64c1+32b .. +31]."""
    rng = np.random.default_rng(3)
    N, K = 64, 256
    w = O.randn_bf16(rng, (N, K), 0.02)
    codes, scales = O.remap_and_quantize_mxfp4(w)
    assert codes.shape == (N // 32, K // 64, 32, 32) and scales.shape == (N // 32, K // 64, 2, 32)
    wd = O.mxfp4_dequant_plain(codes, scales)
    L = O.lib()
    for n, k in [(0, 0), (17, 3), (33, 64), (63, 255), (40, 129)]:
        byte = codes[n // 32, k // 64, (k % 64) // 2, n % 32]
        c = (byte >> 4) if (k & 1) else (byte & 15)
        s = scales[n // 32, k // 64, (k % 64) // 32, n % 32]
        assert wd[n, k] == L.orc_mxfp4_dequant_elem(int(c), int(s))
    # per 32-block the error is bounded by the widest rounding/saturation gap: 2 code units
    err = np.abs(wd - O.bf16_to_f32(w)).reshape(N, K // 32, 32).max(-1)
    sp = np.ascontiguousarray(scales.transpose(0, 3, 1, 2)).reshape(N, K // 32).astype(np.int32)
    assert np.all(err <= 2.0 * np.ldexp(1.0, sp - 127))


def test_int8_layout_addresses():
    rng = np.random.default_rng(4)
    w = O.randn_bf16(rng, (32, 512), 0.02)
    for B in (64, 256):
        q, s, bs = O.remap_and_quantize_qint8(w, B)
        assert q.shape == (2, 512 // B, B // 4, 16, 4) and s.shape == (2, 512 // B, 1, 16)
        qp, sp = O.int8_plain(q, s)
        for n, k in [(0, 0), (17, 70), (31, 511)]:
            assert qp[n, k] == q[n // 16, k // B, (k % B) // 4, n % 16, k % 4]
            assert sp[n, k // B] == s[n // 16, k // B, 0, n % 16]
        wd = O.int8_dequant_plain(q, s, bs)
        assert np.max(np.abs(wd - O.bf16_to_f32(w))) <= np.max(sp) * 0.5 + 1e-9


def test_int8_block_size_fallback():
    """A block size that does not divide K falls back to the largest smaller power of two that does (qtypes.cpp:881-888)."""
    rng = np.random.default_rng(5)
    w = O.randn_bf16(rng, (16, 192), 0.02)
    q, s, bs = O.remap_and_quantize_qint8(w, 256)
    assert bs == 64 and q.shape == (1, 3, 16, 16, 4)


def test_block_unblock_roundtrip():
    rng = np.random.default_rng(6)
    w = O.randn_bf16(rng, (48, 128))
    wb = O.block_weight(w)
    assert wb.shape == (3, 2, 32, 16, 2)
    assert wb[1, 1, 5, 7, 1] == w[16 + 7, 64 + 11]
    assert np.array_equal(O.unblock_weight(wb), w)


def test_packed_linear_equals_dequantised_linear():
    rng = np.random.default_rng(7)
    w = O.randn_bf16(rng, (64, 256), 0.02)
    x = O.randn_bf16(rng, (5, 256))
    codes, scales = O.remap_and_quantize_mxfp4(w)
    wd = O.mxfp4_dequant_plain(codes, scales)
    y1 = O.qlinear(x, wd, act=O.ACT_SILU)
    y2 = O.qlinear_mxfp4_packed(x, codes, scales, act=O.ACT_SILU)
    assert O.rel_err(y2, y1) < 1e-2
    ref = O.bf16_to_f32(x).astype(np.float64) @ wd.astype(np.float64).T
    ref = ref / (1 + np.exp(-ref))
    assert O.rel_err(y1, O.f32_to_bf16(ref.astype(np.float32))) < 1e-2


def test_epilogue_order():
    rng = np.random.default_rng(8)
    wd = (rng.standard_normal((16, 64)) * 0.1).astype(np.float32)
    x = O.randn_bf16(rng, (3, 64))
    b, mi, r = O.randn_bf16(rng, (16,), 0.1), O.randn_bf16(rng, (3, 16)), O.randn_bf16(rng, (3, 16))
    y = O.bf16_to_f32(O.qlinear(x, wd, bias=b, mul_in=mi, res=r, res_scale=0.5, act=O.ACT_GELU))
    from math import erf
    v = O.bf16_to_f32(x) @ wd.T + O.bf16_to_f32(b)
    v = 0.5 * v * (1 + np.vectorize(erf)(v / np.sqrt(2)))
    v = v * O.bf16_to_f32(mi) + O.bf16_to_f32(r) * 0.5
    assert np.max(np.abs(y - v)) < 2e-2 * np.max(np.abs(v))


def test_rope_rms_attention_small():
    rng = np.random.default_rng(9)
    B, S, Nq, Nkv, H = 2, 5, 4, 2, 16
    ep = O.rope_table(64, H, 1e4)
    x = O.randn_bf16(rng, (B, S, Nq * H))
    pos = np.arange(S, dtype=np.int64)[None]
    y = O.bf16_to_f32(O.rope_llama(x, ep, pos, Nq, H)).reshape(B, S, Nq, H)
    xf = O.bf16_to_f32(x).reshape(B, S, Nq, H)
    c, s = ep[0, :S, : H // 2], ep[1, :S, : H // 2]
    want0 = xf[..., : H // 2] * c[None, :, None] - xf[..., H // 2:] * s[None, :, None]
    assert np.max(np.abs(y[..., : H // 2] - want0)) < 2e-2
    # position >= MP leaves the row untouched
    y2 = O.rope_llama(x, ep, np.full((1, S), 64, np.int64), Nq, H)
    assert np.array_equal(y2, x)
    g = O.randn_bf16(rng, (Nq * H,))
    n = O.bf16_to_f32(O.rmsnorm(x, g, 1e-5))
    xf2 = O.bf16_to_f32(x)
    want = xf2 / np.sqrt((xf2 ** 2).mean(-1, keepdims=True) + 1e-5) * O.bf16_to_f32(g)
    assert np.max(np.abs(n - want)) < 3e-2
    # attention vs dense softmax, with a cache that already holds 3 tokens
    cache = O.KVCache()
    k0, v0 = O.randn_bf16(rng, (B, 3, Nkv, H)), O.randn_bf16(rng, (B, 3, Nkv, H))
    cache.update(k0, v0, 0)
    k1, v1 = O.randn_bf16(rng, (B, S, Nkv, H)), O.randn_bf16(rng, (B, S, Nkv, H))
    kc, vc = cache.update(k1, v1, 0)
    assert kc.shape[0] == (3 + S + 128 + 31) // 32 or kc.shape[0] >= 1
    R = Nq // Nkv
    q = O.randn_bf16(rng, (B, Nkv, S, R, H))
    mask = O.align_and_invert_mask(np.ones((B, 3 + S)))
    out = O.bf16_to_f32(O.attention(q, kc, vc, mask, 3 + S))
    K = np.concatenate([O.bf16_to_f32(k0), O.bf16_to_f32(k1)], 1)
    V = np.concatenate([O.bf16_to_f32(v0), O.bf16_to_f32(v1)], 1)
    qf = O.bf16_to_f32(q)
    for b in range(B):
        for n in range(Nkv):
            for i in range(S):
                for r in range(R):
                    sc = K[b, : 3 + i + 1, n] @ qf[b, n, i, r] / np.sqrt(H)
                    p = np.exp(sc - sc.max())
                    p /= p.sum()
                    assert np.max(np.abs(out[b, n, i, r] - p @ V[b, : 3 + i + 1, n])) < 2e-2


def test_empty_and_ragged():
    wd = np.ones((16, 64), np.float32)
    y = O.qlinear(np.zeros((0, 64), np.uint16), wd)
    assert y.shape == (0, 16)


def test_qint8_block_size_rule_matches_oracle():
    """The block size remap_and_quantize_qint8 ends up with (src/csrc/qtypes.cpp:878-889), host-side rule of the package
    against the oracle's remap on the same shapes: a divisor is kept, otherwise the next power of two below the request,
    otherwise the blocked tensor's own inner block."""
    from tpp_pytorch_extension_b200._C._qtype import qint8_block_size_used
    from tpp_pytorch_extension_b200 import _lib
    for K, req in [(4096, 256), (4096, 64), (4096, 32), (11008, 256), (192, 256), (320, 128), (14336, 512)]:
        wb = O.block_weight(np.zeros((16, K), dtype=np.uint16))
        _, bs = O.remap_qint8(wb, req)
        assert qint8_block_size_used(K, wb.shape[2] * wb.shape[4], req) == bs, (K, req, bs)
    assert qint8_block_size_used(4096, 64, 32) == 32
    assert qint8_block_size_used(192, 64, 256) == 64    # 128 and 64 are tried: 64 divides 192
    assert qint8_block_size_used(96, 32, 256) == 32     # nothing from 4096 to 64 divides 96: the tensor's own block
    for bad in (0, -4, 6):
        with pytest.raises(_lib.TpxError):
            qint8_block_size_used(4096, 64, bad)


def test_layernorm_restatement_matches_torch():
    """lyr_norm restated in numpy against torch.nn.functional.layer_norm in fp32 (one bf16 rounding apart)."""
    import torch
    rng = np.random.default_rng(5)
    x = O.f32_to_bf16(O.bf16_to_f32(O.randn_bf16(rng, (6, 320))) * 2.0 - 0.7)
    g, b = O.randn_bf16(rng, (320,), 0.5), O.randn_bf16(rng, (320,), 0.3)
    y = O.bf16_to_f32(O.layernorm(x, g, b, 1e-5))
    want = torch.nn.functional.layer_norm(torch.from_numpy(O.bf16_to_f32(x)), (320,), torch.from_numpy(O.bf16_to_f32(g)),
                                          torch.from_numpy(O.bf16_to_f32(b)), 1e-5).numpy()
    assert np.abs(y - want).max() <= 2.0 ** -7 * np.abs(want).max()


def test_fp8_casts_match_stock_torch_on_every_bf16_value():
    """bfloat8 (E5M2) / hfloat8 (E4M3) weights: the restated round-to-nearest-even cast against torch's float8 casts on
    all 65536 bf16 bit patterns (subnormals, ties, overflow) and the 256-entry decode table against torch's upcast."""
    import torch
    x = O.bf16_to_f32(np.arange(65536, dtype=np.uint16))
    finite = np.isfinite(x)
    for fmt, dt in ((O.FP8_E4M3, torch.float8_e4m3fn), (O.FP8_E5M2, torch.float8_e5m2)):
        t = torch.from_numpy(x.copy()).to(dt)
        want = t.view(torch.uint8).numpy()
        got = O.f32_to_fp8(x, fmt)
        back = t.float().numpy()
        nan = np.isnan(back)
        assert np.array_equal(got[finite & ~nan], want[finite & ~nan])
        assert np.all(np.isnan(O.fp8_dequant(got[finite & nan], fmt)))  # out of range for E4M3: NaN on both sides
        table = O.fp8_to_f32_table(fmt)
        codes = np.arange(256, dtype=np.uint8)
        ref = torch.from_numpy(codes).view(dt).float().numpy()
        assert np.array_equal(table[~np.isnan(ref)], ref[~np.isnan(ref)]) and np.all(np.isnan(table[np.isnan(ref)]))
