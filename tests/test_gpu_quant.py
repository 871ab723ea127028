"""GPU parity: quantize / dequantize / repack through the C ABI against the CPU oracle, bit for bit."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu


def test_cvt_table_is_e2m1(cuda):
    """The in-kernel 4-bit expansion: byte -> (low nibble, high nibble) as f16 pairs."""
    from tpp_pytorch_extension_b200 import _lib
    out = torch.zeros(256, dtype=torch.int32, device=cuda)
    _lib.check(_lib.lib().tpx_e2m1_pair_table(out.data_ptr(), _lib.stream()))
    got = out.cpu().numpy().view(np.uint32)
    lut = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float16)
    for b in range(256):
        lo = np.uint16(got[b] & 0xffff).view(np.float16)
        hi = np.uint16(got[b] >> 16).view(np.float16)
        assert lo == lut[b & 15] and hi == lut[b >> 4], b


@pytest.mark.parametrize("N,K", [(64, 128), (128, 4096), (1024, 1024)])
def test_quantize_mxfp4_bit_exact(cuda, N, K):
    from tpp_pytorch_extension_b200._C import _qtype
    rng = np.random.default_rng(N + K)
    w = O.randn_bf16(rng, (N, K), 0.02)
    w[1, :32] = 0
    w[2, 5] = O.f32_to_bf16(np.array([3.0], np.float32))[0]
    q = _qtype.remap_and_quantize_mxfp4(to_dev_bf16(O.block_weight(w), cuda))
    codes, scales = O.remap_and_quantize_mxfp4(w)
    assert q.shape == codes.shape + (2,)
    assert np.array_equal(q.codes.cpu().numpy(), codes)
    assert np.array_equal(q.scales.cpu().numpy(), scales)
    deq = q.dequantize().cpu().numpy()
    assert np.array_equal(deq.view(np.uint32), O.dequantize_mxfp4(codes, scales).view(np.uint32))


def test_quantize_mxfp4_golden(cuda, golden):
    from tpp_pytorch_extension_b200._C import _qtype
    q = _qtype.remap_and_quantize_mxfp4(to_dev_bf16(O.block_weight(golden["blk_w"]), cuda))
    assert np.array_equal(q.codes.cpu().numpy(), golden["blk_codes"])
    assert np.array_equal(q.scales.cpu().numpy(), golden["blk_scales"])
    assert np.array_equal(q.dequantize().cpu().numpy().view(np.uint32), golden["blk_deq"].view(np.uint32))


def test_quantize_mxfp4_all_bf16_values(cuda):
    """Every finite bf16 value as a weight, grouped so that blocks see many different maxima."""
    from tpp_pytorch_extension_b200._C import _qtype
    vals = np.arange(65536, dtype=np.uint16)
    vals = vals[np.isfinite(O.bf16_to_f32(vals))]
    rng = np.random.default_rng(0)
    w = np.resize(rng.permutation(vals), (512, 128)).astype(np.uint16)
    q = _qtype.remap_and_quantize_mxfp4(to_dev_bf16(O.block_weight(w), cuda))
    codes, scales = O.remap_and_quantize_mxfp4(w)
    assert np.array_equal(q.codes.cpu().numpy(), codes)
    assert np.array_equal(q.scales.cpu().numpy(), scales)


@pytest.mark.parametrize("block", [64, 256])
def test_quantize_int8_bit_exact(cuda, block, golden):
    from tpp_pytorch_extension_b200._C import _qtype
    rng = np.random.default_rng(block)
    w = O.randn_bf16(rng, (64, 1024), 0.02)
    w[3, :256] = 0
    q = _qtype.remap_and_quantize_qint8(to_dev_bf16(O.block_weight(w), cuda), block)
    qq, ss, bs = O.remap_and_quantize_qint8(w, block)
    assert q.block_size == bs
    assert np.array_equal(q.codes.cpu().numpy(), qq)
    assert np.array_equal(q.scales.cpu().numpy().view(np.uint32), ss.view(np.uint32))
    assert np.array_equal(q.dequantize().cpu().numpy().view(np.uint32), O.dequantize_int8(qq, ss, bs).view(np.uint32))
    if block == 64:
        g = _qtype.remap_and_quantize_qint8(to_dev_bf16(O.block_weight(golden["i8_w"]), cuda), 64)
        assert np.array_equal(g.codes.cpu().numpy(), golden["i8_q"])
        assert np.array_equal(g.scales.cpu().numpy().view(np.uint32), golden["i8_scales"].view(np.uint32))


def test_quantize_rejects_bad_shapes(cuda):
    from tpp_pytorch_extension_b200 import _lib
    from tpp_pytorch_extension_b200._C import _qtype
    with pytest.raises(_lib.TpxError):
        _qtype.remap_and_quantize_mxfp4(torch.zeros(3, 2, 32, 16, 2, dtype=torch.bfloat16, device=cuda))  # K1 odd
    with pytest.raises(_lib.TpxError):
        _qtype.remap_and_quantize_mxfp4(torch.zeros(2, 2, 32, 16, 2, dtype=torch.float32, device=cuda))
    with pytest.raises(_lib.TpxError):
        _qtype.remap_and_quantize_mxfp4(torch.zeros(2, 2, 32, 16, 2, dtype=torch.bfloat16))  # CPU tensor


def test_repack_roundtrip_mxfp4(cuda):
    """The streaming layout holds exactly the codes of the interchange tensor (checked by address)."""
    from tpp_pytorch_extension_b200._C import _qtype
    rng = np.random.default_rng(11)
    N, K = 64, 192  # K not a multiple of 128: the last k tile is half padding
    w = O.randn_bf16(rng, (N, K), 0.02)
    q = _qtype.remap_and_quantize_mxfp4(to_dev_bf16(O.block_weight(w), cuda))
    pc, ps = q.packed()
    pc = pc.cpu().numpy()
    assert ps.numel() == 0
    codes, scales = O.remap_and_quantize_mxfp4(w)
    KT = (K + 127) // 128
    tiles = pc.reshape(N // 16, KT, 1088)
    words = np.ascontiguousarray(tiles[:, :, :1024]).view(np.uint32).reshape(N // 16, KT, 2, 32, 4)
    sc = tiles[:, :, 1024:].reshape(N // 16, KT, 16, 4)
    for n in range(N):
        for k in range(KT * 128):
            nt, kt, r = n // 16, k // 128, n % 16
            h, g = r // 8, r % 8
            kk = k % 128
            b, j = kk // 32, (kk % 32)
            hh, rem = j // 16, j % 16
            t, i = rem // 4, rem % 4
            got = (int(words[nt, kt, h, 4 * g + t, b]) >> (4 * (4 * hh + i))) & 15
            if k < K:
                byte = codes[n // 32, k // 64, (k % 64) // 2, n % 32]
                want = (byte >> 4) if (k & 1) else (byte & 15)
                assert sc[nt, kt, r, b] == scales[n // 32, k // 64, (k % 64) // 32, n % 32]
            else:
                want = 0
                assert sc[nt, kt, r, b] == 0
            assert got == want, (n, k)


@pytest.mark.parametrize("K,block", [(256, 32), (192, 256), (4096, 128)])
def test_quantize_qint8_block_sizes(cuda, K, block):
    """Block sizes other than the default: 32 (twice as many scales as blocks of 64), a request that does not divide K
    (the reference falls back to a smaller power of two, src/csrc/qtypes.cpp:881-888), and a bad one refused."""
    from tpp_pytorch_extension_b200 import _lib
    from tpp_pytorch_extension_b200._C import _qtype
    rng = np.random.default_rng(K + block)
    w = O.randn_bf16(rng, (32, K), 0.02)
    wb = O.block_weight(w)
    q = _qtype.remap_and_quantize_qint8(to_dev_bf16(wb, cuda), block)
    qq, ss, bs = O.remap_and_quantize_qint8(w, block)
    assert q.block_size == bs and tuple(q.codes.shape) == qq.shape and tuple(q.scales.shape) == ss.shape
    assert np.array_equal(q.codes.cpu().numpy(), qq)
    assert np.array_equal(q.scales.cpu().numpy().view(np.uint32), ss.view(np.uint32))
    with pytest.raises(_lib.TpxError):
        _qtype.remap_and_quantize_qint8(to_dev_bf16(wb, cuda), 0)
