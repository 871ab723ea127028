"""GPU parity: ternary ("qint2") weights, remap_and_quantize_qint2_intlv (src/csrc/qtypes.cpp:1004-1073), which the
reference multiplies through its int8 GEMM class (src/csrc/fused_gemm.h:1531-1535). Quantizer: bit-exact against the
oracle's restatement. Linear: max |y - ref| / max |ref| <= 2e-2 against the fp32-accumulated oracle on the dequantized
weight (the int8 kernels quantise the activations per block as the reference does)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
TOL = 2e-2


def quantize(w_bits, dev, block_size=None):
    from tpp_pytorch_extension_b200._C import _qtype
    from tpp_pytorch_extension_b200.llm import llm_common
    wb = llm_common.block_weight(to_dev_bf16(w_bits, dev), 16, 64)
    return _qtype.remap_and_quantize_qint2_intlv(wb, block_size)


@pytest.mark.parametrize("N,K,req,used", [(96, 512, None, 256), (64, 320, None, 64), (32, 1024, 512, 512), (128, 384, 256, 128)])
def test_quantizer_is_bit_exact(cuda, N, K, req, used):
    rng = np.random.default_rng(N + K)
    w = O.randn_bf16(rng, (N, K), 0.02)
    w[3, :40] = 0  # part of a block of zeros; a whole zero block below
    w[5, :used] = 0
    q = quantize(w, cuda, req)
    packed, scales, B = O.remap_and_quantize_qint2(w, req or 256)
    assert B == used == q.block_size
    assert q.shape == (N // 32, K // B, B // 4, 32, 4)
    assert np.array_equal(q.codes.cpu().numpy(), packed)
    assert np.array_equal(q.scales.cpu().numpy(), scales)
    wd = O.qint2_dequant_plain(packed, scales, B)
    assert np.array_equal(q.dequantize().cpu().numpy(), wd)
    assert set(np.unique(q.plain_codes().cpu().numpy())) <= {-1, 0, 1}


@pytest.mark.parametrize("M", [1, 9, 64, 200])
def test_linear_on_qint2_weights(cuda, M):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(40 + M)
    N, K = 256, 1024
    wg, wu = O.randn_bf16(rng, (N, K), 0.02), O.randn_bf16(rng, (N, K), 0.02)
    qg, qu = quantize(wg, cuda), quantize(wu, cuda)
    dg = O.qint2_dequant_plain(*O.remap_and_quantize_qint2(wg))
    du = O.qint2_dequant_plain(*O.remap_and_quantize_qint2(wu))
    x = O.randn_bf16(rng, (M, K))
    bias = O.randn_bf16(rng, (N,), 0.1)
    y = to_host_bits(F.fc_plain_act(to_dev_bf16(x, cuda), qg, bias=to_dev_bf16(bias, cuda), act="silu"))
    assert O.rel_err(y, O.qlinear(x, dg, bias=bias, act=O.ACT_SILU)) <= TOL
    y2 = to_host_bits(F.fc_gate_up(to_dev_bf16(x, cuda), qg, qu))
    assert O.rel_err(y2, O.gate_up(x, dg, du)) <= TOL
    assert_no_kernel_error()


def test_llama_on_qint2_weights_runs(cuda):
    """--weight-dtype qint2 end to end on a tiny Llama shape: the fused q/k/v weight is the concatenation of the three
    carriers, prompt logits are finite and greedy decoding completes."""
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    shape = FL.LlamaShape(2, 256, 4, 2, 512, 512, max_position_embeddings=128)
    runner = FL.build_random_llama(shape, "qint2", cuda, seed=3)
    assert type(runner.layers[0].Wqkv).__name__ == "QInt2Tensor"
    ids = torch.randint(0, shape.vocab_size, (2, 17), device=cuda)
    logits, _ = runner.forward(ids)
    assert torch.isfinite(logits.float()).all()
    assert runner.generate(ids, 5).shape == (2, 22)
    assert_no_kernel_error()
