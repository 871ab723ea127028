"""GPU parity: linears on 8-bit floating-point weights (the reference's --weight-dtype bfloat8 / hfloat8,
src/tpp_pytorch_extension/llm/llm_common.py:519-522 and src/csrc/fused_gemm.h:1558-1565) against the fp32-accumulated
oracle on the same cast weights. Tolerance: max |y - ref| / max |ref| <= 2e-2 for bf16 outputs (1e-2 holds: the
products are exact, only the summation order and the final bf16 rounding differ)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
FORMATS = [("hfloat8", O.FP8_E4M3, torch.float8_e4m3fn), ("bfloat8", O.FP8_E5M2, torch.float8_e5m2)]


def make_weight(rng, N, K, name, fmt, dev, std=0.02):
    from tpp_pytorch_extension_b200.llm import llm_common
    w = O.bf16_to_f32(O.randn_bf16(rng, (N, K), std))
    codes = O.f32_to_fp8(w, fmt)
    q = llm_common.quantize_weight(torch.from_numpy(w).to(dev), name)
    # the device cast gives the oracle's codes
    assert np.array_equal(q.codes.cpu().numpy(), codes)
    return q, O.fp8_dequant(codes, fmt)


@pytest.mark.parametrize("name,fmt,dt", FORMATS)
@pytest.mark.parametrize("M", [1, 7, 16, 33, 64, 130, 300])
def test_fc_plain_fp8_matches_oracle(cuda, name, fmt, dt, M):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(10 * M + fmt)
    N, K = 384, 1088  # three tiles; K is not a multiple of the 128-wide k step
    q, wd = make_weight(rng, N, K, name, fmt, cuda)
    x = O.randn_bf16(rng, (M, K))
    bias = O.randn_bf16(rng, (N,), 0.01)
    res = O.randn_bf16(rng, (M, N), 0.5)
    y = to_host_bits(F.fc_plain_act(to_dev_bf16(x, cuda), q, bias=to_dev_bf16(bias, cuda), act="gelu", res=to_dev_bf16(res, cuda), res_scale=0.5))
    assert_no_kernel_error()
    ref = O.qlinear(x, wd, bias=bias, res=res, res_scale=0.5, act=O.ACT_GELU)
    assert O.rel_err(y, ref) <= 1e-2


@pytest.mark.parametrize("name,fmt,dt", FORMATS)
@pytest.mark.parametrize("M", [1, 16, 64, 200])
def test_gate_up_and_long_k_fp8(cuda, name, fmt, dt, M):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(77 + M + fmt)
    N, K = 512, 2048
    qg, wg = make_weight(rng, N, K, name, fmt, cuda)
    qu, wu = make_weight(rng, N, K, name, fmt, cuda)
    x = O.randn_bf16(rng, (M, K))
    y = to_host_bits(F.fc_gate_up(to_dev_bf16(x, cuda), qg, qu))
    assert_no_kernel_error()
    assert O.rel_err(y, O.gate_up(x, wg, wu)) <= 1e-2
    # few tiles and a long K: the K range is cut between the CTAs of a cluster (or a fix-up pass)
    qd, wd = make_weight(rng, 128, 14336, name, fmt, cuda)
    x2 = O.randn_bf16(rng, (M, 14336))
    for _ in range(2):  # twice: the counters in the scratch must come back to zero
        y2 = to_host_bits(F.fc_plain(to_dev_bf16(x2, cuda), qd))
        assert_no_kernel_error()
        assert O.rel_err(y2, O.qlinear(x2, wd)) <= 1e-2


def test_plain_torch_float8_tensor_is_accepted(cuda):
    """fc_plain on a bare [N, K] tensor of a torch float8 dtype (what the reference's cast leaves in nn.Linear.weight),
    and the fused RMSNorm in front of it."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(5)
    N, K, M = 256, 512, 9
    w = O.bf16_to_f32(O.randn_bf16(rng, (N, K), 0.02))
    wt = torch.from_numpy(w).to(cuda).to(torch.float8_e5m2)
    wd = O.fp8_dequant(O.f32_to_fp8(w, O.FP8_E5M2), O.FP8_E5M2)
    x = O.randn_bf16(rng, (M, K))
    gamma = O.randn_bf16(rng, (K,), 1.0)
    y = to_host_bits(F.fc_plain(to_dev_bf16(x, cuda), wt))
    assert O.rel_err(y, O.qlinear(x, wd)) <= 1e-2
    yn = to_host_bits(F.fc_plain_norm(to_dev_bf16(x, cuda), to_dev_bf16(gamma, cuda), 1e-5, wt))
    assert_no_kernel_error()
    # the fused norm keeps the normalised row in fp32 on its way into the split; the oracle rounds it to bf16 first
    assert O.rel_err(yn, O.qlinear(O.rmsnorm(x, gamma, 1e-5), wd)) <= 2e-2


@pytest.mark.parametrize("name,dt", [("bfloat8", torch.float8_e5m2), ("hfloat8", torch.float8_e4m3fn)])
def test_llama_on_fp8_weights_matches_hugging_face(cuda, name, dt):
    """OptimizeModelForLlama(..., weight_dtype="bfloat8" | "hfloat8") against Hugging Face's own fp32 forward of the same
    tiny random model whose linear weights were first rounded to the 8-bit format (casting those again is exact, so
    both sides hold identical weights): prompt logits, one decode step on the cache, greedy generation."""
    transformers = pytest.importorskip("transformers")
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=512, max_position_embeddings=128, rms_norm_eps=1e-5,
                                   tie_word_embeddings=False)
    model = transformers.LlamaForCausalLM(cfg).float().eval()
    for layer in model.model.layers:
        for lin in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.o_proj,
                    layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj):
            lin.weight.data.normal_(0, 0.06)
            lin.weight.data = lin.weight.data.bfloat16().to(dt).float()
    for p in (model.model.embed_tokens.weight, model.lm_head.weight, model.model.norm.weight):
        p.data = p.data.bfloat16().float()
    ids = torch.randint(0, cfg.vocab_size, (2, 23))
    with torch.no_grad():
        want = model(ids).logits[:, -1].float()
    runner = FL.OptimizeModelForLlama(model, torch.bfloat16, cuda, name)
    assert type(runner.layers[0].Wqkv).__name__ == "Fp8Weight"
    logits, cache = runner.forward(ids.to(cuda))
    got = logits[:, -1].float().cpu()
    assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max())
    nxt = want.argmax(-1, keepdim=True)
    with torch.no_grad():
        want2 = model(torch.cat([ids, nxt], 1)).logits[:, -1].float()
    logits2, _ = runner.forward(nxt.to(cuda), cache=cache)
    got2 = logits2[:, -1].float().cpu()
    assert float((got2 - want2).abs().max()) <= 2e-2 * float(want2.abs().max())
    out = runner.generate(ids.to(cuda), 6)
    assert out.shape == (2, 29)
    assert_no_kernel_error()


def test_fp8_weight_state_round_trip(cuda):
    """Fp8Weight.state() / QTensor.from_state (what the packed checkpoints store): the restored weight carries the format,
    the bytes and the kernel layout, and the linear on it gives the same bits."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C import _qtype
    rng = np.random.default_rng(12)
    q, _ = make_weight(rng, 128, 256, "bfloat8", O.FP8_E5M2, cuda)
    x = to_dev_bf16(O.randn_bf16(rng, (5, 256)), cuda)
    want = F.fc_plain(x, q)
    back = _qtype.QTensor.from_state(q.state(), cuda)
    assert type(back).__name__ == "Fp8Weight" and back.fmt == q.fmt and back.shape == q.shape
    assert torch.equal(back.codes, q.codes) and torch.equal(back.packed_tc()[0], q.packed_tc()[0])
    assert torch.equal(F.fc_plain(x, back), want)
    assert_no_kernel_error()
