"""OPT: LayerNorm kernel, the fused OPT decoder layer (torch.classes.tpp_llm.OPTDecoderLayer) against the oracle's
restatement of OPTDecoderLayer::_forward, and the Hugging Face adapter (OptimizeModelForOPT) against Hugging Face's own
fp32 forward and greedy generation of a tiny random OPTForCausalLM whose linear weights were rounded to their
MXFP4-dequantized values. Tolerance: max |y - ref| / max |ref| <= 2e-2."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, make_qweight, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.mark.parametrize("rows,D", [(1, 64), (7, 768), (300, 4096)])
@pytest.mark.parametrize("f32", [False, True])
def test_layernorm_matches_oracle(cuda, rows, D, f32):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(rows + D)
    x = O.f32_to_bf16(O.bf16_to_f32(O.randn_bf16(rng, (rows, D))) * 3.0 + 1.5)  # a mean far from zero
    g, b = O.randn_bf16(rng, (D,), 0.5), O.randn_bf16(rng, (D,), 0.2)
    gd, bd = to_dev_bf16(g, cuda), to_dev_bf16(b, cuda)
    if f32:
        gd, bd = gd.float(), bd.float()
    y = to_host_bits(F.layer_norm(to_dev_bf16(x, cuda), gd, bd, 1e-5))
    ref = O.layernorm(x, g, b, 1e-5)
    # fp32 statistics on both sides: results agree to a bf16 rounding step
    assert O.rel_err(y, ref) <= 2.0 ** -7
    want = torch.nn.functional.layer_norm(torch.from_numpy(O.bf16_to_f32(x)), (D,), torch.from_numpy(O.bf16_to_f32(g)),
                                          torch.from_numpy(O.bf16_to_f32(b)), 1e-5).numpy()
    assert np.abs(O.bf16_to_f32(y) - want).max() <= 2.0 ** -6 * np.abs(want).max()


@pytest.mark.parametrize("before", [True, False])
def test_opt_layer_matches_oracle(cuda, before):
    """Prompt of 40 tokens, then two decode steps, both LayerNorm placements."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C._tpp_attn import TppCache
    rng = np.random.default_rng(11)
    B, D, NH, H, FF = 2, 256, 4, 64, 512
    names = {"q": (D, D), "k": (D, D), "v": (D, D), "o": (D, D), "fc1": (FF, D), "fc2": (D, FF)}
    W, qd = {}, {}
    for n, (N, K) in names.items():
        qd[n], W[n], _ = make_qweight(rng, N, K, "mxfp4", cuda, std=0.05)
    for n, size in (("bq", D), ("bk", D), ("bv", D), ("bo", D), ("b1", FF), ("b2", D)):
        W[n] = O.randn_bf16(rng, (size,), 0.1)
    for n, std, mean in (("g1", 0.2, 1.0), ("b_ln1", 0.1, 0.0), ("g2", 0.2, 1.0), ("b_ln2", 0.1, 0.0)):
        W[n] = O.f32_to_bf16(O.bf16_to_f32(O.randn_bf16(rng, (D,), std)) + mean)
    dv = lambda n: to_dev_bf16(W[n], cuda)
    params = [dv("g1"), dv("b_ln1"), dv("g2"), dv("b_ln2"), qd["q"], dv("bq"), qd["k"], dv("bk"), qd["v"], dv("bv"),
              qd["o"], dv("bo"), qd["fc1"], dv("b1"), qd["fc2"], dv("b2")]
    layer = F.OPTDecoderLayer(params, 0, 1e-5, 1e-5, H, before)
    cache, ocache = TppCache(), O.KVCache()
    past = 0
    for S in (40, 1, 1):
        hs = O.randn_bf16(rng, (B, S, D))
        keep = np.ones((B, past + S), np.float32)
        keep[1, :3] = 0.0  # a left-padded sequence
        am = O.align_and_invert_mask(keep)
        ref = O.opt_layer(hs, am, W, ocache, 0, NH, H, 1e-5, 1e-5, before)
        amd = cache.align_and_invert_mask(torch.from_numpy(keep).to(cuda))
        out = layer.forward([to_dev_bf16(hs, cuda), amd], cache, True)[0]
        assert O.rel_err(to_host_bits(out), ref) <= TOL, (before, S)
        past += S
    assert_no_kernel_error()


def _round_opt_linears_to_mxfp4(model):
    for layer in model.model.decoder.layers:
        a = layer.self_attn
        for lin in (a.q_proj, a.k_proj, a.v_proj, a.out_proj, layer.fc1, layer.fc2):
            w = O.f32_to_bf16(lin.weight.data.numpy().astype(np.float32))
            codes, scales = O.remap_and_quantize_mxfp4(w)
            lin.weight.data = torch.from_numpy(O.mxfp4_dequant_plain(codes, scales).astype(np.float32))
            lin.bias.data = lin.bias.data.bfloat16().float()
    for p in model.parameters():
        p.data = p.data.bfloat16().float()


@pytest.mark.parametrize("before", [True, False])
def test_opt_adapter_matches_hugging_face(cuda, before):
    transformers = pytest.importorskip("transformers")
    from tpp_pytorch_extension_b200.llm import fused_opt_infer as FO
    torch.manual_seed(2)
    cfg = transformers.OPTConfig(hidden_size=256, ffn_dim=512, num_hidden_layers=2, num_attention_heads=4, vocab_size=512,
                                 max_position_embeddings=128, word_embed_proj_dim=256, do_layer_norm_before=before, pad_token_id=1)
    model = transformers.OPTForCausalLM(cfg).float().eval()
    for layer in model.model.decoder.layers:
        a = layer.self_attn
        for lin in (a.q_proj, a.k_proj, a.v_proj, a.out_proj, layer.fc1, layer.fc2):
            lin.weight.data.normal_(0, 0.06)
            lin.bias.data.normal_(0, 0.2)
        for ln in (layer.self_attn_layer_norm, layer.final_layer_norm):
            ln.weight.data.normal_(1.0, 0.2)
            ln.bias.data.normal_(0, 0.1)
    _round_opt_linears_to_mxfp4(model)
    B, P, NEW = 3, 19, 4
    ids = torch.randint(2, cfg.vocab_size, (B, P))
    mask = torch.ones(B, P, dtype=torch.long)
    mask[2, :5] = 0  # sequence 2 is left-padded
    ids[2, :5] = cfg.pad_token_id
    with torch.no_grad():
        want = model(ids, attention_mask=mask).logits[:, -1].float()
        ref_tokens = model.generate(ids, attention_mask=mask, max_new_tokens=NEW, do_sample=False)
    runner = FO.OptimizeModelForOPT(model, torch.bfloat16, cuda, "mxfp4")
    assert type(runner.layers[0]).__name__ == "OPTDecoderLayer"
    pos = (mask.cumsum(-1) - 1).clamp(min=0)
    logits, _ = runner.forward(ids.to(cuda), mask.to(cuda), pos.to(cuda))
    got = logits[:, -1].float().cpu()
    assert float((got - want).abs().max()) <= TOL * float(want.abs().max())
    out = runner.generate(ids.to(cuda), NEW, attention_mask=mask.to(cuda)).cpu()
    assert out.shape == ref_tokens.shape
    tol = TOL * float(want.abs().max())
    for b in range(B):
        ours, theirs = int(out[b, P]), int(ref_tokens[b, P])
        assert ours == theirs or float(want[b, theirs] - want[b, ours]) <= tol, (b, ours, theirs)
    assert_no_kernel_error()
