"""GPT-J: the rotary kernel (adjacent pairs, partial rotary) bit-exact against the oracle, attention at head size 256,
the fused block (torch.classes.tpp_llm.GPTJBlock) against the oracle's restatement of GPTJBlock::_forward, and the
Hugging Face adapter against Hugging Face's own fp32 forward of a tiny random GPTJForCausalLM (head size 256, rotary 64)
whose linear weights were rounded to their MXFP4-dequantized values. Tolerance: max |y - ref| / max |ref| <= 2e-2."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, make_qweight, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _emb_pos(MP, HR):
    inv = 1.0 / (10000 ** (np.arange(0, HR, 2, dtype=np.float32) / HR))
    ang = np.outer(np.arange(MP, dtype=np.float32), inv).astype(np.float32)
    return np.concatenate([np.sin(ang), np.cos(ang)], axis=1).astype(np.float32)


@pytest.mark.parametrize("H,HR", [(64, 32), (256, 64), (128, 128)])
def test_gptj_rotary_and_cache_append_are_bit_exact(cuda, H, HR):
    from tpp_pytorch_extension_b200 import _lib
    rng = np.random.default_rng(H + HR)
    B, S, N, MP = 2, 9, 3, 16
    qkv = O.randn_bf16(rng, (B, S, 3 * N * H))
    ep = _emb_pos(MP, HR)
    pos = np.stack([np.arange(4, 4 + S), np.arange(9, 9 + S)]).astype(np.int64)  # the second row runs past the table
    q_ref = O.rope_gptj(qkv[..., :N * H], ep, pos, N, H)
    k_ref = O.rope_gptj(qkv[..., N * H:2 * N * H], ep, pos, N, H)
    qd = to_dev_bf16(qkv, cuda)
    q_out = torch.empty((B, N, S, 1, H), dtype=torch.bfloat16, device=cuda)
    kc = torch.zeros((1, B, N, 32, H), dtype=torch.bfloat16, device=cuda)
    vc = torch.zeros_like(kc)
    _lib.check(_lib.lib().tpx_rope_kv_update_gptj(qd.data_ptr(), torch.from_numpy(ep).to(cuda).data_ptr(), torch.from_numpy(pos).to(cuda).data_ptr(),
                                                  B, S, N, N, H, MP, HR, 2, 0, 32, None, q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), None, None,
                                                  _lib.stream()))
    got_q = to_host_bits(q_out).reshape(B, N, S, H).transpose(0, 2, 1, 3).reshape(B, S, N * H)
    assert np.array_equal(got_q, q_ref)
    got_k = to_host_bits(kc)[0, :, :, :S].transpose(0, 2, 1, 3).reshape(B, S, N * H)
    assert np.array_equal(got_k, k_ref)
    got_v = to_host_bits(vc)[0, :, :, :S].transpose(0, 2, 1, 3).reshape(B, S, N * H)
    assert np.array_equal(got_v, qkv[..., 2 * N * H:])


@pytest.mark.parametrize("Sq,ctx", [(1, 70), (5, 40), (80, 0)])
def test_attention_head_size_256(cuda, Sq, ctx):
    from tpp_pytorch_extension_b200._C._tpp_attn import attention
    rng = np.random.default_rng(Sq + ctx)
    B, N, H = 2, 2, 256
    key_len = ctx + Sq
    S1 = (key_len + 31) // 32
    q = O.randn_bf16(rng, (B, N, Sq, 1, H))
    kc, vc = O.randn_bf16(rng, (S1, B, N, 32, H)), O.randn_bf16(rng, (S1, B, N, 32, H))
    keep = np.ones((B, key_len), np.float32)
    keep[1, :2] = 0.0
    am = O.align_and_invert_mask(keep)
    ref = O.attention(q, kc, vc, am, key_len, causal=True)
    out = attention(to_dev_bf16(q, cuda), to_dev_bf16(kc, cuda), to_dev_bf16(vc, cuda), to_dev_bf16(am, cuda), key_len, causal=True)
    assert O.rel_err(to_host_bits(out), ref) <= TOL


@pytest.mark.parametrize("H,HR", [(256, 64), (64, 32)])
def test_gptj_block_matches_oracle(cuda, H, HR):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C._tpp_attn import TppCache
    rng = np.random.default_rng(31 + H)
    B, NH, FF, MP = 2, 2, 1024, 128
    D = NH * H
    names = {"q": (D, D), "k": (D, D), "v": (D, D), "o": (D, D), "fc_in": (FF, D), "fc_out": (D, FF)}
    W, qd = {}, {}
    for n, (N, K) in names.items():
        qd[n], W[n], _ = make_qweight(rng, N, K, "mxfp4", cuda, std=0.04)
    W["b_in"], W["b_out"] = O.randn_bf16(rng, (FF,), 0.1), O.randn_bf16(rng, (D,), 0.1)
    W["g"] = O.f32_to_bf16(O.bf16_to_f32(O.randn_bf16(rng, (D,), 0.2)) + 1.0)
    W["b_ln"] = O.randn_bf16(rng, (D,), 0.1)
    ep = _emb_pos(MP, HR)
    dv = lambda n: to_dev_bf16(W[n], cuda)
    block = F.GPTJBlock([dv("g"), dv("b_ln"), qd["q"], qd["k"], qd["v"], qd["o"], qd["fc_in"], dv("b_in"), qd["fc_out"], dv("b_out"),
                         torch.from_numpy(ep).to(cuda)], 0, 1e-5, H, MP, HR)
    cache, ocache = TppCache(), O.KVCache()
    past = 0
    for S in (37, 1, 1):
        hs = O.randn_bf16(rng, (B, S, D))
        pos = np.arange(past, past + S, dtype=np.int64)[None]
        keep = np.ones((B, past + S), np.float32)
        keep[1, :3] = 0.0
        ref = O.gptj_layer(hs, O.align_and_invert_mask(keep), pos, W, ocache, 0, NH, H, 1e-5, ep)
        amd = cache.align_and_invert_mask(torch.from_numpy(keep).to(cuda))
        out = block.forward([to_dev_bf16(hs, cuda), amd, torch.from_numpy(pos).to(cuda)], cache, True)[0]
        assert O.rel_err(to_host_bits(out), ref) <= TOL, S
        past += S
    assert_no_kernel_error()


def test_gptj_adapter_matches_hugging_face(cuda):
    transformers = pytest.importorskip("transformers")
    from tpp_pytorch_extension_b200.llm import fused_gptj_infer as FG
    torch.manual_seed(7)
    cfg = transformers.GPTJConfig(n_embd=512, n_head=2, n_layer=2, n_positions=128, rotary_dim=64, vocab_size=512, n_inner=1024,
                                  pad_token_id=0)
    model = transformers.GPTJForCausalLM(cfg).float().eval()
    for blk in model.transformer.h:
        for lin in (blk.attn.q_proj, blk.attn.k_proj, blk.attn.v_proj, blk.attn.out_proj, blk.mlp.fc_in, blk.mlp.fc_out):
            lin.weight.data.normal_(0, 0.05)
            w = O.f32_to_bf16(lin.weight.data.numpy().astype(np.float32))
            lin.weight.data = torch.from_numpy(O.mxfp4_dequant_plain(*O.remap_and_quantize_mxfp4(w)).astype(np.float32))
        blk.mlp.fc_in.bias.data.normal_(0, 0.1)
        blk.mlp.fc_out.bias.data.normal_(0, 0.1)
        blk.ln_1.weight.data.normal_(1.0, 0.2)
        blk.ln_1.bias.data.normal_(0, 0.1)
    model.lm_head.bias.data.normal_(0, 0.2)
    for p in model.parameters():
        p.data = p.data.bfloat16().float()
    B, P, NEW = 2, 17, 4
    ids = torch.randint(1, cfg.vocab_size, (B, P), generator=torch.Generator().manual_seed(8))
    with torch.no_grad():
        want = model(ids).logits[:, -1].float()
        ref_tokens = model.generate(ids, max_new_tokens=NEW, do_sample=False)
    runner = FG.OptimizeModelForGPTJ(model, torch.bfloat16, cuda, "mxfp4")
    assert type(runner.layers[0]).__name__ == "GPTJBlock" and runner.layers[0].H == 256
    logits, _ = runner.forward(ids.to(cuda))
    got = logits[:, -1].float().cpu()
    tol = TOL * float(want.abs().max())
    assert float((got - want).abs().max()) <= tol
    out = runner.generate(ids.to(cuda), NEW).cpu()
    assert out.shape == ref_tokens.shape
    for b in range(B):
        ours, theirs = int(out[b, P]), int(ref_tokens[b, P])
        assert ours == theirs or float(want[b, theirs] - want[b, ours]) <= tol, (b, ours, theirs)
    assert_no_kernel_error()
