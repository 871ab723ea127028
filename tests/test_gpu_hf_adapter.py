"""The Hugging Face adapters (OptimizeModelForLlama / OptimizeModelForQwen2) against Hugging Face's own fp32 forward of
the same tiny random model whose linear weights were replaced by their MXFP4-dequantized values (quantizing those again
gives the same codes, so both sides hold identical weights): an implementation of the block that shares no code with
this repository or its oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def _round_linears_to_mxfp4(model):
    for layer in model.model.layers:
        for lin in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.o_proj,
                    layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj):
            w = O.f32_to_bf16(lin.weight.data.numpy().astype(np.float32))
            codes, scales = O.remap_and_quantize_mxfp4(w)
            lin.weight.data = torch.from_numpy(O.mxfp4_dequant_plain(codes, scales).astype(np.float32))
            if lin.bias is not None:
                lin.bias.data = lin.bias.data.bfloat16().float()
    for p in (model.model.embed_tokens.weight, model.lm_head.weight, model.model.norm.weight):
        p.data = p.data.bfloat16().float()


@pytest.mark.parametrize("family", ["llama", "qwen2"])
def test_adapter_matches_hugging_face_forward(cuda, family):
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    torch.manual_seed(0)
    kw = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              vocab_size=512, max_position_embeddings=128, rms_norm_eps=1e-5, tie_word_embeddings=False)
    if family == "llama":
        cfg = transformers.LlamaConfig(**kw)
        model = transformers.LlamaForCausalLM(cfg)
    else:
        cfg = transformers.Qwen2Config(**kw)
        model = transformers.Qwen2ForCausalLM(cfg)
        for layer in model.model.layers:  # biases are zero-initialised: make them count
            for lin in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj):
                lin.bias.data.normal_(0, 0.5)
    model = model.float().eval()
    for layer in model.model.layers:  # larger than the default 0.02 so that the logits are not all alike
        for lin in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.o_proj,
                    layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj):
            lin.weight.data.normal_(0, 0.06)
    _round_linears_to_mxfp4(model)
    ids = torch.randint(0, cfg.vocab_size, (2, 23))
    with torch.no_grad():
        want = model(ids).logits[:, -1].float()
    opt = FL.OptimizeModelForQwen2 if family == "qwen2" else FL.OptimizeModelForLlama
    runner = opt(model, torch.bfloat16, cuda, "mxfp4")
    if family == "qwen2":
        assert type(runner.layers[0]).__name__ == "Qwen2DecoderLayer"
    logits, cache = runner.forward(ids.to(cuda))
    got = logits[:, -1].float().cpu()
    assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max())
    # one decode step against Hugging Face run on the extended sequence
    nxt = want.argmax(-1, keepdim=True)
    with torch.no_grad():
        want2 = model(torch.cat([ids, nxt], 1)).logits[:, -1].float()
    logits2, _ = runner.forward(nxt.to(cuda), cache=cache)
    got2 = logits2[:, -1].float().cpu()
    assert float((got2 - want2).abs().max()) <= 2e-2 * float(want2.abs().max())


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 2, 128), (8, 1, 128), (4, 4, 64)])
def test_adapter_gqa_ratios_and_left_padding(cuda, heads, kv_heads, head_dim):
    """Group sizes 4 and 8 at head dimension 128 (the Llama-3 and Llama-2-70B attention shapes) and plain multi-head
    attention, with one left-padded sequence in the batch: prompt logits and greedily generated tokens against Hugging
    Face's own forward / generate on the same weights (positions count the kept tokens only, in both phases)."""
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    torch.manual_seed(1)
    cfg = transformers.LlamaConfig(hidden_size=heads * head_dim, intermediate_size=512, num_hidden_layers=2, num_attention_heads=heads,
                                   num_key_value_heads=kv_heads, head_dim=head_dim, vocab_size=512, max_position_embeddings=128,
                                   rms_norm_eps=1e-5, tie_word_embeddings=False, pad_token_id=0)
    model = transformers.LlamaForCausalLM(cfg).float().eval()
    for layer in model.model.layers:
        for lin in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.o_proj,
                    layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj):
            lin.weight.data.normal_(0, 0.04)
    _round_linears_to_mxfp4(model)
    B, P, NEW = 3, 21, 5
    ids = torch.randint(1, cfg.vocab_size, (B, P))
    mask = torch.ones(B, P, dtype=torch.long)
    mask[1, :6] = 0  # sequence 1 is left-padded by six tokens
    ids[1, :6] = 0
    with torch.no_grad():
        pos = (mask.cumsum(-1) - 1).clamp(min=0)
        want = model(ids, attention_mask=mask, position_ids=pos).logits[:, -1].float()
        ref_tokens = model.generate(ids, attention_mask=mask, max_new_tokens=NEW, do_sample=False)
    runner = FL.OptimizeModelForLlama(model, torch.bfloat16, cuda, "mxfp4")
    logits, _ = runner.forward(ids.to(cuda), mask.to(cuda), pos.to(cuda))
    got = logits[:, -1].float().cpu()
    assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max())
    out = runner.generate(ids.to(cuda), NEW, attention_mask=mask.to(cuda)).cpu()
    assert out.shape == ref_tokens.shape
    # the first generated token: Hugging Face's choice, unless its own margin over our choice is a rounding matter (2e-2 of
    # the largest logit, the bound the logits themselves are held to); later tokens follow the same rule as long as the
    # sequences have not parted
    tol = 2e-2 * float(want.abs().max())
    for b in range(B):
        ours, theirs = int(out[b, P]), int(ref_tokens[b, P])
        assert ours == theirs or float(want[b, theirs] - want[b, ours]) <= tol, (b, ours, theirs)
    same_first = out[:, P] == ref_tokens[:, P]
    if bool(same_first.any()):
        agree = (out[same_first][:, P:] == ref_tokens[same_first][:, P:]).float().mean().item()
        assert agree >= 0.6, (agree, out[:, P:], ref_tokens[:, P:])
