"""The Hugging Face object patched in place (OptimizeModelForLlama(..., patch_model=True), the reference's behaviour):
model(...) and model.generate(...) of transformers run on the fused layers, with greedy decoding and with beam search
(whose cache reordering goes through TppCache.reorder_cache)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def _tiny_llama():
    torch.manual_seed(5)
    cfg = transformers.LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=512, max_position_embeddings=128, rms_norm_eps=1e-5,
                                   tie_word_embeddings=False, pad_token_id=0)
    model = transformers.LlamaForCausalLM(cfg).float().eval()
    for layer in model.model.layers:
        for lin in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.o_proj,
                    layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj):
            lin.weight.data.normal_(0, 0.06)
            w = O.f32_to_bf16(lin.weight.data.numpy().astype(np.float32))
            lin.weight.data = torch.from_numpy(O.mxfp4_dequant_plain(*O.remap_and_quantize_mxfp4(w)).astype(np.float32))
    for p in (model.model.embed_tokens.weight, model.lm_head.weight, model.model.norm.weight):
        p.data = p.data.bfloat16().float()
    return cfg, model


def test_generate_of_the_patched_model(cuda):
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    cfg, model = _tiny_llama()
    B, P, NEW = 3, 14, 5
    ids = torch.randint(1, cfg.vocab_size, (B, P), generator=torch.Generator().manual_seed(9))
    with torch.no_grad():
        want_logits = model(ids).logits[:, -1].float()
        want_greedy = model.generate(ids, max_new_tokens=NEW, do_sample=False)
    runner = FL.OptimizeModelForLlama(model, torch.bfloat16, cuda, "mxfp4", patch_model=True)
    assert model.tpp_runner is runner and len(model.model.layers) == 0
    with torch.no_grad():
        out = model(ids.to(cuda))
    got = out.logits[:, -1].float().cpu()
    tol = 2e-2 * float(want_logits.abs().max())
    assert float((got - want_logits).abs().max()) <= tol
    assert out.logits.shape[1] == P  # all positions unless generate asks for the last one
    assert out.past_key_values.get_seq_length() == P
    with torch.no_grad():
        greedy = model.generate(ids.to(cuda), max_new_tokens=NEW, do_sample=False).cpu()
    assert greedy.shape == want_greedy.shape
    for b in range(B):
        ours, theirs = int(greedy[b, P]), int(want_greedy[b, P])
        assert ours == theirs or float(want_logits[b, theirs] - want_logits[b, ours]) <= tol
    # the patched object and the runner's own greedy loop agree exactly (same kernels, same batch)
    assert torch.equal(greedy, runner.generate(ids.to(cuda), NEW, use_graph=False).cpu())
    with torch.no_grad():
        beams = model.generate(ids.to(cuda), max_new_tokens=NEW, do_sample=False, num_beams=3, num_return_sequences=1).cpu()
    assert beams.shape == (B, P + NEW) and bool((beams[:, :P] == ids).all())
    mine, _ = runner.beam_search(ids.to(cuda), NEW, num_beams=3)
    # Hugging Face normalises by length only between finished hypotheses; with a fixed length its best beam is ours
    assert (beams == mine[:, 0].cpu()).all(dim=1).float().mean().item() >= 2 / 3


def test_assisted_generation_through_the_patched_models(cuda):
    """Speculative (assisted) decoding as the reference's examples/llm/run_spec_decode_llama_70b.py drives it: Hugging
    Face's generate with an assistant model, both objects patched in place; the rollback of rejected draft tokens goes
    through TppCache.crop. With greedy acceptance the result is the target's own greedy continuation."""
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    cfg, target = _tiny_llama()
    torch.manual_seed(6)
    dcfg = transformers.LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=1, num_attention_heads=4,
                                    num_key_value_heads=2, vocab_size=cfg.vocab_size, max_position_embeddings=128,
                                    rms_norm_eps=1e-5, tie_word_embeddings=False, pad_token_id=0)
    draft = transformers.LlamaForCausalLM(dcfg).float().eval()
    FL.OptimizeModelForLlama(target, torch.bfloat16, cuda, "mxfp4", patch_model=True)
    FL.OptimizeModelForLlama(draft, torch.bfloat16, cuda, "mxfp4", patch_model=True)
    ids = torch.randint(1, cfg.vocab_size, (1, 12), generator=torch.Generator().manual_seed(4)).to(cuda)
    NEW = 10
    with torch.no_grad():
        plain = target.generate(ids, max_new_tokens=NEW, do_sample=False)
        cache_len_probe = target(ids).past_key_values.get_seq_length()
        assisted = target.generate(ids, max_new_tokens=NEW, do_sample=False, assistant_model=draft)
    assert cache_len_probe == ids.shape[1]
    assert assisted.shape == plain.shape
    # identical unless a verification batch (several tokens at once) rounds a near-tie the other way: then the sequences
    # part at that position and only the common prefix is comparable
    same = (assisted == plain)[0]
    first_diff = int((~same).float().argmax()) if not bool(same.all()) else plain.shape[1]
    assert first_diff >= ids.shape[1] + NEW // 2, (assisted, plain)
