"""GPU parity of the whole Llama runner (embedding -> fused layers -> norm -> lm_head) against the CPU oracle on a
tiny random model: prefill logits, then greedy decode steps must pick the oracle's tokens."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, to_host_bits

pytestmark = pytest.mark.gpu


def test_tiny_llama_matches_oracle(cuda):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    from tpp_pytorch_extension_b200.llm.llm_common import quantize_weight
    shape = FL.LlamaShape(2, 256, 4, 2, 512, 1024, rms_norm_eps=1e-5, rope_theta=1e4, max_position_embeddings=128)
    H, D, Nq, Nkv, FF = shape.head_dim, 256, 4, 2, 512
    rng = np.random.default_rng(42)
    ep_np = O.rope_table(128, H, 1e4)
    ep = torch.from_numpy(ep_np).to(cuda)
    embed = O.randn_bf16(rng, (shape.vocab_size, D), 0.5)
    lm = O.randn_bf16(rng, (shape.vocab_size, D), 0.05)
    layers, oracle_layers = [], []
    names = {"q": (Nq * H, D), "k": (Nkv * H, D), "v": (Nkv * H, D), "o": (D, Nq * H), "gate": (FF, D), "up": (FF, D), "down": (D, FF)}
    for i in range(shape.num_hidden_layers):
        wt, wo = {}, {}
        for nm, (n, k) in names.items():
            w = O.randn_bf16(rng, (n, k), 0.05)
            wt[nm] = torch.from_numpy(w.view(np.int16)).view(torch.bfloat16)
            c, s = O.remap_and_quantize_mxfp4(w)
            wo[nm] = O.mxfp4_dequant_plain(c, s)
        g1 = O.f32_to_bf16(1 + 0.1 * rng.standard_normal(D).astype(np.float32))
        g2 = O.f32_to_bf16(1 + 0.1 * rng.standard_normal(D).astype(np.float32))
        wt["ln1"] = torch.from_numpy(g1.view(np.int16)).view(torch.bfloat16)
        wt["ln2"] = torch.from_numpy(g2.view(np.int16)).view(torch.bfloat16)
        wo["ln1"], wo["ln2"] = g1, g2
        layers.append(FL.make_layer(shape, wt, i, ep, "mxfp4", cuda))
        oracle_layers.append(wo)
    normw = O.f32_to_bf16(np.ones(D, np.float32))
    runner = FL.LlamaRunner(shape, torch.from_numpy(embed.view(np.int16)).view(torch.bfloat16).to(cuda), layers,
                            torch.from_numpy(normw.view(np.int16)).view(torch.bfloat16).to(cuda),
                            torch.from_numpy(lm.view(np.int16)).view(torch.bfloat16).to(cuda), ep)

    def oracle_step(ids, cache, past):
        B, S = ids.shape
        hs = embed[ids]
        pos = np.arange(past, past + S, dtype=np.int64)[None]
        mask = O.align_and_invert_mask(np.ones((B, past + S)))
        for i, wo in enumerate(oracle_layers):
            hs = O.llama_layer(hs, mask, pos, wo, cache, i, Nq, Nkv, H, 1e-5, ep_np)
        last = O.rmsnorm(hs[:, -1], normw, 1e-5)
        return O.bf16_to_f32(O.qlinear(last, O.bf16_to_f32(lm)))

    B, S = 2, 19
    ids = rng.integers(0, shape.vocab_size, (B, S))
    ocache = O.KVCache()
    ref_logits = oracle_step(ids, ocache, 0)
    ids_t = torch.from_numpy(ids).to(cuda)
    logits, cache = runner.forward(ids_t)
    assert_no_kernel_error()
    got = logits[:, -1].float().cpu().numpy()
    assert np.max(np.abs(got - ref_logits)) <= 2e-2 * np.max(np.abs(ref_logits))
    # greedy decode: same tokens as the oracle for a few steps (ties aside, margins here are large)
    past = S
    nxt = ref_logits.argmax(-1)
    gpu_next = logits[:, -1].argmax(-1).cpu().numpy()
    for _ in range(3):
        assert np.array_equal(gpu_next, nxt)
        ref_logits = oracle_step(nxt[:, None], ocache, past)
        logits, cache = runner.forward(torch.from_numpy(nxt[:, None]).to(cuda), cache=cache)
        past += 1
        got = logits[:, -1].float().cpu().numpy()
        assert np.max(np.abs(got - ref_logits)) <= 2e-2 * np.max(np.abs(ref_logits))
        nxt = ref_logits.argmax(-1)
        gpu_next = got.argmax(-1)
    # generate: eager and CUDA-graph decoding agree token for token, and with the oracle's first tokens
    out_e = runner.generate(ids_t, 8, use_graph=False)
    out_g = runner.generate(ids_t, 8, use_graph=True)
    assert out_e.shape == (B, S + 8)
    assert torch.equal(out_e, out_g)
    assert runner.last_graph is not None, "the decode step was not captured in a CUDA graph"
    assert_no_kernel_error()


def test_generate_reuses_cache_and_recorded_step(cuda):
    """generate() keeps its KV cache and the CUDA graph of the decode step for the next call of the same batch size that
    fits the cache: prompts of other lengths and other padding then replay the same graph (the lengths live in device
    memory). Tokens must equal those of a runner that records anew on every call; a larger batch or a longer request
    starts a new session."""
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    shape = FL.LlamaShape(2, 256, 4, 2, 512, 512, max_position_embeddings=256)
    runner = FL.build_random_llama(shape, "mxfp4", cuda, seed=5, std=0.05)
    g = torch.Generator(device="cpu").manual_seed(7)
    prompts = [torch.randint(1, shape.vocab_size, (3, n), generator=g).to(cuda) for n in (40, 23, 57, 40)]
    masks = [None, None, torch.ones(3, 57, dtype=torch.long, device=cuda), None]
    masks[2][1, :9] = 0  # one left-padded sequence
    runner.reuse_decode_graph = False
    want = [runner.generate(p, 12, attention_mask=m) for p, m in zip(prompts, masks)]
    runner.reuse_decode_graph = True
    graphs = []
    for p, m, w in zip(prompts, masks, want):
        got = runner.generate(p, 12, attention_mask=m)
        graphs.append(runner.last_graph)
        assert torch.equal(got, w)
    # the first call sized the cache for 52 tokens (+ the reference's 128 of slack): every later request fits
    assert graphs[0] is not None and all(gr is graphs[0] for gr in graphs[1:])
    # a request beyond the cache, and another batch size, record anew
    long = runner.generate(prompts[0], 200)
    assert runner.last_graph is not graphs[0] and long.shape == (3, 240)
    runner.reuse_decode_graph = False
    assert torch.equal(long, runner.generate(prompts[0], 200))
    runner.reuse_decode_graph = True
    two = runner.generate(prompts[1][:2], 12)
    runner.reuse_decode_graph = False
    assert torch.equal(two, runner.generate(prompts[1][:2], 12))
    runner.release_session()
    assert_no_kernel_error()
