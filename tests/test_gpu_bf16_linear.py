"""GPU parity of the bf16-weight linear (tcgen05 kind::f16) through the public op against the fp32-accumulated oracle:
ragged shapes, every token-tile size, post-ops, the lm_head shape of the Llama-3-8B configuration on sampled rows, and a
tiny Llama with unquantized weights. Tolerance: max |y - ref| / max |ref| <= 2e-2 (1e-2 held for the plain linear)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.mark.parametrize("M", [1, 5, 16, 17, 40, 64, 100, 129, 300, 700])
@pytest.mark.parametrize("N,K", [(256, 512), (1000, 520), (136, 64), (128, 2056)])
def test_bf16_linear_matches_oracle(cuda, M, N, K):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(M * 7 + N + K)
    w = O.randn_bf16(rng, (N, K), 0.05)
    x = O.randn_bf16(rng, (M, K))
    y = to_host_bits(F.fc_plain(to_dev_bf16(x, cuda), to_dev_bf16(w, cuda)))
    assert O.rel_err(y, O.qlinear(x, O.bf16_to_f32(w))) <= 1e-2
    bias = O.randn_bf16(rng, (N,), 0.1)
    res = O.randn_bf16(rng, (M, N))
    mul = O.randn_bf16(rng, (M, N))
    y = to_host_bits(F.fc_plain_act(to_dev_bf16(x, cuda), to_dev_bf16(w, cuda), bias=to_dev_bf16(bias, cuda), act="gelu",
                                    mul_in=to_dev_bf16(mul, cuda), res=to_dev_bf16(res, cuda), res_scale=0.5))
    ref = O.qlinear(x, O.bf16_to_f32(w), bias=bias, mul_in=mul, res=res, res_scale=0.5, act=O.ACT_GELU)
    assert O.rel_err(y, ref) <= TOL
    assert_no_kernel_error()


@pytest.mark.parametrize("M", [1, 16, 64])
def test_lm_head_shape_matches_oracle(cuda, M):
    """lm_head of the Llama-3-8B configuration, [128256, 4096] bf16: sampled output rows, all tokens."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    g = torch.Generator(device=cuda).manual_seed(3)
    w = (torch.randn(128256, 4096, generator=g, device=cuda) * 0.02).to(torch.bfloat16)
    rng = np.random.default_rng(M)
    x = O.randn_bf16(rng, (M, 4096))
    rows = np.concatenate([np.arange(0, 64), np.arange(64000, 64064), np.arange(128256 - 64, 128256)])
    y = to_host_bits(F.fc_plain(to_dev_bf16(x, cuda), w))
    wr = to_host_bits(w[torch.from_numpy(rows).to(cuda)])
    assert y.shape == (M, 128256)
    assert O.rel_err(y[:, rows], O.qlinear(x, O.bf16_to_f32(wr))) <= 1e-2
    assert_no_kernel_error()


def test_tiny_llama_with_bf16_weights_matches_oracle(cuda):
    """The runner on unquantized bf16 weights (the reference's default weight type) against the oracle's layer."""
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    shape = FL.LlamaShape(2, 256, 4, 2, 512, 1000, rms_norm_eps=1e-5, rope_theta=1e4, max_position_embeddings=128)
    H, D, Nq, Nkv, FF = shape.head_dim, 256, 4, 2, 512
    rng = np.random.default_rng(7)
    ep_np = O.rope_table(128, H, 1e4)
    ep = torch.from_numpy(ep_np).to(cuda)
    embed = O.randn_bf16(rng, (shape.vocab_size, D), 0.5)
    lm = O.randn_bf16(rng, (shape.vocab_size, D), 0.05)
    names = {"q": (Nq * H, D), "k": (Nkv * H, D), "v": (Nkv * H, D), "o": (D, Nq * H), "gate": (FF, D), "up": (FF, D), "down": (D, FF)}
    layers, oracle_layers = [], []
    tb = lambda a: torch.from_numpy(a.view(np.int16)).view(torch.bfloat16)
    for i in range(shape.num_hidden_layers):
        wt, wo = {}, {}
        for nm, (n, k) in names.items():
            w = O.randn_bf16(rng, (n, k), 0.05)
            wt[nm], wo[nm] = tb(w), O.bf16_to_f32(w)
        g1 = O.f32_to_bf16(1 + 0.1 * rng.standard_normal(D).astype(np.float32))
        g2 = O.f32_to_bf16(1 + 0.1 * rng.standard_normal(D).astype(np.float32))
        wt["ln1"], wt["ln2"], wo["ln1"], wo["ln2"] = tb(g1), tb(g2), g1, g2
        layers.append(FL.make_layer(shape, wt, i, ep, "bf16", cuda))
        oracle_layers.append(wo)
    normw = O.f32_to_bf16(np.ones(D, np.float32))
    runner = FL.LlamaRunner(shape, tb(embed).to(cuda), layers, tb(normw).to(cuda), tb(lm).to(cuda), ep)
    B, S = 2, 21
    ids = rng.integers(0, shape.vocab_size, (B, S))
    hs = embed[ids]
    cache = O.KVCache()
    mask = O.align_and_invert_mask(np.ones((B, S)))
    for i, wo in enumerate(oracle_layers):
        hs = O.llama_layer(hs, mask, np.arange(S, dtype=np.int64)[None], wo, cache, i, Nq, Nkv, H, 1e-5, ep_np)
    ref = O.bf16_to_f32(O.qlinear(O.rmsnorm(hs[:, -1], normw, 1e-5), O.bf16_to_f32(lm)))
    logits, _ = runner.forward(torch.from_numpy(ids).to(cuda))
    got = logits[:, -1].float().cpu().numpy()
    assert got.shape == ref.shape
    assert np.max(np.abs(got - ref)) <= TOL * np.max(np.abs(ref))
    out = runner.generate(torch.from_numpy(ids).to(cuda), 6)
    assert out.shape == (B, S + 6) and np.array_equal(out[:, S].cpu().numpy(), ref.argmax(-1))
    assert_no_kernel_error()
