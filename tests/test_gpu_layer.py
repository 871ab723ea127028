"""GPU parity: RMSNorm, RoPE + KV-cache write, attention and the whole Llama decoder layer against the oracle.
Tolerance: max |y - ref| / max |ref| <= 2e-2 (bf16 outputs, fp32-accumulated oracle)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, make_qweight, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
TOL = 2e-2


def test_rmsnorm(cuda):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(1)
    for rows, D in [(1, 4096), (7, 256), (33, 8192)]:
        x, g = O.randn_bf16(rng, (rows, D)), O.randn_bf16(rng, (D,))
        y = to_host_bits(F.rms_norm(to_dev_bf16(x, cuda), to_dev_bf16(g, cuda), 1e-5))
        assert O.rel_err(y, O.rmsnorm(x, g, 1e-5)) <= 1e-2
        y32 = to_host_bits(F.rms_norm(to_dev_bf16(x, cuda), torch.from_numpy(O.bf16_to_f32(g)).to(cuda), 1e-5))
        assert np.array_equal(y32, y)


def _rope_case(cuda, B, S, Nq, Nkv, H, offset, pos):
    from tpp_pytorch_extension_b200 import _lib
    rng = np.random.default_rng(B * 100 + S)
    MP = 64
    ep = O.rope_table(MP, H, 1e4)
    qkv = O.randn_bf16(rng, (B, S, (Nq + 2 * Nkv) * H))
    cap = (offset + S + 31) // 32 * 32 + 32
    kc = torch.zeros((cap // 32, B, Nkv, 32, H), dtype=torch.bfloat16, device=cuda)
    vc = torch.zeros_like(kc)
    R = Nq // Nkv
    q = torch.empty((B, Nkv, S, R, H), dtype=torch.bfloat16, device=cuda)
    pos_t = torch.from_numpy(pos).to(cuda)
    qkv_t, ep_t = to_dev_bf16(qkv, cuda), torch.from_numpy(ep).to(cuda)  # keep the device copies alive across the launch
    _lib.check(_lib.lib().tpx_rope_kv_update(qkv_t.data_ptr(), ep_t.data_ptr(),
                                             pos_t.data_ptr(), B, S, Nq, Nkv, H, MP, H, pos.shape[0], offset, cap,
                                             None, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), _lib.stream()))
    torch.cuda.synchronize()
    qr = qkv[..., : Nq * H]
    kr = qkv[..., Nq * H: (Nq + Nkv) * H]
    vr = qkv[..., (Nq + Nkv) * H:]
    q_ref = O.rope_llama(qr, ep, pos, Nq, H).reshape(B, S, Nkv, R, H).transpose(0, 2, 1, 3, 4)
    k_ref = O.rope_llama(kr, ep, pos, Nkv, H).reshape(B, S, Nkv, H)
    v_ref = vr.reshape(B, S, Nkv, H)
    assert np.array_equal(to_host_bits(q), np.ascontiguousarray(q_ref))
    kh, vh = to_host_bits(kc), to_host_bits(vc)
    for s in range(S):
        t = offset + s
        assert np.array_equal(kh[t // 32, :, :, t % 32], k_ref[:, s])
        assert np.array_equal(vh[t // 32, :, :, t % 32], v_ref[:, s])
    assert not kh[(offset + S + 31) // 32:].any()  # nothing beyond the written tokens


def test_rope_kv_update_bit_exact(cuda):
    _rope_case(cuda, 2, 5, 8, 2, 128, 0, np.arange(5, dtype=np.int64)[None])
    _rope_case(cuda, 3, 1, 4, 4, 64, 37, np.array([[37], [12], [63]], dtype=np.int64))
    # positions at and beyond the table leave the row untouched
    _rope_case(cuda, 1, 3, 2, 1, 128, 30, np.array([[62, 64, 100]], dtype=np.int64))


def test_rope_rejects_overflow(cuda):
    from tpp_pytorch_extension_b200 import _lib
    z = torch.zeros(4096, dtype=torch.bfloat16, device=cuda)
    f = torch.zeros(4096, dtype=torch.float32, device=cuda)
    p = torch.zeros(8, dtype=torch.int64, device=cuda)
    rc = _lib.lib().tpx_rope_kv_update(z.data_ptr(), f.data_ptr(), p.data_ptr(), 1, 4, 2, 1, 64, 8, 64, 1, 30, 32,
                                       None, z.data_ptr(), z.data_ptr(), z.data_ptr(), _lib.stream())
    assert rc == 1 and b"capacity" in _lib.lib().tpx_last_error()


@pytest.mark.parametrize("prefill_kernel", ["tcgen05", "mma_sync"])
@pytest.mark.parametrize("B,Nkv,R,H,ctx,Sq", [(1, 2, 4, 128, 100, 1), (2, 1, 8, 128, 1500, 1), (1, 8, 1, 64, 64, 64),
                                              (2, 2, 4, 128, 300, 37), (16, 8, 4, 128, 2048, 1), (1, 1, 2, 128, 4100, 3),
                                              (2, 2, 1, 64, 333, 333), (1, 1, 4, 128, 700, 260), (1, 2, 4, 128, 2048, 2048)])
def test_attention_matches_oracle(cuda, B, Nkv, R, H, ctx, Sq, prefill_kernel):
    """Decoding (one query), short and long prompts, prompts on top of a cached context, causal 2048 x 2048; prompts of
    64 rows or more run on the tcgen05 kernel or, with TPX_ATTN_TC=0, on the mma.sync kernel."""
    from tests.gpu_util import knob_env
    with knob_env(TPX_ATTN_TC="1" if prefill_kernel == "tcgen05" else "0"):
        _attention_case(cuda, B, Nkv, R, H, ctx, Sq)


def _attention_case(cuda, B, Nkv, R, H, ctx, Sq):
    from tpp_pytorch_extension_b200._C._tpp_attn import TppCache, attention
    rng = np.random.default_rng(ctx + Sq)
    key_len = ctx
    S1 = (key_len + 128 + 31) // 32
    kc = np.zeros((S1, B, Nkv, 32, H), np.uint16)
    vc = np.zeros_like(kc)
    k = O.randn_bf16(rng, (key_len, B, Nkv, H))
    v = O.randn_bf16(rng, (key_len, B, Nkv, H))
    for t in range(key_len):
        kc[t // 32, :, :, t % 32] = k[t]
        vc[t // 32, :, :, t % 32] = v[t]
    q = O.randn_bf16(rng, (B, Nkv, Sq, R, H))
    m01 = np.ones((B, key_len))
    if B > 1:
        m01[1, :5] = 0  # left padding on one sequence
    cache = TppCache()
    am = cache.align_and_invert_mask(torch.from_numpy(m01).to(cuda))
    am_ref = O.align_and_invert_mask(m01)
    assert np.array_equal(to_host_bits(am), am_ref)
    out = attention(to_dev_bf16(q, cuda), to_dev_bf16(kc, cuda), to_dev_bf16(vc, cuda), am, key_len)
    ref = O.attention(q, kc, vc, am_ref, key_len)
    assert O.rel_err(to_host_bits(out), ref) <= TOL
    out2 = attention(to_dev_bf16(q, cuda), to_dev_bf16(kc, cuda), to_dev_bf16(vc, cuda), am, key_len, out_bsnrh=True)
    want = np.ascontiguousarray(ref.transpose(0, 2, 1, 3, 4)).reshape(B, Sq, -1)
    assert O.rel_err(to_host_bits(out2), want) <= TOL
    assert_no_kernel_error()


def test_cache_growth_and_crop(cuda):
    from tpp_pytorch_extension_b200._C._tpp_attn import TppCache
    c = TppCache()
    k = torch.randn(2, 3, 40, 64, device=cuda).bfloat16()
    kc, vc = c.update(k, k, 0)
    assert c.get_seq_length() == 40 and c.get_capacity() == (40 + 128 + 31) // 32 * 32 and c.size() == 1
    assert torch.equal(kc[1, :, :, 7], k[:, :, 39])
    k2 = torch.randn(2, 3, 200, 64, device=cuda).bfloat16()
    kc, _ = c.update(k2, k2, 0)
    assert c.get_seq_length() == 240 and c.get_capacity() >= 240 + 128
    assert torch.equal(kc[1, :, :, 7], k[:, :, 39]) and torch.equal(kc[7, :, :, 15], k2[:, :, 199])
    c.crop(100)
    assert c.get_seq_length() == 100
    c.crop(500)
    assert c.get_seq_length() == 100
    # growth appended pages: the first run of pages is still the tensor the first update returned (nothing was copied)
    lc = c.layers[0]
    assert len(lc.arenas) == 2 and lc.arenas[0][0].data_ptr() == c.layers[0].arenas[0][0].data_ptr()
    assert lc.k_ptrs.numel() == lc.pages() and int(lc.k_ptrs[0].item()) == lc.arenas[0][0].data_ptr()
    assert int(lc.k_ptrs[lc.arenas[0][0].shape[0]].item()) == lc.arenas[1][0].data_ptr()


def test_paged_cache_layer_matches_oracle(cuda, monkeypatch):
    """A decoder layer decoding across page-run boundaries: with no spare capacity (KV_CACHE_INC_SIZE = 0) the cache
    grows by one run of pages every 32 tokens, the kernels follow the page tables (tpx_rope_kv_update_paged,
    tpx_attention_paged), earlier pages never move, and every step matches the oracle; then a prompt chunk on top of the
    paged cache (the mma.sync prefill path) and the gathered cache tensor."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C import _tpp_attn as A
    monkeypatch.setattr(A, "KV_CACHE_INC_SIZE", 0)
    rng = np.random.default_rng(77)
    D, Nq, Nkv, H, FF, B, MP = 256, 4, 2, 64, 512, 2, 256
    eps = 1e-5
    names = {"q": (Nq * H, D), "k": (Nkv * H, D), "v": (Nkv * H, D), "o": (D, Nq * H), "gate": (FF, D), "up": (FF, D), "down": (D, FF)}
    qt, W = {}, {}
    for nm, (n, k) in names.items():
        qt[nm], W[nm], _ = make_qweight(rng, n, k, "mxfp4", cuda, std=0.05)
    W["ln1"], W["ln2"] = O.f32_to_bf16(np.ones(D, np.float32)), O.f32_to_bf16(np.ones(D, np.float32))
    ep = O.rope_table(MP, H, 1e4)
    layer = F.LlamaDecoderLayer([to_dev_bf16(W["ln1"], cuda), qt["q"], qt["k"], qt["v"], qt["o"], to_dev_bf16(W["ln2"], cuda),
                                 qt["gate"], qt["up"], qt["down"], torch.from_numpy(ep).to(cuda)], 0, eps, H, MP, H)
    cache, ocache = A.TppCache(), O.KVCache()
    total = 0
    first_ptr = None
    for S in (37,) + (1,) * 30 + (70, 1):
        hs = O.randn_bf16(rng, (B, S, D))
        pos = np.arange(total, total + S, dtype=np.int64)[None]
        total += S
        m01 = np.ones((B, total))
        am = cache.align_and_invert_mask(torch.from_numpy(m01).to(cuda))
        out = layer.forward([to_dev_bf16(hs, cuda), am, torch.from_numpy(pos).to(cuda)], cache, True)
        ref = O.llama_layer(hs, O.align_and_invert_mask(m01), pos, W, ocache, 0, Nq, Nkv, H, eps, ep)
        assert O.rel_err(to_host_bits(out[0]), ref) <= TOL, (S, total)
        lc = cache.layers[0]
        if first_ptr is None:
            first_ptr = lc.arenas[0][0].data_ptr()
        assert lc.arenas[0][0].data_ptr() == first_ptr and cache.get_seq_length() == total
    assert len(cache.layers[0].arenas) >= 3
    kc_ref = ocache.layers[0]["k"]
    got = to_host_bits(cache.get(0)[0])
    n = min(got.shape[0], kc_ref.shape[0], (total + 31) // 32)
    assert O.rel_err(got[:n], kc_ref[:n]) <= TOL
    assert_no_kernel_error()


@pytest.mark.parametrize("kind", ["mxfp4", "int8"])
def test_llama_layer_prefill_then_decode(cuda, kind):
    """One decoder layer (GQA, 2 kv heads x 2) through prefill of 37 tokens and three decode steps."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C._tpp_attn import TppCache
    rng = np.random.default_rng(5)
    D, Nq, Nkv, H, FF, B, MP = 256, 4, 2, 64, 512, 2, 128
    eps = 1e-5
    names = {"q": (Nq * H, D), "k": (Nkv * H, D), "v": (Nkv * H, D), "o": (D, Nq * H), "gate": (FF, D), "up": (FF, D), "down": (D, FF)}
    qt, W = {}, {}
    for nm, (n, k) in names.items():
        qt[nm], W[nm], _ = make_qweight(rng, n, k, kind, cuda, std=0.05)
    W["ln1"], W["ln2"] = O.f32_to_bf16(1 + 0.1 * rng.standard_normal(D).astype(np.float32)), O.f32_to_bf16(1 + 0.1 * rng.standard_normal(D).astype(np.float32))
    ep = O.rope_table(MP, H, 1e4)
    layer = F.LlamaDecoderLayer([to_dev_bf16(W["ln1"], cuda), qt["q"], qt["k"], qt["v"], qt["o"], to_dev_bf16(W["ln2"], cuda),
                                 qt["gate"], qt["up"], qt["down"], torch.from_numpy(ep).to(cuda)], 0, eps, H, MP, H)
    cache, ocache = TppCache(), O.KVCache()
    total = 0
    for S in (37, 1, 1, 1):
        hs = O.randn_bf16(rng, (B, S, D))
        pos = np.arange(total, total + S, dtype=np.int64)[None]
        total += S
        m01 = np.ones((B, total))
        m01[1, :3] = 0
        am = cache.align_and_invert_mask(torch.from_numpy(m01).to(cuda))
        out = layer.forward([to_dev_bf16(hs, cuda), am, torch.from_numpy(pos).to(cuda)], cache, True)
        ref = O.llama_layer(hs, O.align_and_invert_mask(m01), pos, W, ocache, 0, Nq, Nkv, H, eps, ep)
        assert_no_kernel_error()
        assert O.rel_err(to_host_bits(out[0]), ref) <= TOL, S
        assert cache.get_seq_length(0) == total
        kc_ref, _ = ocache.layers[0]["k"], ocache.layers[0]["v"]
        got = to_host_bits(out[1])
        n = min(got.shape[0], kc_ref.shape[0])
        assert O.rel_err(got[:n], kc_ref[:n]) <= TOL


def test_layer_as_two_c_calls_equals_the_kernel_by_kernel_path(cuda):
    """LlamaDecoderLayer.forward issues the layer as two C calls (tpx_llama_layer_attention / tpx_llama_layer_mlp) where it
    can; with TPX_LAYER_C=0 it launches kernel by kernel from Python. Same kernels, same order: bit-identical outputs and
    caches, through a prompt, decode steps and a cache that grows by pages."""
    from tests.gpu_util import knob_env
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C._tpp_attn import TppCache
    rng = np.random.default_rng(25)
    D, Nq, Nkv, H, FF, B, MP = 256, 4, 2, 64, 512, 2, 512
    names = {"q": (Nq * H, D), "k": (Nkv * H, D), "v": (Nkv * H, D), "o": (D, Nq * H), "gate": (FF, D), "up": (FF, D), "down": (D, FF)}
    qt = {nm: make_qweight(rng, n, k, "mxfp4", cuda, std=0.05)[0] for nm, (n, k) in names.items()}
    g1 = to_dev_bf16(O.f32_to_bf16(1 + 0.1 * rng.standard_normal(D).astype(np.float32)), cuda)
    g2 = to_dev_bf16(O.f32_to_bf16(1 + 0.1 * rng.standard_normal(D).astype(np.float32)), cuda)
    bias = [to_dev_bf16(O.randn_bf16(rng, (n,), 0.1), cuda) for n in (Nq * H, Nkv * H, Nkv * H)]
    ep = torch.from_numpy(O.rope_table(MP, H, 1e4)).to(cuda)
    layer = F.Qwen2DecoderLayer([g1, qt["q"], qt["k"], qt["v"], qt["o"], g2, qt["gate"], qt["up"], qt["down"]] + bias + [ep], 0, 1e-5, H, MP, H)
    assert layer._c_level_ok()
    steps = [(70, None)] + [(1, None)] * 3 + [(200, None), (1, None)]  # the 200-token chunk makes the cache grow: paged from then on
    inputs, total = [], 0
    for S, _ in steps:
        hs = to_dev_bf16(O.randn_bf16(rng, (B, S, D)), cuda)
        pos = torch.arange(total, total + S, device=cuda).unsqueeze(0)
        total += S
        inputs.append((hs, pos, total))
    outs = {}
    for mode in (1, 0):
        with knob_env(TPX_LAYER_C=mode):
            cache = TppCache()
            got = []
            for hs, pos, tot in inputs:
                am = cache.align_and_invert_mask(torch.ones((B, tot), device=cuda))
                got.append(layer.forward([hs, am, pos], cache, True)[0].clone())
            outs[mode] = (got, cache.layers[0].k.clone(), cache.layers[0].v.clone(), cache.layers[0].contiguous())
    assert not outs[1][3]  # the cache did become paged
    for a, b in zip(outs[1][0], outs[0][0]):
        assert torch.equal(a, b)
    assert torch.equal(outs[1][1], outs[0][1]) and torch.equal(outs[1][2], outs[0][2])
    assert_no_kernel_error()


def test_gate_up_hands_its_output_to_down_as_activation_terms(cuda):
    """With at most 64 tokens (by default: 33 to 64) tpx_llama_layer_mlp lets the gate/up kernel's epilogue write the activation terms the down
    projection reads (no split kernel in between) when both kernels chosen for the shapes can: an MLP of the Llama-3-8B
    width (112 whole gate/up tiles). Same arithmetic on the same bf16 values: outputs bit-identical to TPX_HANDOFF=0, with
    one launch fewer per layer call; covers both producers (packed-fp4 kernel up to 32 tokens, wide kernel beyond) and
    both consumers (wide kernel up to 16 tokens, 128-row kernel beyond)."""
    from tests.gpu_util import knob_env
    from tpp_pytorch_extension_b200 import _lib
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C._tpp_attn import TppCache
    rng = np.random.default_rng(31)
    D, Nq, Nkv, H, FF, MP = 512, 4, 2, 64, 14336, 64
    names = {"q": (Nq * H, D), "k": (Nkv * H, D), "v": (Nkv * H, D), "o": (D, Nq * H), "gate": (FF, D), "up": (FF, D), "down": (D, FF)}
    qt = {nm: make_qweight(rng, n, k, "mxfp4", cuda, std=0.05)[0] for nm, (n, k) in names.items()}
    g1 = to_dev_bf16(O.f32_to_bf16(1 + 0.1 * rng.standard_normal(D).astype(np.float32)), cuda)
    g2 = to_dev_bf16(O.f32_to_bf16(1 + 0.1 * rng.standard_normal(D).astype(np.float32)), cuda)
    ep = torch.from_numpy(O.rope_table(MP, H, 1e4)).to(cuda)
    layer = F.LlamaDecoderLayer([g1, qt["q"], qt["k"], qt["v"], qt["o"], g2, qt["gate"], qt["up"], qt["down"], ep], 0, 1e-5, H, MP, H)
    assert layer._c_level_ok()
    for B in (1, 3, 16, 17, 32, 33, 64, 5):  # 5 after 64: rows of the buffer beyond the live tokens hold older terms
        hs = to_dev_bf16(O.randn_bf16(rng, (B, 1, D)), cuda)
        pos = torch.zeros((1, 1), dtype=torch.int64, device=cuda)
        res = {}
        for mode in ("1", "0"):
            with knob_env(TPX_HANDOFF=mode, TPX_HANDOFF_MIN_TOKENS=1):  # by default only 33 to 64 tokens are handed over
                cache = TppCache()
                am = cache.align_and_invert_mask(torch.ones((B, 1), device=cuda))
                layer.forward([hs, am, pos], cache, True)  # warm: buffers, maps
                cache = TppCache()
                c0 = _lib.lib().tpx_launch_count()
                out = layer.forward([hs, am, pos], cache, True)[0].clone()
                res[mode] = (out, _lib.lib().tpx_launch_count() - c0)
        assert torch.equal(res["1"][0], res["0"][0]), B
        assert res["1"][1] == res["0"][1] - 1, (B, res["1"][1], res["0"][1])
    assert_no_kernel_error()


def test_qwen2_layer_has_qkv_bias(cuda):
    """Qwen2DecoderLayer = the Llama block plus q/k/v biases (src/csrc/llm/fused_llm_infer.cpp:1289-1510)."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C._tpp_attn import TppCache
    rng = np.random.default_rng(15)
    D, Nq, Nkv, H, FF, B, MP = 256, 4, 2, 64, 512, 2, 64
    eps = 1e-6
    names = {"q": (Nq * H, D), "k": (Nkv * H, D), "v": (Nkv * H, D), "o": (D, Nq * H), "gate": (FF, D), "up": (FF, D), "down": (D, FF)}
    qt, W = {}, {}
    for nm, (n, k) in names.items():
        qt[nm], W[nm], _ = make_qweight(rng, n, k, "mxfp4", cuda, std=0.05)
    W["ln1"], W["ln2"] = O.f32_to_bf16(np.ones(D, np.float32)), O.f32_to_bf16(np.ones(D, np.float32))
    for nm, n in (("bq", Nq * H), ("bk", Nkv * H), ("bv", Nkv * H)):
        W[nm] = O.randn_bf16(rng, (n,), 0.5)
    ep = O.rope_table(MP, H, 1e6)
    layer = F.Qwen2DecoderLayer([to_dev_bf16(W["ln1"], cuda), qt["q"], qt["k"], qt["v"], qt["o"], to_dev_bf16(W["ln2"], cuda),
                                 qt["gate"], qt["up"], qt["down"], to_dev_bf16(W["bq"], cuda), to_dev_bf16(W["bk"], cuda),
                                 to_dev_bf16(W["bv"], cuda), torch.from_numpy(ep).to(cuda)], 0, eps, H, MP, H)
    cache, ocache = TppCache(), O.KVCache()
    total = 0
    for S in (20, 1):
        hs = O.randn_bf16(rng, (B, S, D))
        pos = np.arange(total, total + S, dtype=np.int64)[None]
        total += S
        m01 = np.ones((B, total))
        am = cache.align_and_invert_mask(torch.from_numpy(m01).to(cuda))
        out = layer.forward([to_dev_bf16(hs, cuda), am, torch.from_numpy(pos).to(cuda)], cache, True)
        ref = O.llama_layer(hs, O.align_and_invert_mask(m01), pos, W, ocache, 0, Nq, Nkv, H, eps, ep)
        assert_no_kernel_error()
        assert O.rel_err(to_host_bits(out[0]), ref) <= TOL, S
    # the biases matter: without them the result is far off
    W0 = {k: v for k, v in W.items() if k not in ("bq", "bk", "bv")}
    no_bias = O.llama_layer(hs, O.align_and_invert_mask(m01), pos, W0, O.KVCache(), 0, Nq, Nkv, H, eps, ep)
    assert O.rel_err(no_bias, ref) > TOL


def test_reorder_cache_gathers_beams(cuda):
    """Beam-search reordering: sequence i continues the history of old sequence beam_idx[i]; a cache of CB sequences
    is first repeated per beam (src/csrc/llm/attn.h:327-403)."""
    from tpp_pytorch_extension_b200._C._tpp_attn import TppCache
    rng = np.random.default_rng(5)
    CB, Nkv, S, H = 2, 2, 40, 64
    k = O.randn_bf16(rng, (CB, Nkv, S, H))
    v = O.randn_bf16(rng, (CB, Nkv, S, H))
    cache = TppCache()
    kc, vc = cache.update(to_dev_bf16(k, cuda), to_dev_bf16(v, cuda), 0)
    beams = torch.tensor([1, 0, 3, 3])  # 2 beams per cached sequence: rows (0,0,1,1) after the repeat
    cache.reorder_cache(beams)
    lc = cache.layer(0)
    assert lc.k.shape[1] == 4 and lc.offset == S
    got_k, got_v = to_host_bits(lc.k), to_host_bits(lc.v)
    src = np.array([0, 0, 1, 1])[beams.numpy()]
    for i in range(4):
        for t in (0, 31, 32, S - 1):
            assert np.array_equal(got_k[t // 32, i, :, t % 32], k[src[i], :, t])
            assert np.array_equal(got_v[t // 32, i, :, t % 32], v[src[i], :, t])
    cache.reorder_cache(torch.tensor([3, 2, 1, 0]))
    got_k = to_host_bits(cache.layer(0).k)
    assert np.array_equal(got_k[0, 0, :, 5], k[src[3], :, 5])
    with pytest.raises(Exception):
        cache.reorder_cache(torch.tensor([0, 1, 2]))
