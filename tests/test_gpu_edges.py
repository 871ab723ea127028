"""Edge cases of the public ops on the GPU: empty batches, one-row shapes, argument errors reported as TpxError (the
reference aborts the process on the same mistakes, src/csrc/utils.h:34-41), and a maximum-size style case (many tokens
through the fused norm + linear and attention over a cache at its capacity)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, make_qweight, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.mark.parametrize("kind", ["mxfp4", "int8"])
def test_empty_batch(cuda, kind):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(1)
    q, _, _ = make_qweight(rng, 64, 128, kind, cuda)
    q2, _, _ = make_qweight(rng, 64, 128, kind, cuda)
    x = torch.empty((0, 128), dtype=torch.bfloat16, device=cuda)
    assert F.fc_plain(x, q).shape == (0, 64)
    assert F.fc_gate_up(x, q, q2).shape == (0, 64)
    x3 = torch.empty((2, 0, 128), dtype=torch.bfloat16, device=cuda)
    assert F.fc_plain(x3, q).shape == (2, 0, 64)
    g = torch.ones(128, dtype=torch.bfloat16, device=cuda)
    assert F.rms_norm(x, g, 1e-5).shape == (0, 128)
    if kind == "mxfp4":
        assert F.fc_plain_norm(x, g, 1e-5, q).shape == (0, 64)


def test_argument_errors_are_reported(cuda):
    from tpp_pytorch_extension_b200 import _lib
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C import _qtype
    from tpp_pytorch_extension_b200._C._tpp_attn import attention
    rng = np.random.default_rng(2)
    q, _, _ = make_qweight(rng, 64, 128, "mxfp4", cuda)
    with pytest.raises(_lib.TpxError):  # in-features mismatch
        F.fc_plain(torch.zeros(3, 64, dtype=torch.bfloat16, device=cuda), q)
    with pytest.raises(_lib.TpxError):  # wrong dtype
        F.fc_plain(torch.zeros(3, 128, dtype=torch.float16, device=cuda), q)
    with pytest.raises(_lib.TpxError):  # host tensor
        F.fc_plain(torch.zeros(3, 128, dtype=torch.bfloat16), q)
    with pytest.raises(_lib.TpxError):  # a plain weight must be bf16 (then it runs on the bf16 kernel)
        F.fc_plain(torch.zeros(3, 128, dtype=torch.bfloat16, device=cuda), torch.zeros(64, 128, dtype=torch.float32, device=cuda))
    y = F.fc_plain(torch.zeros(3, 128, dtype=torch.bfloat16, device=cuda), torch.zeros(64, 128, dtype=torch.bfloat16, device=cuda))
    assert y.shape == (3, 64) and y.abs().max().item() == 0.0
    q_other, _, _ = make_qweight(rng, 32, 128, "mxfp4", cuda)
    with pytest.raises(_lib.TpxError):  # gate/up of different shapes
        F.fc_gate_up(torch.zeros(3, 128, dtype=torch.bfloat16, device=cuda), q, q_other)
    with pytest.raises(_lib.TpxError):  # head dim that no attention kernel is built for
        attention(torch.zeros(1, 1, 1, 1, 96, dtype=torch.bfloat16, device=cuda), torch.zeros(1, 1, 1, 32, 96, dtype=torch.bfloat16, device=cuda),
                  torch.zeros(1, 1, 1, 32, 96, dtype=torch.bfloat16, device=cuda), None, 1)
    # the library keeps working after errors
    y = F.fc_plain(torch.zeros(3, 128, dtype=torch.bfloat16, device=cuda), q)
    assert y.abs().max().item() == 0.0
    assert_no_kernel_error()
    assert isinstance(_lib.lib().tpx_last_error(), bytes)
    assert _qtype is not None


def test_one_token_one_tile(cuda):
    """Smallest shapes the layouts allow: N = 32, K = 64, one token."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(3)
    for kind in ("mxfp4", "int8"):
        q, wd, _ = make_qweight(rng, 32, 64, kind, cuda)
        x = O.randn_bf16(rng, (1, 64))
        y = to_host_bits(F.fc_plain(to_dev_bf16(x, cuda), q))
        assert O.rel_err(y, O.qlinear(x, wd)) <= TOL
    assert_no_kernel_error()


def test_many_tokens_fused_norm_and_full_cache(cuda):
    """1000 tokens through RMSNorm + linear (several token tiles, ragged last tile), then attention with the cache
    filled exactly to its capacity and a causal 1000-row query block."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C._tpp_attn import TppCache, attention
    rng = np.random.default_rng(4)
    M, K, N = 1000, 256, 384
    q, wd, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    x = O.randn_bf16(rng, (M, K), 2.0)
    gamma = O.f32_to_bf16(1 + 0.1 * rng.standard_normal(K).astype(np.float32))
    y = to_host_bits(F.fc_plain_norm(to_dev_bf16(x, cuda), to_dev_bf16(gamma, cuda), 1e-5, q))
    assert O.rel_err(y, O.qlinear(O.rmsnorm(x, gamma, 1e-5), wd)) <= TOL
    B, Nkv, R, H, S = 1, 2, 2, 64, 992  # 992 = 31 blocks: the cache tensor below has exactly that many
    k = O.randn_bf16(rng, (S, B, Nkv, H))
    v = O.randn_bf16(rng, (S, B, Nkv, H))
    kc = np.ascontiguousarray(k.reshape(S // 32, 32, B, Nkv, H).transpose(0, 2, 3, 1, 4))
    vc = np.ascontiguousarray(v.reshape(S // 32, 32, B, Nkv, H).transpose(0, 2, 3, 1, 4))
    qq = O.randn_bf16(rng, (B, Nkv, S, R, H))
    out = attention(to_dev_bf16(qq, cuda), to_dev_bf16(kc, cuda), to_dev_bf16(vc, cuda), None, S)
    ref = O.attention(qq, kc, vc, None, S)
    assert O.rel_err(to_host_bits(out), ref) <= TOL
    assert TppCache().get_seq_length() == 0
    assert_no_kernel_error()


def test_argmax_rows_matches_torch(cuda):
    """Greedy pick: the first of equal maxima, NaN above every number, ragged row lengths (rows not 16-byte aligned)."""
    import torch
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    g = torch.Generator(device="cpu").manual_seed(5)
    for rows, n in [(1, 128256), (16, 128256), (3, 1001), (2, 7), (5, 32000)]:
        x = torch.randn(rows, n, generator=g).bfloat16()  # bf16 rounding makes equal maxima common
        x[0, n // 2] = x[0].max()                          # and one certain tie
        y = F.argmax_rows(x.to(cuda))
        assert torch.equal(y.cpu(), x.float().argmax(-1))
    x = torch.randn(2, 4096, generator=g).bfloat16()
    x[1, 100] = float("nan")
    x[1, 3000] = float("nan")
    y = F.argmax_rows(x.to(cuda))
    assert y[1].item() == 100 and y[0].item() == int(x[0].float().argmax())
    assert F.argmax_rows(torch.empty(0, 16, dtype=torch.bfloat16, device=cuda)).shape == (0,)
