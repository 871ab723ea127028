"""The many-token MXFP4 kernels against the oracle: the CTA-pair kernel (tcgen05.mma.cta_group::2, TPX_TC_P2=1) and the
one-CTA kernel (whole 128 x 128 tiles, three accumulators in tensor memory, TPX_TC_P=1 with TPX_TC_P2=0), forced for
shapes the library would otherwise give to the general kernel:
token counts that are not multiples of the tile, feature counts that end inside a tile, K with a tail, one and two k
steps per pipeline stage, every epilogue, the gate/up pair and the fused RMSNorm.
Tolerance: max |y - ref| / max |ref| <= 2e-2."""
import numpy as np
import pytest

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, knob_env, make_qweight, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(autouse=True, params=[(1, 2, 1), (1, 1, 1), (1, 2, 0), (0, 2, 1), (0, 1, 1)],
                ids=["pair-uks2", "pair-uks1", "pair-blockscales", "one-uks2", "one-uks1"])
def forced(request, cuda):
    """pair: CTA-pair kernel, with one activation scale per token (default) or per 32 values (TPX_TC_P_ROWS=0)."""
    p2, uks, rows = request.param
    with knob_env(TPX_MXFP4_PATH="tc", TPX_TC_P=1, TPX_TC_P2=p2, TPX_TC_P_UKS=uks, TPX_TC_P_ROWS=rows):
        yield


@pytest.mark.parametrize("M,N,K", [(65, 128, 256), (128, 416, 192), (300, 1024, 1088), (1000, 2304, 512)])
def test_plain_and_epilogues(cuda, M, N, K):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(M + N)
    q, wd, _ = make_qweight(rng, N, K, "mxfp4", cuda, std=0.05)
    q.prepare()
    x = O.randn_bf16(rng, (M, K))
    xd = to_dev_bf16(x, cuda)
    for _ in range(2):  # twice: tensor memory and barriers start clean on every launch
        y = to_host_bits(F.fc_plain(xd, q))
        assert O.rel_err(y, O.qlinear(x, wd)) <= TOL
    bias, mul, res = O.randn_bf16(rng, (N,), 0.01), O.randn_bf16(rng, (M, N)), O.randn_bf16(rng, (M, N))
    for act, name in ((O.ACT_SILU, "silu"), (O.ACT_GELU, "gelu"), (O.ACT_RELU, "relu"), (O.ACT_NONE, None)):
        y = to_host_bits(F.fc_plain_act(xd, q, to_dev_bf16(bias, cuda), name, to_dev_bf16(mul, cuda), to_dev_bf16(res, cuda), 0.25))
        assert O.rel_err(y, O.qlinear(x, wd, bias=bias, mul_in=mul, res=res, res_scale=0.25, act=act)) <= TOL
    y = to_host_bits(F.fc_plain_act(xd, q, None, None, None, to_dev_bf16(res, cuda), 1.0))
    assert O.rel_err(y, O.qlinear(x, wd, res=res)) <= TOL
    assert_no_kernel_error()


@pytest.mark.parametrize("M,N,K", [(70, 256, 256), (257, 1056, 1088), (1500, 1408, 512)])
def test_gate_up_pair(cuda, M, N, K):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(7 * M + N)
    qg, wg, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    qu, wu, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    qg.prepare(pair_with=qu)
    x = O.randn_bf16(rng, (M, K))
    for _ in range(2):
        y = to_host_bits(F.fc_gate_up(to_dev_bf16(x, cuda), qg, qu))
        assert O.rel_err(y, O.gate_up(x, wg, wu)) <= TOL
    assert_no_kernel_error()


def test_rows_longer_than_the_per_token_split_serves(cuda):
    """K = 16512: the per-token split keeps a row in registers up to 16384 elements; beyond, block scales are used."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(3)
    M, N, K = 70, 256, 16512
    q, wd, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    q.prepare()
    x = O.randn_bf16(rng, (M, K))
    y = to_host_bits(F.fc_plain(to_dev_bf16(x, cuda), q))
    assert O.rel_err(y, O.qlinear(x, wd)) <= TOL
    assert_no_kernel_error()


def test_outlier_channels_keep_their_precision(cuda):
    """A few activation channels 1000 times larger than the rest (as LLM activations have), with one scale per token: the
    bound holds with the outliers, and for the same rows without them."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(4)
    M, N, K = 130, 256, 1024
    q, wd, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    q.prepare()
    xf = O.bf16_to_f32(O.randn_bf16(rng, (M, K)))
    xf[:, [5, 300, 777]] *= 1000.0
    x = O.f32_to_bf16(xf)
    y = to_host_bits(F.fc_plain(to_dev_bf16(x, cuda), q))
    ref = O.qlinear(x, wd)
    assert O.rel_err(y, ref) <= TOL
    x2f = xf.copy()
    x2f[:, [5, 300, 777]] = 0.0
    x2 = O.f32_to_bf16(x2f)
    y2 = to_host_bits(F.fc_plain(to_dev_bf16(x2, cuda), q))
    assert O.rel_err(y2, O.qlinear(x2, wd)) <= TOL
    assert_no_kernel_error()


def test_rmsnorm_fused_into_the_split(cuda):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(5)
    M, N, K = 200, 384, 448
    q, wd, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    q.prepare()
    x = O.randn_bf16(rng, (M, K))
    gamma = O.randn_bf16(rng, (K,), 0.5)
    y = to_host_bits(F.fc_plain_norm(to_dev_bf16(x, cuda), to_dev_bf16(gamma, cuda), 1e-5, q))
    ref = O.qlinear(O.rmsnorm(x, gamma, 1e-5), wd)
    assert O.rel_err(y, ref) <= TOL
    assert_no_kernel_error()


def test_many_tiles_per_cta_match_the_general_kernel(cuda):
    """4096 tokens x 4096 features: seven tiles per CTA, accumulators reused in rotation; the general kernel is the check
    (both within bf16 rounding of each other: they sum the two activation terms in a different order)."""
    import torch
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(9)
    M, N, K = 4096, 4096, 1024
    q, _, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    q.prepare()
    xd = to_dev_bf16(O.randn_bf16(rng, (M, K)), cuda)
    res = to_dev_bf16(O.randn_bf16(rng, (M, N)), cuda)
    y = F.fc_plain_act(xd, q, None, None, None, res, 1.0).float()
    with knob_env(TPX_TC_P=0, TPX_TC_P2=0):
        y0 = F.fc_plain_act(xd, q, None, None, None, res, 1.0).float()
    assert ((y - y0).abs().max() / y0.abs().max()).item() <= 1e-2
    assert_no_kernel_error()
