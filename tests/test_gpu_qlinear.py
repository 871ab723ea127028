"""GPU parity: the quantized linear through the public op against the fp32-accumulated oracle.

Tolerance (stated by the task): max |y - ref| / max |ref| <= 2e-2 for bf16 outputs."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, knob_env, make_qweight, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(autouse=True, params=["tc", "tc_wide", "tc_f4", "tc_w4", "stream"])
def mxfp4_path(request):
    """Every case runs on each MXFP4 kernel family: the tcgen05 kernel with the weights on the 128-row side of the MMA,
    the tcgen05 kernel with the weights on the wide side (up to 64 tokens), the packed-fp4 tcgen05 kernel (up to 32
    tokens) and the mma.sync streaming kernel."""
    # int8 weights: the tcgen05 kind::i8 kernel (reference arithmetic) with the tensor-core families, else the streaming kernel
    with knob_env(TPX_MXFP4_PATH="stream" if request.param == "stream" else "tc",
                  TPX_TC_WIDE="1" if request.param == "tc_wide" else "0",
                  TPX_TC_F4="1" if request.param == "tc_f4" else "0",
                  TPX_TC_W4="1" if request.param == "tc_w4" else "0",
                  TPX_INT8_PATH="stream" if request.param == "stream" else "tc"):
        yield request.param


def run_fc(x_bits, q, dev, **kw):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    x = to_dev_bf16(x_bits, dev)
    y = F.fc_plain_act(x, q, **kw)
    assert_no_kernel_error()
    return to_host_bits(y)


@pytest.mark.parametrize("kind", ["mxfp4", "int8"])
@pytest.mark.parametrize("M", [1, 3, 8, 13, 32, 45])
def test_fc_plain_matches_oracle(cuda, kind, M, mxfp4_path):
    rng = np.random.default_rng(100 + M)
    N, K = 256, 512
    q, wd, _ = make_qweight(rng, N, K, kind, cuda)
    x = O.randn_bf16(rng, (M, K))
    y = run_fc(x, q, cuda)
    ref = O.qlinear(x, wd)
    assert O.rel_err(y, ref) <= TOL
    if kind == "mxfp4" or mxfp4_path == "stream":
        # exact products + fp32 accumulation: the only differences are summation order and one bf16 rounding
        # (the int8 tensor-core kernel quantises the activations as the reference does: only the wider bound holds)
        assert O.rel_err(y, ref) <= 1e-2


@pytest.mark.parametrize("kind", ["mxfp4", "int8"])
def test_split_k_and_ragged_k(cuda, kind):
    """Long K (forces a K split with the scratch reduction) and K that is not a multiple of the 128-wide tile."""
    rng = np.random.default_rng(7)
    for N, K, M in [(64, 8192, 5), (128, 2112, 16), (32, 14336, 2)]:
        q, wd, _ = make_qweight(rng, N, K, kind, cuda)
        x = O.randn_bf16(rng, (M, K))
        for _ in range(2):  # twice: the counters must come back to zero
            y = run_fc(x, q, cuda)
            assert O.rel_err(y, O.qlinear(x, wd)) <= TOL


@pytest.mark.parametrize("act,name", [(O.ACT_SILU, "silu"), (O.ACT_GELU, "gelu"), (O.ACT_RELU, "relu")])
def test_epilogues(cuda, act, name):
    rng = np.random.default_rng(21)
    N, K, M = 128, 256, 6
    q, wd, _ = make_qweight(rng, N, K, "mxfp4", cuda, std=0.05)
    x = O.randn_bf16(rng, (M, K))
    bias = O.randn_bf16(rng, (N,), 0.01)
    mul = O.randn_bf16(rng, (M, N))
    res = O.randn_bf16(rng, (M, N))
    y = run_fc(x, q, cuda, bias=to_dev_bf16(bias, cuda), act=name, mul_in=to_dev_bf16(mul, cuda),
               res=to_dev_bf16(res, cuda), res_scale=0.25)
    ref = O.qlinear(x, wd, bias=bias, mul_in=mul, res=res, res_scale=0.25, act=act)
    assert O.rel_err(y, ref) <= TOL


@pytest.mark.parametrize("kind", ["mxfp4", "int8"])
@pytest.mark.parametrize("M", [1, 8, 16, 32])
def test_gate_up_pair(cuda, kind, M):
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(33 + M)
    N, K = 512, 1024
    qg, wg, _ = make_qweight(rng, N, K, kind, cuda)
    qu, wu, _ = make_qweight(rng, N, K, kind, cuda)
    x = O.randn_bf16(rng, (M, K))
    y = to_host_bits(F.fc_gate_up(to_dev_bf16(x, cuda), qg, qu))
    assert O.rel_err(y, O.gate_up(x, wg, wu)) <= TOL
    # and against the reference's own rounding points (two GEMMs, bf16 between them)
    assert O.rel_err(y, O.gate_up(x, wg, wu, ref_rounding=True)) <= TOL


@pytest.mark.parametrize("M", [1, 5, 40, 200])
def test_rmsnorm_fused_into_linear(cuda, M):
    """RMSNorm fused into the activation split of the tensor-core linear (and the separate-kernel fallback of the other
    families) against the oracle's rmsnorm -> bf16 -> linear, single weight and gate/up pair, K not a multiple of 128."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(90 + M)
    N, K = 256, 1088
    q, wd, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    qu, wu, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    x = O.randn_bf16(rng, (M, K), 3.0)
    gamma = O.f32_to_bf16(1 + 0.2 * rng.standard_normal(K).astype(np.float32))
    xn = O.rmsnorm(x, gamma, 1e-5)
    xd, gd = to_dev_bf16(x, cuda), to_dev_bf16(gamma, cuda)
    y = to_host_bits(F.fc_plain_norm(xd, gd, 1e-5, q))
    assert_no_kernel_error()
    assert O.rel_err(y, O.qlinear(xn, wd)) <= TOL
    y2 = to_host_bits(F.fc_gate_up(xd, q, qu, "silu", norm=(gd, 1e-5)))
    assert_no_kernel_error()
    assert O.rel_err(y2, O.gate_up(xn, wd, wu)) <= TOL
    # fp32 gamma, as the reference also accepts
    g32 = torch.from_numpy(O.bf16_to_f32(gamma).copy()).to(cuda)
    y3 = to_host_bits(F.fc_plain_norm(xd, g32, 1e-5, q))
    assert np.array_equal(y3, y)


def test_int8_many_tokens(cuda):
    """Prefill-sized calls on int8 weights (unpacked to bf16 + dense GEMM) against the oracle, with post-ops and the pair."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(123)
    N, K, M = 256, 512, 200
    q, wd, _ = make_qweight(rng, N, K, "int8", cuda)
    q2, wd2, _ = make_qweight(rng, N, K, "int8", cuda)
    x = O.randn_bf16(rng, (M, K))
    bias = O.randn_bf16(rng, (N,), 0.01)
    res = O.randn_bf16(rng, (M, N))
    y = run_fc(x, q, cuda, bias=to_dev_bf16(bias, cuda), act="silu", res=to_dev_bf16(res, cuda), res_scale=0.5)
    assert O.rel_err(y, O.qlinear(x, wd, bias=bias, res=res, res_scale=0.5, act=O.ACT_SILU)) <= TOL
    y2 = to_host_bits(F.fc_gate_up(to_dev_bf16(x, cuda), q, q2))
    assert O.rel_err(y2, O.gate_up(x, wd, wd2)) <= TOL


@pytest.mark.parametrize("block", [64, 256])
@pytest.mark.parametrize("M", [1, 7, 16, 33, 64, 100, 128, 300])
def test_int8_tensor_core_kernel_matches_reference_arithmetic(cuda, M, block):
    """The tcgen05 kind::i8 kernel (activations quantised per K block, int32 block products, fp32 scaling) against the
    oracle's restatement of the reference's int8 arithmetic and against the weight-only fp32 oracle; post-ops, a gate/up
    pair, ragged N and a K split over a cluster."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    if F.int8_path() != "tc":
        pytest.skip("runs with the tensor-core families")
    with knob_env(TPX_INT8_DENSE=0):
        rng = np.random.default_rng(300 + M + block)
        N, K = 208, 1024
        q, wd, (qq, ss, bs) = make_qweight(rng, N, K, "int8", cuda, block=block)
        q2, wd2, _ = make_qweight(rng, N, K, "int8", cuda, block=block)
        x = O.randn_bf16(rng, (M, K))
        y = run_fc(x, q, cuda)
        assert O.rel_err(y, O.qlinear_int8_dynact(x, qq, ss, bs)) <= 1.5e-2  # same arithmetic up to the bf16 rounding of the running sum after every block
        assert O.rel_err(y, O.qlinear(x, wd)) <= TOL
        bias = O.randn_bf16(rng, (N,), 0.01)
        res = O.randn_bf16(rng, (M, N))
        y = run_fc(x, q, cuda, bias=to_dev_bf16(bias, cuda), act="silu", res=to_dev_bf16(res, cuda), res_scale=0.5)
        assert O.rel_err(y, O.qlinear(x, wd, bias=bias, res=res, res_scale=0.5, act=O.ACT_SILU)) <= TOL
        y2 = to_host_bits(F.fc_gate_up(to_dev_bf16(x, cuda), q, q2))
        assert O.rel_err(y2, O.gate_up(x, wd, wd2)) <= TOL
        # RMSNorm fused into the activation quantisation
        gamma = O.f32_to_bf16(1 + 0.2 * rng.standard_normal(K).astype(np.float32))
        xs = O.randn_bf16(rng, (M, K), 3.0)
        xn = O.rmsnorm(xs, gamma, 1e-5)
        y3 = to_host_bits(F.fc_plain_norm(to_dev_bf16(xs, cuda), to_dev_bf16(gamma, cuda), 1e-5, q))
        assert O.rel_err(y3, O.qlinear_int8_dynact(xn, qq, ss, bs)) <= 1.5e-2
        y4 = to_host_bits(F.fc_gate_up(to_dev_bf16(xs, cuda), q, q2, "silu", norm=(to_dev_bf16(gamma, cuda), 1e-5)))
        assert O.rel_err(y4, O.gate_up(xn, wd, wd2)) <= TOL
        assert_no_kernel_error()


@pytest.mark.parametrize("dense", [0, 1])
def test_int8_many_tokens_both_routes(cuda, dense):
    """More than 128 tokens: the int8 tensor-core kernel over several token tiles (TPX_INT8_DENSE=0) and the default
    route (weight unpacked to bf16 per call, bf16 tensor-core kernel, weight-only arithmetic), plain, with post-ops, as
    a gate/up pair and behind an RMSNorm."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    if F.int8_path() != "tc":
        pytest.skip("runs with the tensor-core families")
    rng = np.random.default_rng(77)
    M, N, K = 300, 208, 1024
    q, wd, (qq, ss, bs) = make_qweight(rng, N, K, "int8", cuda, block=64)
    q2, wd2, _ = make_qweight(rng, N, K, "int8", cuda, block=64)
    x = O.randn_bf16(rng, (M, K))
    bias, res = O.randn_bf16(rng, (N,), 0.01), O.randn_bf16(rng, (M, N))
    gamma = O.f32_to_bf16(1 + 0.2 * rng.standard_normal(K).astype(np.float32))
    with knob_env(TPX_INT8_DENSE=dense):
        y = run_fc(x, q, cuda)
        assert O.rel_err(y, O.qlinear(x, wd)) <= (TOL if dense == 0 else 1e-2)
        if dense == 0:  # the reference's arithmetic (its bf16 running sum alone moves it about 1e-2 from the exact product)
            assert O.rel_err(y, O.qlinear_int8_dynact(x, qq, ss, bs)) <= 1.5e-2
        y = run_fc(x, q, cuda, bias=to_dev_bf16(bias, cuda), act="gelu", res=to_dev_bf16(res, cuda), res_scale=0.5)
        assert O.rel_err(y, O.qlinear(x, wd, bias=bias, res=res, res_scale=0.5, act=O.ACT_GELU)) <= TOL
        y2 = to_host_bits(F.fc_gate_up(to_dev_bf16(x, cuda), q, q2))
        assert O.rel_err(y2, O.gate_up(x, wd, wd2)) <= TOL
        y3 = to_host_bits(F.fc_plain_norm(to_dev_bf16(x, cuda), to_dev_bf16(gamma, cuda), 1e-5, q))
        assert O.rel_err(y3, O.qlinear(O.rmsnorm(x, gamma, 1e-5), wd)) <= TOL
    assert_no_kernel_error()


def test_int8_reference_arithmetic_is_within_tolerance(cuda):
    """The reference's int8 path quantises activations on the fly; ours is weight-only. Both sit within the
    tolerance of the fp32 oracle, and of each other."""
    rng = np.random.default_rng(55)
    N, K, M = 128, 1024, 8
    q, wd, (qq, ss, bs) = make_qweight(rng, N, K, "int8", cuda)
    x = O.randn_bf16(rng, (M, K))
    y = run_fc(x, q, cuda)
    assert O.rel_err(y, O.qlinear_int8_dynact(x, qq, ss, bs)) <= TOL


def test_large_activations_do_not_overflow(cuda):
    """Activations far outside f16 range: the kernel's power-of-two pre-scale keeps the result exact."""
    rng = np.random.default_rng(66)
    q, wd, _ = make_qweight(rng, 64, 256, "mxfp4", cuda)
    for mag in (1e6, 1e-6, 3e20):
        x = O.f32_to_bf16((rng.standard_normal((4, 256)) * mag).astype(np.float32))
        y = run_fc(x, q, cuda)
        assert O.rel_err(y, O.qlinear(x, wd)) <= TOL


def test_linearity_full_size(cuda):
    """Size-independent property at the benchmark's full shape: f(a) + f(b) = f(a + b) for exactly representable sums."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(77)
    N, K = 14336, 4096
    q, _, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    a = O.f32_to_bf16(rng.integers(-4, 5, (8, K)).astype(np.float32))
    b = O.f32_to_bf16(rng.integers(-4, 5, (8, K)).astype(np.float32))
    ab = O.f32_to_bf16(O.bf16_to_f32(a) + O.bf16_to_f32(b))
    ya = F.fc_plain(to_dev_bf16(a, cuda), q).float()
    yb = F.fc_plain(to_dev_bf16(b, cuda), q).float()
    yab = F.fc_plain(to_dev_bf16(ab, cuda), q).float()
    err = (ya + yb - yab).abs().max().item() / yab.abs().max().item()
    assert err <= TOL
    # a zero input gives exactly zero
    z = F.fc_plain(torch.zeros(3, K, dtype=torch.bfloat16, device=cuda), q)
    assert z.abs().max().item() == 0.0


def test_config1_shape_int8_silu(cuda):
    """The int8 single-op configuration of the benchmark: int8 (block 64) [11008 x 4096], M = 32, bias, SiLU; a sampled check against the oracle."""
    rng = np.random.default_rng(0)
    N, K, M = 11008, 4096, 32
    q, wd, _ = make_qweight(rng, N, K, "int8", cuda, block=64)
    x = O.randn_bf16(rng, (M, K))
    bias = O.randn_bf16(rng, (N,), 0.01)
    y = run_fc(x, q, cuda, bias=to_dev_bf16(bias, cuda), act="silu")
    ref = O.qlinear(x, wd, bias=bias, act=O.ACT_SILU)
    assert O.rel_err(y, ref) <= TOL


@pytest.mark.parametrize("M", [5, 20])
def test_tiles_cut_between_ctas(cuda, M):
    """76 output tiles: more than half the SMs (no cluster per tile), fewer than 70 % of them (no whole tiles), so
    the (tile, k unit) list is cut into equal ranges and partial tiles are completed by the fix-up pass; plain
    linear and gate/up pair, twice (the arrival counters must come back to zero)."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(300 + M)
    N, K = 9728, 512
    q, wd, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    q2, wd2, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    x = O.randn_bf16(rng, (M, K))
    ref = O.qlinear(x, wd)
    ref_pair = O.gate_up(x, wd, wd2)
    for _ in range(2):
        assert O.rel_err(run_fc(x, q, cuda), ref) <= 1e-2
        y = F.fc_gate_up(to_dev_bf16(x, cuda), q, q2)
        assert_no_kernel_error()
        assert O.rel_err(to_host_bits(y), ref_pair) <= TOL


@pytest.mark.parametrize("M", [1, 8, 64, 200])
def test_pinned_host_input_and_output(cuda, M, mxfp4_path):
    """The MXFP4 tensor-core ops accept pinned host memory for the input and for out=: the kernels read and write it
    across the bus. Same kernels on the same values: bit-identical to the device-resident call."""
    from tpp_pytorch_extension_b200 import _lib
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(900 + M)
    N, K = 256, 512
    qg, _, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    qu, _, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    qd, _, _ = make_qweight(rng, K, N, "mxfp4", cuda)
    x_host = torch.from_numpy(O.randn_bf16(rng, (M, K)).view(np.int16)).view(torch.bfloat16).pin_memory()
    y_host = torch.zeros((M, K), dtype=torch.bfloat16).pin_memory()
    if mxfp4_path == "stream":
        with pytest.raises(_lib.TpxError):
            F.fc_gate_up(x_host, qg, qu)
        return
    want = F.fc_plain(F.fc_gate_up(x_host.to(cuda), qg, qu), qd)
    got = F.fc_plain(F.fc_gate_up(x_host, qg, qu), qd, out=y_host)
    assert got is y_host
    torch.cuda.synchronize()
    assert torch.equal(y_host, want.cpu())
    assert_no_kernel_error()
    with pytest.raises(_lib.TpxError):  # pageable host memory is refused
        F.fc_gate_up(x_host.clone(), qg, qu)
