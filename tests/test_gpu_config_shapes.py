"""GPU parity at the benchmark configurations' own shapes, with the kernel choice left to the library.

The full-size weights are drawn on the CPU (seeded), blocked and quantized on the GPU through the C ABI; the oracle
quantizes and multiplies a sample of the output features (groups of 32 consecutive rows, including the first and the last
of the matrix: quantization blocks never span rows, so a row's codes do not depend on which other rows are present) for
ALL tokens, and the GPU result is compared on those columns. Tolerance: max |y - ref| / max |ref| <= 2e-2."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
TOL = 2e-2


def sample_rows(N, groups=8):
    """Row indices of `groups` runs of 32 consecutive output features spread over [0, N), first and last included."""
    starts = sorted({int(round(g * (N - 32) / max(1, groups - 1) / 32)) * 32 for g in range(groups)})
    return np.concatenate([np.arange(s, s + 32) for s in starts])


def quantized(w_bits, kind, dev, block=64):
    from tpp_pytorch_extension_b200._C import _qtype
    wb = to_dev_bf16(O.block_weight(w_bits), dev)
    return _qtype.remap_and_quantize_mxfp4(wb) if kind == "mxfp4" else _qtype.remap_and_quantize_qint8(wb, block)


def oracle_rows(w_bits, rows, kind, block=64):
    sub = np.ascontiguousarray(w_bits[rows])
    if kind == "mxfp4":
        return O.mxfp4_dequant_plain(*O.remap_and_quantize_mxfp4(sub))
    q, s, bs = O.remap_and_quantize_qint8(sub, block)
    return O.int8_dequant_plain(q, s, bs)


@pytest.fixture(scope="module")
def mlp(cuda):
    """The MXFP4 sweep configuration: W_gate, W_up [14336, 4096], W_down [4096, 14336] ~ N(0, 0.02)."""
    rng = np.random.default_rng(0)
    D, FF = 4096, 14336
    ws = {n: O.randn_bf16(rng, s, 0.02) for n, s in (("gate", (FF, D)), ("up", (FF, D)), ("down", (D, FF)))}
    qs = {n: quantized(w, "mxfp4", cuda) for n, w in ws.items()}
    qs["gate"].prepare(pair_with=qs["up"])
    qs["down"].prepare()
    rows_ff, rows_d = sample_rows(FF), sample_rows(D)
    ref = {"gate": oracle_rows(ws["gate"], rows_ff, "mxfp4"), "up": oracle_rows(ws["up"], rows_ff, "mxfp4"),
           "down": oracle_rows(ws["down"], rows_d, "mxfp4")}
    return qs, ref, rows_ff, rows_d


@pytest.mark.parametrize("M", [1, 8, 64, 512, 4096])
def test_mxfp4_sweep_shapes_match_oracle(cuda, mlp, M):
    """gate/up pair with SiLU*mul, then the down projection, at every token count of the sweep."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    qs, ref, rows_ff, rows_d = mlp
    rng = np.random.default_rng(1000 + M)
    x = O.randn_bf16(rng, (M, 4096))
    h = F.fc_gate_up(to_dev_bf16(x, cuda), qs["gate"], qs["up"])
    hb = to_host_bits(h)
    assert O.rel_err(hb[:, rows_ff], O.gate_up(x, ref["gate"], ref["up"])) <= TOL
    y = to_host_bits(F.fc_plain(h, qs["down"]))
    assert O.rel_err(y[:, rows_d], O.qlinear(hb, ref["down"])) <= TOL
    assert_no_kernel_error()


@pytest.mark.parametrize("M", [32, 512])
def test_int8_single_op_config_matches_oracle(cuda, M):
    """The int8 single-op configuration: W [11008, 4096], K blocks of 64, bias ~ N(0, 0.01), SiLU."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(0)
    N, K = 11008, 4096
    w = O.randn_bf16(rng, (N, K), 0.02)
    bias = O.randn_bf16(rng, (N,), 0.01)
    x = O.randn_bf16(rng, (M, K))
    q = quantized(w, "int8", cuda, 64)
    assert q.block_size == 64
    rows = sample_rows(N)
    wd = oracle_rows(w, rows, "int8", 64)
    y = to_host_bits(F.fc_plain_act(to_dev_bf16(x, cuda), q, bias=to_dev_bf16(bias, cuda), act="silu"))
    assert O.rel_err(y[:, rows], O.qlinear(x, wd, bias=bias[rows], act=O.ACT_SILU)) <= TOL
    assert_no_kernel_error()


@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 4096), (1280, 8192), (8192, 1024), (8192, 3584)])
@pytest.mark.parametrize("M", [1, 16, 64, 300])
def test_attention_projection_shapes_match_oracle(cuda, N, K, M):
    """Fused q/k/v and output-projection shapes of the Llama-3-8B configuration (6144 x 4096, 4096 x 4096) and of one
    rank of the 8-way tensor-parallel Llama-2-70B configuration (q/k/v 1280 x 8192, o 8192 x 1024, down 8192 x 3584), with
    the residual epilogue the decoder layer uses."""
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    rng = np.random.default_rng(N + K + M)
    w = O.randn_bf16(rng, (N, K), 0.02)
    q = quantized(w, "mxfp4", cuda)
    rows = sample_rows(N, 6)
    wd = oracle_rows(w, rows, "mxfp4")
    x = O.randn_bf16(rng, (M, K))
    res = O.randn_bf16(rng, (M, N))
    y = to_host_bits(F.fc_plain_act(to_dev_bf16(x, cuda), q, res=to_dev_bf16(res, cuda), res_scale=0.125))
    assert O.rel_err(y[:, rows], O.qlinear(x, wd, res=np.ascontiguousarray(res[:, rows]), res_scale=0.125)) <= TOL
    assert_no_kernel_error()
