"""The reference's own call forms, executed on the GPU against the oracle: the package imported under the reference's
name, operators under torch.ops.tpp_llm, classes under torch.classes.tpp_llm (TORCH_LIBRARY(tpp_llm),
src/csrc/llm/fused_llm_infer.cpp:1589-1611, src/csrc/llm/attn.cpp:1971-1983), used as the reference's Python layer uses
them (src/tpp_pytorch_extension/llm/llm_common.py:87,380; llm/fused_llama_infer.py:93,165), and the debug timers."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import assert_no_kernel_error, make_qweight, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu
TOL = 2e-2


def test_reference_call_forms_match_oracle(cuda, capsys):
    import tpp_pytorch_extension  # noqa: F401  (the reference's package name)
    from tpp_pytorch_extension._C import _qtype  # noqa: F401
    from tpp_pytorch_extension.llm.fused_llama_infer import OptimizeModelForLlama  # noqa: F401
    from tpp_pytorch_extension_b200 import _timers
    rng = np.random.default_rng(21)
    # fc_plain as llm_common.BlockedLinear.forward calls it, on a quantized and on a bf16 weight
    N, K, M = 256, 512, 5
    q, wd, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    x = O.randn_bf16(rng, (M, K))
    bias = O.randn_bf16(rng, (N,), 0.1)
    y = torch.ops.tpp_llm.fc_plain(to_dev_bf16(x, cuda), q, to_dev_bf16(bias, cuda), -1, [])
    assert O.rel_err(to_host_bits(y), O.qlinear(x, wd, bias=bias)) <= TOL
    wb = O.randn_bf16(rng, (N, K), 0.05)
    y = torch.ops.tpp_llm.fc_plain(to_dev_bf16(x, cuda), to_dev_bf16(wb, cuda), torch.Tensor().to(cuda), -1, [])
    assert O.rel_err(to_host_bits(y), O.qlinear(x, O.bf16_to_f32(wb))) <= TOL
    # the decoder block and the cache through the TorchScript class names
    D, Nq, Nkv, H, FF, B, MP = 256, 4, 2, 64, 512, 2, 128
    eps = 1e-5
    names = {"q": (Nq * H, D), "k": (Nkv * H, D), "v": (Nkv * H, D), "o": (D, Nq * H), "gate": (FF, D), "up": (FF, D), "down": (D, FF)}
    qt, W = {}, {}
    for nm, (n, k) in names.items():
        qt[nm], W[nm], _ = make_qweight(rng, n, k, "mxfp4", cuda, std=0.05)
    W["ln1"], W["ln2"] = O.f32_to_bf16(np.ones(D, np.float32)), O.f32_to_bf16(np.ones(D, np.float32))
    ep = O.rope_table(MP, H, 1e4)
    params = [to_dev_bf16(W["ln1"], cuda), qt["q"], qt["k"], qt["v"], qt["o"], to_dev_bf16(W["ln2"], cuda), qt["gate"], qt["up"],
              qt["down"], torch.from_numpy(ep).to(cuda)]
    cpp_block = torch.classes.tpp_llm.LlamaDecoderLayer(params, 0, eps, H, MP, H)
    cache = torch.classes.tpp_llm.TppCache()
    ocache = O.KVCache()
    _timers.enable(True)
    _timers.reset_debug_timers()
    try:
        total = 0
        for S in (19, 1):
            hs = O.randn_bf16(rng, (B, S, D))
            pos = np.arange(total, total + S, dtype=np.int64)[None]
            total += S
            m01 = np.ones((B, total))
            am = cache.align_and_invert_mask(torch.from_numpy(m01).to(cuda))
            out = cpp_block.forward([to_dev_bf16(hs, cuda), am, torch.from_numpy(pos).to(cuda)], cache, True)
            ref = O.llama_layer(hs, O.align_and_invert_mask(m01), pos, W, ocache, 0, Nq, Nkv, H, eps, ep)
            assert O.rel_err(to_host_bits(out[0]), ref) <= TOL
        assert cache.get_seq_length() == 20 and cache.size() == 1
        summ = _timers.summary()
        for scope in ("fqkv_gemm", "rotary", "mha", "proj_gemm", "i_gemm", "o_gemm"):
            assert summ[scope][0] == 2 and summ[scope][1] > 0.0, scope
        tpp_pytorch_extension.print_debug_timers()
        assert "i_gemm" in capsys.readouterr().out
        tpp_pytorch_extension.reset_debug_timers()
        assert not _timers.summary()
    finally:
        _timers.enable(False)
    assert_no_kernel_error()
