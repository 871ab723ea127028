"""Packed checkpoints: a runner saved with save_sharded_model and read back with load_sharded_model (the reference's
--save-sharded-model / --load-sharded-model, examples/llm/run_generation.py:267-275) generates the same tokens without
quantizing or repacking anything, for MXFP4 and int8 Llama models and for OPT."""
import dataclasses

import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny(family, weight_dtype, cuda):
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    from tpp_pytorch_extension_b200.llm import fused_opt_infer as FO
    if family == "opt":
        return FO.build_random_opt(FO.OPTShape(2, 256, 4, 512, 320, 128), weight_dtype, cuda, std=0.05)
    if family == "gptj":
        from tpp_pytorch_extension_b200.llm import fused_gptj_infer as FG
        return FG.build_random_gptj(FG.GPTJShape(2, 256, 4, 512, 320, 32, 128), weight_dtype, cuda, std=0.05)
    shape = FL.LlamaShape(2, 256, 4, 2, 512, 320, max_position_embeddings=128)
    return FL.build_random_llama(shape, weight_dtype, cuda, std=0.05, quantize_lm_head=(weight_dtype == "mxfp4"))


@pytest.mark.parametrize("family,weight_dtype", [("llama", "mxfp4"), ("llama", "qint8"), ("llama", "bf16"), ("opt", "mxfp4"), ("gptj", "mxfp4")])
def test_saved_shard_generates_the_same_tokens(cuda, tmp_path, monkeypatch, family, weight_dtype):
    from tpp_pytorch_extension_b200._C import _qtype
    from tpp_pytorch_extension_b200.llm import llm_common
    runner = _tiny(family, weight_dtype, cuda)
    ids = torch.randint(2, 300, (2, 17), generator=torch.Generator().manual_seed(3)).to(cuda)
    want = runner.generate(ids, 6, use_graph=False)
    path = llm_common.save_sharded_model(runner, str(tmp_path))
    assert path.endswith("r0_1/model.pt")
    calls = []
    for name in ("remap_and_quantize_mxfp4", "remap_and_quantize_qint8"):  # loading must not quantize
        monkeypatch.setattr(_qtype, name, lambda *a, _n=name, **k: calls.append(_n))
    back = llm_common.load_sharded_model(str(tmp_path), cuda)
    got = back.generate(ids, 6, use_graph=False)
    assert not calls
    assert torch.equal(got, want)
    assert dataclasses.asdict(back.shape) == dataclasses.asdict(runner.shape)
    if weight_dtype == "mxfp4" and family == "llama":
        assert back.layers[0].EP is back.ep  # the rotary table is stored once and shared again
