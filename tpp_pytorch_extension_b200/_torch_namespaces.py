"""Publishes the path's operators and classes under the names the reference registers with TorchScript
(TORCH_LIBRARY(tpp_llm), src/csrc/llm/fused_llm_infer.cpp:1589-1611 and src/csrc/llm/attn.cpp:1971-1983), so that code
written against the reference runs unchanged:

    torch.ops.tpp_llm.fc_plain(input, weight, bias, parallel_dim, split_sizes)
    torch.ops.tpp_llm.set_pg(pg) / torch.ops.tpp_llm.allreduce(t)
    torch.classes.tpp_llm.TppCache()
    torch.classes.tpp_llm.LlamaDecoderLayer(params, layer_idx, eps, head_dim, max_positions, rotary_dim).forward(inputs, cache, use_cache)
    torch.classes.tpp_llm.Qwen2DecoderLayer(...)
    torch.classes.tpp_llm.OPTDecoderLayer(params, layer_idx, eps1, eps2, head_dim, do_layer_norm_before)
    torch.classes.tpp_llm.GPTJBlock(params, layer_idx, eps, head_dim, max_positions, rotary_dim)

The quantized weight carrier of this package is a Python object (the reference's custom quantizer tensors cannot exist
on a CUDA device without its C++ classes), which an operator schema cannot name; the entries are therefore attached to
the torch.ops / torch.classes namespace objects directly instead of going through the dispatcher. Calls look and behave
the same; torch.jit.script of code that uses them is not supported."""
import torch


def install():
    from ._C import _fused_llm_infer as F
    from ._C import _tpp_attn as A
    ops = torch.ops.tpp_llm
    for name, fn in (("fc_plain", F.fc_plain), ("set_pg", F.set_pg), ("allreduce", F.allreduce)):
        setattr(ops, name, fn)
    classes = torch.classes.tpp_llm
    for name, cls in (("TppCache", A.TppCache), ("LlamaDecoderLayer", F.LlamaDecoderLayer), ("Qwen2DecoderLayer", F.Qwen2DecoderLayer),
                      ("OPTDecoderLayer", F.OPTDecoderLayer), ("GPTJBlock", F.GPTJBlock)):
        setattr(classes, name, cls)
