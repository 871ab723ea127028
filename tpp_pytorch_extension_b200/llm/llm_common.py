"""Host-side common pieces of the LLM path, mirroring src/tpp_pytorch_extension/llm/llm_common.py:
the cache wrapper, the blocked/quantized linear, tensor-parallel sharding and the process-group plumbing."""
import torch

from .._C import _fused_llm_infer as fused_llm_cpp
from .._C import _qtype as qtype
from .._C._tpp_attn import TppCache as _CppCache
from ..utils.blocked_layout import block_weight

tensor_parallel_enabled = True


class TppCache:
    """llm_common.TppCache (llm_common.py:80-181): the object the model forward carries."""

    # what transformers' generate() asks of a cache object it did not create itself
    is_compileable = False
    is_sliding = [False]

    def __init__(self, **kwargs):
        self.tpp_cache = _CppCache()

    def __len__(self):
        return self.tpp_cache.size()

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        return self.tpp_cache.update(key_states, value_states, layer_idx)

    def get_seq_length(self, layer_idx=0):
        return self.tpp_cache.get_seq_length(layer_idx)

    def get_max_length(self):
        return None

    def get_max_cache_shape(self, layer_idx=0):
        return -1  # grows on demand

    def crop(self, max_length):
        seq_len = self.get_seq_length()
        if max_length < 0:
            max_length = seq_len - abs(max_length)
        if seq_len <= max_length:
            return
        self.tpp_cache.crop(max_length)

    def align_and_invert_mask(self, mask, inputs_embeds):
        if mask is None:
            mask = torch.ones((inputs_embeds.shape[0], inputs_embeds.shape[1]), device=inputs_embeds.device, dtype=inputs_embeds.dtype)
        return self.tpp_cache.align_and_invert_mask(mask.to(inputs_embeds.dtype), torch.finfo(inputs_embeds.dtype).min)

    def reorder_cache(self, beam_idx):
        self.tpp_cache.reorder_cache(beam_idx.to(torch.long))

    def get_cpp(self):
        return self.tpp_cache


def get_rank():
    if not tensor_parallel_enabled:
        return 0
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        return torch.distributed.get_rank()
    return 0


def get_size():
    if not tensor_parallel_enabled:
        return 1
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        return torch.distributed.get_world_size()
    return 1


def set_pg():
    """llm_common.set_pg (llm_common.py:574-578)."""
    if not tensor_parallel_enabled:
        return
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        fused_llm_cpp.set_pg(torch.distributed.distributed_c10d._get_default_group())


def shard_offsets(dim_size, size, block_size=1):
    """Split points of ShardLinear (llm_common.py:517-531): contiguous slices in units of block_size,
    boundary i at ((num_blocks * i) // size) * block_size, so uneven splits are allowed."""
    assert dim_size % block_size == 0, f"dim_size ({dim_size}) is not multiple of block_size ({block_size})"
    nb = dim_size // block_size
    return [0] + [((nb * (i + 1)) // size) * block_size for i in range(size)]


def ShardLinear(m, dim, rank, size, block_size=1):
    """dim 0 shards output features, dim 1 input features; a row-parallel bias is divided by size
    (llm_common.py:517-546)."""
    offs = shard_offsets(m.weight.shape[dim], size, block_size)
    start, end = offs[rank], offs[rank + 1]
    m.split_sizes = [offs[i + 1] - offs[i] for i in range(size)]
    if dim == 0:
        m.weight.data = m.weight.data[start:end, :].contiguous()
    else:
        m.weight.data = m.weight.data[:, start:end].contiguous()
    if m.bias is not None:
        if dim == 0:
            m.bias.data = m.bias.data[start:end].contiguous()
        else:
            m.bias.data = m.bias.data / size


def quantize_weight(w, weight_dtype, bk=16, bc=64):
    """What FixLinear does to one nn.Linear weight (llm_common.py:437-510): block as [N/bk, K/bc, bc/2, bk, 2]
    in bf16, then remap_and_quantize_* by weight_dtype ("mxfp4" | "qint8"); "bfloat8" / "hfloat8" cast the bf16 weight to
    E5M2 / E4M3 (the reference's `.to(weight_dtype)`, llm_common.py:519-522)."""
    if weight_dtype in qtype.FP8_DTYPES or weight_dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return qtype.to_fp8_weight(w, weight_dtype)
    wb = block_weight(w.to(torch.bfloat16), bk, bc)
    if weight_dtype == "mxfp4":
        return qtype.remap_and_quantize_mxfp4(wb)
    if weight_dtype == "qint8":
        return qtype.remap_and_quantize_qint8(wb)
    if weight_dtype == "qint2":
        return qtype.remap_and_quantize_qint2_intlv(wb)
    if weight_dtype in ("bf16", "bfloat16", torch.bfloat16):
        return w.to(torch.bfloat16).contiguous()  # unquantized: the bf16 kernel reads the plain matrix
    raise ValueError(f"Unknown weight_dtype {weight_dtype}")


class BlockedLinear(torch.nn.Module):
    """llm_common.BlockedLinear (llm_common.py:383-426) for quantized weights on CUDA."""

    def __init__(self, qweight, bias=None, parallel_dim=-1, split_sizes=()):
        super().__init__()
        self.weight = qweight
        self.bias = bias
        self.parallel_dim = parallel_dim
        self.split_sizes = list(split_sizes)

    def forward(self, input):
        return fc_plain(input.to(torch.bfloat16), self.weight, self.bias, self.parallel_dim, self.split_sizes)


def FixLinear(m, bk=None, bc=None, layer_dtype=torch.bfloat16, parallel_dim=None, block_size=1, weight_dtype=None):
    """llm_common.FixLinear (llm_common.py:437-510): shard (optionally), block and quantize an nn.Linear;
    returns the BlockedLinear that replaces it."""
    if not isinstance(m, torch.nn.Linear):
        return m
    pd = -1
    if parallel_dim is not None and get_size() > 1:
        ShardLinear(m, parallel_dim, get_rank(), get_size(), block_size)
        pd = parallel_dim
    if weight_dtype not in ("mxfp4", "qint8"):
        raise ValueError("this build carries quantized weights only: weight_dtype must be 'mxfp4' or 'qint8'")
    q = quantize_weight(m.weight.data, weight_dtype, bk or 16, bc or 64)
    bias = m.bias.data.to(torch.bfloat16) if m.bias is not None else None
    return BlockedLinear(q, bias, pd, getattr(m, "split_sizes", ()))


def fc_plain(input, weight, bias=None, parallel_dim=-1, split_sizes=()):
    """torch.ops.tpp_llm.fc_plain (llm_common.py:379-380 -> fc_plain_wrap, src/csrc/llm/fused_llm_infer.cpp:1514-1566)."""
    if parallel_dim == -1 or get_size() == 1:
        return fused_llm_cpp.fc_plain(input, weight, bias)
    return fc_plain_parallel(input, weight, bias, parallel_dim, list(split_sizes))


def fc_plain_parallel(input, weight, bias, parallel_dim, split_sizes):
    """Tensor-parallel linear: row-parallel (parallel_dim 1) takes this rank's slice of the input features and
    all-reduces; column-parallel (0) all-gathers the uneven output slices (fused_llm_infer.cpp:1521-1564)."""
    import torch.distributed as dist
    rank = get_rank()
    if parallel_dim == 1:
        x = input.split(split_sizes, dim=-1)[rank].contiguous()
        y = fused_llm_cpp.fc_plain(x, weight, bias)
        fused_llm_cpp.allreduce(y)
        return y
    y = fused_llm_cpp.fc_plain(input, weight, bias)
    if len(split_sizes) != get_size():
        raise ValueError("Length of split vector doesn't match group size")
    # ranks may own different numbers of output features (ShardLinear cuts in whole blocks); the collective moves
    # equal-sized pieces, so every rank sends its slice padded to the widest one
    widest = max(split_sizes)
    if y.shape[-1] != widest:
        y = torch.nn.functional.pad(y, (0, widest - y.shape[-1]))
    outs = [y.new_empty(y.shape) for _ in split_sizes]
    dist.all_gather(outs, y.contiguous(), group=fused_llm_cpp._pg)
    return torch.cat([o[..., :s] for o, s in zip(outs, split_sizes)], dim=-1)


# --------------------------------------------------------------------------- packed checkpoints
def _pack_value(v):
    if isinstance(v, qtype.QTensor):
        return {"__qtensor__": v.state()}
    if isinstance(v, torch.Tensor):
        return v.detach().cpu()
    if isinstance(v, (list, tuple)):
        return type(v)(_pack_value(x) for x in v)
    return v


def _layer_state(layer, shared_ep):
    # the rotary table is one tensor shared by all layers and the runner: stored once, with the runner
    return {"class": type(layer).__name__,
            "attrs": {k: ("__runner_ep__" if (k == "EP" and shared_ep) else _pack_value(v)) for k, v in vars(layer).items()
                      if k != "_cstruct"}}  # the C-level call's argument block holds device addresses: rebuilt on first use


def _layer_from_state(st, device):
    cls = getattr(fused_llm_cpp, st["class"])
    layer = cls.__new__(cls)
    pending = {}
    for k, v in st["attrs"].items():
        if isinstance(v, dict) and "__qtensor__" in v:
            pending[k] = v["__qtensor__"]
        elif isinstance(v, torch.Tensor):
            setattr(layer, k, v.to(device))
        else:
            setattr(layer, k, v)
    # a gate weight packed together with its up projection finds that layout by the up projection's identity
    for k in sorted(pending, key=lambda n: pending[n]["pair_tc"] is not None):
        pair = getattr(layer, "Wu", None) if pending[k]["pair_tc"] is not None else None
        setattr(layer, k, qtype.QTensor.from_state(pending[k], device, pair))
    return layer


def runner_state(runner):
    """Everything a runner holds (this rank's shard), with the weights in their quantized AND kernel layouts: loading it
    needs no quantization and no repacking."""
    import dataclasses
    st = {"runner": type(runner).__name__, "shape": dataclasses.asdict(runner.shape), "shape_class": type(runner.shape).__name__,
          "rank": get_rank(), "size": get_size(), "layers": [_layer_state(l, getattr(runner, "ep", None) is not None) for l in runner.layers], "extra": {}}
    for k, v in vars(runner).items():
        if k in ("layers", "shape", "last_graph") or k.startswith("_"):
            continue
        if isinstance(v, (torch.Tensor, qtype.QTensor, tuple, list, bool, int, float, type(None))):
            st["extra"][k] = _pack_value(v)
    return st


def runner_from_state(st, device="cuda"):
    from . import fused_llama_infer as FL
    from . import fused_gptj_infer as FG
    from . import fused_opt_infer as FO
    if (st["rank"], st["size"]) != (get_rank(), get_size()):
        raise ValueError(f"this checkpoint holds shard {st['rank']} of {st['size']}, the process is rank {get_rank()} of {get_size()}")
    set_pg()
    dev = torch.device(device)
    shape_cls = {"LlamaShape": FL.LlamaShape, "OPTShape": FO.OPTShape, "GPTJShape": FG.GPTJShape}[st["shape_class"]]
    cls = {"LlamaRunner": FL.LlamaRunner, "OPTRunner": FO.OPTRunner, "GPTJRunner": FG.GPTJRunner}[st["runner"]]
    runner = cls.__new__(cls)
    torch.nn.Module.__init__(runner)
    runner.shape = shape_cls(**st["shape"])
    runner.layers = [_layer_from_state(l, dev) for l in st["layers"]]

    def unpack(v):
        if isinstance(v, dict) and "__qtensor__" in v:
            return qtype.QTensor.from_state(v["__qtensor__"], dev)
        if isinstance(v, torch.Tensor):
            return v.to(dev)
        if isinstance(v, (list, tuple)):
            return type(v)(unpack(x) for x in v)
        return v

    for k, v in st["extra"].items():
        setattr(runner, k, unpack(v))
    for layer in runner.layers:
        if isinstance(getattr(layer, "EP", None), str):
            layer.EP = runner.ep
    return runner


def sharded_model_file(root="./sharded_model"):
    """The reference's per-rank file (examples/llm/run_generation.py:267-275)."""
    import os
    return os.path.join(root, f"r{get_rank()}_{get_size()}", "model.pt")


def save_sharded_model(runner, root="./sharded_model"):
    import os
    path = sharded_model_file(root)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    torch.save(runner_state(runner), path)
    return path


def load_sharded_model(root="./sharded_model", device="cuda"):
    return runner_from_state(torch.load(sharded_model_file(root), weights_only=False), device)


# --------------------------------------------------------------------------- Hugging Face model patched in place
def patch_hf_model(model, runner):
    """Make a Hugging Face causal-LM object run on the fused layers, as the reference's OptimizeModelFor* leave it
    (their patched LlamaModel.forward / LlamaForCausalLM.forward, llm/fused_llama_infer.py:236-408): `model(...)` and
    `model.generate(...)` (greedy, sampling, beam search: the cache object answers get_seq_length, reorder_cache and
    crop) then go through `runner`. The decoder layers of the Hugging Face object are dropped (their weights live, quantized,
    in the runner) and what remains moves to the runner's device so that generate() creates its tensors there. An empty
    cache that generate() supplies is replaced by a TppCache, a non-empty foreign cache is refused, as in the reference
    (:262-270)."""
    import types
    from transformers.modeling_outputs import CausalLMOutputWithPast
    dev = runner.embed.device
    inner = getattr(model, "model", None)
    holder = getattr(inner, "decoder", inner)  # OPT keeps its layers one level further down
    if holder is not None and hasattr(holder, "layers"):
        holder.layers = torch.nn.ModuleList()
    model.to(device=dev, dtype=torch.bfloat16)

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, use_cache=None,
                logits_to_keep=0, **unused):
        if input_ids is None:
            raise ValueError("the fused path takes input_ids (inputs_embeds is not supported)")
        cache = past_key_values
        if not isinstance(cache, TppCache):
            if cache is None or cache.get_seq_length() == 0:
                cache = TppCache()
            else:
                raise ValueError("past_key_values must be of TppCache type")
        keep_last = isinstance(logits_to_keep, int) and logits_to_keep == 1
        old = runner.only_last_logit
        runner.only_last_logit = keep_last
        try:
            logits, cache = runner.forward(input_ids.to(dev), None if attention_mask is None else attention_mask.to(dev),
                                           None if position_ids is None else position_ids.to(dev), cache)
        finally:
            runner.only_last_logit = old
        return CausalLMOutputWithPast(logits=logits, past_key_values=cache)

    model.forward = types.MethodType(forward, model)
    model.tpp_runner = runner
    return model
