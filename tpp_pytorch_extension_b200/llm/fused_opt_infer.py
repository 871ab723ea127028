"""OPT on the fused decoder layers, mirroring src/tpp_pytorch_extension/llm/fused_opt_infer.py.

`OptimizeModelForOPT(model, dtype, device, weight_dtype)` takes a Hugging Face OPTForCausalLM, shards (tensor parallel),
blocks and quantizes the linears of every decoder layer as FixOPTDecoderLayer does (fused_opt_infer.py of the
reference: q/k/v/fc1 column-parallel, out_proj/fc2 row-parallel with the bias divided by the group size) and returns a
runner with the Llama runner's interface (forward, generate, decode with a CUDA-graph decode loop). What differs from
Llama: learned position embeddings added before the first layer (positions = cumsum(mask) - 1 + 2, as OPT's
OPTLearnedPositionalEmbedding), LayerNorm with bias, biases on every linear, ReLU, no rotary embedding, the head tied
to the token embedding. `build_random_opt` builds the same runner from a shape alone."""
from dataclasses import dataclass

import torch

from .._C import _fused_llm_infer as fused_llm_cpp
from . import llm_common
from .fused_llama_infer import LlamaRunner, _lm_head, _shard
from .llm_common import TppCache, get_size, quantize_weight

POSITION_OFFSET = 2  # OPTLearnedPositionalEmbedding keeps two leading rows for padding conventions


@dataclass
class OPTShape:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    ffn_dim: int
    vocab_size: int
    max_position_embeddings: int = 2048
    do_layer_norm_before: bool = True
    layer_norm_eps: float = 1e-5

    @property
    def head_dim(self):
        return self.hidden_size // self.num_attention_heads

    # the names the shared runner reads
    @property
    def num_key_value_heads(self):
        return self.num_attention_heads


def make_opt_layer(shape, w, layer_idx, weight_dtype, device):
    """w: plain [N, K] tensors q,k,v,o,fc1,fc2, their biases bq,bk,bv,bo,b1,b2, LayerNorm parameters g1,b_ln1,g2,b_ln2.
    Sharding: heads for q/k/v (rows) and out_proj (columns), 64-wide blocks for the MLP; a row-parallel bias is divided
    by the group size (ShardLinear, llm_common.py:517-546)."""
    H = shape.head_dim
    size = get_size()
    plan = {"q": (0, H), "k": (0, H), "v": (0, H), "o": (1, H), "fc1": (0, 64), "fc2": (1, 64)}
    qs = {n: quantize_weight(_shard(w[n].to(device), dim, blk), weight_dtype) for n, (dim, blk) in plan.items()}

    def col_bias(name, blk):
        return _shard(w[name].to(device).reshape(-1, 1), 0, blk).reshape(-1).to(torch.bfloat16)

    def row_bias(name):
        return (w[name].to(device).float() / size).to(torch.bfloat16)

    bf = lambda t: t.to(device, torch.bfloat16).contiguous()
    params = [bf(w["g1"]), bf(w["b_ln1"]), bf(w["g2"]), bf(w["b_ln2"]),
              qs["q"], col_bias("bq", H), qs["k"], col_bias("bk", H), qs["v"], col_bias("bv", H), qs["o"], row_bias("bo"),
              qs["fc1"], col_bias("b1", 64), qs["fc2"], row_bias("b2")]
    layer = fused_llm_cpp.OPTDecoderLayer(params, layer_idx, shape.layer_norm_eps, shape.layer_norm_eps, H, shape.do_layer_norm_before)
    for q in (layer.Wqkv, layer.Wp, layer.Wi, layer.Wo):
        if hasattr(q, "codes"):
            q.codes = q.codes.new_empty(0)
    return layer


class OPTRunner(LlamaRunner):
    """The Llama runner with OPT's embedding (tokens + learned positions) and final LayerNorm."""

    def __init__(self, shape, embed, pos_embed, layers, final_ln, lm_head_w):
        super().__init__(shape, embed, layers, None, lm_head_w, None)
        self.pos_embed, self.final_ln = pos_embed, final_ln

    def _embed(self, ids, positions):
        return torch.nn.functional.embedding(ids, self.embed) + torch.nn.functional.embedding(positions + POSITION_OFFSET, self.pos_embed)

    def _final_norm(self, hs):
        if self.final_ln is None:
            return hs.contiguous()
        return fused_llm_cpp.layer_norm(hs.contiguous(), self.final_ln[0], self.final_ln[1], self.shape.layer_norm_eps)


def build_random_opt(shape, weight_dtype="mxfp4", device="cuda", seed=0, std=0.02):
    llm_common.set_pg()
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    D, FF = shape.hidden_size, shape.ffn_dim

    def rnd(*s):
        return (torch.randn(*s, generator=g, device=dev) * std).to(torch.bfloat16)

    embed = rnd(shape.vocab_size, D)
    pos_embed = rnd(shape.max_position_embeddings + POSITION_OFFSET, D)
    layers = []
    for i in range(shape.num_hidden_layers):
        w = {"q": rnd(D, D), "k": rnd(D, D), "v": rnd(D, D), "o": rnd(D, D), "fc1": rnd(FF, D), "fc2": rnd(D, FF),
             "bq": rnd(D), "bk": rnd(D), "bv": rnd(D), "bo": rnd(D), "b1": rnd(FF), "b2": rnd(D),
             "g1": torch.ones(D), "b_ln1": torch.zeros(D), "g2": torch.ones(D), "b_ln2": torch.zeros(D)}
        layers.append(make_opt_layer(shape, w, i, weight_dtype, dev))
    final_ln = (torch.ones(D, device=dev, dtype=torch.bfloat16), torch.zeros(D, device=dev, dtype=torch.bfloat16)) \
        if shape.do_layer_norm_before else None
    return OPTRunner(shape, embed, pos_embed, layers, final_ln, _lm_head(embed, False, weight_dtype))


def OptimizeModelForOPT(model, dtype=torch.bfloat16, device="cuda", weight_dtype="mxfp4", quantize_lm_head=False, patch_model=False):
    """Reference entry point llm/fused_opt_infer.py:OptimizeModelForOPT for a Hugging Face OPTForCausalLM."""
    if dtype != torch.bfloat16:
        raise ValueError("the CUDA path computes in bfloat16")
    llm_common.set_pg()
    cfg = model.config
    if cfg.word_embed_proj_dim != cfg.hidden_size:
        raise ValueError("OPT models with a projected word embedding (word_embed_proj_dim != hidden_size) are not supported")
    if cfg.activation_function != "relu" or not cfg.enable_bias or not cfg.layer_norm_elementwise_affine:
        raise ValueError("only the standard OPT block (ReLU, biases, affine LayerNorm) is supported")
    shape = OPTShape(cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.ffn_dim, cfg.vocab_size,
                     cfg.max_position_embeddings, cfg.do_layer_norm_before, 1e-5)
    dev = torch.device(device)
    dec = model.model.decoder
    layers = []
    for i, l in enumerate(dec.layers):
        a = l.self_attn
        w = {"q": a.q_proj.weight.data, "k": a.k_proj.weight.data, "v": a.v_proj.weight.data, "o": a.out_proj.weight.data,
             "fc1": l.fc1.weight.data, "fc2": l.fc2.weight.data,
             "bq": a.q_proj.bias.data, "bk": a.k_proj.bias.data, "bv": a.v_proj.bias.data, "bo": a.out_proj.bias.data,
             "b1": l.fc1.bias.data, "b2": l.fc2.bias.data,
             "g1": l.self_attn_layer_norm.weight.data, "b_ln1": l.self_attn_layer_norm.bias.data,
             "g2": l.final_layer_norm.weight.data, "b_ln2": l.final_layer_norm.bias.data}
        layers.append(make_opt_layer(shape, w, i, weight_dtype, dev))
    bf = lambda t: t.data.to(dev, torch.bfloat16).contiguous()
    fl = dec.final_layer_norm
    final_ln = (bf(fl.weight), bf(fl.bias)) if fl is not None else None
    embed = bf(dec.embed_tokens.weight)
    lm = _lm_head(bf(model.lm_head.weight), quantize_lm_head, weight_dtype)
    runner = OPTRunner(shape, embed, bf(dec.embed_positions.weight), layers, final_ln, lm)
    if patch_model:
        llm_common.patch_hf_model(model, runner)
    return runner
