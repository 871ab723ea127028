"""GPT-J on the fused block, mirroring src/tpp_pytorch_extension/llm/fused_gptj_infer.py.

`OptimizeModelForGPTJ(model, dtype, device, weight_dtype)` takes a Hugging Face GPTJForCausalLM, shards (tensor
parallel), blocks and quantizes the linears of every block (q/k/v/fc_in column-parallel, out_proj/fc_out row-parallel
with the fc_out bias divided by the group size) and returns a runner with the Llama runner's interface. What differs
from Llama: one LayerNorm per block feeding attention and MLP side by side, rotary embedding on the first rotary_dim
values of a head in adjacent pairs, GELU, a final LayerNorm and a head with a bias. Head size 256 (GPT-J-6B) runs on the
mma.sync attention kernel."""
from dataclasses import dataclass

import torch

from .._C import _fused_llm_infer as fused_llm_cpp
from . import llm_common
from .fused_llama_infer import LlamaRunner, _lm_head, _shard
from .llm_common import get_size, quantize_weight


@dataclass
class GPTJShape:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    intermediate_size: int
    vocab_size: int
    rotary_dim: int = 64
    max_position_embeddings: int = 2048
    layer_norm_eps: float = 1e-5

    @property
    def head_dim(self):
        return self.hidden_size // self.num_attention_heads

    @property
    def num_key_value_heads(self):
        return self.num_attention_heads


def sinusoidal_positions(num_pos, dim, device):
    """GPT-J's embed_positions: cat(sin, cos) of pos * 10000^(-2i/dim), fp32 [num_pos, dim]."""
    inv = 1.0 / (10000 ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    ang = torch.einsum("i,j->ij", torch.arange(num_pos, dtype=torch.int64).float(), inv)
    return torch.cat([ang.sin(), ang.cos()], dim=1).to(device).contiguous()


def make_gptj_block(shape, w, layer_idx, ep, weight_dtype, device):
    """w: plain [N, K] tensors q,k,v,o,fc_in,fc_out, biases b_in,b_out, LayerNorm g,b_ln."""
    H = shape.head_dim
    size = get_size()
    plan = {"q": (0, H), "k": (0, H), "v": (0, H), "o": (1, H), "fc_in": (0, 64), "fc_out": (1, 64)}
    qs = {n: quantize_weight(_shard(w[n].to(device), dim, blk), weight_dtype) for n, (dim, blk) in plan.items()}
    b_in = _shard(w["b_in"].to(device).reshape(-1, 1), 0, 64).reshape(-1).to(torch.bfloat16)
    b_out = (w["b_out"].to(device).float() / size).to(torch.bfloat16)
    bf = lambda t: t.to(device, torch.bfloat16).contiguous()
    params = [bf(w["g"]), bf(w["b_ln"]), qs["q"], qs["k"], qs["v"], qs["o"], qs["fc_in"], b_in, qs["fc_out"], b_out, ep]
    block = fused_llm_cpp.GPTJBlock(params, layer_idx, shape.layer_norm_eps, H, ep.shape[0], shape.rotary_dim)
    for q in (block.Wqkv, block.Wp, block.Wi, block.Wo):
        if hasattr(q, "codes"):
            q.codes = q.codes.new_empty(0)
    return block


class GPTJRunner(LlamaRunner):
    def __init__(self, shape, embed, layers, final_ln, lm_head_w, lm_head_b, ep):
        super().__init__(shape, embed, layers, None, lm_head_w, ep)
        self.final_ln = final_ln
        self.lm_head_b = lm_head_b

    def _final_norm(self, hs):
        return fused_llm_cpp.layer_norm(hs.contiguous(), self.final_ln[0], self.final_ln[1], self.shape.layer_norm_eps)


def build_random_gptj(shape, weight_dtype="mxfp4", device="cuda", seed=0, std=0.02):
    llm_common.set_pg()
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    D, FF = shape.hidden_size, shape.intermediate_size

    def rnd(*s):
        return (torch.randn(*s, generator=g, device=dev) * std).to(torch.bfloat16)

    ep = sinusoidal_positions(shape.max_position_embeddings, shape.rotary_dim, dev)
    embed = rnd(shape.vocab_size, D)
    layers = []
    for i in range(shape.num_hidden_layers):
        w = {"q": rnd(D, D), "k": rnd(D, D), "v": rnd(D, D), "o": rnd(D, D), "fc_in": rnd(FF, D), "fc_out": rnd(D, FF),
             "b_in": rnd(FF), "b_out": rnd(D), "g": torch.ones(D), "b_ln": torch.zeros(D)}
        layers.append(make_gptj_block(shape, w, i, ep, weight_dtype, dev))
    final_ln = (torch.ones(D, device=dev, dtype=torch.bfloat16), torch.zeros(D, device=dev, dtype=torch.bfloat16))
    head_b = (rnd(shape.vocab_size).float() / get_size()).to(torch.bfloat16)
    return GPTJRunner(shape, embed, layers, final_ln, _lm_head(rnd(shape.vocab_size, D), False, weight_dtype), head_b, ep)


def OptimizeModelForGPTJ(model, dtype=torch.bfloat16, device="cuda", weight_dtype="mxfp4", quantize_lm_head=False, patch_model=False):
    """Reference entry point llm/fused_gptj_infer.py:OptimizeModelForGPTJ for a Hugging Face GPTJForCausalLM."""
    if dtype != torch.bfloat16:
        raise ValueError("the CUDA path computes in bfloat16")
    llm_common.set_pg()
    cfg = model.config
    inner = cfg.n_inner if cfg.n_inner is not None else 4 * cfg.n_embd
    shape = GPTJShape(cfg.n_layer, cfg.n_embd, cfg.n_head, inner, cfg.vocab_size, cfg.rotary_dim or cfg.n_embd // cfg.n_head,
                      cfg.n_positions, cfg.layer_norm_epsilon)
    dev = torch.device(device)
    tr = model.transformer
    ep = sinusoidal_positions(shape.max_position_embeddings, shape.rotary_dim, dev)
    layers = []
    for i, blk in enumerate(tr.h):
        a, m = blk.attn, blk.mlp
        w = {"q": a.q_proj.weight.data, "k": a.k_proj.weight.data, "v": a.v_proj.weight.data, "o": a.out_proj.weight.data,
             "fc_in": m.fc_in.weight.data, "fc_out": m.fc_out.weight.data, "b_in": m.fc_in.bias.data, "b_out": m.fc_out.bias.data,
             "g": blk.ln_1.weight.data, "b_ln": blk.ln_1.bias.data}
        layers.append(make_gptj_block(shape, w, i, ep, weight_dtype, dev))
    bf = lambda t: t.data.to(dev, torch.bfloat16).contiguous()
    head_b = None
    if model.lm_head.bias is not None:
        head_b = (model.lm_head.bias.data.to(dev).float() / get_size()).to(torch.bfloat16)
    runner = GPTJRunner(shape, bf(tr.wte.weight), layers, (bf(tr.ln_f.weight), bf(tr.ln_f.bias)),
                        _lm_head(bf(model.lm_head.weight), quantize_lm_head, weight_dtype), head_b, ep)
    if patch_model:
        llm_common.patch_hf_model(model, runner)
    return runner
