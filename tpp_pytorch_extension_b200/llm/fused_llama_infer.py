"""Llama on the fused decoder layers, mirroring src/tpp_pytorch_extension/llm/fused_llama_infer.py.

`OptimizeModelForLlama(model, dtype, device, weight_dtype)` keeps the reference's entry point: it takes a
Hugging Face LlamaForCausalLM, shards (tensor parallel), blocks and quantizes its linears exactly as
FixLlamaDecoderLayer does (fused_llama_infer.py:104-172), and returns a runner whose forward walks the fused
layers (the patched LlamaModel.forward of the reference, :236-335). `build_random_llama` builds the same runner
from a config alone, layer by layer on the GPU, for the random-weight benchmark configurations."""
import math
from dataclasses import dataclass

import torch

from .._C import _fused_llm_infer as fused_llm_cpp
from . import llm_common
from .llm_common import TppCache, get_rank, get_size, quantize_weight, shard_offsets


@dataclass
class LlamaShape:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int
    head_dim: int = 0
    rms_norm_eps: float = 1e-5
    rope_theta: float = 1e4
    max_position_embeddings: int = 4096

    def __post_init__(self):
        if not self.head_dim:
            self.head_dim = self.hidden_size // self.num_attention_heads


def rope_table(max_pos, head_dim, theta, device):
    """cat(cos, sin).view(2, MP, head_dim) in fp32, from HF's default rotary embedding
    (fused_llama_infer.py:186-204): inv_freq = theta^(-2i/d), emb = cat(freqs, freqs)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    fr = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    emb = torch.cat([fr, fr], dim=-1)
    return torch.stack([emb.cos(), emb.sin()]).to(device).contiguous()


def _shard(w, dim, block):
    """This rank's slice of a weight (ShardLinear, llm_common.py:517-546)."""
    size, rank = get_size(), get_rank()
    if size == 1:
        return w
    offs = shard_offsets(w.shape[dim], size, block)
    return (w[offs[rank]:offs[rank + 1], :] if dim == 0 else w[:, offs[rank]:offs[rank + 1]]).contiguous()


def make_layer(shape, weights, layer_idx, ep, weight_dtype, device):
    """weights: dict of plain [N, K] tensors q,k,v,o,gate,up,down and norm vectors ln1, ln2.
    Sharding units follow FixLlamaDecoderLayer (fused_llama_infer.py:119-129): q and o by head_dim * kv groups,
    k and v by head_dim, the MLP by 64."""
    H = shape.head_dim
    grp = H * (shape.num_attention_heads // shape.num_key_value_heads)
    plan = {"q": (0, grp), "k": (0, H), "v": (0, H), "o": (1, grp), "gate": (0, 64), "up": (0, 64), "down": (1, 64)}
    qs = {}
    for name, (dim, blk) in plan.items():
        w = _shard(weights[name].to(device), dim, blk)
        qs[name] = quantize_weight(w, weight_dtype)
    params = [weights["ln1"].to(device, torch.bfloat16), qs["q"], qs["k"], qs["v"], qs["o"],
              weights["ln2"].to(device, torch.bfloat16), qs["gate"], qs["up"], qs["down"]]
    if "bq" in weights:  # Qwen2: biases of the column-parallel q/k/v projections are sharded like their rows
        bs = [_shard(weights[n].to(device).reshape(-1, 1), 0, blk).reshape(-1).to(torch.bfloat16)
              for n, blk in (("bq", grp), ("bk", H), ("bv", H))]
        layer = fused_llm_cpp.Qwen2DecoderLayer(params + bs + [ep], layer_idx, shape.rms_norm_eps, H, ep.shape[1], H)
    else:
        layer = fused_llm_cpp.LlamaDecoderLayer(params + [ep], layer_idx, shape.rms_norm_eps, H, ep.shape[1], H)
    # the interchange tensors are no longer needed once the streaming layouts exist
    for w in (layer.Wqkv, layer.Wp, layer.Wd, layer.Wg, layer.Wu):
        if hasattr(w, "codes"):
            w.codes = w.codes.new_empty(0)
    return layer


class _DecodeSession:
    """What one recorded decode step needs to be replayed by a later generate() call of the same batch size: the KV
    cache (sized once for the longest request so far), the tensors the recorded kernels read their inputs from, and the
    CUDA graph. Recording a step of a 32-layer model costs tens of milliseconds, as much as a dozen decoded tokens."""

    def __init__(self, cache, batch, need):
        self.cache, self.batch, self.need = cache, batch, need
        self.graph = self.tok = self.pos = self.dev_len = self.am = None
        self.capacity, self.arenas = 0, None

    def cache_fits(self, batch, need):
        layers = self.cache.get_cpp().layers
        return self.batch == batch and layers and all(lc.contiguous() and lc.capacity() >= need for lc in layers)

    def graph_fits(self, cpp, cap):
        return (self.graph is not None and self.capacity == cap
                and self.arenas == [id(a[0]) for lc in cpp.layers for a in lc.arenas])


class LlamaRunner(torch.nn.Module):
    _session = None             # cache + recorded decode step kept by generate() for its next call (_DecodeSession)
    reuse_decode_graph = True   # False: every generate() call builds its cache and records its decode step anew

    def __init__(self, shape, embed, layers, norm_w, lm_head_w, ep):
        super().__init__()
        self.shape, self.embed, self.layers, self.norm_w, self.ep = shape, embed, layers, norm_w, ep
        # lm_head stays bf16 as in the reference unless it is quantized separately; with tensor parallelism it is
        # row-parallel followed by an all-reduce (fused_llama_infer.py:218-224)
        self.lm_head_w = lm_head_w
        self.only_last_logit = True

    def _embed(self, ids, positions):
        """Token embedding; model families with learned position embeddings add them here."""
        return torch.nn.functional.embedding(ids, self.embed)

    def _final_norm(self, hs):
        return fused_llm_cpp.rms_norm(hs.contiguous(), self.norm_w, self.shape.rms_norm_eps)

    def _head(self, hs):
        """Final norm + lm_head on the last position (logits slicing of the reference, fused_llama_infer.py:385-390)."""
        if self.only_last_logit:
            hs = hs[:, -1:, :]
        hs = self._final_norm(hs)
        # lm_head_w is a bf16 matrix (the reference's default) or a quantized tensor (its --quantize-lm-head): both go
        # through fc_plain, i.e. this library's own tensor-core kernels
        if get_size() > 1:
            offs = shard_offsets(self.shape.hidden_size, get_size(), 64)
            r = get_rank()
            logits = fused_llm_cpp.fc_plain(hs[..., offs[r]:offs[r + 1]].contiguous(), self.lm_head_w, getattr(self, "lm_head_b", None))
            fused_llm_cpp.allreduce(logits)
        else:
            logits = fused_llm_cpp.fc_plain(hs, self.lm_head_w, getattr(self, "lm_head_b", None))
        if logits.shape[-1] != self.shape.vocab_size:  # a quantized head padded to whole row groups
            logits = logits[..., :self.shape.vocab_size]
        return logits

    @torch.no_grad()
    def forward(self, input_ids, attention_mask=None, position_ids=None, cache=None):
        """Patched LlamaModel.forward + LlamaForCausalLM.forward of the reference (fused_llama_infer.py:236-408)."""
        if cache is None:
            cache = TppCache()
        B, S = input_ids.shape
        past = cache.get_seq_length()
        if position_ids is None:
            position_ids = torch.arange(past, past + S, device=input_ids.device).unsqueeze(0)
        hs = self._embed(input_ids, position_ids)
        if attention_mask is None:
            attention_mask = torch.ones((B, past + S), device=input_ids.device, dtype=hs.dtype)
        am = cache.align_and_invert_mask(attention_mask, hs)
        cpp = cache.get_cpp()
        for layer in self.layers:
            hs = layer.forward([hs, am, position_ids], cpp, True)[0]
        return self._head(hs), cache

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens, attention_mask=None, use_graph=True):
        """Greedy decoding (the reference drives HF generate with --greedy, examples/llm/run_generation.py:337-339).

        With use_graph the decode step (embedding, all layers, head, argmax, length bump) is recorded once in a CUDA
        graph and replayed: the lengths the kernels need live in device memory, the cache is sized up front, and the
        host only replays. Returns [B, prompt + max_new_tokens] token ids."""
        B, P = input_ids.shape
        sess = None
        if use_graph and max_new_tokens - 1 >= 3 and self.reuse_decode_graph:
            # the cache and the recorded step of the previous call serve again when the batch is the same and the
            # request fits the cache; else a new cache is sized for this request in one piece
            need = P + max_new_tokens
            sess = self._session
            if sess is None or not sess.cache_fits(B, need):
                sess = self._session = None  # frees the old cache before the new one is allocated
                sess = self._session = _DecodeSession(TppCache(), B, need)
                cpp = sess.cache.get_cpp()
                for i, layer in enumerate(self.layers):
                    cpp.layer(i).ensure(B, layer.Nkv, layer.H, need, torch.bfloat16, input_ids.device)
            else:
                for lc in sess.cache.get_cpp().layers:
                    lc.offset = 0
        cache = sess.cache if sess is not None else TppCache()
        mask = attention_mask if attention_mask is not None else torch.ones_like(input_ids)
        # positions count the kept tokens only, in the prompt as in the decode steps (HF generate: cumsum(mask) - 1),
        # so that a left-padded sequence rotates its tokens as the unpadded one would
        prompt_pos = (mask.to(torch.int64).cumsum(-1) - 1).clamp_(min=0).contiguous() if attention_mask is not None else None
        logits, cache = self.forward(input_ids, mask, prompt_pos, cache)
        tok = fused_llm_cpp.argmax_rows(logits[:, -1]).unsqueeze(-1)
        new = self.decode(tok, cache, mask, max_new_tokens - 1, use_graph=use_graph, session=sess)
        return torch.cat([input_ids, new], dim=1)

    def release_session(self):
        """Drop the cache and the recorded decode step kept for the next generate() call."""
        self._session = None

    @torch.no_grad()
    def decode(self, tok, cache, mask, steps, use_graph=True, timing=None, session=None):
        """`steps` greedy decode steps from a cache that already holds the context: tok [B, 1] is the first new token
        (not yet in the cache), mask [B, context] the keep-mask of the cached tokens. Returns [B, 1 + steps] tokens.
        timing: optional dict; receives 'events' = (start, end) CUDA events around the replayed steps and 'steps'.
        session: a _DecodeSession whose recorded step is replayed if it was recorded for this cache and capacity, and
        which otherwise receives the step recorded now."""
        cpp = cache.get_cpp()
        B = tok.shape[0]
        dev = tok.device
        P = cpp.get_seq_length()
        tok = tok.clone()
        outs = [tok.clone()]
        if steps <= 0:
            return torch.cat(outs, dim=1)
        # room for every token to come, so that no cache tensor moves during decoding
        for lc in cpp.layers:  # appends pages; nothing cached moves
            _, nkv, hd = lc.dims()
            lc.ensure(B, nkv, hd, steps, lc.arenas[0][0].dtype, dev)
        cap = cpp.layers[0].capacity()
        keep = torch.cat([mask.to(torch.bfloat16), torch.ones((B, cap - P), dtype=torch.bfloat16, device=dev)], dim=1)
        am = cpp.align_and_invert_mask(keep)  # positions not yet written are excluded by the length, not by the mask
        dev_len = torch.full((1,), P, dtype=torch.int32, device=dev)
        pos = mask.sum(-1, keepdim=True).to(torch.int64).contiguous()  # next position per sequence (left padding aware)

        def step():
            hs = self._embed(tok, pos)
            for layer in self.layers:
                hs = layer.forward([hs, am, pos], cpp, True, dev_len=dev_len)[0]
            lg = self._head(hs)
            tok.copy_(fused_llm_cpp.argmax_rows(lg[:, -1]).unsqueeze(-1))
            pos.add_(1)
            dev_len.add_(1)

        done = 0
        graph = None
        if use_graph and steps >= 3 and session is not None and session.graph_fits(cpp, cap):
            # the recorded kernels read these tensors: refill them in place and replay
            session.tok.copy_(tok)
            session.pos.copy_(pos)
            session.dev_len.copy_(dev_len)
            session.am.copy_(am)
            tok, graph = session.tok, session.graph
        elif use_graph and steps >= 3:
            step()  # eager once: sizes scratch buffers and opts kernels in to their shared-memory sizes
            outs.append(tok.clone())
            done = 1
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step()
            except Exception as e:  # capture unsupported here: decode eagerly
                import warnings
                warnings.warn(f"CUDA graph capture of the decode step failed ({e!r}); decoding eagerly")
                graph = None
                torch.cuda.synchronize()
        if timing is not None:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            timing["events"], timing["steps"] = ev, steps - done
            ev[0].record()
        while done < steps:
            if graph is not None:
                graph.replay()
            else:
                step()
            outs.append(tok.clone())
            done += 1
        if timing is not None:
            timing["events"][1].record()
        for lc in cpp.layers:
            lc.offset += steps
        self.last_graph = graph
        if session is not None and graph is not None and session.graph is not graph:
            session.graph, session.tok, session.pos, session.dev_len, session.am = graph, tok, pos, dev_len, am
            session.capacity = cap
            session.arenas = [id(a[0]) for lc in cpp.layers for a in lc.arenas]
        out = torch.cat(outs, dim=1)
        from .. import _lib
        _lib.assert_no_kernel_error()  # a kernel that gave up on a bounded wait would have produced wrong tokens
        return out

    @torch.no_grad()
    def beam_search(self, input_ids, max_new_tokens, num_beams=4, attention_mask=None):
        """Beam search for a fixed number of new tokens (the reference's default driver runs Hugging Face generate with
        num_beams=4, examples/llm/run_generation.py:337-339; its own part is the cache reordering, which this uses).

        Scores are sums of log-softmax over the bf16 logits in fp32; every step keeps the num_beams best continuations
        per sequence and reorders the KV cache rows to follow their parents (TppCache.reorder_cache: after the prompt
        the cache of B sequences is first repeated per beam). No end-of-sequence handling and no length penalty: all
        hypotheses have the same length. Returns ([B, num_beams, prompt + max_new_tokens] token ids, best first,
        [B, num_beams] scores)."""
        B, P = input_ids.shape
        dev = input_ids.device
        nb = int(num_beams)
        cache = TppCache()
        mask = attention_mask if attention_mask is not None else torch.ones_like(input_ids)
        prompt_pos = (mask.to(torch.int64).cumsum(-1) - 1).clamp_(min=0).contiguous() if attention_mask is not None else None
        logits, cache = self.forward(input_ids, mask, prompt_pos, cache)
        logp = torch.log_softmax(logits[:, -1].float(), dim=-1)             # [B, V]
        V = logp.shape[-1]
        scores, tok = logp.topk(nb, dim=-1)                                  # [B, nb]: the first step expands one beam
        seqs = torch.cat([input_ids.unsqueeze(1).expand(B, nb, P), tok.unsqueeze(-1)], dim=-1)
        # sequence b's beams are rows b*nb .. b*nb+nb-1 from here on; the first reorder meets a cache of B rows, repeats
        # each row nb times (indices then address the expanded batch) and every beam continues its own copy
        parent_rows = torch.arange(B * nb, device=dev)
        mask = mask.repeat_interleave(nb, dim=0)
        pos = mask.sum(-1, keepdim=True).to(torch.int64)
        for _ in range(max_new_tokens - 1):
            cache.reorder_cache(parent_rows)
            mask = torch.cat([mask, torch.ones((B * nb, 1), dtype=mask.dtype, device=dev)], dim=1)
            logits, cache = self.forward(tok.reshape(B * nb, 1), mask, pos, cache)
            pos = pos + 1
            logp = torch.log_softmax(logits[:, -1].float(), dim=-1).view(B, nb, V)
            cand = (scores.unsqueeze(-1) + logp).view(B, nb * V)
            scores, idx = cand.topk(nb, dim=-1)
            parent, tok = idx // V, idx % V                                   # [B, nb]
            seqs = torch.cat([seqs.gather(1, parent.unsqueeze(-1).expand(-1, -1, seqs.shape[-1])), tok.unsqueeze(-1)], dim=-1)
            parent_rows = (parent + torch.arange(B, device=dev).unsqueeze(-1) * nb).reshape(-1)
        return seqs, scores

    def synthetic_cache(self, batch, context, room, seed=1):
        """A cache that looks as if `context` tokens per sequence had been prefilled: random keys and values of the
        right shapes (what a decode step costs does not depend on their values). For benchmarks of the decode step on
        long contexts, where running the prefill itself would take most of the run."""
        cache = TppCache()
        cpp = cache.get_cpp()
        g = torch.Generator(device=self.embed.device).manual_seed(seed)
        for i, layer in enumerate(self.layers):
            lc = cpp.layer(i)
            s1 = (context + room + 31) // 32
            shape = (s1, batch, layer.Nkv, 32, layer.H)
            lc.adopt(torch.randn(shape, generator=g, device=self.embed.device, dtype=torch.bfloat16),
                     torch.randn(shape, generator=g, device=self.embed.device, dtype=torch.bfloat16), context)
        return cache


def _lm_head_shard(w):
    if get_size() == 1:
        return w
    offs = shard_offsets(w.shape[1], get_size(), 64)
    r = get_rank()
    return w[:, offs[r]:offs[r + 1]].contiguous()


def _lm_head(w, quantize, weight_dtype):
    """This rank's lm_head: bf16 as it is, or quantized like the decoder linears (examples/llm/run_generation.py:277-282)."""
    w = _lm_head_shard(w)
    if not quantize:
        return w
    if w.shape[0] % 32:  # vocabularies that are not a whole number of MXFP4 row groups get zero rows
        w = torch.nn.functional.pad(w, (0, 0, 0, 32 - w.shape[0] % 32))
    q = quantize_weight(w, weight_dtype)
    q.prepare(drop_interchange=True)
    return q


def build_random_llama(shape, weight_dtype="mxfp4", device="cuda", seed=0, std=0.02, max_positions=None, quantize_lm_head=False):
    """Random N(0, std) linears and embeddings, unit norm weights, quantized layer by layer on the device.
    Every tensor-parallel rank draws the same full weights (same seed) and keeps its shard."""
    llm_common.set_pg()
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    MP = max_positions or shape.max_position_embeddings
    ep = rope_table(MP, shape.head_dim, shape.rope_theta, dev)
    D, H = shape.hidden_size, shape.head_dim
    Nq, Nkv, FF = shape.num_attention_heads, shape.num_key_value_heads, shape.intermediate_size

    def rnd(n, k):
        return (torch.randn(n, k, generator=g, device=dev) * std).to(torch.bfloat16)

    embed = rnd(shape.vocab_size, D)
    layers = []
    for i in range(shape.num_hidden_layers):
        w = {"q": rnd(Nq * H, D), "k": rnd(Nkv * H, D), "v": rnd(Nkv * H, D), "o": rnd(D, Nq * H), "gate": rnd(FF, D),
             "up": rnd(FF, D), "down": rnd(D, FF), "ln1": torch.ones(D), "ln2": torch.ones(D)}
        layers.append(make_layer(shape, w, i, ep, weight_dtype, dev))
        del w
    lm = _lm_head(rnd(shape.vocab_size, D), quantize_lm_head, weight_dtype)
    return LlamaRunner(shape, embed, layers, torch.ones(D, device=dev, dtype=torch.bfloat16), lm, ep)


def OptimizeModelForLlama(model, dtype=torch.bfloat16, device="cuda", weight_dtype="mxfp4", quantize_lm_head=False, patch_model=False):
    """Reference entry point (fused_llama_infer.py:176-233) for a Hugging Face LlamaForCausalLM. Returns the runner;
    with patch_model=True the Hugging Face object is also patched in place, as the reference does, so that
    model(...) and model.generate(...) run on the fused layers (llm_common.patch_hf_model)."""
    if dtype != torch.bfloat16:
        raise ValueError("the CUDA path computes in bfloat16")
    llm_common.set_pg()
    cfg = model.config
    shape = LlamaShape(cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads,
                       getattr(cfg, "num_key_value_heads", cfg.num_attention_heads), cfg.intermediate_size, cfg.vocab_size,
                       getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads, cfg.rms_norm_eps,
                       getattr(cfg, "rope_theta", None) or (getattr(cfg, "rope_parameters", None) or {}).get("rope_theta", 1e4),
                       cfg.max_position_embeddings)
    dev = torch.device(device)
    ep = rope_table(shape.max_position_embeddings, shape.head_dim, shape.rope_theta, dev)
    layers = []
    for i, l in enumerate(model.model.layers):
        w = {}
        if getattr(l.self_attn.q_proj, "bias", None) is not None:  # Qwen2 (fused_qwen2_infer.py of the reference)
            w.update(bq=l.self_attn.q_proj.bias.data, bk=l.self_attn.k_proj.bias.data, bv=l.self_attn.v_proj.bias.data)
        w.update({"q": l.self_attn.q_proj.weight.data, "k": l.self_attn.k_proj.weight.data, "v": l.self_attn.v_proj.weight.data,
             "o": l.self_attn.o_proj.weight.data, "gate": l.mlp.gate_proj.weight.data, "up": l.mlp.up_proj.weight.data,
             "down": l.mlp.down_proj.weight.data, "ln1": l.input_layernorm.weight.data, "ln2": l.post_attention_layernorm.weight.data})
        layers.append(make_layer(shape, w, i, ep, weight_dtype, dev))
    embed = model.model.embed_tokens.weight.data.to(dev, torch.bfloat16)
    lm = _lm_head(model.lm_head.weight.data.to(dev, torch.bfloat16), quantize_lm_head, weight_dtype)
    runner = LlamaRunner(shape, embed, layers, model.model.norm.weight.data.to(dev, torch.bfloat16), lm, ep)
    if patch_model:
        llm_common.patch_hf_model(model, runner)
    return runner


def OptimizeModelForQwen2(model, dtype=torch.bfloat16, device="cuda", weight_dtype="mxfp4", quantize_lm_head=False, patch_model=False):
    """Reference entry point llm/fused_qwen2_infer.py:OptimizeModelForQwen2: the same runner, layers carry q/k/v biases."""
    return OptimizeModelForLlama(model, dtype, device, weight_dtype, quantize_lm_head, patch_model)


LLAMA2_7B = LlamaShape(32, 4096, 32, 32, 11008, 32000, rms_norm_eps=1e-5, rope_theta=1e4)
LLAMA3_8B = LlamaShape(32, 4096, 32, 8, 14336, 128256, rms_norm_eps=1e-5, rope_theta=5e5, max_position_embeddings=8192)
LLAMA2_70B = LlamaShape(80, 8192, 64, 8, 28672, 32000, rms_norm_eps=1e-5, rope_theta=1e4, max_position_embeddings=8192)
