"""Mirror of the reference's `_C._tpp_attn` submodule (src/csrc/llm/attn.cpp:1956-1983): the KV cache object and
the attention op, on CUDA.

The cache keeps the reference's layout and growth rule (src/csrc/llm/attn.h:144-226): per layer two tensors
[S1, B, Nkv, 32, H]; token t lives in block t // 32, slot t % 32; when an update does not fit, the capacity
becomes offset + S + KV_CACHE_INC_SIZE rounded up to a block, by allocating zeros and copying."""
import os

import torch

from .. import _lib

S2 = 32
KV_CACHE_INC_SIZE = int(os.environ.get("KV_CACHE_INC_SIZE", "128"))  # src/csrc/llm/attn.h:31


class LayerCache:
    def __init__(self):
        self.k = None
        self.v = None
        self.offset = 0

    def capacity(self):
        return 0 if self.k is None else self.k.shape[0] * S2

    def ensure(self, B, Nkv, H, S, dtype, device):
        """Make room for S more tokens (LayerCache::update, attn.h:162-178)."""
        if self.k is not None and (self.k.shape[1], self.k.shape[2], self.k.shape[4]) != (B, Nkv, H):
            raise _lib.TpxError("KV cache shape changed between calls")
        if self.capacity() < self.offset + S:
            new_cap = self.offset + S + KV_CACHE_INC_SIZE
            s1 = (new_cap + S2 - 1) // S2
            for name in ("k", "v"):
                old = getattr(self, name)
                new = torch.zeros((s1, B, Nkv, S2, H), dtype=dtype, device=device)
                if old is not None:
                    new[: old.shape[0]] = old
                setattr(self, name, new)


class TppCache:
    """torch.classes.tpp_llm.TppCache (src/csrc/llm/attn.h:229-404)."""

    def __init__(self):
        self.layers = []

    def layer(self, idx):
        while len(self.layers) <= idx:
            self.layers.append(LayerCache())
        return self.layers[idx]

    def update(self, key_states, value_states, layer_idx):
        """Append [B, Nkv, S, H] keys/values (already rotated); returns the cache tensors (attn.h:258-275)."""
        B, N, S, H = key_states.shape
        lc = self.layer(layer_idx)
        lc.ensure(B, N, H, S, key_states.dtype, key_states.device)
        t = torch.arange(lc.offset, lc.offset + S, device=key_states.device)
        lc.k[t // S2, :, :, t % S2, :] = key_states.permute(2, 0, 1, 3)
        lc.v[t // S2, :, :, t % S2, :] = value_states.permute(2, 0, 1, 3)
        lc.offset += S
        return [lc.k, lc.v]

    def get_seq_length(self, layer_idx=0):
        return self.layers[layer_idx].offset if layer_idx < len(self.layers) else 0

    def size(self):
        return len(self.layers)

    def get(self, layer_idx):
        lc = self.layers[layer_idx]
        return [lc.k, lc.v]  # the reference returns the key tensor twice here (attn.h:282); that slip is not mirrored

    def get_capacity(self, layer_idx=0):
        return self.layers[layer_idx].capacity() if layer_idx < len(self.layers) else 0

    def align_and_invert_mask(self, mask, pad_value=None):
        """[B, S] mask of 1 (keep) / 0 (drop) -> additive [B, S rounded up to 32] (attn.h:310-322)."""
        _lib.require_cuda(mask, "mask")
        mask = mask.to(torch.bfloat16).contiguous()
        B, S = mask.shape
        Spad = (S + S2 - 1) // S2 * S2
        out = torch.empty((B, Spad), dtype=torch.bfloat16, device=mask.device)
        if pad_value is None:
            pad_value = torch.finfo(torch.bfloat16).min
        bits = int(torch.tensor(pad_value, dtype=torch.bfloat16).view(torch.int16).item()) & 0xFFFF
        _lib.check(_lib.lib().tpx_align_and_invert_mask(mask.data_ptr(), B, S, Spad, bits, out.data_ptr(), _lib.stream()))
        return out

    def crop(self, max_length):
        for lc in self.layers:
            if lc.offset > max_length:
                lc.offset = max_length

    def reorder_cache(self, beam_idx):
        """TppCache::reorder_cache (src/csrc/llm/attn.h:327-403): after the call, sequence i continues the history
        of the old sequence beam_idx[i]. The reference records the permutations and gathers rows inside attention;
        here the cache rows are gathered once per call (the batch dimension of [S1, B, Nkv, 32, H] is dim 1), which
        yields the same keys and values for every later step. A cache of CB sequences meeting B = CB * beams
        indices is first repeated per beam, as the reference does (attn.h:345-367)."""
        beam_idx = beam_idx.to(torch.long)
        B = beam_idx.shape[0]
        for lc in self.layers:
            if lc.k is None:
                continue
            CB = lc.k.shape[1]
            if CB != B:
                if B % CB != 0:
                    raise _lib.TpxError(f"New batch ({B}) must be multiple of cached batch size ({CB})")
                lc.k = lc.k.repeat_interleave(B // CB, dim=1)
                lc.v = lc.v.repeat_interleave(B // CB, dim=1)
            idx = beam_idx.to(lc.k.device)
            lc.k = lc.k.index_select(1, idx).contiguous()
            lc.v = lc.v.index_select(1, idx).contiguous()


def attention(q, kc, vc, mask, key_len, causal=True, out_bsnrh=False, dev_len=None):
    """attn<T> (src/csrc/llm/attn.cpp:780-955). q [B, Nkv, Sq, R, H] bf16; kc/vc cache tensors; mask additive
    [B, Spad] or None. Returns [B, Nkv, Sq, R, H], or [B, Sq, Nkv*R*H] with out_bsnrh. With dev_len (int32
    device scalar) the key count is read on the device as dev_len + Sq and key_len is the planning maximum."""
    _lib.require_cuda(q, "q")
    B, Nkv, Sq, R, H = q.shape
    L = _lib.lib()
    out = torch.empty((B, Sq, Nkv * R * H) if out_bsnrh else q.shape, dtype=q.dtype, device=q.device)
    nb = L.tpx_attention_scratch_bytes(B, Nkv, Sq, R, H, key_len)
    sc = _lib.aux_scratch(nb, q.device) if nb else None
    Spad = mask.shape[1] if mask is not None else 0
    _lib.check(L.tpx_attention(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), _lib.ptr(mask), B, Nkv, Sq, R, H, key_len, Spad,
                               int(causal), int(out_bsnrh), _lib.ptr(dev_len), out.data_ptr(), _lib.ptr(sc), nb, _lib.stream()))
    return out


def attn(q, k, v, mask, cache, layer_idx, isCausal=True):
    """_tpp_attn.attn (src/csrc/llm/attn.cpp:957-971): update the cache with k, v [B, Nkv, S, H], then attend."""
    kc, vc = cache.update(k, v, layer_idx)
    return attention(q.contiguous(), kc, vc, mask, cache.get_seq_length(layer_idx), isCausal)
