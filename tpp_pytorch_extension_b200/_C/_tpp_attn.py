"""Mirror of the reference's `_C._tpp_attn` submodule (src/csrc/llm/attn.cpp:1956-1983): the KV cache object and
the attention op, on CUDA.

The cache keeps the reference's layout (src/csrc/llm/attn.h:144-226): per layer keys and values as [S1, B, Nkv, 32, H],
token t in block t // 32, slot t % 32, and its growth rule for the capacity (offset + S + KV_CACHE_INC_SIZE rounded up
to a block); but the blocks are pages: growth appends pages instead of allocating a larger tensor and copying."""
import os

import torch

from .. import _lib

S2 = 32
KV_CACHE_INC_SIZE = int(os.environ.get("KV_CACHE_INC_SIZE", "128"))  # src/csrc/llm/attn.h:31


class LayerCache:
    """One layer's keys and values as a sequence of 32-token pages.

    A page is what one index of the reference's leading cache dimension holds: a [B, Nkv, 32, H] slab with the tokens
    32i .. 32i+31 of every sequence (src/csrc/llm/attn.h:144-153). Pages are allocated in runs ("arenas", tensors
    [pages, B, Nkv, 32, H]); when an update does not fit, a new arena with the missing pages is appended and nothing
    already cached moves, where the reference allocates a larger tensor and copies (attn.h:162-178). The capacity after
    growth is the reference's: offset + S + KV_CACHE_INC_SIZE rounded up to a page. The kernels reach the pages through
    two device arrays of page addresses (k_ptrs, v_ptrs); while the cache is a single arena it is also one contiguous
    tensor in the reference's layout, which is what `k` / `v` return and what the TMA-fed prefill kernel reads."""

    def __init__(self):
        self.arenas = []     # [(k, v)] tensors [pages, B, Nkv, 32, H]
        self.k_ptrs = None   # int64 [pages] device addresses of the pages
        self.v_ptrs = None
        self.offset = 0

    def pages(self):
        return sum(a[0].shape[0] for a in self.arenas)

    def capacity(self):
        return self.pages() * S2

    def contiguous(self):
        return len(self.arenas) == 1

    def dims(self):
        k = self.arenas[0][0]
        return k.shape[1], k.shape[2], k.shape[4]

    def _gather(self, which):
        if not self.arenas:
            return None
        if len(self.arenas) == 1:
            return self.arenas[0][which]
        return torch.cat([a[which] for a in self.arenas], dim=0)  # a copy: for inspection, not for the hot path

    @property
    def k(self):
        return self._gather(0)

    @property
    def v(self):
        return self._gather(1)

    def _rebuild_tables(self):
        dev = self.arenas[0][0].device
        tabs = []
        for which in (0, 1):
            addrs = []
            for a in self.arenas:
                t = a[which]
                step = t.stride(0) * t.element_size()
                addrs += [t.data_ptr() + i * step for i in range(t.shape[0])]
            tabs.append(torch.tensor(addrs, dtype=torch.int64, device=dev))
        self.k_ptrs, self.v_ptrs = tabs

    def ensure(self, B, Nkv, H, S, dtype, device):
        """Make room for S more tokens (LayerCache::update, attn.h:162-178) by appending pages."""
        if self.arenas and self.dims() != (B, Nkv, H):
            raise _lib.TpxError("KV cache shape changed between calls")
        if self.capacity() < self.offset + S:
            new_cap = self.offset + S + KV_CACHE_INC_SIZE
            add = (new_cap + S2 - 1) // S2 - self.pages()
            self.arenas.append((torch.zeros((add, B, Nkv, S2, H), dtype=dtype, device=device),
                                torch.zeros((add, B, Nkv, S2, H), dtype=dtype, device=device)))
            self._rebuild_tables()

    def adopt(self, k, v, offset):
        """Take k, v [pages, B, Nkv, 32, H] as the whole cache (one arena) holding `offset` tokens."""
        self.arenas = [(k, v)]
        self.offset = offset
        self._rebuild_tables()

    def write(self, t0, keys, values):
        """keys / values [S, B, Nkv, H] into tokens t0 .. t0+S-1 (host-side path of TppCache.update)."""
        S = keys.shape[0]
        page0 = 0
        for k, v in self.arenas:
            n = k.shape[0]
            lo, hi = max(t0, page0 * S2), min(t0 + S, (page0 + n) * S2)
            if lo < hi:
                t = torch.arange(lo, hi, device=k.device)
                k[t // S2 - page0, :, :, t % S2, :] = keys[lo - t0:hi - t0]
                v[t // S2 - page0, :, :, t % S2, :] = values[lo - t0:hi - t0]
            page0 += n

    def select_batch(self, idx, repeat=1):
        new = []
        for k, v in self.arenas:
            if repeat > 1:
                k, v = k.repeat_interleave(repeat, dim=1), v.repeat_interleave(repeat, dim=1)
            new.append((k.index_select(1, idx).contiguous(), v.index_select(1, idx).contiguous()))
        self.arenas = new
        self._rebuild_tables()


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
        lc.write(lc.offset, key_states.permute(2, 0, 1, 3), value_states.permute(2, 0, 1, 3))
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
            if not lc.arenas:
                continue
            CB = lc.dims()[0]
            rep = 1
            if CB != B:
                if B % CB != 0:
                    raise _lib.TpxError(f"New batch ({B}) must be multiple of cached batch size ({CB})")
                rep = B // CB
            lc.select_batch(beam_idx.to(lc.arenas[0][0].device), rep)


def attention(q, kc, vc, mask, key_len, causal=True, out_bsnrh=False, dev_len=None, pages=None):
    """attn<T> (src/csrc/llm/attn.cpp:780-955). q [B, Nkv, Sq, R, H] bf16; kc/vc cache tensors; mask additive
    [B, Spad] or None. Returns [B, Nkv, Sq, R, H], or [B, Sq, Nkv*R*H] with out_bsnrh. With dev_len (int32
    device scalar) the key count is read on the device as dev_len + Sq and key_len is the planning maximum.
    pages = (k_ptrs, v_ptrs): the cache as device arrays of page addresses instead of the tensors kc / vc."""
    _lib.require_cuda(q, "q")
    B, Nkv, Sq, R, H = q.shape
    L = _lib.lib()
    out = torch.empty((B, Sq, Nkv * R * H) if out_bsnrh else q.shape, dtype=q.dtype, device=q.device)
    nb = L.tpx_attention_scratch_bytes(B, Nkv, Sq, R, H, key_len)
    sc = _lib.aux_scratch(nb, q.device) if nb else None
    Spad = mask.shape[1] if mask is not None else 0
    if pages is not None:
        _lib.check(L.tpx_attention_paged(q.data_ptr(), pages[0].data_ptr(), pages[1].data_ptr(), _lib.ptr(mask), B, Nkv, Sq, R, H, key_len,
                                         Spad, int(causal), int(out_bsnrh), _lib.ptr(dev_len), out.data_ptr(), _lib.ptr(sc), nb, _lib.stream()))
        return out
    _lib.check(L.tpx_attention(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), _lib.ptr(mask), B, Nkv, Sq, R, H, key_len, Spad,
                               int(causal), int(out_bsnrh), _lib.ptr(dev_len), out.data_ptr(), _lib.ptr(sc), nb, _lib.stream()))
    return out


def attn(q, k, v, mask, cache, layer_idx, isCausal=True):
    """_tpp_attn.attn (src/csrc/llm/attn.cpp:957-971): update the cache with k, v [B, Nkv, S, H], then attend."""
    kc, vc = cache.update(k, v, layer_idx)
    return attention(q.contiguous(), kc, vc, mask, cache.get_seq_length(layer_idx), isCausal)
