"""The blocked weight layout of the reference (src/tpp_pytorch_extension/utils/blocked_layout.py:28-91 with the
blocking FixLinear attaches, llm_common.py:468-490), for the one case the quantized path uses."""
import torch


def block_weight(w, bk=16, bc=64, vnni=2):
    """W[N, K] -> [N/bk, K/bc, bc/vnni, bk, vnni] (view [N/bk, bk, K/bc, bc/vnni, vnni], permute [0,2,3,1,4])."""
    N, K = w.shape
    if N % bk or K % bc:
        raise ValueError(f"Blocking factor doesn't divide dim evenly shape = {tuple(w.shape)}, BF = {(bk, bc)}")
    return w.view(N // bk, bk, K // bc, bc // vnni, vnni).permute(0, 2, 3, 1, 4).contiguous()


def unblock_weight(wb):
    K1, C1, C2, K2, C3 = wb.shape
    return wb.permute(0, 3, 1, 2, 4).contiguous().view(K1 * K2, C1 * C2 * C3)


# --------------------------------------------------------------------------- general blocking (BlockingManager,
# BlockedParameter, BlockedModule of the reference, utils/blocked_layout.py:28-91, :248-364): a blocked layout is a view
# that splits some dimensions into (outer, inner...) factors followed by a permutation of the resulting dimensions.
def _split_sizes(shape, factors):
    """View shape after splitting: factors[i] is None (keep), an int f (-> [n // f, f]) or a sequence (-> [n // prod, *seq])."""
    if factors is None:
        factors = [None] * len(shape)
    if len(factors) != len(shape):
        raise ValueError(f"{len(factors)} blocking factors for a {len(shape)}-D tensor")
    sizes = []
    for n, f in zip(shape, factors):
        if f is None:
            sizes.append(n)
            continue
        inner = [f] if isinstance(f, int) else list(f)
        if not inner or not all(isinstance(v, int) and v > 0 for v in inner):
            raise ValueError(f"Unsupported blocking factor: {f!r}")
        total = 1
        for v in inner:
            total *= v
        if n % total:
            raise ValueError(f"Blocking factor doesn't divide dim evenly shape = {tuple(shape)}, BF = {factors}")
        sizes.append(n // total)
        sizes.extend(inner)
    return sizes


class BlockingManager:
    """block(): plain -> view(split sizes) -> permute -> contiguous; unblock() is its inverse."""

    def __init__(self, orig_shape, blocking_factors=None, permute=None):
        self.orig_shape = torch.Size(orig_shape)
        self.view_shape = _split_sizes(self.orig_shape, blocking_factors)
        if permute is not None:
            permute = list(permute)
            if sorted(permute) != list(range(len(self.view_shape))):
                raise ValueError(f"{permute} is not a permutation of the {len(self.view_shape)} blocked dimensions")
        self.permute = permute
        self.back_permute = None if permute is None else [permute.index(i) for i in range(len(permute))]
        self.blocked_shape = list(self.view_shape) if permute is None else [self.view_shape[i] for i in permute]

    def block(self, t):
        if t.shape != self.orig_shape:
            raise ValueError(f"expected a tensor of shape {tuple(self.orig_shape)}, got {tuple(t.shape)}")
        out = t.reshape(self.view_shape)
        return out.permute(self.permute).contiguous() if self.permute is not None else out

    def unblock(self, t):
        if list(t.shape) != self.blocked_shape:
            raise ValueError(f"expected a blocked tensor of shape {self.blocked_shape}, got {list(t.shape)}")
        if self.back_permute is not None:
            t = t.permute(self.back_permute).contiguous()
        return t.reshape(self.orig_shape)


def default_blocking_factors(S, prefered_factor=None, vnni_factor=None):
    """[outer, inner] split of a dimension of size S: the preferred inner factor if it divides S, else the first divisor
    in the reference's priority order (64, 48, 32, 24, 16, then even and odd sizes downwards), divisors that are
    multiples of vnni_factor first; [1, S] when nothing divides (blocked_layout.py:367-386)."""
    if prefered_factor is not None and S % prefered_factor == 0:
        return [S // prefered_factor, prefered_factor]
    order = [64, 48, 32, 24, 16] + list(range(62, 11, -2)) + list(range(63, 10, -2))
    first = [b for b in order if vnni_factor and b % vnni_factor == 0]
    for b in first + order:
        if S % b == 0:
            return [S // b, b]
    return [1, S]


class BlockedParameter(torch.nn.Parameter):
    """A parameter that can switch between its plain and its blocked layout in place. blocking_param =
    (blocking_factors, permute[, blocked_dtype]) as FixLinear attaches it (llm_common.py:468-490)."""

    def __new__(cls, data=None, requires_grad=True):
        self = super().__new__(cls, data, requires_grad)
        self.blocked, self.blocking_param, self.blocking_manager = False, None, None
        return self

    def set_blocking_param(self, blocking_param):
        self.blocking_param = blocking_param

    def is_blocked(self):
        return self.blocked

    def block(self):
        if self.blocked or (self.blocking_manager is None and self.blocking_param is None):
            return
        if self.blocking_manager is None:
            bp = self.blocking_param
            self.unblocked_dtype = self.dtype
            self.blocked_dtype = bp[2] if len(bp) > 2 and bp[2] is not None else self.dtype
            self.blocking_manager = BlockingManager(self.data.shape, blocking_factors=bp[0], permute=bp[1])
        self.data = self.blocking_manager.block(self.data).to(self.blocked_dtype)
        if self.grad is not None:
            self.grad.data = self.blocking_manager.block(self.grad.data).to(self.blocked_dtype)
        self.blocked = True

    def unblock(self):
        if not self.blocked:
            return
        self.data = self.blocking_manager.unblock(self.data).to(self.unblocked_dtype)
        if self.grad is not None:
            self.grad.data = self.blocking_manager.unblock(self.grad.data).to(self.unblocked_dtype)
        self.blocked = False


class BlockedModule(torch.nn.Module):
    """State dicts always hold the plain layout: blocked parameters are unblocked for saving and blocked again
    afterwards, and re-blocked after loading (blocked_layout.py:308-364)."""

    def _own_blocked(self):
        return [p for p in self.parameters(recurse=False) if isinstance(p, BlockedParameter) and p.is_blocked()]

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        blocked = self._own_blocked()
        for p in blocked:
            p.unblock()
        try:
            super()._save_to_state_dict(destination, prefix, keep_vars)
        finally:
            for p in blocked:
                p.block()

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        blocked = self._own_blocked()
        for p in blocked:
            p.unblock()
        try:
            super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)
        finally:
            for p in blocked:
                p.block()


def linear_blocking_param(bk=16, bc=64, vnni=2, blocked_dtype=None):
    """The blocking FixLinear gives a Linear weight [N, K]: [N/bk, K/bc, bc/vnni, bk, vnni]."""
    return ([bk, [bc // vnni, vnni]], [0, 2, 3, 1, 4], blocked_dtype)
