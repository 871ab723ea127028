"""Blocked layouts on the host (no GPU): BlockingManager / BlockedParameter / BlockedModule against the oracle's
index-level definition of the VNNI2 weight layout and as round trips."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tpp_pytorch_extension_b200.utils import blocked_layout as BL


def test_linear_blocking_is_the_vnni2_layout():
    w = torch.arange(64 * 128, dtype=torch.float32).view(64, 128)
    factors, permute, _ = BL.linear_blocking_param(16, 64, 2)
    bm = BL.BlockingManager(w.shape, factors, permute)
    wb = bm.block(w)
    assert list(wb.shape) == [4, 2, 32, 16, 2] == bm.blocked_shape
    # Wb[k1, c1, c2, k2, c3] = W[16 k1 + k2, 64 c1 + 2 c2 + c3]
    k1, c1, c2, k2, c3 = 3, 1, 17, 5, 1
    assert wb[k1, c1, c2, k2, c3] == w[16 * k1 + k2, 64 * c1 + 2 * c2 + c3]
    assert torch.equal(wb, BL.block_weight(w, 16, 64, 2))
    assert torch.equal(bm.unblock(wb), w)
    assert np.array_equal(O.block_weight(w.numpy()), wb.numpy())


def test_blocking_manager_rejects_bad_specs():
    with pytest.raises(ValueError):
        BL.BlockingManager((10, 8), [3, None])          # 3 does not divide 10
    with pytest.raises(ValueError):
        BL.BlockingManager((8, 8), [2, 2], [0, 1, 2])   # permutation of the wrong length
    with pytest.raises(ValueError):
        BL.BlockingManager((8, 8), [2])                 # one factor for two dimensions
    bm = BL.BlockingManager((8, 6), [[2, 2], None], None)
    assert bm.blocked_shape == [2, 2, 2, 6]
    with pytest.raises(ValueError):
        bm.block(torch.zeros(6, 8))


def test_default_blocking_factors_follow_the_priority_order():
    assert BL.default_blocking_factors(4096) == [64, 64]
    assert BL.default_blocking_factors(96) == [2, 48]
    assert BL.default_blocking_factors(100, prefered_factor=25) == [4, 25]
    assert BL.default_blocking_factors(17) == [1, 17]
    assert BL.default_blocking_factors(66, vnni_factor=4) == [3, 22]   # no multiple of 4 divides 66: plain order
    assert BL.default_blocking_factors(120, vnni_factor=4) == [5, 24]


def test_blocked_parameter_and_module_state_dict_round_trip():
    class M(BL.BlockedModule):
        def __init__(self):
            super().__init__()
            self.weight = BL.BlockedParameter(torch.randn(32, 128))
            self.weight.set_blocking_param(BL.linear_blocking_param(16, 64, 2, torch.bfloat16))
            self.bias = torch.nn.Parameter(torch.randn(32))

    m = M()
    plain = m.weight.data.clone()
    m.weight.block()
    assert m.weight.is_blocked() and m.weight.dtype == torch.bfloat16 and list(m.weight.shape) == [2, 2, 32, 16, 2]
    sd = m.state_dict()
    assert m.weight.is_blocked()                                    # blocked again after saving
    assert list(sd["weight"].shape) == [32, 128]                    # the state dict holds the plain layout
    assert torch.equal(sd["weight"], plain.bfloat16().float())
    m2 = M()
    m2.weight.block()
    m2.load_state_dict(sd)
    assert m2.weight.is_blocked()
    m2.weight.unblock()
    assert torch.equal(m2.weight.data, plain.bfloat16().float())
    m2.weight.unblock()                                             # a second unblock is a no-op
    assert not m2.weight.is_blocked()
