"""The linear entry point that allocates nothing (its scratch is an array built into the library), for callers
that cannot allocate device memory at the call site. Checked through the C ABI against the ordinary entry point
on the same inputs, twice in a row: the second call finds the array as the first one left it."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import make_qweight, to_dev_bf16, to_host_bits

pytestmark = pytest.mark.gpu


def _run_pair(cuda, N, K, M, pair, seed):
    from tpp_pytorch_extension_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(seed)
    qg, wg, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    qu, wu, _ = make_qweight(rng, N, K, "mxfp4", cuda)
    wq, sfa = qg.packed_tc(qu if pair else None)
    x_bits = O.randn_bf16(rng, (M, K))
    x = to_dev_bf16(x_bits, cuda)
    act = 2 if pair else 0
    need = L.tpx_qlinear_mxfp4_tc_scratch_bytes(M, N, K, int(pair))
    assert need <= L.tpx_qlinear_mxfp4_tc_static_max_bytes()
    scratch = torch.zeros(need, dtype=torch.uint8, device=cuda)
    y_ref = torch.empty((M, N), dtype=torch.bfloat16, device=cuda)
    _lib.check(L.tpx_qlinear_mxfp4_tc(wq.data_ptr(), sfa.data_ptr(), int(pair), x.data_ptr(), M, N, K, None, act, None, None,
                                      1.0, y_ref.data_ptr(), scratch.data_ptr(), scratch.numel(), _lib.stream()))
    torch.cuda.synchronize()
    want = to_host_bits(y_ref)
    oracle = O.gate_up(x_bits, wg, wu) if pair else O.qlinear(x_bits, wg)
    assert O.rel_err(want, oracle) <= 2e-2
    for _ in range(2):
        y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
        mem_before = torch.cuda.memory_allocated()
        _lib.check(L.tpx_qlinear_mxfp4_tc_static(wq.data_ptr(), sfa.data_ptr(), int(pair), x.data_ptr(), M, N, K, None, act,
                                                 None, None, 1.0, y.data_ptr(), _lib.stream()))
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == mem_before
        # no kernel gave up on a bounded wait: the word lives inside the built-in array, this call copies it out
        status = ctypes.c_uint(0xFFFFFFFF)
        _lib.check(L.tpx_qlinear_mxfp4_tc_static_status(_lib.stream(), ctypes.byref(status)))
        assert status.value == 0
        got = to_host_bits(y)
        assert O.rel_err(got, want) <= 2e-2
        assert np.array_equal(got, want)  # same kernel, same summation order


def test_static_scratch_matches_ordinary_entry_point(cuda):
    _run_pair(cuda, 1024, 4096, 8, pair=False, seed=1)   # K cut between CTAs: partial tiles go through the scratch
    _run_pair(cuda, 512, 1024, 16, pair=True, seed=2)
    _run_pair(cuda, 1024, 4096, 3, pair=False, seed=3)   # a different shape right after: stale contents are harmless


def test_static_scratch_refuses_oversized_shapes(cuda):
    from tpp_pytorch_extension_b200 import _lib
    L = _lib.lib()
    z = torch.zeros(1 << 16, dtype=torch.uint8, device=cuda)
    rc = L.tpx_qlinear_mxfp4_tc_static(z.data_ptr(), z.data_ptr(), 0, z.data_ptr(), 4096, 14336, 4096, None, 0, None, None, 1.0,
                                       z.data_ptr(), _lib.stream())
    assert rc == 4 and b"built-in array" in L.tpx_last_error()
