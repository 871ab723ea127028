"""Helpers shared by the GPU parity tests: numpy bf16 bit patterns <-> torch CUDA tensors."""
import contextlib
import os

import numpy as np
import torch

from oracle import oracle as O


def to_dev_bf16(bits, dev):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(dev).view(torch.bfloat16)


def to_host_bits(t):
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def make_qweight(rng, N, K, kind, dev, block=64, std=0.02):
    """Seeded weight -> (QTensor on the GPU via the C ABI, oracle's dequantised plain fp32 weight, raw oracle tensors)."""
    from tpp_pytorch_extension_b200._C import _qtype
    w = O.randn_bf16(rng, (N, K), std)
    wb = to_dev_bf16(O.block_weight(w), dev)
    if kind == "mxfp4":
        q = _qtype.remap_and_quantize_mxfp4(wb)
        codes, scales = O.remap_and_quantize_mxfp4(w)
        return q, O.mxfp4_dequant_plain(codes, scales), (codes, scales)
    q = _qtype.remap_and_quantize_qint8(wb, block)
    qq, ss, bs = O.remap_and_quantize_qint8(w, block)
    return q, O.int8_dequant_plain(qq, ss, bs), (qq, ss, bs)


def assert_no_kernel_error():
    """The bounded waits inside the kernels report through a word in the scratch buffer."""
    from tpp_pytorch_extension_b200 import _lib
    _lib.assert_no_kernel_error()


@contextlib.contextmanager
def knob_env(**env):
    """Sets TPX_* kernel-selection switches for the enclosed code. The library and the Python layer read them once, so
    both are told to read again on the way in and on the way out."""
    from tpp_pytorch_extension_b200 import _lib
    old = {k: os.environ.get(k) for k in env}
    os.environ.update({k: str(v) for k, v in env.items()})
    _lib.reload_options()
    try:
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
        _lib.reload_options()
