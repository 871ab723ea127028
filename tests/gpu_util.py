"""Helpers shared by the GPU parity tests: numpy bf16 bit patterns <-> torch CUDA tensors."""
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
    torch.cuda.synchronize()
    for buf in _lib._scratch.values():
        assert int(buf[65532:65536].view(torch.int32).item()) == 0, "a kernel gave up on a bounded wait"
