"""Re-exports of the quantizer entry points, as src/tpp_pytorch_extension/qtypes.py:12-24."""
from ._C._qtype import (  # noqa: F401
    Fp8Weight,
    QInt2Tensor,
    QTensor,
    q_per_block_axis,
    q_per_block_block_size,
    q_per_block_pack_size,
    q_per_block_scales,
    remap_and_quantize_mxfp4,
    remap_and_quantize_qint2_intlv,
    remap_and_quantize_qint4,
    remap_and_quantize_qint8,
)
