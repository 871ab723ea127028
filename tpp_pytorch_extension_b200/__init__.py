"""B200 (sm_100a) implementation of the LLM-inference hot path of libxsmm/tpp-pytorch-extension:
weight-only quantized linear, RMSNorm, RoPE + KV-cache attention and the fused Llama decoder layer, behind the
reference's Python names. The compute lives in the in-tree CUDA library (include/tpx_b200.h); there is no CPU path."""
from . import _lib  # noqa: F401


from ._timers import print_debug_timers, reset_debug_timers  # noqa: E402,F401
from . import _torch_namespaces  # noqa: E402

_torch_namespaces.install()
