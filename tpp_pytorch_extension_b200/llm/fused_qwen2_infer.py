"""Mirror of src/tpp_pytorch_extension/llm/fused_qwen2_infer.py: Qwen2 shares the Llama runner; its decoder layers
carry biases on the q, k and v projections (torch.classes.tpp_llm.Qwen2DecoderLayer)."""
from .fused_llama_infer import OptimizeModelForQwen2  # noqa: F401
