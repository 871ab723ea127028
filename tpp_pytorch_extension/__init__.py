"""`import tpp_pytorch_extension` resolves to the B200 implementation of the reference's LLM-inference path: this
package and its submodules are aliases of tpp_pytorch_extension_b200 (same module objects), so that scripts written for
the reference (`from tpp_pytorch_extension.llm.fused_llama_infer import OptimizeModelForLlama`,
`from tpp_pytorch_extension._C import _qtype`) import unchanged. Parts of the reference outside that path (BERT, GNN,
DLRM, AlphaFold, optimizers) are not provided."""
import importlib
import sys

import tpp_pytorch_extension_b200 as _impl

for _name in ("_C", "_C._fused_llm_infer", "_C._qtype", "_C._tpp_attn", "llm", "llm.llm_common", "llm.fused_llama_infer",
              "llm.fused_qwen2_infer", "utils", "utils.blocked_layout", "qtypes"):
    sys.modules[__name__ + "." + _name] = importlib.import_module("tpp_pytorch_extension_b200." + _name)

_C = sys.modules[__name__ + "._C"]
llm = sys.modules[__name__ + ".llm"]
utils = sys.modules[__name__ + ".utils"]
qtypes = sys.modules[__name__ + ".qtypes"]
print_debug_timers = _impl.print_debug_timers
reset_debug_timers = _impl.reset_debug_timers
_C.print_debug_timers = _impl.print_debug_timers
_C.reset_debug_timers = _impl.reset_debug_timers
