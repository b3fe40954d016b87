"""B200-native (sm_100a) KV-cache hot path for MorphServe / SwiftLLM.

Drop-in replacements, behind the reference's own Python names, for

  swiftllm.worker.kernels.paged_attn.paged_attention      -> worker.kernels.paged_attn
  swiftllm.worker.kernels.kvcache_mgmt.store_kvcache      -> worker.kernels.kvcache_mgmt
  swiftllm.worker.kernels.rotary_emb.rotary_embedding_inplace -> worker.kernels.rotary_emb
  swiftllm.worker.kernels.block_mgmt.*                    -> worker.kernels.block_mgmt
  swiftllm.worker.block_manager.BlockManager              -> worker.block_manager
  swiftllm.worker.infer_state.LlamaInferState             -> worker.infer_state
  swiftllm_c.{swap_blocks*, register_kv_cache_info,
              acquire_new_kvcache, ...}                   -> swiftllm_c
  elastic expand / release / compaction bookkeeping       -> server.memory_utils

Everything runs in hand-written CUDA (``libmorphkv.so``, C ABI in
``include/morphkv.h``).  There is no Triton, no CPU path and no fallback:
importing the package without the built library raises.
"""
from __future__ import annotations

import sys
import types

from . import _lib  # noqa: F401  (raises ImportError if libmorphkv.so is missing)
from . import swiftllm_c
from .server import memory_utils
from .worker import block_manager, infer_state, kv_model
from .worker.block_manager import BlockManager
from .worker.infer_state import LlamaInferState
from .worker.kv_model import KVCacheModelState
from .worker.kernels import block_mgmt, kvcache_mgmt, paged_attn, rotary_emb
from .worker.kernels.kvcache_mgmt import set_fused_decode_append, store_kvcache
from .worker.kernels.paged_attn import paged_attention, paged_attention_push, wait_ready
from .worker.kernels.rotary_emb import rotary_embedding_inplace, set_fused_decode_rope, set_rope_rounding

__version__ = "0.1.0"

_ALIASES = {
    "swiftllm.worker.kernels.paged_attn": paged_attn,
    "swiftllm.worker.kernels.kvcache_mgmt": kvcache_mgmt,
    "swiftllm.worker.kernels.block_mgmt": block_mgmt,
    "swiftllm.worker.kernels.rotary_emb": rotary_emb,
    "swiftllm.worker.block_manager": block_manager,
    "swiftllm.worker.infer_state": infer_state,
    "swiftllm_c": swiftllm_c,
}


def install_as_swiftllm(overwrite: bool = True) -> None:
    """Make the reference's import statements resolve to this package.

    Registers the modules above in ``sys.modules`` under the names the
    reference's worker imports (``from swiftllm.worker.kernels.paged_attn import
    paged_attention`` ...).  Call it before importing ``swiftllm.worker.model``.
    If no ``swiftllm`` package is installed the parent packages are created as
    empty namespaces; an installed ``swiftllm`` keeps every module not listed above.
    """
    import importlib.util

    def real_package_exists(top: str) -> bool:
        try:
            return importlib.util.find_spec(top) is not None
        except (ImportError, ValueError):
            return False

    for name, mod in _ALIASES.items():
        parts = name.split(".")
        if not real_package_exists(parts[0]):
            for i in range(1, len(parts)):
                parent = ".".join(parts[:i])
                if parent not in sys.modules:
                    ns = types.ModuleType(parent)
                    ns.__path__ = []
                    sys.modules[parent] = ns
        if overwrite or name not in sys.modules:
            sys.modules[name] = mod
            parent = ".".join(parts[:-1])
            if parent in sys.modules:
                setattr(sys.modules[parent], parts[-1], mod)


__all__ = ["paged_attention", "paged_attention_push", "wait_ready", "store_kvcache", "set_fused_decode_append",
           "rotary_embedding_inplace", "set_fused_decode_rope", "set_rope_rounding", "BlockManager", "LlamaInferState",
           "KVCacheModelState",
           "swiftllm_c", "memory_utils", "install_as_swiftllm"]
