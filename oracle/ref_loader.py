"""Imports the staged reference (``oracle/_ref``, see build_ref.py).  TEST INFRASTRUCTURE ONLY.

The reference's package directory is ``MorphServe/`` while every one of its
modules imports ``swiftllm.*`` and its ``__init__`` pulls ray / awq, which are
not installed.  ``load()`` therefore registers empty namespace packages named
``swiftllm``, ``swiftllm.worker`` ... whose ``__path__`` points into the staged
tree, a stand-in ``swiftllm.utils`` holding the three names the path needs
(the real module imports ``evaluate`` at its top), and - for code that imports
it although decode never calls it - a stand-in ``vllm_flash_attn`` whose
prefill attention is torch's scaled_dot_product_attention per prompt.

With ``interpret=False`` (default) the reference's Triton kernels are compiled
by Triton for the local GPU; with ``interpret=True`` (must be chosen before
triton is first imported in the process) they run on CPU tensors.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
PKG = os.path.join(REF, "MorphServe")

_NAMESPACES = {
    "swiftllm": PKG,
    "swiftllm.worker": os.path.join(PKG, "worker"),
    "swiftllm.worker.kernels": os.path.join(PKG, "worker", "kernels"),
    "swiftllm.worker.layers": os.path.join(PKG, "worker", "layers"),
    "swiftllm.server": os.path.join(PKG, "server"),
}


def available() -> bool:
    return os.path.isfile(os.path.join(PKG, "worker", "kernels", "paged_attn.py"))


def ext_available() -> bool:
    return any(f.startswith("swiftllm_c") and f.endswith(".so") for f in (os.listdir(REF) if os.path.isdir(REF) else []))


def why_unavailable() -> str:
    return ("oracle/_ref is not staged: run `python oracle/build_ref.py <MorphServe checkout>` "
            "(it is git-ignored and travels with the working tree)")


def _flash_attn_stand_in():
    import torch

    def flash_attn_varlen_func(q, k, v, cu_q, cu_k, max_q, max_k, softmax_scale=None, causal=False, **_):
        out = torch.empty_like(q)
        bounds = cu_q.tolist()
        g = q.shape[1] // k.shape[1]
        for a, b in zip(bounds[:-1], bounds[1:]):
            if b <= a:
                continue
            qi = q[a:b].transpose(0, 1).float()
            ki = k[a:b].transpose(0, 1).repeat_interleave(g, dim=0).float()
            vi = v[a:b].transpose(0, 1).repeat_interleave(g, dim=0).float()
            oi = torch.nn.functional.scaled_dot_product_attention(qi, ki, vi, is_causal=causal, scale=softmax_scale)
            out[a:b] = oi.transpose(0, 1).to(q.dtype)
        return out

    m = types.ModuleType("vllm_flash_attn")
    m.flash_attn_varlen_func = flash_attn_varlen_func
    return m


def install_namespaces(skip=()) -> None:
    """Registers the namespace packages and stand-ins; modules already present under a name in `skip`
    (or any submodule registered earlier, e.g. by morphserve_b200.install_as_swiftllm) are left alone."""
    if not available():
        raise ImportError(why_unavailable())
    for name, path in _NAMESPACES.items():
        m = sys.modules.get(name)
        if m is None or not getattr(m, "__path__", None):
            if m is None:
                m = types.ModuleType(name)
                sys.modules[name] = m
            m.__path__ = [path]
        parent, _, leaf = name.rpartition(".")
        if parent:
            setattr(sys.modules[parent], leaf, m)
    if "swiftllm.utils" not in sys.modules:
        u = types.ModuleType("swiftllm.utils")
        u.cdiv = lambda a, b: (a + b - 1) // b
        u.KB, u.MB, u.GB = 1024, 1024 ** 2, 1024 ** 3
        sys.modules["swiftllm.utils"] = u
        sys.modules["swiftllm"].utils = u
    if "vllm_flash_attn" not in sys.modules:
        try:
            importlib.import_module("vllm_flash_attn")
        except Exception:
            sys.modules["vllm_flash_attn"] = _flash_attn_stand_in()


def load_ext():
    """The reference's compiled ``swiftllm_c`` (host C++), or None when it was not built."""
    if not ext_available():
        return None
    import importlib.util
    import sysconfig
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    path = os.path.join(REF, "swiftllm_c" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
    spec = importlib.util.spec_from_file_location("swiftllm_c", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class Reference:
    """Handles on the reference's own functions and classes for the KV-cache path."""

    def __init__(self, with_ext: bool = True):
        install_namespaces()
        K = "swiftllm.worker.kernels."
        self.paged_attn = importlib.import_module(K + "paged_attn")
        self.kvcache_mgmt = importlib.import_module(K + "kvcache_mgmt")
        self.block_mgmt = importlib.import_module(K + "block_mgmt")
        self.rotary_emb = importlib.import_module(K + "rotary_emb")
        self.block_manager = importlib.import_module("swiftllm.worker.block_manager")
        self.infer_state = importlib.import_module("swiftllm.worker.infer_state")
        self.paged_attention = self.paged_attn.paged_attention
        self.store_kvcache = self.kvcache_mgmt.store_kvcache
        self.rotary_embedding_inplace = self.rotary_emb.rotary_embedding_inplace
        self.BlockManager = self.block_manager.BlockManager
        self.LlamaInferState = self.infer_state.LlamaInferState
        self.swiftllm_c = load_ext() if with_ext else None


_cached = None


def load(interpret: bool = False, with_ext: bool = True) -> Reference:
    global _cached
    if interpret:
        if "triton" in sys.modules and os.environ.get("TRITON_INTERPRET") != "1":
            raise RuntimeError("TRITON_INTERPRET must be set before triton is first imported")
        os.environ["TRITON_INTERPRET"] = "1"
    if _cached is None:
        _cached = Reference(with_ext)
    return _cached
