"""Rotary position embedding: drop-in for the reference's
``swiftllm.worker.kernels.rotary_emb.rotary_embedding_inplace``
(worker/kernels/rotary_emb.py:43-58), same signature, q and k rotated in place
with the cos/sin rows the infer state carries for every token
(worker/model.py:432-433).  Rounded the way the reference's kernel rounds once
Triton has compiled it for a GPU (one multiply of each output fused into the
add), so results are bit-identical to it; ``set_rope_rounding("written")`` rounds
every operation on its own instead, which is what the same kernel gives in the
Triton interpreter.
"""
from __future__ import annotations

import torch

from ..._lib import check, lib
from . import kvcache_mgmt
from ._common import device_and_stream, require_cuda

# Opt-in, only together with the fused decode append: when True the rows of the DECODE tokens are not
# rotated here; their cos/sin rows stay with the infer state and the attention call of the same layer
# rotates q as it loads it and the new k row before it stores it (one launch per layer instead of
# three).  q and k of the decode tokens then keep their unrotated values in memory.  Off by default.
FUSE_DECODE_ROPE = False


def set_rope_rounding(mode: str) -> None:
    """"compiled" (default): bit-identical to the reference kernel as Triton compiles it for a GPU;
    "written": every product and sum rounds on its own (the kernel's source, operation by operation)."""
    if mode not in ("compiled", "written"):
        raise ValueError("mode is 'compiled' or 'written'")
    check(lib.mkv_rope_set_rounding(1 if mode == "compiled" else 0), "mkv_rope_set_rounding")


def set_fused_decode_rope(enabled: bool) -> None:
    global FUSE_DECODE_ROPE
    FUSE_DECODE_ROPE = bool(enabled)


def _rotate(q, k, cos, sin, dev, stream) -> None:
    check(lib.mkv_rotary_embedding(dev, stream, q.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                   q.shape[0], q.shape[1], k.shape[1], k.shape[2], q.element_size()),
          "mkv_rotary_embedding")


def flush_pending_rope(infer_state, dev, stream) -> None:
    """Rotate decode rows that were left for a fused attention call that did not come."""
    state = getattr(infer_state, "__dict__", None)
    pending = state.pop("_mkv_pending_rope", None) if state is not None else None
    if pending is not None:
        _rotate(*pending, dev, stream)


def rotary_embedding_inplace(
    q: torch.Tensor,    # [num_tokens, num_q_heads, head_dim]
    k: torch.Tensor,    # [num_tokens, num_kv_heads, head_dim]
    infer_state,
):
    assert q.is_contiguous()
    assert k.is_contiguous()
    require_cuda(q, "q")
    cos, sin = infer_state.position_cos, infer_state.position_sin
    assert cos.is_contiguous() and sin.is_contiguous()
    assert cos.dtype == torch.float16 and sin.dtype == torch.float16, "cos/sin tables are fp16 (worker/model.py:240-241)"
    assert q.dtype == k.dtype and q.dtype in (torch.float16, torch.float32)
    assert cos.shape[0] == q.shape[0] == k.shape[0] and cos.shape[1] * 2 == q.shape[2] == k.shape[2]
    dev, stream = device_and_stream(q)
    flush_pending_rope(infer_state, dev, stream)
    n_tok = q.shape[0]
    state = getattr(infer_state, "__dict__", None)
    n_dec = getattr(infer_state, "num_decoding_seqs", 0)
    if (FUSE_DECODE_ROPE and kvcache_mgmt.FUSE_DECODE_APPEND and state is not None and n_dec > 0
            and q.dtype == torch.float16 and q.shape[2] == 128 and not getattr(infer_state, "ignore_kvcache", False)):
        n_pre = n_tok - n_dec
        state["_mkv_pending_rope"] = (q[n_pre:], k[n_pre:], cos[n_pre:], sin[n_pre:])
        n_tok = n_pre
    if n_tok > 0:
        _rotate(q[:n_tok], k[:n_tok], cos[:n_tok], sin[:n_tok], dev, stream)
