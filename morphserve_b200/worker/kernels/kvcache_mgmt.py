"""KV append / scatter: drop-in for the reference's
``swiftllm.worker.kernels.kvcache_mgmt.store_kvcache``
(worker/kernels/kvcache_mgmt.py:298-478), same signature, in place.

Prefill tokens ``[0, num_prefill_tokens)`` are scattered block by block, decode
tokens after them are appended at position ``len-1``.  Both are byte copies, so
results are bit-identical to the reference's.
"""
from __future__ import annotations

import torch

from ..._lib import check, lib
from ._common import device_and_stream, make_pool, require_cuda

# Opt-in: when True, store_kvcache does not launch the decode append itself; it leaves the new
# K/V rows with the infer state and the paged_attention call of the same layer appends them inside
# its own kernel (one launch per layer instead of two).  The pool then changes when attention runs,
# not when store_kvcache returns - which is when the reference's layer code first reads it anyway
# (worker/layers/transformer_layer.py:117-126 then :181-187).  Off by default.
FUSE_DECODE_APPEND = False


def set_fused_decode_append(enabled: bool) -> None:
    global FUSE_DECODE_APPEND
    FUSE_DECODE_APPEND = bool(enabled)


def flush_pending_append(infer_state, pool, block_table, dev, stream) -> None:
    """Append rows that were left for a fused attention call that did not come."""
    state = getattr(infer_state, "__dict__", None)
    pending = state.pop("_mkv_pending_append", None) if state is not None else None
    if pending is None:
        return
    rope = state.pop("_mkv_pending_rope", None)
    if rope is not None:    # rows must be rotated before they reach the pool
        check(lib.mkv_rotary_embedding(dev, stream, rope[0].data_ptr(), rope[1].data_ptr(), rope[2].data_ptr(),
                                       rope[3].data_ptr(), rope[0].shape[0], rope[0].shape[1], rope[1].shape[1],
                                       rope[1].shape[2], rope[0].element_size()), "mkv_rotary_embedding")
    layer, k_dec, v_dec = pending
    n_pre = infer_state.num_prefill_seqs
    check(lib.mkv_store_kv_decode(
        dev, stream, k_dec.data_ptr(), v_dec.data_ptr(), pool, block_table.data_ptr(), block_table.stride(0),
        infer_state.seq_ids[n_pre:].data_ptr(), infer_state.decoding_seq_lens.data_ptr(),
        infer_state.num_decoding_seqs, layer), "mkv_store_kv_decode")


def store_kvcache(
    k: torch.Tensor,            # [num_tokens, num_kv_heads, head_dim]
    v: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    k_cache_new: list,
    v_cache_new: list,
    block_table: torch.Tensor,
    model_config,
    engine_config,
    infer_state,
    cur_layer: int,
):
    assert k.is_contiguous()
    assert v.is_contiguous()
    assert k_cache.is_contiguous()
    assert v_cache.is_contiguous()
    assert block_table.is_contiguous()
    assert infer_state.seq_ids.is_contiguous()
    assert infer_state.decoding_seq_lens.is_contiguous()
    require_cuda(k, "k")

    dev, stream = device_and_stream(k)
    pool = make_pool(k_cache, v_cache, k_cache_new, v_cache_new,
                     infer_state.num_blocks_org, infer_state.kv_cache_new_block_size)
    stride = block_table.stride(0)
    n_pre = infer_state.num_prefill_seqs
    if n_pre > 0:
        check(lib.mkv_store_kv_prefill(
            dev, stream, k.data_ptr(), v.data_ptr(), pool, block_table.data_ptr(), stride,
            infer_state.seq_ids.data_ptr(), infer_state.prefill_seq_start_locs.data_ptr(),
            infer_state.prefill_seq_lens.data_ptr(), n_pre, int(infer_state.max_prefill_len), cur_layer),
            "mkv_store_kv_prefill")
    n_dec = infer_state.num_decoding_seqs
    if n_dec > 0:
        k_dec = k[infer_state.num_prefill_tokens:]
        v_dec = v[infer_state.num_prefill_tokens:]
        state = getattr(infer_state, "__dict__", None)
        if FUSE_DECODE_APPEND and state is not None and k.dtype == torch.float16:
            flush_pending_append(infer_state, pool, block_table, dev, stream)
            state["_mkv_pending_append"] = (cur_layer, k_dec, v_dec)
            return
        if state is not None and state.get("_mkv_pending_rope") is not None:
            from .rotary_emb import flush_pending_rope      # no fused append for this call: rotate now
            flush_pending_rope(infer_state, dev, stream)
        seq_ids = infer_state.seq_ids[n_pre:]
        check(lib.mkv_store_kv_decode(
            dev, stream, k_dec.data_ptr(), v_dec.data_ptr(), pool, block_table.data_ptr(), stride,
            seq_ids.data_ptr(), infer_state.decoding_seq_lens.data_ptr(), n_dec, cur_layer),
            "mkv_store_kv_decode")


def store_kvcache_performance_test(k, v, k_cache, v_cache, k_cache_new, v_cache_new, block_table, model_config,
                                   engine_config, infer_state, cur_layer: int):
    """Import parity: the reference's layer code imports this name next to ``store_kvcache``
    (worker/layers/transformer_layer.py:14) although it never calls it.  The reference's version
    (worker/kernels/kvcache_mgmt.py:481-524) writes into the original pool only, ignoring the chunk lists."""
    return store_kvcache(k, v, k_cache, v_cache, [], [], block_table, model_config, engine_config, infer_state,
                         cur_layer)


def store_kvcache_org_version(k, v, k_cache, v_cache, block_table, model_config, engine_config, infer_state,
                              cur_layer: int):
    """Import parity: the pre-elastic signature the reference keeps (worker/kernels/kvcache_mgmt.py:254-295)."""
    return store_kvcache(k, v, k_cache, v_cache, [], [], block_table, model_config, engine_config, infer_state,
                         cur_layer)
