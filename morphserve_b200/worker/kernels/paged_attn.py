"""Decode paged attention: drop-in for the reference's
``swiftllm.worker.kernels.paged_attn.paged_attention``
(worker/kernels/paged_attn.py:700-1015), same signature, writes ``o`` in place.

What changes underneath: the two Triton phases become one sm_100a kernel that
packs the query heads of a GQA group on one K/V stream (each tile read once per
KV head), schedules (sequence, chunk) work items longest-first from a plan made
once per decode step, and merges split sequences in the same launch.  There is
no allocation, no host synchronisation and no full-table scan per call (the
reference does ``(block_table >= num_blocks_org).any()`` per layer when elastic
chunks exist, :893-895); elastic blocks are resolved in the kernel.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..._lib import check, lib
from ._common import attn_workspace, device_and_stream, make_pool, require_cuda
from .kvcache_mgmt import flush_pending_append


def _plan_for(infer_state, ws, dev, stream, lens, seq_ids, batch, hq, hkv, d, bs, max_blocks, cur_layer):
    """Plan once per decode step.  A plan made for this infer state is reused by the later layers of the same step
    only: the layer number has to go UP from call to call (the reference's model walks its layers in order,
    worker/model.py:276-291).  A call whose layer is not above the previous one starts a new step - the caller may
    have updated ``decoding_seq_lens`` in place and reused the object - and is planned afresh, as is anything whose
    tensors, batch or workspace changed."""
    token = (ws.generation, dev, stream, batch, max_blocks, lens.data_ptr(), seq_ids.data_ptr())
    state = getattr(infer_state, "__dict__", None)
    if state is not None:
        seen = state.get("_mkv_plan_token")
        if seen is not None and seen[0] == token and cur_layer > seen[1]:
            state["_mkv_plan_token"] = (token, cur_layer)
            return
    ws.generation += 1
    token = (ws.generation,) + token[1:]
    check(lib.mkv_attn_plan(dev, stream, ws.tensor.data_ptr(), ws.nbytes, lens.data_ptr(), seq_ids.data_ptr(), batch,
                            hq, hkv, d, bs, max_blocks), "mkv_attn_plan")
    if state is not None:
        state["_mkv_plan_token"] = (token, cur_layer)


def paged_attention(
    q: torch.Tensor,                # [num_decoding_seqs, num_q_heads, head_dim]
    k_cache: torch.Tensor,          # [num_blocks, num_layers, num_kv_heads, block_size, head_dim]
    v_cache: torch.Tensor,
    k_cache_new: list,              # elastic chunks, each [chunk_blocks, num_layers, num_kv_heads, block_size, head_dim]
    v_cache_new: list,
    block_table: torch.Tensor,      # [max_seqs_in_block_table, max_blocks_per_seq] int32
    model_config,
    engine_config,
    infer_state,
    cur_layer: int,
    o: torch.Tensor,                # [num_decoding_seqs, num_q_heads(*)head_dim]
):
    assert q.is_contiguous()
    assert k_cache.is_contiguous()
    assert v_cache.is_contiguous()
    assert block_table.is_contiguous()
    assert infer_state.seq_block_size % engine_config.block_size == 0
    assert o.is_contiguous()
    require_cuda(q, "q")

    batch = infer_state.num_decoding_seqs
    if batch == 0:
        return
    dev, stream = device_and_stream(q)
    hq, hkv, d = model_config.num_q_heads, model_config.num_kv_heads, model_config.head_dim
    bs = engine_config.block_size
    pool = make_pool(k_cache, v_cache, k_cache_new, v_cache_new,
                     infer_state.num_blocks_org, infer_state.kv_cache_new_block_size)
    lens = infer_state.decoding_seq_lens
    seq_ids = infer_state.seq_ids[infer_state.num_prefill_seqs:]
    max_len = getattr(infer_state, "max_decoding_len", None)
    if not max_len:
        max_len = engine_config.max_blocks_per_seq * bs
    max_blocks = min((max_len + bs - 1) // bs, block_table.shape[1])

    ws = attn_workspace(dev, batch, hq, hkv, d, max_blocks, stream)
    _plan_for(infer_state, ws, dev, stream, lens, seq_ids, batch, hq, hkv, d, bs, max_blocks, cur_layer)
    state = getattr(infer_state, "__dict__", None)
    pending = state.get("_mkv_pending_append") if state is not None else None
    rope = state.get("_mkv_pending_rope") if state is not None else None
    if rope is not None and not (pending is not None and pending[0] == cur_layer
                                 and rope[0].data_ptr() == q.data_ptr() and rope[1].data_ptr() == pending[1].data_ptr()):
        from .rotary_emb import flush_pending_rope      # not this call's rows: rotate them in place now
        flush_pending_rope(infer_state, dev, stream)
        rope = None
    if rope is not None:
        # rotary_embedding_inplace and store_kvcache both left this layer's decode rows to this kernel
        del state["_mkv_pending_rope"], state["_mkv_pending_append"]
        check(lib.mkv_paged_attention_decode_rope_append(
            dev, stream, q.data_ptr(), o.data_ptr(), pending[1].data_ptr(), pending[2].data_ptr(),
            rope[2].data_ptr(), rope[3].data_ptr(), pool, block_table.data_ptr(), block_table.stride(0),
            seq_ids.data_ptr(), lens.data_ptr(), batch, hq, cur_layer, float(infer_state.softmax_scale), max_blocks,
            ws.tensor.data_ptr(), ws.nbytes), "mkv_paged_attention_decode_rope_append")
        return
    if pending is not None and pending[0] == cur_layer:
        # store_kvcache left this layer's new rows to be appended inside the attention kernel
        del state["_mkv_pending_append"]
        check(lib.mkv_paged_attention_decode_append(
            dev, stream, q.data_ptr(), o.data_ptr(), pending[1].data_ptr(), pending[2].data_ptr(), pool,
            block_table.data_ptr(), block_table.stride(0), seq_ids.data_ptr(), lens.data_ptr(), batch, hq,
            cur_layer, float(infer_state.softmax_scale), max_blocks, ws.tensor.data_ptr(), ws.nbytes),
            "mkv_paged_attention_decode_append")
        return
    if pending is not None:
        flush_pending_append(infer_state, pool, block_table, dev, stream)
    check(lib.mkv_paged_attention_decode(
        dev, stream, q.data_ptr(), o.data_ptr(), pool, block_table.data_ptr(), block_table.stride(0),
        seq_ids.data_ptr(), lens.data_ptr(), batch, hq, cur_layer, float(infer_state.softmax_scale),
        max_blocks, ws.tensor.data_ptr(), ws.nbytes), "mkv_paged_attention_decode")


def paged_attention_push(
    q: torch.Tensor,                # [num_decoding_seqs, local num_q_heads, head_dim]
    k_cache: torch.Tensor,          # this rank's KV heads only: [num_blocks, num_layers, local num_kv_heads, 16, 128]
    v_cache: torch.Tensor,
    k_cache_new: list,
    v_cache_new: list,
    block_table: torch.Tensor,
    model_config,                   # num_q_heads / num_kv_heads are the LOCAL counts
    engine_config,
    infer_state,
    cur_layer: int,
    out_ptrs,                       # device addresses of every destination matrix [batch, out_row_stride] fp16
    out_row_stride: int,            # elements per destination row (= total query heads * head_dim)
    out_col_offset: int,            # first column of this rank's slice (= first local query head * head_dim)
    k_new: torch.Tensor = None,     # optional fused append of the newest token's rows [batch, local kv heads, 128]
    v_new: torch.Tensor = None,
    ready_ptrs=None,                # device addresses of this rank's "slice landed" word on every destination
    epoch: int = 0,                 # value written there when the launch's last store is done; grows per launch
):
    """Decode attention for KV-head sharding (no counterpart in the single-GPU reference): the result is
    stored into the same column slice of every matrix in ``out_ptrs`` - the local one and, through
    peer-mapped pointers, the other ranks' - from inside the kernel, replacing attention + all-gather.
    Before anyone reads its matrix the caller either runs a barrier across the ranks, or passes ``ready_ptrs`` /
    ``epoch`` and lets every rank ``wait_ready`` for the other ranks' words."""
    assert q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous() and block_table.is_contiguous()
    require_cuda(q, "q")
    batch = infer_state.num_decoding_seqs
    if batch == 0:
        return
    dev, stream = device_and_stream(q)
    hq, hkv, d = model_config.num_q_heads, model_config.num_kv_heads, model_config.head_dim
    bs = engine_config.block_size
    pool = make_pool(k_cache, v_cache, k_cache_new, v_cache_new,
                     infer_state.num_blocks_org, infer_state.kv_cache_new_block_size)
    lens = infer_state.decoding_seq_lens
    seq_ids = infer_state.seq_ids[infer_state.num_prefill_seqs:]
    max_len = getattr(infer_state, "max_decoding_len", None) or engine_config.max_blocks_per_seq * bs
    max_blocks = min((max_len + bs - 1) // bs, block_table.shape[1])
    ws = attn_workspace(dev, batch, hq, hkv, d, max_blocks, stream)
    _plan_for(infer_state, ws, dev, stream, lens, seq_ids, batch, hq, hkv, d, bs, max_blocks, cur_layer)
    ptrs = (C.c_void_p * len(out_ptrs))(*[int(x) for x in out_ptrs])
    n_ready = len(ready_ptrs) if ready_ptrs else 0
    ready = (C.c_void_p * max(n_ready, 1))(*[int(x) for x in (ready_ptrs or [0])])
    check(lib.mkv_paged_attention_decode_push(
        dev, stream, q.data_ptr(), ptrs, len(out_ptrs), int(out_row_stride), int(out_col_offset),
        ready if n_ready else None, n_ready, int(epoch),
        k_new.data_ptr() if k_new is not None else None, v_new.data_ptr() if v_new is not None else None,
        pool, block_table.data_ptr(), block_table.stride(0), seq_ids.data_ptr(), lens.data_ptr(), batch, hq,
        cur_layer, float(infer_state.softmax_scale), max_blocks, ws.tensor.data_ptr(), ws.nbytes),
        "mkv_paged_attention_decode_push")


def wait_ready(flags: torch.Tensor, epoch: int, status: torch.Tensor, timeout_s: float = 1.0) -> None:
    """Queue, on the current stream, a bounded wait until every int32 word of ``flags`` (this GPU's memory; word r is
    written by rank r's ``paged_attention_push``) has reached ``epoch``.  A word that does not arrive within
    ``timeout_s`` sets its bit in ``status`` (int32 [1] on this GPU, accumulated) and the wait ends."""
    require_cuda(flags, "flags")
    assert flags.dtype == torch.int32 and status.dtype == torch.int32 and flags.is_contiguous()
    dev, stream = device_and_stream(flags)
    check(lib.mkv_wait_ready(dev, stream, flags.data_ptr(), flags.numel(), int(epoch), int(timeout_s * 1e9),
                             status.data_ptr()), "mkv_wait_ready")
