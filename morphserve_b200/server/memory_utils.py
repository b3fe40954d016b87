"""Elastic KV-pool resize: the KV half of the reference's
``server/memory_utils.py`` - expand (:370-420), the release rule (:529-544,
:602-613, :644-651) - plus compaction, which the reference does not have.

Functions take the reference's ``engine`` object duck-typed: they touch
``engine.model.{k_cache,v_cache,k_cache_new,v_cache_new,kv_cache_new_block_size,
gpu_block_manager}`` and ``engine.scheduler.num_gpu_blocks`` only.  Swapping the
transformer layer's weights (the other half of org2quant / quant2org) is not
part of the KV path and stays with the caller.

Compaction rule (defined here; the reference can only release a chunk that is
already empty, :529-544,:622-624).  Given a target size T in blocks:
  src = ascending ids >= T that are in use,
  dst = the first len(src) ascending free ids < T (first-fit, like allocation),
  fail, changing nothing, if there are too few;
  copy K and V of block src[i] to dst[i] (all layers);
  in every row r of the block table, entries [0, num_seq_allocated_blocks[r])
  equal to src[i] become dst[i]; other columns and rows of freed sequences keep
  whatever they held; is_block_free[dst] = False, is_block_free[src] = True;
  num_free_blocks is unchanged and the source blocks keep their bytes.
"""
from __future__ import annotations

import torch

from .._lib import check, lib
from ..worker.kernels._common import device_and_stream, make_pool


def update_kvcache_after_replacing_layer(engine, layer_id, acquire=None):
    """Attach the chunk freed by quantising ``layer_id`` to the pool.
    server/memory_utils.py:370-420.  ``acquire`` defaults to
    ``swiftllm_c.acquire_new_kvcache``."""
    if acquire is None:
        from ..swiftllm_c import acquire_new_kvcache as acquire
    k_cache_new, v_cache_new = acquire(layer_id)
    return attach_kvcache_chunk(engine, k_cache_new, v_cache_new)


def attach_kvcache_chunk(engine, k_cache_new: torch.Tensor, v_cache_new: torch.Tensor) -> int:
    """Bookkeeping of an expand (server/memory_utils.py:389-420)."""
    model = engine.model
    bm = model.gpu_block_manager
    n = len(k_cache_new)
    if model.k_cache_new and n != model.kv_cache_new_block_size:
        raise RuntimeError("elastic KV chunks must all have the same number of blocks")
    model.k_cache_new.append(k_cache_new)
    model.v_cache_new.append(v_cache_new)
    bm.num_blocks += n
    bm.num_free_blocks += n
    model.kv_cache_new_block_size = k_cache_new.shape[0]
    is_block_free_new = torch.ones((n,), dtype=torch.bool, device=bm.is_block_free.device)
    bm.is_block_free = torch.cat((bm.is_block_free, is_block_free_new), dim=0)
    if getattr(engine, "scheduler", None) is not None:
        engine.scheduler.num_gpu_blocks += n
    return n


def if_kv_cache_unused(engine, layer_id=None) -> bool:
    """True when the LAST chunk holds no live block (server/memory_utils.py:529-544)."""
    model = engine.model
    last = len(model.k_cache_new) - 1
    assert last >= 0, f"no elastic KV chunk is attached (layer {layer_id}): nothing to check"
    kv_cache_index = last
    n = model.kv_cache_new_block_size
    start = model.gpu_block_manager.num_blocks_org + n * kv_cache_index
    return bool(model.gpu_block_manager.is_block_free[start:start + n].all())


def free_kv_cache_tensors(engine, layer_id=None) -> None:
    """Drop the last chunk's tensors (server/memory_utils.py:602-613)."""
    model = engine.model
    last = len(model.k_cache_new) - 1
    assert last >= 0, f"no elastic KV chunk is attached (layer {layer_id}): nothing to drop"
    del model.k_cache_new[last]
    del model.v_cache_new[last]


def release_last_kvcache_chunk(engine, layer_id=None) -> bool:
    """The KV half of quant2org_and_update_kvcache (server/memory_utils.py:617-662):
    refuse (return False) unless the last chunk is empty, else drop its tensors and
    shrink the counters and the free bitmap."""
    if not if_kv_cache_unused(engine, layer_id):
        return False
    model = engine.model
    bm = model.gpu_block_manager
    n = model.kv_cache_new_block_size
    free_kv_cache_tensors(engine, layer_id)
    bm.num_blocks -= n
    bm.num_free_blocks -= n
    bm.is_block_free = bm.is_block_free[:-n]
    if getattr(engine, "scheduler", None) is not None:
        engine.scheduler.num_gpu_blocks -= n
    return True


def compact_kvcache_nosync(engine, target_num_blocks: int) -> torch.Tensor:
    """Compaction with no host round trip: plan (one block scans the bitmap, pairs sources with destinations and
    updates the bitmap), block copy and table remap are enqueued back to back, the pair count travelling through
    device memory.  Returns the plan's device record, int64[4]: pairs moved (0 when refused), 1 when refused because
    the low region has too few free blocks (nothing changed), live blocks found at or above the target, free blocks
    found below it.  Capturable in a CUDA graph; `compact_kvcache` is this plus one read of the record."""
    model = engine.model
    bm = model.gpu_block_manager
    free = bm.is_block_free
    total = free.shape[0]
    T = int(target_num_blocks)
    if not 0 <= T <= total:
        raise RuntimeError(f"compaction target {T} outside the pool of {total} blocks")
    dev, stream = device_and_stream(free)
    device = free.device
    capacity = min(total - T, T)               # more sources than ids below the target can never be served
    pairs = torch.empty((2, max(capacity, 1)), dtype=torch.int64, device=device)
    result = torch.empty((4,), dtype=torch.int64, device=device)
    src, dst = pairs[0], pairs[1]
    check(lib.mkv_compact_plan(dev, stream, free.data_ptr(), total, T, src.data_ptr(), dst.data_ptr(), capacity,
                               result.data_ptr()), "mkv_compact_plan")
    if capacity > 0:
        pool = make_pool(model.k_cache, model.v_cache, model.k_cache_new, model.v_cache_new,
                         bm.num_blocks_org, model.kv_cache_new_block_size)
        check(lib.mkv_copy_blocks_counted(dev, stream, pool, src.data_ptr(), dst.data_ptr(), capacity,
                                          result.data_ptr()), "mkv_copy_blocks_counted")
        check(lib.mkv_remap_block_table_counted(dev, stream, bm.block_table.data_ptr(), bm.block_table.stride(0),
                                                bm.block_table.shape[0], bm.num_seq_allocated_blocks.data_ptr(),
                                                src.data_ptr(), dst.data_ptr(), capacity, result.data_ptr()),
              "mkv_remap_block_table_counted")
    return result


def compact_kvcache(engine, target_num_blocks: int) -> int:
    """Move every live block with id >= ``target_num_blocks`` below it and remap the
    block table (rule in the module docstring).  Returns the number of blocks
    moved, or -1 - with nothing changed - when the low region has too few free
    blocks.  The host reads the outcome once, after all of the work is enqueued."""
    moved, refused, _, _ = compact_kvcache_nosync(engine, target_num_blocks).tolist()
    return -1 if refused else moved


def shrink_kvcache(engine, num_chunks_to_release: int) -> int:
    """Compact to the boundary below the last ``num_chunks_to_release`` chunks, then
    release them one by one with the reference's rule.  Returns chunks released."""
    model = engine.model
    bm = model.gpu_block_manager
    k = min(int(num_chunks_to_release), len(model.k_cache_new))
    if k <= 0:
        return 0
    target = bm.num_blocks_org + (len(model.k_cache_new) - k) * model.kv_cache_new_block_size
    if compact_kvcache(engine, target) < 0:
        return 0
    released = 0
    for _ in range(k):
        if not release_last_kvcache_chunk(engine):
            break
        released += 1
    return released


# --------------------------------------------------------------------------
# The KV half of the reference's two elastic transitions, callable from its scheduler
# --------------------------------------------------------------------------
def org2quant_and_update_kvcache(engine, update_kvcache: bool = True, replace_layer=None, acquire=None) -> int:
    """Expand: the next layer (from the last one downward, worker/model.py:81) gives up its fp16 slab and the pool
    gains the chunk carved out of it.  server/memory_utils.py:93-112, KV part and bookkeeping; swapping the layer's
    weights is the caller's `replace_layer(engine, layer_id)` (the reference's swap_layer_in_place, :103), which
    must have put the quantised image into the slab before the chunk behind it is zero-filled.
    Returns the layer that was replaced.  Raises RuntimeError where the reference exits (no layer left, :99-101)."""
    model = engine.model
    layer_id = model.next_unquantized_layer
    if layer_id < 0:
        raise RuntimeError("no fp16 layer left to replace")
    if replace_layer is not None:
        replace_layer(engine, layer_id)
    if update_kvcache:
        update_kvcache_after_replacing_layer(engine, layer_id, acquire)
    model.is_layer_quant_list[layer_id] = True
    model.layer_quant_list.append(layer_id)
    model.next_unquantized_layer -= 1
    return layer_id


def quant2org_and_update_kvcache(engine, update_kvcache: bool = True, restore_layer=None, compact: bool = True) -> bool:
    """Release: the most recently replaced layer gets its fp16 weights back and the pool loses the LAST chunk.
    server/memory_utils.py:617-662.  The reference gives up (returns False, :622-624) whenever a single live
    block sits in that chunk; with `compact` the live blocks are first moved below the chunk
    (`compact_kvcache`, block tables remapped), so the release only fails when the rest of the pool has too few free
    blocks to take them.  The chunk's memory is about to be overwritten by the restored weights - on another stream
    in the reference (csrc/src/memory_manager.cpp:291-322) - so the copies are waited for before `restore_layer(engine,
    layer_id)` (the reference's free_quantized_layer + replace_layer_quant2org + rebuild, :626-641) runs."""
    model = engine.model
    bm = model.gpu_block_manager
    layer_id = model.next_unquantized_layer + 1
    if update_kvcache and not if_kv_cache_unused(engine, layer_id):
        if not compact:
            return False
        boundary = bm.num_blocks_org + (len(model.k_cache_new) - 1) * model.kv_cache_new_block_size
        if compact_kvcache(engine, boundary) < 0:
            return False
        torch.cuda.current_stream(bm.is_block_free.device).synchronize()
    if update_kvcache:
        free_kv_cache_tensors(engine, layer_id)
    if restore_layer is not None:
        restore_layer(engine, layer_id)
    if update_kvcache:
        n = model.kv_cache_new_block_size
        bm.num_blocks -= n
        bm.num_free_blocks -= n
        bm.is_block_free = bm.is_block_free[:-n]
        if getattr(engine, "scheduler", None) is not None:
            engine.scheduler.num_gpu_blocks -= n
    model.is_layer_quant_list[layer_id] = False
    model.layer_quant_list.remove(layer_id)
    model.next_unquantized_layer = layer_id
    return True
