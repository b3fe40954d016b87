"""When the pool grows and shrinks: the elastic decisions of the reference's scheduler
(server/scheduler.py:75-89 ``try_quant2org``, :114-131 and :189-197 the expand conditions), as functions over the
same duck-typed ``scheduler`` / ``engine`` objects, so that the reference's ``Scheduler`` can delegate to them.

Pure host logic: integers in, calls to the two transitions (``org2quant_and_update_kvcache``,
``quant2org_and_update_kvcache`` of ``memory_utils``) out.  The transitions are parameters, which is also how the
tests drive the policy without a GPU.
"""
from __future__ import annotations


def try_quant2org(scheduler, engine, quant2org=None) -> int:
    """server/scheduler.py:75-89.  Shrink only when nothing is waiting and the pool has at least
    ``num_layers_to_quantize`` chunks' worth of free blocks; then release up to that many chunks, each only while
    more than half that many chunks' worth stays free; stop at the first release that does not go through.
    Returns the number of chunks released.

    With the reference's own transition a release fails as soon as the last chunk holds one live block; the
    default transition here compacts first, so the free-block conditions above are what decides."""
    if quant2org is None:
        from .memory_utils import quant2org_and_update_kvcache as quant2org
    model, cfg = engine.model, engine.engine_config
    n = cfg.num_layers_to_quantize
    released = 0
    if (len(model.layer_quant_list) > 0 and not scheduler.waiting_q
            and model.gpu_block_manager.num_free_blocks >= model.kv_cache_new_block_size * n):
        for _ in range(n):
            if (len(model.layer_quant_list) > 0
                    and model.gpu_block_manager.num_free_blocks > model.kv_cache_new_block_size * (n // 2)):
                if not quant2org(engine):
                    break
                released += 1
    return released


def layer_replacements_needed(scheduler, engine, blocks_wanted: int) -> int:
    """server/scheduler.py:116: chunks the pool is short of if `blocks_wanted` more blocks are admitted on top of
    the blocks the decoding requests hold (<= 0: they fit)."""
    chunk = engine.model.kv_cache_new_block_size
    short = blocks_wanted + scheduler.num_decoding_gpu_blocks - scheduler.num_gpu_blocks
    if chunk <= 0:
        return 0 if short <= 0 else 1 << 30
    return (short + chunk - 1) // chunk


def admit_with_expand(scheduler, engine, batch_blocks: int, seq_blocks: int, layers_left: int, org2quant=None):
    """server/scheduler.py:114-131, the admission test of one waiting request when ``quant_serve`` is on.
    Returns (admitted, layers_left).  The request fits as is; or the pool is expanded - by ALL `layers_left`
    replacements at once, as the reference does - if that many suffice, the floor ``num_layers_to_quantize_max``
    has not been reached and enough fp16 layers remain; or it has to wait."""
    if org2quant is None:
        from .memory_utils import org2quant_and_update_kvcache as org2quant
    model, cfg = engine.model, engine.engine_config
    need = layer_replacements_needed(scheduler, engine, batch_blocks + seq_blocks)
    if need <= 0:
        return True, layers_left
    if (model.next_unquantized_layer >= cfg.num_layers_to_quantize_max and need <= layers_left
            and model.next_unquantized_layer - need >= 0):
        for _ in range(layers_left):
            org2quant(engine)
        return True, 0
    return False, layers_left


def expand_before_preempting(scheduler, engine, layers_left: int, org2quant=None):
    """server/scheduler.py:189-197: the decoding requests have outgrown the pool.  While fp16 layers remain and this
    step may still replace some, grow by one chunk instead of swapping a request out.  Returns (expanded,
    layers_left)."""
    if org2quant is None:
        from .memory_utils import org2quant_and_update_kvcache as org2quant
    if engine.model.next_unquantized_layer >= 0 and layers_left > 0:
        org2quant(engine)
        return True, layers_left - 1
    return False, layers_left
