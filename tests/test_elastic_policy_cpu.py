"""The elastic policy (when to expand, when to release) on the host, against the statements of the reference's
scheduler (server/scheduler.py:75-89, :114-131, :189-197), driven with fake engine objects and fake transitions."""
import types
from collections import deque

from morphserve_b200.server import elastic_policy as P


def _engine(free, chunk=100, n_quant=2, quant_list=(31, 30, 29), next_unq=28, floor=20):
    bm = types.SimpleNamespace(num_free_blocks=free)
    model = types.SimpleNamespace(layer_quant_list=list(quant_list), kv_cache_new_block_size=chunk,
                                  gpu_block_manager=bm, next_unquantized_layer=next_unq)
    cfg = types.SimpleNamespace(num_layers_to_quantize=n_quant, num_layers_to_quantize_max=floor)
    return types.SimpleNamespace(model=model, engine_config=cfg)


def _releaser(log, fail_at=None):
    def release(engine):
        if fail_at is not None and len(log) == fail_at:
            return False
        log.append(engine.model.layer_quant_list.pop())
        engine.model.gpu_block_manager.num_free_blocks -= engine.model.kv_cache_new_block_size
        return True
    return release


def test_try_quant2org_follows_the_reference_conditions():
    sched = types.SimpleNamespace(waiting_q=deque())
    # fewer free blocks than n chunks: nothing happens
    log = []
    assert P.try_quant2org(sched, _engine(free=199), _releaser(log)) == 0 and log == []
    # exactly n chunks free: first release (200 > 100), second refused by the half-way condition (100 > 100 is false)
    log = []
    assert P.try_quant2org(sched, _engine(free=200), _releaser(log)) == 1 and log == [29]
    # plenty free: n releases, newest replaced layer first
    log = []
    assert P.try_quant2org(sched, _engine(free=350), _releaser(log)) == 2 and log == [29, 30]
    # a waiting request blocks shrinking altogether
    log = []
    assert P.try_quant2org(types.SimpleNamespace(waiting_q=deque([1])), _engine(free=900), _releaser(log)) == 0
    # nothing quantised
    assert P.try_quant2org(sched, _engine(free=900, quant_list=()), _releaser([])) == 0
    # a release that does not go through ends the attempt
    log = []
    assert P.try_quant2org(sched, _engine(free=900), _releaser(log, fail_at=1)) == 1 and log == [29]
    # the list runs out before n releases
    log = []
    assert P.try_quant2org(sched, _engine(free=900, quant_list=(31,), n_quant=3), _releaser(log)) == 1


def test_admission_expands_by_all_layers_left_or_waits():
    eng = _engine(free=0, chunk=100, n_quant=2, next_unq=28, floor=20)
    sched = types.SimpleNamespace(num_decoding_gpu_blocks=900, num_gpu_blocks=1000)
    calls = []
    grow = lambda e: (calls.append(e.model.next_unquantized_layer),                                # noqa: E731
                      setattr(e.model, "next_unquantized_layer", e.model.next_unquantized_layer - 1))
    assert P.layer_replacements_needed(sched, eng, 100) == 0
    assert P.layer_replacements_needed(sched, eng, 101) == 1
    assert P.layer_replacements_needed(sched, eng, 301) == 3
    assert P.admit_with_expand(sched, eng, 60, 40, 2, grow) == (True, 2) and calls == []          # fits as is
    assert P.admit_with_expand(sched, eng, 60, 141, 2, grow) == (True, 0) and calls == [28, 27]   # 2 needed, 2 left
    assert P.admit_with_expand(sched, eng, 60, 141, 0, grow) == (False, 0)                        # none left this step
    eng = _engine(free=0, next_unq=28, floor=20)
    assert P.admit_with_expand(sched, eng, 0, 401, 2, grow) == (False, 2)                         # needs 4 > 2
    eng = _engine(free=0, next_unq=19, floor=20)
    assert P.admit_with_expand(sched, eng, 0, 150, 2, grow) == (False, 2)                         # floor reached
    eng = _engine(free=0, next_unq=0, floor=0)
    calls.clear()
    assert P.admit_with_expand(sched, eng, 0, 150, 1, grow) == (False, 1)       # need 1, next layer 0: 0 - 1 < 0 ...
    eng = _engine(free=0, next_unq=1, floor=0)
    assert P.admit_with_expand(sched, eng, 0, 150, 1, grow) == (True, 0) and calls == [1]         # ... 1 - 1 >= 0 is


def test_expand_instead_of_preempting():
    calls = []
    grow = lambda e: calls.append(e.model.next_unquantized_layer)                                  # noqa: E731
    assert P.expand_before_preempting(None, _engine(free=0, next_unq=5), 2, grow) == (True, 1) and calls == [5]
    assert P.expand_before_preempting(None, _engine(free=0, next_unq=5), 0, grow) == (False, 0)
    assert P.expand_before_preempting(None, _engine(free=0, next_unq=-1), 2, grow) == (False, 2)
