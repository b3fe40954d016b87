"""Property tests (CPU) of the oracle's integer logic - the rules the CUDA path is held to:
first-fit allocation, the compaction plan and its effect, run coalescing for swaps, chunk sizing."""
import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

from oracle import kv_oracle as O


@settings(max_examples=200, deadline=None)
@given(st.lists(st.booleans(), min_size=1, max_size=200), st.integers(0, 200))
def test_compaction_plan_invariants(free, target):
    free = np.array(free, dtype=bool)
    target = min(target, len(free))
    plan = O.compaction_plan(free, target)
    used_hi = int((~free[target:]).sum())
    free_lo = int(free[:target].sum())
    if free_lo < used_hi:
        assert plan is None
        return
    src, dst = plan
    assert len(src) == len(dst) == used_hi
    assert (np.diff(src) > 0).all() and (np.diff(dst) > 0).all()          # ascending, no duplicates
    assert (src >= target).all() and (dst < target).all()                 # disjoint ranges
    assert (~free[src]).all() and free[dst].all()
    if len(dst):                                                           # first-fit: no free id below the last one is skipped
        assert int(free[: dst[-1] + 1].sum()) == len(dst)


@settings(max_examples=100, deadline=None)
@given(st.integers(0, 2**31 - 1))
def test_compaction_preserves_every_sequence(seed):
    rs = np.random.RandomState(seed)
    nb_org, chunk, n_chunks = 12, 4, 3
    bm = O.BlockManagerOracle(nb_org, 8, 8, 16)
    O.expand(bm, chunk); O.expand(bm, chunk); O.expand(bm, chunk)
    kp = [rs.randint(0, 1000, size=(nb_org, 1, 1, 2, 2)).astype(np.float32)] + \
         [rs.randint(0, 1000, size=(chunk, 1, 1, 2, 2)).astype(np.float32) for _ in range(n_chunks)]
    vp = [p + 0.5 for p in kp]
    for s in range(6):
        n = int(rs.randint(0, 60))
        if (n + 15) // 16 <= bm.num_free_blocks:
            bm.allocate_blocks_for_seqs([s], [n])
    bm.free_blocks_for_seqs(list(rs.permutation(6)[: rs.randint(0, 4)]))

    def content(seq):
        c = int(bm.num_seq_allocated_blocks[seq])
        out = []
        for b in bm.block_table[seq, :c]:
            seg, row = O.locate_block(b, nb_org, chunk)
            out.append((kp[seg][row].copy(), vp[seg][row].copy()))
        return out

    before = [content(s) for s in range(8)]
    nfree = bm.num_free_blocks
    target = nb_org + int(rs.randint(0, n_chunks + 1)) * chunk
    moved = O.compact(bm, kp, vp, target, chunk)
    if moved < 0:
        return
    assert bm.num_free_blocks == nfree and int(bm.is_block_free.sum()) == nfree
    assert bm.is_block_free[target:].all()                                 # everything above the target is free now
    after = [content(s) for s in range(8)]
    for a, b in zip(before, after):
        assert len(a) == len(b)
        for (ka, va), (kb, vb) in zip(a, b):
            assert np.array_equal(ka, kb) and np.array_equal(va, vb)
    live = np.concatenate([bm.block_table[s, : bm.num_seq_allocated_blocks[s]] for s in range(8)])
    assert len(set(live.tolist())) == len(live) and not bm.is_block_free[live].any()


@settings(max_examples=200, deadline=None)
@given(st.lists(st.tuples(st.integers(0, 40), st.integers(0, 40)), min_size=0, max_size=30))
def test_swap_runs_cover_every_pair_once(pairs):
    src = [p[0] for p in pairs]
    dst = [p[1] for p in pairs]
    runs = O.coalesce_runs(src, dst, num_blocks_org=16, chunk_blocks=8)
    assert sum(n for _, n in runs) == len(pairs)
    pos = 0
    for start, n in runs:
        assert start == pos
        for k in range(1, n):
            assert src[start + k] == src[start] + k and dst[start + k] == dst[start] + k
        pos += n


@settings(max_examples=200, deadline=None)
@given(st.integers(1, 1 << 40), st.integers(1, 1 << 30), st.integers(0, 1 << 30), st.integers(1, 48),
       st.sampled_from([1, 2, 4, 8, 32]))
def test_chunk_layout_fits_the_slab(start, size, quant, layers, hkv):
    try:
        k, v, n = O.chunk_layout(start, size, quant, layers, hkv, 16, 128)
    except RuntimeError:
        return
    per = layers * hkv * 16 * 128 * 2
    assert k % 256 == 0 and k >= start + quant and v == k + n * per
    assert v + n * per <= start + size                                      # K and V both inside the slab


@settings(max_examples=100, deadline=None)
@given(st.integers(0, 2**31 - 1))
def test_first_fit_allocation_is_ascending_and_lowest(seed):
    rs = np.random.RandomState(seed)
    bm = O.BlockManagerOracle(64, 10, 8, 16)
    for _ in range(20):
        s = int(rs.randint(0, 10))
        if rs.rand() < 0.3:
            bm.free_blocks_for_seqs([s])
            continue
        have = int(bm.num_seq_allocated_blocks[s])
        want = min(8, have + int(rs.randint(0, 3)))
        if want - have > bm.num_free_blocks:
            continue
        free_before = np.nonzero(bm.is_block_free)[0]
        new = bm.allocate_blocks_for_seqs([s], [want * 16])
        assert np.array_equal(new, free_before[: want - have])
        assert np.array_equal(bm.block_table[s, have:want], new.astype(np.int32))
    assert int(bm.is_block_free.sum()) == bm.num_free_blocks


def test_infer_state_fields_known_answer():
    """worker/model.py:318-436 on a hand-made step: prompts of 3 and 2 tokens, one decoding sequence at length 5."""
    f = O.infer_state_fields([3, 2], [5], num_kv_heads=8, head_dim=128)
    assert (f["batch_size"], f["num_tokens"], f["num_prefill_seqs"], f["num_prefill_tokens"]) == (3, 6, 2, 5)
    assert f["prefill_seq_start_locs"].tolist() == [0, 3]
    assert f["prefill_seq_start_locs_with_end"].tolist() == [0, 3, 6]
    assert f["position_indices"].tolist() == [0, 1, 2, 0, 1, 4]
    assert f["seq_lengths"].tolist() == [3, 2, 5] and f["max_prefill_len"] == 3 and f["max_decoding_len"] == 5
    assert (f["seq_block_size"], f["num_seq_blocks"]) == (64, 1) and f["softmax_scale"] == 128 ** -0.5
    g = O.infer_state_fields([], [700, 20], num_kv_heads=8, head_dim=128)
    assert g["prefill_seq_start_locs_with_end"].tolist() == [2] and g["position_indices"].tolist() == [699, 19]
    assert g["num_prefill_tokens"] == 0 and g["max_prefill_len"] == 0
