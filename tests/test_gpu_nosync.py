"""The sync-free allocate (one launch, no host round trip) against the reference BlockManager's recorded
behaviour, and a decode step captured in a CUDA graph against the same steps launched one by one."""
import os

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from tests import helpers as H
from tests.golden import cases

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def test_nosync_allocate_follows_the_reference_trace():
    """The 38-operation trace recorded from the reference class: every allocate goes through the sync-free
    kernel; tables, counts, bitmap, free count and the new ids (left in the scratch list) must match."""
    from morphserve_b200 import BlockManager
    tr = cases.block_manager_trace()
    gold = np.load(os.path.join(G, "block_manager_trace.npz"))
    bm = BlockManager("GPU", tr["num_blocks"], tr["max_seqs"], tr["max_blocks_per_seq"], tr["block_size"])
    for i, (op, ids, lens) in enumerate(tr["ops"]):
        if op == "alloc":
            assert bm.allocate_blocks_for_seqs_nosync(H.to_dev(ids), H.to_dev(lens)) is None
            n_new = len(gold[f"ret_{i}"])
            np.testing.assert_array_equal(bm._alloc_ids[:n_new].cpu().numpy(), gold[f"ret_{i}"])
        elif op == "free":
            bm.free_blocks_for_seqs(H.to_dev(ids))
        else:
            r = bm.gather_allocated_blocks_and_free(H.to_dev(ids))
            np.testing.assert_array_equal(r.cpu().numpy().astype(np.int64), gold[f"ret_{i}"])
        np.testing.assert_array_equal(bm.block_table.cpu().numpy(), gold[f"table_{i}"])
        np.testing.assert_array_equal(bm.num_seq_allocated_blocks.cpu().numpy(), gold[f"count_{i}"])
        np.testing.assert_array_equal(bm.is_block_free.cpu().numpy(), gold[f"free_{i}"])
        assert int(bm.num_free_blocks) == int(gold[f"nfree_{i}"])


def test_nosync_allocate_errors_arrive_with_the_next_counter_read():
    from morphserve_b200 import BlockManager
    bm = BlockManager("GPU", 8, 4, 6, 16)
    ids = H.to_dev(np.array([0, 1], dtype=np.int32))
    bm.allocate_blocks_for_seqs_nosync(ids, H.to_dev(np.array([40, 17], dtype=np.int32)))    # 3 + 2 blocks
    assert int(bm.num_free_blocks) == 3
    table, count, free = bm.block_table.clone(), bm.num_seq_allocated_blocks.clone(), bm.is_block_free.clone()
    # pool too small (needs 4 more, 3 free): nothing changes, RuntimeError like worker/block_manager.py:69-70
    bm.allocate_blocks_for_seqs_nosync(ids, H.to_dev(np.array([90, 33], dtype=np.int32)))
    with pytest.raises(RuntimeError):
        bm.sync_counters()
    assert torch.equal(bm.block_table, table) and torch.equal(bm.num_seq_allocated_blocks, count)
    assert torch.equal(bm.is_block_free, free) and int(bm.num_free_blocks) == 3
    # shrinking target: the reference's assertion (:95-98)
    bm.allocate_blocks_for_seqs_nosync(ids, H.to_dev(np.array([1, 17], dtype=np.int32)))
    with pytest.raises(AssertionError):
        _ = bm.num_free_blocks
    assert torch.equal(bm.block_table, table) and int(bm.num_free_blocks) == 3
    # a row longer than the table
    bm2 = BlockManager("GPU", 64, 2, 3, 16)
    bm2.allocate_blocks_for_seqs_nosync(H.to_dev(np.array([1], dtype=np.int32)), H.to_dev(np.array([70], dtype=np.int32)))
    with pytest.raises(RuntimeError):
        bm2.sync_counters()
    assert int(bm2.num_free_blocks) == 64 and bool(bm2.is_block_free.all())
    # and it keeps working afterwards; the regular allocate sees a consistent state
    bm.allocate_blocks_for_seqs_nosync(ids, H.to_dev(np.array([48, 32], dtype=np.int32)))
    got = bm.allocate_blocks_for_seqs(H.to_dev(np.array([2], dtype=np.int32)), H.to_dev(np.array([16], dtype=np.int32)))
    assert int(bm.num_free_blocks) == 2 and got.tolist() == [5]


def test_nosync_allocate_large_batch_against_oracle():
    """More sequences than threads, prompts of many blocks, a fragmented bitmap."""
    from morphserve_b200 import BlockManager
    rs = np.random.RandomState(3)
    nb, max_seqs, cols, bs = 60000, 3000, 40, 16
    bm = BlockManager("GPU", nb, max_seqs, cols, bs)
    ob = O.BlockManagerOracle(nb, max_seqs, cols, bs)
    free = rs.rand(nb) < 0.6
    bm.is_block_free.copy_(H.to_dev(free))
    bm.num_free_blocks = int(free.sum())
    ob.is_block_free[:] = free
    ob.num_free_blocks = int(free.sum())
    seq_ids = rs.permutation(max_seqs)[:2500].astype(np.int32)
    lens = rs.randint(1, 200, size=2500).astype(np.int32)
    for step in range(3):
        bm.allocate_blocks_for_seqs_nosync(H.to_dev(seq_ids), H.to_dev(lens))
        ob.allocate_blocks_for_seqs(seq_ids, lens)
        np.testing.assert_array_equal(bm.block_table.cpu().numpy(), ob.block_table)
        np.testing.assert_array_equal(bm.num_seq_allocated_blocks.cpu().numpy(), ob.num_seq_allocated_blocks)
        np.testing.assert_array_equal(bm.is_block_free.cpu().numpy(), ob.is_block_free)
        assert int(bm.num_free_blocks) == int(ob.num_free_blocks)
        lens = (lens + rs.randint(0, 40, size=2500)).astype(np.int32)


def _make_job(L=2, B=24):
    import bench
    w = dict(cfg=77, B=B, Hq=32, Hkv=8, L=L, max_len=700, free_frac=0.2, rope=True)
    w = bench.shard_workload(w, 0, 1)
    return bench.DecodeJob(w, 0, growth_tokens=64, device=torch.device("cuda", 0))


def test_decode_step_captured_in_a_cuda_graph_equals_eager_steps():
    """allocate (sync-free) + plan + L x (rotary + append + attention), all fused forms, captured once and
    replayed: pool bytes, tables, counters and outputs equal the same steps launched one by one."""
    import morphserve_b200 as mk
    steps = 20
    mk.set_fused_decode_append(True)
    mk.set_fused_decode_rope(True)
    try:
        eager = _make_job()
        for _ in range(steps):
            eager.step_resident()
        torch.cuda.synchronize()

        job = _make_job()
        job.capture_step(max_steps=steps + 2)
        for _ in range(steps):
            job.step_graph()
        torch.cuda.synchronize()
    finally:
        mk.set_fused_decode_append(False)
        mk.set_fused_decode_rope(False)
    assert torch.equal(job.lens_dev, eager.lens_dev)
    assert torch.equal(job.bm.block_table, eager.bm.block_table)
    assert torch.equal(job.bm.num_seq_allocated_blocks, eager.bm.num_seq_allocated_blocks)
    assert torch.equal(job.bm.is_block_free, eager.bm.is_block_free)
    assert int(job.bm.num_free_blocks) == int(eager.bm.num_free_blocks)
    assert torch.equal(job.k_cache, eager.k_cache) and torch.equal(job.v_cache, eager.v_cache)
    assert torch.equal(job.o, eager.o)
    from morphserve_b200.worker.kernels._common import read_attn_error_flags
    assert read_attn_error_flags(0) == 0
