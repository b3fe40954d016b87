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
    """The 38-operation trace recorded from the reference class: every allocate and every free goes through the
    sync-free kernels; tables, counts, bitmap, free count and the new ids (left in the scratch list) must match."""
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
            assert bm.free_blocks_for_seqs_nosync(H.to_dev(ids)) is None
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


def test_block_manager_large_batches_against_oracle():
    """allocate / free / gather with thousands of sequences per call (several passes of the one-block kernels'
    scan loops) in lockstep with the oracle: tables, counts, bitmap, returned ids."""
    from morphserve_b200 import BlockManager
    rs = np.random.RandomState(8)
    nb, max_seqs, cols, bs = 130000, 5000, 24, 16
    bm = BlockManager("GPU", nb, max_seqs, cols, bs)
    ob = O.BlockManagerOracle(nb, max_seqs, cols, bs)
    lens = np.zeros(max_seqs, dtype=np.int64)
    for step in range(6):
        ids = rs.permutation(max_seqs)[: rs.randint(1500, 4000)].astype(np.int32)
        new = np.minimum(lens[ids] + rs.randint(0, 120, size=len(ids)), cols * bs).astype(np.int32)
        lens[ids] = new
        got = bm.allocate_blocks_for_seqs(H.to_dev(ids), H.to_dev(new))
        exp = ob.allocate_blocks_for_seqs(ids, new)
        np.testing.assert_array_equal(got.cpu().numpy(), exp)
        drop = rs.permutation(max_seqs)[: rs.randint(1100, 2500)].astype(np.int32)
        if step % 2 == 0:
            bm.free_blocks_for_seqs(H.to_dev(drop))
            ob.free_blocks_for_seqs(drop)
        else:
            g = bm.gather_allocated_blocks_and_free(H.to_dev(drop))
            np.testing.assert_array_equal(g.cpu().numpy(), ob.gather_allocated_blocks_and_free(drop))
        lens[drop] = 0
        np.testing.assert_array_equal(bm.num_seq_allocated_blocks.cpu().numpy(), ob.num_seq_allocated_blocks)
        np.testing.assert_array_equal(bm.is_block_free.cpu().numpy(), ob.is_block_free)
        assert int(bm.num_free_blocks) == int(ob.num_free_blocks)
        live = ob.num_seq_allocated_blocks > 0          # rows of freed sequences keep stale ids on both sides
        np.testing.assert_array_equal(bm.block_table.cpu().numpy()[live], ob.block_table[live])


def test_prefill_scatter_mid_size_against_torch_indexing():
    """48 prompts of up to 1500 tokens plus decode rows, elastic pool of three segments: the scatter kernels against
    the same assignment written with torch advanced indexing (bit-exact)."""
    from morphserve_b200 import store_kvcache
    from morphserve_b200.worker.infer_state import LlamaInferState
    rs = np.random.RandomState(21)
    Hkv, D, L, layer, bs = 4, 128, 3, 2, 16
    plens = rs.randint(1, 1500, size=48)
    dlens = rs.randint(1, 900, size=30)
    all_lens = np.concatenate([plens, dlens])
    need = (all_lens + bs - 1) // bs
    total = int(need.sum()) + 11
    nb_org, chunk = total // 2, (total - total // 2 + 1) // 2
    perm = rs.permutation(nb_org + 2 * chunk)
    nseq = len(all_lens)
    seq_ids = rs.permutation(nseq + 5)[:nseq].astype(np.int32)
    table = np.full((nseq + 5, int(need.max()) + 1), -1, dtype=np.int32)
    pos = 0
    for i in range(nseq):
        table[seq_ids[i], : need[i]] = perm[pos:pos + need[i]]
        pos += need[i]
    ntok = int(plens.sum()) + len(dlens)
    g = torch.Generator(device="cuda").manual_seed(3)
    k = torch.randn((ntok, Hkv, D), generator=g, dtype=torch.float16, device="cuda")
    v = torch.randn((ntok, Hkv, D), generator=g, dtype=torch.float16, device="cuda")
    shapes = [(nb_org, L, Hkv, bs, D), (chunk, L, Hkv, bs, D), (chunk, L, Hkv, bs, D)]
    kp = [torch.randn(sh, generator=g, dtype=torch.float16, device="cuda") for sh in shapes]
    vp = [torch.randn(sh, generator=g, dtype=torch.float16, device="cuda") for sh in shapes]
    ref_k, ref_v = [t.clone() for t in kp], [t.clone() for t in vp]
    # reference: token -> (segment, row, slot) with numpy integer arithmetic, assignment with torch indexing
    tok_seq = np.concatenate([np.repeat(np.arange(len(plens)), plens), len(plens) + np.arange(len(dlens))])
    tok_pos = np.concatenate([np.concatenate([np.arange(n) for n in plens]), dlens - 1])
    blk = table[seq_ids[tok_seq], tok_pos // bs].astype(np.int64)
    seg = np.where(blk < nb_org, 0, 1 + (blk - nb_org) // chunk)
    row = np.where(blk < nb_org, blk, (blk - nb_org) % chunk)
    for s_i in range(3):
        m = np.nonzero(seg == s_i)[0]
        mi, ri, si = H.to_dev(m).long(), H.to_dev(row[m]).long(), H.to_dev(tok_pos[m] % bs).long()
        ref_k[s_i][ri, layer, :, si, :] = k[mi]
        ref_v[s_i][ri, layer, :, si, :] = v[mi]
    z = torch.zeros(0, dtype=torch.int32, device="cuda")
    st = LlamaInferState(
        batch_size=nseq, num_tokens=ntok, seq_ids=H.to_dev(seq_ids), softmax_scale=1.0, num_prefill_seqs=len(plens),
        num_prefill_tokens=int(plens.sum()), prefill_seq_start_locs=H.to_dev((np.cumsum(plens) - plens).astype(np.int32)),
        prefill_seq_start_locs_with_end=z, prefill_seq_lens=H.to_dev(plens.astype(np.int32)),
        max_prefill_len=int(plens.max()), num_decoding_seqs=len(dlens), decoding_seq_lens=H.to_dev(dlens.astype(np.int32)),
        max_decoding_len=int(dlens.max()), seq_block_size=512, num_seq_blocks=2, num_blocks_org=nb_org,
        kv_cache_new_block_size=chunk, org_layer_param_size=0, position_cos=z, position_sin=z, ignore_kvcache=False)
    mc, ec = H.cfgs(dict(L=L, Hkv=Hkv, D=D, bs=bs), table.shape[1])
    store_kvcache(k, v, kp[0], vp[0], kp[1:], vp[1:], H.to_dev(table), mc, ec, st, layer)
    torch.cuda.synchronize()
    for a, b in zip(kp + vp, ref_k + ref_v):
        assert torch.equal(a, b)


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


def test_host_buffer_step_captured_with_its_copies_equals_eager_steps():
    """The step with host-side inputs and outputs (pinned q/k/v in, attention output back) as one graph with copy
    nodes on forked branches: outputs on the host, pool bytes and tables equal the same steps issued call by call."""
    import morphserve_b200 as mk
    steps = 6
    mk.set_fused_decode_append(True)
    mk.set_fused_decode_rope(True)
    try:
        eager = _make_job()
        eager.make_host_buffers()
        for _ in range(steps):
            eager.step_host()
        job = _make_job()
        job.make_host_buffers()
        job.capture_step_host(max_steps=steps + 2)
        for _ in range(steps):
            job.step_host_graph()
        torch.cuda.synchronize()
    finally:
        mk.set_fused_decode_append(False)
        mk.set_fused_decode_rope(False)
    assert torch.equal(job.ho, eager.ho) and bool(job.ho.abs().sum() > 0)
    assert torch.equal(job.bm.block_table, eager.bm.block_table)
    assert int(job.bm.num_free_blocks) == int(eager.bm.num_free_blocks)
    assert torch.equal(job.k_cache, eager.k_cache) and torch.equal(job.v_cache, eager.v_cache)


def test_counter_snapshot_taken_before_a_nosync_call_is_not_trusted():
    """readback_counters_async() -> another sync-free allocate / free -> num_free_blocks: the snapshot was taken
    before the later call, so the read must fetch a fresh one (a stale count would let a later allocate pass its
    capacity check and hand out ids the bitmap does not have)."""
    from morphserve_b200 import BlockManager
    bm = BlockManager("GPU", 10, 4, 6, 16)
    a = H.to_dev(np.array([0], dtype=np.int32))
    b = H.to_dev(np.array([1], dtype=np.int32))
    bm.allocate_blocks_for_seqs_nosync(a, H.to_dev(np.array([48], dtype=np.int32)))      # 3 blocks
    bm.readback_counters_async()
    bm.allocate_blocks_for_seqs_nosync(b, H.to_dev(np.array([64], dtype=np.int32)))      # 4 more, after the snapshot
    torch.cuda.synchronize()
    assert int(bm.num_free_blocks) == 3
    bm.readback_counters_async()
    bm.free_blocks_for_seqs_nosync(a)
    torch.cuda.synchronize()
    assert int(bm.num_free_blocks) == 6
    assert int(bm.is_block_free.sum()) == 6
    # a request for more than the bitmap holds is refused by the synchronous form too, tables untouched
    table = bm.block_table.clone()
    with pytest.raises(RuntimeError):
        bm.allocate_blocks_for_seqs(H.to_dev(np.array([2, 3], dtype=np.int32)),
                                    H.to_dev(np.array([64, 64], dtype=np.int32)))
    assert torch.equal(bm.block_table, table) and int(bm.num_free_blocks) == 6
    # several conditions recorded since the last look are all reported
    bm.allocate_blocks_for_seqs_nosync(b, H.to_dev(np.array([1], dtype=np.int32)))       # shrinking target
    bm.allocate_blocks_for_seqs_nosync(a, H.to_dev(np.array([16 * 8], dtype=np.int32)))  # 8 blocks > 6-column row
    with pytest.raises(RuntimeError) as e:
        bm.sync_counters()
    assert "row" in str(e.value) and "Logic error" in str(e.value)


def test_replacing_the_bitmap_bumps_the_resize_generation():
    """Elastic expand and release assign a new tensor to ``is_block_free`` (server/memory_utils.py:416-417, :650);
    whatever captured the old address (a CUDA graph of the step) checks ``resize_generation``."""
    import types
    from morphserve_b200 import BlockManager, memory_utils
    bm = BlockManager("GPU", 32, 4, 8, 16)
    g0 = bm.resize_generation
    model = types.SimpleNamespace(k_cache_new=[], v_cache_new=[], kv_cache_new_block_size=0, gpu_block_manager=bm)
    eng = types.SimpleNamespace(model=model, scheduler=None)
    chunk = torch.zeros((8, 1, 1, 16, 128), dtype=torch.float16, device="cuda")
    memory_utils.attach_kvcache_chunk(eng, chunk, chunk.clone())
    assert bm.resize_generation == g0 + 1 and bm.is_block_free.shape[0] == 40 and int(bm.num_free_blocks) == 40
    assert memory_utils.release_last_kvcache_chunk(eng)
    assert bm.resize_generation == g0 + 2 and bm.is_block_free.shape[0] == 32


def test_gather_and_free_without_host_round_trip():
    """The sync-free gather against the synchronous one on a twin manager: same ids in batch order, -1 behind them,
    the count on the device, tables / bitmap / free count equal once the counters are read."""
    from morphserve_b200 import BlockManager
    rs = np.random.RandomState(4)
    a, b = BlockManager("GPU", 500, 40, 16, 16), BlockManager("GPU", 500, 40, 16, 16)
    ids = H.to_dev(np.arange(30, dtype=np.int32))
    lens = H.to_dev(rs.randint(0, 200, size=30).astype(np.int32))
    for bm in (a, b):
        bm.allocate_blocks_for_seqs(ids, lens)
    pick = H.to_dev(np.array([7, 0, 29, 12, 3], dtype=np.int32))
    want = a.gather_allocated_blocks_and_free(pick)
    got, count = b.gather_allocated_blocks_and_free_nosync(pick)
    n = int(count.item())
    assert n == want.shape[0] and got.shape[0] == min(5 * 16, 500)
    assert torch.equal(got[:n], want.to(torch.int32)) and bool((got[n:] == -1).all())
    assert int(b.num_free_blocks) == int(a.num_free_blocks)
    assert torch.equal(a.is_block_free, b.is_block_free)
    assert torch.equal(a.num_seq_allocated_blocks, b.num_seq_allocated_blocks)
    # a buffer that is too small: everything is freed, the first `capacity` ids are reported, the count says so
    pick2 = H.to_dev(np.array([1, 2, 4], dtype=np.int32))
    want2 = a.gather_allocated_blocks_and_free(pick2)
    got2, count2 = b.gather_allocated_blocks_and_free_nosync(pick2, capacity=3)
    assert int(count2.item()) == want2.shape[0] > 3 and torch.equal(got2, want2[:3].to(torch.int32))
    assert int(b.num_free_blocks) == int(a.num_free_blocks) and torch.equal(a.is_block_free, b.is_block_free)


def test_mixed_prefill_and_decode_step_captured_in_a_cuda_graph():
    """A step that admits prompts next to the decoding sequences - sync-free allocate for all of them, then per layer
    one store_kvcache call (prompt scatter + decode append) and decode attention - captured once and replayed with
    new contents in the same buffers; pools, tables and outputs equal the same calls issued one by one."""
    import types
    import morphserve_b200 as mk
    dev = torch.device("cuda", 0)
    L, Hq, Hkv, D, bs = 2, 8, 2, 128, 16
    n_pre, n_dec, mbps, nb = 3, 5, 24, 200
    plens = [40, 16, 7]
    mc = types.SimpleNamespace(num_layers=L, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D)
    ec = types.SimpleNamespace(block_size=bs, max_blocks_per_seq=mbps)
    n_tok = sum(plens) + n_dec

    def run(captured: bool):
        g = torch.Generator(device=dev).manual_seed(21)
        bm = mk.BlockManager("GPU", nb, 16, mbps, bs)
        dec_ids = torch.arange(n_pre, n_pre + n_dec, dtype=torch.int32, device=dev)
        dec_lens = torch.tensor([100, 33, 16, 250, 64], dtype=torch.int32, device=dev)
        bm.allocate_blocks_for_seqs(dec_ids, dec_lens)
        kc = torch.randn((nb, L, Hkv, bs, D), generator=g, dtype=torch.float16, device=dev)
        vc = torch.randn((nb, L, Hkv, bs, D), generator=g, dtype=torch.float16, device=dev)
        seq_ids = torch.arange(n_pre + n_dec, dtype=torch.int32, device=dev)
        # fixed-address buffers the graph reads: lengths of all sequences, k / v / q of the step
        lens_all = torch.cat([torch.tensor(plens, dtype=torch.int32, device=dev), dec_lens + 1])
        k = torch.empty((L, n_tok, Hkv, D), dtype=torch.float16, device=dev)
        v = torch.empty_like(k)
        q = torch.empty((L, n_dec, Hq, D), dtype=torch.float16, device=dev)
        o = torch.zeros((L, n_dec, Hq * D), dtype=torch.float16, device=dev)
        starts = torch.tensor(np.cumsum([0] + plens[:-1]), dtype=torch.int32, device=dev)
        z = torch.zeros(0, dtype=torch.int32, device=dev)
        st = mk.LlamaInferState(
            batch_size=n_pre + n_dec, num_tokens=n_tok, seq_ids=seq_ids, softmax_scale=D ** -0.5, num_prefill_seqs=n_pre,
            num_prefill_tokens=sum(plens), prefill_seq_start_locs=starts, prefill_seq_start_locs_with_end=z,
            prefill_seq_lens=lens_all[:n_pre], max_prefill_len=max(plens), num_decoding_seqs=n_dec,
            decoding_seq_lens=lens_all[n_pre:], max_decoding_len=300, seq_block_size=512, num_seq_blocks=1,
            num_blocks_org=nb, kv_cache_new_block_size=0, org_layer_param_size=0, position_cos=z, position_sin=z,
            ignore_kvcache=False)

        def step():
            bm.allocate_blocks_for_seqs_nosync(seq_ids, lens_all)
            for layer in range(L):
                mk.store_kvcache(k[layer], v[layer], kc, vc, [], [], bm.block_table, mc, ec, st, layer)
                mk.paged_attention(q[layer], kc, vc, [], [], bm.block_table, mc, ec, st, layer, o[layer])

        def fill():
            for t in (k, v, q):
                t.normal_(generator=g)

        fill()
        if captured:
            from morphserve_b200.worker.kernels._common import attn_workspace
            bm.prepare_nosync(n_pre + n_dec)
            cs = torch.cuda.Stream(dev)
            attn_workspace(0, n_dec, Hq, Hkv, D, mbps, cs.cuda_stream)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=cs):
                step()
            graph.replay()
            bm.nosync_replayed()
        else:
            step()
        torch.cuda.synchronize()
        return kc, vc, o.clone(), bm

    a, b = run(False), run(True)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    assert bool(a[2].abs().sum() > 0)
    assert torch.equal(a[3].block_table, b[3].block_table) and torch.equal(a[3].is_block_free, b[3].is_block_free)
    assert int(a[3].num_free_blocks) == int(b[3].num_free_blocks)
