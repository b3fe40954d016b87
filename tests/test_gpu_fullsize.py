"""Full-size runs of the benchmark configurations on the GPU, checked through
properties that do not need a CPU copy of a 27-32 GB pool:

* appended K/V rows are read back bit-exact from the position the block table
  names (all sequences, sampled layers);
* attention is compared with the oracle on a sample of sequences whose blocks
  are gathered to the host;
* block tables, counts and the free bitmap are compared EXACTLY with the integer
  oracle driven in lockstep;
* compaction is checked with per-block checksums: every moved block's checksum
  arrives at its destination, every other block keeps its own.
"""
import types

import numpy as np
import pytest
import torch

import bench
from oracle import kv_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu
D, BS = 128, 16


def _gather_seq(pools_k, pools_v, table_row, nblk, layer, nb_org, chunk):
    ks, vs = [], []
    for j in range(nblk):
        seg, row = O.locate_block(int(table_row[j]), nb_org, max(chunk, 1))
        ks.append(pools_k[seg][row, layer].cpu().numpy())
        vs.append(pools_v[seg][row, layer].cpu().numpy())
    return np.concatenate(ks, axis=1), np.concatenate(vs, axis=1)      # [Hkv, nblk*16, D]


def _oracle_attention(q, kk, vv, n, scale):
    Hq, Hkv = q.shape[0], kk.shape[0]
    G = Hq // Hkv
    k = np.repeat(kk[:, :n].astype(np.float64), G, axis=0)
    v = np.repeat(vv[:, :n].astype(np.float64), G, axis=0)
    s = np.einsum("hd,hnd->hn", q.astype(np.float64), k) * scale
    s -= s.max(axis=1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=1, keepdims=True)
    return np.einsum("hn,hnd->hd", p, v)


def _check_append_rows(pools_k, pools_v, table, rows, lens, k_new, v_new, layer, nb_org, chunk):
    """pool[block_table[row, (len-1)//16], layer, :, (len-1)%16, :] == new row, for every sequence."""
    pos = lens.long() - 1
    blk = table[rows.long(), pos // BS].long()
    slot = pos % BS
    if len(pools_k) == 1:
        got_k = pools_k[0][blk, layer, :, slot, :]
        got_v = pools_v[0][blk, layer, :, slot, :]
    else:
        got_k, got_v = torch.empty_like(k_new), torch.empty_like(v_new)
        seg = torch.where(blk < nb_org, torch.zeros_like(blk), 1 + (blk - nb_org) // chunk)
        row = torch.where(blk < nb_org, blk, (blk - nb_org) % chunk)
        for s in seg.unique().tolist():
            m = seg == s
            got_k[m] = pools_k[s][row[m], layer, :, slot[m], :]
            got_v[m] = pools_v[s][row[m], layer, :, slot[m], :]
    assert torch.equal(got_k, k_new), "appended K rows differ"
    assert torch.equal(got_v, v_new), "appended V rows differ"


@pytest.mark.parametrize("name,balance,deal", [("llama3-8b-gqa-decode", None, 1), ("llama2-7b-mha-decode", None, 1),
                                               ("llama3-8b-gqa-decode", 0.0, 0), ("llama3-8b-gqa-decode", 0.0, 1),
                                               ("llama2-7b-mha-decode", None, 2)])
def test_baseline_decode_config_full_size(name, balance, deal):
    """`balance` 0.0 makes the plan cut sequences as finely as its item cap allows, so that the split-KV merge
    runs at full size too (with the default rule these batches are balanced without a cut): once with the chunks
    drawn from the shared counter (`deal` 0) and once with equal ranges per worker (1).  `deal` 2 forces the equal
    ranges on a batch that would not be cut."""
    from morphserve_b200._lib import lib, check
    w = bench.shard_workload(bench.WORKLOADS[name], 0, 1)
    job = bench.DecodeJob(w, 0, growth_tokens=32, device=torch.device("cuda", 0))
    if balance is not None:
        check(lib.mkv_attn_configure(-1, -1, -1.0, balance, -1), "mkv_attn_configure")
    check(lib.mkv_attn_set_static_deal(deal, -1, 1), "mkv_attn_set_static_deal")
    try:
        for _ in range(2):
            job.step_resident()
        torch.cuda.synchronize()
    finally:
        check(lib.mkv_attn_configure(-1, -1, -1.0, 1.5, -1), "mkv_attn_configure")
        check(lib.mkv_attn_set_static_deal(1, -1, 1), "mkv_attn_set_static_deal")
    bm = job.bm
    lens = job.lens_dev
    # integers: every sequence owns exactly ceil(len/16) blocks, all distinct, bitmap consistent
    need = (lens + BS - 1) // BS
    assert torch.equal(bm.num_seq_allocated_blocks[: w["B"]], need)
    owned = torch.cat([bm.block_table[b, : int(need[b])] for b in range(w["B"])]).long()
    assert owned.unique().numel() == owned.numel()
    assert not bm.is_block_free[owned].any()
    assert int(bm.is_block_free.sum()) == int(bm.num_free_blocks) == job.nb - owned.numel()
    # append: bit-exact for all sequences on three layers
    for layer in (0, w["L"] // 2, w["L"] - 1):
        _check_append_rows([job.k_cache], [job.v_cache], bm.block_table, job.seq_ids, lens, job.kn[layer],
                           job.vn[layer], layer, job.nb, 0)
    # attention: longest, shortest and four seeded sequences, two layers, against the oracle
    order = torch.argsort(lens).tolist()
    sample = [order[0], order[-1]] + np.random.RandomState(0).choice(w["B"], 4, replace=False).tolist()
    table = bm.block_table.cpu().numpy()
    for layer in (1, w["L"] - 1):
        o = job.o[layer].view(w["B"], w["Hq"], D)
        for b in sample:
            n = int(lens[b])
            kk, vv = _gather_seq([job.k_cache], [job.v_cache], table[b], (n + BS - 1) // BS, layer, job.nb, 0)
            ex = _oracle_attention(job.q[layer, b].cpu().numpy(), kk, vv, n, D ** -0.5)
            np.testing.assert_allclose(o[b].cpu().numpy().astype(np.float64), ex, rtol=2e-3, atol=1e-2)
    # attention, EVERY sequence and layer: against the library's plain kernel (one warp per query head, fp32 FMA,
    # no plan, no split, no tensor cores - held to the oracle by the small-shape tests)
    st = job.infer_state(job.seq_ids, job.lens_dev)
    check(lib.mkv_attn_configure(-1, -1, -1.0, -1.0, 2), "mkv_attn_configure")
    try:
        plain = torch.empty_like(job.o)
        for layer in range(w["L"]):
            job.mk.paged_attention(job.q[layer], job.k_cache, job.v_cache, [], [], bm.block_table, job.model_config,
                                   job.engine_config, st, layer, plain[layer])
        torch.cuda.synchronize()
    finally:
        check(lib.mkv_attn_configure(-1, -1, -1.0, -1.0, 0), "mkv_attn_configure")
    diff = (job.o.float() - plain.float()).abs()
    assert bool((diff <= 1e-2 + 2e-3 * plain.float().abs()).all()), f"max difference {float(diff.max())}"
    from morphserve_b200.worker.kernels._common import read_attn_error_flags
    assert read_attn_error_flags(0) == 0


def _block_checksums(pool):
    """int64 sum of the 16-bit words of every block (exact, order independent)."""
    out = torch.empty(pool.shape[0], dtype=torch.int64, device=pool.device)
    flat = pool.view(pool.shape[0], -1).view(torch.int16)
    for i in range(0, pool.shape[0], 256):
        out[i:i + 256] = flat[i:i + 256].to(torch.int64).sum(dim=1)
    return out


def _gather_blocks(pools, ids, nb_org, chunk):
    """Bytes of the given blocks ([n, block bytes] uint8), wherever their segment lies."""
    out = torch.empty((len(ids), pools[0][0].numel() * 2), dtype=torch.uint8, device=pools[0].device)
    for i, b in enumerate(ids):
        seg, row = O.locate_block(int(b), nb_org, max(chunk, 1))
        out[i] = pools[seg][row].reshape(-1).view(torch.uint8)
    return out


def test_elastic_resize_trace_full_size():
    """Elastic trace at full size (Llama-3-8B pool shape): 8192 -> 16384 blocks, release 40 % by compaction,
    100 decode steps of batch 128."""
    from morphserve_b200 import BlockManager, paged_attention, store_kvcache
    from morphserve_b200.server import memory_utils as MU
    L, Hq, Hkv = 32, 32, 8
    nb_org, chunk, n_chunks, release = 8192, 1024, 8, 6
    max_len, batch, mbps, max_seqs = 1536, 128, 128, 4096
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(4000)
    rs = np.random.RandomState(4001)

    def new_pool(n):
        t = torch.empty((n, L, Hkv, BS, D), dtype=torch.float16, device=dev)
        flat = t.view(-1)
        for i in range(0, flat.numel(), 1 << 28):
            flat[i:i + (1 << 28)].normal_(generator=g)
        return t

    model = types.SimpleNamespace(k_cache=new_pool(nb_org), v_cache=new_pool(nb_org), k_cache_new=[], v_cache_new=[],
                                  kv_cache_new_block_size=0,
                                  gpu_block_manager=BlockManager("GPU", nb_org, max_seqs, mbps, BS))
    engine = types.SimpleNamespace(model=model, scheduler=types.SimpleNamespace(num_gpu_blocks=nb_org))
    bm = model.gpu_block_manager
    obm = O.BlockManagerOracle(nb_org, max_seqs, mbps, BS)
    lens_of = {}
    next_id = [0]
    mc = types.SimpleNamespace(num_layers=L, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D)
    ec = types.SimpleNamespace(block_size=BS, max_blocks_per_seq=mbps)
    q = torch.randn((L, batch, Hq, D), generator=g, dtype=torch.float16, device=dev)
    kn = torch.randn((L, batch, Hkv, D), generator=g, dtype=torch.float16, device=dev)
    vn = torch.randn((L, batch, Hkv, D), generator=g, dtype=torch.float16, device=dev)
    o = torch.zeros((L, batch, Hq * D), dtype=torch.float16, device=dev)

    def check_ints():
        np.testing.assert_array_equal(bm.block_table.cpu().numpy(), obm.block_table)
        np.testing.assert_array_equal(bm.num_seq_allocated_blocks.cpu().numpy(), obm.num_seq_allocated_blocks)
        np.testing.assert_array_equal(bm.is_block_free.cpu().numpy(), obm.is_block_free)
        assert (bm.num_blocks, int(bm.num_free_blocks)) == (obm.num_blocks, obm.num_free_blocks)
        assert engine.scheduler.num_gpu_blocks == obm.num_blocks

    def admit_until(frac):
        ids, lens = [], []
        used = obm.get_num_used_blocks()
        while used < frac * obm.num_blocks and next_id[0] < max_seqs:
            n = int(rs.randint(1, max_len - 100))
            used += (n + BS - 1) // BS
            ids.append(next_id[0])
            lens.append(n)
            lens_of[next_id[0]] = n
            next_id[0] += 1
        ids, lens = np.array(ids, dtype=np.int32), np.array(lens, dtype=np.int32)
        new = bm.allocate_blocks_for_seqs(H.to_dev(ids), H.to_dev(lens))
        np.testing.assert_array_equal(new.cpu().numpy(), obm.allocate_blocks_for_seqs(ids, lens))

    def decode_steps(running, n_steps):
        ids = np.array(running, dtype=np.int32)
        ids_t = H.to_dev(ids)
        c = dict(scale=D ** -0.5, num_blocks_org=nb_org, chunk_blocks=model.kv_cache_new_block_size)
        for step in range(n_steps):
            for s in running:
                lens_of[s] += 1
            lens = np.array([lens_of[s] for s in running], dtype=np.int32)
            lens_t = H.to_dev(lens)
            new = bm.allocate_blocks_for_seqs(ids_t, lens_t)
            np.testing.assert_array_equal(new.cpu().numpy(), obm.allocate_blocks_for_seqs(ids, lens))
            st = H.decode_state(c, ids_t, lens_t)
            for layer in range(L):
                store_kvcache(kn[layer], vn[layer], model.k_cache, model.v_cache, model.k_cache_new,
                              model.v_cache_new, bm.block_table, mc, ec, st, layer)
                paged_attention(q[layer], model.k_cache, model.v_cache, model.k_cache_new, model.v_cache_new,
                                bm.block_table, mc, ec, st, layer, o[layer])
        # last step: appended rows exact (two layers), attention on three sequences (one layer)
        pk, pv = [model.k_cache] + model.k_cache_new, [model.v_cache] + model.v_cache_new
        for layer in (0, L - 1):
            _check_append_rows(pk, pv, bm.block_table, ids_t, lens_t, kn[layer], vn[layer], layer, nb_org,
                               model.kv_cache_new_block_size)
        table = bm.block_table.cpu().numpy()
        layer = L // 2
        ov = o[layer].view(batch, Hq, D)
        for i in (0, batch // 2, batch - 1):
            n = int(lens[i])
            kk, vv = _gather_seq(pk, pv, table[ids[i]], (n + BS - 1) // BS, layer, nb_org,
                                 model.kv_cache_new_block_size)
            ex = _oracle_attention(q[layer, i].cpu().numpy(), kk, vv, n, D ** -0.5)
            np.testing.assert_allclose(ov[i].cpu().numpy().astype(np.float64), ex, rtol=2e-3, atol=1e-2)

    admit_until(0.90)
    check_ints()
    running = [int(x) for x in rs.permutation(list(lens_of))[:batch]]
    decode_steps(running, 30)
    check_ints()
    for _ in range(n_chunks):                                   # expand 8192 -> 16384
        MU.attach_kvcache_chunk(engine, new_pool(chunk), new_pool(chunk))
        O.expand(obm, chunk)
    check_ints()
    admit_until(0.85)
    check_ints()
    running = [int(x) for x in rs.permutation(list(lens_of))[:batch]]
    decode_steps(running, 40)
    check_ints()
    order = [int(x) for x in rs.permutation(list(lens_of))]       # free a seeded subset: >= 40 % free
    victims = []
    freed = obm.num_free_blocks
    while freed < 0.4 * obm.num_blocks + 1:
        s = order.pop()
        victims.append(s)
        freed += (lens_of.pop(s) + BS - 1) // BS
    bm.free_blocks_for_seqs(H.to_dev(np.array(victims, dtype=np.int32)))
    obm.free_blocks_for_seqs(np.array(victims, dtype=np.int32))
    check_ints()

    target = nb_org + (n_chunks - release) * chunk               # 10240
    pk, pv = [model.k_cache] + model.k_cache_new, [model.v_cache] + model.v_cache_new
    before_k = torch.cat([_block_checksums(p) for p in pk])
    before_v = torch.cat([_block_checksums(p) for p in pv])
    src, dst = O.compaction_plan(obm.is_block_free, target)
    src_bytes_k = _gather_blocks(pk, src, nb_org, chunk)            # 2 x 3.6 GiB: the blocks about to move, byte for byte
    src_bytes_v = _gather_blocks(pv, src, nb_org, chunk)
    moved = MU.compact_kvcache(engine, target)
    assert moved == len(src) > 0
    remap = dict(zip(src.tolist(), dst.tolist()))
    for row in range(obm.block_table.shape[0]):                  # integer side of the oracle's compact()
        cnt = int(obm.num_seq_allocated_blocks[row])
        for j in range(cnt):
            e = int(obm.block_table[row, j])
            if e in remap:
                obm.block_table[row, j] = remap[e]
    obm.is_block_free[dst] = False
    obm.is_block_free[src] = True
    check_ints()
    after_k = torch.cat([_block_checksums(p) for p in pk])
    after_v = torch.cat([_block_checksums(p) for p in pv])
    src_t, dst_t = H.to_dev(src), H.to_dev(dst)
    for before, after in ((before_k, after_k), (before_v, after_v)):
        assert torch.equal(after[dst_t], before[src_t]), "a moved block did not arrive intact"
        keep = torch.ones_like(before, dtype=torch.bool)
        keep[dst_t] = False
        assert torch.equal(after[keep], before[keep]), "a block that was not a destination changed"
    assert torch.equal(_gather_blocks(pk, dst, nb_org, chunk), src_bytes_k), "moved K blocks differ from their sources"
    assert torch.equal(_gather_blocks(pv, dst, nb_org, chunk), src_bytes_v), "moved V blocks differ from their sources"
    assert torch.equal(_gather_blocks(pk, src, nb_org, chunk), src_bytes_k), "a source block was written"
    del src_bytes_k, src_bytes_v
    for _ in range(release):                                     # 16384 -> 10240 by the reference's rule
        assert MU.release_last_kvcache_chunk(engine)
        O.release_last_chunk(obm, chunk)
    check_ints()
    assert bm.num_blocks == target and len(model.k_cache_new) == n_chunks - release
    running = [s for s in running if s in lens_of][:batch]
    while len(running) < batch:
        running.append(next(s for s in lens_of if s not in running))
    decode_steps(running, 30)
    check_ints()
    from morphserve_b200.worker.kernels._common import read_attn_error_flags
    assert read_attn_error_flags(0) == 0
