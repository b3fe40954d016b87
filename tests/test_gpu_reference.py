"""The CUDA path against the REFERENCE'S OWN KERNELS on the same device tensors.

The staged reference (``oracle/_ref``, made by ``oracle/build_ref.py``) is
imported unmodified; Triton compiles its kernels for the local GPU.  Both
implementations then run on the same seeded inputs at the full benchmark sizes:

* ``store_kvcache`` (worker/kernels/kvcache_mgmt.py:298-478): the touched layer
  slice of every pool segment must be BIT-EQUAL, and an untouched layer keeps
  its checksum;
* ``paged_attention`` (worker/kernels/paged_attn.py:700-1015): every sequence
  and every head within rtol 2e-3 / atol 1e-2;
* ``BlockManager`` (worker/block_manager.py): tables, counts, bitmap and the
  returned ids equal after every operation of a seeded trace;
* ``rotary_embedding_inplace`` (worker/kernels/rotary_emb.py:43-58): bit-equal to the COMPILED kernel under the
  library's default rounding.  (Run in the Triton interpreter the same source rounds every operation on its own; the
  committed fixtures hold that, and the library reproduces it under ``set_rope_rounding("written")``.)

The tests skip (with the reason) when ``oracle/_ref`` has not been staged.
"""
import types

import numpy as np
import pytest
import torch

import bench
from oracle import ref_loader
from tests import helpers as H

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_loader.available(), reason=ref_loader.why_unavailable())]
D, BS = 128, 16
RTOL, ATOL = 2e-3, 1e-2


@pytest.fixture(scope="module")
def ref():
    return ref_loader.load()


def _ref_state(ref, st):
    """The same per-step metadata as an instance of the reference's own dataclass."""
    import dataclasses
    return ref.LlamaInferState(**{f.name: getattr(st, f.name) for f in dataclasses.fields(ref.LlamaInferState)})


def _layer_slices(pools, layer):
    return [p[:, layer].clone() for p in pools]


def _restore(pools, layer, saved):
    for p, s in zip(pools, saved):
        p[:, layer].copy_(s)


def _checksum(pools, layer):
    return [int(p[:, layer].contiguous().view(torch.int16).to(torch.int64).sum()) for p in pools]


def _assert_close(o, o_ref, what):
    a, b = o.float(), o_ref.float()
    bad = (a - b).abs() > ATOL + RTOL * b.abs()
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())} of {bad.numel()} outputs outside rtol {RTOL} / atol {ATOL}; "
                                 f"max abs difference {float((a - b).abs().max()):.3e}")


def _compare_layer(ref, mk, layer, other_layer, q, kn, vn, pools_k, pools_v, table, mc, ec, st, modes=("separate", "fused")):
    """One layer of a decode step through both implementations, starting from the same pool bytes."""
    B = q.shape[0]
    st_ref = _ref_state(ref, st)
    kc, vc, kl, vl = pools_k[0], pools_v[0], pools_k[1:], pools_v[1:]
    saved = _layer_slices(pools_k + pools_v, layer)
    before_other = _checksum(pools_k + pools_v, other_layer)
    ref.store_kvcache(kn, vn, kc, vc, kl, vl, table, mc, ec, st_ref, layer)
    o_ref = torch.zeros((B, mc.num_q_heads * D), dtype=torch.float16, device=q.device)
    ref.paged_attention(q, kc, vc, kl, vl, table, mc, ec, st_ref, layer, o_ref)
    torch.cuda.synchronize()
    after_ref = _layer_slices(pools_k + pools_v, layer)
    assert _checksum(pools_k + pools_v, other_layer) == before_other
    for mode in modes:
        _restore(pools_k + pools_v, layer, saved)
        mk.set_fused_decode_append(mode == "fused")
        try:
            mk.store_kvcache(kn, vn, kc, vc, kl, vl, table, mc, ec, st, layer)
            o = torch.zeros_like(o_ref)
            mk.paged_attention(q, kc, vc, kl, vl, table, mc, ec, st, layer, o)
            torch.cuda.synchronize()
        finally:
            mk.set_fused_decode_append(False)
        for i, (a, b) in enumerate(zip(_layer_slices(pools_k + pools_v, layer), after_ref)):
            assert torch.equal(a, b), f"layer {layer}, {mode} append: pool segment {i} differs from the reference's"
        assert _checksum(pools_k + pools_v, other_layer) == before_other, "an untouched layer changed"
        _assert_close(o, o_ref, f"layer {layer}, {mode} append")


@pytest.mark.parametrize("name", ["llama3-8b-gqa-decode", "llama2-7b-mha-decode"])
def test_decode_config_full_size_against_reference_kernels(ref, name):
    """BASELINE configs[2] and configs[1] at full size: every sequence, every head, four layers."""
    w = bench.shard_workload(bench.WORKLOADS[name], 0, 1)
    job = bench.DecodeJob(w, 0, growth_tokens=32, device=torch.device("cuda", 0))
    job.lens_host += 1
    job.lens_dev += 1
    job.bm.allocate_blocks_for_seqs(job.seq_ids, job.lens_dev)
    st = job.infer_state(job.seq_ids, job.lens_dev)
    for layer in (0, 1, w["L"] // 2, w["L"] - 1):
        _compare_layer(ref, job.mk, layer, (layer + 3) % w["L"], job.q[layer], job.kn[layer], job.vn[layer],
                       [job.k_cache], [job.v_cache], job.bm.block_table, job.model_config, job.engine_config, st)
    from morphserve_b200.worker.kernels._common import read_attn_error_flags
    assert read_attn_error_flags(0) == 0


def _slab_chunks(n_chunks, chunk_blocks, L, Hkv, device, gen):
    """Elastic chunks laid out as the reference's address rule expects them (worker/kernels/paged_attn.py:358-360):
    chunk j starts j * org_layer_param_size ELEMENTS below chunk 0, V follows K inside a slab
    (csrc/src/memory_manager.cpp:129-159)."""
    chunk_elems = chunk_blocks * L * Hkv * BS * D
    P = 2 * chunk_elems + 1152                    # "layer parameter size" in elements: two chunks and some slack
    slab = torch.empty(n_chunks * P, dtype=torch.float16, device=device)
    step = 1 << 28
    for i in range(0, slab.numel(), step):
        slab[i:i + step].normal_(generator=gen)
    kl, vl = [], []
    for j in range(n_chunks):
        base = (n_chunks - 1 - j) * P
        shape = (chunk_blocks, L, Hkv, BS, D)
        kl.append(slab[base:base + chunk_elems].view(shape))
        vl.append(slab[base + chunk_elems:base + 2 * chunk_elems].view(shape))
    return kl, vl, P, slab


@pytest.mark.parametrize("L,nb_org,chunk,n_chunks,B,max_len", [(32, 8192, 1024, 8, 128, 1536), (2, 300, 32, 3, 37, 260)])
def test_elastic_pool_against_reference_kernels(ref, L, nb_org, chunk, n_chunks, B, max_len):
    """The config-4 pool shape (8192 original blocks + 8 chunks of 1024, Llama-3-8B GQA, 32 layers) with the
    chunks laid out as weight slabs, block tables drawn over the WHOLE id range so that most sequences mix
    original and elastic blocks; and a small 3-chunk case."""
    import morphserve_b200 as mk
    dev = torch.device("cuda", 0)
    Hq, Hkv = 32, 8
    g = torch.Generator().manual_seed(4000 + L)
    dg = torch.Generator(device=dev).manual_seed(4001 + L)
    lens = torch.randint(1, max_len + 1, (B,), generator=g, dtype=torch.int64)
    need = (lens + BS - 1) // BS
    total = nb_org + chunk * n_chunks
    assert int(need.sum()) <= total
    perm = torch.randperm(total, generator=g)
    mbps = 128
    table = torch.full((B + 5, mbps), -1, dtype=torch.int32)
    rows = torch.randperm(B + 5, generator=g)[:B].to(torch.int32)
    pos = 0
    for b in range(B):
        n = int(need[b])
        table[int(rows[b]), :n] = perm[pos:pos + n].to(torch.int32)
        pos += n
    kc = torch.empty((nb_org, L, Hkv, BS, D), dtype=torch.float16, device=dev)
    vc = torch.empty_like(kc)
    for t in (kc, vc):
        flat = t.view(-1)
        for i in range(0, flat.numel(), 1 << 28):
            flat[i:i + (1 << 28)].normal_(generator=dg)
    kl, vl, P, _slab = _slab_chunks(n_chunks, chunk, L, Hkv, dev, dg)
    table_d, rows_d, lens_d = table.to(dev), rows.to(dev), lens.to(torch.int32).to(dev)
    mc = types.SimpleNamespace(num_layers=L, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D)
    ec = types.SimpleNamespace(block_size=BS, max_blocks_per_seq=mbps)
    c = dict(scale=D ** -0.5, num_blocks_org=nb_org, chunk_blocks=chunk)
    sbs, _ = mk.infer_state.seq_block_size_heuristic(Hkv, lens.tolist())
    st = H.decode_state(c, rows_d, lens_d, sbs=sbs)
    st.org_layer_param_size = P
    for layer in sorted({0, L // 2, L - 1}):
        q = torch.randn((B, Hq, D), generator=dg, dtype=torch.float16, device=dev)
        kn = torch.randn((B, Hkv, D), generator=dg, dtype=torch.float16, device=dev)
        vn = torch.randn((B, Hkv, D), generator=dg, dtype=torch.float16, device=dev)
        _compare_layer(ref, mk, layer, (layer + 1) % L, q, kn, vn, [kc] + kl, [vc] + vl, table_d, mc, ec, st)


def test_mixed_prefill_decode_store_against_reference(ref):
    """One store_kvcache call with prompts and decoding sequences together (worker/kernels/kvcache_mgmt.py:321-373),
    at a serving-sized shape: 24 prompts of up to 2048 tokens and 200 decoding sequences, Llama-3-8B heads."""
    import morphserve_b200 as mk
    dev = torch.device("cuda", 0)
    L, Hkv, Hq, n_pre, n_dec, mbps = 4, 8, 32, 24, 200, 130
    g = torch.Generator().manual_seed(77)
    dg = torch.Generator(device=dev).manual_seed(78)
    plens = torch.randint(1, 2049, (n_pre,), generator=g, dtype=torch.int64)
    dlens = torch.randint(1, 1537, (n_dec,), generator=g, dtype=torch.int64)
    lens = torch.cat([plens, dlens])
    need = (lens + BS - 1) // BS
    nb = int(need.sum() * 1.2) + 8
    perm = torch.randperm(nb, generator=g)
    B = n_pre + n_dec
    table = torch.full((B, mbps), -1, dtype=torch.int32)
    pos = 0
    for b in range(B):
        n = int(need[b])
        table[b, :n] = perm[pos:pos + n].to(torch.int32)
        pos += n
    kc = torch.randn((nb, L, Hkv, BS, D), generator=dg, dtype=torch.float16, device=dev)
    vc = torch.randn((nb, L, Hkv, BS, D), generator=dg, dtype=torch.float16, device=dev)
    n_tok = int(plens.sum()) + n_dec
    k = torch.randn((n_tok, Hkv, D), generator=dg, dtype=torch.float16, device=dev)
    v = torch.randn((n_tok, Hkv, D), generator=dg, dtype=torch.float16, device=dev)
    starts = (torch.cumsum(plens, 0) - plens).to(torch.int32)
    z = torch.zeros(0, dtype=torch.int32, device=dev)
    st = mk.LlamaInferState(
        batch_size=B, num_tokens=n_tok, seq_ids=torch.arange(B, dtype=torch.int32, device=dev), softmax_scale=D ** -0.5,
        num_prefill_seqs=n_pre, num_prefill_tokens=int(plens.sum()), prefill_seq_start_locs=starts.to(dev),
        prefill_seq_start_locs_with_end=z, prefill_seq_lens=plens.to(torch.int32).to(dev),
        max_prefill_len=int(plens.max()), num_decoding_seqs=n_dec, decoding_seq_lens=dlens.to(torch.int32).to(dev),
        max_decoding_len=int(dlens.max()), seq_block_size=512, num_seq_blocks=3, num_blocks_org=nb,
        kv_cache_new_block_size=0, org_layer_param_size=0, position_cos=z, position_sin=z, ignore_kvcache=False)
    mc = types.SimpleNamespace(num_layers=L, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D)
    ec = types.SimpleNamespace(block_size=BS, max_blocks_per_seq=mbps)
    table_d = table.to(dev)
    kr, vr = kc.clone(), vc.clone()
    ref.store_kvcache(k, v, kr, vr, [], [], table_d, mc, ec, _ref_state(ref, st), 2)
    mk.store_kvcache(k, v, kc, vc, [], [], table_d, mc, ec, st, 2)
    torch.cuda.synchronize()
    assert torch.equal(kc, kr) and torch.equal(vc, vr)


def test_block_manager_trace_against_reference_class(ref):
    """The reference's BlockManager (worker/block_manager.py:5-137, its three Triton kernels underneath) and this
    package's, driven through the same seeded sequence of allocate / free / gather-and-free calls: returned ids,
    block table rows of live sequences, counts, bitmap and the free count agree after every call."""
    import morphserve_b200 as mk
    rng = np.random.RandomState(5)
    nb, max_seqs, mbps = 4096, 96, 64
    a = ref.BlockManager("GPU", nb, max_seqs, mbps, BS)
    b = mk.BlockManager("GPU", nb, max_seqs, mbps, BS)
    lens = np.zeros(max_seqs, dtype=np.int64)
    for step in range(60):
        op = rng.choice(["alloc", "alloc", "alloc", "free", "gather"])
        ids = rng.choice(max_seqs, rng.randint(1, 24), replace=False)
        t_ids = torch.tensor(ids, dtype=torch.int32, device="cuda")
        if op == "alloc":
            target = np.minimum(lens[ids] + rng.randint(0, 200, len(ids)), mbps * BS)
            need = int(((target + BS - 1) // BS - (lens[ids] + BS - 1) // BS).sum())
            t_len = torch.tensor(target, dtype=torch.int32, device="cuda")
            if need > int(a.num_free_blocks):
                with pytest.raises(RuntimeError):
                    a.allocate_blocks_for_seqs(t_ids, t_len)
                with pytest.raises(RuntimeError):
                    b.allocate_blocks_for_seqs(t_ids, t_len)
                continue
            ra, rb = a.allocate_blocks_for_seqs(t_ids, t_len), b.allocate_blocks_for_seqs(t_ids, t_len)
            assert torch.equal(ra.long().cpu(), rb.long().cpu()), f"step {step}: allocated ids differ"
            lens[ids] = target
        elif op == "free":
            a.free_blocks_for_seqs(t_ids)
            b.free_blocks_for_seqs(t_ids)
            lens[ids] = 0
        else:
            ra, rb = a.gather_allocated_blocks_and_free(t_ids), b.gather_allocated_blocks_and_free(t_ids)
            assert torch.equal(ra.long().cpu(), rb.long().cpu()), f"step {step}: gathered ids differ"
            lens[ids] = 0
        assert torch.equal(a.num_seq_allocated_blocks, b.num_seq_allocated_blocks), f"step {step}: counts"
        assert torch.equal(a.is_block_free, b.is_block_free), f"step {step}: bitmap"
        assert int(a.num_free_blocks) == int(b.num_free_blocks), f"step {step}: free count"
        assert torch.equal(a.block_table, b.block_table), f"step {step}: block table"
        assert torch.equal(a.get_num_allocated_blocks(t_ids).cpu(), b.get_num_allocated_blocks(t_ids).cpu())


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_rotary_embedding_against_reference_kernel(ref, dtype):
    import morphserve_b200 as mk
    from oracle import kv_oracle as O
    dev = torch.device("cuda", 0)
    dg = torch.Generator(device=dev).manual_seed(9)
    n_tok, Hq, Hkv = 3000, 32, 8
    q = torch.randn((n_tok, Hq, D), generator=dg, dtype=dtype, device=dev)
    k = torch.randn((n_tok, Hkv, D), generator=dg, dtype=dtype, device=dev)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))
    pos = torch.randint(0, 4096, (n_tok,), generator=dg, device=dev).float()
    fr = torch.outer(pos, inv_freq)
    st = types.SimpleNamespace(position_cos=torch.cos(fr).to(torch.float16), position_sin=torch.sin(fr).to(torch.float16),
                               num_decoding_seqs=0)
    q0, k0 = q.cpu().numpy(), k.cpu().numpy()
    qr, kr = q.clone(), k.clone()
    ref.rotary_embedding_inplace(qr, kr, st)
    mk.set_rope_rounding("compiled")
    mk.rotary_embedding_inplace(q, k, st)
    torch.cuda.synchronize()
    assert torch.equal(q, qr) and torch.equal(k, kr), "differs from the reference kernel as Triton compiled it"
    # the oracle's statement of that rounding, and proof that it is not the operation-by-operation one
    qo, ko = O.rotary_embedding(q0, k0, st.position_cos.cpu().numpy(), st.position_sin.cpu().numpy(), rounding="compiled")
    assert qr.cpu().numpy().tobytes() == qo.tobytes() and kr.cpu().numpy().tobytes() == ko.tobytes()
    qw, _ = O.rotary_embedding(q0, k0, st.position_cos.cpu().numpy(), st.position_sin.cpu().numpy(), rounding="written")
    assert qw.tobytes() != qo.tobytes()
