"""This package's ``swiftllm_c`` against the reference's COMPILED extension (csrc/src/*.cpp, built by
``oracle/build_ref.py`` into ``oracle/_ref``), call for call on the same device memory:

* ``swap_blocks`` out and in on pageable host memory (block_swapping.cpp:22-85);
* the swap-OUT half of ``swap_blocks_new_kv_combined`` with chunks laid out as slabs (:88-202).  The reference's
  combined swap-IN is never run: it derives the device address from the source (host) id (:156-161) and would
  write outside the chunk; this package's swap-in is checked against the swap-out it inverts;
* ``register_kv_cache_info`` + ``register_layer_memory_*`` + ``acquire_new_kvcache`` (memory_manager.cpp:57-176):
  addresses, block count, zero fill, exceptions;
* ``replace_layer_org2quant`` / ``replace_layer_quant2org`` (:179-364): slab bytes and the returned views;
* ``get_freed_memory_size`` / ``verify_tensor_continuity`` (:367-405).
"""
import numpy as np
import pytest
import torch

from oracle import ref_loader

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_loader.ext_available(), reason=ref_loader.why_unavailable())]
L, HKV, BS, D = 4, 8, 16, 128


@pytest.fixture(scope="module")
def ref_c():
    c = ref_loader.load_ext()
    yield c
    # The reference keeps the registered tensor maps (Python objects) in C++ statics that are destroyed after the
    # interpreter has shut down (csrc/src/memory_manager.cpp:8-13): leave empty lists behind so that nothing of
    # Python's is left for those destructors to touch.
    for layer in REGISTERED_MAP_LAYERS:
        c.register_layer_memory_tensor_map_quant(layer, [])
        c.register_layer_memory_tensor_map_org(layer, [])


REGISTERED_MAP_LAYERS = (9, 10)


def _same_bits(x, y):
    """Equal as BYTES: the slabs hold random bits, which read as fp16 include NaNs."""
    return torch.equal(x.contiguous().view(torch.uint8), y.contiguous().view(torch.uint8))


def _pools(nb, ncpu, seed, pin=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    shape = (nb, L, HKV, BS, D)
    k = torch.randn(shape, generator=g, dtype=torch.float16, device="cuda")
    v = torch.randn(shape, generator=g, dtype=torch.float16, device="cuda")
    hg = torch.Generator().manual_seed(seed + 1)
    ks = torch.randn((ncpu,) + shape[1:], generator=hg).to(torch.float16)
    vs = torch.randn((ncpu,) + shape[1:], generator=hg).to(torch.float16)
    return k, v, ks, vs


def _id_lists(rs, n_src_space, n_dst_space, n):
    """Distinct ids on both sides with runs of consecutive pairs in between (the case the copy coalesces)."""
    src = rs.permutation(n_src_space)[:n].tolist()
    dst = rs.permutation(n_dst_space)[:n].tolist()
    run = min(12, n // 2, n_src_space - 1, n_dst_space - 1)
    s0, d0 = int(rs.randint(0, n_src_space - run)), int(rs.randint(0, n_dst_space - run))
    keep_s = [x for x in src if not s0 <= x < s0 + run][: n - run]
    keep_d = [x for x in dst if not d0 <= x < d0 + run][: n - run]
    m = min(len(keep_s), len(keep_d))
    return keep_s[:m // 2] + list(range(s0, s0 + run)) + keep_s[m // 2:m], \
        keep_d[:m // 2] + list(range(d0, d0 + run)) + keep_d[m // 2:m]


def test_swap_blocks_matches_the_reference_extension(ref_c):
    from morphserve_b200 import swiftllm_c as ours
    rs = np.random.RandomState(0)
    nb, ncpu = 96, 64
    k, v, ks, vs = _pools(nb, ncpu, 1)
    k2, v2, ks2, vs2 = k.clone(), v.clone(), ks.clone(), vs.clone()
    src, dst = _id_lists(rs, nb, ncpu, 40)
    ref_c.swap_blocks(src, dst, False, k, v, ks, vs)
    ours.swap_blocks(src, dst, False, k2, v2, ks2, vs2)
    torch.cuda.synchronize()
    assert ks.numpy().tobytes() == ks2.numpy().tobytes() and vs.numpy().tobytes() == vs2.numpy().tobytes()
    src, dst = _id_lists(rs, ncpu, nb, 40)
    ref_c.swap_blocks(src, dst, True, k, v, ks, vs)
    ours.swap_blocks(src, dst, True, k2, v2, ks2, vs2)
    torch.cuda.synchronize()
    assert torch.equal(k, k2) and torch.equal(v, v2)
    # the same through a pinned swap space (one zero-copy kernel instead of copies per run), ids as device tensors
    k3, v3 = k.clone(), v.clone()
    ks3, vs3 = ks.clone().pin_memory(), vs.clone().pin_memory()
    src, dst = _id_lists(rs, nb, ncpu, 33)
    ref_c.swap_blocks(src, dst, False, k, v, ks, vs)
    ours.swap_blocks(torch.tensor(src, device="cuda"), torch.tensor(dst, device="cuda"), False, k3, v3, ks3, vs3)
    torch.cuda.synchronize()
    assert ks.numpy().tobytes() == ks3.numpy().tobytes() and vs.numpy().tobytes() == vs3.numpy().tobytes()


def test_combined_swap_out_matches_the_reference_extension(ref_c):
    from morphserve_b200 import swiftllm_c as ours
    rs = np.random.RandomState(1)
    nb_org, chunk, n_chunks, ncpu = 40, 8, 3, 80
    k, v, ks, vs = _pools(nb_org, ncpu, 2)
    chunk_elems = chunk * L * HKV * BS * D
    P = 2 * chunk_elems + 384                                  # elements between chunk starts
    g = torch.Generator(device="cuda").manual_seed(3)
    slab = torch.randn(n_chunks * P, generator=g, dtype=torch.float16, device="cuda")
    kl, vl = [], []
    for j in range(n_chunks):                                   # chunk j sits j*P elements BELOW chunk 0
        base = (n_chunks - 1 - j) * P
        kl.append(slab[base:base + chunk_elems].view(chunk, L, HKV, BS, D))
        vl.append(slab[base + chunk_elems:base + 2 * chunk_elems].view(chunk, L, HKV, BS, D))
    ks2, vs2 = ks.clone(), vs.clone()
    total = nb_org + chunk * n_chunks
    src = rs.permutation(total)[:30].tolist() + list(range(nb_org - 3, nb_org + chunk + 2))   # a run across 2 boundaries
    src = list(dict.fromkeys(src))
    dst = rs.permutation(ncpu)[:len(src)].tolist()
    ref_c.swap_blocks_new_kv_combined(src, dst, False, nb_org, P, chunk, 2, k, v, ks, vs, kl[0], vl[0])
    ours.swap_blocks_new_kv_combined(src, dst, False, nb_org, P, chunk, 2, k, v, ks2, vs2, kl[0], vl[0])
    torch.cuda.synchronize()
    assert ks.numpy().tobytes() == ks2.numpy().tobytes() and vs.numpy().tobytes() == vs2.numpy().tobytes()
    # this package's swap-in inverts it (device address from the TARGET id): every block returns to where it was
    before_k, before_slab = k.clone(), slab.clone()
    k.zero_()
    v.zero_()
    for t in kl + vl:
        t.zero_()
    ours.swap_blocks_new_kv_combined(dst, src, True, nb_org, P, chunk, 2, k, v, ks2, vs2, kl[0], vl[0])
    torch.cuda.synchronize()
    for b in src:
        if b < nb_org:
            assert torch.equal(k[b], before_k[b])
        else:
            j, r = divmod(b - nb_org, chunk)
            lo = (n_chunks - 1 - j) * P + r * (chunk_elems // chunk)
            assert torch.equal(slab[lo:lo + chunk_elems // chunk], before_slab[lo:lo + chunk_elems // chunk])


def test_acquire_new_kvcache_matches_the_reference_extension(ref_c):
    from morphserve_b200 import swiftllm_c as ours
    for c in (ref_c, ours):
        c.register_kv_cache_info(L, HKV, BS, D)
    block_bytes = 2 * L * HKV * D * 2 * BS
    org_size = 9 * block_bytes + 7777
    for layer, quant_size in ((3, 2 * block_bytes + 1001), (4, 5 * block_bytes - 256), (5, 100)):
        slab = torch.full((org_size,), 0x5A, dtype=torch.uint8, device="cuda")
        for c in (ref_c, ours):
            c.register_layer_memory_org_gpu(layer, slab.data_ptr(), org_size)
            c.register_layer_memory_quant(layer, 0, quant_size)
        kr, vr = ref_c.acquire_new_kvcache(layer)
        ptrs = (kr.data_ptr(), vr.data_ptr(), tuple(kr.shape), tuple(vr.shape), kr.dtype)
        torch.cuda.synchronize()
        after_ref = slab.clone()
        slab.fill_(0x5A)
        ko, vo = ours.acquire_new_kvcache(layer)
        torch.cuda.synchronize()
        assert ptrs == (ko.data_ptr(), vo.data_ptr(), tuple(ko.shape), tuple(vo.shape), ko.dtype)
        assert torch.equal(slab, after_ref), "zero fill covers a different byte range"
        assert ko.is_contiguous() and vo.is_contiguous() and ko.device == kr.device
        assert ref_c.get_freed_memory_size(layer, quant_size) == ours.get_freed_memory_size(layer, quant_size)
    assert ref_c.get_freed_memory_size(77, 5) == ours.get_freed_memory_size(77, 5) == 0
    # not registered, and no room for a single block: RuntimeError from both, same message
    for c in (ref_c, ours):
        with pytest.raises(RuntimeError, match="Layer not found in memory maps"):
            c.acquire_new_kvcache(41)
    slab = torch.zeros((org_size,), dtype=torch.uint8, device="cuda")
    for c in (ref_c, ours):
        c.register_layer_memory_org_gpu(42, slab.data_ptr(), org_size)
        c.register_layer_memory_quant(42, 0, org_size - 300)
        with pytest.raises(RuntimeError, match="No space available for new KV cache blocks"):
            c.acquire_new_kvcache(42)


def _tensor_map(rs, total, n):
    """Entries as the reference's layer manager registers them: [{name: {offset, shape, dtype, size}}, ...]."""
    out, off = [], 0
    dtypes = [torch.float16, torch.int32, torch.float16, torch.int8]
    for i in range(n):
        dt = dtypes[i % len(dtypes)]
        rows, cols = int(rs.randint(1, 40)), 8 * int(rs.randint(1, 30))
        size = rows * cols * dt.itemsize
        if off + size > total:
            break
        out.append({f"w{i}.{'qweight' if dt == torch.int32 else 'weight'}":
                    {"offset": off, "shape": [rows, cols], "dtype": dt, "size": size}})
        off += (size + 255) // 256 * 256
    return out


def test_replace_layer_matches_the_reference_extension(ref_c):
    from morphserve_b200 import swiftllm_c as ours
    rs = np.random.RandomState(2)
    org_size, quant_size = 3 << 20, 900_000
    host_org = torch.randint(0, 255, (org_size,), dtype=torch.uint8).pin_memory()
    host_quant = torch.randint(0, 255, (quant_size,), dtype=torch.uint8).pin_memory()
    map_q, map_o = _tensor_map(rs, quant_size, 12), _tensor_map(rs, org_size, 9)
    slabs = {}
    for name, c in (("ref", ref_c), ("ours", ours)):
        slab = slabs[name] = torch.full((org_size,), 0xA5, dtype=torch.uint8, device="cuda")
        c.register_layer_memory_org_gpu(9, slab.data_ptr(), org_size)
        c.register_layer_memory_org_cpu(9, host_org.data_ptr(), org_size)
        c.register_layer_memory_quant(9, host_quant.data_ptr(), quant_size)
        c.register_layer_memory_tensor_map_quant(9, map_q)
        c.register_layer_memory_tensor_map_org(9, map_o)
    for call in ("replace_layer_org2quant", "replace_layer_quant2org"):
        a = getattr(ref_c, call)(9)
        b = getattr(ours, call)(9)
        torch.cuda.synchronize()
        assert torch.equal(slabs["ref"], slabs["ours"]), f"{call}: slab bytes differ"
        assert len(a) == len(b) > 0
        for x, y in zip(a, b):
            assert x.dtype == y.dtype and tuple(x.shape) == tuple(y.shape) and x.is_contiguous() and y.is_contiguous()
            assert x.data_ptr() - slabs["ref"].data_ptr() == y.data_ptr() - slabs["ours"].data_ptr()
            assert _same_bits(x, y)
        assert ref_c.verify_tensor_continuity(a) == ours.verify_tensor_continuity(b)
    for c in (ref_c, ours):
        with pytest.raises(RuntimeError, match="not registered"):
            c.replace_layer_org2quant(1234)
        with pytest.raises(RuntimeError, match="not registered"):
            c.replace_layer_quant2org(1234)
    # a quantised image larger than the slab is refused before any copy
    for c in (ref_c, ours):
        c.register_layer_memory_org_gpu(10, slabs["ref"].data_ptr(), 1000)
        c.register_layer_memory_quant(10, host_quant.data_ptr(), 2000)
        c.register_layer_memory_tensor_map_quant(10, map_q[:1])
        with pytest.raises(RuntimeError, match="bytes available"):
            c.replace_layer_org2quant(10)
