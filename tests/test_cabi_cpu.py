"""CPU-side checks of the C-ABI library: it loads, exports every function that
include/morphkv.h declares, validates arguments on the host before touching the
GPU, and its host-only entry points agree with the oracle.  No kernel runs."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle import kv_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    import __graft_entry__
    __graft_entry__.build()
    from morphserve_b200 import _lib
    return _lib


def declared_functions():
    text = open(os.path.join(ROOT, "include", "morphkv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mkv_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_function(L):
    names = declared_functions()
    assert len(names) >= 19
    for n in names:
        assert hasattr(L.lib, n), f"{n} is declared in morphkv.h but not exported"
    assert sorted(L.SIGNATURES) == names, "ctypes signatures and header disagree"
    assert L.lib.mkv_version() >= 100


def test_status_strings(L):
    assert L.lib.mkv_status_string(0) == b"ok"
    for s in range(-8, 0):
        assert len(L.lib.mkv_status_string(s)) > 0
    assert b"unknown" in L.lib.mkv_status_string(-99)


def test_chunk_layout_matches_oracle(L):
    rs = np.random.RandomState(0)
    for _ in range(200):
        start = int(rs.randint(1, 1 << 30)) * 2
        size = int(rs.randint(1 << 12, 1 << 28))
        quant = int(rs.randint(0, size + 4096))
        Lr, Hkv, bs, D = int(rs.randint(1, 49)), int(rs.choice([1, 2, 8, 32])), 16, 128
        k, v, n = C.c_uint64(), C.c_uint64(), C.c_int64()
        st = L.lib.mkv_chunk_layout(start, size, quant, Lr, Hkv, bs, D, 2, C.byref(k), C.byref(v), C.byref(n))
        try:
            ek, ev, en = O.chunk_layout(start, size, quant, Lr, Hkv, bs, D)
        except RuntimeError:
            assert st == -7
            continue
        assert st == 0 and (k.value, v.value, n.value) == (ek, ev, en)
    # Llama-3-8B numbers: a 436 MB fp16 layer slab with a 118 MB quantised layer
    k, v, n = C.c_uint64(), C.c_uint64(), C.c_int64()
    assert L.lib.mkv_chunk_layout(1 << 32, 436_224_000, 118_000_001, 32, 8, 16, 128, 2,
                                  C.byref(k), C.byref(v), C.byref(n)) == 0
    assert n.value == (436_224_000 - (118_000_001 + 255) // 256 * 256) // (2 * 32 * 8 * 128 * 2 * 16)
    assert k.value % 256 == 0 and v.value == k.value + n.value * (32 * 8 * 16 * 128 * 2)


def _pool(L, **kw):
    p = L.MkvPool()
    p.num_segments, p.elem_bytes, p.num_layers, p.num_kv_heads, p.block_size, p.head_dim = 1, 2, 2, 2, 16, 128
    p.num_blocks_org, p.chunk_blocks = 8, 0
    p.k_base[0] = 0x1000
    p.v_base[0] = 0x2000
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_host_side_argument_validation(L):
    lib = L.lib
    p = _pool(L)
    # NULL pool, bad dtype, bad shapes, bad layer: all refused before any CUDA call
    assert lib.mkv_store_kv_decode(0, None, 1, 1, None, 1, 4, 1, 1, 1, 0) == -1
    assert lib.mkv_store_kv_decode(0, None, 1, 1, C.byref(_pool(L, elem_bytes=3)), 1, 4, 1, 1, 1, 0) == -3
    assert lib.mkv_store_kv_decode(0, None, 1, 1, C.byref(_pool(L, num_segments=66)), 1, 4, 1, 1, 1, 0) == -2
    assert lib.mkv_store_kv_decode(0, None, 1, 1, C.byref(p), 1, 4, 1, 1, 1, 2) == -5      # layer out of range
    assert lib.mkv_store_kv_decode(0, None, None, 1, C.byref(p), 1, 4, 1, 1, 1, 0) == -1    # k is NULL
    assert lib.mkv_store_kv_decode(0, None, 1, 1, C.byref(p), 1, 4, 1, 1, 0, 0) == 0        # empty batch is a no-op
    assert lib.mkv_paged_attention_decode(0, None, 1, 1, C.byref(p), 1, 4, 1, 1, 3, 5, 0, 0.1, 4, None, 0) == -2
    assert lib.mkv_paged_attention_decode(0, None, 1, 1, C.byref(p), 1, 4, 1, 1, 3, 4, 7, 0.1, 4, None, 0) == -5
    assert lib.mkv_paged_attention_decode(0, None, 1, 1, C.byref(p), 1, 4, 1, 1, 0, 4, 0, 0.1, 4, None, 0) == 0
    assert lib.mkv_attn_plan(0, None, None, 0, 1, 1, 4, 4, 2, 128, 16, 8) == -4
    assert lib.mkv_bitmap_select(0, None, 1, 5, 2, 1, 1, 0, 1, None, None) == -2
    assert lib.mkv_copy_blocks(0, None, C.byref(p), None, None, 3) == -1
    assert lib.mkv_copy_blocks(0, None, C.byref(p), None, None, 0) == 0
    assert lib.mkv_remap_block_table(0, None, None, 4, 4, None, None, None, 2) == -1
    assert lib.mkv_block_need(0, None, 1, 8, 1, 1, 4, 0, 1, 1) == -2
    # compaction without a host round trip: target outside the bitmap, no result record, no pair arrays, no count
    assert lib.mkv_compact_plan(0, None, 1, 8, 9, 1, 1, 4, 1) == -2
    assert lib.mkv_compact_plan(0, None, 1, 8, 4, 1, 1, 4, None) == -1
    assert lib.mkv_compact_plan(0, None, 1, 8, 4, None, None, 4, 1) == -1
    assert lib.mkv_copy_blocks_counted(0, None, C.byref(p), 1, 1, 4, None) == -1
    assert lib.mkv_copy_blocks_counted(0, None, C.byref(p), None, None, 0, 1) == 0
    assert lib.mkv_remap_block_table_counted(0, None, 1, 4, 4, 1, 1, 1, 2, None) == -1


def test_swap_validates_ids_on_the_host(L):
    lib = L.lib
    p = _pool(L)
    src = (C.c_int64 * 2)(1, 9)
    dst = (C.c_int64 * 2)(0, 1)
    n = C.c_int64(-1)
    # device id 9 is outside the 8-block pool -> refused before any copy is issued
    assert lib.mkv_swap_blocks(0, None, C.byref(p), 0x10, 0x20, 4, src, dst, 2, 0, C.byref(n)) == -5
    assert n.value == 0
    src = (C.c_int64 * 2)(1, 2)
    dst = (C.c_int64 * 2)(0, 4)
    assert lib.mkv_swap_blocks(0, None, C.byref(p), 0x10, 0x20, 4, src, dst, 2, 0, None) == -5   # host id 4 of 4
    assert lib.mkv_swap_blocks(0, None, C.byref(p), 0x10, 0x20, 4, src, dst, 0, 0, None) == 0


def test_package_refuses_cpu_tensors():
    import torch
    import types
    from morphserve_b200 import store_kvcache
    t = torch.zeros((1, 2, 128), dtype=torch.float16)
    pool = torch.zeros((4, 1, 2, 16, 128), dtype=torch.float16)
    st = types.SimpleNamespace(seq_ids=torch.zeros(1, dtype=torch.int32), decoding_seq_lens=torch.ones(1, dtype=torch.int32),
                               num_prefill_seqs=0, num_prefill_tokens=0, num_decoding_seqs=1, num_blocks_org=4,
                               kv_cache_new_block_size=0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        store_kvcache(t, t, pool, pool, [], [], torch.zeros((2, 2), dtype=torch.int32),
                      types.SimpleNamespace(), types.SimpleNamespace(), st, 0)


def test_swap_run_coalescing_rule():
    # csrc/src/block_swapping.cpp:36-43 and :109-118 restated in the oracle
    assert O.coalesce_runs([3, 4, 5, 9], [0, 1, 2, 3]) == [(0, 3), (3, 1)]
    assert O.coalesce_runs([10, 11, 12, 13], [0, 1, 2, 3], num_blocks_org=12, chunk_blocks=4) == [(0, 2), (2, 2)]
    assert O.coalesce_runs([14, 15, 16, 17], [0, 1, 2, 3], num_blocks_org=12, chunk_blocks=4) == [(0, 2), (2, 2)]


def test_layer_replace_bookkeeping_and_errors_need_no_gpu():
    """Registration state, the two error messages raised before any copy (csrc/src/memory_manager.cpp:
    180-186, :195-200, :275-282) and the pure-host helpers of the layer-replace entry points."""
    import torch
    from morphserve_b200 import swiftllm_c as c
    with pytest.raises(RuntimeError, match="not registered in memory map"):
        c.replace_layer_org2quant(901)
    with pytest.raises(RuntimeError, match="not registered in original memory maps"):
        c.replace_layer_quant2org(901)
    c.register_layer_memory_org_gpu(901, 1 << 20, 100)
    c.register_layer_memory_quant(901, 1 << 21, 200)
    c.register_layer_memory_tensor_map_quant(901, [])
    with pytest.raises(RuntimeError, match="Layer requires 200 bytes, but only 100 bytes available"):
        c.replace_layer_org2quant(901)
    assert c.get_freed_memory_size(901, 30) == 70 and c.get_freed_memory_size(901, 300) == 0
    assert c.get_freed_memory_size(902, 1) == 0
    x = torch.zeros(16)
    assert c.verify_tensor_continuity([x[8:], x[:4], x[4:8]])
    assert not c.verify_tensor_continuity([x[:4], x[8:]])
    assert c.verify_tensor_continuity([])
