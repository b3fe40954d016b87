"""Generate the golden fixtures in this directory by running the REFERENCE's own
kernels on CPU in the Triton interpreter.

Usage (only where a checkout of the reference is available; it is not needed
to run the tests):

    python tests/golden/make_golden.py /path/to/MorphServe-checkout

The reference package directory is ``MorphServe/`` but its modules import each
other as ``swiftllm.*``; empty namespace modules are registered under that name
so that the kernel files import without executing the package ``__init__``
(which needs ray/awq).  Nothing of the reference is copied: its functions are
imported, called on the seeded inputs of ``cases.py`` and only their OUTPUTS are
stored (``*.npz`` + a SHA-256 of the inputs).
"""
from __future__ import annotations

import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests.golden import cases  # noqa: E402


def install_reference_alias(ref_root: str):
    pkg = os.path.join(ref_root, "MorphServe")
    for name, path in (("swiftllm", pkg), ("swiftllm.worker", os.path.join(pkg, "worker")),
                       ("swiftllm.worker.kernels", os.path.join(pkg, "worker", "kernels"))):
        m = types.ModuleType(name)
        m.__path__ = [path]
        sys.modules[name] = m
    utils = types.ModuleType("swiftllm.utils")
    utils.cdiv = lambda a, b: (a + b - 1) // b
    sys.modules["swiftllm.utils"] = utils


class Cfg:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def to_t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def slab_chunks(pools_np, dtype):
    """Lay elastic chunks out as the reference expects: chunk j sits
    j*org_layer_param_size elements BELOW chunk 0; V follows K inside a slab."""
    n_chunks = len(pools_np[0]) - 1
    if n_chunks == 0:
        return [], [], 0, None
    chunk_elems = pools_np[0][1].size
    P = 2 * chunk_elems + 640            # "layer parameter size" in elements, any value >= 2 chunks
    slab = torch.zeros(n_chunks * P, dtype=dtype)
    kl, vl = [], []
    for j in range(n_chunks):
        base = (n_chunks - 1 - j) * P
        shape = pools_np[0][1 + j].shape
        kv = slab[base:base + chunk_elems].view(shape)
        vv = slab[base + chunk_elems:base + 2 * chunk_elems].view(shape)
        kv.copy_(to_t(pools_np[0][1 + j]))
        vv.copy_(to_t(pools_np[1][1 + j]))
        kl.append(kv)
        vl.append(vv)
    return kl, vl, P, slab


def run_decode_case(name, kw):
    from swiftllm.worker.kernels.paged_attn import paged_attention
    from swiftllm.worker.kernels.kvcache_mgmt import store_kvcache
    from oracle.kv_oracle import seq_block_size_heuristic

    c = cases.build_decode_case(**kw)
    tdtype = torch.float16 if c["q"].dtype == np.float16 else torch.float32
    k_cache, v_cache = to_t(c["k_pools"][0]).clone(), to_t(c["v_pools"][0]).clone()
    k_new_l, v_new_l, P, _slab = slab_chunks((c["k_pools"], c["v_pools"]), tdtype)
    sbs, nsb = seq_block_size_heuristic(c["Hkv"], c["seq_lens"])
    block_table = to_t(c["block_table"]).clone()
    model_config = Cfg(num_layers=c["L"], num_q_heads=c["Hq"], num_kv_heads=c["Hkv"], head_dim=c["D"])
    engine_config = Cfg(block_size=c["bs"], max_blocks_per_seq=block_table.shape[1])
    st = Cfg(seq_ids=to_t(c["seq_ids"]), softmax_scale=c["scale"], num_prefill_seqs=0, num_prefill_tokens=0,
             prefill_seq_start_locs=torch.zeros(0, dtype=torch.int32), prefill_seq_lens=torch.zeros(0, dtype=torch.int32),
             max_prefill_len=0, num_decoding_seqs=c["B"], decoding_seq_lens=to_t(c["seq_lens"]),
             max_decoding_len=int(c["seq_lens"].max()), seq_block_size=sbs, num_seq_blocks=nsb,
             num_blocks_org=c["num_blocks_org"], kv_cache_new_block_size=c["chunk_blocks"],
             org_layer_param_size=P, ignore_kvcache=False)
    store_kvcache(to_t(c["k_new"]), to_t(c["v_new"]), k_cache, v_cache, k_new_l, v_new_l, block_table,
                  model_config, engine_config, st, c["layer"])
    o = torch.zeros((c["B"], c["Hq"] * c["D"]), dtype=tdtype)
    paged_attention(to_t(c["q"]), k_cache, v_cache, k_new_l, v_new_l, block_table,
                    model_config, engine_config, st, c["layer"], o)
    k_after = [k_cache.numpy()] + [t.numpy() for t in k_new_l]
    v_after = [v_cache.numpy()] + [t.numpy() for t in v_new_l]
    np.savez_compressed(os.path.join(HERE, f"decode_{name}.npz"),
                        o=o.numpy().reshape(c["B"], c["Hq"], c["D"]),
                        inputs_sha256=np.array(cases.case_inputs_hash(c)),
                        pools_after_sha256=np.array(cases.sha256_of(*k_after, *v_after)),
                        seq_block_size=np.array(sbs))
    print("decode", name, "sbs", sbs, "ok")


def run_prefill_case(name, kw):
    from swiftllm.worker.kernels.kvcache_mgmt import store_kvcache

    c = cases.build_prefill_case(**kw)
    tdtype = torch.float16
    k_cache, v_cache = to_t(c["k_pools"][0]).clone(), to_t(c["v_pools"][0]).clone()
    k_new_l, v_new_l, P, _slab = slab_chunks((c["k_pools"], c["v_pools"]), tdtype)
    block_table = to_t(c["block_table"]).clone()
    npre = len(c["prefill_lens"])
    model_config = Cfg(num_layers=c["L"], num_kv_heads=c["Hkv"], head_dim=c["D"])
    engine_config = Cfg(block_size=c["bs"], max_blocks_per_seq=block_table.shape[1])
    st = Cfg(seq_ids=to_t(c["seq_ids"]), num_prefill_seqs=npre, num_prefill_tokens=c["num_prefill_tokens"],
             prefill_seq_start_locs=to_t(c["prefill_start_locs"]), prefill_seq_lens=to_t(c["prefill_lens"]),
             max_prefill_len=int(c["prefill_lens"].max()), num_decoding_seqs=len(c["decode_lens"]),
             decoding_seq_lens=to_t(c["decode_lens"]), num_blocks_org=c["num_blocks_org"],
             kv_cache_new_block_size=c["chunk_blocks"], org_layer_param_size=P, ignore_kvcache=False)
    store_kvcache(to_t(c["k"]), to_t(c["v"]), k_cache, v_cache, k_new_l, v_new_l, block_table,
                  model_config, engine_config, st, c["layer"])
    k_after = [k_cache.numpy()] + [t.numpy() for t in k_new_l]
    v_after = [v_cache.numpy()] + [t.numpy() for t in v_new_l]
    np.savez_compressed(os.path.join(HERE, f"prefill_{name}.npz"),
                        inputs_sha256=np.array(cases.sha256_of(c["k"], c["v"], c["block_table"], c["seq_ids"])),
                        pools_after_sha256=np.array(cases.sha256_of(*k_after, *v_after)))
    print("prefill", name, "ok")


def run_block_manager_trace():
    import swiftllm.worker.block_manager as ref_bm

    tr = cases.block_manager_trace()
    _empty = torch.empty
    torch.empty = lambda *a, **k: _empty(*a, **{**k, "device": "cpu"})   # the class hard-codes "cuda:0"
    try:
        bm = ref_bm.BlockManager.__new__(ref_bm.BlockManager)
        bm.device_name = "GPU"
        bm.num_free_blocks = bm.num_blocks = tr["num_blocks"]
        bm.num_free_blocks_org = bm.num_blocks_org = tr["num_blocks"]
        bm.block_size = tr["block_size"]
        bm.num_seq_allocated_blocks = torch.zeros(tr["max_seqs"], dtype=torch.int32)
        bm.block_table = torch.full((tr["max_seqs"], tr["max_blocks_per_seq"]), -1, dtype=torch.int32)
        bm.is_block_free = torch.ones(tr["num_blocks"], dtype=torch.bool)
        out = {}
        for i, (op, ids, lens) in enumerate(tr["ops"]):
            if op == "alloc":
                r = bm.allocate_blocks_for_seqs(to_t(ids), to_t(lens))
            elif op == "free":
                bm.free_blocks_for_seqs(to_t(ids))
                r = torch.empty(0)
            else:
                r = bm.gather_allocated_blocks_and_free(to_t(ids))
            out[f"ret_{i}"] = r.numpy().astype(np.int64)
            out[f"table_{i}"] = bm.block_table.numpy().copy()
            out[f"count_{i}"] = bm.num_seq_allocated_blocks.numpy().copy()
            out[f"free_{i}"] = bm.is_block_free.numpy().copy()
            out[f"nfree_{i}"] = np.array(int(bm.num_free_blocks))
    finally:
        torch.empty = _empty
    np.savez_compressed(os.path.join(HERE, "block_manager_trace.npz"), n_ops=np.array(len(tr["ops"])), **out)
    print("block manager trace:", len(tr["ops"]), "ops ok")


def run_rope_case(name, kw):
    from swiftllm.worker.kernels.rotary_emb import rotary_embedding_inplace
    c = cases.build_rope_case(**kw)
    q, k = to_t(c["q"]).clone(), to_t(c["k"]).clone()
    st = Cfg(position_cos=to_t(c["cos"]), position_sin=to_t(c["sin"]))
    rotary_embedding_inplace(q, k, st)
    np.savez_compressed(os.path.join(HERE, f"rope_{name}.npz"), q=q.numpy(), k=k.numpy(),
                        inputs_sha256=np.array(cases.sha256_of(c["q"], c["k"], c["cos"], c["sin"])))
    print("rope", name, "ok")


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MORPHSERVE_REFERENCE", "")
    if not os.path.isdir(os.path.join(ref_root, "MorphServe")):
        raise SystemExit("usage: make_golden.py <reference checkout>")
    install_reference_alias(ref_root)
    only = set(sys.argv[2:])
    for name, kw in cases.DECODE_CASES.items():
        if not only or name in only:
            run_decode_case(name, kw)
    for name, kw in cases.PREFILL_CASES.items():
        if not only or name in only:
            run_prefill_case(name, kw)
    for name, kw in cases.ROPE_CASES.items():
        if not only or "rope" in only:
            run_rope_case(name, kw)
    if not only or "block_manager" in only:
        run_block_manager_trace()


if __name__ == "__main__":
    main()
