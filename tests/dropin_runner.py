"""Runs the REFERENCE'S OWN ``LlamaModel`` (worker/model.py, staged under ``oracle/_ref``) through a
scripted serving scenario on cuda:0 and records what it computed.  Child process of
``tests/test_gpu_dropin.py``.

    python tests/dropin_runner.py --impl reference --out ref.npz
    python tests/dropin_runner.py --impl morphkv [--fused 0|1|2] --out ours.npz

``--impl reference``: every module is the reference's: its Triton kernels for the KV path, its
BlockManager, its compiled ``swiftllm_c``.
``--impl morphkv``: ``morphserve_b200.install_as_swiftllm()`` runs FIRST, so that the very same,
unmodified ``worker/model.py`` and ``worker/layers/transformer_layer.py`` import this package's
``paged_attention``, ``store_kvcache``, ``rotary_embedding_inplace``, ``BlockManager``,
``LlamaInferState`` and ``swiftllm_c`` instead; ``--fused 1`` also folds the decode append into the
attention launch, ``--fused 2`` the rotary embedding too.  Everything else (linear layers, RMSNorm,
SiLU, embedding, the layer code with its two streams and events, ``forward``'s metadata code, ``_swap``)
is the reference's in both runs.

The model is a small Llama (3 layers, 8 query / 2 KV heads of 128, hidden 1024) whose seeded weights are
written as a safetensors checkpoint and loaded by the reference's own loader.  Prefill attention goes through a
stand-in for the absent ``vllm_flash_attn`` (the same in both runs; not part of the path).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

MODEL = dict(model_type="llama", num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2,
             hidden_size=1024, vocab_size=512, max_position_embeddings=4096, intermediate_size=2048,
             rms_norm_eps=1e-5, hidden_act="silu", rope_theta=10000.0)
NUM_BLOCKS, NUM_CPU_BLOCKS, MAX_SEQS, MAX_BLOCKS_PER_SEQ, BLOCK = 96, 48, 32, 40, 16


def scenario():
    """The script both runs follow: a list of (op, args).  Token ids and lengths are seeded."""
    import numpy as np
    rs = np.random.RandomState(11)
    steps = []
    lens = {}
    # prompts of several lengths, including block edges
    first = {0: 5, 1: 16, 2: 17, 3: 150, 4: 33, 5: 260}
    steps.append(("forward", [rs.randint(0, 512, n).tolist() for n in first.values()], list(first), []))
    lens.update(first)
    for _ in range(3):                                      # plain decode steps
        ids = sorted(lens)
        for s in ids:
            lens[s] += 1
        steps.append(("forward", [[int(rs.randint(0, 512))] for _ in ids], ids, [lens[s] for s in ids]))
    steps.append(("swap_out", [1, 3]))
    for _ in range(2):                                      # decode without the swapped-out sequences
        ids = [s for s in sorted(lens) if s not in (1, 3)]
        for s in ids:
            lens[s] += 1
        steps.append(("forward", [[int(rs.randint(0, 512))] for _ in ids], ids, [lens[s] for s in ids]))
    steps.append(("free", [4]))
    del lens[4]
    steps.append(("swap_in", [3, 1]))
    # a mixed step: two new prompts in front of the decoding sequences
    new = {7: 40, 9: 3}
    ids = sorted(lens)
    for s in ids:
        lens[s] += 1
    steps.append(("forward", [rs.randint(0, 512, n).tolist() for n in new.values()]
                  + [[int(rs.randint(0, 512))] for _ in ids], list(new) + ids, [lens[s] for s in ids]))
    lens.update(new)
    for _ in range(14):                                     # decode across several block boundaries
        ids = sorted(lens)
        for s in ids:
            lens[s] += 1
        steps.append(("forward", [[int(rs.randint(0, 512))] for _ in ids], ids, [lens[s] for s in ids]))
    return steps


def write_checkpoint(path):
    """Seeded weights with O(1) activations, in the layout of a Hugging Face Llama checkpoint."""
    import torch
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(1234)
    h, f, v = MODEL["hidden_size"], MODEL["intermediate_size"], MODEL["vocab_size"]
    kv = MODEL["num_key_value_heads"] * (h // MODEL["num_attention_heads"])

    def w(*shape, scale):
        return (torch.randn(shape, generator=g) * scale).to(torch.float16)

    t = {"model.embed_tokens.weight": w(v, h, scale=1.0), "lm_head.weight": w(v, h, scale=h ** -0.5),
         "model.norm.weight": (1.0 + 0.1 * torch.randn(h, generator=g)).to(torch.float16)}
    for i in range(MODEL["num_hidden_layers"]):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = (1.0 + 0.1 * torch.randn(h, generator=g)).to(torch.float16)
        t[p + "post_attention_layernorm.weight"] = (1.0 + 0.1 * torch.randn(h, generator=g)).to(torch.float16)
        t[p + "self_attn.q_proj.weight"] = w(h, h, scale=2.0 * h ** -0.5)     # sharp attention: scores of a few units
        t[p + "self_attn.k_proj.weight"] = w(kv, h, scale=2.0 * h ** -0.5)
        t[p + "self_attn.v_proj.weight"] = w(kv, h, scale=h ** -0.5)
        t[p + "self_attn.o_proj.weight"] = w(h, h, scale=h ** -0.5)
        t[p + "mlp.up_proj.weight"] = w(f, h, scale=h ** -0.5)
        t[p + "mlp.gate_proj.weight"] = w(f, h, scale=h ** -0.5)
        t[p + "mlp.down_proj.weight"] = w(h, f, scale=f ** -0.5)
    save_file(t, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(MODEL, fh)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["reference", "morphkv"], required=True)
    ap.add_argument("--fused", type=int, default=0)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()

    import numpy as np
    import torch
    from oracle import ref_loader
    if a.impl == "morphkv":
        import morphserve_b200 as mk
        mk.install_as_swiftllm()                # before anything of the reference is imported
        mk.set_fused_decode_append(a.fused >= 1)
        mk.set_fused_decode_rope(a.fused >= 2)
    else:
        sys.modules["swiftllm_c"] = ref_loader.load_ext()
        assert sys.modules["swiftllm_c"] is not None, "the reference's swiftllm_c was not built"
    ref_loader.install_namespaces()
    import importlib
    model_mod = importlib.import_module("swiftllm.worker.model")
    EngineConfig = importlib.import_module("swiftllm.engine_config").EngineConfig
    layer_mod = importlib.import_module("swiftllm.worker.layers.transformer_layer")
    if a.impl == "morphkv":
        owner = layer_mod.paged_attention.__module__
        assert owner.startswith("morphserve_b200"), f"the layer code imported {owner}"
        assert model_mod.BlockManager.__module__.startswith("morphserve_b200")
        assert model_mod.swiftllm_c.__name__.startswith("morphserve_b200")
    else:
        assert layer_mod.paged_attention.__module__ == "swiftllm.worker.kernels.paged_attn"
        assert "oracle/_ref" in layer_mod.__file__

    tmp = tempfile.mkdtemp(prefix="mkv_dropin_")
    write_checkpoint(tmp)
    ec = EngineConfig(org_model_path=tmp, use_dummy=False, quantized_model_path="", quantized_q_config={},
                      block_size=BLOCK, gpu_mem_utilization=0.9, gpu_kv_cache_threshold=0.9,
                      num_layers_to_quantize=0, num_layers_to_quantize_max=0, quant_serve=False, awq_mode=False,
                      awq_half_mode=False, num_cpu_blocks=NUM_CPU_BLOCKS, max_seqs_in_block_table=MAX_SEQS,
                      max_blocks_per_seq=MAX_BLOCKS_PER_SEQ, max_batch_size=16, max_tokens_in_batch=2048,
                      req_preempt=0, block_swap=0)
    torch.cuda.set_device(0)
    model = model_mod.LlamaModel(ec, model_path=tmp)
    model.load_weights()
    model.init_kvcache_and_swap(NUM_BLOCKS)

    rec = {}
    cur = {"i": -1}
    post_forward = model.post_layer.forward

    def recording_post(input_embds, infer_state):
        i = cur["i"]
        rec[f"hidden_{i}"] = input_embds.detach().float().cpu().numpy()
        for f in dataclasses.fields(infer_state):
            val = getattr(infer_state, f.name)
            if isinstance(val, torch.Tensor):
                rec[f"state_{i}_{f.name}"] = val.detach().cpu().numpy()
            elif val is not None:
                rec[f"state_{i}_{f.name}"] = np.asarray(val)
        return post_forward(input_embds, infer_state)

    model.post_layer.forward = recording_post

    def snapshot(i):
        for nm, bm in (("gpu", model.gpu_block_manager), ("cpu", model.cpu_block_manager)):
            rec[f"{nm}_table_{i}"] = bm.block_table.cpu().numpy()
            rec[f"{nm}_count_{i}"] = bm.num_seq_allocated_blocks.cpu().numpy()
            rec[f"{nm}_free_{i}"] = bm.is_block_free.cpu().numpy()
            rec[f"{nm}_nfree_{i}"] = np.asarray(int(bm.num_free_blocks))
        rec[f"k_cache_{i}"] = model.k_cache.cpu().numpy()
        rec[f"v_cache_{i}"] = model.v_cache.cpu().numpy()
        rec[f"k_swap_{i}"] = model.k_swap.numpy().copy()
        rec[f"v_swap_{i}"] = model.v_swap.numpy().copy()

    for i, step in enumerate(scenario()):
        cur["i"] = i
        if step[0] == "forward":
            rec[f"tokens_{i}"] = np.asarray(model.forward(step[1], step[2], step[3]))
        elif step[0] == "swap_out":
            model.swap_out_seqs(step[1])
        elif step[0] == "swap_in":
            model.swap_in_seqs(step[1])
        else:
            model.free_seqs_resources(step[1])
        torch.cuda.synchronize()
        snapshot(i)
    rec["n_steps"] = np.asarray(len(scenario()))
    if a.impl == "morphkv":
        from morphserve_b200 import _lib
        from morphserve_b200.worker.kernels._common import read_attn_error_flags
        rec["calls"] = np.asarray(json.dumps(_lib.CALLS))
        rec["attn_error_flags"] = np.asarray(read_attn_error_flags(0))
    np.savez(a.out, **rec)
    print("dropin runner ok:", a.impl, a.fused, len(rec), "arrays")


if __name__ == "__main__":
    main()
