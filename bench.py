#!/usr/bin/env python
"""Decode-step benchmark of the KV-cache hot path (paged-attention decode + KV
append + block allocation) on synthetic inputs shaped like the named model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" = one decode step of the whole batch: allocate blocks for the grown
sequences, then for each of the L layers append one token per sequence
(store_kvcache) and run decode attention (paged_attention).  Lengths advance by
one per step.  Prints ONE JSON line (rank 0).

  value   decode tokens/s, all ranks, inputs resident in HBM, CUDA-event timed
  e2e     the same through the public Python API with HOST inputs: per step the
          q/k/v of every layer are copied from pinned memory and the attention
          output is copied back, inside the timed region
  roofline  KV GB/s of the attention kernel vs the measured HBM copy peak
  cpu_baseline  the reference's PyTorch paged-attention loop on the host cores

With N > 1 (torchrun) every rank owns its own pool, block table and batch
(sequence sharding, no collective on the data path); the step is bracketed by
barriers and the slowest rank's device time is used.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import statistics
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # Llama-3-8B GQA, 256 sequences per GPU: the configuration the tokens/s-at-1/2/4/8-GPUs metric is quoted on
    "llama3-8b-gqa-decode": dict(cfg=3, B=256, Hq=32, Hkv=8, L=32, max_len=1536, free_frac=0.10),
    # Llama-2-7B MHA, 64 sequences, contexts up to 768
    "llama2-7b-mha-decode": dict(cfg=2, B=64, Hq=32, Hkv=32, L=32, max_len=768, free_frac=0.30),
    # CodeLlama-34B GQA, 512 sequences per GPU, sequence-sharded
    "codellama-34b-gqa-decode": dict(cfg=5, B=512, Hq=64, Hkv=8, L=48, max_len=1536, free_frac=0.05),
    # CodeLlama-34B GQA, head-sharded: every rank holds Hkv/N KV heads (and their query heads) of ALL
    # 512*N sequences; the attention outputs are all-gathered over NVLink (NCCL) after every layer
    "codellama-34b-gqa-decode-headshard": dict(cfg=5, B=512, Hq=64, Hkv=8, L=48, max_len=1536, free_frac=0.05,
                                               head_shard=True),
    # elastic-resize pool (Llama-3-8B shape): compaction of a 16384-block pool down to 10240 (copy + remap timing)
    "kv-resize": dict(cfg=4, resize=True, L=32, Hq=32, Hkv=8, B=128, max_len=1536, nb_org=8192, chunk=1024,
                      n_chunks=8, release=6),
    # the same with 4 layers (pool 4 GB) for profiler captures
    "kv-resize-small": dict(cfg=4, resize=True, L=4, Hq=32, Hkv=8, B=128, max_len=1536, nb_org=8192, chunk=1024,
                            n_chunks=8, release=6),
    # llama3-8b batch, 2 layers, every context exactly 768 tokens (no length spread): isolates scheduling effects
    "llama3-8b-gqa-decode-2layer-uniform": dict(cfg=3, B=256, Hq=32, Hkv=8, L=2, min_len=768, max_len=768, free_frac=0.10),
    # prefill scatter of store_kvcache: 32 prompts of up to 2048 tokens into a fragmented pool, 4 layers
    "kv-prefill": dict(cfg=3, prefill=True, L=4, Hq=32, Hkv=8, n_seqs=32, max_len=2048),
    # four times the prompt tokens: shows how much of the figure above is the launch's start and end
    "kv-prefill-large": dict(cfg=3, prefill=True, L=4, Hq=32, Hkv=8, n_seqs=128, max_len=2048),
    # block swap between the pool and the host swap space (Llama-3-8B block = 2 x 1 MiB): 1024 blocks per direction
    "kv-swap": dict(cfg=3, swap=True, L=32, Hq=32, Hkv=8, nb=4096, n_swap=1024),
    # the same with 4 layers (blocks of 2 x 128 KiB, pool 1 GB) for profiler captures
    "kv-swap-small": dict(cfg=3, swap=True, L=4, Hq=32, Hkv=8, nb=4096, n_swap=1024),
    # the same with the all-gather folded into the attention launch: every rank stores its output slice straight
    # into all ranks' full-width matrices (peer-mapped symmetric memory), one barrier per layer
    "codellama-34b-gqa-decode-headshard-push": dict(cfg=5, B=512, Hq=64, Hkv=8, L=48, max_len=1536, free_frac=0.05,
                                                    head_shard=True, push=True),
    # small case for profiler captures and CPU-side dry runs (pool ~1.3 GB: larger than L2)
    "small-gqa-decode": dict(cfg=9, B=64, Hq=32, Hkv=8, L=4, max_len=1536, free_frac=0.10),
    # the llama3-8b batch with 2 layers: same bytes per attention launch as the full workload, pool ~1.8 GB
    "llama3-8b-gqa-decode-2layer": dict(cfg=3, B=256, Hq=32, Hkv=8, L=2, max_len=1536, free_frac=0.10),
    # one 32k-token sequence among 127 short ones, 2 layers: the case that needs split-KV to stay balanced
    "skewed-gqa-decode": dict(cfg=10, B=128, Hq=32, Hkv=8, L=2, max_len=512, free_frac=0.10, n_long=1,
                              long_len=32768),
    # the default workload with the rotary embedding of q and k in front of every layer's append (the step before the
    # path in the reference's layer code); fused into the attention launch unless --no-fused-rope
    "llama3-8b-gqa-decode-rope": dict(cfg=3, B=256, Hq=32, Hkv=8, L=32, max_len=1536, free_frac=0.10, rope=True),
    # layer slab replace (the producer of expand / release events): Llama-3-8B fp16 layer (436 MB) <-> its 4-bit
    # image (~125 MB), host -> device from pinned memory
    "layer-replace": dict(cfg=13, replace=True, org_bytes=436 << 20, quant_bytes=125 << 20),
    # 8 sequences of up to 2k tokens, 32 layers: launches of ~10 us, where issuing the step costs more than running it
    "small-batch-gqa-decode": dict(cfg=12, B=8, Hq=32, Hkv=8, L=32, max_len=2048, free_frac=0.10, rope=True),
    # 8 long sequences (8k-32k tokens), 2 layers: fewer (sequence, head) pairs than worker warps
    "longctx-gqa-decode": dict(cfg=11, B=8, Hq=32, Hkv=8, L=2, min_len=8192, max_len=32768, free_frac=0.10),
}
D, BS = 128, 16
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes (read + write) per attention launch divided by the algorithmic K/V bytes, from an ncu capture of the
# llama3-8b-gqa-decode-2layer workload (same batch and bytes per launch as llama3-8b-gqa-decode): 852.1 and 849.3 MB
# moved by the two captured launches of the fourth step, whose contexts hold 832.6 MB of K/V (840.6 MB counted in
# whole 16-token blocks, which is what the kernel fetches).  Traffic grows with the units processed, so the ratio is
# applied to the live byte count of the timed launches.
NCU_TRAFFIC_RATIO = {"llama3-8b-gqa-decode": 1.0217, "llama3-8b-gqa-decode-2layer": 1.0217}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------------------
# sharding (host logic; covered by the 2-rank gloo tests)
# ----------------------------------------------------------------------------
def shard_workload(w, rank, world):
    """What one rank runs.  Sequence sharding (default): the rank's own batch of
    w["B"] sequences, drawn from its own seed, all KV heads - no data crosses
    ranks.  Head sharding: the global batch of w["B"]*world sequences (same seed
    on every rank, so block tables agree) and the rank's contiguous slice of
    Hkv/world KV heads with their Hq/world query heads."""
    w = dict(w)
    if w.get("head_shard"):
        if w["Hkv"] % world != 0:
            raise ValueError(f"head sharding needs num_kv_heads ({w['Hkv']}) divisible by the number of ranks ({world})")
        w["B_global"] = w["B"] * world
        w["B"] = w["B_global"]
        w["Hq_global"], w["Hkv_global"] = w["Hq"], w["Hkv"]
        w["Hq"], w["Hkv"] = w["Hq"] // world, w["Hkv"] // world
        w["head_offset"] = rank * w["Hq"]
        w["seed"] = 1000 * w["cfg"]
        w["tokens_per_step"] = w["B_global"]          # whole job, counted once
    else:
        w["B_global"] = w["B"] * world
        w["seed"] = 1000 * w["cfg"] + rank
        w["tokens_per_step"] = w["B"] * world
    return w


def bind_to_gpu_numa_node(local_rank):
    """Pin this rank to the CPUs of the NUMA node its GPU hangs off, so that the pinned host buffers it allocates
    afterwards (first touch) and the threads that fill them are local to the GPU's PCIe root: with eight ranks
    copying at once, buffers on the far socket are what the host-buffer leg is limited by.  Returns
    (node, previous affinity) or (None, None) when the topology cannot be read or the CPUs are not ours to use."""
    try:
        p = torch.cuda.get_device_properties(local_rank)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        if node < 0:
            return None, None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        before = os.sched_getaffinity(0)
        cpus &= before
        if not cpus:
            return None, None
        os.sched_setaffinity(0, cpus)
        return node, before
    except Exception:
        return None, None


def max_over_ranks(value, dist, device):
    """Slowest rank's time (dist is torch.distributed or None)."""
    if dist is None:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ----------------------------------------------------------------------------
# synthetic workload
# ----------------------------------------------------------------------------
def draw_lengths_and_tables(w, rank, growth_tokens):
    """Seeded lengths and a block table built from a shuffled free list."""
    g = torch.Generator().manual_seed(w.get("seed", 1000 * w["cfg"] + rank))
    lens = torch.randint(w.get("min_len", 1), w["max_len"] + 1, (w["B"],), generator=g, dtype=torch.int64)
    lens[:w.get("n_long", 0)] = w.get("long_len", 0)
    need = (lens + BS - 1) // BS
    live = int(need.sum())
    growth = w["B"] * ((growth_tokens + BS - 1) // BS + 1)
    nb = int(np.ceil(live / (1.0 - w["free_frac"]))) + growth
    perm = torch.randperm(nb, generator=g)
    mbps = (max(w["max_len"], w.get("long_len", 0)) + growth_tokens + BS - 1) // BS + 1
    return lens, need, nb, perm, mbps, g


class DecodeJob:
    """Pool, block manager and per-step inputs of one rank, on the GPU."""

    def __init__(self, w, rank, growth_tokens, device):
        import morphserve_b200 as mk
        from types import SimpleNamespace
        self.mk = mk
        self.w = w
        self.dev = device
        lens, need, nb, perm, mbps, g = draw_lengths_and_tables(w, rank, growth_tokens)
        B, L, Hq, Hkv = w["B"], w["L"], w["Hq"], w["Hkv"]
        self.model_config = SimpleNamespace(num_layers=L, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D)
        self.engine_config = SimpleNamespace(block_size=BS, max_blocks_per_seq=mbps)
        self.bm = mk.BlockManager("GPU", nb, B, mbps, BS)
        table = torch.full((B, mbps), -1, dtype=torch.int32)
        used = perm[: int(need.sum())]
        pos = 0
        for b in range(B):
            n = int(need[b])
            table[b, :n] = used[pos:pos + n].to(torch.int32)
            pos += n
        self.bm.block_table.copy_(table)
        self.bm.num_seq_allocated_blocks.copy_(need.to(torch.int32))
        free = torch.ones(nb, dtype=torch.bool)
        free[used] = False
        self.bm.is_block_free.copy_(free)
        self.bm.num_free_blocks = type(self.bm.num_free_blocks)(nb - len(used))
        self.lens_host = lens.numpy().astype(np.int64).copy()
        self.seq_ids = torch.arange(B, dtype=torch.int32, device=device)
        self.seq_ids_list = list(range(B))
        self.lens_dev = lens.to(torch.int32).to(device)
        dg = torch.Generator(device=device).manual_seed(1000 * w["cfg"] + rank + 7)
        shape = (nb, L, Hkv, BS, D)
        self.k_cache = torch.empty(shape, dtype=torch.float16, device=device)
        self.v_cache = torch.empty(shape, dtype=torch.float16, device=device)
        for t in (self.k_cache, self.v_cache):       # N(0,1), filled piecewise to bound temporaries
            flat = t.view(-1)
            step = 1 << 28
            for i in range(0, flat.numel(), step):
                flat[i:i + step].normal_(generator=dg)
        self.q = torch.randn((L, B, Hq, D), generator=dg, dtype=torch.float16, device=device)
        self.kn = torch.randn((L, B, Hkv, D), generator=dg, dtype=torch.float16, device=device)
        self.vn = torch.randn((L, B, Hkv, D), generator=dg, dtype=torch.float16, device=device)
        self.o = torch.zeros((L, B, Hq * D), dtype=torch.float16, device=device)
        self.nb = nb
        self._z = torch.zeros(0, dtype=torch.int32, device=device)
        self.cos_table = self.sin_table = None
        if w.get("rope"):
            # the reference's tables (fp32 angles rounded to fp16), long enough for the run
            inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=device, dtype=torch.float32) / D))
            t = torch.arange(mbps * BS + 128, device=device, dtype=torch.float32)
            freqs = torch.outer(t, inv_freq)
            self.cos_table, self.sin_table = torch.cos(freqs).to(torch.float16), torch.sin(freqs).to(torch.float16)
        self.dist = None
        if w.get("head_shard"):
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                self.dist = dist
                n = dist.get_world_size()
                if w.get("push"):
                    # full-width output matrices [layer, sequence, all heads * D] in symmetric memory: every
                    # rank can store into every other rank's copy
                    import torch.distributed._symmetric_memory as symm
                    self.o_full = symm.empty((L, B, w["Hq_global"] * D), dtype=torch.float16, device=device)
                    self.symm = symm.rendezvous(self.o_full, dist.group.WORLD)
                    self.peer_ptrs = [int(x) for x in self.symm.buffer_ptrs]
                    self.layer_bytes = B * w["Hq_global"] * D * 2
                    # one "slice landed" word per source rank, on every rank; rank r writes word r everywhere
                    self.ready = symm.empty((n,), dtype=torch.int32, device=device)
                    self.ready.zero_()
                    self.ready_symm = symm.rendezvous(self.ready, dist.group.WORLD)
                    self.ready_ptrs = [int(x) + 4 * dist.get_rank() for x in self.ready_symm.buffer_ptrs]
                    self.ready_status = torch.zeros((1,), dtype=torch.int32, device=device)
                    self.push_epoch = 0
                    torch.cuda.synchronize()
                    dist.barrier()
                else:
                    # gathered outputs, [rank, sequence, local heads * D]: the consumer reads the permuted view
                    self.o_full = torch.empty((L, n, B, Hq * D), dtype=torch.float16, device=device)

    def infer_state(self, seq_ids, lens_dev, max_len=None):
        B, Hkv = self.w["B"], self.w["Hkv"]
        max_len = max_len or int(self.lens_host.max())
        sbs, nsb = self.mk.infer_state.seq_block_size_heuristic(Hkv, self.lens_host.tolist())
        cos = sin = self._z
        if self.cos_table is not None:      # rows of the newest token's position, gathered once per step
            pos = (lens_dev - 1).long()
            cos, sin = self.cos_table[pos], self.sin_table[pos]
        return self.mk.LlamaInferState(
            batch_size=B, num_tokens=B, seq_ids=seq_ids, softmax_scale=D ** -0.5, num_prefill_seqs=0,
            num_prefill_tokens=0, prefill_seq_start_locs=self._z, prefill_seq_start_locs_with_end=self._z,
            prefill_seq_lens=self._z, max_prefill_len=0, num_decoding_seqs=B, decoding_seq_lens=lens_dev,
            max_decoding_len=max_len, seq_block_size=sbs, num_seq_blocks=nsb, num_blocks_org=self.nb,
            kv_cache_new_block_size=0, org_layer_param_size=0, position_cos=cos, position_sin=sin,
            ignore_kvcache=False)

    def layers(self, st, q, kn, vn, o):
        mk, mc, ec, bt = self.mk, self.model_config, self.engine_config, self.bm.block_table
        if self.dist is not None and self.w.get("push"):
            w = self.w
            for layer in range(w["L"]):
                self.push_epoch += 1
                mk.paged_attention_push(q[layer], self.k_cache, self.v_cache, [], [], bt, mc, ec, st, layer,
                                        [p + layer * self.layer_bytes for p in self.peer_ptrs],
                                        w["Hq_global"] * D, w["head_offset"] * D, k_new=kn[layer], v_new=vn[layer],
                                        ready_ptrs=self.ready_ptrs, epoch=self.push_epoch)
                # every rank's slice of this layer has landed HERE once all words show this epoch (bounded wait;
                # a word that stays behind sets its bit in ready_status); what consumes o_full[layer] queues behind it
                mk.wait_ready(self.ready, self.push_epoch, self.ready_status, timeout_s=1.0)
            # one barrier per step: nobody starts overwriting the matrices of the next step while a peer still reads
            self.symm.barrier()
            return
        for layer in range(self.w["L"]):
            if self.cos_table is not None:
                mk.rotary_embedding_inplace(q[layer], kn[layer], st)
            mk.store_kvcache(kn[layer], vn[layer], self.k_cache, self.v_cache, [], [], bt, mc, ec, st, layer)
            mk.paged_attention(q[layer], self.k_cache, self.v_cache, [], [], bt, mc, ec, st, layer, o[layer])
            if self.dist is not None:      # head sharding: one all-gather of the output shards per layer
                self.dist.all_gather_into_tensor(self.o_full[layer].view(-1, o[layer].shape[-1]), o[layer])

    def step_resident(self):
        """One decode step with every input already in HBM."""
        self.lens_host += 1
        self.lens_dev += 1
        st = self.infer_state(self.seq_ids, self.lens_dev)      # host work first: the allocate below synchronises
        self.bm.allocate_blocks_for_seqs(self.seq_ids, self.lens_dev)
        self.layers(st, self.q, self.kn, self.vn, self.o)

    def capture_step(self, max_steps):
        """Capture one resident decode step in a CUDA graph: lengths + 1, the sync-free allocate, the plan and
        all layers.  Everything the step reads lives at fixed device addresses, so a replay IS the next step.
        `max_steps` bounds how far the contexts may grow (it sizes the plan's table window)."""
        from morphserve_b200.worker.kernels._common import attn_workspace
        w = self.w
        self.bm.prepare_nosync(w["B"])
        self.graph_max_len = min(int(self.lens_host.max()) + max_steps, self.bm.block_table.shape[1] * BS)
        dev = self.dev.index or 0
        max_blocks = min((self.graph_max_len + BS - 1) // BS, self.bm.block_table.shape[1])
        # the attention scratch belongs to the stream the launches run on: allocate it for the capture stream, before
        # the capture
        self.capture_stream = torch.cuda.Stream(self.dev)
        cs = self.capture_stream.cuda_stream
        ws = attn_workspace(dev, w["B"], w["Hq"], w["Hkv"], D, max_blocks, cs)
        self.graph_ws_ptr = ws.tensor.data_ptr()
        torch.cuda.synchronize()
        from morphserve_b200 import _lib
        calls0 = sum(_lib.CALLS.values())
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self.capture_stream,
                              capture_error_mode="thread_local"):   # other threads (NCCL) stay free
            self.lens_dev += 1
            st = self.infer_state(self.seq_ids, self.lens_dev, max_len=self.graph_max_len)
            self.bm.allocate_blocks_for_seqs_nosync(self.seq_ids, self.lens_dev)
            self.layers(st, self.q, self.kn, self.vn, self.o)
        self.graph_launches = sum(_lib.CALLS.values()) - calls0      # library kernels per replay
        self.graph_generation = self.bm.resize_generation
        assert attn_workspace(dev, w["B"], w["Hq"], w["Hkv"], D, max_blocks, cs).tensor.data_ptr() == self.graph_ws_ptr

    def step_graph(self):
        """One decode step = one replay of the captured graph."""
        self.lens_host += 1
        assert int(self.lens_host.max()) <= self.graph_max_len, "captured step outgrown: capture again"
        # an elastic expand / release moves the free bitmap and changes the pool's segments: the graph holds the
        # old addresses and must be captured again
        assert self.bm.resize_generation == self.graph_generation, "pool resized since the capture: capture again"
        self.graph.replay()
        self.bm.nosync_replayed()

    def make_host_buffers(self):
        # per layer one contiguous host record [q | k | v] and its device twin: one copy per layer brings all three
        L, B, Hq, Hkv = self.w["L"], self.w["B"], self.w["Hq"], self.w["Hkv"]
        nq, nk = B * Hq * D, B * Hkv * D
        self.hqkv = torch.empty((L, nq + 2 * nk), dtype=torch.float16).pin_memory()
        self.hqkv[:, :nq].copy_(self.q.view(L, nq))
        self.hqkv[:, nq:nq + nk].copy_(self.kn.view(L, nk))
        self.hqkv[:, nq + nk:].copy_(self.vn.view(L, nk))
        self.dqkv = torch.empty((L, nq + 2 * nk), dtype=torch.float16, device=self.dev)
        self.dq = [self.dqkv[l, :nq].view(B, Hq, D) for l in range(L)]
        self.dk = [self.dqkv[l, nq:nq + nk].view(B, Hkv, D) for l in range(L)]
        self.dv = [self.dqkv[l, nq + nk:].view(B, Hkv, D) for l in range(L)]
        self.ho = torch.empty(self.o.shape, dtype=torch.float16).pin_memory()
        self.h_meta = torch.empty((2, self.w["B"]), dtype=torch.int32).pin_memory()
        self.d_meta = torch.empty((2, self.w["B"]), dtype=torch.int32, device=self.dev)
        self.s_in, self.s_out = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        self.ev_in = [torch.cuda.Event() for _ in range(L)]
        self.ev_out = [torch.cuda.Event() for _ in range(L)]
        return self.hqkv.nbytes + 8 * self.w["B"], self.ho.nbytes

    def _stage_metadata(self):
        """Sequence ids and lengths of the coming step: Python lists (as the reference's LlamaModel.forward
        holds them) -> one pinned staging buffer."""
        self.lens_host += 1
        meta = self.h_meta.numpy()              # a view of the pinned buffer
        meta[0] = self.seq_ids_list
        meta[1] = self.lens_host

    def _enqueue_host_step(self, main, max_len=None):
        """Everything a step with host-side data puts on the GPU's queues, nothing that waits for it: the
        metadata copy, the sync-free allocate, and per layer the q/k/v copies from pinned memory (side stream, one
        layer ahead), rotary/append/attention, and the copy of the layer's output back to pinned memory (second
        side stream)."""
        self.d_meta.copy_(self.h_meta, non_blocking=True)
        seq_ids, lens = self.d_meta[0], self.d_meta[1]
        self.lens_dev = lens
        L = self.w["L"]

        def copy_in(layer):
            with torch.cuda.stream(self.s_in):
                self.dqkv[layer].copy_(self.hqkv[layer], non_blocking=True)
                self.ev_in[layer].record(self.s_in)

        copy_in(0)
        self.bm.allocate_blocks_for_seqs_nosync(seq_ids, lens)      # no host round trip: the layers queue up behind it
        st = self.infer_state(seq_ids, lens, max_len=max_len)
        mk, mc, ec, bt = self.mk, self.model_config, self.engine_config, self.bm.block_table
        for layer in range(L):
            if layer + 1 < L:
                copy_in(layer + 1)                   # next layer's inputs travel while this layer computes
            main.wait_event(self.ev_in[layer])
            if self.cos_table is not None:
                mk.rotary_embedding_inplace(self.dq[layer], self.dk[layer], st)
            mk.store_kvcache(self.dk[layer], self.dv[layer], self.k_cache, self.v_cache, [], [], bt, mc, ec, st, layer)
            mk.paged_attention(self.dq[layer], self.k_cache, self.v_cache, [], [], bt, mc, ec, st, layer,
                               self.o[layer])
            self.ev_out[layer].record(main)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_out[layer])
                self.ho[layer].copy_(self.o[layer], non_blocking=True)
        self.bm.readback_counters_async()       # the allocation record travels to pinned memory with the step

    def step_host(self):
        """One step as a caller with host data makes it; it ends when the last output byte is on the host and
        the host has the allocation result."""
        main = torch.cuda.current_stream()
        self._stage_metadata()
        self._enqueue_host_step(main)
        self.s_out.synchronize()
        main.synchronize()
        _ = self.bm.num_free_blocks     # folds the device-side allocation record into the host counters

    def capture_step_host(self, max_steps):
        """The host-data step as ONE CUDA graph: copy nodes for the metadata, every layer's inputs and outputs
        (pinned buffers at fixed addresses) on two forked branches, the kernels on the main branch."""
        from morphserve_b200.worker.kernels._common import attn_workspace
        w = self.w
        self.bm.prepare_nosync(w["B"])
        self.graph_max_len = min(int(self.lens_host.max()) + max_steps, self.bm.block_table.shape[1] * BS)
        max_blocks = min((self.graph_max_len + BS - 1) // BS, self.bm.block_table.shape[1])
        self.capture_stream_host = torch.cuda.Stream(self.dev)
        attn_workspace(self.dev.index or 0, w["B"], w["Hq"], w["Hkv"], D, max_blocks,
                       self.capture_stream_host.cuda_stream)                              # allocated before the capture
        torch.cuda.synchronize()
        self.graph_host = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_host, stream=self.capture_stream_host, capture_error_mode="thread_local"):
            main = torch.cuda.current_stream()
            self.s_in.wait_stream(main)             # fork: the copy streams join the capture
            self.s_out.wait_stream(main)
            self._enqueue_host_step(main, max_len=self.graph_max_len)
            main.wait_stream(self.s_in)             # join
            main.wait_stream(self.s_out)
        self.graph_generation = self.bm.resize_generation

    def step_host_graph(self):
        """The host-data step as one graph launch: stage the metadata, replay, wait for the outputs."""
        self._stage_metadata()
        assert int(self.lens_host.max()) <= self.graph_max_len, "captured step outgrown: capture again"
        assert self.bm.resize_generation == self.graph_generation, "pool resized since the capture: capture again"
        self.graph_host.replay()
        torch.cuda.current_stream().synchronize()
        self.bm.nosync_replayed(with_readback=True)
        _ = self.bm.num_free_blocks

    def kv_bytes_per_layer(self):
        return 2 * 2 * self.w["Hkv"] * D * int(self.lens_host.sum())

    def snapshot(self):
        """Lengths and block-manager state, so that every timed block starts from the same contexts."""
        torch.cuda.synchronize()
        bm = self.bm
        return dict(lens_host=self.lens_host.copy(), lens_dev=self.lens_dev.clone(), table=bm.block_table.clone(),
                    counts=bm.num_seq_allocated_blocks.clone(), free=bm.is_block_free.clone(),
                    n_free=int(bm.num_free_blocks))

    def restore(self, snap):
        """Back to a snapshot, in place: every tensor keeps its address, so captured graphs stay valid."""
        torch.cuda.synchronize()
        bm = self.bm
        _ = bm.num_free_blocks                  # folds pending sync-free allocations in before the reset
        self.lens_host[:] = snap["lens_host"]
        self.lens_dev.copy_(snap["lens_dev"])
        bm.block_table.copy_(snap["table"])
        bm.num_seq_allocated_blocks.copy_(snap["counts"])
        bm.is_block_free.copy_(snap["free"])
        bm.num_free_blocks = snap["n_free"]
        torch.cuda.synchronize()


# ----------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of the GPUs in use: a separate read-only
    `nvidia-smi --query-gpu ... -lms` process, so that sampling does not compete with the launching
    thread.  It is started before the warm-up (the tool needs up to a few seconds to come up, longer
    with eight GPUs) and its time-stamped samples are cut to the timed region afterwards; if the
    region was too short to hold one, the samples of the warm-up (same load) are reported and marked."""

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, indices):
        self.indices = set(indices)
        self.proc = None
        self.text = ""
        self.t_begin = self.t_end = None

    def start(self):
        if self.indices and self.proc is None:
            import subprocess
            try:
                self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}",
                                              "--format=csv,noheader,nounits", "-lms", "25"],
                                             stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            except Exception:
                self.proc = None
        return self

    def __enter__(self):            # the timed region
        self.start()
        self.t_begin = time.time()
        return self

    def __exit__(self, *a):
        self.t_end = time.time()
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.text, _ = self.proc.communicate(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        import datetime
        rows = []
        for ln in self.text.splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9 or not f[1].isdigit() or int(f[1]) not in self.indices:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[2]), float(f[3]), float(f[4]), f[5:9]))
            except ValueError:
                continue
        inside = [r for r in rows if self.t_begin is not None and self.t_begin <= r[0] <= self.t_end]
        window = "timed region"
        if not inside and rows:     # region shorter than the tool's period or start-up: warm-up samples, same load
            inside = [r for r in rows if r[0] <= (self.t_end or r[0])][-8 * max(1, len(self.indices)):]
            window = "warm-up before the timed region (region too short for a sample)"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        reasons = set()
        for r in inside:
            for nm, val in zip(self.NAMES, r[4]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": inside[-1][2],
                "reasons": sorted(reasons), "samples": len(inside), "power_w_max": max(r[3] for r in inside),
                "window": window}


# ----------------------------------------------------------------------------
# CPU arm: the reference's PyTorch paged-attention path on the host cores
# ----------------------------------------------------------------------------
def cpu_reference_sample(w, steps, warmup, layers_sampled=2, seqs_sampled=None):
    """Times the live restatement of the reference's PyTorch loop (plus the
    indexed-assignment append) on a bounded sample: `seqs_sampled` sequences of
    the workload's length distribution x `layers_sampled` layers per step, and
    scales to the full step (B sequences x L layers).  Returns tokens/s."""
    from oracle import kv_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    B = seqs_sampled or min(w["B"], 64)
    Ls = min(layers_sampled, w["L"])
    g = torch.Generator().manual_seed(1000 * w["cfg"])
    lens = torch.randint(1, w["max_len"] + 1, (w["B"],), generator=g)[:B]
    need = (lens + BS - 1) // BS
    nb = int(need.sum()) + B
    perm = torch.randperm(nb, generator=g)
    mbps = int(need.max()) + 2
    table = torch.full((B, mbps), -1, dtype=torch.int32)
    pos = 0
    for b in range(B):
        table[b, :int(need[b])] = perm[pos:pos + int(need[b])].to(torch.int32)
        pos += int(need[b])
    k_pool = torch.randn((nb, Ls, w["Hkv"], BS, D), generator=g).to(torch.float16)
    v_pool = torch.randn((nb, Ls, w["Hkv"], BS, D), generator=g).to(torch.float16)
    q = torch.randn((Ls, B, w["Hq"], D), generator=g).to(torch.float16)
    kn = torch.randn((Ls, B, w["Hkv"], D), generator=g).to(torch.float16)
    vn = torch.randn((Ls, B, w["Hkv"], D), generator=g).to(torch.float16)
    o = torch.empty((B, w["Hq"] * D), dtype=torch.float16)
    seq_ids = list(range(B))
    lens_l = [int(x) for x in lens]
    kp, vp = [k_pool.numpy()], [v_pool.numpy()]

    def one_step():
        for layer in range(Ls):
            O.store_kvcache_decode(kn[layer].numpy(), vn[layer].numpy(), kp, vp, table.numpy(), seq_ids, lens_l,
                                   layer, nb, 1)
            O.paged_attention_torch_loop(q[layer], [k_pool], [v_pool], table, seq_ids, lens_l, layer, D ** -0.5,
                                         nb, 1, o=o)

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    full_step = dt * (w["B"] / B) * (w["L"] / Ls)
    return w["B"] / full_step, dict(
        cores=os.cpu_count() or 1, kind="port", sample_ms_per_step=dt * 1e3,
        sample=f"{B} of {w['B']} sequences x {Ls} of {w['L']} layers per step, {steps} steps, scaled to the full step")


# ----------------------------------------------------------------------------
# elastic resize: compaction copy + block-table remap
# ----------------------------------------------------------------------------
def resize_bench(w, K, W, device):
    """A pool of nb_org + n_chunks*chunk blocks with 60 % of its blocks live at seeded
    random positions is compacted below the boundary that frees `release` chunks
    (plan + block copies + table remap, one call), K times from the same state."""
    from types import SimpleNamespace

    import morphserve_b200 as mk
    from morphserve_b200.server import memory_utils as MU
    L, Hkv = w["L"], w["Hkv"]
    nb_org, chunk, n_chunks = w["nb_org"], w["chunk"], w["n_chunks"]
    total = nb_org + chunk * n_chunks
    target = nb_org + (n_chunks - w["release"]) * chunk
    g = torch.Generator().manual_seed(1000 * w["cfg"])
    shape = lambda n: (n, L, Hkv, BS, D)                                     # noqa: E731
    model = SimpleNamespace(k_cache=torch.randn(shape(nb_org), dtype=torch.float16, device=device),
                            v_cache=torch.randn(shape(nb_org), dtype=torch.float16, device=device),
                            k_cache_new=[], v_cache_new=[], kv_cache_new_block_size=0,
                            gpu_block_manager=mk.BlockManager("GPU", nb_org, 4096, 128, BS))
    engine = SimpleNamespace(model=model, scheduler=SimpleNamespace(num_gpu_blocks=nb_org))
    for _ in range(n_chunks):
        MU.attach_kvcache_chunk(engine, torch.randn(shape(chunk), dtype=torch.float16, device=device),
                                torch.randn(shape(chunk), dtype=torch.float16, device=device))
    bm = model.gpu_block_manager
    # 60 % live blocks owned by sequences of 48 blocks each, positions from a seeded permutation
    n_live = int(0.6 * total)
    perm = torch.randperm(total, generator=g)[:n_live]
    per_seq = 48
    n_seq = n_live // per_seq
    table = torch.full((4096, 128), -1, dtype=torch.int32)
    table[:n_seq, :per_seq] = perm[: n_seq * per_seq].view(n_seq, per_seq).to(torch.int32)
    counts = torch.zeros(4096, dtype=torch.int32)
    counts[:n_seq] = per_seq
    free = torch.ones(total, dtype=torch.bool)
    free[perm[: n_seq * per_seq]] = False
    state = (table.to(device), counts.to(device), free.to(device))
    block_bytes = 2 * L * Hkv * BS * D * 2
    times, moved = [], 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for it in range(W + K):
        bm.block_table.copy_(state[0])
        bm.num_seq_allocated_blocks.copy_(state[1])
        bm.is_block_free = state[2].clone()
        torch.cuda.synchronize()
        e0.record()
        moved = MU.compact_kvcache(engine, target)
        e1.record()
        torch.cuda.synchronize()
        if it >= W:
            times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    return {"moved_blocks": moved, "ms_per_compaction": ms, "copy_bytes": 2 * moved * block_bytes,
            "copy_gbs_incl_plan_and_remap": 2 * moved * block_bytes / (ms * 1e-3) / 1e9}


# ----------------------------------------------------------------------------
# prefill scatter
# ----------------------------------------------------------------------------
def prefill_bench(w, K, W, device):
    """store_kvcache for a prefill-only batch: every prompt token's K/V row goes to its block."""
    from types import SimpleNamespace

    import morphserve_b200 as mk
    L, Hkv, n_seqs = w["L"], w["Hkv"], w["n_seqs"]
    g = torch.Generator().manual_seed(1000 * w["cfg"] + 5)
    lens = torch.randint(w["max_len"] // 2, w["max_len"] + 1, (n_seqs,), generator=g)
    need = (lens + BS - 1) // BS
    nb = int(need.sum()) * 2
    perm = torch.randperm(nb, generator=g)
    mbps = int(need.max()) + 1
    table = torch.full((n_seqs, mbps), -1, dtype=torch.int32)
    pos = 0
    for i in range(n_seqs):
        table[i, : int(need[i])] = perm[pos:pos + int(need[i])].to(torch.int32)
        pos += int(need[i])
    ntok = int(lens.sum())
    k = torch.randn((ntok, Hkv, D), dtype=torch.float16, device=device)
    v = torch.randn((ntok, Hkv, D), dtype=torch.float16, device=device)
    k_cache = torch.zeros((nb, L, Hkv, BS, D), dtype=torch.float16, device=device)
    v_cache = torch.zeros((nb, L, Hkv, BS, D), dtype=torch.float16, device=device)
    z = torch.zeros(0, dtype=torch.int32, device=device)
    lens_d = lens.to(torch.int32).to(device)
    st = mk.LlamaInferState(
        batch_size=n_seqs, num_tokens=ntok, seq_ids=torch.arange(n_seqs, dtype=torch.int32, device=device),
        softmax_scale=D ** -0.5, num_prefill_seqs=n_seqs, num_prefill_tokens=ntok,
        prefill_seq_start_locs=(torch.cumsum(lens_d, 0, dtype=torch.int32) - lens_d), prefill_seq_start_locs_with_end=z,
        prefill_seq_lens=lens_d, max_prefill_len=int(lens.max()), num_decoding_seqs=0, decoding_seq_lens=z,
        max_decoding_len=0, seq_block_size=512, num_seq_blocks=0, num_blocks_org=nb, kv_cache_new_block_size=0,
        org_layer_param_size=0, position_cos=z, position_sin=z, ignore_kvcache=False)
    mc = SimpleNamespace(num_layers=L, num_q_heads=w["Hq"], num_kv_heads=Hkv, head_dim=D)
    ec = SimpleNamespace(block_size=BS, max_blocks_per_seq=mbps)
    bt = table.to(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(W):
        for layer in range(L):
            mk.store_kvcache(k, v, k_cache, v_cache, [], [], bt, mc, ec, st, layer)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(K):
        for layer in range(L):
            mk.store_kvcache(k, v, k_cache, v_cache, [], [], bt, mc, ec, st, layer)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / (K * L)
    nbytes = 2 * 2 * ntok * Hkv * D * 2          # K and V, read + write
    out = {"tokens": ntok, "ms_per_launch": ms, "bytes_per_launch": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9}
    # rotary embedding of the same prompt tokens (q and k in place), the launch in front of the scatter
    q = torch.randn((ntok, w["Hq"], D), dtype=torch.float16, device=device)
    pos = torch.cat([torch.arange(int(n)) for n in lens]).to(device)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=device, dtype=torch.float32) / D))
    freqs = torch.outer(pos.float(), inv_freq)
    st.position_cos, st.position_sin = torch.cos(freqs).to(torch.float16), torch.sin(freqs).to(torch.float16)
    for _ in range(W):
        mk.rotary_embedding_inplace(q, k, st)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(K * L):
        mk.rotary_embedding_inplace(q, k, st)
    e1.record()
    torch.cuda.synchronize()
    rope_ms = e0.elapsed_time(e1) / (K * L)
    rope_bytes = 2 * ntok * (w["Hq"] + Hkv) * D * 2 + 2 * ntok * (D // 2) * 2   # q, k read + write; cos, sin read
    out["rope"] = {"ms_per_launch": rope_ms, "bytes_per_launch": rope_bytes,
                   "gbs": rope_bytes / (rope_ms * 1e-3) / 1e9}
    return out


# ----------------------------------------------------------------------------
# layer slab replace
# ----------------------------------------------------------------------------
def replace_bench(w, K, W, device):
    """replace_layer_org2quant / replace_layer_quant2org of one layer: a single host->device copy each."""
    from morphserve_b200 import swiftllm_c as c
    slab = torch.zeros(w["org_bytes"], dtype=torch.uint8, device=device)
    org_host = torch.randint(0, 255, (w["org_bytes"],), dtype=torch.uint8).pin_memory()
    q_host = torch.randint(0, 255, (w["quant_bytes"],), dtype=torch.uint8).pin_memory()
    c.register_layer_memory_org_gpu(0, slab.data_ptr(), slab.numel())
    c.register_layer_memory_org_cpu(0, org_host.data_ptr(), org_host.numel())
    c.register_layer_memory_quant(0, q_host.data_ptr(), q_host.numel())
    c.register_layer_memory_tensor_map_org(0, [{"w": dict(offset=0, shape=[w["org_bytes"]], dtype=torch.uint8, size=w["org_bytes"])}])
    c.register_layer_memory_tensor_map_quant(0, [{"w": dict(offset=0, shape=[w["quant_bytes"]], dtype=torch.uint8, size=w["quant_bytes"])}])
    out = {}
    for name, fn, nbytes in (("org2quant", c.replace_layer_org2quant, w["quant_bytes"]),
                             ("quant2org", c.replace_layer_quant2org, w["org_bytes"])):
        for _ in range(W):
            fn(0)
        torch.cuda.synchronize()
        t0 = time.perf_counter()        # the call returns when the copy is complete (it runs on its own stream)
        for _ in range(K):
            fn(0)
        dt = (time.perf_counter() - t0) / K
        out[name] = {"bytes": nbytes, "ms": dt * 1e3, "gbs": nbytes / dt / 1e9}
    assert torch.equal(slab.cpu(), org_host)
    return out


# ----------------------------------------------------------------------------
# block swap
# ----------------------------------------------------------------------------
def swap_bench(w, K, W, device):
    """Swap-out then swap-in of n_swap blocks with fully fragmented (seeded random) ids on both
    sides: the reference-style path (pageable host memory, one cudaMemcpyAsync per run for K and V)
    and the pinned path (one zero-copy kernel per direction, ids on the GPU)."""
    import morphserve_b200 as mk
    L, Hkv, nb, n = w["L"], w["Hkv"], w["nb"], w["n_swap"]
    g = torch.Generator().manual_seed(1000 * w["cfg"] + 3)
    shape = (nb, L, Hkv, BS, D)
    k_cache = torch.randn(shape, dtype=torch.float16, device=device)
    v_cache = torch.randn(shape, dtype=torch.float16, device=device)
    dev_ids = torch.randperm(nb, generator=g)[:n]
    host_ids = torch.randperm(n, generator=g)
    block_bytes = 2 * L * Hkv * BS * D * 2
    out = {"blocks": n, "bytes_per_direction": n * block_bytes}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, pinned in (("pageable_memcpy", False), ("pinned_kernel", True)):
        k_swap = torch.zeros((n, L, Hkv, BS, D), dtype=torch.float16)
        v_swap = torch.zeros((n, L, Hkv, BS, D), dtype=torch.float16)
        if pinned:
            k_swap, v_swap = k_swap.pin_memory(), v_swap.pin_memory()
            d_ids, h_ids = dev_ids.to(device), host_ids.to(device)
        else:
            d_ids, h_ids = dev_ids.tolist(), host_ids.tolist()
        t_out, t_in = [], []
        for it in range(W + K):
            torch.cuda.synchronize()
            e0.record()
            mk.swiftllm_c.swap_blocks(d_ids, h_ids, False, k_cache, v_cache, k_swap, v_swap)
            e1.record()
            torch.cuda.synchronize()
            if it >= W:
                t_out.append(e0.elapsed_time(e1))
            e0.record()
            mk.swiftllm_c.swap_blocks(h_ids, d_ids, True, k_cache, v_cache, k_swap, v_swap)
            e1.record()
            torch.cuda.synchronize()
            if it >= W:
                t_in.append(e0.elapsed_time(e1))
        out[name] = {"swap_out_gbs": n * block_bytes / (statistics.median(t_out) * 1e-3) / 1e9,
                     "swap_in_gbs": n * block_bytes / (statistics.median(t_in) * 1e-3) / 1e9,
                     "swap_out_ms": statistics.median(t_out), "swap_in_ms": statistics.median(t_in)}
        del k_swap, v_swap
    return out


# ----------------------------------------------------------------------------
# one decode workload: resident leg, per-kernel roofline, host-buffer leg
# ----------------------------------------------------------------------------
class RunContext:
    def __init__(self, rank, world, dist, device):
        self.rank, self.world, self.dist, self.device = rank, world, dist, device

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()


def workload_config(name, base, w, world):
    head_shard = bool(base.get("head_shard"))
    return {"workload": name, "baseline_config": base["cfg"], "global_batch": w["B_global"],
            "batch_per_gpu": w["B"], "num_q_heads": base["Hq"], "num_kv_heads": base["Hkv"], "head_dim": D,
            "block_size": BS, "num_layers": w["L"],
            "context_len": f"uniform[{w.get('min_len', 1)},{w['max_len']}] + 1 per step"
            + (f"; first {w['n_long']} at {w['long_len']}" if w.get("n_long") else ""),
            "sharding": ((f"kv heads x{world}, o pushed to all ranks from the attention epilogue" if base.get("push")
                          else f"kv heads x{world} + all-gather of o per layer") if head_shard
                         else f"sequence x{world}"),
            "l2": "inputs_exceed_l2"}


def run_decode(ctx, w, name, K, W, use_graph, min_seconds, clocks=None, with_e2e=False, with_roofline=True,
               job=None, keep_job=False):
    """Times one decode workload on this rank's GPU.  A timed BLOCK is exactly K steps between two CUDA events,
    bracketed by barriers; blocks are repeated from the same starting state (lengths and block tables restored in
    place) until `min_seconds` of blocks have been measured, and the MEDIAN block is reported."""
    from morphserve_b200 import _lib
    rank, world, dist, device = ctx.rank, ctx.world, ctx.dist, ctx.device
    W = max(W, 3)
    if job is None:
        job = DecodeJob(w, rank, growth_tokens=2 * (K + W) + 24, device=device)
    step = job.step_resident
    if use_graph:
        job.step_resident()                       # sizes the workspace, loads the kernels
        job.capture_step(max_steps=K + W + 8)
        step = job.step_graph
    for _ in range(W):
        step()
    snap = job.snapshot()
    ctx.barrier()
    blocks, kv_block, launches = [], 0, 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    own_clocks = clocks is None
    if own_clocks:
        clocks = ClockSampler([])
    t_span = time.perf_counter()
    with clocks:
        while True:
            calls0 = dict(_lib.CALLS)
            kv_block = 0
            ctx.barrier()
            e0.record()
            for _ in range(K):
                step()
                kv_block += job.kv_bytes_per_layer() * w["L"]
            e1.record()
            ctx.barrier()
            launches = sum(v - calls0.get(k, 0) for k, v in _lib.CALLS.items())
            blocks.append(max_over_ranks(e0.elapsed_time(e1), dist, device))
            # every rank takes the same decision: the times above are already the maximum over ranks
            if sum(blocks) >= min_seconds * 1e3 or len(blocks) >= 200:
                break
            job.restore(snap)
    timed_seconds = time.perf_counter() - t_span
    if use_graph:
        launches += K * job.graph_launches          # replays launch the captured kernels without library calls
    ms_block = statistics.median(blocks)
    out = {"value": w["tokens_per_step"] * K / (ms_block * 1e-3), "ms_per_step": ms_block / K, "repeats": len(blocks),
           "timed_seconds": timed_seconds, "ms_per_step_min": min(blocks) / K, "ms_per_step_max": max(blocks) / K,
           "kv_gbs_whole_step": world * kv_block / (ms_block * 1e-3) / 1e9, "launches": launches}
    cs = clocks.summary() if not own_clocks else None
    out["clocks"] = cs
    out["ms_x_mhz"] = (ms_block / K) * cs["sm_mhz"] if cs and cs.get("sm_mhz") else None

    if with_roofline:
        # ---- per-kernel timing for the roofline (attention only, append only) -----
        job.restore(snap)
        st = job.infer_state(job.seq_ids, job.lens_dev)
        mk, mc, ec, bt = job.mk, job.model_config, job.engine_config, job.bm.block_table
        reps = max(3, min(10, K))
        for layer in range(w["L"]):
            mk.paged_attention(job.q[layer], job.k_cache, job.v_cache, [], [], bt, mc, ec, st, layer, job.o[layer])
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # at least 32 launches back to back (layers in turn), as one graph so that no launch waits for Python and
        # the cost of starting a replay is spread thin even for the 2- and 4-layer workloads
        rounds = max(1, -(-32 // w["L"]))
        if use_graph:
            attn_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(attn_graph, capture_error_mode="thread_local"):
                for _ in range(rounds):
                    for layer in range(w["L"]):
                        mk.paged_attention(job.q[layer], job.k_cache, job.v_cache, [], [], bt, mc, ec, st, layer,
                                           job.o[layer])
            attn_graph.replay()
            torch.cuda.synchronize()
        a0.record()
        for _ in range(reps):
            if use_graph:
                attn_graph.replay()
                continue
            for _ in range(rounds):
                for layer in range(w["L"]):
                    mk.paged_attention(job.q[layer], job.k_cache, job.v_cache, [], [], bt, mc, ec, st, layer,
                                       job.o[layer])
        a1.record()
        torch.cuda.synchronize()
        attn_ms = a0.elapsed_time(a1) / (reps * rounds * w["L"])
        was_fused = mk.kvcache_mgmt.FUSE_DECODE_APPEND
        mk.set_fused_decode_append(False)
        a0.record()
        for _ in range(reps):
            for layer in range(w["L"]):
                mk.store_kvcache(job.kn[layer], job.vn[layer], job.k_cache, job.v_cache, [], [], bt, mc, ec, st, layer)
        a1.record()
        torch.cuda.synchronize()
        mk.set_fused_decode_append(was_fused)
        append_ms = a0.elapsed_time(a1) / (reps * w["L"])
        rope_ms = None
        if w.get("rope"):       # the stand-alone rotary kernel on one layer's decode rows
            was_rope = mk.rotary_emb.FUSE_DECODE_ROPE
            mk.set_fused_decode_rope(False)
            a0.record()
            for _ in range(reps):
                for layer in range(w["L"]):
                    mk.rotary_embedding_inplace(job.q[layer], job.kn[layer], st)
            a1.record()
            torch.cuda.synchronize()
            rope_ms = a0.elapsed_time(a1) / (reps * w["L"])
            mk.set_fused_decode_rope(was_rope)
        peak, peak_kind = measured_peak()
        attn_bytes = job.kv_bytes_per_layer()
        achieved = attn_bytes / (attn_ms * 1e-3) / 1e9
        out["roofline"] = {"kernel": "attn_decode_f16_kernel", "bound": "hbm", "achieved": achieved, "peak": peak,
                           "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                           "traffic": NCU_TRAFFIC_RATIO[name] * attn_bytes if name in NCU_TRAFFIC_RATIO else None,
                           "algorithmic_bytes_per_launch": attn_bytes, "ms_per_launch": attn_ms,
                           "append_ms_per_launch": append_ms, "rope_ms_per_launch": rope_ms}

    # ---- host buffers through the public API ----------------------------------
    if with_e2e:
        job.restore(snap)
        h2d, d2h = job.make_host_buffers()
        host_step = job.step_host
        Ke = max(3, min(K, 20))
        if use_graph:
            job.step_host()
            job.capture_step_host(max_steps=Ke + 8)
            host_step = job.step_host_graph
        for _ in range(3):
            host_step()
        ctx.barrier()
        e0.record()
        for _ in range(Ke):
            host_step()
        e1.record()
        ctx.barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1), dist, device)
        e2e = {"value": w["tokens_per_step"] * Ke / (e2e_ms * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": Ke, "ms_per_step": e2e_ms / Ke}
        # the copies alone, every rank at once, each direction by itself: what the host side can feed
        rates = {}
        for nm, fn, nbytes in (("h2d", lambda: job.dqkv.copy_(job.hqkv, non_blocking=True), h2d),
                               ("d2h", lambda: job.ho.copy_(job.o, non_blocking=True), d2h)):
            fn()
            ctx.barrier()
            e0.record()
            for _ in range(5):
                fn()
            e1.record()
            ctx.barrier()
            mine = nbytes * 5 / (e0.elapsed_time(e1) * 1e-3) / 1e9
            rates[nm] = [-max_over_ranks(-mine, dist, device), max_over_ranks(mine, dist, device)]
        e2e["copy_only_gbs_per_rank_min_max"] = rates
        e2e["in_step_gbs_per_rank"] = {"h2d": h2d / (e2e_ms / Ke * 1e-3) / 1e9, "d2h": d2h / (e2e_ms / Ke * 1e-3) / 1e9}
        h2d_ms, d2h_ms = h2d / rates["h2d"][0] * 1e-6, d2h / rates["d2h"][0] * 1e-6     # slowest rank, each alone
        resident_ms = ms_block / K
        e2e["copy_ms_per_step_slowest_rank"] = {"h2d_alone": h2d_ms, "d2h_alone": d2h_ms,
                                                "if_they_overlap_fully": max(h2d_ms, d2h_ms),
                                                "if_they_do_not_overlap": h2d_ms + d2h_ms}
        if e2e_ms / Ke > 1.15 * resident_ms:
            e2e["e2e_limit"] = (f"host memory: the step takes {e2e_ms / Ke:.2f} ms against {resident_ms:.2f} ms resident; with "
                                f"every rank copying at once the two copies of a step need {max(h2d_ms, d2h_ms):.2f} ms "
                                f"(if the directions overlap fully) to {h2d_ms + d2h_ms:.2f} ms (if they share one "
                                "host-memory path) on the slowest rank")
        else:
            e2e["e2e_limit"] = "the GPU step (copies overlap with it)"
        out["e2e"] = e2e
    if keep_job:
        job.restore(snap)
        out["job"] = job
    return out


def reference_gpu_column(job, steps):
    """The reference's own Triton kernels (store_kvcache + paged_attention, worker/kernels/kvcache_mgmt.py:298-478 and
    paged_attn.py:700-1015), compiled by Triton for this GPU, on the same resident batch: decode tokens/s of L x
    (append + attention) per step - no block allocation, no Python beyond the reference's own wrappers."""
    try:
        from oracle import ref_loader
        if not ref_loader.available():
            return {"unavailable": ref_loader.why_unavailable()}
        ref = ref_loader.load(with_ext=False)
        import dataclasses
        import triton
        w = job.w
        st = job.infer_state(job.seq_ids, job.lens_dev)
        st_ref = ref.LlamaInferState(**{f.name: getattr(st, f.name) for f in dataclasses.fields(ref.LlamaInferState)})
        mc, ec, bt = job.model_config, job.engine_config, job.bm.block_table
        o = torch.empty_like(job.o[0])

        def one_step(attn_only=False):
            # the reference's wrappers print timing reports (whenever a call took long, e.g. while Triton compiles):
            # they belong on stderr here, stdout carries the one JSON line
            with contextlib.redirect_stdout(sys.stderr):
                for layer in range(w["L"]):
                    if not attn_only:
                        ref.store_kvcache(job.kn[layer], job.vn[layer], job.k_cache, job.v_cache, [], [], bt, mc, ec,
                                          st_ref, layer)
                    ref.paged_attention(job.q[layer], job.k_cache, job.v_cache, [], [], bt, mc, ec, st_ref, layer, o)

        one_step()                    # Triton compiles here (one variant per specialised layer number)
        one_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            one_step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        e0.record()
        for _ in range(steps):
            one_step(attn_only=True)
        e1.record()
        torch.cuda.synchronize()
        attn_ms = e0.elapsed_time(e1) / (steps * w["L"])
        nbytes = job.kv_bytes_per_layer()
        return {"kind": "triton-jit of the reference's kernels", "triton": triton.__version__,
                "value": w["B"] / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "steps": steps,
                "attention_ms_per_layer": attn_ms, "attention_kv_gbs": nbytes / (attn_ms * 1e-3) / 1e9,
                "seq_block_size": st.seq_block_size, "num_seq_blocks": st.num_seq_blocks,
                "what": "L x (store_kvcache + paged_attention) on the resident batch, launched from Python"}
    except Exception as e:      # a comparison column must not take the bench line down with it
        return {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}


def headshard_column(world, K, W, layers=8, timeout_s=180):
    """The head-sharded CodeLlama-34B variant at the current world size (BASELINE configs[4]): every rank holds
    Hkv / N kv heads of all 512 * N sequences; the output shards are all-gathered per layer (NCCL), or pushed into
    every rank's full-width matrix from the attention epilogue, each rank then waiting for the others' ready flags.
    `layers` of the model's 48 layers are run (the per-layer cost does not depend on the layer count; this bounds
    memory and time next to the main workload).

    Called by rank 0 only, after the main job has released its memory, while the other ranks wait at a barrier: each
    form runs as its OWN torchrun job (fresh processes, fresh communicators) under a hard time limit, so that trouble
    in this side column - a collective that never completes, say - costs the column and never the main line."""
    import signal
    import subprocess
    out = {"layers_run": layers, "layers_of_model": 48, "how": "separate torchrun job per form, bounded time"}
    if 8 % world != 0:
        return {"unavailable": f"8 kv heads do not divide over {world} ranks"}
    env = {k: v for k, v in os.environ.items()
           if not (k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "ROLE_NAME",
                         "ROLE_WORLD_SIZE", "GROUP_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS")
                   or k.startswith("TORCHELASTIC") or k.startswith("TORCH_NCCL") or k.startswith("PET_"))}
    env["NCCL_NVLS_ENABLE"] = "0"
    port = 29700 + os.getpid() % 200
    for i, name in enumerate(("codellama-34b-gqa-decode-headshard", "codellama-34b-gqa-decode-headshard-push")):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
               "--master-addr", "127.0.0.1", "--master-port", str(port + i), os.path.join(ROOT, "bench.py"),
               "--gpus", str(world), "--workload", name, "--layers", str(layers), "--steps", str(K), "--warmup", str(W),
               "--no-e2e", "--no-cpu", "--no-extras", "--min-seconds", "0"]
        try:
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env,
                                    start_new_session=True)
            try:
                stdout, stderr = proc.communicate(timeout=timeout_s)
            except subprocess.TimeoutExpired:
                os.killpg(proc.pid, signal.SIGKILL)         # the job's own process group, nothing else
                proc.communicate()
                out[name] = {"unavailable": f"no result within {timeout_s} s"}
                continue
            lines = [ln for ln in stdout.splitlines() if ln.startswith('{"metric')]
            if proc.returncode != 0 or not lines:
                why = [ln.strip() for ln in stderr.splitlines() if "Error" in ln or "error" in ln]
                out[name] = {"unavailable": f"exit {proc.returncode}: {why[-1][:200] if why else ''}"}
                continue
            r = json.loads(lines[-1])
            out[name] = {"value": r["value"], "unit": "tokens/s", "ms_per_step": r["ms_per_step"],
                         "ms_per_layer": r["ms_per_step"] / layers,
                         "tokens_per_s_at_48_layers": r["value"] * layers / 48}
        except Exception as e:
            out[name] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    return out


# ----------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="llama3-8b-gqa-decode", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true",
                    help="default workload only: skip the further columns (drop-in defaults, the reference's kernels on "
                         "this GPU, the other workloads, the head-sharded variant)")
    ap.add_argument("--layers", type=int, default=0,
                    help="decode workloads: run this many layers instead of the model's (what the head-sharded column does)")
    ap.add_argument("--min-seconds", type=float, default=2.0,
                    help="repeat the timed block of --steps steps (from the same starting state) until this much time "
                         "has been measured; the median block is reported")
    ap.add_argument("--no-cuda-graph", action="store_true",
                    help="resident leg: launch every call of the step from Python instead of capturing the step "
                         "(sync-free allocate + plan + all layers) in a CUDA graph once and replaying it")
    ap.add_argument("--no-fused-rope", action="store_true",
                    help="workloads with rotary embedding: run it as its own launch per layer")
    ap.add_argument("--no-fused-append", action="store_true",
                    help="launch the decode KV append as its own kernel (the reference's two-call structure) "
                         "instead of fusing it into the attention launch")
    args = ap.parse_args()
    K, W = args.steps, max(args.warmup, 0)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    base = WORKLOADS[args.workload]
    if args.layers > 0 and "L" in base:
        base = dict(base, L=args.layers)
    if base.get("prefill"):
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
        torch.cuda.set_device(local_rank)
        if rank == 0:
            r = prefill_bench(base, max(K, 3), max(W, 3), torch.device("cuda", local_rank))
            peak, peak_kind = measured_peak()
            print(json.dumps({"metric": "prefill_scatter_gbs", "value": r["gbs"], "unit": "GB/s", "n_gpus": 1,
                              "higher_is_better": True, "dtype": "u8", "data": "synthetic",
                              "config": {"workload": args.workload},
                              "roofline": {"kernel": "store_kv_prefill_kernel", "bound": "hbm", "achieved": r["gbs"],
                                           "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                                           "frac": r["gbs"] / peak, "traffic": None}, "prefill": r}))
        return
    if base.get("replace"):
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
        torch.cuda.set_device(local_rank)
        if rank == 0:
            r = replace_bench(base, max(K, 3) if K < 10 else 10, 2, torch.device("cuda", local_rank))
            print(json.dumps({"metric": "layer_upload_gbs", "value": r["quant2org"]["gbs"], "unit": "GB/s",
                              "n_gpus": 1, "higher_is_better": True, "dtype": "u8", "data": "synthetic",
                              "config": {"workload": args.workload}, "replace": r}))
        return
    if base.get("swap"):
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
        torch.cuda.set_device(local_rank)
        if rank == 0:
            r = swap_bench(base, max(K, 3) if K < 10 else 5, 2, torch.device("cuda", local_rank))
            print(json.dumps({"metric": "swap_gbs", "value": r["pinned_kernel"]["swap_out_gbs"], "unit": "GB/s",
                              "n_gpus": 1, "higher_is_better": True, "dtype": "u8", "data": "synthetic",
                              "config": {"workload": args.workload}, "swap": r}))
        return
    if base.get("resize"):
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
        torch.cuda.set_device(local_rank)
        if rank == 0:
            r = resize_bench(base, K, max(W, 3), torch.device("cuda", local_rank))
            peak, peak_kind = measured_peak()
            print(json.dumps({"metric": "compaction_copy_gbs", "value": r["copy_gbs_incl_plan_and_remap"],
                              "unit": "GB/s", "n_gpus": 1, "steps": K, "warmup": max(W, 3),
                              "ms_per_step": r["ms_per_compaction"], "higher_is_better": True, "dtype": "u8",
                              "data": "synthetic", "config": {"workload": args.workload, **{k: v for k, v in base.items()
                                                                                          if k != "resize"}},
                              "roofline": {"kernel": "copy_blocks_kernel", "bound": "hbm",
                                           "achieved": r["copy_gbs_incl_plan_and_remap"], "peak": peak,
                                           "peak_kind": peak_kind, "unit": "GB/s",
                                           "frac": r["copy_gbs_incl_plan_and_remap"] / peak, "traffic": None},
                              "resize": r}))
        return
    w = shard_workload(base, rank, world)
    config = workload_config(args.workload, base, w, world)

    if args.impl == "reference":
        if rank != 0:
            return
        val, info = cpu_reference_sample(base, steps=K, warmup=min(W, 2))
        config.update(host_numa_node=None, decode_append=None, step_launch=None)      # same keys as the other arm
        line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": val, "unit": "tokens/s",
                "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": info.pop("sample_ms_per_step"),
                "ms_per_full_step_estimated": 1e3 * base["B"] / val,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
                "data": "synthetic", "config": config,
                "cpu_baseline": dict(value=val, unit="tokens/s", **info),
                "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    numa_node, cpu_affinity_before = bind_to_gpu_numa_node(local_rank)
    config["host_numa_node"] = numa_node
    dist = None
    if world > 1:
        import torch.distributed as dist
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            del os.environ["NCCL_DEBUG"]        # keeps NCCL's banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=device)
    ctx = RunContext(rank, world, dist, device)

    import morphserve_b200
    morphserve_b200.set_fused_decode_append(not args.no_fused_append)
    config["decode_append"] = "own launch" if args.no_fused_append else "fused into the attention launch"
    if w.get("rope"):
        fused_rope = not (args.no_fused_rope or args.no_fused_append)
        morphserve_b200.set_fused_decode_rope(fused_rope)
        config["rotary_embedding"] = "fused into the attention launch" if fused_rope else "own launch"
    use_graph = not args.no_cuda_graph and not base.get("head_shard")   # the captured step has no collective in it
    config["step_launch"] = "cuda graph replay" if use_graph else "python calls"

    clocks = ClockSampler(list(range(world)) if rank == 0 else []).start()     # comes up during the warm-up
    main_run = run_decode(ctx, w, args.workload, K, W, use_graph, min_seconds=args.min_seconds, clocks=clocks,
                          with_e2e=not args.no_e2e, keep_job=True)
    job = main_run.pop("job")
    default_run = args.workload == "llama3-8b-gqa-decode" and not args.no_extras

    extras = {}
    if default_run:
        # what a worker that calls this package exactly like the reference gets: two launches per layer issued from
        # Python, the allocate that returns the new ids (one host synchronisation per step)
        morphserve_b200.set_fused_decode_append(False)
        extras["dropin_default"] = run_decode(ctx, w, args.workload, min(K, 10), 3, False, min_seconds=0.0, job=job,
                                              with_roofline=False)
        extras["dropin_default"]["what"] = ("store_kvcache + paged_attention as two launches per layer issued from "
                                            "Python, BlockManager.allocate_blocks_for_seqs with its host round trip")
        morphserve_b200.set_fused_decode_append(not args.no_fused_append)
        if world == 1:
            extras["reference_gpu"] = reference_gpu_column(job, steps=3)
    del job
    torch.cuda.empty_cache()

    if cpu_affinity_before is not None:
        os.sched_setaffinity(0, cpu_affinity_before)        # the CPU leg below uses every host core
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v, info = cpu_reference_sample(base, steps=3, warmup=1)
        info.pop("sample_ms_per_step")
        cpu = dict(value=v, unit="tokens/s", **info)

    if default_run and world == 1:
        others = {}
        for name in ("llama2-7b-mha-decode", "codellama-34b-gqa-decode", "small-gqa-decode", "skewed-gqa-decode",
                     "longctx-gqa-decode"):
            ww = shard_workload(WORKLOADS[name], 0, 1)
            r = run_decode(ctx, ww, name, 5, 3, use_graph, min_seconds=0.0)
            others[name] = {"value": r["value"], "unit": "tokens/s", "ms_per_step": r["ms_per_step"],
                            "num_layers": ww["L"], "batch": ww["B"], "roofline": r["roofline"]}
            torch.cuda.empty_cache()
        rz = resize_bench(WORKLOADS["kv-resize"], 3, 3, device)
        peak, peak_kind = measured_peak()
        others["kv-resize"] = {"value": rz["copy_gbs_incl_plan_and_remap"], "unit": "GB/s (read + write)",
                               "ms_per_compaction": rz["ms_per_compaction"], "moved_blocks": rz["moved_blocks"],
                               "copy_bytes": rz["copy_bytes"], "frac_of_peak": rz["copy_gbs_incl_plan_and_remap"] / peak,
                               "peak_kind": peak_kind}
        extras["other_workloads"] = others
        torch.cuda.empty_cache()
    if default_run and world > 1:
        # rank 0 runs the column's own jobs; the others wait on the HOST (a key in the rendezvous store), so that no
        # collective kernel of this job spins on the GPUs the column is measured on
        import datetime
        torch.cuda.synchronize()
        store = dist.distributed_c10d._get_default_store()
        if rank == 0:
            extras["headshard"] = headshard_column(world, K=3, W=2)
            store.set("mkv_headshard_done", "1")
        else:
            store.wait(["mkv_headshard_done"], datetime.timedelta(seconds=600))

    if rank == 0:
        line = {
            "metric": "decode_tokens_per_s", "value": main_run["value"], "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": max(W, 3), "ms_per_step": main_run["ms_per_step"], "repeats": main_run["repeats"],
            "timed_seconds": main_run["timed_seconds"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": config,
            "kv_gbs_whole_step": main_run["kv_gbs_whole_step"], "roofline": main_run["roofline"],
            "cpu_baseline": cpu, "e2e": main_run.get("e2e"), "gpu_launches": main_run["launches"],
            "clocks": main_run["clocks"], "ms_per_step_x_sm_mhz": main_run["ms_x_mhz"], **extras,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
