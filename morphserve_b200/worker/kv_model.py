"""The KV-cache half of the reference's ``LlamaModel`` (worker/model.py): pool and swap-space
set-up (:176-227), sequence swap in / out (:468-540) and freeing (:542-550), with the same
attribute and method names, so that the reference's model class can take them over or delegate.

What differs underneath: the swap space is pinned by default, so that a swap is one zero-copy
kernel per direction and the block ids stay on the GPU (the reference allocates pageable memory,
:196-204, turns the ids into Python lists and issues one ``cudaMemcpyAsync`` pair per run of
consecutive ids, :473-504); the choice between the plain and the elastic copy routine needs no
``torch.max`` round trip (:481), because the segment table covers both.
"""
from __future__ import annotations

import torch

import numpy as np

from .. import swiftllm_c
from .block_manager import BlockManager
from .infer_state import LlamaInferState, seq_block_size_heuristic


class KVCacheModelState:
    def __init__(self, model_config, engine_config, pin_swap: bool = True):
        self.model_config = model_config
        self.engine_config = engine_config
        self.pin_swap = pin_swap
        self.k_cache = self.v_cache = None
        self.k_swap = self.v_swap = None
        self.k_cache_new, self.v_cache_new = [], []     # elastic chunks (worker/model.py:75-76)
        self.org_layer_param_size = 0
        self.kv_cache_new_block_size = 0
        self.block_swap = 0                              # blocks swapped so far (worker/model.py:479)
        self.gpu_block_manager = self.cpu_block_manager = None
        self._cos_cached = self._sin_cached = None
        self._staging = [None, None]                     # pinned int32 buffers for the per-step metadata
        self._staging_done = [None, None]
        self._staging_turn = 0

    @torch.inference_mode()
    def _init_to_get_rotary(self):
        """cos / sin tables, fp32 angles rounded to fp16 (worker/model.py:229-241)."""
        mc = self.model_config
        scaling = getattr(mc, "rope_scaling", 1) or 1
        base = getattr(mc, "rope_theta", 10000.0)
        max_seq_len = getattr(mc, "max_position_embeddings", 4096) * scaling
        inv_freq = 1.0 / (base ** (torch.arange(0, mc.head_dim, 2, device="cuda", dtype=torch.float32) / mc.head_dim))
        t = torch.arange(max_seq_len + 128, device="cuda", dtype=torch.float32) / scaling
        freqs = torch.outer(t, inv_freq)
        self._cos_cached = torch.cos(freqs).to(torch.float16)
        self._sin_cached = torch.sin(freqs).to(torch.float16)

    def _stage(self, n: int):
        """A pinned int32 buffer of at least n entries whose previous upload has finished (two take turns)."""
        i = self._staging_turn = self._staging_turn ^ 1
        if self._staging[i] is None or self._staging[i].shape[0] < n:
            self._staging[i] = torch.empty((max(n, 4096),), dtype=torch.int32).pin_memory()
            self._staging_done[i] = torch.cuda.Event()
        else:
            self._staging_done[i].synchronize()
        return self._staging[i], self._staging_done[i]

    @torch.inference_mode()
    def prepare_step(self, input_ids_list, seq_ids_list, decoding_seq_lens_list, ignore_kvcache: bool = False,
                     sync_free: bool = False) -> LlamaInferState:
        """The part of the reference's ``forward`` that turns its Python lists into the step's metadata and block
        allocation (worker/model.py:318-436): prefill sequences come first in ``input_ids_list``, decoding ones
        after them with one token each.  Returns the LlamaInferState the kernels of this package take.

        Underneath, all integer metadata (sequence ids, lengths, prompt start offsets, token positions) is laid out
        in ONE pinned buffer on the host and uploaded with ONE asynchronous copy; the reference builds six small
        tensors from lists and derives the rest with cumsum / arange / cat kernels.  ``sync_free`` takes the
        allocation path without a host round trip (errors then surface with the next ``num_free_blocks`` read)."""
        mc = self.model_config
        n_dec = len(decoding_seq_lens_list)
        n_pre = len(input_ids_list) - n_dec
        prompt_lens = [len(x) for x in input_ids_list[:n_pre]]
        batch = n_pre + n_dec
        n_pre_tok = sum(prompt_lens)
        n_tok = n_pre_tok + n_dec
        # [ seq_ids | seq_lengths | prompt starts + end | token positions ]
        total = 2 * batch + (n_pre + 1) + n_tok
        host, done = self._stage(total)
        h = host.numpy()
        h[:batch] = seq_ids_list
        h[batch:batch + n_pre] = prompt_lens
        h[batch + n_pre:2 * batch] = decoding_seq_lens_list
        o_start = 2 * batch
        if n_pre:
            h[o_start:o_start + n_pre] = np.cumsum(prompt_lens) - np.asarray(prompt_lens)
        h[o_start + n_pre] = n_tok
        o_pos = o_start + n_pre + 1
        p = o_pos
        for n in prompt_lens:
            h[p:p + n] = np.arange(n, dtype=np.int32)
            p += n
        h[p:p + n_dec] = np.asarray(decoding_seq_lens_list, dtype=np.int32) - 1
        dev = torch.empty((total,), dtype=torch.int32, device="cuda")
        dev.copy_(host[:total], non_blocking=True)
        done.record()
        seq_ids, seq_lengths = dev[:batch], dev[batch:2 * batch]
        starts_with_end = dev[o_start:o_start + n_pre + 1]
        positions = dev[o_pos:o_pos + n_tok]
        if not ignore_kvcache:
            if sync_free:
                self.gpu_block_manager.allocate_blocks_for_seqs_nosync(seq_ids, seq_lengths)
            else:
                self.gpu_block_manager.allocate_blocks_for_seqs(seq_ids, seq_lengths)
        if self._cos_cached is None:
            self._init_to_get_rotary()
        seq_block_size, num_seq_blocks = seq_block_size_heuristic(mc.num_kv_heads, decoding_seq_lens_list)
        return LlamaInferState(
            batch_size=batch, num_tokens=n_tok, seq_ids=seq_ids, softmax_scale=mc.head_dim ** -0.5,
            num_prefill_seqs=n_pre, num_prefill_tokens=n_pre_tok, prefill_seq_start_locs=starts_with_end[:n_pre],
            prefill_seq_start_locs_with_end=starts_with_end, prefill_seq_lens=seq_lengths[:n_pre],
            max_prefill_len=max(prompt_lens, default=0), num_decoding_seqs=n_dec, decoding_seq_lens=seq_lengths[n_pre:],
            max_decoding_len=max(decoding_seq_lens_list, default=0), seq_block_size=seq_block_size,
            num_seq_blocks=num_seq_blocks,
            num_blocks_org=self.gpu_block_manager.num_blocks_org if self.gpu_block_manager else None,
            kv_cache_new_block_size=self.kv_cache_new_block_size, org_layer_param_size=self.org_layer_param_size,
            position_cos=self._cos_cached[positions], position_sin=self._sin_cached[positions],
            ignore_kvcache=ignore_kvcache)

    @torch.inference_mode()
    def init_kvcache_and_swap(self, num_blocks: int):
        """worker/model.py:176-227: zero-filled pools ``[blocks, L, Hkv, bs, D]`` fp16 on the GPU and in host
        memory, one BlockManager for each (both keep their tables on the GPU), KV geometry registered with the
        native layer."""
        mc, ec = self.model_config, self.engine_config
        self.num_blocks = num_blocks
        shape = (num_blocks, mc.num_layers, mc.num_kv_heads, ec.block_size, mc.head_dim)
        # zeros, not empty: stale NaN bit patterns in never-written slots would poison masked lanes (:187-188)
        self.k_cache = torch.zeros(shape, dtype=torch.float16, device="cuda")
        self.v_cache = torch.zeros(shape, dtype=torch.float16, device="cuda")
        swap_shape = (ec.num_cpu_blocks,) + shape[1:]
        self.k_swap = torch.zeros(swap_shape, dtype=torch.float16, device="cpu")
        self.v_swap = torch.zeros(swap_shape, dtype=torch.float16, device="cpu")
        if self.pin_swap:
            self.k_swap, self.v_swap = self.k_swap.pin_memory(), self.v_swap.pin_memory()
        self.gpu_block_manager = BlockManager("GPU", num_blocks, ec.max_seqs_in_block_table, ec.max_blocks_per_seq,
                                              ec.block_size)
        self.cpu_block_manager = BlockManager("CPU", ec.num_cpu_blocks, ec.max_seqs_in_block_table,
                                              ec.max_blocks_per_seq, ec.block_size)
        swiftllm_c.register_kv_cache_info(mc.num_layers, mc.num_kv_heads, ec.block_size, mc.head_dim)

    def _swap(self, seq_ids_list, is_swap_in: bool):
        """worker/model.py:468-505: the sequences' blocks leave one manager (gathered and freed) and are
        allocated in the other, then the block contents follow."""
        src_bm = self.cpu_block_manager if is_swap_in else self.gpu_block_manager
        dst_bm = self.gpu_block_manager if is_swap_in else self.cpu_block_manager
        seq_ids = torch.tensor(seq_ids_list, dtype=torch.int32, device="cuda")
        seq_lengths = src_bm.get_num_allocated_blocks(seq_ids) * self.engine_config.block_size
        src_block_ids = src_bm.gather_allocated_blocks_and_free(seq_ids)
        dst_block_ids = dst_bm.allocate_blocks_for_seqs(seq_ids, seq_lengths)
        self.block_swap += len(src_block_ids)
        if len(src_block_ids) == 0:
            return
        if not self.k_cache_new:
            swiftllm_c.swap_blocks(src_block_ids, dst_block_ids, is_swap_in, self.k_cache, self.v_cache,
                                   self.k_swap, self.v_swap)
        else:
            swiftllm_c.swap_blocks_chunk_list(
                src_block_ids, dst_block_ids, is_swap_in, self.gpu_block_manager.num_blocks_org,
                self.kv_cache_new_block_size, self.k_cache, self.v_cache, self.k_swap, self.v_swap,
                self.k_cache_new, self.v_cache_new)

    @torch.inference_mode()
    def swap_seqs_nosync(self, seq_ids: torch.Tensor, is_swap_in: bool) -> torch.Tensor:
        """The same move with no host round trip (pinned swap space only): the source manager's ids stay on the
        GPU (``gather_allocated_blocks_and_free_nosync``), the destination manager allocates with its one-launch
        kernel, and one copy kernel moves the blocks, skipping the unused tail of both id lists.  ``seq_ids`` is an
        int32 CUDA tensor.  Returns the device-side block count (int64 [1]); it is also added to
        ``block_swap_device``.  If the destination has too few free blocks nothing is copied - the id list the copy
        reads is cleared beforehand and the allocation then leaves it untouched - and the next look at the
        destination's ``num_free_blocks`` raises, as for every sync-free allocation."""
        if not (self.k_swap.is_pinned() and self.v_swap.is_pinned()):
            raise RuntimeError("swap_seqs_nosync needs a pinned swap space (pin_swap=True)")
        assert seq_ids.dtype == torch.int32 and seq_ids.is_cuda and seq_ids.is_contiguous()
        src_bm = self.cpu_block_manager if is_swap_in else self.gpu_block_manager
        dst_bm = self.gpu_block_manager if is_swap_in else self.cpu_block_manager
        seq_lengths = (src_bm.get_num_allocated_blocks(seq_ids.long()) * self.engine_config.block_size).to(torch.int32)
        src_ids, count = src_bm.gather_allocated_blocks_and_free_nosync(seq_ids)
        n = min(src_ids.shape[0], dst_bm.is_block_free.shape[0])
        dst_bm.prepare_nosync(seq_ids.shape[0])
        dst_bm._alloc_ids[:n].fill_(-1)
        dst_bm.allocate_blocks_for_seqs_nosync(seq_ids, seq_lengths)
        dst_ids = dst_bm._alloc_ids[:n]
        if getattr(self, "block_swap_device", None) is None:
            self.block_swap_device = torch.zeros((1,), dtype=torch.int64, device=seq_ids.device)
        self.block_swap_device += count
        swiftllm_c.swap_blocks_chunk_list(
            src_ids[:n], dst_ids, is_swap_in, self.gpu_block_manager.num_blocks_org, self.kv_cache_new_block_size,
            self.k_cache, self.v_cache, self.k_swap, self.v_swap, self.k_cache_new, self.v_cache_new)
        return count

    @torch.inference_mode()
    def swap_in_seqs(self, seq_ids_list):
        """Move the blocks of the given sequences from the host swap space to the GPU pool."""
        self._swap(seq_ids_list, True)

    @torch.inference_mode()
    def swap_out_seqs(self, seq_ids_list):
        """Move the blocks of the given sequences from the GPU pool to the host swap space."""
        self._swap(seq_ids_list, False)

    @torch.inference_mode()
    def free_seqs_resources(self, seq_ids_list):
        """worker/model.py:542-550."""
        seq_ids = torch.tensor(seq_ids_list, dtype=torch.int32, device="cuda")
        self.gpu_block_manager.free_blocks_for_seqs(seq_ids)
        self.cpu_block_manager.free_blocks_for_seqs(seq_ids)
