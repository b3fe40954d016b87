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

from .. import swiftllm_c
from .block_manager import BlockManager


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
