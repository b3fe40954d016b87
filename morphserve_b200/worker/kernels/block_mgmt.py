"""Block-table kernels: drop-ins for the three functions of the reference's
``swiftllm.worker.kernels.block_mgmt`` (worker/kernels/block_mgmt.py:26-46,
:66-80, :106-125).  Integer work, exact.
"""
from __future__ import annotations

import torch

from ..._lib import check, lib
from ._common import device_and_stream, require_cuda


def set_block_table_and_num_seq_alloc_blocks(
    num_seq_allocated_blocks: torch.Tensor,     # [max_seqs_in_block_table] int32
    block_table: torch.Tensor,                  # [max_seqs_in_block_table, max_blocks_per_seq] int32
    candidate_blocks: torch.Tensor,             # [sum(block_needed)]
    seq_ids: torch.Tensor,                      # [batch_size] int32
    block_needed: torch.Tensor,                 # [batch_size] int32
):
    """For the i-th sequence (id s): append candidate_blocks[cumsum[i-1]:cumsum[i]]
    to row s starting at column num_seq_allocated_blocks[s], and bump the count."""
    require_cuda(block_table, "block_table")
    dev, stream = device_and_stream(block_table)
    cand = candidate_blocks if candidate_blocks.dtype == torch.int64 else candidate_blocks.to(torch.int64)
    need = block_needed if block_needed.dtype == torch.int32 else block_needed.to(torch.int32)
    check(lib.mkv_block_table_set(dev, stream, num_seq_allocated_blocks.data_ptr(),
                                  num_seq_allocated_blocks.shape[0], block_table.data_ptr(),
                                  block_table.stride(0), cand.contiguous().data_ptr(), seq_ids.data_ptr(),
                                  need.contiguous().data_ptr(), seq_ids.shape[0]), "mkv_block_table_set")


def unset_block_table_and_num_seq_alloc_blocks(
    num_seq_allocated_blocks: torch.Tensor,
    block_table: torch.Tensor,
    seq_ids: torch.Tensor,
    is_block_free: torch.Tensor,                # [num_blocks] bool
):
    """Mark the blocks of the given sequences free and zero their counts (rows keep their ids)."""
    require_cuda(block_table, "block_table")
    dev, stream = device_and_stream(block_table)
    check(lib.mkv_block_table_unset(dev, stream, num_seq_allocated_blocks.data_ptr(),
                                    num_seq_allocated_blocks.shape[0], block_table.data_ptr(),
                                    block_table.stride(0), seq_ids.data_ptr(), seq_ids.shape[0],
                                    is_block_free.data_ptr(), is_block_free.shape[0], None, 0, None, 0),
          "mkv_block_table_unset")


def gather_allocated_blocks_and_unset(
    num_seq_allocated_blocks: torch.Tensor,
    block_table: torch.Tensor,
    seq_ids: torch.Tensor,
    is_block_free: torch.Tensor,
) -> torch.Tensor:
    """Same, and return the freed ids (int32) in batch order."""
    require_cuda(block_table, "block_table")
    dev, stream = device_and_stream(block_table)
    total = torch.empty(1, dtype=torch.int64, device=block_table.device)
    check(lib.mkv_block_table_count(dev, stream, num_seq_allocated_blocks.data_ptr(),
                                    num_seq_allocated_blocks.shape[0], seq_ids.data_ptr(),
                                    seq_ids.shape[0], total.data_ptr()), "mkv_block_table_count")
    n = int(total.item())       # the result's size is data dependent: one sync, as in the reference (:115-116)
    gathered = torch.empty((n,), dtype=torch.int32, device=block_table.device)
    check(lib.mkv_block_table_unset(dev, stream, num_seq_allocated_blocks.data_ptr(),
                                    num_seq_allocated_blocks.shape[0], block_table.data_ptr(),
                                    block_table.stride(0), seq_ids.data_ptr(), seq_ids.shape[0],
                                    is_block_free.data_ptr(), is_block_free.shape[0],
                                    gathered.data_ptr(), n, None, 0), "mkv_block_table_unset")
    return gathered
