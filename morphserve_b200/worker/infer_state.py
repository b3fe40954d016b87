"""Per-step metadata consumed by the KV-cache kernels.

Field-for-field the reference's dataclass (worker/infer_state.py:4-33); the
kernels read ``seq_ids``, ``softmax_scale``, the prefill/decode counts and
lengths, and the three elastic fields.  Any object with these attributes works.
"""
import dataclasses

import torch


@dataclasses.dataclass
class LlamaInferState:
    batch_size: int
    num_tokens: int

    seq_ids: torch.Tensor           # [batch_size]
    softmax_scale: float            # 1/sqrt(head_dim)

    num_prefill_seqs: int
    num_prefill_tokens: int
    prefill_seq_start_locs: torch.Tensor            # [num_prefill_seqs]
    prefill_seq_start_locs_with_end: torch.Tensor   # [num_prefill_seqs+1]
    prefill_seq_lens: torch.Tensor                  # [num_prefill_seqs]
    max_prefill_len: int

    num_decoding_seqs: int
    decoding_seq_lens: torch.Tensor  # [num_decoding_seqs], includes the token being generated
    max_decoding_len: int

    seq_block_size: int              # the reference's split size; the CUDA path plans its own
    num_seq_blocks: int

    num_blocks_org: int              # blocks of the original pool
    kv_cache_new_block_size: int     # blocks per elastic chunk
    org_layer_param_size: int        # elements of one fp16 layer slab (address rule of the reference)

    position_cos: torch.Tensor
    position_sin: torch.Tensor

    ignore_kvcache: bool


def seq_block_size_heuristic(num_kv_heads: int, decoding_seq_lens_list):
    """The reference's split choice (worker/model.py:397-402,426), kept so that
    callers that build an infer state get the same two fields."""
    seq_block_size = 512
    total = sum(decoding_seq_lens_list)
    max_len = max(decoding_seq_lens_list) if decoding_seq_lens_list else 0
    while (num_kv_heads * (total / seq_block_size) < 1024 and seq_block_size // 2 >= 64
           and max_len / (seq_block_size // 2) <= 128):
        seq_block_size //= 2
    return seq_block_size, (max_len + seq_block_size - 1) // seq_block_size
