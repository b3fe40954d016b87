"""GPU-resident block table and free-block bitmap: drop-in for the reference's
``swiftllm.worker.block_manager.BlockManager`` (worker/block_manager.py:5-137).

Same constructor, methods, exceptions and public mutable attributes
(``num_blocks``, ``num_free_blocks``, ``num_blocks_org``, ``block_size``,
``num_seq_allocated_blocks``, ``block_table``, ``is_block_free`` - the elastic
resize code replaces ``is_block_free`` and bumps the counters from outside).
Allocation is first-fit in ascending block id like the reference's
``torch.nonzero(is_block_free)[:n]`` (:75), done by one CUDA kernel without the
nonzero pass; an allocate is one launch and one host synchronisation (the size
of the returned tensor is data dependent) instead of the reference's three.

``allocate_blocks_for_seqs_nosync`` is the same allocation as one launch with
no host round trip at all (nothing is returned; errors and the free-block
count reach the host the next time ``num_free_blocks`` is read), so that a
whole decode step can be enqueued ahead of the GPU or captured in a CUDA graph.
"""
from __future__ import annotations

import torch

from .._lib import check, lib
from .kernels._common import device_and_stream
from .kernels.block_mgmt import gather_allocated_blocks_and_unset


class BlockCount(int):
    """An int that also answers ``.item()``: the reference's ``num_free_blocks``
    turns into a 0-d tensor after the first free (worker/block_manager.py:118)
    and its callers read it with ``.item()`` (server/engine.py:239,247)."""

    def item(self) -> int:
        return int(self)

    def __add__(self, other):
        return BlockCount(int(self) + int(other))

    __radd__ = __add__

    def __sub__(self, other):
        return BlockCount(int(self) - int(other))

    def __rsub__(self, other):
        return BlockCount(int(other) - int(self))


def _as_i32(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.int32:
        t = t.to(torch.int32)
    return t.contiguous()


class BlockManager:
    def __init__(self, device_name: str, num_blocks: int, max_seqs_in_block_table: int,
                 max_blocks_per_seq: int, block_size: int):
        if not torch.cuda.is_available():
            raise RuntimeError("BlockManager keeps its tables on the GPU; no CUDA device is available")
        self.device_name = device_name
        self.resize_generation = 0      # bumped whenever ``is_block_free`` is replaced (elastic expand / release)
        self._nosync_pending = False
        self._readback_enqueued = False
        self._alloc_status = None       # device int64[5]: [0..3] see mkv_block_allocate, [4] blocks freed without sync
        self._alloc_seen = [0, 0, 0, 0, 0]
        self._alloc_need = self._alloc_ids = None
        self.num_free_blocks = BlockCount(num_blocks)
        self.num_blocks = num_blocks
        self.block_size = block_size

        self.num_free_blocks_org = num_blocks
        self.num_blocks_org = num_blocks

        # seq_id |-> number of blocks allocated for this sequence
        self.num_seq_allocated_blocks = torch.zeros((max_seqs_in_block_table,), dtype=torch.int32, device="cuda")
        # (seq_id, block_index) |-> block_id; -1 where never assigned
        self.block_table = torch.full((max_seqs_in_block_table, max_blocks_per_seq), -1,
                                      dtype=torch.int32, device="cuda")
        # block_id |-> free?
        self.is_block_free = torch.ones((num_blocks,), dtype=torch.bool, device="cuda")

    # ``is_block_free`` stays an attribute that outside code REPLACES: the elastic resize assigns a longer or a
    # shorter tensor (server/memory_utils.py:416-417, :650).  Every replacement moves the bitmap to a new address
    # and changes the pool's size, which is what anything that baked the old address in - a captured CUDA graph of
    # the decode step - has to notice: it compares ``resize_generation`` with the value it saw at capture.
    @property
    def is_block_free(self):
        return self._is_block_free

    @is_block_free.setter
    def is_block_free(self, value):
        self._is_block_free = value
        self.resize_generation += 1

    # ``num_free_blocks`` stays an attribute that outside code reads and assigns (the elastic resize does
    # ``+= n`` / ``-= n``); reading it first folds in what sync-free allocations did on the GPU.
    @property
    def num_free_blocks(self):
        if self._nosync_pending:
            self.sync_counters()
        return self._num_free_blocks

    @num_free_blocks.setter
    def num_free_blocks(self, value):
        if self._nosync_pending:
            self.sync_counters()
        self._num_free_blocks = value if isinstance(value, BlockCount) else BlockCount(int(value))

    def allocate_blocks_for_seqs_nosync(self, seq_ids: torch.Tensor, target_lens: torch.Tensor) -> None:
        """``allocate_blocks_for_seqs`` without its return value and without any host synchronisation: one
        kernel computes the need, takes the first free ids in ascending order and extends the rows, or changes
        nothing if the pool is too small.  ``seq_ids`` / ``target_lens`` must be int32 CUDA tensors.  Errors
        (the reference's AssertionError / RuntimeError) are raised by the next ``sync_counters()``, which every
        read of ``num_free_blocks`` implies."""
        assert seq_ids.dtype == torch.int32 and target_lens.dtype == torch.int32
        assert seq_ids.is_contiguous() and target_lens.is_contiguous()
        self.prepare_nosync(seq_ids.shape[0])
        dev, stream = device_and_stream(self.block_table)
        check(lib.mkv_block_allocate(
            dev, stream, self.num_seq_allocated_blocks.data_ptr(), self.num_seq_allocated_blocks.shape[0],
            self.block_table.data_ptr(),
            self.block_table.stride(0), seq_ids.data_ptr(), target_lens.data_ptr(), seq_ids.shape[0], self.block_size,
            self.is_block_free.data_ptr(), self.is_block_free.shape[0], self._alloc_need.data_ptr(),
            self._alloc_ids.data_ptr(), self._alloc_ids.shape[0], self._alloc_status.data_ptr()),
            "mkv_block_allocate")
        self._nosync_pending = True
        self._readback_enqueued = False     # a snapshot taken before this call no longer covers it

    def free_blocks_for_seqs_nosync(self, seq_ids: torch.Tensor) -> None:
        """``free_blocks_for_seqs`` without the host round trip for the number of blocks freed
        (worker/block_manager.py:114-119 reads it with a sum on the device and ends up with a tensor-valued
        counter): the count is accumulated on the device and folded in by the next ``sync_counters()``."""
        assert seq_ids.dtype == torch.int32 and seq_ids.is_contiguous()
        self.prepare_nosync(seq_ids.shape[0])
        dev, stream = device_and_stream(self.block_table)
        check(lib.mkv_block_table_unset(dev, stream, self.num_seq_allocated_blocks.data_ptr(),
                                        self.num_seq_allocated_blocks.shape[0],
                                        self.block_table.data_ptr(), self.block_table.stride(0),
                                        seq_ids.data_ptr(), seq_ids.shape[0], self.is_block_free.data_ptr(),
                                        self.is_block_free.shape[0], None, 0,
                                        self._alloc_status.data_ptr() + 4 * 8, 1), "mkv_block_table_unset")
        self._nosync_pending = True
        self._readback_enqueued = False

    def gather_allocated_blocks_and_free_nosync(self, seq_ids: torch.Tensor, capacity: int = None):
        """``gather_allocated_blocks_and_free`` without the host round trip that sizes its result
        (worker/kernels/block_mgmt.py:115-116 reads the block count back to allocate the output): the ids go into a
        buffer of ``capacity`` entries (default: as many as the sequences' rows could hold, at most the pool) and
        the number of valid entries stays on the device.  Returns ``(ids, count)``: ``ids`` int32 ``[capacity]``,
        batch order, entries from ``count`` on are -1; ``count`` int64 ``[1]`` on the device.  The free-block count
        is folded in by the next ``sync_counters()``.  If the sequences hold more blocks than ``capacity`` the
        surplus ids are freed but not reported; ``count`` then exceeds ``capacity``."""
        assert seq_ids.dtype == torch.int32 and seq_ids.is_contiguous()
        batch = seq_ids.shape[0]
        if capacity is None:
            capacity = min(batch * self.block_table.shape[1], self.is_block_free.shape[0])
        self.prepare_nosync(batch)
        dev, stream = device_and_stream(self.block_table)
        ids = torch.full((max(int(capacity), 1),), -1, dtype=torch.int32, device=self.block_table.device)
        count = torch.zeros((1,), dtype=torch.int64, device=self.block_table.device)
        check(lib.mkv_block_table_unset(dev, stream, self.num_seq_allocated_blocks.data_ptr(),
                                        self.num_seq_allocated_blocks.shape[0],
                                        self.block_table.data_ptr(), self.block_table.stride(0),
                                        seq_ids.data_ptr(), batch, self.is_block_free.data_ptr(),
                                        self.is_block_free.shape[0], ids.data_ptr(), int(capacity),
                                        count.data_ptr(), 0), "mkv_block_table_unset")
        self._alloc_status[4:5] += count        # the running total of blocks freed without a host round trip
        self._nosync_pending = True
        self._readback_enqueued = False
        return ids[:int(capacity)], count

    def prepare_nosync(self, batch: int) -> None:
        """Scratch of the sync-free allocate (status words, need per sequence, id list).  Called by it; call it
        yourself before capturing a CUDA graph, since a capture must not allocate from the regular pool."""
        dev = self.block_table.device
        if (self._alloc_status is not None and self._alloc_need is not None and self._alloc_need.shape[0] >= batch
                and self._alloc_ids is not None and self._alloc_ids.shape[0] >= self.is_block_free.shape[0]):
            return
        with torch.inference_mode(False):   # plain tensors: they are updated from inside and outside inference mode
            self._prepare_nosync_buffers(batch, dev)

    def _prepare_nosync_buffers(self, batch, dev) -> None:
        if self._alloc_status is None:
            self._alloc_status = torch.zeros((5,), dtype=torch.int64, device=dev)
            self._status_host = torch.zeros((5,), dtype=torch.int64).pin_memory()
            self._status_event = torch.cuda.Event()
            self._readback_enqueued = False
        if self._alloc_need is None or self._alloc_need.shape[0] < batch:
            self._alloc_need = torch.empty((max(batch, 64),), dtype=torch.int32, device=dev)
        if self._alloc_ids is None or self._alloc_ids.shape[0] < self.is_block_free.shape[0]:
            self._alloc_ids = torch.empty((self.is_block_free.shape[0],), dtype=torch.int64, device=dev)

    def nosync_replayed(self, with_readback: bool = False) -> None:
        """Tell the manager that a captured graph containing sync-free allocations was replayed (and whether the
        graph also holds ``readback_counters_async()``, in which case the caller synchronises with the stream
        before it reads ``num_free_blocks``)."""
        self._nosync_pending = True
        self._readback_enqueued = with_readback

    def readback_counters_async(self) -> None:
        """Enqueue, on the current stream, the copy of the device-side record into pinned host memory.  A caller
        that synchronises with the stream anyway (end of a step) then gets ``sync_counters()`` without another
        round trip to the GPU; the copy can be captured in a CUDA graph."""
        self.prepare_nosync(1)
        self._status_host.copy_(self._alloc_status, non_blocking=True)
        if not torch.cuda.is_current_stream_capturing():
            self._status_event.record()
        self._readback_enqueued = True

    def sync_counters(self) -> None:
        """Fold the device-side record of the sync-free allocations and frees into the host counters and raise
        what the reference would have raised at allocation time.  One wait for the GPU - none if
        ``readback_counters_async()`` ran after the last sync-free call and the stream has been synchronised."""
        self._nosync_pending = False
        if self._alloc_status is None:
            return
        if not self._readback_enqueued:
            self._status_host.copy_(self._alloc_status, non_blocking=True)
            self._status_event.record()
        self._status_event.synchronize()    # returns at once when the stream was synchronised after the copy
        self._readback_enqueued = False
        st = self._status_host.tolist()
        seen, self._alloc_seen = self._alloc_seen, st
        self._num_free_blocks = BlockCount(self._num_free_blocks - (st[0] - seen[0]) + (st[4] - seen[4]))
        # every condition recorded since the last look is reported, not only the first one
        problems = []
        if st[2] != seen[2]:
            problems.append(f"No enough free blocks available on {self.device_name} ({self.num_blocks} in total, "
                            f"{st[2] - seen[2]} short)")
        if st[3] != seen[3]:
            problems.append(f"(On {self.device_name}) a sequence needs more blocks than a block-table row holds")
        if st[1] != seen[1]:
            shrink = (f"(On {self.device_name}) Logic error: Some sequences have more blocks already allocated "
                      f"than needed.")
            if problems:
                raise RuntimeError("; ".join(problems + [shrink]))
            raise AssertionError(shrink)
        if problems:
            raise RuntimeError("; ".join(problems))

    def get_num_used_blocks(self) -> int:
        return self.num_blocks - self.num_free_blocks

    def _allocate_blocks(self, num_blocks: int) -> torch.Tensor:
        """First ``num_blocks`` free ids in ascending order; marks them used."""
        num_blocks = int(num_blocks)
        if num_blocks > self.num_free_blocks:
            raise RuntimeError(f"No enough free blocks available on {self.device_name} ({self.num_blocks} in total, "
                               f"{self.num_free_blocks} free, {num_blocks} requested)")
        free = self.is_block_free
        dev, stream = device_and_stream(free)
        selected = torch.empty((num_blocks + 1,), dtype=torch.int64, device=free.device)   # ids, then the count found
        check(lib.mkv_bitmap_select(dev, stream, free.data_ptr(), 0, free.shape[0], 1, num_blocks, 1,
                                    selected.data_ptr(), selected[num_blocks:].data_ptr(), None), "mkv_bitmap_select")
        found = int(selected[num_blocks].item())
        self.num_free_blocks = BlockCount(self.num_free_blocks - found)
        if found < num_blocks:      # the host count was ahead of the bitmap: never hand out unwritten ids
            self._free_blocks(selected[:found])
            raise RuntimeError(f"No enough free blocks available on {self.device_name}: the bitmap holds {found} "
                               f"free blocks, {num_blocks} requested")
        return selected[:num_blocks]

    def _free_blocks(self, block_ids: torch.Tensor):
        self.num_free_blocks = BlockCount(self.num_free_blocks + len(block_ids))
        free = self.is_block_free
        dev, stream = device_and_stream(free)
        ids = block_ids.to(torch.int64).contiguous()
        check(lib.mkv_bitmap_scatter(dev, stream, free.data_ptr(), free.shape[0], ids.data_ptr(), ids.shape[0], 1),
              "mkv_bitmap_scatter")

    def allocate_blocks_for_seqs(self, seq_ids: torch.Tensor, target_lens: torch.Tensor) -> torch.Tensor:
        """Make sure sequence i owns ceil(target_lens[i] / block_size) blocks.
        Returns the newly allocated ids (int64), assigned in batch order.

        One launch (the kernel of the sync-free form: need, first-fit ids, rows and counts, all or nothing)
        and one read of its record, which sizes the returned tensor and carries what the reference raises:
        AssertionError when a sequence already owns more blocks than its target (:95-98), RuntimeError when the
        pool is too small (:69-70) - decided against the bitmap itself, so a host-side count that went stale
        cannot let an allocation through - or when a row of the block table is full."""
        seq_ids = _as_i32(seq_ids)
        target_lens = _as_i32(target_lens)
        if self._nosync_pending:
            self.sync_counters()            # earlier sync-free calls: their outcome belongs to them
        before = self._alloc_seen[0]
        self.allocate_blocks_for_seqs_nosync(seq_ids, target_lens)
        self.sync_counters()
        n_new = self._alloc_seen[0] - before
        if n_new == 0:
            return torch.empty(0, device=self.block_table.device, dtype=torch.int64)
        return self._alloc_ids[:n_new].clone()

    def free_blocks_for_seqs(self, seq_ids: torch.Tensor):
        seq_ids = _as_i32(seq_ids)
        dev, stream = device_and_stream(self.block_table)
        total = torch.empty((1,), dtype=torch.int64, device=self.block_table.device)
        check(lib.mkv_block_table_unset(dev, stream, self.num_seq_allocated_blocks.data_ptr(),
                                        self.num_seq_allocated_blocks.shape[0],
                                        self.block_table.data_ptr(), self.block_table.stride(0),
                                        seq_ids.data_ptr(), seq_ids.shape[0], self.is_block_free.data_ptr(),
                                        self.is_block_free.shape[0], None, 0, total.data_ptr(), 0),
              "mkv_block_table_unset")
        self.num_free_blocks = BlockCount(self.num_free_blocks + int(total.item()))

    def gather_allocated_blocks_and_free(self, seq_ids: torch.Tensor) -> torch.Tensor:
        """Ids (int32, batch order) of the blocks of the given sequences; frees them.  Used by swapping."""
        gathered = gather_allocated_blocks_and_unset(self.num_seq_allocated_blocks, self.block_table,
                                                     _as_i32(seq_ids), self.is_block_free)
        self.num_free_blocks = BlockCount(self.num_free_blocks + len(gathered))
        return gathered

    def get_num_allocated_blocks(self, seq_ids: torch.Tensor) -> torch.Tensor:
        return self.num_seq_allocated_blocks[seq_ids]
