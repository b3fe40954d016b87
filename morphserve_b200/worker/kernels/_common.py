"""Plumbing shared by the kernel wrappers: pool descriptors, streams, workspace.

PyTorch appears here only as the owner of device memory and streams; all
computation happens in ``libmorphkv.so``.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..._lib import MKV_MAX_SEGMENTS, MkvPool, check, lib

_pool_cache: dict = {}


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: morphserve_b200 has no CPU path")


def device_and_stream(t: torch.Tensor):
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    return dev, torch.cuda.current_stream(dev).cuda_stream


def make_pool(k_cache, v_cache, k_cache_new, v_cache_new, num_blocks_org, chunk_blocks) -> MkvPool:
    """Segment table for the C ABI: segment 0 = the original pool, segment 1+j =
    elastic chunk j (server/memory_utils.py:389-390 appends them in this order).

    Equals the reference's "chunk j sits j*org_layer_param_size elements below
    chunk 0" addressing (worker/kernels/paged_attn.py:358-360) whenever the list
    was produced by acquire_new_kvcache, and also works for chunks placed
    anywhere.  Descriptors are cached on the identity of the tensors.
    """
    n_new = len(k_cache_new)
    key = (k_cache.data_ptr(), v_cache.data_ptr(), n_new,
           k_cache_new[-1].data_ptr() if n_new else 0, int(num_blocks_org or 0), int(chunk_blocks or 0),
           tuple(k_cache.shape), k_cache.element_size())
    pool = _pool_cache.get(key)
    if pool is not None:
        return pool
    if n_new + 1 > MKV_MAX_SEGMENTS:
        raise RuntimeError(f"too many elastic KV chunks ({n_new}); the library supports {MKV_MAX_SEGMENTS - 1}")
    if k_cache.dtype not in (torch.float16, torch.float32):
        raise RuntimeError(f"unsupported KV dtype {k_cache.dtype}")
    pool = MkvPool()
    pool.num_segments = 1 + n_new
    pool.elem_bytes = k_cache.element_size()
    _, pool.num_layers, pool.num_kv_heads, pool.block_size, pool.head_dim = k_cache.shape
    pool.num_blocks_org = k_cache.shape[0] if not n_new else int(num_blocks_org)
    pool.chunk_blocks = int(chunk_blocks) if n_new else 0
    pool.k_base[0] = k_cache.data_ptr()
    pool.v_base[0] = v_cache.data_ptr()
    for j in range(n_new):
        if k_cache_new[j].shape[0] != pool.chunk_blocks:
            raise RuntimeError("elastic KV chunks must all hold kv_cache_new_block_size blocks")
        pool.k_base[1 + j] = k_cache_new[j].data_ptr()
        pool.v_base[1 + j] = v_cache_new[j].data_ptr()
    if len(_pool_cache) > 256:
        _pool_cache.clear()
    _pool_cache[key] = pool
    return pool


class _Workspace:
    __slots__ = ("tensor", "nbytes", "generation")

    def __init__(self):
        self.tensor = None
        self.nbytes = 0
        self.generation = 0


# One workspace per (device, stream): launches on one stream are ordered and may share scratch, launches on
# different streams may overlap on the GPU and must not (the reference's layer code runs attention on a side
# stream, worker/layers/transformer_layer.py:177-191; two models or two host threads bring their own streams).
# The tensor is allocated while its stream is current, so the caching allocator ties the block to that stream
# and dropping an old entry cannot hand its memory to work that overlaps with launches still queued on it.
_workspaces: dict = {}
_ws_bytes_cache: dict = {}
_MAX_WORKSPACES = 32


def attn_workspace(dev: int, batch: int, hq: int, hkv: int, d: int, max_blocks: int, stream: int = None) -> _Workspace:
    """Persistent scratch of the decode kernel (plan, split-KV partials, counters) for launches on `stream`
    (default: the current stream of `dev`).  Grown when a larger batch arrives, never shrunk."""
    key = (dev, batch, hq, hkv, d, max_blocks)
    need = _ws_bytes_cache.get(key)
    if need is None:
        need = int(lib.mkv_attn_workspace_bytes(dev, batch, hq, hkv, d, max_blocks))
        if need == 0:
            raise RuntimeError("mkv_attn_workspace_bytes failed")
        _ws_bytes_cache[key] = need
    if stream is None:
        stream = torch.cuda.current_stream(dev).cuda_stream
    ws = _workspaces.get((dev, stream))
    if ws is None:
        if len(_workspaces) >= _MAX_WORKSPACES:      # streams come and go: forget the oldest entry
            _workspaces.pop(next(iter(_workspaces)))
        ws = _workspaces[(dev, stream)] = _Workspace()
    if ws.nbytes < need:
        grow = max(need, int(ws.nbytes * 1.5))
        if torch.cuda.current_stream(dev).cuda_stream == stream:
            ws.tensor = torch.empty(grow, dtype=torch.uint8, device=torch.device("cuda", dev))
        else:
            with torch.cuda.stream(torch.cuda.ExternalStream(stream, device=dev)):
                ws.tensor = torch.empty(grow, dtype=torch.uint8, device=torch.device("cuda", dev))
        assert ws.tensor.data_ptr() % 256 == 0
        ws.nbytes = grow
        ws.generation += 1
    return ws


def read_attn_error_flags(dev: int) -> int:
    """Debug helper: the error words of every attention workspace of the device, OR-ed.  Bit 0 = a block-table
    entry pointed outside the pool."""
    out = 0
    for (d, _), ws in list(_workspaces.items()):
        if d != dev or ws.tensor is None:
            continue
        flags = C.c_int(0)
        check(lib.mkv_attn_read_error_flags(dev, torch.cuda.current_stream(dev).cuda_stream,
                                            ws.tensor.data_ptr(), C.byref(flags)), "mkv_attn_read_error_flags")
        out |= flags.value
    return out
