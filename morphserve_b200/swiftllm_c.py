"""Stand-in for the reference's native extension module ``swiftllm_c``
(csrc/src/entrypoints.cpp:6-33): block swap, elastic chunk carving, and the data
movement of a layer replacement (``replace_layer_*`` with the registration calls
around it), which is what produces and retires elastic chunks.  Same function
names and argument order; the work is done by ``libmorphkv.so`` through its C ABI.
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import MKV_MAX_SEGMENTS, MkvPool, MorphKVError, check, lib
from .worker.kernels._common import device_and_stream, make_pool

_state = {"kv_info": None, "org_gpu": {}, "org_cpu": {}, "quant": {}, "map_quant": {}, "map_org": {}}


def _as_list(xs):
    return [int(x) for x in (xs.tolist() if isinstance(xs, torch.Tensor) else xs)]


def _ids(xs):
    xs = _as_list(xs)
    n = len(xs)
    return (C.c_int64 * n)(*xs), n


def _dev_ids(xs, device):
    if isinstance(xs, torch.Tensor):
        return xs.to(device=device, dtype=torch.int64).contiguous()
    return torch.tensor(_as_list(xs), dtype=torch.int64, device=device)


def _swap(src, dst, is_swap_in, pool, k_cache, k_swap, v_swap):
    if len(src) != len(dst):
        raise RuntimeError("source_block_ids and target_block_ids differ in length")
    if k_swap.is_cuda or v_swap.is_cuda:
        raise RuntimeError("k_swap / v_swap must be host tensors")
    dev, stream = device_and_stream(k_cache)
    if k_swap.is_pinned() and v_swap.is_pinned():
        # one kernel reads / writes the pinned swap space directly; ids may stay on the GPU
        if not isinstance(src, torch.Tensor):       # host lists: keep the range check of the copy path
            host_ids = _as_list(src if is_swap_in else dst)
            dev_ids = _as_list(dst if is_swap_in else src)
            total = pool.num_blocks_org + (pool.num_segments - 1) * pool.chunk_blocks
            if host_ids and (min(host_ids) < 0 or max(host_ids) >= k_swap.shape[0]
                             or min(dev_ids) < 0 or max(dev_ids) >= total):
                raise MorphKVError(-5, "mkv_swap_blocks_pinned")
        s, d = _dev_ids(src, k_cache.device), _dev_ids(dst, k_cache.device)
        check(lib.mkv_swap_blocks_pinned(dev, stream, pool, k_swap.data_ptr(), v_swap.data_ptr(), k_swap.shape[0],
                                         s.data_ptr(), d.data_ptr(), s.shape[0], 1 if is_swap_in else 0),
              "mkv_swap_blocks_pinned")
        return
    s, n = _ids(src)
    d, _ = _ids(dst)
    check(lib.mkv_swap_blocks(dev, stream, pool, k_swap.data_ptr(), v_swap.data_ptr(), k_swap.shape[0],
                              s, d, n, 1 if is_swap_in else 0, None), "mkv_swap_blocks")


def swap_blocks(source_block_ids, target_block_ids, is_swap_in, k_cache, v_cache, k_swap, v_swap):
    """csrc/src/block_swapping.cpp:22-85.  Asynchronous on the current stream.  Pageable swap space:
    run-coalesced cudaMemcpyAsync like the reference.  Pinned swap space: one zero-copy kernel; the id
    arguments may then also be device tensors (no .tolist() needed)."""
    pool = make_pool(k_cache, v_cache, [], [], k_cache.shape[0], 0)
    _swap(source_block_ids, target_block_ids, is_swap_in, pool, k_cache, k_swap, v_swap)


def swap_blocks_new_kv_combined(source_block_ids, target_block_ids, is_swap_in, num_blocks_org,
                                org_layer_param_size, kv_cache_new_block_size, k_cache_element_size,
                                k_cache, v_cache, k_swap, v_swap, k_cache_new, v_cache_new):
    """csrc/src/block_swapping.cpp:88-202.  Only chunk 0 is passed in; chunk j is
    taken to sit ``j * org_layer_param_size`` elements below it, the layout the
    reference's allocator produces (:159-160).  The device address always comes
    from the device-side id (the reference uses the source id on swap-in, :156-161)."""
    dev_ids = target_block_ids if is_swap_in else source_block_ids
    top = max(_as_list(dev_ids), default=0)
    n_chunks = 1 + max(0, (top - num_blocks_org) // kv_cache_new_block_size) if top >= num_blocks_org else 1
    if n_chunks + 1 > MKV_MAX_SEGMENTS:
        raise RuntimeError("block id beyond the supported number of elastic chunks")
    pool = MkvPool()
    pool.num_segments = 1 + n_chunks
    pool.elem_bytes = int(k_cache_element_size)
    _, pool.num_layers, pool.num_kv_heads, pool.block_size, pool.head_dim = k_cache.shape
    pool.num_blocks_org = int(num_blocks_org)
    pool.chunk_blocks = int(kv_cache_new_block_size)
    pool.k_base[0] = k_cache.data_ptr()
    pool.v_base[0] = v_cache.data_ptr()
    step = int(org_layer_param_size) * int(k_cache_element_size)
    for j in range(n_chunks):
        pool.k_base[1 + j] = k_cache_new.data_ptr() - j * step
        pool.v_base[1 + j] = v_cache_new.data_ptr() - j * step
    _swap(source_block_ids, target_block_ids, is_swap_in, pool, k_cache, k_swap, v_swap)


def swap_blocks_chunk_list(source_block_ids, target_block_ids, is_swap_in, num_blocks_org, kv_cache_new_block_size,
                           k_cache, v_cache, k_swap, v_swap, k_cache_new: list, v_cache_new: list):
    """The elastic swap for callers that hold the whole chunk LISTS (as the model does, worker/model.py:75-76)
    rather than chunk 0 and a slab stride: chunks may sit anywhere, and with a pinned swap space the ids can
    stay on the GPU (no ``.tolist()``, no scan for the highest id).  No counterpart in the reference."""
    pool = make_pool(k_cache, v_cache, k_cache_new, v_cache_new, int(num_blocks_org), int(kv_cache_new_block_size))
    _swap(source_block_ids, target_block_ids, is_swap_in, pool, k_cache, k_swap, v_swap)


def register_kv_cache_info(num_layers: int, num_kv_heads: int, block_size: int, head_dim: int) -> None:
    """csrc/src/memory_manager.cpp:57-66."""
    _state["kv_info"] = (int(num_layers), int(num_kv_heads), int(block_size), int(head_dim))


def register_layer_memory_org_gpu(layer_id: int, start_addr: int, size: int) -> None:
    """csrc/src/memory_manager.cpp:16-21: the fp16 layer's slab on the GPU."""
    _state["org_gpu"][int(layer_id)] = (int(start_addr), int(size))


def register_layer_memory_quant(layer_id: int, start_addr: int, size: int) -> None:
    """csrc/src/memory_manager.cpp:30-35: only the size of the quantised layer is used here."""
    _state["quant"][int(layer_id)] = (int(start_addr), int(size))


class _RawCudaMemory:
    """Non-owning view of device memory for torch.as_tensor."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 2, "strides": None}


def acquire_new_kvcache(layer_id: int):
    """K and V tensors ``[n, L, Hkv, bs, D]`` fp16 carved out of the part of layer
    ``layer_id``'s slab that the quantised layer does not cover, zero-filled.
    csrc/src/memory_manager.cpp:69-176.  The tensors do not own the memory."""
    layer_id = int(layer_id)
    if layer_id not in _state["org_gpu"] or layer_id not in _state["quant"]:
        raise RuntimeError("Layer not found in memory maps")
    if _state["kv_info"] is None:
        raise RuntimeError("KV cache info not registered")
    L, hkv, bs, d = _state["kv_info"]
    org_start, org_size = _state["org_gpu"][layer_id]
    _, quant_size = _state["quant"][layer_id]
    k_addr, v_addr, n = C.c_uint64(0), C.c_uint64(0), C.c_int64(0)
    st = lib.mkv_chunk_layout(org_start, org_size, quant_size, L, hkv, bs, d, 2,
                              C.byref(k_addr), C.byref(v_addr), C.byref(n))
    if st == -7:
        raise RuntimeError("No space available for new KV cache blocks")
    check(st, "mkv_chunk_layout")
    shape = (n.value, L, hkv, bs, d)
    dev = torch.device("cuda", torch.cuda.current_device())
    k = torch.as_tensor(_RawCudaMemory(k_addr.value, shape, "<f2"), device=dev)
    v = torch.as_tensor(_RawCudaMemory(v_addr.value, shape, "<f2"), device=dev)
    k.zero_()
    v.zero_()
    return k, v


def register_layer_memory_org_cpu(layer_id: int, start_addr: int, size: int) -> None:
    """csrc/src/memory_manager.cpp:23-28: the host copy of the fp16 layer."""
    _state["org_cpu"][int(layer_id)] = (int(start_addr), int(size))


def register_layer_memory_tensor_map_quant(layer_id: int, tensor_map) -> None:
    """csrc/src/memory_manager.cpp:37-45: list of ``{name: {offset, shape, dtype, size}}`` of the quantised layer."""
    _state["map_quant"][int(layer_id)] = [dict(m) for m in tensor_map]


def register_layer_memory_tensor_map_org(layer_id: int, tensor_map) -> None:
    """csrc/src/memory_manager.cpp:47-55."""
    _state["map_org"][int(layer_id)] = [dict(m) for m in tensor_map]


# torch dtype -> (typestr of an equally wide type the CUDA array interface knows, dtype to view as afterwards)
_TYPESTR = {torch.float16: ("<f2", None), torch.float32: ("<f4", None), torch.float64: ("<f8", None),
            torch.int8: ("|i1", None), torch.uint8: ("|u1", None), torch.int16: ("<i2", None),
            torch.int32: ("<i4", None), torch.int64: ("<i8", None), torch.bool: ("|u1", torch.bool),
            torch.bfloat16: ("<i2", torch.bfloat16)}


def _tensors_in_slab(base_addr: int, tensor_map):
    """Non-owning tensors at ``base_addr + offset`` for every entry, in list order; inside one entry names
    come in sorted order like the reference's std::map (csrc/src/memory_manager.cpp:235-268)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    out = []
    for entry in tensor_map:
        for name in sorted(entry):
            info = entry[name]
            shape = tuple(int(x) for x in info["shape"])
            typestr, view_as = _TYPESTR[info["dtype"]]
            t = torch.as_tensor(_RawCudaMemory(base_addr + int(info["offset"]), shape, typestr), device=dev)
            out.append(t.view(view_as) if view_as is not None else t)
    return out


def _upload(dst, src, what: str):
    (dst_addr, dst_size), (src_addr, src_size) = dst, src
    if src_size > dst_size:     # checked before any CUDA call, like csrc/src/memory_manager.cpp:195-200
        raise RuntimeError(f"Layer requires {src_size} bytes, but only {dst_size} bytes available")
    st = lib.mkv_slab_upload(torch.cuda.current_device(), dst_addr, dst_size, src_addr, src_size)
    if st == -7:
        raise RuntimeError(f"Layer requires {src_size} bytes, but only {dst_size} bytes available")
    check(st, what)


def replace_layer_org2quant(layer_id: int):
    """Overwrite the start of layer ``layer_id``'s fp16 slab with its quantised image (host -> device,
    complete on return) and return the quantised tensors as views into the slab, in registration order.
    csrc/src/memory_manager.cpp:179-271."""
    layer_id = int(layer_id)
    if (layer_id not in _state["org_gpu"] or layer_id not in _state["quant"]
            or layer_id not in _state["map_quant"]):
        raise RuntimeError(f"Layer ID {layer_id} not registered in memory map")
    _upload(_state["org_gpu"][layer_id], _state["quant"][layer_id], "mkv_slab_upload")
    return _tensors_in_slab(_state["org_gpu"][layer_id][0], _state["map_quant"][layer_id])


def replace_layer_quant2org(layer_id: int):
    """Restore the fp16 layer from its host copy into the slab and return its tensors as views.
    csrc/src/memory_manager.cpp:274-364.  Elastic KV chunks carved out of the slab must have been
    released before (server/memory_utils.py:617-662 checks that)."""
    layer_id = int(layer_id)
    if (layer_id not in _state["org_gpu"] or layer_id not in _state["org_cpu"]
            or layer_id not in _state["map_org"]):
        raise RuntimeError(f"[MemoryManager C++] Layer ID {layer_id} not registered in original memory maps")
    _upload(_state["org_gpu"][layer_id], _state["org_cpu"][layer_id], "mkv_slab_upload")
    return _tensors_in_slab(_state["org_gpu"][layer_id][0], _state["map_org"][layer_id])


def get_freed_memory_size(layer_id: int, used_size: int) -> int:
    """csrc/src/memory_manager.cpp:367-374."""
    if int(layer_id) not in _state["org_gpu"]:
        return 0
    return max(_state["org_gpu"][int(layer_id)][1] - int(used_size), 0)


def verify_tensor_continuity(tensors) -> bool:
    """True if the tensors, sorted by address, follow each other without a gap.
    csrc/src/memory_manager.cpp:376-405."""
    spans = sorted((t.data_ptr(), t.numel() * t.element_size()) for t in tensors)
    return all(spans[i - 1][0] + spans[i - 1][1] == spans[i][0] for i in range(1, len(spans)))


__all__ = ["swap_blocks", "swap_blocks_new_kv_combined", "swap_blocks_chunk_list", "register_kv_cache_info",
           "register_layer_memory_org_gpu", "register_layer_memory_org_cpu", "register_layer_memory_quant",
           "register_layer_memory_tensor_map_quant", "register_layer_memory_tensor_map_org",
           "acquire_new_kvcache", "replace_layer_org2quant", "replace_layer_quant2org",
           "get_freed_memory_size", "verify_tensor_continuity", "MorphKVError"]
