"""Python mirror of the DSA top-k indexer's entry point (sibling operator of the MoE layer).

Same six tensors in the same order as the reference's entry point for the definition
``dsa_topk_indexer_fp8_h64_d128_topk2048_ps64`` (dsa_indexer/solution/python/dsa_topk_indexer.py:64,
``run(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, topk_indices)``; CUDA variant
dsa_indexer/solution/cuda/dsa_topk_indexer.cu:468-474), destination-passing.  The work is done by the CUDA
kernels of csrc/dsa_indexer.cu behind the C ABI of include/syfi_dsa.h; there is no CPU path.
"""
from __future__ import annotations

import ctypes

import torch

from .moe import MoeError, _check, _stream_ptr, load_library

HEADS, DIM, PAGE, TOPK = 64, 128, 64, 2048
_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
# name -> (restype, argtypes); must list every symbol include/syfi_dsa.h declares
ABI = {
    "syfi_dsa_topk_indexer": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _vp, _vp]),
    "syfi_dsa_check": (ctypes.c_int, [_vp]),
}
_bound = False


def _lib():
    global _bound
    lib = load_library()
    if not _bound:
        for name, (res, args) in ABI.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _bound = True
    return lib


def _expect(t, name, dtypes, shape, dev):
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"{name} must be a torch.Tensor")
    if t.dtype not in dtypes:
        raise ValueError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
    if t.device != dev:
        raise ValueError(f"{name} is on {t.device}, expected {dev}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def run_dsa_topk_indexer(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, topk_indices, *,
                         stream=None):
    """Writes into ``topk_indices`` int32 [B, 2048] the cache token ids of each sequence's 2048 best-scoring
    tokens, best first, -1 beyond the sequence's length.  Enqueues on the current CUDA stream, does not
    synchronise."""
    if not isinstance(q_index_fp8, torch.Tensor) or q_index_fp8.device.type != "cuda":
        raise ValueError("q_index_fp8 must be a CUDA tensor: this library has no CPU path")
    dev = q_index_fp8.device
    B = q_index_fp8.shape[0]
    _expect(q_index_fp8, "q_index_fp8", (torch.float8_e4m3fn, torch.uint8), (B, HEADS, DIM), dev)
    if not isinstance(k_index_cache_fp8, torch.Tensor) or k_index_cache_fp8.dim() != 4:
        raise ValueError("k_index_cache_fp8 must be a 4-D tensor [pages, 64, 1, 132]")
    P = k_index_cache_fp8.shape[0]
    _expect(k_index_cache_fp8, "k_index_cache_fp8", (torch.int8, torch.uint8), (P, PAGE, 1, DIM + 4), dev)
    _expect(weights, "weights", (torch.float32,), (B, HEADS), dev)
    _expect(seq_lens, "seq_lens", (torch.int32,), (B,), dev)
    if not isinstance(block_table, torch.Tensor) or block_table.dim() != 2:
        raise ValueError("block_table must be a 2-D tensor [B, max_pages]")
    max_pages = block_table.shape[1]
    _expect(block_table, "block_table", (torch.int32,), (B, max_pages), dev)
    _expect(topk_indices, "topk_indices", (torch.int32,), (B, TOPK), dev)
    if B == 0:
        return topk_indices
    lib = _lib()
    with torch.cuda.device(dev):
        _check(lib.syfi_dsa_topk_indexer(q_index_fp8.data_ptr(), k_index_cache_fp8.data_ptr(), weights.data_ptr(),
                                         seq_lens.data_ptr(), block_table.data_ptr(), B, P, max_pages,
                                         topk_indices.data_ptr(), _stream_ptr(stream, dev.index)))
    return topk_indices


def dsa_check(device=None, stream=None):
    """Synchronise and raise :class:`MoeError` if a kernel of the indexer gave up on a bounded wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _check(_lib().syfi_dsa_check(_stream_ptr(stream, dev.index)))


__all__ = ["run_dsa_topk_indexer", "dsa_check", "MoeError"]
