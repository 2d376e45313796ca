"""Tensor-core products of the GRU path (tcgen05 GEMM core of ``libb200gru.so``).

``split_bf16`` turns an fp32 tensor into bf16 planes (hi, mid, lo); ``gemm`` multiplies two
plane sets, ``C = alpha * row_scale * col_scale * sum_pairs A_i @ B_j^T + bias``, with fp32
(bf16 planes) or exact int32 (int8 codes) accumulation.  These stand in for the reference's
``F.linear`` input projection (src/gru_qat/gru_layer.py:251-253) and its ``tl.dot`` tiles
(src/gru_qat/triton_kernels/scan.py:153-155, 521-616).  CUDA tensors only; no fallback.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from . import _lib

# plane cross products, most significant first
PAIRS_EXACT_B = {1: [(0, 0)], 2: [(0, 0), (1, 0)], 3: [(0, 0), (1, 0), (2, 0)]}
PAIRS_FULL = [(0, 0), (0, 1), (1, 0), (0, 2), (1, 1), (2, 0)]          # error about 2^-24 of |a||b|
PAIRS_FAST = [(0, 0), (0, 1), (1, 0)]                                  # error about 2^-17 of |a||b|


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def split_bf16(x: torch.Tensor, planes: int = 3, col_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[planes, *x.shape]`` bf16 with ``sum(planes) == x * col_scale`` (to 8 bits per plane)."""
    if not x.is_cuda or x.dtype != torch.float32:
        raise ValueError("split_bf16 needs a CUDA float32 tensor")
    x = x.contiguous()
    n = x.numel()
    if n % 4:
        raise ValueError("element count must be a multiple of 4")
    out = torch.empty((planes,) + tuple(x.shape), device=x.device, dtype=torch.bfloat16)
    ncols = x.shape[-1] if col_scale is not None else 0
    with torch.cuda.device(x.device):
        rc = _lib.load().b200gru_split_bf16(_lib._ptr(x), _lib._ptr(out), n, n, planes, _lib._ptr(col_scale),
                                            ncols, _stream(x))
    if rc:
        _lib._raise(rc, "split_bf16")
    return out


def gemm(A: torch.Tensor, B: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         pairs: Optional[Sequence[Tuple[int, int]]] = None, alpha: float = 1.0,
         row_scale: Optional[torch.Tensor] = None, col_scale: Optional[torch.Tensor] = None,
         bias: Optional[torch.Tensor] = None, split_k: int = 1, tile_n: int = 0, chunk_kblocks: int = 0,
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``A``: ``[planes, M, K]`` (or ``[planes, K, M]`` with ``a_mn``); ``B``: ``[planes, N, K]``
    (or ``[planes, K, N]`` with ``b_mn``); bf16 or int8, contiguous.  Returns fp32 ``[M, N]``
    (``split_k`` partial results are summed in order)."""
    if A.dim() == 2:
        A = A[None]
    if B.dim() == 2:
        B = B[None]
    if not (A.is_cuda and B.is_cuda) or A.dtype != B.dtype or A.dtype not in (torch.bfloat16, torch.int8):
        raise ValueError("gemm needs CUDA operands of one dtype, bfloat16 or int8")
    A, B = A.contiguous(), B.contiguous()
    pa, (M, K) = A.shape[0], ((A.shape[2], A.shape[1]) if a_mn else (A.shape[1], A.shape[2]))
    pb, (N, Kb) = B.shape[0], ((B.shape[2], B.shape[1]) if b_mn else (B.shape[1], B.shape[2]))
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    if pairs is None:
        pairs = [(i, j) for i in range(pa) for j in range(pb)]
    g = _lib.CGemmArgs()
    g.dtype = 1 if A.dtype == torch.int8 else 0
    g.M, g.N, g.K = M, N, K
    g.A, g.B = A.data_ptr(), B.data_ptr()
    g.a_planes, g.b_planes = pa, pb
    g.a_mn_major, g.b_mn_major = int(a_mn), int(b_mn)
    g.lda, g.ldb = A.shape[2], B.shape[2]
    g.a_plane_stride, g.b_plane_stride = A.shape[1] * A.shape[2], B.shape[1] * B.shape[2]
    g.npairs = len(pairs)
    for q, (i, j) in enumerate(pairs):
        g.pair_a[q], g.pair_b[q] = i, j
    g.tile_n, g.alpha, g.chunk_kblocks = tile_n, alpha, chunk_kblocks
    g.row_scale = None if row_scale is None else row_scale.data_ptr()
    g.col_scale = None if col_scale is None else col_scale.data_ptr()
    g.bias = None if bias is None else bias.data_ptr()
    lib = _lib.load()
    g.split_k = 1
    splits = lib.b200gru_tc_gemm_splits(ctypes.byref(g), split_k) if split_k > 1 else 1
    g.split_k = splits
    if splits > 1:
        C = torch.empty((splits, M, N), device=A.device, dtype=torch.float32)
    else:
        C = out if out is not None else torch.empty((M, N), device=A.device, dtype=torch.float32)
    g.C, g.ldc, g.split_stride = C.data_ptr(), N, M * N
    with torch.cuda.device(A.device):
        rc = lib.b200gru_tc_gemm(ctypes.byref(g), _stream(A))
    if rc:
        _lib._raise(rc, "tc gemm")
    if splits > 1:
        res = C[0]
        for s in range(1, splits):
            res = res + C[s]
        if out is not None:
            out.copy_(res)
            return out
        return res
    return C
