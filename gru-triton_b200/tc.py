"""Tensor-core products of the GRU path (tcgen05 GEMM core of ``libb200gru.so``).

* ``split_bf16`` / ``split_f16`` / ``gemm``: operand preparation and the raw product
  ``C = alpha * row_scale * col_scale * sum_pairs A_i @ B_j^T + bias`` with fp32 (bf16 or fp16
  planes) or exact int32 (int8 codes) accumulation.
* ``linear``: the input projection ``gi = x @ Wi^T + bi`` of a whole sequence and its gradients,
  row-chunked so that operand planes stay small; with ``weight_bits <= 8`` the weights are
  fake-quantised per output row on the device and multiplied as exact integer codes.
  Stands in for ``F.linear`` at src/gru_qat/gru_layer.py:251-253 / gru_cell.py:410-435.
* ``gru_scan_dense_q8``: the dense scan on int8 weights (weight fake-quant of
  src/gru_qat/gru_cell.py:239-271 fused into a weight-prep kernel that emits codes and scales).

CUDA tensors only; there is no fallback.
"""

from __future__ import annotations

import ctypes
from typing import Any, Optional, Sequence, Tuple

import torch

from . import _lib

# plane cross products, most significant first
PAIRS_EXACT_B = {1: [(0, 0)], 2: [(0, 0), (1, 0)], 3: [(0, 0), (1, 0), (2, 0)]}
PAIRS_EXACT_A = {1: [(0, 0)], 2: [(0, 0), (0, 1)], 3: [(0, 0), (0, 1), (0, 2)]}
PAIRS_FULL = [(0, 0), (0, 1), (1, 0), (0, 2), (1, 1), (2, 0)]          # error about 2^-24 of |a||b|
PAIRS_FAST = [(0, 0), (0, 1), (1, 0)]                                  # error about 2^-17 of |a||b|
# the same three products on two row-scaled fp16 planes per operand (split_f16): about 2^-22
PAIRS_F16 = PAIRS_FAST

ROW_CHUNK = 32768          # rows of x handled per operand-preparation + GEMM round


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def split_bf16(x: torch.Tensor, planes: int = 3, col_scale: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[planes, *x.shape]`` bf16 with ``sum(planes) == x * col_scale`` (8 mantissa bits per plane)."""
    if not x.is_cuda or x.dtype != torch.float32:
        raise ValueError("split_bf16 needs a CUDA float32 tensor")
    x = x.contiguous()
    n = x.numel()
    if n % 4:
        raise ValueError("element count must be a multiple of 4")
    if out is None:
        out = torch.empty((planes,) + tuple(x.shape), device=x.device, dtype=torch.bfloat16)
    ncols = x.shape[-1] if col_scale is not None else 0
    with torch.cuda.device(x.device):
        rc = _lib.load().b200gru_split_bf16(_lib._ptr(x), _lib._ptr(out), n, n, planes, _lib._ptr(col_scale),
                                            ncols, _stream(x))
    if rc:
        _lib._raise(rc, "split_bf16")
    return out


def split_f16(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(planes [2, R, K] float16, inv_scale [R] float32)`` with
    ``(planes[0] + planes[1]) * inv_scale[:, None] == x`` to 22 significant bits: every row is scaled
    by a power of two of its own before the split, ``inv_scale`` undoes it as the product's
    ``row_scale`` (A operand) or ``col_scale`` (B operand)."""
    if not x.is_cuda or x.dtype != torch.float32 or x.dim() != 2:
        raise ValueError("split_f16 needs a 2-d CUDA float32 tensor")
    x = x.contiguous()
    R, K = x.shape
    if K % 4:
        raise ValueError("row length must be a multiple of 4")
    if out is None:
        out = torch.empty((2, R, K), device=x.device, dtype=torch.float16)
    inv = torch.empty((R,), device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        rc = _lib.load().b200gru_split_f16(_lib._ptr(x), _lib._ptr(out), R, K, R * K, _lib._ptr(inv), _stream(x))
    if rc:
        _lib._raise(rc, "split_f16")
    return out, inv


def gemm(A: torch.Tensor, B: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         pairs: Optional[Sequence[Tuple[int, int]]] = None, alpha: float = 1.0,
         row_scale: Optional[torch.Tensor] = None, col_scale: Optional[torch.Tensor] = None,
         bias: Optional[torch.Tensor] = None, split_k: int = 1, tile_n: int = 0, chunk_kblocks: int = 0,
         out: Optional[torch.Tensor] = None, accumulate: bool = False, reduce_splits: bool = True) -> torch.Tensor:
    """``A``: ``[planes, M, K]`` (or ``[planes, K, M]`` with ``a_mn``); ``B``: ``[planes, N, K]``
    (or ``[planes, K, N]`` with ``b_mn``); bf16, fp16 or int8, contiguous.  Returns fp32 ``[M, N]``.

    ``split_k > 1`` computes that many partial products over slices of K: they are summed in order
    unless ``reduce_splits`` is False, in which case ``out`` (``[splits, M, N]``) receives (or,
    with ``accumulate``, is incremented by) the partial results and is returned as it is."""
    if A.dim() == 2:
        A = A[None]
    if B.dim() == 2:
        B = B[None]
    if not (A.is_cuda and B.is_cuda) or A.dtype != B.dtype or A.dtype not in (torch.bfloat16, torch.float16, torch.int8):
        raise ValueError("gemm needs CUDA operands of one dtype, bfloat16, float16 or int8")
    A, B = A.contiguous(), B.contiguous()
    pa, (M, K) = A.shape[0], ((A.shape[2], A.shape[1]) if a_mn else (A.shape[1], A.shape[2]))
    pb, (N, Kb) = B.shape[0], ((B.shape[2], B.shape[1]) if b_mn else (B.shape[1], B.shape[2]))
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    if pairs is None:
        pairs = [(i, j) for i in range(pa) for j in range(pb)]
    g = _lib.CGemmArgs()
    g.dtype = {torch.bfloat16: 0, torch.int8: 1, torch.float16: 2}[A.dtype]
    g.M, g.N, g.K = M, N, K
    g.A, g.B = A.data_ptr(), B.data_ptr()
    g.a_planes, g.b_planes = pa, pb
    g.a_mn_major, g.b_mn_major = int(a_mn), int(b_mn)
    g.lda, g.ldb = A.shape[2], B.shape[2]
    g.a_plane_stride, g.b_plane_stride = A.shape[1] * A.shape[2], B.shape[1] * B.shape[2]
    g.npairs = len(pairs)
    for q, (i, j) in enumerate(pairs):
        g.pair_a[q], g.pair_b[q] = i, j
    g.tile_n, g.alpha, g.chunk_kblocks, g.accumulate = tile_n, alpha, chunk_kblocks, int(accumulate)
    g.row_scale = None if row_scale is None else row_scale.data_ptr()
    g.col_scale = None if col_scale is None else col_scale.data_ptr()
    g.bias = None if bias is None else bias.data_ptr()
    lib = _lib.load()
    g.split_k = 1
    splits = lib.b200gru_tc_gemm_splits(ctypes.byref(g), split_k) if split_k > 1 else 1
    g.split_k = splits
    if splits > 1 and not (out is not None and not reduce_splits):
        C = torch.empty((splits, M, N), device=A.device, dtype=torch.float32)
    elif out is not None:
        C = out
        if not C.is_contiguous() or C.dtype != torch.float32 or C.numel() < splits * M * N:
            raise ValueError("out must be a contiguous float32 tensor of the result's size")
    else:
        C = torch.empty((M, N), device=A.device, dtype=torch.float32)
    g.C, g.ldc, g.split_stride = C.data_ptr(), N, M * N
    with torch.cuda.device(A.device):
        rc = lib.b200gru_tc_gemm(ctypes.byref(g), _stream(A))
    if rc:
        _lib._raise(rc, "tc gemm")
    if splits > 1 and reduce_splits:
        res = _lib.column_sums(C.reshape(splits, M * N)).reshape(M, N)
        if out is not None:
            out.copy_(res)
            return out
        return res
    return C


def gemm_splits(M: int, N: int, K: int, wanted: int) -> int:
    """Number of K slices a bf16 product of this shape uses when ``wanted`` are asked for."""
    g = _lib.CGemmArgs()
    g.dtype, g.M, g.N, g.K, g.a_planes, g.b_planes, g.npairs = 0, M, N, K, 1, 1, 1
    return int(_lib.load().b200gru_tc_gemm_splits(ctypes.byref(g), wanted))


# ----------------------------------------------------------------------------------------------
# input projection
# ----------------------------------------------------------------------------------------------

class _LinearFunction(torch.autograd.Function):
    """``y[R,N] = x[R,I] @ fq(W)[N,I]^T + bias`` with fp32-accurate tensor-core products."""

    @staticmethod
    def forward(ctx: Any, x, W, bias, weight_bits: int):
        R, I = x.shape
        N = W.shape[0]
        # two row-scaled fp16 planes per fp32 operand: 22 significant bits in three cross products
        # (two when the weights are exact integer codes)
        if weight_bits <= 8:
            codes, scales, _ = _lib.quantize_rows(W, weight_bits)
            Bop, col_scale, pairs = codes.to(torch.float16)[None], scales, PAIRS_EXACT_B[2]
        else:
            Bop, col_scale = split_f16(W)
            pairs = PAIRS_F16
        y = torch.empty((R, N), device=x.device, dtype=torch.float32)
        for r0 in range(0, R, ROW_CHUNK):
            r1 = min(R, r0 + ROW_CHUNK)
            xp, x_inv = split_f16(x[r0:r1])
            gemm(xp, Bop, pairs=pairs, row_scale=x_inv, col_scale=col_scale, bias=bias, out=y[r0:r1])
        ctx.save_for_backward(x, W)
        ctx.weight_bits, ctx.has_bias = weight_bits, bias is not None
        ctx.col_scale, ctx.Bop = col_scale, Bop
        return y

    @staticmethod
    def backward(ctx: Any, dy):
        x, W = ctx.saved_tensors
        dy = dy.contiguous()
        R, I = x.shape
        N = W.shape[0]
        need_x, need_w, need_b = ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2] and ctx.has_bias
        dx = torch.empty_like(x) if need_x else None
        if need_x:
            # dx contracts over the weight rows: the bf16 form of the weights (codes are exact in it)
            Bx = ctx.Bop.to(torch.bfloat16) if ctx.weight_bits <= 8 else split_bf16(W)
        dWq = None
        if need_w:
            chunk_rows = min(R, ROW_CHUNK)
            # K slices: about two waves of (N/128) x (I/256) tiles over the 148 SMs when the contraction
            # is long, one wave when each slice would otherwise be only a few k-blocks
            tiles = -(-N // 128) * -(-I // 256)
            want = 1 if tiles >= 120 else -(-(280 if chunk_rows >= 16384 else 140) // tiles)
            splits = gemm_splits(N, I, chunk_rows, max(1, min(want, chunk_rows // 512)))
            # the first chunk writes the K-slice accumulators, later chunks add to them; a short first chunk
            # may use fewer slices than the rest, then the buffer starts from zero
            first_splits = gemm_splits(N, I, min(R, ROW_CHUNK), splits)
            alloc = torch.empty if first_splits == splits else torch.zeros
            dWq = alloc((splits, N, I), device=x.device, dtype=torch.float32)
        for r0 in range(0, R, ROW_CHUNK):
            r1 = min(R, r0 + ROW_CHUNK)
            dyp = split_bf16(dy[r0:r1], planes=3 if need_x else 2)
            if need_w:
                # weight gradients are held to 1e-4 of their largest entry: two planes per operand and
                # the cross products down to 2^-16 (error about 1e-5 of a term, averaged over the rows)
                xp = split_bf16(x[r0:r1], planes=2)
                k_splits = gemm_splits(N, I, r1 - r0, dWq.shape[0])
                gemm(dyp[:2], xp, a_mn=True, b_mn=True, pairs=PAIRS_FAST, split_k=k_splits, out=dWq,
                     accumulate=(r0 > 0 or first_splits != splits), reduce_splits=False)
            if need_x:
                # dx = dy @ fq(W): W rows are the contraction index (MN-major B)
                if ctx.weight_bits <= 8:
                    dys = split_bf16(dy[r0:r1], col_scale=ctx.col_scale)
                    gemm(dys, Bx, b_mn=True, pairs=PAIRS_EXACT_B[3], out=dx[r0:r1])
                else:
                    gemm(dyp, Bx, b_mn=True, pairs=PAIRS_FULL, out=dx[r0:r1])
        dW = None
        if need_w:
            dWq = _lib.column_sums(dWq.reshape(dWq.shape[0], -1)).reshape(N, I) if dWq.shape[0] > 1 else dWq[0]
            dW = _lib.quantize_rows_backward(W, dWq, ctx.weight_bits) if ctx.weight_bits <= 8 else dWq
        db = _lib.column_sums(dy) if need_b else None
        return dx, dW, db, None


def linear(x: torch.Tensor, W: torch.Tensor, bias: Optional[torch.Tensor] = None, *, weight_bits: int = 32):
    """``x[..., I] @ fq(W)[N, I]^T + bias`` -> ``[..., N]`` (fp32).  ``weight_bits <= 8``: ``W`` is
    fake-quantised per output row (dynamic symmetric scale) on the device, as the reference's
    per-channel weight quantizer does, and multiplied as integer codes."""
    if not (x.is_cuda and W.is_cuda) or x.dtype != torch.float32 or W.dtype != torch.float32:
        raise ValueError("linear needs CUDA float32 tensors")
    if x.shape[-1] != W.shape[1] or x.shape[-1] % 8 or W.shape[0] % 8:
        raise ValueError("linear needs x[..., I] and W[N, I] with I % 8 == 0 and N % 8 == 0")
    lead = x.shape[:-1]
    y = _LinearFunction.apply(x.reshape(-1, x.shape[-1]).contiguous(), W.contiguous(), bias, int(weight_bits))
    return y.reshape(*lead, W.shape[0])


# ----------------------------------------------------------------------------------------------
# dense scan on int8 weights
# ----------------------------------------------------------------------------------------------

class GRUScanDenseQ8Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, gi, h0, Wh_cat, bh_cat, weight_bits, h_in_quant, h_out_quant):
        gi, h0, Wh_cat, bh_cat = (t.contiguous() for t in (gi, h0, Wh_cat, bh_cat))
        codes, scales, Wq = _lib.quantize_rows(Wh_cat, weight_bits)
        want = any(ctx.needs_input_grad[:4])
        out, save = _lib.scan_forward("dense", gi, h0, Wq, bh_cat, h_in_quant, h_out_quant, want_save=want,
                                      codes=codes, scales=scales)
        ctx.save_for_backward(gi, h0, Wh_cat, bh_cat, out, Wq, codes, scales, *([save] if save is not None else []))
        ctx.has_save = save is not None
        ctx.quant, ctx.weight_bits = (h_in_quant, h_out_quant), weight_bits
        return out

    @staticmethod
    def backward(ctx: Any, dout):
        gi, h0, Wh_cat, bh_cat, out, Wq, codes, scales = ctx.saved_tensors[:8]
        save = ctx.saved_tensors[8] if ctx.has_save else None
        dgi, dh0, dWq, dbh = _lib.scan_backward("dense", gi, h0, Wq, bh_cat, out, dout.contiguous(), save,
                                                ctx.quant[0], ctx.quant[1], codes=codes, scales=scales)
        dW = _lib.quantize_rows_backward(Wh_cat, dWq, ctx.weight_bits)
        return dgi, dh0, dW, dbh, None, None, None


def gru_scan_dense_q8(gi, h0, Wh_cat, bh_cat, *, weight_bits: int = 8, h_in_quant=None, h_out_quant=None):
    """Differentiable dense scan on the RAW fp32 weights ``Wh_cat[3H,H]``: the per-output-row
    int8 fake-quant (dynamic symmetric scale) happens on the device and its straight-through
    gradient is applied in the backward.  Equals ``gru_scan_persistent`` on
    ``GRUCellQuant.quantize_weights().Wh_cat`` of a layer with an int8 per-channel weight recipe."""
    from ._scan_common import check_quant, common_shapes, require_cuda, require_f32
    require_cuda(gi=gi, h0=h0, Wh_cat=Wh_cat, bh_cat=bh_cat)
    require_f32(gi=gi, h0=h0, Wh_cat=Wh_cat, bh_cat=bh_cat)
    T, B, H = common_shapes(gi, h0, bh_cat)
    if tuple(Wh_cat.shape) != (3 * H, H):
        raise ValueError(f"Wh_cat shape must be (3H, H)=({3 * H}, {H}); got {tuple(Wh_cat.shape)}")
    if H % 4:
        raise ValueError("int8 weight preparation needs H % 4 == 0")
    check_quant("h_in_quant", h_in_quant)
    check_quant("h_out_quant", h_out_quant)
    return GRUScanDenseQ8Function.apply(gi, h0, Wh_cat, bh_cat, int(weight_bits), h_in_quant, h_out_quant)
