"""Matrix products of the parts: picks the kernel for a product's types and sizes.

float32 anywhere in the operands -> the plain FFMA kernel (true 32-bit, no tensor cores).
bfloat16 x bfloat16 -> the tcgen05 kernel when its size rules hold, else the plain kernel.
"""
from __future__ import annotations

import torch

from ..csrc import ops

# Products with at most this many rows take the weight-streaming kernel (0: never; at most ops.SKINNY_MAX_ROWS),
# unless the matrix is so large that the tensor-core kernel's deep ring streams it faster (measured: 6.2 against
# 4.3 TB/s on a 622 MB output head, 2.5 against 3.5 TB/s on a 25 MB projection).
SKINNY_ROWS = ops.SKINNY_MAX_ROWS
SKINNY_MAX_BYTES = 128 << 20


def linear(ctx, a, w, out_dtype, *, bias=None, a_rows=None, swiglu=False, M=None, out=None):
    """``out = a[a_rows] @ w.T (+ bias)``; with ``swiglu`` w is [2N, K] (gate rows, then up rows)
    and ``out = silu(a @ gate.T) * (a @ up.T)``."""
    rows_w = w.shape[0]
    N = rows_w // 2 if swiglu else rows_w
    if M is None:
        M = a_rows.numel() if a_rows is not None else a.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if M == 0:
        return out
    if (ctx.fast_kernels and M <= SKINNY_ROWS and w.numel() * w.element_size() <= SKINNY_MAX_BYTES
            and ops.skinny_usable(a, w, M, swiglu)):
        # a handful of rows: the product is a stream of w, and the kernel without tiles starts it soonest
        if a_rows is not None:
            a = ops.permute_rows(a, a_rows, M)
        ops.skinny_gemm(a, w, out, bias=bias, swiglu=swiglu, rows=M, err=ctx.err)
        return out
    if ctx.fast_kernels and ops.gemm_fast_usable(a, w, out, bias=bias, a_rows=a_rows, swiglu=swiglu):
        ops.gemm_fast(a, w, out, bias=bias, a_rows=a_rows, swiglu=swiglu, M=M, err=ctx.err)
    else:
        ops.gemm_plain(a, w, out, bias=bias, a_rows=a_rows, swiglu=swiglu, M=M)
    return out


def small_linear(ctx, a32, w):
    """float32 rows times a short matrix, float32 out: router logits and gate logits."""
    out = torch.empty((a32.shape[0], w.shape[0]), dtype=torch.float32, device=a32.device)
    if a32.shape[0]:
        # float32 runs keep one kernel whatever the batch is; bfloat16 runs take the many-rows kernel for prompts
        ops.rowdot(a32, w, out, wide=ctx.fast_kernels and ctx.act_dtype == torch.bfloat16 and a32.shape[0] >= 256)
    return out


def grouped_linear(ctx, a, w, out_dtype, align, *, a_rows=None, swiglu=False, tiles=None, tiles_ready=False, out=None,
                   counter=None):
    """Per-expert product over an expert-sorted row list: row r of the output belongs to the expert
    whose segment of ``align`` holds r and is ``a[a_rows[r]] @ w[expert].T``.  ``counter``: see
    ``ops.gemm_fast_grouped`` (tensor-core path only)."""
    rows_w = w.shape[1]
    N = rows_w // 2 if swiglu else rows_w
    if out is None:
        out = torch.empty((align.TK, N), dtype=out_dtype, device=a.device)
    if align.TK == 0:
        return out
    if ctx.fast_kernels and ops.gemm_fast_usable(a, w, out, a_rows=a_rows, swiglu=swiglu, grouped=True):
        ops.gemm_fast_grouped(a, w, out, align, a_rows=a_rows, swiglu=swiglu, err=ctx.err, tiles=tiles,
                              tiles_ready=tiles_ready, counter=counter)
    else:
        ops.gemm_plain(a, w, out, a_rows=a_rows, swiglu=swiglu, M=align.TK, tiles=align.tiles)
    return out
