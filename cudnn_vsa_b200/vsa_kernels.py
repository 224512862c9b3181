"""Row-movement operators of the VSA path, backed by the sm_100a row gather/scatter kernels.

Mirrors the tensor-op surface of the reference's ``vsa_kernels.py``: ``reorder_tokens``
(:11-63), ``gather`` / ``SlotGather`` and the four padded-slot helpers (:66-116).  Pooling,
routing, attention and the gate merge are fused into larger kernels and live in
``vsa_core``.  All functions need CUDA tensors; there is no CPU path.
"""
from __future__ import annotations

import math

import torch

from . import _cabi
from .vsa_layout import BLOCK  # noqa: F401  (re-exported like the reference module)


def _row_bytes(x):
    return math.prod(x.shape[1:]) * x.element_size()


def _need_cuda(x, what):
    if not x.is_cuda:
        raise ValueError(f"{what} requires a CUDA tensor; this build has no CPU path")


def gather(x, row_map):
    """``out[i] = x[row_map[i]]``, zero where ``row_map[i] < 0`` (reference ``vsa_kernels.py:76-83``)."""
    _need_cuda(x, "gather")
    x = x.contiguous()
    out = torch.empty((row_map.numel(), *x.shape[1:]), device=x.device, dtype=x.dtype)
    if out.numel():
        _cabi.call("vsa_row_gather", _cabi.ptr(x), _cabi.ptr(row_map), _cabi.ptr(out),
                   row_map.numel(), _row_bytes(x), _cabi.stream())
    return out


def _reorder_rows(x, input_rows, inverse, output_tokens):
    """Unique-row gather (forward) or its scatter adjoint (reference ``vsa_kernels.py:29-42``)."""
    _need_cuda(x, "reorder_tokens")
    x = x.contiguous()
    listed = input_rows.numel()
    if not inverse:
        out = x.new_empty((listed, *x.shape[1:]))
        if out.numel():
            _cabi.call("vsa_row_gather", _cabi.ptr(x), _cabi.ptr(input_rows), _cabi.ptr(out),
                       listed, _row_bytes(x), _cabi.stream())
        return out
    shape = (output_tokens, *x.shape[1:])
    # A shard's adjoint leaves unowned rows untouched, so they must start at zero; a full
    # permutation writes every row.
    out = x.new_zeros(shape) if output_tokens != listed else x.new_empty(shape)
    if listed and out.numel():
        _cabi.call("vsa_row_scatter", _cabi.ptr(x), _cabi.ptr(input_rows), _cabi.ptr(out),
                   listed, _row_bytes(x), _cabi.stream())
    return out


class _TokenReorder(torch.autograd.Function):
    """Differentiable to any order: the backward is the same operator, inverted."""

    @staticmethod
    def forward(ctx, x, input_rows, inverse, output_tokens):
        ctx.save_for_backward(input_rows)
        ctx.inverse, ctx.input_tokens = inverse, x.shape[0]
        return _reorder_rows(x, input_rows, inverse, output_tokens)

    @staticmethod
    def backward(ctx, grad):
        input_rows, = ctx.saved_tensors
        return (reorder_tokens(grad, input_rows, inverse=not ctx.inverse,
                               output_tokens=ctx.input_tokens), None, None, None)


def reorder_tokens(x, input_rows, *, inverse=False, output_tokens=None):
    """Gather the unique rows ``input_rows`` of ``x``, or scatter rows back to them
    (reference ``vsa_kernels.py:60-63``)."""
    output_tokens = x.shape[0] if output_tokens is None else output_tokens
    return _TokenReorder.apply(x, input_rows, inverse, output_tokens)


class SlotGather(torch.autograd.Function):
    """Gather through one map; the adjoint is a gather through the inverse map
    (reference ``vsa_kernels.py:86-96``)."""

    @staticmethod
    def forward(ctx, x, row_map, inverse_map):
        ctx.save_for_backward(inverse_map)
        return gather(x, row_map)

    @staticmethod
    def backward(ctx, grad):
        inverse_map, = ctx.saved_tensors
        return gather(grad, inverse_map), None, None


def raster_to_block_w_padding(x, slot_row, row_slot):
    """Raster rows -> zero-padded 64-slot blocks (maps of a raster layout)."""
    return SlotGather.apply(x, slot_row, row_slot)


def block_w_padding_to_raster(x, slot_row, row_slot):
    """Drop block padding and restore raster order (maps of a raster layout)."""
    return SlotGather.apply(x, row_slot, slot_row)


def block_wo_padding_to_block_w_padding(x, slot_row, row_slot):
    """Compact block order -> zero-padded blocks (maps of a block layout)."""
    return SlotGather.apply(x, slot_row, row_slot)


def block_w_padding_to_block_wo_padding(x, slot_row, row_slot):
    """Drop block padding, keeping compact block order (maps of a block layout)."""
    return SlotGather.apply(x, row_slot, slot_row)
