"""Ulysses sequence parallelism around ``vsa_attention``, alone or combined with the ring.

Each of the ``U`` ranks of a Ulysses group holds a slice of ``A`` consecutive rows of the token
stream (raster order without a ring, this ring owner's compact block order with one) and all
``H`` heads.  Before attention an all-to-all turns that into every row of the stream and ``H/U``
heads; after attention the reverse exchange brings the rows home.  The reference keeps this in
caller code (``README.md:294-505``, ``exchange_heads`` / ``exchange_tokens`` of its demo); here it
is a small module with the same semantics so that the composition can be tested:

* :func:`ulysses_plan` - rows per rank ``A``, the transport padding at the tail of the stream
  and which local rows are real (the padding only equalises message sizes; it is removed before
  attention and is separate from the 64-slot block padding inside ``vsa_attention``);
* :func:`exchange_heads` / :func:`exchange_tokens` - the two differentiable all-to-alls (NCCL on
  GPUs, any ``torch.distributed`` backend otherwise); the backward of each is the other exchange
  applied to the gradient;
* :func:`ulysses_attention` - exchange, trim, ``vsa_attention`` on ``H/U`` heads, pad, exchange back.

The layout passed to ``vsa_attention`` is built with ``head_num = H // U`` and, for Ring x Ulysses,
with the ring group of this rank (ranks that share a head slice and own complementary blocks).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .vsa import vsa_attention


@dataclass(frozen=True)
class UlyssesPlan:
    """Row bookkeeping of one Ulysses rank (reference demo, ``README.md:459-470``)."""
    size: int        # U
    rank: int        # position inside the Ulysses group
    rows: int        # A: rows per rank, transport padding included
    tokens: int      # rows of the stream that are real (layout.tokens)
    tail: int        # U * A - tokens
    start: int       # first stream row of this rank

    @property
    def valid(self):
        """Boolean ``[A]``: which local rows hold real tokens."""
        return torch.arange(self.start, self.start + self.rows) < self.tokens


def ulysses_plan(layout, ulysses_size, ulysses_rank):
    """Split the stream that ``vsa_attention`` sees on this ring owner into ``U`` equal slices.

    With a ring every owner's stream may have a different length; all ranks of the job must use
    the same ``A`` so that messages match, hence the maximum over the owners."""
    if ulysses_size < 1 or not 0 <= ulysses_rank < ulysses_size:
        raise ValueError("ulysses_size must be positive and 0 <= ulysses_rank < ulysses_size")
    longest = layout.tokens
    if layout.ring is not None:
        longest = int(layout.ring.peer_block_sizes.sum(dim=1).max().item())
    rows = -(-longest // ulysses_size)
    return UlyssesPlan(ulysses_size, ulysses_rank, rows, layout.tokens, ulysses_size * rows - layout.tokens,
                       ulysses_rank * rows)


def local_slice(stream, plan, fill=0):
    """This rank's ``[A, ...]`` slice of a full ``[tokens, ...]`` stream, tail-padded with ``fill``."""
    if stream.shape[0] != plan.tokens:
        raise ValueError("the stream must hold layout.tokens rows")
    pad = [0, 0] * (stream.dim() - 1) + [0, plan.tail]
    return F.pad(stream, pad, value=fill)[plan.start:plan.start + plan.rows].contiguous()


def _all_to_all(send, group):
    receive = torch.empty_like(send)
    dist.all_to_all_single(receive, send, group=group)
    return receive


class _HeadExchange(torch.autograd.Function):
    """``[A, H, ...] -> [U*A, H/U, ...]``: rows of every rank, this rank's heads."""

    @staticmethod
    def forward(ctx, x, group):
        size = dist.get_world_size(group)
        rows, heads = x.shape[0], x.shape[1]
        if heads % size:
            raise ValueError("the head count must be divisible by the Ulysses size")
        ctx.group, ctx.size = group, size
        send = x.reshape(rows, size, heads // size, *x.shape[2:]).transpose(0, 1).contiguous()  # [U, A, H/U, ...]
        return _all_to_all(send, group).reshape(size * rows, heads // size, *x.shape[2:])

    @staticmethod
    def backward(ctx, grad):
        return _TokenExchange.apply(grad.contiguous(), ctx.group), None


class _TokenExchange(torch.autograd.Function):
    """``[U*A, H/U, ...] -> [A, H, ...]``: this rank's rows, every head."""

    @staticmethod
    def forward(ctx, x, group):
        size = dist.get_world_size(group)
        total, heads = x.shape[0], x.shape[1]
        if total % size:
            raise ValueError("the row count must be divisible by the Ulysses size")
        ctx.group = group
        send = x.reshape(size, total // size, heads, *x.shape[2:]).contiguous()           # [U, A, H/U, ...]
        receive = _all_to_all(send, group)                                                  # [U, A, H/U, ...] by head slice
        return receive.transpose(0, 1).reshape(total // size, size * heads, *x.shape[2:])

    @staticmethod
    def backward(ctx, grad):
        return _HeadExchange.apply(grad.contiguous(), ctx.group), None


def exchange_heads(x, group):
    """``[A, H, ...]`` on every rank -> ``[U*A, H/U, ...]``; identity without a group."""
    return x if group is None else _HeadExchange.apply(x.contiguous(), group)


def exchange_tokens(x, group):
    """``[U*A, H/U, ...]`` -> ``[A, H, ...]``, the inverse of :func:`exchange_heads`."""
    return x if group is None else _TokenExchange.apply(x.contiguous(), group)


def ulysses_attention(mixed, layout, plan, group, *, scale=None):
    """``vsa_attention`` under Ulysses parallelism.

    ``mixed`` is ``[A, H, 4, 128]``: q, k, v and gate of this rank's rows for all heads (the caller's
    fused projection output).  Returns ``[A, H, 128]``; rows of the transport padding come back zero.
    """
    if mixed.dim() != 4 or mixed.shape[0] != plan.rows or mixed.shape[2] != 4:
        raise ValueError("mixed must be [plan.rows, H, 4, D]")
    full = exchange_heads(mixed, group)                                  # [U*A, H/U, 4, D]
    q, k, v, gate = (t[:plan.tokens].contiguous() for t in full.unbind(2))
    out = vsa_attention(q, k, v, gate, layout, scale=scale)              # [tokens, H/U, D]
    out = F.pad(out, (0, 0, 0, 0, 0, plan.tail))                         # [U*A, H/U, D]
    return exchange_tokens(out, group)
