"""Execution core of the B200 VSA path: one autograd function around the fused CUDA kernels.

Forward (one stream, no host synchronisation, CUDA-graph capturable):

1. ``vsa_slots_pool``  Q/K/V rows -> zero-padded slot tensors + FP32 block means + BF16 block
   tokens laid out as the coarse streams (reference ``vsa.py:96-104``, ``vsa_kernels.py:161-188``).
2. ``vsa_route``       FP32 pooled scores and top-k per video region, written into a clone of
   the layout's routing template (reference ``vsa_core.py:61-84``).
3. ``vsa_fine_fwd`` on the block tokens = coarse attention; the same tcgen05 kernel runs it as
   block-sparse attention whose lists name every 64-token chunk of the sample
   (reference ``vsa_core.py:87-97``).
4. ``vsa_fine_fwd`` on the slots with the merge epilogue: fine output, LSE and
   ``out = fine + gate * coarse[block]`` in the caller's row order
   (reference ``vsa_core.py:15-40``, ``vsa.py:111-117``, ``vsa_kernels.py:191-201``).

Backward: ``vsa_merge_bwd`` (dO -> slots, dgate, dcoarse, delta), ``vsa_fine_bwd`` on the block
tokens (coarse adjoint), ``vsa_fine_bwd`` on the slots whose epilogues add the pooled-mean
gradient and scatter dq/dk/dv to the caller's rows.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import _cabi
from .vsa_layout import BLOCK

# Upper bound of the routing score scratch; heads are processed in passes when it is reached.
ROUTE_SCRATCH_BYTES = 1 << 30


@dataclass
class _CoarsePlan:
    """Coarse attention as block-sparse attention over the pooled block tokens.

    Block tokens of each VSA sample occupy consecutive rows of a stream padded to a multiple
    of 64 per sample; every 64-row chunk lists all chunks of its sample.
    """
    q_rows: int                 # rows of the query stream (multiple of 64)
    kv_rows: int                # rows of the key/value stream
    block_q: torch.Tensor       # int32 [blocks]: query-stream row of each local block, -1 = none
    block_kv: torch.Tensor      # int32 [kv source blocks]: kv-stream row, -1 = none
    index: torch.Tensor         # int32 [q_rows/64, cap]
    counts: torch.Tensor        # int32 [q_rows/64]
    kv_sizes: torch.Tensor      # int32 [kv_rows/64]
    q_sizes: torch.Tensor       # int32 [q_rows/64]
    q_src: torch.Tensor         # int64 [q_rows]: local block whose token sits in each row, -1 = padding
    kv_src: torch.Tensor        # int64 [kv_rows]: source (global) block of each row, -1 = padding
    block_kv_rows: torch.Tensor  # block_kv as an int64 row map for the row-gather kernel


@dataclass
class _DevicePlan:
    coarse: _CoarsePlan | None
    spans: tuple                # (q_begin, q_end, kv_first, kv_last, keep, cursor) per region needing top-k
    status: torch.Tensor        # int32 [1] device error word shared by the kernels of this layout
    sizes: torch.Tensor | None  # block sizes, or None when every block is full
    early_kv: tuple = ()        # ring: per owner, leading always-visible KV blocks to schedule first


def _coarse_plan(pairs, q_blocks, kv_blocks, device):
    """``pairs``: per VSA sample ``(q_begin, q_end, kv_begin, kv_end)`` in block ids."""
    block_q = np.full(q_blocks, -1, dtype=np.int32)
    block_kv = np.full(kv_blocks, -1, dtype=np.int32)
    lists, q_sizes, kv_sizes = [], [], []
    q_chunks = kv_chunks = 0
    for q0, q1, k0, k1 in pairs:
        nq, nk = q1 - q0, k1 - k0
        cq, ck = -(-nq // BLOCK), -(-nk // BLOCK)
        block_q[q0:q1] = q_chunks * BLOCK + np.arange(nq, dtype=np.int32)
        block_kv[k0:k1] = kv_chunks * BLOCK + np.arange(nk, dtype=np.int32)
        lists += [np.arange(kv_chunks, kv_chunks + ck, dtype=np.int32)] * cq
        q_sizes += [BLOCK] * (cq - 1) + [nq - BLOCK * (cq - 1)] if cq else []
        kv_sizes += [BLOCK] * (ck - 1) + [nk - BLOCK * (ck - 1)] if ck else []
        q_chunks += cq
        kv_chunks += ck
    cap = max((len(x) for x in lists), default=1)
    index = np.zeros((max(q_chunks, 1), max(cap, 1)), dtype=np.int32)
    counts = np.zeros(max(q_chunks, 1), dtype=np.int32)
    for i, ids in enumerate(lists):
        index[i, :len(ids)] = ids
        counts[i] = len(ids)

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(device)

    def inverse(rows_of_block, rows):
        src = np.full(rows, -1, dtype=np.int64)
        used = rows_of_block >= 0
        src[rows_of_block[used]] = np.nonzero(used)[0]
        return src
    return _CoarsePlan(q_src=dev(inverse(block_q, q_chunks * BLOCK)), kv_src=dev(inverse(block_kv, kv_chunks * BLOCK)),
                       q_rows=q_chunks * BLOCK, kv_rows=kv_chunks * BLOCK, block_q=dev(block_q),
                       block_kv=dev(block_kv), block_kv_rows=dev(block_kv.astype(np.int64)), index=dev(index),
                       counts=dev(counts),
                       kv_sizes=dev(np.asarray(kv_sizes or [0], dtype=np.int32)),
                       q_sizes=dev(np.asarray(q_sizes or [0], dtype=np.int32)))


def _early_kv_blocks(layout):
    """Ring layouts: for each owner, how many of its leading block slots hold always-visible
    (dense) blocks of the first sample.  (On a single device the hint was measured at 2, 4 and 24
    heads and changes nothing: there the long CTAs of one head finish under the next head's work.)  Every local query block of that sample lists them at
    every ring step, so their dK/dV CTAs run far longer than the others and are started first
    (``vsa_fine_bwd``'s scheduling hint).  0 where the dense blocks are not at the front."""
    ring = layout.ring
    if ring is None or not ring.local_groups:
        return ()
    group = ring.local_groups[0][0]
    if group.dense_only or not group.dense_blocks_num:
        return (0,) * ring.size
    capacity = ring.peer_block_sizes.shape[1]
    where = ring.global_to_gather[group.start:group.start + group.dense_blocks_num].cpu().numpy()
    owners, local = where // capacity, where % capacity
    out = []
    for owner in range(ring.size):
        ids = np.sort(local[owners == owner])
        out.append(int(len(ids)) if len(ids) and np.array_equal(ids, np.arange(len(ids))) else 0)
    return tuple(out)


def device_plan(layout):
    """Derived device metadata of a layout, built once and cached on the layout object."""
    plan = getattr(layout, "_b200_plan", None)
    if plan is not None:
        return plan
    device = layout.block_sizes.device
    spans = []
    for group, begin, end, _ in layout.routing_groups:
        cursor = group.dense_blocks_num
        for first, last, keep in group.video_spans:
            if keep < last - first:
                spans.append((begin, end, first, last, keep, cursor))
            cursor += keep
    coarse = None
    if not layout.dense_only:
        if layout.ring is None:
            pairs = [(g.start, g.end, g.start, g.end) for g in layout.groups if not g.dense_only]
            coarse = _coarse_plan(pairs, layout.blocks, layout.blocks, device)
        else:
            pairs = [(b, e, g.start, g.end) for g, b, e, _ in layout.ring.local_groups if not g.dense_only]
            coarse = _coarse_plan(pairs, layout.blocks, layout.ring.global_to_gather.numel(), device)
    plan = _DevicePlan(coarse=coarse, spans=tuple(spans),
                       status=torch.zeros(1, dtype=torch.int32, device=device),
                       sizes=None if layout.all_blocks_full else layout.block_sizes,
                       early_kv=_early_kv_blocks(layout))
    layout._b200_plan = plan
    return plan


def check_status(layout):
    """Raise if a kernel of this layout reported a bounded wait that gave up (synchronises)."""
    code = int(device_plan(layout).status.item())
    if code:
        raise RuntimeError(f"VSA kernel reported device error {code} (a bounded wait timed out)")


def _p(t):
    return _cabi.ptr(t)


def route(q_mean, k_mean, layout, plan=None):
    """Routing table for the current Q/K: the layout's template with every region that needs
    selection filled by the top-``keep`` pooled scores, ascending (reference ``vsa_core.py:75-84``).

    ``q_mean`` is ``[local blocks, H, 128]`` and ``k_mean`` ``[global blocks, H, 128]`` float32,
    both indexed by block id.  Returns the template itself when nothing needs selection.
    """
    plan = device_plan(layout) if plan is None else plan
    if not plan.spans:
        return layout.routing_indices
    index = layout.routing_indices.clone()
    heads, cap = layout.head_num, index.shape[-1]
    need = max(_cabi.load().vsa_route_scratch_bytes(qe - qb, kl - kf, heads)
               for qb, qe, kf, kl, _, _ in plan.spans)
    per_head = need // heads
    scratch = torch.empty(max(per_head, min(need, ROUTE_SCRATCH_BYTES)), dtype=torch.uint8,
                          device=index.device)
    for q_begin, q_end, kv_first, kv_last, keep, cursor in plan.spans:
        per_head = max(1, (q_end - q_begin) * (kv_last - kv_first) * 4)
        passes = -(-heads // max(1, min(heads, scratch.numel() // per_head)))
        _cabi.call("vsa_route", _p(q_mean), _p(k_mean), heads, q_begin, q_end, 0, kv_first, kv_last, 0,
                   keep, cursor, _p(index), index.stride(1), cap, _p(scratch), scratch.numel(),
                   _cabi.stream(), launches=2 * passes)
    return index


def routing_table(q, k, layout):
    """Routing table ``[1, H, B, cap]`` that a single-device forward pass on ``q, k`` (caller row
    order) uses.  Pooling and selection are deterministic, so this reproduces the table of an
    earlier call on the same inputs; benchmarks count useful FLOPs from it and tests hand it to
    the oracle (reference ``vsa_core.py:75-84`` on the means of ``vsa_kernels.py:179-188``)."""
    plan = device_plan(layout)
    if not plan.spans:
        return layout.routing_indices
    heads, dim = q.shape[1], q.shape[2]
    mean = torch.empty((3, layout.blocks, heads, dim), dtype=torch.float32, device=q.device)
    _cabi.call("vsa_slots_pool", _p(q), _p(k), _p(k), None if layout.slots_are_input else _p(layout.slot_row),
               _p(layout.block_sizes), None, None, None, _p(mean), None, None, 0, layout.blocks, heads,
               _cabi.stream())
    return route(mean[0], mean[1], layout, plan)


def _fine_fwd(q, k, v, index, counts, head_strides, kv_sizes, scale, status, *, merge=None):
    """Launch the block-sparse forward; returns ``(o_slots, lse[, out])``."""
    q_blocks, heads = q.shape[0] // BLOCK, q.shape[1]
    o = torch.empty_like(q)
    lse = torch.empty((heads, q.shape[0]), dtype=torch.float32, device=q.device)
    out = None
    slot_row = block_coarse = gate = coarse = None
    out_rows = 0
    if merge is not None:
        slot_row, block_coarse, gate, coarse, out_rows = merge
        out = torch.empty((out_rows, heads, q.shape[2]), dtype=q.dtype, device=q.device)
    _cabi.call("vsa_fine_fwd", _p(q), _p(k), _p(v), q_blocks, k.shape[0] // BLOCK, heads, _p(index),
               _p(counts), head_strides[0], head_strides[1], index.shape[-1], _p(kv_sizes), scale,
               _p(o), _p(lse), _p(slot_row), _p(block_coarse), _p(gate), _p(coarse), _p(out), out_rows,
               _p(status), _cabi.stream())
    return (o, lse) if merge is None else (o, lse, out)


def _fine_bwd(q, k, v, d_o, index, counts, head_strides, q_sizes, kv_sizes, scale, lse, delta, status, *,
              out_rows=None, q_slot_row=None, kv_slot_row=None, pools=None, q_block_coarse=None,
              kv_block_coarse=None):
    """Launch both backward kernels; returns BF16 ``(dq, dk, dv)`` in output-row order."""
    heads = q.shape[1]
    q_blocks, kv_blocks = q.shape[0] // BLOCK, k.shape[0] // BLOCK
    q_rows, kv_rows = (q.shape[0], k.shape[0]) if out_rows is None else out_rows
    dq = torch.empty((q_rows, heads, q.shape[2]), dtype=q.dtype, device=q.device)
    dk = torch.empty((kv_rows, heads, q.shape[2]), dtype=q.dtype, device=q.device)
    dv = torch.empty_like(dk)
    words = _cabi.load().vsa_kv_mask_words(q_blocks)
    mask = torch.empty(heads * kv_blocks * words, dtype=torch.int32, device=q.device)
    dq_pool, dk_pool, dv_pool = pools if pools is not None else (None, None, None)
    _cabi.call("vsa_fine_bwd", _p(q), _p(k), _p(v), _p(d_o), q_blocks, kv_blocks, heads, _p(index), _p(counts),
               head_strides[0], head_strides[1], index.shape[-1], _p(q_sizes), _p(kv_sizes), scale, _p(lse),
               _p(delta), _p(mask), _p(dq), _p(dk), _p(dv), q_rows, kv_rows, _p(q_slot_row), _p(kv_slot_row),
               _p(dq_pool), _p(dk_pool), _p(dv_pool), 0, _p(q_block_coarse), _p(kv_block_coarse), None, None,
               None, 0, 7, _p(status), _cabi.stream(), launches=3)
    return dq, dk, dv


class _VSAFunction(torch.autograd.Function):
    """Single-device VSA: ``out[T,H,128] = fine + gate * coarse`` with all gradients."""

    @staticmethod
    def forward(ctx, q, k, v, gate, layout, scale):
        plan = device_plan(layout)
        tokens, heads, dim = q.shape
        width = heads * dim
        blocks = layout.blocks
        identity = layout.slots_are_input
        coarse = plan.coarse
        need_means = bool(plan.spans)
        mean_f32 = (torch.empty((3, blocks, heads, dim), dtype=torch.float32, device=q.device)
                    if need_means else None)
        tokens_bf16 = (torch.zeros((3, coarse.q_rows, heads, dim), dtype=q.dtype, device=q.device)
                       if coarse is not None else None)
        if identity:
            q_s, k_s, v_s = q, k, v
        else:
            q_s, k_s, v_s = (torch.empty((blocks * BLOCK, heads, dim), dtype=q.dtype, device=q.device)
                             for _ in range(3))
        if not identity or need_means or coarse is not None:
            _cabi.call("vsa_slots_pool", _p(q), _p(k), _p(v), None if identity else _p(layout.slot_row),
                       _p(layout.block_sizes), None if identity else _p(q_s), None if identity else _p(k_s),
                       None if identity else _p(v_s), _p(mean_f32),
                       _p(coarse.block_q) if coarse is not None else None, _p(tokens_bf16),
                       coarse.q_rows if coarse is not None else 0, blocks, heads, _cabi.stream())
        index = route(mean_f32[0], mean_f32[1], layout, plan) if need_means else layout.routing_indices
        coarse_o = coarse_lse = None
        merge = (None if identity else layout.slot_row, None, None, None, tokens)
        if coarse is not None:
            coarse_o, coarse_lse = _fine_fwd(tokens_bf16[0], tokens_bf16[1], tokens_bf16[2], coarse.index,
                                             coarse.counts, (0, 0), coarse.kv_sizes, scale, plan.status)
            merge = (merge[0], coarse.block_q, gate, coarse_o, tokens)
        counts = layout.routing_counts
        from . import vsa_ring  # the pass machinery of the ring steps (imported here: it imports this module)
        bounds, passes = vsa_ring.list_bounds(index, counts, blocks)
        if bounds is None:
            o_s, lse, out = _fine_fwd(q_s, k_s, v_s, index, counts, (index.stride(1), counts.stride(1)),
                                      plan.sizes, scale, plan.status, merge=merge)
        else:
            # K and V of one head do not fit L2: passes over KV ranges into a running FP32 output,
            # exactly like the steps of a ring over one shard (vsa_ring.py).
            out_f32 = torch.zeros((blocks * BLOCK, heads, dim), dtype=torch.float32, device=q.device)
            lse = torch.full((heads, blocks * BLOCK), float("-inf"), dtype=torch.float32, device=q.device)
            flat = bounds[0].flatten()
            for c in range(passes):
                _cabi.call("vsa_fine_fwd_running_range", _p(q_s), _p(k_s), _p(v_s), blocks, blocks, heads, _p(index),
                           _p(flat[c:]), index.stride(1), counts.stride(1), passes + 1, index.shape[-1],
                           _p(plan.sizes), scale, _p(out_f32), _p(lse), _p(plan.status), _cabi.stream())
            o_s = torch.empty((blocks * BLOCK, heads, dim), dtype=q.dtype, device=q.device)
            out = torch.empty((tokens, heads, dim), dtype=q.dtype, device=q.device)
            _cabi.call("vsa_gate_merge", _p(out_f32), _p(merge[0]), _p(merge[1]), _p(merge[2]), _p(merge[3]), _p(o_s),
                       _p(out), blocks, heads, tokens, _cabi.stream())
        ctx.save_for_backward(q_s, k_s, v_s, o_s, lse, index, gate if coarse is not None else None,
                              tokens_bf16, coarse_o, coarse_lse, bounds)
        ctx.layout, ctx.scale, ctx.passes = layout, scale, passes
        return out

    @staticmethod
    def backward(ctx, grad):
        q_s, k_s, v_s, o_s, lse, index, gate, tokens_bf16, coarse_o, coarse_lse, bounds = ctx.saved_tensors
        layout, scale = ctx.layout, ctx.scale
        plan = device_plan(layout)
        coarse = plan.coarse
        grad = grad.contiguous()
        tokens, heads, dim = grad.shape
        blocks = layout.blocks
        identity = layout.slots_are_input
        slot_row = None if identity else layout.slot_row
        grad_s = grad if identity else torch.empty_like(q_s)
        delta = torch.empty((heads, blocks * BLOCK), dtype=torch.float32, device=grad.device)
        dgate = dcoarse = coarse_delta = None
        if coarse is not None:
            dgate = torch.empty_like(grad)
            dcoarse = torch.zeros_like(coarse_o)
            coarse_delta = torch.zeros((heads, coarse.q_rows), dtype=torch.float32, device=grad.device)
        _cabi.call("vsa_merge_bwd", _p(grad), _p(gate), _p(coarse_o), _p(o_s), _p(slot_row),
                   _p(coarse.block_q) if coarse is not None else None, None if identity else _p(grad_s),
                   _p(dgate), _p(dcoarse), _p(delta), _p(coarse_delta), blocks,
                   coarse.q_rows if coarse is not None else 0, heads, _cabi.stream())
        pools = None
        if coarse is not None:
            pools = _fine_bwd(tokens_bf16[0], tokens_bf16[1], tokens_bf16[2], dcoarse, coarse.index,
                              coarse.counts, (0, 0), coarse.q_sizes, coarse.kv_sizes, scale, coarse_lse,
                              coarse_delta, plan.status)
        counts = layout.routing_counts
        if bounds is None:
            dq, dk, dv = _fine_bwd(q_s, k_s, v_s, grad_s, index, counts, (index.stride(1), counts.stride(1)),
                                   layout.block_sizes, plan.sizes, scale, lse, delta, plan.status,
                                   out_rows=(tokens, tokens), q_slot_row=slot_row, kv_slot_row=slot_row,
                                   pools=pools, q_block_coarse=coarse.block_q if coarse is not None else None,
                                   kv_block_coarse=coarse.block_q if coarse is not None else None)
            return dq, dk, dv, dgate, None, None
        # Large layout: FP32 gradients in slot order, dQ in passes over KV ranges, dK / dV in passes
        # over query-block ranges; pooled-mean terms, rounding and the row scatter at the end.
        from . import vsa_ring
        sums = torch.zeros((3, blocks * BLOCK, heads, dim), dtype=torch.float32, device=grad.device)
        words = _cabi.load().vsa_kv_mask_words(blocks)
        mask = torch.empty(heads * blocks * words, dtype=torch.int32, device=grad.device)
        common = (q_s, k_s, v_s, grad_s, index[0], counts[0], layout.block_sizes, plan.sizes, scale, lse, delta, mask,
                  plan.status)
        vsa_ring._bwd_call(*common, parts=3, dq_f32=sums[0], accumulate=1, bounds=bounds[0], passes=ctx.passes)
        vsa_ring._bwd_call(*common, parts=4, dk_f32=sums[1], dv_f32=sums[2], accumulate=1)
        block_q = coarse.block_q if coarse is not None else None
        grads = []
        for acc, pool in zip(sums, pools if pools is not None else (None, None, None)):
            out = torch.empty_like(grad)
            _cabi.call("vsa_grad_finish", _p(acc), _p(slot_row), _p(pool), 0, _p(block_q) if pool is not None else None,
                       _p(layout.block_sizes), _p(out), blocks, heads, tokens, _cabi.stream())
            grads.append(out)
        return grads[0], grads[1], grads[2], dgate, None, None


def _field(mixed, n):
    """Device address of field ``n`` (0..3 = q, k, v, gate) of an interleaved ``[T, H, 4, D]`` tensor."""
    from ctypes import c_void_p
    return c_void_p(mixed.data_ptr() + n * mixed.shape[3] * mixed.element_size())


class _VSAFusedFunction(torch.autograd.Function):
    """Single-device VSA on an interleaved ``[T, H, 4, 128]`` projection output (q, k, v, gate per
    head).  The slot gather reads q, k and v straight out of it, the merge epilogue and its
    adjoint read the gate field in place, and the backward kernels write dq, dk, dv and dgate
    into the four fields of ONE gradient tensor: no ``.contiguous()`` of the four projections
    before the call and no concatenation of four gradients after it (the reference requires
    materialised contiguous inputs, ``vsa.py:50-61``).  Same kernels and arithmetic as
    :class:`_VSAFunction`, so results are bit-identical to the unfused call."""

    @staticmethod
    def forward(ctx, mixed, layout, scale):
        plan = device_plan(layout)
        tokens, heads, _, dim = mixed.shape
        blocks = layout.blocks
        row_stride, head_stride = heads * 4 * dim, 4 * dim
        coarse = plan.coarse
        need_means = bool(plan.spans)
        mean_f32 = (torch.empty((3, blocks, heads, dim), dtype=torch.float32, device=mixed.device)
                    if need_means else None)
        tokens_bf16 = (torch.zeros((3, coarse.q_rows, heads, dim), dtype=mixed.dtype, device=mixed.device)
                       if coarse is not None else None)
        q_s, k_s, v_s = (torch.empty((blocks * BLOCK, heads, dim), dtype=mixed.dtype, device=mixed.device)
                         for _ in range(3))
        slot_row = None if layout.slots_are_input else layout.slot_row
        _cabi.call("vsa_slots_pool_strided", _field(mixed, 0), _field(mixed, 1), _field(mixed, 2), row_stride,
                   head_stride, _p(slot_row), _p(layout.block_sizes), _p(q_s), _p(k_s), _p(v_s), _p(mean_f32),
                   _p(coarse.block_q) if coarse is not None else None, _p(tokens_bf16),
                   coarse.q_rows if coarse is not None else 0, blocks, heads, _cabi.stream())
        index = route(mean_f32[0], mean_f32[1], layout, plan) if need_means else layout.routing_indices
        coarse_o = coarse_lse = None
        if coarse is not None:
            coarse_o, coarse_lse = _fine_fwd(tokens_bf16[0], tokens_bf16[1], tokens_bf16[2], coarse.index,
                                             coarse.counts, (0, 0), coarse.kv_sizes, scale, plan.status)
        counts = layout.routing_counts
        o_s = torch.empty_like(q_s)
        lse = torch.empty((heads, blocks * BLOCK), dtype=torch.float32, device=mixed.device)
        out = torch.empty((tokens, heads, dim), dtype=mixed.dtype, device=mixed.device)
        _cabi.call("vsa_fine_fwd_strided", _p(q_s), _p(k_s), _p(v_s), blocks, blocks, heads, _p(index), _p(counts),
                   index.stride(1), counts.stride(1), index.shape[-1], _p(plan.sizes), scale, _p(o_s), _p(lse),
                   _p(slot_row), _p(coarse.block_q) if coarse is not None else None,
                   _field(mixed, 3) if coarse is not None else None, row_stride, head_stride, _p(coarse_o), _p(out),
                   tokens, _p(plan.status), _cabi.stream())
        ctx.save_for_backward(mixed, q_s, k_s, v_s, o_s, lse, index, tokens_bf16, coarse_o, coarse_lse)
        ctx.layout, ctx.scale = layout, scale
        return out

    @staticmethod
    def backward(ctx, grad):
        mixed, q_s, k_s, v_s, o_s, lse, index, tokens_bf16, coarse_o, coarse_lse = ctx.saved_tensors
        layout, scale = ctx.layout, ctx.scale
        plan = device_plan(layout)
        coarse = plan.coarse
        grad = grad.contiguous()
        tokens, heads, dim = grad.shape
        blocks = layout.blocks
        row_stride, head_stride = heads * 4 * dim, 4 * dim
        slot_row = None if layout.slots_are_input else layout.slot_row
        d_mixed = torch.empty_like(mixed)
        grad_s = torch.empty_like(q_s)
        delta = torch.empty((heads, blocks * BLOCK), dtype=torch.float32, device=grad.device)
        dcoarse = coarse_delta = None
        if coarse is not None:
            dcoarse = torch.zeros_like(coarse_o)
            coarse_delta = torch.zeros((heads, coarse.q_rows), dtype=torch.float32, device=grad.device)
        else:
            d_mixed[:, :, 3].zero_()  # a pack without coarse attention has no gate gradient
        _cabi.call("vsa_merge_bwd_strided", _p(grad), _field(mixed, 3) if coarse is not None else None, row_stride,
                   head_stride, _p(coarse_o), _p(o_s), _p(slot_row),
                   _p(coarse.block_q) if coarse is not None else None, _p(grad_s),
                   _field(d_mixed, 3) if coarse is not None else None, _p(dcoarse), _p(delta), _p(coarse_delta),
                   blocks, coarse.q_rows if coarse is not None else 0, heads, _cabi.stream())
        pools = (None, None, None)
        if coarse is not None:
            pools = _fine_bwd(tokens_bf16[0], tokens_bf16[1], tokens_bf16[2], dcoarse, coarse.index,
                              coarse.counts, (0, 0), coarse.q_sizes, coarse.kv_sizes, scale, coarse_lse,
                              coarse_delta, plan.status)
        counts = layout.routing_counts
        words = _cabi.load().vsa_kv_mask_words(blocks)
        mask = torch.empty(heads * blocks * words, dtype=torch.int32, device=grad.device)
        block_coarse = coarse.block_q if coarse is not None else None
        _cabi.call("vsa_fine_bwd_strided", _p(q_s), _p(k_s), _p(v_s), _p(grad_s), blocks, blocks, heads, _p(index),
                   _p(counts), index.stride(1), counts.stride(1), index.shape[-1], _p(layout.block_sizes),
                   _p(plan.sizes), scale, _p(lse), _p(delta), _p(mask), _field(d_mixed, 0), _field(d_mixed, 1),
                   _field(d_mixed, 2), row_stride, head_stride, tokens, tokens, _p(slot_row), _p(slot_row),
                   _p(pools[0]), _p(pools[1]), _p(pools[2]), 0, _p(block_coarse), _p(block_coarse), 7,
                   _p(plan.status), _cabi.stream(), launches=3)
        return d_mixed, None, None


def attention_fused(mixed, layout, *, scale=None):
    """Single-device packed VSA on validated interleaved inputs; see
    :func:`cudnn_vsa_b200.vsa.vsa_attention_fused`."""
    scale = mixed.shape[-1] ** -0.5 if scale is None else float(scale)
    return _VSAFusedFunction.apply(mixed, layout, scale)


def attention(q, k, v, gate, layout, *, scale=None):
    """Single-device packed VSA on validated inputs; see :func:`cudnn_vsa_b200.vsa.vsa_attention`."""
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    return _VSAFunction.apply(q, k, v, gate, layout, scale)


def ring_attention(q, k, v, gate, layout, *, scale=None):
    """Ring (context-parallel) VSA; see :mod:`cudnn_vsa_b200.vsa_ring`."""
    from . import vsa_ring
    return vsa_ring.ring_attention(q, k, v, gate, layout, scale=scale)
