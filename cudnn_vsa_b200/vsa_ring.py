"""Ring (context-parallel) execution of the VSA path over whole 64-slot blocks.

Each rank owns ``ceil(B / R)`` block slots (see ``build_vsa_layout(ring_cp_group=...)``).  Q, the
running output, LSE and dQ stay local; pooled K/V means are all-gathered so routing and coarse
attention are global; the padded K/V token shard travels around the ring while the block-sparse
kernels work on the shard that is already here (reference ``vsa_core.py:123-315``).

Schedule per forward step ``s`` (owner ``(rank - s) % R``): post the transfer of the current
shard to ``rank + 1`` on a private stream, run ``vsa_fine_fwd_running`` on it with the owner's
lists - its epilogue folds the step's partial result into the FP32 running output and LSE, so
no partial tensor is written and no merge pass runs - then join the transfer.  The backward pass
walks the ring in reverse starting from the last shard held.  The FP32 dK/dV sums travel with
their shard: each step posts the transfer, runs the dQ kernel (which adds into the running FP32
dQ) under it, joins, and then runs the dK/dV kernel, which adds this rank's contribution
straight into the buffer that just arrived; after ``R`` steps the sums are home.  No per-step
allocation, no separate accumulation pass.  Collectives are NCCL through the borrowed process
group; a remote shard always lands in this GPU's memory before any kernel reads it.

A step whose shard is larger than ``RING_CHUNK_BLOCKS`` blocks is run in passes.  K and V of one
head of such a shard do not fit the L2 cache, every CTA then streams its listed blocks from DRAM
and the SM clock drops under the power cap; a pass restricts all lists to one KV range of the
shard (lists are ascending, so that is a contiguous sub-range of each list, found once per call
by ``vsa_list_bounds``), which keeps the CTAs that run together on the same cache-resident part.
The forward and the dQ kernels take KV ranges; the dK/dV kernel, whose streaming side is Q and dO,
takes ranges of query blocks and adds the passes up in the FP32 sums.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _cabi
from .vsa_core import _fine_fwd, _p, device_plan, route
from .vsa_layout import BLOCK


# Largest number of 64-slot blocks one pass of a ring step covers (K and V of a head: 32 KiB per
# block, 64 MiB for 2048 blocks - about half of the L2 cache).
RING_CHUNK_BLOCKS = 2048


@dataclass
class _RingRuntime:
    group: object
    rank: int
    size: int
    stream: object          # private communication stream (None for CPU tensors)
    batch_p2p: bool
    peers: tuple            # global ranks of the group, in group order


def ring_runtime(layout, device):
    """Per-(device, transport) runtime cached on the layout's ring metadata
    (reference ``vsa_core.py:134-155``)."""
    ring = layout.ring
    batch_p2p = ring.batch_p2p
    if batch_p2p is None:
        # Groups bound to a device serialise single P2P calls on one communicator: batch them.
        batch_p2p = getattr(ring.group, "bound_device_id", None) is not None
    key = (str(device), batch_p2p)
    if key not in ring._runtime:
        # The transfers are short next to the kernels they hide under; on a high-priority stream
        # their CTAs are placed as soon as an SM frees up instead of queueing behind the grid of
        # the compute kernel that was launched right after them.
        stream = (torch.cuda.Stream(device=device, priority=-1)
                  if torch.device(device).type == "cuda" else None)
        ring._runtime[key] = _RingRuntime(ring.group, ring.rank, ring.size, stream, batch_p2p,
                                          tuple(dist.get_process_group_ranks(ring.group)))
    return ring._runtime[key]


def ring_exchange(runtime, pairs, *, reverse=False):
    """Send each ``pairs[i][0]`` to the next rank and receive ``pairs[i][1]`` from the previous one
    (directions swapped when ``reverse``), enqueued on the communication stream
    (reference ``vsa_core.py:158-184``).  The caller joins the stream before touching the buffers.
    Odd ranks post the receive first so that lazily created pair communicators cannot wait in a cycle.
    """
    step = -1 if reverse else 1
    to_peer = runtime.peers[(runtime.rank + step) % runtime.size]
    from_peer = runtime.peers[(runtime.rank - step) % runtime.size]
    ops = []
    for send, receive in pairs:
        pair = (dist.P2POp(dist.isend, send, to_peer, runtime.group),
                dist.P2POp(dist.irecv, receive, from_peer, runtime.group))
        ops.extend(pair if runtime.rank % 2 == 0 else pair[::-1])

    def post():
        works = dist.batch_isend_irecv(ops) if runtime.batch_p2p else [op.op(op.tensor, op.peer, op.group)
                                                                       for op in ops]
        for work in works:
            work.wait()

    if runtime.stream is None:
        post()
        return
    runtime.stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(runtime.stream):
        post()


def join_exchange(runtime):
    if runtime.stream is not None:
        with _cabi.mark("ring_exchange_wait"):
            torch.cuda.current_stream().wait_stream(runtime.stream)


def gather_means(k_mean, v_mean, runtime, global_to_gather):
    """All-gather FP32 K means and BF16 V means in one collective and return them in global block
    order (reference ``vsa_core.py:187-204, 296-297``).  The two fields travel as raw bytes."""
    v_mean = v_mean.to(torch.bfloat16)
    if runtime.size == 1:
        return k_mean, v_mean
    key_bytes = k_mean.shape[-1] * 4
    packed = torch.cat((k_mean.contiguous().view(torch.uint8), v_mean.contiguous().view(torch.uint8)), dim=-1)
    gathered = packed.new_empty((runtime.size * packed.shape[0], *packed.shape[1:]))
    dist.all_gather_into_tensor(gathered, packed, group=runtime.group)
    k_all = gathered[..., :key_bytes].view(torch.float32).index_select(0, global_to_gather)
    v_all = gathered[..., key_bytes:].view(torch.bfloat16).index_select(0, global_to_gather)
    return k_all, v_all


def scatter_pooled_grads(dk_global, dv_global, runtime, global_to_gather, local_blocks):
    """Adjoint of :func:`gather_means`: FP32-sum the global pooled gradients over the ranks and keep
    this rank's blocks (reference ``vsa_core.py:206-215``).  Every rank must call it."""
    if runtime.size == 1:
        return dk_global.float(), dv_global.float()
    stacked = torch.stack((dk_global.float(), dv_global.float()), dim=1)
    ordered = stacked.new_zeros((runtime.size * local_blocks, *stacked.shape[1:]))
    ordered.index_copy_(0, global_to_gather, stacked)
    local = ordered.new_empty((local_blocks, *stacked.shape[1:]))
    dist.reduce_scatter_tensor(local, ordered, group=runtime.group)
    return local[:, 0].contiguous(), local[:, 1].contiguous()


def partition(index, counts, layout, runtime):
    """Per-owner lists of owner-local block ids: ``(lists [R, H, C, cap'], counts [R, H, C])``."""
    heads, blocks, cap = index.shape[1], index.shape[2], index.shape[3]
    if runtime.size == 1:
        return index.view(1, heads, blocks, cap), counts.view(1, heads, blocks)
    out_cap = min(blocks, cap)
    rows = heads * blocks
    list_stride, count_stride = -(-rows * out_cap // 4) * 4, -(-rows // 4) * 4
    lists = torch.empty((runtime.size, list_stride), dtype=torch.int32, device=index.device)
    numbers = torch.empty((runtime.size, count_stride), dtype=torch.int32, device=index.device)
    _cabi.call("vsa_partition_indices", _p(index), _p(counts), _p(layout.ring.global_to_gather), _p(lists),
               _p(numbers), rows, cap, out_cap, runtime.size, blocks, list_stride, count_stride, _cabi.stream())
    return (lists[:, :rows * out_cap].view(runtime.size, heads, blocks, out_cap),
            numbers[:, :rows].view(runtime.size, heads, blocks))


def _passes(blocks):
    """Number of passes and blocks per pass for a range of `blocks` blocks (a range up to one and a
    half times the pass size still runs in one pass)."""
    count = max(1, int(blocks / RING_CHUNK_BLOCKS + 0.5))
    return count, -(-blocks // count)


def list_bounds(lists, counts, kv_blocks):
    """``(bounds [R, H, C, passes + 1] or None, passes)``: where each KV range of a shard starts in
    every per-owner list."""
    passes, chunk = _passes(kv_blocks)
    if passes == 1:
        return None, 1
    owners, heads, blocks, cap = lists.shape
    bounds = torch.empty((owners, heads, blocks, passes + 1), dtype=torch.int32, device=lists.device)
    for owner in range(owners):
        _cabi.call("vsa_list_bounds", _p(lists[owner]), _p(counts[owner]), heads * blocks, cap, chunk, passes,
                   _p(bounds[owner]), _cabi.stream())
    return bounds, passes


def _gather_rows(x, row_map):
    out = torch.empty((row_map.numel(), *x.shape[1:]), dtype=x.dtype, device=x.device)
    if out.numel():
        _cabi.call("vsa_row_gather", _p(x), _p(row_map), _p(out), row_map.numel(),
                   x[0].numel() * x.element_size(), _cabi.stream())
    return out


def _bwd_call(q, k, v, d_o, index, counts, sizes_q, sizes_kv, scale, lse, delta, mask, status, *, parts,
              dq=None, dk=None, dv=None, dq_f32=None, dk_f32=None, dv_f32=None, accumulate=0, early_kv=0,
              bounds=None, passes=1):
    """One ring step of the dQ kernel (parts = 3: mask, then dQ) or of the dK/dV kernel (parts = 4),
    in passes over KV ranges / query-block ranges when the shard is large."""
    heads = q.shape[1]
    hint = int(early_kv) << 8  # scheduling hint of the dK/dV kernel
    q_blocks, kv_blocks = q.shape[0] // BLOCK, k.shape[0] // BLOCK
    words = _cabi.load().vsa_kv_mask_words(q_blocks)
    q_passes, _ = _passes(q_blocks)
    with _cabi.mark("ring_step_dq" if parts & 2 else "ring_step_dkv"):
        one_pass = bounds is None if parts & 2 else q_passes == 1
        if one_pass:
            _bwd_launch(q, k, v, d_o, index, counts, sizes_q, sizes_kv, scale, lse, delta, mask, status, parts | hint,
                        dq, dk, dv, dq_f32, dk_f32, dv_f32, accumulate, heads, q_blocks, kv_blocks)
            return

        def launch(now, bound, stride, word_begin, word_end, add):
            _cabi.call("vsa_fine_bwd_range", _p(q), _p(k), _p(v), _p(d_o), q_blocks, kv_blocks, heads, _p(index),
                       _p(counts), _p(bound), index.stride(0), counts.stride(0), stride, index.shape[-1], _p(sizes_q),
                       _p(sizes_kv), scale, _p(lse), _p(delta), _p(mask), word_begin, word_end, _p(dq_f32),
                       _p(dk_f32), _p(dv_f32), add, now, _p(status), _cabi.stream(),
                       launches=bin(now & 7).count("1"))

        if parts & 2:
            flat = bounds.flatten()
            for c in range(passes):
                launch((parts & 1 if c == 0 else 0) | 2, flat[c:], passes + 1, 0, words, accumulate)
        else:
            per = -(-words // q_passes)  # whole 32-block mask words per pass
            for begin in range(0, words, per):
                launch(4 | hint, None, 0, begin, min(words, begin + per), 1 if (accumulate or begin) else 0)


def _bwd_launch(q, k, v, d_o, index, counts, sizes_q, sizes_kv, scale, lse, delta, mask, status, parts, dq, dk, dv,
                dq_f32, dk_f32, dv_f32, accumulate, heads, q_blocks, kv_blocks):
    _cabi.call("vsa_fine_bwd", _p(q), _p(k), _p(v), _p(d_o), q_blocks, kv_blocks, heads, _p(index), _p(counts),
               index.stride(0), counts.stride(0), index.shape[-1], _p(sizes_q), _p(sizes_kv), scale, _p(lse),
               _p(delta), _p(mask), _p(dq), _p(dk), _p(dv), q.shape[0], k.shape[0], None, None, None, None, None,
               0, None, None, _p(dq_f32), _p(dk_f32), _p(dv_f32), accumulate, parts, _p(status), _cabi.stream(),
               launches=bin(parts & 7).count("1"))


class _RingVSAFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, gate, layout, scale):
        rt = ring_runtime(layout, q.device)
        plan = device_plan(layout)
        ring = layout.ring
        tokens, heads, dim = q.shape
        blocks, slots = layout.blocks, layout.blocks * BLOCK
        coarse = plan.coarse
        q_s = torch.empty((slots, heads, dim), dtype=q.dtype, device=q.device)
        kv = torch.empty((2, slots, heads, dim), dtype=q.dtype, device=q.device)
        mean = (torch.empty((3, blocks, heads, dim), dtype=torch.float32, device=q.device)
                if not layout.dense_only else None)
        _cabi.call("vsa_slots_pool", _p(q), _p(k), _p(v), _p(layout.slot_row), _p(layout.block_sizes), _p(q_s),
                   _p(kv[0]), _p(kv[1]), _p(mean), None, None, 0, blocks, heads, _cabi.stream())
        index = layout.routing_indices
        k_all = v_all = None
        if not layout.dense_only:
            k_all, v_all = gather_means(mean[1], mean[2], rt, ring.global_to_gather)
            index = route(mean[0], k_all, layout, plan)
        lists, counts = partition(index, layout.routing_counts, layout, rt)
        bounds, passes = list_bounds(lists, counts, kv.shape[1] // BLOCK)

        out_f32 = torch.zeros((slots, heads, dim), dtype=torch.float32, device=q.device)
        lse = torch.full((heads, slots), float("-inf"), dtype=torch.float32, device=q.device)
        buffers = [kv, torch.empty_like(kv)] if rt.size > 1 else [kv]
        current = kv
        for step in range(rt.size):
            owner = (rt.rank - step) % rt.size
            current = buffers[step % len(buffers)]
            if step + 1 < rt.size:
                ring_exchange(rt, [(current, buffers[(step + 1) % 2])])
            if bounds is None:
                _cabi.call("vsa_fine_fwd_running", _p(q_s), _p(current[0]), _p(current[1]), blocks,
                           current.shape[1] // BLOCK, heads, _p(lists[owner]), _p(counts[owner]), lists.stride(1),
                           counts.stride(1), lists.shape[-1], _p(ring.peer_block_sizes[owner]), scale, _p(out_f32),
                           _p(lse), _p(plan.status), _cabi.stream())
            else:
                flat = bounds[owner].flatten()
                for c in range(passes):
                    _cabi.call("vsa_fine_fwd_running_range", _p(q_s), _p(current[0]), _p(current[1]), blocks,
                               current.shape[1] // BLOCK, heads, _p(lists[owner]), _p(flat[c:]), lists.stride(1),
                               counts.stride(1), passes + 1, lists.shape[-1], _p(ring.peer_block_sizes[owner]),
                               scale, _p(out_f32), _p(lse), _p(plan.status), _cabi.stream())
            if step + 1 < rt.size:
                join_exchange(rt)

        tok = coarse_o = coarse_lse = None
        if coarse is not None and coarse.q_rows:
            tok = (_gather_rows(mean[0].to(q.dtype), coarse.q_src), _gather_rows(k_all.to(q.dtype), coarse.kv_src),
                   _gather_rows(v_all, coarse.kv_src))
            coarse_o, coarse_lse = _fine_fwd(tok[0], tok[1], tok[2], coarse.index, coarse.counts, (0, 0),
                                             coarse.kv_sizes, scale, plan.status)
        o_s = torch.empty_like(q_s)
        out = torch.empty_like(q)
        _cabi.call("vsa_gate_merge", _p(out_f32), _p(layout.slot_row),
                   _p(coarse.block_q) if coarse_o is not None else None, _p(gate) if coarse_o is not None else None,
                   _p(coarse_o), _p(o_s), _p(out), blocks, heads, tokens, _cabi.stream())
        ctx.save_for_backward(q_s, current, o_s, lse, lists, counts, gate if coarse_o is not None else None,
                              coarse_o, coarse_lse, *(tok if tok is not None else (None, None, None)))
        ctx.layout, ctx.scale, ctx.runtime = layout, scale, rt
        ctx.bounds, ctx.passes = bounds, passes
        return out

    @staticmethod
    def backward(ctx, grad):
        q_s, saved_kv, o_s, lse, lists, counts, gate, coarse_o, coarse_lse, tok_q, tok_k, tok_v = ctx.saved_tensors
        layout, scale, rt = ctx.layout, ctx.scale, ctx.runtime
        plan = device_plan(layout)
        ring, coarse = layout.ring, plan.coarse
        grad = grad.contiguous()
        tokens, heads, dim = grad.shape
        blocks, slots = layout.blocks, layout.blocks * BLOCK
        device = grad.device
        grad_s = torch.empty_like(q_s)
        delta = torch.empty((heads, slots), dtype=torch.float32, device=device)
        dgate = dcoarse = coarse_delta = None
        if coarse_o is not None:
            dgate = torch.empty_like(grad)
            dcoarse = torch.zeros_like(coarse_o)
            coarse_delta = torch.zeros((heads, coarse.q_rows), dtype=torch.float32, device=device)
        elif not layout.dense_only:
            dgate = torch.zeros_like(grad)  # a rank without coarse queries still owes a zero gate gradient
        _cabi.call("vsa_merge_bwd", _p(grad), _p(gate), _p(coarse_o), _p(o_s), _p(layout.slot_row),
                   _p(coarse.block_q) if coarse_o is not None else None, _p(grad_s),
                   _p(dgate) if coarse_o is not None else None, _p(dcoarse), _p(delta), _p(coarse_delta), blocks,
                   coarse.q_rows if coarse_o is not None else 0, heads, _cabi.stream())

        dq_tok = dk_pool = dv_pool = None
        if not layout.dense_only:
            total = ring.global_to_gather.numel()
            if coarse_o is not None:
                words = _cabi.load().vsa_kv_mask_words(tok_q.shape[0] // BLOCK)
                mask = torch.empty(heads * (tok_k.shape[0] // BLOCK) * words, dtype=torch.int32, device=device)
                dq_tok, dk_tok, dv_tok = torch.empty_like(tok_q), torch.empty_like(tok_k), torch.empty_like(tok_v)
                index2d, counts2d = coarse.index.unsqueeze(0), coarse.counts.unsqueeze(0)
                _cabi.call("vsa_fine_bwd", _p(tok_q), _p(tok_k), _p(tok_v), _p(dcoarse), tok_q.shape[0] // BLOCK,
                           tok_k.shape[0] // BLOCK, heads, _p(index2d), _p(counts2d), 0, 0, index2d.shape[-1],
                           _p(coarse.q_sizes), _p(coarse.kv_sizes), scale, _p(coarse_lse), _p(coarse_delta),
                           _p(mask), _p(dq_tok), _p(dk_tok), _p(dv_tok), tok_q.shape[0], tok_k.shape[0], None,
                           None, None, None, None, 0, None, None, None, None, None, 0, 7, _p(plan.status),
                           _cabi.stream(), launches=3)
                dk_global = _gather_rows(dk_tok, coarse.block_kv_rows)
                dv_global = _gather_rows(dv_tok, coarse.block_kv_rows)
            else:
                dk_global = torch.zeros((total, heads, dim), dtype=torch.float32, device=device)
                dv_global = torch.zeros_like(dk_global)
            dk_pool, dv_pool = scatter_pooled_grads(dk_global, dv_global, rt, ring.global_to_gather, blocks)

        # Reverse ring: start from the last forward shard; never write into saved tensors.
        kv = saved_kv.clone() if rt.size > 1 else saved_kv
        buffers = [kv, torch.empty_like(kv)] if rt.size > 1 else [kv]
        dq_acc = torch.zeros((slots, heads, dim), dtype=torch.float32, device=device)
        words = _cabi.load().vsa_kv_mask_words(blocks)
        mask = torch.empty(heads * blocks * words, dtype=torch.int32, device=device)
        # Two FP32 dK||dV buffers alternate: the sum that arrives at step s lands in sums[s % 2],
        # the dK/dV kernel adds this rank's part to it in place, and step s + 1 sends it on.
        sums = [torch.empty((2, slots, heads, dim), dtype=torch.float32, device=device)
                for _ in range(min(rt.size, 2))]
        accumulated = None
        for step in range(rt.size):
            owner = (rt.rank - (rt.size - 1 - step)) % rt.size
            current = buffers[step % len(buffers)]
            target = sums[step % len(sums)]
            pairs = []
            if step + 1 < rt.size:
                pairs.append((current, buffers[(step + 1) % 2]))
            if step:
                pairs.append((accumulated, target))
            if pairs:
                ring_exchange(rt, pairs, reverse=True)
            common = (q_s, current[0], current[1], grad_s, lists[owner], counts[owner], layout.block_sizes,
                      ring.peer_block_sizes[owner], scale, lse, delta, mask, plan.status)
            _bwd_call(*common, parts=3, dq_f32=dq_acc, accumulate=1,
                      bounds=None if ctx.bounds is None else ctx.bounds[owner], passes=ctx.passes)
            if pairs:
                join_exchange(rt)
            _bwd_call(*common, parts=4, dk_f32=target[0], dv_f32=target[1], accumulate=1 if step else 0,
                      early_kv=plan.early_kv[owner])
            accumulated = target
        dq, dk, dv = (torch.empty_like(grad) for _ in range(3))
        sizes = layout.block_sizes
        _cabi.call("vsa_grad_finish", _p(dq_acc), _p(layout.slot_row), _p(dq_tok), 0,
                   _p(coarse.block_q) if dq_tok is not None else None, _p(sizes), _p(dq), blocks, heads, tokens,
                   _cabi.stream())
        for acc, pool, out in ((accumulated[0], dk_pool, dk), (accumulated[1], dv_pool, dv)):
            _cabi.call("vsa_grad_finish", _p(acc), _p(layout.slot_row), _p(pool), 1, None, _p(sizes), _p(out),
                       blocks, heads, tokens, _cabi.stream())
        return dq, dk, dv, dgate, None, None


def routing_table(q, k, layout):
    """Routing table of this rank's query blocks over global KV block ids, as the ring forward
    pass computes it (pooling, all-gather of the pooled K, selection).  A collective: every rank
    of the group must call it.  Benchmarks count useful FLOPs from it."""
    rt = ring_runtime(layout, q.device)
    plan = device_plan(layout)
    if layout.dense_only:
        return layout.routing_indices
    heads, dim = q.shape[1], q.shape[2]
    mean = torch.empty((3, layout.blocks, heads, dim), dtype=torch.float32, device=q.device)
    _cabi.call("vsa_slots_pool", _p(q), _p(k), _p(k), _p(layout.slot_row), _p(layout.block_sizes), None, None, None,
               _p(mean), None, None, 0, layout.blocks, heads, _cabi.stream())
    k_all, _ = gather_means(mean[1], mean[2], rt, layout.ring.global_to_gather)
    return route(mean[0], k_all, layout, plan)


def ring_attention(q, k, v, gate, layout, *, scale=None):
    """Ring VSA on validated local inputs ``[layout.tokens, H, 128]`` in compact block order."""
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    return _RingVSAFunction.apply(q, k, v, gate, layout, scale)
