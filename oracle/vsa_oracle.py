"""CPU oracle for the packed video-sparse-attention path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the algorithm that the reference
implements with Triton, cuDNN block-sparse attention and FA4.  It exists to check the
CUDA kernels of this repository; nothing that ships imports it.  Only the test-suite,
the smoke check and the CPU-baseline leg of the benchmark may call it.

Parity status: PINNED.  ``tests/golden/`` holds outputs and gradients produced by the
reference's own CPU code (``tests/reference.py::reference_pack`` and ``::cpu_attention``,
plus its layout planner, router and ring partition reference) on seeded inputs; the
CPU tests check every function below against those vectors.

Each function cites the reference lines it follows.
"""
from __future__ import annotations

import math

import torch

BLOCK = 64


# ----------------------------------------------------------------------------- block planning
def plan_blocks(samples):
    """Per-block raster rows, independent of the vectorised planner (small cases only).

    Follows reference ``vsa_layout.py:334-372``: per sample, dense segments first as
    consecutive <=64-token chunks, then numeric-sparsity videos as 4x4x4 tiles visited
    frame, height, width with width fastest; edge tiles keep only valid tokens.
    Returns ``(blocks, groups)`` with ``blocks`` a list of row lists and ``groups`` a list of
    ``(start, end, dense_blocks, ((first, end, keep), ...))``.
    """
    blocks, groups, token = [], [], 0
    for sample in samples:
        offsets = []
        for seg in sample:
            offsets.append(token)
            token += seg.tokens
        start, spans = len(blocks), []
        for seg, off in zip(sample, offsets):
            if seg.sparsity is None:
                for p in range(0, seg.tokens, BLOCK):
                    blocks.append(list(range(off + p, off + min(p + BLOCK, seg.tokens))))
        dense = len(blocks) - start
        for seg, off in zip(sample, offsets):
            if seg.sparsity is None:
                continue
            frames, height, width = seg.size
            first = len(blocks)
            for f0 in range(0, frames, 4):
                for h0 in range(0, height, 4):
                    for w0 in range(0, width, 4):
                        blocks.append([off + (f * height + h) * width + w
                                       for f in range(f0, min(f0 + 4, frames))
                                       for h in range(h0, min(h0 + 4, height))
                                       for w in range(w0, min(w0 + 4, width))])
            n = len(blocks) - first
            spans.append((first, len(blocks), max(1, math.ceil((1 - seg.sparsity) * n))))
        groups.append((start, len(blocks), dense, tuple(spans)))
    return blocks, groups


def slot_maps(blocks, tokens):
    """``slot_row`` (-1 padding) and ``row_slot`` from per-block rows (reference ``vsa_layout.py:293-297``)."""
    slot_row = []
    for rows in blocks:
        slot_row += rows + [-1] * (BLOCK - len(rows))
    row_slot = [0] * tokens
    for slot, row in enumerate(slot_row):
        if row >= 0:
            row_slot[row] = slot
    return torch.tensor(slot_row, dtype=torch.int64), torch.tensor(row_slot, dtype=torch.int64)


# ----------------------------------------------------------------------------- row movement
def gather_rows(x, row_map):
    """``out[i] = x[row_map[i]]`` or zero where ``row_map[i] < 0`` (reference ``vsa_kernels.py:66-83``,
    CPU twin ``tests/reference.py:18-20``)."""
    picked = x[row_map.clamp_min(0)]
    mask = (row_map < 0).view(-1, *([1] * (x.dim() - 1)))
    return picked.masked_fill(mask, 0)


def reorder_rows(x, input_rows, inverse=False, output_tokens=None):
    """Unique-row gather, or its scatter adjoint into a zero-filled tensor
    (reference ``vsa_kernels.py:11-42``)."""
    if not inverse:
        return x[input_rows]
    tokens = x.shape[0] if output_tokens is None else output_tokens
    out = x.new_zeros((tokens, *x.shape[1:]))
    out[input_rows] = x
    return out


# ----------------------------------------------------------------------------- pooling and routing
def block_means(x_slots, block_sizes):
    """FP32 sum of the 64 zero-padded slots of each block divided by ``max(size, 1)``
    (reference ``vsa_kernels.py:161-176``)."""
    blocks = block_sizes.numel()
    summed = x_slots.view(blocks, BLOCK, *x_slots.shape[1:]).sum(1, dtype=torch.float32)
    return summed / block_sizes.clamp_min(1).view(-1, *([1] * (x_slots.dim() - 1))).float()


def keep_count(sparsity, blocks):
    """KV budget of one video region (reference ``vsa_layout.py:366``)."""
    return max(1, math.ceil((1 - sparsity) * blocks))


def route(q_mean, k_mean, layout, query_blocks=None):
    """Fill the routing template: per video region that needs selection, per (head, query
    block), the ``keep`` highest unscaled FP32 scores ``q_mean . k_mean`` listed in
    ascending block order (reference ``vsa_core.py:61-84``).

    ``q_mean`` / ``k_mean`` are ``[pooled_blocks, H, D]`` float32 in the layout's pooled index
    space (``routing_groups`` carries the offset).  Returns ``[1, H, B, cap]`` int32, or only the
    rows of ``query_blocks`` (a 1-D tensor of block ids) when a bounded sample is wanted.
    """
    if query_blocks is None:
        if not layout.routing_groups:
            return layout.routing_indices
        index = layout.routing_indices.clone()
    else:
        index = layout.routing_indices[:, :, query_blocks].clone()
    for group, begin, end, offset in layout.routing_groups:
        if query_blocks is None:
            rows = slice(begin, end)
            queries = q_mean[begin + offset:end + offset]
        else:
            rows = (query_blocks >= begin) & (query_blocks < end)
            if not bool(rows.any()):
                continue
            queries = q_mean[query_blocks[rows] + offset]
        queries = queries.float().transpose(0, 1)  # [H, nq, D]
        cursor = group.dense_blocks_num
        for first, last, keep in group.video_spans:
            if keep < last - first:
                keys = k_mean[first + offset:last + offset].float().permute(1, 2, 0)  # [H, D, span]
                scores = queries @ keys
                chosen = scores.topk(keep, dim=-1, sorted=False).indices.sort(-1).values
                index[0][:, rows, cursor:cursor + keep] = (chosen + first).to(torch.int32)
            cursor += keep
    return index


def routing_scores(q_mean, k_mean, layout):
    """FP32 pooled scores per routed region, for judging near-ties:
    list of ``(begin, end, first, last, keep, cursor, scores[H, nq, span])``."""
    out = []
    for group, begin, end, offset in layout.routing_groups:
        queries = q_mean[begin + offset:end + offset].float().transpose(0, 1)
        cursor = group.dense_blocks_num
        for first, last, keep in group.video_spans:
            if keep < last - first:
                keys = k_mean[first + offset:last + offset].float().permute(1, 2, 0)
                out.append((begin, end, first, last, keep, cursor, queries @ keys))
            cursor += keep
    return out


# ----------------------------------------------------------------------------- attention
def fine_attention(q, k, v, indices, counts, sizes, scale):
    """Block-sparse softmax(q k^T scale) v over the listed 64-slot KV blocks, FP32, with
    KV slots at or beyond ``sizes[block]`` masked.  Differentiable.

    Same contract as the reference's fine backend call (``vsa_core.py:15-20``; dense CPU
    substitute ``tests/reference.py:57-67``) but evaluated block by block, so it scales to
    long sequences.  ``q, k, v`` are ``[P, H, D]`` slot tensors; ``indices [1,H,B,cap]``,
    ``counts [1,H,B]``.  ``q`` may hold fewer blocks than ``k`` (a sample of query blocks with
    their rows of the table).  All tensors live on one device; a test may place them on a GPU
    when it needs this FP32 restatement at sizes the CPU cannot finish in seconds.
    Returns ``(out [P,H,D] float32, lse [H,P] float32)``; a query block with an empty list gives
    zeros and ``-inf``.
    """
    slots, heads, dim = q.shape
    blocks = slots // BLOCK
    qf, kf, vf = (x.float().view(-1, BLOCK, heads, dim) for x in (q, k, v))
    size_of = (torch.full((kf.shape[0],), BLOCK, dtype=torch.int64, device=q.device) if sizes is None
               else sizes.to(torch.int64))
    slot_ids = torch.arange(BLOCK, device=q.device)
    outs = [[None] * blocks for _ in range(heads)]
    lses = [[None] * blocks for _ in range(heads)]
    count_host = counts[0].tolist()
    for h in range(heads):
        for b in range(blocks):
            n = count_host[h][b]
            if n == 0:
                outs[h][b] = qf.new_zeros(BLOCK, dim)
                lses[h][b] = qf.new_full((BLOCK,), -math.inf)
                continue
            ids = indices[0, h, b, :n].long()
            keys = kf[ids, :, h].reshape(n * BLOCK, dim)
            values = vf[ids, :, h].reshape(n * BLOCK, dim)
            valid = (slot_ids[None, :] < size_of[ids][:, None]).reshape(-1)
            scores = (qf[b, :, h] @ keys.T) * scale
            scores = scores.masked_fill(~valid[None, :], -math.inf)
            lse = scores.logsumexp(-1)
            outs[h][b] = (scores - lse[:, None]).exp() @ values
            lses[h][b] = lse
    out = torch.stack([torch.cat(row) for row in outs], dim=1)
    lse = torch.stack([torch.cat(row) for row in lses], dim=0)
    return out, lse


def coarse_attention(q, k, v, cu_q, cu_kv, scale):
    """Dense attention over block tokens, one independent problem per sample
    (reference ``vsa_core.py:87-97``; CPU substitute ``tests/reference.py:70-78``).  FP32 math."""
    outs, bq, bk = [], cu_q.tolist(), cu_kv.tolist()
    for (q0, q1), (k0, k1) in zip(zip(bq, bq[1:]), zip(bk, bk[1:])):
        qs, ks, vs = q[q0:q1].float(), k[k0:k1].float(), v[k0:k1].float()
        scores = torch.einsum("qhd,khd->hqk", qs, ks) * scale
        outs.append(torch.einsum("hqk,khd->qhd", scores.softmax(-1), vs))
    return torch.cat(outs) if outs else q.new_zeros((0, *q.shape[1:]), dtype=torch.float32)


def merge(fine, gate, coarse, row_coarse):
    """``fine + gate * coarse[row_coarse]``; rows whose index equals ``coarse.shape[0]`` belong to
    fine-only samples, keep ``fine`` and never read ``gate`` (reference ``vsa_kernels.py:191-201``,
    CPU twin ``tests/reference.py:23-29``)."""
    sentinel = row_coarse == coarse.shape[0]
    gate = gate.float().masked_fill(sentinel.view(-1, 1, 1), 0)
    padded = torch.cat((coarse.float(), coarse.new_zeros((1, *coarse.shape[1:]), dtype=torch.float32)))
    return fine.float() + gate * padded[row_coarse]


def vsa_attention(q, k, v, gate, layout, *, scale=None, indices=None, round_like_reference=True):
    """Whole single-device path in FP32 with autograd (reference ``vsa.py:64-121`` and
    ``vsa_core.py:100-120``): slots, pooled means, routing, fine, coarse, restore, merge.

    ``indices`` overrides the router (to judge numerics separately from near-tie choices).
    With ``round_like_reference`` the pooled means used by coarse attention and the coarse and
    fine outputs are rounded to the input dtype where the reference rounds them
    (``vsa_kernels.py:186-188``, backends returning BF16); everything else stays FP32.
    Returns ``(out float32 [T,H,D], indices)``.
    """
    dim = q.shape[-1]
    scale = dim ** -0.5 if scale is None else scale
    low = q.dtype
    rnd = (lambda x: x.to(low).float()) if round_like_reference else (lambda x: x)
    slots = [gather_rows(x, layout.slot_row) for x in (q, k, v)]
    coarse = None
    if not layout.dense_only:
        means = [block_means(x, layout.block_sizes)[layout.coarse_blocks] for x in slots]
        if indices is None:
            indices = route(means[0].detach(), means[1].detach(), layout)
        coarse = rnd(coarse_attention(rnd(means[0]), rnd(means[1]), rnd(means[2]),
                                      layout.coarse_cu_q, layout.coarse_cu_q, scale))
    elif indices is None:
        indices = layout.routing_indices
    sizes = None if layout.all_blocks_full else layout.block_sizes
    fine, _ = fine_attention(*slots, indices, layout.routing_counts, sizes, scale)
    out = gather_rows(rnd(fine), layout.row_slot)
    if coarse is not None:
        out = merge(out, gate, coarse, layout.row_coarse)
    return out, indices


# ----------------------------------------------------------------------------- ring helpers
def partition_indices(index, counts, global_to_gather, ring_size, peer_blocks):
    """Split each routing row into per-owner lists of owner-local block ids, order preserved,
    tails zero (reference ``vsa_kernels.py:285-296``).  Returns
    ``(lists [R,1,H,C,min(peer_blocks,cap)] int32, counts [R,1,H,C] int32)``."""
    cap = index.shape[-1]
    width = min(peer_blocks, cap)
    lists = torch.zeros((ring_size, *index.shape[:-1], width), dtype=torch.int32)
    numbers = torch.zeros((ring_size, *counts.shape), dtype=torch.int32)
    flat_index, flat_counts = index.reshape(-1, cap), counts.reshape(-1)
    flat_lists, flat_numbers = lists.view(ring_size, -1, width), numbers.view(ring_size, -1)
    mapped = global_to_gather[flat_index.long()]
    for row in range(flat_index.shape[0]):
        n = int(flat_counts[row])
        owner, local = mapped[row, :n] // peer_blocks, mapped[row, :n] % peer_blocks
        for peer in range(ring_size):
            mine = local[owner == peer]
            flat_lists[peer, row, :mine.numel()] = mine.to(torch.int32)
            flat_numbers[peer, row] = mine.numel()
    return lists, numbers


def merge_partials(parts, lses):
    """Combine per-step partial attention results: float64 log-sum-exp weights
    (reference ``tests/test_ring_cuda.py:33-38``; kernel ``vsa_kernels.py:375-397``).
    ``parts`` list of ``[P,H,D]``, ``lses`` list of ``[H,P]``; empty rows (-inf everywhere) give 0."""
    stacked = torch.stack([x.double() for x in lses])
    total = stacked.logsumexp(0)
    weights = (stacked - total).exp().nan_to_num()
    out = sum(w.transpose(0, 1).unsqueeze(-1) * p.double() for w, p in zip(weights, parts))
    return out, total


# ----------------------------------------------------------------------------- metrics
def similarity(a, b):
    """Cosine, ``2ab/(a^2+b^2)``, max-abs and relative-L2 (reference ``benchmark/utils.py:17-29``)."""
    if not a.numel():
        return {"cosine": 1., "tensor_similarity": 1., "max_abs": 0., "relative_l2": 0.}
    a, b = a.detach().flatten().double(), b.detach().flatten().double()
    aa, bb, ab = (a * a).sum().item(), (b * b).sum().item(), (a * b).sum().item()
    return {"cosine": ab / (aa * bb) ** 0.5 if aa and bb else float(aa == bb),
            "tensor_similarity": 2 * ab / (aa + bb) if aa + bb else 1.0,
            "max_abs": (a - b).abs().max().item(),
            "relative_l2": ((a - b).square().sum().item() / max(bb, 1e-30)) ** 0.5}


def useful_flops(layout, indices, dim=128):
    """Useful attention FLOPs of one forward pass: valid query-key pairs of the fine lists plus
    the coarse block GEMMs (reference ``benchmark/utils.py:32-75``).  Backward counts twice this."""
    sizes = layout.block_sizes.double().cpu()
    counts = layout.routing_counts[0].cpu()
    idx = indices[0].cpu()
    valid = torch.arange(idx.shape[-1]) < counts[..., None]
    picked = sizes[idx.long()] * valid
    pairs = float((picked.sum(-1) * sizes[None, :]).sum())
    fine = 4 * dim * pairs
    coarse = sum(4 * layout.head_num * dim * g.blocks ** 2 for g in layout.groups if not g.dense_only)
    return {"fine_forward": fine, "coarse_forward": float(coarse), "forward": fine + coarse,
            "total": 3 * (fine + coarse)}
