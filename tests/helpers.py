"""Shared test inputs: geometries of the golden vectors, seeded tensors, tolerance checks."""
from pathlib import Path

import numpy as np
import torch

from cudnn_vsa_b200.vsa_layout import BLOCK, Segment

GOLDEN = Path(__file__).resolve().parent / "golden"
S = Segment

GEOMETRIES = {
    "c1": [[S("video", (8, 16, 16), .75), S("text", 256)]],
    "ragged": [[S("video", (5, 9, 11), .7), S("text", 67)],
               [S("text", 3), S("video", (1, 3, 5))],
               [S("video", (4, 8, 12), .5), S("video", (5, 4, 7), .9), S("audio", 17), S("text", 0)]],
    "partial_blocks": [[S("video", (1, 3, 5), .9), S("text", 7)]],
    "fine_only_peer": [[S("video", (1, 2, 3), .5)], [S("video", (1, 2, 3))]],
    "dense": [[S("video", (1, 9, 11)), S("text", 67)], [S("video", (1, 3, 5)), S("text", 3)]],
    "mixed": [[S("video", (1, 9, 8)), S("text", 7)],
              [S("video", (5, 4, 8), .5), S("text", 65)],
              [S("video", (2, 3, 5), .5), S("text", 9)]],
    "zero_sparsity": [[S("video", (4, 4, 8), 0.0), S("text", 5)]],
    "full_blocks": [[S("video", (4, 4, 8), .5), S("text", 64)], [S("video", (1, 8, 8)), S("text", 64)]],
    "c2": [[S("video", (31, 45, 80), .9), S("text", 2048)]],
    "c3": [[S("video", (31, 45, 80), .9), S("text", 2048)],
           [S("video", (1, 45, 80)), S("text", 2048)], [S("video", (1, 45, 80)), S("text", 2048)]],
    "c4": [[S("video", (21, 30, 52), .8), S("text", 512), S("audio", 1024)]] * 4,
    "c5": [[S("video", (61, 90, 160), .95), S("text", 4096)]],
}

# north_star tolerances for BF16 outputs and gradients against an FP32 reference.
MAX_ABS, REL_L2 = 2e-2, 1e-2


def seeded(tokens, heads, seed, count):
    """The golden vectors' input recipe: CPU generator, FP32 normal, cast to BF16."""
    gen = torch.Generator().manual_seed(seed)
    return [torch.randn(tokens, heads, 128, generator=gen).to(torch.bfloat16) for _ in range(count)]


def golden_cases():
    return np.load(GOLDEN / "cases.npz")


def from_bits(array):
    return torch.from_numpy(np.ascontiguousarray(array)).view(torch.bfloat16)


def error_metrics(actual, expected):
    """``(max_abs, rel_l2, peak)`` of ``actual`` against ``expected`` in float64."""
    a, b = actual.detach().double().flatten(), expected.detach().double().flatten().to(actual.device)
    err = (a - b).abs().max().item() if a.numel() else 0.0
    rel = ((a - b).square().sum() / b.square().sum().clamp_min(1e-30)).sqrt().item() if a.numel() else 0.0
    return err, rel, (b.abs().max().item() if b.numel() else 0.0)


REPORT = []  # (what, max_abs, bound, rel_l2, peak, peak_relative) of every comparison of this process


def assert_close(actual, expected, what, max_abs=MAX_ABS, rel_l2=REL_L2, peak_relative=False):
    """max-abs and relative-L2 bounds; the absolute bound is the stated contract.

    ``peak_relative`` scales the max-abs bound by the reference tensor's peak magnitude when that
    exceeds one.  It is meant for dk / dv only: a BF16 result cannot be closer than half an ulp
    (0.016 at magnitude 4, 0.031 at 8), and the gradient of an always-visible KV block sums
    over every query row of its sample and reaches that size.  Every comparison is appended to
    ``REPORT`` so a run can print which tensors needed the relative form and by what margin.
    """
    assert tuple(actual.shape) == tuple(expected.shape), (what, actual.shape, expected.shape)
    if not actual.numel():
        return
    assert torch.isfinite(actual).all(), f"{what}: non-finite values"
    err, rel, peak = error_metrics(actual, expected)
    bound = max_abs * (max(1.0, peak) if peak_relative else 1.0)
    REPORT.append((what, err, bound, rel, peak, peak_relative))
    assert err <= bound and rel <= rel_l2, (
        f"{what}: max_abs={err:.3e} (bound {bound:.3e}, reference peak {peak:.3g}) rel_l2={rel:.3e}")


def oracle_heads(q, k, v, gate, dy, layout, index, heads, *, chunk=64, scale=None, round_like_reference=False):
    """FP32 oracle of one ``vsa_attention`` call and its backward pass for a subset of heads, at
    sizes where the whole-tensor oracle would not fit: the fine part is evaluated and
    back-propagated ``chunk`` query blocks at a time through ``vsa_oracle.fine_attention``, so
    its autograd graph never holds more than one chunk; pooling, coarse attention and the merge
    follow ``vsa_oracle.vsa_attention``: pure FP32 by default, or with its BF16 roundings of the
    pooled tokens and of the coarse and fine outputs.  Everything runs on ``q.device`` with the
    routing table ``index`` the kernels used.  Returns FP32 ``out, dq, dk, dv, dgate`` of
    shape ``[T, len(heads), 128]`` (``dgate`` is ``None`` for a layout without coarse part).
    """
    from oracle import vsa_oracle
    hs = list(heads)
    dim = q.shape[-1]
    scale = dim ** -0.5 if scale is None else scale
    low = q.dtype
    rnd = (lambda x: x.to(low).float()) if round_like_reference else (lambda x: x)
    slot_row, row_slot = layout.slot_row, layout.row_slot
    slots = [vsa_oracle.gather_rows(x[:, hs], slot_row).float().requires_grad_() for x in (q, k, v)]
    dy_slots = vsa_oracle.gather_rows(dy[:, hs], slot_row).float()
    sizes = None if layout.all_blocks_full else layout.block_sizes
    sub_index, sub_counts = index[:, hs], layout.routing_counts[:, hs]
    fine_slots = torch.zeros_like(dy_slots)
    offsets = torch.arange(BLOCK, device=q.device)
    for first in range(0, layout.blocks, chunk):
        blocks = torch.arange(first, min(first + chunk, layout.blocks), device=q.device)
        rows = (blocks[:, None] * BLOCK + offsets[None, :]).reshape(-1)
        fine, _ = vsa_oracle.fine_attention(slots[0][rows], slots[1], slots[2],
                                            sub_index[:, :, blocks].contiguous(),
                                            sub_counts[:, :, blocks].contiguous(), sizes, scale)
        fine = rnd(fine)
        fine_slots[rows] = fine.detach()
        (fine * dy_slots[rows]).sum().backward()
    out = vsa_oracle.gather_rows(fine_slots, row_slot)
    dgate = None
    if not layout.dense_only:
        gate_leaf = gate[:, hs].float().requires_grad_()
        means = [vsa_oracle.block_means(x, layout.block_sizes)[layout.coarse_blocks] for x in slots]
        coarse = rnd(vsa_oracle.coarse_attention(rnd(means[0]), rnd(means[1]), rnd(means[2]),
                                                 layout.coarse_cu_q, layout.coarse_cu_q, scale))
        term = vsa_oracle.merge(torch.zeros_like(out), gate_leaf, coarse, layout.row_coarse)
        (term * dy[:, hs].float()).sum().backward()
        out = out + term.detach()
        dgate = gate_leaf.grad
    dq, dk, dv = (x.grad[row_slot] for x in slots)
    return out, dq, dk, dv, dgate


def routing_mismatches_are_near_ties(got, want, scores_list, counts, rel=1e-4):
    """Two routing tables may differ only where the swapped blocks' pooled scores are within
    `rel` of the keep-th score (the near-tie rule)."""
    from oracle import vsa_oracle
    bad = 0
    for begin, end, first, last, keep, cursor, scores in scores_list:
        a = got[0, :, begin:end, cursor:cursor + keep].long() - first
        b = want[0, :, begin:end, cursor:cursor + keep].long() - first
        differ = (a != b).any(-1)
        if not differ.any():
            continue
        kth = scores.topk(keep, dim=-1).values[..., -1]
        for h, r in differ.nonzero().tolist():
            sa, sb = set(a[h, r].tolist()), set(b[h, r].tolist())
            for j in sa ^ sb:
                gap = abs(scores[h, r, j] - kth[h, r]) / abs(kth[h, r]).clamp_min(1e-30)
                bad += int(gap >= rel)
    return bad == 0
