"""Shared test inputs: geometries of the golden vectors, seeded tensors, tolerance checks."""
from pathlib import Path

import numpy as np
import torch

from cudnn_vsa_b200.vsa_layout import Segment

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


def assert_close(actual, expected, what, max_abs=MAX_ABS, rel_l2=REL_L2):
    """max-abs and relative-L2 bounds.  The max-abs bound is taken relative to the reference's
    peak magnitude when that exceeds one: a BF16 result cannot be closer than half an ulp
    (0.016 at magnitude 4, 0.031 at 8), and gradients summed over many rows reach that size."""
    a, b = actual.detach().double().cpu().flatten(), expected.detach().double().cpu().flatten()
    assert a.shape == b.shape, (what, a.shape, b.shape)
    if not a.numel():
        return
    assert torch.isfinite(a).all(), f"{what}: non-finite values"
    err = (a - b).abs().max().item()
    bound = max_abs * max(1.0, b.abs().max().item())
    rel = ((a - b).square().sum() / b.square().sum().clamp_min(1e-30)).sqrt().item()
    assert err <= bound and rel <= rel_l2, f"{what}: max_abs={err:.3e} (bound {bound:.3e}) rel_l2={rel:.3e}"


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
