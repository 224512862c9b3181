"""CPU: the oracle is pinned against vectors produced by the reference's own CPU code."""
import numpy as np
import pytest
import torch

from cudnn_vsa_b200.vsa_layout import build_vsa_layout
from oracle import vsa_oracle
from tests.helpers import GEOMETRIES, GOLDEN, assert_close, from_bits, golden_cases, seeded

CASES = golden_cases()
NAMES = ["mixed", "ragged", "partial_blocks", "fine_only_peer", "dense", "zero_sparsity", "full_blocks"]


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("label", ["pack", "cpu"])
def test_oracle_matches_reference_outputs_and_gradients(name, label):
    key = f"{name}/dqf0/{label}"
    if f"{key}/out" not in CASES.files:
        pytest.skip("no vector stored for this combination")
    heads = 2
    layout = build_vsa_layout(GEOMETRIES[name], head_num=heads)
    q, k, v, gate = seeded(layout.tokens, heads, 0, 4)
    dy, = seeded(layout.tokens, heads, 1, 1)
    leaves = [x.float().requires_grad_() for x in (q, k, v, gate)]
    routing = f"{name}/dqf0/routing"
    index = torch.from_numpy(CASES[routing]) if routing in CASES.files else None
    out, _ = vsa_oracle.vsa_attention(*leaves, layout, indices=index)
    grads = torch.autograd.grad(out, leaves, dy.float(), allow_unused=True)
    stride = 4 if layout.tokens > 600 else 1
    for tag, got in zip(("out", "dq", "dk", "dv", "dgate"), (out, *grads)):
        want = from_bits(CASES[f"{key}/{tag}"]).float()
        got = torch.zeros_like(q, dtype=torch.float32) if got is None else got
        # The reference's vectors are BF16 (and its gradients pass through BF16 intermediates).
        assert_close(got[::stride], want, f"{name} {label} {tag}", max_abs=4e-2, rel_l2=1.2e-2,
                     peak_relative=tag in ("dk", "dv"))


@pytest.mark.parametrize("name", ["mixed", "ragged", "c1", "full_blocks", "partial_blocks"])
def test_oracle_routing_and_pooling_match_reference(name):
    heads = 2
    for full in (False, True):
        key = f"{name}/dqf{int(full)}"
        if f"{key}/routing" not in CASES.files:
            continue
        layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, dense_query_full=full)
        q, k, v, _ = seeded(layout.tokens, heads, 0, 4)
        slots = [vsa_oracle.gather_rows(x, layout.slot_row) for x in (q, k, v)]
        means = [vsa_oracle.block_means(s, layout.block_sizes)[layout.coarse_blocks] for s in slots]
        assert np.array_equal(means[0].numpy(), CASES[f"{key}/q_mean"])
        assert torch.equal(means[2].to(torch.bfloat16), from_bits(CASES[f"{key}/coarse_v_mean"]))
        index = vsa_oracle.route(means[0], means[1], layout)
        assert np.array_equal(index.numpy(), CASES[f"{key}/routing"])


def test_oracle_ring_partition_matches_reference(metadata_group):
    ring = np.load(GOLDEN / "ring.npz")
    for name, size in (("ragged", 2), ("ragged", 3), ("mixed", 2), ("partial_blocks", 3)):
        full = build_vsa_layout(GEOMETRIES[name], head_num=2)
        q, k, v, _ = seeded(full.tokens, 2, 0, 4)
        slots = [vsa_oracle.gather_rows(x, full.slot_row) for x in (q, k)]
        qm, km = (vsa_oracle.block_means(s, full.block_sizes) for s in slots)
        for rank in range(size):
            local = build_vsa_layout(GEOMETRIES[name], head_num=2, input_order="block",
                                     ring_cp_group=metadata_group(size, rank))
            ids = local.ring.block_ids
            q_local = qm[ids.clamp_min(0)].masked_fill((ids < 0)[:, None, None], 0)
            index = vsa_oracle.route(q_local, km, local)
            key = f"{name}/ring{size}.{rank}"
            assert np.array_equal(index.numpy(), ring[f"{key}/index"])
            lists, counts = vsa_oracle.partition_indices(index, local.routing_counts,
                                                         local.ring.global_to_gather, size, local.blocks)
            assert np.array_equal(lists.numpy(), ring[f"{key}/lists"])
            assert np.array_equal(counts.numpy(), ring[f"{key}/counts"])


def test_oracle_partial_merge_equals_joint_softmax():
    gen = torch.Generator().manual_seed(5)
    q = torch.randn(128, 2, 128, generator=gen)
    k = torch.randn(256, 2, 128, generator=gen)
    v = torch.randn(256, 2, 128, generator=gen)
    index = torch.tensor([[0, 1, 2, 3], [1, 3, 0, 0]], dtype=torch.int32)[None, None].expand(1, 2, 2, 4)
    counts = torch.tensor([4, 2], dtype=torch.int32)[None, None].expand(1, 2, 2)
    whole, whole_lse = vsa_oracle.fine_attention(q, k, v, index, counts, None, 0.1)
    parts, lses = [], []
    for ids, n in (([[0, 2], [0, 0]], [2, 0]), ([[1, 3], [1, 3]], [2, 2])):
        idx = torch.tensor(ids, dtype=torch.int32)[None, None].expand(1, 2, 2, 2)
        cnt = torch.tensor(n, dtype=torch.int32)[None, None].expand(1, 2, 2)
        o, lse = vsa_oracle.fine_attention(q, k, v, idx, cnt, None, 0.1)
        parts.append(o)
        lses.append(lse)
    merged, total = vsa_oracle.merge_partials(parts, lses)
    torch.testing.assert_close(merged.float(), whole, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(total.float(), whole_lse, atol=1e-5, rtol=1e-5)
