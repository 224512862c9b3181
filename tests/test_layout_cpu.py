"""CPU: the planner reproduces the reference planner's layouts bit for bit (golden hashes),
matches the oracle's independent block planning, and validates its arguments."""
import hashlib
import json
import random

import pytest
import torch

from cudnn_vsa_b200.vsa_layout import (BLOCK, SampleBlocks, Segment, _plan_ring_blocks, build_vsa_layout)
from oracle import vsa_oracle
from tests.helpers import GEOMETRIES, GOLDEN

FIELDS = ("block_sizes", "row_slot", "slot_row", "coarse_blocks", "coarse_kv_blocks", "coarse_cu_q",
          "coarse_cu_kv", "row_coarse", "input_rows", "routing_indices", "routing_counts", "coarse_rows")
RECORDS = json.loads((GOLDEN / "layouts.json").read_text())


def _digest(t):
    t = t.contiguous().cpu()
    return f"{t.dtype}:{tuple(t.shape)}:" + hashlib.sha256(t.numpy().tobytes()).hexdigest()


def _record(layout):
    rec = {name: _digest(getattr(layout, name)) for name in FIELDS}
    rec["scalars"] = [layout.coarse_max_q, layout.coarse_max_kv, layout.dense_only, layout.tokens,
                      layout.blocks, list(layout.sample_lengths),
                      [[g.start, g.end, g.dense_blocks_num, [list(s) for s in g.video_spans]]
                       for g in layout.groups],
                      [[b, e, o, g.start] for g, b, e, o in layout.routing_groups]]
    if layout.ring is not None:
        r = layout.ring
        rec["ring"] = {"block_ids": _digest(r.block_ids), "peer_block_sizes": _digest(r.peer_block_sizes),
                       "global_to_gather": _digest(r.global_to_gather),
                       "scalars": [r.size, r.rank, r.partition, r.global_tokens,
                                   [[b, e, d, g.start] for g, b, e, d in r.local_groups]]}
    return rec


@pytest.mark.parametrize("key", sorted(RECORDS))
def test_layout_equals_reference_planner(key, metadata_group):
    name, mode, extra = key.split("/")
    heads = 1 if name == "c5" else 2
    if mode.startswith("ring"):
        size, rank = (int(x) for x in mode[4:].split("."))
        layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, input_order="block",
                                  ring_partition=extra, ring_cp_group=metadata_group(size, rank))
    else:
        layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, input_order=mode,
                                  dense_query_full=extra == "dqf1")
    assert _record(layout) == RECORDS[key]


@pytest.mark.parametrize("name", ["ragged", "mixed", "partial_blocks", "fine_only_peer", "dense", "c1"])
def test_layout_equals_oracle_block_planning(name):
    samples = GEOMETRIES[name]
    layout = build_vsa_layout(samples, head_num=2)
    blocks, groups = vsa_oracle.plan_blocks(samples)
    slot_row, row_slot = vsa_oracle.slot_maps(blocks, layout.tokens)
    assert torch.equal(layout.slot_row, slot_row) and torch.equal(layout.row_slot, row_slot)
    assert layout.block_sizes.tolist() == [len(b) for b in blocks]
    assert [(g.start, g.end, g.dense_blocks_num, g.video_spans) for g in layout.groups] == groups
    block_layout = build_vsa_layout(samples, head_num=2, input_order="block")
    assert block_layout.input_rows.tolist() == [r for b in blocks for r in b]
    assert block_layout.slot_row[block_layout.slot_row >= 0].tolist() == list(range(layout.tokens))


def test_explicit_tile_order_and_dense_prefix():
    samples = [[Segment("video", (4, 4, 8), .9), Segment("text", 3)],
               [Segment("video", (1, 2, 3)), Segment("text", 0)],
               [Segment("video", (2, 1, 2), .9), Segment("text", 2)]]
    layout = build_vsa_layout(samples, head_num=2)
    tile = lambda w0: [f * 32 + h * 8 + w for f in range(4) for h in range(4) for w in range(w0, w0 + 4)]
    blocks = [[128, 129, 130], tile(0), tile(4), list(range(131, 137)), [141, 142], list(range(137, 141))]
    expected = [r for b in blocks for r in b + [-1] * (BLOCK - len(b))]
    assert layout.slot_row.tolist() == expected
    assert layout.sample_lengths == (131, 6, 6)
    assert layout.sample_slices[2] == (slice(137, 141), slice(141, 143))


def test_keep_uses_python_float_arithmetic():
    # (1 - 0.95) * 14720 = 736.0000000000007 rounds up to 737; (1 - 0.9) * 1920 rounds to 192.
    assert build_vsa_layout(GEOMETRIES["c5"], head_num=1).groups[0].video_spans[0][2] == 737
    assert build_vsa_layout(GEOMETRIES["c2"], head_num=1).groups[0].video_spans[0][2] == 192


@pytest.mark.parametrize("head_num", [0, -1, 1.5, True, None])
@pytest.mark.parametrize("ring", [False, True])
def test_rejects_bad_head_num(head_num, ring, metadata_group):
    kwargs = dict(ring_cp_group=metadata_group(2, 0), input_order="block") if ring else {}
    with pytest.raises(ValueError, match="head_num"):
        build_vsa_layout([[Segment("video", (1, 2, 3))]], head_num=head_num, **kwargs)


@pytest.mark.parametrize("value", [None, 1, "False"])
def test_rejects_bad_dense_query_full(value):
    with pytest.raises(ValueError, match="dense_query_full"):
        build_vsa_layout([[Segment("video", (1, 2, 3))]], head_num=2, dense_query_full=value)


@pytest.mark.parametrize("samples", [[], [[]], [Segment("video", (2, 4, 4))], [[(2, 4, 4)]],
                                     [[Segment("text", 4)]], None])
def test_rejects_bad_samples(samples):
    with pytest.raises(ValueError):
        build_vsa_layout(samples, head_num=2)


@pytest.mark.parametrize("sparsity", [-.1, 1.1, float("nan"), float("inf"), [.5], "0.5"])
def test_rejects_bad_sparsity(sparsity):
    with pytest.raises(ValueError, match="sparsity"):
        Segment("video", (2, 4, 4), sparsity=sparsity)


@pytest.mark.parametrize("kind,size", [("audio", (1, 2, 3)), ("video", 12), ("video", (0, 4, 4)),
                                       ("text", -1), ("image", 3)])
def test_rejects_bad_segments(kind, size):
    with pytest.raises(ValueError):
        Segment(kind, size)
    with pytest.raises(ValueError, match="only supported for video"):
        Segment("text", 3, sparsity=0)


def test_ring_option_validation(metadata_group):
    samples = GEOMETRIES["partial_blocks"]
    with pytest.raises(ValueError, match="require ring_cp_group"):
        build_vsa_layout(samples, head_num=2, ring_partition="contiguous")
    with pytest.raises(ValueError, match="require ring_cp_group"):
        build_vsa_layout(samples, head_num=2, ring_cp_batch_p2p=True)
    with pytest.raises(ValueError, match="input_order"):
        build_vsa_layout(samples, head_num=2, ring_cp_group=metadata_group(2, 0))
    with pytest.raises(ValueError, match="ring_cp_bwd_bucket_size"):
        build_vsa_layout(samples, head_num=2, input_order="block", ring_cp_group=metadata_group(2, 0),
                         ring_cp_bwd_bucket_size=0)
    with pytest.raises(ValueError, match="at least ring_size"):
        build_vsa_layout(samples, head_num=2, input_order="block", ring_cp_group=metadata_group(4, 0))
    with pytest.raises(ValueError, match="ProcessGroup"):
        build_vsa_layout(samples, head_num=2, input_order="block", ring_cp_group="group")


@pytest.mark.parametrize("size", [1, 2, 3, 8, 72])
@pytest.mark.parametrize("partition", ["cyclic", "contiguous"])
def test_ring_planner_covers_balances_and_keeps_order(size, partition):
    rng = random.Random(71 + size)
    for _ in range(40):
        total = rng.randint(size, size + 192)
        cuts = sorted({0, total, *[rng.randrange(total + 1) for _ in range(30)]})
        groups = [SampleBlocks(a, b, b - a, ()) for a, b in zip(cuts, cuts[1:])]
        owned = _plan_ring_blocks(groups, size, partition)
        assert sorted(b for ids in owned for b in ids) == list(range(total))
        assert all(0 < len(ids) <= -(-total // size) for ids in owned)
        for ids in owned:
            assert ids == sorted(ids)
        for g in groups:
            counts = [sum(g.start <= b < g.end for b in ids) for ids in owned]
            upto = [sum(b < g.end for b in ids) for ids in owned]
            assert max(counts) - min(counts) <= 1 and max(upto) - min(upto) <= 1


def test_contiguous_planner_rotates_the_remainder():
    groups = [SampleBlocks(a, b, b - a, ()) for a, b in [(0, 5), (5, 10), (10, 14)]]
    assert _plan_ring_blocks(groups, 4, "contiguous") == [[0, 1, 9, 12], [2, 5, 6, 13], [3, 7, 10], [4, 8, 11]]
