"""GPU parity of the fused kernels, called through the C ABI, against the CPU oracle and the
golden vectors produced by the reference's own CPU code.

Tolerances are the ones stated for BF16 outputs and gradients against an FP32 reference:
max-abs <= 2e-2 and relative L2 <= 1e-2.  Integer results (slots, routing) are bit-exact,
routing up to near-ties (pooled-score gap below 1e-4 relative).
"""
import pytest
import torch

from cudnn_vsa_b200 import _cabi, vsa_core
from cudnn_vsa_b200.vsa import vsa_attention
from cudnn_vsa_b200.vsa_layout import BLOCK, build_vsa_layout
from oracle import vsa_oracle
from tests.helpers import (GEOMETRIES, assert_close, from_bits, golden_cases,
                           routing_mismatches_are_near_ties, seeded)

pytestmark = pytest.mark.gpu
SMALL = ["mixed", "ragged", "partial_blocks", "fine_only_peer", "dense", "zero_sparsity", "full_blocks", "c1"]


def _pooled(layout, q, k, v):
    plan = vsa_core.device_plan(layout)
    heads = q.shape[1]
    mean = torch.empty((3, layout.blocks, heads, 128), dtype=torch.float32, device="cuda")
    slots = [torch.empty((layout.padded_tokens, heads, 128), dtype=q.dtype, device="cuda") for _ in range(3)]
    coarse = plan.coarse
    tokens = (torch.zeros((3, coarse.q_rows, heads, 128), dtype=q.dtype, device="cuda")
              if coarse is not None else None)
    _cabi.call("vsa_slots_pool", _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(layout.slot_row),
               _cabi.ptr(layout.block_sizes), *(_cabi.ptr(s) for s in slots), _cabi.ptr(mean),
               _cabi.ptr(coarse.block_q) if coarse is not None else None, _cabi.ptr(tokens),
               coarse.q_rows if coarse is not None else 0, layout.blocks, heads, _cabi.stream())
    return slots, mean, tokens


@pytest.mark.parametrize("name", SMALL)
def test_slots_and_block_means(name):
    heads = 2
    layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, device="cuda")
    q, k, v = (x.cuda() for x in seeded(layout.tokens, heads, 0, 3))
    slots, mean, tokens = _pooled(layout, q, k, v)
    for got, x in zip(slots, (q, k, v)):
        want = vsa_oracle.gather_rows(x.cpu(), layout.slot_row.cpu())
        assert torch.equal(got.cpu(), want)
    for i, s in enumerate(slots):
        want = vsa_oracle.block_means(s.cpu(), layout.block_sizes.cpu())
        torch.testing.assert_close(mean[i].cpu(), want, atol=1e-6, rtol=1e-5)
    plan = vsa_core.device_plan(layout)
    if plan.coarse is not None:
        rows = plan.coarse.block_q.long()
        used = rows >= 0
        for i in range(3):
            assert torch.equal(tokens[i][rows[used]], mean[i][used].to(torch.bfloat16))
        untouched = torch.ones(plan.coarse.q_rows, dtype=torch.bool, device="cuda")
        untouched[rows[used]] = False
        assert not tokens[:, untouched].count_nonzero()


@pytest.mark.parametrize("name", ["mixed", "ragged", "c1", "full_blocks"])
@pytest.mark.parametrize("dense_query_full", [False, True])
def test_routing_matches_oracle_and_reference(name, dense_query_full):
    heads = 2
    layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, device="cuda",
                              dense_query_full=dense_query_full)
    cpu_layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, dense_query_full=dense_query_full)
    q, k, v = (x.cuda() for x in seeded(layout.tokens, heads, 0, 3))
    slots, mean, _ = _pooled(layout, q, k, v)
    template = layout.routing_indices.clone()
    got = vsa_core.route(mean[0], mean[1], layout).cpu()
    assert torch.equal(layout.routing_indices, template), "the template must never be modified"
    # Oracle means are pooled over the coarse blocks only, like the reference's.
    qm, km = (vsa_oracle.block_means(s.cpu(), cpu_layout.block_sizes)[cpu_layout.coarse_blocks]
              for s in slots[:2])
    want = vsa_oracle.route(qm, km, cpu_layout)
    scores = vsa_oracle.routing_scores(qm, km, cpu_layout)
    counts = cpu_layout.routing_counts
    assert routing_mismatches_are_near_ties(got, want, scores, counts)
    valid = torch.arange(got.shape[-1]) < counts[..., None]
    rows = torch.where(valid, got, torch.iinfo(torch.int32).max)
    assert (rows[..., 1:] > rows[..., :-1]).logical_or(~valid[..., 1:]).all(), "lists must be ascending"
    key = f"{name}/dqf{int(dense_query_full)}/routing"
    cases = golden_cases()
    if key in cases.files:
        assert routing_mismatches_are_near_ties(got, torch.from_numpy(cases[key]), scores, counts)


def test_routing_of_a_14720_block_region_in_several_head_passes():
    """The region of the ring configuration: 14,720 scores per row (more than the 48 KiB of static
    shared memory, so the selection kernel runs with its opt-in size) and 737 kept.  The scratch
    holds one head's score matrix, so the three heads take three passes."""
    heads, rows, region, keep = 3, 8, 14720, 737
    gen = torch.Generator().manual_seed(5)
    q_mean = torch.randn(rows, heads, 128, generator=gen) * 0.2
    k_mean = torch.randn(region, heads, 128, generator=gen) * 0.2
    index = torch.zeros((1, heads, rows, keep), dtype=torch.int32, device="cuda")
    scratch = torch.empty(rows * region * 4, dtype=torch.uint8, device="cuda")
    dq, dk = q_mean.cuda(), k_mean.cuda()
    _cabi.call("vsa_route", _cabi.ptr(dq), _cabi.ptr(dk), heads, 0, rows, 0, 0, region, 0, keep, 0,
               _cabi.ptr(index), index.stride(1), keep, _cabi.ptr(scratch), scratch.numel(), _cabi.stream(),
               launches=2 * heads)
    got = index.cpu()
    scores = torch.einsum("qhd,khd->hqk", q_mean, k_mean)
    want = scores.topk(keep, dim=-1, sorted=False).indices.sort(-1).values.to(torch.int32)[None]
    assert (got[..., 1:] > got[..., :-1]).all(), "ascending, duplicate-free"
    assert got.min() >= 0 and got.max() < region
    spans = [(0, rows, 0, region, keep, 0, scores)]
    assert routing_mismatches_are_near_ties(got, want, spans, None)
    assert (got == want).float().mean().item() > 0.999


def _random_lists(heads, q_blocks, kv_blocks, cap, gen):
    index = torch.zeros((1, heads, q_blocks, cap), dtype=torch.int32)
    counts = torch.zeros((1, heads, q_blocks), dtype=torch.int32)
    for h in range(heads):
        for b in range(q_blocks):
            n = int(torch.randint(0 if b == 1 else 1, min(cap, kv_blocks) + 1, (1,), generator=gen))
            if b == 0 and h == 0:
                n = min(cap, kv_blocks)  # one list of full length in every case
            ids = torch.randperm(kv_blocks, generator=gen)[:n].sort().values
            index[0, h, b, :n] = ids.to(torch.int32)
            counts[0, h, b] = n
    return index, counts


# List lengths from 0 to `cap`: every tail of the pair / stage / buffer rings (odd lists, one pair
# only, lengths around the ring wrap points) occurs in some (head, query block).
# The last case has the list length of the ring configuration (801 blocks: 401 pairs, every ring
# of stages and buffers wraps more than a hundred times) and more than two mask words.
@pytest.mark.parametrize("heads,q_blocks,kv_blocks,cap", [(1, 2, 3, 3), (2, 5, 9, 6), (3, 4, 40, 33), (2, 24, 20, 15),
                                                           (1, 9, 70, 64), (1, 3, 900, 801), (5, 70, 6, 6)])
def test_fine_forward_and_backward_on_given_lists(heads, q_blocks, kv_blocks, cap):
    gen = torch.Generator().manual_seed(11)
    q = torch.randn(q_blocks * BLOCK, heads, 128, generator=gen).to(torch.bfloat16)
    k = torch.randn(kv_blocks * BLOCK, heads, 128, generator=gen).to(torch.bfloat16)
    v = torch.randn(kv_blocks * BLOCK, heads, 128, generator=gen).to(torch.bfloat16)
    d_o = torch.randn(q_blocks * BLOCK, heads, 128, generator=gen).to(torch.bfloat16)
    sizes = torch.randint(1, BLOCK + 1, (kv_blocks,), generator=gen).to(torch.int32)
    sizes[0] = BLOCK
    valid = (torch.arange(BLOCK)[None, :] < sizes[:, None]).reshape(-1)
    k[~valid] = 0
    v[~valid] = 0
    index, counts = _random_lists(heads, q_blocks, kv_blocks, cap, gen)
    scale = 128 ** -0.5
    qf, kf, vf = (x.float().requires_grad_() for x in (q, k, v))
    want_o, want_lse = vsa_oracle.fine_attention(qf, kf, vf, index, counts, sizes, scale)
    want_dq, want_dk, want_dv = torch.autograd.grad(want_o, (qf, kf, vf), d_o.float())
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    dev = [x.cuda() for x in (q, k, v, d_o, index, counts, sizes)]
    strides = (dev[4].stride(1), dev[5].stride(1))
    o, lse = vsa_core._fine_fwd(dev[0], dev[1], dev[2], dev[4], dev[5], strides, dev[6], scale, status)
    assert_close(o.cpu(), want_o, "fine out")
    live = torch.isfinite(want_lse)
    assert torch.equal(torch.isfinite(lse.cpu()), live)
    torch.testing.assert_close(lse.cpu()[live], want_lse[live], atol=2e-3, rtol=1e-3)
    delta = (d_o.float() * o.float().cpu()).sum(-1).transpose(0, 1).contiguous().cuda()
    q_sizes = torch.full((q_blocks,), BLOCK, dtype=torch.int32, device="cuda")
    dq, dk, dv = vsa_core._fine_bwd(dev[0], dev[1], dev[2], dev[3], dev[4], dev[5], strides, q_sizes,
                                    dev[6], scale, lse, delta, status)
    assert int(status.item()) == 0
    assert_close(dq.cpu(), want_dq, "dq")
    assert_close(dk.cpu()[valid], want_dk[valid], "dk", peak_relative=True)
    assert_close(dv.cpu()[valid], want_dv[valid], "dv", peak_relative=True)


def _run(layout, q, k, v, gate, dy):
    leaves = [x.cuda().requires_grad_() for x in (q, k, v, gate)]
    out = vsa_attention(*leaves, layout)
    assert out.is_contiguous() and out.shape == leaves[0].shape and out.dtype == torch.bfloat16
    grads = torch.autograd.grad(out, leaves, dy.cuda(), allow_unused=True)
    vsa_core.check_status(layout)
    return out, grads


@pytest.mark.parametrize("name", SMALL)
@pytest.mark.parametrize("order", ["raster", "block"])
def test_attention_against_fp32_oracle(name, order):
    heads = 2
    layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, device="cuda", input_order=order)
    cpu_layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, input_order=order)
    q, k, v, gate = seeded(layout.tokens, heads, 0, 4)
    dy, = seeded(layout.tokens, heads, 1, 1)
    for group, slices in zip(cpu_layout.groups, cpu_layout.sample_slices):
        if group.dense_only and order == "raster":
            gate[slices[0].start:slices[-1].stop] = float("nan")  # must be ignored
    out, grads = _run(layout, q, k, v, gate, dy)
    # The oracle reuses the kernel's routing table, so numerics are judged apart from near-ties.
    plan = vsa_core.device_plan(layout)
    index = layout.routing_indices
    if plan.spans:
        slots, mean, _ = _pooled(layout, q.cuda(), k.cuda(), v.cuda())
        index = vsa_core.route(mean[0], mean[1], layout)
    leaves = [x.float().requires_grad_() for x in (q, k, v, gate)]
    want, _ = vsa_oracle.vsa_attention(*leaves, cpu_layout, indices=index.cpu())
    want_grads = torch.autograd.grad(want, leaves, dy.float(), allow_unused=True)
    assert_close(out.cpu(), want, f"{name} out")
    for tag, got, ref in zip(("dq", "dk", "dv", "dgate"), grads, want_grads):
        if tag == "dgate" and layout.dense_only:
            assert got is None
            continue
        ref = torch.zeros_like(q, dtype=torch.float32) if ref is None else ref.nan_to_num()
        assert_close(got.cpu(), ref, f"{name} {tag}", peak_relative=tag in ("dk", "dv"))


@pytest.mark.parametrize("name,order,chunk", [("ragged", "raster", 8), ("c1", "block", 10), ("mixed", "raster", 3),
                                              ("full_blocks", "block", 2), ("dense", "raster", 2)])
def test_large_layout_passes_match_the_single_pass_path(name, order, chunk, monkeypatch):
    """A layout with more blocks than one pass covers runs the fine attention in passes over KV
    ranges (forward, dQ) and query-block ranges (dK/dV) into FP32 running results; forced here on
    small geometries by a tiny pass size and compared with the one-pass path on the same inputs."""
    from cudnn_vsa_b200 import vsa_ring
    heads = 2
    layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, device="cuda", input_order=order)
    q, k, v, gate = seeded(layout.tokens, heads, 0, 4)
    dy, = seeded(layout.tokens, heads, 1, 1)
    want_out, want_grads = _run(layout, q, k, v, gate, dy)
    monkeypatch.setattr(vsa_ring, "RING_CHUNK_BLOCKS", chunk)
    assert vsa_ring._passes(layout.blocks)[0] > 1
    out, grads = _run(layout, q, k, v, gate, dy)
    vsa_core.check_status(layout)
    assert_close(out, want_out.float(), f"{name} out in passes", max_abs=8e-3, rel_l2=4e-3)
    for tag, got, ref in zip(("dq", "dk", "dv", "dgate"), grads, want_grads):
        if ref is None:
            assert got is None
            continue
        assert_close(got, ref.float(), f"{name} {tag} in passes", max_abs=2e-2, rel_l2=6e-3,
                     peak_relative=tag in ("dk", "dv"))


@pytest.mark.parametrize("name", SMALL)
def test_attention_against_reference_golden_vectors(name):
    """Output and gradients against the vectors of the reference's own CPU code.  Those carry the
    reference's top-k choices: where the kernel's routing table differs from the stored one (a
    near-tie, checked by the routing test), the rows of the query blocks whose lists differ are
    left out for out / dq / dgate, and the rows of every KV block on such a list for dk / dv.
    Everything else must meet the stated bounds."""
    heads = 2
    cases = golden_cases()
    layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, device="cuda")
    q, k, v, gate = seeded(layout.tokens, heads, 0, 4)
    dy, = seeded(layout.tokens, heads, 1, 1)
    out, grads = _run(layout, q, k, v, gate, dy)
    index = layout.routing_indices
    if vsa_core.device_plan(layout).spans:
        _, mean, _ = _pooled(layout, q.cuda(), k.cuda(), v.cuda())
        index = vsa_core.route(mean[0], mean[1], layout)
    index, counts = index.cpu(), layout.routing_counts.cpu()
    key = f"{name}/dqf0/routing"
    stored = torch.from_numpy(cases[key]) if key in cases.files else index
    listed = torch.arange(index.shape[-1]) < counts[..., None]
    differ = ((index != stored) & listed).any(-1)[0]          # [heads, blocks]
    skip_q = differ.any(0)
    skip_kv = torch.zeros(layout.blocks, dtype=torch.bool)
    for h, b in differ.nonzero().tolist():
        for table in (index, stored):
            skip_kv[table[0, h, b, :counts[0, h, b]].long()] = True
    assert skip_q.float().mean().item() <= 0.1, "routing differs from the reference on too many query blocks"
    row_block = (layout.row_slot.cpu() // BLOCK).long()
    stride = 4 if layout.tokens > 600 else 1
    for tag, got in zip(("out", "dq", "dk", "dv", "dgate"), (out, *grads)):
        want = from_bits(cases[f"{name}/dqf0/pack/{tag}"]).float()
        got = (torch.zeros_like(q).cuda() if got is None else got).float().cpu()
        keep = ~(skip_kv if tag in ("dk", "dv") else skip_q)[row_block]
        assert_close(got[::stride][keep[::stride]], want[keep[::stride]], f"{name} {tag} vs reference",
                     peak_relative=tag in ("dk", "dv"))


def test_cuda_graph_capture_and_replay_with_changed_inputs():
    heads = 2
    layout = build_vsa_layout(GEOMETRIES["mixed"], head_num=heads, device="cuda")
    leaves = [x.cuda().requires_grad_() for x in seeded(layout.tokens, heads, 0, 4)]
    dy = seeded(layout.tokens, heads, 1, 1)[0].cuda()

    def step():
        out = vsa_attention(*leaves, layout)
        return (out, *torch.autograd.grad(out, leaves, dy))

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        captured = step()
    for changed in (False, True):
        if changed:
            with torch.no_grad():
                for x in (*leaves, dy):
                    x.normal_()
        eager = [t.clone() for t in step()]
        graph.replay()
        torch.cuda.synchronize()
        for a, b in zip(captured, eager):
            assert torch.equal(a, b)
    vsa_core.check_status(layout)


def test_retained_graph_second_backward_is_identical():
    heads = 2
    layout = build_vsa_layout(GEOMETRIES["ragged"], head_num=heads, device="cuda")
    leaves = [x.cuda().requires_grad_() for x in seeded(layout.tokens, heads, 0, 4)]
    dy = seeded(layout.tokens, heads, 1, 1)[0].cuda()
    out = vsa_attention(*leaves, layout)
    first = torch.autograd.grad(out, leaves, dy, retain_graph=True)
    second = torch.autograd.grad(out, leaves, dy)
    for a, b in zip(first, second):
        assert torch.equal(a, b)


@pytest.mark.parametrize("name,order", [("ragged", "raster"), ("mixed", "block"), ("full_blocks", "block"),
                                        ("dense", "raster"), ("c1", "raster")])
def test_fused_projection_input_is_bit_identical_to_separate_tensors(name, order):
    """``vsa_attention_fused`` on one interleaved [T, H, 4, 128] tensor against ``vsa_attention`` on
    its four contiguous fields: same kernels, strided reads and writes - output and the gradient
    of the interleaved tensor must match bit for bit."""
    from cudnn_vsa_b200.vsa import vsa_attention_fused
    heads = 3
    layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, device="cuda", input_order=order)
    gen = torch.Generator(device="cuda").manual_seed(3)
    mixed = torch.randn(layout.tokens, heads, 4, 128, device="cuda", dtype=torch.bfloat16, generator=gen)
    dy = torch.randn(layout.tokens, heads, 128, device="cuda", dtype=torch.bfloat16, generator=gen)
    fused_in = mixed.clone().requires_grad_()
    out = vsa_attention_fused(fused_in, layout)
    grad, = torch.autograd.grad(out, fused_in, dy)
    ref_in = mixed.clone().requires_grad_()
    ref_out = vsa_attention(*(t.contiguous() for t in ref_in.unbind(2)), layout)
    ref_grad, = torch.autograd.grad(ref_out, ref_in, dy)
    vsa_core.check_status(layout)
    assert torch.equal(out, ref_out)
    assert torch.equal(grad, ref_grad)
    with pytest.raises(ValueError, match="contiguous"):
        vsa_attention_fused(mixed.transpose(0, 1).contiguous().transpose(0, 1), layout)
    with pytest.raises(ValueError, match="4, head_dim"):
        vsa_attention_fused(mixed[:, :, :3].contiguous(), layout)
