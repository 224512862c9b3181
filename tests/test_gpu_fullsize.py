"""GPU: the configurations named for the benchmark at their full sizes, checked through
properties that do not need a full-size oracle: sampled blocks against the CPU oracle, exact row
maps on wide rows, linearity of the gate term and of the backward pass, fine-only samples."""
import pytest
import torch

from cudnn_vsa_b200 import _cabi, vsa_core
from cudnn_vsa_b200.vsa import block_wo_padding_to_raster, raster_to_block_wo_padding, vsa_attention
from cudnn_vsa_b200.vsa_layout import BLOCK, build_vsa_layout
from oracle import vsa_oracle
from tests.helpers import GEOMETRIES, assert_close

pytestmark = pytest.mark.gpu


def _inputs(tokens, heads, count, seed=0):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    return [torch.randn(tokens, heads, 128, device="cuda", dtype=torch.bfloat16, generator=gen)
            for _ in range(count)]


def test_single_720p_sample_sampled_blocks_match_oracle():
    heads = 12
    layout = build_vsa_layout(GEOMETRIES["c2"], head_num=heads, device="cuda")
    q, k, v, gate, dy = _inputs(layout.tokens, heads, 5)
    leaves = [x.requires_grad_() for x in (q, k, v, gate)]
    out = vsa_attention(*leaves, layout)
    grads = torch.autograd.grad(out, leaves, dy)
    vsa_core.check_status(layout)
    assert all(torch.isfinite(t).all() for t in (out, *grads))
    index = vsa_core.last_routing(layout)
    counts = layout.routing_counts
    assert int(counts.min()) == int(counts.max()) == 224
    valid_rows = index[0]
    assert (valid_rows[..., 1:] > valid_rows[..., :-1]).all(), "ascending, duplicate-free lists"
    assert (valid_rows[..., :32] == torch.arange(32, device="cuda")).all(), "dense blocks always listed"
    # Fine attention of a few query blocks and heads, recomputed by the oracle from the same slots.
    plan = vsa_core.device_plan(layout)
    slots = [torch.empty((layout.padded_tokens, heads, 128), dtype=q.dtype, device="cuda") for _ in range(3)]
    _cabi.call("vsa_slots_pool", _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(layout.slot_row),
               _cabi.ptr(layout.block_sizes), *(_cabi.ptr(s) for s in slots), None, None, None, 0,
               layout.blocks, heads, _cabi.stream())
    strides = (index.stride(1), counts.stride(1))
    fine, lse = vsa_core._fine_fwd(slots[0], slots[1], slots[2], index, counts, strides, plan.sizes,
                                   128 ** -0.5, plan.status)
    picked = torch.tensor([0, 31, 32, 700, 1500, 1951])
    use_heads = [0, 7]
    rows = (picked[:, None] * BLOCK + torch.arange(BLOCK)[None, :]).reshape(-1)
    q_sub = slots[0][rows.cuda()][:, use_heads].cpu()
    k_cpu, v_cpu = (s[:, use_heads].cpu() for s in slots[1:])
    sub_index = index[:, use_heads][:, :, picked.cuda()].cpu().contiguous()
    sub_counts = counts[:, use_heads][:, :, picked.cuda()].cpu().contiguous()
    want, want_lse = vsa_oracle.fine_attention(q_sub, k_cpu, v_cpu, sub_index, sub_counts,
                                               layout.block_sizes.cpu(), 128 ** -0.5)
    assert_close(fine[rows.cuda()][:, use_heads], want, "sampled fine output")
    torch.testing.assert_close(lse[use_heads][:, rows.cuda()].cpu(), want_lse, atol=2e-3, rtol=1e-3)


def test_packed_sample_gate_term_backward_linearity_and_fine_only_samples():
    heads = 4
    layout = build_vsa_layout(GEOMETRIES["c3"], head_num=heads, device="cuda")
    q, k, v, gate, dy = _inputs(layout.tokens, heads, 5)
    dense_rows = slice(layout.sample_lengths[0], layout.tokens)  # samples 1 and 2 are fine-only
    assert layout.groups[1].dense_only and layout.groups[2].dense_only
    base = vsa_attention(q, k, v, torch.zeros_like(gate), layout)
    with_gate = vsa_attention(q, k, v, gate, layout)
    poisoned = gate.clone()
    poisoned[dense_rows] = float("nan")
    assert torch.equal(vsa_attention(q, k, v, poisoned, layout), with_gate), "fine-only rows never read gate"
    assert torch.equal(with_gate[dense_rows], base[dense_rows])
    # out - out(gate=0) = gate * coarse[block]: dividing by the gate recovers one coarse row per block.
    vsa_rows = slice(0, layout.sample_lengths[0])
    ratio = (with_gate[vsa_rows].float() - base[vsa_rows].float()) / gate[vsa_rows].float()
    block_of_row = (layout.row_slot[vsa_rows] // BLOCK).long()
    strong = gate[vsa_rows].float().abs() > 1.0
    ratio = torch.where(strong, ratio, torch.zeros_like(ratio))
    sums = torch.zeros((layout.blocks, heads, 128), device="cuda").index_add_(0, block_of_row, ratio)
    cnt = torch.zeros((layout.blocks, heads, 128), device="cuda").index_add_(0, block_of_row, strong.float())
    mean = sums / cnt.clamp_min(1)
    spread = torch.where(strong, ratio - mean[block_of_row], torch.zeros_like(ratio)).abs().max().item()
    assert spread < 6e-2, spread  # BF16 rounding of out and out(0) divided by |gate| > 1
    # The backward pass is linear in dO.
    leaves = [x.clone().requires_grad_() for x in (q, k, v, gate)]
    out = vsa_attention(*leaves, layout)
    g1 = torch.autograd.grad(out, leaves, dy, retain_graph=True)
    g2 = torch.autograd.grad(out, leaves, dy * 2)
    for a, b, name in zip(g1, g2, ("dq", "dk", "dv", "dgate")):
        assert_close(b, a.float() * 2, f"linearity {name}", max_abs=2e-2, rel_l2=6e-3)
    assert not g1[3][dense_rows].count_nonzero(), "no gate gradient on fine-only samples"
    vsa_core.check_status(layout)


def test_block_order_stack_reuses_one_layout_and_reorders_wide_rows_exactly():
    heads = 4
    layout = build_vsa_layout(GEOMETRIES["c4"], head_num=heads, device="cuda", input_order="block")
    tokens = layout.tokens
    hidden = torch.randn(tokens, 3072, device="cuda", dtype=torch.bfloat16)
    position = torch.arange(tokens * 3, device="cuda", dtype=torch.int64).view(tokens, 3)
    hidden_b = raster_to_block_wo_padding(hidden, vsa_layout=layout)
    position_b = raster_to_block_wo_padding(position, vsa_layout=layout)
    assert torch.equal(hidden_b, hidden[layout.input_rows]) and torch.equal(position_b, position[layout.input_rows])
    assert torch.equal(block_wo_padding_to_raster(hidden_b, vsa_layout=layout), hidden)
    assert torch.equal(block_wo_padding_to_raster(position_b, vsa_layout=layout), position)
    # Three stacked calls through one layout, block-ordered activations, gradients through all.
    x = _inputs(tokens, heads, 1, seed=3)[0].requires_grad_()
    y = x
    for layer in range(3):
        y = vsa_attention(y, y, y, torch.full_like(y, 0.5), layout)
    grad, = torch.autograd.grad(y, x, torch.ones_like(y))
    assert torch.isfinite(y).all() and torch.isfinite(grad).all()
    # Same stack in raster order gives the same result after reordering.
    raster_layout = build_vsa_layout(GEOMETRIES["c4"], head_num=heads, device="cuda")
    xr = block_wo_padding_to_raster(x.detach(), vsa_layout=layout)
    yr = xr
    for layer in range(3):
        yr = vsa_attention(yr, yr, yr, torch.full_like(yr, 0.5), raster_layout)
    assert_close(raster_to_block_wo_padding(yr, vsa_layout=layout), y, "raster vs block order stack")
    vsa_core.check_status(layout)
