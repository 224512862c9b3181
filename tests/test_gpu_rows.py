"""GPU: row gather / scatter, slot helpers and boundary reorder are bit-exact."""
import pytest
import torch

from cudnn_vsa_b200 import _cabi, vsa_core, vsa_kernels
from cudnn_vsa_b200.vsa import block_wo_padding_to_raster, raster_to_block_wo_padding
from cudnn_vsa_b200.vsa_layout import build_vsa_layout
from oracle import vsa_oracle
from tests.helpers import GEOMETRIES

pytestmark = pytest.mark.gpu
DTYPES = [torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.int8, torch.uint8,
          torch.int16, torch.int32, torch.int64, torch.bool]


def _values(shape, dtype):
    x = torch.randint(-100, 100, shape, device="cuda")
    return (x % 2 == 0) if dtype == torch.bool else x.to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("trailing", [(), (1,), (3,), (2, 128), (5, 7)])
def test_gather_matches_oracle_bit_exact(dtype, trailing):
    torch.manual_seed(3)
    x = _values((97, *trailing), dtype)
    row_map = torch.randint(-1, 97, (211,), device="cuda")
    got = vsa_kernels.gather(x, row_map)
    want = vsa_oracle.gather_rows(x.cpu(), row_map.cpu())
    assert got.dtype == dtype and torch.equal(got.cpu(), want)


@pytest.mark.parametrize("name", ["ragged", "mixed", "partial_blocks", "full_blocks", "c1"])
@pytest.mark.parametrize("order", ["raster", "block"])
def test_slot_round_trip_and_adjoint(name, order):
    layout = build_vsa_layout(GEOMETRIES[name], head_num=2, input_order=order, device="cuda")
    pad = (vsa_kernels.block_wo_padding_to_block_w_padding if order == "block"
           else vsa_kernels.raster_to_block_w_padding)
    restore = (vsa_kernels.block_w_padding_to_block_wo_padding if order == "block"
               else vsa_kernels.block_w_padding_to_raster)
    x = torch.randn(layout.tokens, 2, 8, device="cuda", requires_grad=True)
    slots = pad(x, layout.slot_row, layout.row_slot)
    assert slots.shape[0] == layout.padded_tokens
    assert torch.equal(slots.detach().cpu(), vsa_oracle.gather_rows(x.detach().cpu(), layout.slot_row.cpu()))
    assert not slots[layout.slot_row < 0].count_nonzero()
    back = restore(slots, layout.slot_row, layout.row_slot)
    assert torch.equal(back, x)
    dy = torch.randn_like(x)
    grad, = torch.autograd.grad(back, x, dy)
    assert torch.equal(grad, dy)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.int64, torch.bool])
def test_boundary_reorder_matches_indexing(dtype):
    layout = build_vsa_layout(GEOMETRIES["ragged"], head_num=2, input_order="block", device="cuda")
    for trailing in ((3072,), (3,), ()):
        x = _values((layout.tokens, *trailing), dtype)
        y = raster_to_block_wo_padding(x, vsa_layout=layout)
        assert torch.equal(y, x[layout.input_rows])
        assert torch.equal(block_wo_padding_to_raster(y, vsa_layout=layout), x)


def test_boundary_reorder_second_derivative_and_ring_shard(metadata_group):
    samples = GEOMETRIES["ragged"]
    full = build_vsa_layout(samples, head_num=2, input_order="block", device="cuda")
    local = build_vsa_layout(samples, head_num=2, input_order="block", device="cuda",
                             ring_cp_group=metadata_group(3, 1))
    x = torch.randn(full.tokens, 4, device="cuda", dtype=torch.float64, requires_grad=True)
    y = raster_to_block_wo_padding(x, vsa_layout=local)
    assert y.shape[0] == local.tokens and torch.equal(y, x[local.input_rows])
    w = torch.randn_like(y, requires_grad=True)
    grad, = torch.autograd.grad(y, x, w, create_graph=True)
    expected = torch.zeros_like(x)
    expected[local.input_rows] = w.detach()
    assert torch.equal(grad.detach(), expected)
    second, = torch.autograd.grad(grad, w, torch.ones_like(grad))
    assert torch.equal(second, torch.ones_like(w))
    with pytest.raises(ValueError, match="full VSALayout"):
        block_wo_padding_to_raster(y, vsa_layout=local)


def test_offsets_beyond_int32():
    rows, width = 70000, 32768  # 2.29e9 one-byte elements
    x = torch.arange(rows, device="cuda", dtype=torch.int64).view(-1, 1).expand(rows, width // 8)
    x = (x % 251).to(torch.uint8).repeat(1, 8).contiguous()
    perm = torch.randperm(rows, device="cuda")
    y = vsa_kernels.reorder_tokens(x, perm)
    assert torch.equal(y[:, 0], x[perm, 0]) and torch.equal(y[-1], x[perm[-1]])
    assert torch.equal(vsa_kernels.reorder_tokens(y, perm, inverse=True)[:, -1], x[:, -1])


def test_expired_wait_is_reported_and_the_context_stays_usable():
    # Every mbarrier wait in the tcgen05 kernels is bounded; the self-test entry point makes one
    # run out (a barrier that nothing completes, two million clocks: about a millisecond).
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _cabi.call("vsa_selftest_wait_timeout", _cabi.ptr(status), 2_000_000, _cabi.stream())
    torch.cuda.synchronize()
    assert int(status.item()) == 177  # 100 + the self-test's wait site
    # The host side turns a recorded code into an error ...
    layout = build_vsa_layout(GEOMETRIES["ragged"], head_num=2, device="cuda")
    plan = vsa_core.device_plan(layout)
    plan.status.copy_(status)
    with pytest.raises(RuntimeError, match="177"):
        vsa_core.check_status(layout)
    plan.status.zero_()
    # ... and the context is alive: the next kernels run and give the right answer.
    x = _values((50, 3), torch.int32)
    row_map = torch.randint(-1, 50, (77,), device="cuda")
    assert torch.equal(vsa_kernels.gather(x, row_map).cpu(), vsa_oracle.gather_rows(x.cpu(), row_map.cpu()))
