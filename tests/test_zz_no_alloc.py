"""GPU: ``vsa_route_static``, the routing entry point for callers that cannot allocate.

A plugin inside an inference runtime, or a process whose device memory is owned by another
framework's pool, has no way to hand ``vsa_route`` a scratch buffer.  ``vsa_route_static`` keeps
the score matrix in a 16 MiB array built into the library instead.  The array is shared by all
calls and keeps the previous call's contents, so this test calls it twice in a row on different
inputs and checks both results against ``vsa_route`` (same kernels, so the tables must be
identical).  It lives in its own file, collected last, and passes on its own or after the others.
"""
import pytest
import torch

from cudnn_vsa_b200 import _cabi, vsa_core
from cudnn_vsa_b200.vsa_layout import build_vsa_layout
from tests.helpers import GEOMETRIES, seeded

pytestmark = pytest.mark.gpu


def _means(layout, seed):
    heads = layout.head_num
    q, k, v = (x.cuda() for x in seeded(layout.tokens, heads, seed, 3))
    mean = torch.empty((3, layout.blocks, heads, 128), dtype=torch.float32, device="cuda")
    _cabi.call("vsa_slots_pool", _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(layout.slot_row),
               _cabi.ptr(layout.block_sizes), None, None, None, _cabi.ptr(mean), None, None, 0,
               layout.blocks, heads, _cabi.stream())
    return mean


def _route_static(layout, mean):
    plan = vsa_core.device_plan(layout)
    index = layout.routing_indices.clone()
    for q_begin, q_end, kv_first, kv_last, keep, cursor in plan.spans:
        _cabi.call("vsa_route_static", _cabi.ptr(mean[0]), _cabi.ptr(mean[1]), layout.head_num, q_begin, q_end,
                   0, kv_first, kv_last, 0, keep, cursor, _cabi.ptr(index), index.stride(1), index.shape[-1],
                   _cabi.stream(), launches=2)
    return index


def test_static_scratch_routing_matches_vsa_route_on_two_calls_in_a_row():
    calls = [("c1", 2, 0), ("ragged", 3, 5)]
    for name, heads, seed in calls:
        layout = build_vsa_layout(GEOMETRIES[name], head_num=heads, device="cuda")
        assert vsa_core.device_plan(layout).spans, "the geometry must need top-k selection"
        mean = _means(layout, seed)
        want = vsa_core.route(mean[0], mean[1], layout)
        got = _route_static(layout, mean)
        torch.cuda.synchronize()
        assert torch.equal(got, want), name
        assert not torch.equal(got, layout.routing_indices)


def test_static_scratch_call_leaves_device_memory_as_it_found_it():
    """After the first call on the device (which may load the module that holds the array), a
    call neither takes nor returns device memory: the driver's free-byte count and the bytes
    held by this process's tensors are the same before and after."""
    layout = build_vsa_layout(GEOMETRIES["c1"], head_num=2, device="cuda")
    mean = _means(layout, 0)
    first = _route_static(layout, mean)  # set-up call
    plan = vsa_core.device_plan(layout)
    index = layout.routing_indices.clone()
    torch.cuda.synchronize()
    free_before, held_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    for q_begin, q_end, kv_first, kv_last, keep, cursor in plan.spans:
        _cabi.call("vsa_route_static", _cabi.ptr(mean[0]), _cabi.ptr(mean[1]), layout.head_num, q_begin, q_end,
                   0, kv_first, kv_last, 0, keep, cursor, _cabi.ptr(index), index.stride(1), index.shape[-1],
                   _cabi.stream(), launches=2)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_allocated() == held_before
    assert torch.equal(index, first)


def test_static_scratch_refuses_a_region_beyond_its_capacity():
    # 4096 x 2048 scores of one head need 32 MiB; the built-in array holds 16 MiB.
    mean = torch.zeros((4096, 1, 128), dtype=torch.float32, device="cuda")
    index = torch.zeros((1, 1, 4096, 8), dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="built-in scratch"):
        _cabi.call("vsa_route_static", _cabi.ptr(mean), _cabi.ptr(mean), 1, 0, 4096, 0, 0, 2048, 0, 8, 0,
                   _cabi.ptr(index), index.stride(1), 8, _cabi.stream())
    assert not index.count_nonzero()
