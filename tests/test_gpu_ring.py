"""GPU: ring path.  On one GPU the ring's arithmetic is checked without transport (every rank's
steps are replayed one after another in one process); with two or more GPUs the real NCCL ring
runs under torchrun against the single-device result."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist

from cudnn_vsa_b200 import _cabi, vsa_core, vsa_ring
from cudnn_vsa_b200.vsa import raster_to_block_wo_padding, vsa_attention
from cudnn_vsa_b200.vsa_layout import BLOCK, build_vsa_layout
from oracle import vsa_oracle
from tests.helpers import GEOMETRIES, assert_close, seeded

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _slots(layout, x):
    return raster_to_block_wo_padding(x, vsa_layout=layout)


@pytest.mark.parametrize("name,size", [("ragged", 2), ("ragged", 3), ("mixed", 4), ("c1", 8)])
@pytest.mark.parametrize("partition", ["cyclic", "contiguous"])
def test_ring_steps_replayed_on_one_gpu(name, size, partition, metadata_group):
    """Partition of the global routing rows, per-owner fine passes and the running merge give the
    single-device fine output; the per-step backward passes sum to the single-device gradients."""
    heads, scale = 2, 128 ** -0.5
    samples = GEOMETRIES[name]
    full = build_vsa_layout(samples, head_num=heads, device="cuda", input_order="block")
    q, k, v = (x.cuda() for x in seeded(full.tokens, heads, 0, 3))
    d_o = seeded(full.tokens, heads, 1, 1)[0].cuda()
    locals_ = [build_vsa_layout(samples, head_num=heads, device="cuda", input_order="block",
                                ring_cp_group=metadata_group(size, r), ring_partition=partition)
               for r in range(size)]
    p = _cabi.ptr
    shards = []
    for lay in locals_:
        slots = [torch.empty((lay.padded_tokens, heads, 128), dtype=q.dtype, device="cuda") for _ in range(4)]
        mean = torch.empty((3, lay.blocks, heads, 128), dtype=torch.float32, device="cuda")
        xs = [_slots(lay, x) for x in (q, k, v)]
        _cabi.call("vsa_slots_pool", p(xs[0]), p(xs[1]), p(xs[2]), p(lay.slot_row), p(lay.block_sizes),
                   p(slots[0]), p(slots[1]), p(slots[2]), p(mean), None, None, 0, lay.blocks, heads, _cabi.stream())
        slots[3] = vsa_oracle.gather_rows(_slots(lay, d_o).cpu(), lay.slot_row.cpu()).cuda()
        shards.append((slots, mean))
    # Global pooled K in global block order, as the all-gather + reorder would deliver it.
    g2g = locals_[0].ring.global_to_gather
    k_all = torch.cat([m[1] for _, m in shards])[g2g]
    # Single-device reference on the same slots (fine part only).
    fslots = [vsa_oracle.gather_rows(_slots(full, x).cpu(), full.slot_row.cpu()).cuda() for x in (q, k, v, d_o)]
    fmean = torch.empty((3, full.blocks, heads, 128), dtype=torch.float32, device="cuda")
    xs = [_slots(full, x) for x in (q, k, v)]
    _cabi.call("vsa_slots_pool", p(xs[0]), p(xs[1]), p(xs[2]), p(full.slot_row), p(full.block_sizes), None, None,
               None, p(fmean), None, None, 0, full.blocks, heads, _cabi.stream())
    findex = vsa_core.route(fmean[0], fmean[1], full)
    fplan = vsa_core.device_plan(full)
    fcounts = full.routing_counts
    fstr = (findex.stride(1), fcounts.stride(1))
    fo, flse = vsa_core._fine_fwd(fslots[0], fslots[1], fslots[2], findex, fcounts, fstr, fplan.sizes, scale,
                                  fplan.status)
    fdelta = (fslots[3].float() * fo.float()).sum(-1).transpose(0, 1).contiguous()
    fdq, fdk, fdv = vsa_core._fine_bwd(fslots[0], fslots[1], fslots[2], fslots[3], findex, fcounts, fstr,
                                       full.block_sizes, fplan.sizes, scale, flse, fdelta, fplan.status)
    for grad in (fdq, fdk, fdv):  # the kernels leave padding slots unwritten
        grad[full.slot_row < 0] = 0
    dk_acc = [torch.zeros((lay.padded_tokens, heads, 128), dtype=torch.float32, device="cuda") for lay in locals_]
    dv_acc = [torch.zeros_like(x) for x in dk_acc]
    for rank, lay in enumerate(locals_):
        rt = vsa_ring._RingRuntime(None, rank, size, None, False, tuple(range(size)))
        (q_s, _, _, do_s), mean = shards[rank]
        index = vsa_core.route(mean[0], k_all, lay)
        ids = lay.ring.block_ids
        owned = ids >= 0
        assert torch.equal(index[0][:, owned], findex[0][:, ids[owned]]), "global routing of local rows"
        lists, counts = vsa_ring.partition(index, lay.routing_counts, lay, rt)
        want_l, want_c = vsa_oracle.partition_indices(index.cpu(), lay.routing_counts.cpu(), g2g.cpu(), size,
                                                      lay.blocks)
        assert torch.equal(lists.cpu(), want_l[:, 0]) and torch.equal(counts.cpu(), want_c[:, 0])
        slots = lay.padded_tokens
        out = torch.zeros((slots, heads, 128), dtype=torch.float32, device="cuda")
        lse = torch.full((heads, slots), float("-inf"), device="cuda")
        status = vsa_core.device_plan(lay).status
        strides = (lists.stride(1), counts.stride(1))
        # Two ways to the same running state: the ring step kernel that merges in its epilogue,
        # and the plain forward kernel followed by the separate merge kernel.
        out2, lse2 = out.clone(), lse.clone()
        for step in range(size):
            owner = (rank - step) % size
            k_o, v_o = shards[owner][0][1], shards[owner][0][2]
            _cabi.call("vsa_fine_fwd_running", p(q_s), p(k_o), p(v_o), lay.blocks, k_o.shape[0] // BLOCK, heads,
                       p(lists[owner]), p(counts[owner]), strides[0], strides[1], lists.shape[-1],
                       p(lay.ring.peer_block_sizes[owner]), scale, p(out), p(lse), p(status), _cabi.stream())
            part, part_lse = vsa_core._fine_fwd(q_s, k_o, v_o, lists[owner], counts[owner], strides,
                                                lay.ring.peer_block_sizes[owner], scale, status)
            _cabi.call("vsa_merge_partial", p(out2), p(lse2), p(part), p(part_lse), slots, heads, _cabi.stream())
        assert_close(out2, out, f"rank {rank} merge kernel vs merging epilogue", max_abs=1e-2, rel_l2=5e-3)
        assert torch.equal(torch.isfinite(lse2), torch.isfinite(lse))
        live = torch.isfinite(lse)
        torch.testing.assert_close(lse2[live], lse[live], atol=2e-3, rtol=1e-3)
        rows = (ids[owned, None] * BLOCK + torch.arange(BLOCK, device="cuda")).flatten()
        mine = torch.arange(int(owned.sum()) * BLOCK, device="cuda")
        assert_close(out[mine], fo[rows], f"rank {rank} fine out")
        torch.testing.assert_close(lse[:, mine], flse[:, rows], atol=2e-3, rtol=1e-3)
        delta = (do_s.float() * out).sum(-1).transpose(0, 1).contiguous()
        dq_acc = torch.zeros_like(out)
        words = _cabi.load().vsa_kv_mask_words(lay.blocks)
        mask = torch.empty(heads * lay.blocks * words, dtype=torch.int32, device="cuda")
        for step in range(size):
            owner = (rank - (size - 1 - step)) % size
            # Padding slots are never written by the FP32 epilogues: start from zeros.
            part = torch.zeros((2, slots, heads, 128), dtype=torch.float32, device="cuda")
            common = (q_s, shards[owner][0][1], shards[owner][0][2], do_s, lists[owner], counts[owner],
                      lay.block_sizes, lay.ring.peer_block_sizes[owner], scale, lse, delta, mask, status)
            vsa_ring._bwd_call(*common, parts=3, dq_f32=dq_acc, accumulate=1)
            vsa_ring._bwd_call(*common, parts=4, dk_f32=part[0], dv_f32=part[1], accumulate=0)
            dk_acc[owner] += part[0]
            dv_acc[owner] += part[1]
        assert_close(dq_acc[mine], fdq[rows], f"rank {rank} dq")
        assert int(status.item()) == 0
    for rank, lay in enumerate(locals_):
        ids = lay.ring.block_ids
        owned = ids >= 0
        rows = (ids[owned, None] * BLOCK + torch.arange(BLOCK, device="cuda")).flatten()
        mine = torch.arange(int(owned.sum()) * BLOCK, device="cuda")
        assert_close(dk_acc[rank][mine], fdk[rows], f"rank {rank} dk", peak_relative=True)
        assert_close(dv_acc[rank][mine], fdv[rows], f"rank {rank} dv", peak_relative=True)


def test_list_bounds_against_searchsorted():
    """Range starts of ascending lists: rows of different length (empty and full included), ranges
    without entries, a last range shorter than the others."""
    gen = torch.Generator().manual_seed(5)
    rows, capacity, blocks, chunk = 300, 90, 1000, 128
    passes = -(-blocks // chunk)
    counts = torch.randint(0, capacity + 1, (rows,), generator=gen, dtype=torch.int32)
    counts[0], counts[1] = 0, capacity
    lists = torch.zeros((rows, capacity), dtype=torch.int32)
    for r in range(rows):
        n = int(counts[r])
        lists[r, :n] = torch.randperm(blocks, generator=gen)[:n].sort().values.int()
    lists[2, :int(counts[2])] = torch.arange(int(counts[2]), dtype=torch.int32) + 3 * chunk  # one range only
    bounds = torch.full((rows, passes + 1), -1, dtype=torch.int32, device="cuda")
    p = _cabi.ptr
    lists_d, counts_d = lists.cuda(), counts.cuda()
    _cabi.call("vsa_list_bounds", p(lists_d), p(counts_d), rows, capacity, chunk, passes, p(bounds), _cabi.stream())
    want = torch.empty((rows, passes + 1), dtype=torch.int32)
    edges = torch.arange(passes, dtype=torch.int32) * chunk
    for r in range(rows):
        n = int(counts[r])
        want[r, :passes] = torch.searchsorted(lists[r, :n].contiguous(), edges)
        want[r, passes] = n
    assert torch.equal(bounds.cpu(), want)


def test_partial_merge_with_empty_steps():
    torch.manual_seed(61)
    slots, heads = 129 * 1, 2
    out = torch.zeros(slots, heads, 128, device="cuda")
    lse = torch.full((heads, slots), float("-inf"), device="cuda")
    parts, lses = [], []
    for step in range(8):
        part = torch.randn(slots, heads, 128, device="cuda").to(torch.bfloat16)
        part_lse = torch.randn(heads, slots, device="cuda") * 10
        part_lse[:, step::8] = float("-inf")
        part_lse[:, 0] = float("-inf")
        part.masked_fill_(~torch.isfinite(part_lse).transpose(0, 1).unsqueeze(-1), 0)
        parts.append(part.cpu())
        lses.append(part_lse.cpu())
        _cabi.call("vsa_merge_partial", _cabi.ptr(out), _cabi.ptr(lse), _cabi.ptr(part), _cabi.ptr(part_lse), slots,
                   heads, _cabi.stream())
    want, want_lse = vsa_oracle.merge_partials(parts, lses)
    torch.testing.assert_close(out.double().cpu(), want, atol=2e-6, rtol=2e-5)
    torch.testing.assert_close(lse.double().cpu(), want_lse, atol=2e-6, rtol=2e-6)


@pytest.mark.parametrize("chunk", [None, 16, 5])
def test_size_one_ring_group_matches_single_device(chunk, monkeypatch):
    """chunk: blocks per pass of a ring step (None = default, one pass here).  16 gives two KV
    passes and two query-block passes of one mask word each on the 33 blocks; 5 gives seven KV passes."""
    if chunk is not None:
        monkeypatch.setattr(vsa_ring, "RING_CHUNK_BLOCKS", chunk)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29581")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        heads = 2
        samples = GEOMETRIES["ragged"]
        full = build_vsa_layout(samples, head_num=heads, device="cuda", input_order="block")
        ring = build_vsa_layout(samples, head_num=heads, device="cuda", input_order="block",
                                ring_cp_group=dist.group.WORLD)
        data = [_slots(full, x.cuda()) for x in seeded(full.tokens, heads, 0, 4)]
        dy = _slots(full, seeded(full.tokens, heads, 1, 1)[0].cuda())
        results = []
        for layout in (full, ring):
            leaves = [x.detach().requires_grad_() for x in data]
            out = vsa_attention(*leaves, layout)
            results.append((out, *torch.autograd.grad(out, leaves, dy)))
            vsa_core.check_status(layout)
        for tag, a, b in zip(("out", "dq", "dk", "dv", "dgate"), results[1], results[0]):
            assert_close(a, b, f"size-one ring {tag}", peak_relative=tag in ("dk", "dv"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ring_over_nccl_matches_single_device():
    world = min(torch.cuda.device_count(), 4)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29617", str(ROOT / "tests" / "ring_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    log_dir = os.environ.get("VSA_TEST_LOG_DIR")
    if log_dir:  # keep the workers' PARITY lines as evidence of the run
        Path(log_dir, f"ring_worker_r{world}.log").write_text(done.stdout + done.stderr[-3000:])
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ulysses_over_nccl_matches_single_device():
    """Ulysses on two ranks, and Ring x Ulysses (U=2, R=2) when four GPUs are visible."""
    shapes = [(2, 1)] + ([(2, 2)] if torch.cuda.device_count() >= 4 else [])
    for ulysses_size, ring_size in shapes:
        world = ulysses_size * ring_size
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", "29633", str(ROOT / "tests" / "ulysses_worker.py"),
               "--ulysses", str(ulysses_size), "--ring", str(ring_size)]
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        done = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
        log_dir = os.environ.get("VSA_TEST_LOG_DIR")
        if log_dir:
            Path(log_dir, f"ulysses_worker_u{ulysses_size}r{ring_size}.log").write_text(done.stdout + done.stderr[-3000:])
        assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
