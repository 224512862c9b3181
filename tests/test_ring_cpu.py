"""CPU: the ring path's host logic on two gloo ranks - shard rotation order, the reverse pass that
brings accumulated gradients home, the pooled-mean gather and its reduce-scatter adjoint."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cudnn_vsa_b200 import vsa_ring
from cudnn_vsa_b200.vsa_layout import build_vsa_layout
from tests.helpers import GEOMETRIES


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, name, partition, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        layout = build_vsa_layout(GEOMETRIES[name], head_num=2, input_order="block",
                                  ring_cp_group=dist.group.WORLD, ring_partition=partition)
        rt = vsa_ring.ring_runtime(layout, "cpu")
        assert rt.stream is None and rt.size == world and rt.rank == rank
        ring, blocks = layout.ring, layout.blocks
        ids = ring.block_ids
        # 1. gather_means returns every block's mean in global order, bit for bit.
        marks = ids.clamp_min(0).float()[:, None, None].expand(blocks, 2, 128) + 0.25
        k_local = marks.masked_fill((ids < 0)[:, None, None], 0).contiguous()
        v_local = (k_local * 2).contiguous()
        k_all, v_all = vsa_ring.gather_means(k_local, v_local, rt, ring.global_to_gather)
        total = ring.global_to_gather.numel()
        want = torch.arange(total).float()[:, None, None].expand(total, 2, 128) + 0.25
        assert k_all.dtype == torch.float32 and torch.equal(k_all, want)
        assert v_all.dtype == torch.bfloat16 and torch.equal(v_all, (want * 2).to(torch.bfloat16))
        # 2. the adjoint sums over ranks and keeps the local blocks.
        dk = torch.full((total, 2, 128), float(rank + 1))
        dk_local, dv_local = vsa_ring.scatter_pooled_grads(dk, dk * 10, rt, ring.global_to_gather, blocks)
        owned = (ids >= 0)[:, None, None]
        assert torch.equal(dk_local, torch.full_like(dk_local, sum(range(1, world + 1))) * owned)
        assert torch.equal(dv_local, dk_local * 10)
        # 3. forward rotation: step s holds the shard of owner (rank - s) % world.
        shard = torch.full((4,), float(rank))
        buffers, seen = [shard, torch.empty_like(shard)], []
        for step in range(world):
            current = buffers[step % 2]
            if step + 1 < world:
                vsa_ring.ring_exchange(rt, [(current, buffers[(step + 1) % 2])])
            seen.append(int(current[0]))
            vsa_ring.join_exchange(rt)
        assert seen == [(rank - s) % world for s in range(world)]
        # 4. reverse rotation from the last shard: gradients travel with the shard and end at home.
        kv = buffers[(world - 1) % 2].clone()
        buffers = [kv, torch.empty_like(kv)]
        accumulated, incoming = None, torch.empty(4)
        for step in range(world):
            owner = (rank - (world - 1 - step)) % world
            current = buffers[step % 2]
            assert int(current[0]) == owner
            pairs = [(current, buffers[(step + 1) % 2])] if step + 1 < world else []
            if step:
                pairs.append((accumulated, incoming))
            if pairs:
                vsa_ring.ring_exchange(rt, pairs, reverse=True)
            part = torch.full((4,), 10.0 ** rank)   # this rank's contribution to the shard it holds
            vsa_ring.join_exchange(rt)
            accumulated = part + incoming if step else part
        assert torch.equal(accumulated, torch.full((4,), float(sum(10.0 ** r for r in range(world)))))
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("partition", ["cyclic", "contiguous"])
def test_ring_host_logic_on_gloo_ranks(world, partition):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), "ragged", partition, results), nprocs=world, join=True)
    assert dict(results) == {r: "ok" for r in range(world)}


def test_ring_coarse_plan_streams(metadata_group):
    from cudnn_vsa_b200 import vsa_core
    for rank in range(3):
        layout = build_vsa_layout(GEOMETRIES["ragged"], head_num=2, input_order="block",
                                  ring_cp_group=metadata_group(3, rank))
        coarse = vsa_core.device_plan(layout).coarse
        used = coarse.block_q >= 0
        assert torch.equal(coarse.q_src[coarse.block_q[used].long()], used.nonzero().flatten())
        assert (coarse.q_src >= 0).sum() == used.sum() == layout.coarse_blocks.numel()
        assert (coarse.kv_src >= 0).sum() == layout.coarse_kv_blocks.numel()
        assert torch.equal(coarse.kv_src[coarse.kv_src >= 0], layout.coarse_kv_blocks)
        assert coarse.q_rows % 64 == 0 and coarse.kv_rows % 64 == 0
        assert int(coarse.kv_sizes.sum()) == layout.coarse_kv_blocks.numel()


def test_pass_counts_for_the_benchmark_shards():
    """Blocks per pass: a range up to one and a half pass sizes runs in one pass; the ring
    configuration's shards (1848 / 3696 / 7392 blocks at 8 / 4 / 2 ranks) and the whole geometry
    (14784) run in 1 / 2 / 4 / 7 passes; every pass fits the pass size plus its rounding."""
    assert vsa_ring.RING_CHUNK_BLOCKS == 2048
    for blocks, want in ((1, 1), (1848, 1), (3000, 1), (3072, 2), (3696, 2), (7392, 4), (14784, 7)):
        passes, per = vsa_ring._passes(blocks)
        assert passes == want and (passes - 1) * per < blocks <= passes * per
        assert per <= 1.5 * vsa_ring.RING_CHUNK_BLOCKS
