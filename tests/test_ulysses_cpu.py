"""CPU: the Ulysses exchanges on gloo ranks - which rows and heads land where, that the two
exchanges invert each other, their gradients, and the row bookkeeping with and without a ring."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cudnn_vsa_b200 import ulysses
from cudnn_vsa_b200.vsa_layout import build_vsa_layout
from tests.helpers import GEOMETRIES


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        group = dist.group.WORLD
        rows, heads, dim = 5, 2 * world, 3
        # Element (row r of rank k, head h, field n, d) carries its own coordinates.
        grid = torch.stack(torch.meshgrid(torch.arange(world * rows), torch.arange(heads), torch.arange(4),
                                          torch.arange(dim), indexing="ij"), dim=-1).float()
        stream = (grid * torch.tensor([1000., 100., 10., 1.])).sum(-1)            # [U*A, H, 4, D]
        mine = stream[rank * rows:(rank + 1) * rows].clone().requires_grad_()
        got = ulysses.exchange_heads(mine, group)
        per = heads // world
        assert got.shape == (world * rows, per, 4, dim)
        assert torch.equal(got, stream[:, rank * per:(rank + 1) * per])           # every row, my heads
        back = ulysses.exchange_tokens(got, group)
        assert torch.equal(back, mine)                                             # the exchanges invert each other
        # Gradient of a weighted sum of what this rank received: d/dx of sum(w_r * received_r)
        # puts rank s's weight on the head slice s of my rows.
        weight = float(rank + 1)
        (got * weight).sum().backward()
        want = torch.ones_like(mine)
        for s in range(world):
            want[:, s * per:(s + 1) * per] = float(s + 1)
        assert torch.equal(mine.grad, want)
        # Token exchange alone, with its gradient.
        out = stream[:, rank * per:(rank + 1) * per, 0].clone().requires_grad_()   # [U*A, H/U, D]
        home = ulysses.exchange_tokens(out, group)
        assert torch.equal(home, stream[rank * rows:(rank + 1) * rows, :, 0])
        (home * weight).sum().backward()
        want = torch.ones_like(out)
        for s in range(world):
            want[s * rows:(s + 1) * rows] = float(s + 1)
        assert torch.equal(out.grad, want)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_exchanges_route_rows_and_heads_and_are_adjoint(world):
    mp.spawn(_worker, args=(world, _free_port()), nprocs=world, join=True)


def test_plan_without_and_with_a_ring(metadata_group):
    samples = GEOMETRIES["ragged"]
    layout = build_vsa_layout(samples, head_num=2)
    plans = [ulysses.ulysses_plan(layout, 4, r) for r in range(4)]
    rows = -(-layout.tokens // 4)
    assert all(p.rows == rows and p.tokens == layout.tokens and p.tail == 4 * rows - layout.tokens for p in plans)
    assert [p.start for p in plans] == [0, rows, 2 * rows, 3 * rows]
    assert sum(int(p.valid.sum()) for p in plans) == layout.tokens
    stream = torch.arange(layout.tokens * 2).view(layout.tokens, 2)
    pieces = torch.cat([ulysses.local_slice(stream, p, fill=-1) for p in plans])
    assert torch.equal(pieces[:layout.tokens], stream) and (pieces[layout.tokens:] == -1).all()
    # With a ring every owner's stream has its own length; all ranks use the longest one.
    shards = [build_vsa_layout(samples, head_num=2, input_order="block", ring_cp_group=metadata_group(2, r))
              for r in range(2)]
    longest = max(s.tokens for s in shards)
    for shard in shards:
        plan = ulysses.ulysses_plan(shard, 2, 1)
        assert plan.rows == -(-longest // 2) and plan.tokens == shard.tokens and plan.start == plan.rows
    with pytest.raises(ValueError):
        ulysses.ulysses_plan(layout, 2, 2)
