"""torchrun worker: ring VSA on R GPUs against the single-device result on the same seeded data.

    torchrun --nnodes=1 --nproc-per-node R --master-addr 127.0.0.1 tests/ring_worker.py [geometry ...]

Every rank builds the full block-order layout and its own ring shard, runs both paths on
identical global inputs and compares output and all four gradients on the rows it owns - the ring
once with its default pass size and once with ring steps split into several passes over small KV
and query-block ranges (the form large shards run in).  Without
arguments the geometries are the 720p sample (video 31x45x80 at sparsity 0.9 + 2048 text tokens,
the slice the ring configuration is checked on) followed by the small ragged ones; heads = 2.
Every rank prints one ``PARITY`` line per tensor.
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from cudnn_vsa_b200 import vsa_core, vsa_ring  # noqa: E402
from cudnn_vsa_b200.vsa import raster_to_block_wo_padding, vsa_attention  # noqa: E402
from cudnn_vsa_b200.vsa_layout import build_vsa_layout  # noqa: E402
from tests.helpers import GEOMETRIES, REPORT, assert_close, seeded  # noqa: E402


def main():
    names = sys.argv[1:] or ["c2", "ragged", "mixed", "fine_only_peer", "partial_blocks", "c1", "dense"]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    device = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=device)
    heads = 2
    for name in names:
        for partition in ("cyclic", "contiguous"):
            samples = GEOMETRIES[name]
            full = build_vsa_layout(samples, head_num=heads, device=device, input_order="block")
            if full.blocks < world:
                continue
            local = build_vsa_layout(samples, head_num=heads, device=device, input_order="block",
                                     ring_cp_group=dist.group.WORLD, ring_partition=partition)
            raster = [x.to(device) for x in seeded(full.tokens, heads, 0, 4)]
            dy = seeded(full.tokens, heads, 1, 1)[0].to(device)
            # Pass sizes of the ring steps: the default (one pass at these sizes) and a small one,
            # 40 blocks for the 720p sample (more than one 32-block mask word per pass), else 3.
            default_chunk = vsa_ring.RING_CHUNK_BLOCKS
            small_chunk = 40 if local.blocks > 64 else 3
            results = []
            for layout, chunk in ((full, default_chunk), (local, default_chunk), (local, small_chunk)):
                vsa_ring.RING_CHUNK_BLOCKS = chunk
                leaves = [raster_to_block_wo_padding(x, vsa_layout=layout).detach().requires_grad_() for x in raster]
                out = vsa_attention(*leaves, layout)
                grads = torch.autograd.grad(out, leaves, raster_to_block_wo_padding(dy, vsa_layout=layout),
                                            allow_unused=True)
                vsa_core.check_status(layout)
                results.append((out, *grads))
            vsa_ring.RING_CHUNK_BLOCKS = default_chunk
            position = torch.empty(full.tokens, dtype=torch.int64, device=device)
            position[full.input_rows] = torch.arange(full.tokens, device=device)
            mine = position[local.input_rows]
            for form, ring_result in (("one pass", results[1]), (f"passes of {small_chunk}", results[2])):
                for tag, a, b in zip(("out", "dq", "dk", "dv", "dgate"), ring_result, results[0]):
                    if a is None and b is None:
                        continue
                    b = torch.zeros_like(results[0][0]) if b is None else b
                    a = torch.zeros_like(ring_result[0]) if a is None else a
                    assert_close(a, b[mine], f"{name}/{partition}/rank{rank}/{form} {tag}", max_abs=2e-2, rel_l2=1e-2,
                                 peak_relative=tag in ("dk", "dv"))
                    what, err, bound, rel, peak, _ = REPORT[-1]
                    print(f"PARITY ring{world} {what}: max_abs={err:.3e} bound={bound:.3e} rel_l2={rel:.3e} "
                          f"peak={peak:.3g}", flush=True)
            dist.barrier(device_ids=[device.index])
            if rank == 0:
                print(f"ring{world} {name} {partition}: ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
