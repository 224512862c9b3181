"""One rank's ring step on a single GPU, without transport: timing and profiling of the ring path.

    python tests/ring_replay.py [--ring R] [--workload NAME] [--heads H] [--steps K] [--separate-merge]
                                [--chunk-blocks B]

Builds rank 0's shard of an R-rank ring layout from a backend-free process group and runs
``vsa_attention`` on it with the three collectives replaced by local stand-ins: a ring hop is a
device copy on the communication stream, the gathered pooled means are this rank's own means
repeated R times, the reduce-scatter keeps the local part.  Every kernel of the ring path runs
with the shapes, list lengths and launch counts rank 0 sees in a real R-rank job (including the
boundary reorder into the shard and its scatter adjoint), so per-kernel device times and ncu
captures are representative; the VALUES are not those of a real ring (every peer shard holds
this rank's data) and nothing here checks them - parity of the ring path is checked by
``tests/ring_worker.py`` on real NCCL ranks and by ``tests/test_gpu_ring.py``.  Prints one JSON
line with the step time and the device time per C entry point.

``--chunk-blocks`` sets the number of blocks one pass of a ring step covers (default: the
library's ``RING_CHUNK_BLOCKS``; a value above the shard size gives one pass per step).

``--separate-merge`` also runs, per forward step, the plain forward kernel followed by the
stand-alone partial-merge kernel (the unfused form of the same step), so that kernel can be
timed and captured too.
"""
import argparse
import json
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402
from cudnn_vsa_b200 import _cabi, vsa_core, vsa_ring  # noqa: E402
from cudnn_vsa_b200.vsa import raster_to_block_wo_padding, vsa_attention  # noqa: E402
from cudnn_vsa_b200.vsa_layout import BLOCK, build_vsa_layout  # noqa: E402


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--ring", type=int, default=2)
    parser.add_argument("--workload", default="ring_61x90x160_h24", choices=sorted(bench.WORKLOADS))
    parser.add_argument("--heads", type=int, default=None)
    parser.add_argument("--steps", type=int, default=2)
    parser.add_argument("--separate-merge", action="store_true")
    parser.add_argument("--chunk-blocks", type=int, default=None)
    args = parser.parse_args()
    if args.chunk_blocks:
        vsa_ring.RING_CHUNK_BLOCKS = args.chunk_blocks
    samples, heads, _, _ = bench.WORKLOADS[args.workload]
    heads = args.heads or heads
    ring = args.ring
    device = torch.device("cuda", 0)
    full = build_vsa_layout(samples, head_num=heads, device=device)
    layout = build_vsa_layout(samples, head_num=heads, device=device, input_order="block",
                              ring_cp_group=dist.ProcessGroup(0, ring))
    runtime = vsa_ring._RingRuntime(None, 0, ring, torch.cuda.Stream(priority=-1), False, tuple(range(ring)))

    def exchange(rt, pairs, *, reverse=False):
        rt.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(rt.stream):
            for send, receive in pairs:
                receive.copy_(send)

    def gather(k_mean, v_mean, rt, order):
        v_mean = v_mean.to(torch.bfloat16)
        return k_mean.repeat(ring, 1, 1).index_select(0, order), v_mean.repeat(ring, 1, 1).index_select(0, order)

    def scatter(dk, dv, rt, order, local_blocks):
        return dk.float()[:local_blocks].contiguous(), dv.float()[:local_blocks].contiguous()

    vsa_ring.ring_runtime = lambda lay, dev: runtime
    vsa_ring.ring_exchange, vsa_ring.gather_means, vsa_ring.scatter_pooled_grads = exchange, gather, scatter

    gen = torch.Generator(device=device).manual_seed(0)
    raster = [torch.randn(full.tokens, heads, 128, device=device, dtype=torch.bfloat16, generator=gen).requires_grad_()
              for _ in range(4)]
    dy = torch.randn(layout.tokens, heads, 128, device=device, dtype=torch.bfloat16, generator=gen)

    def step():
        local = [raster_to_block_wo_padding(x, vsa_layout=layout) for x in raster]
        out = vsa_attention(*local, layout)
        return torch.autograd.grad(out, raster, dy)

    def separate_merge():
        # The unfused form of the forward steps: plain kernel + stand-alone merge kernel.
        plan = vsa_core.device_plan(layout)
        slots = layout.blocks * BLOCK
        q_s = torch.randn(slots, heads, 128, device=device, dtype=torch.bfloat16, generator=gen)
        kv = torch.randn(2, slots, heads, 128, device=device, dtype=torch.bfloat16, generator=gen)
        index = layout.routing_indices
        lists, counts = vsa_ring.partition(index, layout.routing_counts, layout, runtime)
        out = torch.zeros((slots, heads, 128), dtype=torch.float32, device=device)
        lse = torch.full((heads, slots), float("-inf"), dtype=torch.float32, device=device)
        for owner in range(ring):
            part, part_lse = vsa_core._fine_fwd(q_s, kv[0], kv[1], lists[owner], counts[owner],
                                                (lists.stride(1), counts.stride(1)),
                                                layout.ring.peer_block_sizes[owner], 128 ** -0.5, plan.status)
            _cabi.call("vsa_merge_partial", _cabi.ptr(out), _cabi.ptr(lse), _cabi.ptr(part), _cabi.ptr(part_lse),
                       slots, heads, _cabi.stream())

    step()
    torch.cuda.synchronize()
    vsa_core.check_status(layout)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    with _cabi.trace() as tr:
        step()
        if args.separate_merge:
            separate_merge()
    spans = tr.summary()
    vsa_core.check_status(layout)
    print(json.dumps({"ring": ring, "workload": args.workload, "heads": heads, "local_blocks": layout.blocks,
                      "chunk_blocks": vsa_ring.RING_CHUNK_BLOCKS,
                      "global_tokens": full.tokens, "ms_per_step": start.elapsed_time(stop) / args.steps,
                      "entry_points_ms": {k: [round(v["ms"], 3), v["calls"]]
                                          for k, v in sorted(spans.items(), key=lambda kv: -kv[1]["ms"])}}))


if __name__ == "__main__":
    main()
