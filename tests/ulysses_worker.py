"""torchrun worker: Ulysses (and Ring x Ulysses) VSA on U*R GPUs against the single-device result.

    torchrun --nnodes=1 --nproc-per-node U*R --master-addr 127.0.0.1 tests/ulysses_worker.py --ulysses U [--ring R]

Ranks r*U .. r*U+U-1 form Ulysses group r; ranks with the same position in their Ulysses group
form a ring (the grouping of the reference's demo, ``README.md:416-428``).  Every rank holds a
slice of the token stream with all H heads as one fused ``[A, H, 4, 128]`` tensor (q, k, v, gate),
runs ``ulysses_attention`` and compares its rows of the output and of the gradient of the fused
tensor with the single-device ``vsa_attention`` on all heads.  Prints PARITY lines.
"""
import argparse
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from cudnn_vsa_b200 import ulysses, vsa_core  # noqa: E402
from cudnn_vsa_b200.vsa import raster_to_block_wo_padding, vsa_attention  # noqa: E402
from cudnn_vsa_b200.vsa_layout import build_vsa_layout  # noqa: E402
from tests.helpers import GEOMETRIES, REPORT, assert_close  # noqa: E402


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--ulysses", type=int, default=2)
    parser.add_argument("--ring", type=int, default=1)
    parser.add_argument("--heads", type=int, default=4)
    parser.add_argument("geometries", nargs="*", default=["ragged", "mixed", "c1"])
    args = parser.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    U, R, H = args.ulysses, args.ring, args.heads
    assert world == U * R and H % U == 0
    device = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    ulysses_group = ring_group = None
    for r in range(R):
        group = dist.new_group(list(range(r * U, (r + 1) * U)))
        if rank // U == r:
            ulysses_group = group
    if R > 1:
        for u in range(U):
            group = dist.new_group([r * U + u for r in range(R)])
            if rank % U == u:
                ring_group = group
    for name in args.geometries:
        samples = GEOMETRIES[name]
        full = build_vsa_layout(samples, head_num=H, device=device)
        if R > 1 and full.blocks < R:
            continue
        layout = build_vsa_layout(samples, head_num=H // U, device=device,
                                  input_order="block" if R > 1 else "raster", ring_cp_group=ring_group)
        gen = torch.Generator(device=device).manual_seed(7)
        mixed = torch.randn(full.tokens, H, 4, 128, device=device, dtype=torch.bfloat16, generator=gen)
        dy = torch.randn(full.tokens, H, 128, device=device, dtype=torch.bfloat16, generator=gen)
        # Single device, all heads.
        ref_in = mixed.clone().requires_grad_()
        q, k, v, gate = (t.contiguous() for t in ref_in.unbind(2))
        ref_out = vsa_attention(q, k, v, gate, full)
        ref_grad, = torch.autograd.grad(ref_out, ref_in, dy)
        vsa_core.check_status(full)
        # Context parallel: this ring owner's stream, then this rank's slice of it.
        reorder = (lambda x: raster_to_block_wo_padding(x, vsa_layout=layout)) if R > 1 else (lambda x: x)
        plan = ulysses.ulysses_plan(layout, U, rank % U)
        local = ulysses.local_slice(reorder(mixed), plan).requires_grad_()
        out = ulysses.ulysses_attention(local, layout, plan, ulysses_group)
        grad, = torch.autograd.grad(out, local, ulysses.local_slice(reorder(dy), plan))
        vsa_core.check_status(layout)
        rows = layout.input_rows if R > 1 else torch.arange(full.tokens, device=device)
        mine = rows[plan.start:plan.start + plan.rows]            # global rows of my real rows
        real = mine.numel()
        assert not out[real:].count_nonzero(), "rows of the transport padding come back zero"
        for tag, a, b in (("out", out[:real], ref_out[mine]), ("d_mixed", grad[:real], ref_grad[mine])):
            exact = R == 1 and torch.equal(a, b)  # same kernels on the same heads: bit-identical without a ring
            if not exact:
                assert_close(a, b, f"U{U}R{R} {name} rank{rank} {tag}", peak_relative=tag == "d_mixed")
            line = "bit-identical" if exact else "max_abs=%.3e rel_l2=%.3e" % (REPORT[-1][1], REPORT[-1][3])
            print(f"PARITY ulysses U={U} R={R} {name} rank{rank} {tag}: {line}", flush=True)
        dist.barrier(device_ids=[device.index])
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
