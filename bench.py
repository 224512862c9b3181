"""Benchmark of the VSA hot path: forward + backward of one layer on synthetic inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

N = 1 runs the 720p packed sample (video 31x45x80 at sparsity 0.9 + two dense images, 2048 text
tokens each, 24 heads of 128) through ``vsa_attention`` on one B200.  N > 1 (launched by
torchrun, one rank per GPU) runs the ring configuration (video 61x90x160 at sparsity 0.95 +
4096 text tokens, 24 heads) with whole blocks sharded over the ranks.  A step is one forward and
one backward pass.  Rank 0 prints one JSON line:

``value``  useful attention TFLOP/s of the whole job (valid query-key pairs of the actual
           routing, 4*D per pair forward, backward = 2x forward, plus the coarse block GEMMs),
           inputs resident in HBM.
``e2e``    the same metric through the public Python API with pinned HOST buffers: every step
           copies q, k, v, gate and dO to the device and the output and four gradients back
           (uploads of the next step and downloads of the previous one run on copy streams
           under the current step's kernels, as a prefetching loader would).
``roofline``      the slowest kernel of the step timed alone with CUDA events on its stream.
``cpu_baseline``  the CPU oracle timed on a bounded sample of the same workload (rank 0, N = 1).

``--impl reference`` times the CPU restatement of the reference's algorithm (``oracle/``) on the
host cores instead; the reference itself is Python on top of GPU-only libraries and cannot
travel to the benchmark box.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from cudnn_vsa_b200.vsa_layout import BLOCK, Segment, build_vsa_layout  # noqa: E402

S = Segment
WORKLOADS = {
    # name: (samples, heads, input order)
    "720p_packed_sample_h24": ([[S("video", (31, 45, 80), .9), S("text", 2048)],
                                [S("video", (1, 45, 80)), S("text", 2048)],
                                [S("video", (1, 45, 80)), S("text", 2048)]], 24, "raster"),
    "720p_single_sample_h12": ([[S("video", (31, 45, 80), .9), S("text", 2048)]], 12, "raster"),
    "720p_single_sample_h6": ([[S("video", (31, 45, 80), .9), S("text", 2048)]], 6, "raster"),
    "ring_61x90x160_h24": ([[S("video", (61, 90, 160), .95), S("text", 4096)]], 24, "block"),
    "small_8x16x16_h2": ([[S("video", (8, 16, 16), .75), S("text", 256)]], 2, "raster"),
}
DIM = 128


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"tflops": data["bf16_tflops"], "hbm": data["hbm_gbs"], "source": "measured"}
    return {"tflops": 1590.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            self.proc.wait()
            self.thread.join(timeout=2)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in self.rows),
                "sm_max_mhz": int(self.rows[0][1]), "reasons": reasons, "samples": len(self.rows)}


def useful_flops(layout, index):
    """Forward useful FLOPs from the routing actually used (device tensors, no dense mask)."""
    sizes = layout.block_sizes.double()
    counts = layout.routing_counts[0]
    valid = torch.arange(index.shape[-1], device=index.device) < counts[..., None]
    if layout.ring is None:
        kv_sizes = sizes
    else:  # lists hold global ids; sizes of all global blocks in global order
        flat = layout.ring.peer_block_sizes.double().flatten()
        capacity = layout.ring.peer_block_sizes.shape[1]
        g2g = layout.ring.global_to_gather
        kv_sizes = flat[(g2g // capacity) * capacity + g2g % capacity]
    picked = kv_sizes[index[0].long()] * valid
    pairs = float((picked.sum(-1) * sizes[None, :]).sum().item())
    fine = 4 * DIM * pairs
    coarse = 0.0
    groups = layout.groups if layout.ring is None else [g for g, *_ in layout.ring.local_groups]
    if layout.ring is None:
        coarse = sum(4.0 * layout.head_num * DIM * g.blocks ** 2 for g in groups if not g.dense_only)
    else:
        coarse = sum(4.0 * layout.head_num * DIM * (e - b) * g.blocks
                     for g, b, e, _ in layout.ring.local_groups if not g.dense_only)
    return {"fine_forward": fine, "coarse_forward": coarse, "pairs": pairs}


def cpu_sample(samples, heads_total, block_stride, seed=0):
    """One CPU-oracle pass over a bounded sample: head 0, every `block_stride`-th query block of
    the workload, fine attention forward + backward (routing by the oracle, FP32 math)."""
    from oracle import vsa_oracle
    layout = build_vsa_layout(samples, head_num=1)
    gen = torch.Generator().manual_seed(seed)
    q, k, v, dy = (torch.randn(layout.tokens, 1, DIM, generator=gen).to(torch.bfloat16) for _ in range(4))
    start = time.perf_counter()
    slots = [vsa_oracle.gather_rows(x, layout.slot_row) for x in (q, k, v)]
    index = layout.routing_indices
    if not layout.dense_only:
        means = [vsa_oracle.block_means(x, layout.block_sizes)[layout.coarse_blocks] for x in slots[:2]]
        index = vsa_oracle.route(means[0], means[1], layout)
    picked = torch.arange(0, layout.blocks, block_stride)
    rows = (picked[:, None] * BLOCK + torch.arange(BLOCK)[None, :]).reshape(-1)
    q_sub = slots[0][rows].float().requires_grad_()
    k_all, v_all = (x.float().requires_grad_() for x in slots[1:])
    sub_index = index[:, :, picked].contiguous()
    sub_counts = layout.routing_counts[:, :, picked].contiguous()
    out, _ = vsa_oracle.fine_attention(q_sub, k_all, v_all, sub_index, sub_counts, layout.block_sizes,
                                       DIM ** -0.5)
    dy_sub = vsa_oracle.gather_rows(dy, layout.slot_row)[rows].float()
    torch.autograd.grad(out, (q_sub, k_all, v_all), dy_sub)
    seconds = time.perf_counter() - start
    sizes = layout.block_sizes.double()
    valid = torch.arange(sub_index.shape[-1]) < sub_counts[0][..., None]
    pairs = float(((sizes[sub_index[0].long()] * valid).sum(-1) * sizes[picked][None, :]).sum())
    return 3 * 4 * DIM * pairs, seconds, len(picked)


def reference_arm(args, workload, rank):
    """The CPU restatement of the reference's algorithm, timed on the host cores."""
    if rank != 0:
        return
    samples, heads, _ = WORKLOADS[workload]
    threads = torch.get_num_threads()
    stride = args.cpu_block_stride
    times, flops = [], 0.0
    for i in range(args.warmup + args.steps):
        flops, seconds, blocks = cpu_sample(samples, heads, stride)
        if i >= args.warmup:
            times.append(seconds)
    ms = 1e3 * sum(times) / len(times)
    value = flops / (ms * 1e-3) / 1e12
    sample = (f"head 0 of {heads}, every {stride}th query block ({blocks} blocks) of {workload}: "
              "slots, pooling, routing, fine forward+backward in FP32")
    print(json.dumps({
        "impl": "reference", "metric": "vsa_fwd_bwd_useful_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "heads": heads, "head_dim": DIM},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def timed(fn, steps, stream=None):
    """Average milliseconds of `fn` over `steps` calls, CUDA events on the current stream."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps


def kernel_rooflines(layout, leaves, dy, scale, flops, peaks):
    """Times the three tensor-core kernels alone on this step's tensors."""
    from cudnn_vsa_b200 import _cabi, vsa_core
    plan = vsa_core.device_plan(layout)
    q, k, v, _ = (x.detach() for x in leaves)
    heads, blocks = layout.head_num, layout.blocks
    p = _cabi.ptr
    if layout.slots_are_input:
        slots = [q, k, v]
    else:
        slots = [torch.empty((blocks * BLOCK, heads, DIM), dtype=q.dtype, device=q.device) for _ in range(3)]
    mean = torch.empty((3, blocks, heads, DIM), dtype=torch.float32, device=q.device)
    _cabi.call("vsa_slots_pool", p(q), p(k), p(v), None if layout.slots_are_input else p(layout.slot_row),
               p(layout.block_sizes), *(None if layout.slots_are_input else p(s) for s in slots), p(mean),
               None, None, 0, blocks, heads, _cabi.stream())
    index = vsa_core.route(mean[0], mean[1], layout, plan)
    counts = layout.routing_counts
    strides = (index.stride(1), counts.stride(1))
    dy_slots = torch.randn_like(slots[0])
    holder = {}

    def fwd():
        holder["o"], holder["lse"] = vsa_core._fine_fwd(slots[0], slots[1], slots[2], index, counts, strides,
                                                        plan.sizes, scale, plan.status)
    fwd()
    delta = (dy_slots.float() * holder["o"].float()).sum(-1).transpose(0, 1).contiguous()
    words = _cabi.load().vsa_kv_mask_words(blocks)
    mask = torch.empty(heads * blocks * words, dtype=torch.int32, device=q.device)
    grads = [torch.empty_like(slots[0]) for _ in range(3)]

    def bwd(parts):
        _cabi.call("vsa_fine_bwd", p(slots[0]), p(slots[1]), p(slots[2]), p(dy_slots), blocks, blocks, heads,
                   p(index), p(counts), strides[0], strides[1], index.shape[-1], p(layout.block_sizes),
                   p(plan.sizes), scale, p(holder["lse"]), p(delta), p(mask), p(grads[0]), p(grads[1]),
                   p(grads[2]), blocks * BLOCK, blocks * BLOCK, None, None, None, None, None, 0, None, None,
                   None, None, None, 0, parts, p(plan.status), _cabi.stream(), launches=1)
    bwd(1)
    pairs_flops = flops["fine_forward"] / 4  # D * pairs
    kernels = {
        "fine_fwd_kernel": (fwd, 4 * pairs_flops),
        "fine_bwd_dq_kernel": (lambda: bwd(2), 6 * pairs_flops),
        "fine_bwd_dkv_kernel": (lambda: bwd(4), 8 * pairs_flops),
    }
    out = {}
    for name, (fn, work) in kernels.items():
        fn()
        ms = timed(fn, 3)
        achieved = work / (ms * 1e-3) / 1e12
        out[name] = {"ms": ms, "achieved": achieved, "frac": achieved / peaks["tflops"], "flops": work}
    return out


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default=None)
    parser.add_argument("--cpu-block-stride", type=int, default=48,
                        help="the CPU oracle runs every n-th query block of head 0")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--no-roofline", action="store_true")
    args = parser.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    workload = args.workload or ("720p_packed_sample_h24" if world == 1 else "ring_61x90x160_h24")
    if args.impl == "reference":
        reference_arm(args, workload, rank)
        return

    import torch.distributed as dist
    from cudnn_vsa_b200 import _cabi, vsa_core
    from cudnn_vsa_b200.vsa import raster_to_block_wo_padding, vsa_attention
    _cabi.load()  # fail loudly if the CUDA library was not built
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
    samples, heads, order = WORKLOADS[workload]
    layout = build_vsa_layout(samples, head_num=heads, device=device, input_order=order,
                              ring_cp_group=group if world > 1 else None)
    gen = torch.Generator(device=device).manual_seed(0)
    tokens = layout.tokens
    # Each rank draws its own shard of the synthetic stream (same distribution as a sharded global tensor).
    if world > 1:
        gen.manual_seed(rank)
    leaves = [torch.randn(tokens, heads, DIM, device=device, dtype=torch.bfloat16, generator=gen).requires_grad_()
              for _ in range(4)]
    dy = torch.randn(tokens, heads, DIM, device=device, dtype=torch.bfloat16,
                     generator=torch.Generator(device=device).manual_seed(1 + rank))
    scale = DIM ** -0.5

    def step():
        out = vsa_attention(*leaves, layout)
        return (out, *torch.autograd.grad(out, leaves, dy))

    _cabi.LAUNCHES = 0
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    vsa_core.check_status(layout)
    per_step_launches = _cabi.LAUNCHES // max(args.warmup, 1)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        barrier()
    elapsed = torch.tensor([start.elapsed_time(stop)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_per_step = elapsed.item() / args.steps
    vsa_core.check_status(layout)

    # Useful FLOPs of this rank's queries from the routing table it actually used.
    plan = vsa_core.device_plan(layout)
    index = layout.routing_indices
    if plan.spans:
        index = vsa_core.last_routing(layout)
    flops = useful_flops(layout, index)
    total = torch.tensor([3 * (flops["fine_forward"] + flops["coarse_forward"])], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(total)
    value = total.item() / (ms_per_step * 1e-3) / 1e12

    result = {
        "metric": "vsa_fwd_bwd_useful_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": workload, "tokens": tokens if world == 1 else layout.ring.global_tokens,
                   "heads": heads, "head_dim": DIM, "input_order": order,
                   "useful_flops_per_step": total.item(), "l2": "inputs exceed L2 (no flush needed)",
                   "parallelism": "single" if world == 1 else f"ring{world}"},
        "gpu_launches": per_step_launches * args.steps,
        "clocks": clocks.summary(),
    }
    peaks = measured_peaks()
    if rank == 0 and world == 1 and not args.no_roofline:
        kernels = kernel_rooflines(layout, leaves, dy, scale, flops, peaks)
        name = max(kernels, key=lambda n: kernels[n]["ms"])
        top = kernels[name]
        # DRAM bytes per listed block pair from the ncu captures of the 6-head single sample
        # (profiles/<kernel>_720p_single_sample_h6.md: dram read + write over 2,623,488 pairs),
        # scaled to this workload by its number of listed pairs (traffic grows with the tiles).
        per_pair = {"fine_fwd_kernel": 1515.8, "fine_bwd_dq_kernel": 1508.8, "fine_bwd_dkv_kernel": 2225.6}
        listed = float(layout.routing_counts.sum().item())
        traffic = per_pair[name] * listed
        result["roofline"] = {"kernel": name, "bound": "tensor", "achieved": top["achieved"],
                              "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": top["frac"],
                              "traffic": traffic, "peak_source": f"{peaks['source']} burst BF16",
                              "launch_ms": top["ms"],
                              "all": {n: {"ms": round(k["ms"], 3), "tflops": round(k["achieved"], 1)}
                                      for n, k in kernels.items()}}
    if not args.no_e2e:
        # Host buffers are pinned; the device side is a prefetching loader: two sets of input
        # buffers, uploads on a copy stream (the next step's inputs travel while this step
        # computes), downloads of the output and the four gradients on another (they drain under
        # the next step).  Every step's copies and the final drain are inside the timed region.
        host_in = [x.detach().cpu().pin_memory() for x in (*leaves, dy)]
        host_out = [torch.empty_like(h).pin_memory() for h in host_in]
        dev_in = [[torch.empty_like(x) for x in (*leaves, dy)] for _ in range(2)]
        main = torch.cuda.current_stream()
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        uploaded = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]

        def upload(step):
            buf = step & 1
            with torch.cuda.stream(up):
                if step >= 2:
                    up.wait_event(consumed[buf])  # the step that last used these buffers has finished
                for d, h in zip(dev_in[buf], host_in):
                    d.copy_(h, non_blocking=True)
                uploaded[buf].record(up)

        def e2e_run(steps):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            upload(0)
            for step in range(steps):
                buf = step & 1
                if step + 1 < steps:
                    upload(step + 1)
                main.wait_event(uploaded[buf])
                xs = [d.requires_grad_() for d in dev_in[buf][:4]]
                out = vsa_attention(*xs, layout)
                results = (out, *torch.autograd.grad(out, xs, dev_in[buf][4]))
                consumed[buf].record(main)
                for d in dev_in[buf]:
                    d.requires_grad_(False)
                down.wait_stream(main)
                with torch.cuda.stream(down):
                    for h, r in zip(host_out, results):
                        r.record_stream(down)
                        h.copy_(r, non_blocking=True)
            main.wait_stream(down)
            stop.record()
            torch.cuda.synchronize()
            return start.elapsed_time(stop) / steps
        e2e_run(2)
        barrier()
        e2e_steps = min(args.steps, 10)
        e2e_ms = torch.tensor([e2e_run(e2e_steps)], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
        nbytes = sum(h.numel() * h.element_size() for h in host_in)
        result["e2e"] = {"value": total.item() / (e2e_ms.item() * 1e-3) / 1e12, "unit": "TFLOP/s",
                         "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
                         "ms_per_step": e2e_ms.item(), "steps": e2e_steps}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        work, seconds, blocks = cpu_sample(samples, heads, args.cpu_block_stride)
        result["cpu_baseline"] = {
            "value": work / seconds / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"head 0 of {heads}, every {args.cpu_block_stride}th query block ({blocks} blocks): slots, "
                      f"pooling, routing, fine forward+backward in FP32, {seconds:.1f} s"}
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
