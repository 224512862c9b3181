"""Benchmark of the VSA hot path: forward + backward of one layer on synthetic inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

N = 1 runs the 720p packed sample (video 31x45x80 at sparsity 0.9 + two dense images, 2048 text
tokens each, 24 heads of 128) through ``vsa_attention`` on one B200.  N > 1 (launched by
torchrun, one rank per GPU) runs the ring configuration (video 61x90x160 at sparsity 0.95 +
4096 text tokens, 24 heads) with whole blocks sharded over the ranks; before it is timed, the
ring path is checked against the single-device path on the 720p sample (the reference gates
its benchmark cases the same way, ``benchmark/perf_vsa.py:129-141``).  A step is one forward and
one backward pass.  Rank 0 prints one JSON line:

``value``  useful attention TFLOP/s of the whole job (valid query-key pairs of the actual
           routing, 4*D per pair forward, backward = 2x forward, plus the coarse block GEMMs),
           inputs resident in HBM, mean over the K timed steps, max over ranks.
``phases`` medians of forward, backward and total per step from three events per step
           (one CUDA-graph replay per step on one GPU, eager launches on a ring).
``e2e``    the same metric through the public Python API with pinned HOST buffers: every step
           copies q, k, v, gate and dO to the device and the output and four gradients back
           (uploads of the next step and downloads of the previous one run on copy streams
           under the current step's kernels, as a prefetching loader would).
``roofline``      the slowest kernel of the step timed alone with CUDA events on its stream.
``breakdown_ms``  device time per C entry point over one extra step.
``parity``        (N > 1) the ring-versus-single-device check that gates the timing.
``cpu_baseline``  the CPU oracle timed on a bounded sample of the same workload (rank 0, N = 1).

``--impl reference`` times the CPU restatement of the reference's algorithm (``oracle/``) on the
host cores instead; the reference itself is Python on top of GPU-only libraries and cannot
travel to the benchmark box.  Each of its steps is a sample bounded by wall time.
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
    # name: (samples, heads, input order, stacked layers per step)
    "720p_packed_sample_h24": ([[S("video", (31, 45, 80), .9), S("text", 2048)],
                                [S("video", (1, 45, 80)), S("text", 2048)],
                                [S("video", (1, 45, 80)), S("text", 2048)]], 24, "raster", 1),
    "720p_single_sample_h12": ([[S("video", (31, 45, 80), .9), S("text", 2048)]], 12, "raster", 1),
    "720p_single_sample_h6": ([[S("video", (31, 45, 80), .9), S("text", 2048)]], 6, "raster", 1),
    "block_order_stack_h24_x8": ([[S("video", (21, 30, 52), .8), S("text", 512), S("audio", 1024)]] * 4,
                                 24, "block", 8),
    "ring_61x90x160_h24": ([[S("video", (61, 90, 160), .95), S("text", 4096)]], 24, "block", 1),
    "small_8x16x16_h2": ([[S("video", (8, 16, 16), .75), S("text", 256)]], 2, "raster", 1),
}
PARITY_SAMPLES = [[S("video", (31, 45, 80), .9), S("text", 2048)]]
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
    """Forward useful FLOPs from the routing actually used (device tensors, no dense mask);
    the reference's definition, ``benchmark/utils.py:32-75``."""
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
    if layout.ring is None:
        coarse = sum(4.0 * layout.head_num * DIM * g.blocks ** 2 for g in layout.groups if not g.dense_only)
    else:
        coarse = sum(4.0 * layout.head_num * DIM * (e - b) * g.blocks
                     for g, b, e, _ in layout.ring.local_groups if not g.dense_only)
    return {"fine_forward": fine, "coarse_forward": coarse, "pairs": pairs}


# ------------------------------------------------------------------------------ CPU arm
class CpuSample:
    """The CPU oracle on one head of a workload: slot gather and pooling of the whole head once
    (set-up, untimed), then timed passes over query blocks drawn in a fixed pseudo-random
    order: routing of those blocks' rows plus blockwise FP32 fine attention forward + backward.
    A pass stops at its wall-time budget, so its cost does not depend on the workload's size."""

    def __init__(self, samples, seed=0):
        from oracle import vsa_oracle
        self.oracle = vsa_oracle
        layout = build_vsa_layout(samples, head_num=1)
        gen = torch.Generator().manual_seed(seed)
        q, k, v, dy = (torch.randn(layout.tokens, 1, DIM, generator=gen).to(torch.bfloat16) for _ in range(4))
        self.layout = layout
        self.slots = [vsa_oracle.gather_rows(x, layout.slot_row).float() for x in (q, k, v)]
        self.dy = vsa_oracle.gather_rows(dy, layout.slot_row).float()
        self.means = None
        if not layout.dense_only:
            self.means = [vsa_oracle.block_means(x, layout.block_sizes)[layout.coarse_blocks]
                          for x in self.slots[:2]]
        self.order = torch.randperm(layout.blocks, generator=torch.Generator().manual_seed(seed + 1))

    def run(self, seconds, chunk=None):
        """One pass: returns (useful FLOPs done, seconds spent, query blocks done)."""
        layout, oracle = self.layout, self.oracle
        chunk = chunk or (16 if layout.blocks <= 4096 else 4)
        sizes = layout.block_sizes.double()
        offsets = torch.arange(BLOCK)
        done_blocks, pairs = 0, 0.0
        start = time.perf_counter()
        while done_blocks < layout.blocks and (done_blocks == 0 or time.perf_counter() - start < seconds):
            picked = self.order[done_blocks:done_blocks + chunk].sort().values
            index = (oracle.route(self.means[0], self.means[1], layout, query_blocks=picked)
                     if self.means is not None else layout.routing_indices[:, :, picked].contiguous())
            counts = layout.routing_counts[:, :, picked].contiguous()
            valid = torch.arange(index.shape[-1]) < counts[0][..., None]
            # The oracle runs on the KV blocks these lists name (compact copies, ids remapped), so
            # its gradient tensors have the size of what was touched, not of the whole head.
            needed = index[0][valid].unique().long()
            local = torch.searchsorted(needed, index[0].long().clamp_max(int(needed[-1]))).to(torch.int32)[None]
            kv_rows = (needed[:, None] * BLOCK + offsets[None, :]).reshape(-1)
            k_sub, v_sub = (x[kv_rows].clone().requires_grad_() for x in self.slots[1:])
            rows = (picked[:, None] * BLOCK + offsets[None, :]).reshape(-1)
            q_sub = self.slots[0][rows].clone().requires_grad_()
            out, _ = oracle.fine_attention(q_sub, k_sub, v_sub, local, counts, layout.block_sizes[needed],
                                           DIM ** -0.5)
            torch.autograd.grad(out, (q_sub, k_sub, v_sub), self.dy[rows])
            pairs += float(((sizes[index[0].long()] * valid).sum(-1) * sizes[picked][None, :]).sum())
            done_blocks += len(picked)
        return 3 * 4 * DIM * pairs, time.perf_counter() - start, done_blocks


def host_threads():
    """All host cores for the CPU arm (torchrun pins OMP_NUM_THREADS to 1 for its children)."""
    cores = max(1, min(os.cpu_count() or 1, 64))
    torch.set_num_threads(cores)
    return cores


def reference_arm(args, workload, rank):
    """The CPU restatement of the reference's algorithm, timed on the host cores.  A step is a
    pass bounded by wall time so that warm-up + steps end within a few minutes on any workload."""
    if rank != 0:
        return
    samples, heads, order, layers = WORKLOADS[workload]
    cores = host_threads()
    total_steps = max(1, args.warmup + args.steps)
    budget = max(1.0, min(8.0, 100.0 / total_steps))
    sample = CpuSample(samples)
    times, work, blocks = [], [], 0
    for i in range(total_steps):
        flops, seconds, blocks = sample.run(budget)
        if i >= args.warmup:
            times.append(seconds)
            work.append(flops)
    ms = 1e3 * sum(times) / len(times)
    value = sum(work) / sum(times) / 1e12
    layout = sample.layout
    text = (f"head 0 of {heads}: {blocks} of {layout.blocks} query blocks per step in a fixed random order "
            f"(about {budget:.1f} s): routing of their rows + blockwise fine forward+backward in FP32; "
            "slot gather and pooling of the head are set-up, untimed")
    print(json.dumps({
        "impl": "reference", "metric": "vsa_fwd_bwd_useful_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "tokens": layout.tokens, "heads": heads, "head_dim": DIM,
                   "input_order": order, "layers": layers},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": text},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------ GPU arm
def timed(fn, steps):
    """Average milliseconds of `fn` over `steps` calls, CUDA events on the current stream."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps


def kernel_rooflines(layout, leaves, scale, flops, peaks):
    """Times the three tensor-core kernels alone on this step's tensors."""
    from cudnn_vsa_b200 import _cabi, vsa_core
    plan = vsa_core.device_plan(layout)
    q, k, v = (x.detach() for x in leaves[:3])
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


def ring_parity(group, device, rank, world):
    """Ring path against the single-device path on the 720p sample (2 heads, block order): every
    rank runs both on identical seeded global inputs and compares output and the four gradients
    on the rows it owns.  Bounds: max-abs 2e-2 (dk / dv relative to the reference peak when that
    exceeds one) and relative L2 1e-2.  Returns the worst figures over tensors and ranks."""
    import torch.distributed as dist
    from cudnn_vsa_b200 import vsa_core
    from cudnn_vsa_b200.vsa import raster_to_block_wo_padding, vsa_attention
    heads = 2
    full = build_vsa_layout(PARITY_SAMPLES, head_num=heads, device=device, input_order="block")
    local = build_vsa_layout(PARITY_SAMPLES, head_num=heads, device=device, input_order="block",
                             ring_cp_group=group)
    gen = torch.Generator(device=device).manual_seed(0)
    raster = [torch.randn(full.tokens, heads, DIM, device=device, dtype=torch.bfloat16, generator=gen)
              for _ in range(5)]
    results = []
    for layout in (full, local):
        xs = [raster_to_block_wo_padding(x, vsa_layout=layout).detach().requires_grad_() for x in raster[:4]]
        out = vsa_attention(*xs, layout)
        grads = torch.autograd.grad(out, xs, raster_to_block_wo_padding(raster[4], vsa_layout=layout))
        vsa_core.check_status(layout)
        results.append((out, *grads))
    position = torch.empty(full.tokens, dtype=torch.int64, device=device)
    position[full.input_rows] = torch.arange(full.tokens, device=device)
    mine = position[local.input_rows]
    worst_abs = worst_rel = 0.0
    ok = True
    for tag, got, ref in zip(("out", "dq", "dk", "dv", "dgate"), results[1], results[0]):
        a, b = got.double(), ref[mine].double()
        err = (a - b).abs().max().item()
        rel = ((a - b).square().sum() / b.square().sum().clamp_min(1e-30)).sqrt().item()
        bound = 2e-2 * (max(1.0, b.abs().max().item()) if tag in ("dk", "dv") else 1.0)
        ok = ok and err <= bound and rel <= 1e-2
        worst_abs, worst_rel = max(worst_abs, err), max(worst_rel, rel)
    stats = torch.tensor([worst_abs, worst_rel, 0.0 if ok else 1.0], device=device, dtype=torch.float64)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX, group=group)
    return {"check": "ring vs single device on video 31x45x80@0.9 + text 2048, 2 heads, block order; "
                     "out, dq, dk, dv, dgate on each rank's rows",
            "max_abs": stats[0].item(), "rel_l2": stats[1].item(), "ok": stats[2].item() == 0.0}


def measure_phases(forward, leaves, dy, repeats, world, use_graph):
    """Medians of forward / backward / total from three events per step.  One GPU: the step is
    captured once in a CUDA graph and replayed (the reference's protocol,
    ``benchmark/utils.py:126-190``); a ring: eager launches, every observation reduced with MAX
    over the ranks before the median."""
    import torch.distributed as dist
    mode = "eager"
    graph = None
    if use_graph:
        try:
            events = [torch.cuda.Event(enable_timing=True, external=True) for _ in range(3)]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                xs = [x.detach().clone().requires_grad_() for x in leaves]
                g = dy.clone()
                for _ in range(2):
                    out = forward(xs)
                    torch.autograd.grad(out, xs, g)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                events[0].record()
                out = forward(xs)
                events[1].record()
                kept = torch.autograd.grad(out, xs, g)  # noqa: F841 (keeps the graph's outputs alive)
                events[2].record()
            mode = "cuda_graph"
        except Exception as exc:  # capture is an optimisation of the measurement, not of the product
            graph, mode = None, f"eager (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()
    if graph is None:
        events = [torch.cuda.Event(enable_timing=True) for _ in range(3)]

        def run():
            events[0].record()
            out = forward(leaves)
            events[1].record()
            torch.autograd.grad(out, leaves, dy)
            events[2].record()
    else:
        run = graph.replay
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    rows = []
    for _ in range(repeats):
        run()
        events[2].synchronize()
        rows.append([events[0].elapsed_time(events[1]), events[1].elapsed_time(events[2]),
                     events[0].elapsed_time(events[2])])
    if world > 1:
        t = torch.tensor(rows, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rows = t.cpu().tolist()
    med = [statistics.median(r[i] for r in rows) for i in range(3)]
    return {"fwd_ms": med[0], "bwd_ms": med[1], "total_ms": med[2], "mode": mode, "replays": repeats}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    parser.add_argument("--cpu-seconds", type=float, default=15.0,
                        help="wall-time budget of the CPU-baseline sample of the GPU arm")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--no-roofline", action="store_true")
    parser.add_argument("--no-phases", action="store_true")
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
    from cudnn_vsa_b200 import _cabi, vsa_core, vsa_ring
    from cudnn_vsa_b200.vsa import vsa_attention
    _cabi.load()  # fail loudly if the CUDA library was not built
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    parity = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
        parity = ring_parity(group, device, rank, world)
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"error": "ring parity check failed; nothing was timed", "parity": parity}))
            dist.destroy_process_group()
            sys.exit(1)
    samples, heads, order, layers = WORKLOADS[workload]
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

    def forward(xs):
        q, k, y, gate = xs
        for _ in range(layers):  # a stack shares one layout; v of a layer = the previous layer's output
            y = vsa_attention(q, k, y, gate, layout)
        return y

    def step():
        out = forward(leaves)
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

    # Useful FLOPs of this rank's queries from the routing table the step uses.
    q0, k0 = leaves[0].detach(), leaves[1].detach()
    index = vsa_ring.routing_table(q0, k0, layout) if world > 1 else vsa_core.routing_table(q0, k0, layout)
    flops = useful_flops(layout, index)
    total = torch.tensor([3 * layers * (flops["fine_forward"] + flops["coarse_forward"])], device=device,
                         dtype=torch.float64)
    if world > 1:
        dist.all_reduce(total)
    value = total.item() / (ms_per_step * 1e-3) / 1e12

    result = {
        "metric": "vsa_fwd_bwd_useful_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload, "tokens": tokens if world == 1 else layout.ring.global_tokens,
                   "heads": heads, "head_dim": DIM, "input_order": order, "layers": layers,
                   "ms_per_layer": ms_per_step / layers,
                   "useful_flops_per_step": total.item(), "l2": "inputs exceed L2 (no flush needed)",
                   "parallelism": "single" if world == 1 else f"ring{world}"},
        "gpu_launches": per_step_launches * args.steps,
        "clocks": clocks.summary(),
    }
    if parity is not None:
        result["parity"] = parity
    peaks = measured_peaks()
    if not args.no_phases:
        phases = measure_phases(forward, leaves, dy, min(max(args.steps, 5), 10 if world > 1 else 50), world,
                                use_graph=world == 1)
        phases["tflops_total"] = total.item() / (phases["total_ms"] * 1e-3) / 1e12
        result["phases"] = phases
    with _cabi.trace() as tr:
        step()
    spans = tr.summary()
    if rank == 0:
        result["breakdown_ms"] = {name: round(v["ms"], 3) for name, v in
                                  sorted(spans.items(), key=lambda kv: -kv[1]["ms"])}
    if rank == 0 and world == 1 and not args.no_roofline:
        kernels = kernel_rooflines(layout, leaves, scale, flops, peaks)
        name = max(kernels, key=lambda n: kernels[n]["ms"])
        top = kernels[name]
        # DRAM bytes per listed block pair from the ncu captures of the 6-head single sample
        # (the per-kernel summaries under profiles/: dram read + write over 2,623,488 pairs),
        # scaled to this workload by its number of listed pairs (traffic grows with the tiles).
        per_pair = {"fine_fwd_kernel": 1480.4, "fine_bwd_dq_kernel": 1533.0, "fine_bwd_dkv_kernel": 2199.3}
        listed = float(layout.routing_counts.sum().item())
        traffic = per_pair[name] * listed
        result["roofline"] = {"kernel": name, "bound": "tensor", "achieved": top["achieved"],
                              "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": top["frac"],
                              "traffic": traffic, "traffic_source": "ncu capture of the 6-head sample scaled by listed pairs",
                              "peak_source": f"{peaks['source']} burst BF16", "launch_ms": top["ms"],
                              "all": {n: {"ms": round(k["ms"], 3), "tflops": round(k["achieved"], 1)}
                                      for n, k in kernels.items()}}
    if not args.no_e2e:
        # Host buffers are pinned; the device side is a prefetching loader: two sets of input
        # buffers, uploads on a copy stream (the next step's inputs travel while this step
        # computes), downloads of the output and the gradients on another (they drain under
        # the next step).  The forward pass starts as soon as its four inputs are up (dO follows
        # under it) and the output goes down while the backward pass runs.  Every step's copies
        # and the final drain are inside the timed region.
        host_in = [x.detach().cpu().pin_memory() for x in (*leaves, dy)]
        host_out = [torch.empty_like(h).pin_memory() for h in host_in]
        dev_in = [[torch.empty_like(x) for x in (*leaves, dy)] for _ in range(2)]
        main_stream = torch.cuda.current_stream()
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        uploaded = [torch.cuda.Event() for _ in range(2)]
        uploaded_inputs = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]
        forward_done = torch.cuda.Event()
        inputs = len(leaves)

        def upload(step_no):
            buf = step_no & 1
            with torch.cuda.stream(up):
                if step_no >= 2:
                    up.wait_event(consumed[buf])  # the step that last used these buffers has finished
                for i, (d, h) in enumerate(zip(dev_in[buf], host_in)):
                    d.copy_(h, non_blocking=True)
                    if i + 1 == inputs:
                        uploaded_inputs[buf].record(up)
                uploaded[buf].record(up)

        def e2e_run(steps):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            upload(0)
            for step_no in range(steps):
                buf = step_no & 1
                if step_no + 1 < steps:
                    upload(step_no + 1)
                main_stream.wait_event(uploaded_inputs[buf])
                xs = [d.requires_grad_() for d in dev_in[buf][:inputs]]
                out = forward(xs)
                forward_done.record(main_stream)
                with torch.cuda.stream(down):
                    down.wait_event(forward_done)
                    out.record_stream(down)
                    host_out[0].copy_(out.detach(), non_blocking=True)
                main_stream.wait_event(uploaded[buf])
                grads = torch.autograd.grad(out, xs, dev_in[buf][inputs])
                consumed[buf].record(main_stream)
                for d in dev_in[buf]:
                    d.requires_grad_(False)
                down.wait_stream(main_stream)
                with torch.cuda.stream(down):
                    for h, r in zip(host_out[1:], grads):
                        r.record_stream(down)
                        h.copy_(r, non_blocking=True)
            main_stream.wait_stream(down)
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
        cores = host_threads()
        sample = CpuSample(samples)
        work, seconds, blocks = sample.run(args.cpu_seconds)
        result["cpu_baseline"] = {
            "value": work / seconds / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"head 0 of {heads}: {blocks} of {sample.layout.blocks} query blocks in a fixed random order: "
                      f"routing of their rows + blockwise fine forward+backward in FP32, {seconds:.1f} s; slot "
                      "gather and pooling of the head are set-up, untimed"}
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
