"""Parity, forward/backward timing and useful-FLOP MFU of ``vsa_attention`` with the command line
and the ``vsa-perf/v5`` result file of the reference's ``python -m benchmark.perf_vsa``
(reference ``benchmark/perf_vsa.py:35-213``, ``benchmark/utils.py``, ``benchmark/inputs.py``), run
over this repository's kernels:

    python -m tests.perf_vsa [--cases default single64k ...] [--heads 2 4] [--check-only] ...
    torchrun --nproc-per-node R -m tests.perf_vsa --ring [--cases ragged single64k thd64k] ...

Per case and head count: build the full and the local (raster / block / ring-shard) layouts,
draw seeded inputs (q, k, v, gate, dy from one device generator, in that order), convert them once
at the boundary, check output and the four gradients against a reference - the FP32 oracle for
packs of at most 4096 tokens, the single-device path above that and for ring shards, as the
reference does - with the reference's pass rule (cosine and 2ab/(a^2+b^2) similarity at least
1 - eps for every tensor, all ranks), check a second backward pass through the retained graph,
capture forward + backward in one CUDA graph (checked against eager with changed inputs), time
the replays with three events inside the graph and report medians, useful TFLOP/s and MFU.
The workload names and geometries are the reference's, so result files compare case by case.
It lives under ``tests/`` because the small-case reference is the oracle, which only tests may use.
"""
import argparse
import hashlib
import json
import math
import os
import statistics
import subprocess
import sys
from datetime import timedelta
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from cudnn_vsa_b200 import _cabi, vsa_core, vsa_ring  # noqa: E402
from cudnn_vsa_b200.vsa import raster_to_block_wo_padding, vsa_attention  # noqa: E402
from cudnn_vsa_b200.vsa_layout import Segment, build_vsa_layout  # noqa: E402
from oracle import vsa_oracle  # noqa: E402

HEAD_DIM = 128
TENSORS = ("out", "dq", "dk", "dv", "dgate")


def default_geometry():
    """The 720p 5 s pack of the reference's default case: 24 fps x 5 s + 1 frames, 4x temporal and
    16x spatial compression (a 31 x 45 x 80 video at sparsity 0.9), two dense images of one frame,
    2048 text tokens each."""
    height, width = math.ceil(720 / 16), math.ceil(1280 / 16)
    frames = (24 * 5 + 1 - 1) // 4 + 1
    return [[Segment("video", (frames, height, width), 0.9), Segment("text", 2048)]] + [
        [Segment("video", (1, height, width)), Segment("text", 2048)] for _ in range(2)]


def _v(size, sparsity=None):
    return Segment("video", size, sparsity)


CASES = {
    "single64k": [[_v((16, 60, 64), .9), Segment("text", 4096)]],
    "thd64k": [[_v((12, 48, 64), .9), Segment("text", 2048)], [_v((8, 40, 64), .9), Segment("text", 2048)],
               [_v((1, 32, 64)), Segment("text", 2048)]],
    "thd720p44s": [[_v((265, 45, 80), .9), Segment("text", 2048)], [_v((1, 45, 80)), Segment("text", 2048)]],
    "ragged": [[_v((5, 9, 11), .7), Segment("text", 67)], [Segment("text", 3), _v((1, 3, 5))],
               [_v((4, 8, 12), .5), _v((5, 4, 7), .9), Segment("audio", 17), Segment("text", 0)]],
    "partial_blocks": [[_v((1, 3, 5), .9), Segment("text", 7)]],
    "fine_only_peer": [[_v((1, 2, 3), .5)], [_v((1, 2, 3))]],
    "dense": [[_v((1, 9, 11)), Segment("text", 67)], [_v((1, 3, 5)), Segment("text", 3)]],
}


def case_geometry(name):
    return default_geometry() if name == "default" else CASES[name]


def bucket_argument(value):
    if value in ("auto", "backend"):
        return None if value == "backend" else value
    try:
        number = int(value)
    except ValueError as error:
        raise argparse.ArgumentTypeError("Expected auto, backend, or a positive integer") from error
    if number < 1:
        raise argparse.ArgumentTypeError("Bucket size must be positive")
    return number


def default_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    return json.loads(path.read_text())["bf16_tflops"] if path.exists() else 2250.0


def parse_args(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--ring", action="store_true", help="Run under torchrun with explicit NCCL groups")
    parser.add_argument("--cases", nargs="+", choices=("default", *CASES))
    parser.add_argument("--heads", nargs="+", type=int)
    parser.add_argument("--input-order", choices=("raster", "block"))
    parser.add_argument("--seed", type=int, help="Input seed; default 937 for Ring, 2026 for ordinary VSA")
    parser.add_argument("--dense-query-full", action="store_true")
    parser.add_argument("--eps", type=float, default=1e-5)
    parser.add_argument("--warmup", type=int)
    parser.add_argument("--repeats", type=int)
    parser.add_argument("--peak-tflops", type=float, default=default_peak(),
                        help="Dense BF16 peak per GPU; default: the measured B200 figure, else 2250")
    parser.add_argument("--check-only", action="store_true")
    parser.add_argument("--eager", action="store_true", help="Time eager execution instead of CUDA Graph")
    parser.add_argument("--profile", action=argparse.BooleanOptionalAction, default=None)
    parser.add_argument("--output", type=Path, default=Path("benchmark/results/perf_vsa"),
                        help="JSON file or output directory")
    transport = parser.add_mutually_exclusive_group()
    transport.add_argument("--batch-p2p", action="store_true", default=None)
    transport.add_argument("--unbatched-p2p", dest="batch_p2p", action="store_false")
    parser.add_argument("--eager-group", action="store_true", help="Bind device_id when creating WORLD")
    parser.add_argument("--bwd-bucket-size", type=bucket_argument, default="auto",
                        help="auto (default), backend, or a positive number of query blocks")
    parser.add_argument("--ring-size", type=int, help="Interleaved subgroup size; must divide world size")
    parser.add_argument("--ring-partition", choices=("cyclic", "contiguous"), default="cyclic")
    args = parser.parse_args(argv)
    if not args.ring and (args.ring_size is not None or args.eager_group or args.batch_p2p is not None
                          or args.bwd_bucket_size != "auto" or args.ring_partition != "cyclic"):
        parser.error("Ring transport options require --ring")
    args.cases = args.cases or (["ragged", "single64k", "thd64k"] if args.ring else ["default"])
    args.heads = args.heads or ([2] if args.ring else [2, 4])
    args.seed = (937 if args.ring else 2026) if args.seed is None else args.seed
    if min(args.heads) < 1:
        parser.error("Head counts must be positive")
    args.input_order = args.input_order or ("block" if args.ring else "raster")
    if args.ring and args.input_order != "block":
        parser.error("--ring requires --input-order block")
    if args.ring_size is not None and args.ring_size < 1:
        parser.error("--ring-size must be positive")
    args.warmup = (3 if args.ring else 5) if args.warmup is None else args.warmup
    args.repeats = (30 if args.ring else 80) if args.repeats is None else args.repeats
    if min(args.warmup, args.repeats, args.peak_tflops) <= 0 or not 0 < args.eps < 1:
        parser.error("Warmup, repeats and peak must be positive; eps must be in (0, 1)")
    args.profile = (not args.ring) if args.profile is None else args.profile
    if args.output.suffix != ".json":
        args.output = args.output / "perf.json"
    return args


def init_ring(args):
    """Ordinary-priority NCCL groups shared by forward and backward; ``--ring-size`` splits WORLD
    into interleaved subgroups (reference ``benchmark/perf_vsa.py:88-109``)."""
    options = {"device_id": torch.device("cuda", int(os.environ["LOCAL_RANK"]))} if args.eager_group else {}
    dist.init_process_group("nccl", timeout=timedelta(minutes=15), **options)
    group = dist.group.WORLD
    rank, world = dist.get_rank(), dist.get_world_size()
    if args.ring_size is not None:
        if world % args.ring_size:
            raise ValueError("--ring-size must be positive and divide world size")
        count = world // args.ring_size
        for index in range(count):
            ranks = list(range(index, world, count))
            candidate = dist.new_group(ranks=ranks, backend="nccl", **options)
            if rank in ranks:
                group = candidate
                args.output = args.output.with_stem(f"{args.output.stem}-group{index}")
    return group


def barrier(group):
    if group is not None:
        dist.barrier(group=group, device_ids=[torch.cuda.current_device()])


def make_inputs(samples, heads, seed):
    tokens = sum(seg.tokens for sample in samples for seg in sample)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    xs = [torch.randn(tokens, heads, HEAD_DIM, device="cuda", dtype=torch.bfloat16, generator=gen) for _ in range(5)]
    return tuple(x.requires_grad_() for x in xs[:4]), xs[4]


def backward(out, leaves, dy, retain_graph=False):
    grads = torch.autograd.grad(out, leaves, dy, allow_unused=True, retain_graph=retain_graph)
    return tuple(torch.zeros_like(x) if g is None else g for x, g in zip(leaves, grads))


def forward_backward(fn, leaves, dy, events=None, retain_graph=False):
    if events:
        events[0].record()
    out = fn(*leaves)
    if events:
        events[1].record()
    grads = backward(out, leaves, dy, retain_graph)
    if events:
        events[2].record()
    return (out, *grads)


def oracle_reference(layout_cpu):
    """FP32 oracle of the whole path for small packs (the reference uses its token-level CPU
    math here, ``tests/reference.py:141-177``)."""
    def run(q, k, v, gate):
        xs = [x.detach().float().cpu().requires_grad_() for x in (q, k, v, gate)]
        out, _ = vsa_oracle.vsa_attention(*xs, layout_cpu)
        run.leaves = xs
        return out
    return run


def check_tensors(actual, expected, eps, group, label):
    metrics = {name: vsa_oracle.similarity(a.float().cpu(), b.float().cpu())
               for name, a, b in zip(TENSORS, actual, expected)}
    passed = all(min(m["cosine"], m["tensor_similarity"]) >= 1 - eps for m in metrics.values())
    check = {"passed": passed, "metrics": metrics}
    if group is not None:
        ranks = [None] * dist.get_world_size(group)
        dist.all_gather_object(ranks, check, group=group)
        check = {**check, "passed": all(c["passed"] for c in ranks), "ranks": ranks}
    if not check["passed"]:
        raise AssertionError(f"{label}: {check}")
    return check


def geometry_and_flops(layout, samples, index):
    """Valid routed pairs and coarse block GEMMs per sample, no padding pairs
    (reference ``benchmark/utils.py:32-75``)."""
    heads, sizes = layout.head_num, layout.block_sizes.double()
    records = []
    for i, g in enumerate(layout.groups):
        rows = index[0, :, g.start:g.end]
        count = layout.routing_counts[0, :, g.start:g.end]
        valid = torch.arange(rows.shape[-1], device=rows.device) < count[..., None]
        pairs = int(((sizes[rows.long()] * valid).sum(-1) * sizes[g.start:g.end]).sum().item())
        fine = 4 * HEAD_DIM * pairs
        coarse_blocks = 0 if g.dense_only else g.blocks
        coarse = 4 * heads * HEAD_DIM * coarse_blocks ** 2
        routing = 2 * heads * HEAD_DIM * g.blocks * sum(e - s for s, e, keep in g.video_spans if keep < e - s)
        length = layout.sample_lengths[i]
        flops = {"forward": fine + coarse, "backward": 2 * (fine + coarse), "total": 3 * (fine + coarse),
                 "fine_forward": fine, "coarse_forward": coarse, "routing_forward": routing,
                 "valid_pairs_all_heads": pairs, "dense_pairs_all_heads": heads * length ** 2,
                 "selected_block_pairs_all_heads": int(count.sum().item())}
        records.append({"sample": i, "backend": "vsa_b200", "mode": "dense" if g.dense_only else "vsa",
                        "tokens": length, "blocks": g.blocks, "coarse_blocks": coarse_blocks,
                        "padded_tokens": g.blocks * 64, "flops": flops,
                        "segments": [{"kind": s.kind, "size": s.size, "sparsity": s.sparsity} for s in samples[i]]})
    totals = {key: sum(r["flops"][key] for r in records) for key in records[0]["flops"]}
    return records, totals


def capture_graph(fn, leaves, dy, warmup, eps, group):
    """Capture forward + backward on private buffers and check replay against eager, also after
    the inputs have been overwritten (reference ``benchmark/utils.py:126-166``)."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    events = [torch.cuda.Event(enable_timing=True, external=True) for _ in range(3)]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        leaves = tuple(x.detach().clone().requires_grad_() for x in leaves)
        dy = dy.clone()
        for _ in range(warmup):
            forward_backward(fn, leaves, dy)
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    barrier(group)
    with torch.cuda.graph(graph, stream=stream):
        actual = forward_backward(fn, leaves, dy, events)
    torch.cuda.current_stream().wait_stream(stream)
    saved = [x.detach().clone() for x in (*leaves, dy)]
    checks = []
    try:
        for changed in (False, True):
            if changed:
                with torch.no_grad():
                    for x in (*leaves, dy):
                        x.normal_()
            expected = forward_backward(fn, leaves, dy)
            graph.replay()
            torch.cuda.synchronize()
            checks.append({"changed_inputs": changed,
                           **check_tensors(actual, expected, eps, group, f"graph changed={changed}")})
    finally:
        with torch.no_grad():
            for x, original in zip((*leaves, dy), saved):
                x.copy_(original)
    graph.replay()
    torch.cuda.synchronize()
    return graph, events, leaves, dy, checks


def measure(replay, events, warmup, repeats, group):
    for _ in range(warmup):
        replay()
    torch.cuda.synchronize()
    barrier(group)
    rows = []
    for _ in range(repeats):
        replay()
        events[2].synchronize()
        rows.append([events[0].elapsed_time(events[1]), events[1].elapsed_time(events[2]),
                     events[0].elapsed_time(events[2])])
    if group is not None:  # reduce each observation over the ranks before taking medians
        t = torch.tensor(rows, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        rows = t.cpu().tolist()
    return [dict(zip(("forward", "backward", "total"), row)) for row in rows]


def summarize(samples, flops, peak, world):
    out = {}
    for phase in ("forward", "backward", "total"):
        ms = statistics.median(row[phase] for row in samples)
        tflops = flops[phase] / ms / 1e9 / world
        out[phase] = {"median_ms": ms, "tflops": tflops, "mfu_percent": 100 * tflops / peak}
    return out


def run_case(name, heads, args, group):
    rank, size = (dist.get_rank(group), dist.get_world_size(group)) if group is not None else (0, 1)
    samples = case_geometry(name)
    kwargs = dict(head_num=heads, device="cuda", dense_query_full=args.dense_query_full)
    full = build_vsa_layout(samples, **kwargs)
    if group is not None:
        local = build_vsa_layout(samples, **kwargs, ring_cp_group=group, input_order=args.input_order,
                                 ring_cp_batch_p2p=args.batch_p2p, ring_cp_bwd_bucket_size=args.bwd_bucket_size,
                                 ring_partition=args.ring_partition)
    else:
        local = full if args.input_order == "raster" else build_vsa_layout(samples, **kwargs, input_order="block")
    global_xs, global_dy = make_inputs(samples, heads, args.seed)
    if name == "fine_only_peer":
        with torch.no_grad():
            global_xs[3][full.sample_slices[1][0]] = float("nan")  # gate of a fine-only sample is never read
    convert = ((lambda x: raster_to_block_wo_padding(x, vsa_layout=local)) if local.input_order == "block"
               else (lambda x: x))
    xs = tuple(convert(x.detach()).requires_grad_() for x in global_xs)
    dy = convert(global_dy)
    fn = lambda q, k, v, gate: vsa_attention(q, k, v, gate, local)  # noqa: E731
    small = full.tokens <= 4096
    if small:
        cpu_layout = build_vsa_layout(samples, head_num=heads, dense_query_full=args.dense_query_full)
        ref = oracle_reference(cpu_layout)
        out = ref(*global_xs)
        grads = torch.autograd.grad(out, ref.leaves, global_dy.float().cpu(), allow_unused=True)
        reference = (out, *(torch.zeros_like(out) if g is None else g.nan_to_num() for g in grads))
    else:
        reference = forward_backward(lambda q, k, v, gate: vsa_attention(q, k, v, gate, full), global_xs, global_dy)
    rows = local.input_rows.cpu() if small else local.input_rows
    expected = tuple(x[rows] for x in reference)
    actual = forward_backward(fn, xs, dy, retain_graph=True)
    vsa_core.check_status(local)
    parity = check_tensors(actual, expected, args.eps, group, name)
    repeated = (actual[0], *backward(actual[0], xs, dy))
    retained = check_tensors(repeated, actual, args.eps, group, f"{name} retained backward")
    index = vsa_core.routing_table(global_xs[0].detach(), global_xs[1].detach(), full)
    geometry, flops = geometry_and_flops(full, samples, index)
    record = {"tokens": full.tokens, "heads": heads, "ring_size": size, "input_order": args.input_order,
              "dense_query_full": args.dense_query_full, "threshold": 1 - args.eps,
              "reference": "fp32_oracle" if small else "single_device_vsa",
              "parity": parity, "retained_backward_parity": retained, "sample_geometry": geometry, "flops": flops}
    if group is not None:
        record["ring_partition"] = local.ring.partition
    del global_xs, global_dy, expected, actual, repeated, reference
    if rank == 0:
        print(f"PARITY {name} H={heads} ring={size} input={args.input_order} PASS", flush=True)
    if args.check_only:
        return record
    if args.eager:
        events = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        replay = lambda: forward_backward(fn, xs, dy, events)  # noqa: E731
    else:
        graph, events, _, _, record["graph_parity"] = capture_graph(fn, xs, dy, args.warmup, args.eps, group)
        replay = graph.replay
    record["mode"] = "eager" if args.eager else "cuda_graph"
    record["timing_samples_ms"] = measure(replay, events, args.warmup, args.repeats, group)
    record["timing"] = summarize(record["timing_samples_ms"], flops, args.peak_tflops, size)
    if args.profile:
        trace = args.output.with_name(f"{args.output.stem}-{name}-h{heads}-rank{rank}.trace.json")
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU,
                                                torch.profiler.ProfilerActivity.CUDA]) as prof:
            barrier(group)
            torch.cuda.synchronize()
            replay()
            torch.cuda.synchronize()
        prof.export_chrome_trace(str(trace))
        record["trace"] = trace.name
    if rank == 0:
        print(json.dumps({"case": name, "heads": heads, "mode": record["mode"], "timing": record["timing"]}),
              flush=True)
    return record


def environment():
    props = torch.cuda.get_device_properties(torch.cuda.current_device())
    try:
        smi = subprocess.check_output(["nvidia-smi", "--query-gpu=name,driver_version,clocks.sm,clocks.mem,power.limit",
                                       "--format=csv"], text=True).strip()
    except (OSError, subprocess.CalledProcessError) as exc:
        smi = str(exc)
    sources = sorted((ROOT / "cudnn_vsa_b200").glob("*.py")) + sorted((ROOT / "cudnn_vsa_b200" / "csrc").glob("*.cu*"))
    return {"torch": torch.__version__, "cuda": torch.version.cuda, "backend": "libvsa_b200",
            "abi_version": int(_cabi.load().vsa_abi_version()), "gpu": props.name,
            "compute_capability": [props.major, props.minor], "gpu_memory_bytes": props.total_memory,
            "python": sys.version, "nvidia_smi": smi,
            "source_sha256": {str(p.relative_to(ROOT)): hashlib.sha256(p.read_bytes()).hexdigest() for p in sources}}


def main(argv=None):
    args = parse_args(argv)
    if args.ring:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    torch.set_num_threads(8)
    torch.backends.cuda.matmul.allow_tf32 = False
    group = init_ring(args) if args.ring else None
    writer = group is None or dist.get_rank(group) == 0
    try:
        args.output.parent.mkdir(parents=True, exist_ok=True)
        barrier(group)
        result = {"schema": "vsa-perf/v5", "environment": environment(), "cases": {},
                  "config": {k: (str(v) if isinstance(v, Path) else v) for k, v in vars(args).items() if k != "output"},
                  "scope": "Full forward/backward; timing excludes validation, capture and profiling"}
        if group is not None:
            runtime_batch = (getattr(group, "bound_device_id", None) is not None
                             if args.batch_p2p is None else args.batch_p2p)
            result["batch_p2p_effective"] = runtime_batch
            result["nccl_environment"] = {key: os.environ.get(key) for key in (
                "NCCL_MNNVL_ENABLE", "NCCL_CUMEM_ENABLE", "NCCL_P2P_DISABLE", "NCCL_MIN_P2P_NCHANNELS",
                "NCCL_MAX_P2P_NCHANNELS", "NCCL_NCHANNELS_PER_NET_PEER", "NCCL_NVLS_ENABLE", "NCCL_IB_DISABLE")}
        for name in args.cases:
            for heads in args.heads:
                result["cases"][f"{name}-h{heads}"] = run_case(name, heads, args, group)
                if writer:
                    args.output.write_text(json.dumps(result, indent=2) + "\n")
                torch.cuda.synchronize()
                barrier(group)
                torch.cuda.empty_cache()
        result["environment_after"] = environment()
        if result["environment"]["source_sha256"] != result["environment_after"]["source_sha256"]:
            raise AssertionError("Sources changed during measurement")
        if writer:
            args.output.write_text(json.dumps(result, indent=2) + "\n")
            print(f"Measurements: {args.output}", flush=True)
    finally:
        if group is not None:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
