"""Generate the golden vectors under ``tests/golden/`` from the reference's own CPU code.

Run once, in a container where the reference checkout is available::

    python tests/golden/make_golden.py /path/to/reference

The reference imports two GPU-only third-party backends at import time; this script puts
two stub modules ahead of them on ``sys.path`` (in a temporary directory) so that the
reference's planner, router, pooling, merge and its CPU test substitutes can run
unmodified.  Nothing here is imported by the library or by the tests; the tests only
read the files this script writes:

``layouts.json``   sha256 of every tensor field of the reference planner's layouts
                   (full layouts and ring shards) for a list of geometries.
``cases.npz``      outputs, gradients and routing tables of the reference's token-level
                   math (``reference_pack``) and of its CPU orchestration (``cpu_attention``)
                   on seeded inputs for small geometries, as raw BF16 bit patterns.
``ring.npz``       the reference's ring partition of routing rows and global routing.
"""
import hashlib
import json
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

HERE = Path(__file__).resolve().parent


def install_stubs(reference):
    stub = Path(tempfile.mkdtemp(prefix="vsa_stub_"))
    (stub / "cudnn").mkdir()
    (stub / "cudnn" / "__init__.py").write_text("BSA = None\n")
    (stub / "flash_attn" / "cute").mkdir(parents=True)
    (stub / "flash_attn" / "__init__.py").write_text("")
    (stub / "flash_attn" / "cute" / "__init__.py").write_text("")
    (stub / "flash_attn" / "cute" / "interface.py").write_text(
        "def flash_attn_varlen_func(*a, **k):\n    raise RuntimeError('not installed')\n")
    sys.path[:0] = [str(stub), str(reference)]


def geometries(Segment):
    S = Segment
    return {
        "c1": [[S("video", (8, 16, 16), .75), S("text", 256)]],
        "ragged": [[S("video", (5, 9, 11), .7), S("text", 67)],
                   [S("text", 3), S("video", (1, 3, 5))],
                   [S("video", (4, 8, 12), .5), S("video", (5, 4, 7), .9), S("audio", 17), S("text", 0)]],
        "partial_blocks": [[S("video", (1, 3, 5), .9), S("text", 7)]],
        "fine_only_peer": [[S("video", (1, 2, 3), .5)], [S("video", (1, 2, 3))]],
        "dense": [[S("video", (1, 9, 11)), S("text", 67)], [S("video", (1, 3, 5)), S("text", 3)]],
        "mixed": [[S("video", (1, 9, 8)), S("text", 7)],
                  [S("video", (5, 4, 8), .5), S("text", 65)],
                  [S("video", (2, 3, 5), .5), S("text", 9)]],
        "zero_sparsity": [[S("video", (4, 4, 8), 0.0), S("text", 5)]],
        "full_blocks": [[S("video", (4, 4, 8), .5), S("text", 64)], [S("video", (1, 8, 8)), S("text", 64)]],
        "c2": [[S("video", (31, 45, 80), .9), S("text", 2048)]],
        "c3": [[S("video", (31, 45, 80), .9), S("text", 2048)],
               [S("video", (1, 45, 80)), S("text", 2048)], [S("video", (1, 45, 80)), S("text", 2048)]],
        "c4": [[S("video", (21, 30, 52), .8), S("text", 512), S("audio", 1024)]] * 4,
        "c5": [[S("video", (61, 90, 160), .95), S("text", 4096)]],
    }


LAYOUT_FIELDS = ("block_sizes", "row_slot", "slot_row", "coarse_blocks", "coarse_kv_blocks",
                 "coarse_cu_q", "coarse_cu_kv", "row_coarse", "input_rows", "routing_indices",
                 "routing_counts", "coarse_rows")


def digest(t):
    t = t.contiguous().cpu()
    return f"{t.dtype}:{tuple(t.shape)}:" + hashlib.sha256(t.numpy().tobytes()).hexdigest()


def layout_record(layout):
    rec = {name: digest(getattr(layout, name)) for name in LAYOUT_FIELDS}
    rec["scalars"] = [layout.coarse_max_q, layout.coarse_max_kv, layout.dense_only, layout.tokens,
                      layout.blocks, list(layout.sample_lengths),
                      [[g.start, g.end, g.dense_blocks_num, [list(s) for s in g.video_spans]]
                       for g in layout.groups],
                      [[b, e, o, g.start] for g, b, e, o in layout.routing_groups]]
    if layout.ring is not None:
        r = layout.ring
        rec["ring"] = {"block_ids": digest(r.block_ids), "peer_block_sizes": digest(r.peer_block_sizes),
                       "global_to_gather": digest(r.global_to_gather),
                       "scalars": [r.size, r.rank, r.partition, r.global_tokens,
                                   [[b, e, d, g.start] for g, b, e, d in r.local_groups]]}
    return rec


def seeded(tokens, heads, seed, count):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randn(tokens, heads, 128, generator=gen).to(torch.bfloat16) for _ in range(count)]


def bits(t):
    return t.detach().contiguous().view(torch.int16).numpy()


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference>")
    reference = Path(sys.argv[1])
    install_stubs(reference)
    import vsa_kernels
    import vsa_layout
    from tests import reference as ref
    from vsa_core import route

    # The five substitutions of the reference's cpu_kernels fixture (tests/conftest.py:14-21).
    vsa_kernels.gather = ref.cpu_gather
    vsa_kernels.block_means = vsa_kernels.block_means.__wrapped__
    vsa_kernels.routing_and_coarse_means = vsa_kernels.routing_and_coarse_means.__wrapped__
    vsa_kernels._fine_coarse_gate_add_forward = ref.cpu_merge_forward
    vsa_kernels._fine_coarse_gate_add_backward = ref.cpu_merge_backward

    geo = geometries(vsa_layout.Segment)
    layouts = {}
    for name, samples in geo.items():
        heads = 1 if name == "c5" else 2
        for order in ("raster", "block"):
            for full in (False, True):
                if name in ("c2", "c3", "c4", "c5") and (full or (name == "c5" and order == "raster")):
                    continue
                key = f"{name}/{order}/dqf{int(full)}"
                layouts[key] = layout_record(vsa_layout.build_vsa_layout(
                    samples, head_num=heads, input_order=order, dense_query_full=full))
        blocks = vsa_layout.build_vsa_layout(samples, head_num=1).blocks
        for size in (2, 3, 8):
            if blocks < size or name in ("c3", "c4"):
                continue
            for partition in ("cyclic", "contiguous"):
                for rank in sorted({0, size - 1}):
                    if name in ("c2", "c5") and (size != 8 or partition != "cyclic"):
                        continue
                    key = f"{name}/ring{size}.{rank}/{partition}"
                    layouts[key] = layout_record(vsa_layout.build_vsa_layout(
                        samples, head_num=heads, input_order="block", ring_partition=partition,
                        ring_cp_group=dist.ProcessGroup(rank, size)))
    (HERE / "layouts.json").write_text(json.dumps(layouts, indent=0, sort_keys=True))

    arrays = {}
    for name in ("c1", "ragged", "partial_blocks", "fine_only_peer", "dense", "mixed",
                 "zero_sparsity", "full_blocks"):
        samples, heads = geo[name], 2
        for full in (False, True):
            if full and name not in ("mixed", "full_blocks"):
                continue
            layout = vsa_layout.build_vsa_layout(samples, head_num=heads, dense_query_full=full)
            q, k, v, gate = seeded(layout.tokens, heads, 0, 4)
            dy, = seeded(layout.tokens, heads, 1, 1)
            for label, fn in (("pack", ref.reference_pack(samples, layout.sample_slices,
                                                          dense_query_full=full)),
                              ("cpu", lambda *xs: ref.cpu_attention(*xs, layout))):
                if label == "cpu" and name not in ("ragged", "mixed", "fine_only_peer"):
                    continue
                leaves = [x.clone().requires_grad_() for x in (q, k, v, gate)]
                out = fn(*leaves)
                grads = torch.autograd.grad(out, leaves, dy, allow_unused=True)
                grads = [torch.zeros_like(q) if g is None else g for g in grads]
                stride = 4 if layout.tokens > 600 else 1
                key = f"{name}/dqf{int(full)}/{label}"
                arrays[f"{key}/out"] = bits(out[::stride])
                for tag, g in zip(("dq", "dk", "dv", "dgate"), grads):
                    arrays[f"{key}/{tag}"] = bits(g[::stride])
            if not layout.dense_only:
                slots = [ref.cpu_gather(x, layout.slot_row) for x in (q, k, v)]
                qr, kr, qc, kc, vc = vsa_kernels.routing_and_coarse_means(
                    *slots, layout.block_sizes, layout.coarse_blocks)
                arrays[f"{name}/dqf{int(full)}/routing"] = route(qr, kr, layout).numpy()
                arrays[f"{name}/dqf{int(full)}/q_mean"] = qr.numpy()
                arrays[f"{name}/dqf{int(full)}/coarse_v_mean"] = bits(vc)
    np.savez_compressed(HERE / "cases.npz", **arrays)

    ring = {}
    for name, size in (("ragged", 2), ("ragged", 3), ("mixed", 2), ("partial_blocks", 3)):
        samples = geo[name]
        full = vsa_layout.build_vsa_layout(samples, head_num=2)
        q, k, v, _ = seeded(full.tokens, 2, 0, 4)
        slots = [ref.cpu_gather(x, full.slot_row) for x in (q, k, v)]
        qm, km, _ = vsa_kernels.block_means(*slots, full.block_sizes)
        for rank in range(size):
            local = vsa_layout.build_vsa_layout(samples, head_num=2, input_order="block",
                                                ring_cp_group=dist.ProcessGroup(rank, size))
            ids = local.ring.block_ids
            q_local = qm[ids.clamp_min(0)].masked_fill((ids < 0)[:, None, None], 0)
            index = route(q_local, km, local)
            lists, counts = vsa_kernels._partition_indices_reference(
                index, local.routing_counts, local.ring.global_to_gather, size, local.blocks)
            key = f"{name}/ring{size}.{rank}"
            ring[f"{key}/index"] = index.numpy()
            ring[f"{key}/lists"] = lists.numpy()
            ring[f"{key}/counts"] = counts.numpy()
    np.savez_compressed(HERE / "ring.npz", **ring)
    print("wrote", len(layouts), "layout records,", len(arrays), "case arrays,", len(ring), "ring arrays")


if __name__ == "__main__":
    main()
