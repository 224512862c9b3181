"""Static geometry of a packed VSA batch: segments, 64-slot blocks, row maps, routing templates.

Host-side planner for the B200 video-sparse-attention path.  It produces the same
public objects, field names, dtypes and values as the reference planner
(reference ``vsa_layout.py:12-489``) but is written as vectorised numpy index
arithmetic instead of per-token Python lists, so that a 880k-token ring geometry
plans in well under a second.

Vocabulary
    block        up to 64 tokens processed together: a <=64-token chunk of a dense
                 segment or one 4x4x4 (frame, height, width) tile of a sparse video.
    slot         position inside the zero-padded block stream, ``block * 64 + i``.
    slot_row     ``[64 * blocks]`` int64, input row held by a slot, ``-1`` for padding.
    row_slot     ``[tokens]`` int64, inverse of ``slot_row``.
    input_rows   ``[tokens]`` int64, row of the global raster stream each input row holds.
    routing      per (head, query block) ascending list of visible KV blocks
                 (``routing_indices [1,H,B,cap]`` int32, ``routing_counts [1,H,B]`` int32).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch
import torch.distributed as dist

BLOCK = 64
_TILE = 4
_DENSE_KINDS = ("text", "audio", "keyframe")


@dataclass(frozen=True)
class Segment:
    """One ordered token region of a sample (reference ``vsa_layout.py:12-45``).

    ``kind`` is ``"video"`` with ``size=(frames, height, width)`` or one of
    ``"text" / "audio" / "keyframe"`` with an integer ``size``.  ``sparsity`` is the
    fraction of a video's KV blocks each query block drops; ``None`` keeps the
    segment dense (raster chunks, no tiling).  A numeric value, including 0, enables
    4x4x4 tiling and block selection.
    """
    kind: str
    size: int | tuple[int, int, int]
    sparsity: float | None = None

    def __post_init__(self):
        if self.kind != "video" and self.kind not in _DENSE_KINDS:
            raise ValueError(f"Unknown segment kind: {self.kind}")
        if self.kind == "video":
            if not isinstance(self.size, tuple) or len(self.size) != 3:
                raise ValueError("Video size must be a (frames, height, width) tuple")
            extents, lowest = self.size, 1
            s = self.sparsity
            if s is not None and not (isinstance(s, (int, float)) and 0 <= s <= 1):
                raise ValueError("Video sparsity must be None or a finite number between 0 and 1")
        else:
            if not isinstance(self.size, int):
                raise ValueError("Dense segment size must be an integer")
            if self.sparsity is not None:
                raise ValueError("sparsity is only supported for video segments")
            extents, lowest = (self.size,), 0
        for n in extents:
            if not isinstance(n, int) or n < lowest:
                raise ValueError(
                    "Video dimensions must be positive; dense lengths must be nonnegative integers")

    @property
    def tokens(self):
        return math.prod(self.size) if isinstance(self.size, tuple) else self.size


@dataclass(frozen=True)
class SampleBlocks:
    """Global block range of one sample and its per-video KV budgets.

    Blocks are ordered ``[dense chunks..., video tiles...]``; ``video_spans`` holds one
    ``(first_block, end_block, keep)`` triple per numeric-sparsity video
    (reference ``vsa_layout.py:48-70``).
    """
    start: int
    end: int
    dense_blocks_num: int
    video_spans: tuple[tuple[int, int, int], ...]

    @property
    def dense_only(self):
        return len(self.video_spans) == 0

    @property
    def blocks(self):
        return self.end - self.start

    @property
    def kept(self):
        return self.dense_blocks_num + sum(span[2] for span in self.video_spans)


@dataclass(frozen=True)
class _RingMetadata:
    """Borrowed process group plus block ownership of one ring shard
    (reference ``vsa_layout.py:73-88``)."""
    group: dist.ProcessGroup = field(repr=False)
    size: int
    rank: int
    partition: str
    batch_p2p: bool | None
    bwd_bucket_size: str | int | None
    global_tokens: int
    # (sample, first local query block, end local query block, end of its dense query blocks)
    local_groups: tuple[tuple[SampleBlocks, int, int, int], ...]
    block_ids: torch.Tensor
    peer_block_sizes: torch.Tensor
    global_to_gather: torch.Tensor
    _runtime: dict = field(default_factory=dict, repr=False)


def _row_template(group, row_kind, capacity):
    """One routing row of a sample: ids written where they are static, count beside it.

    ``row_kind`` is ``"all"`` (every block of the sample is visible) or ``"routed"``
    (dense prefix, then each video's budget; a video kept in full is listed, a video
    that needs top-k leaves zeros for the router to fill).
    """
    row = np.zeros(capacity, dtype=np.int32)
    if row_kind == "all":
        row[:group.blocks] = np.arange(group.start, group.end, dtype=np.int32)
        return row, group.blocks
    dense = group.dense_blocks_num
    row[:dense] = np.arange(group.start, group.start + dense, dtype=np.int32)
    cursor = dense
    for first, end, keep in group.video_spans:
        if keep == end - first:
            row[cursor:cursor + keep] = np.arange(first, end, dtype=np.int32)
        cursor += keep
    return row, group.kept


@dataclass
class VSALayout:
    """Geometry, row maps and prepared routing templates of one packed batch.

    Built by :func:`build_vsa_layout`; field names, dtypes and contents follow the
    reference dataclass (``vsa_layout.py:91-207``) so callers can switch planners.
    ``input_order="raster"`` means inputs arrive in sample/segment order (frames,
    height, width inside a video); ``"block"`` means compact block order without
    padding.  ``ring`` is ``None`` for a full layout, otherwise the maps describe the
    local shard while ``groups`` / ``sample_slices`` stay global.
    """
    samples: tuple[tuple[Segment, ...], ...]
    head_num: int
    block_sizes: torch.Tensor
    row_slot: torch.Tensor
    slot_row: torch.Tensor
    groups: tuple[SampleBlocks, ...]
    coarse_blocks: torch.Tensor
    coarse_kv_blocks: torch.Tensor
    coarse_cu_q: torch.Tensor
    coarse_cu_kv: torch.Tensor
    coarse_max_q: int
    coarse_max_kv: int
    row_coarse: torch.Tensor
    input_rows: torch.Tensor
    input_order: str = "raster"
    dense_query_full: bool = False
    sample_slices: tuple = ()
    ring: _RingMetadata | None = None
    routing_indices: torch.Tensor = field(init=False, repr=False)
    routing_counts: torch.Tensor = field(init=False, repr=False)
    # (sample, first routed row, end routed row, offset of the sample in the pooled means)
    routing_groups: tuple = field(init=False, repr=False)
    coarse_rows: torch.Tensor = field(init=False, repr=False)
    dense_only: bool = field(init=False)

    def __post_init__(self):
        if self.input_order not in ("raster", "block"):
            raise ValueError('input_order must be "raster" or "block"')
        if self.ring is not None and self.input_order != "block":
            raise ValueError('Ring input_order must be "block" (compact, without padding)')
        if isinstance(self.head_num, bool) or not isinstance(self.head_num, int) or self.head_num <= 0:
            raise ValueError("head_num must be a positive integer")
        if not isinstance(self.dense_query_full, bool):
            raise ValueError("dense_query_full must be a bool")
        device = self.block_sizes.device
        exempt = self.dense_query_full
        capacity = max(g.blocks if exempt and g.dense_blocks_num else g.kept for g in self.groups)
        if self.ring is not None:
            local_groups = self.ring.local_groups
        else:
            local_groups = tuple((g, g.start, g.end, g.start + g.dense_blocks_num)
                                 for g in self.groups)
        # One [blocks, capacity] host template, broadcast over heads on the device.
        rows = np.zeros((self.blocks, capacity), dtype=np.int32)
        counts = np.zeros(self.blocks, dtype=np.int32)
        routing_groups, pooled = [], 0
        for g, begin, end, dense_end in local_groups:
            routed_from = dense_end if exempt else begin
            if g.kept == g.blocks:
                rows[begin:end], counts[begin:end] = _row_template(g, "all", capacity)
            else:
                if exempt and g.dense_blocks_num:
                    rows[begin:dense_end], counts[begin:dense_end] = _row_template(g, "all", capacity)
                rows[routed_from:end], counts[routed_from:end] = _row_template(g, "routed", capacity)
            offset = 0 if self.ring is not None else pooled - g.start
            if not g.dense_only:
                pooled += g.blocks
            if g.kept < g.blocks and routed_from < end:
                routing_groups.append((g, routed_from, end, offset))
        heads = self.head_num
        self.routing_indices = (torch.from_numpy(rows).to(device)[None, None]
                                .expand(1, heads, self.blocks, capacity).contiguous())
        self.routing_counts = (torch.from_numpy(counts).to(device)[None, None]
                               .expand(1, heads, self.blocks).contiguous())
        self.routing_groups = tuple(routing_groups)
        # Input rows of every coarse block (-1 = padding), used by the merge adjoint.
        self.coarse_rows = self.slot_row.view(self.blocks, BLOCK)[self.coarse_blocks]
        self.dense_only = all(g.dense_only for g in self.groups)

    @property
    def tokens(self):
        return self.row_slot.numel()

    @property
    def blocks(self):
        return self.block_sizes.numel()

    @property
    def padded_tokens(self):
        return self.blocks * BLOCK

    @property
    def all_blocks_full(self):
        return self.padded_tokens == self.tokens

    @property
    def slots_are_input(self):
        return self.input_order == "block" and self.all_blocks_full

    @property
    def sample_lengths(self):
        return tuple(sum(s.stop - s.start for s in slices) for slices in self.sample_slices)


# --------------------------------------------------------------------------- planning

def _dense_segment_blocks(tokens, offset):
    """Rows and sizes of the <=64-token raster chunks of a dense segment."""
    count = -(-tokens // BLOCK)
    sizes = np.full(count, BLOCK, dtype=np.int64)
    if count:
        sizes[-1] = tokens - (count - 1) * BLOCK
    return np.arange(offset, offset + tokens, dtype=np.int64), sizes


def _video_segment_blocks(size, offset):
    """Rows and sizes of the 4x4x4 tiles of a video, tiles and tokens visited F, H, W."""
    frames, height, width = size
    padded = [-(-n // _TILE) * _TILE for n in size]
    grid = np.full(padded, -1, dtype=np.int64)
    grid[:frames, :height, :width] = (
        offset + np.arange(frames * height * width, dtype=np.int64).reshape(size))
    tiles = grid.reshape(padded[0] // _TILE, _TILE, padded[1] // _TILE, _TILE,
                         padded[2] // _TILE, _TILE)
    tiles = tiles.transpose(0, 2, 4, 1, 3, 5).reshape(-1, BLOCK)
    valid = tiles >= 0
    return tiles[valid], valid.sum(1).astype(np.int64)


def _plan_sample(segments, token_offset, block_offset):
    """Block rows, sizes, routing group and segment slices of one sample
    (behaviour of reference ``vsa_layout.py:347-372``)."""
    slices = []
    for seg in segments:
        slices.append(slice(token_offset, token_offset + seg.tokens))
        token_offset += seg.tokens
    rows, sizes, spans = [], [], []
    blocks = 0
    dense_blocks = 0
    for want_dense in (True, False):
        for seg, where in zip(segments, slices):
            if (seg.sparsity is None) != want_dense:
                continue
            if want_dense:
                r, s = _dense_segment_blocks(seg.tokens, where.start)
            else:
                r, s = _video_segment_blocks(seg.size, where.start)
            first = block_offset + blocks
            rows.append(r)
            sizes.append(s)
            blocks += len(s)
            if not want_dense:
                end = block_offset + blocks
                # Python float arithmetic on purpose: (1-0.95)*14720 rounds up to 737.
                keep = max(1, math.ceil((1 - seg.sparsity) * (end - first)))
                spans.append((first, end, keep))
        if want_dense:
            dense_blocks = blocks
    group = SampleBlocks(start=block_offset, end=block_offset + blocks,
                         dense_blocks_num=dense_blocks, video_spans=tuple(spans))
    rows = np.concatenate(rows) if rows else np.zeros(0, dtype=np.int64)
    sizes = np.concatenate(sizes) if sizes else np.zeros(0, dtype=np.int64)
    return rows, sizes, group, tuple(slices)


def _plan_samples(samples):
    """Validate the nested sample description and plan all global blocks.

    Returns ``(samples, rows, sizes, groups, sample_slices)`` where ``rows`` is the
    concatenation of every block's raster rows in block order and ``sizes`` the token
    count of each block.
    """
    try:
        samples = tuple(tuple(sample) for sample in samples)
    except TypeError as error:
        raise ValueError("samples must be a nested sequence of Segment objects") from error
    if not samples:
        raise ValueError("samples must be nonempty")
    all_rows, all_sizes, groups, sample_slices = [], [], [], []
    token_offset = block_offset = 0
    for sample in samples:
        if not sample or any(not isinstance(seg, Segment) for seg in sample):
            raise ValueError("Each sample must be a nonempty sequence of Segment objects")
        if not any(seg.kind == "video" for seg in sample):
            raise ValueError("Each sample requires at least one video segment")
        rows, sizes, group, slices = _plan_sample(sample, token_offset, block_offset)
        all_rows.append(rows)
        all_sizes.append(sizes)
        groups.append(group)
        sample_slices.append(slices)
        token_offset = slices[-1].stop
        block_offset = group.end
    return samples, np.concatenate(all_rows), np.concatenate(all_sizes), groups, sample_slices


def _plan_ring_blocks(groups, ring_size, partition="cyclic"):
    """Owned global block ids per rank (lists), behaviour of reference ``vsa_layout.py:210-235``.

    ``"cyclic"`` gives block ``b`` to rank ``b % ring_size`` using global ids;
    ``"contiguous"`` gives each rank one interval per sample and rotates which ranks
    take a sample's remainder blocks, so per-sample and cumulative counts stay within one.
    """
    if partition not in ("cyclic", "contiguous"):
        raise ValueError('ring_partition must be "cyclic" or "contiguous"')
    if partition == "cyclic":
        owned = [[] for _ in range(ring_size)]
        for g in groups:
            for rank in range(ring_size):
                first = g.start + (rank - g.start) % ring_size
                owned[rank].extend(range(first, g.end, ring_size))
        return owned
    owned = [[] for _ in range(ring_size)]
    lead = 0
    for g in groups:
        base, extra = divmod(g.end - g.start, ring_size)
        cursor = g.start
        for step in range(ring_size):
            take = base + (1 if step < extra else 0)
            owned[(lead + step) % ring_size].extend(range(cursor, cursor + take))
            cursor += take
        lead = (lead + extra) % ring_size
    return owned


def _finalize_layout(samples, rows, sizes, groups, sample_slices, *, head_num,
                     dense_query_full, device, input_order, ring_size, ring_rank,
                     ring_cp_group, ring_cp_batch_p2p, ring_cp_bwd_bucket_size,
                     ring_partition="cyclic") -> VSALayout:
    """Derive padding maps, coarse metadata and (optionally) the ring shard."""
    def tensor(values, dtype=torch.int64):
        array = np.asarray(values)
        return torch.from_numpy(np.ascontiguousarray(array)).to(dtype).to(device)

    starts = np.concatenate(([0], np.cumsum(sizes)))  # first position of each block in `rows`
    ring = None
    if ring_size is not None:
        total = len(sizes)
        capacity = -(-total // ring_size)
        peer_ids = _plan_ring_blocks(groups, ring_size, ring_partition)
        owned = np.asarray(peer_ids[ring_rank], dtype=np.int64)
        local_groups = []
        for g in groups:
            begin, end = np.searchsorted(owned, [g.start, g.end])
            if begin < end:
                dense_end = begin + np.searchsorted(owned[begin:end], g.start + g.dense_blocks_num)
                local_groups.append((g, int(begin), int(end), int(dense_end)))
        peer_sizes = np.zeros((ring_size, capacity + (-capacity % 4)), dtype=np.int32)
        global_to_gather = np.zeros(total, dtype=np.int64)
        for rank, ids in enumerate(peer_ids):
            ids = np.asarray(ids, dtype=np.int64)
            peer_sizes[rank, :len(ids)] = sizes[ids]
            global_to_gather[ids] = rank * capacity + np.arange(len(ids))
        block_ids = np.full(capacity, -1, dtype=np.int64)
        block_ids[:len(owned)] = owned
        ring = _RingMetadata(
            group=ring_cp_group, batch_p2p=ring_cp_batch_p2p,
            bwd_bucket_size=ring_cp_bwd_bucket_size, size=ring_size, rank=ring_rank,
            partition=ring_partition, global_tokens=int(sizes.sum()),
            local_groups=tuple(local_groups), block_ids=tensor(block_ids),
            # Row stride padded to a multiple of four int32 so every peer row starts 16-byte aligned.
            peer_block_sizes=tensor(peer_sizes, torch.int32)[:, :capacity],
            global_to_gather=tensor(global_to_gather))
        local_sizes = np.zeros(capacity, dtype=np.int64)
        local_sizes[:len(owned)] = sizes[owned]
        if len(owned):
            pick = np.concatenate([np.arange(starts[b], starts[b + 1]) for b in owned])
        else:
            pick = np.zeros(0, dtype=np.int64)
        local_rows = rows[pick]
    else:
        local_groups = [(g, g.start, g.end, g.start + g.dense_blocks_num) for g in groups]
        local_sizes, local_rows = sizes, rows
    blocks = len(local_sizes)
    tokens = int(local_sizes.sum())
    if input_order == "raster":
        input_rows = np.arange(tokens, dtype=np.int64)
        held_rows = local_rows
    else:
        input_rows = local_rows
        held_rows = np.arange(tokens, dtype=np.int64)
    # Slot of the i-th valid token in block order.
    local_starts = np.concatenate(([0], np.cumsum(local_sizes)))[:-1]
    block_of_token = np.repeat(np.arange(blocks, dtype=np.int64), local_sizes)
    slot_of_token = block_of_token * BLOCK + (np.arange(tokens, dtype=np.int64)
                                              - np.repeat(local_starts, local_sizes))
    slot_row = np.full(blocks * BLOCK, -1, dtype=np.int64)
    slot_row[slot_of_token] = held_rows
    row_slot = np.zeros(tokens, dtype=np.int64)
    row_slot[held_rows] = slot_of_token
    coarse_q, coarse_kv, cu_q, cu_kv = [], [], [0], [0]
    for g, begin, end, _ in local_groups:
        if g.dense_only:
            continue
        coarse_q.append(np.arange(begin, end, dtype=np.int64))
        coarse_kv.append(np.arange(g.start, g.end, dtype=np.int64))
        cu_q.append(cu_q[-1] + end - begin)
        cu_kv.append(cu_kv[-1] + g.end - g.start)
    coarse_q = np.concatenate(coarse_q) if coarse_q else np.zeros(0, dtype=np.int64)
    coarse_kv = np.concatenate(coarse_kv) if coarse_kv else np.zeros(0, dtype=np.int64)
    # Blocks of fine-only samples point at a sentinel one past the last coarse row.
    block_to_coarse = np.full(blocks, len(coarse_q), dtype=np.int64)
    block_to_coarse[coarse_q] = np.arange(len(coarse_q), dtype=np.int64)
    coarse_blocks = tensor(coarse_q)
    coarse_cu_q = tensor(cu_q, torch.int32)
    return VSALayout(
        samples=samples, head_num=head_num, dense_query_full=dense_query_full,
        block_sizes=tensor(local_sizes, torch.int32),
        row_slot=tensor(row_slot), slot_row=tensor(slot_row), groups=tuple(groups),
        coarse_blocks=coarse_blocks,
        coarse_kv_blocks=coarse_blocks if ring is None else tensor(coarse_kv),
        coarse_cu_q=coarse_cu_q,
        coarse_cu_kv=coarse_cu_q if ring is None else tensor(cu_kv, torch.int32),
        coarse_max_q=int(np.diff(cu_q).max()) if len(cu_q) > 1 else 0,
        coarse_max_kv=int(np.diff(cu_kv).max()) if len(cu_kv) > 1 else 0,
        row_coarse=tensor(block_to_coarse[row_slot // BLOCK]),
        input_rows=tensor(input_rows), input_order=input_order,
        sample_slices=tuple(sample_slices), ring=ring)


def build_vsa_layout(samples, *, head_num, dense_query_full=False, device="cpu",
                     input_order="raster", ring_cp_group=None, ring_cp_batch_p2p=None,
                     ring_cp_bwd_bucket_size="auto", ring_partition="cyclic") -> VSALayout:
    """Plan one packed batch (reference ``vsa_layout.py:375-465``).

    ``samples`` is a sequence of samples, each a sequence of :class:`Segment`; every
    sample needs at least one video segment and samples never attend to each other.
    Inside a sample, dense (``sparsity=None``) segments come first in block order, cut
    into consecutive <=64-token chunks; numeric-sparsity videos follow as 4x4x4 tiles,
    each with its own budget ``keep = max(1, ceil((1 - sparsity) * blocks))``.  A sample
    with only dense segments runs fine attention alone (no pooling, coarse or gate).

    ``dense_query_full=True`` lets dense query blocks see every KV block of their sample;
    dense KV blocks are always visible.  ``input_order`` is ``"raster"`` or ``"block"``
    (compact block order, produced once by ``raster_to_block_wo_padding``).

    Passing ``ring_cp_group`` (an existing process group containing this rank, size one
    allowed) builds this rank's ring shard: whole blocks are owned ``"cyclic"`` (global
    block ``b`` on rank ``b % size``) or ``"contiguous"`` (one interval per sample per
    rank); every rank holds ``ceil(blocks / size)`` block slots, padded with empty blocks.
    The group is borrowed, never created or destroyed.  ``ring_cp_batch_p2p`` and
    ``ring_cp_bwd_bucket_size`` are transport options validated exactly like the
    reference's and require a group.
    """
    if input_order not in ("raster", "block"):
        raise ValueError('input_order must be "raster" or "block"')
    if ring_partition not in ("cyclic", "contiguous"):
        raise ValueError('ring_partition must be "cyclic" or "contiguous"')
    if ring_cp_batch_p2p is not None and not isinstance(ring_cp_batch_p2p, bool):
        raise ValueError("ring_cp_batch_p2p must be a bool or None")
    bucket = ring_cp_bwd_bucket_size
    if bucket is not None and not (isinstance(bucket, str) and bucket == "auto"):
        if isinstance(bucket, bool) or not isinstance(bucket, int) or bucket < 1:
            raise ValueError('ring_cp_bwd_bucket_size must be "auto", a positive integer or None')
    ring_size = ring_rank = None
    if ring_cp_group is not None:
        if input_order != "block":
            raise ValueError('Ring input_order must be "block" (compact, without padding)')
        if not isinstance(ring_cp_group, dist.ProcessGroup):
            raise ValueError("ring_cp_group must be a ProcessGroup containing this rank")
        ring_size, ring_rank = ring_cp_group.size(), ring_cp_group.rank()
        if ring_size < 1 or not 0 <= ring_rank < ring_size:
            raise ValueError("ring_cp_group must contain this rank and have positive size")
        if isinstance(head_num, bool) or not isinstance(head_num, int) or head_num < 1:
            raise ValueError("head_num must be a positive integer")
        if not isinstance(dense_query_full, bool):
            raise ValueError("dense_query_full must be a bool")
    elif (ring_cp_batch_p2p is not None or ring_cp_bwd_bucket_size != "auto"
          or ring_partition != "cyclic"):
        raise ValueError("Ring transport options require ring_cp_group")
    samples, rows, sizes, groups, sample_slices = _plan_samples(samples)
    if ring_size is not None and len(sizes) < ring_size:
        raise ValueError("Ring requires at least ring_size global blocks; "
                         f"got global_blocks={len(sizes)}, ring_size={ring_size}")
    return _finalize_layout(samples, rows, sizes, groups, sample_slices,
                            head_num=head_num, dense_query_full=dense_query_full, device=device,
                            input_order=input_order, ring_size=ring_size, ring_rank=ring_rank,
                            ring_cp_group=ring_cp_group, ring_cp_batch_p2p=ring_cp_batch_p2p,
                            ring_cp_bwd_bucket_size=ring_cp_bwd_bucket_size,
                            ring_partition=ring_partition)
