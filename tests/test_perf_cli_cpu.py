"""CPU: command line and workloads of ``tests/perf_vsa.py`` (the reference pins the same facts for
its own benchmark in ``tests/test_benchmark.py:27-40, 124-154``)."""
import pytest

from tests import perf_vsa


def test_default_workload_is_the_720p_pack():
    samples = perf_vsa.case_geometry("default")
    lengths = [sum(seg.tokens for seg in sample) for sample in samples]
    assert lengths == [113648, 5648, 5648]
    assert samples[0][0].size == (31, 45, 80) and samples[0][0].sparsity == 0.9
    assert samples[1][0].sparsity is None and samples[2][0].size == (1, 45, 80)
    assert sum(seg.tokens for sample in perf_vsa.case_geometry("thd720p44s") for seg in sample) == 961696


def test_defaults_follow_the_reference_cli():
    args = perf_vsa.parse_args([])
    assert (args.cases, args.heads, args.seed, args.input_order) == (["default"], [2, 4], 2026, "raster")
    assert (args.warmup, args.repeats, args.profile) == (5, 80, True)
    assert args.output.name == "perf.json"
    ring = perf_vsa.parse_args(["--ring"])
    assert (ring.cases, ring.heads, ring.seed, ring.input_order) == (["ragged", "single64k", "thd64k"], [2], 937, "block")
    assert (ring.warmup, ring.repeats, ring.profile, ring.ring_partition) == (3, 30, False, "cyclic")
    assert perf_vsa.parse_args(["--ring", "--bwd-bucket-size", "backend"]).bwd_bucket_size is None
    assert perf_vsa.parse_args(["--ring", "--bwd-bucket-size", "7"]).bwd_bucket_size == 7


@pytest.mark.parametrize("argv", [["--ring-size", "2"], ["--batch-p2p"], ["--ring-partition", "contiguous"],
                                  ["--ring", "--input-order", "raster"], ["--heads", "0"], ["--eps", "1.5"],
                                  ["--ring", "--bwd-bucket-size", "0"], ["--repeats", "0"]])
def test_invalid_combinations_are_rejected(argv):
    with pytest.raises(SystemExit):
        perf_vsa.parse_args(argv)
