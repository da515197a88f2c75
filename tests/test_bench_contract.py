"""What needs no GPU of the measurement side: the command line's refusals, the reference arm's
answer, the byte and flop counts that the fractions rest on, and the launch plans of the
tensor-core products."""
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _bench(*args, env=None):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=120, env=env)


def test_more_than_one_gpu_is_refused_with_one_line():
    p = _bench("--gpus", "2")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "single-GPU" in p.stdout


def test_reference_arm_says_why_it_is_unavailable(tmp_path):
    """Without a built copy of the reference (here: an empty folder in its place) the arm prints one line that says so."""
    import os
    p = _bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1", env=dict(os.environ, LLAISYS_REF_DIR=str(tmp_path)))
    assert p.returncode == 0 and len(p.stdout.strip().splitlines()) == 1
    line = json.loads(p.stdout.strip())
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]
    assert "--reference-src" in line["unavailable"]


def test_own_workload_needs_a_shape_that_has_one():
    p = _bench("--workload", "own")
    assert p.returncode == 2 and "--shape" in p.stdout


def test_weight_counts_of_the_benchmark_shapes():
    sys.path.insert(0, str(ROOT))
    import bench
    lin, head = bench.linear_params(bench.QWEN2_1_5B, 28)
    # 28 layers x (2048 x 1536 + 1536 x 1536 + 3 x 8960 x 1536) and the head 151936 x 1536
    assert lin == 28 * (2048 * 1536 + 1536 * 1536 + 3 * 8960 * 1536) and head == 151936 * 1536
    assert abs((lin + head) * 2 / 1e9 - 3.087) < 0.01          # bytes a decode step streams, in GB
    name, cfg7 = bench.SHAPES["7b"]
    lin7, head7 = bench.linear_params(cfg7, 28)
    assert abs((lin7 + head7) * 2 / 1e9 - 14.14) < 0.02
    assert set(bench.OWN_WORKLOADS) == {"7b", "32b"}


@pytest.mark.parametrize("T", [1, 8, 16, 17, 32, 64, 100, 128, 200, 2048])
@pytest.mark.parametrize("rows,K,dual", [(2048, 1536, False), (1536, 1536, False), (8960, 1536, True), (1536, 8960, False),
                                         (151936, 1536, False), (136, 72, False), (300, 1096, False), (18944, 3584, True)])
def test_launch_plans_are_launchable(T, rows, K, dual):
    from llaisys_b200.kernels import ops
    bn, splits = ops.tc_plan(T, rows, K, 148, dual)
    assert bn in (16, 32, 64, 128, 256) and bn >= min(T, 256) and (bn == 16 or bn // 2 < T)
    kblocks = math.ceil(K / 64)
    assert splits in (1, 2, 4, 8, 16) and splits <= max(1, kblocks // 2)
    if splits > 1:
        assert bn <= 128                                             # the cluster reduction takes tiles up to 128 tokens
        chunk = math.ceil(kblocks / splits)
        assert (splits - 1) * chunk < kblocks                        # no CTA of the cluster is left without a k-block
        tiles = math.ceil(rows / 128) * math.ceil(T / bn)
        assert tiles * splits <= 2 * 148                             # all resident at once, at most two per SM
    if splits == 16:
        assert bn == 64 or T <= 4


@pytest.mark.parametrize("T,N,K,want", [(2048, 1536, 8960, 3), (2048, 1536, 1536, 1), (4096, 1536, 8960, 3), (8192, 1536, 8960, 1),
                                        (2048, 3584, 18944, 3), (4096, 3584, 18944, 2), (300, 200, 72, 1), (100000, 5120, 27648, 1)])
def test_k_ranges_of_the_prefill_projection_that_ends_in_the_residual_add(T, N, K, want):
    """Where one round of 256 x 256 tiles would leave SM pairs idle (48 tiles on 74 pairs), the K range is cut so
    that the units fill the rounds; where the tiles fill many rounds anyway, it is not (the plan is host code)."""
    import ctypes
    from llaisys_b200.csrc.build import load_module
    f = load_module("gemm_tc2.cu").llb_gemm_tc2_into_ksplit
    f.restype, f.argtypes = ctypes.c_int, [ctypes.c_int] * 4
    ks = f(T, N, K, 74)
    assert ks == want
    kblocks = math.ceil(K / 64)
    assert 1 <= ks <= 4 and (ks - 1) * math.ceil(kblocks / ks) < kblocks          # no K range is empty


def test_clock_summary_is_over_the_samples_of_the_timed_region():
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench
    clk = bench.ClockSampler()
    row = lambda mhz, cap: [str(mhz), "1965", "Not Active", "Not Active", "Not Active", "Active" if cap else "Not Active"]
    clk.rows = [(10.00, row(300, False)), (10.05, row(1900, False)), (10.10, row(1950, True)), (10.15, row(1920, True)),
                (10.40, row(500, False))]
    clk.t0, clk.t1 = 10.04, 10.12
    s = clk.summary()                      # the samples at 10.05, 10.10 and (within a period and a half of the end) 10.15
    assert s == {"sm_mhz": 1920, "sm_max_mhz": 1965, "reasons": ["sw_power_cap"], "samples": 3}
    clk.t0, clk.t1 = 11.0, 11.001          # a region no sample fell into: all of them
    assert clk.summary()["samples"] == 5
