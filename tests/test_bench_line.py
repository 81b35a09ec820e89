"""The bench's JSON line is assembled by pure functions; build it here for every world size and
every --fused-exchange value without a device, so that a typo in the line-building code cannot
surface only on a multi-GPU box."""
import json

import pytest

import bench


def _line(world, decode=None):
    clocks = {"sm_mhz": 1965.0, "sm_max_mhz": 1965.0, "samples": 6, "reasons": []}
    return bench.make_line(world=world, steps=20, warmup=5, layers=128, passes=80, order="relaxed", ms=530.0,
                           ms_other=None if world > 1 else 780.0, graphed=True, e2e_s=0.2, e2e_blocking_s=0.4,
                           e2e_steps=5, e2e_passes=20, clocks=clocks, peak=6546.6, peak_kind="measured", decode=decode,
                           cpu={"value": 6.0, "unit": "GB/s", "cores": 16, "kind": "port", "sample": "x"} if world == 1 else None)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_line_builds_for_every_world_size(world):
    decode = {"tok_s": 500.0, "unit": "tok/s", "scaling": "strong",
              "batch1": {"tok_s": 500.0, "ms_per_step": 2.0, "parallelism": bench.decode_parallelism(world, "auto", 1)},
              "batch16": {"tok_s": 4000.0, "ms_per_step": 4.0, "parallelism": bench.decode_parallelism(world, "auto", 16)}}
    line = _line(world, decode)
    json.dumps(line)                                    # serialisable
    assert line["metric"] == "q4k_matvec_gbs" and line["unit"] == "GB/s" and line["n_gpus"] == world
    assert line["scaling"] == "weak" and line["higher_is_better"] is True and line["vs_baseline"] is None
    # whole-job value: bytes of all ranks over the timed region
    total = world * 128 * 80 * bench.ALG_BYTES * 20
    assert line["value"] == pytest.approx(total / 0.530 / 1e9)
    assert line["ms_per_step"] == pytest.approx(530.0 / 20)
    assert line["gpu_launches"] == 128 * 80 * 20
    # the roofline is per launch on one GPU, whatever the world size
    us = 530.0 * 1e3 / (20 * 128 * 80)
    assert line["roofline"]["us_per_launch"] == pytest.approx(us)
    assert line["roofline"]["achieved"] == pytest.approx(bench.ALG_BYTES / us / 1e3)
    assert line["roofline"]["frac"] == pytest.approx(line["roofline"]["achieved"] / 6546.6)
    assert line["roofline"]["traffic"] == bench.DRAM_TRAFFIC_PER_LAUNCH
    assert line["detail"]["timed_region_s"] == pytest.approx(0.53)
    assert line["detail"]["us_per_launch_x_sm_mhz"] == pytest.approx(us * 1965.0)
    assert line["e2e"]["h2d_bytes_per_step"] == 128 * 20 * 4 * 4096
    assert line["e2e"]["value"] == pytest.approx(world * 128 * 20 * 5 * bench.ALG_BYTES / 0.2 / 1e9)
    assert line["decode"]["batch1"]["tok_s"] == 500.0
    assert ("cpu_baseline" in line) == (world == 1)
    assert (line["detail"]["other_order"] is None) == (world > 1)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_both_arms_print_the_same_config(world):
    assert _line(world)["config"] == bench.workload_config(world, 128)
    assert bench.workload_config(world, 128)["workload"] == "cfg1: Q4_K matvec 4096x4096, M=1, fp32 x"
    assert ("none" == bench.workload_config(world, 128)["sharding"]) == (world == 1)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("fused", ["auto", "on", "off"])
@pytest.mark.parametrize("batch", [1, 2, 16])
def test_decode_parallelism_wording(world, fused, batch):
    s = bench.decode_parallelism(world, fused, batch)
    if world == 1:
        assert s == "none"
        return
    assert s.startswith(f"tp{world}")
    want_fused = batch <= 2 and fused == "on"
    assert ("fused" in s) == want_fused


def test_decode_legs_survive_a_failed_leg_and_a_stuck_one():
    """guarded_decode_legs: a leg that raises is replaced by its error and the next one still runs; a leg that
    never returns (ranks out of step in a collective) is given up after the deadline with the finished legs kept,
    and the give-up hook is not called when every leg returns in time."""
    import threading
    import time
    gave_up = []

    def leg_ok(B):
        if B == 16:
            raise RuntimeError("boom")
        return {"tok_s": 500.0, "batch": B}

    d = bench.guarded_decode_legs(leg_ok, (1, 16), 5.0, gave_up.append, None)
    assert d["batch1"]["tok_s"] == 500.0 and "RuntimeError: boom" in d["batch16"]["error"]
    assert d["tok_s"] == 500.0 and d["unit"] == "tok/s" and d["scaling"] == "strong" and gave_up == []

    release = threading.Event()

    def leg_stuck(B):
        if B == 16:
            release.wait(10.0)          # stands for a collective that never completes
        return {"tok_s": 100.0 * B, "batch": B}

    t0 = time.perf_counter()
    seen = []

    def hook(partial):
        seen.append(partial)
        release.set()                   # (the bench leaves the process here)

    d = bench.guarded_decode_legs(leg_stuck, (1, 16), 0.3, hook, None)
    assert time.perf_counter() - t0 < 5.0
    assert len(seen) == 1 and seen[0]["batch1"]["tok_s"] == 100.0 and "not finished" in seen[0]["batch16"]["error"]
    assert seen[0]["tok_s"] == 100.0
    assert "batch16" not in d          # the late leg's result is dropped: the line has been printed without it
    json.dumps(seen[0])
