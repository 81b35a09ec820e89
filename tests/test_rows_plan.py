"""Launch geometry of the many-row matvec, checked on the CPU through skn_rows_plan_query (the library's own
planning and per-CTA group arithmetic, no device): for the projections of the 32-layer decoder and of its
tensor-parallel shards (1, 2, 4, 8 ranks), for odd sizes, and for a sweep of group counts, no CTA is left
without a group, no CTA owns more groups than its partial-sum space holds, and the shared memory fits.

Why it exists: the gate / up shard of an 8-way decoder (224 groups for 148 CTAs) once left every third CTA
without a group after the SwiGLU form's rounding to whole pairs, and such a CTA sat out a two-second bounded wait
in every launch."""
import ctypes

import pytest

from skainet_b200 import _ffi

Q4_K, Q8_0, Q4_0 = 12, 8, 2


def query(sm, qt, groups, K, na, swiglu):
    out = (ctypes.c_int64 * 8)()
    rc = _ffi.lib().skn_rows_plan_query(sm, qt, groups, K, na, 1 if swiglu else 0, out)
    assert rc == 0
    return dict(zip(("ok", "grid", "most", "room", "empty", "chunks", "stages", "smem"), list(out)))


def check(p, groups):
    assert p["empty"] == 0, p
    assert 1 <= p["most"] <= p["room"], p
    assert p["grid"] * p["most"] >= groups, p
    assert p["stages"] >= 2 and p["smem"] <= 220 * 1024, p


@pytest.mark.parametrize("ranks", [1, 2, 4, 8])
@pytest.mark.parametrize("na", [3, 4, 5, 8, 16])
def test_decoder_projections_and_their_shards(ranks, na):
    d, F = 4096, 14336
    qd, kd = 4096 // ranks, 1024 // ranks
    shapes = [((qd + 2 * kd) // 16, d, False), (d // 16, d // ranks, False), (2 * (F // ranks) // 16, d, True),
              (d // 16, F // ranks, False)]
    covered = 0
    for groups, K, swiglu in shapes:
        p = query(148, Q4_K, groups, K, na, swiglu)
        if p["ok"]:
            covered += 1
            check(p, groups)
    assert covered >= 3          # (the unsharded gate / up pair is the four-rows-per-launch path's)


@pytest.mark.parametrize("qt", [Q4_K, Q8_0, Q4_0])
@pytest.mark.parametrize("swiglu", [False, True])
def test_sweep_of_group_counts(qt, swiglu):
    for sm in (148, 132, 16):
        for K in (512, 768, 1792, 4096, 14336):
            for na in (3, 7, 16):
                for groups in list(range(2, 40, 2)) + [100, 148, 150, 224, 296, 298, 448, 1000, 1184]:
                    p = query(sm, qt, groups, K, na, swiglu)
                    if p["ok"]:
                        check(p, groups)


def test_the_eight_way_gate_up_shard_gets_one_cta_per_pair():
    p = query(148, Q4_K, 224, 4096, 16, True)
    assert p["ok"] and p["grid"] == 112 and p["most"] == 2 and p["empty"] == 0


def test_uncovered_shapes_and_bad_arguments():
    assert query(148, 14, 64, 4096, 4, False)["ok"] == 0          # Q6_K is not on this kernel
    assert query(148, Q4_K, 64, 256, 4, False)["ok"] == 0         # a single super-block per row
    assert query(148, Q4_K, 64, 4100, 4, False)["ok"] == 0        # not whole super-blocks
    out = (ctypes.c_int64 * 8)()
    assert _ffi.lib().skn_rows_plan_query(0, Q4_K, 64, 4096, 4, 0, out) != 0
    assert _ffi.lib().skn_rows_plan_query(148, Q4_K, 64, 4096, 17, 0, out) != 0
    assert _ffi.lib().skn_rows_plan_query(148, Q4_K, 64, 4096, 4, 0, None) != 0
