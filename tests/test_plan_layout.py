"""Host-side arithmetic of the compact plan: the closed-form range offsets match a running sum."""
from minference_b200 import _cabi


def rng_index(m, cap_s):      # mirror of plan_rng_index in csrc/plan_layout.h
    k = m if m < cap_s - 1 else max(cap_s - 1, 0)
    return k * (k - 1) // 2 + 2 * k + (m - k) * cap_s


def test_range_offsets_are_prefix_sums_of_capacities():
    for cap_s in (1, 2, 3, 50, 100, 6096):
        run = 0
        for m in range(0, 300):
            assert rng_index(m, cap_s) == run, (cap_s, m)
            run += min(cap_s, m + 2)


def test_plan_bytes_monotone(built_lib):
    lib = _cabi.lib()
    a = lib.minf_plan_bytes(1, 1, 8192, 1000, 6096)
    b = lib.minf_plan_bytes(1, 2, 8192, 1000, 6096)
    c = lib.minf_plan_bytes(1, 1, 16384, 1000, 6096)
    assert b == 2 * a and c > a
    rows = 8192 // 64
    need = rows * 4 + rows * ((1000 + 31) // 32) * 4 + rng_index(rows, 6096) * 8
    assert a >= need and a < need + 1024
