"""Writes tests/golden/known_answers.npz.

The reference holds no golden vectors for this path and cannot be run here, so these are
closed-form known answers (written down independently of the oracle's code) plus the first
draws of the counter-based generator (a regression pin for the synthetic inputs).
Run:  python tests/golden/make_golden.py
"""
from pathlib import Path

import numpy as np

out = {}
# sum(1:n) = n(n+1)/2, cumsum(ones)[i] = i, alternating +-1 scan, Int32 wrap-around
n = 100_000
out["iota_n"] = np.int64(n)
out["iota_sum"] = np.int64(n * (n + 1) // 2)
out["alt_scan_first8"] = np.array([1, 0, 1, 0, 1, 0, 1, 0], dtype=np.int32)
out["wrap_in"] = np.array([2**31 - 1, 1, 1], dtype=np.int32)
out["wrap_scan"] = np.array([2**31 - 1, -2**31, -2**31 + 1], dtype=np.int32)
# exact Float32 sums: 2^-k patterns
out["pow2_in"] = np.array([0.5, 0.25, 0.125, 0.0625, 1.0, 2.0, 4.0, 8.0], dtype=np.float32)
out["pow2_sum"] = np.float32(15.9375)
out["pow2_scan"] = np.array([0.5, 0.75, 0.875, 0.9375, 1.9375, 3.9375, 7.9375, 15.9375], dtype=np.float32)
# isless ordering: -Inf < -1 < -0.0 < +0.0 < 3 < Inf < NaN; stable among the two +0.0
x = np.array([3.0, -0.0, 0.0, np.nan, -1.0, np.inf, -np.inf, 0.0], dtype=np.float32)
out["order_in"] = x
out["order_sorted"] = np.array([-np.inf, -1.0, -0.0, 0.0, 0.0, 3.0, np.inf, np.nan], dtype=np.float32)
out["order_perm"] = np.array([7, 5, 2, 3, 8, 1, 6, 4], dtype=np.int64)
out["order_perm_rev"] = np.array([4, 6, 1, 3, 8, 2, 5, 7], dtype=np.int64)
# max/min semantics of Base: NaN propagates, max(-0.0, 0.0) = 0.0, min(-0.0, 0.0) = -0.0
out["mm_a"] = np.array([1.0, np.nan, -0.0, 0.0, 2.0], dtype=np.float32)
out["mm_b"] = np.array([2.0, 1.0, 0.0, -0.0, np.nan], dtype=np.float32)
out["mm_max"] = np.array([2.0, np.nan, 0.0, 0.0, np.nan], dtype=np.float32)
out["mm_min"] = np.array([1.0, np.nan, -0.0, -0.0, np.nan], dtype=np.float32)
# a .* x .+ y rounds twice: pick values where fused and unfused differ
a = np.float32(1.0 + 2.0**-12)
xx = np.array([1.0 + 2.0**-12], dtype=np.float32)
yy = np.array([-1.0], dtype=np.float32)
out["axpy_a"], out["axpy_x"], out["axpy_y"] = a, xx, yy
out["axpy_unfused"] = (np.float32(a * xx[0]) + yy[0]).astype(np.float32).reshape(1)
# 3x4 matrix reductions (column-major semantics checked by hand)
A = np.arange(1, 13, dtype=np.float32).reshape(3, 4, order="F")
out["mat"] = A
out["mat_sum_dims1"] = np.array([[6.0, 15.0, 24.0, 33.0]], dtype=np.float32)
out["mat_max_dims2"] = np.array([[10.0], [11.0], [12.0]], dtype=np.float32)
out["mat_sumsq"] = np.float32(650.0)
# generator pin (splitmix64 stream keyed by seed and stream id)
import sys
sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import __graft_entry__ as entry
rnd = entry.load_package().random
out["draws_seed0_stream0"] = rnd.host_draw(0, 0, 0, 8)
out["draws_seed3_stream1_at1000"] = rnd.host_draw(3, 1, 1000, 4)
np.savez(Path(__file__).with_name("known_answers.npz"), **out)
print("wrote", len(out), "entries")
