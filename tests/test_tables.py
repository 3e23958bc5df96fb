"""The TQ4 format tables (warp34_b200/csrc/tq4_tables.h).

The reference ships them as generated constants (crates/warp34-kernels/csrc/tq/tq4_codebook.cuh:
46-101) and states how they were made: Lloyd-Max centroids on the coordinate density of a
uniformly random unit vector in R^256, boundaries = adjacent mid-points, a fixed +-1 diagonal.
These tests check the stored numbers against that definition, independently of the reference
file."""
import numpy as np
from scipy import integrate


def _tables(oracle_lib):
    L = oracle_lib.lib()
    c = np.array([L.w34o_centroid(i) for i in range(16)], np.float32)
    b = np.array([L.w34o_boundary(i) for i in range(15)], np.float32)
    s = np.array([L.w34o_sign(i) for i in range(256)], np.float32)
    return c, b, s


def test_symmetry_order_and_midpoints(oracle_lib):
    c, b, s = _tables(oracle_lib)
    assert (np.diff(c) > 0).all() and (np.diff(b) > 0).all()
    assert (c == -c[::-1]).all() and (b == -b[::-1]).all() and b[7] == 0.0
    mid = ((c[1:].astype(np.float64) + c[:-1]) / 2)
    assert np.abs(mid - b).max() < 1e-8
    assert set(np.unique(s)) == {-1.0, 1.0}
    assert 96 <= int((s < 0).sum()) <= 160


def test_centroids_are_a_lloyd_max_fixed_point_of_the_sphere_coordinate_density(oracle_lib):
    c, b, _ = _tables(oracle_lib)
    d = 256
    a = (d - 3) / 2.0
    edges = np.concatenate([[-1.0], b.astype(np.float64), [1.0]])
    for i in range(16):
        num = integrate.quad(lambda x: x * (1 - x * x) ** a, edges[i], edges[i + 1], epsabs=0, epsrel=1e-12)[0]
        den = integrate.quad(lambda x: (1 - x * x) ** a, edges[i], edges[i + 1], epsabs=0, epsrel=1e-12)[0]
        assert abs(num / den - c[i]) <= 2e-6 * abs(c[i]) + 1e-9, (i, num / den, c[i])
    # unit-vector scaling: the quantiser's mean squared output is close to 1/d
    probs = [integrate.quad(lambda x: (1 - x * x) ** a, edges[i], edges[i + 1])[0] for i in range(16)]
    probs = np.array(probs) / sum(probs)
    assert abs((probs * c.astype(np.float64) ** 2).sum() * d - (1 - 0.009408)) < 2e-3
