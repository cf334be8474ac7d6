"""CPU tests of the host-side pieces of the layer path: the window sums that stand in for the zero-point
cross-term convolutions, and the table construction for sign-magnitude operands."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle_np as O

GEOMS = [(8, 8, 3, 3, 1, 1, 1), (9, 7, 3, 3, 2, 1, 1), (6, 6, 1, 1, 2, 0, 1), (10, 10, 3, 3, 1, 2, 2), (12, 12, 5, 5, 2, 2, 1)]


@pytest.mark.parametrize("geom", GEOMS)
def test_window_sums_equal_the_ones_kernel_convolutions(geom):
    from lutgemm_layers import _out_hw, _valid_taps, _window_sum, _window_sum_adjoint
    H, W, kh, kw, stride, pad, dil = geom
    torch.manual_seed(0)
    img = torch.randint(0, 500, (3, H, W)).float()
    ones_k = torch.ones(1, 1, kh, kw)
    want = F.conv2d(img.unsqueeze(1), ones_k, stride=stride, padding=pad, dilation=dil)[:, 0]
    got = _window_sum(img, geom)
    assert torch.equal(got, want)
    Ho, Wo = _out_hw(H, W, kh, kw, stride, pad, dil)
    assert got.shape == (3, Ho, Wo)
    # adjoint: <window_sum(x), g> == <x, adjoint(g)>
    g = torch.randint(-50, 50, (3, Ho, Wo)).float()
    adj = _window_sum_adjoint(g, geom)
    assert adj.shape == img.shape
    assert float((got * g).sum()) == float((img * adj).sum())
    valid = _valid_taps(geom, torch.device("cpu"))
    taps = F.conv2d(torch.ones(1, 1, H, W), ones_k, stride=stride, padding=pad, dilation=dil).reshape(-1)
    assert valid.shape == (kh * kw, Ho * Wo) and torch.equal(valid.sum(dim=0), taps)


def test_signed_tables_follow_the_sign_magnitude_definition():
    from lutgemm_signed import signed_dense_tables
    bits = 5
    q = 1 << bits
    fp, ga, gb = O.synthetic_tables(bits, seed=2)
    fp_s, ga_s, gb_s, offset = signed_dense_tables(fp, ga, gb)
    assert fp_s.shape == (2 * q, 2 * q) and fp_s.min() >= 0 and offset == fp.max()
    rng = np.random.default_rng(0)
    for _ in range(200):
        a, w = rng.integers(0, q, 2)
        na, nw = rng.integers(0, 2, 2)
        sa, sw = 1 - 2 * na, 1 - 2 * nw
        ca, cw = a | (na << bits), w | (nw << bits)
        assert fp_s[ca, cw] - offset == sa * sw * fp[a, w]
        assert ga_s[ca, cw] == sw * round(ga[a, w] * 16)
        assert gb_s[ca, cw] == sa * round(gb[a, w] * 16)


def test_config0_on_the_cpu_oracle():
    """Benchmark configuration 0 (7-bit magnitudes with sign bits, M=256, K=512, N=256) evaluated on the CPU: the
    signed tables through the C oracle's 8-bit unsigned forward equal the direct signed sum."""
    from lutgemm_signed import signed_dense_tables
    from oracle.oracle_c import OracleC
    bits, M, K, N = 7, 256, 512, 256
    q = 1 << bits
    fp, ga, gb = O.synthetic_tables(bits, seed=0, half_window=8)
    fp_s, ga_s, gb_s, offset = signed_dense_tables(fp, ga, gb)
    rng = np.random.default_rng(0)
    a_mag, w_mag = rng.integers(0, q, (M, K)), rng.integers(0, q, (K, N))
    a_neg, w_neg = rng.random((M, K)) < 0.5, rng.random((K, N)) < 0.5
    a_codes = (a_mag | (a_neg.astype(np.int64) << bits)).astype(np.uint8)
    w_codes = (w_mag | (w_neg.astype(np.int64) << bits)).astype(np.uint8)
    lf = O.pack_padded(fp_s, bits + 1, np.uint16)
    c = OracleC().forward(a_codes, w_codes, lf, bits + 1).astype(np.int64) - K * offset
    sa, sw = np.where(a_neg, -1, 1).astype(np.int64), np.where(w_neg, -1, 1).astype(np.int64)
    want = np.zeros((M, N), np.int64)
    for k in range(K):
        want += (sa[:, k, None] * sw[None, k, :]) * fp[a_mag[:, k, None], w_mag[None, k, :]]
    assert np.array_equal(c, want)
    out = c * (0.05 * 0.01)  # the configuration's activation and weight scales
    assert np.isfinite(out).all()
