"""CPU tests: the oracle (C restatement and NumPy restatement) against the fixtures generated from
the reference's own Python layer, and the table tools against the reference's checked-in tables."""
import numpy as np
import pytest

from oracle import oracle_np as O

N_GEMM, N_CONV = 7, 4


def test_geometry_matches_wire_format(oracle_c):
    assert [O.geometry(b)[2] for b in (4, 6, 7, 8)] == [1024, 5120, 17408, 66306]
    assert [oracle_c.lut_elem_num(b) for b in (4, 6, 7, 8)] == [1024, 5120, 17408, 66306]
    assert oracle_c.lut_elem_num(5) == -1
    with pytest.raises(NotImplementedError):
        O.geometry(5)


def test_oracle_forward_bit_exact_vs_golden(golden, oracle_c):
    bits = int(golden["bits"])
    for i in range(N_GEMM):
        a, b = golden[f"gemm{i}_a"], golden[f"gemm{i}_b"]
        want = golden[f"gemm{i}_c"]
        got_c = oracle_c.forward(a, b, golden["lut_fp"], bits)
        got_np = O.forward_np(a, b, golden["lut_fp"], bits)
        assert np.array_equal(got_c, got_np)
        # the reference hands back uint32 sums converted to fp32 (round to nearest)
        assert np.array_equal(got_c.astype(np.float32), want)


def test_oracle_backward_vs_golden(golden, oracle_c):
    """fp32, tolerance 1e-5 relative to the largest gradient magnitude (the golden values come from a
    pairwise PyTorch sum, the oracle from the reference's sequential FMA order)."""
    bits = int(golden["bits"])
    for i in range(N_GEMM):
        a, b, gc = golden[f"gemm{i}_a"], golden[f"gemm{i}_b"], golden[f"gemm{i}_gc"]
        ga, gw = oracle_c.backward(gc, a, b, golden["lut_ga"], golden["lut_gb"], bits)
        for got, want in ((ga, golden[f"gemm{i}_ga"]), (gw, golden[f"gemm{i}_gb"])):
            scale = max(np.abs(want).max(), 1e-30)
            assert np.abs(got - want).max() / scale <= 1e-5
        r64 = O.backward_np_f64(gc, a, b, golden["lut_ga"], golden["lut_gb"], bits)
        c64 = oracle_c.backward_f64(gc, a, b, golden["lut_ga"], golden["lut_gb"], bits)
        for x, y in zip(r64, c64):
            assert np.allclose(x, y, rtol=1e-12, atol=1e-9)
        # every fp32 element is within 1e-5 of the sum of its absolute terms
        assert (np.abs(ga - r64[0]) <= 1e-5 * r64[2] + 1e-30).all()
        assert (np.abs(gw - r64[1]) <= 1e-5 * r64[3] + 1e-30).all()


def test_oracle_conv_vs_golden(golden, oracle_c):
    bits = int(golden["bits"])
    for i in range(N_CONV):
        B, Cin, H, W, Cout, k, s, p, d = [int(v) for v in golden[f"conv{i}_cfg"]]
        x, wt, gy = golden[f"conv{i}_x"], golden[f"conv{i}_w"], golden[f"conv{i}_gy"]
        col = oracle_c.im2col(x, k, k, s, p, d)
        assert np.array_equal(col, O.im2col_codes(x, k, k, s, p, d))
        wmat = np.ascontiguousarray(wt.reshape(Cout, -1).T)
        c = oracle_c.forward(col, wmat, golden["lut_fp"], bits)
        Ho, Wo = golden[f"conv{i}_y"].shape[2:]
        y = c.astype(np.float32).reshape(B, Ho * Wo, Cout).transpose(0, 2, 1).reshape(B, Cout, Ho, Wo)
        assert np.array_equal(y, golden[f"conv{i}_y"])
        gcm = np.ascontiguousarray(gy.reshape(B, Cout, Ho * Wo).transpose(0, 2, 1).reshape(B * Ho * Wo, Cout))
        gcol, gwm = oracle_c.backward(gcm, col, wmat, golden["lut_ga"], golden["lut_gb"], bits)
        gx = oracle_c.col2im(gcol, x.shape, k, k, s, p, d)
        gx64 = O.col2im_f64(gcol, x.shape, k, k, s, p, d)
        gwt = gwm.T.reshape(Cout, Cin, k, k)
        for got, want in ((gx, golden[f"conv{i}_gx"]), (gx64, golden[f"conv{i}_gx"]), (gwt, golden[f"conv{i}_gw"])):
            assert np.abs(got - want).max() / max(np.abs(want).max(), 1e-30) <= 1e-5


def test_reference_gradient_rule_reproduces_checked_in_tables():
    """The restated smoothing/central-difference rule, applied to the forward section of the
    reference's tables, must reproduce their two gradient sections entry for entry."""
    from tests.conftest import load_golden
    for name, half_ws in (("mult7_med63", 8), ("mul8u_17C8", 16), ("trunc6", 2)):
        g = load_golden(name)
        bits = int(g["bits"])
        fp = O.unpack_padded(g["lut_fp"], bits).astype(np.int64)
        qa, qb = O.reference_gradient_tables(fp, half_ws)
        assert np.array_equal(qa, O.unpack_padded(g["lut_ga"], bits))
        assert np.array_equal(qb, O.unpack_padded(g["lut_gb"], bits))


def test_padded_tables_have_zero_null_code(golden):
    bits = int(golden["bits"])
    row, col, elems = O.geometry(bits)
    q = 1 << bits
    for key in ("lut_fp", "lut_ga", "lut_gb"):
        flat = golden[key]
        assert flat.shape == (elems,)
        t = flat[: row * col].reshape(row, col)
        assert not t[q:, :].any() and not t[:, q:].any() and not flat[row * col:].any()
        assert np.array_equal(O.pack_padded(O.unpack_padded(flat, bits), bits, flat.dtype), flat)


def test_synthetic_tables_follow_the_benchmark_definition():
    fp, ga, gb = O.synthetic_tables(7, seed=0)
    x = np.arange(128)
    e = fp - x[:, None] * x[None, :]
    nz = fp > 0
    assert e[nz].min() >= -64 and e[nz].max() <= 64 and fp.min() >= 0
    assert np.isclose(ga[20, 5], (fp[28, 5] - fp[12, 5]) / 16) and np.isclose(ga[2, 9], (fp[10, 9] - fp[0, 9]) / 10)
    assert np.isclose(gb[7, 127], (fp[7, 127] - fp[7, 119]) / 8)
    lf, la, lb = O.to_wire(fp, ga, gb, 7)
    assert lf.dtype == np.uint16 and la.dtype == np.int16 and lf.shape == (17408,)
    fp8, ga8, gb8 = O.synthetic_tables(8, seed=0)
    assert fp8.max() < 65536
    O.to_wire(fp8, ga8, gb8, 8)
