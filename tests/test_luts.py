"""CPU tests of the table generators and the LUT file writer (lutgemm_luts) against the reference's
checked-in tables (through the golden fixtures) and against the oracle's restatement."""
import numpy as np

import lutgemm_luts as LU
import self_ops
from oracle import oracle_np as O
from self_ops.ops_py import approx_ops as py_ops
from tests.conftest import load_golden


def test_smoothed_difference_rule_reproduces_the_reference_tables():
    for name, hws in (("mult7_med63", 8), ("mul8u_17C8", 16), ("trunc6", 2)):
        g = load_golden(name)
        bits = int(g["bits"])
        fp = O.unpack_padded(g["lut_fp"], bits).astype(np.int64)
        ga, gb = LU.smoothed_difference_gradients(fp, hws)
        assert np.array_equal(ga, O.unpack_padded(g["lut_ga"], bits))
        assert np.array_equal(gb, O.unpack_padded(g["lut_gb"], bits))


def test_window_rule_and_synthetic_multiplier_match_the_oracle():
    for bits in (4, 6, 7, 8):
        fp = LU.synthetic_multiplier(bits, seed=3)
        o_fp, o_ga, o_gb = O.synthetic_tables(bits, seed=3)
        assert np.array_equal(fp, o_fp)
        ga, gb = LU.window_difference_gradients(fp, max(1, (1 << bits) // 16))
        assert np.array_equal(ga, np.round(o_ga * 16).astype(np.int64))
        assert np.array_equal(gb, np.round(o_gb * 16).astype(np.int64))


def test_written_file_loads_back_identically(tmp_path):
    bits = 6
    fp = LU.synthetic_multiplier(bits, seed=1)
    ga, gb = LU.smoothed_difference_gradients(fp, 2)
    path = tmp_path / "synthetic_6_6_lutfp+bp.txt"
    LU.write_lut_file(str(path), fp, ga, gb, header="test")
    self_ops.init_lookup_tables("cpu", str(path), bits)
    assert np.array_equal(py_ops.lut_appmult.numpy(), O.pack_padded(fp, bits, np.uint16))
    assert np.array_equal(py_ops.lut_grad_a.numpy(), O.pack_padded(ga, bits, np.int16))
    assert np.array_equal(py_ops.lut_grad_b.numpy(), O.pack_padded(gb, bits, np.int16))
    got = O.parse_lut_file(str(path), bits)
    assert all(np.array_equal(x, y) for x, y in zip(got, (fp, ga, gb)))


def test_error_metrics_match_the_reference_header():
    g = load_golden("mult7_med63")
    m = LU.error_metrics(O.unpack_padded(g["lut_fp"], 7))
    assert abs(m["med"] - 63.5938720703125) < 1e-9 and abs(m["mse"] - 9228.21875) < 1e-6 and m["max_ed"] == 713.0


def test_load_lut_file_parses_caches_and_checks_the_header(tmp_path):
    import lutgemm_luts as L
    bits = 6
    fp = L.synthetic_multiplier(bits, seed=5)
    ga, gb = L.window_difference_gradients(fp, 4)
    path = str(tmp_path / "lut.txt")
    L.write_lut_file(path, fp, ga, gb)
    t1 = L.load_lut_file(path, bits)
    assert all(np.array_equal(x, y) for x, y in zip(t1, (fp, ga, gb)))
    import os
    assert os.path.exists(path + f".b{bits}.npz")
    t2 = L.load_lut_file(path, bits)  # from the cache
    assert all(np.array_equal(x, y) for x, y in zip(t2, (fp, ga, gb)))
    # a header that does not match the table is refused
    text = open(path).read().replace("Mean error distance between lut_appmult and lut_mult: ", "Mean error distance between lut_appmult and lut_mult: 9")
    bad = str(tmp_path / "bad.txt")
    open(bad, "w").write(text)
    import pytest
    with pytest.raises(ValueError, match="does not match"):
        L.load_lut_file(bad, bits, cache=False)
