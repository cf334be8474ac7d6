"""CPU tests of the Python operator layer's host logic (argument checks, table loading).  The
compute paths need the GPU and are covered by the gpu-marked parity tests."""
import numpy as np
import pytest
import torch

import approx_ops
import self_ops
from self_ops.ops_py import approx_ops as py_ops


def test_public_api_names_match_the_reference():
    for name in ("init_lookup_tables", "approx_gemm_op", "approx_gemm_baseline_op", "approx_conv2d_op",
                 "approx_conv2d_baseline_op"):
        assert callable(getattr(self_ops, name))
    for name in ("approx_gemm_forward", "approx_gemm_backward", "acc_gemm_forward_fp32"):
        assert callable(getattr(approx_ops, name))


def test_cpu_tensors_are_rejected_like_check_input():
    a = torch.zeros(4, 4, dtype=torch.uint8)
    c = torch.zeros(4, 4, dtype=torch.uint32)
    lut = torch.zeros(17408, dtype=torch.uint16)
    with pytest.raises(RuntimeError, match="must be a CUDAtensor"):
        approx_ops.approx_gemm_forward(a, a, c, lut)
    g = torch.zeros(4, 4)
    l16 = torch.zeros(17408, dtype=torch.int16)
    with pytest.raises(RuntimeError, match="must be a CUDAtensor"):
        approx_ops.approx_gemm_backward(g, a, a, g.clone(), g.clone(), l16, l16)


def test_set_lookup_tables_packs_the_wire_format(golden):
    bits = int(golden["bits"])
    from oracle import oracle_np as O
    fp, ga, gb = (O.unpack_padded(golden[k], bits) for k in ("lut_fp", "lut_ga", "lut_gb"))
    self_ops.set_lookup_tables("cpu", fp, ga, gb, bits)
    assert np.array_equal(py_ops.lut_appmult.numpy(), golden["lut_fp"])
    assert np.array_equal(py_ops.lut_grad_a.numpy(), golden["lut_ga"])
    assert np.array_equal(py_ops.lut_grad_b.numpy(), golden["lut_gb"])
    assert py_ops.lut_appmult.dtype == torch.uint16 and py_ops.lut_grad_a.dtype == torch.int16


def test_parse_lut_file_round_trip(tmp_path, golden):
    bits = int(golden["bits"])
    if bits == 8:
        pytest.skip("the 6- and 7-bit tables cover the parser; the 8-bit text is large")
    from oracle import oracle_np as O
    tabs = [O.unpack_padded(golden[k], bits) for k in ("lut_fp", "lut_ga", "lut_gb")]
    titles = ["LUT for approximate multiplier:",
              "LUT for the gradient of the approximate multiplier w.r.t. the first operand:",
              "LUT for the gradient of the approximate multiplier w.r.t. the second operand:"]
    q = 1 << bits
    path = tmp_path / "lut.txt"
    with open(path, "w") as f:
        f.write("INFO: header line that must be skipped\nINFO: another 1 2 3\n")
        for title, t in zip(titles, tabs):
            f.write(title + "\n")
            for a in range(q):
                f.write("".join(f"{a} {b} {int(t[a, b])}\n" for b in range(q)))
    self_ops.init_lookup_tables("cpu", str(path), bits)
    assert np.array_equal(py_ops.lut_appmult.numpy(), golden["lut_fp"])
    assert np.array_equal(py_ops.lut_grad_b.numpy(), golden["lut_gb"])
    got = O.parse_lut_file(str(path), bits)
    assert all(np.array_equal(x, y) for x, y in zip(got, tabs))


def test_unsupported_bit_width():
    with pytest.raises(NotImplementedError):
        self_ops.set_lookup_tables("cpu", np.zeros((32, 32)), np.zeros((32, 32)), np.zeros((32, 32)), 5)


def test_conv_op_rejects_bias_and_groups():
    x = torch.zeros(1, 2, 4, 4)
    w = torch.zeros(3, 2, 3, 3)
    with pytest.raises(AssertionError):
        self_ops.approx_conv2d_op(x, w, bias=torch.zeros(3), stride=(1, 1), padding=(1, 1), dilation=(1, 1), groups=1)
    with pytest.raises(AssertionError):
        self_ops.approx_conv2d_op(x, w, bias=None, stride=(1, 1), padding=(1, 1), dilation=(1, 1), groups=2)


def test_bench_reads_dram_traffic_from_the_committed_capture_summary():
    """bench.py's roofline.traffic is parsed from the ncu summary under profiles/, only for the captured workload."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    for kernel in ("forward", "grad_w", "grad_a"):
        nbytes, source = bench.ncu_dram_traffic(kernel, (8, 4096, 4096))
        assert nbytes is not None and 50e6 < nbytes < 2e9, kernel
        assert "profiles/" in source
    assert bench.ncu_dram_traffic("forward", (7, 4096, 4096)) == (None, None)
    assert bench.ncu_dram_traffic("no such kernel", (8, 4096, 4096)) == (None, None)
