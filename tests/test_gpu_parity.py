"""GPU parity tests (run with -m gpu on the B200 box): the CUDA path, called through the C-ABI via the
`approx_ops` module, against the CPU oracle and the committed golden fixtures.

Forward: bit-exact uint32.  Backward: fp32, tolerance 1e-5 - per element |got - f64| must not exceed
1e-5 times the sum of the element's absolute terms (the natural scale of an fp32 sum in any order),
and the max error relative to the largest gradient magnitude must not exceed 1e-5."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle_np as O

pytestmark = pytest.mark.gpu

TOL = 1e-5


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test started without a CUDA device")
    import approx_ops
    approx_ops.library()  # raises if liblutgemm_b200.so is missing: there is no fallback to test
    return torch.device("cuda:0")


def run_forward(dev, a, w, lut):
    import approx_ops
    at, wt = torch.from_numpy(a).to(dev), torch.from_numpy(w).to(dev)
    c = torch.full((a.shape[0], w.shape[1]), 0xDEADBEEF, dtype=torch.uint32, device=dev)
    approx_ops.approx_gemm_forward(at, wt, c, torch.from_numpy(lut).to(dev))
    torch.cuda.synchronize()
    return c.cpu().numpy()


def run_backward(dev, gc, a, w, lut_ga, lut_gw):
    import approx_ops
    ga = torch.full(a.shape, float("nan"), dtype=torch.float32, device=dev)
    gw = torch.full(w.shape, float("nan"), dtype=torch.float32, device=dev)
    approx_ops.approx_gemm_backward(torch.from_numpy(gc).to(dev), torch.from_numpy(a).to(dev),
                                    torch.from_numpy(w).to(dev), ga, gw, torch.from_numpy(lut_ga).to(dev),
                                    torch.from_numpy(lut_gw).to(dev))
    torch.cuda.synchronize()
    return ga.cpu().numpy(), gw.cpu().numpy()


def check_backward(oracle_c, gc, a, w, lga, lgw, bits, ga, gw):
    r_ga, r_gw, r_gaa, r_gwa = oracle_c.backward_f64(gc, a, w, lga, lgw, bits)
    for got, ref, refabs in ((ga, r_ga, r_gaa), (gw, r_gw, r_gwa)):
        assert np.isfinite(got).all()
        assert (np.abs(got - ref) <= TOL * refabs + 1e-30).all()
        assert np.abs(got - ref).max() <= TOL * max(np.abs(ref).max(), 1e-30)


def synth_wire(bits, seed=0):
    return O.to_wire(*O.synthetic_tables(bits, seed=seed), bits)


def rand_problem(bits, M, K, N, seed):
    rng = np.random.default_rng(seed)
    q = 1 << bits
    a = rng.integers(0, q, (M, K), dtype=np.uint8) if bits < 8 else rng.integers(0, 256, (M, K)).astype(np.uint8)
    w = rng.integers(0, q, (K, N), dtype=np.uint8) if bits < 8 else rng.integers(0, 256, (K, N)).astype(np.uint8)
    gc = rng.standard_normal((M, N)).astype(np.float32)
    return a, w, gc


# ---------------------------------------------------------------------------------------------
def test_golden_gemm(dev, golden, oracle_c):
    bits = int(golden["bits"])
    for i in range(7):
        a, w, gc = golden[f"gemm{i}_a"], golden[f"gemm{i}_b"], golden[f"gemm{i}_gc"]
        c = run_forward(dev, a, w, golden["lut_fp"])
        assert np.array_equal(c.astype(np.float32), golden[f"gemm{i}_c"])
        assert np.array_equal(c, oracle_c.forward(a, w, golden["lut_fp"], bits))
        ga, gw = run_backward(dev, gc, a, w, golden["lut_ga"], golden["lut_gb"])
        check_backward(oracle_c, gc, a, w, golden["lut_ga"], golden["lut_gb"], bits, ga, gw)
        for got, want in ((ga, golden[f"gemm{i}_ga"]), (gw, golden[f"gemm{i}_gb"])):
            assert np.abs(got - want).max() <= TOL * max(np.abs(want).max(), 1e-30)


RAGGED = [(1, 1, 1), (2, 3, 5), (5, 127, 3), (127, 129, 65), (129, 31, 127), (64, 512, 256), (256, 512, 256),
          (300, 27, 64), (77, 576, 64), (33, 1152, 128), (50, 200, 300), (513, 16, 10), (16, 2304, 257),
          (700, 45, 70), (1025, 130, 33), (512, 16, 64), (2100, 300, 200), (1536, 17, 96),
          (100, 50, 600), (70, 33, 1030), (513, 20, 512), (1100, 40, 1100)]


@pytest.mark.parametrize("bits", [4, 6, 7, 8])
def test_ragged_shapes_all_bit_widths(dev, oracle_c, bits):
    lf, la, lw = synth_wire(bits, seed=bits)
    for s, (M, K, N) in enumerate(RAGGED):
        a, w, gc = rand_problem(bits, M, K, N, seed=100 * bits + s)
        c = run_forward(dev, a, w, lf)
        assert np.array_equal(c, oracle_c.forward(a, w, lf, bits)), (bits, M, K, N)
        ga, gw = run_backward(dev, gc, a, w, la, lw)
        check_backward(oracle_c, gc, a, w, la, lw, bits, ga, gw)


@pytest.fixture
def kernel_choice():
    """approx_ops.set_kernel_choice for the duration of one test; the automatic choice is restored afterwards."""
    import approx_ops
    yield approx_ops.set_kernel_choice
    approx_ops.set_kernel_choice()


@pytest.mark.parametrize("kernel", ["rowbcast", "slab"])
@pytest.mark.parametrize("bits", [4, 6, 7, 8])
def test_each_forward_kernel_on_every_shape_class(dev, oracle_c, bits, kernel, kernel_choice):
    """Every forward kernel (selected through lutgemm_set_kernel_choice) must be bit-exact on shapes the
    dispatcher would normally send to another one, including tiles that are almost empty."""
    kernel_choice(forward=kernel)
    lf, _, _ = synth_wire(bits, seed=10 + bits)
    for s, (M, K, N) in enumerate([(1, 1, 1), (5, 33, 3), (130, 16, 64), (515, 31, 67), (1024, 48, 128), (600, 257, 65)]):
        a, w, _ = rand_problem(bits, M, K, N, seed=7 * bits + s)
        assert np.array_equal(run_forward(dev, a, w, lf), oracle_c.forward(a, w, lf, bits)), (kernel, bits, M, K, N)


@pytest.mark.parametrize("kernel", ["bcast", "slab-wide", "slab-tall"])
@pytest.mark.parametrize("bits", [4, 6, 7, 8])
def test_each_backward_kernel_on_every_shape_class(dev, oracle_c, bits, kernel, kernel_choice):
    """Every family of gradient kernels (selected through lutgemm_set_kernel_choice: fp32 slab with the
    512 x 64 and the 1024 x 32 tile, broadcast) on shapes of either class."""
    kernel_choice(backward=kernel.split("-")[0], grad_tile="tall" if kernel.endswith("-tall") else "wide")
    _, la, lw = synth_wire(bits, seed=20 + bits)
    shapes = [(1, 1, 1), (5, 33, 3), (130, 16, 64), (515, 31, 67), (1024, 48, 128), (66, 35, 520)]
    if kernel.endswith("-tall"):
        shapes += [(2100, 40, 70), (40, 57, 2050), (1030, 130, 1100)]
    for s, (M, K, N) in enumerate(shapes):
        a, w, gc = rand_problem(bits, M, K, N, seed=11 * bits + s)
        ga, gw = run_backward(dev, gc, a, w, la, lw)
        check_backward(oracle_c, gc, a, w, la, lw, bits, ga, gw)


@pytest.mark.parametrize("bits", [6, 8])
def test_forward_tiles_cut_across_ctas(dev, oracle_c, bits):
    """Few tiles and a long K: the forward slab kernel gives every CTA an equal share of the (tile, k chunk) pairs, so
    each tile is cut many times and its parts are combined with integer atomics - the sums must stay bit-exact, with
    and without 16-byte aligned output rows, and whole tiles (16-byte stores) next to cut ones."""
    lf, _, _ = synth_wire(bits, seed=40 + bits)
    for s, (M, K, N) in enumerate([(1100, 4096, 200), (512, 8192, 64), (3000, 1040, 130), (9000, 528, 128)]):
        a, w, _ = rand_problem(bits, M, K, N, seed=13 * bits + s)
        assert np.array_equal(run_forward(dev, a, w, lf), oracle_c.forward(a, w, lf, bits)), (bits, M, K, N)


@pytest.mark.parametrize("bits", [7, 8])
def test_extreme_codes(dev, oracle_c, bits):
    lf, la, lw = synth_wire(bits, seed=3)
    q = 1 << bits
    M, K, N = 96, 160, 272
    for fill_a, fill_w in ((0, 0), (q - 1, q - 1), (0, q - 1), (q - 1, 0)):
        a = np.full((M, K), fill_a, np.uint8)
        w = np.full((K, N), fill_w, np.uint8)
        gc = np.ones((M, N), np.float32)
        assert np.array_equal(run_forward(dev, a, w, lf), oracle_c.forward(a, w, lf, bits))
        ga, gw = run_backward(dev, gc, a, w, la, lw)
        check_backward(oracle_c, gc, a, w, la, lw, bits, ga, gw)


def test_config0_single_layer(dev, oracle_c):
    """The CPU-runnable benchmark case: M=256, K=512, N=256, 7-bit, seed 0."""
    bits = 7
    lf, la, lw = synth_wire(bits, seed=0)
    a, w, gc = rand_problem(bits, 256, 512, 256, seed=0)
    assert np.array_equal(run_forward(dev, a, w, lf), oracle_c.forward(a, w, lf, bits))
    ga, gw = run_backward(dev, gc, a, w, la, lw)
    check_backward(oracle_c, gc, a, w, la, lw, bits, ga, gw)


def test_split_m_weight_gradient_on_a_conv_shape(dev, oracle_c):
    """A long-M, small-output problem makes the weight-gradient kernel split M into slabs."""
    bits = 7
    lf, la, lw = synth_wire(bits, seed=5)
    a, w, gc = rand_problem(bits, 20000, 72, 64, seed=9)
    ga, gw = run_backward(dev, gc, a, w, la, lw)
    check_backward(oracle_c, gc, a, w, la, lw, bits, ga, gw)


@pytest.mark.parametrize("bits", [7, 8])
def test_full_size_properties(dev, oracle_c, bits):
    """At a benchmark-sized problem the oracle is too slow for every element, so check (1) sampled rows
    and columns against the oracle, (2) additivity over a split of K (forward is a sum over k),
    (3) invariance under a joint permutation of k, (4) linearity of the backward in grad_out."""
    lf, la, lw = synth_wire(bits, seed=1)
    M = K = N = 2048
    a, w, gc = rand_problem(bits, M, K, N, seed=77)
    c = run_forward(dev, a, w, lf)
    rows = np.array([0, 1, 777, 1024, M - 1])
    cols = np.array([0, 5, 1000, N - 1])
    assert np.array_equal(c[rows], oracle_c.forward(a[rows], w, lf, bits))
    assert np.array_equal(c[:, cols], oracle_c.forward(a, np.ascontiguousarray(w[:, cols]), lf, bits))
    c1 = run_forward(dev, np.ascontiguousarray(a[:, :1000]), np.ascontiguousarray(w[:1000]), lf)
    c2 = run_forward(dev, np.ascontiguousarray(a[:, 1000:]), np.ascontiguousarray(w[1000:]), lf)
    assert np.array_equal(c1 + c2, c)
    perm = np.random.default_rng(5).permutation(K)
    assert np.array_equal(run_forward(dev, np.ascontiguousarray(a[:, perm]), np.ascontiguousarray(w[perm]), lf), c)

    ga, gw = run_backward(dev, gc, a, w, la, lw)
    r_ga, _, r_gaa, _ = oracle_c.backward_f64(gc[rows], a[rows], w, la, lw, bits)
    assert (np.abs(ga[rows] - r_ga) <= TOL * r_gaa + 1e-30).all()
    kk = np.array([0, 3, 999, K - 1])
    _, r_gw, _, r_gwa = oracle_c.backward_f64(gc, np.ascontiguousarray(a[:, kk]), np.ascontiguousarray(w[kk]), la, lw, bits)
    assert (np.abs(gw[kk] - r_gw) <= TOL * r_gwa + 1e-30).all()
    ga2, gw2 = run_backward(dev, 2.0 * gc, a, w, la, lw)  # scaling by 2 is exact in fp32
    assert np.array_equal(ga2, 2.0 * ga) and np.array_equal(gw2, 2.0 * gw)


def test_autograd_ops_and_conv_against_golden(dev, golden):
    """The reference-facing Python ops (self_ops.*) on the GPU against the golden conv fixtures."""
    import self_ops
    bits = int(golden["bits"])
    fp, ga_t, gb_t = (O.unpack_padded(golden[k], bits) for k in ("lut_fp", "lut_ga", "lut_gb"))
    self_ops.set_lookup_tables(dev, fp, ga_t, gb_t, bits)
    for i in range(4):
        B, Cin, H, W, Cout, k, s, p, d = [int(v) for v in golden[f"conv{i}_cfg"]]
        x = torch.from_numpy(golden[f"conv{i}_x"]).to(dev).float().requires_grad_(True)
        wt = torch.from_numpy(golden[f"conv{i}_w"]).to(dev).float().requires_grad_(True)
        y = self_ops.approx_conv2d_op(x, wt, bias=None, stride=(s, s), padding=(p, p), dilation=(d, d), groups=1)
        assert np.array_equal(y.detach().cpu().numpy(), golden[f"conv{i}_y"])
        y.backward(torch.from_numpy(golden[f"conv{i}_gy"]).to(dev))
        for got, want in ((x.grad, golden[f"conv{i}_gx"]), (wt.grad, golden[f"conv{i}_gw"])):
            got = got.cpu().numpy()
            assert np.abs(got - want).max() <= TOL * max(np.abs(want).max(), 1e-30)
    # straight-through variant: same forward, matmul backward
    a = torch.from_numpy(golden["gemm4_a"]).to(dev).float().requires_grad_(True)
    b = torch.from_numpy(golden["gemm4_b"]).to(dev).float().requires_grad_(True)
    c = self_ops.approx_gemm_baseline_op(a, b)
    assert np.array_equal(c.detach().cpu().numpy(), golden["gemm4_c"])
    gc = torch.from_numpy(golden["gemm4_gc"]).to(dev)
    c.backward(gc)
    assert torch.allclose(a.grad, gc @ b.detach().t(), rtol=1e-4, atol=1e-2)


CONV_CASES = [  # B, Cin, H, W, Cout, k, stride, pad, dil
    (2, 3, 8, 8, 5, 3, 1, 1, 1), (1, 4, 9, 7, 6, 3, 2, 1, 1), (2, 2, 6, 6, 3, 1, 1, 0, 1), (1, 3, 10, 10, 4, 3, 1, 2, 2),
    (3, 3, 32, 32, 64, 3, 1, 1, 1), (2, 16, 16, 16, 40, 3, 2, 1, 1), (4, 8, 12, 12, 32, 1, 2, 0, 1),
    (2, 64, 16, 16, 64, 3, 1, 1, 1), (1, 24, 20, 20, 400, 3, 1, 1, 1), (2, 5, 7, 9, 33, 5, 1, 2, 1),
    # activation gradient without an unfolded intermediate: several row blocks per pixel tile (3x3, 128 and 320
    # output channels), stride classes with 1 to 16 taps (3x3, 5x5 and 7x7 at stride 2, 4x4 at stride 3)
    (2, 20, 10, 10, 128, 3, 1, 1, 1), (1, 8, 16, 16, 320, 3, 2, 1, 1), (2, 6, 11, 13, 24, 5, 2, 2, 1),
    (1, 3, 21, 18, 16, 7, 2, 3, 1), (2, 4, 13, 11, 12, 4, 3, 1, 1),
    # windows that do not overlap (grad_a written in place): 2x2 stride 2, 4x4 stride 4 (patches), 3x3 stride 3
    # with padding, 2x2 stride 3 (positions nobody reads), 1x1 with a long reduction (slab kernels)
    (2, 5, 8, 8, 9, 2, 2, 0, 1), (1, 3, 16, 16, 40, 4, 4, 0, 1), (2, 4, 10, 10, 7, 3, 3, 1, 1),
    (1, 6, 11, 11, 10, 2, 3, 0, 1), (1, 8, 12, 12, 800, 1, 1, 0, 1)]


@pytest.mark.parametrize("bits", [4, 6, 7, 8])
@pytest.mark.parametrize("tile", ["auto", "tall"])
def test_fused_conv_kernels_against_oracle(dev, oracle_c, bits, tile, kernel_choice):
    """lutgemm_conv2d_forward / _backward (implicit im2col) against im2col + GEMM + col2im on the oracle;
    once with the dispatcher's own choice and once with the tall-tile slab gradient kernels forced."""
    import approx_ops
    if tile == "tall":
        kernel_choice(backward="slab", grad_tile="tall")
    lf, la, lw = synth_wire(bits, seed=30 + bits)
    lft, lat, lwt = (torch.from_numpy(t).to(dev) for t in (lf, la, lw))
    for s_, (B, Cin, H, W, Cout, k, st, p, d) in enumerate(CONV_CASES):
        rng = np.random.default_rng(1000 * bits + s_)
        q = 1 << bits
        x = rng.integers(0, q, (B, Cin, H, W)).astype(np.uint8)
        wt = rng.integers(0, q, (Cout, Cin, k, k)).astype(np.uint8)
        wmat = np.ascontiguousarray(wt.reshape(Cout, -1).T)
        Ho, Wo = (H + 2 * p - d * (k - 1) - 1) // st + 1, (W + 2 * p - d * (k - 1) - 1) // st + 1
        gy = rng.standard_normal((B * Ho * Wo, Cout)).astype(np.float32)
        col = oracle_c.im2col(x, k, k, st, p, d)
        want_y = oracle_c.forward(col, wmat, lf, bits)
        xt, wm = torch.from_numpy(x).to(dev), torch.from_numpy(wmat).to(dev)
        y = torch.full((B * Ho * Wo, Cout), 0xDEADBEEF, dtype=torch.uint32, device=dev)
        approx_ops.approx_conv2d_forward(xt, wm, y, lft, k, k, st, p, d)
        assert np.array_equal(y.cpu().numpy(), want_y), (bits, B, Cin, H, W, Cout, k, st, p, d)
        gx = torch.full(x.shape, float("nan"), dtype=torch.float32, device=dev)
        gw = torch.full(wmat.shape, float("nan"), dtype=torch.float32, device=dev)
        approx_ops.approx_conv2d_backward(torch.from_numpy(gy).to(dev), xt, wm, gx, gw, lat, lwt, k, k, st, p, d)
        r_ga, r_gw, r_gaa, r_gwa = oracle_c.backward_f64(gy, col, wmat, la, lw, bits)
        gw_n, gx_n = gw.cpu().numpy(), gx.cpu().numpy()
        assert (np.abs(gw_n - r_gw) <= TOL * r_gwa + 1e-30).all()
        r_gx = O.col2im_f64(r_ga, x.shape, k, k, st, p, d)
        r_gxa = O.col2im_f64(r_gaa, x.shape, k, k, st, p, d)
        assert np.isfinite(gx_n).all()
        assert (np.abs(gx_n - r_gx) <= TOL * r_gxa + 1e-30).all(), (bits, B, Cin, H, W, Cout, k, st, p, d)


def test_fused_conv_op_against_golden(dev, golden):
    """self_ops.approx_conv2d_op (convolution entry points of the library, no F.unfold) must reproduce the golden
    conv fixtures, which the reference's own unfold-based Python layer produced."""
    import self_ops
    bits = int(golden["bits"])
    fp, ga_t, gb_t = (O.unpack_padded(golden[k], bits) for k in ("lut_fp", "lut_ga", "lut_gb"))
    self_ops.set_lookup_tables(dev, fp, ga_t, gb_t, bits)
    for i in range(4):
        B, Cin, H, W, Cout, k, s, p, d = [int(v) for v in golden[f"conv{i}_cfg"]]
        x = torch.from_numpy(golden[f"conv{i}_x"]).to(dev).float().requires_grad_(True)
        wt = torch.from_numpy(golden[f"conv{i}_w"]).to(dev).float().requires_grad_(True)
        y = self_ops.approx_conv2d_op(x, wt, bias=None, stride=(s, s), padding=(p, p), dilation=(d, d), groups=1)
        assert np.array_equal(y.detach().cpu().numpy(), golden[f"conv{i}_y"])
        y.backward(torch.from_numpy(golden[f"conv{i}_gy"]).to(dev))
        for got, want in ((x.grad, golden[f"conv{i}_gx"]), (wt.grad, golden[f"conv{i}_gw"])):
            got = got.cpu().numpy()
            assert np.abs(got - want).max() <= TOL * max(np.abs(want).max(), 1e-30)


def test_errors_raise_instead_of_printing(dev):
    import approx_ops
    a = torch.zeros(4, 4, dtype=torch.uint8, device=dev)
    c = torch.zeros(4, 4, dtype=torch.uint32, device=dev)
    with pytest.raises(RuntimeError, match="size should be"):
        approx_ops.approx_gemm_forward(a, a, c, torch.zeros(1000, dtype=torch.uint16, device=dev))
    with pytest.raises(RuntimeError, match="shape should be"):
        approx_ops.approx_gemm_forward(a, a[:3].contiguous(), c, torch.zeros(17408, dtype=torch.uint16, device=dev))
    with pytest.raises(RuntimeError, match="contiguous"):
        approx_ops.approx_gemm_forward(a.t(), a, c, torch.zeros(17408, dtype=torch.uint16, device=dev))


def test_bounded_wait_times_out_and_reports(dev):
    """A barrier wait that can never be satisfied must give up, report its id through the error word and
    leave the context usable (no hang, no fault)."""
    import approx_ops
    assert approx_ops.device_error() == 0  # nothing above ran into a time-out
    assert approx_ops.library().lutgemm_selftest_bounded_wait(None) == 0
    torch.cuda.synchronize()
    assert approx_ops.device_error() == 99
    assert approx_ops.device_error() == 0  # reading clears it
    x = torch.ones(8, device=dev)
    assert float(x.sum()) == 8.0


@pytest.mark.parametrize("bits", [7, 8])
def test_whole_layer_kernels_match_the_reference_expression(dev, bits, monkeypatch):
    """AppConv2d with conv_impl="layer" (quantisation prologue, LUT convolution, de-quantisation epilogue and
    their fused backward) against the reference's layer expression evaluated by autograd - F.unfold + LUT-GEMM
    for the product term, three library convolutions for the zero-point cross terms
    (tests/reference_expression.py, after micronet+/app_layers.py:147-184): same outputs and gradients to
    fp32 rounding."""
    import self_ops
    from lutgemm_layers import AppConv2d
    from reference_expression import approx_conv_layer
    fp, ga_t, gb_t = O.synthetic_tables(bits, seed=40 + bits)
    self_ops.set_lookup_tables(dev, fp, ga_t, gb_t, bits)
    # the reference expression evaluates its cross terms with library convolutions: keep those in full fp32
    monkeypatch.setattr(torch.backends.cudnn, "allow_tf32", False)
    unfold_op = lambda a, b, **kw: self_ops.unfold_conv2d(self_ops.approx_gemm_op, a, b, **kw)
    cases = [(4, 3, 12, 12, 8, 3, 1, 1, False, False), (2, 40, 9, 11, 33, 3, 2, 1, True, True),
             (3, 64, 8, 8, 64, 1, 2, 0, False, True), (2, 16, 10, 10, 24, 3, 1, 2, True, False),
             (2, 8, 40, 40, 64, 3, 1, 1, False, False)]
    for s_, (B, Cin, H, W, Cout, k, st, p, bias, cl) in enumerate(cases):
        torch.manual_seed(100 * bits + s_)
        new = AppConv2d(Cin, Cout, k, st, p, 1, 1, bias, bits, bits, False, "layer").to(dev).train()
        x = torch.randn(B, Cin, H, W, device=dev) * 1.5 + 0.3
        if cl:
            x = x.contiguous(memory_format=torch.channels_last)
        xr, xn = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        yn = new(xn)  # refreshes the layer's scales and zero points from this input, as the reference layer would
        w_ref = new.weight.detach().clone().requires_grad_(True)
        b_ref = new.bias.detach().clone().requires_grad_(True) if bias else None
        yr = approx_conv_layer(unfold_op, xr, w_ref, b_ref, new.activation_scale, new.activation_zp_neg,
                               new.weight_scale, new.weight_zp_neg, new.a_qmax, new.w_qmax, (st, st), (p, p), (1, 1))
        assert yr.shape == yn.shape
        # The output is a small difference of large terms (LUT sum against zero-point cross terms), and the
        # library convolutions of the reference expression are not exact in fp32: allow a few fp32 roundings of
        # the largest term.
        qmax = float((1 << bits) - 1)
        s_a, z_a, s_w, z_w = (float(t) for t in (new.activation_scale, new.activation_zp_neg, new.weight_scale,
                                                  new.weight_zp_neg))
        kdim = Cin * k * k
        mag = s_a * s_w * kdim * (qmax * qmax + (abs(z_a) + abs(z_w)) * qmax + abs(z_a * z_w))
        assert float((yr - yn).detach().abs().max()) <= 4 * 1.2e-7 * mag, (bits, s_)
        g = torch.randn_like(yr)
        yr.backward(g)
        yn.backward(g)
        # Each gradient is the sum of a LUT term and a zero-point cross term that largely cancel, and the two
        # evaluations round them in different places: the tolerance is 1e-5 of the size of the terms, not of
        # their (smaller) sum.
        s_a, z_a, s_w, z_w = new.activation_scale, new.activation_zp_neg, new.weight_scale, new.weight_zp_neg
        ones_k = torch.ones(1, 1, k, k, device=dev)
        Ho, Wo = yr.shape[2], yr.shape[3]
        opad = (H - ((Ho - 1) * st - 2 * p + (k - 1) + 1), W - ((Wo - 1) * st - 2 * p + (k - 1) + 1))
        box_t = F.conv_transpose2d(g.sum(dim=1, keepdim=True), ones_k, stride=st, padding=p, output_padding=opad)
        tap = torch.nn.grad.conv2d_weight(torch.ones(1, 1, H, W, device=dev), (Cout, 1, k, k), g.sum(dim=0, keepdim=True),
                                          stride=st, padding=p)
        cross = {"x": float((s_w * z_w * box_t).abs().max()), "w": float((s_a * z_a * tap).abs().max())}
        for a_, b_, name in ((xr.grad, xn.grad, "x"), (w_ref.grad, new.weight.grad, "w")):
            scale_ = float(a_.abs().max()) + 2.0 * cross[name]
            assert float((a_ - b_).abs().max()) <= 1e-5 * scale_ + 1e-30, (bits, s_, name)
        if bias:
            assert torch.allclose(b_ref.grad, new.bias.grad, rtol=1e-5, atol=1e-6)
        assert xn.grad.stride() == xn.stride()


@pytest.mark.parametrize("bits", [7, 8])
def test_workspace_entry_points_match_the_plain_ones(dev, bits):
    """lutgemm_forward_ws (activation codes transposed into a workspace first) against lutgemm_forward, and
    a convolution backward fed the forward pass's transposed codes against one that makes its own."""
    import ctypes
    import approx_ops
    lib = approx_ops.library()
    lf, la, lw = (torch.from_numpy(t).to(dev) for t in synth_wire(bits, seed=50 + bits))
    stream = torch.cuda.current_stream(dev).cuda_stream
    # a shape the row-broadcast kernel takes has no use for a workspace
    assert lib.lutgemm_forward_scratch_bytes(bits, 100, 64, 16) == 0
    for s_, (M, K, N) in enumerate([(1024, 48, 64), (1000, 45, 120), (960, 31, 62)]):
        a, w, _ = rand_problem(bits, M, K, N, seed=60 * bits + s_)
        at, wt = torch.from_numpy(a).to(dev), torch.from_numpy(w).to(dev)
        c0 = torch.zeros(M, N, dtype=torch.uint32, device=dev)
        c1 = torch.zeros(M, N, dtype=torch.uint32, device=dev)
        assert lib.lutgemm_forward(at.data_ptr(), wt.data_ptr(), c0.data_ptr(), lf.data_ptr(), bits, M, K, N, stream) == 0
        nbytes = lib.lutgemm_forward_scratch_bytes(bits, M, K, N)
        assert nbytes == K * ((M + 15) // 16 * 16)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        assert lib.lutgemm_forward_ws(at.data_ptr(), wt.data_ptr(), c1.data_ptr(), lf.data_ptr(), bits, M, K, N,
                                      ws.data_ptr(), nbytes, stream) == 0
        assert torch.equal(c0.view(torch.int32), c1.view(torch.int32))
        assert torch.equal(ws.view(K, -1)[:, :M], at.t())            # the workspace holds the transposed codes
        assert lib.lutgemm_forward_ws(at.data_ptr(), wt.data_ptr(), c1.data_ptr(), lf.data_ptr(), bits, M, K, N,
                                      ws.data_ptr(), nbytes - 1, stream) == -4   # LUTGEMM_E_SCRATCH
        # the GEMM backward fed the forward pass's transposed codes gives the same gradients as one making its own
        gct = torch.randn(M, N, device=dev)
        res = []
        for given in (None, ws):
            ga_, gw_ = torch.empty(M, K, device=dev), torch.empty(K, N, device=dev)
            approx_ops.approx_gemm_backward(gct, at, wt, ga_, gw_, la, lw, codes_t=given)
            res.append((ga_, gw_))
        assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    B, Cin, H, W, Cout, k, st, p = 3, 16, 32, 32, 64, 3, 1, 1
    rng = np.random.default_rng(7 + bits)
    x = torch.from_numpy(rng.integers(0, 1 << bits, (B, Cin, H, W)).astype(np.uint8)).to(dev)
    wm = torch.from_numpy(rng.integers(0, 1 << bits, (Cin * k * k, Cout)).astype(np.uint8)).to(dev)
    M = B * H * W
    y = torch.empty(M, Cout, dtype=torch.uint32, device=dev)
    codes_t = approx_ops.approx_conv2d_forward(x, wm, y, lf, k, k, st, p, 1)
    assert codes_t is not None and codes_t.numel() == Cin * k * k * M
    gy = torch.randn(M, Cout, device=dev)
    out = []
    for given in (None, codes_t):
        gx, gw = torch.empty(x.shape, device=dev), torch.empty(wm.shape, device=dev)
        approx_ops.approx_conv2d_backward(gy, x, wm, gx, gw, la, lw, k, k, st, p, 1, codes_t=given)
        out.append((gx, gw))
    assert torch.equal(out[0][0], out[1][0]) and torch.equal(out[0][1], out[1][1])


@pytest.mark.parametrize("bits", [4, 6, 7, 8])
def test_random_shapes_through_the_dispatcher(dev, oracle_c, bits):
    """Seeded random shapes (tile edges, ragged K, rows and columns that are not multiples of anything) through
    whatever kernels the dispatcher picks, GEMM and convolution, against the oracle."""
    import approx_ops
    lf, la, lw = synth_wire(bits, seed=90 + bits)
    rng = np.random.default_rng(9000 + bits)
    shapes = []
    while len(shapes) < 14:
        M, K, N = (int(v) for v in np.exp(rng.uniform(0, np.log(2600), 3)))
        if M * K * N <= 40_000_000:
            shapes.append((M, K, N))
    shapes += [(1030, 17, 33), (2049, 5, 70), (1023, 100, 31), (3000, 9, 800), (40, 60, 1025), (1024, 16, 32)]
    for s_, (M, K, N) in enumerate(shapes):
        a, w, gc = rand_problem(bits, M, K, N, seed=31 * bits + s_)
        c = run_forward(dev, a, w, lf)
        assert np.array_equal(c, oracle_c.forward(a, w, lf, bits)), (bits, M, K, N)
        ga, gw = run_backward(dev, gc, a, w, la, lw)
        check_backward(oracle_c, gc, a, w, la, lw, bits, ga, gw)
    lft, lat, lwt = (torch.from_numpy(t).to(dev) for t in (lf, la, lw))
    for s_ in range(8):
        B, Cin, Cout = int(rng.integers(1, 5)), int(rng.integers(1, 40)), int(rng.integers(1, 90))
        k, st, d = int(rng.choice([1, 2, 3, 5])), int(rng.choice([1, 2, 3])), int(rng.choice([1, 2]))
        p = int(rng.integers(0, k))
        H, W = int(rng.integers(d * (k - 1) + 1, 40)), int(rng.integers(d * (k - 1) + 1, 40))
        x = rng.integers(0, 1 << bits, (B, Cin, H, W)).astype(np.uint8)
        wmat = rng.integers(0, 1 << bits, (Cin * k * k, Cout)).astype(np.uint8)
        Ho, Wo = (H + 2 * p - d * (k - 1) - 1) // st + 1, (W + 2 * p - d * (k - 1) - 1) // st + 1
        gy = rng.standard_normal((B * Ho * Wo, Cout)).astype(np.float32)
        col = oracle_c.im2col(x, k, k, st, p, d)
        xt, wm = torch.from_numpy(x).to(dev), torch.from_numpy(wmat).to(dev)
        y = torch.empty((B * Ho * Wo, Cout), dtype=torch.uint32, device=dev)
        codes_t = approx_ops.approx_conv2d_forward(xt, wm, y, lft, k, k, st, p, d)
        assert np.array_equal(y.cpu().numpy(), oracle_c.forward(col, wmat, lf, bits)), (bits, B, Cin, H, W, Cout, k, st, p, d)
        gx = torch.full(x.shape, float("nan"), dtype=torch.float32, device=dev)
        gw = torch.full(wmat.shape, float("nan"), dtype=torch.float32, device=dev)
        approx_ops.approx_conv2d_backward(torch.from_numpy(gy).to(dev), xt, wm, gx, gw, lat, lwt, k, k, st, p, d,
                                          codes_t=codes_t)
        r_ga, r_gw, r_gaa, r_gwa = oracle_c.backward_f64(gy, col, wmat, la, lw, bits)
        assert (np.abs(gw.cpu().numpy() - r_gw) <= TOL * r_gwa + 1e-30).all(), (bits, B, Cin, H, W, Cout, k, st, p, d)
        r_gx = O.col2im_f64(r_ga, x.shape, k, k, st, p, d)
        r_gxa = O.col2im_f64(r_gaa, x.shape, k, k, st, p, d)
        assert (np.abs(gx.cpu().numpy() - r_gx) <= TOL * r_gxa + 1e-30).all(), (bits, B, Cin, H, W, Cout, k, st, p, d)


def test_straight_through_conv_op_matches_the_unfold_formulation(dev, golden):
    """approx_conv2d_baseline_op (LUT convolution forward, exact-convolution gradients) against the reference's
    formulation of it (F.unfold + LUT-GEMM forward, two matmuls backward, self_ops/ops_py/approx_ops.py:576-619):
    identical forward (the LUT sums), straight-through gradients equal to fp32 rounding."""
    import self_ops
    bits = int(golden["bits"])
    fp, ga_t, gb_t = (O.unpack_padded(golden[k], bits) for k in ("lut_fp", "lut_ga", "lut_gb"))
    self_ops.set_lookup_tables(dev, fp, ga_t, gb_t, bits)
    for i in range(4):
        B, Cin, H, W, Cout, k, s, p, d = [int(v) for v in golden[f"conv{i}_cfg"]]
        kw = dict(bias=None, stride=(s, s), padding=(p, p), dilation=(d, d), groups=1)
        outs = []
        unfold_op = lambda a, b, **k_: self_ops.unfold_conv2d(self_ops.approx_gemm_baseline_op, a, b, **k_)
        for op in (unfold_op, self_ops.approx_conv2d_baseline_op):
            x = torch.from_numpy(golden[f"conv{i}_x"]).to(dev).float().requires_grad_(True)
            wt = torch.from_numpy(golden[f"conv{i}_w"]).to(dev).float().requires_grad_(True)
            y = op(x, wt, **kw)
            y.backward(torch.from_numpy(golden[f"conv{i}_gy"]).to(dev))
            outs.append((y.detach(), x.grad, wt.grad))
        assert torch.equal(outs[0][0], outs[1][0])
        assert np.array_equal(outs[1][0].cpu().numpy(), golden[f"conv{i}_y"])
        for a_, b_ in zip(outs[0][1:], outs[1][1:]):
            assert torch.allclose(a_, b_, rtol=1e-4, atol=1e-5 * float(a_.abs().max()))
