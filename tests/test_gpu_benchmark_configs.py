"""GPU parity on the shapes and operand formats of the benchmark's other configurations:

* configuration 0 - one linear layer, M=256, K=512, N=256, 7-bit magnitudes with independent sign bits, the
  synthetic multiplier L[x][y] = max(0, x*y + e); run on the 8-bit kernels through `lutgemm_signed.SignedTables`
  and checked against a direct NumPy evaluation (forward exact, backward 1e-5);
* configuration 3 - layer geometries of ResNet-50 at ImageNet shape (7x7 stride-2 stem, 1x1 / 3x3 bottleneck
  convolutions, strided shortcuts, the 2048 -> 1000 classifier) at 8 bits, reduced batch;
* configuration 4 - the linears of ViT-S/16 (d=384, MLP 1536, 197 tokens per image) and its 16x16 patch
  embedding at 7 bits, reduced batch.
The full-size models are benchmark material, not test material: what is checked here is that every layer shape
they contain goes through the C-ABI bit-exactly (forward) and within 1e-5 (backward)."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as O

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "gpu-marked test started without a CUDA device"
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def oracle_c():
    from oracle.oracle_c import OracleC
    return OracleC()


def test_config0_signed_linear_layer(dev):
    from lutgemm_signed import SignedTables
    bits, M, K, N = 7, 256, 512, 256
    q = 1 << bits
    fp, ga, gb = O.synthetic_tables(bits, seed=0, half_window=8)
    tables = SignedTables(dev, fp, ga, gb, bits)
    rng = np.random.default_rng(0)
    a_mag, w_mag = rng.integers(0, q, (M, K)), rng.integers(0, q, (K, N))
    a_neg, w_neg = rng.random((M, K)) < 0.5, rng.random((K, N)) < 0.5
    gc = rng.standard_normal((M, N)).astype(np.float32)
    act_scale, w_scale = 0.05, 0.01
    a_codes = tables.codes(torch.from_numpy(a_mag).to(dev), torch.from_numpy(a_neg).to(dev))
    w_codes = tables.codes(torch.from_numpy(w_mag).to(dev), torch.from_numpy(w_neg).to(dev))
    out = tables.forward(a_codes, w_codes)
    sa, sw = np.where(a_neg, -1, 1).astype(np.int64), np.where(w_neg, -1, 1).astype(np.int64)
    want = np.zeros((M, N), np.int64)
    for k in range(K):  # exact integer reference, one k at a time
        want += (sa[:, k, None] * sw[None, k, :]) * fp[a_mag[:, k, None], w_mag[None, k, :]]
    assert np.array_equal(out.cpu().numpy(), want)
    scaled = out.to(torch.float64) * (act_scale * w_scale)
    assert np.allclose(scaled.cpu().numpy(), want * (act_scale * w_scale), rtol=0, atol=0)
    # gradients w.r.t. the signed operand values, against the gradient tables as the wire format holds them
    qa, qb = np.round(ga * 16.0) / 16.0, np.round(gb * 16.0) / 16.0
    g_a, g_w = tables.backward(torch.from_numpy(gc).to(dev), a_codes, w_codes)
    ref_a, abs_a = np.zeros((M, K)), np.zeros((M, K))
    ref_w, abs_w = np.zeros((K, N)), np.zeros((K, N))
    gc64 = gc.astype(np.float64)
    for k in range(K):
        ta = sw[None, k, :] * qa[a_mag[:, k, None], w_mag[None, k, :]] * gc64   # [M, N]
        tw = sa[:, k, None] * qb[a_mag[:, k, None], w_mag[None, k, :]] * gc64
        ref_a[:, k], abs_a[:, k] = ta.sum(axis=1), np.abs(ta).sum(axis=1)
        ref_w[k, :], abs_w[k, :] = tw.sum(axis=0), np.abs(tw).sum(axis=0)
    assert (np.abs(g_a.cpu().numpy() - ref_a) <= TOL * abs_a + 1e-30).all()
    assert (np.abs(g_w.cpu().numpy() - ref_w) <= TOL * abs_w + 1e-30).all()


@pytest.mark.parametrize("bits,shape", [(7, (256, 512, 256)), (6, (1030, 70, 45)), (4, (33, 129, 2100)), (7, (2500, 64, 96))])
def test_fp32_gradient_tables(dev, bits, shape):
    """lutgemm_backward_f32lut with the benchmark's un-rounded window-difference gradient tables (fp32 entries
    that are not multiples of 1/16) against their definition evaluated in float64:
    ga[m,k] = sum_n gc[m,n] * Ga[a[m,k]][w[k,n]], gw[k,n] = sum_m Gw[a[m,k]][w[k,n]] * gc[m,n]; tolerance 1e-5
    of the sum of the absolute terms of each element."""
    import approx_ops
    M, K, N = shape
    q = 1 << bits
    _, ga_t, gb_t = O.synthetic_tables(bits, seed=bits, half_window=3 if bits == 4 else q // 16)
    ga_t, gb_t = ga_t.astype(np.float32), gb_t.astype(np.float32)
    assert np.abs(ga_t * 16 - np.round(ga_t * 16)).max() > 1e-3  # really off the 1/16 grid
    n_el = approx_ops.library().lutgemm_lut_elem_num(bits)

    def wire(dense):
        flat = np.zeros(n_el, np.float32)
        flat[: (q + 1) * (q + 2)].reshape(q + 1, q + 2)[:q, :q] = dense
        return torch.from_numpy(flat).to(dev)

    rng = np.random.default_rng(5 * bits + M)
    a, w = rng.integers(0, q, (M, K)).astype(np.uint8), rng.integers(0, q, (K, N)).astype(np.uint8)
    gc = rng.standard_normal((M, N)).astype(np.float32)
    ga = torch.full((M, K), float("nan"), device=dev)
    gw = torch.full((K, N), float("nan"), device=dev)
    approx_ops.approx_gemm_backward_f32lut(torch.from_numpy(gc).to(dev), torch.from_numpy(a).to(dev),
                                           torch.from_numpy(w).to(dev), ga, gw, wire(ga_t), wire(gb_t))
    gc64, Ga, Gw = gc.astype(np.float64), ga_t.astype(np.float64), gb_t.astype(np.float64)
    ref_a, abs_a, ref_w, abs_w = np.zeros((M, K)), np.zeros((M, K)), np.zeros((K, N)), np.zeros((K, N))
    for k in range(K):
        ta = Ga[a[:, k, None], w[None, k, :]] * gc64
        tw = Gw[a[:, k, None], w[None, k, :]] * gc64
        ref_a[:, k], abs_a[:, k] = ta.sum(axis=1), np.abs(ta).sum(axis=1)
        ref_w[k, :], abs_w[k, :] = tw.sum(axis=0), np.abs(tw).sum(axis=0)
    assert (np.abs(ga.cpu().numpy() - ref_a) <= TOL * abs_a + 1e-30).all()
    assert (np.abs(gw.cpu().numpy() - ref_w) <= TOL * abs_w + 1e-30).all()
    # 8-bit fp32 tables do not fit in shared memory next to the slabs: refused, not approximated
    lib = approx_ops.library()
    assert lib.lutgemm_backward_f32lut(1, 1, 1, 1, 1, 1, 1, 8, 4, 4, 4, None, 0, None) == -2


def _check_gemm(dev, oracle_c, bits, M, K, N, seed, tables):
    import approx_ops
    lf, la, lw = tables
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 1 << bits, (M, K)).astype(np.uint8)
    w = rng.integers(0, 1 << bits, (K, N)).astype(np.uint8)
    gc = rng.standard_normal((M, N)).astype(np.float32)
    at, wt = torch.from_numpy(a).to(dev), torch.from_numpy(w).to(dev)
    c = torch.empty((M, N), dtype=torch.uint32, device=dev)
    approx_ops.approx_gemm_forward(at, wt, c, torch.from_numpy(lf).to(dev))
    assert np.array_equal(c.cpu().numpy(), oracle_c.forward(a, w, lf, bits)), (M, K, N)
    ga = torch.full((M, K), float("nan"), device=dev)
    gw = torch.full((K, N), float("nan"), device=dev)
    approx_ops.approx_gemm_backward(torch.from_numpy(gc).to(dev), at, wt, ga, gw, torch.from_numpy(la).to(dev),
                                    torch.from_numpy(lw).to(dev))
    r_ga, r_gw, r_gaa, r_gwa = oracle_c.backward_f64(gc, a, w, la, lw, bits)
    assert (np.abs(ga.cpu().numpy() - r_ga) <= TOL * r_gaa + 1e-30).all(), (M, K, N)
    assert (np.abs(gw.cpu().numpy() - r_gw) <= TOL * r_gwa + 1e-30).all(), (M, K, N)


def _check_conv(dev, oracle_c, bits, case, seed, tables):
    import approx_ops
    lf, la, lw = tables
    B, Cin, H, W, Cout, k, st, p = case
    rng = np.random.default_rng(seed)
    x = rng.integers(0, 1 << bits, (B, Cin, H, W)).astype(np.uint8)
    wmat = rng.integers(0, 1 << bits, (Cin * k * k, Cout)).astype(np.uint8)
    Ho, Wo = (H + 2 * p - k) // st + 1, (W + 2 * p - k) // st + 1
    gy = rng.standard_normal((B * Ho * Wo, Cout)).astype(np.float32)
    col = oracle_c.im2col(x, k, k, st, p, 1)
    xt, wm = torch.from_numpy(x).to(dev), torch.from_numpy(wmat).to(dev)
    y = torch.empty((B * Ho * Wo, Cout), dtype=torch.uint32, device=dev)
    approx_ops.approx_conv2d_forward(xt, wm, y, torch.from_numpy(lf).to(dev), k, k, st, p, 1)
    assert np.array_equal(y.cpu().numpy(), oracle_c.forward(col, wmat, lf, bits)), case
    gx = torch.full(x.shape, float("nan"), dtype=torch.float32, device=dev)
    gw = torch.full(wmat.shape, float("nan"), dtype=torch.float32, device=dev)
    approx_ops.approx_conv2d_backward(torch.from_numpy(gy).to(dev), xt, wm, gx, gw, torch.from_numpy(la).to(dev),
                                      torch.from_numpy(lw).to(dev), k, k, st, p, 1)
    r_ga, r_gw, r_gaa, r_gwa = oracle_c.backward_f64(gy, col, wmat, la, lw, bits)
    assert (np.abs(gw.cpu().numpy() - r_gw) <= TOL * r_gwa + 1e-30).all(), case
    r_gx = O.col2im_f64(r_ga, x.shape, k, k, st, p, 1)
    r_gxa = O.col2im_f64(r_gaa, x.shape, k, k, st, p, 1)
    assert (np.abs(gx.cpu().numpy() - r_gx) <= TOL * r_gxa + 1e-30).all(), case


# B, Cin, H, W, Cout, kernel, stride, pad - one layer of each kind in ResNet-50 at 224 x 224
RESNET50_LAYERS = [(1, 3, 224, 224, 64, 7, 2, 3), (1, 64, 56, 56, 64, 1, 1, 0), (1, 64, 56, 56, 64, 3, 1, 1),
                   (1, 64, 56, 56, 256, 1, 1, 0), (1, 256, 56, 56, 128, 1, 1, 0), (1, 128, 56, 56, 128, 3, 2, 1),
                   (1, 256, 56, 56, 512, 1, 2, 0), (2, 512, 14, 14, 512, 3, 1, 1), (2, 1024, 14, 14, 2048, 1, 2, 0),
                   (3, 512, 7, 7, 2048, 1, 1, 0)]


def test_config3_resnet50_layer_shapes(dev, oracle_c):
    bits = 8
    tables = O.to_wire(*O.synthetic_tables(bits, seed=3), bits)
    for s_, case in enumerate(RESNET50_LAYERS):
        _check_conv(dev, oracle_c, bits, case, 300 + s_, tables)
    _check_gemm(dev, oracle_c, bits, 4, 2048, 1000, 399, tables)   # classifier, batch 4


def test_config4_vit_small_layer_shapes(dev, oracle_c):
    bits = 7
    tables = O.to_wire(*O.synthetic_tables(bits, seed=4), bits)
    tokens = 2 * 197
    for s_, (K, N) in enumerate([(384, 1152), (384, 384), (384, 1536), (1536, 384)]):   # QKV, proj, MLP up / down
        _check_gemm(dev, oracle_c, bits, tokens, K, N, 400 + s_, tables)
    _check_conv(dev, oracle_c, bits, (1, 3, 224, 224, 384, 16, 16, 0), 450, tables)    # patch embedding


@pytest.mark.parametrize("name,kw,shape,bits", [
    ("resnet50", dict(base=8, blocks=(1, 1, 1, 1)), (2, 3, 64, 64), 8),
    ("vit_s", dict(image=32, dim=48, depth=2, heads=3, mlp=96), (2, 3, 32, 32), 7)])
def test_reduced_models_take_a_training_step(dev, name, kw, shape, bits):
    """A narrow ResNet-50 (bottleneck blocks, 7x7 stem) and a small ViT (patch embedding, attention with exact
    softmax, approximate linears) run forward, backward and an SGD step through the approximate layers."""
    import self_ops
    import torch.nn.functional as F
    from lutgemm_layers import AppConv2d, AppLinear, prepare
    from lutgemm_models import MODELS
    fp, ga, gb = O.synthetic_tables(bits, seed=bits)
    self_ops.set_lookup_tables(dev, fp, ga, gb, bits)
    torch.manual_seed(0)
    model = MODELS[name][0](10, **kw).to(dev)
    prepare(model, a_bits=bits, w_bits=bits, conv_impl="layer")
    assert any(isinstance(m, AppConv2d) for m in model.modules()) and any(isinstance(m, AppLinear) for m in model.modules())
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    x = torch.randn(*shape, device=dev)
    y = torch.randint(0, 10, (shape[0],), device=dev)
    losses = []
    for _ in range(2):
        opt.zero_grad(set_to_none=True)
        loss = F.cross_entropy(model(x), y)
        loss.backward()
        assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters() if p.requires_grad)
        opt.step()
        losses.append(float(loss.detach()))
    assert all(np.isfinite(losses))


@pytest.mark.parametrize("bits", [7, 8])
def test_whole_layer_linear_matches_the_reference_expression(dev, bits):
    """AppLinear with impl="layer" against the reference's layer expression carried over to a linear layer
    (tests/reference_expression.py: LUT-GEMM product term plus three exact cross-term products, evaluated by
    autograd), 3-D token input, with bias."""
    import self_ops
    from lutgemm_layers import AppLinear
    from reference_expression import approx_linear_layer
    fp, ga, gb = O.synthetic_tables(bits, seed=70 + bits)
    self_ops.set_lookup_tables(dev, fp, ga, gb, bits)
    for s_, (B, T, K, N, bias) in enumerate([(2, 197, 384, 96, True), (3, 5, 33, 17, False), (1, 600, 64, 64, True)]):
        torch.manual_seed(10 * bits + s_)
        new = AppLinear(K, N, bias, bits, bits, False, "layer").to(dev).train()
        x = torch.randn(B, T, K, device=dev) * 1.3 - 0.2
        xr, xn = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        yn = new(xn)  # refreshes the layer's scales and zero points from this input
        w_ref = new.weight.detach().clone().requires_grad_(True)
        b_ref = new.bias.detach().clone().requires_grad_(True) if bias else None
        yr = approx_linear_layer(self_ops.approx_gemm_op, xr.reshape(-1, K), w_ref, b_ref, new.activation_scale,
                                 new.activation_zp_neg, new.weight_scale, new.weight_zp_neg, new.a_qmax,
                                 new.w_qmax).reshape(B, T, N)
        qmax = float((1 << bits) - 1)
        s_a, z_a, s_w, z_w = (float(t) for t in (new.activation_scale, new.activation_zp_neg, new.weight_scale,
                                                  new.weight_zp_neg))
        mag = s_a * s_w * K * (qmax * qmax + (abs(z_a) + abs(z_w)) * qmax + abs(z_a * z_w))
        assert float((yr - yn).detach().abs().max()) <= 4 * 1.2e-7 * mag, (bits, s_)
        g = torch.randn_like(yr)
        yr.backward(g)
        yn.backward(g)
        g2 = g.reshape(-1, N)
        cross = {"x": abs(s_w * z_w) * float(g2.sum(dim=1).abs().max()), "w": abs(s_a * z_a) * float(g2.sum(dim=0).abs().max())}
        for a_, b_, name in ((xr.grad, xn.grad, "x"), (w_ref.grad, new.weight.grad, "w")):
            scale_ = float(a_.abs().max()) + 2.0 * cross[name]
            assert float((a_ - b_).abs().max()) <= 1e-5 * scale_ + 1e-30, (bits, s_, name)
        if bias:
            assert torch.allclose(b_ref.grad, new.bias.grad, rtol=1e-5, atol=1e-6)
