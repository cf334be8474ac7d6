"""GPU tests of the small one-pass kernels of the layer wiring (lutgemm_layer_aux.cu), called through the C-ABI via
`approx_ops`, each against the PyTorch expression it replaces in the layer - the expressions the reference's
ApproxConv2d and observers evaluate (micronet+/app_layers.py:21-53, 147-184).  Sums of integer codes are exact, so
those comparisons are bit-exact; the others allow fp32 rounding of one operation."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GEOMS = [  # B, Cin, H, W, Cout, kh, kw, stride, pad, dil
    (2, 5, 9, 11, 7, 3, 3, 1, 1, 1), (3, 4, 12, 12, 6, 3, 3, 2, 1, 1), (1, 3, 10, 8, 4, 5, 5, 1, 2, 1),
    (2, 2, 13, 13, 3, 3, 3, 1, 2, 2), (2, 6, 8, 8, 5, 1, 1, 2, 0, 1), (1, 2, 7, 9, 3, 2, 2, 3, 0, 1)]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "gpu-marked test started without a CUDA device"
    import approx_ops
    approx_ops.library()
    return torch.device("cuda:0")


def test_observers_and_quantisation_parameters_in_one_launch(dev):
    """layer_update_ranges against the PyTorch observers of lutgemm_layers (running weight range, moving-average
    activation range, scales, zero points) over four steps: identical buffers."""
    import approx_ops
    from lutgemm_layers import AppConv2d
    torch.manual_seed(0)
    ref = AppConv2d(4, 6, 3, 1, 1, 1, 1, False, 7, 7, False, "fused").to(dev).train()
    new = AppConv2d(4, 6, 3, 1, 1, 1, 1, False, 7, 7, False, "layer").to(dev).train()
    new.load_state_dict(ref.state_dict())
    for step in range(4):
        x = torch.randn(2, 4, 8, 8, device=dev) * (1.0 + step) - 0.3 * step
        with torch.no_grad():
            ref.weight.add_(0.05 * torch.randn_like(ref.weight))
            new.weight.copy_(ref.weight)
        ref._refresh(x, ref.weight)
        new._refresh(x, new.weight, fused=True)
        assert torch.equal(ref.quant, new.quant), step
        for a_, b_ in zip(ref.act_range.state() + ref.weight_range.state(), new.act_range.state() + new.weight_range.state()):
            assert torch.equal(a_, b_), step


@pytest.mark.parametrize("channels_last", [False, True])
def test_weight_codes_and_cross_terms(dev, channels_last):
    import approx_ops
    from lutgemm_layers import _valid_taps
    for s_, (B, Cin, H, W, Cout, kh, kw, st, p, d) in enumerate(GEOMS):
        torch.manual_seed(s_)
        weight = torch.randn(Cout, Cin, kh, kw, device=dev)
        if channels_last:
            weight = weight.contiguous(memory_format=torch.channels_last)
        qmax = 127.0
        quant = torch.tensor([0.03, -20.0, 0.02, -70.0], device=dev)
        wmat, wsum = approx_ops.layer_weight_prep(weight, quant, qmax)
        qw = torch.clamp(torch.round(weight / quant[2] - quant[3]), 0.0, qmax)
        assert torch.equal(wmat, qw.reshape(Cout, -1).t().to(torch.uint8))
        assert torch.equal(wsum, qw.sum(dim=1).reshape(Cout, kh * kw))
        sumw_t, taps = approx_ops.layer_cross_terms(wsum, Cin, H, W, kh, kw, st, p, d)
        if kh == kw:
            valid = _valid_taps((H, W, kh, kw, st, p, d), dev)  # [kh*kw, L]
            assert torch.equal(sumw_t, valid.t() @ wsum.t())
            assert torch.equal(taps, valid.sum(dim=0) * float(Cin))
        # gradient of the fp32 weight from the gradient of its codes
        gwmat = torch.randn(Cin * kh * kw, Cout, device=dev)
        tapg = torch.randn(Cout, kh * kw, device=dev)
        gw = approx_ops.layer_weight_grad(gwmat, tapg, weight, quant, qmax)
        g_qw = gwmat.t().reshape(weight.shape) + quant[1] * tapg.reshape(Cout, 1, kh, kw)
        q = torch.round(weight / quant[2] - quant[3])
        want = torch.where((q >= 0) & (q <= qmax), quant[0] * g_qw, torch.zeros_like(g_qw))
        assert gw.is_contiguous() and torch.equal(gw, want.contiguous())


def test_window_sums(dev):
    import approx_ops
    from lutgemm_layers import _out_hw, _window_sum, _window_sum_adjoint
    for s_, (B, Cin, H, W, Cout, kh, kw, st, p, d) in enumerate(GEOMS):
        if kh != kw:
            continue
        torch.manual_seed(10 + s_)
        geom = (H, W, kh, kw, st, p, d)
        img = torch.randint(0, 128 * Cin, (B, H, W), device=dev).float()   # channel sums of codes: integers
        box = approx_ops.layer_window_sum(img, kh, kw, st, p, d)
        assert torch.equal(box, _window_sum(img, geom).reshape(-1))
        Ho, Wo = _out_hw(H, W, kh, kw, st, p, d)
        g = torch.randn(B, Ho, Wo, device=dev)
        adj = approx_ops.layer_window_sum_adjoint(g, H, W, kh, kw, st, p, d)
        want = _window_sum_adjoint(g, geom)
        assert torch.allclose(adj, want, rtol=0, atol=1e-6 * float(want.abs().max()))
        # <window_sum(u), g> = <u, adjoint(g)>
        u = torch.randn(B, H, W, device=dev)
        lhs = float((approx_ops.layer_window_sum(u, kh, kw, st, p, d).double() * g.reshape(-1).double()).sum())
        rhs = float((u.double() * adj.double()).sum())
        assert abs(lhs - rhs) <= 1e-5 * max(abs(lhs), 1.0)


def test_quantisation_division_matches_ieee_division_for_awkward_scales(dev):
    """The quantisation kernels divide by the common scale with a reciprocal and one fused correction; the codes must
    equal clamp(round(x / scale - zp)) evaluated with PyTorch's IEEE division for scales whose mantissa is all ones,
    a power of two, or random, and for activations that are zero, tiny, huge or infinite."""
    import approx_ops
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(4, 40, 9, 33, device=dev, generator=g) * 3.0
    flat = x.view(-1)
    flat[::97] = 0.0
    flat[1::193] = 1e-38
    flat[2::211] = -3e37
    flat[3::389] = float("inf")
    flat[4::401] = -float("inf")
    x = x.contiguous(memory_format=torch.channels_last)
    mant = [0x7FFFFF, 0x7FFFFE, 0x000000, 0x000001, 0x400000, 0x2AAAAB, 0x555555, 0x123457]
    for bits, qmax in ((7, 127.0), (8, 255.0)):
        for i, m in enumerate(mant):
            for e in (110, 121, 127, 130):
                scale = torch.tensor([(e << 23) | m], dtype=torch.int32, device=dev).view(torch.float32)
                zp = torch.tensor([float(-(17 + 9 * i) % int(qmax))], device=dev).neg()
                codes, _ = approx_ops.quantize_activations(x, scale, zp, qmax, want_chansum=False)
                want = torch.clamp(torch.round(x / scale - zp), 0.0, qmax)
                want = torch.nan_to_num(want, nan=0.0).to(torch.uint8)
                assert torch.equal(codes, want.contiguous()), (bits, hex(m), e)
