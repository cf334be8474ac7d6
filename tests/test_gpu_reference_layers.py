"""The reference's own layer and trainer sources, UNMODIFIED, running on top of this package (GPU, -m gpu).

`build()` stages the reference project's `micronet+` directory in baseline/_ref/ (git-ignored).  With this
package's directory first on sys.path, `import self_ops` inside micronet+/app_layers.py:5 and
micronet+/app_train.py:8 resolves to this package, so ApproxConv2d.forward (app_layers.py:152-185) calls this
library's `approx_conv2d_op` / `approx_conv2d_baseline_op` and everything else - observers, fake quantisation,
cross-term convolutions, `prepare`, `train`, `calibrate` - is the reference's code as it stands.

Checked: (1) every ApproxConv2d of a reference-prepared network gives the outputs and gradients of this
package's AppConv2d (whole-layer kernels) on the same input; (2) the reference's `calibrate` and `train` loops
(app_train.py:23-46) step a reference ResNet-18 (models.py:151-211) with Adam, through this library's kernels."""
import copy
import os
import sys
import types

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import oracle_np as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGE = os.path.join(ROOT, "baseline", "_ref")
MICRONET = os.path.join(STAGE, "micronet+")


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test started without a CUDA device")
    import approx_ops
    approx_ops.library()
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def ref_modules():
    """(app_layers, models, app_train) imported from the staged, unmodified reference sources."""
    if not os.path.isfile(os.path.join(MICRONET, "app_layers.py")):
        if os.path.exists(os.path.join(ROOT, "oracle", "_build", "reference_trainer_staged.txt")):
            pytest.fail("build() staged the reference's micronet+ sources but baseline/_ref/micronet+/app_layers.py "
                        "is not there")
        pytest.skip("no reference checkout was at hand when build() ran (baseline/_ref/micronet+ is absent)")
    import self_ops
    assert os.path.dirname(os.path.abspath(self_ops.__file__)).startswith(os.path.join(ROOT, "appmult-aware-retraining_b200"))
    sys.path.append(MICRONET)
    try:
        import app_layers
        import models
        import app_train
    finally:
        sys.path.remove(MICRONET)
    for m in (app_layers, models, app_train):
        assert os.path.abspath(m.__file__).startswith(MICRONET)
    assert app_layers.self_ops is self_ops
    return app_layers, models, app_train


class SmallNet(nn.Module):
    """Two convolutions (one strided, one with bias), pooling and a classifier - every module kind the
    reference's add_quant_op (app_layers.py:285-339) replaces."""

    def __init__(self):
        super().__init__()
        self.c1 = nn.Conv2d(3, 16, 3, padding=1, bias=False)
        self.bn = nn.BatchNorm2d(16)
        self.pool = nn.MaxPool2d(2)
        self.c2 = nn.Conv2d(16, 40, 3, stride=2, padding=1, bias=True)
        self.avg = nn.AvgPool2d(2)
        self.fc = nn.Linear(40 * 4 * 4, 10)

    def forward(self, x):
        x = self.pool(torch.relu(self.bn(self.c1(x))))
        x = self.avg(torch.relu(self.c2(x)))
        return self.fc(x.flatten(1))


def _count_calls(monkeypatch):
    """Counts the calls the reference layer makes into this library's convolution entry points."""
    import approx_ops
    counts = {"fwd": 0, "bwd": 0}
    fwd, bwd = approx_ops.approx_conv2d_forward, approx_ops.approx_conv2d_backward

    def fwd_counted(*a, **k):
        counts["fwd"] += 1
        return fwd(*a, **k)

    def bwd_counted(*a, **k):
        counts["bwd"] += 1
        return bwd(*a, **k)

    monkeypatch.setattr(approx_ops, "approx_conv2d_forward", fwd_counted)
    monkeypatch.setattr(approx_ops, "approx_conv2d_backward", bwd_counted)
    return counts


@pytest.mark.parametrize("bits,ste", [(7, False), (8, False), (7, True)])
def test_reference_layers_on_this_package_match_the_whole_layer_kernels(dev, ref_modules, bits, ste, monkeypatch):
    import self_ops
    from lutgemm_layers import AppConv2d
    app_layers = ref_modules[0]
    fp, ga_t, gb_t = O.synthetic_tables(bits, seed=90 + bits)
    self_ops.set_lookup_tables(dev, fp, ga_t, gb_t, bits)
    monkeypatch.setattr(torch.backends.cudnn, "allow_tf32", False)  # the reference's cross-term convolutions in full fp32
    counts = _count_calls(monkeypatch)
    torch.manual_seed(bits)
    net = SmallNet().to(dev)
    app_layers.prepare(net, inplace=True, a_bits=bits, w_bits=bits, use_ste_gradient=ste)
    net = net.to(dev).train()
    assert isinstance(net.c1, app_layers.ApproxConv2d) and isinstance(net.c2, app_layers.ApproxConv2d)
    assert isinstance(net.fc, app_layers.QuantLinear) and isinstance(net.pool, app_layers.QuantMaxPool2d)
    seen = {}
    hooks = [m.register_forward_hook(lambda mod, inp, out, n=n: seen.__setitem__(n, (inp[0].detach().clone(), out)))
             for n, m in (("c1", net.c1), ("c2", net.c2))]
    opt = torch.optim.Adam(net.parameters(), lr=1e-3, weight_decay=0.0)  # app_train.py:257
    x = torch.randn(6, 3, 32, 32, device=dev)
    target = torch.randint(0, 10, (6,), device=dev)
    for step in range(2):  # the second step exercises the moving-average observer branch
        opt.zero_grad()
        out = net(x + 0.1 * step)
        loss = nn.functional.cross_entropy(out, target)
        for n in seen:
            seen[n][1].retain_grad()
        loss.backward()
        assert torch.isfinite(loss)
        # --- every approximate convolution against this package's whole-layer kernels on the same input -----
        for n, layer in (("c1", net.c1), ("c2", net.c2)):
            xin, yref = seen[n]
            mine = AppConv2d(layer.in_channels, layer.out_channels, layer.kernel_size, layer.stride, layer.padding,
                             layer.dilation, 1, layer.bias is not None, bits, bits, ste,
                             "fused" if ste else "layer").to(dev).eval()
            mine.weight.data.copy_(layer.weight.data)
            if layer.bias is not None:
                mine.bias.data.copy_(layer.bias.data)
            for name in ("activation_scale", "activation_zp_neg", "weight_scale", "weight_zp_neg"):
                getattr(mine, name).copy_(getattr(layer, name).reshape(1))
            xm = xin.clone().requires_grad_(True)
            ym = mine(xm)
            qmax = float((1 << bits) - 1)
            s_a, z_a, s_w, z_w = (float(getattr(layer, k_)) for k_ in ("activation_scale", "activation_zp_neg",
                                                                        "weight_scale", "weight_zp_neg"))
            kdim = layer.in_channels * layer.kernel_size[0] * layer.kernel_size[1]
            mag = s_a * s_w * kdim * (qmax * qmax + (abs(z_a) + abs(z_w)) * qmax + abs(z_a * z_w))
            assert float((yref - ym).detach().abs().max()) <= 4 * 1.2e-7 * mag, (bits, step, n)
            g = yref.grad
            ym.backward(g)
            wg_ref, wg = layer.weight.grad, mine.weight.grad
            # gradients are sums of a LUT term and a zero-point cross term that largely cancel: tolerance relative
            # to the size of the terms (1e-5 of the cross term's magnitude added to that of the result)
            gsum = float(g.abs().sum(dim=(0, 2, 3)).max())
            tol_w = 1e-5 * (float(wg_ref.abs().max()) + 2.0 * abs(s_a * z_a) * gsum)
            assert float((wg_ref - wg).abs().max()) <= tol_w + 1e-30, (bits, step, n)
            if layer.bias is not None:
                assert torch.allclose(layer.bias.grad, mine.bias.grad, rtol=1e-5, atol=1e-6)
        opt.step()
    for h in hooks:
        h.remove()
    assert counts["fwd"] >= 4  # two convolutions, two steps, plus the comparison layers
    assert ste or counts["bwd"] >= 4


def test_reference_trainer_steps_resnet18(dev, ref_modules, monkeypatch, capsys):
    """app_train.calibrate and app_train.train (micronet+/app_train.py:23-46), unmodified, on the reference's
    ResNet-18 (models.resnet18, 100 classes) prepared by the reference's `prepare`, with Adam as in
    app_train.py:257: every convolution runs this library's kernels, the loss is finite and the weights move."""
    import self_ops
    app_layers, models, app_train = ref_modules
    bits = 7
    fp, ga_t, gb_t = O.synthetic_tables(bits, seed=7)
    self_ops.set_lookup_tables(dev, fp, ga_t, gb_t, bits)
    counts = _count_calls(monkeypatch)
    torch.manual_seed(0)
    model = models.resnet18().to(dev)
    app_layers.prepare(model, inplace=True, a_bits=bits, w_bits=bits, q_type=1, q_level=1, weight_observer=0,
                       bn_fuse=False, bn_fuse_calib=False, pretrained_model=True, qaft=False, ptq=False,
                       percentile=0.999999, use_ste_gradient=False)  # the call of app_train.py:234-249
    model = model.to(dev)
    n_convs = sum(isinstance(m, app_layers.ApproxConv2d) for m in model.modules())
    assert n_convs == 20
    gen = torch.Generator().manual_seed(1)
    batches = [(torch.randn(8, 3, 32, 32, generator=gen), torch.randint(0, 100, (8,), generator=gen)) for _ in range(2)]

    class Loader(list):
        dataset = list(range(16))

    loader = Loader(batches)
    before = {k: v.detach().clone() for k, v in model.named_parameters()}
    app_train.calibrate(model, dev, loader)
    assert counts["fwd"] == n_convs * len(batches)
    optimizer = torch.optim.Adam(model.parameters(), lr=1e-3, weight_decay=0.0)
    app_train.train(model, dev, loader, optimizer, 0)
    torch.cuda.synchronize()
    assert counts["fwd"] == 2 * n_convs * len(batches)
    assert counts["bwd"] == n_convs * len(batches)
    printed = capsys.readouterr().out
    assert "Train Epoch 0" in printed and "nan" not in printed.lower()
    moved = [float((p.detach() - before[k]).abs().max()) for k, p in model.named_parameters()]
    # (with random initial weights the gradients of the first layers of this 18-layer network reach ~1e22; their
    # squares overflow Adam's second moment, which freezes those few parameters - in the reference's own setting,
    # a pretrained network, that does not happen; everything else must have moved)
    assert all(np.isfinite(moved)) and np.mean(np.array(moved) > 0.0) > 0.9
