"""Benchmark models built from the shapes the benchmark configuration names (plain PyTorch modules; their
convolutions and linears are swapped for the approximate layers by `lutgemm_layers.prepare`).

`resnet18_cifar` is the CIFAR variant the reference trains (3x3 stem, four stages of two basic blocks,
widths 64/128/256/512, global average pool, linear classifier; cf. micronet+/models.py:151-211)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class BasicBlock(nn.Module):
    def __init__(self, cin: int, cout: int, stride: int):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(cout)
        self.conv2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(cout)
        self.shortcut = None
        if stride != 1 or cin != cout:
            self.shortcut = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, 0, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        out = F.relu(self.bn1(self.conv1(x)))
        out = self.bn2(self.conv2(out))
        return F.relu(out + (x if self.shortcut is None else self.shortcut(x)))


class ResNetCifar(nn.Module):
    def __init__(self, blocks=(2, 2, 2, 2), widths=(64, 128, 256, 512), num_classes: int = 10):
        super().__init__()
        self.conv1 = nn.Conv2d(3, widths[0], 3, 1, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(widths[0])
        layers, cin = [], widths[0]
        for i, (n, w) in enumerate(zip(blocks, widths)):
            for j in range(n):
                layers.append(BasicBlock(cin, w, 2 if (j == 0 and i > 0) else 1))
                cin = w
        self.layers = nn.Sequential(*layers)
        self.fc = nn.Linear(cin, num_classes)
        for m in self.modules():
            if isinstance(m, (nn.Conv2d, nn.Linear)):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def forward(self, x):
        x = F.relu(self.bn1(self.conv1(x)))
        x = self.layers(x)
        x = F.adaptive_avg_pool2d(x, 1).flatten(1)
        return self.fc(x)


def resnet18_cifar(num_classes: int = 10) -> ResNetCifar:
    return ResNetCifar((2, 2, 2, 2), (64, 128, 256, 512), num_classes)


def lut_macs_per_image(model: nn.Module, image_shape=(3, 32, 32)) -> int:
    """Forward LUT-MACs per image of every Conv2d/Linear in `model` (one per (m, k, n) triple)."""
    total = 0
    hooks = []

    def conv_hook(mod, inp, out):
        nonlocal total
        total += out.shape[2] * out.shape[3] * mod.out_channels * mod.in_channels * mod.kernel_size[0] * mod.kernel_size[1]

    def lin_hook(mod, inp, out):
        nonlocal total
        total += mod.in_features * mod.out_features

    for m in model.modules():
        if isinstance(m, nn.Conv2d):
            hooks.append(m.register_forward_hook(conv_hook))
        elif isinstance(m, nn.Linear):
            hooks.append(m.register_forward_hook(lin_hook))
    was = model.training
    model.eval()
    with torch.no_grad():
        model(torch.zeros(1, *image_shape, device=next(model.parameters()).device))
    model.train(was)
    for h in hooks:
        h.remove()
    return total
