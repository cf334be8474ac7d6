"""Benchmark models built from the shapes the benchmark configurations name (plain PyTorch modules; their
convolutions and linears are swapped for the approximate layers by `lutgemm_layers.prepare`).

`resnet18_cifar` is the CIFAR variant the reference trains (3x3 stem, four stages of two basic blocks,
widths 64/128/256/512, global average pool, linear classifier; cf. micronet+/models.py:151-211).
`resnet50_imagenet` (7x7 stride-2 stem, max pool, bottleneck stages [3,4,6,3], 1000-way classifier) and
`vit_small_16` (patch 16, 12 blocks, width 384, 6 heads, MLP 1536; attention scores and softmax stay exact
fp32, the QKV / projection / MLP linears and the patch embedding are swapped) are the two larger
configurations."""
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


class Bottleneck(nn.Module):
    def __init__(self, cin: int, mid: int, stride: int):
        super().__init__()
        cout = 4 * mid
        self.conv1, self.bn1 = nn.Conv2d(cin, mid, 1, 1, 0, bias=False), nn.BatchNorm2d(mid)
        self.conv2, self.bn2 = nn.Conv2d(mid, mid, 3, stride, 1, bias=False), nn.BatchNorm2d(mid)
        self.conv3, self.bn3 = nn.Conv2d(mid, cout, 1, 1, 0, bias=False), nn.BatchNorm2d(cout)
        self.shortcut = None
        if stride != 1 or cin != cout:
            self.shortcut = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, 0, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        out = F.relu(self.bn1(self.conv1(x)))
        out = F.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        return F.relu(out + (x if self.shortcut is None else self.shortcut(x)))


class ResNetBottleneck(nn.Module):
    def __init__(self, blocks=(3, 4, 6, 3), base: int = 64, num_classes: int = 1000):
        super().__init__()
        self.conv1 = nn.Conv2d(3, base, 7, 2, 3, bias=False)
        self.bn1 = nn.BatchNorm2d(base)
        layers, cin = [], base
        for i, n in enumerate(blocks):
            for j in range(n):
                layers.append(Bottleneck(cin, base << i, 2 if (j == 0 and i > 0) else 1))
                cin = 4 * (base << i)
        self.layers = nn.Sequential(*layers)
        self.fc = nn.Linear(cin, num_classes)
        for m in self.modules():
            if isinstance(m, (nn.Conv2d, nn.Linear)):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.bn1(self.conv1(x))), 3, 2, 1)
        x = self.layers(x)
        return self.fc(F.adaptive_avg_pool2d(x, 1).flatten(1))


def resnet50_imagenet(num_classes: int = 1000, base: int = 64, blocks=(3, 4, 6, 3)) -> ResNetBottleneck:
    return ResNetBottleneck(blocks, base, num_classes)


class ViTBlock(nn.Module):
    def __init__(self, dim: int, heads: int, mlp: int):
        super().__init__()
        self.heads = heads
        self.norm1, self.norm2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.qkv, self.proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        self.fc1, self.fc2 = nn.Linear(dim, mlp), nn.Linear(mlp, dim)

    def forward(self, x):
        B, T, D = x.shape
        q, k, v = self.qkv(self.norm1(x)).view(B, T, 3, self.heads, D // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v)  # exact fp32 scores and softmax
        x = x + self.proj(a.transpose(1, 2).reshape(B, T, D))
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x))))


class ViT(nn.Module):
    def __init__(self, image: int = 224, patch: int = 16, dim: int = 384, depth: int = 12, heads: int = 6,
                 mlp: int = 1536, num_classes: int = 1000):
        super().__init__()
        self.patch_embed = nn.Conv2d(3, dim, patch, patch, 0)
        tokens = (image // patch) ** 2 + 1
        self.cls = nn.Parameter(torch.zeros(1, 1, dim))
        self.pos = nn.Parameter(torch.randn(1, tokens, dim) * 0.02)
        self.blocks = nn.Sequential(*[ViTBlock(dim, heads, mlp) for _ in range(depth)])
        self.norm = nn.LayerNorm(dim)
        self.head = nn.Linear(dim, num_classes)

    def forward(self, x):
        x = self.patch_embed(x).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls.expand(x.shape[0], -1, -1), x], dim=1) + self.pos
        return self.head(self.norm(self.blocks(x))[:, 0])


def vit_small_16(num_classes: int = 1000, **kw) -> ViT:
    return ViT(num_classes=num_classes, **kw)


# name -> (constructor, image shape, classes): the models `lutgemm_train.py` and `bench.py --workload` know
MODELS = {
    "resnet18": (resnet18_cifar, (3, 32, 32), 10),
    "resnet50": (resnet50_imagenet, (3, 224, 224), 1000),
    "vit_s": (vit_small_16, (3, 224, 224), 1000),
}


def lut_macs_per_image(model: nn.Module, image_shape=(3, 32, 32)) -> int:
    """Forward LUT-MACs per image of every Conv2d/Linear in `model` (one per (m, k, n) triple)."""
    total = 0
    hooks = []

    def conv_hook(mod, inp, out):
        nonlocal total
        total += out.shape[2] * out.shape[3] * mod.out_channels * mod.in_channels * mod.kernel_size[0] * mod.kernel_size[1]

    def lin_hook(mod, inp, out):
        nonlocal total
        total += (out.numel() // out.shape[-1]) * mod.in_features * mod.out_features  # rows x K x N

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
