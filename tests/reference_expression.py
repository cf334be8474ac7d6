"""Test-side restatement of the reference's layer arithmetic, used as the expected value of the whole-layer
kernels.  Test infrastructure only: nothing in the package imports it.

`approx_conv_layer` follows ApproxConv2d.forward, micronet+/app_layers.py:147-150 (quantize_v2: affine map,
straight-through rounding, clamp) and :163-184 (LUT convolution of the codes plus the three zero-point cross
terms as exact library convolutions, one common scale, bias last).  `approx_linear_layer` is the same
expression for a linear layer (the reference's QuantLinear, :78-113, never reaches the approximate
multiplier; the benchmark configurations route linears through it, so the conv expression is carried over
term by term with F.linear in place of F.conv2d)."""
import torch
import torch.nn.functional as F


def codes_ste(t, scale, zp_neg, qmax):
    """Float tensor of integer codes; d codes / d t = 1 / scale inside the clamp range, 0 outside."""
    affine = t / scale - zp_neg
    return torch.clamp(affine - affine.detach() + torch.round(affine), 0, qmax)


def approx_conv_layer(conv_op, x, weight, bias, s_a, z_a, s_w, z_w, a_qmax, w_qmax, stride, padding, dilation):
    geo = dict(bias=None, stride=stride, padding=padding, dilation=dilation, groups=1)
    xq = codes_ste(x, s_a, z_a, a_qmax)
    wq = codes_ste(weight, s_w, z_w, w_qmax)
    zw_img, za_img = torch.full_like(wq, float(z_w)), torch.full_like(xq, float(z_a))
    acc = conv_op(xq, wq, **geo) + F.conv2d(xq, zw_img, **geo) + F.conv2d(za_img, wq, **geo) \
        + F.conv2d(za_img, zw_img, **geo)
    out = s_a * s_w * acc
    if bias is not None:
        out = out + bias.view(1, -1, 1, 1)
    return out


def approx_linear_layer(gemm_op, x2, weight, bias, s_a, z_a, s_w, z_w, a_qmax, w_qmax):
    xq = codes_ste(x2, s_a, z_a, a_qmax)
    wq = codes_ste(weight, s_w, z_w, w_qmax)
    zw_mat, za_mat = torch.full_like(wq, float(z_w)), torch.full_like(xq, float(z_a))
    acc = gemm_op(xq, wq.t()) + F.linear(xq, zw_mat) + F.linear(za_mat, wq) + F.linear(za_mat, zw_mat)
    out = s_a * s_w * acc
    if bias is not None:
        out = out + bias
    return out
