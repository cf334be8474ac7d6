"""Approximate-multiplier layers on top of the LUT-GEMM ops: `AppConv2d`, `AppLinear`, `prepare`.

They follow the layer contract of the reference's `ApproxConv2d` (micronet+/app_layers.py:116-185):
activation and weight are fake-quantised to unsigned b-bit codes with asymmetric (min/max) ranges -
an exponential-moving-average observer for activations (momentum 0.1, :38-53) and a running min/max
observer for weights (:21-35), scales and zero points refreshed every training step (:155-160) - the
code x code product goes through the approximate multiplier, and the three zero-point cross terms of

    (s_a (q_a + z_a)) * (s_w (q_w + z_w)) = s_a s_w (q_a q_w + z_w q_a + z_a q_w + z_a z_w)

are exact (:175-181, equation 8 of the paper).  Rounding uses the straight-through estimator (:147-150).

Differences from the reference, on purpose: the cross terms are computed as window sums (a one-channel
box filter of the channel-summed codes, one batch-independent convolution of a ones image with the
weight codes, a tap count) instead of three full convolutions - identical in exact arithmetic; linear
layers go through the approximate multiplier too (`AppLinear`), which the reference's `QuantLinear`
(:78-113) does not do; the convolution can use the fused implicit-im2col kernels instead of
`F.unfold` (conv_impl="fused"), and the whole layer - quantisation, convolution, cross terms, scaling - can
run as two kernels in the forward pass - quantisation prologue, LUT convolution with the de-quantisation
applied where it stores (conv_impl="layer").  Spatial padding is code 0 and therefore contributes LUT[0][w], as in the reference
(self_ops/ops_py/approx_ops.py:556)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

import approx_ops
import self_ops
from self_ops.ops_py import approx_ops as _ops_state


def _out_hw(H, W, kh, kw, stride, pad, dil):
    return (H + 2 * pad - dil * (kh - 1) - 1) // stride + 1, (W + 2 * pad - dil * (kw - 1) - 1) // stride + 1


# The zero-point cross terms are window sums.  They are evaluated with slices and small fp32 matrix products
# rather than library convolutions, which may round their inputs to TF32 (channel sums of codes need 16 bits).
def _tap_slices(geom):
    H, W, kh, kw, stride, pad, dil = geom
    Ho, Wo = _out_hw(H, W, kh, kw, stride, pad, dil)
    for i in range(kh):
        for j in range(kw):
            yield (slice(i * dil, i * dil + (Ho - 1) * stride + 1, stride),
                   slice(j * dil, j * dil + (Wo - 1) * stride + 1, stride))


def _window_sum(img, geom):
    """[B, H, W] -> [B, Ho, Wo]: sum of the kernel window at every output position (zero padding).  PyTorch
    statement of what `approx_ops.layer_window_sum` computes in one kernel; the tests hold the kernel against it."""
    pad = geom[5]
    padded = F.pad(img, (pad, pad, pad, pad))
    out = None
    for sh, sw in _tap_slices(geom):
        out = padded[:, sh, sw].clone() if out is None else out.add_(padded[:, sh, sw])
    return out


def _window_sum_adjoint(g, geom):
    """[B, Ho, Wo] -> [B, H, W]: adjoint of `_window_sum`."""
    H, W, pad = geom[0], geom[1], geom[5]
    padded = torch.zeros(g.shape[0], H + 2 * pad, W + 2 * pad, dtype=g.dtype, device=g.device)
    for sh, sw in _tap_slices(geom):
        padded[:, sh, sw] += g
    return padded[:, pad:pad + H, pad:pad + W].contiguous()


_VALID_TAPS = {}


def _valid_taps(geom, device):
    """[kh*kw, Ho*Wo] fp32: 1 where tap (i, j) of output position l falls inside the image (geometry only)."""
    key = (geom, str(device))
    if key not in _VALID_TAPS:
        H, W, kh, kw, stride, pad, dil = geom
        padded = F.pad(torch.ones(1, H, W, device=device), (pad, pad, pad, pad))
        _VALID_TAPS[key] = torch.stack([padded[0, sh, sw].reshape(-1) for sh, sw in _tap_slices(geom)]).contiguous()
    return _VALID_TAPS[key]


class _AppConvLayer(torch.autograd.Function):
    """The whole approximate convolution layer around the fused implicit-im2col kernels: quantisation prologue
    (one pass over the activations, any dense layout), LUT convolution, de-quantisation epilogue with the three
    zero-point cross terms (one pass over the accumulators); backward: LUT gradients on the un-scaled grad_out,
    then one pass that applies clamp mask, weight scale and the cross-term gradient in the layout of the input.
    Same values and gradients as the expression in `AppConv2d.forward` evaluated by autograd."""

    @staticmethod
    def forward(ctx, x, weight, bias, quant, a_qmax, w_qmax, stride, padding, dilation):
        # quant = [s_a, z_a, s_w, z_w] (one device tensor, so nothing here synchronises with the host)
        if _ops_state.lut_appmult is None:
            raise RuntimeError("lookup tables are not initialised: call init_lookup_tables first")
        s_a, z_a, s_w, z_w = (quant[i:i + 1] for i in range(4))
        B, Cin, H, W = x.shape
        Cout, _, kh, kw = weight.shape
        Ho, Wo = _out_hw(H, W, kh, kw, stride, padding, dilation)
        L, M = Ho * Wo, B * Ho * Wo
        if not (x.is_contiguous() or x.is_contiguous(memory_format=torch.channels_last)):
            x = x.contiguous()
        codes, chansum = approx_ops.quantize_activations(x, s_a, z_a, a_qmax)
        # weight codes as the [K, Cout] matrix of the LUT kernels + their per-tap sums; the two z_a cross terms per
        # output position; the window sums of the channel-summed activation codes (one small kernel each)
        wmat, wsum = approx_ops.layer_weight_prep(weight, quant, w_qmax)
        sumw_t, taps = approx_ops.layer_cross_terms(wsum, Cin, H, W, kh, kw, stride, padding, dilation)
        box = approx_ops.layer_window_sum(chansum, kh, kw, stride, padding, dilation)
        # one kernel: LUT convolution with the de-quantisation applied to the sums in registers
        out, codes_t = approx_ops.approx_conv2d_forward_layer(codes, wmat, _ops_state.lut_appmult, kh, kw, stride, padding,
                                                              dilation, box, sumw_t, taps, s_a, s_w, z_a, z_w, bias)
        ctx.save_for_backward(x, codes, wmat, weight, quant)
        ctx.codes_t = codes_t  # transposed unfolded codes of the forward kernel: the grad_w kernel reuses them
        ctx.cfg = (a_qmax, w_qmax, stride, padding, dilation, Ho, Wo, bias is not None)
        return out.view(B, Ho, Wo, Cout).permute(0, 3, 1, 2)  # NCHW view of channels-last memory

    @staticmethod
    def backward(ctx, g_out):
        x, codes, wmat, weight, quant = ctx.saved_tensors
        a_qmax, w_qmax, stride, padding, dilation, Ho, Wo, has_bias = ctx.cfg
        s_a, z_a, s_w, z_w = (quant[i:i + 1] for i in range(4))
        B, Cin, H, W = x.shape
        Cout, _, kh, kw = weight.shape
        L, M = Ho * Wo, B * Ho * Wo
        gy = g_out.permute(0, 2, 3, 1).reshape(M, Cout).contiguous()  # a view when g_out is channels-last
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gcodes = torch.empty(codes.shape, dtype=torch.float32, device=gy.device) if need_x else None
        gwmat = torch.empty(wmat.shape, dtype=torch.float32, device=gy.device) if need_w else None
        if need_x or need_w:
            approx_ops.approx_conv2d_backward(gy, codes, wmat, gcodes, gwmat, _ops_state.lut_grad_a, _ops_state.lut_grad_b,
                                              kh, kw, stride, padding, dilation, codes_t=ctx.codes_t if need_w else None)
        ctx.codes_t = None
        geom = (H, W, kh, kw, stride, padding, dilation)
        gx = gw = gb = None
        if need_x:
            # cross term z_w * box(q_a): its adjoint spreads the channel sum of grad_out over each window
            box_t = approx_ops.layer_window_sum_adjoint(gy.sum(dim=1).view(B, Ho, Wo), H, W, kh, kw, stride, padding, dilation)
            gx = approx_ops.quantize_activations_backward(x, s_a, z_a, a_qmax, gcodes, box_t, s_w, z_w)
        if need_w:
            # cross term z_a * sum_w(q_w): every input channel of a tap sees the same sum of grad_out; then clamp
            # mask and activation scale in one pass
            gsum_b = gy.view(B, L, Cout).sum(dim=0)                                          # [L, Cout]
            tap_grad = (_valid_taps(geom, gy.device) @ gsum_b).t().contiguous()              # [Cout, kh*kw]
            gw = approx_ops.layer_weight_grad(gwmat, tap_grad, weight, quant, w_qmax)
        if has_bias and ctx.needs_input_grad[2]:
            gb = gy.sum(dim=0)
        return gx, gw, gb, None, None, None, None, None, None


class _AppLinearLayer(torch.autograd.Function):
    """The whole approximate linear layer: quantisation prologue, LUT-GEMM, de-quantisation epilogue with the
    zero-point cross terms (one output position, so the window sums are a row sum of the activation codes, a
    column sum of the weight codes and K), and their backward.  Same values and gradients as the expression
    in `AppLinear.forward` evaluated by autograd."""

    @staticmethod
    def forward(ctx, x2, weight, bias, quant, a_qmax, w_qmax):
        if _ops_state.lut_appmult is None:
            raise RuntimeError("lookup tables are not initialised: call init_lookup_tables first")
        s_a, z_a, s_w, z_w = (quant[i:i + 1] for i in range(4))
        M, K = x2.shape
        N = weight.shape[0]
        x2 = x2.contiguous()
        # rows as the channel dimension of a one-row image: the kernel's 32 x 32 tiles are then all payload
        codes, _ = approx_ops.quantize_activations(x2.view(1, M, 1, K), s_a, z_a, a_qmax, want_chansum=False)
        codes = codes.view(M, K)
        wmat, wsum = approx_ops.layer_weight_prep(weight.view(N, K, 1, 1), quant, w_qmax)  # [K, N] codes, [N, 1] sums
        box = codes.sum(dim=1, dtype=torch.float32)
        sumw_t = wsum.view(1, N)
        taps = torch.full((1,), float(K), device=x2.device)
        out, codes_t = approx_ops.approx_gemm_forward_layer(codes, wmat, _ops_state.lut_appmult, box, sumw_t, taps, s_a, s_w,
                                                            z_a, z_w, bias)
        ctx.save_for_backward(x2, codes, wmat, weight, quant)
        ctx.codes_t = codes_t  # transposed codes of the forward kernel: the grad_w kernel reuses them
        ctx.cfg = (a_qmax, w_qmax, bias is not None)
        return out

    @staticmethod
    def backward(ctx, g_out):
        x2, codes, wmat, weight, quant = ctx.saved_tensors
        a_qmax, w_qmax, has_bias = ctx.cfg
        s_a, z_a, s_w, z_w = (quant[i:i + 1] for i in range(4))
        M, K = x2.shape
        gy = g_out.contiguous()
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        ga = torch.empty((M, K), dtype=torch.float32, device=gy.device)
        gw = torch.empty(wmat.shape, dtype=torch.float32, device=gy.device)
        approx_ops.approx_gemm_backward(gy, codes, wmat, ga, gw, _ops_state.lut_grad_a, _ops_state.lut_grad_b,
                                        codes_t=ctx.codes_t)
        ctx.codes_t = None
        gx = gwt = gb = None
        if need_x:
            ga.add_(z_w * gy.sum(dim=1, keepdim=True))  # cross term z_w * rowsum(q_a)
            gx = approx_ops.quantize_activations_backward(x2.view(1, M, 1, K), s_a, z_a, a_qmax, ga.view(1, M, 1, K),
                                                          None, s_w, z_w).view(M, K)
        if need_w:
            # cross term z_a * colsum(q_w), clamp mask and activation scale in one pass
            gwt = approx_ops.layer_weight_grad(gw, gy.sum(dim=0).view(-1, 1).contiguous(), weight.view(-1, K, 1, 1), quant,
                                               w_qmax).view(weight.shape)
        if has_bias and ctx.needs_input_grad[2]:
            gb = gy.sum(dim=0)
        return gx, gwt, gb, None, None, None


class _MinMax(nn.Module):
    """Running min/max (weights) or exponential moving average of min/max (activations)."""

    def __init__(self, momentum: float | None):
        super().__init__()
        self.momentum = momentum
        self.register_buffer("min_val", torch.zeros(1))
        self.register_buffer("max_val", torch.zeros(1))
        self.register_buffer("seen", torch.zeros(1))

    def state(self):
        return self.min_val, self.max_val, self.seen

    @torch.no_grad()
    def update(self, x: torch.Tensor) -> None:
        lo, hi = torch.aminmax(x)
        first = self.seen == 0
        if self.momentum is None:
            new_lo, new_hi = torch.minimum(lo, self.min_val), torch.maximum(hi, self.max_val)
        else:
            new_lo = (1 - self.momentum) * self.min_val + self.momentum * lo
            new_hi = (1 - self.momentum) * self.max_val + self.momentum * hi
        self.min_val.copy_(torch.where(first, lo, new_lo))
        self.max_val.copy_(torch.where(first, hi, new_hi))
        self.seen.fill_(1)


class _AppQuant(nn.Module):
    """Shared quantisation state of the approximate layers."""

    def _init_quant(self, a_bits: int, w_bits: int) -> None:
        self.act_range = _MinMax(momentum=0.1)
        self.weight_range = _MinMax(momentum=None)
        self.a_qmax = float((1 << a_bits) - 1)
        self.w_qmax = float((1 << w_bits) - 1)
        # {activation scale, activation zero point, weight scale, weight zero point}: one buffer, so that the kernels
        # read all four from one place; the names below are views into it
        self.register_buffer("quant", torch.tensor([1.0, 0.0, 1.0, 0.0]))

    activation_scale = property(lambda self: self.quant[0:1])
    activation_zp_neg = property(lambda self: self.quant[1:2])
    weight_scale = property(lambda self: self.quant[2:3])
    weight_zp_neg = property(lambda self: self.quant[3:4])

    def _refresh(self, x: torch.Tensor, w: torch.Tensor, fused: bool = False) -> None:
        if not self.training:
            return
        if fused:
            # the two range reductions, then ONE launch for both observers and the four quantisation parameters
            a_lo, a_hi = torch.aminmax(x.detach())
            w_lo, w_hi = torch.aminmax(w.detach())
            approx_ops.layer_update_ranges(a_lo, a_hi, w_lo, w_hi, self.act_range.state(), self.weight_range.state(),
                                           self.act_range.momentum, self.a_qmax, self.w_qmax, self.quant)
            return
        eps = torch.finfo(torch.float32).eps
        with torch.no_grad():
            self.act_range.update(x)
            self.weight_range.update(w)
            self.activation_scale.copy_(torch.clamp((self.act_range.max_val - self.act_range.min_val) / self.a_qmax, min=eps))
            self.activation_zp_neg.copy_(torch.round(self.act_range.min_val / self.activation_scale))
            self.weight_scale.copy_(torch.clamp((self.weight_range.max_val - self.weight_range.min_val) / self.w_qmax, min=eps))
            self.weight_zp_neg.copy_(torch.round(self.weight_range.min_val / self.weight_scale))

    @staticmethod
    def _codes(x: torch.Tensor, scale: torch.Tensor, zp_neg: torch.Tensor, qmax: float) -> torch.Tensor:
        """Float tensor of integer codes in [0, qmax]; gradient of the rounding is the identity."""
        q = x / scale - zp_neg
        q = q + (torch.round(q) - q).detach()
        return torch.clamp(q, 0.0, qmax)


class AppConv2d(nn.Conv2d, _AppQuant):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 a_bits=7, w_bits=7, use_ste_gradient=False, conv_impl="fused"):
        nn.Conv2d.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias)
        assert groups == 1, "groups is not supported in approximate convolution"
        self._init_quant(a_bits, w_bits)
        self.use_ste_gradient = use_ste_gradient
        self.conv_impl = conv_impl

    def _approx_conv(self, xq, wq):
        kw = dict(bias=None, stride=self.stride, padding=self.padding, dilation=self.dilation, groups=1)
        if self.conv_impl == "unfold":  # the reference's F.unfold formulation, for comparisons
            gemm = self_ops.approx_gemm_baseline_op if self.use_ste_gradient else self_ops.approx_gemm_op
            return _ops_state.unfold_conv2d(gemm, xq, wq, **kw)
        if self.use_ste_gradient:
            return self_ops.approx_conv2d_baseline_op(xq, wq, **kw)
        return self_ops.approx_conv2d_op(xq, wq, **kw)

    def forward(self, x):
        if self.conv_impl == "layer" and not self.use_ste_gradient and x.is_cuda:
            self._refresh(x, self.weight, fused=True)
            # (a copy: the layer's buffer is overwritten by the next step's refresh before this step's backward is
            # necessarily done with it only when forward passes are stacked; four floats)
            return _AppConvLayer.apply(x, self.weight, self.bias, self.quant.clone(), self.a_qmax, self.w_qmax,
                                       self.stride[0], self.padding[0], self.dilation[0])
        self._refresh(x, self.weight)
        xq = self._codes(x, self.activation_scale, self.activation_zp_neg, self.a_qmax)
        wq = self._codes(self.weight, self.weight_scale, self.weight_zp_neg, self.w_qmax)
        geo = dict(stride=self.stride, padding=self.padding, dilation=self.dilation)
        kh, kw_ = self.kernel_size
        ones_k = torch.ones(1, 1, kh, kw_, device=x.device, dtype=x.dtype)
        ones_img = torch.ones(1, 1, x.shape[2], x.shape[3], device=x.device, dtype=x.dtype)
        # z_w * sum_{valid taps, channels} q_a ; z_a * sum_{valid taps} q_w ; z_a z_w * (#valid taps * Cin)
        box_a = F.conv2d(xq.sum(dim=1, keepdim=True), ones_k, **geo)
        sum_w = F.conv2d(ones_img.expand(1, self.in_channels, -1, -1), wq, **geo)
        taps = F.conv2d(ones_img, ones_k, **geo) * float(self.in_channels)
        acc = self._approx_conv(xq, wq) + self.weight_zp_neg * box_a + self.activation_zp_neg * sum_w \
            + (self.activation_zp_neg * self.weight_zp_neg) * taps
        out = (self.activation_scale * self.weight_scale) * acc
        if self.bias is not None:
            out = out + self.bias.view(1, -1, 1, 1)
        return out


class AppLinear(nn.Linear, _AppQuant):
    def __init__(self, in_features, out_features, bias=True, a_bits=7, w_bits=7, use_ste_gradient=False,
                 impl="ops"):
        nn.Linear.__init__(self, in_features, out_features, bias)
        self._init_quant(a_bits, w_bits)
        self.use_ste_gradient = use_ste_gradient
        self.impl = impl  # "ops": PyTorch quantisation around the LUT-GEMM op; "layer": the whole-layer kernels

    def forward(self, x):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if self.impl == "layer" and not self.use_ste_gradient and x.is_cuda:
            self._refresh(x, self.weight, fused=True)
            out = _AppLinearLayer.apply(x2, self.weight, self.bias, self.quant.clone(), self.a_qmax, self.w_qmax)
            return out.reshape(*lead, self.out_features)
        self._refresh(x, self.weight)
        xq = self._codes(x2, self.activation_scale, self.activation_zp_neg, self.a_qmax)
        wq = self._codes(self.weight, self.weight_scale, self.weight_zp_neg, self.w_qmax)
        gemm = self_ops.approx_gemm_baseline_op if self.use_ste_gradient else self_ops.approx_gemm_op
        acc = gemm(xq, wq.t()) + self.weight_zp_neg * xq.sum(dim=1, keepdim=True) \
            + self.activation_zp_neg * wq.sum(dim=1).unsqueeze(0) \
            + (self.activation_zp_neg * self.weight_zp_neg) * float(self.in_features)
        out = (self.activation_scale * self.weight_scale) * acc
        if self.bias is not None:
            out = out + self.bias
        return out.reshape(*lead, self.out_features)


def prepare(model: nn.Module, a_bits: int = 7, w_bits: int = 7, use_ste_gradient: bool = False,
            conv_impl: str = "fused", linear: bool = True) -> nn.Module:
    """Swaps every nn.Conv2d (and, with linear=True, nn.Linear) of `model` in place for its approximate
    counterpart; parameters are shared with the replaced module (cf. add_quant_op,
    micronet+/app_layers.py:270-339)."""
    for name, child in list(model.named_children()):
        if isinstance(child, (AppConv2d, AppLinear)):
            continue
        if isinstance(child, nn.Conv2d) and child.groups == 1:
            new = AppConv2d(child.in_channels, child.out_channels, child.kernel_size, child.stride, child.padding,
                            child.dilation, 1, child.bias is not None, a_bits, w_bits, use_ste_gradient, conv_impl)
            new.weight = child.weight
            new.bias = child.bias
            setattr(model, name, new.to(child.weight.device))
        elif linear and isinstance(child, nn.Linear):
            new = AppLinear(child.in_features, child.out_features, child.bias is not None, a_bits, w_bits, use_ste_gradient,
                            "layer" if conv_impl == "layer" else "ops")
            new.weight = child.weight
            new.bias = child.bias
            setattr(model, name, new.to(child.weight.device))
        else:
            prepare(child, a_bits, w_bits, use_ste_gradient, conv_impl, linear)
    return model
