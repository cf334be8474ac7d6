"""Python operator layer over the compiled `approx_ops` module - same public functions, argument
meaning and autograd contract as the reference's self_ops/ops_py/approx_ops.py:

    init_lookup_tables(device, file_name, quantization_bit)            (reference :18-79)
    approx_gemm_op(a, b) / approx_gemm_baseline_op(a, b)               (reference :148-264)
    approx_conv2d_op / approx_conv2d_baseline_op(input, weight, bias,
                                 stride, padding, dilation, groups)    (reference :530-619)

Inputs are float tensors that hold integer codes in [0, 2^bits); outputs are fp32.  Gradients flow
to both operands: through the difference-based gradient tables for the `*_op` functions and through
the straight-through estimator (two exact matmuls on the float codes) for the `*_baseline_op` ones.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F
from torch.autograd import Function

import approx_ops  # the ctypes-backed module next to this package (no fallback if it cannot load)

# Module-level tables, same names as the reference keeps (self_ops/ops_py/approx_ops.py:13-15).
lut_appmult = None   # uint16 [LUT_ELEM_NUM]  forward products
lut_grad_a = None    # int16  [LUT_ELEM_NUM]  round(16 * dAM/d first operand)
lut_grad_b = None    # int16  [LUT_ELEM_NUM]  round(16 * dAM/d second operand)

_TAIL_PAD = {4: 718, 6: 830, 7: 638, 8: 0}
_SECTIONS = (
    ("LUT for approximate multiplier:", 0),
    ("LUT for the gradient of the approximate multiplier w.r.t. the first operand:", 1),
    ("LUT for the gradient of the approximate multiplier w.r.t. the second operand:", 2),
)


def _geometry(quantization_bit: int):
    if quantization_bit not in _TAIL_PAD:
        raise NotImplementedError(f"quantization_bit = {quantization_bit} is not supported")
    q = 1 << quantization_bit
    row, col = q + 1, q + 2
    return q, row, col, row * col + _TAIL_PAD[quantization_bit]


def _pack(dense: np.ndarray, quantization_bit: int, np_dtype) -> np.ndarray:
    q, row, col, elems = _geometry(quantization_bit)
    flat = np.zeros(elems, dtype=np_dtype)
    flat[: row * col].reshape(row, col)[:q, :q] = dense
    return flat


def parse_lut_file(file_name: str, quantization_bit: int):
    """Reads the three `a b value` sections of a LUT text file into dense int64 [2^b, 2^b] arrays.
    Header lines before the first section title are ignored; a missing section stays zero."""
    q = 1 << quantization_bit
    tabs = [np.zeros((q, q), np.int64) for _ in range(3)]
    with open(file_name, "r") as f:
        text = f.read()
    marks = sorted((text.find(title), sec, len(title)) for title, sec in _SECTIONS if text.find(title) >= 0)
    for i, (pos, sec, tlen) in enumerate(marks):
        end = marks[i + 1][0] if i + 1 < len(marks) else len(text)
        vals = np.array(text[pos + tlen:end].split(), dtype=np.int64)
        if vals.size % 3:
            raise ValueError(f"{file_name}: section {sec} is not a list of `a b value` triples")
        vals = vals.reshape(-1, 3)
        if vals.size and (vals[:, :2].min() < 0 or vals[:, :2].max() >= q):
            raise ValueError(f"{file_name}: operand outside [0, {q}) - wrong quantization_bit?")
        tabs[sec][vals[:, 0], vals[:, 1]] = vals[:, 2]
    return tabs


def set_lookup_tables(device, fp, grad_a, grad_b, quantization_bit: int) -> None:
    """Installs dense [2^b, 2^b] tables (forward products, 16x gradients as integers) as the module's
    lookup tables on `device`, in the padded flat wire format the compiled operators take."""
    global lut_appmult, lut_grad_a, lut_grad_b
    fp, grad_a, grad_b = (np.asarray(t) for t in (fp, grad_a, grad_b))
    if fp.min() < 0 or fp.max() > 0xFFFF:
        raise ValueError("forward table entries must fit uint16")
    for g in (grad_a, grad_b):
        if g.min() < -32768 or g.max() > 32767:
            raise ValueError("gradient table entries must fit int16")
    lut_appmult = torch.from_numpy(_pack(fp, quantization_bit, np.uint16)).to(device)
    lut_grad_a = torch.from_numpy(_pack(grad_a, quantization_bit, np.int16)).to(device)
    lut_grad_b = torch.from_numpy(_pack(grad_b, quantization_bit, np.int16)).to(device)


def init_lookup_tables(device, file_name, quantization_bit):
    """Loads a `*_lutfp+bp_*.txt` file into the module's lookup tables on `device`."""
    print(f"Initializing lookup tables from {file_name}...")
    fp, ga, gb = parse_lut_file(file_name, quantization_bit)
    set_lookup_tables(device, fp, ga, gb, quantization_bit)


def _forward_codes(a_u8: torch.Tensor, b_u8: torch.Tensor) -> torch.Tensor:
    if lut_appmult is None:
        raise RuntimeError("lookup tables are not initialised: call init_lookup_tables first")
    c = torch.empty((a_u8.shape[0], b_u8.shape[1]), dtype=torch.uint32, device=a_u8.device)
    approx_ops.approx_gemm_forward(a_u8, b_u8, c, lut_appmult)
    return c.to(torch.float32)


class ApproxGemm(Function):
    """c = LUT-GEMM(a, b); backward through the gradient tables (reference ApproxGemm, :148-205)."""

    @staticmethod
    def forward(ctx, a, b):
        a_u8 = a.to(torch.uint8).contiguous()
        b_u8 = b.to(torch.uint8).contiguous()
        ctx.save_for_backward(a_u8, b_u8)
        return _forward_codes(a_u8, b_u8)

    @staticmethod
    def backward(ctx, g_c):
        assert g_c.dtype == torch.float32
        a_u8, b_u8 = ctx.saved_tensors
        g_a = torch.empty(a_u8.shape, dtype=torch.float32, device=g_c.device)
        g_b = torch.empty(b_u8.shape, dtype=torch.float32, device=g_c.device)
        approx_ops.approx_gemm_backward(g_c.contiguous(), a_u8, b_u8, g_a, g_b, lut_grad_a, lut_grad_b)
        return g_a, g_b


class ApproxGemmBaseline(Function):
    """Same forward; straight-through backward g_a = g_c b^T, g_b = a^T g_c on the float codes
    (reference ApproxGemmBaseline, :210-262)."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return _forward_codes(a.to(torch.uint8).contiguous(), b.to(torch.uint8).contiguous())

    @staticmethod
    def backward(ctx, g_c):
        assert g_c.dtype == torch.float32
        a, b = ctx.saved_tensors
        g_c = g_c.contiguous()
        return torch.matmul(g_c, b.t()), torch.matmul(a.t(), g_c)


approx_gemm_op = ApproxGemm.apply
approx_gemm_baseline_op = ApproxGemmBaseline.apply


def unfold_conv2d(gemm_op, input, weight, bias, stride, padding, dilation, groups):
    """The reference's formulation of the convolution (self_ops/ops_py/approx_ops.py:545-571): pad with code 0,
    `F.unfold`, one LUT-GEMM on the materialised [B*Ho*Wo, Cin*kh*kw] matrix.  Kept as the comparison the
    tests hold the fused kernels against; the public ops below do not use it."""
    assert bias is None, "bias is not supported in approximate convolution"
    assert groups == 1, "groups is not supported in approximate convolution"
    s, p, d = stride[0], padding[0], dilation[0]
    B, Cin, H, W = input.shape
    Cout, _, kh, kw = weight.shape
    Ho = (H + 2 * p - d * (kh - 1) - 1) // s + 1
    Wo = (W + 2 * p - d * (kw - 1) - 1) // s + 1
    # spatial padding is CODE 0 (it looks up LUT[0][w]), rows ordered (b, oh, ow), K ordered (cin, kh, kw)
    cols = F.unfold(F.pad(input, (p, p, p, p), value=0.0), kernel_size=(kh, kw), dilation=d, stride=s)
    a = cols.transpose(1, 2).reshape(B * Ho * Wo, Cin * kh * kw)
    out = gemm_op(a, weight.reshape(Cout, -1).t())
    return out.view(B, Ho * Wo, Cout).transpose(1, 2).reshape(B, Cout, Ho, Wo)


class ApproxConv2dFused(Function):
    """Approximate convolution on the convolution entry points of the library: the fp32 unfolded activations
    the reference materialises twice (:556-563) never exist.  Large layers write ONE uint8 copy of the unfolded
    codes, transposed ([K][M], a quarter of one fp32 unfold), which the forward and the weight-gradient kernels
    both read; small layers gather the codes from the NCHW image inside the kernels' operand loaders.  Same
    values and gradients as the reference's `approx_conv2d_op` (unfold + LUT-GEMM)."""

    @staticmethod
    def forward(ctx, input, weight, stride, padding, dilation):
        B, Cin, H, W = input.shape
        Cout, _, kh, kw = weight.shape
        x_u8 = input.to(torch.uint8).contiguous()
        wmat = weight.reshape(Cout, -1).t().to(torch.uint8).contiguous()  # [K, Cout], K ordered (cin, kh, kw)
        Ho = (H + 2 * padding - dilation * (kh - 1) - 1) // stride + 1
        Wo = (W + 2 * padding - dilation * (kw - 1) - 1) // stride + 1
        if lut_appmult is None:
            raise RuntimeError("lookup tables are not initialised: call init_lookup_tables first")
        y = torch.empty((B * Ho * Wo, Cout), dtype=torch.uint32, device=input.device)
        ctx.codes_t = approx_ops.approx_conv2d_forward(x_u8, wmat, y, lut_appmult, kh, kw, stride, padding, dilation)
        ctx.save_for_backward(x_u8, wmat)
        ctx.geom = (kh, kw, stride, padding, dilation, tuple(weight.shape), Ho, Wo)
        # rows are (b, oh, ow): an NCHW tensor in channels-last memory, no copy
        return y.to(torch.float32).view(B, Ho, Wo, Cout).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, g_out):
        x_u8, wmat = ctx.saved_tensors
        kh, kw, stride, padding, dilation, wshape, Ho, Wo = ctx.geom
        B, Cout = x_u8.shape[0], wshape[0]
        gy = g_out.permute(0, 2, 3, 1).reshape(B * Ho * Wo, Cout).contiguous()
        # a gradient nobody asked for (e.g. w.r.t. the input image of the first layer) is not computed
        gx = torch.empty(x_u8.shape, dtype=torch.float32, device=gy.device) if ctx.needs_input_grad[0] else None
        gw = torch.empty(wmat.shape, dtype=torch.float32, device=gy.device) if ctx.needs_input_grad[1] else None
        if gx is not None or gw is not None:
            approx_ops.approx_conv2d_backward(gy, x_u8, wmat, gx, gw, lut_grad_a, lut_grad_b, kh, kw, stride, padding,
                                              dilation, codes_t=ctx.codes_t if gw is not None else None)
        ctx.codes_t = None
        return gx, (gw.t().reshape(wshape) if gw is not None else None), None, None, None


def approx_conv2d_op(input, weight, bias, stride, padding, dilation, groups):
    """Approximate convolution of code tensors: input [B,Cin,H,W], weight [Cout,Cin,kh,kw] ->
    [B,Cout,Ho,Wo]; bias must be None, groups 1, stride / padding / dilation square (their first entries are
    used), as in the reference's approx_conv2d_op (:530-573), whose arguments, values and gradients this
    reproduces without `F.unfold`."""
    assert bias is None, "bias is not supported in approximate convolution"
    assert groups == 1, "groups is not supported in approximate convolution"
    return ApproxConv2dFused.apply(input, weight, stride[0], padding[0], dilation[0])


class ApproxConv2dFusedBaseline(Function):
    """Straight-through variant of `ApproxConv2dFused`: the same LUT forward; the backward treats the product
    as exact, i.e. the plain convolution gradients on the float codes (what the reference computes through
    unfold + matmul, self_ops/ops_py/approx_ops.py:576-619)."""

    @staticmethod
    def forward(ctx, input, weight, stride, padding, dilation):
        B, Cin, H, W = input.shape
        Cout, _, kh, kw = weight.shape
        x_u8 = input.to(torch.uint8).contiguous()
        wmat = weight.reshape(Cout, -1).t().to(torch.uint8).contiguous()
        Ho = (H + 2 * padding - dilation * (kh - 1) - 1) // stride + 1
        Wo = (W + 2 * padding - dilation * (kw - 1) - 1) // stride + 1
        if lut_appmult is None:
            raise RuntimeError("lookup tables are not initialised: call init_lookup_tables first")
        y = torch.empty((B * Ho * Wo, Cout), dtype=torch.uint32, device=input.device)
        approx_ops.approx_conv2d_forward(x_u8, wmat, y, lut_appmult, kh, kw, stride, padding, dilation)
        ctx.save_for_backward(input, weight)
        ctx.geom = (stride, padding, dilation)
        return y.to(torch.float32).view(B, Ho, Wo, Cout).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, g_out):
        input, weight = ctx.saved_tensors
        stride, padding, dilation = ctx.geom
        gx = gw = None
        # full fp32 like the reference's two matmuls (:259-260): no TF32 rounding of grad_out or of the codes
        with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
            if ctx.needs_input_grad[0]:
                gx = torch.nn.grad.conv2d_input(input.shape, weight, g_out, stride=stride, padding=padding,
                                                dilation=dilation)
            if ctx.needs_input_grad[1]:
                gw = torch.nn.grad.conv2d_weight(input, weight.shape, g_out, stride=stride, padding=padding,
                                                 dilation=dilation)
        return gx, gw, None, None, None


def approx_conv2d_baseline_op(input, weight, bias, stride, padding, dilation, groups):
    """Same forward with the straight-through backward (reference approx_conv2d_baseline_op, :576-619): the
    gradients are those of an exact convolution of the float codes."""
    assert bias is None, "bias is not supported in approximate convolution"
    assert groups == 1, "groups is not supported in approximate convolution"
    return ApproxConv2dFusedBaseline.apply(input, weight, stride[0], padding[0], dilation[0])


# earlier names of the two functions above
approx_conv2d_fused_op = approx_conv2d_op
approx_conv2d_fused_baseline_op = approx_conv2d_baseline_op
