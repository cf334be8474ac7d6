"""`approx_ops` - the compiled-operator module the reference Python layer imports by absolute name
(`import approx_ops`, self_ops/ops_py/approx_ops.py:3), re-implemented on liblutgemm_b200.so.

It exposes the three functions the reference registers in self_ops/src/op_register.cpp:16-19 with
the same positional signatures, in-place outputs and precondition checks
(self_ops/src/cuda_helper.h:64-74, approx_gemm_forward.cu:243-259, approx_gemm_backward.cu:508-529):

    approx_gemm_forward (a: u8[M,K], b: u8[K,N], c: u32[M,N] (out), lut: u16[LUT_ELEM_NUM])
    approx_gemm_backward(gc: f32[M,N], a, b, ga: f32[M,K] (out), gb: f32[K,N] (out),
                         lut_ga: i16[LUT_ELEM_NUM], lut_gb: i16[LUT_ELEM_NUM])
    acc_gemm_forward_fp32(a: f32[M,K], b: f32[K,N], c: f32[M,N] (out))

Differences from the reference, all on the safe side: the bit-width is inferred from the table
length instead of a compile-time macro; kernels run on the current PyTorch stream instead of the
legacy default stream; a failed launch raises RuntimeError instead of printing and carrying on.
There is no CPU or PyTorch fallback: without the CUDA library every call raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liblutgemm_b200.so")
_lib = None


def _load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build_ext.py')}` "
            "(there is no fallback path for the LUT-GEMM operators)")
    lib = ctypes.CDLL(_LIB_PATH)
    vp, ci, cl, sz, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_size_t, ctypes.c_float
    lib.lutgemm_version.restype = ci
    lib.lutgemm_status_string.restype = ctypes.c_char_p
    lib.lutgemm_status_string.argtypes = [ci]
    lib.lutgemm_lut_elem_num.restype = ci
    lib.lutgemm_lut_elem_num.argtypes = [ci]
    lib.lutgemm_bits_from_elem_num.restype = ci
    lib.lutgemm_bits_from_elem_num.argtypes = [cl]
    lib.lutgemm_forward.restype = ci
    lib.lutgemm_forward.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, vp]
    lib.lutgemm_forward_scratch_bytes.restype = sz
    lib.lutgemm_forward_scratch_bytes.argtypes = [ci, ci, ci, ci]
    lib.lutgemm_forward_ws.restype = ci
    lib.lutgemm_forward_ws.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, vp, sz, vp]
    lib.lutgemm_conv2d_forward_scratch_bytes.restype = sz
    lib.lutgemm_conv2d_forward_scratch_bytes.argtypes = [ci] * 11
    lib.lutgemm_conv2d_forward_ws.restype = ci
    lib.lutgemm_conv2d_forward_ws.argtypes = [vp, vp, vp, vp] + [ci] * 11 + [vp, sz, vp]
    lib.lutgemm_conv2d_backward_ws.restype = ci
    lib.lutgemm_conv2d_backward_ws.argtypes = [vp] * 7 + [ci] * 11 + [vp, vp, sz, vp]
    lib.lutgemm_backward_scratch_bytes.restype = sz
    lib.lutgemm_backward_scratch_bytes.argtypes = [ci, ci, ci, ci]
    lib.lutgemm_backward.restype = ci
    lib.lutgemm_backward.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp, sz, vp]
    lib.lutgemm_backward_ws.restype = ci
    lib.lutgemm_backward_ws.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp, vp, sz, vp]
    lib.lutgemm_conv2d_forward.restype = ci
    lib.lutgemm_conv2d_forward.argtypes = [vp, vp, vp, vp] + [ci] * 11 + [vp]
    lib.lutgemm_conv2d_backward_scratch_bytes.restype = sz
    lib.lutgemm_conv2d_backward_scratch_bytes.argtypes = [ci] * 11
    lib.lutgemm_conv2d_backward.restype = ci
    lib.lutgemm_conv2d_backward.argtypes = [vp] * 7 + [ci] * 11 + [vp, sz, vp]
    cf = ctypes.c_float
    lib.lutgemm_quantize_activations.restype = ci
    lib.lutgemm_quantize_activations.argtypes = [vp, cl, cl, cl, cl, ci, ci, ci, ci, vp, vp, cf, vp, vp, vp]
    lib.lutgemm_quantize_activations_backward.restype = ci
    lib.lutgemm_quantize_activations_backward.argtypes = [vp, cl, cl, cl, cl, ci, ci, ci, ci, vp, vp, cf, vp, vp, vp, vp, vp, vp]
    lib.lutgemm_conv2d_epilogue.restype = ci
    lib.lutgemm_conv2d_epilogue.argtypes = [vp] * 10 + [cl, ci, ci, vp]
    lib.lutgemm_kernel_launches.restype = ctypes.c_ulonglong
    lib.lutgemm_kernel_launches.argtypes = []
    lib.lutgemm_layer_update_ranges.restype = ci
    lib.lutgemm_layer_update_ranges.argtypes = [vp] * 10 + [cf] * 5 + [vp, vp]
    lib.lutgemm_layer_weight_prep.restype = ci
    lib.lutgemm_layer_weight_prep.argtypes = [vp, cl, cl, cl, cl, ci, ci, ci, ci, vp, cf, vp, vp, vp]
    lib.lutgemm_layer_cross_terms.restype = ci
    lib.lutgemm_layer_cross_terms.argtypes = [vp] + [ci] * 9 + [vp, vp, vp]
    lib.lutgemm_layer_window_sum.restype = ci
    lib.lutgemm_layer_window_sum.argtypes = [vp] + [ci] * 8 + [vp, vp]
    lib.lutgemm_layer_window_sum_adjoint.restype = ci
    lib.lutgemm_layer_window_sum_adjoint.argtypes = [vp] + [ci] * 8 + [vp, vp]
    lib.lutgemm_layer_weight_grad.restype = ci
    lib.lutgemm_layer_weight_grad.argtypes = [vp, vp, vp, cl, cl, cl, cl, ci, ci, ci, ci, vp, cf, vp, vp]
    lib.lutgemm_conv2d_forward_layer_scratch_bytes.restype = sz
    lib.lutgemm_conv2d_forward_layer_scratch_bytes.argtypes = [ci] * 11
    lib.lutgemm_forward_layer_scratch_bytes.restype = sz
    lib.lutgemm_forward_layer_scratch_bytes.argtypes = [ci, ci, ci, ci]
    lib.lutgemm_conv2d_forward_layer.restype = ci
    lib.lutgemm_conv2d_forward_layer.argtypes = [vp, vp, vp] + [ci] * 11 + [vp] * 9 + [vp, sz, vp]
    lib.lutgemm_forward_layer.restype = ci
    lib.lutgemm_forward_layer.argtypes = [vp, vp, vp] + [ci] * 4 + [vp] * 9 + [vp, sz, vp]
    lib.lutgemm_backward_f32lut_scratch_bytes.restype = sz
    lib.lutgemm_backward_f32lut_scratch_bytes.argtypes = [ci, ci, ci, ci]
    lib.lutgemm_backward_f32lut.restype = ci
    lib.lutgemm_backward_f32lut.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp, sz, vp]
    lib.lutgemm_set_tma.restype = ci
    lib.lutgemm_set_tma.argtypes = [ci]
    lib.lutgemm_set_handover.restype = ci
    lib.lutgemm_set_handover.argtypes = [ci]
    lib.lutgemm_set_kernel_choice.restype = ci
    lib.lutgemm_set_kernel_choice.argtypes = [ci, ci, ci]
    lib.lutgemm_device_error.restype = ci
    lib.lutgemm_device_error.argtypes = [ctypes.POINTER(ci)]
    lib.lutgemm_selftest_bounded_wait.restype = ci
    lib.lutgemm_selftest_bounded_wait.argtypes = [vp]
    _lib = lib
    return lib


def library():
    """The loaded ctypes handle of liblutgemm_b200.so (raises if it has not been built)."""
    return _load()


_FORWARD_CHOICES = {"auto": 0, "rowbcast": 1, "slab": 2}
_BACKWARD_CHOICES = {"auto": 0, "bcast": 1, "slab": 2}
_TILE_CHOICES = {"auto": 0, "wide": 1, "tall": 2}


def set_kernel_choice(forward: str = "auto", backward: str = "auto", grad_tile: str = "auto") -> None:
    """Process-wide kernel-family override (tests, A/B timing); all "auto" restores the choice by shape.
    forward: "rowbcast" | "slab"; backward: "bcast" | "slab"; grad_tile: "wide" (512 x 64) | "tall" (1024 x 32)."""
    _check(_load().lutgemm_set_kernel_choice(_FORWARD_CHOICES[forward], _BACKWARD_CHOICES[backward],
                                             _TILE_CHOICES[grad_tile]), "set_kernel_choice")


def device_error() -> int:
    """Reads and clears the device-side error word of the pipelined kernels (0 = no error).  A non-zero
    value names the bounded barrier wait that ran out; results since the last call are then invalid."""
    v = ctypes.c_int(0)
    _check(_load().lutgemm_device_error(ctypes.byref(v)), "lutgemm_device_error")
    return v.value


def _check(status: int, what: str) -> None:
    if status != 0:
        msg = _load().lutgemm_status_string(status).decode()
        raise RuntimeError(f"{what} failed with status {status}: {msg}")


def _check_input(x: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if not isinstance(x, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not x.is_cuda:
        raise RuntimeError(f"{name} must be a CUDAtensor")
    if not x.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if x.dtype != dtype:
        raise RuntimeError(f"{name} must be of type {dtype}")


def _bits_of(lut: torch.Tensor, name: str) -> int:
    bits = _load().lutgemm_bits_from_elem_num(lut.numel())
    if lut.dim() != 1 or bits < 0:
        raise RuntimeError(f"{name} size should be one of 1024/5120/17408/66306 (4/6/7/8-bit tables), got "
                           f"{tuple(lut.shape)}; please check the quantization bit-width")
    return bits


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def approx_gemm_forward(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, lut: torch.Tensor):
    """c[m,n] = sum_k lut[a[m,k]*(2^bits+2) + b[k,n]], written in place into the uint32 tensor c.
    Returns the transposed activation codes the kernel worked from (a uint8 tensor that
    `approx_gemm_backward(..., codes_t=...)` of the same `a` can reuse), or None; callers of the reference
    signature simply ignore it."""
    _check_input(a, torch.uint8, "a_tensor")
    _check_input(b, torch.uint8, "b_tensor")
    _check_input(c, torch.uint32, "c_tensor")
    _check_input(lut, torch.uint16, "lut_appmult_tensor")
    if a.dim() != 2 or b.dim() != 2 or c.dim() != 2:
        raise RuntimeError("a_tensor, b_tensor and c_tensor must be 2-D")
    M, K = a.shape
    N = b.shape[1]
    if b.shape[0] != K:
        raise RuntimeError(f"b_tensor's shape should be {K} x {N}")
    if tuple(c.shape) != (M, N):
        raise RuntimeError(f"c_tensor's shape should be {M} x {N}")
    bits = _bits_of(lut, "lut_appmult_tensor")
    dev = a.device
    if b.device != dev or c.device != dev or lut.device != dev:
        raise RuntimeError("device id not match")
    if M == 0 or N == 0:
        return
    if K == 0:
        c.zero_()
        return
    lib = _load()
    with torch.cuda.device(dev):
        # workspace for the transposed activation codes (0 bytes when the kernel for this shape has no use for it)
        nbytes = lib.lutgemm_forward_scratch_bytes(bits, M, K, N)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
        rc = lib.lutgemm_forward_ws(a.data_ptr(), b.data_ptr(), c.data_ptr(), lut.data_ptr(), bits, M, K, N,
                                    scratch.data_ptr() if nbytes else None, nbytes, _stream_ptr(dev))
    _check(rc, "approx_gemm_forward")
    return scratch


def approx_gemm_backward(gc: torch.Tensor, a: torch.Tensor, b: torch.Tensor, ga: torch.Tensor, gb: torch.Tensor,
                         lut_grad_a: torch.Tensor, lut_grad_b: torch.Tensor, codes_t: torch.Tensor = None) -> None:
    """ga = 1/16 * sum_n gc * LUTa[a][b],  gb = 1/16 * sum_m LUTb[a][b] * gc, written in place."""
    _check_input(gc, torch.float32, "gc_tensor")
    _check_input(a, torch.uint8, "a_tensor")
    _check_input(b, torch.uint8, "b_tensor")
    _check_input(ga, torch.float32, "ga_tensor")
    _check_input(gb, torch.float32, "gb_tensor")
    _check_input(lut_grad_a, torch.int16, "lut_grad_a_tensor")
    _check_input(lut_grad_b, torch.int16, "lut_grad_b_tensor")
    if a.dim() != 2 or b.dim() != 2:
        raise RuntimeError("a_tensor and b_tensor must be 2-D")
    M, K = a.shape
    N = b.shape[1]
    if tuple(gc.shape) != (M, N):
        raise RuntimeError(f"gc_tensor's shape should be {M} x {N}")
    if b.shape[0] != K:
        raise RuntimeError(f"b_tensor's shape should be {K} x {N}")
    if tuple(ga.shape) != (M, K):
        raise RuntimeError(f"ga_tensor's shape should be {M} x {K}")
    if tuple(gb.shape) != (K, N):
        raise RuntimeError(f"gb_tensor's shape should be {K} x {N}")
    bits = _bits_of(lut_grad_a, "lut_grad_a_tensor")
    if _bits_of(lut_grad_b, "lut_grad_b_tensor") != bits:
        raise RuntimeError("lut_grad_a_tensor and lut_grad_b_tensor must have the same length")
    dev = gc.device
    for t in (a, b, ga, gb, lut_grad_a, lut_grad_b):
        if t.device != dev:
            raise RuntimeError("All tensors should be on the same device")
    if M == 0 or K == 0 or N == 0:
        ga.zero_()
        gb.zero_()
        return
    lib = _load()
    with torch.cuda.device(dev):
        nbytes = lib.lutgemm_backward_scratch_bytes(bits, M, K, N)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
        if codes_t is not None:
            _check_input(codes_t, torch.uint8, "codes_t")
            if codes_t.numel() != K * ((M + 15) // 16 * 16):
                raise RuntimeError("codes_t does not belong to this a_tensor")
        rc = lib.lutgemm_backward_ws(gc.data_ptr(), a.data_ptr(), b.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                     lut_grad_a.data_ptr(), lut_grad_b.data_ptr(), bits, M, K, N,
                                     codes_t.data_ptr() if codes_t is not None else None,
                                     scratch.data_ptr() if scratch is not None else None, nbytes, _stream_ptr(dev))
    _check(rc, "approx_gemm_backward")


def acc_gemm_forward_fp32(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> None:
    """Exact fp32 GEMM c = a @ b written in place.  The reference carries a hand-written SGEMM for this
    (approx_gemm_forward.cu:340-571) that only its unused AccGemm wrapper calls; the symbol is kept
    for API parity and forwards to the library GEMM."""
    _check_input(a, torch.float32, "a_tensor")
    _check_input(b, torch.float32, "b_tensor")
    _check_input(c, torch.float32, "c_tensor")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise RuntimeError(f"b_tensor's shape should be {a.shape[1]} x N")
    if tuple(c.shape) != (a.shape[0], b.shape[1]):
        raise RuntimeError(f"c_tensor's shape should be {a.shape[0]} x {b.shape[1]}")
    torch.mm(a, b, out=c)


def _conv_out(H, W, kh, kw, stride, pad, dil):
    return (H + 2 * pad - dil * (kh - 1) - 1) // stride + 1, (W + 2 * pad - dil * (kw - 1) - 1) // stride + 1


def approx_conv2d_forward(x: torch.Tensor, wmat: torch.Tensor, y: torch.Tensor, lut: torch.Tensor, kh: int, kw: int,
                          stride: int, pad: int, dil: int):
    """Fused-im2col convolution forward.  x: u8 codes [B,C,H,W]; wmat: u8 [C*kh*kw, Cout]; y: u32
    [B*Ho*Wo, Cout] (NHWC), written in place.  The reference declares such an op
    (`approx_conv2d_forward`, self_ops/src/op_register.cpp:11,22) but ships no source for it.
    Returns the transposed unfolded codes the kernel worked from (a uint8 tensor to hand to
    `approx_conv2d_backward(..., codes_t=...)` of the same layer), or None when the shape did not need them."""
    _check_input(x, torch.uint8, "input_tensor")
    _check_input(wmat, torch.uint8, "weight_tensor")
    _check_input(y, torch.uint32, "output_tensor")
    _check_input(lut, torch.uint16, "lut_appmult_tensor")
    if x.dim() != 4 or wmat.dim() != 2 or y.dim() != 2:
        raise RuntimeError("input_tensor must be 4-D, weight_tensor and output_tensor 2-D")
    B, C, H, W = x.shape
    K, Cout = wmat.shape
    Ho, Wo = _conv_out(H, W, kh, kw, stride, pad, dil)
    if K != C * kh * kw:
        raise RuntimeError(f"weight_tensor's shape should be {C * kh * kw} x Cout")
    if tuple(y.shape) != (B * Ho * Wo, Cout):
        raise RuntimeError(f"output_tensor's shape should be {B * Ho * Wo} x {Cout}")
    bits = _bits_of(lut, "lut_appmult_tensor")
    if wmat.device != x.device or y.device != x.device or lut.device != x.device:
        raise RuntimeError("device id not match")
    lib = _load()
    with torch.cuda.device(x.device):
        nbytes = lib.lutgemm_conv2d_forward_scratch_bytes(bits, B, C, H, W, Cout, kh, kw, stride, pad, dil)
        codes_t = torch.empty(nbytes, dtype=torch.uint8, device=x.device) if nbytes else None
        rc = lib.lutgemm_conv2d_forward_ws(x.data_ptr(), wmat.data_ptr(), y.data_ptr(), lut.data_ptr(), bits, B, C, H,
                                           W, Cout, kh, kw, stride, pad, dil, codes_t.data_ptr() if nbytes else None,
                                           nbytes, _stream_ptr(x.device))
    _check(rc, "approx_conv2d_forward")
    return codes_t


def _epilogue_args(box, sumw_t, taps, s_a, s_w, z_a, z_w, bias, M, L, Cout):
    for t, shape, name in ((box, (M,), "box"), (sumw_t, (L, Cout), "sumw_t"), (taps, (L,), "taps")):
        _check_input(t, torch.float32, name)
        if tuple(t.shape) != shape:
            raise RuntimeError(f"{name} has shape {tuple(t.shape)}, expected {shape}")
    return [box.data_ptr(), sumw_t.data_ptr(), taps.data_ptr(), s_a.data_ptr(), s_w.data_ptr(), z_a.data_ptr(),
            z_w.data_ptr(), bias.data_ptr() if bias is not None else None]


def approx_conv2d_forward_layer(x: torch.Tensor, wmat: torch.Tensor, lut: torch.Tensor, kh: int, kw: int, stride: int,
                                pad: int, dil: int, box, sumw_t, taps, s_a, s_w, z_a, z_w, bias):
    """Whole-layer convolution forward in one kernel: the LUT sums of `approx_conv2d_forward` de-quantised as by
    `conv2d_epilogue` while still in registers.  Returns (out f32 [B*Ho*Wo, Cout], codes_t or None)."""
    _check_input(x, torch.uint8, "input_tensor")
    _check_input(wmat, torch.uint8, "weight_tensor")
    _check_input(lut, torch.uint16, "lut_appmult_tensor")
    B, C, H, W = x.shape
    K, Cout = wmat.shape
    Ho, Wo = _conv_out(H, W, kh, kw, stride, pad, dil)
    if K != C * kh * kw:
        raise RuntimeError(f"weight_tensor's shape should be {C * kh * kw} x Cout")
    bits = _bits_of(lut, "lut_appmult_tensor")
    M, L = B * Ho * Wo, Ho * Wo
    epi = _epilogue_args(box, sumw_t, taps, s_a, s_w, z_a, z_w, bias, M, L, Cout)
    out = torch.empty((M, Cout), dtype=torch.float32, device=x.device)
    lib = _load()
    with torch.cuda.device(x.device):
        ncodes = lib.lutgemm_conv2d_forward_scratch_bytes(bits, B, C, H, W, Cout, kh, kw, stride, pad, dil)
        nbytes = lib.lutgemm_conv2d_forward_layer_scratch_bytes(bits, B, C, H, W, Cout, kh, kw, stride, pad, dil)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device) if nbytes else None
        rc = lib.lutgemm_conv2d_forward_layer(x.data_ptr(), wmat.data_ptr(), lut.data_ptr(), bits, B, C, H, W, Cout, kh, kw,
                                              stride, pad, dil, *epi, out.data_ptr(),
                                              scratch.data_ptr() if nbytes else None, nbytes, _stream_ptr(x.device))
    _check(rc, "approx_conv2d_forward_layer")
    return out, (scratch[:ncodes] if ncodes else None)


def approx_gemm_forward_layer(a: torch.Tensor, b: torch.Tensor, lut: torch.Tensor, box, sumw_t, taps, s_a, s_w, z_a, z_w,
                              bias):
    """Whole-layer linear forward in one kernel (L = 1: box [M] row sums of the codes, sumw_t [1, N], taps [1]).
    Returns (out f32 [M, N], codes_t or None)."""
    _check_input(a, torch.uint8, "a_tensor")
    _check_input(b, torch.uint8, "b_tensor")
    _check_input(lut, torch.uint16, "lut_appmult_tensor")
    M, K = a.shape
    N = b.shape[1]
    if b.shape[0] != K:
        raise RuntimeError(f"b_tensor's shape should be {K} x {N}")
    bits = _bits_of(lut, "lut_appmult_tensor")
    epi = _epilogue_args(box, sumw_t, taps, s_a, s_w, z_a, z_w, bias, M, 1, N)
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    lib = _load()
    with torch.cuda.device(a.device):
        ncodes = lib.lutgemm_forward_scratch_bytes(bits, M, K, N)
        nbytes = lib.lutgemm_forward_layer_scratch_bytes(bits, M, K, N)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=a.device) if nbytes else None
        rc = lib.lutgemm_forward_layer(a.data_ptr(), b.data_ptr(), lut.data_ptr(), bits, M, K, N, *epi, out.data_ptr(),
                                       scratch.data_ptr() if nbytes else None, nbytes, _stream_ptr(a.device))
    _check(rc, "approx_gemm_forward_layer")
    return out, (scratch[:ncodes] if ncodes else None)


def approx_conv2d_backward(gy: torch.Tensor, x: torch.Tensor, wmat: torch.Tensor, gx: torch.Tensor, gw: torch.Tensor,
                           lut_grad_a: torch.Tensor, lut_grad_b: torch.Tensor, kh: int, kw: int, stride: int, pad: int,
                           dil: int, codes_t: torch.Tensor = None) -> None:
    """Fused-im2col convolution backward.  gy: f32 [B*Ho*Wo, Cout]; gx: f32 [B,C,H,W] and gw: f32
    [C*kh*kw, Cout] are written in place; either may be None to skip that gradient.  codes_t: what
    `approx_conv2d_forward` returned for the same x and geometry (optional)."""
    _check_input(gy, torch.float32, "grad_output_tensor")
    _check_input(x, torch.uint8, "input_tensor")
    _check_input(wmat, torch.uint8, "weight_tensor")
    if gx is not None:
        _check_input(gx, torch.float32, "grad_input_tensor")
    if gw is not None:
        _check_input(gw, torch.float32, "grad_weight_tensor")
    _check_input(lut_grad_a, torch.int16, "lut_grad_a_tensor")
    _check_input(lut_grad_b, torch.int16, "lut_grad_b_tensor")
    B, C, H, W = x.shape
    K, Cout = wmat.shape
    Ho, Wo = _conv_out(H, W, kh, kw, stride, pad, dil)
    if K != C * kh * kw or tuple(gy.shape) != (B * Ho * Wo, Cout) \
            or (gx is not None and tuple(gx.shape) != tuple(x.shape)) \
            or (gw is not None and tuple(gw.shape) != (K, Cout)):
        raise RuntimeError("approx_conv2d_backward: tensor shapes do not match the convolution geometry")
    bits = _bits_of(lut_grad_a, "lut_grad_a_tensor")
    if _bits_of(lut_grad_b, "lut_grad_b_tensor") != bits:
        raise RuntimeError("lut_grad_a_tensor and lut_grad_b_tensor must have the same length")
    dev = gy.device
    for t in (x, wmat, gx, gw, lut_grad_a, lut_grad_b):
        if t is not None and t.device != dev:
            raise RuntimeError("All tensors should be on the same device")
    lib = _load()
    with torch.cuda.device(dev):
        nbytes = lib.lutgemm_conv2d_backward_scratch_bytes(bits, B, C, H, W, Cout, kh, kw, stride, pad, dil)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        if codes_t is not None:
            _check_input(codes_t, torch.uint8, "codes_t")
            if codes_t.numel() != K * ((B * Ho * Wo + 15) // 16 * 16):
                raise RuntimeError("codes_t does not belong to this convolution")
        rc = lib.lutgemm_conv2d_backward_ws(gy.data_ptr(), x.data_ptr(), wmat.data_ptr(),
                                            gx.data_ptr() if gx is not None else None,
                                            gw.data_ptr() if gw is not None else None,
                                            lut_grad_a.data_ptr(), lut_grad_b.data_ptr(), bits, B, C, H, W, Cout, kh, kw,
                                            stride, pad, dil, codes_t.data_ptr() if codes_t is not None else None,
                                            scratch.data_ptr(), nbytes, _stream_ptr(dev))
    _check(rc, "approx_conv2d_backward")


def approx_gemm_backward_f32lut(gc: torch.Tensor, a: torch.Tensor, b: torch.Tensor, ga: torch.Tensor, gb: torch.Tensor,
                                lut_grad_a: torch.Tensor, lut_grad_b: torch.Tensor) -> None:
    """ga = sum_n gc * LUTa[a][b],  gb = sum_m LUTb[a][b] * gc with fp32 gradient tables (padded flat layout, float
    entries, bit-widths up to 7), written in place; no 1/16 factor."""
    for t, dt, name in ((gc, torch.float32, "gc_tensor"), (a, torch.uint8, "a_tensor"), (b, torch.uint8, "b_tensor"),
                        (ga, torch.float32, "ga_tensor"), (gb, torch.float32, "gb_tensor"),
                        (lut_grad_a, torch.float32, "lut_grad_a_tensor"), (lut_grad_b, torch.float32, "lut_grad_b_tensor")):
        _check_input(t, dt, name)
    M, K = a.shape
    N = b.shape[1]
    if tuple(gc.shape) != (M, N) or b.shape[0] != K or tuple(ga.shape) != (M, K) or tuple(gb.shape) != (K, N):
        raise RuntimeError("approx_gemm_backward_f32lut: tensor shapes do not agree")
    lib = _load()
    bits = lib.lutgemm_bits_from_elem_num(lut_grad_a.numel())
    if bits < 0 or bits > 7 or lut_grad_b.numel() != lut_grad_a.numel():
        raise RuntimeError("fp32 gradient tables must both have the padded length of a bit-width up to 7")
    dev = gc.device
    with torch.cuda.device(dev):
        nbytes = lib.lutgemm_backward_f32lut_scratch_bytes(bits, M, K, N)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
        rc = lib.lutgemm_backward_f32lut(gc.data_ptr(), a.data_ptr(), b.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                         lut_grad_a.data_ptr(), lut_grad_b.data_ptr(), bits, M, K, N,
                                         scratch.data_ptr() if scratch is not None else None, nbytes, _stream_ptr(dev))
    _check(rc, "approx_gemm_backward_f32lut")


def _dense_4d(x: torch.Tensor, name: str) -> None:
    if not x.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if x.dtype != torch.float32 or x.dim() != 4:
        raise RuntimeError(f"{name} must be a 4-D float32 tensor")
    if not (x.is_contiguous() or x.is_contiguous(memory_format=torch.channels_last)):
        raise RuntimeError(f"{name} must be dense (NCHW or channels-last)")


def quantize_activations(x: torch.Tensor, scale: torch.Tensor, zp_neg: torch.Tensor, qmax: float,
                         want_chansum: bool = True):
    """codes = uint8(clamp(round(x / scale - zp_neg), 0, qmax)), NCHW-contiguous, and (optionally) their sums over
    the channels [B, H, W]; one pass over x in whichever dense layout it has.  scale / zp_neg: 1-element device
    tensors."""
    _dense_4d(x, "input_tensor")
    B, C, H, W = x.shape
    codes = torch.empty((B, C, H, W), dtype=torch.uint8, device=x.device)
    chansum = torch.zeros((B, H, W), dtype=torch.float32, device=x.device) if want_chansum else None
    sb, sc, sh, sw = x.stride()
    with torch.cuda.device(x.device):
        rc = _load().lutgemm_quantize_activations(x.data_ptr(), sb, sc, sh, sw, B, C, H, W, scale.data_ptr(),
                                                  zp_neg.data_ptr(), float(qmax), codes.data_ptr(),
                                                  chansum.data_ptr() if want_chansum else None, _stream_ptr(x.device))
    _check(rc, "quantize_activations")
    return codes, chansum


def quantize_activations_backward(x: torch.Tensor, scale: torch.Tensor, zp_neg: torch.Tensor, qmax: float,
                                  gcodes: torch.Tensor, box_t, s_w: torch.Tensor, z_w: torch.Tensor) -> torch.Tensor:
    """Gradient w.r.t. x of the quantised layer input (clamp mask, straight-through rounding), in the layout of x:
    mask * s_w * (gcodes + z_w * box_t).  gcodes: f32 NCHW-contiguous; box_t: f32 [B, H, W] or None."""
    _dense_4d(x, "input_tensor")
    _check_input(gcodes, torch.float32, "grad_codes_tensor")
    if tuple(gcodes.shape) != tuple(x.shape):
        raise RuntimeError("grad_codes_tensor must have the shape of input_tensor")
    B, C, H, W = x.shape
    gx = torch.empty_like(x)  # preserves the (dense) strides of x
    sb, sc, sh, sw = x.stride()
    if gx.stride() != x.stride():
        raise RuntimeError("could not allocate a gradient with the strides of input_tensor")
    if box_t is not None:
        _check_input(box_t, torch.float32, "box_t_tensor")
    with torch.cuda.device(x.device):
        rc = _load().lutgemm_quantize_activations_backward(
            x.data_ptr(), sb, sc, sh, sw, B, C, H, W, scale.data_ptr(), zp_neg.data_ptr(), float(qmax), gcodes.data_ptr(),
            box_t.data_ptr() if box_t is not None else None, s_w.data_ptr(), z_w.data_ptr(), gx.data_ptr(),
            _stream_ptr(x.device))
    _check(rc, "quantize_activations_backward")
    return gx


def conv2d_epilogue(y: torch.Tensor, box: torch.Tensor, sumw_t: torch.Tensor, taps: torch.Tensor, s_a: torch.Tensor,
                    s_w: torch.Tensor, z_a: torch.Tensor, z_w: torch.Tensor, bias, L: int) -> torch.Tensor:
    """out[m, co] = s_a s_w (y + z_w box[m] + z_a sumw_t[l, co] + z_a z_w taps[l]) (+ bias[co]);  y: u32 [M, Cout]."""
    _check_input(y, torch.uint32, "accumulator_tensor")
    M, Cout = y.shape
    for t, shape, name in ((box, (M,), "box"), (sumw_t, (L, Cout), "sumw_t"), (taps, (L,), "taps")):
        _check_input(t, torch.float32, name)
        if tuple(t.shape) != shape:
            raise RuntimeError(f"{name} has shape {tuple(t.shape)}, expected {shape}")
    out = torch.empty((M, Cout), dtype=torch.float32, device=y.device)
    with torch.cuda.device(y.device):
        rc = _load().lutgemm_conv2d_epilogue(y.data_ptr(), box.data_ptr(), sumw_t.data_ptr(), taps.data_ptr(),
                                             s_a.data_ptr(), s_w.data_ptr(), z_a.data_ptr(), z_w.data_ptr(),
                                             bias.data_ptr() if bias is not None else None, out.data_ptr(), M, L, Cout,
                                             _stream_ptr(y.device))
    _check(rc, "conv2d_epilogue")
    return out


# ---- small one-pass kernels of the layer wiring (lutgemm_layers.py) ---------------------------------------------------
def layer_update_ranges(act_lo, act_hi, w_lo, w_hi, act_state, w_state, momentum: float, a_qmax: float, w_qmax: float,
                        quant: torch.Tensor) -> None:
    """Observers and quantisation parameters of one layer in one launch.  act_lo / act_hi / w_lo / w_hi: device
    scalars (this batch's activation range, the weights' range); act_state / w_state: (min, max, seen) buffers,
    updated in place - exponential moving average for activations, running range for weights; quant (4 floats) =
    {s_a, z_a, s_w, z_w}."""
    dev = quant.device
    eps = float(torch.finfo(torch.float32).eps)
    with torch.cuda.device(dev):
        rc = _load().lutgemm_layer_update_ranges(
            act_lo.data_ptr(), act_hi.data_ptr(), w_lo.data_ptr(), w_hi.data_ptr(), act_state[0].data_ptr(),
            act_state[1].data_ptr(), act_state[2].data_ptr(), w_state[0].data_ptr(), w_state[1].data_ptr(),
            w_state[2].data_ptr(), float(1 - momentum), float(momentum), float(a_qmax), float(w_qmax), eps,
            quant.data_ptr(), _stream_ptr(dev))
    _check(rc, "layer_update_ranges")


def layer_weight_prep(weight: torch.Tensor, quant: torch.Tensor, qmax: float):
    """(wmat u8 [Cin*kh*kw, Cout], wsum f32 [Cout, kh*kw]) of a 4-D fp32 weight in any dense layout: the weight
    codes transposed for the LUT kernels and their sums over the input channels per tap."""
    Cout, Cin, kh, kw = weight.shape
    wmat = torch.empty((Cin * kh * kw, Cout), dtype=torch.uint8, device=weight.device)
    wsum = torch.empty((Cout, kh * kw), dtype=torch.float32, device=weight.device)
    s = weight.stride()
    with torch.cuda.device(weight.device):
        rc = _load().lutgemm_layer_weight_prep(weight.data_ptr(), s[0], s[1], s[2], s[3], Cout, Cin, kh, kw, quant.data_ptr(),
                                               float(qmax), wmat.data_ptr(), wsum.data_ptr(), _stream_ptr(weight.device))
    _check(rc, "layer_weight_prep")
    return wmat, wsum


def layer_cross_terms(wsum: torch.Tensor, Cin: int, H: int, W: int, kh: int, kw: int, stride: int, pad: int, dil: int):
    """(sumw_t f32 [Ho*Wo, Cout], taps f32 [Ho*Wo]): per output position the weight-code sums over the taps inside
    the image, and Cin times the number of those taps."""
    Cout = wsum.shape[0]
    Ho, Wo = _conv_out(H, W, kh, kw, stride, pad, dil)
    sumw_t = torch.empty((Ho * Wo, Cout), dtype=torch.float32, device=wsum.device)
    taps = torch.empty((Ho * Wo,), dtype=torch.float32, device=wsum.device)
    with torch.cuda.device(wsum.device):
        rc = _load().lutgemm_layer_cross_terms(wsum.data_ptr(), Cout, Cin, H, W, kh, kw, stride, pad, dil, sumw_t.data_ptr(),
                                               taps.data_ptr(), _stream_ptr(wsum.device))
    _check(rc, "layer_cross_terms")
    return sumw_t, taps


def layer_window_sum(img: torch.Tensor, kh: int, kw: int, stride: int, pad: int, dil: int) -> torch.Tensor:
    """[B, H, W] f32 -> [B*Ho*Wo] f32: sum of the kernel window at every output position (zero padding)."""
    _check_input(img, torch.float32, "image")
    B, H, W = img.shape
    Ho, Wo = _conv_out(H, W, kh, kw, stride, pad, dil)
    box = torch.empty((B * Ho * Wo,), dtype=torch.float32, device=img.device)
    with torch.cuda.device(img.device):
        rc = _load().lutgemm_layer_window_sum(img.data_ptr(), B, H, W, kh, kw, stride, pad, dil, box.data_ptr(),
                                              _stream_ptr(img.device))
    _check(rc, "layer_window_sum")
    return box


def layer_window_sum_adjoint(gsum: torch.Tensor, H: int, W: int, kh: int, kw: int, stride: int, pad: int, dil: int):
    """[B, Ho, Wo] f32 -> [B, H, W] f32: adjoint of `layer_window_sum`."""
    _check_input(gsum, torch.float32, "grad_sum")
    B = gsum.shape[0]
    out = torch.empty((B, H, W), dtype=torch.float32, device=gsum.device)
    with torch.cuda.device(gsum.device):
        rc = _load().lutgemm_layer_window_sum_adjoint(gsum.data_ptr(), B, H, W, kh, kw, stride, pad, dil, out.data_ptr(),
                                                      _stream_ptr(gsum.device))
    _check(rc, "layer_window_sum_adjoint")
    return out


def layer_weight_grad(gwmat: torch.Tensor, tapg: torch.Tensor, weight: torch.Tensor, quant: torch.Tensor, qmax: float):
    """Gradient w.r.t. the fp32 weight [Cout, Cin, kh, kw] (contiguous) from the gradient w.r.t. its codes
    gwmat f32 [Cin*kh*kw, Cout] and the cross-term gradient tapg f32 [Cout, kh*kw]."""
    _check_input(gwmat, torch.float32, "grad_codes")
    _check_input(tapg, torch.float32, "tap_grad")
    Cout, Cin, kh, kw = weight.shape
    gw = torch.empty((Cout, Cin, kh, kw), dtype=torch.float32, device=weight.device)
    s = weight.stride()
    with torch.cuda.device(weight.device):
        rc = _load().lutgemm_layer_weight_grad(gwmat.data_ptr(), tapg.data_ptr(), weight.data_ptr(), s[0], s[1], s[2], s[3],
                                               Cout, Cin, kh, kw, quant.data_ptr(), float(qmax), gw.data_ptr(),
                                               _stream_ptr(weight.device))
    _check(rc, "layer_weight_grad")
    return gw
