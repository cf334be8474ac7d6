"""Sign-magnitude operands on the unsigned LUT kernels.

The reference's operator multiplies unsigned b-bit codes.  The benchmark's first configuration uses b-bit
magnitudes with independent sign bits: out[m,n] = sum_k s_a s_w L[|a|][|w|].  That product is again a table
look-up - of the (b+1)-bit codes  c = sign << b | magnitude  in a table twice as large in each direction:

    forward    L'[(s_a,a)][(s_w,w)] = s_a s_w L[a][w] + C     C = max L, so that the entries stay unsigned 16-bit;
                                                              the K offsets are subtracted after the exact sum
    d/d a      Ga'[(s_a,a)][(s_w,w)] = s_w Ga[a][w]           (a is the signed VALUE s_a * magnitude)
    d/d w      Gw'[(s_a,a)][(s_w,w)] = s_a Gw[a][w]

so the signed operator runs on the (b+1)-bit kernels unchanged and exactly: magnitudes of 3, 5, 6 and 7 bits
map to the 4-, 6-, 7- and 8-bit kernels.  A negative zero keeps its own table row, as a sign-magnitude
multiplier circuit would."""
from __future__ import annotations

import numpy as np
import torch

import approx_ops

_GRAD_SCALE = 16
_MAG_TO_KERNEL_BITS = {3: 4, 5: 6, 6: 7, 7: 8}


def _pack(dense: np.ndarray, bits: int, dtype) -> np.ndarray:
    q = 1 << bits
    flat = np.zeros(approx_ops.library().lutgemm_lut_elem_num(bits), dtype=dtype)
    flat[: (q + 1) * (q + 2)].reshape(q + 1, q + 2)[:q, :q] = dense.astype(dtype)  # entry (a, w) at a*(2^b+2) + w
    return flat


def signed_dense_tables(fp: np.ndarray, grad_a: np.ndarray, grad_b: np.ndarray):
    """Dense [2Q, 2Q] tables of the codes `sign << b | magnitude`: (forward + offset, round(16 d/da), round(16 d/dw),
    offset) with offset = max(fp)."""
    fp = np.asarray(fp, dtype=np.int64)
    q = fp.shape[0]
    offset = int(fp.max())
    sign = np.concatenate([np.ones(q, np.int64), -np.ones(q, np.int64)])
    big = lambda t: np.tile(np.asarray(t), (2, 2))  # index (sign << b | magnitude) in both directions
    fp_s = sign[:, None] * sign[None, :] * big(fp) + offset
    ga_s = sign[None, :] * np.round(big(np.asarray(grad_a, np.float64)) * _GRAD_SCALE).astype(np.int64)
    gb_s = sign[:, None] * np.round(big(np.asarray(grad_b, np.float64)) * _GRAD_SCALE).astype(np.int64)
    return fp_s, ga_s, gb_s, offset


class SignedTables:
    """Device tables of the signed operator built from magnitude tables fp [2^b, 2^b] (non-negative integers),
    grad_a / grad_b (floats, d product / d magnitude)."""

    def __init__(self, device, fp: np.ndarray, grad_a: np.ndarray, grad_b: np.ndarray, magnitude_bits: int):
        if magnitude_bits not in _MAG_TO_KERNEL_BITS:
            raise ValueError("magnitude bit-width must be one of 3, 5, 6, 7")
        q = 1 << magnitude_bits
        fp = np.asarray(fp, dtype=np.int64)
        if fp.shape != (q, q) or fp.min() < 0 or 2 * int(fp.max()) > 0xFFFF:
            raise ValueError("forward table must be [2^b, 2^b], non-negative, with 2*max <= 65535")
        self.magnitude_bits, self.kernel_bits = magnitude_bits, _MAG_TO_KERNEL_BITS[magnitude_bits]
        fp_s, ga_s, gb_s, self.offset = signed_dense_tables(fp, grad_a, grad_b)
        for t in (ga_s, gb_s):
            if t.min() < -32768 or t.max() > 32767:
                raise ValueError("gradient table does not fit the 16-bit wire format")
        dev = torch.device(device)
        self.fp = torch.from_numpy(_pack(fp_s, self.kernel_bits, np.uint16)).to(dev)
        self.ga = torch.from_numpy(_pack(ga_s, self.kernel_bits, np.int16)).to(dev)
        self.gb = torch.from_numpy(_pack(gb_s, self.kernel_bits, np.int16)).to(dev)

    def codes(self, magnitude: torch.Tensor, negative: torch.Tensor) -> torch.Tensor:
        """uint8 kernel codes from magnitudes in [0, 2^b) and sign bits (True = negative)."""
        return (magnitude.to(torch.uint8) | (negative.to(torch.uint8) << self.magnitude_bits)).contiguous()

    def forward(self, a_codes: torch.Tensor, w_codes: torch.Tensor) -> torch.Tensor:
        """int64 [M, N]: sum_k s_a s_w L[|a|][|w|], exact.  a_codes [M, K], w_codes [K, N] from `codes`."""
        M, K = a_codes.shape
        c = torch.empty((M, w_codes.shape[1]), dtype=torch.uint32, device=a_codes.device)
        approx_ops.approx_gemm_forward(a_codes, w_codes, c, self.fp)
        return c.to(torch.int64) - K * self.offset

    def backward(self, grad_out: torch.Tensor, a_codes: torch.Tensor, w_codes: torch.Tensor):
        """fp32 gradients w.r.t. the signed operand values: (grad_a [M, K], grad_w [K, N])."""
        ga = torch.empty(a_codes.shape, dtype=torch.float32, device=grad_out.device)
        gw = torch.empty(w_codes.shape, dtype=torch.float32, device=grad_out.device)
        approx_ops.approx_gemm_backward(grad_out.contiguous(), a_codes, w_codes, ga, gw, self.ga, self.gb)
        return ga, gw
