"""NumPy restatement of the reference LUT-GEMM semantics (TEST INFRASTRUCTURE, not product code).

Only tests, the smoke check and the benchmark's cpu_baseline / reference legs may import this
module.  Every function cites the reference lines it follows (paths relative to the reference
project).  The reference ships no golden vectors for this path, so the pins are: fixtures generated
by importing the reference's own Python LUT loader and evaluating its gather expression
(tests/golden/make_golden.py), and the self-consistency of the reference's checked-in LUT files.
"""
from __future__ import annotations

import numpy as np

FACTOR = 1.0 / 16.0  # self_ops/src/approx_mult.h:41

_TAIL_PAD = {4: 718, 6: 830, 7: 638, 8: 0}  # self_ops/src/approx_mult.h:14-38


def geometry(bits: int):
    """(ROW, COL, ELEM_NUM) of the padded flat table, self_ops/src/approx_mult.h:13-40 and
    self_ops/ops_py/approx_ops.py:21-41."""
    if bits not in _TAIL_PAD:
        raise NotImplementedError(f"quantization_bit = {bits} is not supported")
    row, col = (1 << bits) + 1, (1 << bits) + 2
    return row, col, row * col + _TAIL_PAD[bits]


def bits_from_elem_num(n: int) -> int:
    for b in _TAIL_PAD:
        if geometry(b)[2] == n:
            return b
    raise ValueError(f"no bit-width has a padded table of {n} elements")


def pack_padded(dense: np.ndarray, bits: int, dtype) -> np.ndarray:
    """dense[2^b, 2^b] -> flat padded table; everything outside [0,2^b)^2 stays zero, which is what
    makes code 2^b the null code (self_ops/ops_py/approx_ops.py:51-53,70-77)."""
    row, col, elems = geometry(bits)
    q = 1 << bits
    assert dense.shape == (q, q)
    flat = np.zeros(elems, dtype=dtype)
    view = flat[: row * col].reshape(row, col)
    view[:q, :q] = dense.astype(dtype)
    return flat


def unpack_padded(flat: np.ndarray, bits: int) -> np.ndarray:
    row, col, elems = geometry(bits)
    q = 1 << bits
    assert flat.shape == (elems,)
    return flat[: row * col].reshape(row, col)[:q, :q].copy()


def parse_lut_file(path: str, bits: int):
    """Text LUT -> three dense int64 [2^b, 2^b] arrays (forward, d/da, d/db), following the state
    machine of self_ops/ops_py/approx_ops.py:54-79: header lines are skipped until the first section
    title, each data line is `a b value`."""
    q = 1 << bits
    tabs = {"fp": np.zeros((q, q), np.int64), "ga": np.zeros((q, q), np.int64), "gb": np.zeros((q, q), np.int64)}
    state = None
    with open(path, "r") as f:
        for line in f:
            if line.startswith("LUT for approximate multiplier:"):
                state = "fp"
                continue
            if line.startswith("LUT for the gradient of the approximate multiplier w.r.t. the first operand:"):
                state = "ga"
                continue
            if line.startswith("LUT for the gradient of the approximate multiplier w.r.t. the second operand:"):
                state = "gb"
                continue
            if state is None:
                continue
            a, b, res = line.split()
            tabs[state][int(a), int(b)] = int(res)
    return tabs["fp"], tabs["ga"], tabs["gb"]


def forward_np(a: np.ndarray, w: np.ndarray, lut_padded: np.ndarray, bits: int) -> np.ndarray:
    """C[m,n] = sum_k lut[a[m,k]*COL + w[k,n]] as uint32 (approx_gemm_forward.cu:183-208)."""
    _, col, _ = geometry(bits)
    M, K = a.shape
    K2, N = w.shape
    assert K == K2
    lut = lut_padded.astype(np.uint32)
    out = np.zeros((M, N), dtype=np.uint32)
    step = max(1, (1 << 24) // max(1, K * N))
    wi = w.astype(np.int64)[None, :, :]
    for m0 in range(0, M, step):
        ai = a[m0 : m0 + step].astype(np.int64)[:, :, None] * col
        out[m0 : m0 + step] = lut[ai + wi].sum(axis=1, dtype=np.uint32)
    return out


def backward_np_f64(gc, a, w, lut_ga_padded, lut_gw_padded, bits):
    """float64 evaluation of approx_gemm_backward.cu:213-241 / :447-475; returns (gA, gW, |gA|, |gW|)
    where the last two are the sums of absolute terms (the natural scale for an fp32 error bound)."""
    _, col, _ = geometry(bits)
    M, K = a.shape
    _, N = w.shape
    la = lut_ga_padded.astype(np.float64)
    lw = lut_gw_padded.astype(np.float64)
    ga = np.zeros((M, K)); ga_abs = np.zeros((M, K))
    gw = np.zeros((K, N)); gw_abs = np.zeros((K, N))
    step = max(1, (1 << 22) // max(1, K * N))
    wi = w.astype(np.int64)[None, :, :]
    g64 = gc.astype(np.float64)
    for m0 in range(0, M, step):
        idx = a[m0 : m0 + step].astype(np.int64)[:, :, None] * col + wi  # [m,k,n]
        g = g64[m0 : m0 + step][:, None, :]
        ta = la[idx] * g
        ga[m0 : m0 + step] = ta.sum(axis=2)
        ga_abs[m0 : m0 + step] = np.abs(ta).sum(axis=2)
        tw = lw[idx] * g
        gw += tw.sum(axis=0)
        gw_abs += np.abs(tw).sum(axis=0)
    return ga * FACTOR, gw * FACTOR, ga_abs * FACTOR, gw_abs * FACTOR


def im2col_codes(x: np.ndarray, kh: int, kw: int, stride: int, pad: int, dil: int) -> np.ndarray:
    """x[B,C,H,W] codes -> [B*Ho*Wo, C*kh*kw]; padding is code 0, K ordered (c,kh,kw)
    (self_ops/ops_py/approx_ops.py:556-563)."""
    B, C, H, W = x.shape
    Ho = (H + 2 * pad - dil * (kh - 1) - 1) // stride + 1
    Wo = (W + 2 * pad - dil * (kw - 1) - 1) // stride + 1
    xp = np.zeros((B, C, H + 2 * pad, W + 2 * pad), dtype=x.dtype)
    xp[:, :, pad : pad + H, pad : pad + W] = x
    cols = np.zeros((B, Ho, Wo, C, kh, kw), dtype=x.dtype)
    for i in range(kh):
        for j in range(kw):
            cols[:, :, :, :, i, j] = xp[:, :, i * dil : i * dil + stride * (Ho - 1) + 1 : stride,
                                        j * dil : j * dil + stride * (Wo - 1) + 1 : stride].transpose(0, 2, 3, 1)
    return cols.reshape(B * Ho * Wo, C * kh * kw)


def col2im_f64(gcol: np.ndarray, xshape, kh, kw, stride, pad, dil) -> np.ndarray:
    """adjoint of im2col_codes for gradients (autograd of F.unfold + F.pad in the reference)."""
    B, C, H, W = xshape
    Ho = (H + 2 * pad - dil * (kh - 1) - 1) // stride + 1
    Wo = (W + 2 * pad - dil * (kw - 1) - 1) // stride + 1
    g = gcol.reshape(B, Ho, Wo, C, kh, kw).astype(np.float64)
    gxp = np.zeros((B, C, H + 2 * pad, W + 2 * pad))
    for i in range(kh):
        for j in range(kw):
            gxp[:, :, i * dil : i * dil + stride * (Ho - 1) + 1 : stride,
                j * dil : j * dil + stride * (Wo - 1) + 1 : stride] += g[:, :, :, :, i, j].transpose(0, 3, 1, 2)
    return gxp[:, :, pad : pad + H, pad : pad + W]


# ---------------------------------------------------------------------------------------------
# Table generators
# ---------------------------------------------------------------------------------------------

def synthetic_tables(bits: int, seed: int = 0, half_window: int | None = None):
    """The benchmark's synthetic multiplier: L[x][y] = max(0, x*y + e), e integer uniform in
    [-2^(b-1), 2^(b-1)]; gradient tables are the clipped window difference
    (L[min(x+h,max)][y] - L[max(x-h,0)][y]) / (min(x+h,max) - max(x-h,0)) (and symmetrically in y).
    Returns (fp int64, ga float64, gb float64); h defaults to 2^b / 16 (8 for 7 bits)."""
    q = 1 << bits
    h = half_window if half_window is not None else max(1, q // 16)
    rng = np.random.default_rng(seed)
    e = rng.integers(-(q // 2), q // 2 + 1, size=(q, q))
    x = np.arange(q)
    L = np.maximum(0, x[:, None] * x[None, :] + e).astype(np.int64)
    hi = np.minimum(x + h, q - 1)
    lo = np.maximum(x - h, 0)
    ga = (L[hi, :] - L[lo, :]) / (hi - lo)[:, None]
    gb = (L[:, hi] - L[:, lo]) / (hi - lo)[None, :]
    return L, ga, gb


def to_wire(fp, ga, gb, bits):
    """dense tables -> the reference wire format: uint16 forward, int16 round(16*grad)
    (scripts/gen_bp_lut.py:164-183)."""
    assert fp.min() >= 0 and fp.max() < 2 ** 16
    qa = np.round(np.asarray(ga, dtype=np.float64) * 16.0).astype(np.int64)
    qb = np.round(np.asarray(gb, dtype=np.float64) * 16.0).astype(np.int64)
    assert qa.min() >= -2 ** 15 and qa.max() < 2 ** 15 and qb.min() >= -2 ** 15 and qb.max() < 2 ** 15
    return (pack_padded(fp, bits, np.uint16), pack_padded(qa, bits, np.int16), pack_padded(qb, bits, np.int16))


def reference_gradient_tables(fp: np.ndarray, half_ws: int):
    """Restatement of scripts/gen_bp_lut.py:7-62,171-183: moving-average smoothing (float32 means),
    central difference inside (half_ws, 2^b-1-half_ws), (max-min)/2^b at the borders, then
    round(16*g) -> int.  Reproduces the reference quirk at :58-59, where the border rule for the
    first-operand gradient takes max/min over ROW b of the table instead of column b."""
    q = fp.shape[0]
    lut = fp.astype(np.float32)
    smooth_a = np.zeros((q, q), np.float32)
    smooth_b = np.zeros((q, q), np.float32)
    for i in range(q):
        s, e = max(0, i - half_ws), min(q, i + half_ws + 1)
        smooth_a[i, :] = np.mean(lut[s:e, :], axis=0, dtype=np.float32)
        smooth_b[:, i] = np.mean(lut[:, s:e], axis=1, dtype=np.float32)
    grad_a = np.zeros((q, q), np.float32)
    grad_b = np.zeros((q, q), np.float32)
    inner = np.arange(q)
    inner = inner[(inner >= half_ws + 1) & (inner <= q - 1 - half_ws - 1)]
    border = np.setdiff1d(np.arange(q), inner)
    grad_a[inner, :] = (smooth_a[inner + 1, :] - smooth_a[inner - 1, :]) / 2
    grad_b[:, inner] = (smooth_b[:, inner + 1] - smooth_b[:, inner - 1]) / 2
    row_rng = (lut.max(axis=1) - lut.min(axis=1)) / q  # per row a
    grad_b[:, border] = row_rng[:, None]
    grad_a[border, :] = row_rng[None, :]  # quirk: indexed by b but computed over row b
    return (np.round(grad_a * np.float32(16.0)).astype(np.int64), np.round(grad_b * np.float32(16.0)).astype(np.int64))
