"""Look-up-table files: gradient-table generators and the text format the training scripts load.

Covers what the reference does offline with `scripts/gen_bp_lut.py` (forward table -> the two
difference-based gradient tables, written as a three-section text file that
`self_ops.init_lookup_tables` reads): the same smoothing + central-difference rule, vectorised, plus the
clipped window-difference rule of the synthetic benchmark multiplier, and a writer for the file format.
Tables are dense NumPy arrays [2^b, 2^b]; gradients are returned as integers scaled by 16 (the fixed
point of the wire format, `FACTOR = 1/16` in self_ops/src/approx_mult.h:41)."""
from __future__ import annotations

import numpy as np

GRAD_SCALE = 16

TITLES = (
    "LUT for approximate multiplier:",
    "LUT for the gradient of the approximate multiplier w.r.t. the first operand:",
    "LUT for the gradient of the approximate multiplier w.r.t. the second operand:",
)


def smoothed_difference_gradients(fp: np.ndarray, half_window: int):
    """The reference's rule (scripts/gen_bp_lut.py:7-62): moving-average smoothing of the forward table
    along the differentiated operand (window 2*half_window+1, clipped at the borders, float32 means),
    then (s[i+1] - s[i-1]) / 2 for half_window < i < 2^b - 1 - half_window and (max - min) / 2^b of the
    unsmoothed table at the borders.  At the borders the reference takes max/min over ROW b of the
    table also for the first-operand gradient (its :58-59 index a row where a column is meant); that is
    reproduced so that files generated here equal the reference's checked-in ones.
    Returns (grad_a, grad_b) as int64 = round(16 * gradient)."""
    if half_window < 1:
        raise ValueError("half_window must be >= 1")
    q = fp.shape[0]
    lut = np.asarray(fp, dtype=np.float32)
    idx = np.arange(q)
    smooth_a = np.empty((q, q), np.float32)
    smooth_b = np.empty((q, q), np.float32)
    for i in range(q):  # float32 means over the clipped window, one table line at a time
        lo, hi = max(0, i - half_window), min(q, i + half_window + 1)
        smooth_a[i, :] = np.mean(lut[lo:hi, :], axis=0, dtype=np.float32)
        smooth_b[:, i] = np.mean(lut[:, lo:hi], axis=1, dtype=np.float32)
    inner = idx[(idx >= half_window + 1) & (idx <= q - 2 - half_window)]
    border = np.setdiff1d(idx, inner)
    grad_a = np.zeros((q, q), np.float32)
    grad_b = np.zeros((q, q), np.float32)
    grad_a[inner, :] = (smooth_a[inner + 1, :] - smooth_a[inner - 1, :]) / np.float32(2)
    grad_b[:, inner] = (smooth_b[:, inner + 1] - smooth_b[:, inner - 1]) / np.float32(2)
    row_range = (lut.max(axis=1) - lut.min(axis=1)) / np.float32(q)
    grad_b[:, border] = row_range[:, None]
    grad_a[border, :] = row_range[None, :]
    scale = np.float32(GRAD_SCALE)
    return np.round(grad_a * scale).astype(np.int64), np.round(grad_b * scale).astype(np.int64)


def window_difference_gradients(fp: np.ndarray, half_window: int):
    """The benchmark's rule: (L[min(x+h, max)][y] - L[max(x-h, 0)][y]) / (min(x+h, max) - max(x-h, 0)) for
    the first operand and symmetrically for the second.  Returns int64 = round(16 * gradient)."""
    q = fp.shape[0]
    L = np.asarray(fp, dtype=np.float64)
    x = np.arange(q)
    hi, lo = np.minimum(x + half_window, q - 1), np.maximum(x - half_window, 0)
    ga = (L[hi, :] - L[lo, :]) / (hi - lo)[:, None]
    gb = (L[:, hi] - L[:, lo]) / (hi - lo)[None, :]
    return np.round(ga * GRAD_SCALE).astype(np.int64), np.round(gb * GRAD_SCALE).astype(np.int64)


def synthetic_multiplier(bits: int, seed: int = 0) -> np.ndarray:
    """L[x][y] = max(0, x*y + e), e integer uniform in [-2^(b-1), 2^(b-1)] (the benchmark's multiplier)."""
    q = 1 << bits
    rng = np.random.default_rng(seed)
    e = rng.integers(-(q // 2), q // 2 + 1, size=(q, q))
    x = np.arange(q)
    return np.maximum(0, x[:, None] * x[None, :] + e).astype(np.int64)


def error_metrics(fp: np.ndarray) -> dict:
    """The self-consistency figures the reference prints into its file headers (gen_bp_lut.py:118-126)."""
    q = fp.shape[0]
    x = np.arange(q)
    exact = (x[:, None] * x[None, :]).astype(np.float64)
    err = np.abs(np.asarray(fp, np.float64) - exact)
    return {"mse": float((err ** 2).mean()), "error_rate_pct": float((err != 0).mean() * 100),
            "med": float(err.mean()), "nmed_pct": float(err.mean() / q ** 2 * 100), "max_ed": float(err.max())}


def write_lut_file(path: str, fp: np.ndarray, grad_a: np.ndarray, grad_b: np.ndarray, header: str = "") -> None:
    """Writes the three-section text format (`a b value` lines) that init_lookup_tables parses."""
    q = fp.shape[0]
    for name, t, lo, hi in (("forward", fp, 0, 0xFFFF), ("grad_a", grad_a, -32768, 32767), ("grad_b", grad_b, -32768, 32767)):
        if t.shape != (q, q) or t.min() < lo or t.max() > hi:
            raise ValueError(f"{name} table does not fit the wire format")
    a, b = np.meshgrid(np.arange(q), np.arange(q), indexing="ij")
    with open(path, "w") as f:
        m = error_metrics(fp)
        f.write(f"INFO: generated by lutgemm_luts.write_lut_file {header}\n")
        f.write(f"INFO: Mean squared error between lut_appmult and lut_accmult: {m['mse']}\n")
        f.write(f"INFO: Mean error distance between lut_appmult and lut_mult: {m['med']}\n")
        for title, t in zip(TITLES, (fp, grad_a, grad_b)):
            f.write(title + "\n")
            rows = np.stack([a.ravel(), b.ravel(), np.asarray(t, np.int64).ravel()], axis=1)
            f.write("\n".join(" ".join(map(str, r)) for r in rows.tolist()) + "\n")


def load_lut_file(path: str, bits: int, cache: bool = True):
    """Three dense int64 [2^b, 2^b] tables (forward, d/da * 16, d/db * 16) from a LUT text file, with a binary
    cache beside it: parsing a 8-bit file means 196 608 text lines, the cache (`<file>.b<bits>.npz`, rewritten
    whenever the text file is newer) loads in milliseconds.  The `INFO:` header's mean error distance, when
    present, is checked against the parsed forward table."""
    import os
    import re
    cache_path = f"{path}.b{bits}.npz"
    if cache and os.path.exists(cache_path) and os.path.getmtime(cache_path) >= os.path.getmtime(path):
        z = np.load(cache_path)
        return z["fp"], z["grad_a"], z["grad_b"]
    q = 1 << bits
    tables = [np.zeros((q, q), np.int64) for _ in range(3)]
    section, med = -1, None
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line in TITLES:
                section = TITLES.index(line)
                continue
            if section < 0:
                m = re.search(r"Mean error distance[^:]*:\s*([0-9.eE+-]+)", line)
                if m:
                    med = float(m.group(1))
                continue
            parts = line.split()
            if len(parts) == 3:
                a, b, v = int(parts[0]), int(parts[1]), int(parts[2])
                if a < q and b < q:
                    tables[section][a, b] = v
    if section != 2:
        raise ValueError(f"{path}: expected three table sections, found {section + 1}")
    if med is not None and abs(error_metrics(tables[0])["med"] - med) > 1e-3 * max(1.0, med):
        raise ValueError(f"{path}: header mean error distance {med} does not match the table")
    if cache:
        try:
            np.savez(cache_path, fp=tables[0], grad_a=tables[1], grad_b=tables[2])
        except OSError:
            pass  # read-only location: just skip the cache
    return tuple(tables)
