"""ctypes front-end of oracle/lutgemm_oracle.c (TEST INFRASTRUCTURE)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .build_oracle import load_oracle


def _p(arr, ctype):
    return arr.ctypes.data_as(C.POINTER(ctype)) if arr is not None else None


class OracleC:
    """NumPy-array interface to the C restatement; see the C file for the reference citations."""

    def __init__(self):
        self.lib = load_oracle()
        L = self.lib
        L.oracle_forward.restype = C.c_int
        L.oracle_backward.restype = C.c_int
        L.oracle_backward_f64.restype = C.c_int
        L.oracle_lut_elem_num.restype = C.c_int
        L.oracle_num_threads.restype = C.c_int

    def num_threads(self) -> int:
        return int(self.lib.oracle_num_threads())

    def set_num_threads(self, n: int) -> None:
        self.lib.oracle_set_num_threads(C.c_int(n))

    def lut_elem_num(self, bits: int) -> int:
        return int(self.lib.oracle_lut_elem_num(C.c_int(bits)))

    def forward(self, a, w, lut, bits):
        a = np.ascontiguousarray(a, np.uint8); w = np.ascontiguousarray(w, np.uint8)
        lut = np.ascontiguousarray(lut, np.uint16)
        M, K = a.shape; _, N = w.shape
        c = np.empty((M, N), np.uint32)
        rc = self.lib.oracle_forward(_p(a, C.c_uint8), _p(w, C.c_uint8), _p(c, C.c_uint32), _p(lut, C.c_uint16),
                                     C.c_int(bits), C.c_long(M), C.c_long(K), C.c_long(N))
        assert rc == 0
        return c

    def backward(self, gc, a, w, lut_ga, lut_gw, bits):
        gc = np.ascontiguousarray(gc, np.float32)
        a = np.ascontiguousarray(a, np.uint8); w = np.ascontiguousarray(w, np.uint8)
        lut_ga = np.ascontiguousarray(lut_ga, np.int16); lut_gw = np.ascontiguousarray(lut_gw, np.int16)
        M, K = a.shape; _, N = w.shape
        ga = np.empty((M, K), np.float32); gw = np.empty((K, N), np.float32)
        rc = self.lib.oracle_backward(_p(gc, C.c_float), _p(a, C.c_uint8), _p(w, C.c_uint8), _p(ga, C.c_float),
                                      _p(gw, C.c_float), _p(lut_ga, C.c_int16), _p(lut_gw, C.c_int16),
                                      C.c_int(bits), C.c_long(M), C.c_long(K), C.c_long(N))
        assert rc == 0
        return ga, gw

    def backward_f64(self, gc, a, w, lut_ga, lut_gw, bits):
        gc = np.ascontiguousarray(gc, np.float32)
        a = np.ascontiguousarray(a, np.uint8); w = np.ascontiguousarray(w, np.uint8)
        lut_ga = np.ascontiguousarray(lut_ga, np.int16); lut_gw = np.ascontiguousarray(lut_gw, np.int16)
        M, K = a.shape; _, N = w.shape
        ga = np.empty((M, K)); gw = np.empty((K, N)); gaa = np.empty((M, K)); gwa = np.empty((K, N))
        rc = self.lib.oracle_backward_f64(_p(gc, C.c_float), _p(a, C.c_uint8), _p(w, C.c_uint8), _p(ga, C.c_double),
                                          _p(gw, C.c_double), _p(gaa, C.c_double), _p(gwa, C.c_double),
                                          _p(lut_ga, C.c_int16), _p(lut_gw, C.c_int16),
                                          C.c_int(bits), C.c_long(M), C.c_long(K), C.c_long(N))
        assert rc == 0
        return ga, gw, gaa, gwa

    def im2col(self, x, kh, kw, stride, pad, dil):
        x = np.ascontiguousarray(x, np.uint8)
        B, Cc, H, W = x.shape
        Ho = (H + 2 * pad - dil * (kh - 1) - 1) // stride + 1
        Wo = (W + 2 * pad - dil * (kw - 1) - 1) // stride + 1
        col = np.empty((B * Ho * Wo, Cc * kh * kw), np.uint8)
        self.lib.oracle_im2col_u8(_p(x, C.c_uint8), _p(col, C.c_uint8), C.c_long(B), C.c_long(Cc), C.c_long(H),
                                  C.c_long(W), C.c_long(kh), C.c_long(kw), C.c_long(stride), C.c_long(pad), C.c_long(dil))
        return col

    def col2im(self, gcol, xshape, kh, kw, stride, pad, dil):
        gcol = np.ascontiguousarray(gcol, np.float32)
        B, Cc, H, W = xshape
        gx = np.empty((B, Cc, H, W), np.float32)
        self.lib.oracle_col2im_f32(_p(gcol, C.c_float), _p(gx, C.c_float), C.c_long(B), C.c_long(Cc), C.c_long(H),
                                   C.c_long(W), C.c_long(kh), C.c_long(kw), C.c_long(stride), C.c_long(pad), C.c_long(dil))
        return gx
