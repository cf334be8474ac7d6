"""Generates the golden fixtures under tests/golden/ from the reference's own Python layer.

Needs a checkout of the reference project (the fixtures it writes are what the tests read):

    python tests/golden/make_golden.py [/path/to/reference]

The reference has no CPU kernel, so its compiled `approx_ops` module is replaced by a stand-in whose
two functions evaluate the reference's LUT-gather semantics with plain PyTorch indexing on the CPU
(index a*COL + b into the padded flat table, exactly the tensors the reference's own
`init_lookup_tables` builds).  Everything above that stand-in - the LUT text parser, the autograd
Functions, the unfold-based convolution wrapper - is the reference's unmodified Python, imported
from the checkout.  Each fixture stores seeded inputs, the padded tables and the resulting outputs.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("APPMULT_REFERENCE", "")
if not os.path.isdir(REF):
    raise SystemExit("usage: make_golden.py REFERENCE_CHECKOUT  (or set APPMULT_REFERENCE)")
OUT = os.path.dirname(os.path.abspath(__file__))

LUT_FILES = {
    "mult7_med63": ("app_mults/resub_als/Mult_7_7_MED_63.6771_size_178_depth_23_lutfp+bp_avg_8_8.txt", 7),
    "mul8u_17C8": ("app_mults/evo_selected/mult8u/mul8u_17C8_lutfp+bp_avg_16_16.txt", 8),
    "trunc6": ("app_mults/vert_trunc/mult6u/6_6_U_SP_WT_CL_GenMul_vertical_truncation_4cols_lutfp+bp_avg_2_2.txt", 6),
}

GEMM_SHAPES = [(1, 1, 1), (3, 5, 2), (17, 27, 10), (33, 64, 65), (64, 96, 80), (129, 40, 257), (70, 150, 33)]
CONV_CASES = [  # (B, Cin, H, W, Cout, k, stride, pad, dil)
    (2, 3, 8, 8, 5, 3, 1, 1, 1),
    (1, 4, 9, 7, 6, 3, 2, 1, 1),
    (2, 2, 6, 6, 3, 1, 1, 0, 1),
    (1, 3, 10, 10, 4, 3, 1, 2, 2),
]


def install_stub():
    stub = types.ModuleType("approx_ops")

    def _col(lut):
        n = lut.numel()
        return {1024: 18, 5120: 66, 17408: 130, 66306: 258}[n]

    def approx_gemm_forward(a, b, c, lut):
        col = _col(lut)
        idx = a.long()[:, :, None] * col + b.long()[None, :, :]
        s = lut.to(torch.int64)[idx].sum(dim=1)
        c.copy_((s & 0xFFFFFFFF).to(torch.uint32))

    def approx_gemm_backward(gc, a, b, ga, gb, lut_ga, lut_gb):
        col = _col(lut_ga)
        idx = a.long()[:, :, None] * col + b.long()[None, :, :]  # [M,K,N]
        ga.copy_((gc[:, None, :] * lut_ga.to(torch.float32)[idx]).sum(dim=2) * (1 / 16.0))
        gb.copy_((lut_gb.to(torch.float32)[idx] * gc[:, None, :]).sum(dim=0) * (1 / 16.0))

    def acc_gemm_forward_fp32(a, b, c):
        c.copy_(a @ b)

    stub.approx_gemm_forward = approx_gemm_forward
    stub.approx_gemm_backward = approx_gemm_backward
    stub.acc_gemm_forward_fp32 = acc_gemm_forward_fp32
    sys.modules["approx_ops"] = stub


def main():
    install_stub()
    sys.path.insert(0, REF)
    import self_ops as ref_self_ops  # the reference package, unmodified
    from self_ops.ops_py import approx_ops as ref_ops

    for name, (rel, bits) in LUT_FILES.items():
        ref_self_ops.init_lookup_tables("cpu", os.path.join(REF, rel), bits)
        lut_fp = ref_ops.lut_appmult.numpy().copy()
        lut_ga = ref_ops.lut_grad_a.numpy().copy()
        lut_gb = ref_ops.lut_grad_b.numpy().copy()
        q = 1 << bits
        data = {"bits": np.int64(bits), "lut_fp": lut_fp, "lut_ga": lut_ga, "lut_gb": lut_gb}
        g = torch.Generator().manual_seed(1234 + bits)
        for i, (M, K, N) in enumerate(GEMM_SHAPES):
            a = torch.randint(0, q, (M, K), generator=g).float().requires_grad_(True)
            b = torch.randint(0, q, (K, N), generator=g).float().requires_grad_(True)
            if i == 0:  # extremes
                a.data.fill_(q - 1); b.data.fill_(q - 1)
            gc = torch.randn(M, N, generator=g)
            c = ref_self_ops.approx_gemm_op(a, b)
            c.backward(gc)
            data[f"gemm{i}_a"] = a.detach().numpy().astype(np.uint8)
            data[f"gemm{i}_b"] = b.detach().numpy().astype(np.uint8)
            data[f"gemm{i}_gc"] = gc.numpy()
            data[f"gemm{i}_c"] = c.detach().numpy()
            data[f"gemm{i}_ga"] = a.grad.numpy().copy()
            data[f"gemm{i}_gb"] = b.grad.numpy().copy()
        for i, (B, Cin, H, W, Cout, k, s, p, d) in enumerate(CONV_CASES):
            x = torch.randint(0, q, (B, Cin, H, W), generator=g).float().requires_grad_(True)
            wt = torch.randint(0, q, (Cout, Cin, k, k), generator=g).float().requires_grad_(True)
            y = ref_self_ops.approx_conv2d_op(x, wt, bias=None, stride=(s, s), padding=(p, p), dilation=(d, d), groups=1)
            gy = torch.randn(y.shape, generator=g)
            y.backward(gy)
            data[f"conv{i}_cfg"] = np.array([B, Cin, H, W, Cout, k, s, p, d], np.int64)
            data[f"conv{i}_x"] = x.detach().numpy().astype(np.uint8)
            data[f"conv{i}_w"] = wt.detach().numpy().astype(np.uint8)
            data[f"conv{i}_gy"] = gy.numpy()
            data[f"conv{i}_y"] = y.detach().numpy()
            data[f"conv{i}_gx"] = x.grad.numpy().copy()
            data[f"conv{i}_gw"] = wt.grad.numpy().copy()
        path = os.path.join(OUT, f"golden_{name}.npz")
        np.savez_compressed(path, **data)
        print(path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
