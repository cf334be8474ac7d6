"""Times the reference's own CUDA kernels (oracle/_ref/, see build_reference_ext.py) next to this
library's on the same GPU and inputs: forward, and backward (both gradients), CUDA events.

    python oracle/time_reference_ext.py [size | MxKxN] [bits ...]

TEST INFRASTRUCTURE: a measurement aid, not part of the product path."""
import glob
import importlib.util
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "appmult-aware-retraining_b200")]
import approx_ops  # noqa: E402
from oracle import oracle_np as O  # noqa: E402


def timed(fn, reps):
    fn(); fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def main():
    shape = sys.argv[1] if len(sys.argv) > 1 else "4096"
    dims = [int(v) for v in shape.split("x")]
    size = dims[0]
    widths = [int(a) for a in sys.argv[2:]] or [7, 8]
    dev = torch.device("cuda:0")
    for bits in widths:
        hits = glob.glob(os.path.join(ROOT, "oracle", "_ref", f"approx_ops_ref{bits}*.so"))
        if not hits:
            print(json.dumps({"bits": bits, "unavailable": "oracle/_ref module not built"}))
            continue
        spec = importlib.util.spec_from_file_location(f"approx_ops_ref{bits}", hits[0])
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
        lf, la, lw = (torch.from_numpy(t).to(dev) for t in O.to_wire(*O.synthetic_tables(bits, seed=0), bits))
        M, K, N = dims if len(dims) == 3 else (size, size, size)
        a = torch.randint(0, 1 << bits, (M, K), dtype=torch.uint8, device=dev)
        w = torch.randint(0, 1 << bits, (K, N), dtype=torch.uint8, device=dev)
        gc = torch.randn(M, N, device=dev)
        c = torch.zeros(M, N, dtype=torch.uint32, device=dev)
        ga, gw = torch.zeros(M, K, device=dev), torch.zeros(K, N, device=dev)
        reps = 3
        out = {"bits": bits, "M": M, "K": K, "N": N,
               "reference_forward_ms": timed(lambda: ref.approx_gemm_forward(a, w, c, lf), reps),
               "reference_backward_ms": timed(lambda: ref.approx_gemm_backward(gc, a, w, ga, gw, la, lw), reps),
               "ours_forward_ms": timed(lambda: approx_ops.approx_gemm_forward(a, w, c, lf), reps),
               "ours_backward_ms": timed(lambda: approx_ops.approx_gemm_backward(gc, a, w, ga, gw, la, lw), reps)}
        out["speedup_fwd_bwd"] = (out["reference_forward_ms"] + out["reference_backward_ms"]) / \
                                 (out["ours_forward_ms"] + out["ours_backward_ms"])
        print(json.dumps(out))


if __name__ == "__main__":
    main()
