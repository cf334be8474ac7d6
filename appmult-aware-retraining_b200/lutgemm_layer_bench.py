"""Per-layer timing of the ResNet-18 (CIFAR shape) convolutions through the fused kernels:

    python lutgemm_layer_bench.py [bits] [batch]

For every distinct convolution of the network: implicit-im2col forward, grad_w and grad_x (LUT gradient +
col2im) in ms (CUDA events) and as a fraction of the shared-memory look-up roofline (SMs x clock x 32), with the
per-step totals weighted by how often the layer occurs.  Each call is timed on its own, so the grad_w figure
includes the code transposition that a training step shares with the forward pass."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import approx_ops  # noqa: E402
from lutgemm_luts import synthetic_multiplier, window_difference_gradients  # noqa: E402

# name, Cin, H = W, Cout, kernel, stride, pad, occurrences in the network
LAYERS = [("stem", 3, 32, 64, 3, 1, 1, 1), ("s1", 64, 32, 64, 3, 1, 1, 4), ("s2a", 64, 32, 128, 3, 2, 1, 1),
          ("s2", 128, 16, 128, 3, 1, 1, 3), ("s2sc", 64, 32, 128, 1, 2, 0, 1), ("s3a", 128, 16, 256, 3, 2, 1, 1),
          ("s3", 256, 8, 256, 3, 1, 1, 3), ("s3sc", 128, 16, 256, 1, 2, 0, 1), ("s4a", 256, 8, 512, 3, 2, 1, 1),
          ("s4", 512, 4, 512, 3, 1, 1, 3), ("s4sc", 256, 8, 512, 1, 2, 0, 1)]


def wire(dense, bits, dtype):
    q = 1 << bits
    flat = np.zeros(approx_ops.library().lutgemm_lut_elem_num(bits), dtype=dtype)
    flat[: (q + 1) * (q + 2)].reshape(q + 1, q + 2)[:q, :q] = dense
    return flat


def timeit(fn, reps=3):
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
    bits = int(sys.argv[1]) if len(sys.argv) > 1 else 7
    B = int(sys.argv[2]) if len(sys.argv) > 2 else 256
    dev = torch.device("cuda:0")
    fp = synthetic_multiplier(bits, seed=0)
    ga, gb = window_difference_gradients(fp, max(1, (1 << bits) // 16))
    lf = torch.from_numpy(wire(fp, bits, np.uint16)).to(dev)
    la = torch.from_numpy(wire(ga, bits, np.int16)).to(dev)
    lw = torch.from_numpy(wire(gb, bits, np.int16)).to(dev)
    props = torch.cuda.get_device_properties(dev)
    roof = props.multi_processor_count * 1965e6 * 32
    tot = [0.0, 0.0, 0.0]
    print("layer      M      K    N  cnt |  fwd ms  %roof |   gw ms  %roof |   gx ms  %roof")
    for name, cin, hw, cout, k, st, p, cnt in LAYERS:
        x = torch.randint(0, 1 << bits, (B, cin, hw, hw), dtype=torch.uint8, device=dev)
        wm = torch.randint(0, 1 << bits, (cin * k * k, cout), dtype=torch.uint8, device=dev)
        ho = (hw + 2 * p - k) // st + 1
        M, K = B * ho * ho, cin * k * k
        y = torch.empty(M, cout, dtype=torch.uint32, device=dev)
        gy = torch.randn(M, cout, device=dev)
        gx, gw = torch.empty(B, cin, hw, hw, device=dev), torch.empty(K, cout, device=dev)
        tf = timeit(lambda: approx_ops.approx_conv2d_forward(x, wm, y, lf, k, k, st, p, 1))
        tw = timeit(lambda: approx_ops.approx_conv2d_backward(gy, x, wm, None, gw, la, lw, k, k, st, p, 1))
        tx = timeit(lambda: approx_ops.approx_conv2d_backward(gy, x, wm, gx, None, la, lw, k, k, st, p, 1)) if name != "stem" else 0.0
        look = M * K * cout
        pr = lambda t: 100 * look / (t * 1e-3) / roof if t > 0 else 0.0
        print(f"{name:6s} {M:6d} {K:5d} {cout:4d} x{cnt} | {tf:7.3f} {pr(tf):5.1f}  | {tw:7.3f} {pr(tw):5.1f}  | {tx:7.3f} {pr(tx):5.1f}",
              flush=True)
        for i, t in enumerate((tf, tw, tx)):
            tot[i] += t * cnt
    print("totals per step (ms): fwd %.2f gw %.2f gx %.2f sum %.2f" % (tot[0], tot[1], tot[2], sum(tot)))


if __name__ == "__main__":
    main()
