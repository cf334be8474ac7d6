"""GPU test of the entry point that allocates nothing (lutgemm_backward_gw_noalloc), called through the
C-ABI.  It lives in a file of its own that is collected last, so a run that stops at the first failure
has already been through every other test.

The entry point serves callers that may not allocate device memory when the weight gradient is due (a
host runtime with a fixed memory budget, a binding that cannot reach the framework's allocator, a path
where cudaMalloc's implicit synchronisation is unacceptable): its partial sums go to a fixed 32 MiB array
inside the library instead of a scratch buffer from the caller.  Checked here: two calls in a row give
the same weight gradient as the regular entry point with a caller-allocated scratch buffer and as the CPU
oracle, to the tolerance the other gradient tests use (1e-5); the driver's count of free device memory does
not move across the calls (cudaMemGetInfo sees every allocation, whoever makes it - PyTorch's own counters
would only see PyTorch's); a call on a second stream gives the same result; problems whose partial sums
exceed the array are refused."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _problem(dev, bits, M, K, N, seed):
    from oracle import oracle_np as O
    g = torch.Generator(device="cpu").manual_seed(seed)
    _, _, lw = O.to_wire(*O.synthetic_tables(bits, seed=seed), bits)
    a = torch.randint(0, 1 << bits, (M, K), generator=g, dtype=torch.uint8).to(dev)
    w = torch.randint(0, 1 << bits, (K, N), generator=g, dtype=torch.uint8).to(dev)
    gc = torch.randn(M, N, generator=g).to(dev)
    return a, w, gc, torch.from_numpy(lw).to(dev)


def test_no_alloc_weight_gradient_matches_regular_entry_point_twice_in_a_row(oracle_c):
    assert torch.cuda.is_available(), "gpu-marked test started without a CUDA device"
    import approx_ops
    from oracle import oracle_np as O
    lib = approx_ops.library()
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.lutgemm_backward_gw_noalloc.restype = ci
    lib.lutgemm_backward_gw_noalloc.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]
    lib.lutgemm_noalloc_scratch_capacity.restype = ctypes.c_size_t
    cap = lib.lutgemm_noalloc_scratch_capacity()
    assert cap == 32 << 20

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    # first a slab-path problem with several row blocks of partial sums, then a split-M problem of another
    # shape: the second call finds the first call's partial sums in the array and must not be affected
    cases = [(8, 4096, 256, 320, 1), (6, 6000, 48, 64, 2), (8, 4096, 256, 320, 3)]
    for bits, M, K, N, seed in cases:
        a, w, gc, lw = _problem(dev, bits, M, K, N, seed)
        nbytes = lib.lutgemm_backward_scratch_bytes(bits, M, K, N)
        assert 0 < nbytes <= cap, "the case is meant to need scratch memory that fits the fixed array"
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        ref = torch.full((K, N), float("nan"), device=dev)
        rc = lib.lutgemm_backward(gc.data_ptr(), a.data_ptr(), w.data_ptr(), None, ref.data_ptr(), None, lw.data_ptr(),
                                  bits, M, K, N, scratch.data_ptr(), nbytes, stream)
        assert rc == 0
        got = torch.full((K, N), float("nan"), device=dev)
        got2 = torch.full((K, N), float("nan"), device=dev)
        side = torch.cuda.Stream(dev)
        # one call first: it looks up the array's address on this device and makes the driver load the kernels,
        # which may take device memory once per process; the calls measured below must take none
        rc = lib.lutgemm_backward_gw_noalloc(gc.data_ptr(), a.data_ptr(), w.data_ptr(), got.data_ptr(), lw.data_ptr(),
                                             bits, M, K, N, stream)
        assert rc == 0, lib.lutgemm_status_string(rc)
        torch.cuda.synchronize()
        got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        torch_before = torch.cuda.memory_allocated(dev)
        rc = lib.lutgemm_backward_gw_noalloc(gc.data_ptr(), a.data_ptr(), w.data_ptr(), got.data_ptr(), lw.data_ptr(),
                                             bits, M, K, N, stream)
        assert rc == 0, lib.lutgemm_status_string(rc)
        torch.cuda.synchronize()  # the calls share the one array: the second starts after the first has finished
        rc = lib.lutgemm_backward_gw_noalloc(gc.data_ptr(), a.data_ptr(), w.data_ptr(), got2.data_ptr(), lw.data_ptr(),
                                             bits, M, K, N, side.cuda_stream)
        assert rc == 0, lib.lutgemm_status_string(rc)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before, "device memory was taken during the calls"
        assert torch.cuda.memory_allocated(dev) == torch_before
        ref_n, got_n = ref.cpu().numpy(), got.cpu().numpy()
        assert np.isfinite(got_n).all()
        assert np.abs(got_n - ref_n).max() <= TOL * max(np.abs(ref_n).max(), 1e-30)
        assert torch.equal(got, got2), "the call on a second stream gave another result"
        # and against the CPU oracle (weight gradient only; its float64 sums and the sums of absolute terms)
        _, r_gw, _, r_gwa = oracle_c.backward_f64(gc.cpu().numpy(), a.cpu().numpy(), w.cpu().numpy(),
                                                  np.zeros_like(lw.cpu().numpy()), lw.cpu().numpy(), bits)
        assert (np.abs(got_n - r_gw) <= TOL * r_gwa + 1e-30).all()
    assert approx_ops.device_error() == 0


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    assert torch.cuda.is_available(), "gpu-marked test started without a CUDA device"
    import approx_ops
    lib = approx_ops.library()
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.lutgemm_backward_gw_noalloc.restype = ci
    lib.lutgemm_backward_gw_noalloc.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]
    dev = torch.device("cuda:0")
    bits, M, K, N = 8, 4096, 2048, 2048  # four 1024-row blocks x 16 MiB of partial sums = 64 MiB > 32 MiB
    a, w, gc, lw = _problem(dev, bits, M, K, N, 5)
    gw = torch.zeros(K, N, device=dev)
    rc = lib.lutgemm_backward_gw_noalloc(gc.data_ptr(), a.data_ptr(), w.data_ptr(), gw.data_ptr(), lw.data_ptr(),
                                         bits, M, K, N, None)
    assert rc == -5  # LUTGEMM_E_TOOLARGE
    assert b"size" in lib.lutgemm_status_string(rc)
    assert lib.lutgemm_backward_gw_noalloc(None, a.data_ptr(), w.data_ptr(), gw.data_ptr(), lw.data_ptr(),
                                           bits, M, K, N, None) == -1
    assert lib.lutgemm_backward_gw_noalloc(gc.data_ptr(), a.data_ptr(), w.data_ptr(), gw.data_ptr(), lw.data_ptr(),
                                           5, M, K, N, None) == -2
    torch.cuda.synchronize()
