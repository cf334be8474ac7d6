"""Builds the reference's own CUDA extension (unmodified kernel sources) for sm_100a into oracle/_ref/,
once per bit-width, as a second GPU-side oracle and as the "reference kernel on the same B200" timing.

    python oracle/build_reference_ext.py [/path/to/reference] [bits ...]

The reference fixes the bit-width with an unconditional `#define QUANTIZATION_BIT 7`
(self_ops/src/approx_mult.h:12), so for every width the five source files are copied to a temporary
directory, that one line is rewritten there, and the copy is compiled under a distinct module name
(approx_ops_ref7, approx_ops_ref8).  Nothing of the reference is copied into this repository: only the
built shared objects land in oracle/_ref/ (git-ignored).  Building needs a reference checkout, nvcc and the
PyTorch headers; running needs only the built modules and a GPU.
TEST INFRASTRUCTURE: nothing in the product path imports these modules."""
import os
import re
import shutil
import subprocess
import sys
import sysconfig
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
FILES = ["op_register.cpp", "approx_gemm_forward.cu", "approx_gemm_backward.cu", "approx_mult.h", "cuda_helper.h"]


def build(ref: str, bits: int) -> str:
    from torch.utils import cpp_extension as ce
    import torch
    name = f"approx_ops_ref{bits}"
    so = os.path.join(OUT, name + sysconfig.get_config_var("EXT_SUFFIX"))
    os.makedirs(OUT, exist_ok=True)
    srcs = [os.path.join(ref, "self_ops", "src", f) for f in FILES]
    if os.path.exists(so) and os.path.getmtime(so) >= max(os.path.getmtime(f) for f in srcs + [__file__]):
        return so  # up to date
    with tempfile.TemporaryDirectory() as tmp:
        for f in FILES:
            shutil.copy(os.path.join(ref, "self_ops", "src", f), tmp)
        hdr = os.path.join(tmp, "approx_mult.h")
        text = open(hdr).read()
        text, n = re.subn(r"#define QUANTIZATION_BIT \d+", f"#define QUANTIZATION_BIT {bits}", text)
        assert n == 1
        open(hdr, "w").write(text)
        inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
        common = ["-O3", "-std=c++17", f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                  f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
        objs = []
        for f in FILES[:3]:
            obj = os.path.join(tmp, f + ".o")
            if f.endswith(".cu"):
                cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-c",
                       os.path.join(tmp, f), "-o", obj, *common, *inc, "--expt-relaxed-constexpr"]
            else:
                cmd = ["g++", "-fPIC", "-c", os.path.join(tmp, f), "-o", obj, *common, *inc]
            subprocess.run(cmd, check=True)
            objs.append(obj)
        libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
        subprocess.run(["g++", "-shared", "-o", so, *objs, f"-L{libdir}", "-lc10", "-ltorch", "-ltorch_cpu",
                        "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-L/usr/local/cuda/lib64", "-lcudart",
                        f"-Wl,-rpath,{libdir}"], check=True)
    return so


if __name__ == "__main__":
    args = sys.argv[1:]
    ref = args[0] if args and not args[0].isdigit() else os.environ.get("APPMULT_REFERENCE", "")
    if not os.path.isdir(ref):
        raise SystemExit("usage: build_reference_ext.py REFERENCE_CHECKOUT [bits ...]  (or set APPMULT_REFERENCE)")
    widths = [int(a) for a in args if a.isdigit()] or [7, 8]
    for b in widths:
        print(build(ref, b))
