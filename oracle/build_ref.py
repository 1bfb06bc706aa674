"""Build the reference's own CUDA implementation of the path as a GPU oracle (TEST INFRASTRUCTURE).

Compiles, straight from the reference tree where it lies (nothing is copied into this repository), the
"Route L" sources its setup.py lists (plugin/setup.py:57-82: lcpp_shim.cu, lcpp_owned_{k4,iq3_mma,mma_k}.cu,
the vendored mmvq.cu, quantize.cu and nine mmq template instances) with the same nvcc flags
(plugin/setup.py:34-42, 74-82) for sm_100a, and links them into  oracle/_ref/ref_C_gguf.so , a torch op
library that defines torch.ops._C_gguf.lcpp_* exactly as the reference does. Those kernels carry no sm_100
code path; on a B200 they run their mma.sync / dp4a code.

The library defines the same op names as this repository's own registration, so it is only ever loaded in a
separate process (oracle/ref_runner.py). Used by tests/test_gpu_vs_reference.py; never by the product.

    python oracle/build_ref.py [/path/to/reference]
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "ref_C_gguf.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def reference_root() -> str | None:
    """Where the reference tree is: $GSQ_REFERENCE, else a checkout named `reference` beside this repository."""
    cand = os.environ.get("GSQ_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(cand) else None


def build(ref: str | None = None, force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension

    ref = ref or reference_root()
    if ref is None:
        raise FileNotFoundError("no reference tree: set GSQ_REFERENCE")
    csrc = os.path.join(ref, "plugin", "vllm_gguf_plugin", "csrc")
    if not os.path.isdir(csrc):
        raise FileNotFoundError(csrc)
    if os.path.exists(OUT) and not force:
        return OUT
    lcpp = os.path.join(csrc, "lcpp")
    cuda = os.path.join(lcpp, "ggml", "src", "ggml-cuda")
    srcs = [os.path.join(csrc, f) for f in ("lcpp_shim.cu", "lcpp_owned_k4.cu", "lcpp_owned_iq3_mma.cu", "lcpp_owned_mma_k.cu")]
    srcs += [os.path.join(cuda, f) for f in ("mmvq.cu", "quantize.cu")]
    srcs += [os.path.join(cuda, "template-instances", f"mmq-instance-{t}.cu")
             for t in ("iq2_s", "iq2_xs", "iq2_xxs", "iq3_s", "iq3_xxs", "iq4_xs", "q2_k", "q4_k", "q6_k")]
    incs = [os.path.join(lcpp, "ggml", "include"), os.path.join(lcpp, "ggml", "src"), cuda, csrc, os.path.join(csrc, "gguf")]
    incs += cpp_extension.include_paths("cuda")
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--use_fast_math", "-DUSE_CUDA", "-DNDEBUG",
             "--extended-lambda", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
             "-U__CUDA_NO_HALF2_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-Xcompiler", "-fPIC",
             "-DTORCH_EXTENSION_NAME=ref_C_gguf", "-D_GLIBCXX_USE_CXX11_ABI=1", "--expt-relaxed-constexpr"]
    try:
        import nvidia

        for base in nvidia.__path__:
            for sub in sorted(os.listdir(base)):
                inc = os.path.join(base, sub, "include")
                if os.path.exists(os.path.join(inc, "cublas_v2.h")):
                    flags += ["-Xcompiler", f"-idirafter,{inc}"]
    except ImportError:
        pass
    os.makedirs(OUT_DIR, exist_ok=True)
    objs = []

    def compile_one(src):
        obj = os.path.join(OUT_DIR, os.path.basename(src)[:-3] + ".o")
        cmd = [NVCC, *flags, *[f"-I{i}" for i in incs], "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on " + src + "\n" + r.stderr[-3000:])
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, srcs))
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [NVCC, "-shared", "-o", OUT, *objs, f"-L{libdir}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           "-Xlinker", f"-rpath={libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed\n" + r.stderr[-3000:])
    for o in objs:
        os.remove(o)
    return OUT


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
