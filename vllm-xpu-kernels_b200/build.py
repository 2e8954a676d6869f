"""In-tree build of the B200 fused-MoE binaries.

    python vllm-xpu-kernels_b200/build.py [--force]

Produces, next to the Python package:
  vllm_xpu_kernels/libb200moe.so     CUDA kernels + C ABI (nvcc, sm_100a only)
  vllm_xpu_kernels/_b200_torch_ops.so  torch operator registry (g++), links the above

Objects are cached under build/ by source hash, so a second run only relinks
what changed.  nvcc cross-compiles: no GPU is needed to build.
"""
import concurrent.futures
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CAPI = os.path.join(HERE, "csrc", "capi")
TORCH_SRC = os.path.join(HERE, "csrc", "torch", "bindings.cpp")
PKG = os.path.join(HERE, "vllm_xpu_kernels")
BUILD = os.path.join(HERE, "build")
INCLUDE = os.path.join(ROOT, "include")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CAPI]


def _hash(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    return r


def build_capi(force=False):
    os.makedirs(BUILD, exist_ok=True)
    headers = [os.path.join(CAPI, f) for f in os.listdir(CAPI) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(INCLUDE, "b200moe.h"))
    sources = sorted(os.path.join(CAPI, f) for f in os.listdir(CAPI) if f.endswith(".cu"))
    objs, jobs = [], []
    for src in sources:
        tag = _hash([src] + headers, " ".join(NVCC_FLAGS))
        obj = os.path.join(BUILD, os.path.basename(src)[:-3] + "." + tag + ".o")
        objs.append(obj)
        stem = os.path.basename(src)[:-3] + "."
        for old in os.listdir(BUILD):  # objects of earlier versions of this source
            if old.startswith(stem) and old.endswith(".o") and os.path.join(BUILD, old) != obj:
                os.remove(os.path.join(BUILD, old))
        if force or not os.path.exists(obj):
            jobs.append(["nvcc"] + NVCC_FLAGS + ["-c", src, "-o", obj])
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(_run, jobs))
    lib = os.path.join(PKG, "libb200moe.so")
    stamp = os.path.join(BUILD, "libb200moe.stamp")
    want = _hash(objs)
    if force or not os.path.exists(lib) or not os.path.exists(stamp) or open(stamp).read() != want:
        _run(["nvcc", "-shared", "-o", lib + ".tmp"] + objs + ["-lcudart"])
        os.replace(lib + ".tmp", lib)  # a reader (or a snapshot of the tree) never sees half a file
        open(stamp, "w").write(want)
    return lib


def build_torch_ops(force=False):
    import torch
    from torch.utils import cpp_extension as ce
    out = os.path.join(PKG, "_b200_torch_ops.so")
    stamp = os.path.join(BUILD, "torch_ops.stamp")
    want = _hash([TORCH_SRC, os.path.join(INCLUDE, "b200moe.h")], torch.__version__)
    if not force and os.path.exists(out) and os.path.exists(stamp) and open(stamp).read() == want:
        return out
    inc = []
    for p in ce.include_paths() + ["/usr/local/cuda/include", INCLUDE]:
        inc += ["-I", p]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi,
           "-DTORCH_EXTENSION_NAME=_b200_torch_ops"] + inc + [TORCH_SRC, "-o", out + ".tmp",
           "-L", tlib, "-L", PKG, "-L", "/usr/local/cuda/lib64",
           "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda", "-lb200moe", "-lcudart",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib]
    _run(cmd)
    os.replace(out + ".tmp", out)
    open(stamp, "w").write(want)
    return out


def build_all(force=False):
    return build_capi(force), build_torch_ops(force)


if __name__ == "__main__":
    for path in build_all("--force" in sys.argv):
        print("built", path)
