"""In-tree build of the CUDA extension.

Every ``.cu`` under ``csrc/`` is compiled by nvcc for ``sm_100a`` only (no torch headers, so a
file builds in seconds), ``bindings.cpp`` by g++ against the torch headers, and everything is
linked into ``picotron_b200/_C.so`` next to this package, where a GPU box finds it without a
rebuild. A stamp file holds the hash of all sources and flags; ``build()`` is a no-op while it
matches.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent.parent
REPO_DIR = PKG_DIR.parent
CSRC = REPO_DIR / "csrc"
OBJ_DIR = REPO_DIR / "build" / "obj"
SO_PATH = PKG_DIR / "_C.so"
STAMP_PATH = PKG_DIR / "_C.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _sources():
    cu = sorted(CSRC.rglob("*.cu"))
    cpp = sorted(CSRC.rglob("*.cpp"))
    hdr = sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")))
    return cu, cpp, hdr


def source_hash() -> str:
    cu, cpp, hdr = _sources()
    h = hashlib.sha256()
    for f in cu + cpp + hdr:
        h.update(str(f.relative_to(CSRC)).encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return SO_PATH.exists() and STAMP_PATH.exists() and STAMP_PATH.read_text().strip() == source_hash()


def _run(cmd, log_path=None):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path is not None:
        Path(log_path).write_text(" ".join(map(str, cmd)) + "\n" + p.stdout)
    if p.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd))}\n{p.stdout}")
    return p.stdout


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link the extension unless an up-to-date one exists. Returns the .so path."""
    if not force and is_current():
        return SO_PATH
    import torch
    from torch.utils import cpp_extension

    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cu, cpp, _ = _sources()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    jobs = []
    objs = []
    for src in cu:
        obj = OBJ_DIR / (str(src.relative_to(CSRC)).replace("/", "_") + ".o")
        objs.append(obj)
        jobs.append(([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
                     str(obj) + ".log"))
    torch_inc = cpp_extension.include_paths()
    py_inc = sysconfig.get_paths()["include"]
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for src in cpp:
        obj = OBJ_DIR / (str(src.relative_to(CSRC)).replace("/", "_") + ".o")
        objs.append(obj)
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
               "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
               "-I", str(CSRC), "-I", py_inc, "-I", cuda_inc]
        for inc in torch_inc:
            cmd += ["-isystem", inc]
        cmd += ["-c", str(src), "-o", str(obj)]
        jobs.append((cmd, str(obj) + ".log"))
    with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        outs = list(ex.map(lambda j: _run(*j), jobs))
    if verbose:
        for o in outs:
            sys.stderr.write(o)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    site = os.path.dirname(os.path.dirname(torch.__file__))
    cudart_dir = os.path.join(site, "nvidia", "cuda_runtime", "lib")
    link = ["g++", "-shared", *map(str, objs), "-o", str(SO_PATH),
            f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-ltorch_python", f"-Wl,-rpath,{torch_lib}"]
    if os.path.exists(os.path.join(cudart_dir, "libcudart.so.12")):
        link += [f"-L{cudart_dir}", "-l:libcudart.so.12", f"-Wl,-rpath,{cudart_dir}"]
    else:
        link += ["-L/usr/local/cuda/lib64", "-lcudart"]
    _run(link)
    STAMP_PATH.write_text(source_hash() + "\n")
    return SO_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
