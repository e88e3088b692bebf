"""In-tree build of the native extension.

Every ``.cu`` file under ``csrc/kernels`` is compiled by nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``); the ``.cpp`` files under ``csrc/host`` and
``csrc/bindings.cpp`` are compiled by the host compiler; everything is linked into
``async_grpo_nccl_b200/_C.so`` next to this file, so that the shared object travels with the
source tree. Objects are rebuilt only when the content hash of the source (and of every header
under ``csrc``) changes.
"""
from __future__ import annotations

import hashlib
import json
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR.parent / "build" / "agrpo_ext"
SO_PATH = PKG_DIR / "_C.so"
STAMP_PATH = PKG_DIR / "_C.stamp.json"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "--use_fast_math",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function"]


def _cuda_home() -> str:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return cand
    raise RuntimeError("nvcc not found; set CUDA_HOME")


def _sources():
    cu = sorted((CSRC / "kernels").glob("*.cu"))
    cpp = sorted((CSRC / "host").glob("*.cpp")) + [CSRC / "bindings.cpp"]
    headers = sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")))
    return cu, cpp, headers


def _hash(paths, extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(str(p.relative_to(CSRC)).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def source_hash() -> str:
    cu, cpp, headers = _sources()
    return _hash(cu + cpp + headers, " ".join(NVCC_FLAGS + CXX_FLAGS))


def is_current() -> bool:
    if not SO_PATH.exists() or not STAMP_PATH.exists():
        return False
    try:
        return json.loads(STAMP_PATH.read_text()).get("hash") == source_hash()
    except Exception:
        return False


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout)
    return r.stdout


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile (if needed) and return the path of the shared object."""
    if not force and is_current():
        return SO_PATH
    import torch.utils.cpp_extension as ce

    cuda_home = _cuda_home()
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    cxx = os.environ.get("CXX", "g++")
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    cu, cpp, headers = _sources()
    header_hash = _hash(headers)
    torch_inc = ce.include_paths()
    py_inc = sysconfig.get_paths()["include"]
    inc_cuda = ["-I" + os.path.join(cuda_home, "include")]
    inc_all = ["-I" + p for p in torch_inc] + ["-I" + py_inc] + inc_cuda

    obj_stamp_path = BUILD_DIR / "objects.json"
    obj_stamps = {}
    if obj_stamp_path.exists():
        try:
            obj_stamps = json.loads(obj_stamp_path.read_text())
        except Exception:
            obj_stamps = {}

    jobs = []
    objects = []
    for src in cu:
        obj = BUILD_DIR / (src.stem + ".cu.o")
        objects.append(obj)
        key = _hash([src], header_hash + " ".join(NVCC_FLAGS))
        if force or not obj.exists() or obj_stamps.get(obj.name) != key:
            jobs.append((obj, key, [nvcc, *NVCC_FLAGS, *inc_cuda, "-c", str(src), "-o", str(obj)]))
    for src in cpp:
        obj = BUILD_DIR / (src.stem + ".cpp.o")
        objects.append(obj)
        key = _hash([src], header_hash + " ".join(CXX_FLAGS))
        if force or not obj.exists() or obj_stamps.get(obj.name) != key:
            flags = list(CXX_FLAGS)
            if src.name == "bindings.cpp":
                flags += ["-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1"]
                incs = inc_all
            else:
                incs = inc_cuda
            jobs.append((obj, key, [cxx, *flags, *incs, "-c", str(src), "-o", str(obj)]))

    def _do(job):
        obj, key, cmd = job
        if verbose:
            print("[build]", " ".join(cmd), flush=True)
        out = _run(cmd)
        if verbose and out.strip():
            print(out)
        return obj.name, key

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        for name, key in ex.map(_do, jobs):
            obj_stamps[name] = key
    obj_stamp_path.write_text(json.dumps(obj_stamps))

    lib_dirs = ce.library_paths() + [os.path.join(cuda_home, "lib64")]
    link = [cxx, "-shared", "-o", str(SO_PATH), *map(str, objects)]
    for d in lib_dirs:
        link += ["-L" + d, "-Wl,-rpath," + d]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    _run(link)
    STAMP_PATH.write_text(json.dumps({"hash": source_hash()}))
    return SO_PATH


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)
