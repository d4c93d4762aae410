"""In-tree build of the native library ``modular_b200/_C.so``.

Kernel sources (``csrc/kernels/*.cu``) are compiled straight with ``nvcc`` for
``sm_100a`` and know nothing about torch; only ``csrc/bindings.cpp`` sees torch headers.
Objects are cached by content hash under ``_native/build/`` so an unchanged file is never
recompiled; the link step produces one shared object that Python loads by explicit path
(no JIT cache outside the tree is involved).

The role matches the reference's kernel build + compile cache (``warm-cache`` CLI,
max/python/max/engine/_precompiled_mefs.py): turn kernel source into device code once and
reuse it on every start.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
BUILD = Path(__file__).resolve().parent / "build"
TARGET = PKG / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wno-attributes"]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _sources() -> list[Path]:
    out = sorted(CSRC.rglob("*.cu")) + sorted(CSRC.rglob("*.cpp"))
    return out


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))):
        h.update(p.read_bytes())
    return h.hexdigest()


def _torch_paths():
    import torch
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths()
    lib = ce.library_paths()
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return inc, lib, abi


def _compile_one(src: Path, obj: Path, verbose: bool) -> None:
    cuda = _cuda_home()
    if src.suffix == ".cu":
        cmd = [f"{cuda}/bin/nvcc", *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    else:
        inc, _, abi = _torch_paths()
        # every host file uses the pybind11 that ships inside torch, so all translation
        # units agree on one pybind11 ABI
        cmd = ["g++", *CXX_FLAGS, f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C",
               "-DTORCH_API_INCLUDE_EXTENSION_H", "-I", str(CSRC), "-I", f"{cuda}/include",
               "-I", sysconfig.get_paths()["include"]]
        for i in inc:
            cmd += ["-isystem", i]
        cmd += ["-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{r.stdout}\n{r.stderr}")


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile what changed and link ``_C.so``. Returns the path of the library."""
    BUILD.mkdir(parents=True, exist_ok=True)
    hdr = _headers_digest()
    flags_sig = " ".join(NVCC_FLAGS + CXX_FLAGS)
    jobs, objs = [], []
    for src in _sources():
        key = hashlib.sha256(src.read_bytes() + hdr.encode() + flags_sig.encode()).hexdigest()[:16]
        obj = BUILD / f"{src.stem}.{key}.o"
        objs.append(obj)
        if force or not obj.exists():
            for old in BUILD.glob(f"{src.stem}.*.o"):
                old.unlink()
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _compile_one(j[0], j[1], verbose), jobs))
    stamp = BUILD / "link.stamp"
    link_sig = " ".join(o.name for o in objs)
    if jobs or not TARGET.exists() or not stamp.exists() or stamp.read_text() != link_sig:
        _, libdirs, _ = _torch_paths()
        cuda = _cuda_home()
        cmd = ["g++", "-shared", "-o", str(TARGET), *[str(o) for o in objs]]
        for d in libdirs:
            cmd += [f"-L{d}", f"-Wl,-rpath,{d}"]
        cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
                f"-L{cuda}/lib64", f"-Wl,-rpath,{cuda}/lib64", "-lcudart", "-ldl", "-lpthread"]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed\n{r.stdout}\n{r.stderr}")
        stamp.write_text(link_sig)
    return TARGET


def is_stale() -> bool:
    """True when a source changed since the library was linked."""
    if not TARGET.exists():
        return True
    t = TARGET.stat().st_mtime
    return any(p.stat().st_mtime > t for p in CSRC.rglob("*") if p.is_file())


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)
