"""In-tree native build: every CUDA source is compiled for sm_100a with nvcc and linked into
``mstar_b200/lib/libmstar_kernels.so``; the C++ host runtime (control mesh, shared-memory arena, HTTP
frontend) is compiled with g++ into ``mstar_b200/lib/libmstar_runtime.so`` and ``mstar_b200/lib/mstar-server``.

The libraries expose a plain C ABI and are loaded with ctypes, so no Python headers are needed and a
source file compiles in seconds. Run ``python -m mstar_b200.build`` (add ``--force`` to rebuild all).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha1()
    h.update(extra.encode())
    h.update(path.read_bytes())
    # headers are few and small: fold all of them in so that a header edit rebuilds every object
    for hdr in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.inc")) +
                      list((CSRC / "runtime").glob("*.h"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile(cmd: list[str], src: Path, obj: Path, force: bool, verbose: bool) -> bool:
    stamp = obj.with_suffix(obj.suffix + ".sha1")
    dig = _digest(src, " ".join(cmd))
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return False
    full = cmd + ["-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(full), flush=True)
    res = subprocess.run(full, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {src.name}\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr.strip():
        print(res.stderr, flush=True)
    stamp.write_text(dig)
    return True


def kernel_sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def runtime_sources() -> list[Path]:
    return sorted(p for p in (CSRC / "runtime").glob("*.cpp") if p.name != "http_frontend_main.cpp")


def build_kernels(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    out = LIB / "libmstar_kernels.so"
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
    srcs = kernel_sources()
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as ex:
        changed = list(ex.map(lambda so: _compile([_nvcc()] + flags + ["-I", str(CSRC)], so[0], so[1], force,
                                                  verbose or ptxas_info), zip(srcs, objs)))
    if any(changed) or not out.exists():
        cmd = [_nvcc(), "-shared", "-o", str(out)] + [str(o) for o in objs] + ["-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed\n{res.stdout}\n{res.stderr}")
    return out


def build_runtime(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    out = LIB / "libmstar_runtime.so"
    srcs = runtime_sources()
    if not srcs:
        return out
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    objs = [OBJ / ("rt_" + s.stem + ".o") for s in srcs]
    with ThreadPoolExecutor(max_workers=8) as ex:
        changed = list(ex.map(lambda so: _compile([cxx] + CXX_FLAGS + ["-I", str(CSRC / "runtime")], so[0], so[1],
                                                  force, verbose), zip(srcs, objs)))
    if any(changed) or not out.exists():
        cmd = [cxx, "-shared", "-o", str(out)] + [str(o) for o in objs] + ["-pthread", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed\n{res.stdout}\n{res.stderr}")
    main = CSRC / "runtime" / "http_frontend_main.cpp"
    exe = LIB / "mstar-server"
    if main.exists():
        mobj = OBJ / "rt_http_frontend_main.o"
        ch = _compile([cxx] + CXX_FLAGS + ["-I", str(CSRC / "runtime")], main, mobj, force, verbose)
        if ch or any(changed) or not exe.exists():
            cmd = [cxx, "-o", str(exe), str(mobj)] + [str(o) for o in objs] + ["-pthread", "-lrt"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"link failed\n{res.stdout}\n{res.stderr}")
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_runtime(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv or "--ptxas" in sys.argv)
    if "--ptxas" in sys.argv:
        build_kernels(force=True, ptxas_info=True)
    print("built:", *(p.name for p in LIB.glob("*.so")))
