"""In-tree build of the native parts (no setuptools, no JIT cache).

Produces, next to this file:

* ``lib/libtgo_mmq.so``  - the C-ABI CUDA library (``include/tgo_mmq.h``), compiled by nvcc for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a``);
* ``_C.abi3.so``         - the libtorch stable-ABI module that registers the
  ``torch_ggml_ops::*`` operators over that C ABI (reference build recipe: setup.py:23-44,
  ``-DTORCH_TARGET_VERSION=0x020A000000000000 -DTORCH_STABLE_ONLY``).

The IQ2_S codebook is not kept in the source tree: it is written to ``build/iq2s_grid.inc`` from
the installed ``gguf`` package (the same table the reference vendors at
csrc/vendor/llama_cpp/iq2_s_grid.cuh:7-263) and its SHA-256 is asserted.

Run as ``python torch_ggml_ops_b200/_build.py`` (a plain script: the package itself cannot be
imported before its native module exists) or load this file and call :func:`build`.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
BUILD = ROOT / "build"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libtgo_mmq.so"
SHIM_PATH = PKG / "_C.abi3.so"

IQ2S_GRID_SHA256 = "e1aa1473412b0552c2174c30ef22ab4073f6a181b85a17056e8249bd2932fd88"
QUANT_TYPES = (11, 12, 13, 14, 22)
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--threads", "2"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _host_cxx() -> str:
    """Host C++ compiler for the stable-ABI module.  The distribution compiler is preferred over
    whatever is first on PATH because it is the one whose shared libstdc++ is installed."""
    if os.environ.get("TGO_CXX"):
        return os.environ["TGO_CXX"]
    return "/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"


def _newer(target: Path, sources) -> bool:
    """True if target exists and is newer than every source."""
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def generate_iq2s_table() -> Path:
    out = BUILD / "iq2s_grid.inc"
    if out.exists():
        return out
    import numpy as np
    from gguf import quants

    quants.IQ2_S.init_grid()
    raw = np.ascontiguousarray(quants.IQ2_S.grid.reshape(1024, 8).astype(np.uint8))
    digest = hashlib.sha256(raw.tobytes()).hexdigest()
    if digest != IQ2S_GRID_SHA256:
        raise RuntimeError(f"IQ2_S codebook hash mismatch: {digest}")
    words = raw.view("<u8").reshape(1024)
    BUILD.mkdir(parents=True, exist_ok=True)
    out.write_text("".join(f"0x{int(w):016x}ULL,\n" for w in words))
    return out


def _run(cmd) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    generate_iq2s_table()
    BUILD.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [ROOT / "include" / "tgo_mmq.h",
                                                                      BUILD / "iq2s_grid.inc"]
    jobs = []
    for qt in QUANT_TYPES:
        jobs.append((CSRC / "mmq_inst.cu", BUILD / f"mmq_inst_{qt}.o", [f"-DTGO_QT={qt}"]))
    for src in sorted(CSRC.glob("*.cu")):
        if src.name != "mmq_inst.cu":
            jobs.append((src, BUILD / (src.stem + ".o"), []))
    todo = [(s, o, f) for (s, o, f) in jobs if force or not _newer(o, [s, *headers])]

    def compile_one(job):
        src, obj, flags = job
        cmd = [_nvcc(), "-ccbin", _host_cxx(), *NVCC_FLAGS, *flags, "-I", str(BUILD), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        _run(cmd)

    if todo:
        with ThreadPoolExecutor(max(1, min(len(todo), (os.cpu_count() or 2) // 2))) as ex:
            list(ex.map(compile_one, todo))
    objs = [o for (_, o, _) in jobs]
    if force or todo or not _newer(LIB_PATH, objs):
        _run([_nvcc(), "-ccbin", _host_cxx(), "-shared", "-cudart", "shared", "-o", str(LIB_PATH), *map(str, objs),
              "-Xlinker", "-rpath,/usr/local/cuda/lib64"])
    return LIB_PATH


def build_shim(force: bool = False) -> Path:
    import torch

    src = CSRC / "torch_shim.cpp"
    if not force and _newer(SHIM_PATH, [src, ROOT / "include" / "tgo_mmq.h", LIB_PATH]):
        return SHIM_PATH
    tdir = Path(torch.__file__).resolve().parent
    inc = [tdir / "include", tdir / "include" / "torch" / "csrc" / "api" / "include",
           Path(sysconfig.get_paths()["include"])]
    cmd = [_host_cxx(), "-O2", "-std=c++17", "-fPIC", "-shared",
           "-DTORCH_TARGET_VERSION=0x020A000000000000", "-DTORCH_STABLE_ONLY", "-DUSE_CUDA", "-DPy_LIMITED_API=0x030A0000",
           *[f"-I{p}" for p in inc], str(src), "-o", str(SHIM_PATH),
           f"-L{LIB_DIR}", "-ltgo_mmq", f"-L{tdir / 'lib'}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10",
           "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{tdir / 'lib'}"]
    _run(cmd)
    # The module must use the process-wide shared libstdc++ (the one libtorch uses): a toolchain
    # that silently links libstdc++.a gives it private iostream state and crashes in operator<<.
    syms = subprocess.run(["nm", "-D", "--defined-only", str(SHIM_PATH)], capture_output=True, text=True).stdout
    if "_ZNSo9_M_insertIlEERSoT_" in syms:
        raise RuntimeError("the stable-ABI module was linked against a static libstdc++; set TGO_CXX to a g++ "
                           "whose libstdc++.so is installed")
    return SHIM_PATH


def build(force: bool = False, verbose: bool = False) -> None:
    build_library(force=force, verbose=verbose)
    build_shim(force=force)


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB_PATH)
    print(SHIM_PATH)
