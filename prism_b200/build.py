"""In-tree build of libprism_b200.so (sm_100a) with nvcc.

    python -m prism_b200.build [--force] [--verbose]

The library is written next to this file so that it travels with the source
tree; nothing is installed into site-packages and nothing is cached elsewhere.
nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libprism_b200.so"
SOURCES = ["api.cu", "scan.cu", "sgemm.cu", "gemm_bf16.cu", "host_plan.cu", "peer_gather.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-cudart", "static",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libprism_b200.so cannot be built")
    return exe


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


STAMP_PATH = PKG_DIR / "libprism_b200.stamp"


def _source_digest() -> str:
    """Hash of everything the library is compiled from (contents, not time stamps: a copied tree keeps
    its contents but not necessarily the order of its modification times)."""
    import hashlib
    h = hashlib.sha256()
    deps = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "prism_b200.h"]
    for d in deps:
        if d.exists():
            h.update(d.name.encode())
            h.update(d.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def stale() -> bool:
    """True if the library is missing or was built from other sources than the ones in the tree."""
    if not LIB_PATH.exists() or not STAMP_PATH.exists():
        return True
    return STAMP_PATH.read_text().strip() != _source_digest()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel source into one shared library; returns its path."""
    if not force and not stale():
        return LIB_PATH
    objdir = PKG_DIR / "build"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stdout.write(out)
        if p.returncode != 0:
            failed = True
            print(f"nvcc failed on {src.name}", file=sys.stderr)
    if failed:
        raise RuntimeError("libprism_b200.so: compilation failed")
    tmp = LIB_PATH.with_suffix(".so.tmp")
    link = [nvcc, *NVCC_FLAGS, "-shared", *objs, "-o", str(tmp)]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stdout.write(r.stdout)
        raise RuntimeError("libprism_b200.so: link failed")
    os.replace(tmp, LIB_PATH)
    STAMP_PATH.write_text(_source_digest() + "\n")
    return LIB_PATH


def build_evals() -> Path:
    """Compile the evaluation programs under prism_b200/evals (needs the library built)."""
    evals = PKG_DIR / "evals"
    r = subprocess.run(["make", "-C", str(evals), f"NVCC={_nvcc()}"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                       text=True)
    if r.returncode != 0:
        sys.stdout.write(r.stdout)
        raise RuntimeError("prism_b200/evals: build failed")
    return evals / "build"


def build_generated_tile_gemm(force: bool = False) -> Path:
    """Compile the kernel that the Prism generator emitted for sm_100a (prism_b200/codegen/generated/tile_gemm.cu)
    into a shared library of its own beside the source; it is an example of the code-generation target, not part
    of libprism_b200.so."""
    src = PKG_DIR / "codegen" / "generated" / "tile_gemm.cu"
    out = src.with_name("libtile_gemm.so")
    if not force and out.exists() and out.stat().st_mtime >= src.stat().st_mtime:
        return out
    tmp = out.with_suffix(".so.tmp")
    cmd = [_nvcc(), *NVCC_FLAGS, "-diag-suppress", "177", "-shared", str(src), "-o", str(tmp)]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stdout.write(r.stdout)
        raise RuntimeError("codegen/generated/tile_gemm.cu: compilation failed")
    os.replace(tmp, out)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build_library(force=a.force, verbose=a.verbose))
