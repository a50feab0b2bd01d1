"""Builds the checkers under oracle/ -- TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [--reference /path/to/prism]

1. oracle/liboracle_cpu.so     the plain-C restatement (oracle_cpu.c), gcc + OpenMP.
2. oracle/_ref/libref_cpu.so   the reference's own CPU scan loop (scan_harness.cuh) behind a C symbol.
3. oracle/_ref/libprism_ref.so the reference's generated SGEMM and scan kernels with the harness launch
                               geometry, compiled for sm_100 with the reference Makefile's flags
                               (-O3 --use_fast_math -w; evals/4090_sgemm/Makefile:12-18, evals/4090_scan/Makefile:3-4).

4. oracle/_ref/relink_sgemm_sweep  the reference's SGEMM sweep program (evals/4090_sgemm/main.cu), unmodified, linked
                               against libprism_b200.so through relink_sgemm_runner.cu instead of its own runner.cu.

5. oracle/_ref/relink_scan_main  the reference's scan harness program (evals/4090_scan/main.cu and scan_harness.cuh), unmodified,
                               on libprism_b200.so through relink_scan_main.cu.

Steps 2 to 5 compile the reference's sources from where they lie (include path
= the reference root); nothing is copied.  They are skipped when the reference
tree is absent (e.g. on a GPU box, which uses the files built beforehand).
The bf16 kernel is not built: wgmma does not assemble for sm_100.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_OUT = HERE / "_ref"
# Root of a checkout of manya-bansal/prism; set PRISM_REFERENCE to point elsewhere.
DEFAULT_REFERENCE = os.environ.get("PRISM_REFERENCE", str(HERE.parent.parent / "reference"))


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stdout.write(r.stdout)
        raise RuntimeError("command failed: " + " ".join(cmd))


def _newer(target: Path, deps: list[Path]) -> bool:
    return target.exists() and all(target.stat().st_mtime >= d.stat().st_mtime for d in deps if d.exists())


def build_oracle_c(force: bool = False) -> Path:
    out = HERE / "liboracle_cpu.so"
    src = HERE / "oracle_cpu.c"
    if not force and _newer(out, [src]):
        return out
    _run(["gcc", "-O3", "-march=native", "-fopenmp", "-shared", "-fPIC", str(src), "-o", str(out)])
    return out


def build_reference(reference: str = DEFAULT_REFERENCE, force: bool = False) -> dict[str, Path] | None:
    ref = Path(reference)
    if not (ref / "generated" / "scan_kernel.cu").exists():
        return None
    REF_OUT.mkdir(exist_ok=True)
    built = {}
    cpu_out = REF_OUT / "libref_cpu.so"
    cpu_src = HERE / "ref_cpu_shim.cpp"
    if force or not _newer(cpu_out, [cpu_src]):
        cuda_inc = Path(shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc").resolve().parent.parent / "include"
        _run(["g++", "-O2", "-w", "-shared", "-fPIC", f"-I{ref}", f"-I{cuda_inc}", str(cpu_src), "-o", str(cpu_out)])
    built["cpu"] = cpu_out
    gpu_out = REF_OUT / "libprism_ref.so"
    gpu_src = HERE / "ref_shim.cu"
    if force or not _newer(gpu_out, [gpu_src]):
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        _run([nvcc, "-arch=sm_100", "-O3", "--use_fast_math", "-w", "-cudart", "static", "-shared", "-Xcompiler", "-fPIC",
              f"-I{ref}", str(gpu_src), "-o", str(gpu_out)])
    built["gpu"] = gpu_out
    relink = build_relinked_sgemm_sweep(ref, force)
    if relink is not None:
        built["relink_sgemm_sweep"] = relink
    relink = build_relinked_scan_main(ref, force)
    if relink is not None:
        built["relink_scan_main"] = relink
    relink = build_relinked_h100_main(ref, force)
    if relink is not None:
        built["relink_h100_main"] = relink
    return built


def build_relinked_scan_main(ref: Path, force: bool = False) -> Path | None:
    """The reference's own scan harness main and header, compiled in place, on this library's scan."""
    main_cu = ref / "evals" / "4090_scan" / "main.cu"
    lib = HERE.parent / "prism_b200" / "libprism_b200.so"
    if not main_cu.exists() or not lib.exists():
        return None
    out = REF_OUT / "relink_scan_main"
    shim = HERE / "relink_scan_main.cu"
    if force or not _newer(out, [shim, lib]):
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        # flags of evals/4090_scan/Makefile:3-4 with the architecture changed; include path = the reference root
        _run([nvcc, "-arch=sm_100", "-O3", "-w", "-std=c++17", f"-I{ref}", f"-I{HERE.parent / 'include'}", str(shim),
              "-o", str(out), f"-L{lib.parent}", "-lprism_b200", "-Xlinker", "-rpath", "-Xlinker",
              "$ORIGIN/../../prism_b200"])
    return out


def build_relinked_sgemm_sweep(ref: Path, force: bool = False) -> Path | None:
    """The reference's own sweep main, compiled in place, on this library's `run_my_kernel`."""
    main_cu = ref / "evals" / "4090_sgemm" / "main.cu"
    lib = HERE.parent / "prism_b200" / "libprism_b200.so"
    if not main_cu.exists() or not lib.exists():
        return None
    out = REF_OUT / "relink_sgemm_sweep"
    runner = HERE / "relink_sgemm_runner.cu"
    if force or not _newer(out, [runner, lib]):
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        _run([nvcc, "-arch=sm_100", "-O3", "-w", "-std=c++17", f"-I{main_cu.parent}", f"-I{HERE.parent / 'include'}",
              str(main_cu), str(runner), "-o", str(out), "-lcublas", f"-L{lib.parent}", "-lprism_b200",
              "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../prism_b200"])
    return out


def build_relinked_h100_main(ref: Path, force: bool = False) -> Path | None:
    """The reference's own bf16 benchmark main, compiled from where it lies, on this library's `runmyh100`.

    The program includes "utils.cuh" from its own directory, which is where the Hopper-only kernel lives; the
    stand-in (oracle/relink_h100_utils.cuh) therefore goes, under that name, into a directory that holds nothing else
    but a symbolic link to the reference's main.cu: a quoted include is looked up beside the file as it was named."""
    main_cu = ref / "evals" / "h100_bench" / "main.cu"
    lib = HERE.parent / "prism_b200" / "libprism_b200.so"
    if not main_cu.exists() or not lib.exists():
        return None
    out = REF_OUT / "relink_h100_main"
    stand_in = HERE / "relink_h100_utils.cuh"
    if force or not _newer(out, [stand_in, lib]):
        work = REF_OUT / "h100_relink"
        work.mkdir(exist_ok=True)
        link = work / "main.cu"
        if link.is_symlink() or link.exists():
            link.unlink()
        link.symlink_to(main_cu)
        shutil.copyfile(stand_in, work / "utils.cuh")
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        _run([nvcc, "-arch=sm_100", "-O3", "-w", "-std=c++17", f"-I{HERE.parent / 'include'}", str(link), "-o", str(out),
              "-lcublas", "-lcuda", f"-L{lib.parent}", "-lprism_b200", "-Xlinker", "-rpath", "-Xlinker",
              "$ORIGIN/../../prism_b200"])
        shutil.rmtree(work)      # the link points into the reference checkout: nothing to keep, nothing to ship
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle_c(a.force))
    print(build_reference(a.reference, a.force) or "reference tree absent: oracle/_ref not (re)built")
