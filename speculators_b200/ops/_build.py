"""In-tree build of the native extension (``speculators_b200/ops/_sb200.so``).

The kernels are plain CUDA translation units (no torch headers, so each compiles
in seconds) built with ``nvcc -gencode arch=compute_100a,code=sm_100a``; only
``bindings.cpp`` sees torch.  Objects and a source hash are kept under
``ops/build/`` so an unchanged tree is not rebuilt, and the shared object sits
next to this file so that a snapshot of the source tree carries it along.
"""

from __future__ import annotations

import hashlib
import os
import re
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
BUILD_CHECKED = HERE / "build_checked"
LIB = HERE / "_sb200.so"
# Debug flavour: same sources with -DSB200_CHECK_BOUNDS (data-dependent row indices are
# validated in the kernels, violations recorded and skipped); selected with
# SB200_CHECKED_BUILD=1, built on demand with build(checked=True).
LIB_CHECKED = HERE / "_sb200_checked.so"
CHECKED = os.environ.get("SB200_CHECKED_BUILD", "0") == "1"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-diag-suppress", "177",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _sources() -> tuple[list[Path], list[Path]]:
    cu = sorted(CSRC.glob("*.cu"))
    cpp = sorted(CSRC.glob("*.cpp"))
    return cu, cpp


def _digest(extra: str = "") -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.glob("*")):
        if p.is_file():
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(extra.encode())
    return h.hexdigest()


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def active_lib() -> Path:
    return LIB_CHECKED if CHECKED else LIB


def is_current(checked: bool | None = None) -> bool:
    import torch

    checked = CHECKED if checked is None else checked
    lib = LIB_CHECKED if checked else LIB
    stamp = (BUILD_CHECKED if checked else BUILD) / "stamp"
    return lib.exists() and stamp.exists() and stamp.read_text() == _digest(torch.__version__ + ("+checked" if checked else ""))


def build(force: bool = False, verbose: bool = False, checked: bool | None = None) -> Path:
    """Compile every kernel for sm_100a and link the extension; returns the .so path."""
    import torch
    from torch.utils import cpp_extension

    checked = CHECKED if checked is None else checked
    if not force and is_current(checked):
        return LIB_CHECKED if checked else LIB
    return _build_into(BUILD_CHECKED if checked else BUILD, LIB_CHECKED if checked else LIB,
                       ["-DSB200_CHECK_BOUNDS"] if checked else [], "+checked" if checked else "", verbose, torch, cpp_extension)


def _build_into(BUILD: Path, LIB: Path, defines: list[str], tag: str, verbose: bool, torch, cpp_extension) -> Path:  # noqa: N803
    BUILD.mkdir(exist_ok=True)
    cu, cpp = _sources()
    nvcc = _nvcc()
    cuda_home = Path(nvcc).resolve().parent.parent
    torch_inc = cpp_extension.include_paths()
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)  # noqa: SLF001

    jobs: list[list[str]] = []
    objs: list[Path] = []
    for src in cu:
        obj = BUILD / (src.stem + ".o")
        objs.append(obj)
        jobs.append([nvcc, *NVCC_FLAGS, *defines, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
    for src in cpp:
        obj = BUILD / (src.stem + ".cpp.o")
        objs.append(obj)
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", *defines, f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
               "-I", str(CSRC), "-I", str(cuda_home / "include")]
        for inc in torch_inc:
            cmd += ["-isystem", inc]
        cmd += ["-c", str(src), "-o", str(obj)]
        jobs.append(cmd)
    if verbose:
        for j in jobs:
            print(" ".join(j), file=sys.stderr)
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        list(pool.map(_run, jobs))

    torch_lib = Path(torch.__file__).parent / "lib"
    link = ["g++", "-shared", "-o", str(LIB), *map(str, objs), f"-L{torch_lib}",
            f"-L{cuda_home / 'lib64'}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-lcudart", f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{cuda_home / 'lib64'}"]
    _run(link)
    (BUILD / "stamp").write_text(_digest(torch.__version__ + tag))
    return LIB


_ENTRY = re.compile(r"Compiling entry function '([^']+)'")
_SPILL = re.compile(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads")
_USED = re.compile(r"Used (\d+) registers")
_SMEM = re.compile(r"(\d+) bytes smem")


def parse_ptxas_info(text: str) -> list[dict]:
    """Rows ``{kernel, registers, smem, stack, spill_stores, spill_loads}`` from the text
    ``nvcc -Xptxas -v`` writes to stderr (one row per entry function)."""
    rows: list[dict] = []
    current: dict | None = None
    for line in text.splitlines():
        if m := _ENTRY.search(line):
            current = {"kernel": m.group(1), "registers": 0, "smem": 0, "stack": 0, "spill_stores": 0, "spill_loads": 0}
            rows.append(current)
        elif current is not None and (m := _SPILL.search(line)):
            current["stack"], current["spill_stores"], current["spill_loads"] = (int(g) for g in m.groups())
        elif current is not None and (m := _USED.search(line)):
            current["registers"] = int(m.group(1))
            if sm := _SMEM.search(line):
                current["smem"] = int(sm.group(1))
    return rows


def _demangle(names: list[str]) -> list[str]:
    try:
        proc = subprocess.run(["c++filt", "-p"], input="\n".join(names), capture_output=True, text=True, check=True)
        out = proc.stdout.splitlines()
        return out if len(out) == len(names) else names
    except (OSError, subprocess.CalledProcessError):
        return names


def resource_usage(only: list[str] | None = None) -> list[dict]:
    """Compile the CUDA sources with ``-Xptxas -v`` into a scratch folder and return registers,
    static shared memory and spills of every kernel (``only``: file stems to restrict to)."""
    scratch = BUILD / "resources"
    scratch.mkdir(parents=True, exist_ok=True)
    cu, _ = _sources()
    nvcc = _nvcc()
    rows: list[dict] = []
    for src in cu:
        if only and src.stem not in only:
            continue
        proc = subprocess.run([nvcc, *NVCC_FLAGS, "-Xptxas", "-v", "-I", str(CSRC), "-c", str(src), "-o", str(scratch / (src.stem + ".o"))],
                              capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}\n{proc.stderr}")
        found = parse_ptxas_info(proc.stderr)
        for row, name in zip(found, _demangle([r["kernel"] for r in found])):
            row["kernel"], row["file"] = name, src.name
        rows.extend(found)
    return rows


if __name__ == "__main__":
    if "--resources" in sys.argv:
        stems = [a for a in sys.argv[1:] if not a.startswith("--")]
        print(f"{'file':<22} {'regs':>4} {'smem':>6} {'stack':>5} {'spill st/ld':>11}  kernel")
        for r in resource_usage(stems or None):
            print(f"{r['file']:<22} {r['registers']:>4} {r['smem']:>6} {r['stack']:>5} {r['spill_stores']:>5}/{r['spill_loads']:<5}  {r['kernel'][:110]}")
    else:
        print(build(force="--force" in sys.argv, verbose=True, checked=True if "--checked" in sys.argv else None))
