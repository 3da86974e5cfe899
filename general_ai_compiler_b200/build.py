"""Build recipe for ``libgacb.so`` (nvcc, sm_100a only).

``python -m general_ai_compiler_b200.build`` compiles every ``csrc/*.cu`` into
one shared library next to this file.  The library links the CUDA runtime
statically and exports only the ``extern "C"`` entry points declared in
``include/gacb.h``.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libgacb.so"
OBJ_DIR = PKG_DIR / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("GACB_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set GACB_NVCC")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    stamp = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "gacb.h"]
    return any(p.stat().st_mtime > stamp for p in deps)


def build_native(force: bool = False, verbose: bool = False, ptxas_info: bool = False,
                 extra_flags: tuple = (), output: Path | None = None) -> Path:
    """Compile and link; returns the library path.  Raises on any compiler error.

    ``extra_flags`` (e.g. ``("-DGACB_MSDA_UNROLL=2",)``) and ``output`` build a tuning variant elsewhere."""
    if extra_flags or output is not None:
        return _build_variant(tuple(extra_flags), Path(output) if output else LIB_PATH, verbose)
    if not force and not needs_build():
        return LIB_PATH
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "gacb.h"]
    newest_header = max(p.stat().st_mtime for p in headers)
    objs = []
    procs = []
    for src in sources():
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, newest_header):
            continue
        cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if ptxas_info else []), "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
        if verbose or ptxas_info:
            print(out, end="")
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC"]
    if verbose:
        print(" ".join(link), flush=True)
    subprocess.run(link, check=True)
    return LIB_PATH


def _build_variant(extra_flags: tuple, output: Path, verbose: bool) -> Path:
    nvcc = _nvcc()
    cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-shared", "-o", str(output), *map(str, sources())]
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{proc.stdout}")
    return output


# Test builds of the same sources, kept beside the library (git-ignored, they travel with the tree):
#   libgacb_checked.so      every kernel index range-checked (gacb_checked_violations)
#   libgacb_faultinject.so  short bounded-wait limit and a flag that makes the DCNv2 weight loader skip its copies,
#                           so that a wait runs out and the kernel leaves through its abort path
VARIANTS = {
    "libgacb_checked.so": ("-DGACB_CHECKED=1",),
    "libgacb_faultinject.so": ("-DGACB_DCN_FAULT_INJECT=1", "-DGACB_DCN_SPIN_LIMIT=4096"),
}


def build_variants(force: bool = False, verbose: bool = False) -> list[Path]:
    """Build the test variants whose file is missing or older than a source; returns their paths."""
    from concurrent.futures import ThreadPoolExecutor

    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "gacb.h"]
    newest = max(p.stat().st_mtime for p in deps)
    todo = [(name, flags) for name, flags in VARIANTS.items()
            if force or not (PKG_DIR / name).exists() or (PKG_DIR / name).stat().st_mtime < newest]
    with ThreadPoolExecutor(max_workers=max(1, len(todo))) as pool:
        list(pool.map(lambda nf: _build_variant(nf[1], PKG_DIR / nf[0], verbose), todo))
    return [PKG_DIR / name for name in VARIANTS]


RUNNER_SRC = CSRC / "runner" / "gacb_run.cpp"
RUNNER_PATH = PKG_DIR / "gacb-run"


def build_runner(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``gacb-run`` (the plan.json runner in C++) against the library; it finds ``libgacb.so`` next to itself."""
    build_native()
    deps = [RUNNER_SRC, CSRC / "runner" / "json_lite.h", PKG_DIR.parent / "include" / "gacb.h", LIB_PATH]
    if not force and RUNNER_PATH.exists() and all(p.stat().st_mtime <= RUNNER_PATH.stat().st_mtime for p in deps):
        return RUNNER_PATH
    cmd = [_nvcc(), "-O2", "-std=c++17", f"-I{PKG_DIR.parent / 'include'}", f"-I{CSRC / 'runner'}", str(RUNNER_SRC), "-o",
           str(RUNNER_PATH), f"-L{PKG_DIR}", "-l:libgacb.so", "-Xlinker", "-rpath=$ORIGIN"]
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {RUNNER_SRC.name}:\n{proc.stdout}")
    return RUNNER_PATH


if __name__ == "__main__":
    path = build_native(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas-info" in sys.argv)
    print(path)
    print(build_runner(force="--force" in sys.argv, verbose=True))
