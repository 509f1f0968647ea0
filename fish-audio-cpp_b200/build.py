"""Builds libw8a8.so in-tree with nvcc for sm_100a.

Every .cu under csrc/ is compiled to an object in _build/ (only when it or a header is
newer than the object) and linked into lib/libw8a8.so. No JIT cache is involved, so the
built library travels with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "_build"
LIB = HERE / "lib" / "libw8a8.so"
INCLUDE = HERE.parent / "include"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr", "-DW8A8_BUILDING"]


def nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC")
    return cand


def _newest_header() -> float:
    hs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False, defines=(), out_dir=None) -> Path:
    """defines / out_dir: a diagnostic build with extra -D flags goes to a directory of its own
    (out_dir/_build, out_dir/libw8a8.so) and leaves the product library alone."""
    OBJ = globals()["OBJ"] if out_dir is None else Path(out_dir) / "_build"
    LIB = globals()["LIB"] if out_dir is None else Path(out_dir) / "libw8a8.so"
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    hdr = _newest_header()
    defines = [f"-D{d}" for d in defines]
    jobs = []
    for src in sources():
        obj = OBJ / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr)
        if stale:
            cmd = [nvcc(), *ARCH, *NVCC_FLAGS, *defines, "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(run, jobs):
            if verbose or r.returncode != 0 or ptxas_info:
                sys.stderr.write(f"[nvcc] {src.name}\n{r.stdout}{r.stderr}")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [str(OBJ / (s.stem + ".o")) for s in sources()]
    if jobs or not LIB.exists():
        cmd = [nvcc(), *ARCH, "-shared", "-o", str(LIB), *objs, "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    # python build.py [-v] [-f] [--ptxas] [--define NAME[=VALUE]]... [--out DIR]
    #   --define W8A8_TRACE --out DIR   the diagnostic build whose kernels record a device-side timeline
    #                                   (bench.py --trace reads it; point W8A8_LIBRARY at DIR/libw8a8.so)
    argv = sys.argv[1:]
    defs, out = [], None
    i = 0
    while i < len(argv):
        if argv[i] == "--define" and i + 1 < len(argv):
            defs.append(argv[i + 1]); i += 2
        elif argv[i] == "--out" and i + 1 < len(argv):
            out = argv[i + 1]; i += 2
        else:
            i += 1
    print(build(verbose="-v" in argv, force="-f" in argv, ptxas_info="--ptxas" in argv, defines=defs, out_dir=out))
