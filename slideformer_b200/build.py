"""In-tree build of libslideformer_b200.so for sm_100a.

    python -m slideformer_b200.build [--force] [--verbose]

The shared library lands next to this file so that it travels with the source tree; it is
never installed into site-packages.  nvcc cross-compiles without a GPU present.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "libslideformer_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    # No fast-math of any kind: the kernels must round like the reference's IEEE CPU code.
    "-fmad=false", "-ftz=false", "-prec-div=true", "-prec-sqrt=true",
    "-Xcompiler", "-fPIC,-O2,-Wall,-fno-fast-math,-ffp-contract=off",
    "-shared", "-cudart", "static",
]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = sources() + list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h")) + [Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    nvcc = [nvcc_path()]
    # The host compiler must be the system g++; an exported CXX may point elsewhere.
    if Path("/usr/bin/g++").exists():
        nvcc += ["-ccbin", "/usr/bin/g++"]
    flags = [f for f in NVCC_FLAGS if f not in ("-shared",)]
    common = [*flags, f"-I{ROOT / 'include'}", f"-I{CSRC}"] + (["-Xptxas", "-v"] if verbose else [])
    env = dict(os.environ)
    obj_dir = Path(tempfile.mkdtemp(prefix="sf_b200_obj_"))
    # one nvcc process per translation unit, side by side
    jobs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        cmd = [*nvcc, *common, "-c", str(src), "-o", str(obj)]
        jobs.append((cmd, obj, subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = ""
    for cmd, obj, proc in jobs:
        out, _ = proc.communicate()
        log += out
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + out)
    link = [*nvcc, *flags, "-shared", *[str(o) for _, o, _ in jobs], "-o", str(LIB)]
    res = subprocess.run(link, env=env, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + " ".join(link) + "\n" + res.stdout + res.stderr)
    shutil.rmtree(obj_dir, ignore_errors=True)
    if verbose:
        print(log + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
