"""Build the reference's own CPU Adam kernel into oracle/_ref/ (test infrastructure).

The two translation units are compiled where they lie in the reference checkout
(optimizer/layer_adam/csrc/cpu_adam.cpp and cpu_adam_impl.cpp); nothing is copied.  The
flags are the ones the reference's loader passes (optimizer/layer_adam/builder.py:55-82)
with one change: -march=native becomes -march=x86-64-v4, because the resulting module is
built on one machine and run on another.  The vector body is written with explicit
AVX-512 intrinsics and the tail's contraction is decided before instruction selection, so
the results are bit-identical for both -march values (checked by tests/golden/make_golden.py
--check-march when it is run where the reference is mounted).

Output: oracle/_ref/cpu_adam.so, a pybind11 module exporting create_adam / adam_update /
destroy_adam (cpu_adam.cpp:8-13).  It is used to pin the C restatement, to generate the
golden vectors and as the "reference" CPU baseline of the benchmark.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent


def default_reference() -> Path | None:
    """Where the reference checkout is: $SLIDEFORMER_REFERENCE, else a directory named `reference`
    next to this repository; None when neither exists."""
    env = os.environ.get("SLIDEFORMER_REFERENCE")
    if env:
        return Path(env)
    sibling = HERE.parents[1] / "reference"
    return sibling if sibling.is_dir() else None



def ref_sources(reference: Path) -> list[Path]:
    csrc = reference / "optimizer" / "layer_adam" / "csrc"
    return [csrc / "cpu_adam.cpp", csrc / "cpu_adam_impl.cpp"]


def build(reference: Path | None = None, out_dir: Path = HERE / "_ref",
          march: str = "x86-64-v4", force: bool = False, verbose: bool = True) -> Path | None:
    """Compile the reference kernel.  Returns the .so path, or None if the sources are absent."""
    reference = Path(reference) if reference is not None else default_reference()
    srcs = ref_sources(reference) if reference is not None else []
    if not srcs or not all(s.exists() for s in srcs):
        if verbose:
            print("[build_ref] reference sources not found (set SLIDEFORMER_REFERENCE to the checkout); "
                  "keeping any prebuilt module")
        so = out_dir / "cpu_adam.so"
        return so if so.exists() else None
    out_dir.mkdir(parents=True, exist_ok=True)
    so = out_dir / "cpu_adam.so"
    newest_src = max(p.stat().st_mtime for p in list(srcs[0].parent.glob("*.h")) + srcs)
    if so.exists() and not force and so.stat().st_mtime >= newest_src:
        return so

    from torch.utils import cpp_extension as ce
    import torch

    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}",
                                                    f"-I{srcs[0].parent}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cflags = ["-DTORCH_EXTENSION_NAME=cpu_adam", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
              "-DVERSION_GE_1_1", "-DVERSION_GE_1_3", "-DVERSION_GE_1_5", "-D__AVX512__",
              "-O3", "-std=c++17", "-g", "-Wno-reorder", "-fopenmp", f"-march={march}", "-fPIC"]
    objs = []
    t0 = time.time()
    procs = []
    for s in srcs:
        o = out_dir / (s.stem + ".o")
        objs.append(o)
        cmd = ["g++", *cflags, *inc, "-c", str(s), "-o", str(o)]
        procs.append((cmd, subprocess.Popen(cmd)))
    for cmd, p in procs:
        if p.wait() != 0:
            raise RuntimeError("reference compile failed: " + " ".join(cmd))
    libdirs = ce.library_paths()
    link = ["g++", "-shared", *map(str, objs), "-o", str(so), "-fopenmp",
            *[f"-L{d}" for d in libdirs], *[f"-Wl,-rpath,{d}" for d in libdirs],
            "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    subprocess.check_call(link)
    for o in objs:
        o.unlink()
    if verbose:
        print(f"[build_ref] built {so} in {time.time() - t0:.1f}s (march={march})")
    return so


def host_can_run_ref() -> bool:
    """The module needs AVX-512 F/BW/DQ/VL; say so instead of dying on an illegal instruction."""
    try:
        flags = Path("/proc/cpuinfo").read_text()
    except OSError:
        return False
    return all(f" {f}" in flags for f in ("avx512f", "avx512bw", "avx512dq", "avx512vl", "fma"))


def load(out_dir: Path = HERE / "_ref"):
    """Import the prebuilt reference module, or return None when it is absent or unusable here."""
    so = out_dir / "cpu_adam.so"
    if not so.exists() or not host_can_run_ref():
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    spec = importlib.util.spec_from_file_location("cpu_adam", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, default=None,
                    help="reference checkout (default: $SLIDEFORMER_REFERENCE, else ../reference next to this repository)")
    ap.add_argument("--out", type=Path, default=HERE / "_ref")
    ap.add_argument("--march", default="x86-64-v4")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    r = build(a.reference, a.out, a.march, a.force)
    sys.exit(0 if r is not None else 1)
