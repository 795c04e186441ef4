#!/usr/bin/env python3
"""Build the CPU checker: TEST INFRASTRUCTURE ONLY, never part of the shipped library.

Two artefacts, both git-ignored:

  oracle/libtq_oracle.so       the C restatement in tq_oracle.c (always built)
  oracle/_ref/libtq_ref.so     the upstream project's own C++ core
                               (csrc/core/turboquant_core.cpp, compiled from where it lies in an
                               upstream checkout, never copied) behind the C shim ref_shim.cpp.
  oracle/_ref/libtq_ref_cpu.so the upstream project's own CPU kernels (csrc/cpu/quant_cpu.cpp, OpenMP,
                               compiled where it lies against the installed torch headers) behind
                               ref_cpu_shim.cpp: the timed CPU reference of the decode benchmark.
                               Both are built only when an upstream checkout is found (--reference, the
                               TURBOQUANT_REFERENCE environment variable, or a directory `reference` beside
                               this repository); built files are kept and reused.

Usage:  python oracle/build.py [--reference /path/to/turboquant-kv]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _default_reference() -> str:
    """The upstream checkout: $TURBOQUANT_REFERENCE, else a directory `reference` beside this repository."""
    env = os.environ.get("TURBOQUANT_REFERENCE", "")
    if env:
        return env
    sibling = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return sibling if os.path.isdir(os.path.join(sibling, "csrc")) else ""


DEFAULT_REFERENCE = _default_reference()


def _cc(candidates):
    for c in candidates:
        path = c if os.path.isabs(c) else shutil.which(c)
        if path and os.path.exists(path):
            return path
    raise RuntimeError(f"no compiler found among {candidates}")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "tq_oracle.c")
    out = os.path.join(HERE, "libtq_oracle.so")
    if not force and _newer(out, [src]):
        return out
    gcc = _cc(["/usr/bin/gcc", "gcc"])  # the system gcc links -fopenmp; some bundled ones do not
    cmd = [gcc, "-O2", "-std=gnu11", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden",
           "-fno-fast-math", "-ffp-contract=off", "-Wno-stringop-overflow", src, "-o", out, "-lm"]
    subprocess.check_call(cmd)
    return out


def build_ref(reference: str = DEFAULT_REFERENCE, force: bool = False):
    """Compile the upstream C++ core in place.  Returns the path, or None without a checkout."""
    core = os.path.join(reference, "csrc", "core", "turboquant_core.cpp") if reference else ""
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libtq_ref.so")
    if not core or not os.path.exists(core):
        return out if os.path.exists(out) else None
    shim = os.path.join(HERE, "ref_shim.cpp")
    if not force and _newer(out, [shim, core]):
        return out
    os.makedirs(out_dir, exist_ok=True)
    gxx = _cc(["/usr/bin/g++", "g++"])
    cmd = [gxx, "-O3", "-std=c++17", "-fopenmp", "-fPIC", "-shared",
           "-I", os.path.join(reference, "csrc", "core"), core, shim, "-o", out]
    subprocess.check_call(cmd)
    return out


def build_ref_cpu(reference: str = DEFAULT_REFERENCE, force: bool = False):
    """Compile the upstream CPU kernels in place (needs torch's headers).  Returns the path, or None."""
    src = os.path.join(reference, "csrc", "cpu", "quant_cpu.cpp") if reference else ""
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libtq_ref_cpu.so")
    if not src or not os.path.exists(src):
        return out if os.path.exists(out) else None
    shim = os.path.join(HERE, "ref_cpu_shim.cpp")
    if not force and _newer(out, [shim, src]):
        return out
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    os.makedirs(out_dir, exist_ok=True)
    gxx = _cc(["/usr/bin/g++", "g++"])
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [gxx, "-O3", "-std=c++17", "-fopenmp", "-fPIC", "-shared", "-w",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in cpp_extension.include_paths() + [sysconfig.get_paths()["include"]]:
        cmd += ["-isystem", inc]
    cmd += [src, shim, "-o", out, f"-L{libdir}", "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{libdir}"]
    subprocess.check_call(cmd)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    print("oracle:", build_oracle(args.force))
    ref = build_ref(args.reference, args.force)
    print("upstream core:", ref if ref else "no upstream checkout, skipped")
    cpu = build_ref_cpu(args.reference, args.force)
    print("upstream CPU kernels:", cpu if cpu else "no upstream checkout, skipped")


if __name__ == "__main__":
    sys.exit(main())
