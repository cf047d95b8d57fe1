"""Compile libflare_attn.so (sm_100a) in-tree with nvcc.

    python -m flarellm_b200.build [--force] [-v]

One object per .cu file, linked into flarellm_b200/libflare_attn.so.  The CUDA runtime is
linked statically, so the library has no dependency beyond the driver.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
SO = os.path.join(HERE, "libflare_attn.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, flags=(), suffix: str = "") -> str:
    """flags / suffix: a variant of the library (extra nvcc flags, e.g. -DFLARE_DEBUG_BOUNDS) built beside the
    product as libflare_attn<suffix>.so from its own object directory."""
    OBJ = os.path.join(HERE, "build" + suffix)
    SO = os.path.join(HERE, "libflare_attn" + suffix + ".so")
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hpp"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "flare_attn.h"))
    jobs = []
    objs = []
    for src in sources():
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [NVCC, *ARCH, *CFLAGS, *flags, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed for " + cmd[-3])

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(run, jobs))
    if jobs or force or _stale(SO, objs):
        run([NVCC, *ARCH, "-shared", "-o", SO, *objs, "-cudart", "static"])
    return SO


if __name__ == "__main__":
    # python -m flarellm_b200.build [--force] [-v] [--variant SUFFIX -DFLAG ...]
    argv = sys.argv[1:]
    suffix = argv[argv.index("--variant") + 1] if "--variant" in argv else ""
    print(build(force="--force" in argv, verbose="-v" in argv, flags=[a for a in argv if a.startswith("-D")], suffix=suffix))
