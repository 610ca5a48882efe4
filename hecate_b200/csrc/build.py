"""Builds libhecate_moe_b200.so in-tree with nvcc for sm_100a (no torch headers, links cudart only).

    python -m hecate_b200.csrc.build [--force] [--verbose]
    python -m hecate_b200.csrc.build --probe-waits      # diagnostic build libhecate_moe_b200_probe.so: the prefill GEMMs count the cycles
                                                        # every role spends in its waits, and the decode chain's kernels stamp the global
                                                        # timer at a few points (select it with HECATE_MOE_LIB; bench.py reports both)
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libhecate_moe_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--shared",
         "-cudart", "shared"]


def sources():
    return sorted(glob.glob(os.path.join(HERE, "*.cu")))


def build(force=False, verbose=False, defines=(), lib=None, obj_suffix=".o"):
    LIB = lib or globals()["LIB"]
    deps = sources() + glob.glob(os.path.join(HERE, "*.cuh")) + glob.glob(os.path.join(HERE, "*.h")) + \
        [os.path.join(HERE, "..", "..", "include", "hecate_moe.h")]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(d) for d in deps):
        return LIB
    objs = []
    procs = []
    for src in sources():
        obj = src[:-3] + obj_suffix
        cmd = [NVCC, *[f for f in FLAGS if f != "--shared"], *defines, "-c", src, "-o", obj] + (["-Xptxas", "-v"] if verbose else [])
        procs.append((subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT), src))
        objs.append(obj)
    bad = False
    for p, src in procs:
        out = p.communicate()[0].decode()
        if p.returncode != 0 or verbose:
            print(f"--- {os.path.basename(src)}\n{out}")
        bad |= p.returncode != 0
    if bad:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([NVCC, "--shared", "-cudart", "shared", "-o", LIB, *objs, "-lcuda"])
    return LIB


if __name__ == "__main__":
    if "--probe-waits" in sys.argv:
        print(build(force=True, verbose="--verbose" in sys.argv, defines=["-DHMOE_PROBE_WAITS", "-DHMOE_PROBE_TIMELINE"],
                    lib=os.path.join(HERE, "libhecate_moe_b200_probe.so"), obj_suffix=".probe.o"))
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
