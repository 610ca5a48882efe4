"""TEST INFRASTRUCTURE: builds the CPU checker.

  python oracle/build.py          # builds oracle/hmoe_oracle.so, and oracle/_ref/cpuband_ref*.so when the reference tree
                                  # is present on this machine

`hmoe_oracle.so` is this repository's own restatement (oracle/hmoe_oracle.cpp). `_ref/cpuband_ref` is the reference's
CPU expert engine compiled from its own source file where it lies (runtime/tier/cpuband.cpp under the reference root):
the source is AArch64 code, so it is compiled for x86-64 against the stand-in `ref_shim/arm_neon.h`, with two textual
substitutions applied to the stream that is piped into the compiler (the AArch64 `yield` hint becomes the x86 pause
builtin, `__fp16` becomes `_Float16`). No reference source is written into this repository; only the binary lands in the
git-ignored `_ref/` folder.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))


def ref_root():
    """Where the reference project's tree lies: HECATE_REFERENCE_ROOT, else a folder named `reference` beside this repository
    (None if neither exists)."""
    for cand in (os.environ.get("HECATE_REFERENCE_ROOT"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isdir(cand):
            return cand
    return None

CXXFLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-mavx2", "-mfma", "-mf16c", "-ffp-contract=off", "-fopenmp"]


def _newer(dst, *srcs):
    return os.path.exists(dst) and all(os.path.getmtime(dst) >= os.path.getmtime(s) for s in srcs)


def build_oracle(force=False):
    src = os.path.join(HERE, "hmoe_oracle.cpp")
    dst = os.path.join(HERE, "hmoe_oracle.so")
    if force or not _newer(dst, src):
        subprocess.check_call(["g++", *CXXFLAGS, src, "-o", dst])
    return dst


# Builds of the reference engine: the same source with three versions of the shim's inner-loop intrinsics (see
# ref_shim/arm_neon.h). The module name carries the variant, so several can be loaded into one process.
REF_VARIANTS = {
    "avx2": ("cpuband_ref", []),
    "vnni": ("cpuband_ref_vnni", ["-DHMOE_SHIM_VNNI", "-mavx512f", "-mavx512vl", "-mavx512vnni"]),
    "scalar": ("cpuband_ref_scalar", ["-DHMOE_SHIM_SCALAR", "-fno-tree-vectorize", "-fno-tree-slp-vectorize"]),
}


def ref_module_path(variant="avx2"):
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(HERE, "_ref", REF_VARIANTS[variant][0] + suffix)


def host_has_vnni():
    try:
        return "avx512_vnni" in open("/proc/cpuinfo").read()
    except OSError:
        return False


def build_ref(force=False, variant="avx2"):
    """Compile the reference CPU engine as a python module (needs the reference tree and torch headers)."""
    root = ref_root()
    src = os.path.join(root, "runtime", "tier", "cpuband.cpp") if root else ""
    dst = ref_module_path(variant)
    if not root or not os.path.exists(src):
        return dst if os.path.exists(dst) else None
    shim = os.path.join(HERE, "ref_shim", "arm_neon.h")
    if not force and _newer(dst, src, shim):
        return dst
    import torch.utils.cpp_extension as ce
    os.makedirs(os.path.dirname(dst), exist_ok=True)
    text = open(src).read()
    text = text.replace('asm volatile("yield")', "__builtin_ia32_pause()").replace("__fp16", "_Float16")
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", f"-I{os.path.join(HERE, 'ref_shim')}"]
    libdir = ce.library_paths()[0]
    name, extra = REF_VARIANTS[variant]
    cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-mavx2", "-mfma", "-mf16c", "-ffp-contract=off", "-pthread", *extra,
           f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1",
           *inc, "-x", "c++", "-", "-o", dst, f"-L{libdir}", f"-Wl,-rpath,{libdir}",
           "-ltorch_python", "-ltorch", "-ltorch_cpu", "-lc10"]
    subprocess.run(cmd, input=text.encode(), check=True)
    return dst


def build_ref_all(force=False):
    return {v: build_ref(force, v) for v in REF_VARIANTS}


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref_all(force="--force" in sys.argv))
