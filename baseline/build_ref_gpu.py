"""BASELINE INFRASTRUCTURE: builds the reference's own GPU kernels of the MoE expert path, unchanged, for sm_100a.

    python baseline/build_ref_gpu.py [--force] [moe4 moe4t router ...]

What is built (python extension modules, written only into the git-ignored folder baseline/_ref/):
  moe4    runtime/tier/moe4/moe4.cu     decode kernels (<= 8 rows) + combine + dequant       (tier_split.py:65-66)
  moe4t   runtime/tier/moe4/moe4t.cu    tcgen05 prefill kernels                              (tier_split.py:74-76)
  cn      runtime/tier/cn.cu            combine fused into the next input norm               (tier_split.py:79-81)
  router  the CUDA source text embedded in runtime/core/exl3_router.py (`_K_SRC`), compiled the way its own
          `load_inline` call does (runtime/core/exl3_router.py:153-160)
The sources are compiled where they lie under the reference root (HECATE_REFERENCE_ROOT, or a folder `reference` beside
this repository); the router's source string is
piped to a temporary file outside this repository. Flags are the reference's own (-O3 --use_fast_math plus the flags
torch.utils.cpp_extension.load adds to every CUDA extension), with its arch (compute_103a, the GB300) replaced by
arch=compute_100a,code=sm_100a (B200). No reference source is copied into this repository.

The modules are baselines and second parity references for tests and bench.py; nothing under hecate_b200/ loads them.
"""
import os
import subprocess
import sys
import sysconfig
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"

CUDA_SOURCES = {
    "moe4": ("runtime", "tier", "moe4", "moe4.cu"),
    "moe4t": ("runtime", "tier", "moe4", "moe4t.cu"),
    "cn": ("runtime", "tier", "cn.cu"),
}
ROUTER_PY = ("runtime", "core", "exl3_router.py")
ROUTER_DECL = ("void router_fused(at::Tensor x, at::Tensor wt, c10::optional<at::Tensor> bias, at::Tensor logits, at::Tensor ctr, "
               "at::Tensor sel, at::Tensor rw, int64_t topk, double scale);")


def ref_root():
    """HECATE_REFERENCE_ROOT, else a folder named `reference` beside this repository ("" if neither exists)."""
    for cand in (os.environ.get("HECATE_REFERENCE_ROOT"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isdir(cand):
            return cand
    return ""


def module_path(name):
    return os.path.join(OUT, name + SUFFIX)


def _cmd(name, src):
    import torch.utils.cpp_extension as ce
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    libdir = ce.library_paths("cuda")[0]
    return [NVCC, "-O3", "-gencode=arch=compute_100a,code=sm_100a", "--use_fast_math", "-std=c++17", *ce.COMMON_NVCC_FLAGS,
            "--shared", "-Xcompiler", "-fPIC", f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-D_GLIBCXX_USE_CXX11_ABI=1", *inc, src, "-o", module_path(name), f"-L{libdir}", "-Xlinker", f"-rpath={libdir}",
            "-ltorch_python", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-lcudart"]


def _router_source(root):
    """The CUDA text the reference hands to load_inline, plus the binding load_inline generates for `functions=[...]`."""
    text = open(os.path.join(root, *ROUTER_PY)).read()
    start = text.index('_K_SRC = r"""') + len('_K_SRC = r"""')
    body = text[start:text.index('"""', start)]
    return ("#include <torch/extension.h>\n" + body + "\n" + ROUTER_DECL +
            "\nPYBIND11_MODULE(TORCH_EXTENSION_NAME, m) { m.def(\"router_fused\", &router_fused, \"router_fused\"); }\n")


def build(names=None, force=False, verbose=True):
    """Builds the named modules (default: all) in parallel. Returns {name: path or None}."""
    root = ref_root()
    names = list(names or [*CUDA_SOURCES, "router"])
    out = {n: (module_path(n) if os.path.exists(module_path(n)) else None) for n in names}
    if not root or not os.path.isdir(root):
        return out                                           # no reference tree on this machine: use what was built before
    os.makedirs(OUT, exist_ok=True)
    procs, tmp = [], None
    for n in names:
        if n == "router":
            src_time = os.path.getmtime(os.path.join(root, *ROUTER_PY))
        else:
            src_time = os.path.getmtime(os.path.join(root, *CUDA_SOURCES[n]))
        if not force and out[n] and os.path.getmtime(out[n]) >= src_time:
            continue
        if n == "router":
            tmp = tempfile.TemporaryDirectory()
            src = os.path.join(tmp.name, "exl3_router_fused4.cu")
            open(src, "w").write(_router_source(root))
        else:
            src = os.path.join(root, *CUDA_SOURCES[n])
        procs.append((n, subprocess.Popen(_cmd(n, src), stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    for n, p in procs:
        log = p.communicate()[0].decode()
        if p.returncode != 0:
            print(f"--- {n}: nvcc failed\n{log[-4000:]}")
            out[n] = None
        else:
            out[n] = module_path(n)
            if verbose:
                print(f"built {out[n]}")
    if tmp is not None:
        tmp.cleanup()
    return out


def load(name):
    """Imports a built module (torch must be imported first: the modules link against it). None if it is not built."""
    p = module_path(name)
    if not os.path.exists(p):
        return None
    import importlib.util
    import torch  # noqa: F401
    spec = importlib.util.spec_from_file_location(name, p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(args or None, force="--force" in sys.argv))
