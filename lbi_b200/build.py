"""Build the CUDA extension in-tree:  python -m lbi_b200.build

Kernels are compiled by nvcc for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``) into object files,
the pybind11 binding is compiled against the installed PyTorch, and everything is linked into
``lbi_b200/_C<abi suffix>.so`` next to the Python sources so that it travels with the tree.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG / "build"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUDA_SOURCES = ["elementwise.cu", "suffix_scan.cu", "interface_jac.cu", "gated_norm.cu", "siso_prep.cu", "mamba_small.cu", "gemm_tcgen05.cu", "attn_pullback.cu", "attn_fwd.cu", "ssd.cu", "peer.cu", "noalloc.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _ext_path(name: str = "_C") -> Path:
    return PKG / f"{name}{sysconfig.get_config_var('EXT_SUFFIX')}"


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if os.environ.get("LBI_B200_BUILD_VERBOSE") and (proc.stdout or proc.stderr):
        print(proc.stdout, proc.stderr, file=sys.stderr)


def build(force: bool = False, verbose_ptxas: bool = False, bounds_check: bool = False) -> Path:
    """``bounds_check``: the debug extension ``lbi_b200/_Cdbg*.so`` compiled with -DLBI_BOUNDS_CHECK (index checks that record a
    site code and skip the access; ``LBI_B200_DEBUG_EXT=1`` makes ``lbi_b200.ops`` load it instead of ``_C``)."""
    import torch
    from torch.utils import cpp_extension

    name = "_Cdbg" if bounds_check else "_C"
    BUILD = PKG / ("build_dbg" if bounds_check else "build")
    extra = ["-DLBI_BOUNDS_CHECK"] if bounds_check else []
    BUILD.mkdir(exist_ok=True)
    sources = [CSRC / s for s in CUDA_SOURCES if (CSRC / s).exists()]
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh"))
    binding = CSRC / "binding.cpp"
    stamp = BUILD / "stamp.txt"
    digest = _digest([*sources, *headers, binding]) + torch.__version__
    out = _ext_path(name)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out

    include_dirs = cpp_extension.include_paths(device_type="cuda")
    inc = [f"-I{d}" for d in include_dirs] + [f"-I{CSRC}", f"-I{sysconfig.get_paths()['include']}"]
    objects: list[Path] = []
    jobs = []
    for src in sources:
        obj = BUILD / (src.stem + ".o")
        objects.append(obj)
        flags = list(NVCC_FLAGS) + extra + (["-Xptxas", "-v"] if verbose_ptxas else [])
        jobs.append([NVCC, *flags, f"-I{CSRC}", "-I/usr/local/cuda/include", "-c", str(src), "-o", str(obj)])
    bind_obj = BUILD / "binding.o"
    objects.append(bind_obj)
    cxx11_abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    jobs.append([
        "g++", "-O2", "-std=c++17", "-fPIC", f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H", *extra,
        f"-D_GLIBCXX_USE_CXX11_ABI={cxx11_abi}", *inc, "-c", str(binding), "-o", str(bind_obj),
    ])
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        list(pool.map(_run, jobs))
    lib_dirs = cpp_extension.library_paths(device_type="cuda")
    link = ["g++", "-shared", *map(str, objects), "-o", str(out)]
    for d in lib_dirs:
        link += [f"-L{d}", f"-Wl,-rpath,{d}"]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    _run(link)
    stamp.write_text(digest)
    return out


def main() -> None:
    """python -m lbi_b200.build [--force] [--ptxas] [--bounds-check]"""
    path = build(force="--force" in sys.argv, verbose_ptxas="--ptxas" in sys.argv, bounds_check="--bounds-check" in sys.argv)
    print(path)


if __name__ == "__main__":
    main()
