"""In-tree build of every native part.

Three products, all placed inside the package directory so that they travel
with a copy of the source tree:

* ``_ctl*.so``    control plane bindings (g++, pybind11; no CUDA, no torch)
* ``bin/fabricd`` and the other host executables (g++)
* ``_C*.so``      the sm_100a kernels and their torch bindings (nvcc through
                  ``torch.utils.cpp_extension``; compiles without a GPU)

``python -m skygdr_b200.build [ctl|bin|cuda|all]``. Each product is rebuilt only
when one of its sources is newer than it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
CTL = CSRC / "ctl"
KERNELS = CSRC / "kernels"
BIN = PKG / "bin"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _ext_suffix() -> str:
    return sysconfig.get_config_var("EXT_SUFFIX") or ".so"


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, **kw):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, **kw)
    if r.returncode != 0:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + r.stdout)
        raise RuntimeError(f"build step failed: {cmd[0]} (exit {r.returncode})")
    return r.stdout


def ctl_path() -> Path:
    return PKG / ("_ctl" + _ext_suffix())


def build_ctl(force: bool = False) -> Path:
    import pybind11

    out = ctl_path()
    srcs = sorted(CTL.glob("*.hpp")) + sorted(CTL.glob("*.h")) + [CTL / "ctl_py.cc"]
    if force or _newer(out, srcs):
        inc = [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{CTL}"]
        _run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", *inc,
              str(CTL / "ctl_py.cc"), "-o", str(out), "-ldl", "-pthread"])
    return out


HOST_BINARIES = {
    "fabricd": ["fabricd.cc"],
    "cpu_client": ["cpu_client.cc"],
    "gpu_server": ["gpu_server.cc"],
}


def _nvtx_flags() -> list:
    """NVTX v3 is header-only; the control plane's timeline ranges (csrc/ctl/trace.hpp) are compiled in where the CUDA
    toolkit's headers are present and are empty otherwise."""
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "include" / "nvtx3" / "nvToolsExt.h").exists():
            return ["-DSKYGDR_WITH_NVTX", f"-isystem{Path(root) / 'include'}"]
    return []


def build_bin(force: bool = False) -> Path:
    BIN.mkdir(exist_ok=True)
    hdrs = sorted(CTL.glob("*.hpp")) + sorted(CTL.glob("*.h"))
    for name, files in HOST_BINARIES.items():
        srcs = [CTL / f for f in files]
        if not all(s.exists() for s in srcs):
            continue
        out = BIN / name
        if force or _newer(out, srcs + hdrs):
            _run(["g++", "-std=c++17", "-O2", "-Wall", f"-I{CTL}", *_nvtx_flags(), *map(str, srcs), "-o", str(out), "-ldl", "-pthread"])
    return BIN


def build_sanitized(kind: str = "address") -> Path:
    """fabricd with a sanitizer: ``address`` = ASan + UBSan, ``thread`` = TSan. Used by the CPU tests to run a
    daemon session (connections, window timer, lease expiry) under the sanitizer; the reference has no such runs."""
    assert kind in ("address", "thread")
    BIN.mkdir(exist_ok=True)
    out = BIN / f"fabricd_{'asan' if kind == 'address' else 'tsan'}"
    srcs = [CTL / "fabricd.cc"]
    hdrs = sorted(CTL.glob("*.hpp")) + sorted(CTL.glob("*.h"))
    if _newer(out, srcs + hdrs):
        flags = ["-fsanitize=address,undefined", "-fno-omit-frame-pointer"] if kind == "address" else ["-fsanitize=thread"]
        _run(["g++", "-std=c++17", "-O1", "-g", *flags, f"-I{CTL}", str(srcs[0]), "-o", str(out), "-ldl", "-pthread"])
    return out


def cuda_path() -> Path:
    return PKG / ("_C" + _ext_suffix())


def cuda_sources():
    return sorted(KERNELS.glob("*.cu")) + sorted(KERNELS.glob("*.cpp"))


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the kernels for sm_100a. Needs nvcc, not a GPU."""
    out = cuda_path()
    srcs = cuda_sources()
    deps = srcs + sorted(KERNELS.glob("*.cuh")) + sorted(KERNELS.glob("*.h")) + sorted(CTL.glob("*.h"))
    if not force and not _newer(out, deps):
        return out
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    from torch.utils import cpp_extension

    build_dir = PKG / "build" / "_C"
    build_dir.mkdir(parents=True, exist_ok=True)
    cpp_extension.load(
        name="_C",
        sources=[str(s) for s in srcs],
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xptxas", "-v", *NVCC_ARCH,
                           "--expt-relaxed-constexpr"],
        extra_include_paths=[str(KERNELS), str(CTL)],
        build_directory=str(build_dir),
        verbose=verbose,
        is_python_module=False,
    )
    built = build_dir / "_C.so"
    shutil.copy2(built, out)
    return out


def build_all(force: bool = False, verbose: bool = False):
    build_ctl(force)
    build_bin(force)
    build_cuda(force, verbose)


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    force = "--force" in sys.argv
    verbose = "-v" in sys.argv
    if what in ("ctl", "all"):
        print("built", build_ctl(force))
    if what in ("bin", "all"):
        print("built", build_bin(force))
    if what in ("cuda", "all"):
        print("built", build_cuda(force, verbose))
