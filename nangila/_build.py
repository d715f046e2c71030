"""In-tree build of the native parts of nangila.

Three artefacts, all written next to the Python sources so that an importing process finds them
without an install step:

* ``nangila/_C*.so``        host-side core (C++17 + pybind11, no CUDA, no torch);
* ``nangila/libnangila_kernels.so``  the sm_100a kernels with plain C launchers (nvcc only);
* ``nangila/_cuda*.so``     torch glue: tensor-typed wrappers of the launchers and the C++ DDP
  communication hook (g++ against libtorch).

Plus two small executables, ``nangila/cli/nangila-dump`` and ``nangila/cli/nangila-profile``, and the
circuit simulator's module and solver process (``nangila_spice/_native*.so``, ``nangila_spice/bin/nangila-node``).

The role of the reference's ``nangila-cuda/build.rs:15-156`` (find CUDA, compile every kernel for a
list of architectures, archive and link) is played by :func:`build_kernels`; the only architecture
is ``sm_100a``.

Run ``python -m nangila._build`` to build everything; ``--core`` / ``--kernels`` / ``--glue`` /
``--cli`` select parts. A part is rebuilt only when one of its sources is newer than its output.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "nangila"
CSRC = ROOT / "csrc"
OBJ = ROOT / "build"
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"

GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _cuda_home() -> str:
    for key in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(key):
            return os.environ[key]
    nvcc = shutil.which("nvcc")
    if nvcc:
        return str(Path(nvcc).resolve().parent.parent)
    return "/usr/local/cuda"


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build command failed:\n  " + " ".join(cmd) + "\n" + proc.stdout)
    if os.environ.get("NANGILA_BUILD_VERBOSE") and proc.stdout.strip():
        print(proc.stdout)


def _stale(out: Path, sources: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources if s.exists())


def _headers(*dirs: Path) -> list[Path]:
    out: list[Path] = []
    for d in dirs:
        out += list(d.glob("**/*.hpp")) + list(d.glob("**/*.cuh")) + list(d.glob("**/*.h"))
    return out


def core_path() -> Path:
    return PKG / f"_C{EXT_SUFFIX}"


def kernels_path() -> Path:
    return PKG / "libnangila_kernels.so"


def glue_path() -> Path:
    return PKG / f"_cuda{EXT_SUFFIX}"


def build_core(force: bool = False) -> Path:
    import pybind11

    out = core_path()
    srcs = [CSRC / "core" / "bindings.cpp", CSRC / "core" / "c_api.cpp"]
    srcs = [s for s in srcs if s.exists()]
    if not force and not _stale(out, srcs + _headers(CSRC / "core")):
        return out
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall",
           "-Wno-unused-function",
           f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
           f"-I{CSRC / 'core'}", *map(str, srcs), "-o", str(out)]
    _run(cmd)
    return out


def kernel_sources() -> list[Path]:
    return sorted((CSRC / "kernels").glob("*.cu"))


def build_kernels(force: bool = False, verbose_ptxas: bool = False) -> Path:
    out = kernels_path()
    srcs = kernel_sources()
    if not srcs:
        raise RuntimeError("no kernel sources found")
    hdrs = _headers(CSRC / "kernels", CSRC / "comm")
    if not force and not _stale(out, srcs + hdrs):
        return out
    nvcc = str(Path(_cuda_home()) / "bin" / "nvcc")
    OBJ.mkdir(exist_ok=True)
    flags = [*GENCODE, "-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
             "-Xcompiler", "-fvisibility=default", f"-I{CSRC / 'kernels'}", f"-I{CSRC / 'comm'}", f"-I{CSRC}"]
    if verbose_ptxas:
        flags += ["-Xptxas", "-v"]
    objs = []
    jobs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append([nvcc, *flags, "-c", str(s), "-o", str(o)])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(_run, jobs))
    _run([nvcc, *GENCODE, "-shared", "-Xcompiler", "-fPIC", *map(str, objs), "-o", str(out), "-lcudart", "-lcuda"])
    return out


def build_glue(force: bool = False) -> Path:
    import pybind11  # noqa: F401  (torch ships its own copy; ours is only a fallback include)
    import torch
    from torch.utils import cpp_extension as ce

    out = glue_path()
    srcs = sorted((CSRC / "ddp").glob("*.cpp"))
    if not srcs:
        raise RuntimeError("no glue sources found")
    if not force and not _stale(out, srcs + _headers(CSRC / "ddp", CSRC / "kernels", CSRC / "comm")):
        return out
    build_kernels()
    torch_lib = Path(torch.__file__).parent / "lib"
    cuda = _cuda_home()
    incs = [f"-I{p}" for p in ce.include_paths()] + [f"-I{cuda}/include", f"-I{sysconfig.get_paths()['include']}",
                                                    f"-I{CSRC / 'kernels'}", f"-I{CSRC / 'comm'}", f"-I{CSRC}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    OBJ.mkdir(exist_ok=True)
    objs, jobs = [], []
    for s in srcs:
        o = OBJ / ("glue_" + s.stem + ".o")
        objs.append(o)
        if force or _stale(o, [s] + _headers(CSRC / "ddp", CSRC / "kernels", CSRC / "comm")):
            jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", "-Wno-unused-function", "-DTORCH_EXTENSION_NAME=_cuda",
                         "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DUSE_C10D_NCCL",
                         *incs, "-c", str(s), "-o", str(o)])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(_run, jobs))
    _run(["g++", "-shared", "-fPIC", *map(str, objs), "-o", str(out),
          f"-L{torch_lib}", f"-L{cuda}/lib64", f"-L{PKG}", "-lnangila_kernels",
          "-ltorch_python", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-lcudart",
          f"-Wl,-rpath,{torch_lib}", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{cuda}/lib64"])
    return out


def build_cli(force: bool = False) -> list[Path]:
    outs = []
    for name in ("nangila_dump", "nangila_profile"):
        src = CSRC / "cli" / f"{name}.cpp"
        if not src.exists():
            continue
        out = PKG / "cli" / name.replace("_", "-")
        outs.append(out)
        if force or _stale(out, [src] + _headers(CSRC / "core")):
            _run(["g++", "-O2", "-std=c++17", f"-I{CSRC / 'core'}", str(src), "-o", str(out)])
    return outs


SPICE_PKG = ROOT / "nangila_spice"


def spice_native_path() -> Path:
    return SPICE_PKG / f"_native{EXT_SUFFIX}"


def build_spice(force: bool = False) -> list[Path]:
    """The circuit simulator: ``nangila_spice/_native*.so`` (pybind11 module over ``csrc/spice``) and
    the ``nangila_spice/bin/nangila-node`` executable. Host code only; its device kernel
    (``csrc/kernels/spmv_csr.cu``) is part of ``libnangila_kernels.so``."""
    import pybind11

    hdrs = _headers(CSRC / "spice")
    outs = []
    mod = spice_native_path()
    src = CSRC / "spice" / "bindings.cpp"
    if force or _stale(mod, [src] + hdrs):
        _run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall", "-pthread",
              f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC / 'spice'}",
              str(src), "-o", str(mod)])
    outs.append(mod)
    exe = SPICE_PKG / "bin" / "nangila-node"
    exe.parent.mkdir(exist_ok=True)
    src = CSRC / "spice" / "node_main.cpp"
    if force or _stale(exe, [src] + hdrs):
        _run(["g++", "-O2", "-std=c++17", "-Wall", "-pthread", f"-I{CSRC / 'spice'}", str(src), "-o", str(exe), "-ldl"])
    outs.append(exe)
    return outs


def build_all(force: bool = False) -> None:
    build_core(force)
    build_cli(force)
    build_spice(force)
    build_kernels(force)
    build_glue(force)


def main(argv: list[str]) -> int:
    force = "--force" in argv
    parts = [a for a in argv if a in ("--core", "--kernels", "--glue", "--cli", "--spice")]
    if not parts:
        build_all(force)
    else:
        if "--core" in parts:
            build_core(force)
        if "--cli" in parts:
            build_cli(force)
        if "--spice" in parts:
            build_spice(force)
        if "--kernels" in parts:
            build_kernels(force, verbose_ptxas="--ptxas-v" in argv)
        if "--glue" in parts:
            build_glue(force)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
