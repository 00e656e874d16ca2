"""In-tree build of the native library (``rustorch_b200/_C*.so``) for sm_100a.

Every ``csrc/**/*.cu`` is compiled by nvcc with ``-gencode arch=compute_100a,code=sm_100a``
(kernel translation units are torch-free and compile in seconds), the tensor glue
``csrc/*.cpp`` by g++ against the torch headers, and everything is linked into one Python
extension module that sits next to this file.  Objects are cached under ``build/`` keyed by a
content hash of the source and the headers it can see, so rebuilds only touch what changed.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
BUILD = ROOT / "build" / "obj"
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
TARGET = Path(__file__).resolve().parent / f"_C{EXT_SUFFIX}"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "--threads", "2",
] + os.environ.get("RUSTORCH_NVCC_EXTRA", "").split()          # e.g. "-DRT_ATTN_PROF" for an instrumented build
# RUSTORCH_BOUNDS_CHECK=1: the checked build.  Guarded global accesses compare their index with the extent passed by
# the host and record an error code instead of touching memory outside (csrc/common/ptx.cuh, RT_GUARD);
# ``_C.bounds_check_build()`` tells which build is loaded.
if os.environ.get("RUSTORCH_BOUNDS_CHECK", "0") == "1":
    NVCC_FLAGS.append("-DRT_BOUNDS_CHECK")


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".h", ".cuh", ".hpp"):
            h.update(p.read_bytes())
    return h.hexdigest()


def _obj_for(src: Path, hdr_digest: str, extra: str) -> Path:
    h = hashlib.sha256(src.read_bytes())
    h.update(hdr_digest.encode())
    h.update(extra.encode())
    rel = "_".join(src.relative_to(CSRC).with_suffix("").parts)
    return BUILD / f"{rel}.{h.hexdigest()[:16]}.o"


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n  " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def sources() -> tuple[list[Path], list[Path]]:
    cu = sorted(CSRC.rglob("*.cu"))
    cpp = sorted(CSRC.glob("*.cpp"))
    return cu, cpp


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile what changed and (re)link ``_C``.  Returns the path of the shared object."""
    import torch  # noqa: F401  (headers + libs come from the installed torch)
    from torch.utils import cpp_extension as ce

    BUILD.mkdir(parents=True, exist_ok=True)
    cu, cpp = sources()
    hdr = _headers_digest()
    nvcc = str(Path(_cuda_home()) / "bin" / "nvcc")
    torch_inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    cxx_flags = [
        "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        f"-I{_cuda_home()}/include", "-Wno-deprecated-declarations",
    ]
    jobs: list[tuple[Path, list[str]]] = []
    objs: list[Path] = []
    for s in cu:
        o = _obj_for(s, hdr, " ".join(NVCC_FLAGS))
        objs.append(o)
        if force or not o.exists():
            jobs.append((o, [nvcc, *NVCC_FLAGS, f"-I{CSRC}", "-c", str(s), "-o", str(o)]))
    for s in cpp:
        o = _obj_for(s, hdr, " ".join(cxx_flags) + torch.__version__)
        objs.append(o)
        if force or not o.exists():
            jobs.append((o, ["g++", *cxx_flags, *torch_inc, f"-I{CSRC}", "-c", str(s), "-o", str(o)]))

    def _do(job):
        o, cmd = job
        if verbose:
            print("[build]", " ".join(cmd[-4:]), flush=True)
        _run(cmd)
        return o

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(_do, jobs))
    # drop stale objects of sources that changed
    keep = {o.name for o in objs}
    hflags_probe = "runtime_"
    for old in BUILD.glob("*.o"):
        if old.name.startswith(hflags_probe):
            continue
        if old.name not in keep:
            old.unlink()
    stamp = BUILD / "link.stamp"
    want = "\n".join(sorted(keep))
    if force or jobs or not TARGET.exists() or not stamp.exists() or stamp.read_text() != want:
        lib_dirs = ce.library_paths()
        tmp = TARGET.with_suffix(".so.tmp")       # link beside the target, then rename: readers never see a partial file
        link = ["g++", "-shared", "-o", str(tmp), *map(str, objs)]
        for d in lib_dirs:
            link += [f"-L{d}", f"-Wl,-rpath,{d}"]
        link += [f"-L{_cuda_home()}/lib64", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
                 "-ltorch", "-ltorch_python", "-lcudart"]
        if verbose:
            print("[build] link", TARGET.name, flush=True)
        _run(link)
        os.replace(tmp, TARGET)
        stamp.write_text(want)
    build_host(verbose, force)
    return TARGET


HOST_TARGET = Path(__file__).resolve().parent / f"_host{EXT_SUFFIX}"


def build_host(verbose: bool = False, force: bool = False) -> Path:
    """``csrc/runtime/*.cpp`` -> ``rustorch_b200/_host*.so``: the host-only native runtime (pybind11, no CUDA and
    no torch), so it also loads where there is no GPU."""
    import pybind11
    BUILD.mkdir(parents=True, exist_ok=True)
    srcs = sorted((CSRC / "runtime").glob("*.cpp"))
    hdr = _headers_digest()
    flags = ["-O2", "-std=c++17", "-fPIC", "-pthread", "-fvisibility=hidden", f"-I{pybind11.get_include()}",
             f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC}"]
    objs, rebuilt = [], False
    for s in srcs:
        o = _obj_for(s, hdr, "host " + " ".join(flags))
        objs.append(o)
        if force or not o.exists():
            if verbose:
                print("[build]", s.name, flush=True)
            _run(["g++", *flags, "-c", str(s), "-o", str(o)])
            rebuilt = True
    if rebuilt or force or not HOST_TARGET.exists():
        _run(["g++", "-shared", "-pthread", "-o", str(HOST_TARGET), *map(str, objs)])
    return HOST_TARGET


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv))
