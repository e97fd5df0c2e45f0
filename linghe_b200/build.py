"""Build the CUDA library in-tree for sm_100a.

    python -m linghe_b200.build [--force] [--verbose]

Compiles every ``csrc/*.cu`` with nvcc (``-gencode arch=compute_100a,code=sm_100a``,
relocatable device code, one process per file) and links ``lib/liblinghe_b200.so``.
nvcc cross-compiles, so no GPU is needed to build.
"""

from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")
LIBNAME = "liblinghe_b200.so"
HOSTDIR = os.path.join(PKG, "host")
HOSTNAME = "_lh_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]


WHOLE_PROGRAM = {"lh_duo.cu"}


def nvcc_path() -> str:
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found; the CUDA 12.9 toolkit is required to build linghe_b200")
    return p


def lib_path() -> str:
    return os.path.join(LIBDIR, LIBNAME)


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    inc = os.path.join(os.path.dirname(PKG), "include", "linghe_b200.h")
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))] + [inc]
    files += [os.path.join(HOSTDIR, f) for f in sorted(os.listdir(HOSTDIR)) if f.endswith(".cpp")]
    for f in files:
        with open(f, "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJDIR, src[:-3] + ".o")
    # relocatable device code everywhere except the files that use setmaxnreg (ptxas ignores it there)
    mode = ["-c"] if src in WHOLE_PROGRAM else ["-rdc=true", "-dc"]
    cmd = [nvcc_path(), *NVCC_FLAGS, *mode, os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = os.path.join(OBJDIR, src[:-3] + ".ptxas.log")
    with open(log, "w") as fh:
        fh.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    stamp = os.path.join(LIBDIR, "build.stamp")
    dig = _digest()
    if not force and os.path.exists(lib_path()) and os.path.exists(stamp):
        if open(stamp).read().strip() == dig:
            return lib_path()
    srcs = _sources()
    with cf.ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), srcs))
    cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC",
           *objs, "-o", lib_path(), "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    _build_host(verbose)
    with open(stamp, "w") as fh:
        fh.write(dig)
    return lib_path()


def host_path() -> str:
    return os.path.join(LIBDIR, HOSTNAME)


def _gen_host_bindings(path: str) -> None:
    """One pybind11 definition per entry point of include/linghe_b200.h, generated from the
    header: pointers travel as integers (tensor.data_ptr()), scalars as they are.  A call through
    these costs about a microsecond; the same call through ctypes costs four."""
    import re
    hdr = open(os.path.join(os.path.dirname(PKG), "include", "linghe_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    lines = []
    for m in re.finditer(r"(int|int64_t|const char\*)\s+(lh_\w+)\s*\(([^)]*)\)\s*;", hdr):
        ret, name, args = m.group(1), m.group(2), m.group(3).strip()
        params, call = [], []
        if args not in ("", "void"):
            for i, a in enumerate(x.strip() for x in args.split(",")):
                typ = a[:a.rindex(" ")].strip() if not a.endswith("*") else a
                if "*" in a:
                    typ = a[:a.rindex("*") + 1].strip()
                if typ == "const char*":
                    params.append(f"const std::string& a{i}")
                    call.append(f"a{i}.c_str()")
                elif "*" in typ:
                    params.append(f"uintptr_t a{i}")
                    call.append(f"reinterpret_cast<{typ}>(a{i})")
                else:
                    params.append(f"{typ} a{i}")
                    call.append(f"a{i}")
        body = f"{name}({', '.join(call)})"
        if ret == "const char*":
            body = f"std::string({body})"
        lines.append(f'm.def("{name}", []({", ".join(params)}) {{ return {body}; }});')
    with open(path, "w") as fh:
        fh.write("// generated from include/linghe_b200.h by linghe_b200/build.py\n" + "\n".join(lines) + "\n")


def _build_host(verbose: bool) -> None:
    """The C++ argument handling of the hottest wrappers (host/lh_host.cpp): a Python extension module
    linked against the library above.  Optional: without it the wrappers go through ctypes (the
    same C ABI and kernels, a few microseconds more host time per call), so a failure here is
    reported and does not fail the build."""
    if os.path.exists(host_path()):
        os.remove(host_path())
    try:
        import sysconfig

        import torch
        from torch.utils import cpp_extension as ce
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        _gen_host_bindings(os.path.join(OBJDIR, "lh_host_bindings.inc"))
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", os.path.join(HOSTDIR, "lh_host.cpp"), "-o", host_path(),
               "-I" + os.path.join(os.path.dirname(PKG), "include"), "-I" + OBJDIR, "-I/usr/local/cuda/include",
               "-I" + sysconfig.get_paths()["include"], *["-I" + d for d in ce.include_paths()],
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-DTORCH_EXTENSION_NAME=_lh_host",
               "-DTORCH_API_INCLUDE_EXTENSION_H", "-L" + tlib, "-lc10", "-lc10_cuda", "-ltorch", "-ltorch_cpu",
               "-ltorch_python", "-L" + LIBDIR, "-llinghe_b200", "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(r.stderr[-2000:])
        if verbose:
            print(r.stderr)
    except Exception as e:  # noqa: BLE001 -- optional component, see the docstring
        print(f"linghe_b200.build: host module not built ({e}); the wrappers will use ctypes", file=sys.stderr)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))


if __name__ == "__main__":
    sys.exit(main())
