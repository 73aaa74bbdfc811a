"""In-tree build of the native library.

Steps (each skipped when its outputs are newer than its inputs):

1. every kernel source under ``csrc/kernels`` -> one sm_100a code object
   (``nvcc -cubin -gencode arch=compute_100a,code=sm_100a -lineinfo``) under
   ``build/``;
2. the code objects are embedded through an assembler ``.incbin`` table;
3. the C++23 runtime, registry, harness and C ABI are compiled with ``g++`` and
   linked into ``libkernelh_b200.so`` (the CUDA driver is only ever dlopen'ed);
4. the ``kernelh`` command-line tool is linked against that library;
5. ``csrc/noalloc`` sources, if any, are compiled by nvcc as ordinary CUDA
   runtime code into the same library.

Run as ``python kernelh_b200/csrc/build.py`` or through ``__graft_entry__.build()``. The
script lives outside the Python package on purpose: importing the package loads
the library, which must not be a precondition for building it.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(CSRC)
ROOT = os.path.dirname(PKG)
BUILD = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libkernelh_b200.so")
CLI = os.path.join(PKG, "bin", "kernelh")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

KERNELS = ["vecadd", "fused_gelu", "scan", "softmax", "layernorm", "gemm", "attention"]
IMAGES = KERNELS  # code objects: one per kernel template
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = NVCC_ARCH + ["-lineinfo", "-O3", "-std=c++17"]
CXX = "g++"  # plain g++ from PATH: an inherited CXX may be a wrapper without C++23 support
CXXFLAGS = ["-std=c++23", "-O2", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter",
            "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA_HOME, "include")]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"build step failed ({res.returncode}): {' '.join(cmd)}")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout + res.stderr, flush=True)


def _headers(subdir: str) -> list[str]:
    d = os.path.join(CSRC, subdir)
    return [os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith((".hpp", ".cuh", ".h"))]


def _cpp_sources() -> list[str]:
    out = []
    for sub in ("runtime", "registry", "harness", "capi"):
        d = os.path.join(CSRC, sub)
        out += [os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith(".cpp")]
    return out


def build_cubins(verbose: bool = False, ptxas_info: bool = False) -> list[str]:
    """One code object per kernel source. ptxas runs verbosely every time and its per-entry
    resource lines (registers, static shared memory, spills, barriers) are kept beside the
    code object as ``<name>.ptxas.txt``: the library embeds that text and serves it as the
    kernel's resources.json."""
    os.makedirs(BUILD, exist_ok=True)
    outs = []
    headers = _headers("kernels")
    for name in IMAGES:
        src = os.path.join(CSRC, "kernels", name + ".cu")
        out = os.path.join(BUILD, name + ".cubin")
        report = os.path.join(BUILD, name + ".ptxas.txt")
        outs.append(out)
        if _newer(out, [src] + headers) and _newer(report, [out]) and not ptxas_info:
            continue
        cmd = [NVCC, "-cubin"] + NVCC_FLAGS + ["-Xptxas", "-v", "-o", out, src]
        if verbose or ptxas_info:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError(f"build step failed ({res.returncode}): {' '.join(cmd)}")
        text = "".join(line + "\n" for line in (res.stdout + res.stderr).splitlines() if "ptxas info" in line
                       or "bytes stack frame" in line)
        with open(report, "w") as f:
            f.write(text)
        if ptxas_info:
            print(text, flush=True)
    return outs


def _write_blob_table(cubins: list[str]) -> tuple[str, str]:
    asm = os.path.join(BUILD, "cubin_blobs.S")
    cpp = os.path.join(BUILD, "cubin_blobs.cpp")
    lines = ['.section .rodata, "a"']
    for name, path in zip(IMAGES, cubins):
        lines += [f".balign 64", f".global kh_cubin_{name}", f"kh_cubin_{name}:",
                  f'.incbin "{path}"', f".global kh_cubin_{name}_end", f"kh_cubin_{name}_end:"]
    lines.append('.section .note.GNU-stack, "", @progbits')
    text = "\n".join(lines) + "\n"
    if not os.path.exists(asm) or open(asm).read() != text:
        with open(asm, "w") as f:
            f.write(text)
    body = ['// generated by kernelh_b200/build.py: table of embedded sm_100a code objects',
            '#include "../csrc/registry/registry.hpp"', 'extern "C" {']
    for name in IMAGES:
        body.append(f"extern const unsigned char kh_cubin_{name}[], kh_cubin_{name}_end[];")
    body += ["}", "namespace kh {", "const CodeObject *code_objects_begin() {",
             "  static const CodeObject objects[] = {"]
    for name, path in zip(IMAGES, cubins):
        with open(path[:-len(".cubin")] + ".ptxas.txt") as f:
            report = f.read()
        literal = "".join('\n          "' + line.replace("\\", "\\\\").replace('"', '\\"') + '\\n"'
                          for line in report.splitlines()) or ' ""'
        body.append(f'      {{"{name}", kh_cubin_{name}, '
                    f"static_cast<size_t>(kh_cubin_{name}_end - kh_cubin_{name}),{literal}}},")
    body += ["  };", "  return objects;", "}",
             f"extern const int kCodeObjectCount = {len(IMAGES)};", "} // namespace kh", ""]
    text = "\n".join(body)
    if not os.path.exists(cpp) or open(cpp).read() != text:
        with open(cpp, "w") as f:
            f.write(text)
    return asm, cpp


def build_library(verbose: bool = False) -> str:
    cubins = build_cubins(verbose)
    asm, blob_cpp = _write_blob_table(cubins)
    all_headers = sum((_headers(s) for s in ("runtime", "registry", "harness")), []) + [
        os.path.join(ROOT, "include", "kernelh_b200.h")]
    objs = []
    for src in _cpp_sources() + [blob_cpp]:
        obj = os.path.join(BUILD, os.path.basename(src).replace(".cpp", ".o"))
        objs.append(obj)
        if _newer(obj, [src] + all_headers):
            continue
        _run([CXX] + CXXFLAGS + ["-c", src, "-o", obj], verbose)
    blob_obj = os.path.join(BUILD, "cubin_blobs_data.o")
    if not _newer(blob_obj, [asm] + cubins):
        _run(["gcc", "-c", asm, "-o", blob_obj], verbose)
    objs.append(blob_obj)
    extra_libs = []
    noalloc_dir = os.path.join(CSRC, "noalloc")
    if os.path.isdir(noalloc_dir):
        for f in sorted(os.listdir(noalloc_dir)):
            if not f.endswith(".cu"):
                continue
            src = os.path.join(noalloc_dir, f)
            obj = os.path.join(BUILD, f.replace(".cu", "_rt.o"))
            objs.append(obj)
            # these sources #include kernel sources, so every file under kernels/ is an input
            kernel_dir = os.path.join(CSRC, "kernels")
            deps = [os.path.join(kernel_dir, k) for k in sorted(os.listdir(kernel_dir))]
            if not _newer(obj, [src] + deps):
                _run([NVCC] + NVCC_FLAGS + ["-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"),
                                            "-I", os.path.join(CSRC, "kernels"), "-c", src, "-o", obj], verbose)
            extra_libs = ["-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart_static", "-lrt", "-lpthread"]
    if not _newer(LIB, objs):
        _run([CXX, "-shared", "-o", LIB] + objs + extra_libs + ["-ldl"], verbose)
    return LIB


def build_cli(verbose: bool = False) -> str:
    src = os.path.join(CSRC, "cli", "kernelh_main.cpp")
    if not os.path.exists(src):
        return ""
    os.makedirs(os.path.dirname(CLI), exist_ok=True)
    if not _newer(CLI, [src, LIB]):
        _run([CXX] + CXXFLAGS + [src, "-o", CLI, "-L", PKG, "-lkernelh_b200",
                                 "-Wl,-rpath,$ORIGIN/..", "-ldl"], verbose)
    return CLI


def _source_digest() -> str:
    """Content hash of everything the build reads, so a copied tree with fresh
    mtimes is recognised as already built."""
    h = hashlib.sha256()
    files = [os.path.abspath(__file__), os.path.join(ROOT, "include", "kernelh_b200.h")]
    for sub in sorted(os.listdir(CSRC)):
        d = os.path.join(CSRC, sub)
        if os.path.isdir(d):
            files += [os.path.join(d, f) for f in sorted(os.listdir(d))
                      if os.path.isfile(os.path.join(d, f))]
    for path in files:
        h.update(path[len(ROOT):].encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def build_all(verbose: bool = False) -> None:
    stamp = os.path.join(BUILD, "stamp.txt")
    digest = _source_digest()
    have_cli = os.path.exists(CLI) or not os.path.exists(os.path.join(CSRC, "cli", "kernelh_main.cpp"))
    if os.path.exists(LIB) and have_cli and os.path.exists(stamp) and open(stamp).read() == digest:
        return
    if shutil.which(NVCC) is None and not os.path.exists(NVCC):
        raise RuntimeError(f"nvcc not found at {NVCC}: the sm_100a kernels cannot be built")
    build_library(verbose)
    build_cli(verbose)
    with open(stamp, "w") as f:
        f.write(digest)


if __name__ == "__main__":
    if "--ptxas-info" in sys.argv:
        build_cubins(verbose=True, ptxas_info=True)
    else:
        build_all(verbose="-v" in sys.argv)
        print(LIB)
