"""In-tree native build: compiles every CUDA translation unit for sm_100a into
``lib/libtfb_kernels.so`` and every host C++ library (codec, tokenizer, server) into its own
shared object next to it.  Objects are rebuilt only when a source or header is newer.

    python -m transformers_fusion_b200.build            # build everything
    python -m transformers_fusion_b200.build --force    # rebuild from scratch

nvcc cross-compiles without a GPU, so this also serves as the "does it build" check.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall", "-Wno-unused-function"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _newer(src_list, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in src_list)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def _compile_many(jobs, workers):
    with cf.ThreadPoolExecutor(max_workers=workers) as ex:
        for out in ex.map(_run, jobs):
            if out.strip() and os.environ.get("TFB_BUILD_VERBOSE"):
                print(out)


def build_kernels(force=False, verbose=False, bounds_check=False) -> Path:
    """All .cu files under csrc/kernels and csrc/comm -> lib/libtfb_kernels.so.  ``bounds_check`` builds the variant
    with -DTFB_BOUNDS_CHECK into lib/libtfb_kernels_check.so (loaded when the environment has TFB_BOUNDS_CHECK=1)."""
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    suffix, extra = ("_check", ["-DTFB_BOUNDS_CHECK"]) if bounds_check else ("", [])
    srcs = sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu"))
    hdrs = list((CSRC / "kernels").glob("*.cuh")) + list((CSRC / "kernels").glob("*.h")) + \
        list((CSRC / "comm").glob("*.cuh")) + list((CSRC / "comm").glob("*.h"))
    jobs, objs = [], []
    for s in srcs:
        o = OBJ / (s.stem + suffix + ".o")
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            cmd = [nvcc] + NVCC_FLAGS + extra + ["-I", str(CSRC / "kernels"), "-I", str(CSRC / "comm"), "-c", str(s), "-o", str(o)]
            if verbose:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)
    _compile_many(jobs, workers=min(8, os.cpu_count() or 4))
    so = LIB / f"libtfb_kernels{suffix}.so"
    if force or jobs or not so.exists():
        _run([nvcc, "-shared", "-o", str(so)] + [str(o) for o in objs] + ["-cudart", "static"])
    return so


def build_host_lib(name: str, subdir: str, force=False, extra_libs=()) -> Path | None:
    """All .cpp files under csrc/<subdir> -> lib/lib<name>.so (skipped when the folder is empty)."""
    d = CSRC / subdir
    srcs = sorted(d.glob("*.cpp"))
    if not srcs:
        return None
    hdrs = list(d.glob("*.h")) + list(d.glob("*.hpp"))
    OBJ.mkdir(parents=True, exist_ok=True)
    jobs, objs = [], []
    cxx = os.environ.get("TFB_CXX", "g++")  # not $CXX: a toolchain with a static libstdc++ would clash with torch's
    for s in srcs:
        o = OBJ / f"{subdir}_{s.stem}.o"
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            jobs.append([cxx] + CXX_FLAGS + ["-I", str(d), "-c", str(s), "-o", str(o)])
    _compile_many(jobs, workers=min(8, os.cpu_count() or 4))
    so = LIB / f"lib{name}.so"
    if force or jobs or not so.exists():
        _run([cxx, "-shared", "-pthread", "-o", str(so)] + [str(o) for o in objs] + list(extra_libs))
    return so


def build_capi(force=False) -> Path | None:
    """csrc/capi -> lib/libtfb_capi.so, linked against the running interpreter's libpython (skipped when the
    development headers are not installed)."""
    import sysconfig
    inc = sysconfig.get_paths()["include"]
    if not (Path(inc) / "Python.h").exists():
        return None
    d = CSRC / "capi"
    src, so = d / "tfb_capi.cpp", LIB / "libtfb_capi.so"
    if force or _newer([src, d / "tfb_capi.h"], so):
        cxx = os.environ.get("TFB_CXX", "g++")
        libdir = sysconfig.get_config_var("LIBDIR") or "/usr/lib"
        ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
        _run([cxx] + CXX_FLAGS + ["-shared", "-I", inc, "-I", str(d), str(src), "-o", str(so), f"-L{libdir}", f"-lpython{ver}",
              f"-Wl,-rpath,{libdir}"])
    return so


def build_tools(force=False):
    """Native command-line front ends (csrc/tools/*.cpp) -> lib/bin/<name>."""
    d = CSRC / "tools"
    out = []
    if not d.exists():
        return out
    bind = LIB / "bin"
    bind.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("TFB_CXX", "g++")  # not $CXX: a toolchain with a static libstdc++ would clash with torch's
    for s in sorted(d.glob("*.cpp")):
        exe = bind / s.stem
        deps = [s] + list((CSRC / "codec").glob("*.h")) + list((CSRC / "serve").glob("*.h")) + \
            list((CSRC / "tokenizer").glob("*.h"))
        if force or _newer(deps, exe):
            _run([cxx] + CXX_FLAGS + ["-I", str(CSRC / "codec"), "-I", str(CSRC / "serve"), "-I", str(CSRC / "tokenizer"),
                  str(s), "-o", str(exe), f"-L{LIB}", "-ltfb_codec", "-ltfb_tokenizer", "-ltfb_serve",
                  f"-Wl,-rpath,$ORIGIN/.."])
        out.append(exe)
    return out


def build_sanitized(kind: str = "asan", force=False) -> Path:
    """The host-side native sources (codec + container, tokenizer, HTTP server) and the harness csrc/san/san_driver.cpp as
    one executable under a sanitizer: kind "asan" = -fsanitize=address,undefined, "tsan" = -fsanitize=thread.
    Product: lib/bin/tfb_san_<kind> (run it with a scratch directory as its argument)."""
    flags = {"asan": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "tsan": ["-fsanitize=thread"]}[kind]
    bind = LIB / "bin"
    bind.mkdir(parents=True, exist_ok=True)
    exe = bind / f"tfb_san_{kind}"
    srcs = [CSRC / "san" / "san_driver.cpp"] + sorted((CSRC / "codec").glob("*.cpp")) + sorted((CSRC / "tokenizer").glob("*.cpp")) + \
        sorted((CSRC / "serve").glob("*.cpp"))
    deps = srcs + list((CSRC / "codec").glob("*.h"))
    if force or _newer(deps, exe):
        cxx = os.environ.get("TFB_CXX", "g++")
        _run([cxx, "-O1", "-g", "-fno-omit-frame-pointer", "-std=c++17", "-pthread", "-Wall", "-Wno-unused-function"] + flags +
             ["-I", str(CSRC / "codec")] + [str(s) for s in srcs] + ["-o", str(exe)])
    return exe


def build_all(force=False, verbose=False, bounds_check=True):
    LIB.mkdir(exist_ok=True)
    built = [build_kernels(force, verbose)]
    if bounds_check:
        built.append(build_kernels(force, False, bounds_check=True))
    for name, sub in (("tfb_codec", "codec"), ("tfb_tokenizer", "tokenizer"), ("tfb_serve", "serve")):
        so = build_host_lib(name, sub, force)
        if so:
            built.append(so)
    capi = build_capi(force)
    if capi:
        built.append(capi)
    built += build_tools(force)
    return built


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="pass -Xptxas -v (set TFB_BUILD_VERBOSE=1 to print)")
    ap.add_argument("--no-bounds-check", action="store_true", help="skip the -DTFB_BOUNDS_CHECK variant of the kernel library")
    ap.add_argument("--sanitize", choices=["asan", "tsan"], help="only build the sanitizer harness of the host-side native code "
                                                                "(lib/bin/tfb_san_asan: address + undefined behaviour; tfb_san_tsan: threads)")
    a = ap.parse_args(argv)
    if a.sanitize:
        print("built", build_sanitized(a.sanitize, a.force))
        return
    for p in build_all(a.force, a.verbose, not a.no_bounds_check):
        print("built", p)


if __name__ == "__main__":
    main(sys.argv[1:])
