"""In-tree native build for the sm_100a kernels and the libtorch C++ core.

Two shared objects are produced next to this file:

* ``libtitb200_kernels.so`` -- every ``csrc/kernels/*.cu`` file, compiled with
  ``nvcc -gencode arch=compute_100a,code=sm_100a``.  It depends on the CUDA
  runtime only and exports a plain C API (``csrc/kernels/api.h``).
* ``_C.so`` -- the libtorch side: op bindings (``csrc/binding``) and the C++
  framework core (``csrc/core``), linked against the kernel library.

Objects are cached under ``build/`` keyed by source + header mtimes and flags,
so a second call is a no-op.  ``nvcc`` cross-compiles without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import re
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG.parent / "build" / "titb200"

KERNEL_LIB = PKG / "libtitb200_kernels.so"
CORE_LIB = PKG / "_C.so"

NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
# The distribution's own g++ is used on purpose (override with TITB200_CXX): a toolchain wrapper found
# through $CXX on some images links parts of a static libstdc++ into the module, whose iostream state
# is then never initialised inside the Python process.
CXX = os.environ.get("TITB200_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
CUDA_HOME = Path(NVCC).resolve().parent.parent

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--expt-extended-lambda", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden", "-DNDEBUG",
]


def _torch_paths():
    import torch  # noqa: F401
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths()
    lib = ce.library_paths()
    return inc, lib


def _hdr_stamp(dirs) -> str:
    h = hashlib.sha1()
    for d in dirs:
        for p in sorted(Path(d).rglob("*")):
            if p.suffix in (".h", ".cuh", ".hpp"):
                h.update(str(p).encode())
                h.update(str(p.stat().st_mtime_ns).encode())
    return h.hexdigest()


def _obj_key(src: Path, flags, stamp: str) -> str:
    h = hashlib.sha1()
    h.update(str(src).encode())
    h.update(str(src.stat().st_mtime_ns).encode())
    h.update(" ".join(flags).encode())
    h.update(stamp.encode())
    # a source that includes another source file (a second compilation of the same kernel under other macros) is
    # rebuilt when that file changes
    if src.suffix == ".cu":
        for line in src.read_text().splitlines():
            m = re.match(r'\s*#include\s+"([^"]+\.cu)"', line)
            if m and (src.parent / m.group(1)).exists():
                h.update(str((src.parent / m.group(1)).stat().st_mtime_ns).encode())
    return h.hexdigest()[:16]


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        sys.stderr.write(r.stderr)
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd[:6]))} ...")
    if verbose and (r.stdout or r.stderr):
        sys.stderr.write(r.stdout + r.stderr)


def _compile_all(jobs, verbose):
    """jobs: list of (cmd, obj_path). Skips those whose obj exists."""
    todo = [(c, o) for c, o in jobs if not o.exists()]
    if not todo:
        return False
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        list(ex.map(lambda co: _run(co[0], verbose), todo))
    return True


def build(verbose: bool = False, force: bool = False) -> None:
    BUILD.mkdir(parents=True, exist_ok=True)
    stamp = _hdr_stamp([CSRC])

    # ---- 1. kernel library (pure CUDA) -------------------------------------
    cu_srcs = sorted((CSRC / "kernels").glob("*.cu"))
    kflags = NVCC_FLAGS + ["-I", str(CSRC / "kernels")]
    if os.environ.get("TITB200_PTXAS_V"):
        kflags = kflags + ["-Xptxas", "-v"]
    kjobs, kobjs = [], []
    for s in cu_srcs:
        o = BUILD / f"{s.stem}.{_obj_key(s, kflags, stamp)}.o"
        if force and o.exists():
            o.unlink()
        kobjs.append(o)
        kjobs.append(([NVCC, *kflags, "-c", s, "-o", o], o))
    changed = _compile_all(kjobs, verbose)
    if changed or not KERNEL_LIB.exists():
        _run([NVCC, "-shared", "-o", KERNEL_LIB, *kobjs, "-cudart", "shared",
              "-Xlinker", f"-rpath={CUDA_HOME}/lib64"], verbose)

    # ---- 2. libtorch core + bindings ---------------------------------------
    inc, lib = _torch_paths()
    py_inc = sysconfig.get_paths()["include"]
    cc_srcs = sorted((CSRC / "binding").glob("*.cpp")) + sorted((CSRC / "core").rglob("*.cc"))
    cflags = [
        "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-DNDEBUG",
        "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
        "-D_GLIBCXX_USE_CXX11_ABI=1", "-Wno-deprecated-declarations",
        "-I", str(CSRC), "-I", str(CSRC / "kernels"), "-I", str(CUDA_HOME / "include"),
        "-I", py_inc,
    ]
    for i in inc:
        cflags += ["-isystem", i]
    # TITB200_SANITIZE=1: AddressSanitizer + UBSan build of the host-side C++ (run the CPU tests with
    # LD_PRELOAD=$(g++ -print-file-name=libasan.so) and ASAN_OPTIONS=detect_leaks=0); rebuild without it afterwards.
    sanitize = ["-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-g"] if os.environ.get("TITB200_SANITIZE") else []
    cflags += sanitize
    cjobs, cobjs = [], []
    for s in cc_srcs:
        tag = hashlib.sha1(str(s.relative_to(CSRC)).encode()).hexdigest()[:6]
        o = BUILD / f"{s.stem}.{tag}.{_obj_key(s, cflags, stamp)}.o"
        if force and o.exists():
            o.unlink()
        cobjs.append(o)
        cjobs.append(([CXX, *cflags, "-c", s, "-o", o], o))
    changed2 = _compile_all(cjobs, verbose)
    if changed or changed2 or not CORE_LIB.exists() or sanitize:
        link = [CXX, "-shared", *sanitize, "-o", CORE_LIB, *cobjs,
                f"-L{PKG}", "-ltitb200_kernels", "-Wl,-rpath,$ORIGIN"]
        for l in lib:
            link += [f"-L{l}", f"-Wl,-rpath,{l}"]
        link += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python",
                 f"-L{CUDA_HOME}/lib64", "-lcudart", "-lc10_cuda", "-ltorch_cuda"]
        _run(link, verbose)

    # stale objects from earlier source versions
    live = {o.name for o in kobjs + cobjs}
    for p in BUILD.glob("*.o"):
        if p.name not in live:
            p.unlink()


def build_cpp(verbose: bool = False) -> dict:
    """The C++ API as a stand-alone library plus its test program and the C++ training example (no Python involved at
    run time): ``libtitb200_framework.so`` from ``csrc/core`` without the binding files, ``facade_api_test`` from
    ``tests/cpp`` and ``train_gpt2`` from ``examples/cpp``.  Returns the paths."""
    if not is_built():                        # the kernel library the framework links against; never rebuilt here when
        build(verbose=verbose)                # present, because a running process may have it loaded
    inc, lib = _torch_paths()
    root = PKG.parent
    srcs = [s for s in sorted((CSRC / "core").rglob("*.cc")) if not s.name.endswith("_binding.cc")]
    cflags = ["-O2", "-std=c++17", "-fPIC", "-DNDEBUG", "-D_GLIBCXX_USE_CXX11_ABI=1", "-Wno-deprecated-declarations",
              "-I", str(CSRC), "-I", str(CSRC / "kernels"), "-I", str(CUDA_HOME / "include")]
    for i in inc:
        cflags += ["-isystem", i]
    out_dir = BUILD / "cpp"
    out_dir.mkdir(parents=True, exist_ok=True)
    stamp = _hdr_stamp([CSRC])
    jobs, objs = [], []
    for s in srcs:
        tag = hashlib.sha1(str(s.relative_to(CSRC)).encode()).hexdigest()[:6]
        o = out_dir / f"{s.stem}.{tag}.{_obj_key(s, cflags, stamp)}.o"
        objs.append(o)
        jobs.append(([CXX, *cflags, "-c", s, "-o", o], o))
    changed = _compile_all(jobs, verbose)
    libs = []
    for l in lib:
        libs += [f"-L{l}", f"-Wl,-rpath,{l}"]
    libs += ["-lc10", "-ltorch_cpu", "-ltorch", f"-L{CUDA_HOME}/lib64", f"-Wl,-rpath,{CUDA_HOME}/lib64", "-lcudart",
             "-lc10_cuda", "-ltorch_cuda"]
    fw = PKG / "libtitb200_framework.so"
    if changed or not fw.exists():
        _run([CXX, "-shared", "-o", fw, *objs, f"-L{PKG}", "-ltitb200_kernels", "-Wl,-rpath,$ORIGIN", *libs], verbose)
    live = {o.name for o in objs}
    for p in out_dir.glob("*.o"):
        if p.name not in live:
            p.unlink()
    exes = {}
    for name, src in (("facade_api_test", root / "tests" / "cpp" / "facade_api_test.cc"),
                      ("train_gpt2", root / "examples" / "cpp" / "train_gpt2.cc")):
        exe = out_dir / name
        if changed or not exe.exists() or exe.stat().st_mtime < src.stat().st_mtime:
            _run([CXX, *cflags, src, "-o", exe, f"-L{PKG}", "-ltitb200_framework", "-ltitb200_kernels",
                  f"-Wl,-rpath,{PKG}", "-Wl,--no-as-needed", *libs], verbose)
        exes[name] = exe
    return {"library": fw, **exes}


def is_built() -> bool:
    return KERNEL_LIB.exists() and CORE_LIB.exists()


if __name__ == "__main__":
    build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    if "--cpp" in sys.argv:
        for k, v in build_cpp(verbose="-v" in sys.argv).items():
            print(f"{k}: {v}")
    print("built:", KERNEL_LIB.name, CORE_LIB.name)
