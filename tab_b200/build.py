"""In-tree build of the CUDA library and the ``TAB_CUDA`` extension module, for sm_100a only.

    python -m tab_b200.build            # libtab_b200.so + TAB_CUDA module
    python -m tab_b200.build --lib      # libtab_b200.so only

``libtab_b200.so`` (the C ABI of ``include/tab_b200.h``) is compiled with nvcc directly;
``TAB_CUDA`` (the reference-named PyTorch extension) is built by ``Setup_CUDA.py`` at the repository root
and links against it.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtab_b200.so")
SOURCES = ["c_abi.cu", "quantize_sm100.cu", "conv_sm100.cu", "conv_umma_sm100.cu", "umma_probe.cu", "conv_static_sm100.cu", "chain_sm100.cu", "pipe_probe.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile_one(args):
    nvcc, src, obj = args
    r = subprocess.run([nvcc] + NVCC_FLAGS + ["-c", "-o", obj, src], capture_output=True, text=True)
    return src, r.returncode, r.stdout, r.stderr


def build_library(force=False, verbose=False):
    """nvcc -> tab_b200/libtab_b200.so (one object per source, compiled in parallel under ``build/``).  Returns the
    ptxas resource report, which is also kept as ``build/libtab_b200.ptxas.txt``."""
    from concurrent.futures import ThreadPoolExecutor
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    hdrs = [os.path.join(CSRC, "tab_kernels.cuh"), os.path.join(CSRC, "umma_common.cuh"),
            os.path.join(ROOT, "include", "tab_b200.h"), __file__]
    objdir = os.path.join(ROOT, "build", "libtab_b200")
    os.makedirs(objdir, exist_ok=True)
    log = os.path.join(ROOT, "build", "libtab_b200.ptxas.txt")
    nvcc = os.environ.get("NVCC", "nvcc")
    jobs, objs = [], []
    for s in srcs:
        obj = os.path.join(objdir, os.path.basename(s) + ".o")
        objs.append(obj)
        if force or _stale(obj, [s] + hdrs):
            jobs.append((nvcc, s, obj))
    if not jobs and not _stale(LIB, objs):
        return open(log).read() if os.path.exists(log) else ""
    report = []
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        for src, rc, out, err in ex.map(_compile_one, jobs):
            if rc != 0:
                raise RuntimeError("nvcc failed on %s:\n%s\n%s" % (src, out, err))
            report.append("==== %s\n%s" % (os.path.basename(src), err))
    r = subprocess.run([nvcc, "-shared", "-o", LIB] + objs, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc link failed:\n%s\n%s" % (r.stdout, r.stderr))
    text = "\n".join(report)
    with open(log, "a" if len(jobs) < len(srcs) and os.path.exists(log) else "w") as f:
        f.write(text)
    if verbose:
        print(text)
    return text


def module_path():
    import glob
    hits = glob.glob(os.path.join(ROOT, "TAB_CUDA*.so"))
    return hits[0] if hits else None


def build_module(force=False):
    """``python Setup_CUDA.py build_ext --inplace`` -> TAB_CUDA*.so at the repository root."""
    deps = [os.path.join(CSRC, "tab_api.cpp"), os.path.join(ROOT, "include", "tab_b200.h"), os.path.join(ROOT, "Setup_CUDA.py")]
    mp = module_path()
    if not force and mp and not _stale(mp, deps):
        return mp
    r = subprocess.run([sys.executable, "Setup_CUDA.py", "build_ext", "--inplace"], cwd=ROOT, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("Setup_CUDA.py failed:\n%s\n%s" % (r.stdout[-4000:], r.stderr[-4000:]))
    return module_path()


def build_all(force=False):
    build_library(force=force)
    return build_module(force=force)


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_library(force=force, verbose=True) if "--lib" in sys.argv else build_all(force=force))
