"""Build the CPU oracle (``liboracle*.so``) and, where the reference source tree is present, the
reference's own CPU GEMMs (``oracle/_ref/libtab_ref*.so``) and its CUDA kernel bodies compiled for the
host (``oracle/_ref/libtab_ref_cuda.so``).  TEST INFRASTRUCTURE ONLY.

Two flag sets are built for each: the flags of the reference's ``Setup_GCC.py:12`` split into
separate arguments plus ``-DGCC`` ("shipped": no ``-mpopcnt``, so the 64-bit popcount is a libgcc
call), and the same plus ``-march=x86-64-v3`` ("v3": hardware POPCNT / AVX2).

The reference's ``TAB_CPU.cpp`` does not compile as a whole (undefined identifiers in its wrappers),
so only its ``*GEMM_baseline`` functions are used: they are located by signature in the file where it
lies, written to a temporary include outside this repository, compiled through ``ref_shim.cpp`` and
the temporary is deleted.  Only the resulting ``.so`` files are kept (git-ignored).

The reference's ``TAB_GEMM.cu`` does not compile under nvcc 12.9 either (``goto`` across initialisations
in its host functions) and there is no GPU where this is built, but its *kernels* are plain C bodies:
they are located by signature in ``TAB_GEMM.cu`` / ``TAB_GEMM.cuh``, written to a temporary include and
compiled for the host through ``ref_cuda_shim.cpp``, which supplies the index variables and loops the
reference's launch shapes.  That library executes the reference's quantise, BTN_Weight, pad, im2row and
GEMM code itself, so every stage of the oracle is checked against reference code that ran.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
# where the reference source tree lies: TAB_REFERENCE_DIR, else a "reference" directory beside this repository
REF_DIR = os.environ.get("TAB_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
SHIPPED = ["-fopenmp", "-flax-vector-conversions", "-funsafe-math-optimizations", "-fbuiltin", "-O3"]  # Setup_GCC.py:12
VARIANTS = {"shipped": SHIPPED, "v3": SHIPPED + ["-march=x86-64-v3"]}


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "tab_oracle.c")
    out = []
    for name, flags in VARIANTS.items():
        so = os.path.join(HERE, "liboracle_%s.so" % name)
        if force or not _newer(so, [src, __file__]):
            _run(["gcc", "-std=c11", "-shared", "-fPIC"] + flags + ["-o", so, src])
        out.append(so)
    return out


def _extract_gemms(text):
    """The four ``std::vector<int> XXXGEMM_baseline(...) { ... }`` definitions, by signature."""
    parts = []
    for name in ("TNNGEMM_baseline", "TBNGEMM_baseline", "BTNGEMM_baseline", "BNNGEMM_baseline"):
        m = re.search(r"^std::vector<int>\s+%s\s*\(" % name, text, flags=re.M)
        if not m:
            raise RuntimeError("reference function %s not found" % name)
        end = text.index("\n}\n", m.start()) + 3
        parts.append(text[m.start():end])
    return "\n".join(parts)


def build_ref(force=False):
    """Returns the list of built libraries, or [] when the reference tree is not available."""
    cpp = os.path.join(REF_DIR, "TAB_CPU.cpp")
    hdr = os.path.join(REF_DIR, "TAB_CPU.h")
    out_dir = os.path.join(HERE, "_ref")
    shim = os.path.join(HERE, "ref_shim.cpp")
    if not (os.path.exists(cpp) and os.path.exists(hdr)):
        return [p for p in (os.path.join(out_dir, "libtab_ref_%s.so" % n) for n in VARIANTS) if os.path.exists(p)]
    os.makedirs(out_dir, exist_ok=True)
    out = []
    with tempfile.TemporaryDirectory(prefix="tab_ref_") as tmp:
        inc = os.path.join(tmp, "ref_gemm_extract.inc")
        with open(cpp, "r", errors="replace") as f:
            code = _extract_gemms(f.read())
        with open(inc, "w") as f:
            f.write(code)
        for name, flags in VARIANTS.items():
            so = os.path.join(out_dir, "libtab_ref_%s.so" % name)
            if force or not _newer(so, [shim, cpp, hdr, __file__]):
                _run(["g++", "-std=c++17", "-shared", "-fPIC"] + flags +
                     ["-I", REF_DIR, '-DREF_GEMM_INC="%s"' % inc, "-o", so, shim])
            out.append(so)
    return out


CUDA_KERNELS_CU = ["GetIdx", "TNNGEMM", "TBNGEMM", "BTNGEMM", "BNNGEMM", "BTN_Weight", "TerOnlyKernel", "BinOnlyKernel"]
CUDA_KERNELS_CUH = ["PadKernel", "Img2RowKernel"]


def _extract_cuda_function(text, name):
    """The definition ``[template<...>] __global__|__device__ void name(...) { ... }`` (not a prototype)."""
    for m in re.finditer(r"^(template\s*<[^>]*>\s*\n)?__(?:global|device)__\s+void\s+%s\s*\(" % name, text, flags=re.M):
        close = text.index(")", m.end())
        rest = text[close + 1:].lstrip()
        if not rest.startswith("{"):
            continue                                  # a declaration
        start = text.index("{", close)
        depth, i = 0, start
        while True:
            ch = text[i]
            if ch == "{":
                depth += 1
            elif ch == "}":
                depth -= 1
                if depth == 0:
                    return text[m.start():i + 1]
            i += 1
    raise RuntimeError("reference kernel %s not found" % name)


def build_ref_cuda(force=False):
    """``oracle/_ref/libtab_ref_cuda.so``: the reference's CUDA kernel bodies run on the host.  Returns its path,
    or None when neither the reference tree nor a prebuilt library is available."""
    cu = os.path.join(REF_DIR, "TAB_GEMM.cu")
    cuh = os.path.join(REF_DIR, "TAB_GEMM.cuh")
    out_dir = os.path.join(HERE, "_ref")
    so = os.path.join(out_dir, "libtab_ref_cuda.so")
    shim = os.path.join(HERE, "ref_cuda_shim.cpp")
    if not (os.path.exists(cu) and os.path.exists(cuh)):
        return so if os.path.exists(so) else None
    if not force and _newer(so, [shim, cu, cuh, __file__]):
        return so
    os.makedirs(out_dir, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="tab_ref_") as tmp:
        inc = os.path.join(tmp, "ref_cuda_extract.inc")
        with open(cu, "r", errors="replace") as f:
            text_cu = f.read()
        with open(cuh, "r", errors="replace") as f:
            text_cuh = f.read()
        parts = [_extract_cuda_function(text_cu, n) for n in CUDA_KERNELS_CU]
        parts += [_extract_cuda_function(text_cuh, n) for n in CUDA_KERNELS_CUH]
        with open(inc, "w") as f:
            f.write("\n\n".join(parts) + "\n")
        _run(["g++", "-std=c++17", "-shared", "-fPIC", "-O2", "-fopenmp", "-march=x86-64-v3",
              '-DREF_CUDA_INC="%s"' % inc, "-o", so, shim])
    return so


if __name__ == "__main__":
    print("\n".join(build_oracle(force="--force" in sys.argv)))
    print("\n".join(build_ref(force="--force" in sys.argv)) or "reference tree not present: oracle/_ref not rebuilt")
    print(build_ref_cuda(force="--force" in sys.argv) or "reference tree not present: libtab_ref_cuda.so not rebuilt")
