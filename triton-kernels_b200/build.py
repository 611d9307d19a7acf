"""Build libema_b200.so (sm_100a only) in-tree with nvcc.

    python triton-kernels_b200/build.py [--force] [--verbose] [--checked]

--checked builds lib/libema_b200_checked.so as well: the same sources with -DEMA_BOUNDS_CHECK, every plain global-memory
access of the fused kernels checked against the call's buffers (csrc/ema_bounds.cuh).

The library lands in triton-kernels_b200/lib/ next to the sources, so that it travels with the
repository checkout; nothing is installed into site-packages or a JIT cache.
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libema_b200.so")
LIB_CHECKED = os.path.join(LIB_DIR, "libema_b200_checked.so")

def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def needs_build(lib=LIB):
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "ema_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, defines=(), out=None):
    """Compiles every .cu under csrc/ and links the library.  `defines` (e.g. ["EMA_TRYWAIT_HINT_NS=1000"]) and `out`
    (another library path; objects go next to it) build a variant beside the default library for A/B measurements."""
    lib = out or LIB
    if not force and not out and not needs_build():
        return LIB
    obj_dir = os.path.join(os.path.dirname(lib), "obj_" + os.path.basename(lib)[:-3]) if out else LIB_DIR
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
               "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c", src, "-o", obj]
        cmd += [f"-D{d}" for d in defines]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write(f"--- {os.path.basename(src)}\n{out}\n")
        failed = failed or pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc, "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"])
    return lib


def build_checked(force=False, verbose=False):
    """The bounds-checking variant, beside the default library."""
    if not force and not needs_build(LIB_CHECKED):
        return LIB_CHECKED
    return build(force=True, verbose=verbose, defines=["EMA_BOUNDS_CHECK"], out=LIB_CHECKED)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("-D", dest="defines", action="append", default=[], help="preprocessor definition for a variant build")
    ap.add_argument("--out", help="path of the variant library (default: the package's lib/libema_b200.so)")
    ap.add_argument("--checked", action="store_true", help="also build the bounds-checking variant")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.defines, a.out))
    if a.checked:
        print(build_checked(a.force, a.verbose))
