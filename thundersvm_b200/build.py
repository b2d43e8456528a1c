"""Builds libthundersvm_b200.so (CUDA kernels + C ABI + host classes) in-tree for sm_100a."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libthundersvm_b200.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler",
              "-fPIC,-fopenmp", "--expt-relaxed-constexpr"]


def sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cpp")):
                out.append(os.path.join(root, f))
    return sorted(out)


def headers():
    out = [os.path.join(HERE, "..", "include", "thundersvm_b200.h")]
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".cuh", ".h", ".hpp"))]
    return out


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > t for p in sources() + headers())


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs, procs = [], []
    for src in sources():
        obj = os.path.join(objdir, os.path.relpath(src, CSRC).replace(os.sep, "_") + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(
                [os.path.getmtime(src)] + [os.path.getmtime(h) for h in headers()]):
            cmd = [nvcc] + NVCC_FLAGS + os.environ.get("TSVM_NVCC_EXTRA", "").split() + (["-Xptxas", "-v"] if verbose else []) + [
                "-x", "cu", "-I", os.path.join(HERE, "..", "include"), "-I", os.path.join(CSRC, "host", "include"),
                "-c", src, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write("== %s\n%s\n" % (src, out))
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc, "-shared", "-o", LIB] + objs + ["-lcudart", "-Xcompiler", "-fopenmp"])
    build_cli(nvcc)
    return LIB


def build_cli(nvcc):
    """thundersvm-train / thundersvm-predict next to the library (rpath $ORIGIN/..)."""
    bindir = os.path.join(HERE, "bin")
    os.makedirs(bindir, exist_ok=True)
    for name in ("thundersvm-train", "thundersvm-predict"):
        src = os.path.join(HERE, "cli", name + ".cpp")
        subprocess.check_call([nvcc, "-O2", "-std=c++17", "-I", os.path.join(CSRC, "host", "include"), src, "-o",
                               os.path.join(bindir, name), "-L", HERE, "-lthundersvm_b200", "-Xlinker",
                               "-rpath=$ORIGIN/.."])


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
