"""Build libbam_b200.so in-tree with nvcc for sm_100a (explicit command, no JIT cache)."""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libbam_b200.so")
SOURCES = ["bam_lib.cu", "bam_noalloc.cu", "bam_graph.cu", "bam_exchange.cu", "bam_nvm_host.cu"]


def _newer_than(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _deps():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    inc = os.path.join(ROOT, "include")
    for base, _, files in os.walk(inc):
        deps += [os.path.join(base, f) for f in files]
    return deps


def nvcc_path():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


PROFILE_LIB = os.path.join(HERE, "libbam_b200_prof.so")


def build_library(force=False, verbose=False, profile=False):
    """Compile the CUDA library; returns the path of the .so.  profile=True builds a second library with
    -DBAM_PROFILE (cycle and event counters of the queue protocol, the cache and the controller, read with
    bam_ctrl_profile); select it at run time with BAM_B200_LIB=<path>."""
    lib = PROFILE_LIB if profile else LIB
    if not force and not _newer_than(lib, _deps()):
        return lib
    cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xptxas", "-v", "-shared", "-Xcompiler", "-fPIC"] + (["-DBAM_PROFILE"] if profile else []) + [
           "-I" + os.path.join(ROOT, "include"), "-I" + CSRC, "-o", lib + ".tmp"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode == 0:
        os.replace(lib + ".tmp", lib)          # a reader never sees a half-written library
    if verbose or res.returncode != 0:
        print(res.stdout)
        print(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building " + os.path.basename(lib))
    return lib


def build_cpp_bench(force=False, name="array_bench"):
    """Compile tests/cpp/<name>.cu (a benchmark of the reference written against the drop-in C++
    headers) and link it against the in-tree library."""
    src = os.path.join(ROOT, "tests", "cpp", name + ".cu")
    exe = os.path.join(ROOT, "tests", "cpp", name)
    build_library()
    if not force and not _newer_than(exe, _deps() + [src, LIB]):
        return exe
    cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-I" + os.path.join(ROOT, "include"), "-o", exe, src, "-L" + HERE, "-lbam_b200",
           "-Xlinker", "-rpath", "-Xlinker", HERE]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        print(res.stdout)
        print(res.stderr)
        raise RuntimeError("nvcc failed building tests/cpp/" + name)
    return exe
