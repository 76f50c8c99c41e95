"""Builds oracle/_ref/libref_nerf_kernels.so: the reference's own training-step kernels (src/testbed_nerf.cu, included where it
lies in a reference checkout) behind extern "C" launchers (oracle/ref_kernels/ref_nerf_kernels.cu).  Test infrastructure: the
GPU tests run these kernels and this repository's kernels on the same inputs.  Needs a reference checkout (next to this
repository or named by NEUS2_REFERENCE) and nlohmann/json.hpp; without them nothing is built and the tests skip.

The translation unit defines many Testbed member functions that call into parts of the reference that are not compiled here
(GUI, other primitives): the shared object is linked with those symbols left undefined, which is harmless as long as only
the launchers are called.

Compiled with -fmad=false: the comparison is about the sequence of arithmetic operations, and this repository's ray marcher and
its CPU restatement are built without multiply-add contraction so that they agree bit for bit with each other.  (The
reference's own build lets the compiler contract, which moves last bits of ray directions and sample positions; the per-ray
sample counts of the test scenes are the same either way.)"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref", "libref_nerf_kernels.so")


def build(verbose=False):
    sys.path.insert(0, ROOT)
    from neus2_b200 import build as B
    ref, flags = B.reference_root(), B.header_include_flags(with_reference=True)
    if ref is None or flags is None:
        return None
    src = os.path.join(HERE, "ref_kernels", "ref_nerf_kernels.cu")
    deps = [src, os.path.abspath(__file__), os.path.join(ref, "src", "testbed_nerf.cu")] + [os.path.join(d, f) for d, _, fs in os.walk(os.path.join(ROOT, "include")) for f in fs]
    if os.path.exists(OUT) and os.path.getmtime(OUT) > max(os.path.getmtime(p) for p in deps):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    tmp = os.path.dirname(OUT)
    obj, stubs_c, stubs_o = os.path.join(tmp, "ref_nerf_kernels.o"), os.path.join(tmp, "stubs.c"), os.path.join(tmp, "stubs.o")

    def run(cmd):
        r = subprocess.run(cmd, capture_output=not verbose, text=True)
        if r.returncode != 0:
            raise RuntimeError("building libref_nerf_kernels.so failed (%s):\n%s%s" % (" ".join(cmd[:3]), r.stdout or "", r.stderr or ""))
        return r

    run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17", "--extended-lambda", "--expt-relaxed-constexpr", "-w",
         '-DNGP_VERSION="1.0dev"', "-DTCNN_MIN_GPU_ARCH=100", "-fmad=false", "-Xcompiler", "-fPIC", "-I" + ref] + flags + ["-c", src, "-o", obj])
    link = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", OUT, obj, "-L" + os.path.join(ROOT, "neus2_b200", "_build"), "-lneus2b",
            "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../neus2_b200/_build"]
    run(link)
    # The reference's functions this object refers to but that live in sources not compiled here (mesh extraction, dataset
    # loader, snapshot code: none of them is reached from the launchers) get a definition that aborts, so that the library
    # loads with immediate binding (ctypes always binds immediately).
    names = subprocess.run(["nm", "-D", "-u", OUT], capture_output=True, text=True, check=True).stdout.split()
    missing = sorted(n for n in names if n.startswith("_ZN3ngp"))
    with open(stubs_c, "w") as f:
        f.write("#include <stdio.h>\n#include <stdlib.h>\n")
        for n in missing:
            f.write('void %s(void) { fputs("libref_nerf_kernels: %s is not part of this build\\n", stderr); abort(); }\n' % (n, n))
    run(["gcc", "-fPIC", "-c", stubs_c, "-o", stubs_o])
    run(link[:6] + [stubs_o] + link[6:])
    return OUT


TESTBED_OUT = os.path.join(HERE, "_ref", "libref_testbed.so")
BENIGN_STUBS = {"_ZN3ngp13CudaSurface2D4freeEv"}  # CudaSurface2D::free() of a surface that holds nothing
TESTBED_SOURCES = ["src/testbed.cu", "src/testbed_nerf.cu", "src/marching_cubes.cu", "src/nerf_loader.cu", "src/common_device.cu", "src/camera_path.cu",
                   "src/triangle_bvh.cu", "src/thread_pool.cpp", "src/tinyobj_loader_wrapper.cpp"]


def build_testbed(verbose=False):
    """oracle/_ref/libref_testbed.so: the reference's headless training loop (its own sources, compiled where they lie, with the
    reference's default compiler settings) behind ref_testbed_train (oracle/ref_kernels/ref_testbed.cu)."""
    sys.path.insert(0, ROOT)
    from neus2_b200 import build as B
    ref, flags = B.reference_root(), B.header_include_flags(with_reference=True)
    if ref is None or flags is None:
        return None
    wrapper = os.path.join(HERE, "ref_kernels", "ref_testbed.cu")
    srcs = [os.path.join(ref, s) for s in TESTBED_SOURCES] + [wrapper]
    deps = srcs + [os.path.abspath(__file__)] + [os.path.join(d, f) for d, _, fs in os.walk(os.path.join(ROOT, "include")) for f in fs]
    if os.path.exists(TESTBED_OUT) and os.path.getmtime(TESTBED_OUT) > max(os.path.getmtime(p) for p in deps):
        return TESTBED_OUT
    tmp = os.path.join(HERE, "_ref", "tb")
    os.makedirs(tmp, exist_ok=True)
    base = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17", "--extended-lambda", "--expt-relaxed-constexpr", "-w",
            '-DNGP_VERSION="1.0dev"', "-DTCNN_MIN_GPU_ARCH=100", "-Xcompiler", "-fPIC", "-I" + os.path.join(ref, "dependencies", "tinyobjloader")] + flags
    jobs, objs = [], []
    for s in srcs:
        o = os.path.join(tmp, os.path.splitext(os.path.basename(s))[0] + ".o")
        objs.append(o)
        jobs.append((s, subprocess.Popen(base + ["-x", "cu", "-c", s, "-o", o], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, p in jobs:
        log, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("building libref_testbed.so failed at %s:\n%s" % (s, log[-4000:]))
    link = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", TESTBED_OUT] + objs + [
        "-L" + os.path.join(ROOT, "neus2_b200", "_build"), "-lneus2b", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../neus2_b200/_build"]

    def run(cmd):
        r = subprocess.run(cmd, capture_output=not verbose, text=True)
        if r.returncode != 0:
            raise RuntimeError("building libref_testbed.so failed (%s):\n%s%s" % (" ".join(cmd[:3]), r.stdout or "", r.stderr or ""))

    run(link)
    # what the headless NeRF path never reaches (GUI, render buffer, other primitives, EXR): functions that abort, and one
    # vtable (data, so that the library loads with immediate binding)
    names = subprocess.run(["nm", "-D", "-u", TESTBED_OUT], capture_output=True, text=True, check=True).stdout.split()
    missing = sorted(n for n in names if n.startswith("_ZN3ngp") or n.startswith("_ZNK3ngp"))
    vtables = sorted(n for n in names if n.startswith("_ZTVN3ngp"))
    stubs_c, stubs_o = os.path.join(tmp, "stubs.c"), os.path.join(tmp, "stubs.o")
    with open(stubs_c, "w") as f:
        f.write("#include <stdio.h>\n#include <stdlib.h>\n")
        for n in missing:
            if n in BENIGN_STUBS:  # reached by destructors of members that were never filled
                f.write("void %s(void) {}\n" % n)
            else:
                f.write('void %s(void) { fputs("libref_testbed: %s is not part of this build\\n", stderr); abort(); }\n' % (n, n))
        for n in vtables:
            f.write("void* %s[16] = {0};\n" % n)
    run(["gcc", "-fPIC", "-c", stubs_c, "-o", stubs_o])
    run(link[:6] + [stubs_o] + link[6:])
    return TESTBED_OUT


if __name__ == "__main__":
    print(build(verbose=True))
    print(build_testbed(verbose=True))
