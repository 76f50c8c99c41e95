"""Builds libneus2b.so (sm_100a) in-tree with nvcc via csrc/Makefile.  `python -m neus2_b200.build`."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "libneus2b.so")


def build(verbose=False, extra=""):
    env = dict(os.environ)
    cmd = ["make", "-C", os.path.join(HERE, "csrc"), "-j8"]
    if extra:
        cmd.append("EXTRA=" + extra)
    r = subprocess.run(cmd, env=env, capture_output=not verbose, text=True)
    if r.returncode != 0:
        raise RuntimeError("building libneus2b.so failed:\n" + (r.stdout or "") + (r.stderr or ""))
    return LIB


def reference_root():
    """A checkout of the reference next to this repository (or named by NEUS2_REFERENCE), or None.  Only the build-time
    compile checks and the C++ test that instantiates the reference's NerfNetwork look at it; nothing at run time does."""
    for cand in (os.environ.get("NEUS2_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "include", "neural-graphics-primitives", "nerf_network.h")):
            return cand
    return None


def nlohmann_include_dir():
    """A directory that holds nlohmann/json.hpp (include/json/json.hpp forwards to it), or None."""
    import glob
    import sysconfig
    cands = [os.environ.get("NLOHMANN_JSON_INCLUDE"), "/usr/include", "/usr/local/include"]
    site = sysconfig.get_paths().get("purelib")
    if site:
        cands += [os.path.join(site, "include", "cudnn_frontend", "thirdparty")]
        cands += [os.path.dirname(os.path.dirname(p)) for p in glob.glob(os.path.join(site, "**", "nlohmann", "json.hpp"), recursive=True)]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "nlohmann", "json.hpp")):
            return c
    return None


def header_include_flags(with_reference=False):
    """nvcc -I flags for a translation unit that includes <tiny-cuda-nn/...> (and, with_reference, the reference's own
    headers and the third-party trees it vendors)."""
    root = os.path.dirname(HERE)
    nl = nlohmann_include_dir()
    if nl is None:
        return None
    flags = ["-I" + os.path.join(root, "include"), "-I" + nl]
    if with_reference:
        ref = reference_root()
        if ref is None:
            return None
        flags += ["-I" + os.path.join(ref, "include")] + ["-I" + os.path.join(ref, "dependencies", d) for d in ("", "eigen", "filesystem", "tinylogger")]
    return flags


if __name__ == "__main__":
    print(build(verbose=True))
