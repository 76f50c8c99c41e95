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


if __name__ == "__main__":
    print(build(verbose=True))
