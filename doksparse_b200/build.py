"""In-tree build of libdoksparse.so: nvcc, -gencode arch=compute_100a,code=sm_100a (see csrc/Makefile)."""
import os
import subprocess

_CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")


def build(verbose=False):
    cmd = ["make", "-C", _CSRC, "-j4"]
    out = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or out.returncode != 0:
        print(out.stdout)
    if out.returncode != 0:
        raise RuntimeError("building libdoksparse.so failed")
    return os.path.join(_CSRC, "libdoksparse.so")


if __name__ == "__main__":
    print(build(verbose=True))
