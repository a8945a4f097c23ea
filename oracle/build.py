"""Builds the test-only CPU checkers.

  oracle/libdsa_oracle.so      the C restatement in dsa_oracle.c (always)
  oracle/_ref/libdsa_ref.so    the reference's own host.cc compiled through ref_wrap.cu
                               (only when a checkout of the reference is present; the sources
                               are compiled from where they lie and never copied)

The reference checkout is looked for in $DSA_REFERENCE_ROOT, else in a directory named
`reference` beside the repository.  Nothing here is part of the shipped library.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libdsa_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libdsa_ref.so")


def reference_root():
    root = os.environ.get("DSA_REFERENCE_ROOT")
    if not root:
        root = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    lab = os.path.join(root, "opus_attn", "dsa_v32")
    return lab if os.path.isfile(os.path.join(lab, "common", "host.cc")) else None


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "dsa_oracle.c")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    cmd = ["gcc", "-O3", "-std=gnu11", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-pthread",
           "-o", ORACLE_SO, src, "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_ref(force=False):
    lab = reference_root()
    if lab is None:
        return REF_SO if os.path.exists(REF_SO) else None
    src = os.path.join(HERE, "ref_wrap.cu")
    shim = os.path.join(HERE, "ref_shim")
    deps = [src, os.path.join(shim, "opus", "hip_minimal.hpp"), os.path.join(lab, "common", "host.cc"),
            os.path.join(lab, "common", "defs.h")]
    if not force and _newer(REF_SO, deps):
        return REF_SO
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = [nvcc, "-std=c++20", "-O3", "-arch=sm_100a", "-Xcompiler", "-pthread,-fPIC", "-shared",
           "-D_BitInt(n)=char", "-DMLA_DECODE_ARCH_GFX950", "-I" + shim, "-I" + lab,
           "-I" + os.path.join(lab, "common"), "-o", REF_SO, src]
    subprocess.check_call(cmd)
    return REF_SO


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
