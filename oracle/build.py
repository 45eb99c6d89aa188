"""Build recipe for the CPU oracle (test infrastructure, never part of the shipped library).

Produces, next to this file:
  liboracle.so                    the C++ restatement in vearo_oracle.cpp
  _ref/libvearo_ref_matmul.so     the reference's own 4x8 AVX2 matmul block, assembled from the
                                  reference source where it lies (only when the reference tree is
                                  present; the built file travels with the repository snapshot).
Nothing of the reference is copied: the assembler reads the file in place.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# where a checkout of the reference lives (VEARO_REFERENCE_DIR overrides); absent: the assembly kernel is simply not built
REF_DIR = os.environ.get("VEARO_REFERENCE_DIR", "/root/reference")
REF_ASM = os.path.join(REF_DIR, "crates/vearo-backend-cpu/src/asm/x86_64/matmul.s")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build(verbose=False):
    src = os.path.join(HERE, "vearo_oracle.cpp")
    out = os.path.join(HERE, "liboracle.so")
    if _stale(out, [src]):
        cmd = ["g++", "-std=c++17", "-O3", "-mavx2", "-mfma", "-ffp-contract=off", "-fno-fast-math",
               "-shared", "-fPIC", "-pthread", src, "-o", out]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    ref_out = os.path.join(HERE, "_ref", "libvearo_ref_matmul.so")
    if os.path.exists(REF_ASM) and _stale(ref_out, [REF_ASM]):
        os.makedirs(os.path.dirname(ref_out), exist_ok=True)
        cmd = ["gcc", "-shared", "-fPIC", "-Wl,-z,noexecstack", "-x", "assembler", REF_ASM, "-o", ref_out]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    build(verbose=True)
    print("ok", file=sys.stderr)
