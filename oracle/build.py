"""Compiles oracle/cpu_ref.c (test / benchmark infrastructure) into
oracle/_build/: an AVX2+FMA build and a plain one; cpu_ref.py loads the first
the host CPU supports.  The reference itself (Metal kernels, XLA, Bazel) cannot
be compiled here, so there is no oracle/_ref."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")
VARIANTS = {"cpu_ref_avx2.so": ["-mavx2", "-mfma"], "cpu_ref_base.so": []}


def build(force=False):
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(HERE, "cpu_ref.c")
    for name, extra in VARIANTS.items():
        dst = os.path.join(OUT, name)
        if not force and os.path.exists(dst) and os.path.getmtime(dst) >= os.path.getmtime(src):
            continue
        subprocess.run(["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-ffp-contract=off", *extra, src, "-o", dst,
                        "-lm"], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
