"""Builds oracle/_build/libitex_oracle.so from oracle/itex_oracle_c.c with gcc.

-ffp-contract=off keeps fp32 multiply and add separate; -mavx2 (no FMA, no AVX-512) is
the widest ISA assumed of the host that runs the CPU baseline.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build", "libitex_oracle.so")


def build(force=False):
    src = os.path.join(HERE, "itex_oracle_c.c")
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(src):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = ["gcc", "-O3", "-mavx2", "-fopenmp", "-ffp-contract=off", "-fno-math-errno", "-shared", "-fPIC",
           "-fvisibility=hidden", "-o", OUT, src, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
