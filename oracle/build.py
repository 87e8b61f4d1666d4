"""Build recipe of the CPU checker (test infrastructure, not the product).

`build()` compiles oracle/oracle.cpp into oracle/_build/liboracle.so with
`g++ -O2 -ffp-contract=off -fopenmp`.  The reference implementation itself is
Rust and no Rust toolchain exists where this runs, so there is no reference
binary to build; the checker is the restatement in oracle.cpp.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")  # the restatement compiled here: not a build of the reference itself
LIB = os.path.join(OUT_DIR, "liboracle.so")
SRC = os.path.join(HERE, "oracle.cpp")
DEPS = [SRC, os.path.join(HERE, "..", "include", "ruai_b200.h"), os.path.join(HERE, "..", "include", "ruai_b200_synth.h")]


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in DEPS)


def build(force=False):
    if not force and not needs_build():
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-O2", "-ffp-contract=off", "-fopenmp", "-std=c++17", "-shared", "-fPIC",
           "-fvisibility=hidden", "-o", LIB, SRC]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
