"""Build recipe for the CPU oracle (test infrastructure): g++ on oracle/thrml_oracle.cpp -> oracle/liboracle.so.

Floating-point contraction is switched off so that the deterministic f32 routines evaluate exactly the
operation sequence written in the source.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "thrml_oracle.cpp")
OUT = os.path.join(HERE, "liboracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", "-ffp-contract=off", "-fvisibility=hidden",
           "-o", OUT, SRC]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
