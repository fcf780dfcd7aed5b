"""Build the CPU oracle (test infrastructure, not product) into oracle/libnvfp4_oracle.so.

The reference implementation of this path is Rust; no Rust toolchain exists where
this runs, so there is no `oracle/_ref` build of the reference itself -- the C
restatement in nvfp4_oracle.c is the only oracle, pinned by the reference's own
known-answer tests restated under tests/.
"""
import pathlib
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
SRC = HERE / "nvfp4_oracle.c"
OUT = HERE / "libnvfp4_oracle.so"


def build(force: bool = False) -> pathlib.Path:
    if not force and OUT.exists() and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    cmd = ["gcc", "-O2", "-fopenmp", "-fno-fast-math", "-ffp-contract=off", "-shared", "-fPIC",
           "-o", str(OUT), str(SRC), "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
