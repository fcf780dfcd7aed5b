"""Build the host emulation of the CUDA library: the product's own .cu sources compiled as C++ with
-DNVK_EMU against tests/emu (see cuda_emu.h).  Output: tests/emu/build/libnvk_b200_emu.so, loaded
only by the tests.

    python tests/emu/build_emu.py [--force] [--sanitize] [--tsan]

--sanitize builds tests/emu/build/libnvk_b200_emu_san.so with -fsanitize=alignment,shift,
signed-integer-overflow,bounds (no recovery): a misaligned vector load or store in a kernel -- a fault on
the GPU -- aborts the run.  Use it with
    NVK_EMU_LIB=tests/emu/build/libnvk_b200_emu_san.so python -m pytest tests -m gpu --emu

--tsan builds tests/emu/build/libnvk_b200_emu_tsan.so: a race checker.  The kernels are compiled with
-fsanitize=thread, every emulated CUDA thread is a ThreadSanitizer fiber, and the only ordering between
threads is what CUDA's barriers and launch boundaries give (see emu_rt.cpp).  Use it with
    LD_PRELOAD=$(gcc -print-file-name=libtsan.so) TSAN_OPTIONS=halt_on_error=1 \
    NVK_EMU_LIB=tests/emu/build/libnvk_b200_emu_tsan.so python -m pytest tests -m gpu --emu -p no:cacheprovider
"""
from __future__ import annotations

import pathlib
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = pathlib.Path(__file__).resolve().parent
ROOT = HERE.parents[1]
CSRC = ROOT / "speaches-plus_b200" / "csrc"
OUT_DIR = HERE / "build"
LIB = OUT_DIR / "libnvk_b200_emu.so"
# -O1: fast enough to run, quick to compile; no fast-math and no FMA contraction, so float
# expressions round the way the kernels' source says (nvcc is likewise given no fast-math).
CXX_FLAGS = ["-std=c++17", "-O1", "-g", "-fPIC", "-fno-fast-math", "-ffp-contract=off", "-DNVK_EMU", "-Wall",
             "-Wno-unknown-pragmas", "-Wno-unused-function", "-Wno-unused-variable", "-Wno-sign-compare",
             f"-I{HERE / 'shim'}", f"-I{HERE}", f"-I{CSRC}"]


def _deps_mtime() -> float:
    files = (list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(HERE.glob("*.h")) + list(HERE.glob("*.cpp")) +
             list(HERE.glob("*.cu")))
    return max(f.stat().st_mtime for f in files)


SAN_FLAGS = ["-fsanitize=alignment,shift,signed-integer-overflow,bounds", "-fno-sanitize-recover=all"]


def build(force: bool = False, sanitize: bool = False, tsan: bool = False) -> pathlib.Path:
    lib = OUT_DIR / ("libnvk_b200_emu_tsan.so" if tsan else "libnvk_b200_emu_san.so") if (sanitize or tsan) else LIB
    if not force and lib.exists() and lib.stat().st_mtime >= _deps_mtime():
        return lib
    OUT_DIR.mkdir(exist_ok=True)
    newest_header = max(f.stat().st_mtime for f in list(CSRC.glob("*.cuh")) + list(HERE.glob("*.h")))

    def compile_one(src: pathlib.Path) -> pathlib.Path:
        obj = OUT_DIR / (src.stem + (".tsan.o" if tsan else ".san.o" if sanitize else ".emu.o"))
        if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, newest_header):
            return obj
        lang = ["-x", "c++"] if src.suffix == ".cu" else []
        extra = list(SAN_FLAGS) if sanitize else []
        if tsan:   # kernels instrumented; the runtime only told that fibers exist
            extra = ["-DNVK_EMU_TSAN"] + ([] if src.name == "emu_rt.cpp" else ["-fsanitize=thread"])
        r = subprocess.run(["g++", *CXX_FLAGS, *extra, *lang, "-c", str(src), "-o", str(obj)],
                           capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError(f"emulation build failed on {src.name}")
        return obj

    srcs = sorted(CSRC.glob("*.cu")) + [HERE / "emu_rt.cpp"]
    if tsan:
        srcs.append(HERE / "selftest_kernels.cu")   # a barrier left out on purpose, for the checker's own test
    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, srcs))
    libs = ["-lubsan"] if sanitize else ["-ltsan"] if tsan else []
    subprocess.run(["g++", "-shared", "-o", str(lib), *map(str, objs), "-lpthread", *libs], check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, sanitize="--sanitize" in sys.argv, tsan="--tsan" in sys.argv))
