"""Compile the CUDA sources under csrc/ into libnvk_b200.so (sm_100a only), in-tree.

    python speaches-plus_b200/build.py [--force] [--verbose]

Two plain C-ABI shared objects (see include/nvk_b200.h), each linking the CUDA runtime statically:
libnvk_b200.so (csrc/: every decode-path kernel) and libnvk_b200_prefill.so (csrc_prefill/: the
prefill block-scaled GEMM, built from CUTLASS headers when they are found).  The split keeps the
CUTLASS-derived kernel out of multi-GPU runs, which only need the first library.
"""
from __future__ import annotations

import pathlib
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
CSRC_PREFILL = HERE / "csrc_prefill"
OBJ = HERE / "build"
LIB = HERE / "libnvk_b200.so"
LIB_PREFILL = HERE / "libnvk_b200_prefill.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def sources():
    return sorted(CSRC.glob("*.cu"))


def cutlass_include_dirs() -> list[str]:
    """CUTLASS/CuTe headers for the prefill GEMM: $NVK_CUTLASS_DIR, or a tree vendored inside an
    installed Python package.  Empty when none is found (the prefill entry points then refuse)."""
    import importlib.util
    import os
    cands = []
    if os.environ.get("NVK_CUTLASS_DIR"):
        cands.append(pathlib.Path(os.environ["NVK_CUTLASS_DIR"]))
    for pkg, rel in (("flashinfer", "data/cutlass"), ("tilelang", "3rdparty/cutlass")):
        spec = importlib.util.find_spec(pkg)
        if spec and spec.origin:
            cands.append(pathlib.Path(spec.origin).parent / rel)
    for root in cands:
        if (root / "include" / "cutlass" / "gemm" / "collective" / "builders" / "sm100_blockscaled_umma_builder.inl").exists():
            dirs = [str(root / "include")]
            if (root / "tools" / "util" / "include").exists():
                dirs.append(str(root / "tools" / "util" / "include"))
            return dirs
    return []


def _newest_header() -> float:
    return max([f.stat().st_mtime for f in CSRC.glob("*.cuh")] + [0.0])


def _newest_dep() -> float:
    return max(f.stat().st_mtime for f in list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) +
               list(CSRC_PREFILL.glob("*.cu")))


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    have_prefill_src = CSRC_PREFILL.exists() and any(CSRC_PREFILL.glob("*.cu"))
    up_to_date = LIB.exists() and LIB.stat().st_mtime >= _newest_dep()
    if have_prefill_src:
        up_to_date = up_to_date and LIB_PREFILL.exists() and LIB_PREFILL.stat().st_mtime >= _newest_dep()
    if not force and up_to_date:
        return LIB
    OBJ.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []
    cutlass = cutlass_include_dirs()

    def compile_one(src: pathlib.Path) -> pathlib.Path:
        obj = OBJ / (src.stem + ".o")
        per_file = []
        if src.parent == CSRC_PREFILL and cutlass:
            per_file = ["--expt-relaxed-constexpr", "-DNVK_HAVE_CUTLASS", *[f"-I{d}" for d in cutlass]]
        if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, _newest_header()):
            return obj
        cmd = ["nvcc", *NVCC_FLAGS, *extra, *per_file, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    prefill_srcs = sorted(CSRC_PREFILL.glob("*.cu")) if have_prefill_src else []
    with ThreadPoolExecutor(max_workers=8) as ex:
        all_objs = list(ex.map(compile_one, sources() + prefill_srcs))
    objs, pre_objs = all_objs[:len(sources())], all_objs[len(sources()):]
    link = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
    subprocess.run([*link, "-o", str(LIB), *map(str, objs)], check=True)
    if pre_objs:
        subprocess.run([*link, "-o", str(LIB_PREFILL), *map(str, pre_objs)], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
