"""Writes tests/golden/reference_prototypes.json: for every entry point of the NVFP4 linear path, the
parameter kinds (pointer / int / 64-bit int / float / size_t, in order) and the parameter names that
the reference's C header declares.  The drop-in claim is that include/nvk_b200.h declares the same
prototypes; tests/test_abi_load.py compares the two.

Run where the reference tree is available:
    python tests/golden/extract_reference_prototypes.py /path/to/reference
"""
import json
import pathlib
import re
import sys

HEADER = "rust/crates/nv-kernels/include/nv_kernels.h"


def kind_of(param: str) -> str:
    if "*" in param:
        return "ptr"
    if re.match(r"(const\s+)?(long long|int64_t)\b", param):
        return "i64"
    if re.match(r"(const\s+)?size_t\b", param):
        return "size_t"
    if re.match(r"(const\s+)?float\b", param):
        return "float"
    if re.match(r"(const\s+)?(int|int32_t|unsigned|uint32_t)\b", param):
        return "int"
    raise ValueError(f"parameter type not understood: {param!r}")


def prototypes(text: str) -> dict:
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    out = {}
    for name, params in re.findall(r"\bint\s+(nv_kernels_\w+)\s*\(([^)]*)\)\s*;", text):
        plist = [re.sub(r"\s+", " ", q.strip()) for q in params.split(",") if q.strip() not in ("", "void")]
        out[name] = {"kinds": [kind_of(q) for q in plist],
                     "names": [re.findall(r"(\w+)\s*$", q)[0] for q in plist]}
    return out


if __name__ == "__main__":
    ref_root = pathlib.Path(sys.argv[1])
    repo = pathlib.Path(__file__).resolve().parents[2]
    mine = (repo / "include" / "nvk_b200.h").read_text()
    wanted = sorted(set(re.findall(r"\b(nv_kernels_\w+)\s*\(", re.sub(r"/\*.*?\*/", "", mine, flags=re.S))))
    ref = prototypes((ref_root / HEADER).read_text())
    missing = [n for n in wanted if n not in ref]
    if missing:
        raise SystemExit(f"not declared by the reference header: {missing}")
    out = {"source": HEADER, "prototypes": {n: ref[n] for n in wanted}}
    path = pathlib.Path(__file__).with_name("reference_prototypes.json")
    path.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    print(path, len(wanted), "prototypes")
