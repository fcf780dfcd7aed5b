"""CPU-side checks of the drop-in boundary: the library loads without a GPU and exports every
symbol that include/nvk_b200.h declares; the Python binding covers the same set."""
import ctypes
import pathlib
import re

import speaches_plus_b200 as sp

ROOT = pathlib.Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "nvk_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|size_t)\s+((?:nv_kernels|nvk_b200)_\w+)\s*\(", text)))


def test_header_declares_the_path_entry_points():
    syms = declared_symbols()
    for must in ("nv_kernels_nvfp4_gemv_bf16act", "nv_kernels_gemv_nvfp4_w4a16_dual_m1",
                 "nv_kernels_gemv_nvfp4_w4a16_silu_gate_up_in_m1", "nv_kernels_gemm_nvfp4_w4a16_mk_dual",
                 "nv_kernels_moe_grouped_fp4_gemv_m1_bf16", "nv_kernels_quantize_nvfp4_bf16",
                 "nv_kernels_moe_route_topk", "nv_kernels_gemv_bf16", "nv_kernels_capability"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    """The decode-path symbols come from libnvk_b200.so, the prefill GEMM's from libnvk_b200_prefill.so."""
    lib = ctypes.CDLL(str(sp.ffi.LIB_PATH))
    pre = ctypes.CDLL(str(sp.ffi.PREFILL_LIB_PATH))
    for name in declared_symbols():
        owner = pre if name in sp.ffi.PREFILL_SIGNATURES else lib
        assert hasattr(owner, name), f"{name} declared in include/nvk_b200.h but not exported"


def test_binding_matches_header():
    assert sorted(list(sp.ffi.SIGNATURES) + list(sp.ffi.PREFILL_SIGNATURES)) == declared_symbols()
    sp.ffi.lib()  # resolves every symbol, raises if one is missing
    sp.ffi.prefill_lib()


def test_header_compiles_as_c(tmp_path):
    import subprocess
    src = tmp_path / "t.c"
    src.write_text('#include "nvk_b200.h"\nint main(void){return 0;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), "-c", str(src), "-o",
                    str(tmp_path / "t.o")], check=True)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import pytest
    monkeypatch.setattr(sp.ffi, "_lib", None)
    monkeypatch.setattr(sp.ffi, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        sp.ffi.lib()


def declared_prototypes():
    """name -> list of parameter kinds ('ptr', 'int', 'i64', 'float', 'size_t') parsed from the header."""
    text = (ROOT / "include" / "nvk_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for name, params in re.findall(r"\b(?:int|size_t)\s+((?:nv_kernels|nvk_b200)_\w+)\s*\(([^)]*)\)\s*;", text):
        kinds = []
        for prm in (q.strip() for q in params.split(",")):
            if prm in ("", "void"):
                continue
            if "*" in prm:
                kinds.append("ptr")
            elif re.match(r"(const\s+)?(long long|int64_t)\b", prm):
                kinds.append("i64")
            elif re.match(r"(const\s+)?size_t\b", prm):
                kinds.append("size_t")
            elif re.match(r"(const\s+)?float\b", prm):
                kinds.append("float")
            elif re.match(r"(const\s+)?(int|int32_t|unsigned)\b", prm):
                kinds.append("int")
            else:
                raise AssertionError(f"{name}: parameter type not understood: {prm!r}")
        out[name] = kinds
    return out


def test_binding_argument_types_match_the_header():
    """Every ctypes signature has the header's parameter count and kinds, in order: a drifted binding
    would pass garbage through the C ABI without any error."""
    kind = {ctypes.c_void_p: "ptr", ctypes.c_int: "int", ctypes.c_uint: "int", ctypes.c_float: "float",
            ctypes.c_size_t: "size_t", ctypes.c_longlong: "i64"}
    protos = declared_prototypes()
    sigs = dict(sp.ffi.SIGNATURES)
    sigs.update(sp.ffi.PREFILL_SIGNATURES)
    assert sorted(protos) == sorted(sigs)
    for name, argtypes in sigs.items():
        assert [kind[a] for a in argtypes] == protos[name], name


def test_header_prototypes_equal_the_reference_headers():
    """tests/golden/reference_prototypes.json holds what the reference's own header declares for these
    entry points (written by tests/golden/extract_reference_prototypes.py): same parameter kinds in
    the same order, so an existing caller binds to this library unchanged."""
    import json
    ref = json.loads((ROOT / "tests" / "golden" / "reference_prototypes.json").read_text())["prototypes"]
    mine = declared_prototypes()
    shared = sorted(n for n in mine if n.startswith("nv_kernels_"))
    assert shared == sorted(ref)
    for name in shared:
        assert mine[name] == ref[name]["kinds"], name
