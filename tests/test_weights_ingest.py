"""On-disk NVFP4 ingestion (host side, no GPU): safetensors shards, quantization config, tensor-name
layouts, global-scale conventions, host swizzle, fused pairs, small-module expansion.  The cases
follow the reference's own tests (rust/crates/nv-weights/src/lib.rs:744-1015) and loader rules
(rust/crates/nv-layers/src/moe.rs:574-992); byte layouts are checked against the oracle."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import ref
from speaches_plus_b200 import weights as W


def write_safetensors(path, tensors: dict, metadata=None):
    """tensors: name -> (dtype tag, shape, bytes-like).  Minimal writer of the public format."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, (dtype, shape, payload) in tensors.items():
        payload = bytes(payload)
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + len(payload)]}
        blobs.append(payload)
        off += len(payload)
    hdr = json.dumps(header).encode()
    hdr += b" " * (-len(hdr) % 8)
    with open(path, "wb") as f:
        f.write(len(hdr).to_bytes(8, "little"))
        f.write(hdr)
        for b in blobs:
            f.write(b)
    return path


def f32(*v):
    return np.asarray(v, np.float32).tobytes()


def make_module(rng, n, k, stored_global=None):
    w = ref.f32_to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    g = np.float32(ref.weight_global(ref.bf16_to_f32(w))) if stored_global is None else np.float32(stored_global)
    packed, lin = ref.quantize_rows_bf16(w, float(g))
    return packed, lin, g


def ct_tensors(prefix, packed, lin, g, gx=None):
    """compressed-tensors names: the file stores the quantization multipliers themselves."""
    t = {f"{prefix}.weight_packed": ("U8", packed.shape, packed.tobytes()),
         f"{prefix}.weight_scale": ("F8_E4M3", lin.shape, lin.tobytes()),
         f"{prefix}.weight_global_scale": ("F32", (1,), f32(g))}
    if gx is not None:
        t[f"{prefix}.input_global_scale"] = ("F32", (1,), f32(gx))
    return t


def modelopt_tensors(prefix, packed, lin, g, gx=None):
    """ModelOpt names: the file stores the dequantization multipliers (reciprocals)."""
    t = {f"{prefix}.weight": ("U8", packed.shape, packed.tobytes()),
         f"{prefix}.weight_scale": ("F8_E4M3", lin.shape, lin.tobytes()),
         f"{prefix}.weight_scale_2": ("F32", (), f32(np.float32(1.0) / np.float32(g)))}
    if gx is not None:
        t[f"{prefix}.input_scale"] = ("F32", (), f32(np.float32(1.0) / np.float32(gx)))
    return t


# ---- safetensors shards ---------------------------------------------------------------------
def test_typed_reads_and_raw_bytes(tmp_path):
    i64 = np.array([1, -2, 3_000_000_000], "<i8")
    bf = ref.f32_to_bf16(np.array([1.5, -2.0, 0.1], np.float32))
    p = write_safetensors(tmp_path / "m.safetensors", {
        "ids": ("I64", (3,), i64.tobytes()),
        "w": ("BF16", (1, 3), bf.tobytes()),
        "flag": ("BOOL", (2,), bytes([1, 0])),
        "fp8": ("F8_E4M3", (4,), bytes([0x38, 0x40, 0, 0x7E])),
    }, metadata={"format": "pt"})
    wl = W.WeightLoader.open_file(p)
    assert wl.names() == ["flag", "fp8", "ids", "w"]
    assert wl.has("w") and not wl.has("nope")
    assert wl.shape_of("w") == [1, 3] and wl.shape_of("nope") is None
    assert torch.equal(wl.get("ids", torch.int64), torch.tensor(i64))              # i64 round trip
    assert wl.get("w").dtype == torch.bfloat16
    assert np.array_equal(wl.get("w", torch.float32).numpy().ravel(), ref.bf16_to_f32(bf))
    assert wl.dtype_of("flag") == "U8" and wl.get("flag").dtype == torch.uint8     # bool reads as u8
    assert wl.get("flag", torch.float32).tolist() == [1.0, 0.0]
    assert bytes(wl.raw_bytes("fp8")) == bytes([0x38, 0x40, 0, 0x7E])              # byte-only dtype
    assert wl.dtype_of("fp8") is None and wl.st_dtype_of("fp8") == "F8_E4M3"
    with pytest.raises(W.WeightError, match="unsupported source dtype"):
        wl.get("fp8")
    with pytest.raises(W.WeightError, match="tensor not found: nope"):
        wl.raw_bytes("nope")


def test_bad_headers_are_refused(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(W.WeightError, match="too short"):
        W.WeightLoader.open_file(p)
    p = tmp_path / "long.safetensors"
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(W.WeightError, match="exceeds the file"):
        W.WeightLoader.open_file(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p = tmp_path / "size.safetensors"
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + bytes(8))
    with pytest.raises(W.WeightError, match="bad data_offsets"):
        W.WeightLoader.open_file(p)


def test_open_dir_with_index_without_index_and_lfs_pointer(tmp_path):
    d = tmp_path / "ckpt"
    d.mkdir()
    write_safetensors(d / "a.safetensors", {"x": ("F32", (1,), f32(1.0))})
    write_safetensors(d / "b.safetensors", {"y": ("F32", (1,), f32(2.0))})
    wl = W.WeightLoader.open_dir(d)
    assert wl.names() == ["x", "y"] and float(wl.scalar_f32("y")) == 2.0
    # an index file decides which shard serves which name; a git-lfs pointer shard is skipped
    (d / "c.safetensors").write_bytes(b"version https://git-lfs.github.com/spec/v1\noid sha256:0\nsize 1\n")
    (d / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "a.safetensors", "y": "b.safetensors", "z": "c.safetensors"}}))
    wl = W.WeightLoader.open_dir(d)
    assert wl.names() == ["x", "y"]
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"q": "a.safetensors"}}))
    with pytest.raises(W.WeightError, match="missing tensor q"):
        W.WeightLoader.open_dir(d)
    # without an index, the same name in two shards is an error
    os.remove(d / "model.safetensors.index.json")
    os.remove(d / "c.safetensors")
    write_safetensors(d / "b.safetensors", {"x": ("F32", (1,), f32(3.0))})
    with pytest.raises(W.WeightError, match="duplicate tensor x"):
        W.WeightLoader.open_dir(d)
    e = tmp_path / "empty"
    e.mkdir()
    with pytest.raises(W.WeightError, match="no .safetensors files"):
        W.WeightLoader.open_dir(e)
    with pytest.raises(W.WeightError, match="not a directory"):
        W.WeightLoader.open_dir(tmp_path / "missing")


# ---- quantization config (rust/crates/nv-weights/src/lib.rs:912-998) ----------------------------
def _cfg(qc):
    return json.dumps({"quantization_config": qc})


def test_nvfp4_group_size_16_is_accepted():
    q = W.QuantizationConfig.from_hf_json_str(_cfg({
        "quant_method": "compressed-tensors",
        "config_groups": {"group_0": {"weights": {"num_bits": 4, "type": "float", "group_size": 16}}}}))
    assert q.scheme is W.QuantScheme.NVFP4 and q.group_size == 16 and q.effective_group_size() == 16


def test_nvfp4_without_group_size_uses_the_implemented_one():
    q = W.QuantizationConfig.from_hf_json_str(_cfg({"quant_method": "modelopt", "quant_algo": "NVFP4"}))
    assert q.scheme is W.QuantScheme.NVFP4 and q.group_size is None and q.effective_group_size() == 16


def test_nvfp4_group_size_32_is_rejected():
    with pytest.raises(W.WeightError) as e:
        W.QuantizationConfig.from_hf_json_str(_cfg({
            "quant_method": "compressed-tensors",
            "config_groups": {"group_0": {"weights": {"num_bits": 4, "type": "float", "group_size": 32}}}}))
    assert "32" in str(e.value) and "MXFP4" in str(e.value) and "16" in str(e.value)


def test_fp8_group_size_is_rejected_and_plain_fp8_loads():
    with pytest.raises(W.WeightError, match="per output row"):
        W.QuantizationConfig.from_hf_json_str(_cfg({
            "quant_method": "compressed-tensors",
            "config_groups": {"group_0": {"weights": {"num_bits": 8, "type": "float", "group_size": 128}}}}))
    with pytest.raises(W.WeightError):
        W.QuantizationConfig.from_hf_json_str(_cfg({
            "quant_method": "modelopt", "quant_algo": "FP8",
            "config_groups": {"group_0": {"weights": {"group_size": 128}}}}))
    q = W.QuantizationConfig.from_hf_json_str(_cfg({
        "quant_method": "compressed-tensors",
        "config_groups": {"group_0": {"weights": {"num_bits": 8, "type": "float"}}}, "ignore": ["lm_head"]}))
    assert q.scheme is W.QuantScheme.FP8_E4M3 and q.effective_group_size() is None
    assert q.is_module_ignored("lm_head") and not q.is_module_ignored("lm_head2")


def test_config_formats_and_ignore_patterns():
    assert W.QuantizationConfig.from_hf_json_str("{}").scheme is W.QuantScheme.NONE
    assert W.QuantizationConfig.from_hf_json_str(_cfg({"format": "nvfp4-pack-quantized"})).scheme is W.QuantScheme.NVFP4
    with pytest.raises(W.WeightError, match="must be an object"):
        W.QuantizationConfig.from_hf_json_str(_cfg([1]))
    q = W.QuantizationConfig.from_hf_value({"quant_method": "modelopt", "quant_algo": "nvfp4_awq",
                                            "ignored_modules": ["model.layers.0.*", "lm_head", 7]})
    assert q.scheme is W.QuantScheme.NVFP4 and q.ignored_modules == ["model.layers.0.*", "lm_head"]
    assert q.is_module_ignored("model.layers.0.mlp.gate") and not q.is_module_ignored("model.layers.1.mlp.gate")


# ---- layouts and scale conventions --------------------------------------------------------------
@pytest.mark.parametrize("rows,kb", [(128, 8), (256, 256), (300, 10), (1, 1), (129, 5)])
def test_host_swizzle_equals_the_oracle(rows, kb):
    rng = np.random.default_rng(rows * 1000 + kb)
    lin = rng.integers(0, 0x7F, (rows, kb), dtype=np.uint8)
    sw = W.swizzle_scales(lin, rows, kb)
    assert np.array_equal(sw, ref.swizzle_scales(lin, rows, kb))
    assert np.array_equal(W.unswizzle_scales(sw, rows, kb), lin)
    assert sw.size == ref.swizzled_len(rows, kb)


@pytest.mark.parametrize("layout", ["compressed-tensors", "modelopt"])
def test_module_read_applies_the_layouts_global_convention(tmp_path, layout):
    rng = np.random.default_rng(5)
    n, k = 256, 128
    packed, lin, g = make_module(rng, n, k)
    gx = np.float32(37.5)
    if layout == "modelopt":
        tensors, sfx = modelopt_tensors("m.q", packed, lin, g, gx), W.Nvfp4Suffixes.GEMMA_MODELOPT
    else:
        tensors, sfx = ct_tensors("m.q", packed, lin, g, gx), W.Nvfp4Suffixes.QWEN_COMPRESSED_TENSORS
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", tensors))
    parts = W.read_nvfp4_module(wl, "m.q", n, k, sfx)
    assert np.array_equal(parts.packed, packed)
    assert np.array_equal(parts.scales_swizzled, ref.swizzle_scales(lin))
    want_alpha = (np.float32(1) / g) * (np.float32(1) / gx)
    assert abs(float(parts.weight_alpha) / float(want_alpha) - 1) < 3e-7
    assert abs(float(parts.stored_input_global) / float(gx) - 1) < 3e-7
    if layout == "compressed-tensors":   # no reciprocal of a reciprocal on this layout: exact
        assert parts.weight_alpha == want_alpha and parts.stored_input_global == gx
    # dequantized through the oracle, the module is the quantized weight again
    deq = ref.dequantize_packed_swizzled(parts.packed, parts.scales_swizzled, n, k, float(1 / parts.stored_weight_global))
    assert np.allclose(deq, ref.dequantize_packed_linear(packed, lin, n, k, float(np.float32(1) / g)), rtol=3e-7, atol=0)


def test_missing_input_global_and_degenerate_globals(tmp_path):
    rng = np.random.default_rng(6)
    packed, lin, g = make_module(rng, 128, 128)
    t = ct_tensors("a", packed, lin, g)                       # no input global: 1.0
    t.update(modelopt_tensors("b", packed, lin, g))
    t["b.weight_scale_2"] = ("F32", (), f32(0.0))             # zero and non-finite multipliers read as 1.0
    t["b.input_scale"] = ("F32", (), f32(np.inf))
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", t))
    a = W.read_nvfp4_module(wl, "a", 128, 128)
    assert a.stored_input_global == 1.0 and a.weight_alpha == np.float32(1) / g
    b = W.read_nvfp4_module(wl, "b", 128, 128, W.Nvfp4Suffixes.GEMMA_MODELOPT)
    assert b.weight_alpha == 1.0 and b.stored_input_global == 1.0


def test_shape_and_length_checks(tmp_path):
    rng = np.random.default_rng(7)
    packed, lin, g = make_module(rng, 128, 128)
    t = ct_tensors("a", packed, lin, g)
    t["b.weight_packed"] = t["a.weight_packed"]
    t["b.weight_scale"] = ("F8_E4M3", (128, 4), lin[:, :4].tobytes())
    t["b.weight_global_scale"] = t["a.weight_global_scale"]
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", t))
    with pytest.raises(W.WeightError, match=r"shape expected \[256, 64\]"):
        W.read_nvfp4_module(wl, "a", 256, 128)
    with pytest.raises(W.WeightError, match="missing c.weight_packed"):
        W.read_nvfp4_module(wl, "c", 128, 128)
    with pytest.raises(W.WeightError, match="weight_scale byte length"):
        W.read_nvfp4_module(wl, "b", 128, 128)


def test_fused_pair_concatenates_and_checks(tmp_path):
    rng = np.random.default_rng(8)
    n, k = 256, 256
    pg, lg, g = make_module(rng, n, k, stored_global=2000.0)
    pu, lu, _ = make_module(rng, n, k, stored_global=2000.0)
    pd, ld, gd = make_module(rng, n, k, stored_global=1000.0)
    t = {}
    t.update(ct_tensors("mlp.gate", pg, lg, g, 3.0))
    t.update(ct_tensors("mlp.up", pu, lu, g, 3.0))
    t.update(ct_tensors("mlp.other", pd, ld, gd, 3.0))
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", t))
    f = W.read_nvfp4_fused_pair(wl, "mlp.gate", "mlp.up", n, k)
    assert f.out_features == 2 * n and np.array_equal(f.packed, np.concatenate([pg, pu]))
    # each part is whole 128-row tiles, so the fused tiled layout is the two tiled layouts back to back
    assert np.array_equal(f.scales_swizzled, np.concatenate([ref.swizzle_scales(lg), ref.swizzle_scales(lu)]))
    assert np.array_equal(f.scales_swizzled, ref.swizzle_scales(np.concatenate([lg, lu])))
    assert f.weight_alpha == (np.float32(1) / np.float32(2000.0)) * (np.float32(1) / np.float32(3.0))
    with pytest.raises(W.WeightError, match="global scales must match"):
        W.read_nvfp4_fused_pair(wl, "mlp.gate", "mlp.other", n, k)
    with pytest.raises(W.WeightError, match="multiple of 128"):
        W.read_nvfp4_fused_pair(wl, "mlp.gate", "mlp.up", 192, k)


@pytest.mark.parametrize("n,k", [(64, 64), (16, 128), (96, 32)])
def test_small_module_expansion_equals_the_oracle(tmp_path, n, k):
    rng = np.random.default_rng(n + k)
    packed, lin, g = make_module(rng, n, k)
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", ct_tensors("s", packed, lin, g)))
    got = W.dequantize_nvfp4_to_bf16(wl, "s", n, k)
    want = ref.dequantize_to_bf16(packed, ref.swizzle_scales(lin), n, k, float(np.float32(1) / g))
    assert got.dtype == np.uint16 and np.array_equal(got, want)


def test_device_constructors_refuse_a_cpu_device(tmp_path):
    rng = np.random.default_rng(9)
    packed, lin, g = make_module(rng, 128, 128)
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", ct_tensors("a", packed, lin, g)))
    with pytest.raises(W.WeightError, match="requires a CUDA device"):
        W.nvfp4_linear_from_disk(wl, "a", 128, 128, "cpu")
    with pytest.raises(W.WeightError, match="requires a CUDA device"):
        W.moe_grouped_weights_from_disk(wl, ["a"], 128, 128, "cpu")


def test_host_dequantize_equals_the_oracle_and_serves_dequant_weight():
    """dequantize_packed_to_bf16_bits == the oracle's bf16 expansion, bit for bit; Nvfp4Linear.dequant_weight
    (a host-side helper, run here on CPU tensors) returns it for the linear's own buffers."""
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(13)
    n, k = 256, 384
    packed, lin, g = make_module(rng, n, k)
    alpha = np.float32(1) / g
    want = ref.dequantize_to_bf16(packed, ref.swizzle_scales(lin), n, k, float(alpha))
    assert np.array_equal(W.dequantize_packed_to_bf16_bits(packed, lin, n, k, alpha), want)
    layer = sp.Nvfp4Linear.new_nvfp4(torch.from_numpy(packed), torch.from_numpy(ref.swizzle_scales(lin)), float(alpha), k, n)
    got = layer.dequant_weight()
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == (n, k)
    assert np.array_equal(got.view(torch.int16).numpy().view(np.uint16), want)
    with pytest.raises(W.WeightError, match="too few bytes"):
        W.dequantize_packed_to_bf16_bits(packed[:10], lin, n, k, alpha)


def test_interoperates_with_the_safetensors_library(tmp_path):
    """Files written by the `safetensors` package load here, and files written by this test's
    minimal writer load there (skipped when the package is not installed)."""
    st = pytest.importorskip("safetensors.numpy")
    rng = np.random.default_rng(14)
    a = rng.standard_normal((3, 5)).astype(np.float32)
    b = rng.integers(0, 255, (4, 8), dtype=np.uint8)
    c = np.array([7, -9], np.int64)
    path = tmp_path / "lib.safetensors"
    st.save_file({"a": a, "b": b, "c": c}, str(path), metadata={"format": "np"})
    wl = W.WeightLoader.open_file(path)
    assert wl.names() == ["a", "b", "c"]
    assert np.array_equal(wl.get("a").numpy(), a) and wl.shape_of("b") == [4, 8]
    assert np.array_equal(np.asarray(wl.raw_bytes("b")).reshape(4, 8), b)
    assert wl.get("c").tolist() == [7, -9]
    mine = write_safetensors(tmp_path / "mine.safetensors", {"a": ("F32", a.shape, a.tobytes()),
                                                             "b": ("U8", b.shape, b.tobytes())})
    back = st.load_file(str(mine))
    assert np.array_equal(back["a"], a) and np.array_equal(back["b"], b)


def test_host_nvfp4_tensor_is_byte_exact_with_the_oracle():
    """The host container and its quantizer (rust/crates/nv-quant/src/nvfp4.rs:91-210) against the C
    oracle: codes, scale bytes, swizzle, column-major scales and dequantization, on random data, ties,
    zeros, huge and tiny magnitudes and odd globals."""
    import numpy as np

    from oracle import ref
    from speaches_plus_b200 import weights as W
    rng = np.random.default_rng(21)
    rows, cols = 37, 256
    x = (rng.standard_normal((rows, cols)) * np.exp(rng.uniform(-12, 12, (rows, 1)))).astype(np.float32)
    x[0, :16] = 0.0
    x[1, :16] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0]  # ties at unit scale
    x[2, :16] = 1e30
    x[3, :16] = 1e-30
    for g in (1.0, 3.7, 2688.0 / 0.31, 0.0, float("nan"), float("inf")):
        t = W.Nvfp4Tensor.quantize_rows_with_global(x, g)
        packed, lin = ref.quantize_rows(x, g if np.isfinite(g) and g != 0 else 1.0)
        assert np.array_equal(t.data, packed), g
        assert np.array_equal(t.scales, lin), g
        assert np.array_equal(t.scales_swizzled(), ref.swizzle_scales(lin))
        assert np.array_equal(t.scales_column_major().reshape(cols // 16, rows), lin.T)
        want = ref.dequantize_packed_linear(packed, lin, rows, cols, 0.5).reshape(rows, cols)
        assert np.array_equal(t.dequantize_scaled(0.5), want)
    assert W.Nvfp4Tensor.quantize_rows(x).scales.shape == (rows, cols // 16)
    # every scale the encoder can meet: a dense sweep against the oracle's scalar encoder
    s = np.concatenate([np.float32(2.0) ** rng.uniform(-12, 10, 4000).astype(np.float32),
                        np.array([0, -1, np.nan, np.inf, 448, 449, 1e9, 2 ** -6, 2 ** -9, 2 ** -10], np.float32)])
    assert np.array_equal(W.encode_ue4m3_host(s), np.array([ref.encode_ue4m3(float(v)) for v in s], np.uint8))
    v = np.concatenate([rng.uniform(-7, 7, 4000).astype(np.float32),
                        np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.0, 0.0], np.float32)])
    assert np.array_equal(W.encode_e2m1_host(v), np.array([ref.encode_e2m1(float(q)) for q in v], np.uint8))
