"""On-disk NVFP4 checkpoints -> device-resident NVFP4 linears.

Host-side mirror of the reference's ingestion for this path:
  * `WeightLoader` (rust/crates/nv-weights/src/lib.rs:52-238,580-598): memory-mapped safetensors
    shards, opened from one file or a directory (index file, or every `*.safetensors`);
  * `QuantizationConfig` (lib.rs:313-520): which scheme a `config.json` declares, group-size check,
    ignore list;
  * `Nvfp4Suffixes`, `load_linear_maybe_quant`, `nvfp4_linear_from_disk[_with_suffixes]`,
    `nvfp4_linear_from_disk_fused_pair`, `dequantize_nvfp4_to_bf16`
    (rust/crates/nv-layers/src/moe.rs:574-992): tensor names of the two checkpoint layouts, global
    scale conventions, host swizzle of the block scales, fused gate+up concatenation.

Everything up to the host->device copy is plain numpy on memory-mapped bytes, as it is load-time
work on the host in the reference too; the linears it returns run on the CUDA library only.
"""
from __future__ import annotations

import dataclasses
import enum
import json
import mmap
import os
from typing import Iterable

import numpy as np

BLOCK_SIZE = 16
MIN_TILE = 128
NVFP4_GROUP_SIZE = BLOCK_SIZE

# safetensors dtype tag -> bytes per element
_ST_ITEMSIZE = {"BOOL": 1, "U8": 1, "I8": 1, "F8_E5M2": 1, "F8_E4M3": 1, "I16": 2, "U16": 2, "F16": 2, "BF16": 2,
                "I32": 4, "U32": 4, "F32": 4, "F64": 8, "I64": 8, "U64": 8}
# Source dtypes a typed read accepts (lib.rs:277-288); anything else is reachable as raw bytes only.
_TYPED = {"BF16", "F16", "F32", "I64", "U8", "BOOL"}


class WeightError(ValueError):
    """A checkpoint that cannot be loaded as asked; the message names the tensor."""


# ------------------------------------------------------------------------------------------------
# safetensors shards
@dataclasses.dataclass(frozen=True)
class TensorHeader:
    dtype: str
    shape: tuple
    offset_start: int
    offset_end: int


class _Shard:
    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            size = os.fstat(f.fileno()).st_size
            if size < 8:
                raise WeightError(f"parse safetensors header in {path}: file too short")
            self._mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        self.bytes = np.frombuffer(self._mm, dtype=np.uint8)
        n = int.from_bytes(self._mm[:8], "little")
        if n > size - 8:
            raise WeightError(f"parse safetensors header in {path}: header length {n} exceeds the file")
        try:
            meta = json.loads(self._mm[8:8 + n].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightError(f"parse safetensors header in {path}: {e}") from e
        if not isinstance(meta, dict):
            raise WeightError(f"parse safetensors header in {path}: not an object")
        base = 8 + n
        self.headers: dict[str, TensorHeader] = {}
        for name, h in meta.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (a, b) = h["dtype"], tuple(int(d) for d in h["shape"]), h["data_offsets"]
            except (KeyError, TypeError, ValueError) as e:
                raise WeightError(f"parse safetensors header in {path}: tensor {name}: {e}") from e
            if dtype not in _ST_ITEMSIZE:
                raise WeightError(f"parse safetensors header in {path}: tensor {name}: unknown dtype {dtype}")
            count = 1
            for d in shape:
                count *= d
            if not (0 <= a <= b and base + b <= size) or b - a != count * _ST_ITEMSIZE[dtype]:
                raise WeightError(f"parse safetensors header in {path}: tensor {name}: bad data_offsets")
            self.headers[name] = TensorHeader(dtype, shape, base + a, base + b)


def _is_lfs_pointer(path: str) -> bool:
    """A git-lfs pointer left in place of a shard (lib.rs:266-275)."""
    if os.path.getsize(path) > 1024:
        return False
    with open(path, "rb") as f:
        return f.read(64).startswith(b"version https://git-lfs.github.com/spec/")


class WeightLoader:
    """Name -> tensor over one or more memory-mapped safetensors shards."""

    def __init__(self, shards: list, name_to_shard: dict):
        self._shards, self._name_to_shard = shards, name_to_shard

    @classmethod
    def open_file(cls, path) -> "WeightLoader":
        shard = _Shard(os.fspath(path))
        return cls([shard], {name: 0 for name in shard.headers})

    @classmethod
    def open_dir(cls, directory) -> "WeightLoader":
        directory = os.fspath(directory)
        if not os.path.isdir(directory):
            raise WeightError(f"not a directory: {directory}")
        index_path = os.path.join(directory, "model.safetensors.index.json")
        weight_map = None
        if os.path.isfile(index_path):
            with open(index_path, "rb") as f:
                try:
                    weight_map = json.load(f)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError) as e:
                    raise WeightError(f"parse {index_path}: {e}") from e
            paths = sorted({os.path.join(directory, fn) for fn in weight_map.values()})
        else:
            paths = sorted(os.path.join(directory, fn) for fn in os.listdir(directory) if fn.endswith(".safetensors"))
            if not paths:
                raise WeightError(f"no .safetensors files in {directory}")
        shards, path_to_idx, skipped = [], {}, set()
        for p in paths:
            if _is_lfs_pointer(p):
                skipped.add(p)
                continue
            path_to_idx[p] = len(shards)
            shards.append(_Shard(p))
        name_to_shard: dict[str, int] = {}
        if weight_map is not None:
            for name, fn in weight_map.items():
                full = os.path.join(directory, fn)
                if full in skipped:
                    continue
                if full not in path_to_idx:
                    raise WeightError(f"index references missing shard {full}")
                idx = path_to_idx[full]
                if name not in shards[idx].headers:
                    raise WeightError(f"shard {full} missing tensor {name}")
                name_to_shard[name] = idx
        else:
            for idx, shard in enumerate(shards):
                for name in shard.headers:
                    if name in name_to_shard:
                        raise WeightError(f"duplicate tensor {name} in shards "
                                          f"{shards[name_to_shard[name]].path} and {shard.path}")
                    name_to_shard[name] = idx
        return cls(shards, name_to_shard)

    # -- queries --
    def names(self) -> list:
        return sorted(self._name_to_shard)

    def has(self, name: str) -> bool:
        return name in self._name_to_shard

    def _header(self, name: str):
        if name not in self._name_to_shard:
            raise WeightError(f"tensor not found: {name}")
        shard = self._shards[self._name_to_shard[name]]
        return shard, shard.headers[name]

    def shape_of(self, name: str):
        return list(self._header(name)[1].shape) if self.has(name) else None

    def st_dtype_of(self, name: str):
        return self._header(name)[1].dtype if self.has(name) else None

    def dtype_of(self, name: str):
        """The dtype a typed read yields before any cast: BOOL reads as U8; None for byte-only dtypes."""
        d = self.st_dtype_of(name)
        if d == "BOOL":
            return "U8"
        return d if d in _TYPED else None

    def raw_bytes(self, name: str) -> np.ndarray:
        """The tensor's bytes as stored (a read-only view of the mapping), whatever its dtype."""
        shard, h = self._header(name)
        return shard.bytes[h.offset_start:h.offset_end]

    def get_numpy_f32(self, name: str) -> np.ndarray:
        """The tensor widened to float32 on the host (BF16, F16, F32, I64, U8, BOOL sources)."""
        shard, h = self._header(name)
        raw = shard.bytes[h.offset_start:h.offset_end]
        if h.dtype == "BF16":
            out = (raw.view("<u2").astype(np.uint32) << 16).view(np.float32)
        elif h.dtype == "F16":
            out = raw.view("<f2").astype(np.float32)
        elif h.dtype == "F32":
            out = raw.view("<f4").astype(np.float32)
        elif h.dtype == "I64":
            out = raw.view("<i8").astype(np.float32)
        elif h.dtype in ("U8", "BOOL"):
            out = raw.astype(np.float32)
        else:
            raise WeightError(f"unsupported source dtype {h.dtype} for {name}")
        return out.reshape(h.shape)

    def get(self, name: str, dtype=None):
        """The tensor as a host torch tensor, cast to `dtype` when given (lib.rs:174-208)."""
        import torch
        shard, h = self._header(name)
        if h.dtype not in _TYPED:
            raise WeightError(f"unsupported source dtype {h.dtype} for {name}")
        raw = np.array(shard.bytes[h.offset_start:h.offset_end])  # private copy: torch wants writable memory
        t = torch.from_numpy(raw)
        view = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "I64": torch.int64,
                "U8": torch.uint8, "BOOL": torch.uint8}[h.dtype]
        t = t.view(view).reshape(h.shape)
        return t if dtype is None or dtype == t.dtype else t.to(dtype)

    def scalar_f32(self, name: str, default: float = 1.0) -> np.float32:
        """First element of a tensor read as f32; `default` for an empty tensor."""
        v = self.get_numpy_f32(name).reshape(-1)
        return np.float32(v[0]) if v.size else np.float32(default)


# ------------------------------------------------------------------------------------------------
# config.json -> scheme
class QuantScheme(enum.Enum):
    NONE = "none"
    FP8_E4M3 = "fp8_e4m3"
    NVFP4 = "nvfp4"


def _detect_group_size(obj: dict):
    groups = obj.get("config_groups")
    if isinstance(groups, dict):
        for group in groups.values():
            w = group.get("weights") if isinstance(group, dict) else None
            if isinstance(w, dict) and isinstance(w.get("group_size"), int) and w["group_size"] >= 0:
                return w["group_size"]
    return None


@dataclasses.dataclass
class QuantizationConfig:
    scheme: QuantScheme = QuantScheme.NONE
    ignored_modules: list = dataclasses.field(default_factory=list)
    group_size: int | None = None

    @staticmethod
    def implemented_group_size(scheme: QuantScheme):
        return NVFP4_GROUP_SIZE if scheme is QuantScheme.NVFP4 else None

    def effective_group_size(self):
        return self.group_size if self.group_size is not None else self.implemented_group_size(self.scheme)

    def validate(self) -> None:
        """Refuse a declared group size this build would mis-scale (lib.rs:342-370)."""
        g = self.group_size
        if g is None or self.scheme is QuantScheme.NONE:
            return
        if self.scheme is QuantScheme.NVFP4:
            if g != NVFP4_GROUP_SIZE:
                raise WeightError(
                    f"quantization_config declares group_size {g} for 4-bit float weights, but NVFP4 here has "
                    f"exactly {NVFP4_GROUP_SIZE} elements per ue4m3 scale. group_size 32 with 4-bit weights is "
                    f"MXFP4 (per-32 ue8m0 scales), a different format; loading it as NVFP4 would mis-scale "
                    f"every block. Refusing.")
            return
        raise WeightError(
            f"quantization_config declares group_size {g} for FP8 weights, but FP8 is scaled per output row "
            f"here, not per {g}-element block. Refusing.")

    @classmethod
    def none(cls) -> "QuantizationConfig":
        return cls()

    @classmethod
    def from_hf_value(cls, v) -> "QuantizationConfig":
        q = cls._parse(v)
        q.validate()
        return q

    @classmethod
    def _parse(cls, v) -> "QuantizationConfig":
        if v is None:
            return cls.none()
        if not isinstance(v, dict):
            raise WeightError("quantization_config must be an object")
        ign = v.get("ignore", v.get("ignored_modules"))
        ignored = [x for x in ign if isinstance(x, str)] if isinstance(ign, list) else []
        gs = _detect_group_size(v)
        if v.get("quant_method") == "modelopt" and isinstance(v.get("quant_algo"), str):
            algo = v["quant_algo"].upper()
            if "FP4" in algo:
                return cls(QuantScheme.NVFP4, ignored, gs)
            if "FP8" in algo:
                return cls(QuantScheme.FP8_E4M3, ignored, gs)
        fmt = v.get("format") if isinstance(v.get("format"), str) else ""
        qtype = v.get("quantization_type") if isinstance(v.get("quantization_type"), str) else ""
        if "fp4" in fmt.lower():
            return cls(QuantScheme.NVFP4, ignored, gs)
        if qtype.lower() == "fp8" or "fp8" in fmt.lower():
            return cls(QuantScheme.FP8_E4M3, ignored, gs)
        groups = v.get("config_groups")
        if isinstance(groups, dict):
            for group in groups.values():
                w = group.get("weights") if isinstance(group, dict) else None
                if not isinstance(w, dict):
                    continue
                bits = w.get("num_bits") if isinstance(w.get("num_bits"), int) else 0
                typ = w.get("type") if isinstance(w.get("type"), str) else ""
                g = w.get("group_size") if isinstance(w.get("group_size"), int) else None
                if typ.lower() == "float" and bits == 4:
                    return cls(QuantScheme.NVFP4, ignored, g)
                if typ.lower() == "float" and bits == 8:
                    return cls(QuantScheme.FP8_E4M3, ignored, g)
        return cls.none()

    @classmethod
    def from_hf_json_str(cls, s: str) -> "QuantizationConfig":
        try:
            v = json.loads(s)
        except json.JSONDecodeError as e:
            raise WeightError(f"parse config.json: {e}") from e
        return cls.from_hf_value(v.get("quantization_config") if isinstance(v, dict) else None)

    @classmethod
    def from_hf_json_file(cls, path) -> "QuantizationConfig":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_hf_json_str(f.read())

    def is_module_ignored(self, name: str) -> bool:
        """Exact match, or prefix match for a pattern ending in `*` (lib.rs:491-520)."""
        for pat in self.ignored_modules:
            if (name.startswith(pat[:-1]) if pat.endswith("*") else name == pat):
                return True
        return False


# ------------------------------------------------------------------------------------------------
# NVFP4 tensors of one module
@dataclasses.dataclass(frozen=True)
class Nvfp4Suffixes:
    """Tensor-name suffixes of one checkpoint layout (moe.rs:605-632)."""
    packed: str
    block_scale: str
    weight_global_scale: str
    input_global_scale: str
    global_scale_is_inverse: bool  # True: the file stores the multiplier used when quantizing (448*6/amax)


Nvfp4Suffixes.QWEN_COMPRESSED_TENSORS = Nvfp4Suffixes("weight_packed", "weight_scale", "weight_global_scale",
                                                      "input_global_scale", True)
Nvfp4Suffixes.GEMMA_MODELOPT = Nvfp4Suffixes("weight", "weight_scale", "weight_scale_2", "input_scale", False)


def _safe_recip(x) -> np.float32:
    x = np.float32(x)
    return np.float32(1.0) if (x == 0 or not np.isfinite(x)) else np.float32(1.0) / x


def swizzle_scales(linear: np.ndarray, rows: int, k_blocks: int) -> np.ndarray:
    """Row-major [rows, k_blocks] scale bytes -> the 128x4-tiled layout the kernels read, padded
    with zero bytes to whole tiles (rust/crates/nv-quant/src/nvfp4.rs:231-249):
    dst = ((m/128 * ceil(k_blocks/4) + kb/4) * 32 + m%32) * 16 + ((m/32)%4) * 4 + kb%4."""
    linear = np.ascontiguousarray(linear, dtype=np.uint8).reshape(-1)
    if linear.size != rows * k_blocks:
        raise WeightError(f"swizzle_scales: {linear.size} bytes for {rows} x {k_blocks} scales")
    m_tiles, k_tiles = (rows + 127) // 128, (k_blocks + 3) // 4
    padded = np.zeros((m_tiles * 128, k_tiles * 4), dtype=np.uint8)
    padded[:rows, :k_blocks] = linear.reshape(rows, k_blocks)
    # [m_tile, (m/32)%4, m%32, k_tile, kb%4] -> [m_tile, k_tile, m%32, (m/32)%4, kb%4]
    t = padded.reshape(m_tiles, 4, 32, k_tiles, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(t).reshape(-1)


def unswizzle_scales(swz: np.ndarray, rows: int, k_blocks: int) -> np.ndarray:
    """Inverse of `swizzle_scales` (nvfp4.rs:251-264): the row-major [rows, k_blocks] bytes."""
    m_tiles, k_tiles = (rows + 127) // 128, (k_blocks + 3) // 4
    swz = np.asarray(swz, dtype=np.uint8).reshape(-1)[: m_tiles * k_tiles * 512]
    t = swz.reshape(m_tiles, k_tiles, 32, 4, 4).transpose(0, 3, 2, 1, 4).reshape(m_tiles * 128, k_tiles * 4)
    return np.ascontiguousarray(t[:rows, :k_blocks])


@dataclasses.dataclass
class Nvfp4HostParts:
    """One module's NVFP4 tensors on the host, ready to upload."""
    packed: np.ndarray            # [out, in/2] bytes, as stored
    scales_swizzled: np.ndarray   # 128x4-tiled ue4m3 bytes
    scales_linear: np.ndarray     # [out, in/16] bytes, as stored
    weight_alpha: np.float32      # 1/(weight global) * 1/(input global)
    stored_input_global: np.float32
    stored_weight_global: np.float32
    out_features: int
    in_features: int


def _read_module(weights: WeightLoader, module: str, out_features: int, in_features: int, sfx: Nvfp4Suffixes,
                 what: str = "nvfp4"):
    packed_name, scale_name = f"{module}.{sfx.packed}", f"{module}.{sfx.block_scale}"
    shape = weights.shape_of(packed_name)
    if shape is None:
        raise WeightError(f"missing {packed_name}")
    if in_features % BLOCK_SIZE != 0:
        raise WeightError(f"{what} {module}: in_features {in_features} is not a multiple of {BLOCK_SIZE}")
    if shape != [out_features, in_features // 2]:
        raise WeightError(f"{what} {module}: {sfx.packed} shape expected [{out_features}, {in_features // 2}], "
                          f"got {shape}")
    packed = weights.raw_bytes(packed_name)
    if packed.size != out_features * in_features // 2:
        raise WeightError(f"{what} {module}: {sfx.packed} byte length {packed.size} != expected "
                          f"{out_features * in_features // 2}")
    if not weights.has(scale_name):
        raise WeightError(f"missing {scale_name}")
    scales = weights.raw_bytes(scale_name)
    if scales.size != out_features * (in_features // BLOCK_SIZE):
        raise WeightError(f"{what} {module}: {sfx.block_scale} byte length {scales.size} != "
                          f"{out_features} x {in_features // BLOCK_SIZE}")
    raw_w = weights.scalar_f32(f"{module}.{sfx.weight_global_scale}")
    in_name = f"{module}.{sfx.input_global_scale}"
    raw_x = weights.scalar_f32(in_name) if weights.has(in_name) else np.float32(1.0)
    return packed, scales, raw_w, raw_x


def _globals(raw_w, raw_x, sfx: Nvfp4Suffixes):
    """(stored weight global, stored input global, weight_alpha) from the file's numbers: a layout that
    stores the dequantization multipliers is inverted first (moe.rs:787-792)."""
    if sfx.global_scale_is_inverse:
        gw, gx = np.float32(raw_w), np.float32(raw_x)
    else:
        gw, gx = _safe_recip(raw_w), _safe_recip(raw_x)
    return gw, gx, np.float32(_safe_recip(gw) * _safe_recip(gx))


def read_nvfp4_module(weights: WeightLoader, module: str, out_features: int, in_features: int,
                      sfx: Nvfp4Suffixes = Nvfp4Suffixes.QWEN_COMPRESSED_TENSORS) -> Nvfp4HostParts:
    """Host half of `nvfp4_linear_from_disk_inner` (moe.rs:706-815): check shapes and byte counts,
    read the globals, swizzle the block scales."""
    packed, scales, raw_w, raw_x = _read_module(weights, module, out_features, in_features, sfx)
    gw, gx, alpha = _globals(raw_w, raw_x, sfx)
    return Nvfp4HostParts(packed.reshape(out_features, in_features // 2),
                          swizzle_scales(scales, out_features, in_features // BLOCK_SIZE),
                          scales.reshape(out_features, in_features // BLOCK_SIZE), alpha, gx, gw,
                          out_features, in_features)


def read_nvfp4_fused_pair(weights: WeightLoader, module_a: str, module_b: str, out_features_each: int,
                          in_features: int, sfx: Nvfp4Suffixes = Nvfp4Suffixes.QWEN_COMPRESSED_TENSORS
                          ) -> Nvfp4HostParts:
    """Two modules with the same input (gate and up) as one [2*out_each, in] linear
    (moe.rs:817-953).  Each part must be a multiple of 128 rows so that the tiled scale layouts
    concatenate, and both must carry the same global scales."""
    if out_features_each % 128 != 0:
        raise WeightError(f"fused NVFP4 pair: out_features_each ({out_features_each}) must be a multiple of 128 "
                          f"so the swizzled scale layout concatenates cleanly")
    pa, sa, wa, xa = _read_module(weights, module_a, out_features_each, in_features, sfx, "fused")
    pb, sb, wb, xb = _read_module(weights, module_b, out_features_each, in_features, sfx, "fused")
    if wa != wb or xa != xb:
        raise WeightError(f"fused NVFP4 pair ({module_a} + {module_b}): global scales must match. "
                          f"gate(w={wa:.6e} x={xa:.6e}) up(w={wb:.6e} x={xb:.6e})")
    gw, gx, alpha = _globals(wa, xa, sfx)
    n, kb = 2 * out_features_each, in_features // BLOCK_SIZE
    scales = np.concatenate([sa, sb])
    return Nvfp4HostParts(np.concatenate([pa, pb]).reshape(n, in_features // 2), swizzle_scales(scales, n, kb),
                          scales.reshape(n, kb), alpha, gx, gw, n, in_features)


_E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], np.float32)


def _ue4m3_table() -> np.ndarray:
    b = np.arange(256, dtype=np.int64)
    e, m = (b >> 3) & 0xF, (b & 7).astype(np.float32)
    sub = m * np.float32(2.0 ** -9)
    nor = (np.float32(1.0) + m / np.float32(8.0)) * np.exp2((e - 7).astype(np.float32))
    return np.where(e == 0, sub, nor).astype(np.float32)


_UE4M3 = _ue4m3_table()


def _f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u + (np.uint32(0x7FFF) + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    return np.where(np.isnan(x), np.uint16(0x7FC0), r).astype(np.uint16)


def dequantize_packed_to_bf16_bits(packed: np.ndarray, scales_linear: np.ndarray, rows: int, cols: int,
                                   weight_mult) -> np.ndarray:
    """Packed e2m1 [rows, cols/2] + row-major ue4m3 scales [rows, cols/16] -> bf16 bits [rows, cols]:
    value = e2m1 * (ue4m3 * weight_mult), each product one f32 operation, rounded to bf16 (nearest
    even) -- rust/crates/nv-quant/src/nvfp4.rs:266-292 followed by the bf16 cast of its callers."""
    kb = cols // BLOCK_SIZE
    packed = np.asarray(packed, dtype=np.uint8).reshape(-1)
    scales_linear = np.asarray(scales_linear, dtype=np.uint8).reshape(-1)
    if cols % BLOCK_SIZE != 0 or packed.size < rows * cols // 2 or scales_linear.size < rows * kb:
        raise WeightError(f"nvfp4 dequantize: too few bytes for [{rows}, {cols}]")
    block = (_UE4M3[scales_linear[: rows * kb]] * np.float32(weight_mult)).astype(np.float32).reshape(rows, kb, 1)
    p = packed[: rows * cols // 2].reshape(rows, kb, BLOCK_SIZE // 2)
    vals = np.empty((rows, kb, BLOCK_SIZE), dtype=np.float32)
    vals[:, :, 0::2] = _E2M1[p & 0xF] * block
    vals[:, :, 1::2] = _E2M1[p >> 4] * block
    return _f32_to_bf16_bits(vals.reshape(rows, cols))


# ---- host-side NVFP4 container and quantizer (load-time tools; the decode path quantizes on the GPU) ----
def encode_e2m1_host(x: np.ndarray) -> np.ndarray:
    """f32 -> 4-bit e2m1 codes (sign in bit 3): nearest codebook value, the FIRST minimum winning, i.e.
    ties go to the lower code (rust/crates/nv-quant/src/nvfp4.rs:6-22).  Midpoints with strict `>`."""
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x)
    code = np.zeros(x.shape, dtype=np.uint8)
    for mid in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        code += (a > np.float32(mid)).astype(np.uint8)
    return code | (np.signbit(x).astype(np.uint8) << 3)


def encode_ue4m3_host(s: np.ndarray) -> np.ndarray:
    """f32 scale -> ue4m3 byte (nvfp4.rs:38-74): <= 0 / NaN / Inf -> 0; clamp to 448; below 2^-6 the
    subnormal grid m * 2^-9; else mantissa rounded half away from zero with carry; 0x7F -> 0x7E."""
    s = np.asarray(s, dtype=np.float32)
    ok = np.isfinite(s) & (s > 0)
    c = np.minimum(np.where(ok, s, np.float32(1.0)), np.float32(448.0)).astype(np.float32)
    half_away = lambda v: np.floor(v + np.float32(0.5))   # noqa: E731  (arguments are non-negative)
    sub_m = half_away((c / np.float32(2.0 ** -9)).astype(np.float32))
    sub = np.where(sub_m <= 0, 0, np.where(sub_m <= 7, sub_m, 8)).astype(np.int64)
    _, e2 = np.frexp(c)
    ex = e2.astype(np.int64) - 1
    mf = (np.ldexp(c, -ex.astype(np.int32)) - np.float32(1.0)).astype(np.float32)
    mant = half_away((mf * np.float32(8.0)).astype(np.float32)).astype(np.int64)
    mant = np.maximum(mant, 0)
    carry = mant > 7
    mant = np.where(carry, 0, mant)
    ex = ex + carry
    biased = np.clip(ex + 7, 1, 15)
    byte = (biased << 3) | mant
    byte = np.where(byte == 0x7F, 0x7E, byte)
    out = np.where(c < np.float32(2.0 ** -6), sub, byte)
    return np.where(ok, out, 0).astype(np.uint8)


def quantize_rows_host(x: np.ndarray, stored_global: float = 1.0):
    """f32 [rows, cols] -> (packed [rows, cols/2], row-major scales [rows, cols/16]) by the block rule of
    nvfp4.rs:91-120: local = amax/6 (1 for an all-zero block); byte = ue4m3(G * local); inv = G / decode(byte)
    (1 when that is 0); code = e2m1(clamp(v * inv, +-6)); G in {0, NaN, Inf} counts as 1.  All in f32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    if cols % BLOCK_SIZE != 0:
        raise WeightError(f"cols must be a multiple of {BLOCK_SIZE}")
    g = np.float32(stored_global)
    if g == 0 or not np.isfinite(g):
        g = np.float32(1.0)
    b = x.reshape(rows, cols // BLOCK_SIZE, BLOCK_SIZE)
    amax = np.max(np.abs(b), axis=2).astype(np.float32)
    local = np.where(amax == 0, np.float32(1.0), (amax / np.float32(6.0)).astype(np.float32)).astype(np.float32)
    scales = encode_ue4m3_host((g * local).astype(np.float32))
    dec = _UE4M3[scales]
    inv = np.where(dec == 0, np.float32(1.0), (g / np.where(dec == 0, np.float32(1.0), dec)).astype(np.float32))
    q = np.clip((b * inv[:, :, None].astype(np.float32)).astype(np.float32), np.float32(-6.0), np.float32(6.0))
    codes = encode_e2m1_host(q)
    packed = (codes[:, :, 0::2] | (codes[:, :, 1::2] << 4)).astype(np.uint8).reshape(rows, cols // 2)
    return packed, scales.astype(np.uint8)


@dataclasses.dataclass
class Nvfp4Tensor:
    """Row-major NVFP4 container on the host (nvfp4.rs:131-210): `data` [rows, cols/2] packed e2m1 (even
    element in the low nibble), `scales` [rows, cols/16] ue4m3, row-major."""
    data: np.ndarray
    scales: np.ndarray
    rows: int
    cols: int

    @classmethod
    def quantize_rows(cls, rows) -> "Nvfp4Tensor":
        return cls.quantize_rows_with_global(rows, 1.0)

    @classmethod
    def quantize_rows_with_global(cls, rows, stored_global: float) -> "Nvfp4Tensor":
        x = np.asarray(rows, dtype=np.float32)
        packed, scales = quantize_rows_host(x, stored_global)
        return cls(packed, scales, x.shape[0], x.shape[1])

    def scales_swizzled(self) -> np.ndarray:
        return swizzle_scales(self.scales, self.rows, self.cols // BLOCK_SIZE)

    def scales_column_major(self) -> np.ndarray:
        return np.ascontiguousarray(self.scales.reshape(self.rows, self.cols // BLOCK_SIZE).T).reshape(-1)

    def dequantize(self) -> np.ndarray:
        return self.dequantize_scaled(1.0)

    def dequantize_scaled(self, weight_mult: float) -> np.ndarray:
        """f32 [rows, cols]: (e2m1 * ue4m3) then * weight_mult, as nvfp4.rs:178-209 multiplies."""
        kb = self.cols // BLOCK_SIZE
        block = _UE4M3[self.scales.reshape(self.rows, kb)].reshape(self.rows, kb, 1)
        p = self.data.reshape(self.rows, kb, BLOCK_SIZE // 2)
        vals = np.empty((self.rows, kb, BLOCK_SIZE), dtype=np.float32)
        vals[:, :, 0::2] = _E2M1[p & 0xF] * block
        vals[:, :, 1::2] = _E2M1[p >> 4] * block
        return (vals.reshape(self.rows, self.cols) * np.float32(weight_mult)).astype(np.float32)


def dequantize_nvfp4_to_bf16(weights: WeightLoader, module: str, out_features: int, in_features: int) -> np.ndarray:
    """A module too small for the NVFP4 kernels, expanded to bf16 bits on the host
    (moe.rs:955-992), with 1/stored_global as the multiplier.  Reads the compressed-tensors names, as
    the reference does."""
    g = weights.scalar_f32(f"{module}.weight_global_scale")
    inv = np.float32(1.0) if g == 0 else np.float32(1.0) / g
    try:
        return dequantize_packed_to_bf16_bits(weights.raw_bytes(f"{module}.weight_packed"),
                                              weights.raw_bytes(f"{module}.weight_scale"), out_features, in_features,
                                              inv)
    except WeightError as e:
        raise WeightError(f"nvfp4 {module}: {e}") from e


# ------------------------------------------------------------------------------------------------
# device-side constructors
def _upload(parts: Nvfp4HostParts, device):
    import torch

    from .linear import Nvfp4Linear
    packed = torch.from_numpy(np.array(parts.packed, copy=True)).to(device)
    scales = torch.from_numpy(np.array(parts.scales_swizzled, copy=True)).to(device)
    return Nvfp4Linear.new_nvfp4_scaled(packed, scales, parts.in_features, parts.out_features, None,
                                        float(parts.weight_alpha), float(parts.stored_input_global))


def _require_cuda(device):
    import torch
    if torch.device(device).type != "cuda":
        raise WeightError("nvfp4 ingest requires a CUDA device")


def nvfp4_linear_from_disk_with_suffixes(weights, module, out_features, in_features, device, sfx):
    _require_cuda(device)
    return _upload(read_nvfp4_module(weights, module, out_features, in_features, sfx), device)


def nvfp4_linear_from_disk(weights, module, out_features, in_features, device):
    return nvfp4_linear_from_disk_with_suffixes(weights, module, out_features, in_features, device,
                                                Nvfp4Suffixes.QWEN_COMPRESSED_TENSORS)


def nvfp4_linear_from_disk_fused_pair(weights, module_a, module_b, out_features_each, in_features, device,
                                      sfx=Nvfp4Suffixes.QWEN_COMPRESSED_TENSORS):
    _require_cuda(device)
    return _upload(read_nvfp4_fused_pair(weights, module_a, module_b, out_features_each, in_features, sfx), device)


def load_linear(weights: WeightLoader, name: str, out_features: int, in_features: int, device):
    """A plain (unquantized) weight as a bf16 linear (moe.rs:548-572)."""
    import torch

    from .linear import Bf16Linear
    w = weights.get(name, torch.bfloat16)
    if list(w.shape) != [out_features, in_features]:
        raise WeightError(f"linear {name}: expected [{out_features}, {in_features}], got {list(w.shape)}")
    return Bf16Linear(w.to(device))


def load_linear_maybe_quant(weights: WeightLoader, name: str, out_features: int, in_features: int,
                            qconfig: QuantizationConfig, device):
    """The reference's dispatch for one `<module>.weight` (moe.rs:574-602): ignored modules and
    modules stored unquantized load as they are; a packed module below the kernels' minimum size is
    expanded to bf16; every other packed module becomes an NVFP4 linear."""
    import torch

    from .linear import Bf16Linear
    module = name[: -len(".weight")] if name.endswith(".weight") else name
    if qconfig.is_module_ignored(module) or weights.has(name) or not weights.has(f"{module}.weight_packed"):
        return load_linear(weights, name, out_features, in_features, device)
    if in_features < MIN_TILE or out_features < MIN_TILE:
        bits = dequantize_nvfp4_to_bf16(weights, module, out_features, in_features)
        return Bf16Linear(torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).to(device))
    return nvfp4_linear_from_disk(weights, module, out_features, in_features, device)


def moe_grouped_weights_from_disk(weights: WeightLoader, expert_prefixes: Iterable[str], hidden: int, inter: int,
                                  device, sfx: Nvfp4Suffixes = Nvfp4Suffixes.QWEN_COMPRESSED_TENSORS,
                                  names=("gate_proj", "up_proj", "down_proj"), rank: int = 0, world: int = 1):
    """Expert banks for the grouped decode path straight from a checkpoint: for each prefix
    `<prefix>.{gate,up,down}_proj`, the same per-expert layout `MoeGroupedWeights.build_from_experts`
    produces (rust/crates/nv-layers/src/moe_grouped.rs:97-280), without a device round trip.  Gate and
    up of one expert must share their input global.  With world > 1 only this rank's block of experts
    is read and uploaded (expert parallelism)."""
    _require_cuda(device)
    import torch

    from .moe import MoeGroupedWeights, expert_shard_range
    prefixes = list(expert_prefixes)
    if not prefixes:
        raise WeightError("MoeGroupedWeights: no experts")
    total = len(prefixes)
    first, last = expert_shard_range(total, rank, world)
    prefixes = prefixes[first:last]
    dims = {0: (inter, hidden), 1: (inter, hidden), 2: (hidden, inter)}
    banks = []
    per_expert = [[read_nvfp4_module(weights, f"{p}.{names[i]}", *dims[i], sfx) for i in range(3)] for p in prefixes]
    for e, (g, u, _) in enumerate(per_expert):
        if abs(float(g.stored_input_global) - float(u.stored_input_global)) > 1e-6:
            raise WeightError(f"expert {first + e}: gate and up have different input_global_scale "
                              f"({g.stored_input_global} vs {u.stored_input_global})")
    for i in range(3):
        parts = [pe[i] for pe in per_expert]
        packed = torch.from_numpy(np.stack([p.packed for p in parts])).to(device)
        scales = torch.from_numpy(np.stack([p.scales_swizzled for p in parts])).to(device)
        # the grouped kernels keep activations in bf16: multiplier = reciprocal of the weight global alone
        alphas = torch.tensor([float(np.float32(p.weight_alpha) * np.float32(p.stored_input_global)) for p in parts],
                              dtype=torch.float32, device=device)
        banks.append((packed, scales, alphas))
    return MoeGroupedWeights(banks[0], banks[1], banks[2], hidden, inter, len(prefixes), first, total)
