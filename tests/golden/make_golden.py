"""Writes tests/golden/nvfp4_small.npz: seeded inputs and the CPU oracle's outputs for one small case
of every stage of the NVFP4 linear path.

Provenance: the reference is Rust and cannot be run where these were made, and it ships no golden
files for this path, so the outputs come from the oracle (oracle/nvfp4_oracle.c) AFTER it has been
pinned to the reference's known-answer tests (tests/test_oracle_kats.py).  The file freezes those
answers: a later change to the oracle or to a kernel that moves any of them fails the fixture tests.
Byte, index and bf16-bit arrays are exact expectations; `y_f64` is the f64 statement of the
contraction, compared within the tolerance the tests write down.

Run from the repository root:  python tests/golden/make_golden.py
"""
import pathlib
import sys

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import ref  # noqa: E402

SEED = 20240607


def build() -> dict:
    rng = np.random.default_rng(SEED)
    out = {}
    # weight [N, K] ~ N(0, 0.02) as bf16, quantized with global 448*6/amax (linear.rs:2161-2175)
    n, k = 128, 512
    w = ref.f32_to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    g = np.float32(ref.weight_global(ref.bf16_to_f32(w)))
    packed, lin = ref.quantize_rows_bf16(w, float(g))
    sw = ref.swizzle_scales(lin)
    alpha = np.float32(1.0) / g
    out.update(w_bf16=w, w_global=np.array([g], np.float32), w_packed=packed, w_scales_linear=lin,
               w_scales_swizzled=sw, alpha=np.array([alpha], np.float32))
    # activations [M, K] ~ N(0, 1) as bf16; W4A16 linear in f64 and through the Cpu-backend linear
    x = ref.f32_to_bf16(rng.standard_normal((5, k)).astype(np.float32))
    out["x_bf16"] = x
    out["y_f64"] = ref.linear_w4a16_f64(packed, sw, x, float(alpha), n, k)
    out["w_dequant_bf16"] = ref.dequantize_to_bf16(packed, sw, n, k, float(alpha))
    out["y_cpu_backend_bf16"] = ref.linear_cpu_backend(out["w_dequant_bf16"], x, threads=1)
    # activation quantizer (global 1.0, rows padded to 128) and the W4A4 product
    a_packed, a_lin = ref.quantize_rows_bf16(x, 1.0, m_padded=128)
    out.update(a_packed=a_packed, a_scales_linear=a_lin, a_scales_swizzled=ref.swizzle_scales(a_lin))
    out["d_w4a4_bf16"] = ref.matmul_w4a4(a_packed, a_lin, packed, lin, 128, n, k, float(alpha))[:5]
    # SwiGLU activation, both roundings
    gate = ref.f32_to_bf16(rng.standard_normal((2, 64)).astype(np.float32) * 2)
    up = ref.f32_to_bf16(rng.standard_normal((2, 64)).astype(np.float32))
    out.update(gate_bf16=gate, up_bf16=up, silu_mul_f32=ref.silu_mul(gate, up, round_bf16=False),
               silu_mul_bf16_rounded=ref.silu_mul(gate, up, round_bf16=True))
    # router: top-8 of 128, softmax over the winners
    logits = rng.standard_normal((6, 128)).astype(np.float32)
    logits[5, 10] = logits[5, 70] = logits[5].max() + 1  # a tie at the top: the lower index wins
    ids, wts = ref.moe_route_topk(logits, 8)
    out.update(router_logits=logits, router_ids=ids, router_weights=wts)
    return out


if __name__ == "__main__":
    path = pathlib.Path(__file__).with_name("nvfp4_small.npz")
    np.savez_compressed(path, **build())
    print(path, path.stat().st_size, "bytes")
