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
    # sigmoid router with a selection bias and a routed scaling (mode 1), top-4 of 40
    lg1 = rng.standard_normal((5, 40)).astype(np.float32)
    bias1 = (rng.standard_normal(40) * 0.1).astype(np.float32)
    ids1, wts1 = ref.moe_route_topk(lg1, 4, bias=bias1, mode=1, norm_topk=True, routed_scaling=2.5)
    out.update(router1_logits=lg1, router1_bias=bias1, router1_ids=ids1, router1_weights=wts1)
    # stable slot sort of the first router's ids: offsets, sorted slot -> token, slot -> sorted position
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable")
    inv = np.empty(flat.size, np.int32)
    inv[order] = np.arange(flat.size, dtype=np.int32)
    out.update(sort_offsets=np.concatenate([[0], np.cumsum(np.bincount(flat, minlength=128))]).astype(np.int32),
               sort_perm_token=(order // ids.shape[1]).astype(np.int32), sort_inv_perm=inv)
    # int8 activation rows (W4A8 route): exact integers and scales, the product with and without a residual
    x8 = (rng.standard_normal((3, k)) * np.array([[0.3], [1.0], [4.0]])).astype(np.float32)
    q8, s8 = ref.rowquant_i8(x8)
    resid = ref.f32_to_bf16(rng.standard_normal((3, n)).astype(np.float32))
    out.update(x8_f32=x8, x8_q=q8, x8_scales=s8, w4a8_residual_bf16=resid,
               y_w4a8_f64=ref.linear_w4a8_f64(packed, sw, q8, s8, float(alpha), n, k),
               y_w4a8_residual_f64=ref.linear_w4a8_f64(packed, sw, q8, s8, float(alpha), n, k, resid))
    # residual RMSNorm: new residual (exact bits) and the normed row
    hx = ref.f32_to_bf16(rng.standard_normal((2, 256)).astype(np.float32))
    hres = ref.f32_to_bf16(rng.standard_normal((2, 256)).astype(np.float32) * 2)
    hw = ref.f32_to_bf16((1.0 + 0.1 * rng.standard_normal(256)).astype(np.float32))
    res_out, normed = ref.rmsnorm_residual(hx, hres, hw, 1e-6)
    out.update(norm_x_bf16=hx, norm_res_bf16=hres, norm_w_bf16=hw, norm_res_out_bf16=res_out, norm_out_bf16=normed)
    return out


if __name__ == "__main__":
    path = pathlib.Path(__file__).with_name("nvfp4_small.npz")
    np.savez_compressed(path, **build())
    print(path, path.stat().st_size, "bytes")
