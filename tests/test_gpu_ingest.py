"""Checkpoint -> device: linears built from safetensors files run on the CUDA library and agree with
the oracle; both tensor-name layouts give the same linear; expert banks built from disk equal the
banks built from device linears byte for byte."""
import numpy as np
import pytest
import torch

from oracle import ref
from speaches_plus_b200 import weights as W
from tests import _util as U
from tests.test_gpu_linear import TOL_F64
from tests.test_weights_ingest import ct_tensors, make_module, modelopt_tensors, write_safetensors

pytestmark = pytest.mark.gpu


def test_linear_from_disk_both_layouts(tmp_path):
    U.require_gpu()
    rng = np.random.default_rng(21)
    n, k = 512, 1024
    packed, lin, g = make_module(rng, n, k)
    gx = np.float32(8.0)  # a power of two: its reciprocal's reciprocal is exact, so both layouts give the same bits
    t = ct_tensors("ct.proj", packed, lin, g, gx)
    t.update(modelopt_tensors("mo.proj", packed, lin, g, gx))
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", t))
    a = W.nvfp4_linear_from_disk(wl, "ct.proj", n, k, "cuda")
    b = W.nvfp4_linear_from_disk_with_suffixes(wl, "mo.proj", n, k, "cuda", W.Nvfp4Suffixes.GEMMA_MODELOPT)
    assert a.input_stored_global == 8.0 and abs(b.input_stored_global / 8.0 - 1) < 3e-7
    # activations stay bf16 on this route: the multiplier is the reciprocal of the weight global alone
    alpha = float(np.float32(1) / g)
    assert abs(a.alpha_w4a16 / alpha - 1) < 3e-7
    for m in (1, 5):
        x = U.gauss_bf16(rng, (m, k))
        xt = U.dev(x).view(torch.bfloat16)
        ya, yb = a.forward(xt), b.forward(xt)
        torch.cuda.synchronize()
        want = ref.linear_w4a16_f64(packed, ref.swizzle_scales(lin), x, alpha, n, k)
        assert U.rel_err_floor(ya.float().cpu().numpy(), want) < TOL_F64
        assert U.rel_err_floor(yb.float().cpu().numpy(), want) < TOL_F64


def test_fused_pair_from_disk_equals_the_two_linears(tmp_path):
    U.require_gpu()
    rng = np.random.default_rng(22)
    n, k = 256, 512
    pg, lg, g = make_module(rng, n, k, stored_global=3000.0)
    pu, lu, _ = make_module(rng, n, k, stored_global=3000.0)
    t = ct_tensors("mlp.gate_proj", pg, lg, g)
    t.update(ct_tensors("mlp.up_proj", pu, lu, g))
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", t))
    fused = W.nvfp4_linear_from_disk_fused_pair(wl, "mlp.gate_proj", "mlp.up_proj", n, k, "cuda")
    gate = W.nvfp4_linear_from_disk(wl, "mlp.gate_proj", n, k, "cuda")
    up = W.nvfp4_linear_from_disk(wl, "mlp.up_proj", n, k, "cuda")
    x = U.dev(U.gauss_bf16(rng, (3, k))).view(torch.bfloat16)
    # The split of K over CTAs is chosen from the number of rows; pin it so that the fused and the
    # separate launches add each row's products in the same order.
    assert U.ffi.call("nvk_b200_set_tuning", 1, 0) == 0
    try:
        yf, yg, yu = fused.forward(x), gate.forward(x), up.forward(x)
        torch.cuda.synchronize()
    finally:
        U.ffi.call("nvk_b200_set_tuning", 0, 0)
    # rows are computed independently of their neighbours: the fused linear is the two, bit for bit
    assert torch.equal(yf[:, :n].contiguous().view(torch.int16), yg.view(torch.int16))
    assert torch.equal(yf[:, n:].contiguous().view(torch.int16), yu.view(torch.int16))


def test_load_linear_maybe_quant_dispatch(tmp_path):
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(23)
    big_p, big_l, big_g = make_module(rng, 256, 256)
    small_p, small_l, small_g = make_module(rng, 64, 64)
    plain = U.gauss_bf16(rng, (128, 256), 0.02)
    t = ct_tensors("model.big", big_p, big_l, big_g)
    t.update(ct_tensors("model.small", small_p, small_l, small_g))
    t["lm_head.weight"] = ("BF16", plain.shape, plain.tobytes())
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", t))
    q = W.QuantizationConfig(W.QuantScheme.NVFP4, ["lm_head"], 16)
    big = W.load_linear_maybe_quant(wl, "model.big.weight", 256, 256, q, "cuda")
    small = W.load_linear_maybe_quant(wl, "model.small.weight", 64, 64, q, "cuda")
    head = W.load_linear_maybe_quant(wl, "lm_head.weight", 128, 256, q, "cuda")
    assert isinstance(big, sp.Nvfp4Linear) and isinstance(small, sp.Bf16Linear) and isinstance(head, sp.Bf16Linear)
    # the small module holds exactly the oracle's bf16 expansion
    want = ref.dequantize_to_bf16(small_p, ref.swizzle_scales(small_l), 64, 64, float(np.float32(1) / small_g))
    assert np.array_equal(U.host_u16(small.weight), want)
    assert np.array_equal(U.host_u16(head.weight), plain)
    x = U.gauss_bf16(rng, (1, 64))
    y = small.forward(U.dev(x).view(torch.bfloat16))
    torch.cuda.synchronize()
    ref_y = ref.bf16_to_f32(want).astype(np.float64) @ ref.bf16_to_f32(x)[0].astype(np.float64)
    assert U.rel_err_floor(y.float().cpu().numpy()[0], ref_y) < TOL_F64
    with pytest.raises(W.WeightError, match="expected"):
        W.load_linear_maybe_quant(wl, "lm_head.weight", 256, 256, q, "cuda")


def test_expert_banks_from_disk_equal_banks_from_device_linears(tmp_path):
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(24)
    E, hidden, inter = 16, 256, 384
    t, experts = {}, []
    for e in range(E):
        trip = []
        for name, (n, k) in (("gate_proj", (inter, hidden)), ("up_proj", (inter, hidden)),
                             ("down_proj", (hidden, inter))):
            p, l, g = make_module(rng, n, k)
            t.update(ct_tensors(f"experts.{e}.{name}", p, l, g))
            trip.append(sp.Nvfp4Linear.new_nvfp4(U.dev(p), U.dev(ref.swizzle_scales(l)), float(np.float32(1) / g), k, n))
        experts.append(tuple(trip))
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", t))
    disk = W.moe_grouped_weights_from_disk(wl, [f"experts.{e}" for e in range(E)], hidden, inter, "cuda")
    dev = sp.MoeGroupedWeights.build_from_experts(experts)
    assert (disk.hidden, disk.inter, disk.num_experts) == (dev.hidden, dev.inter, dev.num_experts)
    for a, b in zip((disk.gate, disk.up, disk.down), (dev.gate, dev.up, dev.down)):
        assert torch.equal(a[0].reshape(-1), b[0].reshape(-1))
        assert torch.equal(a[1].reshape(-1), b[1].reshape(-1))
        assert torch.equal(a[2], b[2])
    # and the banks run: one decode step over them agrees between the two constructions
    ctx = sp.GroupedDecodeContext(disk, 8, 4, "cuda")
    x = U.dev(U.gauss_bf16(rng, (3, hidden))).view(torch.bfloat16)
    logits = U.dev(rng.standard_normal((3, E)).astype(np.float32))
    y1 = sp.forward_grouped_decode(disk, ctx, x, logits).clone()
    y2 = sp.forward_grouped_decode(dev, ctx, x, logits).clone()
    torch.cuda.synchronize()
    assert torch.equal(y1, y2) and bool(torch.isfinite(y1.float()).all())
