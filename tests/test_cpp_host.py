"""The C++ host layer (include/nvk_b200_host.hpp) driven by a C++ program, checked against the oracle.

The program (tests/cpp/host_check.cpp) is compiled here with g++ and linked against the host emulation of
the library, so it runs without a GPU: operands are written to a directory, the program runs a linear
(plain, M = 1, residual update, RMSNorm in front), an MLP and a grouped MoE decode step through the host
layer, and its outputs are compared with the oracle's with the bounds of the Python-driven tests."""
import pathlib
import subprocess

import numpy as np

from oracle import ref
from tests import _util as U

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _build_program() -> pathlib.Path:
    from tests.emu import harness as H
    lib = pathlib.Path(H._build_module().build())
    exe = lib.parent / "host_check"
    src = ROOT / "tests" / "cpp" / "host_check.cpp"
    hdrs = [ROOT / "include" / "nvk_b200_host.hpp", ROOT / "include" / "nvk_b200.h"]
    if not exe.exists() or exe.stat().st_mtime < max(f.stat().st_mtime for f in [src, lib, *hdrs]):
        subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Werror", f"-I{ROOT / 'include'}", str(src), "-o", str(exe),
                        f"-L{lib.parent}", "-lnvk_b200_emu", f"-Wl,-rpath,{lib.parent}"], check=True)
    return exe


def _weight(rng, n, k, std=0.02):
    w = U.gauss_bf16(rng, (n, k), std)
    return ref.quantize_weight_bf16(w)     # packed, swizzled scales, alpha


def test_cpp_host_layer_matches_the_oracle(tmp_path):
    exe = _build_program()
    rng = np.random.default_rng(2024)
    d = tmp_path
    meta = {}

    def put(name, a):
        np.ascontiguousarray(a).tofile(d / name)

    # linear
    m, n, k, eps = 11, 256, 512, 1e-6
    lp, ls, la = _weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    resid = U.gauss_bf16(rng, (m, n), 2.0)
    nw = U.gauss_bf16(rng, (k,), 1.0)
    meta.update(lin_m=m, lin_n=n, lin_k=k, lin_alpha=la, eps=eps)
    put("lin_packed.bin", lp), put("lin_scales.bin", ls), put("lin_x.bin", x), put("lin_residual.bin", resid)
    put("lin_norm_w.bin", nw)
    # mlp
    mm, hidden, inter = 5, 256, 384
    g, u, dn = _weight(rng, inter, hidden), _weight(rng, inter, hidden), _weight(rng, hidden, inter)
    xm = U.gauss_bf16(rng, (mm, hidden))
    meta.update(mlp_m=mm, mlp_hidden=hidden, mlp_inter=inter, mlp_gate_alpha=g[2], mlp_up_alpha=u[2], mlp_down_alpha=dn[2])
    for name, w in (("gate", g), ("up", u), ("down", dn)):
        put(f"mlp_{name}_packed.bin", w[0]), put(f"mlp_{name}_scales.bin", w[1])
    put("mlp_x.bin", xm)
    # moe
    nt, E, topk, mh, mi = 3, 8, 2, 128, 256
    experts = [[_weight(rng, mi, mh, 0.05), _weight(rng, mi, mh, 0.05), _weight(rng, mh, mi, 0.05)] for _ in range(E)]
    for j, name in enumerate(("gate", "up", "down")):
        put(f"moe_{name}_packed.bin", np.stack([e[j][0] for e in experts]))
        put(f"moe_{name}_scales.bin", np.stack([e[j][1] for e in experts]))
        put(f"moe_{name}_alphas.bin", np.array([e[j][2] for e in experts], np.float32))
    xmoe = U.gauss_bf16(rng, (nt, mh))
    logits = rng.standard_normal((nt, E)).astype(np.float32)
    meta.update(moe_n=nt, moe_E=E, moe_topk=topk, moe_hidden=mh, moe_inter=mi)
    put("moe_x.bin", xmoe), put("moe_logits.bin", logits)
    (d / "meta.txt").write_text("".join(f"{k_} {float(v)!r}\n" for k_, v in meta.items()))

    r = subprocess.run([str(exe), str(d)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "host_check ok" in r.stdout, (r.stdout + r.stderr)[-3000:]
    # refusals surface as exceptions naming the entry point (K = 144: K % 32 for the residual form)
    assert "residual refusal: nvk_b200_linear_nvfp4_w4a16_residual -1" in r.stdout

    def out(name, dtype, shape):
        return np.fromfile(d / name, dtype=dtype).reshape(shape)

    want = ref.linear_w4a16_f64(lp, ls, x, la, n, k)
    y = out("out_lin.bin", np.uint16, (m, n))
    assert U.rel_err_floor(ref.bf16_to_f32(y), want) < 1e-4 + 1e-2
    assert np.array_equal(out("out_lin_m1.bin", np.uint16, (n,)), y[0])            # a row's bits do not depend on M
    assert "tp fused: 1 err 0" in r.stdout
    assert np.array_equal(out("out_lin_tp1.bin", np.uint16, (8, n)), y[:8])        # a world of one: the plain linear
    yr = out("out_lin_residual.bin", np.uint16, (m, n))
    assert U.rel_err_floor(ref.bf16_to_f32(yr), want + ref.bf16_to_f32(resid).astype(np.float64)) < 1e-4 + 1e-2
    xf = ref.bf16_to_f32(x)
    rstd = (1.0 / np.sqrt((xf.astype(np.float64) ** 2).mean(1) + eps)).astype(np.float32)
    rows = ref.f32_to_bf16((xf * rstd[:, None]) * ref.bf16_to_f32(nw)[None, :])
    want_n = ref.linear_w4a16_f64(lp, ls, rows, la, n, k)
    yn = out("out_lin_prenorm.bin", np.uint16, (m, n))
    assert U.rel_err_floor(ref.bf16_to_f32(yn), want_n) < 2e-2
    assert np.array_equal(out("out_lin_prenorm_few.bin", np.uint16, (8, n)), yn[:8])   # fused norm == norm kernel + linear

    gate = ref.f32_to_bf16(ref.linear_w4a16_f64(g[0], g[1], xm, g[2], inter, hidden).astype(np.float32))
    up = ref.f32_to_bf16(ref.linear_w4a16_f64(u[0], u[1], xm, u[2], inter, hidden).astype(np.float32))
    act = ref.f32_to_bf16(ref.silu_mul(gate, up, round_bf16=True))
    want_mlp = ref.linear_w4a16_f64(dn[0], dn[1], act, dn[2], hidden, inter)
    assert U.rel_err_floor(ref.bf16_to_f32(out("out_mlp.bin", np.uint16, (mm, hidden))), want_mlp) < 2e-2

    ids, wts = ref.moe_route_topk(logits, topk)
    assert np.array_equal(out("out_moe_ids.bin", np.int32, (nt, topk)), ids)
    assert out("out_moe_status.bin", np.int32, (1,))[0] == 0
    want_moe = np.zeros((nt, mh), np.float64)
    for t in range(nt):
        for j in range(topk):
            (pg, sg, ag), (pu, su, au), (pd, sd, ad) = experts[ids[t, j]]
            gt = ref.f32_to_bf16(ref.linear_w4a16_f64(pg, sg, xmoe[t:t + 1], ag, mi, mh).astype(np.float32))
            ut = ref.f32_to_bf16(ref.linear_w4a16_f64(pu, su, xmoe[t:t + 1], au, mi, mh).astype(np.float32))
            a = ref.f32_to_bf16(ref.silu_mul(gt, ut, round_bf16=True))
            dd = ref.f32_to_bf16(ref.linear_w4a16_f64(pd, sd, a, ad, mh, mi).astype(np.float32))
            want_moe[t] += np.float64(wts[t, j]) * ref.bf16_to_f32(dd)[0].astype(np.float64)
    assert U.rel_err_floor(out("out_moe.bin", np.float32, (nt, mh)), want_moe) < 1e-2
