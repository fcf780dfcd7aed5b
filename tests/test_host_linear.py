"""Host-side rules of the NVFP4 linear that need no GPU: constructor refusals
(rust/crates/nv-layers/src/linear.rs:1565-1579, 2059-2120; tests/linear_quant.rs bad-shape cases),
buffer sizes, the W4A16 multiplier."""
import numpy as np
import pytest
import torch

import speaches_plus_b200 as sp
from speaches_plus_b200 import linear as L


def parts(n, k):
    return (torch.zeros((n, k // 2), dtype=torch.uint8), torch.zeros(L.swizzled_scale_bytes(n, k), dtype=torch.uint8))


def test_swizzled_scale_bytes():
    assert L.swizzled_scale_bytes(4096, 4096) == 4096 * 256          # no padding at the benchmark shapes
    assert L.swizzled_scale_bytes(130, 144) == 256 * 12               # rows to 128, blocks to 4
    assert L.swizzled_scale_bytes(768, 2048) * 2 + 768 * 2048 // 2 * 2 + L.swizzled_scale_bytes(2048, 768) + 2048 * 768 // 2 \
        == 2_654_208                                                  # bytes of one expert of the MoE benchmark (768 x 2048 x 3 matrices)


def test_constructor_refusals():
    p, s = parts(128, 128)
    sp.Nvfp4Linear.new_nvfp4(p, s, 0.5, 128, 128)
    with pytest.raises(ValueError, match="multiple of 16"):
        sp.Nvfp4Linear.new_nvfp4(p, s, 0.5, 136, 128)
    with pytest.raises(ValueError, match="MIN_TILE"):
        sp.Nvfp4Linear.new_nvfp4(*parts(64, 128), 0.5, 128, 64)
    with pytest.raises(ValueError, match="MIN_TILE"):
        sp.Nvfp4Linear.new_nvfp4(*parts(128, 64), 0.5, 64, 128)
    with pytest.raises(ValueError, match="wrong number of bytes"):
        sp.Nvfp4Linear.new_nvfp4(p[:100], s, 0.5, 128, 128)
    with pytest.raises(ValueError, match="scale buffer too small"):
        sp.Nvfp4Linear.new_nvfp4(p, s[:100], 0.5, 128, 128)


def test_forward_checks_the_input_width_before_any_launch():
    lin = sp.Nvfp4Linear.new_nvfp4(*parts(128, 128), 0.5, 128, 128)
    with pytest.raises(ValueError, match="input last dim 64 != 128"):
        lin.forward(torch.zeros((1, 64), dtype=torch.bfloat16))


def test_w4a16_multiplier_drops_the_input_global():
    p, s = parts(128, 128)
    plain = sp.Nvfp4Linear.new_nvfp4(p, s, 0.25, 128, 128)
    assert plain.alpha_w4a16 == 0.25 and plain.nvfp4_parts()[2] == 0.25
    ckpt = sp.Nvfp4Linear.new_nvfp4_scaled(p, s, 128, 128, None, float(np.float32(0.25) * np.float32(1 / 8)), 8.0)
    assert ckpt.alpha_w4a16 == 0.25 and ckpt.nvfp4_parts_full()[3] == 8.0


def test_stored_global_rule():
    assert L.stored_global_from_amax(0.0) == 1.0 and L.stored_global_from_amax(float("inf")) == 1.0
    assert L.stored_global_from_amax(0.5) == 448.0 * 6.0 / 0.5


def test_moe_block_constructor_refusals():
    """rust/crates/nv-layers/src/moe.rs:33-80: expert count, top-k range, router shape."""
    def banks(E, hidden=128, inter=128):
        z = (torch.zeros((E, 1), dtype=torch.uint8),) * 2 + (torch.zeros(E),)
        return sp.MoeGroupedWeights(z, z, z, hidden, inter, E)

    def router(E, hidden=128):
        return sp.Bf16Linear(torch.zeros((E, hidden), dtype=torch.bfloat16))

    cfg = sp.MoeConfig(128, 4, 2, 128)
    sp.MoeBlock(cfg, router(4), banks(4))
    with pytest.raises(ValueError, match="experts=3"):
        sp.MoeBlock(cfg, router(4), banks(3))
    with pytest.raises(ValueError, match="num_experts_per_tok=5"):
        sp.MoeBlock(sp.MoeConfig(128, 4, 5, 128), router(4), banks(4))
    with pytest.raises(ValueError, match="num_experts_per_tok=0"):
        sp.MoeBlock(sp.MoeConfig(128, 4, 0, 128), router(4), banks(4))
    with pytest.raises(ValueError, match="gate shape mismatch"):
        sp.MoeBlock(cfg, router(5), banks(4))
    with pytest.raises(ValueError, match="configured sizes"):
        sp.MoeBlock(cfg, router(4), banks(4, inter=256))
    with pytest.raises(ValueError, match="come together"):
        sp.MoeBlock(cfg, router(4), banks(4), shared_expert=object())
    blk = sp.MoeBlock(cfg, router(4), banks(4))
    with pytest.raises(ValueError, match="last dim 64 != hidden_size 128"):
        blk.forward(torch.zeros((1, 64), dtype=torch.bfloat16))


def test_draft_twin_range_check_needs_no_device():
    lin = sp.Bf16Linear(torch.zeros((256, 128), dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="out of range"):
        lin.nvfp4_draft_twin_rows(200, 128)
    with pytest.raises(ValueError, match="out of range"):
        lin.nvfp4_draft_twin_rows(0, 0)
    with pytest.raises(ValueError, match="2-D"):
        sp.Nvfp4Linear.from_bf16_quantized_nvfp4(torch.zeros(4, dtype=torch.bfloat16))


def test_persistent_step_protocol_cannot_deadlock():
    """A model of the persistent step's scheduling (csrc/w4a16_stack.cu): every CTA walks the
    operations in order, claims items from a per-operation counter, and an item may only run once the
    operation it depends on has counted all of its items.  Under any interleaving -- here random
    ones, with far fewer CTAs than items -- every item runs exactly once and never before its
    dependency is complete; a CTA blocked on a dependency is always waiting for items that other CTAs
    hold and can finish."""
    import random
    for seed in range(50):
        rnd = random.Random(seed)
        n_ops = rnd.randint(1, 8)
        items = [rnd.randint(1, 12) for _ in range(n_ops)]
        deps = [rnd.randint(-1, o - 1) for o in range(n_ops)]
        n_cta = rnd.randint(1, 5)
        next_item, done = [0] * n_ops, [0] * n_ops
        ran = [[0] * items[o] for o in range(n_ops)]
        # per CTA: (operation, claimed item or None)
        state = [[0, None] for _ in range(n_cta)]
        steps = 0
        while any(s[0] < n_ops for s in state):
            steps += 1
            assert steps < 100000, "no progress: deadlock"
            live = [c for c in range(n_cta) if state[c][0] < n_ops]
            c = rnd.choice(live)
            o, item = state[c]
            if item is None:                      # claim
                item = next_item[o]
                next_item[o] += 1
                if item >= items[o]:
                    state[c] = [o + 1, None]      # nothing left in this operation
                else:
                    state[c][1] = item
                continue
            if deps[o] >= 0 and done[deps[o]] < items[deps[o]]:
                continue                          # still waiting (weights already in flight)
            ran[o][item] += 1
            if deps[o] >= 0:
                assert done[deps[o]] == items[deps[o]]
            done[o] += 1
            state[c][1] = None
        assert all(all(v == 1 for v in r) for r in ran) and done == items


# ---- the GEMM runner's host logic (rust/crates/nv-quant/src/nvfp4.rs:359-1084) ----

def test_runner_knob_parsers_follow_the_reference_pins():
    from speaches_plus_b200 import runner as R
    # nvfp4.rs:1133-1170 (streamk_k256_gate_tests and the sibling gates)
    assert not R.streamk_k256_from(None) and not R.streamk_k256_from("") and not R.streamk_k256_from("0")
    assert R.streamk_k256_from("1") and R.streamk_k256_from("yes")
    assert R.k256_from(None) and R.k256_from("1") and not R.k256_from("0")
    assert R.skinny_lt_from(None) and not R.skinny_lt_from("0")
    assert R.streamk_down_splits_from(None) == 0 and R.streamk_down_splits_from("1") == 0
    assert R.streamk_down_splits_from(" 4 ") == 4 and R.streamk_down_splits_from("x") == 0
    assert R.streamk_mode_from("0") is R.StreamkMode.NEVER and R.streamk_mode_from("1") is R.StreamkMode.ALWAYS
    assert R.streamk_mode_from(None) is R.StreamkMode.AUTO
    assert R.Nvfp4Backend.from_env("CUBLAS ") is R.Nvfp4Backend.CUBLASLT
    assert R.Nvfp4Backend.from_env("bogus") is R.Nvfp4Backend.AUTO


def test_runner_scheduler_rule():
    from speaches_plus_b200 import runner as R
    # nvfp4.rs:1116-1124 skinny_tiles_covers_verify_shapes_not_prefill
    assert R.skinny_tiles(128, 5376) and R.skinny_tiles(128, 5376 * 2) and R.skinny_tiles(128, 20480)
    assert not R.skinny_tiles(128, 43008) and not R.skinny_tiles(2048, 5376) and not R.skinny_tiles(1024, 43008)
    # the 148-SM addition: 640 tiles leave a last wave of 48; 3200 tiles are 21 waves and a bit
    assert R.ragged_last_wave(2048, 5120) and not R.ragged_last_wave(2048, 25600)
    assert not R.ragged_last_wave(128 * 148, 128)          # exactly one wave
    r = R.Nvfp4GemmRunner(env={})
    assert r.streamk_wanted(2048, 5120) and not r.streamk_wanted(2048, 25600)
    assert not R.Nvfp4GemmRunner(env={"NV_NVFP4_STREAMK": "0"}).streamk_wanted(128, 128)
    assert R.Nvfp4GemmRunner(env={"NV_NVFP4_STREAMK": "1"}).streamk_wanted(8192, 8192)
    assert R.Nvfp4GemmRunner(env={"SPEACHES_NVFP4_BACKEND": "cublaslt"}).backend is R.Nvfp4Backend.CUBLASLT
    assert R.Nvfp4GemmRunner(env={"SPEACHES_NVFP4_BACKEND": "nonsense"}).backend is R.Nvfp4Backend.AUTO


def test_runner_library_backend_and_shape_refusals(monkeypatch):
    """nvfp4.rs:564-590: k % 16, n and k at least 128 for every backend, m at least 128 for the library
    route, which is given the host copy of alpha and the stream's workspace."""
    import pytest
    from speaches_plus_b200 import runner as R
    monkeypatch.setattr(R, "ensure_workspace_for_stream", lambda: None)
    r = R.Nvfp4GemmRunner(env={})
    with pytest.raises(ValueError, match="multiple of 16"):
        r.matmul(None, None, None, None, None, None, 128, 128, 136)
    with pytest.raises(ValueError, match="n,k >= 128"):
        r.matmul(None, None, None, None, None, None, 128, 64, 128)
    with pytest.raises(ValueError, match="m >= 1"):
        r.matmul(None, None, None, None, None, None, 0, 128, 128)
    lt = R.Nvfp4GemmRunner(env={"SPEACHES_NVFP4_BACKEND": "cublaslt"})
    with pytest.raises(ValueError, match="alpha_host"):
        lt.matmul(None, None, None, None, None, None, 128, 128, 128)
    with pytest.raises(ValueError, match="requires m >= 128"):
        lt.matmul(None, None, None, None, None, None, 64, 128, 128, alpha_host=1.0)


def test_runner_choice_tree_and_permanent_fallback(monkeypatch):
    from speaches_plus_b200 import runner as R
    tiled, sk, dp = ("nv_kernels_cutlass_fp4_gemm_sm120_bf16_tiled", "nv_kernels_cutlass_fp4_gemm_sm120_bf16_streamk",
                     "nv_kernels_cutlass_fp4_gemm_sm120_bf16")
    r = R.Nvfp4GemmRunner(env={})
    assert r.plan(256, 256, 512, False) == (tiled, (1, 0))          # K % 256 == 0: the K256 tile id
    assert r.plan(256, 256, 384, False) == (dp, ())
    assert r.plan(256, 256, 512, True) == (sk, ())                   # stream-K K256 ships off
    assert R.Nvfp4GemmRunner(env={"NV_NVFP4_STREAMK_K256": "1"}).plan(256, 256, 512, True) == (tiled, (1, 1))
    assert R.Nvfp4GemmRunner(env={"NV_NVFP4_STREAMK_DOWN_SPLITS": "4"}).plan(256, 256, 512, True) == (tiled, (0, 4))
    assert R.Nvfp4GemmRunner(env={"NV_NVFP4_K256": "0"}).plan(256, 256, 512, False) == (dp, ())
    # a failing stream-K launch falls back to the data-parallel scheduler and stays there
    calls = []

    def fake_launch(self, entry, extra, *a):
        calls.append(entry)
        return -1 if "streamk" in entry else 0

    monkeypatch.setattr(R.Nvfp4GemmRunner, "_launch", fake_launch)
    monkeypatch.setattr(R, "ensure_workspace_for_stream", lambda: None)
    r = R.Nvfp4GemmRunner(env={"NV_NVFP4_STREAMK": "1", "NV_NVFP4_K256": "0"})
    r.matmul(None, None, None, None, None, None, 128, 128, 384)
    assert calls == [sk, dp] and r.streamk_failed
    calls.clear()
    r.matmul(None, None, None, None, None, None, 128, 128, 384)
    assert calls == [dp]


def test_backend_registry_knows_one_backend():
    """rust/crates/nv-layers/src/backend.rs:16-233: the selection values parse as in the reference; only
    cuda resolves, and it serves every kernel id of the path."""
    import pytest

    from speaches_plus_b200 import backend as B
    assert B.BackendSel.parse(" AUTO ") is B.BackendSel.AUTO and B.BackendSel.parse("") is B.BackendSel.AUTO
    assert B.BackendSel.parse("wgpu") is B.BackendSel.WGPU and B.BackendSel.parse("metal") is None
    assert B.BackendSel.from_env({}) is B.BackendSel.AUTO
    assert B.BackendSel.from_env({B.BACKEND_ENV: "Cuda"}) is B.BackendSel.CUDA
    with pytest.raises(B.BackendError, match="not one of auto"):
        B.BackendSel.from_env({B.BACKEND_ENV: "vulkan"})
    assert B.resolve(B.BackendSel.AUTO) is B.BackendKind.CUDA and B.resolve(B.BackendSel.CUDA) is B.BackendKind.CUDA
    for sel in (B.BackendSel.CPU, B.BackendSel.WGPU):
        with pytest.raises(B.BackendError, match="no CPU or wgpu fallback"):
            B.resolve(sel)
    assert all(B.kind_supports(B.BackendKind.CUDA, k) for k in B.KernelId)
    assert B.missing_on(B.BackendKind.CPU, list(B.KernelId)) == list(B.KernelId)
    assert B.supporting_backends(B.KernelId.GEMV_NVFP4) == [B.BackendKind.CUDA]
    assert B.library_for(B.KernelId.GEMM_NVFP4) == "libnvk_b200_prefill.so"
    assert B.library_for(B.KernelId.GEMV_NVFP4) == "libnvk_b200.so"
    assert str(B.BackendKind.CUDA) == "cuda"


# ---- stream epochs and activation staging (rust/crates/nv-layers/tests/nvfp4_staging_lifecycle.rs) ----
def test_stream_epoch_registry_bumps_and_reads():
    from speaches_plus_b200 import runner as R
    key = 0xDEADBEEF
    e0 = R.stream_epoch(key)
    R.bump_stream_epoch(key)
    R.bump_stream_epoch(key)
    assert R.stream_epoch(key) == e0 + 2
    assert R.stream_epoch(key ^ 1) == 0


def test_staging_evicts_on_epoch_bump_and_zeros_on_shrink():
    """The cache's rules, with numpy buffers standing in for device memory: the high-water mark tracks
    the live rows; fewer rows than last time zero the entry first; a released stream's entries are
    rebuilt under the new epoch; a capture that finds no entry gets None and creates nothing."""
    import numpy as np
    from speaches_plus_b200 import runner as R
    cache, key, allocs, zeroed = R.StagingCache(), 0x51A6E, [], []

    def alloc():
        allocs.append(1)
        return np.zeros(64, np.uint8), np.zeros(16, np.uint8)

    def zero(buf):
        zeroed.append(id(buf))
        buf[:] = 0

    e = cache.acquire(key, 128, 5, False, alloc, zero)
    e.packed[:] = 7                       # the quantizer wrote rows
    assert cache.diag(key, 128) == (R.stream_epoch(key), 5) and len(allocs) == 1 and not zeroed
    e2 = cache.acquire(key, 128, 9, False, alloc, zero)
    assert e2 is e and cache.diag(key, 128)[1] == 9 and not zeroed       # growing: nothing to clear
    e3 = cache.acquire(key, 128, 2, False, alloc, zero)
    assert e3 is e and cache.diag(key, 128)[1] == 2 and len(zeroed) == 2 and not e.packed.any()
    assert cache.acquire(key, 256, 130, True, alloc, zero) is None and len(allocs) == 1   # capturing, no entry
    assert cache.acquire(key, 128, 2, True, alloc, zero) is e                             # capturing, entry exists
    other = cache.acquire(key + 1, 128, 3, False, alloc, zero)
    epoch_before = cache.diag(key, 128)[0]
    R.release_stream_resources(key)
    e4 = cache.acquire(key, 128, 2, False, alloc, zero)
    assert e4 is not e and cache.diag(key, 128)[0] > epoch_before and len(allocs) == 3
    assert cache.acquire(key + 1, 128, 3, False, alloc, zero) is other    # another stream's entry survives
    assert cache.diag(key, 512) is None
