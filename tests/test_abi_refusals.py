"""Refusals of the C ABI, checked without a GPU: a refused call returns its code before any CUDA
call is made, so these run anywhere.  Order of the checks: empty problem (0), shape (-1), argument /
alignment (-2), resource (-3), grid axis (-9); a NULL operand is refused with -2 after the shape
checks."""
import speaches_plus_b200 as sp

f = sp.ffi.call
P = 0x1000   # a 16-byte aligned, non-null address; never dereferenced on a refused call
S = 0        # the default stream


def test_empty_problems_are_no_ops():
    assert f("nv_kernels_nvfp4_gemv_bf16act", S, 0, 0, 0, 0, 1.0, 0, 128) == 0
    assert f("nvk_b200_linear_nvfp4_w4a16", S, 0, 0, None, None, 0, None, 0, None, 1.0, 0.0, 4, 0, 128) == 0
    assert f("nv_kernels_quantize_nvfp4_bf16", S, 0, 0, 0, 1.0, 0, 0, 64) == 0
    assert f("nv_kernels_gemv_bf16", S, 0, 0, 0, 0, 64) == 0
    assert f("nv_kernels_moe_route_topk", S, 0, 0, 0, 0, 0, 8, 2, 0, 0.0, 1, 1.0) == 0
    assert f("nv_kernels_moe_permute", S, 0, 0, 0, 0, 0, 0, 2, 8) == 0
    assert f("nvk_b200_tp_allreduce_bf16", S, 0, 0, 2, 0, 0, 0, 64, 0, 0) == 0


def test_shape_refusals():
    assert f("nv_kernels_nvfp4_gemv_bf16act", S, P, P, P, P, 1.0, 64, 250) == -1              # K % 16
    assert f("nv_kernels_gemv_nvfp4_w4a16_dual_m1", S, P, P, None, None, P, P, None, 1.0, 1.0, 64, 48) == -1  # K % 32
    assert f("nv_kernels_gemv_nvfp4_w4a16_dual_m1", S, P, P, P, None, P, P, None, 1.0, 1.0, 64, 64) == -1     # half-null arm
    assert f("nv_kernels_gemv_nvfp4_w4a16_silu_gate_up_in_m1", S, P, P, P, P, P, 1.0, 0, 64) == -1
    assert f("nv_kernels_gemm_nvfp4_w4a16_mk_dual", S, P, P, None, None, P, P, None, 1.0, 1.0, 17, 64, 64) == -1  # M > 16
    assert f("nv_kernels_gemm_nvfp4_w4a16_mk_dual", S, P, P, None, None, P, P, None, 1.0, 1.0, 4, 48, 64) == -1   # N % 32
    assert f("nvk_b200_linear_nvfp4_w4a16", S, P, P, None, None, P, None, P, None, 1.0, 0.0, 65, 128, 128) == -1  # M > 64
    assert f("nv_kernels_quantize_nvfp4_bf16", S, P, P, P, 1.0, 4, 4, 40) == -1
    assert f("nvk_b200_moe_grouped_w4a16", S, P, P, None, None, P, None, P, None, None, P, None, None, P, None, 4, 64, 48, 8, 8, None) == -1
    assert f("nv_kernels_moe_grouped_fp4_gemv_m1_bf16", S, P, P, P, P, P, P, P, 4, 8, 64, 64, 100, 64) == -1    # tile stride


def test_argument_refusals():
    assert f("nv_kernels_nvfp4_gemv_bf16act", S, 0, 0, 0, 0, 1.0, 128, 128) == -2             # NULL operands
    assert f("nv_kernels_nvfp4_gemv_bf16act", S, P, P, P, 0, 1.0, 128, 128) == -2             # NULL output
    assert f("nv_kernels_gemv_nvfp4_w4a16_silu_gate_up_in_m1", S, P, P, P, 0, P, 1.0, 128, 128) == -2  # NULL up
    assert f("nv_kernels_quantize_nvfp4_bf16", S, P, P, P, 1.0, 4, 5, 64) == -2               # logical > padded rows
    assert f("nv_kernels_quantize_nvfp4_bf16", S, P + 2, P, P, 1.0, 4, 4, 64) == -2           # misaligned x
    assert f("nv_kernels_quantize_nvfp4_bf16", S, 0, P, P, 1.0, 4, 4, 64) == -2               # NULL x with live rows
    assert f("nv_kernels_gemv_bf16", S, 0, 0, 0, 4, 8) == -2
    assert f("nv_kernels_moe_route_topk", S, P, 0, P, P, 1, 8, 9, 0, 0.0, 1, 1.0) == -2       # K > E
    assert f("nv_kernels_moe_route_topk", S, 0, 0, 0, 0, 1, 8, 2, 0, 0.0, 1, 1.0) == -2       # NULL operands
    assert f("nv_kernels_moe_permute", S, 0, 0, 0, 0, 0, 4, 2, 8) == -2
    assert f("nv_kernels_moe_unpermute_scatter", S, P, P, P, P, 4, 2, 64, 32) == -2           # row stride < hidden
    assert f("nv_kernels_moe_grouped_fp4_gemv_m1_bf16", S, 4, P, P, P, P, P, P, 4, 8, 64, 64, 128, 64) == -2     # alignment
    assert f("nvk_b200_moe_route_permute", S, P, 0, P, P, P, P, P, None, None, 4, 8, 9, 0, 0.0, 1, 1.0) == -2
    assert f("nvk_b200_set_tuning", 3, 0) == -2 and f("nvk_b200_set_tuning", 0, 48) == -2
    assert f("nvk_b200_set_tuning", 0, 0) == 0
    assert f("nvk_b200_set_row_balance", 3) == -2 and f("nvk_b200_set_row_balance", -1) == -2
    assert f("nvk_b200_set_row_balance", 0) == 0
    assert f("nvk_b200_tp_allreduce_bf16", S, P, 2, 2, P, P, 8, 64, P, P) == -2               # rank outside the world
    assert f("nvk_b200_tp_allreduce_bf16", S, P, 0, 2, P, P, 12, 64, P, P) == -2              # n % 8
    assert f("nvk_b200_tp_allreduce_bf16", S, P, 0, 9, P, P, 8, 64, P, P) == -2               # more than 8 ranks


def test_resource_and_grid_refusals():
    assert f("nvk_b200_moe_route_permute", S, P, 0, P, P, P, P, P, None, None, 4, 257, 4, 0, 0.0, 1, 1.0) == -3   # > 256 experts
    assert f("nvk_b200_moe_route_permute", S, P, 0, P, P, P, P, P, None, None, 2000, 8, 4, 0, 0.0, 1, 1.0) == -3  # > 4096 slots
    assert f("nvk_b200_moe_permute_static", S, P, P, P, P, 4, 2, 4097) == -3
    assert f("nv_kernels_rmsnorm_quantize_nvfp4_bf16", S, P, P, P, P, 1.0, 1e-6, 1, 1, 32768) == -3  # row > 48 KiB
    assert f("nv_kernels_gather_rows_bf16_strided", S, P, P, P, 9, 64, 4, 4) == -3
    assert f("nv_kernels_moe_route_topk_shared_tail", S, P, 0, P, P, 1, 8, 2, 0, 0.0, 1, 1.0, -1) == -3
    assert f("nv_kernels_moe_grouped_fp4_gemv_m1_bf16", S, P, P, P, P, P, P, P, 70000, 8, 64, 64, 128, 64) == -9


def test_buffer_size_queries():
    lib = sp.ffi.lib()
    assert lib.nvk_b200_tp_allreduce_buffer_bytes(8, 64 * 5120) == 4096 + 2 * 8 * 64 * 5120 * 2
    assert lib.nvk_b200_tp_allreduce_buffer_bytes(9, 64) == 0 and lib.nvk_b200_tp_allreduce_buffer_bytes(2, 0) == 0
    assert lib.nvk_b200_linear_workspace_bytes(16, 4096) == 256 + 16 * 16 * 512
    assert lib.nvk_b200_linear_workspace_bytes(0, 4096) == 0


def test_w4a4_single_gemv_refusals():
    assert f("nv_kernels_nvfp4_gemv_bf16", S, P, P, P, P, P, 1.0, 0, 64) == 0
    assert f("nv_kernels_nvfp4_gemv_bf16", S, P, P, P, P, P, 1.0, 8, 40) == -1
    assert f("nv_kernels_nvfp4_gemv_bf16", S, P, P, 0, P, P, 1.0, 8, 64) == -2
    assert f("nv_kernels_nvfp4_gemv_bf16", S, P + 4, P, P, P, P, 1.0, 8, 64) == -2


def _stack_op(**kw):
    o = sp.ffi.NvkStackOp()
    for k, v in dict(wq_a=P, sc_a=P, x=P, y_a=P, N=128, K=128, dep=-1).items():
        setattr(o, k, v)
    for k, v in kw.items():
        setattr(o, k, v)
    return o


def _stack_build(ops, m=1, plan=P, nbytes=1 << 20):
    import ctypes as C
    arr = (sp.ffi.NvkStackOp * len(ops))(*ops)
    out = (C.c_int * 2)()
    return f("nvk_b200_stack_build", C.addressof(arr), len(ops), m, plan, nbytes, C.addressof(out))


def test_persistent_step_refusals():
    """nvk_b200_stack_build validates every operation before it touches the device."""
    lib = sp.ffi.lib()
    assert lib.nvk_b200_stack_plan_bytes(0) == 0 and lib.nvk_b200_stack_plan_bytes(1025) == 0
    assert lib.nvk_b200_stack_plan_bytes(4) >= 4 * 88 + 2 * 16
    assert _stack_build([_stack_op(K=48)]) == -1                  # K % 32
    assert _stack_build([_stack_op()], m=9) == -1                 # more than 8 tokens
    assert _stack_build([_stack_op(wq_b=P)]) == -1                # half-null second arm
    assert _stack_build([_stack_op(dep=0)]) == -2                 # may only wait for an earlier operation
    assert _stack_build([_stack_op(), _stack_op(dep=1)]) == -2
    assert _stack_build([_stack_op(x=0)]) == -2                   # NULL operand
    assert _stack_build([_stack_op(wq_a=P + 4)]) == -2            # alignment
    assert _stack_build([_stack_op(rows_per_item=64)]) == -2
    assert _stack_build([_stack_op()], nbytes=16) == -2           # plan buffer too small
    assert _stack_build([_stack_op()], plan=0) == -2
    assert f("nvk_b200_stack_run", S, 0, 1, 1, 148, 1024, P) == -2
    assert f("nvk_b200_stack_run", S, P, 1, 9, 148, 1024, P) == -2
    assert f("nvk_b200_stack_run", S, P, 1, 1, 0, 1024, P) == -2


def test_decode_step_wrapper_checks():
    import pytest
    import torch
    z = torch.zeros
    lin = sp.Nvfp4Linear.new_nvfp4(z((128, 64), dtype=torch.uint8), z(128 * 8, dtype=torch.uint8), 1.0, 128, 128)
    wide = sp.Nvfp4Linear.new_nvfp4(z((256, 64), dtype=torch.uint8), z(256 * 8, dtype=torch.uint8), 1.0, 128, 256)
    x, y = z((1, 128), dtype=torch.bfloat16), z((1, 128), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="1..8"):
        sp.DecodeStep(9, "cpu")
    step = sp.DecodeStep(1, "cpu")
    assert step.add(lin, x, y) == 0
    with pytest.raises(ValueError, match="earlier operation"):
        step.add(lin, x, y, dep=1)
    with pytest.raises(ValueError, match="come together"):
        step.add(lin, x, y, lin_b=lin)
    with pytest.raises(ValueError, match="same shape"):
        step.add(lin, x, y, lin_b=wide, y_b=z((1, 256), dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="contiguous bf16"):
        step.add(lin, z((1, 128)), y)
    with pytest.raises(ValueError, match="contiguous bf16"):
        step.add(lin, z((2, 128), dtype=torch.bfloat16), y)
    assert step.add(lin, y, x, x2=y, dep=0) == 1
    with pytest.raises(RuntimeError, match="build"):
        step.run()


def test_rowgate_refusals():
    assert f("nv_kernels_mul_sigmoid_rowgate_f32", S, P, P, P, 0, 64) == 0
    assert f("nv_kernels_mul_sigmoid_rowgate_f32", S, P, 0, P, 2, 64) == -2


def test_rmsnorm_refusals():
    assert f("nv_kernels_rmsnorm_bf16", S, P, P, P, 0, 64, 1e-6) == 0
    assert f("nv_kernels_rmsnorm_bf16", S, P, 0, P, 2, 64, 1e-6) == -2


def test_row_balance_rule():
    """The dealt launch is chosen exactly when the 128-row tile CTAs fit the GPU at once but unevenly."""
    g = lambda ctas, smem=90 * 1024, per_sm=3: f("nvk_b200_row_balance_grid", ctas, smem, per_sm)
    assert g(224) == 296          # 224 tiles, two 90 KiB CTAs per SM: 76 SMs would hold two tiles, 72 one
    assert g(150) == 296          # two SMs would do double work
    assert g(148) == 0 and g(100) == 0 and g(0) == 0      # at most one tile per SM: nothing to even out
    assert g(296) == 0            # two tiles on every SM already
    assert g(290) == 0            # ceil(2320 / 296) = 8 units per CTA: dealing would not lower the maximum
    assert g(297) == 0            # more than one wave at two CTAs per SM
    assert g(300, 60 * 1024) == 444   # three 60 KiB CTAs per SM are resident: one wave again
    assert g(224, 120 * 1024) == 0    # one 120 KiB CTA per SM: 224 tiles take two waves
    assert g(224, 90 * 1024, 1) == 0  # registers allow one CTA per SM


def test_library_route_refusals():
    """The cuBLASLt route refuses before it opens the library: empty problems are no-ops, the reference's
    shape rule for this route (k % 16, every dimension at least 128), null and misaligned operands."""
    g = lambda *a: f("nvk_b200_cublaslt_fp4_gemm_bf16", S, *a)
    assert g(0, 0, 0, 0, 0, 0, 128, 128, 1.0, 0, 0) == 0
    assert g(P, P, P, P, P, 128, 128, 136, 1.0, P, 1024) == -1      # k % 16
    assert g(P, P, P, P, P, 64, 128, 128, 1.0, P, 1024) == -1       # m < 128: pad the activation
    assert g(P, P, P, P, P, 128, 96, 128, 1.0, P, 1024) == -1
    assert g(P, P, P, P, P, 128, 128, 64, 1.0, P, 1024) == -1
    assert g(P, P, 0, P, P, 128, 128, 128, 1.0, P, 1024) == -2      # null weights
    assert g(P + 8, P, P, P, P, 128, 128, 128, 1.0, P, 1024) == -2  # misaligned activations
    assert g(P, P, P, P, P, 128, 128, 128, 1.0, 0, 1024) == -2      # workspace size without a workspace
    assert sp.ffi.prefill_lib().nvk_b200_cublaslt_fp4_workspace_bytes() == 64 << 20


def test_residual_linear_refusals():
    g = lambda *a: f("nvk_b200_linear_nvfp4_w4a16_residual", S, *a)
    assert g(0, 0, 0, None, 0, 0, 1.0, 4, 0, 128) == 0                   # empty problem
    assert g(P, P, P, None, P, P, 1.0, 0, 128, 128) == -1 and g(P, P, P, None, P, P, 1.0, 65, 128, 128) == -1
    assert g(P, P, P, None, P, P, 1.0, 4, 128, 144) == -1                # K % 32
    assert g(P, P, P, None, 0, P, 1.0, 4, 128, 128) == -2                # no residual
    assert g(P, P, P + 2, None, P, P, 1.0, 4, 128, 128) == -2            # misaligned x
    assert g(P, P, P, P + 4, P, P, 1.0, 4, 128, 128) == -2               # misaligned x2


def test_normed_linear_and_rstd_emit_refusals():
    g = lambda *a: f("nvk_b200_linear_nvfp4_w4a16_normed", S, *a)
    assert g(0, 0, None, None, 0, 0, None, 1e-6, 0, None, 1.0, 0.0, 1, 0, 128) == 0
    assert g(P, P, None, None, P, P, None, 1e-6, P, None, 1.0, 0.0, 9, 128, 128) == -1     # no rstd: M <= 8
    assert g(P, P, None, None, P, P, P, 1e-6, P, None, 1.0, 0.0, 65, 128, 128) == -1       # with rstd: M <= 64
    assert g(P, P, None, None, P, P, None, 1e-6, P, None, 1.0, 0.0, 1, 128, 144) == -1     # K % 32
    assert g(P, P, P, None, P, P, None, 1e-6, P, None, 1.0, 0.0, 1, 128, 128) == -1        # half-given second matrix
    assert g(P, P, None, None, P, 0, None, 1e-6, P, None, 1.0, 0.0, 1, 128, 128) == -2     # no norm weight
    assert g(P, P, None, None, P, P + 2, None, 1e-6, P, None, 1.0, 0.0, 1, 128, 128) == -2
    e = lambda *a: f("nvk_b200_linear_nvfp4_w4a16_residual_rstd_emit", S, *a)
    assert e(P, P, P, None, P, P, 1.0, 0, 1e-6, 128, 128) == -2                             # no pack
    assert e(P, P, P, None, P, P, 1.0, P, 1e-6, 0, 128) == 0
    assert e(P, P, P, None, 0, P, 1.0, P, 1e-6, 128, 128) == -2


def test_fused_linear_allreduce_refusals():
    g = lambda *a: f("nvk_b200_tp_linear_nvfp4_w4a16_allreduce", S, *a)
    assert g(P, 0, 2, P, P, P, None, None, P, 1.0, 1, 0, 128, 64, 8, P, P) == 0                 # empty problem
    assert g(P, 0, 2, P, P, P, None, None, P, 1.0, 9, 128, 128, 64, 8, P, P) == -1              # more rows than the buffers hold
    assert g(P, 0, 2, P, P, P, None, None, P, 1.0, 1, 128, 128, 64, 65, P, P) == -2             # row capacity > 64
    assert g(P, 0, 2, P, P, P, None, None, P, 1.0, 1, 128, 144, 64, 8, P, P) == -1              # K % 32
    assert g(P, 2, 2, P, P, P, None, None, P, 1.0, 1, 128, 128, 64, 8, P, P) == -2              # rank outside the world
    assert g(P, 0, 9, P, P, P, None, None, P, 1.0, 1, 128, 128, 64, 8, P, P) == -2              # more than 8 ranks
    assert g(0, 0, 2, P, P, P, None, None, P, 1.0, 1, 128, 128, 64, 8, P, P) == -2              # no buffers
    assert g(P, 0, 2, P, P, P, None, None, P, 1.0, 1, 128, 128, 64, 8, 0, P) == -2              # no call counters
    assert g(P, 0, 2, P, P, P + 4, None, None, P, 1.0, 1, 128, 128, 64, 8, P, P) == -2          # misaligned x
    assert f("nvk_b200_tp_fused_buffer_bytes", 0, 64, 8) == 0 and f("nvk_b200_tp_fused_buffer_bytes", 2, 5000, 8) == 0
    assert f("nvk_b200_tp_fused_buffer_bytes", 2, 64, 16) == 64 * 32 + 2 * 2 * 64 * 128 * 16 * 2


def test_combine_allreduce_refusals():
    g = lambda *a: f("nvk_b200_moe_combine_allreduce", S, *a)
    assert g(P, 0, 2, P, P, P, P, 0, 2, 256, 256, 8, None, 64, P, P) == 0                    # no tokens
    assert g(P, 0, 2, P, P, P, P, 1, 2, 252, 256, 8, None, 64, P, P) == -2                   # hidden % 8
    assert g(P, 0, 2, P, P, P, P, 1, 2, 256, 128, 8, None, 64, P, P) == -2                   # row stride < hidden
    assert g(P, 3, 2, P, P, P, P, 1, 2, 256, 256, 8, None, 64, P, P) == -2                   # rank outside the world
    assert g(P, 0, 2, P, P, P, P, 65, 2, 2048, 2048, 8, None, 64, P, P) == -3                # 130 CTAs > 64
    assert g(P, 0, 2, P, P, P, P, 1, 2, 256, 256, 8, None, 64, 0, P) == -2                   # no call counters
    assert f("nvk_b200_moe_combine_buffer_bytes", 2, 64) == 64 * 32 + 2 * 2 * 64 * 4096
