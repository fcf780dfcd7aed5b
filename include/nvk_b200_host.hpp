// C++ host layer over the C ABI of nvk_b200.h: the operator interface of the reference's quantized
// Linear, Mlp and grouped MoE decode step (rust/crates/nv-layers/src/linear.rs, mlp.rs, moe_grouped.rs)
// for a host written in a compiled language.  Header-only, C++17, no dependency beyond the C header:
// every tensor is a raw device pointer owned by the caller, every call is enqueued on the stream it is
// given, nothing allocates, nothing synchronises -- a step built from these can be captured in a graph.
// A non-zero status from the library becomes an nvk::host::Error naming the entry point, as the
// reference turns launcher codes into errors.  The Python package in this repository is the same
// layer for a Python host; both sit on the same entry points.
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "nvk_b200.h"

namespace nvk {
namespace host {

struct Error : std::runtime_error {
    std::string entry;
    int status;
    Error(const char* e, int rc)
        : std::runtime_error(std::string(e) + " returned " + std::to_string(rc)), entry(e), status(rc) {}
};

inline void check(const char* entry, int rc) {
    if (rc != 0) throw Error(entry, rc);
}

constexpr int kBlock = 16;         // values per ue4m3 scale
constexpr int kMinTile = 128;      // the reference refuses NVFP4 linears with a dimension below this
constexpr int kMaxDecodeRows = 64; // rows one launch of the W4A16 kernel takes

// Bytes of a 128x4-swizzled scale buffer for a [rows, cols] operand (linear.rs:2178-2180).
inline size_t swizzled_scale_bytes(size_t rows, size_t cols) {
    return (rows + 127) / 128 * 128 * ((cols / kBlock + 3) / 4 * 4);
}

// NVFP4 weight-only linear, y = x W^T: packed weights [out, in/2], swizzled block scales, and
// weight_alpha = 1 / stored weight global (times 1 / stored input global where a checkpoint has one).
// The decode-sized routes: one row through the M = 1 GEMV, up to 64 rows in one launch, more rows in
// chunks of 64 (rows are independent, so the chunking does not change a bit).
class Nvfp4Linear {
public:
    Nvfp4Linear(const uint8_t* weight_u8, const uint8_t* weight_scales, float weight_alpha, int in_features,
                int out_features, float input_stored_global = 1.0f)
        : w_(weight_u8), sc_(weight_scales), alpha_(weight_alpha), in_(in_features), out_(out_features),
          input_global_(input_stored_global) {
        if (in_features % kBlock != 0)
            throw std::invalid_argument("nvfp4 linear: in_features is not a multiple of 16");
        if (in_features < kMinTile || out_features < kMinTile)
            throw std::invalid_argument("nvfp4 linear: a dimension is below MIN_TILE = 128");
        if (weight_u8 == nullptr || weight_scales == nullptr) throw std::invalid_argument("nvfp4 linear: null weights");
    }

    int in_features() const { return in_; }
    int out_features() const { return out_; }
    const uint8_t* weight_u8() const { return w_; }
    const uint8_t* weight_scales() const { return sc_; }
    float weight_alpha() const { return alpha_; }
    // Output multiplier when the activations stay bf16: the input global is multiplied back out
    // (rust/crates/nv-models/src/qwen3_5_moe.rs:718-727).
    float alpha_w4a16() const { return alpha_ * input_global_; }

    // Which kernels m rows take: "gemv" or "decode".
    static const char* route_for(int m) { return m == 1 ? "gemv" : "decode"; }

    // x [m, in] bf16 -> y [m, out] bf16.
    void forward_into(void* stream, const uint16_t* x, uint16_t* y, int m) const {
        if (m <= 0) return;
        if (m == 1) {
            check("nv_kernels_nvfp4_gemv_bf16act",
                  nv_kernels_nvfp4_gemv_bf16act(stream, w_, sc_, x, y, alpha_w4a16(), out_, in_));
            return;
        }
        for (int r0 = 0; r0 < m; r0 += kMaxDecodeRows) {
            const int mm = m - r0 < kMaxDecodeRows ? m - r0 : kMaxDecodeRows;
            check("nvk_b200_linear_nvfp4_w4a16",
                  nvk_b200_linear_nvfp4_w4a16(stream, w_, sc_, nullptr, nullptr, x + (size_t)r0 * in_, nullptr,
                                              y + (size_t)r0 * out_, nullptr, alpha_w4a16(), 0.f, mm, out_, in_));
        }
    }

    // y = bf16(residual + alpha * a W^T), one rounding; a = x, or bf16(SiLU(x) * up) when `up` is given.
    // y may be `residual` itself.
    void forward_residual_into(void* stream, const uint16_t* x, const uint16_t* up, const uint16_t* residual,
                               uint16_t* y, int m) const {
        for (int r0 = 0; r0 < m; r0 += kMaxDecodeRows) {
            const int mm = m - r0 < kMaxDecodeRows ? m - r0 : kMaxDecodeRows;
            check("nvk_b200_linear_nvfp4_w4a16_residual",
                  nvk_b200_linear_nvfp4_w4a16_residual(stream, w_, sc_, x + (size_t)r0 * in_,
                                                       up ? up + (size_t)r0 * in_ : nullptr,
                                                       residual + (size_t)r0 * out_, y + (size_t)r0 * out_,
                                                       alpha_w4a16(), mm, out_, in_));
        }
    }

    // RMSNorm in front (the reference's FusedPreNorm on the decode route): up to 8 rows in one launch with
    // the norm in the linear's prologue; more rows through `normed_scratch` [m, in] and the norm kernel.
    void forward_prenorm_decode_into(void* stream, const uint16_t* x, const uint16_t* norm_weight, float eps,
                                     uint16_t* y, int m, uint16_t* normed_scratch) const {
        if (m <= 8 && in_ % 32 == 0) {
            check("nvk_b200_linear_nvfp4_w4a16_normed",
                  nvk_b200_linear_nvfp4_w4a16_normed(stream, w_, sc_, nullptr, nullptr, x, norm_weight, nullptr, eps, y,
                                                     nullptr, alpha_w4a16(), 0.f, m, out_, in_));
            return;
        }
        if (normed_scratch == nullptr) throw std::invalid_argument("forward_prenorm_decode: scratch needed for m > 8");
        check("nv_kernels_rmsnorm_bf16",
              nv_kernels_rmsnorm_bf16(stream, x, norm_weight, normed_scratch, (size_t)m, (size_t)in_, eps));
        forward_into(stream, normed_scratch, y, m);
    }

private:
    const uint8_t* w_;
    const uint8_t* sc_;
    float alpha_;
    int in_, out_;
    float input_global_;
};

// SwiGLU MLP on the W4A16 route: gate and up in one launch sharing x, then down with SiLU(gate) * up
// formed in its prologue.  `gate_out` / `up_out`: [m, inter] bf16 scratch of the caller.
class Nvfp4Mlp {
public:
    Nvfp4Mlp(const Nvfp4Linear& gate, const Nvfp4Linear& up, const Nvfp4Linear& down) : g_(gate), u_(up), d_(down) {
        if (gate.in_features() != up.in_features() || gate.out_features() != up.out_features() ||
            down.in_features() != gate.out_features())
            throw std::invalid_argument("nvfp4 mlp: gate / up / down shapes do not fit");
    }

    void gate_up_into(void* stream, const uint16_t* x, uint16_t* gate_out, uint16_t* up_out, int m) const {
        const int inter = g_.out_features(), hidden = g_.in_features();
        for (int r0 = 0; r0 < m; r0 += kMaxDecodeRows) {
            const int mm = m - r0 < kMaxDecodeRows ? m - r0 : kMaxDecodeRows;
            check("nvk_b200_linear_nvfp4_w4a16",
                  nvk_b200_linear_nvfp4_w4a16(stream, g_.weight_u8(), g_.weight_scales(), u_.weight_u8(),
                                              u_.weight_scales(), x + (size_t)r0 * hidden, nullptr,
                                              gate_out + (size_t)r0 * inter, up_out + (size_t)r0 * inter,
                                              g_.alpha_w4a16(), u_.alpha_w4a16(), mm, inter, hidden));
        }
    }

    void forward_into(void* stream, const uint16_t* x, uint16_t* gate_out, uint16_t* up_out, uint16_t* y, int m) const {
        gate_up_into(stream, x, gate_out, up_out, m);
        const int inter = g_.out_features(), hidden = d_.out_features();
        for (int r0 = 0; r0 < m; r0 += kMaxDecodeRows) {
            const int mm = m - r0 < kMaxDecodeRows ? m - r0 : kMaxDecodeRows;
            check("nvk_b200_linear_nvfp4_w4a16",
                  nvk_b200_linear_nvfp4_w4a16(stream, d_.weight_u8(), d_.weight_scales(), nullptr, nullptr,
                                              gate_out + (size_t)r0 * inter, up_out + (size_t)r0 * inter,
                                              y + (size_t)r0 * hidden, nullptr, d_.alpha_w4a16(), 0.f, mm, hidden, inter));
        }
    }

    // residual + MLP(x), rounded once; y may be `residual`.
    void forward_residual_into(void* stream, const uint16_t* x, const uint16_t* residual, uint16_t* gate_out,
                               uint16_t* up_out, uint16_t* y, int m) const {
        gate_up_into(stream, x, gate_out, up_out, m);
        d_.forward_residual_into(stream, gate_out, up_out, residual, y, m);
    }

private:
    Nvfp4Linear g_, u_, d_;
};

// Expert banks addressable by expert id (moe_grouped.rs `MoeGroupedWeights`): packed weights
// [E, N, K/2], swizzled scales [E, scale bytes per expert], alphas [E] in device memory.
struct ExpertBank {
    const uint8_t* packed;
    const uint8_t* scales;
    const float* alphas;
};

struct MoeGroupedWeights {
    ExpertBank gate, up, down;   // gate / up: [inter, hidden] per expert; down: [hidden, inter]
    int hidden, inter, num_experts;
};

// The caller's buffers for up to max_tokens tokens with top_k experts each (moe_grouped.rs
// `GroupedDecodeContext`); `bytes()` says how large each must be.
struct GroupedDecodeContext {
    int max_tokens, top_k;
    int32_t* topk_ids;       // [max_tokens, top_k]
    float* topk_weights;     // [max_tokens, top_k]
    int32_t* perm_token;     // [slots]
    int32_t* offsets;        // [E + 1]
    int32_t* inv_perm;       // [slots]
    int32_t* counts;         // [E]
    int32_t* active;         // [min(E, slots)]
    int32_t* n_active;       // [1]
    int32_t* status;         // [1], zero before the first step
    uint16_t* gate_out;      // [slots, inter]
    uint16_t* up_out;        // [slots, inter]
    uint16_t* down_out;      // [slots, hidden]
    float* y_acc;            // [max_tokens, hidden]
    int slots() const { return max_tokens * top_k; }
};

// One decode step (moe_grouped.rs:810-1134 on the route that keeps activations in bf16): route and sort
// the slots by expert, gate+up over each expert's tokens, down with the SiLU prologue, f32 weighted
// combine into ctx.y_acc [n, hidden].  mode 0: softmax over the winners; 1: sigmoid scores with bias.
inline void forward_grouped_decode(void* stream, const MoeGroupedWeights& w, const GroupedDecodeContext& ctx,
                                   const uint16_t* x, const float* router_logits, int n, const float* bias = nullptr,
                                   int mode = 0, float softcap = 0.f, bool norm_topk = true,
                                   float routed_scaling = 1.f) {
    if (n <= 0) return;
    if (n > ctx.max_tokens) throw std::invalid_argument("forward_grouped_decode: more tokens than the context holds");
    const int k = ctx.top_k, E = w.num_experts, slots = n * k;
    const bool fused = E <= 256 && slots <= 4096;
    const int32_t* active = nullptr;
    const int32_t* n_active = nullptr;
    if (fused) {
        check("nvk_b200_moe_route_permute",
              nvk_b200_moe_route_permute(stream, router_logits, bias, ctx.topk_ids, ctx.topk_weights, ctx.perm_token,
                                         ctx.offsets, ctx.inv_perm, ctx.active, ctx.n_active, n, E, k, mode, softcap,
                                         norm_topk ? 1 : 0, routed_scaling));
        active = ctx.active;
        n_active = ctx.n_active;
    } else {
        check("nv_kernels_moe_route_topk",
              nv_kernels_moe_route_topk(stream, router_logits, bias, ctx.topk_ids, ctx.topk_weights, n, E, k, mode,
                                        softcap, norm_topk ? 1 : 0, routed_scaling));
        check("nv_kernels_moe_permute", nv_kernels_moe_permute(stream, ctx.topk_ids, ctx.perm_token, ctx.offsets,
                                                               ctx.inv_perm, ctx.counts, n, k, E));
    }
    check("nvk_b200_moe_grouped_w4a16",
          nvk_b200_moe_grouped_w4a16(stream, w.gate.packed, w.gate.scales, w.up.packed, w.up.scales, w.gate.alphas,
                                     w.up.alphas, x, nullptr, ctx.perm_token, ctx.offsets, active, n_active,
                                     ctx.gate_out, ctx.up_out, E, w.inter, w.hidden, slots, n, ctx.status));
    check("nvk_b200_moe_grouped_w4a16",
          nvk_b200_moe_grouped_w4a16(stream, w.down.packed, w.down.scales, nullptr, nullptr, w.down.alphas, nullptr,
                                     ctx.gate_out, ctx.up_out, nullptr, ctx.offsets, active, n_active, ctx.down_out,
                                     nullptr, E, w.hidden, w.inter, slots, slots, ctx.status));
    check("nvk_b200_moe_combine", nvk_b200_moe_combine(stream, ctx.down_out, ctx.topk_weights, ctx.inv_perm, ctx.y_acc,
                                                       n, k, w.hidden, w.hidden, slots, ctx.status));
}

// ---- tensor / expert parallelism over peer memory ---------------------------------------------------
// The exchange buffers of a group of GPUs as one rank sees them: `bufs[r]` is rank r's buffer mapped in
// this process (nvk_b200_tp_buffer_alloc / _ipc_export / _ipc_open, handles exchanged by the host),
// `epoch` max_ctas zeroed uint32 of local device memory, `err` one zeroed int.  One such object per kind
// of exchange (they differ in buffer size: nvk_b200_tp_fused_buffer_bytes, nvk_b200_moe_combine_buffer_bytes).
struct PeerExchange {
    const void* const* bufs;
    int rank, world;
    int max_ctas, max_rows;
    uint32_t* epoch;
    int* err;
};

// Row-parallel linear (this rank's K slice in `shard`, this rank's activation slice in x) with the sum
// over the ranks inside the linear's own launch; y [m, out] is complete and identical on every rank.
// False when the launch does not fit the buffers: run shard.forward_into and an all-reduce instead.
inline bool tp_linear_allreduce(void* stream, const PeerExchange& px, const Nvfp4Linear& shard, const uint16_t* x,
                                const uint16_t* up, const uint16_t* residual, uint16_t* y, int m) {
    if (m > px.max_rows) return false;
    const int rc = nvk_b200_tp_linear_nvfp4_w4a16_allreduce(
        stream, px.bufs, px.rank, px.world, shard.weight_u8(), shard.weight_scales(), x, up, residual, y,
        shard.alpha_w4a16(), m, shard.out_features(), shard.in_features(), px.max_ctas, px.max_rows, px.epoch, px.err);
    if (rc == -3) return false;
    check("nvk_b200_tp_linear_nvfp4_w4a16_allreduce", rc);
    return true;
}

// Expert-parallel tail of forward_grouped_decode: the weighted combine of this rank's experts' slots and
// the sum over the ranks in one launch.  False when it does not fit the buffers.
inline bool moe_combine_allreduce(void* stream, const PeerExchange& px, const MoeGroupedWeights& w,
                                  const GroupedDecodeContext& ctx, int n) {
    const int slots = n * ctx.top_k;
    const int rc = nvk_b200_moe_combine_allreduce(stream, px.bufs, px.rank, px.world, ctx.down_out, ctx.topk_weights,
                                                  ctx.inv_perm, ctx.y_acc, n, ctx.top_k, w.hidden, w.hidden, slots,
                                                  ctx.status, px.max_ctas, px.epoch, px.err);
    if (rc == -3) return false;
    check("nvk_b200_moe_combine_allreduce", rc);
    return true;
}

}  // namespace host
}  // namespace nvk
