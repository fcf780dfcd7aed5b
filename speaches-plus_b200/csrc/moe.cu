// MoE decode plumbing for the NVFP4 expert path: router top-k, row gather into expert tiles,
// weighted combine, token permutation, and the grouped M=1 expert GEMV with NVFP4 activations.
#include "nvk_common.cuh"

namespace {

constexpr int kRouteMaxE = 4096;
constexpr int kRouteMaxK = 32;

// ---- router ------------------------------------------------------------------------------
// One CTA per token.  Scores live in shared memory; K rounds of a block-wide arg-max pick the
// winners (ties to the lower expert id).  mode 0: softmax over the K winning logits;
// mode 1: sigmoid scores, selection on score + bias, optional renormalisation.
__global__ void __launch_bounds__(256) moe_route_topk_kernel(const float* __restrict__ logits,
                                                             const float* __restrict__ bias,
                                                             int32_t* __restrict__ topk_ids,
                                                             float* __restrict__ topk_weights, int n_tokens, int E,
                                                             int K, int mode, float softcap, int norm_topk,
                                                             float routed_scaling, int out_stride,
                                                             int shared_tail_id) {
    extern __shared__ float rsm[];
    float* sel = rsm;
    float* raw = rsm + E;
    __shared__ float wv[8];
    __shared__ int wi[8];
    __shared__ int win_ids[kRouteMaxK];
    __shared__ float win_w[kRouteMaxK];
    const int n = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int e = tid; e < E; e += blockDim.x) {
        float x = logits[(size_t)n * E + e];
        if (softcap > 0.f) x = softcap * tanhf(x / softcap);
        if (mode == 1) {
            const float s = 1.f / (1.f + expf(-x));
            raw[e] = s;
            sel[e] = s + (bias ? bias[e] : 0.f);
        } else {
            raw[e] = x;
            sel[e] = x;
        }
    }
    __syncthreads();

    for (int j = 0; j < K; ++j) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = tid; e < E; e += blockDim.x) {
            const float v = sel[e];
            if (v > bv || (v == bv && e < bi)) {
                bv = v;
                bi = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        if (lane == 0) {
            wv[warp] = bv;
            wi[warp] = bi;
        }
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
                if (wv[w] > bv || (wv[w] == bv && wi[w] < bi)) {
                    bv = wv[w];
                    bi = wi[w];
                }
            const bool ok = bi < E;
            win_ids[j] = ok ? bi : -1;
            win_w[j] = ok ? raw[bi] : 0.f;
            if (ok) sel[bi] = -INFINITY;
        }
        __syncthreads();
    }

    if (tid == 0) {
        if (mode == 0) {
            float mx = -INFINITY;
            for (int j = 0; j < K; ++j) mx = fmaxf(mx, win_w[j]);
            float sum = 0.f;
            for (int j = 0; j < K; ++j) {
                win_w[j] = expf(win_w[j] - mx);
                sum += win_w[j];
            }
            for (int j = 0; j < K; ++j) win_w[j] /= sum;
        } else if (norm_topk) {
            float sum = 0.f;
            for (int j = 0; j < K; ++j) sum += win_w[j];
            if (sum > 0.f)
                for (int j = 0; j < K; ++j) win_w[j] /= sum;
        }
        for (int j = 0; j < K; ++j) {
            topk_ids[(size_t)n * out_stride + j] = win_ids[j];
            topk_weights[(size_t)n * out_stride + j] = win_w[j] * routed_scaling;
        }
        if (shared_tail_id >= 0 && out_stride > K) {
            topk_ids[(size_t)n * out_stride + K] = shared_tail_id;
            topk_weights[(size_t)n * out_stride + K] = 1.f;
        }
    }
}

int launch_route(void* stream, const float* logits, const float* bias, int32_t* ids, float* w, int n_tokens, int E,
                 int K, int mode, float softcap, int norm_topk, float routed_scaling, int out_stride, int tail) {
    const size_t shmem = (size_t)2 * E * sizeof(float);
    const int threads = E <= 32 ? 32 : (E <= 64 ? 64 : (E <= 128 ? 128 : 256));
    moe_route_topk_kernel<<<(unsigned)n_tokens, threads, shmem, (cudaStream_t)stream>>>(
        logits, bias, ids, w, n_tokens, E, K, mode, softcap, norm_topk, routed_scaling, out_stride, tail);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

// ---- gathers -----------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_rows_bf16_kernel(const uint16_t* __restrict__ x,
                                                               const int32_t* __restrict__ src_idx,
                                                               uint16_t* __restrict__ out, int m_total_padded,
                                                               int hidden, int n_tokens, int row_mul) {
    const int r = blockIdx.x * row_mul;
    if (r >= m_total_padded) return;
    const int s = src_idx[r];
    const bool ok = s >= 0 && s < n_tokens;
    const uint16_t* src = x + (size_t)(ok ? s : 0) * hidden;
    uint16_t* dst = out + (size_t)r * hidden;
    const bool vec = (hidden & 7) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    if (vec) {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        for (int i = threadIdx.x; i < (hidden >> 3); i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = ok ? reinterpret_cast<const uint4*>(src)[i] : z;
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? src[i] : (uint16_t)0;
    }
}

__global__ void gather_f32_by_ids_kernel(const float* __restrict__ src, const int32_t* __restrict__ ids,
                                         float* __restrict__ dst, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = ids[i];
    dst[i] = e >= 0 ? src[e] : 0.f;
}

// ---- combine -----------------------------------------------------------------------------
// TAIL == false: y_acc[n,h] = sum_s w[n,s] * y_sorted[inv_perm[n,s], h] (f32, s ascending).
// TAIL == true : out = bf16( resid + bf16( acc + shared ) ).
template <bool TAIL>
__global__ void __launch_bounds__(256) moe_unpermute_kernel(const uint16_t* __restrict__ y_sorted,
                                                            const float* __restrict__ topk_weights,
                                                            const int32_t* __restrict__ inv_perm,
                                                            float* __restrict__ y_acc,
                                                            const float* __restrict__ shared_f32,
                                                            const uint16_t* __restrict__ resid,
                                                            uint16_t* __restrict__ out, int n_tokens, int k, int H,
                                                            int row_stride) {
    const int n = blockIdx.x;
    const int h = blockIdx.y * blockDim.x + threadIdx.x;
    if (n >= n_tokens || h >= H) return;
    float acc = 0.f;
#pragma unroll 1
    for (int s = 0; s < k; ++s) {
        const int slot = n * k + s;
        const int row = inv_perm[slot];
        const float w = topk_weights[slot];
        const float v = nvk::bf16_bits_to_f32(y_sorted[(size_t)row * row_stride + h]);
        acc += w * v;
    }
    const size_t i = (size_t)n * H + h;
    if (TAIL) {
        const float t = (acc + shared_f32[i]) * 1.0f;
        const float fb = nvk::bf16_bits_to_f32(nvk::f32_to_bf16_bits(t));
        out[i] = nvk::f32_to_bf16_bits((nvk::bf16_bits_to_f32(resid[i]) + fb) * 1.0f);
    } else {
        y_acc[i] = acc;
    }
}

// ---- permutation (sort token slots by expert) ----------------------------------------------
__global__ void permute_count_kernel(const int32_t* __restrict__ topk_ids, int32_t* __restrict__ counts, int total) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < total) atomicAdd(&counts[topk_ids[t]], 1);
}

__global__ void permute_scan_kernel(const int32_t* __restrict__ counts, int32_t* __restrict__ offsets, int E) {
    if (threadIdx.x != 0) return;
    int32_t acc = 0;
    offsets[0] = 0;
    for (int e = 0; e < E; ++e) {
        acc += counts[e];
        offsets[e + 1] = acc;
    }
}

// Stable assignment: slot t goes after every earlier slot routed to the same expert, so the
// permutation does not depend on thread scheduling (one thread per expert walks the slots).
__global__ void permute_assign_kernel(const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ offsets,
                                      int32_t* __restrict__ permuted_token_idx, int32_t* __restrict__ inv_perm,
                                      int n_tokens, int k, int E) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    int pos = offsets[e];
    const int total = n_tokens * k;
    for (int t = 0; t < total; ++t) {
        if (topk_ids[t] == e) {
            permuted_token_idx[pos] = t / k;
            inv_perm[t] = pos;
            ++pos;
        }
    }
}

// ---- router + permutation in one launch (decode-sized batches) -------------------------------
// One CTA: each warp routes tokens w, w+8, ... (E <= 256 scores per token live in registers, 8 per
// lane), then the CTA counts, scans and stably assigns the routed slots.  Outputs are exactly those
// of moe_route_topk_kernel followed by the permute kernels.
constexpr int kFusedMaxE = 256, kFusedMaxSlots = 4096;

__global__ void __launch_bounds__(256) moe_route_permute_kernel(
    const float* __restrict__ logits, const float* __restrict__ bias, int32_t* __restrict__ topk_ids,
    float* __restrict__ topk_weights, int32_t* __restrict__ permuted_token_idx, int32_t* __restrict__ expert_offsets,
    int32_t* __restrict__ inv_perm, int n_tokens, int E, int K, int mode, float softcap, int norm_topk,
    float routed_scaling) {
    __shared__ int s_ids[kFusedMaxSlots];
    __shared__ int s_counts[kFusedMaxE + 1];
    // The logits usually come from the kernel just before this one.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int e = tid; e <= E; e += blockDim.x) s_counts[e] = 0;
    __syncthreads();
    for (int n = warp; n < n_tokens; n += 8) {
        float sel[8], raw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            sel[i] = -INFINITY;
            raw[i] = 0.f;
            if (e < E) {
                float x = logits[(size_t)n * E + e];
                if (softcap > 0.f) x = softcap * tanhf(x / softcap);
                if (mode == 1) {
                    const float sg = 1.f / (1.f + expf(-x));
                    raw[i] = sg;
                    sel[i] = sg + (bias ? bias[e] : 0.f);
                } else {
                    raw[i] = x;
                    sel[i] = x;
                }
            }
        }
        float my_w = 0.f;   // lane j keeps winner j's raw score
        int my_id = -1;
        for (int j = 0; j < K; ++j) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            float br = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int e = lane + 32 * i;
                if (e < E && (sel[i] > bv || (sel[i] == bv && e < bi))) {
                    bv = sel[i];
                    bi = e;
                    br = raw[i];
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                const float orr = __shfl_xor_sync(0xffffffffu, br, o);
                if (ov > bv || (ov == bv && oi < bi)) {
                    bv = ov;
                    bi = oi;
                    br = orr;
                }
            }
            const bool ok = bi < E;
            if (lane == j) {
                my_id = ok ? bi : -1;
                my_w = ok ? br : 0.f;
            }
            if (ok && (bi & 31) == lane) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (i == (bi >> 5)) sel[i] = -INFINITY;
            }
        }
        // weights: the same sequential sums the per-token router does, evaluated by every lane
        float w = my_w;
        if (mode == 0) {
            float mx = -INFINITY;
            for (int j = 0; j < K; ++j) mx = fmaxf(mx, __shfl_sync(0xffffffffu, my_w, j));
            const float ex = expf(my_w - mx);
            float sum = 0.f;
            for (int j = 0; j < K; ++j) sum += __shfl_sync(0xffffffffu, ex, j);
            w = ex / sum;
        } else if (norm_topk) {
            float sum = 0.f;
            for (int j = 0; j < K; ++j) sum += __shfl_sync(0xffffffffu, my_w, j);
            if (sum > 0.f) w = my_w / sum;
        }
        if (lane < K) {
            topk_ids[(size_t)n * K + lane] = my_id;
            topk_weights[(size_t)n * K + lane] = w * routed_scaling;
            s_ids[n * K + lane] = my_id;
            if (my_id >= 0) atomicAdd(&s_counts[my_id], 1);
        }
    }
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int e = 0; e < E; ++e) {
            const int c = s_counts[e];
            s_counts[e] = acc;
            acc += c;
        }
        s_counts[E] = acc;
    }
    __syncthreads();
    for (int e = tid; e <= E; e += blockDim.x) expert_offsets[e] = s_counts[e];
    const int total = n_tokens * K;
    for (int e = tid; e < E; e += blockDim.x) {
        int pos = s_counts[e];
        const int end = s_counts[e + 1];
        for (int t = 0; t < total && pos < end; ++t) {
            if (s_ids[t] == e) {
                permuted_token_idx[pos] = t / K;
                inv_perm[t] = pos;
                ++pos;
            }
        }
    }
}

// ---- grouped M=1 expert GEMV, NVFP4 weights and NVFP4 activations ---------------------------
// d[g, n] = bf16( alphas[e] * sum_kb (ws * as) * dot16(w, a) ),  e = ids[g]; the activation of
// group g is row 0 of its 128-row tile.  One warp per output row; the 16 e2m1 x e2m1 products of
// a block are exact in f16 (multiples of 1/4 up to 36), and each half of an f16x2 accumulator
// sums 8 of them exactly (at most 288), so the block dot is exact before it meets the scales.
__global__ void __launch_bounds__(256) moe_grouped_fp4_gemv_kernel(
    const uint8_t* __restrict__ a_packed, const uint8_t* __restrict__ a_scales, const uint8_t* __restrict__ b_packed,
    const uint8_t* __restrict__ b_scales, const float* __restrict__ alphas, uint16_t* __restrict__ d,
    const int32_t* __restrict__ ids, int num_experts_total, int n_dim, int k_dim, int a_tile_stride_rows,
    long long d_group_stride) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int g = blockIdx.y;
    if (n >= n_dim) return;
    const long long d_idx = (long long)g * d_group_stride + n;
    const int e = ids[g];
    if (e < 0 || e >= num_experts_total) {
        if (lane == 0) d[d_idx] = 0;
        return;
    }
    const int half_k = k_dim >> 1, group_k = k_dim >> 4;
    const int k_tiles = (group_k + 3) >> 2;
    const size_t group_k_pad = (size_t)k_tiles * 4;
    const size_t n_pad = ((size_t)n_dim + 127) / 128 * 128;
    const uint2* w_row = reinterpret_cast<const uint2*>(b_packed + ((size_t)e * n_dim + n) * half_k);
    const uint2* a_row = reinterpret_cast<const uint2*>(a_packed + (size_t)g * a_tile_stride_rows * half_k);
    const uint8_t* w_sf = b_scales + (size_t)e * n_pad * group_k_pad;
    const uint8_t* a_sf = a_scales + (size_t)g * (size_t)(a_tile_stride_rows / 128) * group_k_pad * 128;

    float acc = 0.f;
    for (int kb = lane; kb < group_k; kb += 32) {
        const float ws = nvk::ue4m3_to_f32(w_sf[nvk::swz_offset(n, kb, group_k)]);
        const float as = nvk::ue4m3_to_f32(a_sf[(size_t)(kb >> 2) * 512 + (kb & 3)]);
        const uint2 wq = __ldg(&w_row[kb]);
        const uint2 aq = __ldg(&a_row[kb]);
        uint32_t wh[8], ah[8];
        nvk::e2m1x8_to_f16x2x4(wq.x, wh[0], wh[1], wh[2], wh[3]);
        nvk::e2m1x8_to_f16x2x4(wq.y, wh[4], wh[5], wh[6], wh[7]);
        nvk::e2m1x8_to_f16x2x4(aq.x, ah[0], ah[1], ah[2], ah[3]);
        nvk::e2m1x8_to_f16x2x4(aq.y, ah[4], ah[5], ah[6], ah[7]);
        uint32_t s2 = 0u;
#pragma unroll
        for (int i = 0; i < 8; ++i) s2 = nvk::hfma2_u32(wh[i], ah[i], s2);
        const float2 sf = __half22float2(*reinterpret_cast<__half2*>(&s2));
        acc += (ws * as) * (sf.x + sf.y);
    }
    acc = nvk::warp_sum(acc);
    if (lane == 0) d[d_idx] = nvk::f32_to_bf16_bits(acc * __ldg(&alphas[e]));
}

// ---- single M=1 GEMV with NVFP4 weights and an NVFP4 activation row ---------------------------
// y[n] = bf16( alpha * sum_kb (ws[n,kb] * xs[kb]) * dot16(w, x) ): the grouped kernel's block dot for
// one matrix; the activation's scales are a flat [K/16] array (the row quantizer's layout), the
// weight's are swizzled.  One warp per output row.
__global__ void __launch_bounds__(256) nvfp4_w4a4_gemv_kernel(const uint8_t* __restrict__ w_packed,
                                                              const uint8_t* __restrict__ w_scales,
                                                              const uint8_t* __restrict__ x_packed,
                                                              const uint8_t* __restrict__ x_scales,
                                                              uint16_t* __restrict__ y, float alpha, int n_dim,
                                                              int k_dim) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= n_dim) return;
    const int half_k = k_dim >> 1, group_k = k_dim >> 4;
    const uint2* w_row = reinterpret_cast<const uint2*>(w_packed + (size_t)n * half_k);
    const uint2* x_row = reinterpret_cast<const uint2*>(x_packed);
    float acc = 0.f;
    for (int kb = lane; kb < group_k; kb += 32) {
        const float ws = nvk::ue4m3_to_f32(w_scales[nvk::swz_offset(n, kb, group_k)]);
        const float xs = nvk::ue4m3_to_f32(x_scales[kb]);
        const uint2 wq = __ldg(&w_row[kb]);
        const uint2 xq = __ldg(&x_row[kb]);
        uint32_t wh[8], xh[8];
        nvk::e2m1x8_to_f16x2x4(wq.x, wh[0], wh[1], wh[2], wh[3]);
        nvk::e2m1x8_to_f16x2x4(wq.y, wh[4], wh[5], wh[6], wh[7]);
        nvk::e2m1x8_to_f16x2x4(xq.x, xh[0], xh[1], xh[2], xh[3]);
        nvk::e2m1x8_to_f16x2x4(xq.y, xh[4], xh[5], xh[6], xh[7]);
        uint32_t s2 = 0u;
#pragma unroll
        for (int i = 0; i < 8; ++i) s2 = nvk::hfma2_u32(wh[i], xh[i], s2);
        const float2 sf = __half22float2(*reinterpret_cast<__half2*>(&s2));
        acc += (ws * xs) * (sf.x + sf.y);
    }
    acc = nvk::warp_sum(acc);
    if (lane == 0) y[n] = nvk::f32_to_bf16_bits(acc * alpha);
}

// y[r, h] = x[r, h] * sigmoid(gate_logits[r]): the shared expert's gate (one logit per token).
__global__ void __launch_bounds__(256) mul_sigmoid_rowgate_kernel(const float* __restrict__ x,
                                                                  const float* __restrict__ gate_logits,
                                                                  float* __restrict__ y, int rows, int hidden) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * hidden) return;
    const float g = 1.f / (1.f + expf(-gate_logits[(int)(i / hidden)]));
    y[i] = x[i] * g;
}

}  // namespace

extern "C" {

int nv_kernels_mul_sigmoid_rowgate_f32(void* stream, const float* x, const float* gate_logits, float* y, int rows,
                                       int hidden) {
    if (rows <= 0 || hidden <= 0) return 0;
    if (nvk::any_null(x, gate_logits, y)) return NVK_ERR_ARG;
    const long long total = (long long)rows * hidden;
    const long long grid = (total + 255) / 256;
    if (grid > 0x7FFFFFFFLL) return NVK_ERR_GRID_AXIS;
    mul_sigmoid_rowgate_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(x, gate_logits, y, rows, hidden);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int nv_kernels_nvfp4_gemv_bf16(void* stream, const uint8_t* W_packed, const uint8_t* W_scales, const uint8_t* x_packed,
                               const uint8_t* x_scales, uint16_t* y, float alpha, int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    if ((K & 15) != 0) return NVK_ERR_SHAPE;
    if (nvk::any_null(W_packed, W_scales, x_packed, x_scales, y)) return NVK_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(W_packed) & 7) != 0 || (reinterpret_cast<uintptr_t>(x_packed) & 7) != 0)
        return NVK_ERR_ARG;
    nvfp4_w4a4_gemv_kernel<<<(unsigned)((N + 7) / 8), 256, 0, (cudaStream_t)stream>>>(W_packed, W_scales, x_packed,
                                                                                       x_scales, y, alpha, N, K);
    return (int)cudaGetLastError();
}

int nv_kernels_moe_route_topk(void* stream, const float* logits, const float* bias, int32_t* topk_ids,
                              float* topk_weights, int n_tokens, int E, int K, int mode, float softcap,
                              int norm_topk, float routed_scaling) {
    if (n_tokens <= 0 || E <= 0 || K <= 0) return 0;
    if (E > kRouteMaxE || K > kRouteMaxK || K > E) return NVK_ERR_ARG;
    if (nvk::any_null(logits, topk_ids, topk_weights)) return NVK_ERR_ARG;
    return launch_route(stream, logits, bias, topk_ids, topk_weights, n_tokens, E, K, mode, softcap, norm_topk,
                        routed_scaling, K, -1);
}

int nv_kernels_moe_route_topk_shared_tail(void* stream, const float* logits, const float* bias, int32_t* topk_ids,
                                          float* topk_weights, int n_tokens, int E, int K, int mode, float softcap,
                                          int norm_topk, float routed_scaling, int shared_tail_id) {
    if (n_tokens <= 0 || E <= 0 || K <= 0) return 0;
    if (E > kRouteMaxE || K + 1 > kRouteMaxK || K > E) return NVK_ERR_ARG;
    if (shared_tail_id < 0) return NVK_ERR_RESOURCE;
    if (nvk::any_null(logits, topk_ids, topk_weights)) return NVK_ERR_ARG;
    return launch_route(stream, logits, bias, topk_ids, topk_weights, n_tokens, E, K, mode, softcap, norm_topk,
                        routed_scaling, K + 1, shared_tail_id);
}

static int gather_rows(void* stream, const uint16_t* x, const int32_t* src_idx, uint16_t* out, int m_total_padded,
                       int hidden, int n_tokens, int row_stride) {
    int block = 256;
    if (hidden < block) block = ((hidden + 31) / 32) * 32;
    if (block < 32) block = 32;
    gather_rows_bf16_kernel<<<(unsigned)(m_total_padded / row_stride), block, 0, (cudaStream_t)stream>>>(
        x, src_idx, out, m_total_padded, hidden, n_tokens, row_stride);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int nv_kernels_gather_rows_bf16(void* stream, const uint16_t* x_bf16, const int32_t* src_idx, uint16_t* out_bf16,
                                int m_total_padded, int hidden, int n_tokens) {
    if (m_total_padded <= 0 || hidden <= 0) return 0;
    if (nvk::any_null(x_bf16, src_idx, out_bf16)) return NVK_ERR_ARG;
    return gather_rows(stream, x_bf16, src_idx, out_bf16, m_total_padded, hidden, n_tokens, 1);
}

int nv_kernels_gather_rows_bf16_strided(void* stream, const uint16_t* x_bf16, const int32_t* src_idx,
                                        uint16_t* out_bf16, int m_total_padded, int hidden, int n_tokens,
                                        int row_stride) {
    if (m_total_padded <= 0 || hidden <= 0) return 0;
    if (row_stride <= 0 || (m_total_padded % row_stride) != 0) return NVK_ERR_RESOURCE;
    if (nvk::any_null(x_bf16, src_idx, out_bf16)) return NVK_ERR_ARG;
    return gather_rows(stream, x_bf16, src_idx, out_bf16, m_total_padded, hidden, n_tokens, row_stride);
}

int nv_kernels_gather_f32_by_ids(void* stream, const float* src, const int32_t* ids, float* dst, int n) {
    if (n <= 0) return 0;
    if (nvk::any_null(src, ids, dst)) return NVK_ERR_ARG;
    gather_f32_by_ids_kernel<<<(unsigned)((n + 127) / 128), 128, 0, (cudaStream_t)stream>>>(src, ids, dst, n);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int nv_kernels_moe_unpermute_scatter(void* stream, const uint16_t* y_sorted_bf16, const float* topk_weights,
                                     const int32_t* inv_perm, float* y_acc_f32, int n_tokens, int k, int hidden,
                                     int y_sorted_row_stride) {
    if (n_tokens <= 0 || k <= 0 || hidden <= 0) return 0;
    if (y_sorted_row_stride < hidden) return NVK_ERR_ARG;
    if (nvk::any_null(y_sorted_bf16, topk_weights, inv_perm, y_acc_f32)) return NVK_ERR_ARG;
    dim3 grid((unsigned)n_tokens, (unsigned)((hidden + 255) / 256));
    moe_unpermute_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(y_sorted_bf16, topk_weights, inv_perm,
                                                                        y_acc_f32, nullptr, nullptr, nullptr,
                                                                        n_tokens, k, hidden, y_sorted_row_stride);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int nv_kernels_moe_unpermute_scatter_tail(void* stream, const uint16_t* y_sorted_bf16, const float* topk_weights,
                                          const int32_t* inv_perm, const float* shared_f32,
                                          const uint16_t* resid_bf16, uint16_t* out_bf16, int n_tokens, int k,
                                          int hidden, int y_sorted_row_stride) {
    if (n_tokens <= 0 || k <= 0 || hidden <= 0) return 0;
    if (y_sorted_row_stride < hidden) return NVK_ERR_ARG;
    if (nvk::any_null(y_sorted_bf16, topk_weights, inv_perm, out_bf16)) return NVK_ERR_ARG;
    dim3 grid((unsigned)n_tokens, (unsigned)((hidden + 255) / 256));
    moe_unpermute_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(y_sorted_bf16, topk_weights, inv_perm, nullptr,
                                                                       shared_f32, resid_bf16, out_bf16, n_tokens, k,
                                                                       hidden, y_sorted_row_stride);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int nv_kernels_moe_permute(void* stream, const int32_t* topk_ids, int32_t* permuted_token_idx,
                           int32_t* expert_offsets, int32_t* inv_perm, int32_t* scratch_counts, int n_tokens, int k,
                           int num_experts) {
    if (n_tokens <= 0 || k <= 0 || num_experts <= 0) return 0;
    if (nvk::any_null(topk_ids, permuted_token_idx, expert_offsets, inv_perm, scratch_counts)) return NVK_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int total = n_tokens * k;
    cudaError_t err = cudaMemsetAsync(scratch_counts, 0, sizeof(int32_t) * num_experts, s);
    if (err != cudaSuccess) return (int)err;
    permute_count_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(topk_ids, scratch_counts, total);
    permute_scan_kernel<<<1, 32, 0, s>>>(scratch_counts, expert_offsets, num_experts);
    permute_assign_kernel<<<(unsigned)((num_experts + 127) / 128), 128, 0, s>>>(
        topk_ids, expert_offsets, permuted_token_idx, inv_perm, n_tokens, k, num_experts);
    err = cudaGetLastError();
    return err == cudaSuccess ? 0 : (int)err;
}

// Router and permutation in one launch for decode-sized batches (no counterpart in the reference,
// whose decode step launches them separately): same outputs as nv_kernels_moe_route_topk followed by
// nv_kernels_moe_permute, no scratch.  Limits: E <= 256, K <= 32, n_tokens * K <= 4096 (else -3).
int nvk_b200_moe_route_permute(void* stream, const float* logits, const float* bias, int32_t* topk_ids,
                               float* topk_weights, int32_t* permuted_token_idx, int32_t* expert_offsets,
                               int32_t* inv_perm, int n_tokens, int E, int K, int mode, float softcap, int norm_topk,
                               float routed_scaling) {
    if (n_tokens <= 0 || E <= 0 || K <= 0) return 0;
    if (K > E || K > kRouteMaxK) return NVK_ERR_ARG;
    if (E > kFusedMaxE || (long long)n_tokens * K > kFusedMaxSlots) return NVK_ERR_RESOURCE;
    if (nvk::any_null(logits, topk_ids, topk_weights, permuted_token_idx, expert_offsets, inv_perm)) return NVK_ERR_ARG;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, moe_route_permute_kernel, logits, bias, topk_ids, topk_weights,
                                       permuted_token_idx, expert_offsets, inv_perm, n_tokens, E, K, mode, softcap,
                                       norm_topk, routed_scaling);
    return e == cudaSuccess ? 0 : (int)e;
}

// ---- token permutation for callers that may not allocate device memory -------------------------
// Some hosts of this library cannot hand it a scratch buffer at the point of the call: a serving
// engine that claimed all of HBM for its KV-cache pool at start-up has nothing left to cudaMalloc
// from, a decode loop cannot afford the device-wide synchronisation an allocation implies, and an
// FFI host whose ownership rule is "the C side never allocates" has no allocator to lend.  For them
// the per-expert counters of the permutation live in the fixed array below instead of in a
// caller-supplied buffer.  The array is part of the library image: every GPU that loads the library
// holds these 16 KiB until the process exits.
constexpr int kStaticPermuteMaxExperts = 4096;
static __device__ __align__(256) int32_t g_permute_counts[kStaticPermuteMaxExperts];

int nvk_b200_moe_permute_static(void* stream, const int32_t* topk_ids, int32_t* permuted_token_idx,
                                int32_t* expert_offsets, int32_t* inv_perm, int n_tokens, int k,
                                int num_experts) {
    if (n_tokens <= 0 || k <= 0 || num_experts <= 0) return 0;
    if (num_experts > kStaticPermuteMaxExperts) return NVK_ERR_RESOURCE;  // more experts than the fixed array holds
    if (nvk::any_null(topk_ids, permuted_token_idx, expert_offsets, inv_perm)) return NVK_ERR_ARG;
    // In host code `g_permute_counts` is only a handle for the symbol, not an address the GPU can
    // use; the device address is looked up once per device (with that device current) and kept.
    constexpr int kMaxDevices = 64;
    static int32_t* dev_ptr[kMaxDevices] = {};
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return (int)err;
    if (dev < 0 || dev >= kMaxDevices) return NVK_ERR_ARG;
    if (dev_ptr[dev] == nullptr) {
        int32_t* ptr = nullptr;
        err = cudaGetSymbolAddress((void**)&ptr, g_permute_counts);
        if (err != cudaSuccess) return (int)err;
        if (ptr == nullptr) return NVK_ERR_RESOURCE;
        dev_ptr[dev] = ptr;
    }
    int32_t* counts = dev_ptr[dev];
    cudaStream_t s = (cudaStream_t)stream;
    const int total = n_tokens * k;
    // The array still holds whatever the previous call left in it: the counters start from zero.
    err = cudaMemsetAsync(counts, 0, sizeof(int32_t) * num_experts, s);
    if (err != cudaSuccess) return (int)err;
    permute_count_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(topk_ids, counts, total);
    permute_scan_kernel<<<1, 32, 0, s>>>(counts, expert_offsets, num_experts);
    permute_assign_kernel<<<(unsigned)((num_experts + 127) / 128), 128, 0, s>>>(
        topk_ids, expert_offsets, permuted_token_idx, inv_perm, n_tokens, k, num_experts);
    err = cudaGetLastError();
    return err == cudaSuccess ? 0 : (int)err;
}

int nv_kernels_moe_grouped_fp4_gemv_m1_bf16(void* stream, const uint8_t* a_packed, const uint8_t* a_scales,
                                            const uint8_t* b_packed, const uint8_t* b_scales, const float* alphas,
                                            uint16_t* d_bf16, const int32_t* group_expert_ids, int num_groups,
                                            int num_experts_total, int n, int k, int a_tile_stride_rows,
                                            long long d_group_stride_elems) {
    if (num_groups <= 0 || num_experts_total <= 0 || n <= 0 || k <= 0) return NVK_ERR_SHAPE;
    if ((k & 15) != 0) return NVK_ERR_SHAPE;
    if (a_tile_stride_rows <= 0 || (a_tile_stride_rows & 127) != 0) return NVK_ERR_SHAPE;
    if (d_group_stride_elems < (long long)n) return NVK_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(a_packed) & 7) != 0 || (reinterpret_cast<uintptr_t>(b_packed) & 7) != 0)
        return NVK_ERR_ARG;
    if (num_groups > 65535) return NVK_ERR_GRID_AXIS;
    if (nvk::any_null(a_packed, a_scales, b_packed, b_scales, alphas, d_bf16, group_expert_ids)) return NVK_ERR_ARG;
    dim3 grid((unsigned)((n + 7) / 8), (unsigned)num_groups);
    moe_grouped_fp4_gemv_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        a_packed, a_scales, b_packed, b_scales, alphas, d_bf16, group_expert_ids, num_experts_total, n, k,
        a_tile_stride_rows, d_group_stride_elems);
    return (int)cudaGetLastError();
}

}  // extern "C"
