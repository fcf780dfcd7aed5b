// bf16 -> NVFP4 quantizers (packed e2m1 + swizzled ue4m3 block scales), byte-exact with the
// host rule: local = amax/6 (1 when the block is all zero), byte = ue4m3(G*local),
// inv = G/decode(byte) (1 when that is 0), code = e2m1(clamp(v*inv, +-6)), even element in the
// low nibble.  G == 0, NaN or Inf is treated as 1.  One thread owns one 16-value block: two
// 128-bit loads in, one 64-bit store of codes and one scale byte out.
#include "nvk_common.cuh"

namespace {

struct QuantParams {
    const uint16_t* x;       // [rows, K] bf16 (gate when SRC == 1)
    const uint16_t* x2;      // up when SRC == 1
    const uint16_t* norm_w;  // RMSNorm weight when SRC == 2
    uint8_t* packed;         // [rows, K/2]
    uint8_t* scales;         // swizzled, or [K/16] linear when `linear_scales`
    const float* globals;    // per row-tile stored global (device), or null
    float global;            // stored global when `globals` is null
    float eps;
    int rows;                // rows written
    int rows_logical;        // rows >= this quantize zeros
    int K;
    int row_mul;             // row = index * row_mul (strided variants touch one row per tile)
    int m_per_expert;        // rows per entry of `globals`
    int linear_scales;
};

__device__ __forceinline__ float fix_global(float g) { return (g == 0.f || !isfinite(g)) ? 1.f : g; }

__device__ __forceinline__ void quantize_block(const float (&v)[16], float stored, uint2& codes, uint32_t& sbyte) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float local = (amax == 0.f) ? 1.f : (amax / 6.f);
    sbyte = nvk::encode_ue4m3(stored * local);
    const float dec = nvk::ue4m3_to_f32(sbyte);
    const float inv = (dec == 0.f) ? 1.f : (stored / dec);
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float q = fminf(fmaxf(v[i] * inv, -6.f), 6.f);
        w[i >> 3] |= nvk::encode_e2m1(q) << (4 * (i & 7));
    }
    codes = make_uint2(w[0], w[1]);
}

// SRC 0: plain bf16; SRC 1: SiLU(gate)*up evaluated in f32 (not rounded to bf16 first).
template <int SRC>
__global__ void __launch_bounds__(256) quantize_blocks_kernel(const QuantParams p) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int bpr = p.K >> 4;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)p.rows * bpr;
    if (idx >= total) return;
    const int ri = (int)(idx / bpr);
    const int kb = (int)(idx - (long long)ri * bpr);
    const int row = ri * p.row_mul;
    float stored = p.globals ? p.globals[row / p.m_per_expert] : p.global;
    stored = fix_global(stored);

    float v[16];
    if (row < p.rows_logical) {
        const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)row * p.K + (size_t)kb * 16);
        const uint4 a = src[0], b = src[1];
        const uint32_t ws[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[2 * i] = nvk::bf16_bits_to_f32(ws[i] & 0xFFFFu);
            v[2 * i + 1] = nvk::bf16_bits_to_f32(ws[i] >> 16);
        }
        if (SRC == 1) {
            const uint4* src2 = reinterpret_cast<const uint4*>(p.x2 + (size_t)row * p.K + (size_t)kb * 16);
            const uint4 c = src2[0], d = src2[1];
            const uint32_t us[8] = {c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float u0 = nvk::bf16_bits_to_f32(us[i] & 0xFFFFu), u1 = nvk::bf16_bits_to_f32(us[i] >> 16);
                const float g0 = v[2 * i], g1 = v[2 * i + 1];
                v[2 * i] = (g0 / (1.f + expf(-g0))) * u0;
                v[2 * i + 1] = (g1 / (1.f + expf(-g1))) * u1;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
    }
    uint2 codes;
    uint32_t sb;
    quantize_block(v, stored, codes, sb);
    *reinterpret_cast<uint2*>(p.packed + (size_t)row * (p.K >> 1) + (size_t)kb * 8) = codes;
    const size_t so = p.linear_scales ? (size_t)row * bpr + kb : nvk::swz_offset(row, kb, bpr);
    p.scales[so] = (uint8_t)sb;
}

// RMSNorm fused in front of the quantizer: one CTA per row, the row staged once in shared memory.
// The quantized value is bf16(x * rsqrt(mean(x^2) + eps) * w): one rounding to bf16, then the
// plain block quantizer.
__global__ void __launch_bounds__(256) rmsnorm_quantize_kernel(const QuantParams p) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    NVK_DYN_SMEM_AS(uint16_t, row_s);
    __shared__ float red[8];
    const int row = blockIdx.x;
    const int bpr = p.K >> 4;
    const bool live = row < p.rows_logical;
    float ss = 0.f;
    if (live) {
        for (int i = threadIdx.x; i < p.K; i += blockDim.x) {
            const uint16_t b = p.x[(size_t)row * p.K + i];
            row_s[i] = b;
            const float f = nvk::bf16_bits_to_f32(b);
            ss = fmaf(f, f, ss);   // an explicit fma: every copy of this sum rounds alike
        }
    }
    ss = nvk::warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float rstd = rsqrtf(tot / (float)p.K + p.eps);
    const float stored = fix_global(p.global);
    for (int kb = threadIdx.x; kb < bpr; kb += blockDim.x) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (live) {
                const float w = nvk::bf16_bits_to_f32(p.norm_w[kb * 16 + i]);
                v[i] = nvk::bf16_bits_to_f32(
                    nvk::f32_to_bf16_bits(nvk::bf16_bits_to_f32(row_s[kb * 16 + i]) * rstd * w));
            } else {
                v[i] = 0.f;
            }
        }
        uint2 codes;
        uint32_t sb;
        quantize_block(v, stored, codes, sb);
        *reinterpret_cast<uint2*>(p.packed + (size_t)row * (p.K >> 1) + (size_t)kb * 8) = codes;
        p.scales[nvk::swz_offset(row, kb, bpr)] = (uint8_t)sb;
    }
}

// Plain RMSNorm over bf16 rows: y = bf16(x * rsqrt(mean(x^2) + eps) * w), fp32 arithmetic, one
// rounding -- the statement the fused quantizer above applies before it quantizes.  One CTA per row.
__global__ void __launch_bounds__(256) rmsnorm_bf16_kernel(const uint16_t* __restrict__ x,
                                                           const uint16_t* __restrict__ w, uint16_t* __restrict__ y,
                                                           size_t hidden, float eps) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    __shared__ float red[8];
    const uint16_t* xr = x + (size_t)blockIdx.x * hidden;
    uint16_t* yr = y + (size_t)blockIdx.x * hidden;
    float ss = 0.f;
    for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float f = nvk::bf16_bits_to_f32(xr[i]);
        ss = fmaf(f, f, ss);   // an explicit fma: every copy of this sum rounds alike
    }
    ss = nvk::warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float rstd = rsqrtf(tot / (float)hidden + eps);
    for (size_t i = threadIdx.x; i < hidden; i += blockDim.x)
        yr[i] = nvk::f32_to_bf16_bits(nvk::bf16_bits_to_f32(xr[i]) * rstd * nvk::bf16_bits_to_f32(w[i]));
}

template <int SRC>
int launch_blocks(cudaStream_t s, const QuantParams& p) {
    const long long total = (long long)p.rows * (p.K >> 4);
    const long long grid = (total + 255) / 256;
    if (grid > 0x7FFFFFFFLL) return NVK_ERR_GRID_AXIS;
    return nvk::launch(nvk::launch_1d(s, (unsigned)grid, 256, 0, true), quantize_blocks_kernel<SRC>, p);
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

}  // namespace

extern "C" {

int nv_kernels_quantize_nvfp4_bf16(void* stream, const uint16_t* x_bf16, uint8_t* packed_out,
                                   uint8_t* scales_out_swizzled, float stored_global, int m_padded,
                                   int m_logical, int K) {
    if (m_padded <= 0 || K <= 0) return 0;
    if (m_logical < 0 || m_logical > m_padded) return NVK_ERR_ARG;
    if ((K % 16) != 0) return NVK_ERR_SHAPE;
    if (!aligned16(x_bf16) || (reinterpret_cast<uintptr_t>(packed_out) & 7u)) return NVK_ERR_ARG;
    // x is not read when every row is a pad row
    if (nvk::any_null(packed_out, scales_out_swizzled) || (m_logical > 0 && x_bf16 == nullptr)) return NVK_ERR_ARG;
    QuantParams p = {};
    p.x = x_bf16; p.packed = packed_out; p.scales = scales_out_swizzled;
    p.global = stored_global; p.rows = m_padded; p.rows_logical = m_logical; p.K = K;
    p.row_mul = 1; p.m_per_expert = 1;
    return launch_blocks<0>((cudaStream_t)stream, p);
}

int nv_kernels_quantize_nvfp4_bf16_rows(void* stream, const uint16_t* x_bf16, uint8_t* packed_out,
                                        uint8_t* scales_out_swizzled, float stored_global, int m_rows, int K) {
    if (m_rows <= 0 || K <= 0) return 0;
    return nv_kernels_quantize_nvfp4_bf16(stream, x_bf16, packed_out, scales_out_swizzled, stored_global, m_rows,
                                          m_rows, K);
}

// Flat-layout single-row quantizer: scales are written linearly ([K/16]), not swizzled.
int nv_kernels_nvfp4_quantize_row_bf16(void* stream, const uint16_t* x, uint8_t* packed_out, uint8_t* scales_out,
                                       float stored_global, int K) {
    if (K <= 0) return 0;
    if ((K & 15) != 0) return NVK_ERR_SHAPE;
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(packed_out) & 7u)) return NVK_ERR_ARG;
    if (nvk::any_null(x, packed_out, scales_out)) return NVK_ERR_ARG;
    QuantParams p = {};
    p.x = x; p.packed = packed_out; p.scales = scales_out;
    p.global = stored_global; p.rows = 1; p.rows_logical = 1; p.K = K;
    p.row_mul = 1; p.m_per_expert = 1; p.linear_scales = 1;
    return launch_blocks<0>((cudaStream_t)stream, p);
}

static int per_expert(void* stream, const uint16_t* a, const uint16_t* b, uint8_t* packed, uint8_t* scales,
                      const float* globals, int m_per_expert, int m_total, int K, bool strided, bool silu) {
    if (m_total <= 0 || K <= 0 || m_per_expert <= 0) return 0;
    if ((K % 16) != 0) return NVK_ERR_SHAPE;
    if (strided && (m_total % m_per_expert) != 0) return NVK_ERR_RESOURCE;
    if (!aligned16(a) || (silu && !aligned16(b)) || (reinterpret_cast<uintptr_t>(packed) & 7u)) return NVK_ERR_ARG;
    if (nvk::any_null(a, packed, scales, globals) || (silu && b == nullptr)) return NVK_ERR_ARG;
    QuantParams p = {};
    p.x = a; p.x2 = b; p.packed = packed; p.scales = scales; p.globals = globals;
    p.K = K; p.m_per_expert = m_per_expert;
    p.row_mul = strided ? m_per_expert : 1;
    p.rows = strided ? m_total / m_per_expert : m_total;
    p.rows_logical = m_total;
    return silu ? launch_blocks<1>((cudaStream_t)stream, p) : launch_blocks<0>((cudaStream_t)stream, p);
}

int nv_kernels_quantize_nvfp4_bf16_per_expert(void* stream, const uint16_t* x_bf16, uint8_t* packed_out,
                                              uint8_t* scales_out_swizzled, const float* stored_globals,
                                              int m_per_expert, int m_total, int K) {
    return per_expert(stream, x_bf16, nullptr, packed_out, scales_out_swizzled, stored_globals, m_per_expert,
                      m_total, K, false, false);
}

int nv_kernels_quantize_nvfp4_bf16_per_expert_strided(void* stream, const uint16_t* x_bf16, uint8_t* packed_out,
                                                      uint8_t* scales_out_swizzled, const float* stored_globals,
                                                      int m_per_expert, int m_total, int K) {
    return per_expert(stream, x_bf16, nullptr, packed_out, scales_out_swizzled, stored_globals, m_per_expert,
                      m_total, K, true, false);
}

int nv_kernels_silu_mul_quantize_nvfp4_bf16_per_expert(void* stream, const uint16_t* y_gate_bf16,
                                                       const uint16_t* y_up_bf16, uint8_t* packed_out,
                                                       uint8_t* scales_out_swizzled, const float* stored_globals,
                                                       int m_per_expert, int m_total, int K) {
    return per_expert(stream, y_gate_bf16, y_up_bf16, packed_out, scales_out_swizzled, stored_globals,
                      m_per_expert, m_total, K, false, true);
}

int nv_kernels_silu_mul_quantize_nvfp4_bf16_per_expert_strided(void* stream, const uint16_t* y_gate_bf16,
                                                               const uint16_t* y_up_bf16, uint8_t* packed_out,
                                                               uint8_t* scales_out_swizzled,
                                                               const float* stored_globals, int m_per_expert,
                                                               int m_total, int K) {
    return per_expert(stream, y_gate_bf16, y_up_bf16, packed_out, scales_out_swizzled, stored_globals,
                      m_per_expert, m_total, K, true, true);
}

int nv_kernels_rmsnorm_bf16(void* stream, const uint16_t* x, const uint16_t* weight, uint16_t* y, size_t batch,
                            size_t hidden, float eps) {
    if (batch == 0 || hidden == 0) return 0;
    if (nvk::any_null(x, weight, y)) return NVK_ERR_ARG;
    if (batch > 0x7FFFFFFFull) return NVK_ERR_GRID_AXIS;
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, (unsigned)batch, 256, 0, true), rmsnorm_bf16_kernel, x, weight, y,
                       hidden, eps);
}

int nv_kernels_rmsnorm_quantize_nvfp4_bf16(void* stream, const uint16_t* x_bf16, const uint16_t* weight_bf16,
                                           uint8_t* packed_out, uint8_t* scales_out_swizzled, float stored_global,
                                           float eps, int m_padded, int m_logical, int K) {
    if (m_padded <= 0 || K <= 0) return 0;
    if (m_logical < 0 || m_logical > m_padded) return NVK_ERR_ARG;
    if ((K % 16) != 0) return NVK_ERR_SHAPE;
    const size_t smem = (size_t)K * sizeof(uint16_t);
    if (smem > 48 * 1024) return NVK_ERR_RESOURCE;
    if (reinterpret_cast<uintptr_t>(packed_out) & 7u) return NVK_ERR_ARG;
    if (nvk::any_null(weight_bf16, packed_out, scales_out_swizzled) || (m_logical > 0 && x_bf16 == nullptr))
        return NVK_ERR_ARG;
    QuantParams p = {};
    p.x = x_bf16; p.norm_w = weight_bf16; p.packed = packed_out; p.scales = scales_out_swizzled;
    p.global = stored_global; p.eps = eps; p.rows = m_padded; p.rows_logical = m_logical; p.K = K;
    p.row_mul = 1; p.m_per_expert = 1;
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, (unsigned)m_padded, 256, smem, true), rmsnorm_quantize_kernel, p);
}

}  // extern "C"
