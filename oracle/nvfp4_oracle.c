/*
 * CPU oracle for the NVFP4 weight-only linear path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped library links, loads or calls this file; it is the
 * checker that the CUDA path is compared against, and the CPU baseline that the
 * benchmark times beside it.
 *
 * Every function restates, in plain C, the arithmetic of the reference project
 * (eordano/speaches-plus); the citation beside each one is the reference file and
 * line it follows.  The reference is Rust and cannot be built where this runs, so
 * parity is pinned by the reference's own known-answer tests
 * (rust/crates/nv-quant/src/nvfp4.rs:1180-1563 and
 * rust/crates/nv-quant/tests/nvfp4_oracle_fuzz.rs), restated in tests/.
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC (see oracle/build.py).  -ffast-math must
 * not be used: rounding of each f32 operation is part of the contract.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define NVO_BLOCK 16

/* ---- bf16 <-> f32 (half 2.7.1 `bf16::from_f32`: round-to-nearest-even, NaN kept quiet) ---- */
float nvo_bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

uint16_t nvo_f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t round_bit = 0x00008000u;
    if ((u & round_bit) != 0 && (u & (3u * round_bit - 1u)) != 0) return (uint16_t)((u >> 16) + 1u);
    return (uint16_t)(u >> 16);
}

/* ---- e2m1: rust/crates/nv-quant/src/nvfp4.rs:4-36 ----
 * Nearest codebook entry, the FIRST minimum wins, so a tie goes to the lower code. */
static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

uint8_t nvo_encode_e2m1(float x) {
    uint8_t sign = signbit(x) ? 0x8 : 0x0;
    float a = fabsf(x);
    uint8_t best = 0;
    float best_err = INFINITY;
    for (int i = 0; i < 8; ++i) {
        float err = fabsf(a - kE2M1[i]);
        if (err < best_err) {
            best_err = err;
            best = (uint8_t)i;
        }
    }
    return (uint8_t)(sign | best);
}

float nvo_decode_e2m1(uint8_t code) {
    float m = kE2M1[code & 7];
    return (code & 8) ? -m : m;
}

/* ---- ue4m3: rust/crates/nv-quant/src/nvfp4.rs:38-85 ----
 * The reference takes floor(log2(x)); frexpf gives the same exponent exactly
 * (the reference pins this against f32 neighbours of powers of two in
 * rust/crates/nv-kernels/tests/ue4m3_log2f_boundary.rs). */
uint8_t nvo_encode_ue4m3(float scale) {
    if (!isfinite(scale) || scale <= 0.0f) return 0;
    float c = fminf(scale, 448.0f);
    if (c < 0.015625f) {
        int m = (int)roundf(c / 0.001953125f);
        if (m <= 0) return 0;
        if (m <= 7) return (uint8_t)m;
        return 0x08;
    }
    int e2;
    (void)frexpf(c, &e2);
    int exp = e2 - 1;
    float mant_f = c / ldexpf(1.0f, exp) - 1.0f;
    int mant = (int)roundf(mant_f * 8.0f);
    if (mant >= 8) {
        mant = 0;
        exp += 1;
    }
    if (mant < 0) mant = 0;
    if (mant > 7) mant = 7;
    int biased = exp + 7;
    if (biased < 1) biased = 1;
    if (biased > 15) biased = 15;
    uint8_t byte = (uint8_t)((biased << 3) | (mant & 7));
    return byte == 0x7F ? 0x7E : byte;
}

float nvo_decode_ue4m3(uint8_t byte) {
    int exp = (byte >> 3) & 0x0F;
    float mant = (float)(byte & 0x07);
    if (exp == 0) return mant * 0.001953125f;
    return (1.0f + mant / 8.0f) * ldexpf(1.0f, exp - 7);
}

/* ---- block quantizer: rust/crates/nv-quant/src/nvfp4.rs:91-129 ---- */
void nvo_quantize_block(const float* v, float stored_global, uint8_t* packed8, uint8_t* scale_byte) {
    float amax = 0.0f;
    for (int i = 0; i < NVO_BLOCK; ++i) amax = fmaxf(amax, fabsf(v[i]));
    float stored = (stored_global == 0.0f || !isfinite(stored_global)) ? 1.0f : stored_global;
    float local = (amax == 0.0f) ? 1.0f : amax / 6.0f;
    float stored_scale = stored * local;
    uint8_t sb = nvo_encode_ue4m3(stored_scale);
    float dec = nvo_decode_ue4m3(sb);
    float inv = (dec == 0.0f) ? 1.0f : stored / dec;
    for (int i = 0; i < NVO_BLOCK / 2; ++i) {
        float lo_v = fminf(fmaxf(v[2 * i] * inv, -6.0f), 6.0f);
        float hi_v = fminf(fmaxf(v[2 * i + 1] * inv, -6.0f), 6.0f);
        uint8_t lo = nvo_encode_e2m1(lo_v);
        uint8_t hi = nvo_encode_e2m1(hi_v);
        packed8[i] = (uint8_t)((hi << 4) | (lo & 0x0F));
    }
    *scale_byte = sb;
}

void nvo_dequantize_block(const uint8_t* packed8, uint8_t scale_byte, float* out16) {
    float s = nvo_decode_ue4m3(scale_byte);
    for (int i = 0; i < NVO_BLOCK / 2; ++i) {
        out16[2 * i] = nvo_decode_e2m1(packed8[i] & 0x0F) * s;
        out16[2 * i + 1] = nvo_decode_e2m1((packed8[i] >> 4) & 0x0F) * s;
    }
}

/* ---- row container: rust/crates/nv-quant/src/nvfp4.rs:131-165 (quantize_rows_with_global) ----
 * packed is [rows, cols/2], scales_linear is [rows, cols/16]. */
int nvo_quantize_rows(const float* x, int rows, int cols, float stored_global, uint8_t* packed,
                      uint8_t* scales_linear) {
    if (cols % NVO_BLOCK != 0) return -1;
    int bpr = cols / NVO_BLOCK;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        for (int b = 0; b < bpr; ++b) {
            nvo_quantize_block(x + (size_t)r * cols + (size_t)b * NVO_BLOCK, stored_global,
                               packed + (size_t)r * (cols / 2) + (size_t)b * 8,
                               scales_linear + (size_t)r * bpr + b);
        }
    }
    return 0;
}

/* Same, from bf16 bits: what the reference's device quantizer is fed
 * (rust/crates/nv-kernels/cuda/quantize_nvfp4_bf16.cu:73-120: each element is
 * widened to f32 first; rows at or past m_logical quantize as zeros). */
int nvo_quantize_rows_bf16(const uint16_t* x, int m_padded, int m_logical, int cols,
                           float stored_global, uint8_t* packed, uint8_t* scales_linear) {
    if (cols % NVO_BLOCK != 0) return -1;
    int bpr = cols / NVO_BLOCK;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < m_padded; ++r) {
        float v[NVO_BLOCK];
        for (int b = 0; b < bpr; ++b) {
            for (int i = 0; i < NVO_BLOCK; ++i)
                v[i] = (r < m_logical) ? nvo_bf16_to_f32(x[(size_t)r * cols + (size_t)b * NVO_BLOCK + i])
                                       : 0.0f;
            nvo_quantize_block(v, stored_global, packed + (size_t)r * (cols / 2) + (size_t)b * 8,
                               scales_linear + (size_t)r * bpr + b);
        }
    }
    return 0;
}

/* ---- scale swizzle: rust/crates/nv-quant/src/nvfp4.rs:231-264 ---- */
size_t nvo_swizzled_len(int rows, int k_blocks) {
    size_t m_tiles = ((size_t)rows + 127) / 128;
    size_t k_tiles = ((size_t)k_blocks + 3) / 4;
    return m_tiles * 128 * k_tiles * 4;
}

static size_t swz_index(int m, int kb, int k_blocks) {
    size_t k_tiles = ((size_t)k_blocks + 3) / 4;
    size_t m_tile = (size_t)m / 128;
    size_t d2 = ((size_t)m / 32) % 4;
    size_t d3 = (size_t)m % 32;
    size_t k_tile = (size_t)kb / 4;
    size_t d5 = (size_t)kb % 4;
    return ((m_tile * k_tiles + k_tile) * 32 + d3) * 16 + d2 * 4 + d5;
}

void nvo_swizzle_scales(const uint8_t* linear, int rows, int k_blocks, uint8_t* out) {
    memset(out, 0, nvo_swizzled_len(rows, k_blocks));
    for (int m = 0; m < rows; ++m)
        for (int kb = 0; kb < k_blocks; ++kb)
            out[swz_index(m, kb, k_blocks)] = linear[(size_t)m * k_blocks + kb];
}

void nvo_unswizzle_scales(const uint8_t* sw, int rows, int k_blocks, uint8_t* out) {
    for (int m = 0; m < rows; ++m)
        for (int kb = 0; kb < k_blocks; ++kb)
            out[(size_t)m * k_blocks + kb] = sw[swz_index(m, kb, k_blocks)];
}

/* ---- dequant: rust/crates/nv-quant/src/nvfp4.rs:266-305 ----
 * The scale is multiplied by weight_mult in f32 FIRST, then by the e2m1 value. */
int nvo_dequantize_packed_linear(const uint8_t* packed, const uint8_t* scales_linear, int rows,
                                 int cols, float weight_mult, float* out) {
    if (cols % NVO_BLOCK != 0) return -1;
    int bpr = cols / NVO_BLOCK;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        for (int b = 0; b < bpr; ++b) {
            float s = nvo_decode_ue4m3(scales_linear[(size_t)r * bpr + b]) * weight_mult;
            const uint8_t* p = packed + (size_t)r * (cols / 2) + (size_t)b * 8;
            float* o = out + (size_t)r * cols + (size_t)b * NVO_BLOCK;
            for (int i = 0; i < 8; ++i) {
                o[2 * i] = nvo_decode_e2m1(p[i] & 0x0F) * s;
                o[2 * i + 1] = nvo_decode_e2m1((p[i] >> 4) & 0x0F) * s;
            }
        }
    }
    return 0;
}

int nvo_dequantize_packed_swizzled(const uint8_t* packed, const uint8_t* scales_sw, int rows,
                                   int cols, float weight_mult, float* out) {
    if (cols % NVO_BLOCK != 0) return -1;
    int bpr = cols / NVO_BLOCK;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        for (int b = 0; b < bpr; ++b) {
            float s = nvo_decode_ue4m3(scales_sw[swz_index(r, b, bpr)]) * weight_mult;
            const uint8_t* p = packed + (size_t)r * (cols / 2) + (size_t)b * 8;
            float* o = out + (size_t)r * cols + (size_t)b * NVO_BLOCK;
            for (int i = 0; i < 8; ++i) {
                o[2 * i] = nvo_decode_e2m1(p[i] & 0x0F) * s;
                o[2 * i + 1] = nvo_decode_e2m1((p[i] >> 4) & 0x0F) * s;
            }
        }
    }
    return 0;
}

/* Dequantize straight to bf16 bits: the weight tensor the reference's Cpu backend
 * holds for an NVFP4 checkpoint (rust/crates/nv-models/src/train_runner.rs:101-127:
 * dequantize_packed_linear -> f32 tensor -> to_dtype(bf16)). */
int nvo_dequantize_to_bf16(const uint8_t* packed, const uint8_t* scales_sw, int rows, int cols,
                           float weight_mult, uint16_t* out) {
    if (cols % NVO_BLOCK != 0) return -1;
    int bpr = cols / NVO_BLOCK;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        for (int b = 0; b < bpr; ++b) {
            float s = nvo_decode_ue4m3(scales_sw[swz_index(r, b, bpr)]) * weight_mult;
            const uint8_t* p = packed + (size_t)r * (cols / 2) + (size_t)b * 8;
            uint16_t* o = out + (size_t)r * cols + (size_t)b * NVO_BLOCK;
            for (int i = 0; i < 8; ++i) {
                o[2 * i] = nvo_f32_to_bf16(nvo_decode_e2m1(p[i] & 0x0F) * s);
                o[2 * i + 1] = nvo_f32_to_bf16(nvo_decode_e2m1((p[i] >> 4) & 0x0F) * s);
            }
        }
    }
    return 0;
}

/* ---- the Cpu-backend linear: rust/crates/nv-layers/src/linear.rs:1148-1161 ----
 * bf16 weight and bf16 activation are widened to f32, y = x W^T with f32
 * accumulation, result cast to bf16.  The reference's matmul is the `gemm` crate
 * (candle-core 0.10.2 -> gemm 0.18; not in the reference tree); its blocked
 * summation order is not reproduced, the sum here runs k = 0..K-1 in order, as the
 * reference's own hand-written CPU GEMV does
 * (rust/crates/nv-layers/src/backend.rs:846-857).  threads <= 0 uses every core. */
int nvo_linear_cpu_backend(const uint16_t* w_bf16, const uint16_t* x_bf16, uint16_t* y_bf16, int M,
                           int N, int K, int threads) {
#ifdef _OPENMP
    int nt = threads > 0 ? threads : omp_get_max_threads();
#else
    int nt = 1;
    (void)threads;
#endif
    float* xf = (float*)__builtin_malloc((size_t)M * K * sizeof(float));
    if (!xf) return -1;
    for (size_t i = 0; i < (size_t)M * K; ++i) xf[i] = nvo_bf16_to_f32(x_bf16[i]);
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int n = 0; n < N; ++n) {
        const uint16_t* wr = w_bf16 + (size_t)n * K;
        for (int m = 0; m < M; ++m) {
            const float* xr = xf + (size_t)m * K;
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += nvo_bf16_to_f32(wr[k]) * xr[k];
            y_bf16[(size_t)m * N + n] = nvo_f32_to_bf16(acc);
        }
    }
    __builtin_free(xf);
    return 0;
}

/* The same linear with the summation order of a SIMD matmul: the reference's Cpu backend multiplies
 * through the `gemm` crate, which keeps several partial sums per output and adds them at the end
 * (its exact blocking is not in the reference tree).  Here each output keeps 16 partial sums -- lane j
 * takes k = j, j+16, j+32, ... in order -- which are then added pairwise (8+8, 4+4, 2+2, 1+1).  Every
 * product and sum is a separate f32 operation (no FMA), so the result is the same on every host; the
 * compiler turns the 16 lanes into vector instructions (AVX-512 / AVX2 / SSE chosen at load time).
 * This is the variant timed as the CPU baseline: a sequential scalar dot would understate what the
 * reference's multithreaded SIMD matmul does on the same cores. */
__attribute__((target_clones("avx512f", "avx2", "default"), optimize("O3")))
static float nvo_dot_bf16_f32_lanes16(const uint16_t* w, const float* x, int K) {
    float acc[16];
    for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
    int k = 0;
    for (; k + 16 <= K; k += 16) {
        for (int j = 0; j < 16; ++j) {
            union { uint32_t u; float f; } c;
            c.u = (uint32_t)w[k + j] << 16;
            acc[j] += c.f * x[k + j];
        }
    }
    for (; k < K; ++k) acc[k & 15] += nvo_bf16_to_f32(w[k]) * x[k];
    for (int s = 8; s >= 1; s >>= 1)
        for (int j = 0; j < s; ++j) acc[j] += acc[j + s];
    return acc[0];
}

int nvo_linear_cpu_backend_lanes16(const uint16_t* w_bf16, const uint16_t* x_bf16, uint16_t* y_bf16, int M,
                                   int N, int K, int threads) {
#ifdef _OPENMP
    int nt = threads > 0 ? threads : omp_get_max_threads();
#else
    int nt = 1;
    (void)threads;
#endif
    float* xf = (float*)__builtin_malloc((size_t)M * K * sizeof(float));
    if (!xf) return -1;
    for (size_t i = 0; i < (size_t)M * K; ++i) xf[i] = nvo_bf16_to_f32(x_bf16[i]);
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int n = 0; n < N; ++n) {
        const uint16_t* wr = w_bf16 + (size_t)n * K;
        for (int m = 0; m < M; ++m)
            y_bf16[(size_t)m * N + n] = nvo_f32_to_bf16(nvo_dot_bf16_f32_lanes16(wr, xf + (size_t)m * K, K));
    }
    __builtin_free(xf);
    return 0;
}

/* ---- exact-ish statement of the W4A16 contraction, f64 accumulate ----
 * y[m,n] = alpha * sum_k dequant(W)[n,k] * x[m,k]; the form the reference's GPU
 * parity test uses as its oracle (rust/crates/nv-quant/tests/nvfp4_m1_gemv_ab.rs:93-102:
 * dequantize_packed_swizzled with multiplier 1, f64 dot, alpha applied last). */
int nvo_linear_w4a16_f64(const uint8_t* packed, const uint8_t* scales_sw, const uint16_t* x_bf16,
                         float alpha, int M, int N, int K, double* y) {
    if (K % NVO_BLOCK != 0) return -1;
    int bpr = K / NVO_BLOCK;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            const uint16_t* xr = x_bf16 + (size_t)m * K;
            double acc = 0.0;
            for (int b = 0; b < bpr; ++b) {
                float s = nvo_decode_ue4m3(scales_sw[swz_index(n, b, bpr)]);
                const uint8_t* p = packed + (size_t)n * (K / 2) + (size_t)b * 8;
                for (int i = 0; i < 8; ++i) {
                    float w0 = nvo_decode_e2m1(p[i] & 0x0F) * s;
                    float w1 = nvo_decode_e2m1((p[i] >> 4) & 0x0F) * s;
                    acc += (double)w0 * (double)nvo_bf16_to_f32(xr[b * 16 + 2 * i]);
                    acc += (double)w1 * (double)nvo_bf16_to_f32(xr[b * 16 + 2 * i + 1]);
                }
            }
            y[(size_t)m * N + n] = acc * (double)alpha;
        }
    }
    return 0;
}

/* ---- W4A4 matmul oracle: rust/crates/nv-quant/src/nvfp4.rs:1086-1106 ----
 * Both operands dequantized with linear scales (multiplier 1), sequential f32 dot,
 * bf16 out; `alpha` (1.0 in the reference function) is applied in f32 before the cast. */
int nvo_matmul_w4a4(const uint8_t* a_packed, const uint8_t* a_scales_lin, const uint8_t* b_packed,
                    const uint8_t* b_scales_lin, float alpha, int M, int N, int K, uint16_t* d_bf16) {
    if (K % NVO_BLOCK != 0) return -1;
    float* a = (float*)__builtin_malloc((size_t)M * K * sizeof(float));
    float* b = (float*)__builtin_malloc((size_t)N * K * sizeof(float));
    if (!a || !b) {
        __builtin_free(a);
        __builtin_free(b);
        return -1;
    }
    nvo_dequantize_packed_linear(a_packed, a_scales_lin, M, K, 1.0f, a);
    nvo_dequantize_packed_linear(b_packed, b_scales_lin, N, K, 1.0f, b);
#pragma omp parallel for schedule(static)
    for (int j = 0; j < N; ++j) {
        for (int i = 0; i < M; ++i) {
            float acc = 0.0f;
            for (int p = 0; p < K; ++p) acc += a[(size_t)i * K + p] * b[(size_t)j * K + p];
            d_bf16[(size_t)i * N + j] = nvo_f32_to_bf16(alpha == 1.0f ? acc : acc * alpha);
        }
    }
    __builtin_free(a);
    __builtin_free(b);
    return 0;
}

/* ---- SiLU(gate)*up, the two roundings the reference uses ----
 * round_bf16 != 0: rust/crates/nv-kernels/cuda/gemv_nvfp4_w4a16_decode.cu:165-170
 *   (f32 silu, product rounded to bf16 before the down projection);
 * round_bf16 == 0: rust/crates/nv-kernels/cuda/quantize_nvfp4_bf16.cu:193-200
 *   (f32 silu, product kept in f32 and quantized). */
void nvo_silu_mul(const uint16_t* gate, const uint16_t* up, size_t n, int round_bf16, float* out) {
    for (size_t i = 0; i < n; ++i) {
        float g = nvo_bf16_to_f32(gate[i]);
        float u = nvo_bf16_to_f32(up[i]);
        float act = (g / (1.0f + expf(-g))) * u;
        out[i] = round_bf16 ? nvo_bf16_to_f32(nvo_f32_to_bf16(act)) : act;
    }
}

/* ---- router: rust/crates/nv-kernels/cuda/moe_route.cu:75-250 and
 * rust/crates/nv-layers/src/moe.rs:312-335 ----
 * mode 0: top-k of the (optionally tanh soft-capped) logits, softmax over the k
 * winners; mode 1: sigmoid scores, selection on score + bias, optional
 * renormalisation.  Ties go to the lower expert id.  Weights are multiplied by
 * routed_scaling last. */
int nvo_moe_route_topk(const float* logits, const float* bias, int32_t* ids, float* weights,
                       int n_tokens, int E, int K, int mode, float softcap, int norm_topk,
                       float routed_scaling) {
    if (K > E || K > 32) return -2;
    float* sel = (float*)__builtin_malloc((size_t)E * 2 * sizeof(float));
    if (!sel) return -1;
    float* raw = sel + E;
    for (int n = 0; n < n_tokens; ++n) {
        for (int e = 0; e < E; ++e) {
            float x = logits[(size_t)n * E + e];
            if (softcap > 0.0f) x = softcap * tanhf(x / softcap);
            if (mode == 1) {
                float s = 1.0f / (1.0f + expf(-x));
                raw[e] = s;
                sel[e] = s + (bias ? bias[e] : 0.0f);
            } else {
                raw[e] = x;
                sel[e] = x;
            }
        }
        float w[32];
        int id[32];
        for (int j = 0; j < K; ++j) {
            int bi = -1;
            float bv = -INFINITY;
            for (int e = 0; e < E; ++e) {
                if (sel[e] > bv || (bi < 0 && sel[e] == bv)) {
                    bv = sel[e];
                    bi = e;
                }
            }
            id[j] = bi;
            w[j] = bi >= 0 ? raw[bi] : 0.0f;
            if (bi >= 0) sel[bi] = -INFINITY;
        }
        if (mode == 0) {
            float mx = -INFINITY;
            for (int j = 0; j < K; ++j) mx = fmaxf(mx, w[j]);
            float sum = 0.0f;
            for (int j = 0; j < K; ++j) {
                w[j] = expf(w[j] - mx);
                sum += w[j];
            }
            for (int j = 0; j < K; ++j) w[j] /= sum;
        } else if (norm_topk) {
            float sum = 0.0f;
            for (int j = 0; j < K; ++j) sum += w[j];
            if (sum > 0.0f)
                for (int j = 0; j < K; ++j) w[j] /= sum;
        }
        for (int j = 0; j < K; ++j) {
            ids[(size_t)n * K + j] = id[j];
            weights[(size_t)n * K + j] = w[j] * routed_scaling;
        }
    }
    __builtin_free(sel);
    return 0;
}

/* ---- combine: rust/crates/nv-kernels/cuda/moe_unpermute_scatter.cu:6-32 ----
 * y_acc[n,h] = sum_s w[n,s] * bf16(y_sorted[inv_perm[n,s], h]), f32, s in order.  The reference
 * statement `acc += w * v` is device code, which nvcc contracts to one fused multiply-add; fmaf
 * states that rounding explicitly.  A negative row (a slot the slot sort left out because its
 * expert id was outside [0, E); the reference has no such rule and would index with it) adds nothing. */
void nvo_moe_unpermute_scatter(const uint16_t* y_sorted, const float* w, const int32_t* inv_perm,
                               float* y_acc, int n_tokens, int k, int H, int row_stride) {
    for (int n = 0; n < n_tokens; ++n)
        for (int h = 0; h < H; ++h) {
            float acc = 0.0f;
            for (int s = 0; s < k; ++s) {
                int row = inv_perm[n * k + s];
                if (row < 0) continue;
                acc = fmaf(w[n * k + s], nvo_bf16_to_f32(y_sorted[(size_t)row * row_stride + h]), acc);
            }
            y_acc[(size_t)n * H + h] = acc;
        }
}

int nvo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
