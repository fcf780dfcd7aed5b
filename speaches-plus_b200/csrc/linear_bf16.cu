// bf16 linear for a few tokens (2 <= M <= 64): y[m, n] = bf16( sum_k W[n, k] * x[m, k] ), fp32
// accumulate -- the lm_head of a batched decode step, where one pass over a 1.5 GB matrix has to serve
// every token of the batch.
//
// HBM-bound on W, which is streamed exactly once with 16-byte loads that bypass L1.  A warp owns 16
// weight rows (the A operand of mma.sync m16n8k16, bf16 in, fp32 out); the tokens are the columns of
// B, eight per MMA.  K is consumed in a permuted order: lane (g, tg) loads the 8 consecutive values
// W[row][k0 + 8 tg ..] of its two rows (one 16-byte load each) and the same 8 values of each token
// row of x, and the four register pairs feed two MMAs.  Both operands use the same permutation, so
// the dot product is unchanged.  x (M x K bf16, at most a few hundred KB) is read through L1/L2 by
// every CTA; nothing is staged in shared memory when a warp walks all of K.
//
// For matrices with few rows (a router's [experts, hidden]) the warps of a CTA split K instead and the
// partial tiles are added in a fixed order through shared memory.
#include "nvk_common.cuh"

namespace {

struct Bf16LinearArgs {
    const uint16_t* W;   // [N, K]
    const uint16_t* x;   // [M, K]
    uint16_t* y;         // [M, N]
    int M, N, K;
};

__device__ __forceinline__ uint4 zero4() { return make_uint4(0u, 0u, 0u, 0u); }

// NT: 8-token column tiles.  KW: warps of the CTA along K (1: a warp sums all of K for its 16 rows).
template <int NT, int KW>
__global__ void __launch_bounds__(256) linear_bf16_kernel(const Bf16LinearArgs a) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    constexpr int UNITS = 8 / KW;   // 16-row units per CTA
    __shared__ float s_red[KW > 1 ? KW * UNITS * 16 * 8 * NT : 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int unit = warp % UNITS, kw = warp / UNITS;
    const int gid = lane >> 2, tg = lane & 3;
    const int row0 = (blockIdx.x * UNITS + unit) * 16 + gid;   // second row is 8 further
    const int K = a.K, N = a.N, M = a.M;
    // rows past N read row N - 1 (valid memory) and are never stored
    const uint16_t* w0 = a.W + (size_t)min(row0, N - 1) * K + 8 * tg;
    const uint16_t* w1 = a.W + (size_t)min(row0 + 8, N - 1) * K + 8 * tg;
    const uint16_t* xr[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) xr[n] = a.x + (size_t)min(8 * n + gid, M - 1) * K + 8 * tg;

    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;

    // this warp's K range, in steps of 32 values (4 lanes x 8)
    const int steps = nvk::ceil_div(K, 32);
    const int per = nvk::ceil_div(steps, KW);
    const int s_begin = kw * per, s_end = min(steps, s_begin + per);
    constexpr int U = 4;   // steps in flight per lane: 2 * U independent 16-byte weight loads
    for (int s = s_begin; s < s_end; s += U) {
        uint4 wa[U], wb[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (s + u) * 32 + 8 * tg;
            const bool live = s + u < s_end && k < K;   // K % 8 == 0: a lane's 8 values are all in or all out
            wa[u] = live ? nvk::ptx::ldg_stream_v4(w0 + (size_t)(s + u) * 32) : zero4();
            wb[u] = live ? nvk::ptx::ldg_stream_v4(w1 + (size_t)(s + u) * 32) : zero4();
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (s + u) * 32 + 8 * tg;
            const bool live = s + u < s_end && k < K;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const uint4 xv = live ? __ldg(reinterpret_cast<const uint4*>(xr[n] + (size_t)(s + u) * 32)) : zero4();
                nvk::ptx::mma_m16n8k16_bf16(acc[n], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);
                nvk::ptx::mma_m16n8k16_bf16(acc[n], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv.z, xv.w);
            }
        }
    }

    if (KW > 1) {
        // red[kw][unit][token][row]: add the K-warps in order
        float* mine = s_red + ((size_t)(kw * UNITS + unit) * 8 * NT) * 16;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) mine[(8 * n + 2 * tg + (j & 1)) * 16 + gid + 8 * (j >> 1)] = acc[n][j];
        __syncthreads();
        if (kw != 0) return;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float v = 0.f;
                for (int w = 0; w < KW; ++w)
                    v += s_red[((size_t)(w * UNITS + unit) * 8 * NT + 8 * n + 2 * tg + (j & 1)) * 16 + gid + 8 * (j >> 1)];
                acc[n][j] = v;
            }
    }
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = 8 * n + 2 * tg + (j & 1);
            const int r = row0 + 8 * (j >> 1);
            if (m < M && r < N) a.y[(size_t)m * N + r] = nvk::f32_to_bf16_bits(acc[n][j]);
        }
}

template <int NT>
int launch_nt(cudaStream_t stream, const Bf16LinearArgs& a) {
    // a warp per 16 rows when that alone fills the GPU, else the eight warps of a CTA share 16 rows
    const bool split = nvk::ceil_div(a.N, 128) < 148;
    const unsigned grid = (unsigned)nvk::ceil_div(a.N, split ? 16 : 128);
    const nvk::Launch l = nvk::launch_1d(stream, grid, 256, 0, true);
    return split ? nvk::launch(l, linear_bf16_kernel<NT, 8>, a) : nvk::launch(l, linear_bf16_kernel<NT, 1>, a);
}

}  // namespace

extern "C" {

int nv_kernels_gemv_bf16(void* stream, const uint16_t* W, const uint16_t* x, uint16_t* y, int N, int K);

// y [M, N] = x [M, K] W^T for bf16 W [N, K], 1 <= M <= 64 (no counterpart with this signature in the
// reference, which sends bf16 linears with several rows to a library GEMM).  One pass over W for all
// rows of x when K % 8 == 0 and W and x are 16-byte aligned; other shapes, and M == 1, run the M = 1
// GEMV once per row.  -1 if M is outside [1, 64].
int nvk_b200_linear_bf16(void* stream, const uint16_t* W, const uint16_t* x, uint16_t* y, int M, int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    if (M <= 0 || M > 64) return NVK_ERR_SHAPE;
    if (nvk::any_null(W, x, y)) return NVK_ERR_ARG;
    const bool fast = M > 1 && (K & 7) == 0 &&
                      ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(x)) & 15u) == 0;
    if (!fast) {
        for (int m = 0; m < M; ++m)
            if (int rc = nv_kernels_gemv_bf16(stream, W, x + (size_t)m * K, y + (size_t)m * N, N, K)) return rc;
        return 0;
    }
    Bf16LinearArgs a;
    a.W = W; a.x = x; a.y = y; a.M = M; a.N = N; a.K = K;
    cudaStream_t s = (cudaStream_t)stream;
    if (M <= 8) return launch_nt<1>(s, a);
    if (M <= 16) return launch_nt<2>(s, a);
    if (M <= 32) return launch_nt<4>(s, a);
    return launch_nt<8>(s, a);
}

}  // extern "C"
