// MoE decode plumbing around the NVFP4 expert linears: router, slot sort, row gathers, weighted
// combine, and the single-token route + quantize step.
//
// Router.  A score becomes a 32-bit ORDER KEY (the float's bits remapped so that unsigned order is
// float order, NaN -> 0 = "cannot win"); every thread owns a contiguous run of experts in registers.
// One winner is two warp reductions (redux.sync): the largest key, then the smallest expert id among
// the lanes that hold it -- larger score first, lower id on ties.  An expert wins at most once; a row
// with fewer than K usable scores pads with id -1 / weight 0.  The weights use the same float
// operations in the same order as the per-winner loop they replace (max, exp, running sum over the
// winners in order, one division each), so ids and weights are reproducible bit for bit.
//
// Slot sort.  Routed slots (token-major) are sorted by expert with a counting sort that is stable
// by construction: one warp walks the slots 32 at a time in order, match.sync groups the lanes that
// name the same expert, and each lane's position is the expert's cursor plus the number of lower
// lanes in its group.  Expert ids outside [0, E) -- a router's -1 included -- are never used as an
// index: such slots get inv_perm = -1 and take no part, and the combine skips them.
#include "nvk_common.cuh"

namespace {

constexpr int kRouteMaxE = 4096;
constexpr int kRouteMaxK = 32;
constexpr unsigned kFullMask = 0xffffffffu;
constexpr uint32_t kNoWinner = 0xffffffffu;

// ---- order keys -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t order_key(float v) {
    if (v != v) return 0u;                       // NaN never wins
    if (v == 0.f) v = 0.f;                       // -0 and +0 compare equal: one key
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);   // >= 0x007FFFFF for every non-NaN value
}

struct RouteArgs {
    const float* logits;      // [n_tokens, E]
    const float* bias;        // [E] or null (mode 1 only)
    int32_t* topk_ids;        // [n_tokens, out_stride]
    float* topk_weights;      // [n_tokens, out_stride]
    int n_tokens, E, K, mode;
    float softcap;
    int norm_topk;
    float routed_scaling;
    int out_stride;           // K, or K + 1 with a shared-expert tail
    int shared_tail_id;       // < 0: none
};

// score of expert e for selection (`key`) and for the weights (`raw`)
__device__ __forceinline__ void score(const RouteArgs& a, const float* row, int e, uint32_t& key, float& raw) {
    float x = row[e];
    if (a.softcap > 0.f) x = a.softcap * tanhf(x / a.softcap);
    if (a.mode == 1) {
        const float s = 1.f / (1.f + expf(-x));
        raw = s;
        key = order_key(s + (a.bias ? a.bias[e] : 0.f));
    } else {
        raw = x;
        key = order_key(x);
    }
}

// Lane j < K holds winner j's raw score in `raw_j` (0 for a missing winner, which still takes part
// exactly like a present one, as a padded loop over K entries would).  Returns lane j's weight.
__device__ __forceinline__ float winner_weight(float raw_j, int K, int mode, int norm_topk, float routed_scaling) {
    float w = raw_j;
    if (mode == 0) {
        float mx = -INFINITY;
        for (int j = 0; j < K; ++j) mx = fmaxf(mx, __shfl_sync(kFullMask, raw_j, j));
        const float ex = expf(raw_j - mx);
        float sum = 0.f;
        for (int j = 0; j < K; ++j) sum += __shfl_sync(kFullMask, ex, j);
        w = ex / sum;
    } else if (norm_topk) {
        float sum = 0.f;
        for (int j = 0; j < K; ++j) sum += __shfl_sync(kFullMask, raw_j, j);
        if (sum > 0.f) w = raw_j / sum;
    }
    return w * routed_scaling;
}

// One token per warp, E <= 32 * R: lane L owns experts [L * R, L * R + R).  After the call lane
// j < K holds winner j in (id_j, raw_j).
template <int R>
__device__ __forceinline__ void route_token_warp(const RouteArgs& a, const float* row, int lane, int& id_j,
                                                 float& raw_j) {
    uint32_t key[R];
    float raw[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int e = lane * R + i;
        key[i] = 0u;
        raw[i] = 0.f;
        if (e < a.E) score(a, row, e, key[i], raw[i]);
    }
    id_j = -1;
    raw_j = 0.f;
    for (int j = 0; j < a.K; ++j) {
        uint32_t bk = 0u;
        int bi = 0;
        float br = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i)
            if (key[i] > bk) {   // strict: the lowest id of the lane's run keeps a tie
                bk = key[i];
                bi = i;
                br = raw[i];
            }
        const uint32_t top = __reduce_max_sync(kFullMask, bk);
        const uint32_t win = __reduce_min_sync(kFullMask, (top != 0u && bk == top) ? (uint32_t)(lane * R + bi) : kNoWinner);
        const bool found = win != kNoWinner;
        const int owner = found ? (int)(win / R) : 0;
        const float wr = __shfl_sync(kFullMask, br, owner);
        if (found && lane == owner) {
#pragma unroll
            for (int i = 0; i < R; ++i)
                if (i == bi) key[i] = 0u;
        }
        if (lane == j) {
            id_j = found ? (int)win : -1;
            raw_j = found ? wr : 0.f;
        }
    }
}

__device__ __forceinline__ void store_winner(const RouteArgs& a, int n, int lane, int id_j, float w_j) {
    if (lane < a.K) {
        a.topk_ids[(size_t)n * a.out_stride + lane] = id_j;
        a.topk_weights[(size_t)n * a.out_stride + lane] = w_j;
    }
    if (lane == 0 && a.shared_tail_id >= 0 && a.out_stride > a.K) {
        a.topk_ids[(size_t)n * a.out_stride + a.K] = a.shared_tail_id;
        a.topk_weights[(size_t)n * a.out_stride + a.K] = 1.f;
    }
}

// Router for E <= 256: eight tokens per CTA, one per warp, no shared memory, no barrier.
template <int R>
__global__ void __launch_bounds__(256) route_warp_kernel(const RouteArgs a) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= a.n_tokens) return;   // whole warps leave together
    int id_j;
    float raw_j;
    route_token_warp<R>(a, a.logits + (size_t)n * a.E, lane, id_j, raw_j);
    const float w_j = winner_weight(raw_j, a.K, a.mode, a.norm_topk, a.routed_scaling);
    store_winner(a, n, lane, id_j, w_j);
}

// Router for larger E (<= 256 * R): one token per CTA, thread t owns experts [t * R, t * R + R).
// A round is the warp reduction of route_token_warp followed by the same reduction over the eight
// warps' candidates, done redundantly by every warp from shared memory.
template <int R>
__global__ void __launch_bounds__(256) route_cta_kernel(const RouteArgs a) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    __shared__ uint32_t s_top[8], s_win[8];
    __shared__ float s_raw[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = blockIdx.x;
    const float* row = a.logits + (size_t)n * a.E;
    uint32_t key[R];
    float raw[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int e = tid * R + i;
        key[i] = 0u;
        raw[i] = 0.f;
        if (e < a.E) score(a, row, e, key[i], raw[i]);
    }
    int id_j = -1;
    float raw_j = 0.f;
    for (int j = 0; j < a.K; ++j) {
        uint32_t bk = 0u;
        int bi = 0;
        float br = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i)
            if (key[i] > bk) {
                bk = key[i];
                bi = i;
                br = raw[i];
            }
        const uint32_t top = __reduce_max_sync(kFullMask, bk);
        const uint32_t win = __reduce_min_sync(kFullMask, (top != 0u && bk == top) ? (uint32_t)(tid * R + bi) : kNoWinner);
        const int owner = win != kNoWinner ? (int)(win / R) & 31 : 0;
        const float wr = __shfl_sync(kFullMask, br, owner);
        if (lane == 0) {
            s_top[warp] = top;
            s_win[warp] = win;
            s_raw[warp] = wr;
        }
        __syncthreads();
        // every warp finishes the reduction over the eight candidates (lanes 8.. repeat lanes 0..7)
        const uint32_t ctop = __reduce_max_sync(kFullMask, s_top[lane & 7]);
        const uint32_t cwin =
            __reduce_min_sync(kFullMask, (ctop != 0u && s_top[lane & 7] == ctop) ? s_win[lane & 7] : kNoWinner);
        const bool found = cwin != kNoWinner;
        const float cr = found ? s_raw[(cwin / R) >> 5] : 0.f;
        if (found && tid == (int)(cwin / R)) {
#pragma unroll
            for (int i = 0; i < R; ++i)
                if (i == (int)(cwin % R)) key[i] = 0u;
        }
        if (warp == 0 && lane == j) {
            id_j = found ? (int)cwin : -1;
            raw_j = cr;
        }
        __syncthreads();   // the candidates are consumed before the next round overwrites them
    }
    if (warp == 0) {
        const float w_j = winner_weight(raw_j, a.K, a.mode, a.norm_topk, a.routed_scaling);
        store_winner(a, n, lane, id_j, w_j);
    }
}

int launch_router(cudaStream_t stream, const RouteArgs& a) {
    if (a.E <= 256) {
        const nvk::Launch l = nvk::launch_1d(stream, (unsigned)nvk::ceil_div(a.n_tokens, 8), 256, 0, true);
        if (a.E <= 32) return nvk::launch(l, route_warp_kernel<1>, a);
        if (a.E <= 64) return nvk::launch(l, route_warp_kernel<2>, a);
        if (a.E <= 128) return nvk::launch(l, route_warp_kernel<4>, a);
        return nvk::launch(l, route_warp_kernel<8>, a);
    }
    const nvk::Launch l = nvk::launch_1d(stream, (unsigned)a.n_tokens, 256, 0, true);
    if (a.E <= 512) return nvk::launch(l, route_cta_kernel<2>, a);
    if (a.E <= 1024) return nvk::launch(l, route_cta_kernel<4>, a);
    if (a.E <= 2048) return nvk::launch(l, route_cta_kernel<8>, a);
    return nvk::launch(l, route_cta_kernel<16>, a);
}

// ---- slot sort ----------------------------------------------------------------------------------
// `cursor[e]` holds the first sorted position of expert e on entry and is advanced as slots are
// placed.  Called by ONE warp; slots are visited in order, so the sort is stable.  `ids` may be
// shared or global memory.
__device__ __forceinline__ void place_slots_stable(const int32_t* ids, int32_t* cursor, int32_t* perm_token,
                                                   int32_t* inv_perm, int total, int k, int E, int lane) {
    for (int base = 0; base < total; base += 32) {
        const int t = base + lane;
        const int e = t < total ? ids[t] : -1;
        const bool ok = e >= 0 && e < E;
        // lanes with the same expert form a group; lanes without a valid expert group under -1
        const unsigned group = __match_any_sync(kFullMask, ok ? e : -1);
        if (ok) {
            const int before = __popc(group & ((1u << lane) - 1u));
            const int pos = cursor[e] + before;
            perm_token[pos] = t / k;
            inv_perm[t] = pos;
        } else if (t < total) {
            inv_perm[t] = -1;
        }
        __syncwarp();   // every lane has read its cursor before the group leaders advance them
        if (ok && (group & ((1u << lane) - 1u)) == 0u) cursor[e] += __popc(group);
        __syncwarp();
    }
}

// Exclusive scan of counts[0..E) by one CTA of 256 threads: offsets[0..E] and, in place, the cursors.
// GLOBAL: `counts` is global memory that other threads of the CTA updated with atomics; those live in
// L2, so the counts are read with L1 bypassed.
template <bool GLOBAL>
__device__ __forceinline__ int read_count(const int32_t* p) {
    return GLOBAL ? __ldcg(p) : *p;
}

template <bool GLOBAL>
__device__ __forceinline__ void scan_counts_cta(int32_t* counts, int32_t* offsets, int E, int32_t* s_part /*[257]*/) {
    const int tid = threadIdx.x;
    const int per = nvk::ceil_div(E, 256);
    const int e0 = min(E, tid * per), e1 = min(E, e0 + per);
    int sum = 0;
    for (int e = e0; e < e1; ++e) sum += read_count<GLOBAL>(counts + e);
    s_part[tid + 1] = sum;
    if (tid == 0) s_part[0] = 0;
    __syncthreads();
    if (tid < 32) {   // 256 partial sums: each lane owns eight in order, then a warp scan
        int local[8], run = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            local[i] = s_part[1 + tid * 8 + i];
            run += local[i];
        }
        int incl = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(kFullMask, incl, o);
            if (tid >= o) incl += up;
        }
        int acc = incl - run;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            acc += local[i];
            s_part[1 + tid * 8 + i] = acc;
        }
    }
    __syncthreads();
    int acc = s_part[tid];
    for (int e = e0; e < e1; ++e) {
        const int c = read_count<GLOBAL>(counts + e);
        offsets[e] = acc;
        counts[e] = acc;   // becomes the cursor
        acc += c;
    }
    if (tid == 255) offsets[E] = s_part[256];
    __syncthreads();
}

// Stand-alone sort: one CTA.  `counts` is caller scratch of E ints (any contents on entry).
__global__ void __launch_bounds__(256) slot_sort_kernel(const int32_t* __restrict__ topk_ids,
                                                        int32_t* __restrict__ perm_token,
                                                        int32_t* __restrict__ offsets, int32_t* __restrict__ inv_perm,
                                                        int32_t* __restrict__ counts, int total, int k, int E) {
    __shared__ int32_t s_part[257];
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += 256) counts[e] = 0;   // the scratch keeps the last call's contents
    __syncthreads();
    for (int t = tid; t < total; t += 256) {
        const int e = topk_ids[t];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    scan_counts_cta<true>(counts, offsets, E, s_part);
    if (tid < 32) place_slots_stable(topk_ids, counts, perm_token, inv_perm, total, k, E, tid);
}

// ---- router + sort in one launch (decode-sized steps) ---------------------------------------------
constexpr int kFusedMaxE = 256, kFusedMaxSlots = 4096;

struct RouteSortArgs {
    RouteArgs r;
    int32_t* perm_token;      // [n_tokens * K]
    int32_t* offsets;         // [E + 1]
    int32_t* inv_perm;        // [n_tokens * K]
    int32_t* active;          // optional [min(E, n_tokens * K)]: experts that received slots, ascending
    int32_t* n_active;        // optional [1]
};

template <int R>
__global__ void __launch_bounds__(256) route_sort_kernel(const RouteSortArgs a) {
    __shared__ int32_t s_ids[kFusedMaxSlots];
    __shared__ int32_t s_counts[kFusedMaxE];
    __shared__ int32_t s_offsets[kFusedMaxE + 1];
    __shared__ int32_t s_part[257];
    // The logits usually come from the kernel just before this one.
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int E = a.r.E, K = a.r.K, total = a.r.n_tokens * K;
    for (int e = tid; e < E; e += 256) s_counts[e] = 0;
    __syncthreads();
    for (int n = warp; n < a.r.n_tokens; n += 8) {
        int id_j;
        float raw_j;
        route_token_warp<R>(a.r, a.r.logits + (size_t)n * E, lane, id_j, raw_j);
        const float w_j = winner_weight(raw_j, K, a.r.mode, a.r.norm_topk, a.r.routed_scaling);
        store_winner(a.r, n, lane, id_j, w_j);
        if (lane < K) {
            s_ids[n * K + lane] = id_j;
            if (id_j >= 0) atomicAdd(&s_counts[id_j], 1);
        }
    }
    __syncthreads();
    if (a.active != nullptr && warp == 1) {
        // compact list of the experts with at least one slot, in ascending order (one warp, in order)
        int n_act = 0;
        for (int base = 0; base < E; base += 32) {
            const int e = base + lane;
            const bool on = e < E && s_counts[e] > 0;
            const unsigned m = __ballot_sync(kFullMask, on);
            if (on) a.active[n_act + __popc(m & ((1u << lane) - 1u))] = e;
            n_act += __popc(m);
        }
        if (lane == 0 && a.n_active != nullptr) *a.n_active = n_act;
    }
    __syncthreads();
    scan_counts_cta<false>(s_counts, s_offsets, E, s_part);
    for (int e = tid; e <= E; e += 256) a.offsets[e] = s_offsets[e];
    if (warp == 0) place_slots_stable(s_ids, s_counts, a.perm_token, a.inv_perm, total, K, E, lane);
}

// ---- gathers --------------------------------------------------------------------------------------
// out[r] = x[src_idx[r]] for the rows r = i * row_step; an index outside [0, n_tokens) gives a zero row.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint16_t* __restrict__ x,
                                                          const int32_t* __restrict__ src_idx,
                                                          uint16_t* __restrict__ out, int rows, int hidden,
                                                          int n_tokens, int row_step) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int r = blockIdx.x * row_step;
    if (r >= rows) return;
    const int s = src_idx[r];
    const bool live = s >= 0 && s < n_tokens;
    const uint16_t* src = x + (size_t)(live ? s : 0) * hidden;
    uint16_t* dst = out + (size_t)r * hidden;
    if ((hidden & 7) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0) {
        for (int i = threadIdx.x; i < (hidden >> 3); i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = live ? reinterpret_cast<const uint4*>(src)[i] : make_uint4(0u, 0u, 0u, 0u);
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = live ? src[i] : (uint16_t)0;
    }
}

__global__ void __launch_bounds__(128) gather_f32_kernel(const float* __restrict__ src, const int32_t* __restrict__ ids,
                                                         float* __restrict__ dst, int n) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = ids[i];
    dst[i] = e >= 0 ? src[e] : 0.f;
}

// ---- combine --------------------------------------------------------------------------------------
// acc[n, h] = sum over the token's slots s, in order, of w[n, s] * y_sorted[inv_perm[n, s], h] in f32
// (one fused multiply-add per slot).
// A slot whose row is negative (a slot the sort left out) or not below `sorted_rows` contributes
// nothing.  TAIL: out = bf16(resid + bf16(acc + shared)) instead of storing acc.
// Each thread owns eight consecutive h of one token (one 16-byte load per slot).
struct CombineArgs {
    const uint16_t* y_sorted;
    const float* weights;
    const int32_t* inv_perm;
    float* y_acc;
    const float* shared_f32;
    const uint16_t* resid;
    uint16_t* out;
    int n_tokens, k, hidden, row_stride;
    int sorted_rows;   // rows of y_sorted; INT_MAX when the caller gives no bound
    int* status;       // optional: bit 2 set when a row index was not below sorted_rows
};

template <bool TAIL, bool VEC>
__global__ void __launch_bounds__(128) combine_kernel(const CombineArgs a) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    constexpr int W = VEC ? 8 : 1;
    const int n = blockIdx.y;
    const int h0 = (blockIdx.x * 128 + threadIdx.x) * W;
    if (h0 >= a.hidden) return;
    float acc[W];
#pragma unroll
    for (int i = 0; i < W; ++i) acc[i] = 0.f;
    for (int s = 0; s < a.k; ++s) {
        const int slot = n * a.k + s;
        const int row = a.inv_perm[slot];
        if (row < 0) continue;
        if (row >= a.sorted_rows) {
            if (a.status != nullptr && threadIdx.x == 0 && blockIdx.x == 0) atomicOr(a.status, 4);
            continue;
        }
        const float w = a.weights[slot];
        const uint16_t* src = a.y_sorted + (size_t)row * a.row_stride + h0;
        if (VEC) {
            const uint4 v = *reinterpret_cast<const uint4*>(src);
            const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[2 * i] = fmaf(w, nvk::bf16_bits_to_f32(ws[i] & 0xFFFFu), acc[2 * i]);
                acc[2 * i + 1] = fmaf(w, nvk::bf16_bits_to_f32(ws[i] >> 16), acc[2 * i + 1]);
            }
        } else {
            acc[0] = fmaf(w, nvk::bf16_bits_to_f32(src[0]), acc[0]);
        }
    }
    const size_t o = (size_t)n * a.hidden + h0;
#pragma unroll
    for (int i = 0; i < W; ++i) {
        if (TAIL) {
            const float moe = nvk::bf16_bits_to_f32(nvk::f32_to_bf16_bits(acc[i] + a.shared_f32[o + i]));
            a.out[o + i] = nvk::f32_to_bf16_bits(nvk::bf16_bits_to_f32(a.resid[o + i]) + moe);
        } else {
            a.y_acc[o + i] = acc[i];
        }
    }
}

// ---- expert-parallel combine: the weighted sum and the sum over GPUs in one launch --------------------
// Every GPU ran the slots of its own experts (the other slots' rows are zeros or skipped), so its combine
// yields a partial y_acc.  Each CTA stores its 128 x 8 f32 partials into its own region of every GPU's
// inbox (plain peer stores), raises one flag per GPU, waits -- bounded -- for the CTA of the same index
// on every other GPU and writes the sum in rank order: the same bits on every GPU.  Buffer layout (one
// per rank): [flags: max_ctas x 8 uint32][inbox: 2 parities x world x max_ctas x 1024 f32].
struct CombineXchArgs {
    uint8_t* peer[8];
    uint32_t* epoch;
    int* err;
    int rank, world, max_ctas;
    unsigned wait_limit;
};
constexpr int kCombineCtaElems = 1024;
__host__ __device__ inline size_t combine_xch_flag_bytes(int max_ctas) { return (size_t)max_ctas * 8 * sizeof(uint32_t); }

__global__ void __launch_bounds__(128) combine_allreduce_kernel(const CombineArgs a, const __grid_constant__ CombineXchArgs x) {
    __shared__ int s_ok;
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int n = blockIdx.y;
    const int h0 = (blockIdx.x * 128 + threadIdx.x) * 8;
    const int cta = (int)(blockIdx.y * gridDim.x + blockIdx.x);
    const uint32_t call = x.epoch[cta] + 1u;
    const bool live = h0 < a.hidden;          // hidden % 8 == 0: a thread's eight values are all in or all out
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (live) {
        for (int s = 0; s < a.k; ++s) {
            const int slot = n * a.k + s;
            const int row = a.inv_perm[slot];
            if (row < 0) continue;
            if (row >= a.sorted_rows) {
                if (a.status != nullptr && threadIdx.x == 0 && blockIdx.x == 0) atomicOr(a.status, 4);
                continue;
            }
            const float w = a.weights[slot];
            const uint4 v = *reinterpret_cast<const uint4*>(a.y_sorted + (size_t)row * a.row_stride + h0);
            const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[2 * i] = fmaf(w, nvk::bf16_bits_to_f32(ws[i] & 0xFFFFu), acc[2 * i]);
                acc[2 * i + 1] = fmaf(w, nvk::bf16_bits_to_f32(ws[i] >> 16), acc[2 * i + 1]);
            }
        }
    }
    const size_t region = (size_t)x.world * x.max_ctas * kCombineCtaElems;    // f32 per parity
    auto slot_of = [&](int src_rank) {
        return (size_t)(call & 1u) * region + ((size_t)src_rank * x.max_ctas + cta) * kCombineCtaElems + threadIdx.x * 8;
    };
    if (live) {
        const float4 lo = make_float4(acc[0], acc[1], acc[2], acc[3]), hi = make_float4(acc[4], acc[5], acc[6], acc[7]);
        for (int g = 0; g < x.world; ++g) {
            float* inbox = reinterpret_cast<float*>(x.peer[g] + combine_xch_flag_bytes(x.max_ctas));
            float4* dst = reinterpret_cast<float4*>(inbox + slot_of(x.rank));
            dst[0] = lo;
            dst[1] = hi;
        }
    }
    if (threadIdx.x == 0) s_ok = 1;
    __threadfence_system();
    __syncthreads();
    uint8_t* own = x.peer[x.rank];
    if ((int)threadIdx.x < x.world) {
        const int g = (int)threadIdx.x;
        nvk::ptx::st_release_sys(reinterpret_cast<uint32_t*>(x.peer[g]) + cta * 8 + x.rank, call);
        if (!nvk::bounded_wait_ge(reinterpret_cast<const uint32_t*>(own) + cta * 8 + g, call, x.wait_limit)) {
            atomicExch(x.err, 1 + g);
            s_ok = 0;
        }
    }
    __syncthreads();
    if (s_ok && live) {
        const float* inbox = reinterpret_cast<const float*>(own + combine_xch_flag_bytes(x.max_ctas));
        float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int g = 0; g < x.world; ++g) {
            const float4* src = reinterpret_cast<const float4*>(inbox + slot_of(g));
            const float4 lo = src[0], hi = src[1];
            sum[0] += lo.x; sum[1] += lo.y; sum[2] += lo.z; sum[3] += lo.w;
            sum[4] += hi.x; sum[5] += hi.y; sum[6] += hi.z; sum[7] += hi.w;
        }
        float4* out = reinterpret_cast<float4*>(a.y_acc + (size_t)n * a.hidden + h0);
        out[0] = make_float4(sum[0], sum[1], sum[2], sum[3]);
        out[1] = make_float4(sum[4], sum[5], sum[6], sum[7]);
    }
    __syncthreads();
    if (threadIdx.x == 0) x.epoch[cta] = call;   // also after a failed wait: the ranks stay in step
}

template <bool TAIL>
int launch_combine(cudaStream_t stream, const CombineArgs& a) {
    const bool vec = (a.hidden & 7) == 0 && (a.row_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(a.y_sorted) & 15u) == 0;
    nvk::Launch l;
    l.grid = dim3((unsigned)nvk::ceil_div(a.hidden, 128 * (vec ? 8 : 1)), (unsigned)a.n_tokens, 1);
    l.block = dim3(128, 1, 1);
    l.stream = stream;
    l.pdl = true;
    if (a.n_tokens > 65535) return NVK_ERR_GRID_AXIS;
    return vec ? nvk::launch(l, combine_kernel<TAIL, true>, a) : nvk::launch(l, combine_kernel<TAIL, false>, a);
}

// y[r, h] = x[r, h] * sigmoid(gate_logits[r]): the shared expert's gate (one logit per token).
__global__ void __launch_bounds__(256) rowgate_kernel(const float* __restrict__ x, const float* __restrict__ gate_logits,
                                                      float* __restrict__ y, int rows, int hidden) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * hidden) return;
    const float g = 1.f / (1.f + expf(-gate_logits[(int)(i / hidden)]));
    y[i] = x[i] * g;
}

// ---- single-token route + per-tile quantize -----------------------------------------------------------
// One decode token: route it, look up each winner's (and the shared tail's) activation globals, and
// quantize the token's row once per tile with that tile's gate/up global -- row t * min_tile of x_fp4
// and its swizzled scale.  A 16-value block is loaded and its maximum taken once; only the global
// differs between tiles.
struct RouteQuantArgs {
    RouteArgs r;              // n_tokens = 1, out_stride = K + (tail ? 1 : 0)
    const uint16_t* x;        // [hidden] bf16
    const float* globals_gu;  // [E (+ tail)] stored activation globals of gate/up
    const float* globals_dn;  // the same for down
    float* gu_mini;           // [tiles]
    float* dn_mini;           // [tiles]
    uint8_t* x_fp4;           // [tiles * min_tile, hidden / 2]
    uint8_t* x_sf;            // swizzled scales of those rows
    int hidden, min_tile;
};

template <int R>
__global__ void __launch_bounds__(256) route_quant_m1_kernel(const RouteQuantArgs a) {
    __shared__ float s_stored[kRouteMaxK];
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = a.r.K;
    const int tiles = K + (a.r.shared_tail_id >= 0 ? 1 : 0);
    if (warp == 0) {
        int id_j;
        float raw_j;
        route_token_warp<R>(a.r, a.r.logits, lane, id_j, raw_j);
        const float w_j = winner_weight(raw_j, K, a.r.mode, a.r.norm_topk, a.r.routed_scaling);
        store_winner(a.r, 0, lane, id_j, w_j);
        if (lane < tiles) {
            const int id = lane < K ? id_j : a.r.shared_tail_id;
            const float g_gu = id >= 0 ? a.globals_gu[id] : 0.f;
            const float g_dn = id >= 0 ? a.globals_dn[id] : 0.f;
            a.gu_mini[lane] = g_gu;
            a.dn_mini[lane] = g_dn;
            s_stored[lane] = (g_gu == 0.f || !isfinite(g_gu)) ? 1.f : g_gu;
        }
    }
    __syncthreads();
    const int blocks = a.hidden >> 4;
    for (int kb = tid; kb < blocks; kb += 256) {
        const uint4* src = reinterpret_cast<const uint4*>(a.x + (size_t)kb * 16);
        const uint4 p0 = src[0], p1 = src[1];
        const uint32_t ws[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        float v[16], amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[2 * i] = nvk::bf16_bits_to_f32(ws[i] & 0xFFFFu);
            v[2 * i + 1] = nvk::bf16_bits_to_f32(ws[i] >> 16);
            amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
        }
        const float local = amax == 0.f ? 1.f : amax / 6.f;
        for (int t = 0; t < tiles; ++t) {
            const float stored = s_stored[t];
            const uint32_t sb = nvk::encode_ue4m3(stored * local);
            const float dec = nvk::ue4m3_to_f32(sb);
            const float inv = dec == 0.f ? 1.f : stored / dec;
            uint32_t w[2] = {0u, 0u};
#pragma unroll
            for (int i = 0; i < 16; ++i)
                w[i >> 3] |= nvk::encode_e2m1(fminf(fmaxf(v[i] * inv, -6.f), 6.f)) << (4 * (i & 7));
            const int row = t * a.min_tile;
            *reinterpret_cast<uint2*>(a.x_fp4 + (size_t)row * (a.hidden >> 1) + (size_t)kb * 8) = make_uint2(w[0], w[1]);
            a.x_sf[nvk::swz_offset(row, kb, blocks)] = (uint8_t)sb;
        }
    }
}

// ---- device timestamp -------------------------------------------------------------------------------
__global__ void timestamp_kernel(unsigned long long* out) { *out = nvk::ptx::globaltimer_ns(); }

RouteArgs route_args(const float* logits, const float* bias, int32_t* ids, float* w, int n_tokens, int E, int K, int mode,
                     float softcap, int norm_topk, float routed_scaling, int out_stride, int tail) {
    RouteArgs a;
    a.logits = logits; a.bias = bias; a.topk_ids = ids; a.topk_weights = w;
    a.n_tokens = n_tokens; a.E = E; a.K = K; a.mode = mode; a.softcap = softcap; a.norm_topk = norm_topk;
    a.routed_scaling = routed_scaling; a.out_stride = out_stride; a.shared_tail_id = tail;
    return a;
}

int gather_rows(void* stream, const uint16_t* x, const int32_t* src_idx, uint16_t* out, int rows, int hidden,
                int n_tokens, int row_step) {
    const int block = hidden >= 2048 ? 256 : (hidden >= 512 ? 64 : 32);
    const unsigned grid = (unsigned)(rows / row_step);
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, grid, (unsigned)block, 0, true), gather_rows_kernel, x, src_idx, out,
                       rows, hidden, n_tokens, row_step);
}

int slot_sort(void* stream, const int32_t* topk_ids, int32_t* perm_token, int32_t* offsets, int32_t* inv_perm,
              int32_t* counts, int n_tokens, int k, int E) {
    const long long total = (long long)n_tokens * k;
    if (total > 0x7FFFFFFFLL) return NVK_ERR_GRID_AXIS;
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, 1, 256, 0, true), slot_sort_kernel, topk_ids, perm_token,
                       offsets, inv_perm, counts, (int)total, k, E);
}

}  // namespace

extern "C" {

int nv_kernels_mul_sigmoid_rowgate_f32(void* stream, const float* x, const float* gate_logits, float* y, int rows,
                                       int hidden) {
    if (rows <= 0 || hidden <= 0) return 0;
    if (nvk::any_null(x, gate_logits, y)) return NVK_ERR_ARG;
    const long long grid = ((long long)rows * hidden + 255) / 256;
    if (grid > 0x7FFFFFFFLL) return NVK_ERR_GRID_AXIS;
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, (unsigned)grid, 256, 0, true), rowgate_kernel, x, gate_logits, y, rows,
                       hidden);
}

int nv_kernels_moe_route_topk(void* stream, const float* logits, const float* bias, int32_t* topk_ids,
                              float* topk_weights, int n_tokens, int E, int K, int mode, float softcap,
                              int norm_topk, float routed_scaling) {
    if (n_tokens <= 0 || E <= 0 || K <= 0) return 0;
    if (E > kRouteMaxE || K > kRouteMaxK || K > E) return NVK_ERR_ARG;
    if (nvk::any_null(logits, topk_ids, topk_weights)) return NVK_ERR_ARG;
    return launch_router((cudaStream_t)stream, route_args(logits, bias, topk_ids, topk_weights, n_tokens, E, K, mode,
                                                          softcap, norm_topk, routed_scaling, K, -1));
}

int nv_kernels_moe_route_topk_shared_tail(void* stream, const float* logits, const float* bias, int32_t* topk_ids,
                                          float* topk_weights, int n_tokens, int E, int K, int mode, float softcap,
                                          int norm_topk, float routed_scaling, int shared_tail_id) {
    if (n_tokens <= 0 || E <= 0 || K <= 0) return 0;
    if (E > kRouteMaxE || K + 1 > kRouteMaxK || K > E) return NVK_ERR_ARG;
    if (shared_tail_id < 0) return NVK_ERR_RESOURCE;
    if (nvk::any_null(logits, topk_ids, topk_weights)) return NVK_ERR_ARG;
    return launch_router((cudaStream_t)stream, route_args(logits, bias, topk_ids, topk_weights, n_tokens, E, K, mode,
                                                          softcap, norm_topk, routed_scaling, K + 1, shared_tail_id));
}

int nv_kernels_moe_route_gather_quant_m1(void* stream, const float* logits, const float* bias, const uint16_t* x_bf16,
                                         const float* globals_gu, const float* globals_dn, int32_t* topk_ids,
                                         float* topk_weights, float* gu_mini, float* dn_mini, uint8_t* x_fp4,
                                         uint8_t* x_sf, int E, int K, int mode, float softcap, int norm_topk,
                                         float routed_scaling, int shared_tail_id, int hidden, int min_tile) {
    if (E <= 0 || K <= 0 || hidden <= 0 || min_tile <= 0) return NVK_ERR_SHAPE;
    if (E > 256 || K + 1 > kRouteMaxK || K > E) return NVK_ERR_ARG;
    if ((hidden % 16) != 0 || (min_tile % 128) != 0) return NVK_ERR_RESOURCE;
    if (nvk::any_null(logits, x_bf16, globals_gu, globals_dn, topk_ids, topk_weights, gu_mini, dn_mini, x_fp4, x_sf))
        return NVK_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) || (reinterpret_cast<uintptr_t>(x_fp4) & 7u)) return NVK_ERR_ARG;
    RouteQuantArgs a;
    const int tiles = K + (shared_tail_id >= 0 ? 1 : 0);
    a.r = route_args(logits, bias, topk_ids, topk_weights, 1, E, K, mode, softcap, norm_topk, routed_scaling, tiles,
                     shared_tail_id);
    a.x = x_bf16; a.globals_gu = globals_gu; a.globals_dn = globals_dn; a.gu_mini = gu_mini; a.dn_mini = dn_mini;
    a.x_fp4 = x_fp4; a.x_sf = x_sf; a.hidden = hidden; a.min_tile = min_tile;
    const nvk::Launch l = nvk::launch_1d((cudaStream_t)stream, 1, 256, 0, true);
    if (E <= 32) return nvk::launch(l, route_quant_m1_kernel<1>, a);
    if (E <= 64) return nvk::launch(l, route_quant_m1_kernel<2>, a);
    if (E <= 128) return nvk::launch(l, route_quant_m1_kernel<4>, a);
    return nvk::launch(l, route_quant_m1_kernel<8>, a);
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
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, (unsigned)((n + 127) / 128), 128, 0, true), gather_f32_kernel, src, ids,
                       dst, n);
}

static int combine(void* stream, const uint16_t* y_sorted, const float* w, const int32_t* inv_perm, float* y_acc,
                   const float* shared_f32, const uint16_t* resid, uint16_t* out, int n_tokens, int k, int hidden,
                   int row_stride, int sorted_rows, int* status, bool tail) {
    CombineArgs a;
    a.y_sorted = y_sorted; a.weights = w; a.inv_perm = inv_perm; a.y_acc = y_acc; a.shared_f32 = shared_f32;
    a.resid = resid; a.out = out; a.n_tokens = n_tokens; a.k = k; a.hidden = hidden; a.row_stride = row_stride;
    a.sorted_rows = sorted_rows; a.status = status;
    return tail ? launch_combine<true>((cudaStream_t)stream, a) : launch_combine<false>((cudaStream_t)stream, a);
}

int nv_kernels_moe_unpermute_scatter(void* stream, const uint16_t* y_sorted_bf16, const float* topk_weights,
                                     const int32_t* inv_perm, float* y_acc_f32, int n_tokens, int k, int hidden,
                                     int y_sorted_row_stride) {
    if (n_tokens <= 0 || k <= 0 || hidden <= 0) return 0;
    if (y_sorted_row_stride < hidden) return NVK_ERR_ARG;
    if (nvk::any_null(y_sorted_bf16, topk_weights, inv_perm, y_acc_f32)) return NVK_ERR_ARG;
    return combine(stream, y_sorted_bf16, topk_weights, inv_perm, y_acc_f32, nullptr, nullptr, nullptr, n_tokens, k,
                   hidden, y_sorted_row_stride, 0x7FFFFFFF, nullptr, false);
}

int nv_kernels_moe_unpermute_scatter_tail(void* stream, const uint16_t* y_sorted_bf16, const float* topk_weights,
                                          const int32_t* inv_perm, const float* shared_f32,
                                          const uint16_t* resid_bf16, uint16_t* out_bf16, int n_tokens, int k,
                                          int hidden, int y_sorted_row_stride) {
    if (n_tokens <= 0 || k <= 0 || hidden <= 0) return 0;
    if (y_sorted_row_stride < hidden) return NVK_ERR_ARG;
    if (nvk::any_null(y_sorted_bf16, topk_weights, inv_perm, shared_f32, resid_bf16, out_bf16)) return NVK_ERR_ARG;
    return combine(stream, y_sorted_bf16, topk_weights, inv_perm, nullptr, shared_f32, resid_bf16, out_bf16, n_tokens, k,
                   hidden, y_sorted_row_stride, 0x7FFFFFFF, nullptr, true);
}

// The weighted combine with the sorted buffer's row count known (no counterpart in the reference,
// whose entry point trusts inv_perm): a row index not below `sorted_rows` is skipped and reported in
// bit 2 of `status` (one device int zeroed by the caller; may be NULL).
int nvk_b200_moe_combine(void* stream, const uint16_t* y_sorted_bf16, const float* topk_weights, const int32_t* inv_perm,
                         float* y_acc_f32, int n_tokens, int k, int hidden, int y_sorted_row_stride, int sorted_rows,
                         int* status) {
    if (n_tokens <= 0 || k <= 0 || hidden <= 0) return 0;
    if (y_sorted_row_stride < hidden || sorted_rows < 0) return NVK_ERR_ARG;
    if (nvk::any_null(y_sorted_bf16, topk_weights, inv_perm, y_acc_f32)) return NVK_ERR_ARG;
    return combine(stream, y_sorted_bf16, topk_weights, inv_perm, y_acc_f32, nullptr, nullptr, nullptr, n_tokens, k,
                   hidden, y_sorted_row_stride, sorted_rows, status, false);
}

// Bytes of the exchange buffer every rank provides (zero before the first call) for
// nvk_b200_moe_combine_allreduce launches of up to max_ctas CTAs; 0 for arguments out of range.
size_t nvk_b200_moe_combine_buffer_bytes(int world, int max_ctas) {
    if (world <= 0 || world > 8 || max_ctas <= 0 || max_ctas > 4096) return 0;
    return combine_xch_flag_bytes(max_ctas) + (size_t)2 * world * max_ctas * kCombineCtaElems * sizeof(float);
}

// Expert-parallel combine (no counterpart in the reference, which has no multi-GPU path): every rank
// passes the rows of ITS experts' slots (inv_perm < 0 or zero rows for the others); y_acc [n_tokens,
// hidden] receives the sum over ranks of the ranks' weighted combines, added in rank order -- the same
// bits on every rank -- without a separate all-reduce.  hidden % 8 == 0, the sorted rows 16-byte
// aligned.  peer_bufs / epoch (max_ctas uint32, zero before the first call) / err as for
// nvk_b200_tp_linear_nvfp4_w4a16_allreduce; all ranks make the same sequence of calls.  -2 for bad
// arguments, -3 when ceil(hidden / 1024) * n_tokens exceeds max_ctas.
int nvk_b200_moe_combine_allreduce(void* stream, const void* const* peer_bufs, int rank, int world,
                                   const uint16_t* y_sorted_bf16, const float* topk_weights, const int32_t* inv_perm,
                                   float* y_acc_f32, int n_tokens, int k, int hidden, int y_sorted_row_stride,
                                   int sorted_rows, int* status, int max_ctas, uint32_t* epoch, int* err) {
    if (n_tokens <= 0 || k <= 0 || hidden <= 0) return 0;
    if (y_sorted_row_stride < hidden || sorted_rows < 0 || (hidden & 7) != 0 || (y_sorted_row_stride & 7) != 0)
        return NVK_ERR_ARG;
    if (world <= 0 || world > 8 || rank < 0 || rank >= world || max_ctas <= 0 || max_ctas > 4096) return NVK_ERR_ARG;
    if (!peer_bufs || nvk::any_null(y_sorted_bf16, topk_weights, inv_perm, y_acc_f32, epoch, err)) return NVK_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(y_sorted_bf16) | reinterpret_cast<uintptr_t>(y_acc_f32)) & 15u) return NVK_ERR_ARG;
    const long ctas = (long)nvk::ceil_div(hidden, 1024) * n_tokens;
    if (ctas > max_ctas || n_tokens > 65535) return NVK_ERR_RESOURCE;
    CombineArgs a = {};
    a.y_sorted = y_sorted_bf16; a.weights = topk_weights; a.inv_perm = inv_perm; a.y_acc = y_acc_f32;
    a.n_tokens = n_tokens; a.k = k; a.hidden = hidden; a.row_stride = y_sorted_row_stride;
    a.sorted_rows = sorted_rows; a.status = status;
    CombineXchArgs x = {};
    for (int r = 0; r < world; ++r) {
        if (!peer_bufs[r]) return NVK_ERR_ARG;
        x.peer[r] = static_cast<uint8_t*>(const_cast<void*>(peer_bufs[r]));
    }
    x.epoch = epoch; x.err = err; x.rank = rank; x.world = world; x.max_ctas = max_ctas;
    x.wait_limit = nvk::wait_limit_setting();
    nvk::Launch l;
    l.grid = dim3((unsigned)nvk::ceil_div(hidden, 1024), (unsigned)n_tokens, 1);
    l.block = dim3(128, 1, 1);
    l.stream = (cudaStream_t)stream;
    l.pdl = true;
    return nvk::launch(l, combine_allreduce_kernel, a, x);
}

int nv_kernels_moe_permute(void* stream, const int32_t* topk_ids, int32_t* permuted_token_idx,
                           int32_t* expert_offsets, int32_t* inv_perm, int32_t* scratch_counts, int n_tokens, int k,
                           int num_experts) {
    if (n_tokens <= 0 || k <= 0 || num_experts <= 0) return 0;
    if (nvk::any_null(topk_ids, permuted_token_idx, expert_offsets, inv_perm, scratch_counts)) return NVK_ERR_ARG;
    return slot_sort(stream, topk_ids, permuted_token_idx, expert_offsets, inv_perm, scratch_counts, n_tokens, k,
                     num_experts);
}

// Router and slot sort in one launch for decode-sized steps (no counterpart in the reference, whose
// decode step launches them separately): the outputs of nv_kernels_moe_route_topk followed by
// nv_kernels_moe_permute, no scratch, plus -- when `active_experts` is given -- the ascending list of
// experts that received at least one slot ([min(E, n_tokens * K)] ints) and its length in `n_active`.
// Limits: E <= 256, K <= 32, n_tokens * K <= 4096 (else -3).
int nvk_b200_moe_route_permute(void* stream, const float* logits, const float* bias, int32_t* topk_ids,
                               float* topk_weights, int32_t* permuted_token_idx, int32_t* expert_offsets,
                               int32_t* inv_perm, int32_t* active_experts, int32_t* n_active, int n_tokens, int E, int K,
                               int mode, float softcap, int norm_topk, float routed_scaling) {
    if (n_tokens <= 0 || E <= 0 || K <= 0) return 0;
    if (K > E || K > kRouteMaxK) return NVK_ERR_ARG;
    if (E > kFusedMaxE || (long long)n_tokens * K > kFusedMaxSlots) return NVK_ERR_RESOURCE;
    if (nvk::any_null(logits, topk_ids, topk_weights, permuted_token_idx, expert_offsets, inv_perm)) return NVK_ERR_ARG;
    if ((active_experts == nullptr) != (n_active == nullptr)) return NVK_ERR_ARG;
    RouteSortArgs a;
    a.r = route_args(logits, bias, topk_ids, topk_weights, n_tokens, E, K, mode, softcap, norm_topk, routed_scaling, K, -1);
    a.perm_token = permuted_token_idx; a.offsets = expert_offsets; a.inv_perm = inv_perm;
    a.active = active_experts; a.n_active = n_active;
    const nvk::Launch l = nvk::launch_1d((cudaStream_t)stream, 1, 256, 0, true);
    if (E <= 32) return nvk::launch(l, route_sort_kernel<1>, a);
    if (E <= 64) return nvk::launch(l, route_sort_kernel<2>, a);
    if (E <= 128) return nvk::launch(l, route_sort_kernel<4>, a);
    return nvk::launch(l, route_sort_kernel<8>, a);
}

// ---- slot sort for callers that may not allocate device memory ------------------------------------
// Some hosts of this library cannot hand it a scratch buffer at the point of the call: a serving
// engine that claimed all of HBM for its KV-cache pool at start-up has nothing left to cudaMalloc
// from, a decode loop cannot afford the device-wide synchronisation an allocation implies, and an
// FFI host whose ownership rule is "the C side never allocates" has no allocator to lend.  For them
// the per-expert counters of the sort live in the fixed array below instead of in a caller-supplied
// buffer.  The array is part of the library image: every GPU that loads the library holds these
// 16 KiB until the process exits.
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
    // The array still holds whatever the previous call left in it; the kernel clears the counters it
    // uses before it counts.
    return slot_sort(stream, topk_ids, permuted_token_idx, expert_offsets, inv_perm, dev_ptr[dev], n_tokens, k,
                     num_experts);
}

// Writes the GPU's global nanosecond timer into *out when the stream reaches this point; usable
// inside a captured graph to time the kernels between two stamps.
int nv_kernels_prof_timestamp(void* stream, unsigned long long* out) {
    if (out == nullptr) return NVK_ERR_ARG;
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, 1, 1), timestamp_kernel, out);
}

}  // extern "C"
