// A whole decode step's NVFP4 W4A16 linears in ONE persistent launch.
//
// A batch-1 GEMV launched on its own spends more time in the hand-over between kernels (release of
// the previous grid, first touch of the activations, the split-K sum) than in moving its 10-60 MB
// of weights.  Here the linears of a step are a list of operations in device memory and one
// cooperative kernel walks the list:
//
//   * every CTA takes work items (a 128-row or 16-row slab of one operation's matrix over all of K)
//     from a per-operation counter, so the SMs stay evenly loaded whatever the shapes;
//   * an operation whose activations are another operation's outputs waits for that operation's
//     arrival counter, not for a grid-wide barrier -- and the tile code fills its weight ring BEFORE
//     that wait, so the weight stream does not stop between dependent linears;
//   * the per-tile arithmetic is w4a16_tile (w4a16_tile.cuh), unchanged: an item computes exactly
//     what the stand-alone launch with the same rows-per-CTA and no K split computes, bit for bit.
//
// Every wait is bounded: after the wait limit (nvk_b200_set_wait_limit) the CTA records an error and goes on (its
// results are then meaningless, the launch still ends).  The launch is cooperative, so all CTAs are
// resident together and a CTA never waits for one that is not running.
#include <map>

#include "w4a16_tile.cuh"

namespace {

constexpr int kStackThreads = 256;
constexpr int kMaxOps = 1024;

// One linear of the step, as the kernel reads it.
struct StackOp {
    const uint8_t* wq[2];
    const uint8_t* sc[2];
    const uint16_t* x;     // [M, K] bf16 (gate when x2 != null)
    const uint16_t* x2;    // up: the activation is bf16(SiLU(x) * x2)
    uint16_t* y[2];        // [M, N] bf16 per arm
    float alpha[2];
    int N, K;
    int dep;               // operation that writes x (and x2), or -1
    int ug;                // 16-row units per item: 8 (one 128-row scale tile) or 1 (16 rows, 8 warps along K)
    int items;             // arms * ceil(N / 128) * (8 / ug)
    int tiles_per_arm;     // items per arm
    int k_tiles, nsc, ph, x_stride, ring_off;
};

// Tiles inside the persistent launch: no cluster (an item owns all of K for its rows), activations
// written earlier in the SAME launch -- so they are read from L2 (another SM wrote them; this SM's L1
// may hold a stale line from an earlier operation) after the producer's arrival counter says so.
struct StackHooks {
    __device__ static __forceinline__ int crank() { return 0; }
    __device__ static __forceinline__ int nranks() { return 1; }
    __device__ static __forceinline__ void before_activations(const TileView& t) {
        if (t.gate == nullptr) return;   // uniform over the CTA
        if (threadIdx.x == 0 && !nvk::bounded_wait_ge(t.gate, t.gate_target, t.gate_limit)) atomicExch(t.gate_err, 1);
        __syncthreads();
    }
    __device__ static __forceinline__ uint4 load_x(const uint16_t* q) {
        return __ldcg(reinterpret_cast<const uint4*>(q));
    }
};

template <int UG, int KW>
__device__ __forceinline__ void run_item(const StackOp& op, int item, int M, const unsigned* done, const StackOp* ops,
                                         int* err, unsigned wait_limit) {
    GemmParams p = {};
    p.wq[0] = op.wq[0]; p.wq[1] = op.wq[1];
    p.sc[0] = op.sc[0]; p.sc[1] = op.sc[1];
    p.x = op.x; p.x2 = op.x2;
    p.y[0] = op.y[0]; p.y[1] = op.y[1];
    p.alpha[0] = op.alpha[0]; p.alpha[1] = op.alpha[1];
    p.M = M; p.N = op.N; p.K = op.K;
    p.tiles_per_arm = op.tiles_per_arm;
    p.k_tiles = op.k_tiles;
    p.nsc = op.nsc;
    p.spc = op.nsc;          // the item's K slice is all of K
    p.ph = op.ph;
    p.x_stride = op.x_stride;
    p.ring_off = op.ring_off;
    const int arm = item >= op.tiles_per_arm ? 1 : 0;
    TileView t = {};
    t.wq = op.wq[arm];
    t.sc = op.sc[arm];
    t.x = op.x;
    t.x2 = op.x2;
    t.xrows = nullptr;
    t.x_rows = 0;
    t.status = nullptr;
    t.y = op.y[arm];
    t.alpha = op.alpha[arm];
    t.xrow0 = 0;
    t.M = M;
    t.sub = item - arm * op.tiles_per_arm;
    t.pdl = false;
    t.ws = nullptr;
    t.gate = op.dep >= 0 ? done + op.dep : nullptr;
    t.gate_target = op.dep >= 0 ? (unsigned)ops[op.dep].items : 0u;
    t.gate_err = err;
    t.gate_limit = wait_limit;
    if (op.x2 != nullptr)
        w4a16_tile<1, 1, UG, KW, false, StackHooks>(p, t);
    else
        w4a16_tile<1, 0, UG, KW, false, StackHooks>(p, t);
}

// next_item[o]: the next unclaimed item of operation o; done[o]: items of operation o completed.
// Both start at zero (the launcher clears them on the stream before every launch).
__global__ void __launch_bounds__(kStackThreads, 2) w4a16_stack_kernel(const StackOp* __restrict__ ops, int n_ops, int M,
                                                                       unsigned* next_item, unsigned* done, int* err,
                                                                       unsigned wait_limit) {
    __shared__ int s_item;
    for (int o = 0; o < n_ops; ++o) {
        const StackOp op = ops[o];
        for (;;) {
            __syncthreads();   // the previous item's shared-memory reads are over
            if (threadIdx.x == 0) s_item = (int)atomicAdd(next_item + o, 1u);
            __syncthreads();
            const int item = s_item;
            if (item >= op.items) break;
            if (op.ug == 8)
                run_item<8, 1>(op, item, M, done, ops, err, wait_limit);
            else
                run_item<1, 8>(op, item, M, done, ops, err, wait_limit);
            __syncthreads();   // every thread's outputs of this item are written ...
            if (threadIdx.x == 0) {
                __threadfence();            // ... and visible device-wide before the arrival is counted
                atomicAdd(done + o, 1u);
            }
        }
    }
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

// What nvk_b200_stack_build laid a plan out for.  nvk_b200_stack_run checks its arguments against
// this record: a step run with more tokens than the plan's shared-memory layout was sized for, or
// with another operation count, would compute garbage without any error.
struct PlanRecord {
    int n_ops, M, grid, smem;
};
std::mutex g_plans_mu;
std::map<const void*, PlanRecord> g_plans;

size_t plan_bytes(int n_ops) {
    // [StackOp x n_ops | next_item x n_ops | done x n_ops], each part 256-byte aligned
    const size_t ops_b = ((size_t)n_ops * sizeof(StackOp) + 255) / 256 * 256;
    const size_t ctr_b = ((size_t)n_ops * sizeof(unsigned) + 255) / 256 * 256;
    return ops_b + 2 * ctr_b;
}

}  // namespace

extern "C" {

// Public description of one linear: the same members, in the same order, as NvkStackOp in the C
// header of this library.
struct NvkStackOp {
    const uint8_t* wq_a;
    const uint8_t* sc_a;
    const uint8_t* wq_b;
    const uint8_t* sc_b;
    const uint16_t* x;
    const uint16_t* x2;
    uint16_t* y_a;
    uint16_t* y_b;
    float alpha_a, alpha_b;
    int N, K;
    int dep;
    int rows_per_item;   // 0 = chosen here; 128 or 16
};
static_assert(sizeof(NvkStackOp) == 8 * sizeof(void*) + 2 * sizeof(float) + 4 * sizeof(int), "NvkStackOp layout");

size_t nvk_b200_stack_plan_bytes(int n_ops) {
    if (n_ops <= 0 || n_ops > kMaxOps) return 0;
    return plan_bytes(n_ops);
}

// Set-up call (copies to the device and synchronises; not for the decode loop): checks the
// operations, lays out each one's shared memory, writes the plan into `plan_dev` and returns the
// launch shape in launch_out[0] (CTAs) and launch_out[1] (dynamic shared memory bytes).
int nvk_b200_stack_build(const NvkStackOp* ops, int n_ops, int M, void* plan_dev, size_t plan_dev_bytes,
                         int* launch_out) {
    if (ops == nullptr || plan_dev == nullptr || launch_out == nullptr) return NVK_ERR_ARG;
    if (n_ops <= 0 || n_ops > kMaxOps) return NVK_ERR_RESOURCE;
    if (M <= 0 || M > 8) return NVK_ERR_SHAPE;
    if (plan_dev_bytes < plan_bytes(n_ops) || !aligned16(plan_dev)) return NVK_ERR_ARG;
    StackOp* host = static_cast<StackOp*>(malloc((size_t)n_ops * sizeof(StackOp)));
    if (host == nullptr) return NVK_ERR_RESOURCE;
    size_t smem_max = 0;
    int rc = 0;
    for (int i = 0; i < n_ops && rc == 0; ++i) {
        const NvkStackOp& s = ops[i];
        const bool dual = s.wq_b != nullptr;
        if (s.N <= 0 || s.K <= 0 || (s.K & 31) != 0) rc = NVK_ERR_SHAPE;
        else if ((s.wq_b == nullptr) != (s.sc_b == nullptr) || (s.wq_b == nullptr) != (s.y_b == nullptr)) rc = NVK_ERR_SHAPE;
        else if (s.dep >= i || s.dep < -1) rc = NVK_ERR_ARG;   // only earlier operations can be waited for
        else if (nvk::any_null(s.wq_a, s.sc_a, s.x, s.y_a)) rc = NVK_ERR_ARG;
        else if (!aligned16(s.wq_a) || !aligned16(s.sc_a) || !aligned16(s.x) || (s.x2 && !aligned16(s.x2)) ||
                 (dual && (!aligned16(s.wq_b) || !aligned16(s.sc_b))))
            rc = NVK_ERR_ARG;
        else if (s.rows_per_item != 0 && s.rows_per_item != 16 && s.rows_per_item != 128) rc = NVK_ERR_ARG;
        if (rc) break;
        StackOp& d = host[i];
        d = StackOp{};
        d.wq[0] = s.wq_a; d.wq[1] = s.wq_b;
        d.sc[0] = s.sc_a; d.sc[1] = s.sc_b;
        d.x = s.x; d.x2 = s.x2;
        d.y[0] = s.y_a; d.y[1] = s.y_b;
        d.alpha[0] = s.alpha_a; d.alpha[1] = s.alpha_b;
        d.N = s.N; d.K = s.K; d.dep = s.dep;
        const int arms = dual ? 2 : 1;
        const int row_tiles = nvk::ceil_div(s.N, kRowsPerCta);
        // 128-row items when they alone give every SM work, else 16-row items (8 warps along K)
        d.ug = s.rows_per_item == 128 ? 8 : s.rows_per_item == 16 ? 1 : (arms * row_tiles >= 148 ? 8 : 1);
        const int kw = d.ug == 8 ? 1 : 8;
        d.tiles_per_arm = row_tiles * (8 / d.ug);
        d.items = arms * d.tiles_per_arm;
        d.k_tiles = nvk::ceil_div(s.K, 64);
        d.nsc = nvk::ceil_div(s.K, kSuper);
        // the same shared-memory layout rule as the stand-alone launch
        int ph_cap = (48 * 1024) / (M * 512);
        ph_cap = ph_cap / kw * kw;
        if (ph_cap < kw) ph_cap = kw;
        const int spc_up = nvk::ceil_div(d.nsc, kw) * kw;
        d.ph = ph_cap < spc_up ? ph_cap : spc_up;
        d.x_stride = d.ph * 512 + 64;
        const size_t smem_x = (size_t)M * d.x_stride;
        const size_t smem_red = (size_t)(kw + 1) * 8 * (16 * d.ug + 4) * sizeof(float);
        const size_t lo = smem_x > smem_red ? smem_x : smem_red;
        d.ring_off = (int)((lo + 127) / 128 * 128);
        const size_t smem = (size_t)d.ring_off + (size_t)8 * kDepth * kSlotBytes;
        if (smem > smem_max) smem_max = smem;
    }
    if (rc == 0) {
        static nvk::SmemOptin optin;
        rc = optin.ensure((const void*)w4a16_stack_kernel, smem_max);
    }
    int per_sm = 0, sms = 0, dev = 0;
    if (rc == 0) {
        cudaError_t e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess)
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, w4a16_stack_kernel, kStackThreads, smem_max);
        if (e != cudaSuccess) rc = (int)e;
        else if (per_sm < 1 || sms < 1) rc = NVK_ERR_RESOURCE;
    }
    if (rc == 0) {
        cudaError_t e = cudaMemset(plan_dev, 0, plan_bytes(n_ops));
        if (e == cudaSuccess) e = cudaMemcpy(plan_dev, host, (size_t)n_ops * sizeof(StackOp), cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        if (e != cudaSuccess) rc = (int)e;
    }
    free(host);
    if (rc == 0) {
        launch_out[0] = (per_sm > 2 ? 2 : per_sm) * sms;   // all of them resident together
        launch_out[1] = (int)smem_max;
        std::lock_guard<std::mutex> lock(g_plans_mu);
        g_plans[plan_dev] = PlanRecord{n_ops, M, launch_out[0], launch_out[1]};
    }
    return rc;
}

// Enqueue one step: clears the plan's counters on the stream, then launches the cooperative kernel
// with the shape nvk_b200_stack_build returned.  `err` (device int, owned by the caller, zeroed by
// the caller) is set to 1 if a wait inside the kernel gave up.  Allocates nothing, never synchronises.
int nvk_b200_stack_run(void* stream, void* plan_dev, int n_ops, int M, int grid, int smem_bytes, int* err) {
    if (plan_dev == nullptr || err == nullptr) return NVK_ERR_ARG;
    if (n_ops <= 0 || n_ops > kMaxOps || M <= 0 || M > 8 || grid <= 0 || smem_bytes <= 0) return NVK_ERR_ARG;
    {
        // the plan must be one this process built, run with the shape it was built for (a smaller
        // grid is allowed: the work items are drawn from counters)
        std::lock_guard<std::mutex> lock(g_plans_mu);
        auto it = g_plans.find(plan_dev);
        if (it == g_plans.end()) return NVK_ERR_ARG;
        const PlanRecord& r = it->second;
        if (n_ops != r.n_ops || M != r.M || smem_bytes != r.smem || grid > r.grid) return NVK_ERR_ARG;
    }
    cudaStream_t s = (cudaStream_t)stream;
    uint8_t* base = static_cast<uint8_t*>(plan_dev);
    const size_t ops_b = ((size_t)n_ops * sizeof(StackOp) + 255) / 256 * 256;
    const size_t ctr_b = ((size_t)n_ops * sizeof(unsigned) + 255) / 256 * 256;
    unsigned* next_item = reinterpret_cast<unsigned*>(base + ops_b);
    unsigned* done = reinterpret_cast<unsigned*>(base + ops_b + ctr_b);
    cudaError_t e = cudaMemsetAsync(next_item, 0, 2 * ctr_b, s);
    if (e != cudaSuccess) return (int)e;
    nvk::Launch l = nvk::launch_1d(s, (unsigned)grid, kStackThreads, (size_t)smem_bytes);
    l.cooperative = true;
    const StackOp* ops = reinterpret_cast<const StackOp*>(base);
    return nvk::launch(l, w4a16_stack_kernel, ops, n_ops, M, next_item, done, err, nvk::wait_limit_setting());
}

}  // extern "C"
