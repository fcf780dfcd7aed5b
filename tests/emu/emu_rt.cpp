// Runtime of the host-side SIMT emulation (see cuda_emu.h): fibers, barriers, warp exchange,
// cp.async queues, clusters, guard-paged memory.  Test infrastructure only.
#include <pthread.h>
#include <signal.h>
#include <stdio.h>
#include <sys/mman.h>
#include <ucontext.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <mutex>
#include <thread>
#include <unordered_set>

#include "cuda_emu.h"

// Race checking (build_emu.py --tsan): the kernels are compiled with -fsanitize=thread and every
// emulated CUDA thread is a ThreadSanitizer fiber.  Switching fibers establishes NO ordering; the only
// happens-before edges are the ones CUDA gives -- block, warp and cluster barriers, launch boundaries --
// so two threads of a block that touch the same shared or global bytes without a barrier between them
// are reported, although the fibers here always run one after the other.  This file itself is compiled
// without instrumentation: the emulation's own bookkeeping is not part of the check.
#ifdef NVK_EMU_TSAN
extern "C" {
void* __tsan_get_current_fiber(void);
void* __tsan_create_fiber(unsigned flags);
void __tsan_destroy_fiber(void* fiber);
void __tsan_switch_to_fiber(void* fiber, unsigned flags);
void __tsan_acquire(void* addr);
void __tsan_release(void* addr);
}
#define TSAN_ACQUIRE(p) __tsan_acquire((void*)(p))
#define TSAN_RELEASE(p) __tsan_release((void*)(p))
#define TSAN_SWITCH(f) __tsan_switch_to_fiber((f), 1u /* no synchronisation */)
#else
#define TSAN_ACQUIRE(p) ((void)0)
#define TSAN_RELEASE(p) ((void)0)
#define TSAN_SWITCH(f) ((void)0)
#endif

namespace emu {

namespace {
constexpr size_t kPage = 4096;
constexpr size_t kStackBytes = 256 * 1024;
constexpr size_t kSmemMax = 232448;         // 227 KiB: the opt-in limit per block on sm_100
constexpr size_t kSmemDefault = 48 * 1024;  // without cudaFuncSetAttribute
constexpr uint32_t kSharedWindow = 0x01000000u;

struct Options {
    std::atomic<int> cp_async_early{0};
    std::atomic<int> sms{8};
    std::atomic<int> threads{0};
} g_opt;

struct Warp {
    uint32_t tab[2][32][8];
    int arrived = 0, alive = 0;
    unsigned gen = 0;
    char sync_w[2] = {0, 0};   // race-checker edges of the warp barrier, by generation parity
};
}  // namespace

struct Cluster {
    unsigned size = 1;
    Block* blocks[16] = {};
    pthread_barrier_t bar;
    char sync_all[2] = {0, 0};   // by barrier generation parity, like Block::sync_block
};

struct Copy {
    uint32_t dst;
    const void* src;
    int bytes, src_bytes;
    unsigned group;
};

struct Fiber {
    FiberPublic pub;
    ucontext_t ctx;
    bool done = false;
    std::vector<Copy> pending;
    unsigned groups = 0;
    void* tsan = nullptr;
};

struct Block {
    BlockPublic pub;
    int nthreads = 0;
    std::vector<Fiber> fibers;
    ucontext_t sched;
    int bar_arrived = 0, alive = 0;
    unsigned bar_gen = 0;
    int cbar_arrived = 0;
    unsigned cbar_gen = 0;
    std::vector<Warp> warps;
    Cluster* cluster = nullptr;
    unsigned long progress = 0;
    bool external_wait = false;
    const std::function<void()>* body = nullptr;
    void* tsan_sched = nullptr;
    // Addresses that the race checker's happens-before edges hang on.  A barrier uses two, by the parity
    // of its generation: a thread that has left barrier g and already arrived at barrier g + 1 must not
    // pass what it wrote in between to a thread that has yet to leave g.
    char sync_block[2] = {0, 0};
    char sync_start = 0, sync_end = 0;   // scheduler -> threads at block start, threads -> scheduler at its end
    char* sync_worker = nullptr;         // orders successive blocks on one arena (its shared memory, its stacks)
    // 32-byte sectors of global memory this block fetched with cp.async or streaming loads (see note_fetch)
    std::unordered_set<uintptr_t> fetched;
};

thread_local Block* g_block = nullptr;
thread_local Fiber* g_fiber = nullptr;

FiberPublic& fiber() { return g_fiber->pub; }
BlockPublic& block() { return g_block->pub; }

namespace {

[[noreturn]] void die(const char* what) {
    fprintf(stderr, "EMU: %s", what);
    if (g_block && g_fiber)
        fprintf(stderr, " (block %u,%u,%u thread %u)", g_block->pub.bidx.x, g_block->pub.bidx.y, g_block->pub.bidx.z,
                g_fiber->pub.tidx.x);
    fprintf(stderr, "\n");
    fflush(stderr);
    _exit(97);
}

// launch boundaries: what ran before a launch -> its threads (begin); its threads -> what comes next (end).
// Two addresses, so that the blocks of ONE launch are not ordered with each other through them.
char g_launch_begin = 0, g_launch_end = 0;

// weight-stream accounting (note_fetch below)
std::atomic<unsigned long long> g_fetch_sectors{0};
std::atomic<int> g_fetch_on{0};


inline void yield() {
    TSAN_SWITCH(g_block->tsan_sched);
    swapcontext(&g_fiber->ctx, &g_block->sched);
}

// ---- per-OS-thread resources: fiber stacks and the dynamic shared memory window ----------------
struct Arena {
    uint8_t* stacks = nullptr;   // 1024 x (guard page + stack)
    uint8_t* smem = nullptr;     // guard | kSmemMax (+ slack) | guard
    char sync = 0;               // orders the blocks that use this arena one after the other
    Arena() {
        const size_t per = kStackBytes + kPage;
        stacks = (uint8_t*)mmap(nullptr, 1024 * per, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE,
                                -1, 0);
        if (stacks == MAP_FAILED) die("mmap of fiber stacks failed");
        for (int i = 0; i < 1024; ++i) mprotect(stacks + i * per, kPage, PROT_NONE);
        const size_t body = (kSmemMax + kPage - 1) / kPage * kPage;
        smem = (uint8_t*)mmap(nullptr, body + 2 * kPage, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
        if (smem == MAP_FAILED) die("mmap of shared memory failed");
        mprotect(smem, kPage, PROT_NONE);
        mprotect(smem + kPage + body, kPage, PROT_NONE);
    }
    uint8_t* stack(int i) const { return stacks + (size_t)i * (kStackBytes + kPage) + kPage; }
    // the dynamic shared memory of a launch ends right at the trailing guard page
    uint8_t* smem_for(size_t bytes) const {
        const size_t body = (kSmemMax + kPage - 1) / kPage * kPage;
        const size_t rounded = (bytes + 127) / 128 * 128;
        return smem + kPage + body - rounded;
    }
};
std::mutex g_arena_mu;
std::vector<Arena*> g_arena_free;
Arena* arena_get() {
    std::lock_guard<std::mutex> l(g_arena_mu);
    if (!g_arena_free.empty()) {
        Arena* a = g_arena_free.back();
        g_arena_free.pop_back();
        return a;
    }
    return new Arena();
}
void arena_put(Arena* a) {
    std::lock_guard<std::mutex> l(g_arena_mu);
    g_arena_free.push_back(a);
}

void on_barrier_release(Block* b) { b->progress++; }

void fiber_exit_bookkeeping(Block* b, Fiber* f) {
    if (!f->pending.empty() && !g_opt.cp_async_early.load())
        die("a thread left the kernel with cp.async copies it never waited for");
    b->alive--;
    Warp& w = b->warps[f->pub.warp];
    w.alive--;
    if (w.arrived > 0 && w.arrived == w.alive) {
        w.arrived = 0;
        w.gen++;
        on_barrier_release(b);
    }
    if (b->bar_arrived > 0 && b->bar_arrived == b->alive) {
        b->bar_arrived = 0;
        b->bar_gen++;
        on_barrier_release(b);
    }
    if (b->cbar_arrived > 0 && b->cbar_arrived == b->alive) die("a thread exited while its block waits in cluster.sync()");
    b->progress++;
}

void trampoline(unsigned lo, unsigned hi) {
    Fiber* f = reinterpret_cast<Fiber*>(((uintptr_t)hi << 32) | (uintptr_t)lo);
    Block* b = g_block;
    // a thread starts knowing what preceded the launch and the block's set-up, and nothing that another
    // thread of the launch has done: threads only ever release to sync_end / g_launch_end
    TSAN_ACQUIRE(&g_launch_begin);
    TSAN_ACQUIRE(&b->sync_start);
    (*b->body)();
    TSAN_RELEASE(&b->sync_end);
    TSAN_RELEASE(&g_launch_end);
    f->done = true;
    fiber_exit_bookkeeping(b, f);
    TSAN_SWITCH(b->tsan_sched);
    swapcontext(&f->ctx, &b->sched);
    die("a finished fiber was resumed");
}

void run_block(Block& b, Arena* arena) {
    g_block = &b;
    b.sync_worker = &arena->sync;
    TSAN_ACQUIRE(b.sync_worker);   // the block that used this arena's shared memory before us is over
    b.pub.dyn_smem = arena->smem_for(b.pub.dyn_bytes);
    const unsigned n = (unsigned)b.nthreads;
    b.fibers.clear();
    b.fibers.resize(n);
    b.warps.assign((n + 31) / 32, Warp());
    b.alive = (int)n;
    b.bar_arrived = b.cbar_arrived = 0;
    for (unsigned t = 0; t < n; ++t) {
        Fiber& f = b.fibers[t];
        f.pub.tidx.x = t % b.pub.bdim.x;
        f.pub.tidx.y = (t / b.pub.bdim.x) % b.pub.bdim.y;
        f.pub.tidx.z = t / (b.pub.bdim.x * b.pub.bdim.y);
        f.pub.lane = (int)(t & 31);
        f.pub.warp = (int)(t >> 5);
        b.warps[t >> 5].alive++;
#ifdef NVK_EMU_TSAN
        f.tsan = __tsan_create_fiber(0);
#endif
        getcontext(&f.ctx);
        f.ctx.uc_stack.ss_sp = arena->stack((int)t);
        f.ctx.uc_stack.ss_size = kStackBytes;
        f.ctx.uc_link = &b.sched;
        const uintptr_t p = reinterpret_cast<uintptr_t>(&f);
        makecontext(&f.ctx, (void (*)())trampoline, 2, (unsigned)(p & 0xFFFFFFFFu), (unsigned)(p >> 32));
    }
#ifdef NVK_EMU_TSAN
    b.tsan_sched = __tsan_get_current_fiber();
#endif
    TSAN_RELEASE(&b.sync_start);
    unsigned remaining = n;
    unsigned idle_passes = 0;
    while (remaining) {
        const unsigned long before = b.progress;
        b.external_wait = false;
        for (unsigned t = 0; t < n; ++t) {
            Fiber& f = b.fibers[t];
            if (f.done) continue;
            g_fiber = &f;
            TSAN_SWITCH(f.tsan);
            swapcontext(&b.sched, &f.ctx);
            if (f.done) --remaining;
        }
        if (b.progress == before && !b.external_wait) {
            if (++idle_passes > 2) die("deadlock: every thread of the block waits at a barrier that cannot complete");
        } else {
            idle_passes = 0;
        }
    }
    if (!b.fetched.empty()) {
        g_fetch_sectors.fetch_add(b.fetched.size(), std::memory_order_relaxed);
        b.fetched.clear();
    }
    TSAN_ACQUIRE(&b.sync_end);     // the threads are done: the worker may reuse or free what they used
    TSAN_RELEASE(b.sync_worker);
#ifdef NVK_EMU_TSAN
    for (unsigned t = 0; t < n; ++t) __tsan_destroy_fiber(b.fibers[t].tsan);
#endif
    g_fiber = nullptr;
    g_block = nullptr;
}

std::mutex g_attr_mu;
std::map<const void*, size_t> g_func_smem;

}  // namespace

// ---- barriers ----------------------------------------------------------------------------------
void syncthreads() {
    Block* b = g_block;
    const unsigned gen = b->bar_gen;
    char* const edge = &b->sync_block[gen & 1u];
    TSAN_RELEASE(edge);
    if (++b->bar_arrived == b->alive) {
        b->bar_arrived = 0;
        b->bar_gen++;
        on_barrier_release(b);
        TSAN_ACQUIRE(edge);
        return;
    }
    while (b->bar_gen == gen) yield();
    TSAN_ACQUIRE(edge);
}

void syncwarp() {
    Block* b = g_block;
    Warp& w = b->warps[g_fiber->pub.warp];
    const unsigned gen = w.gen;
    char* const edge = &w.sync_w[gen & 1u];
    TSAN_RELEASE(edge);
    if (++w.arrived == w.alive) {
        w.arrived = 0;
        w.gen++;
        on_barrier_release(b);
        TSAN_ACQUIRE(edge);
        return;
    }
    while (w.gen == gen) yield();
    TSAN_ACQUIRE(edge);
}

const uint32_t (*warp_publish(const uint32_t* words, int n_words))[8] {
    Block* b = g_block;
    Warp& w = b->warps[g_fiber->pub.warp];
    const unsigned p = w.gen & 1u;   // the same for every lane: gen moves only when the last lane arrives
    uint32_t* mine = w.tab[p][g_fiber->pub.lane];
    for (int i = 0; i < 8; ++i) mine[i] = i < n_words ? words[i] : 0u;
    syncwarp();
    return w.tab[p];
}

void cluster_sync() {
    Block* b = g_block;
    if (b->cluster == nullptr || b->cluster->size <= 1) {
        syncthreads();
        return;
    }
    const unsigned gen = b->cbar_gen;
    char* const edge = &b->cluster->sync_all[gen & 1u];
    TSAN_RELEASE(edge);
    if (++b->cbar_arrived == b->alive) {
        pthread_barrier_wait(&b->cluster->bar);   // every fiber of this block is parked: block the OS thread
        b->cbar_arrived = 0;
        b->cbar_gen++;
        on_barrier_release(b);
        TSAN_ACQUIRE(edge);
        return;
    }
    while (b->cbar_gen == gen) yield();
    TSAN_ACQUIRE(edge);
}

void* cluster_map(void* p, unsigned rank) {
    Block* b = g_block;
    uint8_t* q = static_cast<uint8_t*>(p);
    if (q < b->pub.dyn_smem || q >= b->pub.dyn_smem + b->pub.dyn_bytes)
        die("map_shared_rank: only dynamic shared memory can be mapped in the emulation");
    if (b->cluster == nullptr) {
        if (rank != 0) die("map_shared_rank: rank outside the cluster");
        return p;
    }
    if (rank >= b->cluster->size) die("map_shared_rank: rank outside the cluster");
    return b->cluster->blocks[rank]->pub.dyn_smem + (q - b->pub.dyn_smem);
}

void spin_yield() {
    g_block->external_wait = true;
    yield();
    if (g_block->cluster == nullptr && g_block->alive == 1) sched_yield();
}

// ---- cp.async ------------------------------------------------------------------------------------
uint32_t shared_addr(const void* p) {
    Block* b = g_block;
    const uint8_t* q = static_cast<const uint8_t*>(p);
    if (q < b->pub.dyn_smem || q > b->pub.dyn_smem + b->pub.dyn_bytes)
        die("__cvta_generic_to_shared: pointer is not in dynamic shared memory");
    return kSharedWindow + (uint32_t)(q - b->pub.dyn_smem);
}

void* shared_ptr(uint32_t a, size_t bytes) {
    Block* b = g_block;
    if (a < kSharedWindow || (size_t)(a - kSharedWindow) + bytes > b->pub.dyn_bytes) {
        fprintf(stderr, "EMU: shared-memory access [%u, +%zu) outside the launch's %zu bytes\n", a - kSharedWindow, bytes,
                b->pub.dyn_bytes);
        die("shared window overrun");
    }
    return b->pub.dyn_smem + (a - kSharedWindow);
}

static void do_copy(const Copy& c) {
    uint8_t* d = static_cast<uint8_t*>(shared_ptr(c.dst, (size_t)c.bytes));
    if (c.src_bytes > 0) memcpy(d, c.src, (size_t)c.src_bytes);
    if (c.src_bytes < c.bytes) memset(d + c.src_bytes, 0, (size_t)(c.bytes - c.src_bytes));
}

// Weight-stream accounting: every global address range a block fetches with cp.async or a streaming load
// is recorded as 32-byte sectors, once per block (a second fetch of a sector by the same block is what a
// warp's coalescer or L1 would absorb); the sum over the blocks of a launch is the traffic its SMs ask
// of L2 for those streams.  Equal to the algorithmic bytes when every byte is fetched by exactly one block.

void note_fetch(const void* src, int bytes) {
    if (!g_fetch_on.load(std::memory_order_relaxed) || bytes <= 0 || g_block == nullptr) return;
    const uintptr_t a0 = (uintptr_t)src >> 5, a1 = ((uintptr_t)src + (uintptr_t)bytes - 1) >> 5;
    for (uintptr_t a = a0; a <= a1; ++a) g_block->fetched.insert(a);
}

void cp_async(uint32_t dst, const void* src, int bytes, int src_bytes) {
    note_fetch(src, src_bytes);
    if (src_bytes < 0 || src_bytes > bytes) die("cp.async: src-size larger than the copy");
    if ((dst & (uint32_t)(bytes - 1)) != 0) die("cp.async: misaligned shared destination");
    if (src_bytes > 0 && ((uintptr_t)src & (uintptr_t)(bytes - 1)) != 0) die("cp.async: misaligned global source");
    (void)shared_ptr(dst, (size_t)bytes);
    Copy c{dst, src, bytes, src_bytes, g_fiber->groups};
    if (g_opt.cp_async_early.load())
        do_copy(c);
    else
        g_fiber->pending.push_back(c);
}

void cp_async_commit() { g_fiber->groups++; }

void cp_async_wait(int allowed_pending) {
    Fiber* f = g_fiber;
    // groups [0, groups - allowed) are complete after this; later ones may still be in flight
    const long done_below = (long)f->groups - allowed_pending;
    size_t keep = 0;
    for (size_t i = 0; i < f->pending.size(); ++i) {
        if ((long)f->pending[i].group < done_below)
            do_copy(f->pending[i]);
        else
            f->pending[keep++] = f->pending[i];
    }
    f->pending.resize(keep);
}

// ---- launches ------------------------------------------------------------------------------------
int func_set_max_dyn_smem(const void* func, int bytes) {
    if (bytes < 0 || (size_t)bytes > kSmemMax) return cudaErrorInvalidValue;
    std::lock_guard<std::mutex> l(g_attr_mu);
    size_t& cur = g_func_smem[func];
    cur = (size_t)bytes;
    return 0;
}

int sm_count() { return g_opt.sms.load(); }

int run_grid(const LaunchCfg& c, const void* func, const std::function<void()>& body) {
    const unsigned long nthreads = (unsigned long)c.block.x * c.block.y * c.block.z;
    if (nthreads == 0 || nthreads > 1024 || c.block.z > 64) return cudaErrorInvalidConfiguration;
    if (c.grid.x == 0 || c.grid.y == 0 || c.grid.z == 0 || c.grid.y > 65535 || c.grid.z > 65535 ||
        c.grid.x > 0x7FFFFFFFu)
        return cudaErrorInvalidConfiguration;
    size_t limit = kSmemDefault;
    {
        std::lock_guard<std::mutex> l(g_attr_mu);
        auto it = g_func_smem.find(func);
        if (it != g_func_smem.end() && it->second > limit) limit = it->second;
    }
    if (c.smem > limit) return cudaErrorInvalidValue;   // the opt-in was not raised for this kernel
    const unsigned cs = c.cluster_x ? c.cluster_x : 1;
    if (cs > 8 || (c.grid.x % cs) != 0) return cudaErrorInvalidConfiguration;
    const unsigned long nblocks = (unsigned long)c.grid.x * c.grid.y * c.grid.z;
    if (c.cooperative && nblocks > 64) return cudaErrorInvalidConfiguration;   // keep co-resident grids small here

    auto init_block = [&](Block& b, unsigned long linear) {
        b.pub.bidx.x = (unsigned)(linear % c.grid.x);
        b.pub.bidx.y = (unsigned)((linear / c.grid.x) % c.grid.y);
        b.pub.bidx.z = (unsigned)(linear / ((unsigned long)c.grid.x * c.grid.y));
        b.pub.bdim = c.block;
        b.pub.gdim = c.grid;
        b.pub.dyn_bytes = c.smem;
        b.pub.cluster_rank = 0;
        b.pub.cluster_size = 1;
        b.nthreads = (int)nthreads;
        b.body = &body;
    };

    int hw = g_opt.threads.load();
    if (hw <= 0) hw = (int)std::thread::hardware_concurrency();
    if (hw <= 0) hw = 4;
    TSAN_RELEASE(&g_launch_begin);   // stream order: what ran before this launch is visible to its threads
    struct AfterLaunch {
        ~AfterLaunch() {   // ... and what they did, to whatever comes next (the next launch included)
            TSAN_ACQUIRE(&g_launch_end);
        }
    } after_launch;

    if (c.cooperative) {
        // every block resident at once, as a cooperative launch guarantees
        std::vector<Block> blocks(nblocks);
        std::vector<std::thread> th;
        for (unsigned long i = 0; i < nblocks; ++i) init_block(blocks[i], i);
        for (unsigned long i = 0; i < nblocks; ++i)
            th.emplace_back([&, i] {
                Arena* a = arena_get();
                run_block(blocks[i], a);
                arena_put(a);
            });
        for (auto& t : th) t.join();
        return 0;
    }

    if (cs == 1) {
        std::atomic<unsigned long> next{0};
        const int workers = (int)std::min<unsigned long>((unsigned long)hw, nblocks);
        auto work = [&] {
            Arena* a = arena_get();
            Block b;
            for (;;) {
                const unsigned long i = next.fetch_add(1);
                if (i >= nblocks) break;
                init_block(b, i);
                run_block(b, a);
            }
            arena_put(a);
        };
        if (workers <= 1) {
            work();
        } else {
            std::vector<std::thread> th;
            for (int w = 0; w < workers; ++w) th.emplace_back(work);
            for (auto& t : th) t.join();
        }
        return 0;
    }

    // clusters: the blocks of one cluster run together, each on its own OS thread
    const unsigned long nclusters = nblocks / cs;
    std::atomic<unsigned long> next{0};
    const int groups = (int)std::min<unsigned long>((unsigned long)std::max(1, hw / (int)cs), nclusters);
    auto run_clusters = [&] {
        for (;;) {
            const unsigned long ci = next.fetch_add(1);
            if (ci >= nclusters) break;
            // x is the fastest grid axis and the cluster spans x, so a cluster's blocks are consecutive
            Cluster cl;
            cl.size = cs;
            pthread_barrier_init(&cl.bar, nullptr, cs);
            std::vector<Block> blocks(cs);
            for (unsigned r = 0; r < cs; ++r) {
                init_block(blocks[r], ci * cs + r);
                blocks[r].cluster = &cl;
                blocks[r].pub.cluster_rank = r;
                blocks[r].pub.cluster_size = cs;
                cl.blocks[r] = &blocks[r];
            }
            // shared-memory windows must exist before any block maps a peer's
            std::vector<Arena*> arenas(cs);
            for (unsigned r = 0; r < cs; ++r) {
                arenas[r] = arena_get();
                blocks[r].pub.dyn_smem = arenas[r]->smem_for(c.smem);
            }
            std::vector<std::thread> th;
            for (unsigned r = 0; r < cs; ++r) th.emplace_back([&, r] { run_block(blocks[r], arenas[r]); });
            for (auto& t : th) t.join();
            for (unsigned r = 0; r < cs; ++r) arena_put(arenas[r]);
            pthread_barrier_destroy(&cl.bar);
        }
    };
    std::vector<std::thread> th;
    for (int g = 0; g < groups; ++g) th.emplace_back(run_clusters);
    for (auto& t : th) t.join();
    return 0;
}

// ---- guard-paged "device" memory -------------------------------------------------------------------
namespace {
struct Alloc {
    uint8_t* map;
    size_t map_bytes, bytes;
};
std::mutex g_alloc_mu;
std::map<uintptr_t, Alloc> g_allocs;   // user pointer -> mapping

void* guarded_alloc(size_t bytes, int front) {
    const size_t body = (std::max<size_t>(bytes, 1) + kPage - 1) / kPage * kPage;
    uint8_t* m = (uint8_t*)mmap(nullptr, body + 2 * kPage, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    if (m == MAP_FAILED) return nullptr;
    mprotect(m, kPage, PROT_NONE);
    mprotect(m + kPage + body, kPage, PROT_NONE);
    // front: the buffer starts right after the leading guard page (catches reads before it);
    // otherwise it ends right at the trailing guard page, up to the 256-byte alignment cudaMalloc gives
    uint8_t* p = front ? m + kPage : m + kPage + body - (bytes + 255) / 256 * 256;
    if (!front && bytes == 0) p = m + kPage;
    memset(m + kPage, 0xA5, body);   // stale garbage, not zeros
    std::lock_guard<std::mutex> l(g_alloc_mu);
    g_allocs[(uintptr_t)p] = Alloc{m, body + 2 * kPage, bytes};
    return p;
}

void segv_handler(int, siginfo_t* si, void*) {
    const uintptr_t a = (uintptr_t)si->si_addr;
    char buf[256];
    int n = snprintf(buf, sizeof buf, "EMU: memory fault at %p", si->si_addr);
    // async-signal-safety is moot: the process ends here
    for (auto& kv : g_allocs) {
        const uintptr_t lo = (uintptr_t)kv.second.map, hi = lo + kv.second.map_bytes;
        if (a >= lo && a < hi) {
            n += snprintf(buf + n, sizeof buf - n, " -- %ld bytes past the start of a %zu-byte buffer",
                          (long)(a - kv.first), kv.second.bytes);
            break;
        }
    }
    n += snprintf(buf + n, sizeof buf - n, " (out-of-bounds access in an emulated kernel)\n");
    (void)!write(2, buf, (size_t)n);
    _exit(98);
}
}  // namespace

}  // namespace emu

cudaError_t cudaMalloc(void** p, size_t n) {
    *p = emu::guarded_alloc(n, 0);
    return *p ? cudaSuccess : cudaErrorMemoryAllocation;
}

cudaError_t cudaFree(void* p) {
    if (!p) return cudaSuccess;
    std::lock_guard<std::mutex> l(emu::g_alloc_mu);
    auto it = emu::g_allocs.find((uintptr_t)p);
    if (it == emu::g_allocs.end()) return cudaErrorInvalidValue;
    munmap(it->second.map, it->second.map_bytes);
    emu::g_allocs.erase(it);
    return cudaSuccess;
}

extern "C" {

// Buffers for the tests: `front` != 0 puts the leading guard page right before the buffer, else the
// trailing guard page right after it (rounded up to 256 bytes, the alignment a device allocation has).
void* emu_alloc(size_t bytes, int front) { return emu::guarded_alloc(bytes, front); }
void emu_free(void* p) { (void)cudaFree(p); }

// Options: "cp_async_early" (0: copies land at the matching wait_group, the latest the ISA allows;
// 1: at once), "sms" (what cudaDevAttrMultiProcessorCount reports), "threads" (host threads per launch).
// Start (on != 0: counter to zero) or stop the weight-stream accounting; read the sectors counted so far.
void emu_fetch_accounting(int on) {
    if (on) emu::g_fetch_sectors.store(0);
    emu::g_fetch_on.store(on ? 1 : 0);
}
unsigned long long emu_fetched_bytes(void) { return emu::g_fetch_sectors.load() * 32ull; }

int emu_set_option(const char* name, int value) {
    if (!strcmp(name, "cp_async_early")) emu::g_opt.cp_async_early = value;
    else if (!strcmp(name, "sms")) emu::g_opt.sms = value;
    else if (!strcmp(name, "threads")) emu::g_opt.threads = value;
    else return -1;
    return 0;
}

void emu_install_fault_handler(void) {
    // the handler needs its own stack: a fault on a fiber's guard page leaves none to run on
    static uint8_t alt[64 * 1024];
    stack_t ss;
    ss.ss_sp = alt;
    ss.ss_size = sizeof alt;
    ss.ss_flags = 0;
    sigaltstack(&ss, nullptr);
    struct sigaction sa;
    memset(&sa, 0, sizeof sa);
    sa.sa_sigaction = emu::segv_handler;
    sa.sa_flags = SA_SIGINFO | SA_ONSTACK;
    sigaction(SIGSEGV, &sa, nullptr);
    sigaction(SIGBUS, &sa, nullptr);
}

}  // extern "C"
