// One way to launch a kernel: grid, block, dynamic shared memory, stream, and the optional launch
// attributes this library uses (thread-block cluster along x, programmatic dependent launch,
// cooperative launch).  Returns 0 or the cudaError_t of the launch; never synchronises.
#pragma once
#include "nvk_ptx.cuh"

namespace nvk {

struct Launch {
    dim3 grid = dim3(1, 1, 1), block = dim3(1, 1, 1);
    size_t smem = 0;
    cudaStream_t stream = nullptr;
    unsigned cluster_x = 1;    // > 1: clusters of that many CTAs along grid x
    bool pdl = false;          // the kernel calls ptx::pdl_wait() before touching its predecessor's output
    bool cooperative = false;  // all CTAs resident together
};

// Programmatic dependent launch for the calling thread's launches (nvk_b200_set_pdl): when 0, a launch
// that asks for it is an ordinary stream-ordered launch (the kernels' waits are then no-ops).
inline thread_local int g_pdl_enabled = 1;

inline Launch launch_1d(cudaStream_t stream, unsigned grid, unsigned block, size_t smem = 0, bool pdl = false) {
    Launch l;
    l.grid = dim3(grid, 1, 1);
    l.block = dim3(block, 1, 1);
    l.smem = smem;
    l.stream = stream;
    l.pdl = pdl;
    return l;
}

template <class... P, class... A>
inline int launch(const Launch& l, void (*kernel)(P...), A&&... args) {
#ifdef NVK_EMU
    emu::LaunchCfg c;
    c.grid = l.grid;
    c.block = l.block;
    c.smem = l.smem;
    c.cluster_x = l.cluster_x;
    c.cooperative = l.cooperative;
    return emu::run_grid(c, reinterpret_cast<const void*>(kernel), [&] { kernel(static_cast<P>(args)...); });
#else
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = l.grid;
    cfg.blockDim = l.block;
    cfg.dynamicSmemBytes = l.smem;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[3];
    unsigned na = 0;
    if (l.cluster_x > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = l.cluster_x;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (l.pdl && g_pdl_enabled != 0) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (l.cooperative) {
        attr[na].id = cudaLaunchAttributeCooperative;
        attr[na].val.cooperative = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
#endif
}

}  // namespace nvk
