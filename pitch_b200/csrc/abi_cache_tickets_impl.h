// The whole-cache decode / step launch for caches that mix per-channel and TurboQuant planes: the
// instances of cache_decode_kernel that deal their items by drawn tickets.  Included by two translation
// units, one per deal (PITCH_TICKET_DEAL 1: abi_cache_tickets.cu; 2, which also asks the L2 for the items
// ahead: abi_cache_tickets_ahead.cu), so that the two sets of instances compile side by side.
#include "abi_internal.h"

#include <atomic>

#ifndef PITCH_TICKET_DEAL
#error "define PITCH_TICKET_DEAL (1 or 2) before including this file"
#endif

#include "cache_kernels.cuh"
#include "common.cuh"

using namespace pitch;
using namespace pitch_abi;

namespace {

template <typename T, int D, int BITS, int DEAL>
int launch_tickets_impl(const Cache64Params& p, int64_t tokens_for_grid, cudaStream_t s) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    constexpr int smem = cache64_smem_bytes<T>();
    if (dev >= 0 && dev < 64 && !configured[dev].load(std::memory_order_acquire)) {
        // idempotent: two threads racing here both set the same attribute
        if (cudaFuncSetAttribute(cache_decode_kernel<T, D, BITS, DEAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return launch_status(false, "cache_decode (shared memory opt-in)");
        configured[dev].store(true, std::memory_order_release);
    }
    // one CTA per multiprocessor, fewer when there is less than one item per warp
    const int64_t items = ceil_div(tokens_for_grid, 2048 / D);
    const int64_t work = (int64_t)p.segments * (items > 0 ? items : 1);
    int64_t ctas = ceil_div(work, CD_WARPS);
    if (ctas > sm_count()) ctas = sm_count();
    // Programmatic dependent launch: the kernel may start while the previous kernel of the stream
    // is still running; it builds its lookup tables, then waits for that kernel to complete before
    // it reads any cache memory.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(CD_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, cache_decode_kernel<T, D, BITS, DEAL>, p);
    return PITCH_OK;
}

template <typename T>
int launch_tickets(const Cache64Params& p, int dim, int bits, int64_t tokens_for_grid, cudaStream_t s) {
    if (dim == 64)
        return bits == 4 ? launch_tickets_impl<T, 64, 4, PITCH_TICKET_DEAL>(p, tokens_for_grid, s)
                         : launch_tickets_impl<T, 64, 3, PITCH_TICKET_DEAL>(p, tokens_for_grid, s);
    return bits == 4 ? launch_tickets_impl<T, 128, 4, PITCH_TICKET_DEAL>(p, tokens_for_grid, s)
                     : launch_tickets_impl<T, 128, 3, PITCH_TICKET_DEAL>(p, tokens_for_grid, s);
}

}  // namespace

namespace pitch_abi {

#if PITCH_TICKET_DEAL == 1
int launch_cache64_tickets(const Cache64Params& p, int dim, int bits, int dtype, int64_t tokens_for_grid, cudaStream_t s) {
    // fewer than 32 items per warp: the variant that also asks the L2 for the items ahead (abi_cache_tickets_ahead.cu)
    const int64_t items = ceil_div(tokens_for_grid, 2048 / dim) * p.segments * p.n_planes;
    if (items < (int64_t)32 * CD_WARPS * sm_count()) return launch_cache64_tickets_ahead(p, dim, bits, dtype, tokens_for_grid, s);
    int st = 0;
    PITCH_DISPATCH_DTYPE(dtype, st = (launch_tickets<T>(p, dim, bits, tokens_for_grid, s)));
    return st;
}
#else
int launch_cache64_tickets_ahead(const Cache64Params& p, int dim, int bits, int dtype, int64_t tokens_for_grid, cudaStream_t s) {
    int st = 0;
    PITCH_DISPATCH_DTYPE(dtype, st = (launch_tickets<T>(p, dim, bits, tokens_for_grid, s)));
    return st;
}
#endif

}  // namespace pitch_abi
