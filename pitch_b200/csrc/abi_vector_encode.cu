// C ABI, per-vector encoders (TurboQuant, PolarQuant variant): pitch_enqueue_encode.
// Declarations and the reference interfaces they replace: include/pitch_b200.h.
#include "abi_internal.h"

#include <atomic>
#include <cstring>

#include "common.cuh"
#include "vector_kernels.cuh"

using namespace pitch;
using namespace pitch_abi;

namespace {

template <int BITS>
bool fetch_book(int dim, Codebook<BITS>& out) { return book_get(dim, BITS, out.c); }

// Picks the quantiser grid for a codebook: the smallest power-of-two cell count (16...8192) whose
// cells each hold at most one decision boundary, verified with the very formula the kernel uses.
// Returns false when no such grid exists (the binary-search kernel is used instead).
bool quant_grid_for(const float* centroids, int bits, QuantGrid& g) {
    const int nedges = (1 << bits) - 1;
    float edges[255];
    float mingap = 4.0f;
    for (int k = 0; k < nedges; ++k) {
        edges[k] = 0.5f * (centroids[k] + centroids[k + 1]);
        if (!(std::fabs(edges[k]) <= 1.0f)) return false;
        if (k > 0) mingap = std::fmin(mingap, edges[k] - edges[k - 1]);
    }
    if (!(mingap > 0.0f)) return false;
    for (int cells = 16; cells <= 8192; cells <<= 1) {
        if (2.25f / cells >= 0.9f * mingap) continue;
        g.cells = cells;
        g.scale8 = 8.0f * cells / 2.25f;
        g.magic8 = 12582912.0f + 4.0f * cells;
        const uint32_t mask8 = (uint32_t)(cells - 1) << 3;
        bool ok = true;
        uint32_t prev = 0;
        for (int k = 0; k < nedges && ok; ++k) {
            const uint32_t c = quant_cell8(edges[k], g.scale8, g.magic8, mask8);
            if (k > 0 && c <= prev) ok = false;       // two boundaries in one cell, or not monotone
            prev = c;
        }
        if (ok) return true;
    }
    return false;
}

template <int BITS, typename T>
int launch_turbo_encode(int dim, uint32_t seed, const void* in, void* codes, void* scales, int64_t count,
                        cudaStream_t s) {
    Codebook<BITS> book;
    if (!fetch_book<BITS>(dim, book))
        return fail(PITCH_ERR_INVALID_INPUT, "no TurboQuant codebook for dim %d, bits %d", dim, BITS);
    if (dim < 32) {
        turbo_encode_kernel<BITS, T, true><<<vec_grid(count, dim), VEC_THREADS, 0, s>>>(
            static_cast<const T*>(in), static_cast<uint32_t*>(codes), static_cast<float*>(scales), count, dim, seed,
            rsqrt_dim(dim), aligned16(in) ? 1 : 0, book);
        return PITCH_OK;
    }
    QuantGrid grid;
    if (quant_grid_for(book.c, BITS, grid)) {
        // table-driven quantiser, CTAs loop over warp tiles
        int64_t ctas = vec_grid(count, dim);
        const int64_t cap = (int64_t)sm_count() * 8;
        if (ctas > cap) ctas = cap;
        const int smem = grid.cells * 8;
        if (smem > 4 * 1024) {                 // static staging buffers (about 40 KB) + table may pass the 48 KB default
            static std::atomic<bool> configured[64];
            int dev = 0;
            cudaGetDevice(&dev);
            if (dev >= 0 && dev < 64 && !configured[dev].load(std::memory_order_acquire)) {
                cudaFuncSetAttribute(turbo_encode_grid_kernel<BITS, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
                configured[dev].store(true, std::memory_order_release);
            }
        }
        turbo_encode_grid_kernel<BITS, T><<<(unsigned)ctas, VEC_THREADS, smem, s>>>(
            static_cast<const T*>(in), static_cast<uint32_t*>(codes), static_cast<float*>(scales), count, dim, seed,
            rsqrt_dim(dim), aligned16(in) ? 1 : 0, grid, book);
        return PITCH_OK;
    }
    turbo_encode_kernel<BITS, T, false><<<vec_grid(count, dim), VEC_THREADS, 0, s>>>(
        static_cast<const T*>(in), static_cast<uint32_t*>(codes), static_cast<float*>(scales), count, dim, seed,
        rsqrt_dim(dim), aligned16(in) ? 1 : 0, book);
    return PITCH_OK;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------- per-vector
int pitch_enqueue_encode(int method, int dim, int bits, uint32_t seed, int dtype, pitch_buffer input,
                         pitch_buffer codes, pitch_buffer scales, int64_t count, void* stream) {
    int st = check_vector_config(method, dim, bits, dtype);
    if (st) return st;
    if (count < 1) return fail(PITCH_ERR_INVALID_INPUT, "count must be at least 1");
    const int64_t stride = pitch_code_stride(dim, bits);
    if ((st = check_buffer(input, count * dim * elem_size(dtype), "input"))) return st;
    if ((st = check_buffer(codes, count * stride, "codes"))) return st;
    if ((st = check_buffer(scales, count * 4, "scales"))) return st;
    const pitch_buffer bufs[3] = {input, codes, scales};
    const char* const names[3] = {"input", "codes", "scales"};
    int dev;
    if ((st = check_same_device(bufs, names, 3, &dev))) return st;
    DeviceGuard guard(dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float rs = rsqrt_dim(dim);
    if (method == PITCH_TURBO_QUANT) {
        PITCH_DISPATCH_BITS(bits, PITCH_DISPATCH_DTYPE(dtype, st = (launch_turbo_encode<BITS, T>(
                                                                  dim, seed, at(input), at(codes), at(scales), count, s))));
        if (st) return st;
    } else {
        if (dim < 32) {
            PITCH_DISPATCH_BITS(bits, PITCH_DISPATCH_DTYPE(dtype, (polar_encode_kernel<BITS, T, true><<<vec_grid(count, dim), VEC_THREADS, 0, s>>>(
                                                                      reinterpret_cast<const T*>(at(input)),
                                                                      reinterpret_cast<uint32_t*>(at(codes)),
                                                                      reinterpret_cast<float*>(at(scales)), count, dim, seed, rs,
                                                                      aligned16(at(input)) ? 1 : 0))));
        } else {
            unsigned ctas = vec_grid(count, dim);                       // CTAs loop over warp tiles
            if (ctas > (unsigned)sm_count() * 8u) ctas = (unsigned)sm_count() * 8u;
            PITCH_DISPATCH_BITS(bits, PITCH_DISPATCH_DTYPE(dtype, (polar_encode_kernel<BITS, T, false><<<ctas, VEC_THREADS, 0, s>>>(
                                                                      reinterpret_cast<const T*>(at(input)),
                                                                      reinterpret_cast<uint32_t*>(at(codes)),
                                                                      reinterpret_cast<float*>(at(scales)), count, dim, seed, rs,
                                                                      aligned16(at(input)) ? 1 : 0))));
        }
    }
    return launch_status(true, method == PITCH_TURBO_QUANT ? "turbo_encode" : "polar_encode");
}

}  // extern "C"
