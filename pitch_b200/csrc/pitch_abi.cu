// C ABI of the B200 KV-cache codec: argument validation, kernel selection and launch.
// Declarations and the reference interfaces they replace: include/pitch_b200.h.
//
// Validation mirrors Codec.params / Codec.check (Sources/PITCH/Core/Codec.swift:28-47) and
// ChannelCodec.params / check (Sources/PITCH/PerChannel.swift:308-329), QuantConfig.init
// (Sources/PITCH/Models/QuantConfig.swift:24-35) and ChannelQuantConfig.init
// (Sources/PITCH/PerChannel.swift:30-43).  Nothing here allocates device memory.
#include "../../include/pitch_b200.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>
#include <string>

#include "append_kernels.cuh"
#include "attention_kernels.cuh"
#include "bias_kernels.cuh"
#include "cache_kernels.cuh"
#include "channel_kernels.cuh"
#include "common.cuh"
#include "vector_kernels.cuh"

using namespace pitch;

namespace {

thread_local std::string g_error;

int fail(int status, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
    return status;
}

// ---- host-side codebook table (TurboCodebooks.codebook(dim:bits:)) --------------------------
struct BookTable {
    std::mutex lock;
    bool present[11][9] = {};
    float values[11][9][256];
} g_books;

int log2_exact(int v) {
    int l = 0;
    while ((1 << l) < v) ++l;
    return l;
}

bool valid_vector_dim(int dim) { return dim >= 2 && dim <= PITCH_MAX_DIM && (dim & (dim - 1)) == 0; }
bool valid_bits(int bits) { return bits >= PITCH_MIN_BITS && bits <= PITCH_MAX_BITS; }

template <int BITS>
bool fetch_book(int dim, Codebook<BITS>& out) {
    std::lock_guard<std::mutex> guard(g_books.lock);
    const int l = log2_exact(dim);
    if (!g_books.present[l][BITS]) return false;
    memcpy(out.c, g_books.values[l][BITS], sizeof(float) << BITS);
    return true;
}

// ---- buffer checks (Codec.check) ------------------------------------------------------------
int check_buffer(const pitch_buffer& b, int64_t needs, const char* name) {
    if (b.base == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "%s buffer is null", name);
    if (b.offset < 0 || (b.offset & 3) != 0)
        return fail(PITCH_ERR_INVALID_INPUT, "%s offset %lld must be a non-negative multiple of 4", name,
                    (long long)b.offset);
    if (b.length < b.offset + needs)
        return fail(PITCH_ERR_INVALID_INPUT, "%s buffer has %lld bytes after offset; needs %lld", name,
                    (long long)(b.length - b.offset), (long long)needs);
    return PITCH_OK;
}

// All buffers of a call must be device-accessible memory of one GPU ("belongs to a different
// MTLDevice", Codec.swift:38-40).  Returns that GPU's ordinal in *device.
int check_same_device(const pitch_buffer* bufs, const char* const* names, int n, int* device) {
    int dev = -1;
    for (int i = 0; i < n; ++i) {
        cudaPointerAttributes attr;
        cudaError_t e = cudaPointerGetAttributes(&attr, bufs[i].base);
        if (e != cudaSuccess) {
            cudaGetLastError();
            if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver)
                return fail(PITCH_ERR_DEVICE_NOT_SUPPORTED, "no usable CUDA device: %s", cudaGetErrorString(e));
            return fail(PITCH_ERR_INVALID_INPUT, "%s buffer: %s", names[i], cudaGetErrorString(e));
        }
        if (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)
            return fail(PITCH_ERR_INVALID_INPUT, "%s buffer is not device memory", names[i]);
        if (dev >= 0 && attr.type == cudaMemoryTypeDevice && attr.device != dev)
            return fail(PITCH_ERR_INVALID_INPUT, "%s buffer belongs to a different GPU", names[i]);
        if (attr.type == cudaMemoryTypeDevice) dev = attr.device;
    }
    if (dev < 0) cudaGetDevice(&dev);
    *device = dev;
    return PITCH_OK;
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev); else prev = -1;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

int launch_status(bool encode, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return PITCH_OK;
    if (e == cudaErrorNoKernelImageForDevice || e == cudaErrorInvalidDeviceFunction)
        return fail(PITCH_ERR_KERNEL_UNAVAILABLE, "%s: %s (library is built for sm_100a)", what, cudaGetErrorString(e));
    return fail(encode ? PITCH_ERR_ENCODING_FAILED : PITCH_ERR_DECODING_FAILED, "%s: %s", what, cudaGetErrorString(e));
}

inline unsigned char* at(const pitch_buffer& b) { return static_cast<unsigned char*>(b.base) + b.offset; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline float rsqrt_dim(int dim) { return (float)(1.0 / std::sqrt((double)dim)); }
inline int elem_size(int dtype) { return dtype == PITCH_F32 ? 4 : 2; }

int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

int check_vector_config(int method, int dim, int bits, int dtype) {
    if (method != PITCH_TURBO_QUANT && method != PITCH_POLAR_QUANT)
        return fail(PITCH_ERR_INVALID_INPUT, "unknown method %d", method);
    if (!valid_vector_dim(dim))
        return fail(PITCH_ERR_INVALID_DIMENSION, "Invalid dimension %d. Must be a power of two in [2, %d].", dim, PITCH_MAX_DIM);
    if (!valid_bits(bits)) return fail(PITCH_ERR_INVALID_BIT_WIDTH, "Invalid bit width %d. Must be in 2...8.", bits);
    if (dtype < PITCH_F32 || dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", dtype);
    return PITCH_OK;
}

int check_channel_config(int dim, int bits, int group_size, int dtype) {
    if (dim < 1 || dim > PITCH_MAX_DIM)
        return fail(PITCH_ERR_INVALID_INPUT, "per-channel dimension %d must be in 1...%d", dim, PITCH_MAX_DIM);
    if (!valid_bits(bits)) return fail(PITCH_ERR_INVALID_BIT_WIDTH, "Invalid bit width %d. Must be in 2...8.", bits);
    if (group_size < 1 || group_size > PITCH_MAX_GROUP)
        return fail(PITCH_ERR_INVALID_INPUT, "group size %d must be in 1...%d", group_size, PITCH_MAX_GROUP);
    if (dtype < PITCH_F32 || dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", dtype);
    return PITCH_OK;
}

// ---- dispatch helpers -------------------------------------------------------------------------
#define PITCH_DISPATCH_BITS(bits, ...)                   \
    switch (bits) {                                      \
        case 2: { constexpr int BITS = 2; __VA_ARGS__; break; } \
        case 3: { constexpr int BITS = 3; __VA_ARGS__; break; } \
        case 4: { constexpr int BITS = 4; __VA_ARGS__; break; } \
        case 5: { constexpr int BITS = 5; __VA_ARGS__; break; } \
        case 6: { constexpr int BITS = 6; __VA_ARGS__; break; } \
        case 7: { constexpr int BITS = 7; __VA_ARGS__; break; } \
        default: { constexpr int BITS = 8; __VA_ARGS__; break; } \
    }

#define PITCH_DISPATCH_DTYPE(dtype, ...)                                  \
    switch (dtype) {                                                      \
        case PITCH_F32: { typedef float T; __VA_ARGS__; break; }          \
        case PITCH_F16: { typedef __half T; __VA_ARGS__; break; }         \
        default: { typedef __nv_bfloat16 T; __VA_ARGS__; break; }         \
    }

unsigned vec_grid(int64_t count, int dim);
int sm_count();
// Grid of a kernel whose CTAs loop over warp tiles: enough CTAs for every SM's registers, no more.
unsigned vec_grid_looping(int64_t count, int dim) {
    const unsigned all = vec_grid(count, dim), cap = (unsigned)sm_count() * 8u;
    return all < cap ? all : cap;
}

unsigned vec_grid(int64_t count, int dim) {
    const int vpw = dim < 32 ? 32 : 1024 / dim;
    return (unsigned)ceil_div(ceil_div(count, vpw), VEC_WARPS);
}

// Persistent whole-cache decode: one CTA per SM, opt-in dynamic shared memory.
int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);     // idempotent: racing threads store the same value
    }
    return n;
}

template <typename T, int D, int BITS>
int launch_cache64_impl(const Cache64Params& p, cudaStream_t s) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    constexpr int smem = cache64_smem_bytes<T>();
    if (dev >= 0 && dev < 64 && !configured[dev].load(std::memory_order_acquire)) {
        // idempotent: two threads racing here both set the same attribute
        if (cudaFuncSetAttribute(cache_decode_kernel<T, D, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return launch_status(false, "cache_decode (shared memory opt-in)");
        configured[dev].store(true, std::memory_order_release);
    }
    const int64_t work = (int64_t)p.segments * (p.full_items > 0 ? p.full_items : 1);
    int64_t ctas = ceil_div(work, CD_WARPS);
    if (ctas > sm_count()) ctas = sm_count();
    // Programmatic dependent launch: the kernel may start while the previous kernel of the stream
    // (typically the append of the same step) is still running; it builds its lookup table, then
    // waits for that kernel to complete before it reads any cache memory.
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
    cudaLaunchKernelEx(&cfg, cache_decode_kernel<T, D, BITS>, p);
    return PITCH_OK;
}

// dim in {64, 128}, bits (of the TurboQuant planes) in {3, 4}
template <typename T>
int launch_cache64(const Cache64Params& p, int dim, int bits, cudaStream_t s) {
    if (dim == 64) return bits == 4 ? launch_cache64_impl<T, 64, 4>(p, s) : launch_cache64_impl<T, 64, 3>(p, s);
    return bits == 4 ? launch_cache64_impl<T, 128, 4>(p, s) : launch_cache64_impl<T, 128, 3>(p, s);
}

// Fills the geometry of a fast-path launch: `tokens` tokens per segment at head dimension `dim`.
void cache64_geometry(Cache64Params& p, int dim, int64_t segments, int64_t tokens) {
    const int per_item = 2048 / dim;
    p.segments = (int)segments;
    p.full_items = (int)(tokens / per_item);
    p.tail = (int)(tokens % per_item);
    p.rs = rsqrt_dim(dim);
}

void cache64_signs(Plane64& q, uint32_t seed) {
    for (int j = 0; j < 4; ++j) q.neg[j] = negate_mask32(seed, 32u * j);
}

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

template <int BITS, typename T>
int launch_turbo_decode(int dim, uint32_t seed, const void* codes, const void* scales, void* out, int64_t count,
                        cudaStream_t s) {
    Codebook<BITS> book;
    if (!fetch_book<BITS>(dim, book))
        return fail(PITCH_ERR_INVALID_INPUT, "no TurboQuant codebook for dim %d, bits %d", dim, BITS);
    if ((BITS == 4 || BITS == 3) && (dim == 64 || dim == 128) && aligned16(codes) && aligned16(out) &&
        count / (2048 / dim) <= 0x3FFFFFFF) {
        // the persistent whole-cache kernel with a single TurboQuant plane
        Cache64Params p;
        memset(&p, 0, sizeof p);
        p.n_planes = 1;
        cache64_geometry(p, dim, 1, count);
        p.plane[0].kind = 0;
        p.plane[0].group_items = 1;
        cache64_signs(p.plane[0], seed);
        p.plane[0].codes = static_cast<const unsigned char*>(codes);
        p.plane[0].side = static_cast<const unsigned char*>(scales);
        p.plane[0].out = static_cast<unsigned char*>(out);
        memcpy(p.book.c, book.c, sizeof(float) << BITS);
        return launch_cache64<T>(p, dim, BITS, s);
    }
    if (dim < 32)
        turbo_decode_kernel<BITS, T, true><<<vec_grid(count, dim), VEC_THREADS, 0, s>>>(
            static_cast<const uint32_t*>(codes), static_cast<const float*>(scales), static_cast<T*>(out), count, dim, seed,
            rsqrt_dim(dim), aligned16(out) ? 1 : 0, book);
    else
        turbo_decode_kernel<BITS, T, false><<<vec_grid_looping(count, dim), VEC_THREADS, 0, s>>>(
            static_cast<const uint32_t*>(codes), static_cast<const float*>(scales), static_cast<T*>(out), count, dim, seed,
            rsqrt_dim(dim), aligned16(out) ? 1 : 0, book);
    return PITCH_OK;
}

// slab mapping applies when dim/8 is a power of two in 1...32 and the buffers allow 16-byte access
bool slab_ok(int dim, int bits) {
    if (bits != 2 && bits != 4 && bits != 8) return false;
    if (dim % 8 != 0) return false;
    const int slabs = dim / 8;
    return slabs <= 32 && (slabs & (slabs - 1)) == 0;
}

__global__ void pack_codes_kernel(const int32_t* __restrict__ codes, uint32_t* __restrict__ packed, int64_t count,
                                  int dim, int bits, int wpv) {
    const int64_t total = count * wpv;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = e / wpv;
        const int w = (int)(e - v * wpv);
        const int bit0 = w * 32;
        const int i0 = bit0 / bits;
        int i1 = (bit0 + 31) / bits;
        if (i1 > dim - 1) i1 = dim - 1;
        uint32_t word = 0;
        for (int i = i0; i <= i1; ++i) {
            const uint32_t c = (uint32_t)codes[v * dim + i] & ((1u << bits) - 1u);
            const int shift = i * bits - bit0;
            word |= shift >= 0 ? (c << shift) : (c >> (-shift));
        }
        packed[e] = word;
    }
}

__global__ void unpack_codes_kernel(const uint32_t* __restrict__ packed, int32_t* __restrict__ codes, int64_t count,
                                    int dim, int bits, int wpv) {
    const int64_t total = count * dim;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = e / dim;
        const int i = (int)(e - v * dim);
        codes[e] = (int32_t)read_code(packed + v * wpv, i, bits);
    }
}

__global__ void checksum_kernel(const uint32_t* __restrict__ words, int64_t n, unsigned long long* result) {
    unsigned long long acc = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        acc += ((unsigned long long)words[i] + 1ull) * (2ull * (unsigned long long)i + 1ull);
    for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(FULL, acc, m);
    if ((threadIdx.x & 31) == 0 && acc != 0) atomicAdd(result, acc);
}

}  // namespace

// =================================================================================================
extern "C" {

int pitch_abi_version(void) { return PITCH_ABI_VERSION; }

const char* pitch_status_string(int status) {
    switch (status) {
        case PITCH_OK: return "ok";
        case PITCH_ERR_INVALID_INPUT: return "invalid input";
        case PITCH_ERR_INVALID_BIT_WIDTH: return "invalid bit width";
        case PITCH_ERR_INVALID_DIMENSION: return "invalid dimension";
        case PITCH_ERR_CONFIGURATION_MISMATCH: return "configuration mismatch";
        case PITCH_ERR_KERNEL_UNAVAILABLE: return "no kernel image for this GPU";
        case PITCH_ERR_ENCODING_FAILED: return "encoding failed";
        case PITCH_ERR_DECODING_FAILED: return "decoding failed";
        case PITCH_ERR_DEVICE_NOT_SUPPORTED: return "CUDA device not supported";
        default: return "unknown status";
    }
}

const char* pitch_last_error(void) { return g_error.c_str(); }

int pitch_code_stride(int dim, int bits) { return words_per_vector(dim, bits) * 4; }

int pitch_set_codebook(int dim, int bits, const float* centroids) {
    if (!valid_vector_dim(dim))
        return fail(PITCH_ERR_INVALID_DIMENSION, "Invalid dimension %d. Must be a power of two in [2, %d].", dim, PITCH_MAX_DIM);
    if (!valid_bits(bits)) return fail(PITCH_ERR_INVALID_BIT_WIDTH, "Invalid bit width %d. Must be in 2...8.", bits);
    if (centroids == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "centroids is null");
    const int n = 1 << bits;
    for (int i = 0; i < n; ++i) {
        if (!std::isfinite(centroids[i])) return fail(PITCH_ERR_INVALID_INPUT, "centroid %d is not finite", i);
        if (i > 0 && !(centroids[i] > centroids[i - 1]))
            return fail(PITCH_ERR_INVALID_INPUT, "centroids must be strictly ascending (index %d)", i);
    }
    std::lock_guard<std::mutex> guard(g_books.lock);
    const int l = log2_exact(dim);
    memcpy(g_books.values[l][bits], centroids, sizeof(float) * n);
    g_books.present[l][bits] = true;
    return PITCH_OK;
}

int pitch_has_codebook(int dim, int bits) {
    if (!valid_vector_dim(dim) || !valid_bits(bits)) return 0;
    std::lock_guard<std::mutex> guard(g_books.lock);
    return g_books.present[log2_exact(dim)][bits] ? 1 : 0;
}

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

int pitch_enqueue_decode(int method, int dim, int bits, uint32_t seed, int dtype, pitch_buffer codes,
                         pitch_buffer scales, pitch_buffer output, int64_t count, void* stream) {
    int st = check_vector_config(method, dim, bits, dtype);
    if (st) return st;
    if (count < 1) return fail(PITCH_ERR_INVALID_INPUT, "count must be at least 1");
    const int64_t stride = pitch_code_stride(dim, bits);
    if ((st = check_buffer(codes, count * stride, "codes"))) return st;
    if ((st = check_buffer(scales, count * 4, "scales"))) return st;
    if ((st = check_buffer(output, count * dim * elem_size(dtype), "output"))) return st;
    const pitch_buffer bufs[3] = {codes, scales, output};
    const char* const names[3] = {"codes", "scales", "output"};
    int dev;
    if ((st = check_same_device(bufs, names, 3, &dev))) return st;
    DeviceGuard guard(dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float rs = rsqrt_dim(dim);
    if (method == PITCH_TURBO_QUANT) {
        PITCH_DISPATCH_BITS(bits, PITCH_DISPATCH_DTYPE(dtype, st = (launch_turbo_decode<BITS, T>(
                                                                  dim, seed, at(codes), at(scales), at(output), count, s))));
        if (st) return st;
    } else {
        if (dim < 32) {
            PITCH_DISPATCH_BITS(bits, PITCH_DISPATCH_DTYPE(dtype, (polar_decode_kernel<BITS, T, true><<<vec_grid(count, dim), VEC_THREADS, 0, s>>>(
                                                                      reinterpret_cast<const uint32_t*>(at(codes)),
                                                                      reinterpret_cast<const float*>(at(scales)),
                                                                      reinterpret_cast<T*>(at(output)), count, dim, seed, rs,
                                                                      aligned16(at(output)) ? 1 : 0))));
        } else {
            PITCH_DISPATCH_BITS(bits, PITCH_DISPATCH_DTYPE(dtype, (polar_decode_kernel<BITS, T, false><<<vec_grid_looping(count, dim), VEC_THREADS, 0, s>>>(
                                                                      reinterpret_cast<const uint32_t*>(at(codes)),
                                                                      reinterpret_cast<const float*>(at(scales)),
                                                                      reinterpret_cast<T*>(at(output)), count, dim, seed, rs,
                                                                      aligned16(at(output)) ? 1 : 0))));
        }
    }
    return launch_status(false, method == PITCH_TURBO_QUANT ? "turbo_decode" : "polar_decode");
}

// --------------------------------------------------------------------------------- per-channel
int pitch_enqueue_channel_encode(int dim, int bits, int group_size, int dtype, pitch_buffer input,
                                 pitch_buffer codes, pitch_buffer ranges, int64_t count, void* stream) {
    int st = check_channel_config(dim, bits, group_size, dtype);
    if (st) return st;
    if (count < 1) return fail(PITCH_ERR_INVALID_INPUT, "count must be at least 1");
    const int64_t stride = pitch_code_stride(dim, bits);
    const int64_t groups = ceil_div(count, group_size);
    if ((st = check_buffer(input, count * dim * elem_size(dtype), "input"))) return st;
    if ((st = check_buffer(codes, count * stride, "codes"))) return st;
    if ((st = check_buffer(ranges, groups * 4 * dim, "ranges"))) return st;
    const pitch_buffer bufs[3] = {input, codes, ranges};
    const char* const names[3] = {"input", "codes", "ranges"};
    int dev;
    if ((st = check_same_device(bufs, names, 3, &dev))) return st;
    DeviceGuard guard(dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool slab = slab_ok(dim, bits) && aligned16(at(input)) && aligned16(at(ranges)) &&
                      (reinterpret_cast<uintptr_t>(at(codes)) % (bits == 8 ? 8 : 4)) == 0;
    if (slab) {
        const int l2 = log2_exact(dim / 8);
        const unsigned grid = (unsigned)ceil_div(groups, CH_WARPS);
#define PITCH_SLAB_ENC(B)                                                                                      \
    PITCH_DISPATCH_DTYPE(dtype, (channel_encode_slab_kernel<B, T><<<grid, CH_THREADS, 0, s>>>(                 \
                                    reinterpret_cast<const T*>(at(input)), at(codes),                          \
                                    reinterpret_cast<__half*>(at(ranges)), count, dim, l2, group_size, groups)))
        if (bits == 2) { PITCH_SLAB_ENC(2); } else if (bits == 4) { PITCH_SLAB_ENC(4); } else { PITCH_SLAB_ENC(8); }
#undef PITCH_SLAB_ENC
    } else {
        PITCH_DISPATCH_DTYPE(dtype, (channel_encode_general_kernel<T><<<(unsigned)groups, 256, 0, s>>>(
                                        reinterpret_cast<const T*>(at(input)), reinterpret_cast<uint32_t*>(at(codes)),
                                        reinterpret_cast<__half*>(at(ranges)), count, dim, bits, group_size)));
    }
    return launch_status(true, "channel_encode");
}

int pitch_enqueue_channel_decode(int dim, int bits, int group_size, int dtype, pitch_buffer codes,
                                 pitch_buffer ranges, pitch_buffer output, int64_t count, void* stream) {
    int st = check_channel_config(dim, bits, group_size, dtype);
    if (st) return st;
    if (count < 1) return fail(PITCH_ERR_INVALID_INPUT, "count must be at least 1");
    const int64_t stride = pitch_code_stride(dim, bits);
    const int64_t groups = ceil_div(count, group_size);
    if ((st = check_buffer(codes, count * stride, "codes"))) return st;
    if ((st = check_buffer(ranges, groups * 4 * dim, "ranges"))) return st;
    if ((st = check_buffer(output, count * dim * elem_size(dtype), "output"))) return st;
    const pitch_buffer bufs[3] = {codes, ranges, output};
    const char* const names[3] = {"codes", "ranges", "output"};
    int dev;
    if ((st = check_same_device(bufs, names, 3, &dev))) return st;
    DeviceGuard guard(dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool slab = slab_ok(dim, bits) && aligned16(at(output)) && aligned16(at(ranges)) &&
                      (reinterpret_cast<uintptr_t>(at(codes)) % (bits == 8 ? 8 : 4)) == 0;
    if (slab && (dim == 64 || dim == 128) && bits == 4 && group_size % (2048 / dim) == 0 && aligned16(at(codes)) &&
        count / (2048 / dim) <= 0x3FFFFFFF) {
        // the persistent whole-cache kernel with a single per-channel plane
        Cache64Params p;
        memset(&p, 0, sizeof p);
        p.n_planes = 1;
        cache64_geometry(p, dim, 1, count);
        p.plane[0].kind = 1;
        p.plane[0].group_items = group_size / (2048 / dim);
        p.plane[0].codes = at(codes);
        p.plane[0].side = at(ranges);
        p.plane[0].out = at(output);
        PITCH_DISPATCH_DTYPE(dtype, st = (launch_cache64<T>(p, dim, 4, s)));
        if (st) return st;
        return launch_status(false, "channel_decode");
    }
    if (slab) {
        const int l2 = log2_exact(dim / 8);
        const int chunks = (int)ceil_div(group_size, CH_CHUNK);
        const int64_t tiles = groups * chunks;
        const unsigned grid = (unsigned)ceil_div(tiles, CH_WARPS);
#define PITCH_SLAB_DEC(B)                                                                                      \
    PITCH_DISPATCH_DTYPE(dtype, (channel_decode_slab_kernel<B, T><<<grid, CH_THREADS, 0, s>>>(                 \
                                    at(codes), reinterpret_cast<const __half*>(at(ranges)),                    \
                                    reinterpret_cast<T*>(at(output)), count, dim, l2, group_size, chunks, tiles)))
        if (bits == 2) { PITCH_SLAB_DEC(2); } else if (bits == 4) { PITCH_SLAB_DEC(4); } else { PITCH_SLAB_DEC(8); }
#undef PITCH_SLAB_DEC
    } else {
        const int64_t total = count * dim;
        int64_t blocks = ceil_div(total, 256);
        if (blocks > 148 * 64) blocks = 148 * 64;
        PITCH_DISPATCH_DTYPE(dtype, (channel_decode_general_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(
                                        reinterpret_cast<const uint32_t*>(at(codes)),
                                        reinterpret_cast<const __half*>(at(ranges)), reinterpret_cast<T*>(at(output)),
                                        count, dim, bits, group_size)));
    }
    return launch_status(false, "channel_decode");
}

// ------------------------------------------------------------------------------------ rotation
int pitch_enqueue_rotate(int mode, int dim, uint32_t seed, pitch_buffer input, pitch_buffer output, int64_t count,
                         void* stream) {
    if (mode < 0 || mode > 2) return fail(PITCH_ERR_INVALID_INPUT, "unknown rotation mode %d", mode);
    if (!valid_vector_dim(dim))
        return fail(PITCH_ERR_INVALID_DIMENSION, "Invalid dimension %d. Must be a power of two in [2, %d].", dim, PITCH_MAX_DIM);
    if (count < 1) return fail(PITCH_ERR_INVALID_INPUT, "count must be at least 1");
    int st;
    if ((st = check_buffer(input, count * dim * 4, "input"))) return st;
    if ((st = check_buffer(output, count * dim * 4, "output"))) return st;
    const pitch_buffer bufs[2] = {input, output};
    const char* const names[2] = {"input", "output"};
    int dev;
    if ((st = check_same_device(bufs, names, 2, &dev))) return st;
    DeviceGuard guard(dev);
    if (dim < 32)
        rotate_kernel<true><<<vec_grid(count, dim), VEC_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
            reinterpret_cast<const float*>(at(input)), reinterpret_cast<float*>(at(output)), count, dim, seed,
            rsqrt_dim(dim), mode, aligned16(at(input)) ? 1 : 0, aligned16(at(output)) ? 1 : 0);
    else
        rotate_kernel<false><<<vec_grid(count, dim), VEC_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
            reinterpret_cast<const float*>(at(input)), reinterpret_cast<float*>(at(output)), count, dim, seed,
            rsqrt_dim(dim), mode, aligned16(at(input)) ? 1 : 0, aligned16(at(output)) ? 1 : 0);
    return launch_status(true, "rotate");
}

// ----------------------------------------------------------------------------- pack / unpack
static int pack_common(bool pack, int dim, int bits, pitch_buffer codes_i32, pitch_buffer packed, int64_t count,
                       void* stream) {
    if (dim < 1 || dim > PITCH_MAX_DIM) return fail(PITCH_ERR_INVALID_INPUT, "dimension %d must be in 1...%d", dim, PITCH_MAX_DIM);
    if (!valid_bits(bits)) return fail(PITCH_ERR_INVALID_BIT_WIDTH, "Invalid bit width %d. Must be in 2...8.", bits);
    if (count < 1) return fail(PITCH_ERR_INVALID_INPUT, "count must be at least 1");
    int st;
    const int wpv = words_per_vector(dim, bits);
    if ((st = check_buffer(codes_i32, count * dim * 4, "codes_i32"))) return st;
    if ((st = check_buffer(packed, count * wpv * 4, "packed"))) return st;
    const pitch_buffer bufs[2] = {codes_i32, packed};
    const char* const names[2] = {"codes_i32", "packed"};
    int dev;
    if ((st = check_same_device(bufs, names, 2, &dev))) return st;
    DeviceGuard guard(dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int64_t blocks = ceil_div(count * (pack ? wpv : dim), 256);
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (pack)
        pack_codes_kernel<<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const int32_t*>(at(codes_i32)),
                                                           reinterpret_cast<uint32_t*>(at(packed)), count, dim, bits, wpv);
    else
        unpack_codes_kernel<<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const uint32_t*>(at(packed)),
                                                             reinterpret_cast<int32_t*>(at(codes_i32)), count, dim, bits, wpv);
    return launch_status(pack, pack ? "pack_codes" : "unpack_codes");
}

int pitch_enqueue_pack_codes(int dim, int bits, pitch_buffer codes_i32, pitch_buffer packed, int64_t count, void* stream) {
    return pack_common(true, dim, bits, codes_i32, packed, count, stream);
}
int pitch_enqueue_unpack_codes(int dim, int bits, pitch_buffer packed, pitch_buffer codes_i32, int64_t count, void* stream) {
    return pack_common(false, dim, bits, codes_i32, packed, count, stream);
}

// ------------------------------------------------------------------------------- whole cache
static int64_t plane_side_bytes(const pitch_plane& pl, int dim, int64_t tokens) {
    if (pl.kind == PITCH_PLANE_CHANNEL) return ceil_div(tokens, pl.group_size) * 4 * dim;
    return tokens * 4;
}

int pitch_enqueue_cache_decode(const pitch_cache_desc* d, void* stream) {
    if (d == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "descriptor is null");
    if (d->n_planes < 1 || d->n_planes > 4) return fail(PITCH_ERR_INVALID_INPUT, "n_planes %d must be in 1...4", d->n_planes);
    if (d->segments < 1 || d->tokens < 1) return fail(PITCH_ERR_INVALID_INPUT, "segments and tokens must be at least 1");
    if (d->out_dtype < PITCH_F32 || d->out_dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", d->out_dtype);
    const int dim = d->dim;
    bool fused = dim == 64 || dim == 128;
    int turbo_bits = 0;                       // all TurboQuant planes of a fast-path launch share one width
    for (int i = 0; i < d->n_planes; ++i) {
        const pitch_plane& pl = d->planes[i];
        int st;
        if (pl.kind == PITCH_PLANE_CHANNEL) {
            if ((st = check_channel_config(dim, pl.bits, pl.group_size, d->out_dtype))) return st;
        } else if (pl.kind == PITCH_PLANE_TURBO || pl.kind == PITCH_PLANE_POLAR) {
            if ((st = check_vector_config(pl.kind, dim, pl.bits, d->out_dtype))) return st;
        } else {
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: unknown kind %d", i, pl.kind);
        }
        if (!pl.codes || !pl.side || !pl.out) return fail(PITCH_ERR_INVALID_INPUT, "plane %d: null pointer", i);
        if (!aligned16(pl.codes) || !aligned16(pl.side) || !aligned16(pl.out) || (pl.codes_seg_stride & 15) ||
            (pl.side_seg_stride & 15) || (pl.out_seg_stride & 15))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: pointers and segment strides must be multiples of 16", i);
        const int64_t stride = pitch_code_stride(dim, pl.bits);
        if (d->segments > 1 && (pl.codes_seg_stride < d->tokens * stride ||
                                pl.side_seg_stride < plane_side_bytes(pl, dim, d->tokens) ||
                                pl.out_seg_stride < d->tokens * dim * elem_size(d->out_dtype)))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: a segment stride is smaller than one segment", i);
        if (pl.kind == PITCH_PLANE_POLAR) fused = false;
        if (pl.kind == PITCH_PLANE_CHANNEL && (pl.bits != 4 || dim > 128 || pl.group_size % (2048 / (dim > 128 ? 128 : dim)) != 0))
            fused = false;
        if (pl.kind == PITCH_PLANE_TURBO) {
            if (pl.bits != 3 && pl.bits != 4) fused = false;
            if (turbo_bits != 0 && turbo_bits != pl.bits) fused = false;
            turbo_bits = pl.bits;
        }
        if (d->segments > 0x7FFFFFFF / (d->tokens / 16 + 1)) fused = false;      // 32-bit item indices in the kernel
    }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, d->planes[0].out) != cudaSuccess ||
        (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)) {
        cudaGetLastError();
        return fail(PITCH_ERR_INVALID_INPUT, "plane 0: output is not device memory");
    }
    int dev = attr.device;
    DeviceGuard guard(dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    if (fused) {
        Cache64Params p;
        memset(&p, 0, sizeof p);
        p.n_planes = d->n_planes;
        cache64_geometry(p, dim, d->segments, d->tokens);
        if (turbo_bits == 0) turbo_bits = 4;
        for (int i = 0; i < d->n_planes; ++i) {
            const pitch_plane& pl = d->planes[i];
            Plane64& q = p.plane[i];
            q.kind = pl.kind == PITCH_PLANE_CHANNEL ? 1 : 0;
            q.group_items = pl.kind == PITCH_PLANE_CHANNEL ? pl.group_size / (2048 / dim) : 1;
            cache64_signs(q, pl.seed);
            q.codes = static_cast<const unsigned char*>(pl.codes);
            q.codes_seg_stride = pl.codes_seg_stride;
            q.side = static_cast<const unsigned char*>(pl.side);
            q.side_seg_stride = pl.side_seg_stride;
            q.out = static_cast<unsigned char*>(pl.out);
            q.out_seg_stride = pl.out_seg_stride;
            if (q.kind == 0) {
                std::lock_guard<std::mutex> guardb(g_books.lock);
                const int l = log2_exact(dim);
                if (!g_books.present[l][turbo_bits])
                    return fail(PITCH_ERR_INVALID_INPUT, "no TurboQuant codebook for dim %d, bits %d", dim, turbo_bits);
                memcpy(p.book.c, g_books.values[l][turbo_bits], sizeof(float) << turbo_bits);
            }
        }
        int st = 0;
        PITCH_DISPATCH_DTYPE(d->out_dtype, st = (launch_cache64<T>(p, dim, turbo_bits, s)));
        if (st) return st;
        return launch_status(false, "cache_decode");
    }

    // Any other shape: one stand-alone decode per (plane, segment), same results.
    for (int i = 0; i < d->n_planes; ++i) {
        const pitch_plane& pl = d->planes[i];
        const int64_t stride = pitch_code_stride(dim, pl.bits);
        for (int64_t sgm = 0; sgm < d->segments; ++sgm) {
            pitch_buffer codes = {pl.codes, sgm * pl.codes_seg_stride + d->tokens * stride, sgm * pl.codes_seg_stride};
            pitch_buffer side = {pl.side, sgm * pl.side_seg_stride + plane_side_bytes(pl, dim, d->tokens), sgm * pl.side_seg_stride};
            pitch_buffer out = {pl.out, sgm * pl.out_seg_stride + d->tokens * dim * elem_size(d->out_dtype), sgm * pl.out_seg_stride};
            int st;
            if (pl.kind == PITCH_PLANE_CHANNEL)
                st = pitch_enqueue_channel_decode(dim, pl.bits, pl.group_size, d->out_dtype, codes, side, out, d->tokens, stream);
            else
                st = pitch_enqueue_decode(pl.kind, dim, pl.bits, pl.seed, d->out_dtype, codes, side, out, d->tokens, stream);
            if (st) return st;
        }
    }
    return PITCH_OK;
}

int pitch_enqueue_cache_append(const pitch_cache_desc* d, const pitch_append_src* src, int in_dtype, int64_t n_new,
                               void* stream) {
    if (d == nullptr || src == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "descriptor is null");
    if (d->n_planes < 1 || d->n_planes > 4) return fail(PITCH_ERR_INVALID_INPUT, "n_planes %d must be in 1...4", d->n_planes);
    if (d->segments < 1 || d->segments > 65535) return fail(PITCH_ERR_INVALID_INPUT, "segments must be in 1...65535");
    if (d->tokens < 0) return fail(PITCH_ERR_INVALID_INPUT, "tokens must not be negative");
    if (n_new < 1 || n_new > 65535) return fail(PITCH_ERR_INVALID_INPUT, "n_new must be in 1...65535");
    if (in_dtype < PITCH_F32 || in_dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", in_dtype);
    const int dim = d->dim;
    for (int i = 0; i < d->n_planes; ++i) {
        const pitch_plane& pl = d->planes[i];
        int st;
        if (pl.kind == PITCH_PLANE_CHANNEL) {
            if ((st = check_channel_config(dim, pl.bits, pl.group_size, in_dtype))) return st;
            if (src[i].residual == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "plane %d: residual buffer is null", i);
            if (src[i].residual_seg_stride < ((int64_t)pl.group_size + 2) * dim * 4 || (src[i].residual_seg_stride & 3))
                return fail(PITCH_ERR_INVALID_INPUT, "plane %d: residual segment stride too small", i);
            if (d->tokens % pl.group_size + n_new > pl.group_size)
                return fail(PITCH_ERR_INVALID_INPUT, "plane %d: new tokens must fall into one group of %d", i, pl.group_size);
        } else if (pl.kind == PITCH_PLANE_TURBO || pl.kind == PITCH_PLANE_POLAR) {
            if ((st = check_vector_config(pl.kind, dim, pl.bits, in_dtype))) return st;
        } else {
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: unknown kind %d", i, pl.kind);
        }
        if (!pl.codes || !pl.side || !src[i].input) return fail(PITCH_ERR_INVALID_INPUT, "plane %d: null pointer", i);
        if ((reinterpret_cast<uintptr_t>(pl.codes) & 3) || (reinterpret_cast<uintptr_t>(pl.side) & 3) ||
            (reinterpret_cast<uintptr_t>(src[i].input) & 3) || (pl.codes_seg_stride & 3) || (pl.side_seg_stride & 3) ||
            (src[i].input_seg_stride & 3))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: pointers and strides must be multiples of 4", i);
    }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, d->planes[0].codes) != cudaSuccess ||
        (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)) {
        cudaGetLastError();
        return fail(PITCH_ERR_INVALID_INPUT, "plane 0: codes is not device memory");
    }
    DeviceGuard guard(attr.device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // one launch for every segment and plane; the descriptor (with the codebooks) travels as the kernel parameter
    static thread_local AppendParams p;
    p.n_planes = d->n_planes;
    p.dim = dim;
    p.n_new = (int)n_new;
    p.rs = rsqrt_dim(dim);
    p.first_token = d->tokens;
    for (int i = 0; i < d->n_planes; ++i) {
        const pitch_plane& pl = d->planes[i];
        AppendPlane& q = p.plane[i];
        q.kind = pl.kind == PITCH_PLANE_CHANNEL ? 2 : (pl.kind == PITCH_PLANE_TURBO ? 0 : 1);
        q.bits = pl.bits;
        q.group_size = pl.group_size;
        q.seed = pl.seed;
        q.in = static_cast<const unsigned char*>(src[i].input);
        q.in_seg_stride = src[i].input_seg_stride;
        q.codes = static_cast<unsigned char*>(pl.codes);
        q.codes_seg_stride = pl.codes_seg_stride;
        q.side = static_cast<unsigned char*>(pl.side);
        q.side_seg_stride = pl.side_seg_stride;
        q.residual = static_cast<float*>(src[i].residual);
        q.residual_seg_elems = src[i].residual_seg_stride / 4;
        if (pl.kind == PITCH_PLANE_TURBO) {
            std::lock_guard<std::mutex> guardb(g_books.lock);
            const int l = log2_exact(dim);
            if (!g_books.present[l][pl.bits])
                return fail(PITCH_ERR_INVALID_INPUT, "no TurboQuant codebook for dim %d, bits %d", dim, pl.bits);
            memcpy(p.book[i], g_books.values[l][pl.bits], sizeof(float) << pl.bits);
        }
    }
    const dim3 grid((unsigned)d->segments, (unsigned)d->n_planes);
    const unsigned threads = dim < APPEND_MIN_THREADS ? APPEND_MIN_THREADS : dim;
    // programmatic dependent launch: the grid may be scheduled while the previous kernel of the stream
    // drains; it waits for that kernel before it touches memory (first statement of the kernel)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.stream = s;
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = pdl;
    cfg.numAttrs = 1;
    PITCH_DISPATCH_DTYPE(in_dtype, (cudaLaunchKernelEx(&cfg, cache_append_kernel<T>, p)));
    return launch_status(true, "cache_append");
}

// ------------------------------------------------------------------ append without allocations
// Residual scratch of pitch_enqueue_cache_append_noalloc: lives in the library image, so every
// GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) float g_noalloc_residual[PITCH_NOALLOC_RESIDUAL_FLOATS];

namespace {
struct NoallocDevice {
    float* base = nullptr;        // device address of g_noalloc_residual on this GPU
    const void* owner = nullptr;  // codes pointer of plane 0 of the cache whose newest group is held
    int64_t tokens = -1;          // tokens that cache held after its last call
};
std::mutex g_noalloc_lock;
NoallocDevice g_noalloc[64];
}  // namespace

int pitch_enqueue_cache_append_noalloc(const pitch_cache_desc* d, const pitch_append_src* src, int in_dtype,
                                       int64_t n_new, void* stream) {
    if (d == nullptr || src == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "descriptor is null");
    if (d->n_planes < 1 || d->n_planes > 4) return fail(PITCH_ERR_INVALID_INPUT, "n_planes %d must be in 1...4", d->n_planes);
    if (d->segments < 1 || d->tokens < 0) return fail(PITCH_ERR_INVALID_INPUT, "segments must be at least 1 and tokens not negative");
    if (d->planes[0].codes == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "plane 0: null pointer");
    // how much of the static array this cache needs, and whether every per-channel plane starts a new group
    int64_t need = 0;
    bool fresh_group = true;
    for (int i = 0; i < d->n_planes; ++i) {
        const pitch_plane& pl = d->planes[i];
        if (pl.kind != PITCH_PLANE_CHANNEL) continue;
        if (pl.group_size < 1 || d->dim < 1) return fail(PITCH_ERR_INVALID_INPUT, "plane %d: bad group size or dimension", i);
        need += d->segments * ((int64_t)pl.group_size + 2) * d->dim;
        if (d->tokens % pl.group_size != 0) fresh_group = false;
    }
    if (need > (int64_t)PITCH_NOALLOC_RESIDUAL_FLOATS)
        return fail(PITCH_ERR_INVALID_INPUT,
                    "the per-channel planes need %lld floats of residual; the built-in buffer holds %lld "
                    "(segments * (group_size + 2) * dim per plane): use pitch_enqueue_cache_append with your own buffer",
                    (long long)need, (long long)PITCH_NOALLOC_RESIDUAL_FLOATS);
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, d->planes[0].codes) != cudaSuccess ||
        (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)) {
        cudaGetLastError();
        return fail(PITCH_ERR_INVALID_INPUT, "plane 0: codes is not device memory");
    }
    const int dev = attr.device;
    if (dev < 0 || dev >= 64) return fail(PITCH_ERR_DEVICE_NOT_SUPPORTED, "device ordinal %d is out of range", dev);
    DeviceGuard guard(dev);
    float* base;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_lock);
        NoallocDevice& nd = g_noalloc[dev];
        if (nd.base == nullptr) {
            // once per GPU, with that GPU current: the array's name is only a host-side handle
            float* ptr = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_residual);
            if (e != cudaSuccess || ptr == nullptr) {
                cudaGetLastError();
                return fail(PITCH_ERR_KERNEL_UNAVAILABLE, "cannot locate the built-in residual buffer on GPU %d: %s", dev,
                            cudaGetErrorString(e));
            }
            nd.base = ptr;
        }
        if (!fresh_group && (nd.owner != d->planes[0].codes || nd.tokens != d->tokens))
            return fail(PITCH_ERR_CONFIGURATION_MISMATCH,
                        "the built-in residual buffer does not hold the newest group of this cache at %lld tokens "
                        "(it serves one cache at a time; switch caches only on a group boundary)", (long long)d->tokens);
        base = nd.base;
    }
    pitch_append_src mine[4];
    int64_t at_float = 0;
    for (int i = 0; i < d->n_planes; ++i) {
        mine[i] = src[i];
        mine[i].residual = nullptr;
        mine[i].residual_seg_stride = 0;
        if (d->planes[i].kind == PITCH_PLANE_CHANNEL) {
            const int64_t seg_floats = ((int64_t)d->planes[i].group_size + 2) * d->dim;
            mine[i].residual = base + at_float;
            mine[i].residual_seg_stride = seg_floats * 4;
            at_float += d->segments * seg_floats;
        }
    }
    const int st = pitch_enqueue_cache_append(d, mine, in_dtype, n_new, stream);
    if (st == PITCH_OK) {
        std::lock_guard<std::mutex> lock(g_noalloc_lock);
        g_noalloc[dev].owner = d->planes[0].codes;
        g_noalloc[dev].tokens = d->tokens + n_new;
    }
    return st;
}

// -------------------------------------------------------------------------------- attention
// How a segment's tokens are cut into runs (one warp each).  Depends on the shape only, so that
// the workspace size can be computed ahead of the call: runs of whole 32-token tiles, about one
// run per warp that a 148-SM GPU keeps resident (16 per SM), at least 4 tiles long.
static void attention_slices(int64_t segments, int64_t tokens, int* splits, int* tokens_per_split) {
    const int64_t tiles = ceil_div(tokens, 32), slots = 148 * 16;
    int64_t run = ceil_div(segments * tiles, slots);
    if (run < 4) run = 4;
    // rounding the runs per segment up must not push the total past the resident warps: a few
    // left-over runs would cost a whole second round
    while (run < tiles && segments * ceil_div(tiles, run) > slots && segments <= slots) ++run;
    if (run > tiles) run = tiles;
    *tokens_per_split = (int)(run * 32);
    *splits = (int)ceil_div(tiles, run);
}

static int check_attention_shape(const pitch_cache_desc* d, int n_queries) {
    if (d == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "descriptor is null");
    if (n_queries < 1 || n_queries > AT_MAX_QUERIES)
        return fail(PITCH_ERR_INVALID_INPUT, "n_queries %d must be in 1...%d", n_queries, AT_MAX_QUERIES);
    if (d->segments < 1 || d->segments > 65535 || d->tokens < 1 || d->tokens > 0x7FFFFFFF - 1024)
        return fail(PITCH_ERR_INVALID_INPUT, "segments must be in 1...65535 and tokens in 1...2^31-1025");
    if (d->dim != 64 || d->n_planes != 2)
        return fail(PITCH_ERR_INVALID_INPUT, "cache attention needs dim 64 and two planes (keys, values)");
    const pitch_plane& k = d->planes[0];
    const pitch_plane& v = d->planes[1];
    if (k.kind != PITCH_PLANE_CHANNEL || k.bits != 4 || k.group_size < 32 || k.group_size % 32 != 0 || k.group_size > PITCH_MAX_GROUP)
        return fail(PITCH_ERR_INVALID_INPUT, "cache attention needs per-channel 4-bit keys with a group size that is a multiple of 32");
    if (v.kind != PITCH_PLANE_TURBO || v.bits != 4)
        return fail(PITCH_ERR_INVALID_INPUT, "cache attention needs TurboQuant 4-bit values");
    return PITCH_OK;
}

int64_t pitch_cache_attention_workspace(const pitch_cache_desc* d, int n_queries) {
    if (check_attention_shape(d, n_queries)) return -1;
    int splits, tps;
    attention_slices(d->segments, d->tokens, &splits, &tps);
    return d->segments * splits * n_queries * AT_PART_FLOATS * (int64_t)sizeof(float);
}

int pitch_enqueue_cache_attention(const pitch_cache_desc* d, const pitch_attention_args* a, void* stream) {
    if (a == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "arguments are null");
    int st;
    if ((st = check_attention_shape(d, a->n_queries))) return st;
    if (!(a->scale > 0.0f) || !std::isfinite(a->scale)) return fail(PITCH_ERR_INVALID_INPUT, "scale must be positive and finite");
    if (!a->queries || !a->out || !a->workspace) return fail(PITCH_ERR_INVALID_INPUT, "queries, out or workspace is null");
    if (!aligned16(a->queries) || !aligned16(a->out) || !aligned16(a->workspace))
        return fail(PITCH_ERR_INVALID_INPUT, "queries, out and workspace must be 16-byte aligned");
    const int64_t need = pitch_cache_attention_workspace(d, a->n_queries);
    if (a->workspace_bytes < need)
        return fail(PITCH_ERR_INVALID_INPUT, "workspace has %lld bytes; needs %lld", (long long)a->workspace_bytes, (long long)need);
    for (int i = 0; i < 2; ++i) {
        const pitch_plane& pl = d->planes[i];
        if (!pl.codes || !pl.side) return fail(PITCH_ERR_INVALID_INPUT, "plane %d: null pointer", i);
        if (!aligned16(pl.codes) || !aligned16(pl.side) || (pl.codes_seg_stride & 15) || (pl.side_seg_stride & 15))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: pointers and segment strides must be multiples of 16", i);
        if (d->segments > 1 && (pl.codes_seg_stride < d->tokens * 32 || pl.side_seg_stride < plane_side_bytes(pl, 64, d->tokens)))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: a segment stride is smaller than one segment", i);
    }
    const pitch_buffer bufs[5] = {{const_cast<void*>(a->queries), 0, 0}, {a->out, 0, 0}, {a->workspace, 0, 0},
                                  {d->planes[0].codes, 0, 0}, {d->planes[1].codes, 0, 0}};
    const char* const names[5] = {"queries", "out", "workspace", "key codes", "value codes"};
    int dev;
    if ((st = check_same_device(bufs, names, 5, &dev))) return st;
    DeviceGuard guard(dev);

    AttentionParams p;
    memset(&p, 0, sizeof p);
    p.segments = (int)d->segments;
    p.tokens = (int)d->tokens;
    attention_slices(d->segments, d->tokens, &p.splits, &p.tokens_per_split);
    if ((int64_t)p.segments * p.splits > 0x7FFFFFFF) return fail(PITCH_ERR_INVALID_INPUT, "segments x runs exceeds 2^31 - 1");
    p.n_queries = a->n_queries;
    p.group_size = d->planes[0].group_size;
    p.scale_log2 = (float)((double)a->scale * 1.4426950408889634);
    p.neg_lo = negate_mask32(d->planes[1].seed, 0);
    p.neg_hi = negate_mask32(d->planes[1].seed, 32);
    p.k_codes = static_cast<const unsigned char*>(d->planes[0].codes);
    p.k_codes_seg = d->planes[0].codes_seg_stride;
    p.k_ranges = static_cast<const unsigned char*>(d->planes[0].side);
    p.k_ranges_seg = d->planes[0].side_seg_stride;
    p.v_codes = static_cast<const unsigned char*>(d->planes[1].codes);
    p.v_codes_seg = d->planes[1].codes_seg_stride;
    p.v_norms = static_cast<const unsigned char*>(d->planes[1].side);
    p.v_norms_seg = d->planes[1].side_seg_stride;
    p.q = static_cast<const float*>(a->queries);
    p.work = static_cast<float*>(a->workspace);
    p.out = static_cast<float*>(a->out);
    {
        std::lock_guard<std::mutex> guardb(g_books.lock);
        if (!g_books.present[6][4]) return fail(PITCH_ERR_INVALID_INPUT, "no TurboQuant codebook for dim 64, bits 4");
        memcpy(p.book.c, g_books.values[6][4], sizeof(float) * 16);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    {
        static std::atomic<bool> configured[64];
        if (dev >= 0 && dev < 64 && !configured[dev].load(std::memory_order_acquire)) {
            if (cudaFuncSetAttribute(attention_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES) != cudaSuccess)
                return launch_status(false, "cache_attention (shared memory opt-in)");
            configured[dev].store(true, std::memory_order_release);
        }
        // one CTA of sixteen warps per SM; a warp takes runs warp, warp + all warps, ...
        int64_t ctas = ceil_div((int64_t)p.segments * p.splits, AT_WARPS);
        if (ctas > sm_count()) ctas = sm_count();
        // Both launches are programmatic dependent launches: each grid may be scheduled while the
        // kernel before it in the stream is still running, sets itself up, then waits for that
        // kernel to complete before it reads what it wrote.
        cudaLaunchAttribute pdl[1];
        pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        pdl[0].val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)ctas);
        cfg.blockDim = dim3(AT_THREADS);
        cfg.dynamicSmemBytes = AT_SMEM_BYTES;
        cfg.stream = s;
        cfg.attrs = pdl;
        cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, attention_partial_kernel, p);
        if ((st = launch_status(false, "cache_attention"))) return st;
        cfg.gridDim = dim3((unsigned)p.n_queries, (unsigned)p.segments);
        cfg.blockDim = dim3(32 * AT_COMBINE_WARPS);
        cfg.dynamicSmemBytes = 0;
        cudaLaunchKernelEx(&cfg, attention_combine_kernel, p);
    }
    return launch_status(false, "cache_attention (combine)");
}

// ------------------------------------------------------------------------- key-bias removal
int pitch_enqueue_rope_bias(int dim, int dtype, int subtract, void* data, int64_t data_seg_stride, int64_t segments,
                            int64_t first_position, int64_t count, const pitch_rope_bias* rope, void* stream) {
    if (dim < 8 || dim > PITCH_MAX_DIM || (dim & 7)) return fail(PITCH_ERR_INVALID_DIMENSION, "dimension %d must be a multiple of 8 in 8...%d", dim, PITCH_MAX_DIM);
    if (dtype < PITCH_F32 || dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", dtype);
    if (rope == nullptr || data == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "data or rope description is null");
    if (!rope->bias || !rope->cos_table || !rope->sin_table) return fail(PITCH_ERR_INVALID_INPUT, "bias or rotary tables are null");
    if (segments < 1 || segments > 65535) return fail(PITCH_ERR_INVALID_INPUT, "segments must be in 1...65535");
    if (count < 0 || first_position < 0 || first_position + count > rope->positions)
        return fail(PITCH_ERR_INVALID_INPUT, "positions %lld...%lld are outside the rotary tables (%lld rows)",
                    (long long)first_position, (long long)(first_position + count), (long long)rope->positions);
    if (!aligned16(data) || (data_seg_stride & 15) || !aligned16(rope->cos_table) || !aligned16(rope->sin_table) ||
        (rope->bias_seg_stride & 3) || (reinterpret_cast<uintptr_t>(rope->bias) & 3))
        return fail(PITCH_ERR_INVALID_INPUT, "data and tables must be 16-byte aligned, strides multiples of 16 (data) and 4 (bias)");
    if (segments > 1 && data_seg_stride < count * dim * elem_size(dtype))
        return fail(PITCH_ERR_INVALID_INPUT, "data segment stride is smaller than one segment");
    const pitch_buffer bufs[4] = {{data, 0, 0}, {const_cast<float*>(rope->bias), 0, 0}, {const_cast<float*>(rope->cos_table), 0, 0},
                                  {const_cast<float*>(rope->sin_table), 0, 0}};
    const char* const names[4] = {"data", "bias", "cos table", "sin table"};
    int dev, st;
    if ((st = check_same_device(bufs, names, 4, &dev))) return st;
    if (count == 0) return PITCH_OK;
    DeviceGuard guard(dev);
    const int seg_tile = rope_bias_seg_tile(dim, segments);
    const int64_t tiles = ceil_div(segments, seg_tile);
    const int64_t chunks = count * dim * elem_size(dtype) / 16;
    int64_t blocks = ceil_div(chunks, RB_THREADS);
    if (blocks > 0x7FFFFFFF) blocks = 0x7FFFFFFF;                             // the kernel strides over what is left
    if (tiles > 65535) return fail(PITCH_ERR_INVALID_INPUT, "too many segments for dimension %d", dim);
    const dim3 grid((unsigned)blocks, (unsigned)tiles);
    const size_t smem = 2 * (size_t)dim * sizeof(float) * seg_tile;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PITCH_DISPATCH_DTYPE(dtype, (rope_bias_kernel<T><<<grid, RB_THREADS, smem, s>>>(
        static_cast<unsigned char*>(data), data_seg_stride, reinterpret_cast<const unsigned char*>(rope->bias),
        rope->bias_seg_stride, rope->cos_table, rope->sin_table, dim, segments, seg_tile, first_position, count, subtract)));
    return launch_status(subtract != 0, "rope_bias");
}

// --------------------------------------------------------------------------------- checksum
int pitch_enqueue_checksum(pitch_buffer buf, int64_t bytes, uint64_t* result_device, void* stream) {
    if (bytes < 0 || (bytes & 3)) return fail(PITCH_ERR_INVALID_INPUT, "bytes %lld must be a non-negative multiple of 4", (long long)bytes);
    if (result_device == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "result pointer is null");
    int st;
    if ((st = check_buffer(buf, bytes, "buffer"))) return st;
    const pitch_buffer bufs[1] = {buf};
    const char* const names[1] = {"buffer"};
    int dev;
    if ((st = check_same_device(bufs, names, 1, &dev))) return st;
    if (bytes == 0) return PITCH_OK;
    DeviceGuard guard(dev);
    const int64_t n = bytes / 4;
    int64_t blocks = ceil_div(n, 256 * 8);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    checksum_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint32_t*>(at(buf)), n, reinterpret_cast<unsigned long long*>(result_device));
    return launch_status(false, "checksum");
}

}  // extern "C"
