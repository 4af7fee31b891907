// C ABI, common part: status reporting, the host-side codebook table, buffer and configuration
// checks, and the small entry points (rotation, pack / unpack, key-bias pass, checksum).
// Declarations and the reference interfaces they replace: include/pitch_b200.h.
//
// Validation mirrors Codec.params / Codec.check (Sources/PITCH/Core/Codec.swift:28-47) and
// ChannelCodec.params / check (Sources/PITCH/PerChannel.swift:308-329), QuantConfig.init
// (Sources/PITCH/Models/QuantConfig.swift:24-35) and ChannelQuantConfig.init
// (Sources/PITCH/PerChannel.swift:30-43).  Nothing here allocates device memory.
#include "abi_internal.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "bias_kernels.cuh"
#include "common.cuh"
#include "vector_kernels.cuh"

using namespace pitch;

namespace {

thread_local std::string g_error;

// ---- host-side codebook table (TurboCodebooks.codebook(dim:bits:)) --------------------------
struct BookTable {
    std::mutex lock;
    bool present[11][9] = {};
    float values[11][9][256];
} g_books;

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

namespace pitch_abi {

int fail(int status, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
    return status;
}

bool book_get(int dim, int bits, float* out) {
    if (!valid_vector_dim(dim) || !valid_bits(bits)) return false;
    std::lock_guard<std::mutex> guard(g_books.lock);
    const int l = log2_exact(dim);
    if (!g_books.present[l][bits]) return false;
    memcpy(out, g_books.values[l][bits], sizeof(float) << bits);
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

int launch_status(bool encode, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return PITCH_OK;
    if (e == cudaErrorNoKernelImageForDevice || e == cudaErrorInvalidDeviceFunction)
        return fail(PITCH_ERR_KERNEL_UNAVAILABLE, "%s: %s (library is built for sm_100a)", what, cudaGetErrorString(e));
    return fail(encode ? PITCH_ERR_ENCODING_FAILED : PITCH_ERR_DECODING_FAILED, "%s: %s", what, cudaGetErrorString(e));
}

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

unsigned vec_grid(int64_t count, int dim) {
    const int vpw = dim < 32 ? 32 : 1024 / dim;
    return (unsigned)ceil_div(ceil_div(count, vpw), VEC_WARPS);
}

unsigned vec_grid_looping(int64_t count, int dim) {
    const unsigned all = vec_grid(count, dim), cap = (unsigned)sm_count() * 8u;
    return all < cap ? all : cap;
}

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

}  // namespace pitch_abi

using namespace pitch_abi;

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
