// Host-side helpers shared by the translation units of the C ABI (abi_*.cu): status reporting,
// the buffer checks of Codec.check (Sources/PITCH/Core/Codec.swift:37-47), configuration checks
// of QuantConfig.init / ChannelQuantConfig.init (Sources/PITCH/Models/QuantConfig.swift:24-35,
// Sources/PITCH/PerChannel.swift:30-43), the host-side codebook table and launch plumbing.
// Definitions live in abi_core.cu unless noted.
#pragma once

#include "../../include/pitch_b200.h"

#include <cuda_runtime.h>
#include <stdint.h>

#include <cmath>

namespace pitch {
struct Cache64Params;
}

namespace pitch_abi {

// Records the detail of a failure for pitch_last_error() on this thread and returns `status`.
int fail(int status, const char* fmt, ...);

// Copies the 2^bits centroids registered for (dim, bits) into `out`; false when there are none.
bool book_get(int dim, int bits, float* out);

int check_buffer(const pitch_buffer& b, int64_t needs, const char* name);
// All buffers of a call must be device-accessible memory of one GPU ("belongs to a different
// MTLDevice", Codec.swift:38-40).  Returns that GPU's ordinal in *device.
int check_same_device(const pitch_buffer* bufs, const char* const* names, int n, int* device);
int check_vector_config(int method, int dim, int bits, int dtype);
int check_channel_config(int dim, int bits, int group_size, int dtype);
// Status of the launch just made on this thread (cudaGetLastError), as a pitch_status.
int launch_status(bool encode, const char* what);
// Multiprocessors of the current device (cached per device).
int sm_count();

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev); else prev = -1;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

inline int log2_exact(int v) {
    int l = 0;
    while ((1 << l) < v) ++l;
    return l;
}
inline bool valid_vector_dim(int dim) { return dim >= 2 && dim <= PITCH_MAX_DIM && (dim & (dim - 1)) == 0; }
inline bool valid_bits(int bits) { return bits >= PITCH_MIN_BITS && bits <= PITCH_MAX_BITS; }
inline unsigned char* at(const pitch_buffer& b) { return static_cast<unsigned char*>(b.base) + b.offset; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline float rsqrt_dim(int dim) { return (float)(1.0 / std::sqrt((double)dim)); }
inline int elem_size(int dtype) { return dtype == PITCH_F32 ? 4 : 2; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Grid of the per-vector kernels: one warp tile of 32 x min(dim, 32) coordinates per warp, 4 warps per CTA.
unsigned vec_grid(int64_t count, int dim);
// Grid of a kernel whose CTAs loop over warp tiles: enough CTAs for every SM's registers, no more.
unsigned vec_grid_looping(int64_t count, int dim);

// The persistent whole-cache kernel run over a single plane of a single segment (abi_cache.cu): the
// fast path of the stand-alone TurboQuant and per-channel decoders at dim 64 / 128.
// kind: PITCH_PLANE_TURBO (bits 3 or 4) or PITCH_PLANE_CHANNEL (bits 4, group_size a multiple of 2048/dim).
int cache64_single_plane(int kind, int dim, int bits, int group_size, uint32_t seed, int dtype, const void* codes,
                         const void* side, void* out, int64_t count, cudaStream_t s);

// The same kernel family with exact key-bias removal on plane 0 (abi_cache_bias.cu); `p` carries the
// bias row pointer and the rotary tables.  dim in {64, 128}, bits (of the TurboQuant planes) in {3, 4}.
int launch_cache64_bias(const pitch::Cache64Params& p, int dim, int bits, int dtype, int64_t tokens_for_grid, cudaStream_t s);
// The whole-cache launch with its items dealt by drawn tickets (cache_decode_kernel<..., true>): abi_cache_tickets.cu.
int launch_cache64_tickets(const pitch::Cache64Params& p, int dim, int bits, int dtype, int64_t tokens_for_grid, cudaStream_t s);
int launch_cache64_tickets_ahead(const pitch::Cache64Params& p, int dim, int bits, int dtype, int64_t tokens_for_grid, cudaStream_t s);

}  // namespace pitch_abi

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
