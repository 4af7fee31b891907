// C ABI, per-channel key codec: pitch_enqueue_channel_encode / _decode.
// Declarations and the reference interfaces they replace: include/pitch_b200.h.
#include "abi_internal.h"

#include "channel_kernels.cuh"
#include "common.cuh"

using namespace pitch;
using namespace pitch_abi;

namespace {

// slab mapping applies when dim/8 is a power of two in 1...32 and the buffers allow 16-byte access
bool slab_ok(int dim, int bits) {
    if (bits != 2 && bits != 4 && bits != 8) return false;
    if (dim % 8 != 0) return false;
    const int slabs = dim / 8;
    return slabs <= 32 && (slabs & (slabs - 1)) == 0;
}

}  // namespace

extern "C" {

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
        if ((st = cache64_single_plane(PITCH_PLANE_CHANNEL, dim, 4, group_size, 0, dtype, at(codes), at(ranges), at(output), count, s)))
            return st;
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

}  // extern "C"
