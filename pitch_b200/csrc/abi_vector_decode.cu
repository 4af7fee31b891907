// C ABI, per-vector decoders (TurboQuant, PolarQuant variant): pitch_enqueue_decode.
// Declarations and the reference interfaces they replace: include/pitch_b200.h.
#include "abi_internal.h"

#include <cstring>
#include <type_traits>

#include "common.cuh"
#include "vector_kernels.cuh"

using namespace pitch;
using namespace pitch_abi;

namespace {

template <int BITS>
bool fetch_book(int dim, Codebook<BITS>& out) { return book_get(dim, BITS, out.c); }

template <int BITS, typename T>
int launch_turbo_decode(int dim, uint32_t seed, const void* codes, const void* scales, void* out, int64_t count,
                        cudaStream_t s) {
    Codebook<BITS> book;
    if (!fetch_book<BITS>(dim, book))
        return fail(PITCH_ERR_INVALID_INPUT, "no TurboQuant codebook for dim %d, bits %d", dim, BITS);
    if ((BITS == 4 || BITS == 3) && (dim == 64 || dim == 128) && aligned16(codes) && aligned16(out) &&
        count / (2048 / dim) <= 0x3FFFFFFF) {
        // the persistent whole-cache kernel with a single TurboQuant plane
        return cache64_single_plane(PITCH_PLANE_TURBO, dim, BITS, 0, seed, std::is_same<T, float>::value ? PITCH_F32 :
                                    (std::is_same<T, __half>::value ? PITCH_F16 : PITCH_BF16), codes, scales, out, count, s);
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

}  // namespace

extern "C" {

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

}  // extern "C"
