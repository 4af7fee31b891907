// C ABI, whole-cache entry points: pitch_enqueue_cache_decode / _append / _step / _append_noalloc.
// Declarations and the reference interfaces they replace: include/pitch_b200.h.
//
// Validation follows Codec.check (Sources/PITCH/Core/Codec.swift:37-47): every buffer must be
// device memory of one GPU and long enough for what the call addresses.  The arithmetic part
// (sizes, strides, alignment) runs on every call; the queries that ask the driver which GPU a
// pointer belongs to are remembered per set of pointers, so the per-token path asks only about the
// pointers that change from step to step (the new tokens).  Nothing here allocates device memory.
#include "abi_internal.h"

#include <atomic>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "append_kernels.cuh"
#include "cache_kernels.cuh"
#include "common.cuh"

using namespace pitch;
using namespace pitch_abi;

namespace {

int64_t plane_side_bytes(const pitch_plane& pl, int dim, int64_t tokens) {
    if (pl.kind == PITCH_PLANE_CHANNEL) return ceil_div(tokens, pl.group_size) * 4 * dim;
    return tokens * 4;
}

// ---- which GPU a set of pointers lives on, remembered --------------------------------------------
// (device addresses are unique across the GPUs of a process, so a remembered answer stays right
// for as long as the same pointers are passed)
struct PointerSet {
    const void* p[24];
    int n = 0;
    void add(const void* q) { if (q != nullptr && n < 24) p[n++] = q; }
};

struct CheckedPointers {
    static const int SLOTS = 16;
    std::mutex lock;
    PointerSet key[SLOTS];
    int device[SLOTS];
    int used = 0, next = 0;

    bool find(const PointerSet& k, int* dev) {
        std::lock_guard<std::mutex> guard(lock);
        for (int i = 0; i < used; ++i)
            if (key[i].n == k.n && memcmp(key[i].p, k.p, sizeof(void*) * k.n) == 0) {
                *dev = device[i];
                return true;
            }
        return false;
    }
    void store(const PointerSet& k, int dev) {
        std::lock_guard<std::mutex> guard(lock);
        const int slot = used < SLOTS ? used++ : (next++ % SLOTS);
        key[slot] = k;
        device[slot] = dev;
    }
} g_checked;

// Asks the driver about one pointer: device (or managed) memory, and of which GPU.
int pointer_device(const void* ptr, const char* what, int plane, int* dev) {
    cudaPointerAttributes attr;
    const cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver)
            return fail(PITCH_ERR_DEVICE_NOT_SUPPORTED, "no usable CUDA device: %s", cudaGetErrorString(e));
        return fail(PITCH_ERR_INVALID_INPUT, "plane %d: %s: %s", plane, what, cudaGetErrorString(e));
    }
    if (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)
        return fail(PITCH_ERR_INVALID_INPUT, "plane %d: %s is not device memory", plane, what);
    if (attr.type == cudaMemoryTypeDevice) {
        if (*dev >= 0 && attr.device != *dev)
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: %s belongs to a different GPU", plane, what);
        *dev = attr.device;
    }
    return PITCH_OK;
}

struct DescNeeds {
    int64_t tokens;      // tokens per segment the call addresses (after an append)
    bool out;            // the planes' out buffers are used
    int align;           // required alignment of pointers and segment strides (16: vector paths, 4: append)
    int value_dtype;     // element type the plane configurations are checked with
};

// Shape, alignment and extent of every plane (the arithmetic half of Codec.check).
int check_desc_shape(const pitch_cache_desc* d, const DescNeeds& need) {
    if (d == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "descriptor is null");
    if (d->n_planes < 1 || d->n_planes > 4) return fail(PITCH_ERR_INVALID_INPUT, "n_planes %d must be in 1...4", d->n_planes);
    if (d->segments < 1) return fail(PITCH_ERR_INVALID_INPUT, "segments must be at least 1");
    if (d->capacity < 0) return fail(PITCH_ERR_INVALID_INPUT, "capacity must not be negative");
    if (d->capacity > 0 && need.tokens > d->capacity)
        return fail(PITCH_ERR_INVALID_INPUT, "the call addresses %lld tokens per segment; the cache was sized for %lld",
                    (long long)need.tokens, (long long)d->capacity);
    const int64_t sized = d->capacity > 0 ? d->capacity : need.tokens;      // tokens the extents must cover
    const int dim = d->dim;
    const uintptr_t mask = (uintptr_t)need.align - 1;
    for (int i = 0; i < d->n_planes; ++i) {
        const pitch_plane& pl = d->planes[i];
        int st;
        if (pl.kind == PITCH_PLANE_CHANNEL) {
            if ((st = check_channel_config(dim, pl.bits, pl.group_size, need.value_dtype))) return st;
        } else if (pl.kind == PITCH_PLANE_TURBO || pl.kind == PITCH_PLANE_POLAR) {
            if ((st = check_vector_config(pl.kind, dim, pl.bits, need.value_dtype))) return st;
        } else {
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: unknown kind %d", i, pl.kind);
        }
        if (!pl.codes || !pl.side || (need.out && !pl.out)) return fail(PITCH_ERR_INVALID_INPUT, "plane %d: null pointer", i);
        if ((reinterpret_cast<uintptr_t>(pl.codes) & mask) || (reinterpret_cast<uintptr_t>(pl.side) & mask) ||
            (need.out && (reinterpret_cast<uintptr_t>(pl.out) & mask)) || (pl.codes_seg_stride & mask) ||
            (pl.side_seg_stride & mask) || (need.out && (pl.out_seg_stride & mask)))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: pointers and segment strides must be multiples of %d", i, need.align);
        const int64_t code_need = sized * pitch_code_stride(dim, pl.bits);
        const int64_t side_need = plane_side_bytes(pl, dim, sized);
        const int64_t out_need = sized * dim * elem_size(d->out_dtype);
        if (d->segments > 1 && (pl.codes_seg_stride < code_need || pl.side_seg_stride < side_need ||
                                (need.out && pl.out_seg_stride < out_need)))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: a segment stride is smaller than one segment of %lld tokens", i,
                        (long long)sized);
        const int64_t last = d->segments - 1;
        if (pl.codes_bytes < last * pl.codes_seg_stride + code_need)
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: codes buffer has %lld bytes; needs %lld", i, (long long)pl.codes_bytes,
                        (long long)(last * pl.codes_seg_stride + code_need));
        if (pl.side_bytes < last * pl.side_seg_stride + side_need)
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: side-information buffer has %lld bytes; needs %lld", i,
                        (long long)pl.side_bytes, (long long)(last * pl.side_seg_stride + side_need));
        if (need.out && pl.out_bytes < last * pl.out_seg_stride + out_need)
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: output buffer has %lld bytes; needs %lld", i, (long long)pl.out_bytes,
                        (long long)(last * pl.out_seg_stride + out_need));
    }
    if (d->key_bias != nullptr) {
        const pitch_rope_bias& r = *d->key_bias;
        if (!r.bias || !r.cos_table || !r.sin_table) return fail(PITCH_ERR_INVALID_INPUT, "key bias: bias or rotary tables are null");
        if (dim < 8 || (dim & 7)) return fail(PITCH_ERR_INVALID_DIMENSION, "key bias: dimension %d must be a multiple of 8", dim);
        if (r.positions < sized)
            return fail(PITCH_ERR_INVALID_INPUT, "key bias: the rotary tables hold %lld positions; the cache addresses %lld",
                        (long long)r.positions, (long long)sized);
        if (!aligned16(r.cos_table) || !aligned16(r.sin_table) || (reinterpret_cast<uintptr_t>(r.bias) & 3) || (r.bias_seg_stride & 3))
            return fail(PITCH_ERR_INVALID_INPUT, "key bias: tables must be 16-byte aligned, bias and its stride multiples of 4");
    }
    return PITCH_OK;
}

// The other half of Codec.check: all buffers are device memory of one GPU (returned in *device).
// `extra` are further pointers of the call that stay the same from step to step (residual buffers).
int check_desc_device(const pitch_cache_desc* d, bool with_out, const PointerSet& extra, int* device) {
    PointerSet key;
    for (int i = 0; i < d->n_planes; ++i) {
        key.add(d->planes[i].codes);
        key.add(d->planes[i].side);
        if (with_out) key.add(d->planes[i].out);
    }
    if (d->key_bias != nullptr) {
        key.add(d->key_bias->bias);
        key.add(d->key_bias->cos_table);
        key.add(d->key_bias->sin_table);
    }
    for (int i = 0; i < extra.n; ++i) key.add(extra.p[i]);
    if (g_checked.find(key, device)) return PITCH_OK;
    int dev = -1, st, at = 0;
    for (int i = 0; i < d->n_planes; ++i) {
        if ((st = pointer_device(key.p[at++], "codes", i, &dev))) return st;
        if ((st = pointer_device(key.p[at++], "side information", i, &dev))) return st;
        if (with_out && (st = pointer_device(key.p[at++], "output", i, &dev))) return st;
    }
    for (; at < key.n; ++at)
        if ((st = pointer_device(key.p[at], "auxiliary buffer (key-bias tables, residual, token counter)", 0, &dev))) return st;
    if (dev < 0) cudaGetDevice(&dev);
    g_checked.store(key, dev);
    *device = dev;
    return PITCH_OK;
}

// The new tokens (and the residual buffers) of an append or a step.
int check_append_src(const pitch_cache_desc* d, const pitch_append_src* src, int in_dtype, int64_t n_new, int device,
                     PointerSet* residuals, int residual_align = 4) {
    if (src == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "source description is null");
    if (in_dtype < PITCH_F32 || in_dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", in_dtype);
    const int dim = d->dim;
    const int64_t last = d->segments - 1;
    for (int i = 0; i < d->n_planes; ++i) {
        const pitch_plane& pl = d->planes[i];
        if (!src[i].input) return fail(PITCH_ERR_INVALID_INPUT, "plane %d: null pointer", i);
        if ((reinterpret_cast<uintptr_t>(src[i].input) & 3) || (src[i].input_seg_stride & 3))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: pointers and strides must be multiples of 4", i);
        const int64_t in_need = n_new * dim * elem_size(in_dtype);
        if (d->segments > 1 && src[i].input_seg_stride < in_need)
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: input segment stride is smaller than the new tokens of a segment", i);
        if (src[i].input_bytes < last * src[i].input_seg_stride + in_need)
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: input buffer has %lld bytes; needs %lld", i, (long long)src[i].input_bytes,
                        (long long)(last * src[i].input_seg_stride + in_need));
        if (device >= 0) {
            int dev = device, st;
            if ((st = pointer_device(src[i].input, "input", i, &dev))) return st;
        }
        if (pl.kind == PITCH_PLANE_CHANNEL && residuals != nullptr) {
            if (src[i].residual == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "plane %d: residual buffer is null", i);
            const int64_t res_need = ((int64_t)pl.group_size + 2) * dim * 4;
            const uintptr_t rmask = (uintptr_t)residual_align - 1;
            if (src[i].residual_seg_stride < res_need || (src[i].residual_seg_stride & rmask) ||
                (reinterpret_cast<uintptr_t>(src[i].residual) & rmask))
                return fail(PITCH_ERR_INVALID_INPUT, "plane %d: residual needs %d-byte alignment and a segment stride of at least %lld bytes",
                            i, residual_align, (long long)res_need);
            if (src[i].residual_bytes < last * src[i].residual_seg_stride + res_need)
                return fail(PITCH_ERR_INVALID_INPUT, "plane %d: residual buffer has %lld bytes; needs %lld", i,
                            (long long)src[i].residual_bytes, (long long)(last * src[i].residual_seg_stride + res_need));
            residuals->add(src[i].residual);
        }
    }
    return PITCH_OK;
}

// ---- the persistent kernel ---------------------------------------------------------------------------
template <typename T, int D, int BITS>
int launch_cache64_impl(const Cache64Params& p, int64_t tokens_for_grid, cudaStream_t s) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    constexpr int smem = cache64_smem_bytes<T>();
    if (dev >= 0 && dev < 64 && !configured[dev].load(std::memory_order_acquire)) {
        // idempotent: two threads racing here both set the same attribute
        if (cudaFuncSetAttribute(cache_decode_kernel<T, D, BITS, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
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
    cudaLaunchKernelEx(&cfg, cache_decode_kernel<T, D, BITS, 0>, p);
    return PITCH_OK;
}

// dim in {64, 128}, bits (of the TurboQuant planes) in {3, 4}.  A cache that mixes per-channel and
// TurboQuant planes takes the kernel that deals its items by drawn tickets (instances in abi_cache_tickets.cu).
template <typename T>
int launch_cache64(const Cache64Params& p, int dim, int bits, int64_t tokens_for_grid, cudaStream_t s) {
    bool turbo = false, channel = false;
    for (int i = 0; i < p.n_planes; ++i) (p.plane[i].kind == 0 ? turbo : channel) = true;
    if (turbo && channel) return launch_cache64_tickets(p, dim, bits, std::is_same<T, float>::value ? PITCH_F32 : (std::is_same<T, __half>::value ? PITCH_F16 : PITCH_BF16), tokens_for_grid, s);
    if (dim == 64)
        return bits == 4 ? launch_cache64_impl<T, 64, 4>(p, tokens_for_grid, s) : launch_cache64_impl<T, 64, 3>(p, tokens_for_grid, s);
    return bits == 4 ? launch_cache64_impl<T, 128, 4>(p, tokens_for_grid, s) : launch_cache64_impl<T, 128, 3>(p, tokens_for_grid, s);
}

void cache64_signs(Plane64& q, uint32_t seed) {
    for (int j = 0; j < 4; ++j) q.neg[j] = negate_mask32(seed, 32u * j);
}

// Whether the persistent kernel covers this cache (otherwise: stand-alone launches per plane and
// segment).  Returns the width of the TurboQuant planes in *turbo_bits (4 when there are none).
bool fused_shape(const pitch_cache_desc* d, int64_t tokens, int* turbo_bits) {
    const int dim = d->dim;
    if (dim != 64 && dim != 128) return false;
    int tb = 0;
    for (int i = 0; i < d->n_planes; ++i) {
        const pitch_plane& pl = d->planes[i];
        if (pl.kind == PITCH_PLANE_POLAR) return false;
        if (pl.kind == PITCH_PLANE_CHANNEL && (pl.bits != 4 || pl.group_size % (2048 / dim) != 0)) return false;
        if (pl.kind == PITCH_PLANE_TURBO) {
            if (pl.bits != 3 && pl.bits != 4) return false;
            if (tb != 0 && tb != pl.bits) return false;
            tb = pl.bits;
        }
    }
    if (d->segments > 0x7FFFFFFF / (tokens / 16 + 2)) return false;          // 32-bit item indices in the kernel
    *turbo_bits = tb == 0 ? 4 : tb;
    return true;
}

// Fills the kernel parameters from a descriptor (planes, signs, codebook).
int fill_cache64(Cache64Params& p, const pitch_cache_desc* d, int turbo_bits) {
    memset(&p, 0, sizeof p);
    const int dim = d->dim;
    p.n_planes = d->n_planes;
    p.segments = (int)d->segments;
    p.tokens = d->tokens;
    p.capacity = d->capacity;
    p.rs = rsqrt_dim(dim);
    bool any_turbo = false;
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
        any_turbo |= q.kind == 0;
    }
    if (any_turbo && !book_get(dim, turbo_bits, p.book.c))
        return fail(PITCH_ERR_INVALID_INPUT, "no TurboQuant codebook for dim %d, bits %d", dim, turbo_bits);
    if (d->key_bias != nullptr) {
        p.bias = reinterpret_cast<const unsigned char*>(d->key_bias->bias);
        p.bias_seg_stride = d->key_bias->bias_seg_stride;
        p.cos_table = d->key_bias->cos_table;
        p.sin_table = d->key_bias->sin_table;
    }
    return PITCH_OK;
}

}  // namespace

namespace pitch_abi {

int cache64_single_plane(int kind, int dim, int bits, int group_size, uint32_t seed, int dtype, const void* codes,
                         const void* side, void* out, int64_t count, cudaStream_t s) {
    Cache64Params p;
    memset(&p, 0, sizeof p);
    p.n_planes = 1;
    p.segments = 1;
    p.tokens = count;
    p.rs = rsqrt_dim(dim);
    Plane64& q = p.plane[0];
    q.kind = kind == PITCH_PLANE_CHANNEL ? 1 : 0;
    q.group_items = kind == PITCH_PLANE_CHANNEL ? group_size / (2048 / dim) : 1;
    cache64_signs(q, seed);
    q.codes = static_cast<const unsigned char*>(codes);
    q.side = static_cast<const unsigned char*>(side);
    q.out = static_cast<unsigned char*>(out);
    const int turbo_bits = kind == PITCH_PLANE_CHANNEL ? 4 : bits;
    if (q.kind == 0 && !book_get(dim, turbo_bits, p.book.c))
        return fail(PITCH_ERR_INVALID_INPUT, "no TurboQuant codebook for dim %d, bits %d", dim, turbo_bits);
    int st = 0;
    PITCH_DISPATCH_DTYPE(dtype, st = (launch_cache64<T>(p, dim, turbo_bits, count, s)));
    return st;
}

}  // namespace pitch_abi

// =================================================================================================
extern "C" {

int pitch_enqueue_cache_decode(const pitch_cache_desc* d, void* stream) {
    if (d == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "descriptor is null");
    if (d->tokens < 1) return fail(PITCH_ERR_INVALID_INPUT, "segments and tokens must be at least 1");
    if (d->out_dtype < PITCH_F32 || d->out_dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", d->out_dtype);
    int st;
    if ((st = check_desc_shape(d, DescNeeds{d->tokens, true, 16, d->out_dtype}))) return st;
    int dev;
    if ((st = check_desc_device(d, true, PointerSet(), &dev))) return st;
    DeviceGuard guard(dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int dim = d->dim;

    int turbo_bits = 4;
    if (fused_shape(d, d->tokens, &turbo_bits)) {
        Cache64Params p;
        if ((st = fill_cache64(p, d, turbo_bits))) return st;
        if (d->key_bias != nullptr) {
            // the rotated key bias is added to plane 0 inside the launch
            if ((st = launch_cache64_bias(p, dim, turbo_bits, d->out_dtype, d->tokens, s))) return st;
            return launch_status(false, "cache_decode with key bias");
        }
        PITCH_DISPATCH_DTYPE(d->out_dtype, st = (launch_cache64<T>(p, dim, turbo_bits, d->tokens, s)));
        if (st) return st;
        if ((st = launch_status(false, "cache_decode"))) return st;
    } else {
        // Any other shape: one stand-alone decode per (plane, segment), same results.
        for (int i = 0; i < d->n_planes; ++i) {
            const pitch_plane& pl = d->planes[i];
            const int64_t stride = pitch_code_stride(dim, pl.bits);
            for (int64_t sgm = 0; sgm < d->segments; ++sgm) {
                pitch_buffer codes = {pl.codes, sgm * pl.codes_seg_stride + d->tokens * stride, sgm * pl.codes_seg_stride};
                pitch_buffer side = {pl.side, sgm * pl.side_seg_stride + plane_side_bytes(pl, dim, d->tokens), sgm * pl.side_seg_stride};
                pitch_buffer out = {pl.out, sgm * pl.out_seg_stride + d->tokens * dim * elem_size(d->out_dtype), sgm * pl.out_seg_stride};
                if (pl.kind == PITCH_PLANE_CHANNEL)
                    st = pitch_enqueue_channel_decode(dim, pl.bits, pl.group_size, d->out_dtype, codes, side, out, d->tokens, stream);
                else
                    st = pitch_enqueue_decode(pl.kind, dim, pl.bits, pl.seed, d->out_dtype, codes, side, out, d->tokens, stream);
                if (st) return st;
            }
        }
    }
    if (d->key_bias != nullptr) {
        // add the rotated key bias back to the decoded keys (plane 0)
        const pitch_plane& k = d->planes[0];
        return pitch_enqueue_rope_bias(dim, d->out_dtype, 0, k.out, k.out_seg_stride, d->segments, 0, d->tokens, d->key_bias, stream);
    }
    return PITCH_OK;
}

int pitch_enqueue_cache_append(const pitch_cache_desc* d, const pitch_append_src* src, int in_dtype, int64_t n_new,
                               void* stream) {
    if (d == nullptr || src == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "descriptor is null");
    if (d->segments < 1 || d->segments > 65535) return fail(PITCH_ERR_INVALID_INPUT, "segments must be in 1...65535");
    if (d->tokens < 0) return fail(PITCH_ERR_INVALID_INPUT, "tokens must not be negative");
    if (n_new < 1 || n_new > 65535) return fail(PITCH_ERR_INVALID_INPUT, "n_new must be in 1...65535");
    if (in_dtype < PITCH_F32 || in_dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", in_dtype);
    if (d->key_bias != nullptr)
        return fail(PITCH_ERR_INVALID_INPUT, "append with key-bias removal: remove the bias from the new keys with "
                                             "pitch_enqueue_rope_bias first, or use pitch_enqueue_cache_step");
    int st;
    if ((st = check_desc_shape(d, DescNeeds{d->tokens + n_new, false, 4, in_dtype}))) return st;
    const int dim = d->dim;
    for (int i = 0; i < d->n_planes; ++i) {
        const pitch_plane& pl = d->planes[i];
        if (pl.kind == PITCH_PLANE_CHANNEL && d->tokens % pl.group_size + n_new > pl.group_size)
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: new tokens must fall into one group of %d", i, pl.group_size);
    }
    PointerSet residuals;
    if ((st = check_append_src(d, src, in_dtype, n_new, -1, &residuals))) return st;
    int dev;
    if ((st = check_desc_device(d, false, residuals, &dev))) return st;
    if ((st = check_append_src(d, src, in_dtype, n_new, dev, nullptr))) return st;
    DeviceGuard guard(dev);
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
        if (pl.kind == PITCH_PLANE_TURBO && !book_get(dim, pl.bits, p.book[i]))
            return fail(PITCH_ERR_INVALID_INPUT, "no TurboQuant codebook for dim %d, bits %d", dim, pl.bits);
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

int pitch_enqueue_cache_step(const pitch_cache_desc* d, const pitch_append_src* src, int in_dtype, pitch_cache_state* state,
                             void* stream) {
    if (d == nullptr || src == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "descriptor is null");
    if (d->segments < 1 || d->segments > 65535) return fail(PITCH_ERR_INVALID_INPUT, "segments must be in 1...65535");
    if (d->out_dtype < PITCH_F32 || d->out_dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", d->out_dtype);
    if (in_dtype < PITCH_F32 || in_dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", in_dtype);
    if (state != nullptr && d->capacity < 1)
        return fail(PITCH_ERR_INVALID_INPUT, "a step with a device-side token counter needs desc->capacity");
    if (state != nullptr && (reinterpret_cast<uintptr_t>(state) & 15))
        return fail(PITCH_ERR_INVALID_INPUT, "the token counter must be 16-byte aligned");
    if (state == nullptr && d->tokens < 0) return fail(PITCH_ERR_INVALID_INPUT, "tokens must not be negative");
    const int64_t after = state != nullptr ? d->capacity : d->tokens + 1;      // tokens the buffers must hold
    int st;
    if ((st = check_desc_shape(d, DescNeeds{after, true, 16, d->out_dtype}))) return st;
    PointerSet residuals;
    if ((st = check_append_src(d, src, in_dtype, 1, -1, &residuals, 16))) return st;
    residuals.add(state);
    int dev;
    if ((st = check_desc_device(d, true, residuals, &dev))) return st;
    if ((st = check_append_src(d, src, in_dtype, 1, dev, nullptr))) return st;

    int turbo_bits = 4;
    const bool fused = fused_shape(d, after, &turbo_bits);
    if (!fused) {
        if (state != nullptr)
            return fail(PITCH_ERR_INVALID_INPUT, "a device-side token counter needs a cache shape the one-launch step covers "
                                                 "(dim 64 or 128; TurboQuant planes of 3 or 4 bits; per-channel planes of 4 bits)");
        // the same step as separate launches: [bias removal,] append, decode [+ bias]
        pitch_cache_desc now = *d;
        const pitch_rope_bias* bias = d->key_bias;
        now.key_bias = nullptr;
        if (bias != nullptr)
            return fail(PITCH_ERR_INVALID_INPUT, "a step with key-bias removal on this cache shape: subtract the bias with "
                                                 "pitch_enqueue_rope_bias, then append and decode");
        if ((st = pitch_enqueue_cache_append(&now, src, in_dtype, 1, stream))) return st;
        now.tokens = d->tokens + 1;
        return pitch_enqueue_cache_decode(&now, stream);
    }
    DeviceGuard guard(dev);
    Cache64Params p;
    if ((st = fill_cache64(p, d, turbo_bits))) return st;
    p.append = 1;
    p.in_dtype = in_dtype;
    p.state = reinterpret_cast<CacheState*>(state);
    for (int i = 0; i < d->n_planes; ++i) {
        p.step[i].in = static_cast<const unsigned char*>(src[i].input);
        p.step[i].in_seg_stride = src[i].input_seg_stride;
        p.step[i].residual = static_cast<float*>(src[i].residual);
        p.step[i].residual_seg_elems = src[i].residual_seg_stride / 4;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d->key_bias != nullptr) {
        if ((st = launch_cache64_bias(p, d->dim, turbo_bits, d->out_dtype, after, s))) return st;
        return launch_status(false, "cache_step with key bias");
    }
    PITCH_DISPATCH_DTYPE(d->out_dtype, st = (launch_cache64<T>(p, d->dim, turbo_bits, after, s)));
    if (st) return st;
    return launch_status(false, "cache_step");
}

int pitch_enqueue_cache_newest(const pitch_cache_desc* d, const pitch_cache_state* state, void* dst, int64_t dst_bytes, void* stream) {
    if (d == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "descriptor is null");
    if (d->out_dtype < PITCH_F32 || d->out_dtype > PITCH_BF16) return fail(PITCH_ERR_INVALID_INPUT, "unknown dtype %d", d->out_dtype);
    if (state != nullptr && d->capacity < 1)
        return fail(PITCH_ERR_INVALID_INPUT, "reading the newest token with a device-side token counter needs desc->capacity");
    if (state == nullptr && d->tokens < 1) return fail(PITCH_ERR_INVALID_INPUT, "the cache holds no token");
    const int64_t held = state != nullptr ? d->capacity : d->tokens;
    int st;
    if ((st = check_desc_shape(d, DescNeeds{held, true, 16, d->out_dtype}))) return st;
    if (d->segments > 0x7FFFFF) return fail(PITCH_ERR_INVALID_INPUT, "segments must be below 2^23");
    const int64_t row_bytes = (int64_t)d->dim * elem_size(d->out_dtype);
    if (row_bytes & 15) return fail(PITCH_ERR_INVALID_DIMENSION, "a token row of %lld bytes is not a multiple of 16", (long long)row_bytes);
    const int64_t need = d->n_planes * d->segments * row_bytes;
    if (dst == nullptr || !aligned16(dst)) return fail(PITCH_ERR_INVALID_INPUT, "destination must be a 16-byte aligned device pointer");
    if (dst_bytes < need)
        return fail(PITCH_ERR_INVALID_INPUT, "destination has %lld bytes; needs %lld", (long long)dst_bytes, (long long)need);
    if (need > 0x7FFFFFFF) return fail(PITCH_ERR_INVALID_INPUT, "more than 2^31 - 1 bytes of newest tokens");
    PointerSet extra;
    extra.add(dst);
    if (state != nullptr) extra.add(state);
    int dev;
    if ((st = check_desc_device(d, true, extra, &dev))) return st;
    DeviceGuard guard(dev);
    NewestParams p;
    p.n_planes = d->n_planes;
    p.segments = (int)d->segments;
    p.row_bytes = (int)row_bytes;
    p.tokens = d->tokens;
    p.state = reinterpret_cast<const CacheState*>(state);
    for (int i = 0; i < 4; ++i) {
        p.out[i] = i < d->n_planes ? static_cast<const unsigned char*>(d->planes[i].out) : nullptr;
        p.out_seg_stride[i] = i < d->n_planes ? d->planes[i].out_seg_stride : 0;
    }
    p.dst = static_cast<unsigned char*>(dst);
    const int chunks = (int)(need / 16);
    const int ctas = chunks < 256 * 64 ? (chunks + 255) / 256 : 64;
    cache_newest_kernel<uint4><<<ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return launch_status(false, "cache_newest");
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
    if (d->segments < 1 || d->segments > 65535 || d->tokens < 0)
        return fail(PITCH_ERR_INVALID_INPUT, "segments must be in 1...65535 and tokens not negative");
    if (d->dim < 1 || d->dim > PITCH_MAX_DIM) return fail(PITCH_ERR_INVALID_INPUT, "dimension %d must be in 1...%d", d->dim, PITCH_MAX_DIM);
    if (d->planes[0].codes == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "plane 0: null pointer");
    // how much of the static array this cache needs (every factor was range-checked above or is
    // checked here, so the product cannot overflow), and whether every per-channel plane starts a new group
    int64_t need = 0;
    bool fresh_group = true;
    for (int i = 0; i < d->n_planes; ++i) {
        const pitch_plane& pl = d->planes[i];
        if (pl.kind != PITCH_PLANE_CHANNEL) continue;
        if (pl.group_size < 1 || pl.group_size > PITCH_MAX_GROUP)
            return fail(PITCH_ERR_INVALID_INPUT, "group size %d must be in 1...%d", pl.group_size, PITCH_MAX_GROUP);
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
        mine[i].residual_bytes = 0;
        if (d->planes[i].kind == PITCH_PLANE_CHANNEL) {
            const int64_t seg_floats = ((int64_t)d->planes[i].group_size + 2) * d->dim;
            mine[i].residual = base + at_float;
            mine[i].residual_seg_stride = seg_floats * 4;
            mine[i].residual_bytes = d->segments * seg_floats * 4;
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

}  // extern "C"
