// Whole-cache decode for head dimension 64 at 4 bits: the per-step bottleneck of a
// compressed KV cache (all tokens of every layer and KV head are decoded each step).
//
// One launch covers every plane (K, V) and every segment (layer x KV head).  A CTA of 128
// threads decodes 128 consecutive tokens of one (plane, segment):
//   * TurboQuant plane  - one vector per thread: the thread's 32 code bytes arrive as two
//     128-bit loads, the 64-point Walsh-Hadamard transform runs entirely in registers, and the
//     result leaves through a padded warp-private shared tile so that every global store
//     instruction writes 512 contiguous bytes per warp.
//   * per-channel plane - a lane owns 8 channels of 4 tokens per step (see channel_kernels.cuh);
//     loads are 4 bytes and stores 16 bytes per lane, both contiguous across the warp.
// The kernel is bound by HBM traffic: per token it reads 32 code bytes plus 4 bytes of side
// information and writes 64 elements.
#pragma once

#include "channel_kernels.cuh"
#include "common.cuh"

namespace pitch {

constexpr int C64_THREADS = 128;
constexpr int C64_WARPS = 4;
constexpr int C64_TILE = 128;   // tokens per CTA

struct Book16 { float c[16]; };

// 32 vectors (d = 64, b = 4) per warp, one per lane.  `codes`, `norms`, `out` point at the
// warp's first vector; nvalid in 1...32.
template <typename T>
__device__ __forceinline__ void turbo64_decode_warp(const uint4* __restrict__ codes, const float* __restrict__ norms,
                                                    T* __restrict__ out, int nvalid, const float* s_book,
                                                    uint32_t neg_lo, uint32_t neg_hi, unsigned char* stage, int lane) {
    const bool valid = lane < nvalid;
    uint4 c0 = make_uint4(0, 0, 0, 0), c1 = c0;
    float norm = 0.0f;
    if (valid) {
        c0 = ldg_stream(codes + 2 * lane);
        c1 = ldg_stream(codes + 2 * lane + 1);
        norm = __ldg(norms + lane);
    }
    const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    float x[64];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int k = 0; k < 8; ++k) x[8 * j + k] = s_book[(w[j] >> (4 * k)) & 15u];
    }
    wht_regs(x, 64);
    // 1/sqrt(64) is a power of two, so (x * rs) * norm == x * (rs * norm) in float32.
    const float scale = 0.125f * norm;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        x[i] = flip_if(x[i], neg_lo, i) * scale;
        x[32 + i] = flip_if(x[32 + i], neg_hi, i) * scale;
    }
    WarpStage<T, 64>::store(out, nvalid * 64, true, stage, lane, x);
}

// 32 tokens (d = 64, b = 4, all inside one group) per warp: lane = (token lane 0..3, slab 0..7).
template <typename T>
__device__ __forceinline__ void channel64_decode_warp(const uint32_t* __restrict__ codes,
                                                      const __half* __restrict__ group_ranges, T* __restrict__ out,
                                                      int nvalid, int lane) {
    const int slab = lane & 7, tok_lane = lane >> 3;
    float lo[8], step[8];
    load_slab_range(group_ranges, 0, 64, slab, 15.0f, lo, step);
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int t = 4 * k + tok_lane;
        w[k] = 0;
        if (t < nvalid) w[k] = __ldg(codes + t * 8 + slab);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int t = 4 * k + tok_lane;
        if (t < nvalid) decode_slab<4, T>(w[k], lo, step, out + t * 64 + slab * 8);
    }
}

struct Plane64 {
    int kind;                 // PITCH_PLANE_TURBO or PITCH_PLANE_CHANNEL
    int group_size;           // channel planes: multiple of 32
    uint32_t neg_lo, neg_hi;  // sign diagonal of the rotation (turbo planes)
    const unsigned char* codes;
    int64_t codes_seg_stride;
    const unsigned char* side;
    int64_t side_seg_stride;
    unsigned char* out;
    int64_t out_seg_stride;
};

struct Cache64Params {
    int n_planes;
    int tiles_per_seg;
    int64_t tokens;
    Plane64 plane[4];
    Book16 book;              // TurboQuant centroids for (64, 4)
};

// grid = segments * tiles_per_seg * n_planes; the plane index varies fastest so that CTAs
// running side by side mix the two kinds of work.
template <typename T>
__global__ void __launch_bounds__(C64_THREADS)
cache_decode_d64b4_kernel(const __grid_constant__ Cache64Params p) {
    __shared__ float s_book[16];
    __shared__ __align__(16) unsigned char s_stage[C64_WARPS][WarpStage<T, 64>::BYTES];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pl = blockIdx.x % p.n_planes;
    const int64_t rest = blockIdx.x / p.n_planes;
    const int64_t seg = rest / p.tiles_per_seg;
    const int tile = (int)(rest - seg * p.tiles_per_seg);
    const Plane64& P = p.plane[pl];

    const int64_t t0 = (int64_t)tile * C64_TILE + warp * 32;   // this warp's first token
    if (P.kind == 0) {
        if (threadIdx.x < 16) s_book[threadIdx.x] = p.book.c[threadIdx.x];
        __syncthreads();
        if (t0 >= p.tokens) return;
        const int64_t left = p.tokens - t0;
        const int nvalid = left < 32 ? (int)left : 32;
        const unsigned char* codes = P.codes + seg * P.codes_seg_stride + t0 * 32;
        const float* norms = reinterpret_cast<const float*>(P.side + seg * P.side_seg_stride) + t0;
        T* out = reinterpret_cast<T*>(P.out + seg * P.out_seg_stride) + t0 * 64;
        turbo64_decode_warp<T>(reinterpret_cast<const uint4*>(codes), norms, out, nvalid, s_book, P.neg_lo, P.neg_hi,
                               s_stage[warp], lane);
    } else {
        if (t0 >= p.tokens) return;
        const int64_t left = p.tokens - t0;
        const int nvalid = left < 32 ? (int)left : 32;
        const int64_t g = t0 / P.group_size;
        const unsigned char* codes = P.codes + seg * P.codes_seg_stride + t0 * 32;
        const __half* ranges = reinterpret_cast<const __half*>(P.side + seg * P.side_seg_stride) + g * 128;
        T* out = reinterpret_cast<T*>(P.out + seg * P.out_seg_stride) + t0 * 64;
        channel64_decode_warp<T>(reinterpret_cast<const uint32_t*>(codes), ranges, out, nvalid, lane);
    }
}

// Stand-alone TurboQuant decode, d = 64, b = 4, 16-byte aligned buffers: same warp routine.
template <typename T>
__global__ void __launch_bounds__(C64_THREADS)
turbo64_decode_kernel(const uint4* __restrict__ codes, const float* __restrict__ norms, T* __restrict__ out,
                      int64_t count, uint32_t neg_lo, uint32_t neg_hi, const Book16 book) {
    __shared__ float s_book[16];
    __shared__ __align__(16) unsigned char s_stage[C64_WARPS][WarpStage<T, 64>::BYTES];
    if (threadIdx.x < 16) s_book[threadIdx.x] = book.c[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t v0 = ((int64_t)blockIdx.x * C64_WARPS + warp) * 32;
    if (v0 >= count) return;
    const int64_t left = count - v0;
    turbo64_decode_warp<T>(codes + v0 * 2, norms + v0, out + v0 * 64, left < 32 ? (int)left : 32, s_book, neg_lo,
                           neg_hi, s_stage[warp], lane);
}

// ------------------------------------------------------------------------------------------
// Appending tokens to a cache.  The work is tiny (one vector per segment and plane per step),
// so these kernels favour one launch for all segments over throughput: one CTA per vector,
// one thread per coordinate, Walsh-Hadamard stages through shared memory.  The arithmetic
// (operation order included) is that of the bulk encoders, so an appended token has the
// same codes as the same token encoded in bulk.
// ------------------------------------------------------------------------------------------
struct Book256 { float c[256]; };

// blockDim.x = max(dim, 32) threads; grid = (n_new, segments).
// kind 0 = TurboQuant, 1 = PolarQuant variant.
template <typename T>
__global__ void __launch_bounds__(1024)
cache_append_vector_kernel(const unsigned char* __restrict__ in, int64_t in_seg_stride,
                           unsigned char* __restrict__ codes, int64_t codes_seg_stride,
                           unsigned char* __restrict__ side, int64_t side_seg_stride, int64_t first_token,
                           int dim, int bits, int kind, uint32_t seed, float rs, const Book256 book) {
    __shared__ float s[1024];
    __shared__ float s_edges[256];
    __shared__ uint32_t s_codes[1024];
    __shared__ float s_red[32];
    const int tid = threadIdx.x;
    const int64_t seg = blockIdx.y, j = blockIdx.x, tok = first_token + j;
    const int wpv = words_per_vector(dim, bits);
    const T* x_in = reinterpret_cast<const T*>(in + seg * in_seg_stride) + j * dim;
    uint32_t* out_codes = reinterpret_cast<uint32_t*>(codes + seg * codes_seg_stride) + tok * wpv;
    float* out_scale = reinterpret_cast<float*>(side + seg * side_seg_stride) + tok;
    const bool active = tid < dim;
    const float x = active ? Elem<T>::to_f32(x_in[tid]) : 0.0f;
    const float sign = (pcg_hash(seed + (uint32_t)tid) & 1u) ? 1.0f : -1.0f;
    if (kind == 0)
        for (int k = tid; k < (1 << bits) - 1; k += blockDim.x) s_edges[k] = 0.5f * (book.c[k] + book.c[k + 1]);

    float norm = 0.0f, inv = 1.0f;
    if (kind == 0) {
        // balanced adjacent-pair tree, as tree_sum_regs + lanes_sum
        if (active) s[tid] = x * x;
        __syncthreads();
        for (int n = dim; n > 1; n >>= 1) {
            float t = 0.0f;
            if (tid < n / 2) t = s[2 * tid] + s[2 * tid + 1];
            __syncthreads();
            if (tid < n / 2) s[tid] = t;
            __syncthreads();
        }
        norm = sqrtf(s[0]);
        inv = norm > 0.0f ? 1.0f / norm : 0.0f;
        __syncthreads();
    }
    if (active) s[tid] = kind == 0 ? sign * x * inv : sign * x;
    __syncthreads();
    for (int len = 1; len < dim; len <<= 1) {
        float v = 0.0f;
        if (active) {
            const float lo = s[tid & ~len], hi = s[tid | len];
            v = (tid & len) ? (lo - hi) : (lo + hi);
        }
        __syncthreads();
        if (active) s[tid] = v;
        __syncthreads();
    }
    uint32_t code = 0;
    float scale = norm;
    if (kind == 0) {
        if (active) {
            const float u = s[tid] * rs;
            for (int step = (1 << bits) >> 1; step > 0; step >>= 1) {
                const uint32_t cand = code + step;
                if (u > s_edges[cand - 1]) code = cand;
            }
        }
    } else {
        float a = 0.0f, c = 0.0f, r = 0.0f;
        if (active) {
            a = s[tid & ~1] * rs;
            c = s[(tid & ~1) + 1] * rs;
            const float aa = a * a, cc = c * c;
            r = sqrtf(aa + cc);
        }
        float m = r;
        for (int k = 16; k > 0; k >>= 1) m = fmaxf(m, __shfl_xor_sync(FULL, m, k));
        if ((tid & 31) == 0) s_red[tid >> 5] = m;
        __syncthreads();
        float rmax = 0.0f;
        for (int k = 0; k < (int)((blockDim.x + 31) >> 5); ++k) rmax = fmaxf(rmax, s_red[k]);
        const float safe = rmax > 0.0f ? rmax : 1.0f;
        const float RL = (float)((1u << bits) - 1u), NB = (float)(1u << bits);
        if (active) {
            if ((tid & 1) == 0) {
                float q = floorf(r / safe * RL + 0.5f);
                q = fminf(fmaxf(q, 0.0f), RL);
                code = (uint32_t)q;
            } else {
                float theta = atan2f(c, a);
                if (theta < 0.0f) theta += TWO_PI_F;
                code = (uint32_t)floorf(theta / TWO_PI_F * NB + 0.5f) & ((1u << bits) - 1u);
            }
        }
        scale = rmax;
    }
    if (active) s_codes[tid] = code;
    __syncthreads();
    for (int w = tid; w < wpv; w += blockDim.x) {
        const int bit0 = w * 32;
        const int i0 = bit0 / bits;
        int i1 = (bit0 + 31) / bits;
        if (i1 > dim - 1) i1 = dim - 1;
        uint32_t word = 0;
        for (int i = i0; i <= i1; ++i) {
            const int shift = i * bits - bit0;
            word |= shift >= 0 ? (s_codes[i] << shift) : (s_codes[i] >> (-shift));
        }
        out_codes[w] = word;
    }
    if (tid == 0) *out_scale = scale;
}

// Per-channel plane: the newest, still growing group of every segment is kept in float32 in
// `residual` ([segments][group_size][dim]) and re-encoded from there each time tokens arrive,
// so the stored codes always equal a bulk encode of the tokens seen so far.
// grid = segments, 256 threads.  All new tokens must fall into one group.
template <typename T>
__global__ void __launch_bounds__(256)
cache_append_channel_kernel(const unsigned char* __restrict__ in, int64_t in_seg_stride, float* __restrict__ residual,
                            int64_t residual_seg_elems, unsigned char* __restrict__ codes, int64_t codes_seg_stride,
                            unsigned char* __restrict__ ranges, int64_t ranges_seg_stride, int64_t first_token,
                            int n_new, int dim, int bits, int group_size) {
    __shared__ float s_lo[1024], s_step[1024];
    const int64_t seg = blockIdx.x;
    const int64_t g = first_token / group_size;
    const int pos = (int)(first_token - g * group_size);
    const int n = pos + n_new;
    const float levels = (float)((1u << bits) - 1u);
    const int wpv = words_per_vector(dim, bits);
    const T* x_in = reinterpret_cast<const T*>(in + seg * in_seg_stride);
    float* res = residual + seg * residual_seg_elems;
    uint32_t* out_codes = reinterpret_cast<uint32_t*>(codes + seg * codes_seg_stride) + g * group_size * wpv;
    __half* out_ranges = reinterpret_cast<__half*>(ranges + seg * ranges_seg_stride) + g * 2 * dim;

    for (int e = threadIdx.x; e < n_new * dim; e += blockDim.x) res[pos * dim + e] = Elem<T>::to_f32(x_in[e]);
    __syncthreads();

    for (int ch = threadIdx.x; ch < dim; ch += blockDim.x) {
        float lo = res[ch], hi = lo;
        for (int t = 1; t < n; ++t) {
            const float x = res[t * dim + ch];
            lo = fminf(lo, x);
            hi = fmaxf(hi, x);
        }
        const __half lo16 = __float2half_rn(lo), hi16 = __float2half_rn(hi);
        out_ranges[ch] = lo16;
        out_ranges[dim + ch] = hi16;
        const float base = __half2float(lo16);
        s_lo[ch] = base;
        s_step[ch] = step_of(base, __half2float(hi16), levels);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int t = warp; t < n; t += nwarps) {
        const float* row = res + t * dim;
        for (int w = lane; w < wpv; w += 32) {
            const int bit0 = w * 32;
            const int i0 = bit0 / bits;
            int i1 = (bit0 + 31) / bits;
            if (i1 > dim - 1) i1 = dim - 1;
            uint32_t word = 0;
            for (int i = i0; i <= i1; ++i) {
                const uint32_t c = quantise(row[i], s_lo[i], s_step[i], levels);
                const int shift = i * bits - bit0;
                word |= shift >= 0 ? (c << shift) : (c >> (-shift));
            }
            out_codes[t * wpv + w] = word;
        }
    }
}

}  // namespace pitch
