// Per-channel (KIVI-style) key codec.  Per group of G tokens and per channel the encoder keeps
// an fp16 minimum and maximum; step = (max - min) / (2^b - 1), or 1 when the channel is
// constant; code = clamp(floor((x - min) / step + 0.5), 0, 2^b - 1); decode = code * step + min.
// All arithmetic is float32, one rounding per operation, exactly as the specification
// (reference/pitch_reference.py:145-174; PITCHKernels.metal:262-325).
//
// Two mappings:
//  * slab kernels - dim a multiple of 8 with dim/8 a power of two (8...256) and b in {2,4,8}:
//    a lane owns 8 consecutive channels ("slab"), 32/(dim/8) tokens are processed per warp
//    step, the per-channel range lives in registers for the whole group, and every global
//    access of the full-precision tensor is a contiguous 16-byte piece per lane.
//  * general kernels - any dim 1...1024, any b, any G.
#pragma once

#include "common.cuh"

namespace pitch {

constexpr int CH_THREADS = 128;
constexpr int CH_WARPS = CH_THREADS / 32;
constexpr int CH_CHUNK = 256;   // tokens of one group handled by one warp in the slab decoder

__device__ __forceinline__ float step_of(float lo, float hi, float levels) {
    const float s = (hi - lo) / levels;
    return s == 0.0f ? 1.0f : s;
}

__device__ __forceinline__ uint32_t quantise(float x, float lo, float step, float levels) {
    float q = floorf((x - lo) / step + 0.5f);
    q = fminf(fmaxf(q, 0.0f), levels);
    return (uint32_t)q;
}

// The same code from a precomputed reciprocal of the step, without a division per element.
// With rcp = RN(1 / step) (correctly rounded: __frcp_rn), q0 = RN(d * rcp) lies within one ulp of
// d / step; the remainder rem = d - step * q0 is then exactly representable and fma(-step, q0, d)
// returns it without error; and q = RN(q0 + rem * rcp) is the correctly rounded quotient RN(d / step),
// i.e. the very float the division of `quantise` produces.  This is the final correction step of
// FMA-based division (P. Markstein, "IA-64 and Elementary Functions", ch. 8: a correctly rounded
// reciprocal, a quotient estimate within one ulp, an exact remainder and one fused correction give
// the correctly rounded quotient).  Its premises hold here: step is a normal float in
// [2^-24 / 255, 131008 / 3] (a difference of two finite fp16 values over the number of levels, or 1),
// so neither rcp nor step * q0 can overflow; the remainder can lose bits to underflow only when
// |d| < 2^-100, where the quotient is below 2^-70 and the code is 0 whatever its last bits.  The
// rounding q + 0.5, the floor and the clamp are those of `quantise` (the conversion saturates).
// Checked in addition against the division on 4e8 random and adversarial pairs (steps with an
// all-ones significand, quotients next to k + 1/2).
__device__ __forceinline__ uint32_t quantise_rcp(float x, float lo, float step, float rcp, float levels) {
    const float d = x - lo;
    const float q0 = d * rcp;
    const int q = __float2int_rd(__fmaf_rn(__fmaf_rn(-step, q0, d), rcp, q0) + 0.5f);     // floor, saturating
    return (uint32_t)min(max(q, 0), (int)levels);
}

// ------------------------------------------------------------------------------------------
// General decode: one thread per coordinate.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
channel_decode_general_kernel(const uint32_t* __restrict__ codes, const __half* __restrict__ ranges,
                              T* __restrict__ out, int64_t count, int dim, int bits, int group_size) {
    const int64_t total = count * dim;
    const float levels = (float)((1u << bits) - 1u);
    const int wpv = words_per_vector(dim, bits);
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t tok = e / dim;
        const int ch = (int)(e - tok * dim);
        const int64_t g = tok / group_size;
        const float lo = __half2float(ranges[g * 2 * dim + ch]);
        const float hi = __half2float(ranges[g * 2 * dim + dim + ch]);
        const float step = step_of(lo, hi, levels);
        const float c = (float)read_code(codes + tok * wpv, ch, bits);
        out[e] = Elem<T>::from_f32(c * step + lo);
    }
}

// ------------------------------------------------------------------------------------------
// General encode: one CTA per group.  Pass 1: a thread per channel scans the group's tokens
// (coalesced across channels).  Pass 2: a warp per token, a lane per packed word.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
channel_encode_general_kernel(const T* __restrict__ in, uint32_t* __restrict__ codes, __half* __restrict__ ranges,
                              int64_t count, int dim, int bits, int group_size) {
    __shared__ float s_lo[1024], s_step[1024];
    const int64_t g = blockIdx.x;
    const int64_t first = g * group_size;
    const int n = (int)((count - first) < group_size ? (count - first) : group_size);
    const float levels = (float)((1u << bits) - 1u);
    const int wpv = words_per_vector(dim, bits);

    for (int ch = threadIdx.x; ch < dim; ch += blockDim.x) {
        float lo = Elem<T>::to_f32(in[first * dim + ch]), hi = lo;
        for (int t = 1; t < n; ++t) {
            const float x = Elem<T>::to_f32(in[(first + t) * dim + ch]);
            lo = fminf(lo, x);
            hi = fmaxf(hi, x);
        }
        const __half lo16 = __float2half_rn(lo), hi16 = __float2half_rn(hi);
        ranges[g * 2 * dim + ch] = lo16;
        ranges[g * 2 * dim + dim + ch] = hi16;
        const float base = __half2float(lo16);
        s_lo[ch] = base;
        s_step[ch] = step_of(base, __half2float(hi16), levels);
    }
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int t = warp; t < n; t += nwarps) {
        const T* row = in + (first + t) * dim;
        for (int w = lane; w < wpv; w += 32) {
            const int bit0 = w * 32;
            const int i0 = bit0 / bits;
            int i1 = (bit0 + 31) / bits;
            if (i1 > dim - 1) i1 = dim - 1;
            uint32_t word = 0;
            for (int i = i0; i <= i1; ++i) {
                const uint32_t c = quantise(Elem<T>::to_f32(row[i]), s_lo[i], s_step[i], levels);
                const int shift = i * bits - bit0;
                word |= shift >= 0 ? (c << shift) : (c >> (-shift));
            }
            codes[(first + t) * wpv + w] = word;
        }
    }
}

// ------------------------------------------------------------------------------------------
// Slab mapping helpers.  A slab is 8 channels: 8*BITS bits = BITS bytes of codes.
// ------------------------------------------------------------------------------------------
template <int BITS> struct SlabCodes;   // packed codes of one slab
template <> struct SlabCodes<2> {
    typedef uint16_t type;
    static __device__ __forceinline__ uint32_t code(type w, int i) { return (w >> (2 * i)) & 3u; }
};
template <> struct SlabCodes<4> {
    typedef uint32_t type;
    static __device__ __forceinline__ uint32_t code(type w, int i) { return (w >> (4 * i)) & 15u; }
};
template <> struct SlabCodes<8> {
    typedef uint2 type;
    static __device__ __forceinline__ uint32_t code(type w, int i) {
        return ((i < 4 ? w.x : w.y) >> (8 * (i & 3))) & 255u;
    }
};

// float(code) without an integer-to-float conversion: 2^23 + code is exact in float32.
__device__ __forceinline__ float small_uint_to_float(uint32_t c) {
    return __uint_as_float(0x4B000000u | c) - 8388608.0f;
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]) {
    uint32_t w[Packer<T, 8>::WORDS];
    Packer<T, 8>::pack(v, w);
    stg_stream(reinterpret_cast<uint4*>(p), make_uint4(w[0], w[1], w[2], w[3]));
    if constexpr (sizeof(T) == 4)
        stg_stream(reinterpret_cast<uint4*>(p) + 1, make_uint4(w[4], w[5], w[6], w[7]));
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
    uint32_t w[Packer<T, 8>::WORDS];
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    if constexpr (sizeof(T) == 4) {
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
        w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    }
    Packer<T, 8>::unpack(w, v);
}

// Reads the fp16 range of this lane's slab for group g and turns it into (lo, step).
__device__ __forceinline__ void load_slab_range(const __half* __restrict__ ranges, int64_t g, int dim, int slab,
                                                float levels, float (&lo)[8], float (&step)[8]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(ranges + g * 2 * dim + slab * 8));
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(ranges + g * 2 * dim + dim + slab * 8));
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 l = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
        const float2 h = __half22float2(*reinterpret_cast<const __half2*>(&bw[i]));
        lo[2 * i] = l.x;
        lo[2 * i + 1] = l.y;
        step[2 * i] = step_of(l.x, h.x, levels);
        step[2 * i + 1] = step_of(l.y, h.y, levels);
    }
}

// Decodes one slab of one token: 8 outputs.
template <int BITS, typename T>
__device__ __forceinline__ void decode_slab(typename SlabCodes<BITS>::type w, const float (&lo)[8],
                                            const float (&step)[8], T* out) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = small_uint_to_float(SlabCodes<BITS>::code(w, i)) * step[i] + lo[i];
    store8<T>(out, v);
}

// ------------------------------------------------------------------------------------------
// Slab decode.  One warp per (group, chunk of up to CH_CHUNK tokens).  log2_slabs = log2(dim/8).
// Requires 16-byte aligned ranges and output, code rows aligned to BITS bytes (always true).
// ------------------------------------------------------------------------------------------
template <int BITS, typename T>
__global__ void __launch_bounds__(CH_THREADS)
channel_decode_slab_kernel(const unsigned char* __restrict__ codes, const __half* __restrict__ ranges,
                           T* __restrict__ out, int64_t count, int dim, int log2_slabs, int group_size,
                           int chunks_per_group, int64_t total_tiles) {
    const int lane = threadIdx.x & 31;
    const int64_t tile = (int64_t)blockIdx.x * CH_WARPS + (threadIdx.x >> 5);
    if (tile >= total_tiles) return;
    const int64_t g = tile / chunks_per_group;
    const int chunk = (int)(tile - g * chunks_per_group);
    const int64_t first = g * group_size + (int64_t)chunk * CH_CHUNK;
    int64_t last = first + CH_CHUNK;
    if (last > (g + 1) * (int64_t)group_size) last = (g + 1) * (int64_t)group_size;
    if (last > count) last = count;

    const int slab = lane & ((1 << log2_slabs) - 1);
    const int tok_lane = lane >> log2_slabs;
    const int tok_lanes = 32 >> log2_slabs;
    const int stride = words_per_vector(dim, BITS) * 4;   // bytes of codes per token
    constexpr float LEVELS = (float)((1 << BITS) - 1);

    float lo[8], step[8];
    load_slab_range(ranges, g, dim, slab, LEVELS, lo, step);

    typedef typename SlabCodes<BITS>::type W;
    for (int64_t t = first + tok_lane; t < last; t += 4 * tok_lanes) {
        // four tokens in flight per lane
        W w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t tk = t + (int64_t)k * tok_lanes;
            if (tk < last) w[k] = __ldg(reinterpret_cast<const W*>(codes + tk * stride + slab * BITS));
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t tk = t + (int64_t)k * tok_lanes;
            if (tk < last) decode_slab<BITS, T>(w[k], lo, step, out + tk * dim + slab * 8);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Slab encode.  One warp per group: pass 1 scans the group for the per-channel range, pass 2
// re-reads (L1/L2 resident) and quantises.  Requires 16-byte aligned input and ranges.
// ------------------------------------------------------------------------------------------
template <int BITS, typename T>
__global__ void __launch_bounds__(CH_THREADS)
channel_encode_slab_kernel(const T* __restrict__ in, unsigned char* __restrict__ codes, __half* __restrict__ ranges,
                           int64_t count, int dim, int log2_slabs, int group_size, int64_t groups) {
    const int lane = threadIdx.x & 31;
    const int64_t g = (int64_t)blockIdx.x * CH_WARPS + (threadIdx.x >> 5);
    if (g >= groups) return;
    const int64_t first = g * group_size;
    int64_t last = first + group_size;
    if (last > count) last = count;

    const int slab = lane & ((1 << log2_slabs) - 1);
    const int tok_lane = lane >> log2_slabs;
    const int tok_lanes = 32 >> log2_slabs;
    const int stride = words_per_vector(dim, BITS) * 4;
    constexpr float LEVELS = (float)((1 << BITS) - 1);

    // every lane starts from the group's first token, so lanes without a token of their own stay neutral
    float lo[8], hi[8];
    load8<T>(in + first * dim + slab * 8, lo);
#pragma unroll
    for (int i = 0; i < 8; ++i) hi[i] = lo[i];
    for (int64_t t = first + tok_lane; t < last; t += 4 * tok_lanes) {
        // four tokens in flight per lane
        float x[4][8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t tk = t + (int64_t)k * tok_lanes;
            load8<T>(in + (tk < last ? tk : first) * dim + slab * 8, x[k]);      // a token of the group either way
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                lo[i] = fminf(lo[i], x[k][i]);
                hi[i] = fmaxf(hi[i], x[k][i]);
            }
    }
    for (int m = 1 << log2_slabs; m < 32; m <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo[i] = fminf(lo[i], __shfl_xor_sync(FULL, lo[i], m));
            hi[i] = fmaxf(hi[i], __shfl_xor_sync(FULL, hi[i], m));
        }
    }
    float step[8];
    uint32_t lo_w[4], hi_w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 l = __floats2half2_rn(lo[2 * i], lo[2 * i + 1]);
        const __half2 h = __floats2half2_rn(hi[2 * i], hi[2 * i + 1]);
        lo_w[i] = *reinterpret_cast<const uint32_t*>(&l);
        hi_w[i] = *reinterpret_cast<const uint32_t*>(&h);
        const float2 lf = __half22float2(l), hf = __half22float2(h);
        lo[2 * i] = lf.x;
        lo[2 * i + 1] = lf.y;
        step[2 * i] = step_of(lf.x, hf.x, LEVELS);
        step[2 * i + 1] = step_of(lf.y, hf.y, LEVELS);
    }
    float rcp[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) rcp[i] = __frcp_rn(step[i]);
    if (tok_lane == 0) {
        *reinterpret_cast<uint4*>(ranges + g * 2 * dim + slab * 8) = make_uint4(lo_w[0], lo_w[1], lo_w[2], lo_w[3]);
        *reinterpret_cast<uint4*>(ranges + g * 2 * dim + dim + slab * 8) = make_uint4(hi_w[0], hi_w[1], hi_w[2], hi_w[3]);
    }

    for (int64_t t0 = first + tok_lane; t0 < last; t0 += 4 * tok_lanes) {
      float xs[4][8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
          const int64_t tk = t0 + (int64_t)k * tok_lanes;
          if (tk < last) load8<T>(in + tk * dim + slab * 8, xs[k]);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t t = t0 + (int64_t)k * tok_lanes;
        if (t >= last) break;
        const float (&x)[8] = xs[k];
        uint32_t c[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) c[i] = quantise_rcp(x[i], lo[i], step[i], rcp[i], LEVELS);
        unsigned char* dst = codes + t * stride + slab * BITS;
        if (BITS == 2) {
            uint32_t w = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) w |= c[i] << (2 * i);
            *reinterpret_cast<uint16_t*>(dst) = (uint16_t)w;
        } else if (BITS == 4) {
            uint32_t w = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) w |= c[i] << (4 * i);
            *reinterpret_cast<uint32_t*>(dst) = w;
        } else {
            uint2 w = make_uint2(0, 0);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                w.x |= c[i] << (8 * i);
                w.y |= c[i + 4] << (8 * i);
            }
            *reinterpret_cast<uint2*>(dst) = w;
        }
      }
    }
}

}  // namespace pitch
