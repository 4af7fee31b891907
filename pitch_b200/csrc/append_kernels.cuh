// Appending tokens to a compressed cache: one launch encodes the new token(s) of every segment
// (layer x KV head) for every plane (K, V).  The work is tiny - one vector per segment and
// plane per generated token - so the kernel is built for latency, not throughput: grid =
// (segments, planes), one CTA per (segment, plane), one thread per coordinate, Walsh-Hadamard
// stages through shared memory.  The arithmetic, operation order included, is that of the bulk
// encoders, so an appended token has exactly the codes of the same token encoded in bulk.
//
// Per-channel planes keep the newest, still growing group of each segment in float32 in a
// residual buffer, rows [0, G) = tokens of the group, row G = running per-channel minimum, row
// G+1 = running maximum.  A new token updates the running range (min and max are exact in any
// order), and the whole group is re-quantised against the new fp16 range, so the stored codes
// and ranges always equal a bulk encode of the tokens seen so far.
#pragma once

#include "channel_kernels.cuh"
#include "common.cuh"

namespace pitch {

constexpr int APPEND_MIN_THREADS = 256;

struct AppendPlane {
    int kind;            // 0 TurboQuant, 1 PolarQuant variant, 2 per-channel
    int bits;
    int group_size;      // per-channel
    uint32_t seed;       // rotation seed (kinds 0, 1)
    const unsigned char* in;   // [segments][n_new][dim] of T
    int64_t in_seg_stride;
    unsigned char* codes;
    int64_t codes_seg_stride;
    unsigned char* side;
    int64_t side_seg_stride;
    float* residual;     // per-channel: [segments][group_size + 2][dim]
    int64_t residual_seg_elems;
};

struct AppendParams {
    int n_planes, dim, n_new;
    float rs;                    // 1/sqrt(dim)
    int64_t first_token;         // tokens held before the call
    AppendPlane plane[4];
    float book[4][256];          // TurboQuant centroids per plane (kind 0)
};

// One vector (TurboQuant or PolarQuant variant) by the whole CTA; threads >= dim only take part
// in the barriers.  s, s_codes: dim words each; s_edges: 2^bits floats; s_red: 32 floats.
template <typename T>
__device__ __forceinline__ void append_vector_cta(const T* __restrict__ x_in, uint32_t* __restrict__ out_codes,
                                                  float* __restrict__ out_scale, int dim, int bits, int kind,
                                                  uint32_t seed, float rs, const float* s_edges, float* s,
                                                  uint32_t* s_codes, float* s_red) {
    const int tid = threadIdx.x;
    const int wpv = words_per_vector(dim, bits);
    const bool active = tid < dim;
    const float x = active ? Elem<T>::to_f32(x_in[tid]) : 0.0f;
    const float sign = (pcg_hash(seed + (uint32_t)tid) & 1u) ? 1.0f : -1.0f;

    float norm = 0.0f, inv = 1.0f;
    if (kind == 0) {
        // balanced adjacent-pair tree, the order of tree_sum_regs + lanes_sum
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
        // same operations as polar_encode_kernel: approximate square root per pair, one correctly
        // rounded square root of the largest squared radius for the scale
        float a = 0.0f, c = 0.0f, r = 0.0f, r2 = 0.0f;
        if (active) {
            a = s[tid & ~1] * rs;
            c = s[(tid & ~1) + 1] * rs;
            const float aa = a * a, cc = c * c;
            r2 = aa + cc;
            asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(r2));
        }
        float m = r2;
        for (int k = 16; k > 0; k >>= 1) m = fmaxf(m, __shfl_xor_sync(FULL, m, k));
        if ((tid & 31) == 0) s_red[tid >> 5] = m;
        __syncthreads();
        float rmax2 = 0.0f;
        for (int k = 0; k < (int)((blockDim.x + 31) >> 5); ++k) rmax2 = fmaxf(rmax2, s_red[k]);
        const float rmax = sqrtf(rmax2);
        const float safe = rmax > 0.0f ? rmax : 1.0f;
        const int RL = (1 << bits) - 1;
        const float radius_scale = (float)RL / safe;
        if (active) {
            if ((tid & 1) == 0) {
                const int q = __float2int_rd(r * radius_scale + 0.5f);
                code = (uint32_t)min(q, RL);
            } else {
                code = angle_bin(a, c, bits);
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
    __syncthreads();      // s, s_codes, s_red are reused by the next vector
}

// Per-channel plane, one segment: fold the new tokens into the running range, then re-quantise
// the group's n tokens.  s_lo, s_step: dim floats each.
template <typename T>
__device__ __forceinline__ void append_channel_cta(const T* __restrict__ x_in, float* __restrict__ res,
                                                   uint32_t* __restrict__ group_codes, __half* __restrict__ group_ranges,
                                                   int pos, int n_new, int dim, int bits, int group_size,
                                                   float* s_lo, float* s_step) {
    const float levels = (float)((1u << bits) - 1u);
    const int wpv = words_per_vector(dim, bits);
    const int n = pos + n_new;
    float* run_lo = res + (int64_t)group_size * dim;
    float* run_hi = run_lo + dim;
    for (int ch = threadIdx.x; ch < dim; ch += blockDim.x) {
        float x = Elem<T>::to_f32(x_in[ch]);
        float lo = x, hi = x;
        if (pos > 0) {
            lo = fminf(run_lo[ch], x);
            hi = fmaxf(run_hi[ch], x);
        }
        res[pos * dim + ch] = x;
        for (int j = 1; j < n_new; ++j) {
            x = Elem<T>::to_f32(x_in[j * dim + ch]);
            res[(pos + j) * dim + ch] = x;
            lo = fminf(lo, x);
            hi = fmaxf(hi, x);
        }
        run_lo[ch] = lo;
        run_hi[ch] = hi;
        const __half lo16 = __float2half_rn(lo), hi16 = __float2half_rn(hi);
        group_ranges[ch] = lo16;
        group_ranges[dim + ch] = hi16;
        const float base = __half2float(lo16);
        s_lo[ch] = base;
        s_step[ch] = step_of(base, __half2float(hi16), levels);
    }
    __syncthreads();      // residual rows and the range are visible to the whole CTA
    for (int idx = threadIdx.x; idx < n * wpv; idx += blockDim.x) {
        const int t = idx / wpv, w = idx - t * wpv;
        const float* row = res + t * dim;
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
        group_codes[idx] = word;
    }
}

// grid = (segments, n_planes); blockDim.x = max(APPEND_MIN_THREADS, dim).
template <typename T>
__global__ void __launch_bounds__(1024)
cache_append_kernel(const __grid_constant__ AppendParams p) {
    __shared__ float s_a[1024];        // vector: WHT scratch      | per-channel: lo
    __shared__ float s_b[1024];        // vector: codes (as words) | per-channel: step
    __shared__ float s_edges[256];
    __shared__ float s_red[32];
    // Programmatic dependent launch on both sides: wait for the previous kernel of the stream (the
    // decode of the previous step reads the codes this grid rewrites), then let the next kernel (the
    // decode of this step) start its prologue; it still waits for this grid to finish before it
    // reads what is written here.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int64_t seg = blockIdx.x;
    const AppendPlane& P = p.plane[blockIdx.y];
    const int dim = p.dim;
    const int wpv = words_per_vector(dim, P.bits);
    const T* x_in = reinterpret_cast<const T*>(P.in + seg * P.in_seg_stride);
    if (P.kind == 2) {
        const int64_t g = p.first_token / P.group_size;
        const int pos = (int)(p.first_token - g * P.group_size);
        append_channel_cta<T>(x_in, P.residual + seg * P.residual_seg_elems,
                              reinterpret_cast<uint32_t*>(P.codes + seg * P.codes_seg_stride) + g * P.group_size * wpv,
                              reinterpret_cast<__half*>(P.side + seg * P.side_seg_stride) + g * 2 * dim, pos, p.n_new, dim,
                              P.bits, P.group_size, s_a, s_b);
    } else {
        if (P.kind == 0)
            for (int k = threadIdx.x; k < (1 << P.bits) - 1; k += blockDim.x)
                s_edges[k] = 0.5f * (p.book[blockIdx.y][k] + p.book[blockIdx.y][k + 1]);
        __syncthreads();
        for (int j = 0; j < p.n_new; ++j) {
            const int64_t tok = p.first_token + j;
            append_vector_cta<T>(x_in + (int64_t)j * dim,
                                 reinterpret_cast<uint32_t*>(P.codes + seg * P.codes_seg_stride) + tok * wpv,
                                 reinterpret_cast<float*>(P.side + seg * P.side_seg_stride) + tok, dim, P.bits, P.kind,
                                 P.seed, p.rs, s_edges, s_a, reinterpret_cast<uint32_t*>(s_b), s_red);
        }
    }
}

}  // namespace pitch
