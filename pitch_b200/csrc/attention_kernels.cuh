// Single-token attention straight from the compressed cache (head dimension 64, per-channel 4-bit
// keys, TurboQuant 4-bit values): the decoded cache is never written to memory.  This is the step
// the reference names as what has to come next for long contexts (README.md:96, "decoding needs
// to move inside the attention kernel").
//
// For one segment (layer x KV head) with R query vectors q_r (grouped-query attention: the query
// heads that share this KV head) and T cached tokens:
//
//   scores   s_r,t = scale * sum_c q_r,c * K_t,c        with K_t,c = code_t,c * step_g,c + lo_g,c
//                  = sum_c (scale * q_r,c * step_g,c) * code_t,c  +  scale * sum_c q_r,c * lo_g,c
//            -> per group g of tokens the query is folded into the quantisation grid once
//               (qk_r,c and a bias qb_r); a score is then a dot product with the 4-bit codes.
//   output   o_r = sum_t p_r,t V_t / sum_t p_r,t        with V_t = norm_t/8 * D H cb[codes_t]
//                = D H ( sum_t p_r,t norm_t cb[codes_t] ) / (8 sum_t p_r,t)
//            -> centroids are accumulated in the rotated domain and the Walsh-Hadamard transform
//               and the sign diagonal are applied once per query at the very end, instead of once
//               per cached token.
//
// Kernel 1 (attention_partial_kernel): grid (splits, segments); a CTA of 8 warps walks one slice of
// the tokens of one segment in tiles of 32 tokens.  For the scores a lane owns a token (its 32 code
// bytes arrive as two 128-bit loads, the folded query is read from shared memory as broadcasts);
// softmax is online (running maximum and sum per query, base-2 exponentials); for the value
// accumulation a lane owns two of the 64 output coordinates: it reads its code byte of every token
// of the tile from a shared tile and maps it to two centroids through a lane-replicated, conflict
// free table.  Each CTA writes (max, sum, 64 accumulators) per query to a workspace.
// Kernel 2 (attention_combine_kernel): merges the slices of a segment, normalises, un-rotates.
#pragma once

#include "cache_kernels.cuh"
#include "common.cuh"

namespace pitch {

constexpr int AT_THREADS = 256;
constexpr int AT_WARPS = AT_THREADS / 32;
constexpr int AT_MAX_QUERIES = 8;
constexpr int AT_PART_FLOATS = 66;                     // per (segment, split, query): max, sum, 64 accumulators
constexpr int AT_WARP_SMEM = 1024 + 1024 + AT_MAX_QUERIES * 64 * 4 + 32;   // value codes, weights, folded query, bias
constexpr int AT_SMEM_BYTES = CD_TABLE_BYTES + AT_WARPS * AT_WARP_SMEM;

struct AttentionParams {
    int segments, tokens, splits, tokens_per_split;    // tokens_per_split is a multiple of 256
    int n_queries, group_size;
    float scale_log2;                                  // softmax scale * log2(e)
    uint32_t neg_lo, neg_hi;                           // sign diagonal of the values' rotation
    const unsigned char* k_codes; int64_t k_codes_seg;
    const unsigned char* k_ranges; int64_t k_ranges_seg;
    const unsigned char* v_codes; int64_t v_codes_seg;
    const unsigned char* v_norms; int64_t v_norms_seg;
    const float* q;                                    // [segments][n_queries][64]
    float* work;                                       // [segments][splits][n_queries][66]
    float* out;                                        // [segments][n_queries][64]
    Book16 book;                                       // TurboQuant centroids (64, 4)
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, m));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, m);
    return v;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int R>
__global__ void __launch_bounds__(AT_THREADS, 2)
attention_partial_kernel(const __grid_constant__ AttentionParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* table = smem;                                       // entry e, slot l: (c[e & 15], c[e >> 4])
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char* mine = smem + CD_TABLE_BYTES + warp * AT_WARP_SMEM;
    unsigned char* vtile = mine;                                       // [32 tokens][32 code bytes]
    float* wtile = reinterpret_cast<float*>(mine + 1024);              // [32 tokens][8 weights]
    float* qk = reinterpret_cast<float*>(mine + 2048);                 // [R][64] folded query
    float* qb = reinterpret_cast<float*>(mine + 2048 + AT_MAX_QUERIES * 256);   // [R] bias

    for (int idx = threadIdx.x; idx < 256 * 32; idx += AT_THREADS) {
        const int e = idx >> 5;
        *reinterpret_cast<float2*>(table + idx * 8) = make_float2(p.book.c[e & 15], p.book.c[e >> 4]);
    }
    const int64_t seg = blockIdx.y;
    const int split = blockIdx.x;
    const int t_begin = split * p.tokens_per_split;
    int t_end = t_begin + p.tokens_per_split;
    if (t_end > p.tokens) t_end = p.tokens;

    // this lane's two channels of every query, pre-multiplied by the softmax scale (base 2)
    float q0[R], q1[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float2 v = *reinterpret_cast<const float2*>(p.q + (seg * R + r) * 64 + 2 * lane);
        q0[r] = v.x * p.scale_log2;
        q1[r] = v.y * p.scale_log2;
    }
    __syncthreads();

    const unsigned char* k_codes = p.k_codes + seg * p.k_codes_seg;
    const __half* k_ranges = reinterpret_cast<const __half*>(p.k_ranges + seg * p.k_ranges_seg);
    const unsigned char* v_codes = p.v_codes + seg * p.v_codes_seg;
    const float* v_norms = reinterpret_cast<const float*>(p.v_norms + seg * p.v_norms_seg);
    const uint32_t slot = (uint32_t)lane * 8u;

    float m[R], l[R];
    float2 acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) { m[r] = -INFINITY; l[r] = 0.0f; acc[r] = make_float2(0.0f, 0.0f); }
    int cur_group = -1;

    for (int t0 = t_begin + warp * 32; t0 < t_end; t0 += AT_WARPS * 32) {
        const int nvalid = t_end - t0 < 32 ? t_end - t0 : 32;
        const bool valid = lane < nvalid;
        // ---- loads of this tile: key codes and value codes of token t0 + lane, its norm
        uint4 ka = make_uint4(0, 0, 0, 0), kb = ka, va = ka, vb = ka;
        float norm = 0.0f;
        if (valid) {
            const uint4* kp = reinterpret_cast<const uint4*>(k_codes + (int64_t)(t0 + lane) * 32);
            const uint4* vp = reinterpret_cast<const uint4*>(v_codes + (int64_t)(t0 + lane) * 32);
            ka = ldg_stream(kp); kb = ldg_stream(kp + 1);
            va = ldg_stream(vp); vb = ldg_stream(vp + 1);
            norm = __ldg(v_norms + t0 + lane);
        }
        // ---- a new group of tokens: fold the queries into its quantisation grid
        const int group = t0 / p.group_size;
        if (group != cur_group) {
            cur_group = group;
            const __half2 lo2 = *reinterpret_cast<const __half2*>(k_ranges + (int64_t)group * 128 + 2 * lane);
            const __half2 hi2 = *reinterpret_cast<const __half2*>(k_ranges + (int64_t)group * 128 + 64 + 2 * lane);
            const float2 lo = __half22float2(lo2), hi = __half22float2(hi2);
            const float s0 = step15(lo.x, hi.x), s1 = step15(lo.y, hi.y);
            __syncwarp();                               // the previous tile's reads of qk are done
#pragma unroll
            for (int r = 0; r < R; ++r) {
                *reinterpret_cast<float2*>(qk + r * 64 + 2 * lane) = make_float2(q0[r] * s0, q1[r] * s1);
                const float b = warp_sum(q0[r] * lo.x + q1[r] * lo.y);
                if (lane == 0) qb[r] = b;
            }
        }
        *reinterpret_cast<uint4*>(vtile + lane * 32) = va;
        *reinterpret_cast<uint4*>(vtile + lane * 32 + 16) = vb;
        __syncwarp();

        // ---- scores of token t0 + lane against every query
        const uint32_t kw[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
        float2 s2[R];
#pragma unroll
        for (int r = 0; r < R; ++r) s2[r] = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float2 f[4];
            codes8_to_pairs(kw[j], f);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float4 a = *reinterpret_cast<const float4*>(qk + r * 64 + 8 * j);        // broadcast
                const float4 b = *reinterpret_cast<const float4*>(qk + r * 64 + 8 * j + 4);
                s2[r] = __ffma2_rn(f[0], make_float2(a.x, a.y), s2[r]);
                s2[r] = __ffma2_rn(f[1], make_float2(a.z, a.w), s2[r]);
                s2[r] = __ffma2_rn(f[2], make_float2(b.x, b.y), s2[r]);
                s2[r] = __ffma2_rn(f[3], make_float2(b.z, b.w), s2[r]);
            }
        }
        // ---- online softmax (base 2) and the weights of this tile
        float w[AT_MAX_QUERIES];
#pragma unroll
        for (int r = 0; r < AT_MAX_QUERIES; ++r) w[r] = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float s = valid ? (s2[r].x + s2[r].y + qb[r]) : -INFINITY;
            const float mn = fmaxf(m[r], warp_max(s));          // finite: every tile has a valid token
            const float corr = fast_exp2(m[r] - mn);            // 0 on the first tile (m = -inf)
            const float pr = fast_exp2(s - mn);                 // 0 for tokens that do not exist
            l[r] = l[r] * corr + warp_sum(pr);
            acc[r].x *= corr;
            acc[r].y *= corr;
            m[r] = mn;
            w[r] = pr * norm;
        }
        *reinterpret_cast<float4*>(wtile + lane * 8) = make_float4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<float4*>(wtile + lane * 8 + 4) = make_float4(w[4], w[5], w[6], w[7]);
        __syncwarp();

        // ---- values: this lane accumulates output coordinates 2*lane and 2*lane + 1 over the tile
#pragma unroll 8
        for (int t = 0; t < 32; ++t) {
            const uint32_t byte = vtile[t * 32 + lane];
            const float2 c = *reinterpret_cast<const float2*>(table + __byte_perm(byte, slot, 0x5504));
            const float4 wa = *reinterpret_cast<const float4*>(wtile + t * 8);                 // broadcast
            const float4 wb = *reinterpret_cast<const float4*>(wtile + t * 8 + 4);
            const float ws[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int r = 0; r < R; ++r) {
                acc[r].x = fmaf(c.x, ws[r], acc[r].x);
                acc[r].y = fmaf(c.y, ws[r], acc[r].y);
            }
        }
        __syncwarp();
    }

    // ---- merge the eight warps of the CTA (the table is no longer needed: reuse its space)
    __syncthreads();
    float* merge = reinterpret_cast<float*>(smem);                    // [warp][R][66]
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float* dst = merge + (warp * R + r) * AT_PART_FLOATS;
        if (lane == 0) { dst[0] = m[r]; dst[1] = l[r]; }
        *reinterpret_cast<float2*>(dst + 2 + 2 * lane) = acc[r];
    }
    __syncthreads();
    float* out = p.work + ((seg * p.splits + split) * R) * AT_PART_FLOATS;
    for (int idx = threadIdx.x; idx < R * 64; idx += AT_THREADS) {
        const int r = idx >> 6, c = idx & 63;
        float mm = -INFINITY;
        for (int wv = 0; wv < AT_WARPS; ++wv) mm = fmaxf(mm, merge[(wv * R + r) * AT_PART_FLOATS]);
        float a = 0.0f, ll = 0.0f;
        for (int wv = 0; wv < AT_WARPS; ++wv) {
            const float* src = merge + (wv * R + r) * AT_PART_FLOATS;
            const float f = src[0] == -INFINITY ? 0.0f : fast_exp2(src[0] - mm);   // a warp that saw no tile
            a += src[2 + c] * f;
            ll += src[1] * f;
        }
        out[r * AT_PART_FLOATS + 2 + c] = a;
        if (c == 0) { out[r * AT_PART_FLOATS] = mm; out[r * AT_PART_FLOATS + 1] = ll; }
    }
}

// grid = segments, blockDim = 32 * n_queries: one warp per (segment, query).
__global__ void __launch_bounds__(32 * AT_MAX_QUERIES)
attention_combine_kernel(const __grid_constant__ AttentionParams p) {
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int64_t seg = blockIdx.x;
    const int R = p.n_queries;
    const float* base = p.work + (seg * p.splits * R + r) * AT_PART_FLOATS;
    const int64_t stride = (int64_t)R * AT_PART_FLOATS;
    float mm = -INFINITY;
    for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, base[s * stride]);
    float2 a = make_float2(0.0f, 0.0f);
    float ll = 0.0f;
    for (int s = 0; s < p.splits; ++s) {
        const float* src = base + s * stride;
        const float f = src[0] == -INFINITY ? 0.0f : fast_exp2(src[0] - mm);        // an empty slice
        const float2 v = *reinterpret_cast<const float2*>(src + 2 + 2 * lane);
        a.x += v.x * f;
        a.y += v.y * f;
        ll += src[1] * f;
    }
    // normalise, then rotate back once: H over 64 coordinates (two per lane), 1/8, sign diagonal
    const float inv = 0.125f / ll;
    float x0 = a.x + a.y, x1 = a.x - a.y;                    // stage 1 inside the lane
#pragma unroll
    for (int mbit = 1; mbit < 32; mbit <<= 1) {              // stages 2 ... 32 across lanes
        const float o0 = __shfl_xor_sync(0xFFFFFFFFu, x0, mbit), o1 = __shfl_xor_sync(0xFFFFFFFFu, x1, mbit);
        const bool upper = (lane & mbit) != 0;
        x0 = upper ? o0 - x0 : x0 + o0;
        x1 = upper ? o1 - x1 : x1 + o1;
    }
    const uint32_t neg = lane < 16 ? p.neg_lo : p.neg_hi;
    const int bit = (2 * lane) & 31;
    x0 = flip_if(x0 * inv, neg, bit);
    x1 = flip_if(x1 * inv, neg, bit + 1);
    *reinterpret_cast<float2*>(p.out + (seg * R + r) * 64 + 2 * lane) = make_float2(x0, x1);
}

}  // namespace pitch
