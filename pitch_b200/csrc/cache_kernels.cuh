// Whole-cache decode for head dimensions 64 and 128 at 3 or 4 bits: the per-step bottleneck
// of a compressed KV cache (all tokens of every layer and KV head are decoded each step).
//
// One persistent launch covers every plane (K, V) and every segment (layer x KV head): one CTA
// of 16 warps per SM; a warp takes work items round-robin - an item is 2048 consecutive
// coordinates of one plane of one segment (32 tokens at dim 64, 16 at dim 128) - and the loads
// of the next item are in flight while the current one is decoded.  Per token the kernel reads
// dim*bits/8 code bytes plus 4 bytes of side information and writes dim elements, so it is bound
// by HBM traffic as long as the instruction count per token stays low; the two paths are built
// around that:
//
//   * TurboQuant plane - a lane owns 64 consecutive coordinates (a whole vector at dim 64, half
//     of one at dim 128).  Each pair of adjacent codes (a, b) - one byte at 4 bits, a 6-bit field
//     at 3 bits - indexes a table in shared memory that holds (c[a] + c[b], c[a] - c[b]), i.e.
//     centroid lookup and the first Walsh-Hadamard stage in one 64-bit load.  The table is
//     replicated over 32 lane slots (entry e, slot l at byte e*256 + l*8), so a lookup is
//     bank-conflict free for any codes and, at 4 bits, its address is a single byte permute of the
//     code word.  Stages 2...32 run on float2 pairs with packed fp32x2 instructions; at dim 128
//     the last stage is one exchange between the two lanes of a vector.  The result is scaled,
//     rounded, sign-flipped as packed words, and leaves through a padded warp-private shared tile
//     so that every global store instruction writes 512 contiguous bytes per warp.
//   * per-channel plane (4 bits) - a lane owns 8 channels ("slab") of every 4th (dim 64) or 2nd
//     (dim 128) token of the item; codes become floats by byte permutes into the mantissa of
//     2^23; loads are 4 bytes and stores 16 bytes per lane, both contiguous across the warp.
#pragma once

#include "channel_kernels.cuh"
#include "common.cuh"

namespace pitch {

constexpr int CD_THREADS = 512;
constexpr int CD_WARPS = CD_THREADS / 32;
constexpr int CD_TABLE_BYTES = 256 * 32 * 8;   // byte-pair table: 256 entries x 32 lane slots x float2

struct Book16 { float c[16]; };     // TurboQuant centroids, 2^bits of them used

// float2 arithmetic on the packed fp32x2 pipe; each component is one IEEE rounding.
// Caution, measured on sm_100a: a packed multiply whose only use is a packed add is contracted
// into one fused operation by the assembler even for the round-to-nearest forms and with
// contraction disabled.  Where the two roundings matter (per-channel decode) the add is
// therefore done per component with scalar round-to-nearest adds, which are never contracted.
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return __ffma2_rn(b, make_float2(-1.0f, -1.0f), a); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 mul2_then_add(float2 a, float2 b, float2 c) {
    const float2 m = __fmul2_rn(a, b);
    return make_float2(__fadd_rn(m.x, c.x), __fadd_rn(m.y, c.y));
}

// Walsh-Hadamard stages h = 2, 4, ..., 32 on 64 values held as 32 adjacent pairs
// (pair p = elements 2p, 2p+1); stage h = 1 is already folded into the table lookup.
__device__ __forceinline__ void wht64_pairs_from_stage2(float2 (&v)[32]) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {          // pair-index bit h = element bit 2h
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (!(i & h)) {
                const float2 a = v[i], b = v[i | h];
                v[i] = add2(a, b);
                v[i | h] = sub2(a, b);
            }
        }
    }
}

template <typename T> struct PairStore;   // 32 float2 -> this lane's 64-element row in the staging tile
template <> struct PairStore<float> {
    static __device__ __forceinline__ void row(const float2 (&v)[32], const uint32_t* sign, unsigned char* dst) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint2 m = *reinterpret_cast<const uint2*>(sign + 2 * j);      // same address in every lane: broadcast
            uint4 q;
            q.x = __float_as_uint(v[2 * j].x) ^ ((m.x & 0x8000u) << 16);
            q.y = __float_as_uint(v[2 * j].y) ^ (m.x & 0x80000000u);
            q.z = __float_as_uint(v[2 * j + 1].x) ^ ((m.y & 0x8000u) << 16);
            q.w = __float_as_uint(v[2 * j + 1].y) ^ (m.y & 0x80000000u);
            *reinterpret_cast<uint4*>(dst + j * 16) = q;
        }
    }
};
template <> struct PairStore<__half> {
    static __device__ __forceinline__ uint32_t cvt(float2 f) {
        const __half2 h = __float22half2_rn(f);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    static __device__ __forceinline__ void row(const float2 (&v)[32], const uint32_t* sign, unsigned char* dst) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint4 m = *reinterpret_cast<const uint4*>(sign + 4 * j);      // same address in every lane: broadcast
            *reinterpret_cast<uint4*>(dst + j * 16) =
                make_uint4(cvt(v[4 * j]) ^ m.x, cvt(v[4 * j + 1]) ^ m.y, cvt(v[4 * j + 2]) ^ m.z, cvt(v[4 * j + 3]) ^ m.w);
        }
    }
};
template <> struct PairStore<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t cvt(float2 f) {
        const __nv_bfloat162 h = __float22bfloat162_rn(f);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    static __device__ __forceinline__ void row(const float2 (&v)[32], const uint32_t* sign, unsigned char* dst) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint4 m = *reinterpret_cast<const uint4*>(sign + 4 * j);      // same address in every lane: broadcast
            *reinterpret_cast<uint4*>(dst + j * 16) =
                make_uint4(cvt(v[4 * j]) ^ m.x, cvt(v[4 * j + 1]) ^ m.y, cvt(v[4 * j + 2]) ^ m.z, cvt(v[4 * j + 3]) ^ m.w);
        }
    }
};

// What one lane needs from global memory to decode its share of one work item.  Fetched one
// item ahead of its use, so the loads of item k+1 are in flight while item k is being decoded.
struct Prefetch64 {
    uint4 a, b;   // TurboQuant: the lane's code bytes (32 at 4 bits, 24 at 3).  Per-channel: code words of tokens k*TOK_LANES + tok_lane, k = 0..7
    uint4 c, d;   // TurboQuant: c.x = norm bits.  Per-channel: fp16 minima (c) and maxima (d) of the lane's 8 channels
};

// Geometry of a work item for head dimension D.
template <int D> struct Item64 {
    static constexpr int LPV = D / 64;          // lanes per vector (TurboQuant)
    static constexpr int TOKENS = 32 / LPV;     // tokens per item
    static constexpr int SLABS = D / 8;         // 8-channel slabs per token (per-channel)
    static constexpr int TOK_LANES = 32 / SLABS;
};

// FULL: all tokens of the item exist (no bounds checks); otherwise nvalid in 1...TOKENS-1.
// `codes` points at the item's first code byte, `norms` at its first norm.
template <int D, int BITS, bool FULL>
__device__ __forceinline__ void prefetch_turbo64(Prefetch64& f, const unsigned char* __restrict__ codes,
                                                 const float* __restrict__ norms, int nvalid, int lane) {
    constexpr int LPV = Item64<D>::LPV;
    f.a = f.b = make_uint4(0, 0, 0, 0);
    f.c.x = 0;
    if (FULL || lane / LPV < nvalid) {
        if (BITS == 4) {
            f.a = ldg_stream(reinterpret_cast<const uint4*>(codes) + 2 * lane);
            f.b = ldg_stream(reinterpret_cast<const uint4*>(codes) + 2 * lane + 1);
        } else {
            const uint2* q = reinterpret_cast<const uint2*>(codes) + 3 * lane;      // 24 bytes per lane
            const uint2 q0 = ldg_stream64(q), q1 = ldg_stream64(q + 1), q2 = ldg_stream64(q + 2);
            f.a = make_uint4(q0.x, q0.y, q1.x, q1.y);
            f.b = make_uint4(q2.x, q2.y, 0, 0);
        }
        f.c.x = ldg_stream32(reinterpret_cast<const uint32_t*>(norms) + lane / LPV);
    }
}

template <int D, bool FULL>
__device__ __forceinline__ void prefetch_channel64(Prefetch64& f, const uint32_t* __restrict__ codes,
                                                   const __half* __restrict__ group_ranges, int nvalid, int lane) {
    constexpr int SLABS = Item64<D>::SLABS, TOK_LANES = Item64<D>::TOK_LANES;
    const int slab = lane & (SLABS - 1), tok_lane = lane / SLABS;
    const uint32_t* mine = codes + lane;      // token k*TOK_LANES + tok_lane, slab: word k*32 + lane
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        w[k] = 0;
        if (FULL || TOK_LANES * k + tok_lane < nvalid) w[k] = ldg_stream32(mine + 32 * k);
    }
    f.a = make_uint4(w[0], w[1], w[2], w[3]);
    f.b = make_uint4(w[4], w[5], w[6], w[7]);
    f.c = __ldg(reinterpret_cast<const uint4*>(group_ranges + slab * 8));
    f.d = __ldg(reinterpret_cast<const uint4*>(group_ranges + D + slab * 8));
}

// Byte offset into the pair table of code pair p (codes 2p, 2p+1 of the lane's 64), lane slot included.
template <int BITS>
__device__ __forceinline__ uint32_t pair_offset(const uint32_t (&w)[8], int p, uint32_t slot) {
    if (BITS == 4) {
        // byte p of the code words -> (byte << 8) | slot with one permute
        return __byte_perm(w[p >> 2], slot, 0x5504 | ((p & 3) << 4));
    } else {
        const int bit = 6 * p, word = bit >> 5, off = bit & 31;       // 6-bit field, may straddle two words
        uint32_t x;
        if (off + 6 <= 32) x = off >= 8 ? (w[word] >> (off - 8)) : (w[word] << (8 - off));
        else x = __funnelshift_r(w[word], w[word + 1], off - 8);
        return (x & 0x3F00u) | slot;
    }
}

// ---- exact key-bias removal inside the decode (reference/mechanism_eval.py:82-91) -----------------
// R_t b for coordinate c: fl(fl(b[c] * cos[t][c]) + fl(rh[c] * sin[t][c])), rh = rotate_half(b) =
// (-b[D/2:], b[:D/2]): the arithmetic of rope_bias_kernel, one rounding per operation.
__device__ __forceinline__ float rotated_bias_at(float b, float rh, float c, float s) {
    return __fadd_rn(__fmul_rn(b, c), __fmul_rn(rh, s));
}

// The rotary tables of one token block (TOKENS tokens) staged in shared memory: token t, table j
// (0 cosine, 1 sine), 4-float chunk q at chunk index (t*2 + j) * D/4 + (q ^ ((q >> 3) & 1)).  The
// swizzle makes the two access patterns of the decoders (8 lanes reading every second chunk, or 8
// lanes reading 8 consecutive chunks) free of bank conflicts.
template <int D>
__device__ __forceinline__ float4 tile_chunk(const float* tile, int t, int j, int q) {
    return reinterpret_cast<const float4*>(tile)[(t * 2 + j) * (D / 4) + (q ^ ((q >> 3) & 1))];
}

// b and rotate_half(b) for N consecutive coordinates starting at c0 (a multiple of N, N <= 8, so the
// block lies in one half of the vector); brow is the segment's bias row in global memory.
template <int D, int N>
__device__ __forceinline__ void load_bias_block(const float* __restrict__ brow, int c0, float (&b)[N], float (&rh)[N]) {
    const bool low = c0 < D / 2;
    const float* partner = brow + (low ? c0 + D / 2 : c0 - D / 2);
#pragma unroll
    for (int i = 0; i < N; ++i) {
        b[i] = __ldg(brow + c0 + i);
        const float o = __ldg(partner + i);
        rh[i] = low ? -o : o;
    }
}

// x[i] -> T(T(x[i]) + R_t b): what a separate pass over the stored (already rounded) output gives.
// cq = index of this lane's N-coordinate block inside the vector, t = token inside the block's tile.
template <typename T, int D, int N>
__device__ __forceinline__ void add_bias_block(float (&x)[N], const float* tile, int t, int cq, const float (&b)[N],
                                               const float (&rh)[N]) {
    float c[N], s[N];
#pragma unroll
    for (int h = 0; h < N / 4; ++h) {
        const float4 c4 = tile_chunk<D>(tile, t, 0, cq * (N / 4) + h), s4 = tile_chunk<D>(tile, t, 1, cq * (N / 4) + h);
        c[4 * h] = c4.x; c[4 * h + 1] = c4.y; c[4 * h + 2] = c4.z; c[4 * h + 3] = c4.w;
        s[4 * h] = s4.x; s[4 * h + 1] = s4.y; s[4 * h + 2] = s4.z; s[4 * h + 3] = s4.w;
    }
    // two coordinates at a time on the packed pipe: both products packed, their sum with scalar adds (a
    // packed add fed only by a packed multiply would be fused into one operation by the assembler and
    // lose a rounding), the final add packed again.  Same roundings as rotated_bias_at.
#pragma unroll
    for (int i = 0; i < N; i += 2) {
        const float2 pc = __fmul2_rn(make_float2(b[i], b[i + 1]), make_float2(c[i], c[i + 1]));
        const float2 ps = __fmul2_rn(make_float2(rh[i], rh[i + 1]), make_float2(s[i], s[i + 1]));
        const float2 rb = make_float2(__fadd_rn(pc.x, ps.x), __fadd_rn(pc.y, ps.y));
        const float2 y = __fadd2_rn(make_float2(x[i], x[i + 1]), rb);
        x[i] = y.x;
        x[i + 1] = y.y;
    }
}

// 64 coordinates per lane (BITS-bit codes): a whole vector at D = 64, half of one at D = 128.
// `table` is the pair table, `sign` 32 words for this lane's 64 coordinates whose bit 15 / bit 31 say
// whether coordinate 2p / 2p+1 is negated by the rotation's diagonal.  `out` points at the item's
// first output element.
// BIAS: the rotated key bias of each token (tables of the token block in `tile`, the segment's bias row
// at `brow`) is added to the rounded output on its way from the staging tile to global memory.
template <typename T, int D, int BITS, bool FULL, bool BIAS = false>
__device__ __forceinline__ void turbo64_decode_warp(const Prefetch64& f, T* __restrict__ out, int nvalid,
                                                    const unsigned char* table, const uint32_t* sign,
                                                    unsigned char* stage, int lane, float rs,
                                                    const float* tile = nullptr, const float* brow = nullptr) {
    typedef WarpStage<T, 64> Stage;
    const uint32_t w[8] = {f.a.x, f.a.y, f.a.z, f.a.w, f.b.x, f.b.y, f.b.z, f.b.w};
    const float norm = __uint_as_float(f.c.x);
    const uint32_t slot = (uint32_t)lane * 8u;
    float2 v[32];
    if (D == 128 && BITS == 4) {
        // The stage that pairs coordinate i with i + 64 (held by the other lane of the pair) is done
        // first and inside the table: the lanes swap their 32 code bytes (8 shuffles instead of the
        // 64 a float exchange takes), each interleaves its own nibbles with the partner's, and the
        // table gives c[own] + c[partner] to even lanes (output coordinates 0...63) and
        // c[partner] - c[own] to odd lanes (64...127) in one 4-byte lookup.
        const uint32_t slot4 = (uint32_t)lane * 4u;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, w[k], 1);
            const uint32_t even = (w[k] & 0x0F0F0F0Fu) | ((other << 4) & 0xF0F0F0F0u);     // coordinates 8k, 8k+2, 8k+4, 8k+6
            const uint32_t odd = ((w[k] >> 4) & 0x0F0F0F0Fu) | (other & 0xF0F0F0F0u);      // coordinates 8k+1, ...
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float x = *reinterpret_cast<const float*>(table + __byte_perm(even, slot4, 0x5504 | (j << 4)));
                const float y = *reinterpret_cast<const float*>(table + __byte_perm(odd, slot4, 0x5504 | (j << 4)));
                v[4 * k + j] = make_float2(x + y, x - y);                                   // stage 1
            }
        }
        wht64_pairs_from_stage2(v);
        const float2 r2 = make_float2(rs, rs), n2 = make_float2(norm, norm);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = mul2(mul2(v[i], r2), n2);
        PairStore<T>::row(v, sign, stage + lane * Stage::PITCHB);
    } else {
#pragma unroll
    for (int p = 0; p < 32; ++p) v[p] = *reinterpret_cast<const float2*>(table + pair_offset<BITS>(w, p, slot));
    wht64_pairs_from_stage2(v);
    if (D == 128) {
        // stage 64: coordinate i of the even lane pairs with coordinate i of the odd lane
        const float sg = (lane & 1) ? -1.0f : 1.0f;
        const float2 sgn = make_float2(sg, sg);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float2 o;
            o.x = __shfl_xor_sync(0xFFFFFFFFu, v[i].x, 1);
            o.y = __shfl_xor_sync(0xFFFFFFFFu, v[i].y, 1);
            v[i] = __ffma2_rn(v[i], sgn, o);          // even: v + o, odd: o - v
        }
        const float2 r2 = make_float2(rs, rs), n2 = make_float2(norm, norm);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = mul2(mul2(v[i], r2), n2);
    } else {
        // 1/sqrt(64) is a power of two, so (x * rs) * norm == x * (rs * norm) in float32.
        const float sc = 0.125f * norm;
        const float2 scale = make_float2(sc, sc);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = mul2(v[i], scale);
    }
    PairStore<T>::row(v, sign, stage + lane * Stage::PITCHB);
    }
    __syncwarp();
    // transposed read-out: chunk c = k*32 + lane of the item's contiguous output
    const unsigned char* src = stage + (lane / Stage::CPR) * Stage::PITCHB + (lane % Stage::CPR) * 16;
    uint4* dst = reinterpret_cast<uint4*>(out) + lane;
    const int valid_chunks = nvalid * (D / Stage::EPC);
    if constexpr (BIAS) {
        constexpr int EPC = Stage::EPC, CPT = D / EPC;            // elements per 16-byte chunk, chunks per token
        const int cq = lane % CPT;                                // this lane's coordinate block, the same for every k
        float bb[EPC], rh[EPC];
        load_bias_block<D, EPC>(brow, cq * EPC, bb, rh);
#pragma unroll
        for (int k = 0; k < Stage::CPR; ++k) {
            const uint4 q = *reinterpret_cast<const uint4*>(src + k * (32 / Stage::CPR) * Stage::PITCHB);
            if (FULL || k * 32 + lane < valid_chunks) {
                uint32_t w4[4] = {q.x, q.y, q.z, q.w};
                float x[EPC];
                Packer<T, EPC>::unpack(w4, x);
                add_bias_block<T, D, EPC>(x, tile, (k * 32 + lane) / CPT, cq, bb, rh);
                Packer<T, EPC>::pack(x, w4);
                stg_stream(dst + k * 32, make_uint4(w4[0], w4[1], w4[2], w4[3]));
            }
        }
    } else {
#pragma unroll
        for (int k = 0; k < Stage::CPR; ++k) {
            const uint4 q = *reinterpret_cast<const uint4*>(src + k * (32 / Stage::CPR) * Stage::PITCHB);
            if (FULL || k * 32 + lane < valid_chunks) stg_stream(dst + k * 32, q);
        }
    }
    __syncwarp();
}

// float(code) for the 8 codes of a word without integer-to-float conversions: the code byte is
// permuted into the mantissa of 2^23 (0x4B0000cc = 2^23 + code exactly), then 2^23 is subtracted.
// Returned as adjacent pairs for the packed pipe.
__device__ __forceinline__ void codes8_to_pairs(uint32_t w, float2 (&f)[4]) {
    const uint32_t even = w & 0x0F0F0F0Fu, odd = (w >> 4) & 0x0F0F0F0Fu;
    const float2 magic = make_float2(8388608.0f, 8388608.0f);
    f[0] = sub2(make_float2(__uint_as_float(__byte_perm(even, 0x4B000000u, 0x7440)),
                            __uint_as_float(__byte_perm(odd, 0x4B000000u, 0x7440))), magic);
    f[1] = sub2(make_float2(__uint_as_float(__byte_perm(even, 0x4B000000u, 0x7441)),
                            __uint_as_float(__byte_perm(odd, 0x4B000000u, 0x7441))), magic);
    f[2] = sub2(make_float2(__uint_as_float(__byte_perm(even, 0x4B000000u, 0x7442)),
                            __uint_as_float(__byte_perm(odd, 0x4B000000u, 0x7442))), magic);
    f[3] = sub2(make_float2(__uint_as_float(__byte_perm(even, 0x4B000000u, 0x7443)),
                            __uint_as_float(__byte_perm(odd, 0x4B000000u, 0x7443))), magic);
}

template <typename T> struct Pairs8;   // 4 float2 -> 8 elements of T, stored as one or two 16-byte pieces
template <> struct Pairs8<float> {
    // A lane's 8 floats are 32 bytes.  Adjacent lanes (slabs 2j, 2j+1) swap 16-byte halves first, so
    // that each store instruction fills whole 32-byte sectors (lane pair -> 32 contiguous bytes)
    // instead of half of every sector.  Must be called by all lanes of the warp.
    static __device__ __forceinline__ void store(float* p, const float2 (&v)[4], bool write = true) {
        const bool odd = threadIdx.x & 1;
        // even lane gives away its second half, odd lane its first half
        const float2 g0 = odd ? v[0] : v[2], g1 = odd ? v[1] : v[3];
        float2 r0, r1;
        r0.x = __shfl_xor_sync(FULL, g0.x, 1); r0.y = __shfl_xor_sync(FULL, g0.y, 1);
        r1.x = __shfl_xor_sync(FULL, g1.x, 1); r1.y = __shfl_xor_sync(FULL, g1.y, 1);
        // even lane: own first half at +0, partner's first half at +32 (partner's slab base is +32 bytes)
        // odd lane: partner's second half at partner's +16, own second half at own +16
        const float2 a0 = odd ? r0 : v[0], a1 = odd ? r1 : v[1];      // goes to the lower 32-byte sector of the pair
        const float2 b0 = odd ? v[2] : r0, b1 = odd ? v[3] : r1;      // goes to the upper 32-byte sector of the pair
        float* pair_base = p - (odd ? 8 : 0);                         // first float of the even lane's slab
        if (write) {
            stg_stream(reinterpret_cast<uint4*>(pair_base) + (odd ? 1 : 0),
                       make_uint4(__float_as_uint(a0.x), __float_as_uint(a0.y), __float_as_uint(a1.x), __float_as_uint(a1.y)));
            stg_stream(reinterpret_cast<uint4*>(pair_base) + (odd ? 3 : 2),
                       make_uint4(__float_as_uint(b0.x), __float_as_uint(b0.y), __float_as_uint(b1.x), __float_as_uint(b1.y)));
        }
    }
};
template <> struct Pairs8<__half> {
    static __device__ __forceinline__ void store(__half* p, const float2 (&v)[4], bool write = true) {
        if (write) stg_stream(reinterpret_cast<uint4*>(p), make_uint4(PairStore<__half>::cvt(v[0]), PairStore<__half>::cvt(v[1]),
                                                           PairStore<__half>::cvt(v[2]), PairStore<__half>::cvt(v[3])));
    }
};
template <> struct Pairs8<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float2 (&v)[4], bool write = true) {
        if (write) stg_stream(reinterpret_cast<uint4*>(p),
                   make_uint4(PairStore<__nv_bfloat16>::cvt(v[0]), PairStore<__nv_bfloat16>::cvt(v[1]),
                              PairStore<__nv_bfloat16>::cvt(v[2]), PairStore<__nv_bfloat16>::cvt(v[3])));
    }
};

// (hi - lo) / 15, correctly rounded, as a multiply by the rounded reciprocal and two fused
// corrections (q = x*r; q += fma(-15, q, x) * r).  Checked against the IEEE quotient for every
// non-negative float32 x, subnormals included; the result is then forced to 1 when it is 0,
// as the specification does for a constant channel.
__device__ __forceinline__ float step15(float lo, float hi) {
    const float x = hi - lo;
    const float r = 1.0f / 15.0f;
    const float q = x * r;
    const float s = __fmaf_rn(__fmaf_rn(-15.0f, q, x), r, q);
    return s == 0.0f ? 1.0f : s;
}

// TOKENS tokens (4-bit codes, all inside one group) per warp: lane = (token lane, slab).
// code * step + lo with one rounding per operation.
template <typename T, int D, bool FULL, bool BIAS = false>
__device__ __forceinline__ void channel64_decode_warp(const Prefetch64& f, T* __restrict__ out, int nvalid, int lane,
                                                      const float* tile = nullptr, const float* brow = nullptr) {
    constexpr int SLABS = Item64<D>::SLABS, TOK_LANES = Item64<D>::TOK_LANES;
    const int tok_lane = lane / SLABS, slab = lane & (SLABS - 1);
    const uint32_t w[8] = {f.a.x, f.a.y, f.a.z, f.a.w, f.b.x, f.b.y, f.b.z, f.b.w};
    const uint32_t lo16[4] = {f.c.x, f.c.y, f.c.z, f.c.w}, hi16[4] = {f.d.x, f.d.y, f.d.z, f.d.w};
    float2 lo[4], step[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        lo[i] = __half22float2(*reinterpret_cast<const __half2*>(&lo16[i]));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&hi16[i]));
        step[i] = make_float2(step15(lo[i].x, hi.x), step15(lo[i].y, hi.y));
    }
    float bb[8], rh[8];
    if constexpr (BIAS) load_bias_block<D, 8>(brow, slab * 8, bb, rh);
    T* mine = out + lane * 8;                 // token k*TOK_LANES + tok_lane, slab: element k*256 + lane*8
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float2 v[4];
        codes8_to_pairs(w[k], v);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = mul2_then_add(v[i], step[i], lo[i]);
        if constexpr (BIAS) {
            // the value as stored by a decode without the option (rounded to T), plus R_t b
            float x[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                x[2 * i] = Elem<T>::to_f32(Elem<T>::from_f32(v[i].x));
                x[2 * i + 1] = Elem<T>::to_f32(Elem<T>::from_f32(v[i].y));
            }
            add_bias_block<T, D, 8>(x, tile, TOK_LANES * k + tok_lane, slab, bb, rh);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = make_float2(x[2 * i], x[2 * i + 1]);
        }
        Pairs8<T>::store(mine + 256 * k, v, FULL || TOK_LANES * k + tok_lane < nvalid);
    }
}

struct Plane64 {
    int kind;                 // 0 = TurboQuant, 1 = per-channel
    int group_items;          // per-channel planes: group size / tokens per item
    uint32_t neg[4];          // rotation diagonal: bit i of word j set when coordinate 32j + i is negated
    const unsigned char* codes;
    int64_t codes_seg_stride;
    const unsigned char* side;
    int64_t side_seg_stride;
    unsigned char* out;
    int64_t out_seg_stride;
};

// What a step (append one token, then decode) needs on top of Plane64.
struct StepPlane {
    const unsigned char* in;      // new token of segment s at in + s * in_seg_stride: dim elements of in_dtype
    int64_t in_seg_stride;
    float* residual;              // per-channel planes: [segments][group + 2][dim] float32 (tokens, running min, running max)
    int64_t residual_seg_elems;
};

// Device-side token counter of a cache (pitch_cache_state of the C interface).
struct CacheState {
    long long tokens;
    int status;
    unsigned arrivals;
};

struct Cache64Params {
    int n_planes;
    int segments;
    int append;               // 0: decode `tokens` tokens.  1: append one token at position `tokens`, then decode tokens + 1
    int in_dtype;             // element type of the new tokens (0 float32, 1 float16, 2 bfloat16)
    int64_t tokens;           // tokens held before the launch (read from *state instead when state is set)
    int64_t capacity;         // append with a device-side counter: refuse when tokens >= capacity
    CacheState* state;
    float rs;                 // 1/sqrt(dim), correctly rounded
    Plane64 plane[4];
    StepPlane step[4];
    Book16 book;              // TurboQuant centroids for (dim, bits)
    // exact key-bias removal on plane 0 (cache_decode_bias_kernel only)
    const unsigned char* bias;      // float32 [segments][dim]
    int64_t bias_seg_stride;
    const float* cos_table;         // float32 [positions][dim]
    const float* sin_table;
};

constexpr int CD_SIGN_BYTES = 4 * 64 * 4;      // [plane][pair of the vector] sign words
constexpr int CD_EDGE_BYTES = 16 * 4;          // TurboQuant decision boundaries (append)
template <typename T>
constexpr int cache64_smem_bytes() { return CD_TABLE_BYTES + CD_SIGN_BYTES + CD_EDGE_BYTES + CD_WARPS * WarpStage<T, 64>::BYTES; }

// A work item: 2048 coordinates of one plane of one segment.
struct Cursor64 {
    int pl, seg, item;
};

__device__ __forceinline__ float load_elem_f32(const unsigned char* p, int dtype, int idx) {
    if (dtype == 0) return reinterpret_cast<const float*>(p)[idx];
    if (dtype == 1) return __half2float(reinterpret_cast<const __half*>(p)[idx]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
}
__device__ __forceinline__ float round_to_dtype(float v, int dtype) {
    if (dtype == 0) return v;
    if (dtype == 1) return __half2float(__float2half_rn(v));
    return __bfloat162float(__float2bfloat16_rn(v));
}

// Key-bias removal for the token a step appends: the segment's bias row and the rotary table rows of
// the token's position (all in global memory).  A null brow means "no bias".
struct RopeNew {
    const float* brow;
    const float* cos_row;
    const float* sin_row;
};

// x - R_t b for coordinate c of the new token, rounded to the element type the token arrived in
// (what subtracting in place from a copy of the input gives).
template <int D>
__device__ __forceinline__ float remove_bias(float x, int c, const RopeNew& rn, int in_dtype) {
    const float b = __ldg(rn.brow + c);
    const float rh = c < D / 2 ? -__ldg(rn.brow + c + D / 2) : __ldg(rn.brow + c - D / 2);
    return round_to_dtype(__fsub_rn(x, rotated_bias_at(b, rh, __ldg(rn.cos_row + c), __ldg(rn.sin_row + c))), in_dtype);
}

// TurboQuant encode of ONE vector by a whole warp (the token a step appends): lane l owns the
// D/32 consecutive coordinates l*D/32 ...; the float operations and their order are those of
// turbo_encode_kernel (balanced adjacent-pair sum of squares, unit vector, sign flip,
// Walsh-Hadamard stages from the lowest coordinate bit up, 1/sqrt(D), number of decision
// boundaries strictly below).  Writes the packed codes and the norm to the cache and patches
// them into the prefetch registers of the lanes that decode this token, so the decode that
// follows does not depend on reading back what was just written.
template <int D, int BITS>
__device__ __forceinline__ void turbo_append_warp(Prefetch64& f, const unsigned char* __restrict__ in, int in_dtype,
                                                  uint32_t* __restrict__ codes_tok, float* __restrict__ norm_out,
                                                  int tok_in_item, const uint32_t* neg, const float* s_edges, float rs,
                                                  unsigned char* stage, int lane, const RopeNew rn = RopeNew{nullptr, nullptr, nullptr}) {
    constexpr int E = D / 32, LPV = Item64<D>::LPV, WPV = D * BITS / 32;
    float x[E], t[E];
#pragma unroll
    for (int i = 0; i < E; ++i) {
        x[i] = load_elem_f32(in, in_dtype, lane * E + i);
        if (rn.brow != nullptr) x[i] = remove_bias<D>(x[i], lane * E + i, rn, in_dtype);
        t[i] = x[i] * x[i];
    }
    const float norm = sqrtf(lanes_sum(tree_sum_regs(t), 32));
    const float inv = norm > 0.0f ? 1.0f / norm : 0.0f;
#pragma unroll
    for (int i = 0; i < E; ++i) {
        const int c = lane * E + i;
        x[i] = flip_if(x[i], neg[c >> 5], c & 31) * inv;
    }
    wht_regs(x, E);
    wht_lanes(x, 32, lane);
    uint32_t* s_code = reinterpret_cast<uint32_t*>(stage);          // D code values, then WPV packed words
    uint32_t* s_word = s_code + D;
#pragma unroll
    for (int i = 0; i < E; ++i) {
        const float u = x[i] * rs;
        uint32_t code = 0;
#pragma unroll
        for (int step = (1 << BITS) >> 1; step > 0; step >>= 1) {
            const uint32_t cand = code + step;
            if (u > s_edges[cand - 1]) code = cand;
        }
        s_code[lane * E + i] = code;
    }
    __syncwarp();
    if (lane < WPV) {
        const int bit0 = lane * 32;
        const int i0 = bit0 / BITS;
        int i1 = (bit0 + 31) / BITS;
        if (i1 > D - 1) i1 = D - 1;
        uint32_t word = 0;
        for (int i = i0; i <= i1; ++i) {
            const int shift = i * BITS - bit0;
            word |= shift >= 0 ? (s_code[i] << shift) : (s_code[i] >> (-shift));
        }
        s_word[lane] = word;
        codes_tok[lane] = word;
    }
    if (lane == 0) *norm_out = norm;
    __syncwarp();
    if (lane / LPV == tok_in_item) {
        const uint32_t* mine = s_word + (lane % LPV) * 2 * BITS;
        f.a = make_uint4(mine[0], mine[1], mine[2], mine[3]);
        f.b = BITS == 4 ? make_uint4(mine[4], mine[5], mine[6], mine[7]) : make_uint4(mine[4], mine[5], 0, 0);
        f.c.x = __float_as_uint(norm);
    }
    __syncwarp();
}

// The newest group of a per-channel plane during a step, one item of it per warp: fold the new
// token into the group's running range, re-quantise the item's tokens from the float32 residual
// against the new fp16 range (4-bit codes), store the codes, and decode them in the same breath.
// A group that spans several items is handled by several warps; each derives the new range on its
// own (minimum and maximum are idempotent, so it does not matter whether a warp sees the running
// range before or after the holder of the new token has updated it), and only the holder writes
// the residual row, the running range and the fp16 range.  Arithmetic as channel_encode_slab_kernel.
template <typename T, int D, bool BIAS = false>
__device__ __forceinline__ void channel_step_warp(const Plane64& P, const StepPlane& S, int in_dtype, int64_t seg,
                                                  int item, int64_t t_old, T* __restrict__ out, int nvalid, int lane,
                                                  const RopeNew rn = RopeNew{nullptr, nullptr, nullptr}, const float* tile = nullptr) {
    constexpr int SLABS = Item64<D>::SLABS, TOK_LANES = Item64<D>::TOK_LANES, TOKENS = Item64<D>::TOKENS;
    const int slab = lane & (SLABS - 1), tok_lane = lane / SLABS;
    const int G = P.group_items * TOKENS;
    const int64_t g = t_old / G;
    const int pos = (int)(t_old - g * G);                              // index of the new token inside its group
    const int j = item - (int)(g * P.group_items);                     // this item inside the group
    const bool holder = j == pos / TOKENS;
    float* res = S.residual + seg * S.residual_seg_elems;
    const unsigned char* in = S.in + seg * S.in_seg_stride;

    float xn[8], lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        xn[i] = load_elem_f32(in, in_dtype, slab * 8 + i);
        if (BIAS) xn[i] = remove_bias<D>(xn[i], slab * 8 + i, rn, in_dtype);
    }
    if (pos > 0) {
        const float4 l0 = *reinterpret_cast<const float4*>(res + (int64_t)G * D + slab * 8);
        const float4 l1 = *reinterpret_cast<const float4*>(res + (int64_t)G * D + slab * 8 + 4);
        const float4 h0 = *reinterpret_cast<const float4*>(res + (int64_t)(G + 1) * D + slab * 8);
        const float4 h1 = *reinterpret_cast<const float4*>(res + (int64_t)(G + 1) * D + slab * 8 + 4);
        const float rl[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
        const float rh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo[i] = fminf(rl[i], xn[i]);
            hi[i] = fmaxf(rh[i], xn[i]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) lo[i] = hi[i] = xn[i];
    }
    const bool writer = holder && tok_lane == 0;
    if (writer) {
        *reinterpret_cast<float4*>(res + (int64_t)G * D + slab * 8) = make_float4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<float4*>(res + (int64_t)G * D + slab * 8 + 4) = make_float4(lo[4], lo[5], lo[6], lo[7]);
        *reinterpret_cast<float4*>(res + (int64_t)(G + 1) * D + slab * 8) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<float4*>(res + (int64_t)(G + 1) * D + slab * 8 + 4) = make_float4(hi[4], hi[5], hi[6], hi[7]);
    }
    Prefetch64 f;
    float step[8], rcp[8];
    {
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
            step[2 * i] = step_of(lf.x, hf.x, 15.0f);
            step[2 * i + 1] = step_of(lf.y, hf.y, 15.0f);
        }
        f.c = make_uint4(lo_w[0], lo_w[1], lo_w[2], lo_w[3]);
        f.d = make_uint4(hi_w[0], hi_w[1], hi_w[2], hi_w[3]);
        if (writer) {
            __half* ranges = reinterpret_cast<__half*>(const_cast<unsigned char*>(P.side) + seg * P.side_seg_stride) + g * 2 * D;
            *reinterpret_cast<uint4*>(ranges + slab * 8) = f.c;
            *reinterpret_cast<uint4*>(ranges + D + slab * 8) = f.d;
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) rcp[i] = __frcp_rn(step[i]);

    uint32_t* item_codes = reinterpret_cast<uint32_t*>(const_cast<unsigned char*>(P.codes) + seg * P.codes_seg_stride +
                                                       (int64_t)item * 1024);
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int tg = j * TOKENS + k * TOK_LANES + tok_lane;          // token index inside the group
        w[k] = 0;
        if (tg <= pos) {
            float row[8];
            if (tg == pos) {
#pragma unroll
                for (int i = 0; i < 8; ++i) row[i] = xn[i];
                *reinterpret_cast<float4*>(res + (int64_t)pos * D + slab * 8) = make_float4(xn[0], xn[1], xn[2], xn[3]);
                *reinterpret_cast<float4*>(res + (int64_t)pos * D + slab * 8 + 4) = make_float4(xn[4], xn[5], xn[6], xn[7]);
            } else {
                const float4 r0 = *reinterpret_cast<const float4*>(res + (int64_t)tg * D + slab * 8);
                const float4 r1 = *reinterpret_cast<const float4*>(res + (int64_t)tg * D + slab * 8 + 4);
                row[0] = r0.x; row[1] = r0.y; row[2] = r0.z; row[3] = r0.w;
                row[4] = r1.x; row[5] = r1.y; row[6] = r1.z; row[7] = r1.w;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) w[k] |= quantise_rcp(row[i], lo[i], step[i], rcp[i], 15.0f) << (4 * i);
            item_codes[k * 32 + lane] = w[k];
        }
    }
    f.a = make_uint4(w[0], w[1], w[2], w[3]);
    f.b = make_uint4(w[4], w[5], w[6], w[7]);
    channel64_decode_warp<T, D, false, BIAS>(f, out, nvalid, lane, tile, rn.brow);
}

// grid = number of SMs (persistent), CD_THREADS threads, cache64_smem_bytes<T>() dynamic shared memory.
// D in {64, 128}; BITS in {3, 4} is the width of the TurboQuant planes (per-channel planes are 4-bit).
//
// Work of a launch that holds `total` tokens per segment after an optional append at position t_old:
//   * main items  - items [0, main) of every segment and plane, none touched by the append: the
//     software-pipelined, unchecked path.  main = total / tokens-per-item without an append; with
//     one it is the first item of the newest group of the per-channel planes (or of the new token).
//   * edge items  - items [main, ceil(total / tokens-per-item)): the partial last item, the items
//     of a per-channel plane's newest group (re-quantised from the residual) and the item that
//     receives the new TurboQuant vector (encoded by the warp that decodes it).  One warp each,
//     taken first, by the warps that come last in the round-robin of the main items.
//
// DEAL selects how the main items are dealt to the warps.  0: a fixed deal - warp w of CTA c is
// worker w * gridDim + c and takes every (gridDim * 16)-th position, planes innermost; nothing to compute
// per item.  1: the positions are dealt to the CTAs round-robin and the warps of a CTA draw them, one
// plane at a time, from a counter in shared memory as they become free: no warp idles at the end while
// another still has a whole item more to do, and warps that got the costlier items fall behind no one.
// That costs about 30 instructions per item.  It pays for a cache that mixes per-channel (cheap) and
// TurboQuant (costly) planes - 2.7 % of the whole step at config 4's size, 12 % for an eighth of it, where
// a warp has five items - and does not for a cache of TurboQuant planes only, whose launch is bound by
// instruction issue (6 % slower at config 5's shape): the host picks.
// DEAL 2 is the drawn deal plus a request to the L2, with every item fetched, for the item the CTA reaches 16
// positions later: worth its instructions (and registers) only where a warp has few items and the start of
// the launch weighs - a quarter or an eighth of config 4's cache: 23.3 -> 22.2 us and 13.7 -> 13.2 us per
// step; the whole cache loses to it, 81.4 -> 82.3 us.
template <typename T, int D, int BITS, int DEAL>
__global__ void __launch_bounds__(CD_THREADS, 1)
cache_decode_kernel(const __grid_constant__ Cache64Params p) {
    constexpr bool TICKETS = DEAL != 0;
    constexpr int TOKENS = Item64<D>::TOKENS, LPV = Item64<D>::LPV;
    constexpr int ITEM_CODE_BYTES = 32 * 8 * BITS;          // TurboQuant: 32 lanes x 64 codes
    constexpr int CH_ITEM_CODE_BYTES = 1024;                // per-channel, 4 bits: 2048 codes
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* table = smem;
    uint32_t* s_sign = reinterpret_cast<uint32_t*>(smem + CD_TABLE_BYTES);           // [4][64]
    float* s_edges = reinterpret_cast<float*>(smem + CD_TABLE_BYTES + CD_SIGN_BYTES);
    unsigned char* stage_base = smem + CD_TABLE_BYTES + CD_SIGN_BYTES + CD_EDGE_BYTES;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    bool any_turbo = false;
    for (int pl = 0; pl < p.n_planes; ++pl) any_turbo |= p.plane[pl].kind == 0;
    if (any_turbo) {
        constexpr int ENTRIES = 1 << (2 * BITS);
        for (int idx = threadIdx.x; idx < ENTRIES * 32; idx += CD_THREADS) {
            const int e = idx >> 5;
            const float a = p.book.c[e & ((1 << BITS) - 1)], b = p.book.c[e >> BITS];
            if (D == 128 && BITS == 4)      // 4-byte entries, own code in the low nibble: see turbo64_decode_warp
                *reinterpret_cast<float*>(table + e * 256 + (idx & 31) * 4) = (idx & 1) ? b - a : a + b;
            else
                *reinterpret_cast<float2*>(table + idx * 8) = make_float2(a + b, a - b);
        }
        if (threadIdx.x < 4 * 64) {
            const int pl = threadIdx.x >> 6, i = threadIdx.x & 63;       // packed pair i = coordinates 2i, 2i+1
            const uint32_t m = p.plane[pl].neg[i >> 4];
            const int bit = (2 * i) & 31;
            s_sign[threadIdx.x] = (((m >> bit) & 1u) << 15) | (((m >> (bit + 1)) & 1u) << 31);
        }
        if (threadIdx.x < (1 << BITS) - 1) s_edges[threadIdx.x] = 0.5f * (p.book.c[threadIdx.x] + p.book.c[threadIdx.x + 1]);
    }
    int* s_next = reinterpret_cast<int*>(s_edges) + 15;       // the CTA's work counter (the boundaries use 15 slots at most)
    if (TICKETS && threadIdx.x == 0) *s_next = 0;
    __syncthreads();
    // Everything above touched only kernel parameters and shared memory.  Under programmatic
    // dependent launch this grid may have started before the previous kernel of the stream ended:
    // wait for it (and for its memory to be visible) before reading the cache, then let the next
    // kernel of the stream be scheduled as soon as multiprocessors free up (it waits for this grid
    // in the same way before it touches memory).
    if (p.state == nullptr) {
        // While waiting: ask the L2 for the codes and side information of the items this CTA takes first
        // (drawn deal: those its first round of tickets stands for, warp w: ticket w; fixed deal: every plane
        // of the warp's first position), so that the first fetches after the wait do not start from a cold
        // cache.  A prefetch changes nothing that can be observed; the addresses are inside the planes'
        // buffers whatever the previous kernel is still writing there.  (Measured at config 4's size: 83.0 us
        // per step without, 81.5 us with one round, 81.7 with two, 82.4 with four.)
        const int items_guess = (int)(p.tokens / TOKENS);
        for (int k = TICKETS ? warp : 0; k < (TICKETS ? CD_WARPS : p.n_planes) && items_guess > 0; k += TICKETS ? CD_WARPS : 1) {
            const int kp = TICKETS ? k / p.n_planes : 0, pl = TICKETS ? k - kp * p.n_planes : k;
            const int64_t pos = TICKETS ? blockIdx.x + (int64_t)gridDim.x * kp : (int64_t)warp * gridDim.x + blockIdx.x;
            if (pos >= (int64_t)p.segments * items_guess) break;
            const int seg = (int)(pos / items_guess), item = (int)(pos - (int64_t)seg * items_guess);
            const Plane64& P = p.plane[pl];
            const unsigned char* codes = P.codes + seg * P.codes_seg_stride + (int64_t)item * (P.kind == 0 ? ITEM_CODE_BYTES : CH_ITEM_CODE_BYTES);
            const unsigned char* side = P.side + seg * P.side_seg_stride +
                                        (P.kind == 0 ? (int64_t)item * TOKENS * 4 : (int64_t)(item / P.group_items) * (2 * D) * 2);
            // whole 128-byte pieces inside the item's own bytes only (at least the piece its first byte lies in)
            const int code_lines = (P.kind == 0 ? ITEM_CODE_BYTES : CH_ITEM_CODE_BYTES) / 128;
            const int side_bytes = P.kind == 0 ? TOKENS * 4 : 2 * D * 2;
            const int side_lines = side_bytes >= 128 ? side_bytes / 128 : 1;
            if (lane < code_lines) asm volatile("prefetch.global.L2 [%0];" :: "l"(codes + lane * 128));
            else if (lane < code_lines + side_lines) asm volatile("prefetch.global.L2 [%0];" :: "l"(side + (lane - code_lines) * 128));
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    unsigned char* stage = stage_base + warp * WarpStage<T, 64>::BYTES;
    // warp w of CTA c is worker w * gridDim + c: when the item count is not a multiple of the worker
    // count, the workers that take one item more are spread evenly over the SMs
    const int warp_id = warp * gridDim.x + blockIdx.x;
    const int warp_stride = gridDim.x * CD_WARPS;
    const uint32_t* my_sign_base = s_sign + (LPV == 2 ? (lane & 1) * 32 : 0);

    // ---- geometry of this launch (uniform over the grid)
    const int64_t t_old = p.state != nullptr ? p.state->tokens : p.tokens;
    const bool refuse = p.append && p.state != nullptr && t_old >= p.capacity;
    const int64_t total = t_old + (p.append ? 1 : 0);
    const int last_items = (int)((total + TOKENS - 1) / TOKENS);          // items per segment and plane, partial one included
    int full_items = (int)(total / TOKENS);
    if (p.append) {
        full_items = (int)(t_old / TOKENS);
        for (int pl = 0; pl < p.n_planes; ++pl)
            if (p.plane[pl].kind == 1) {
                const int G = p.plane[pl].group_items * TOKENS;
                const int first = (int)(t_old / G) * p.plane[pl].group_items;
                full_items = first < full_items ? first : full_items;
            }
    }
    const int edge_items = last_items - full_items;

    // Addresses of an item.  Whole items take the FULL (unchecked) paths.
    auto fetch = [&](const Cursor64& c, Prefetch64& f) {
        const Plane64& P = p.plane[c.pl];
        const unsigned char* side = P.side + c.seg * P.side_seg_stride;
        if (P.kind == 0)
            prefetch_turbo64<D, BITS, true>(f, P.codes + c.seg * P.codes_seg_stride + (int64_t)c.item * ITEM_CODE_BYTES,
                                            reinterpret_cast<const float*>(side) + (int64_t)c.item * TOKENS, TOKENS, lane);
        else
            prefetch_channel64<D, true>(
                f, reinterpret_cast<const uint32_t*>(P.codes + c.seg * P.codes_seg_stride + (int64_t)c.item * CH_ITEM_CODE_BYTES),
                reinterpret_cast<const __half*>(side) + (int64_t)(c.item / P.group_items) * (2 * D), TOKENS, lane);
    };
    auto decode = [&](const Cursor64& c, const Prefetch64& f) {
        const Plane64& P = p.plane[c.pl];
        T* out = reinterpret_cast<T*>(P.out + c.seg * P.out_seg_stride) + (int64_t)c.item * 2048;
        if (P.kind == 0)
            turbo64_decode_warp<T, D, BITS, true>(f, out, TOKENS, table, my_sign_base + c.pl * 64, stage, lane, p.rs);
        else
            channel64_decode_warp<T, D, true>(f, out, TOKENS, lane);
    };
    // Next item of this warp: planes innermost, then the warp's next position (round-robin over the grid).
    auto advance = [&](Cursor64& c) {
        if (++c.pl < p.n_planes) return true;
        c.pl = 0;
        c.item += warp_stride;
        if (c.item >= full_items) {
            const int q = c.item / full_items;
            c.seg += q;
            c.item -= q * full_items;
        }
        return c.seg < p.segments;
    };
    // The drawn deal.  A ticket is drawn (by lane 0) one item ahead of its use, so that the counter's
    // latency is never on the warp's path: ticket() while an item is decoded, resolve() when the next one
    // is to be fetched.  (segments x items fits 31 bits: the host checks it.)
    const int positions = p.segments * full_items;
    const int my_positions = positions > (int)blockIdx.x ? (positions - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const float inv_items = full_items > 0 ? __frcp_rd(__int2float_ru(full_items)) : 0.0f;     // never above 1 / full_items
    auto ticket = [&]() { return lane == 0 ? atomicAdd(s_next, 1) : 0; };
    auto resolve = [&](int drawn, Cursor64& c) {
        const int k = __shfl_sync(0xFFFFFFFFu, drawn, 0);
        const int np = p.n_planes;
        const int kp = np == 2 ? (k >> 1) : (np == 1 ? k : k / np);
        if (kp >= my_positions) return false;
        const int pos = (int)blockIdx.x + (int)gridDim.x * kp;
        c.pl = k - kp * np;
        // pos / full_items without an integer division: every rounding of the float quotient goes down, so
        // it is the quotient or one less (segments < 2^16 keeps the error below one)
        int seg = __float2int_rd(__fmul_rd(__int2float_rd(pos), inv_items));
        int item = pos - seg * full_items;
        if (item >= full_items) { ++seg; item -= full_items; }
        c.seg = seg;
        c.item = item;
        return true;
    };

    // The item the CTA will reach AHEAD positions after the one just fetched (same plane): asked of the L2
    // now, so that whichever warp draws it finds its codes there.  Every item is asked for once, by the warp
    // that holds the ticket AHEAD positions before it.
    constexpr int AHEAD = 16;                         // 8 and 32 measured slower (a quarter of the cache: 22.5 and 23.0 us against 22.2)
    auto ask_ahead = [&](const Cursor64& c) {
        if constexpr (DEAL != 2) return;
        const int pos = c.seg * full_items + c.item + AHEAD * (int)gridDim.x;
        if (pos >= positions) return;
        int seg = __float2int_rd(__fmul_rd(__int2float_rd(pos), inv_items));
        int item = pos - seg * full_items;
        if (item >= full_items) { ++seg; item -= full_items; }
        const Plane64& P = p.plane[c.pl];
        const unsigned char* codes = P.codes + seg * P.codes_seg_stride + (int64_t)item * (P.kind == 0 ? ITEM_CODE_BYTES : CH_ITEM_CODE_BYTES);
        const int code_lines = (P.kind == 0 ? ITEM_CODE_BYTES : CH_ITEM_CODE_BYTES) / 128;
        if (lane < code_lines) asm volatile("prefetch.global.L2 [%0];" :: "l"(codes + lane * 128));
        else if (lane == code_lines && P.kind == 0)
            asm volatile("prefetch.global.L2 [%0];" :: "l"(P.side + seg * P.side_seg_stride + (int64_t)item * TOKENS * 4));
    };

    if (!refuse) {
    // ---- edge items: the partial last item and everything an append touches
    if (edge_items > 0) {
        const int per_seg = p.n_planes * edge_items;
        for (int work = warp_stride - 1 - warp_id; work < p.segments * per_seg; work += warp_stride) {
            const int seg = work / per_seg, r = work - seg * per_seg;
            const int pl = r / edge_items, item = full_items + (r - pl * edge_items);
            const Plane64& P = p.plane[pl];
            const int64_t left = total - (int64_t)item * TOKENS;
            const int nvalid = left < TOKENS ? (int)left : TOKENS;
            const unsigned char* side = P.side + seg * P.side_seg_stride;
            T* out = reinterpret_cast<T*>(P.out + seg * P.out_seg_stride) + (int64_t)item * 2048;
            Prefetch64 f;
            if (P.kind == 0) {
                const bool has_new = p.append && item == (int)(t_old / TOKENS);
                const unsigned char* item_codes = P.codes + seg * P.codes_seg_stride + (int64_t)item * ITEM_CODE_BYTES;
                const float* item_norms = reinterpret_cast<const float*>(side) + (int64_t)item * TOKENS;
                prefetch_turbo64<D, BITS, false>(f, item_codes, item_norms, has_new ? nvalid - 1 : nvalid, lane);
                if (has_new) {
                    const int tok = nvalid - 1;
                    turbo_append_warp<D, BITS>(f, p.step[pl].in + seg * p.step[pl].in_seg_stride, p.in_dtype,
                                               reinterpret_cast<uint32_t*>(const_cast<unsigned char*>(item_codes)) + tok * (D * BITS / 32),
                                               const_cast<float*>(item_norms) + tok, tok, P.neg, s_edges, p.rs, stage, lane);
                }
                turbo64_decode_warp<T, D, BITS, false>(f, out, nvalid, table, my_sign_base + pl * 64, stage, lane, p.rs);
            } else if (p.append && item / P.group_items == (int)(t_old / (P.group_items * TOKENS))) {
                channel_step_warp<T, D>(P, p.step[pl], p.in_dtype, seg, item, t_old, out, nvalid, lane);
            } else {
                prefetch_channel64<D, false>(
                    f, reinterpret_cast<const uint32_t*>(P.codes + seg * P.codes_seg_stride + (int64_t)item * CH_ITEM_CODE_BYTES),
                    reinterpret_cast<const __half*>(side) + (int64_t)(item / P.group_items) * (2 * D), nvalid, lane);
                channel64_decode_warp<T, D, false>(f, out, nvalid, lane);
            }
        }
    }

    // ---- main items, software pipelined with two register buffers used alternately
    if constexpr (TICKETS) {
        if (full_items > 0) {
            Cursor64 cur, nxt;
            int drawn = ticket();
            if (resolve(drawn, cur)) {
                Prefetch64 fa, fb;
                fetch(cur, fa);
                drawn = ticket();
#pragma unroll 1
                while (true) {
                    bool more = resolve(drawn, nxt);
                    if (more) { fetch(nxt, fb); drawn = ticket(); ask_ahead(nxt); }
                    decode(cur, fa);
                    if (!more) break;
                    cur = nxt;
                    more = resolve(drawn, nxt);
                    if (more) { fetch(nxt, fa); drawn = ticket(); ask_ahead(nxt); }
                    decode(cur, fb);
                    if (!more) break;
                    cur = nxt;
                }
            }
        }
    } else if (full_items > 0) {
        Cursor64 cur;
        cur.pl = 0;
        cur.seg = warp_id / full_items;
        cur.item = warp_id - cur.seg * full_items;
        if (cur.seg < p.segments) {
            Prefetch64 fa, fb;
            fetch(cur, fa);
#pragma unroll 1
            while (true) {
                Cursor64 nxt = cur;
                bool more = advance(nxt);
                if (more) fetch(nxt, fb);
                decode(cur, fa);
                if (!more) break;
                cur = nxt;
                more = advance(nxt);
                if (more) fetch(nxt, fa);
                decode(cur, fb);
                if (!more) break;
                cur = nxt;
            }
        }
    }
    }

    // ---- device-side token counter: the last CTA to finish publishes the new count.  The counter is
    // read again here (nothing has changed it since the start of the grid: only the last arrival
    // writes) so that no register has to carry it through the main loop.
    if (p.append && p.state != nullptr) {
        __syncthreads();
        if (threadIdx.x == 0) {
            const long long held = p.state->tokens;
            if (held >= p.capacity) {
                p.state->status = 1;
            } else {
                __threadfence();
                if (atomicAdd(&p.state->arrivals, 1u) == gridDim.x - 1) {
                    p.state->arrivals = 0;
                    p.state->tokens = held + 1;
                }
            }
        }
    }
}

// --------------------------------------------------------------------------------------------------
// The same launch with exact key-bias removal on plane 0 (README.md:100 of the reference lists it as
// missing from its kernels; arithmetic of rope_bias_kernel): the rotated bias R_t b of every token is
// added to the decoded keys on their way out, and taken off the new key before it is encoded, so the
// decoded keys never make a second trip through memory.  R_t b needs the rotary tables of the token:
// 2 x dim floats per token, four times the bf16 output of that token.  Read per item they would
// dominate the traffic, so the work is arranged by TOKEN BLOCK instead: a CTA takes one block of
// tokens (one item's worth), stages the block's cos/sin rows in shared memory once (asynchronous
// copies, the next block's rows in flight while this one is used), and its 16 warps then decode that
// block for every segment and plane.  The tables are read once per launch instead of once per segment.
// Results equal the launch without the option followed by the separate element-wise pass, bit for bit.
// --------------------------------------------------------------------------------------------------
constexpr int CD_TILE_BYTES = 2048 * 2 * 4;                   // cos and sin of one item's 2048 coordinates
template <typename T> struct TileBuffers { static constexpr int N = sizeof(T) == 2 ? 2 : 1; };
template <typename T>
constexpr int cache64_bias_smem_bytes() { return cache64_smem_bytes<T>() + TileBuffers<T>::N * CD_TILE_BYTES; }

template <typename T, int D, int BITS>
__global__ void __launch_bounds__(CD_THREADS, 1)
cache_decode_bias_kernel(const __grid_constant__ Cache64Params p) {
    constexpr int TOKENS = Item64<D>::TOKENS, LPV = Item64<D>::LPV;
    constexpr int ITEM_CODE_BYTES = 32 * 8 * BITS;
    constexpr int CH_ITEM_CODE_BYTES = 1024;
    constexpr int NBUF = TileBuffers<T>::N;
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* table = smem;
    uint32_t* s_sign = reinterpret_cast<uint32_t*>(smem + CD_TABLE_BYTES);
    float* s_edges = reinterpret_cast<float*>(smem + CD_TABLE_BYTES + CD_SIGN_BYTES);
    unsigned char* stage_base = smem + CD_TABLE_BYTES + CD_SIGN_BYTES + CD_EDGE_BYTES;
    float* tiles = reinterpret_cast<float*>(stage_base + CD_WARPS * WarpStage<T, 64>::BYTES);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    bool any_turbo = false;
    for (int pl = 0; pl < p.n_planes; ++pl) any_turbo |= p.plane[pl].kind == 0;
    if (any_turbo) {
        constexpr int ENTRIES = 1 << (2 * BITS);
        for (int idx = threadIdx.x; idx < ENTRIES * 32; idx += CD_THREADS) {
            const int e = idx >> 5;
            const float a = p.book.c[e & ((1 << BITS) - 1)], b = p.book.c[e >> BITS];
            if (D == 128 && BITS == 4)
                *reinterpret_cast<float*>(table + e * 256 + (idx & 31) * 4) = (idx & 1) ? b - a : a + b;
            else
                *reinterpret_cast<float2*>(table + idx * 8) = make_float2(a + b, a - b);
        }
        if (threadIdx.x < 4 * 64) {
            const int pl = threadIdx.x >> 6, i = threadIdx.x & 63;
            const uint32_t m = p.plane[pl].neg[i >> 4];
            const int bit = (2 * i) & 31;
            s_sign[threadIdx.x] = (((m >> bit) & 1u) << 15) | (((m >> (bit + 1)) & 1u) << 31);
        }
        if (threadIdx.x < (1 << BITS) - 1) s_edges[threadIdx.x] = 0.5f * (p.book.c[threadIdx.x] + p.book.c[threadIdx.x + 1]);
    }
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    unsigned char* stage = stage_base + warp * WarpStage<T, 64>::BYTES;
    const uint32_t* my_sign_base = s_sign + (LPV == 2 ? (lane & 1) * 32 : 0);

    // ---- geometry of this launch (as in cache_decode_kernel)
    const int64_t t_old = p.state != nullptr ? p.state->tokens : p.tokens;
    const bool refuse = p.append && p.state != nullptr && t_old >= p.capacity;
    const int64_t total = t_old + (p.append ? 1 : 0);
    const int last_items = (int)((total + TOKENS - 1) / TOKENS);
    int full_items = (int)(total / TOKENS);
    if (p.append) {
        full_items = (int)(t_old / TOKENS);
        for (int pl = 0; pl < p.n_planes; ++pl)
            if (p.plane[pl].kind == 1) {
                const int G = p.plane[pl].group_items * TOKENS;
                const int first = (int)(t_old / G) * p.plane[pl].group_items;
                full_items = first < full_items ? first : full_items;
            }
    }
    // (plane, segment) pairs, all at the CTA's token block; plane-major, so that the 16 warps of a CTA,
    // which take every 16th unit, each get their share of the costlier biased plane
    const int units = p.segments * p.n_planes;

    // cos and sin rows of token block tb -> shared memory (16-byte asynchronous copies, swizzled chunks)
    auto load_tile = [&](int tb, float* dst) {
        const uint32_t base = (uint32_t)__cvta_generic_to_shared(dst);
        constexpr int CPRW = D / 4;                            // 4-float chunks per table row
        for (int c = threadIdx.x; c < TOKENS * 2 * CPRW; c += CD_THREADS) {
            const int t = c / (2 * CPRW), r = c - t * (2 * CPRW), j = r / CPRW, q = r - j * CPRW;
            const int64_t tok = (int64_t)tb * TOKENS + t;
            const bool live = tok < total;
            const float* src = (j ? p.sin_table : p.cos_table) + (live ? tok * D + q * 4 : 0);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                         :: "r"(base + (uint32_t)(((t * 2 + j) * CPRW + (q ^ ((q >> 3) & 1))) * 16)), "l"(src), "r"(live ? 16 : 0) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // one (segment, plane) of token block `item`: prefetch ...
    auto fetch = [&](int u, int item, Prefetch64& f) {
        const int pl = u / p.segments, seg = u - pl * p.segments;
        const Plane64& P = p.plane[pl];
        const unsigned char* side = P.side + seg * P.side_seg_stride;
        const bool whole = item < full_items;
        const int64_t left = total - (int64_t)item * TOKENS;
        const int nvalid = left < TOKENS ? (int)left : TOKENS;
        if (P.kind == 0) {
            const unsigned char* codes = P.codes + seg * P.codes_seg_stride + (int64_t)item * ITEM_CODE_BYTES;
            const float* norms = reinterpret_cast<const float*>(side) + (int64_t)item * TOKENS;
            if (whole) prefetch_turbo64<D, BITS, true>(f, codes, norms, TOKENS, lane);
            else prefetch_turbo64<D, BITS, false>(f, codes, norms, (p.append && item == (int)(t_old / TOKENS)) ? nvalid - 1 : nvalid, lane);
        } else {
            const uint32_t* codes = reinterpret_cast<const uint32_t*>(P.codes + seg * P.codes_seg_stride + (int64_t)item * CH_ITEM_CODE_BYTES);
            const __half* ranges = reinterpret_cast<const __half*>(side) + (int64_t)(item / P.group_items) * (2 * D);
            if (whole) prefetch_channel64<D, true>(f, codes, ranges, TOKENS, lane);
            else if (!(p.append && item / P.group_items == (int)(t_old / (P.group_items * TOKENS))))
                prefetch_channel64<D, false>(f, codes, ranges, nvalid, lane);
        }
    };
    // ... and decode (with the append work where the item is touched by it)
    auto decode = [&](int u, int item, Prefetch64& f, const float* tile) {
        const int pl = u / p.segments, seg = u - pl * p.segments;
        const Plane64& P = p.plane[pl];
        const bool whole = item < full_items;
        const int64_t left = total - (int64_t)item * TOKENS;
        const int nvalid = left < TOKENS ? (int)left : TOKENS;
        T* out = reinterpret_cast<T*>(P.out + seg * P.out_seg_stride) + (int64_t)item * 2048;
        const float* brow = reinterpret_cast<const float*>(p.bias + seg * p.bias_seg_stride);
        RopeNew rn = RopeNew{nullptr, nullptr, nullptr};
        if (pl == 0) rn = RopeNew{brow, p.cos_table + t_old * D, p.sin_table + t_old * D};
        if (P.kind == 0) {
            if (whole) {
                if (pl == 0) turbo64_decode_warp<T, D, BITS, true, true>(f, out, TOKENS, table, my_sign_base + pl * 64, stage, lane, p.rs, tile, brow);
                else turbo64_decode_warp<T, D, BITS, true>(f, out, TOKENS, table, my_sign_base + pl * 64, stage, lane, p.rs);
                return;
            }
            if (p.append && item == (int)(t_old / TOKENS)) {
                const int tok = nvalid - 1;
                unsigned char* item_codes = const_cast<unsigned char*>(P.codes) + seg * P.codes_seg_stride + (int64_t)item * ITEM_CODE_BYTES;
                float* item_norms = reinterpret_cast<float*>(const_cast<unsigned char*>(P.side) + seg * P.side_seg_stride) + (int64_t)item * TOKENS;
                turbo_append_warp<D, BITS>(f, p.step[pl].in + seg * p.step[pl].in_seg_stride, p.in_dtype,
                                           reinterpret_cast<uint32_t*>(item_codes) + tok * (D * BITS / 32), item_norms + tok, tok,
                                           P.neg, s_edges, p.rs, stage, lane, rn);
            }
            if (pl == 0) turbo64_decode_warp<T, D, BITS, false, true>(f, out, nvalid, table, my_sign_base + pl * 64, stage, lane, p.rs, tile, brow);
            else turbo64_decode_warp<T, D, BITS, false>(f, out, nvalid, table, my_sign_base + pl * 64, stage, lane, p.rs);
        } else {
            if (whole) {
                if (pl == 0) channel64_decode_warp<T, D, true, true>(f, out, TOKENS, lane, tile, brow);
                else channel64_decode_warp<T, D, true>(f, out, TOKENS, lane);
            } else if (p.append && item / P.group_items == (int)(t_old / (P.group_items * TOKENS))) {
                if (pl == 0) channel_step_warp<T, D, true>(P, p.step[pl], p.in_dtype, seg, item, t_old, out, nvalid, lane, rn, tile);
                else channel_step_warp<T, D, false>(P, p.step[pl], p.in_dtype, seg, item, t_old, out, nvalid, lane);
            } else {
                if (pl == 0) channel64_decode_warp<T, D, false, true>(f, out, nvalid, lane, tile, brow);
                else channel64_decode_warp<T, D, false>(f, out, nvalid, lane);
            }
        }
    };

    if (!refuse) {
        int tb = blockIdx.x, buf = 0;
        Prefetch64 fa, fb;
        if (tb < last_items) {
            load_tile(tb, tiles);
            if (warp < units) fetch(warp, tb, fa);
        }
        for (; tb < last_items; tb += gridDim.x) {
            cp_async_wait<0>();
            __syncthreads();                                   // this block's rows are in place; nobody still reads the other buffer
            const int tb_next = tb + gridDim.x;
            if (NBUF == 2 && tb_next < last_items) load_tile(tb_next, tiles + (buf ^ 1) * (CD_TILE_BYTES / 4));
            const float* tile = tiles + buf * (CD_TILE_BYTES / 4);
#pragma unroll 1
            for (int u = warp; u < units; u += CD_WARPS) {
                int nu = u + CD_WARPS, ntb = tb;
                if (nu >= units) { nu = warp; ntb = tb_next; }
                const bool more = ntb < last_items;
                if (more) fetch(nu, ntb, fb);
                decode(u, tb, fa, tile);
                fa = fb;
            }
            if (NBUF == 1) {
                __syncthreads();                               // everyone is done with the only buffer
                if (tb_next < last_items) load_tile(tb_next, tiles);
            } else {
                buf ^= 1;
            }
        }
    }

    if (p.append && p.state != nullptr) {
        __syncthreads();
        if (threadIdx.x == 0) {
            const long long held = p.state->tokens;
            if (held >= p.capacity) {
                p.state->status = 1;
            } else {
                __threadfence();
                if (atomicAdd(&p.state->arrivals, 1u) == gridDim.x - 1) {
                    p.state->arrivals = 0;
                    p.state->tokens = held + 1;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// The decoded token at the newest position of every plane and segment, gathered into one contiguous
// buffer [plane][segment][dim]: what a host reads back after a step.  The position comes from the
// device-side token counter when there is one, so a captured graph of (step, this) stays valid
// from token to token.
// ------------------------------------------------------------------------------------------
struct NewestParams {
    int n_planes, segments;
    int row_bytes;                     // dim * sizeof(out element), a multiple of 16
    int64_t tokens;                    // tokens held (read from *state instead when state is set)
    const CacheState* state;
    const unsigned char* out[4];
    int64_t out_seg_stride[4];
    unsigned char* dst;
};

template <typename Chunk>                  // uint4: rows are copied in 16-byte chunks
__global__ void __launch_bounds__(256)
cache_newest_kernel(const __grid_constant__ NewestParams p) {
    const int64_t tokens = p.state != nullptr ? p.state->tokens : p.tokens;
    if (tokens < 1) return;
    const int cpr = p.row_bytes / (int)sizeof(Chunk);                  // chunks per token row
    const int total = p.n_planes * p.segments * cpr;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int c = i % cpr, row = i / cpr;
        const int seg = row % p.segments, pl = row / p.segments;
        const unsigned char* src = p.out[pl] + (int64_t)seg * p.out_seg_stride[pl] + (tokens - 1) * p.row_bytes + c * (int)sizeof(Chunk);
        reinterpret_cast<Chunk*>(p.dst)[i] = *reinterpret_cast<const Chunk*>(src);
    }
}

}  // namespace pitch
