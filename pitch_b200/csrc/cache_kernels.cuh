// Whole-cache decode for head dimension 64 at 4 bits: the per-step bottleneck of a
// compressed KV cache (all tokens of every layer and KV head are decoded each step).
//
// One persistent launch covers every plane (K, V) and every segment (layer x KV head): one CTA
// of 16 warps per SM; a warp takes tiles of 32 consecutive tokens of one segment round-robin and
// decodes that tile for every plane before moving on.  Per token the kernel reads 32 code bytes
// plus 4 bytes of side information and writes 64 elements, so it is bound by HBM traffic as
// long as the instruction count per token stays low; the two paths are built around that:
//
//   * TurboQuant plane - one vector per lane.  Two 128-bit loads bring the lane's 32 code
//     bytes.  Each byte holds two codes (a, b); a 256-entry table in shared memory maps the byte
//     to (c[a] + c[b], c[a] - c[b]), i.e. centroid lookup and the first Walsh-Hadamard stage in
//     one 64-bit load.  The table is replicated over 32 lane slots (entry e, slot l at byte
//     e*256 + l*8), so a lookup is bank-conflict free for any codes and its address is a single
//     byte permute of the code word.  The remaining five stages run on float2 pairs with packed
//     fp32x2 instructions, the result is scaled, rounded, sign-flipped as packed words, and
//     leaves through a padded warp-private shared tile so that every global store instruction
//     writes 512 contiguous bytes per warp.
//   * per-channel plane - a lane owns 8 channels ("slab") of 4 of the 32 tokens per step; codes
//     become floats by byte permutes into the mantissa of 2^23; loads are 4 bytes and stores 16
//     bytes per lane, both contiguous across the warp.
#pragma once

#include "channel_kernels.cuh"
#include "common.cuh"

namespace pitch {

constexpr int CD_THREADS = 512;
constexpr int CD_WARPS = CD_THREADS / 32;
constexpr int CD_TABLE_BYTES = 256 * 32 * 8;   // byte-pair table: 256 entries x 32 lane slots x float2

struct Book16 { float c[16]; };

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

// What one lane needs from global memory to decode its share of a 32-token tile of one plane.
// Fetched one work item ahead of its use, so the loads of item k+1 are in flight while item k
// is being decoded.
struct Prefetch64 {
    uint4 a, b;   // TurboQuant: the lane's 32 code bytes.  Per-channel: code words of tokens 4k + (lane >> 3), k = 0..7
    uint4 c, d;   // TurboQuant: c.x = norm bits.  Per-channel: fp16 minima (c) and maxima (d) of the lane's 8 channels
};

__device__ __forceinline__ uint32_t ldg_stream32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// FULL: all 32 tokens of the tile exist (no bounds checks); otherwise nvalid in 1...31.
template <bool FULL>
__device__ __forceinline__ void prefetch_turbo64(Prefetch64& f, const uint4* __restrict__ codes,
                                                 const float* __restrict__ norms, int nvalid, int lane) {
    if (FULL || lane < nvalid) {
        f.a = ldg_stream(codes + 2 * lane);
        f.b = ldg_stream(codes + 2 * lane + 1);
        f.c.x = ldg_stream32(reinterpret_cast<const uint32_t*>(norms) + lane);
    } else {
        f.a = f.b = make_uint4(0, 0, 0, 0);
        f.c.x = 0;
    }
}

template <bool FULL>
__device__ __forceinline__ void prefetch_channel64(Prefetch64& f, const uint32_t* __restrict__ codes,
                                                   const __half* __restrict__ group_ranges, int nvalid, int lane) {
    const int slab = lane & 7, tok_lane = lane >> 3;
    const uint32_t* mine = codes + tok_lane * 8 + slab;      // token 4k + tok_lane is 32k words further
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        w[k] = 0;
        if (FULL || 4 * k + tok_lane < nvalid) w[k] = ldg_stream32(mine + 32 * k);
    }
    f.a = make_uint4(w[0], w[1], w[2], w[3]);
    f.b = make_uint4(w[4], w[5], w[6], w[7]);
    f.c = __ldg(reinterpret_cast<const uint4*>(group_ranges + slab * 8));
    f.d = __ldg(reinterpret_cast<const uint4*>(group_ranges + 64 + slab * 8));
}

// 32 vectors (d = 64, b = 4) per warp, one per lane.  `table` is the byte-pair table, `sign` 32
// words whose bit 15 / bit 31 say whether element 2p / 2p+1 is negated by the rotation's diagonal.
template <typename T, bool FULL>
__device__ __forceinline__ void turbo64_decode_warp(const Prefetch64& f, T* __restrict__ out, int nvalid,
                                                    const unsigned char* table, const uint32_t* sign,
                                                    unsigned char* stage, int lane) {
    typedef WarpStage<T, 64> Stage;
    const uint32_t w[8] = {f.a.x, f.a.y, f.a.z, f.a.w, f.b.x, f.b.y, f.b.z, f.b.w};
    const float norm = __uint_as_float(f.c.x);
    const uint32_t slot = (uint32_t)lane * 8u;
    float2 v[32];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        // byte k of the word -> table offset (byte << 8) | slot, one permute each
        v[4 * j + 0] = *reinterpret_cast<const float2*>(table + __byte_perm(w[j], slot, 0x5504));
        v[4 * j + 1] = *reinterpret_cast<const float2*>(table + __byte_perm(w[j], slot, 0x5514));
        v[4 * j + 2] = *reinterpret_cast<const float2*>(table + __byte_perm(w[j], slot, 0x5524));
        v[4 * j + 3] = *reinterpret_cast<const float2*>(table + __byte_perm(w[j], slot, 0x5534));
    }
    wht64_pairs_from_stage2(v);
    // 1/sqrt(64) is a power of two, so (x * rs) * norm == x * (rs * norm) in float32.
    const float sc = 0.125f * norm;
    const float2 scale = make_float2(sc, sc);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = mul2(v[i], scale);
    PairStore<T>::row(v, sign, stage + lane * Stage::PITCHB);
    __syncwarp();
    // transposed read-out: chunk c = k*32 + lane of the tile's contiguous output
    const unsigned char* src = stage + (lane / Stage::CPR) * Stage::PITCHB + (lane % Stage::CPR) * 16;
    uint4* dst = reinterpret_cast<uint4*>(out) + lane;
    const int valid_chunks = nvalid * Stage::CPR;
#pragma unroll
    for (int k = 0; k < Stage::CPR; ++k) {
        const uint4 q = *reinterpret_cast<const uint4*>(src + k * (32 / Stage::CPR) * Stage::PITCHB);
        if (FULL || k * 32 + lane < valid_chunks) stg_stream(dst + k * 32, q);
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

// 32 tokens (d = 64, b = 4, all inside one group) per warp: lane = (token lane 0..3, slab 0..7).
// code * step + lo with one rounding per operation.
template <typename T, bool FULL>
__device__ __forceinline__ void channel64_decode_warp(const Prefetch64& f, T* __restrict__ out, int nvalid, int lane) {
    const int slab = lane & 7, tok_lane = lane >> 3;
    const uint32_t w[8] = {f.a.x, f.a.y, f.a.z, f.a.w, f.b.x, f.b.y, f.b.z, f.b.w};
    const uint32_t lo16[4] = {f.c.x, f.c.y, f.c.z, f.c.w}, hi16[4] = {f.d.x, f.d.y, f.d.z, f.d.w};
    float2 lo[4], step[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        lo[i] = __half22float2(*reinterpret_cast<const __half2*>(&lo16[i]));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&hi16[i]));
        step[i] = make_float2(step15(lo[i].x, hi.x), step15(lo[i].y, hi.y));
    }
    T* mine = out + tok_lane * 64 + slab * 8;                // token 4k + tok_lane is 256k elements further
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float2 v[4];
        codes8_to_pairs(w[k], v);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = mul2_then_add(v[i], step[i], lo[i]);
        Pairs8<T>::store(mine + 256 * k, v, FULL || 4 * k + tok_lane < nvalid);
    }
}

struct Plane64 {
    int kind;                 // 0 = TurboQuant, 1 = per-channel
    int group_tiles;          // per-channel planes: group size / 32
    uint32_t neg_lo, neg_hi;  // rotation diagonal: bit i set when element i (resp. 32 + i) is negated
    const unsigned char* codes;
    int64_t codes_seg_stride;
    const unsigned char* side;
    int64_t side_seg_stride;
    unsigned char* out;
    int64_t out_seg_stride;
};

struct Cache64Params {
    int n_planes;
    int segments;
    int full_tiles;           // whole 32-token tiles per segment (tokens / 32)
    int tail;                 // tokens in the partial last tile of every segment (tokens % 32)
    Plane64 plane[4];
    Book16 book;              // TurboQuant centroids for (64, 4)
};

template <typename T>
constexpr int cache64_smem_bytes() { return CD_TABLE_BYTES + 4 * 32 * 4 + CD_WARPS * WarpStage<T, 64>::BYTES; }

// A work item: one 32-token tile of one plane of one segment.
struct Cursor64 {
    int pl, seg, tile;
};

// grid = number of SMs (persistent), CD_THREADS threads, cache64_smem_bytes<T>() dynamic shared memory.
template <typename T>
__global__ void __launch_bounds__(CD_THREADS, 1)
cache_decode_d64b4_kernel(const __grid_constant__ Cache64Params p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* table = smem;
    uint32_t* s_sign = reinterpret_cast<uint32_t*>(smem + CD_TABLE_BYTES);           // [4][32]
    unsigned char* stage_base = smem + CD_TABLE_BYTES + 4 * 32 * 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    bool any_turbo = false;
    for (int pl = 0; pl < p.n_planes; ++pl) any_turbo |= p.plane[pl].kind == 0;
    if (any_turbo) {
        for (int idx = threadIdx.x; idx < 256 * 32; idx += CD_THREADS) {
            const int e = idx >> 5;
            const float a = p.book.c[e & 15], b = p.book.c[e >> 4];
            *reinterpret_cast<float2*>(table + idx * 8) = make_float2(a + b, a - b);
        }
        if (threadIdx.x < 4 * 32) {
            const int pl = threadIdx.x >> 5, i = threadIdx.x & 31;       // packed pair i = elements 2i, 2i+1
            const uint32_t m = i < 16 ? p.plane[pl].neg_lo : p.plane[pl].neg_hi;
            const int bit = (2 * i) & 31;
            s_sign[threadIdx.x] = (((m >> bit) & 1u) << 15) | (((m >> (bit + 1)) & 1u) << 31);
        }
    }
    __syncthreads();
    // Everything above touched only kernel parameters and shared memory.  Under programmatic
    // dependent launch this grid may have started before the previous kernel of the stream ended:
    // wait for it (and for its memory to be visible) before reading the cache.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    unsigned char* stage = stage_base + warp * WarpStage<T, 64>::BYTES;
    // warp w of CTA c is worker w * gridDim + c: when the tile count is not a multiple of the worker
    // count, the workers that take one tile more are spread evenly over the SMs
    const int warp_id = warp * gridDim.x + blockIdx.x;
    const int warp_stride = gridDim.x * CD_WARPS;

    // Addresses of an item.  Whole tiles take the FULL (unchecked) paths.
    auto fetch = [&](const Cursor64& c, Prefetch64& f) {
        const Plane64& P = p.plane[c.pl];
        const unsigned char* codes = P.codes + c.seg * P.codes_seg_stride + (int64_t)c.tile * 1024;
        const unsigned char* side = P.side + c.seg * P.side_seg_stride;
        if (P.kind == 0)
            prefetch_turbo64<true>(f, reinterpret_cast<const uint4*>(codes),
                                   reinterpret_cast<const float*>(side) + c.tile * 32, 32, lane);
        else
            prefetch_channel64<true>(f, reinterpret_cast<const uint32_t*>(codes),
                                     reinterpret_cast<const __half*>(side) + (c.tile / P.group_tiles) * 128, 32, lane);
    };
    auto decode = [&](const Cursor64& c, const Prefetch64& f) {
        const Plane64& P = p.plane[c.pl];
        T* out = reinterpret_cast<T*>(P.out + c.seg * P.out_seg_stride) + (int64_t)c.tile * 2048;
        if (P.kind == 0)
            turbo64_decode_warp<T, true>(f, out, 32, table, s_sign + c.pl * 32, stage, lane);
        else
            channel64_decode_warp<T, true>(f, out, 32, lane);
    };
    // Next item of this warp: planes innermost, then the warp's next tile (round-robin over the grid).
    auto advance = [&](Cursor64& c) {
        if (++c.pl < p.n_planes) return true;
        c.pl = 0;
        c.tile += warp_stride;
        if (c.tile >= p.full_tiles) {
            const int q = c.tile / p.full_tiles;
            c.seg += q;
            c.tile -= q * p.full_tiles;
        }
        return c.seg < p.segments;
    };

    // ---- whole tiles, software pipelined with two register buffers used alternately
    if (p.full_tiles > 0) {
        Cursor64 cur;
        cur.pl = 0;
        cur.seg = warp_id / p.full_tiles;
        cur.tile = warp_id - cur.seg * p.full_tiles;
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

    // ---- the partial last tile of every segment (at most one per segment and plane)
    if (p.tail > 0) {
        for (int item = warp_id; item < p.segments * p.n_planes; item += warp_stride) {
            const int seg = item / p.n_planes, pl = item - seg * p.n_planes;
            const Plane64& P = p.plane[pl];
            const unsigned char* codes = P.codes + seg * P.codes_seg_stride + (int64_t)p.full_tiles * 1024;
            const unsigned char* side = P.side + seg * P.side_seg_stride;
            T* out = reinterpret_cast<T*>(P.out + seg * P.out_seg_stride) + (int64_t)p.full_tiles * 2048;
            Prefetch64 f;
            if (P.kind == 0) {
                prefetch_turbo64<false>(f, reinterpret_cast<const uint4*>(codes),
                                        reinterpret_cast<const float*>(side) + p.full_tiles * 32, p.tail, lane);
                turbo64_decode_warp<T, false>(f, out, p.tail, table, s_sign + pl * 32, stage, lane);
            } else {
                prefetch_channel64<false>(f, reinterpret_cast<const uint32_t*>(codes),
                                          reinterpret_cast<const __half*>(side) + (p.full_tiles / P.group_tiles) * 128,
                                          p.tail, lane);
                channel64_decode_warp<T, false>(f, out, p.tail, lane);
            }
        }
    }
}

}  // namespace pitch
