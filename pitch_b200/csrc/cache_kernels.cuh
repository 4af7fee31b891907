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

__device__ __forceinline__ void prefetch_turbo64(Prefetch64& f, const uint4* __restrict__ codes,
                                                 const float* __restrict__ norms, int nvalid, int lane) {
    f.a = f.b = f.c = f.d = make_uint4(0, 0, 0, 0);
    if (lane < nvalid) {
        f.a = ldg_stream(codes + 2 * lane);
        f.b = ldg_stream(codes + 2 * lane + 1);
        f.c.x = ldg_stream32(reinterpret_cast<const uint32_t*>(norms) + lane);
    }
}

__device__ __forceinline__ void prefetch_channel64(Prefetch64& f, const uint32_t* __restrict__ codes,
                                                   const __half* __restrict__ group_ranges, int nvalid, int lane) {
    const int slab = lane & 7, tok_lane = lane >> 3;
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int t = 4 * k + tok_lane;
        w[k] = 0;
        if (t < nvalid) w[k] = ldg_stream32(codes + t * 8 + slab);
    }
    f.a = make_uint4(w[0], w[1], w[2], w[3]);
    f.b = make_uint4(w[4], w[5], w[6], w[7]);
    f.c = __ldg(reinterpret_cast<const uint4*>(group_ranges + slab * 8));
    f.d = __ldg(reinterpret_cast<const uint4*>(group_ranges + 64 + slab * 8));
}

// 32 vectors (d = 64, b = 4) per warp, one per lane; nvalid in 1...32.  `table` is the byte-pair
// table, `sign` 32 words whose bit 15 / bit 31 say whether element 2p / 2p+1 is negated by the
// rotation's diagonal.
template <typename T>
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
    const int valid_elems = nvalid * 64;
#pragma unroll
    for (int k = 0; k < Stage::CPR; ++k) {
        const int c = k * 32 + lane;
        const uint4 q = *reinterpret_cast<const uint4*>(stage + (c / Stage::CPR) * Stage::PITCHB + (c % Stage::CPR) * 16);
        if (c * Stage::EPC < valid_elems) stg_stream(reinterpret_cast<uint4*>(out) + c, q);
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
    static __device__ __forceinline__ void store(float* p, const float2 (&v)[4]) {
        stg_stream(reinterpret_cast<uint4*>(p), make_uint4(__float_as_uint(v[0].x), __float_as_uint(v[0].y),
                                                           __float_as_uint(v[1].x), __float_as_uint(v[1].y)));
        stg_stream(reinterpret_cast<uint4*>(p) + 1, make_uint4(__float_as_uint(v[2].x), __float_as_uint(v[2].y),
                                                               __float_as_uint(v[3].x), __float_as_uint(v[3].y)));
    }
};
template <> struct Pairs8<__half> {
    static __device__ __forceinline__ void store(__half* p, const float2 (&v)[4]) {
        stg_stream(reinterpret_cast<uint4*>(p), make_uint4(PairStore<__half>::cvt(v[0]), PairStore<__half>::cvt(v[1]),
                                                           PairStore<__half>::cvt(v[2]), PairStore<__half>::cvt(v[3])));
    }
};
template <> struct Pairs8<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float2 (&v)[4]) {
        stg_stream(reinterpret_cast<uint4*>(p),
                   make_uint4(PairStore<__nv_bfloat16>::cvt(v[0]), PairStore<__nv_bfloat16>::cvt(v[1]),
                              PairStore<__nv_bfloat16>::cvt(v[2]), PairStore<__nv_bfloat16>::cvt(v[3])));
    }
};

// 32 tokens (d = 64, b = 4, all inside one group) per warp: lane = (token lane 0..3, slab 0..7).
// code * step + lo with one rounding per operation.
template <typename T>
__device__ __forceinline__ void channel64_decode_warp(const Prefetch64& f, T* __restrict__ out, int nvalid, int lane) {
    const int slab = lane & 7, tok_lane = lane >> 3;
    const uint32_t w[8] = {f.a.x, f.a.y, f.a.z, f.a.w, f.b.x, f.b.y, f.b.z, f.b.w};
    const uint32_t lo16[4] = {f.c.x, f.c.y, f.c.z, f.c.w}, hi16[4] = {f.d.x, f.d.y, f.d.z, f.d.w};
    float2 lo[4], step[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        lo[i] = __half22float2(*reinterpret_cast<const __half2*>(&lo16[i]));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&hi16[i]));
        step[i] = make_float2(step_of(lo[i].x, hi.x, 15.0f), step_of(lo[i].y, hi.y, 15.0f));
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int t = 4 * k + tok_lane;
        float2 v[4];
        codes8_to_pairs(w[k], v);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = mul2_then_add(v[i], step[i], lo[i]);
        if (t < nvalid) Pairs8<T>::store(out + t * 64 + slab * 8, v);
    }
}

struct Plane64 {
    int kind;                 // 0 = TurboQuant, 1 = per-channel
    int group_size;           // per-channel planes: multiple of 32
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
    int tiles_per_seg;        // warp tiles (32 tokens) per segment
    int64_t tokens;
    int64_t total_tiles;      // segments * tiles_per_seg
    Plane64 plane[4];
    Book16 book;              // TurboQuant centroids for (64, 4)
};

template <typename T>
constexpr int cache64_smem_bytes() { return CD_TABLE_BYTES + 4 * 32 * 4 + CD_WARPS * WarpStage<T, 64>::BYTES; }

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
    unsigned char* stage = stage_base + warp * WarpStage<T, 64>::BYTES;

    // Work items of this warp: (tile, plane) pairs, tiles round-robin over all warps of the grid,
    // planes innermost.  Item k+1 is fetched before item k is decoded.
    const int64_t warp_id = (int64_t)blockIdx.x * CD_WARPS + warp;
    const int64_t warp_stride = (int64_t)gridDim.x * CD_WARPS;
    if (warp_id >= p.total_tiles) return;
    const int64_t my_tiles = (p.total_tiles - warp_id + warp_stride - 1) / warp_stride;
    const int64_t items = my_tiles * p.n_planes;

    struct Item { int pl; int nvalid; int64_t seg, t0; };
    auto locate = [&](int64_t k) {
        Item it;
        const int64_t tile = warp_id + (k / p.n_planes) * warp_stride;
        it.pl = (int)(k % p.n_planes);
        it.seg = tile / p.tiles_per_seg;
        it.t0 = (tile - it.seg * p.tiles_per_seg) * 32;
        const int64_t left = p.tokens - it.t0;
        it.nvalid = left < 32 ? (int)left : 32;
        return it;
    };
    auto fetch = [&](const Item& it, Prefetch64& f) {
        const Plane64& P = p.plane[it.pl];
        const unsigned char* codes = P.codes + it.seg * P.codes_seg_stride + it.t0 * 32;
        const unsigned char* side = P.side + it.seg * P.side_seg_stride;
        if (P.kind == 0)
            prefetch_turbo64(f, reinterpret_cast<const uint4*>(codes), reinterpret_cast<const float*>(side) + it.t0,
                             it.nvalid, lane);
        else
            prefetch_channel64(f, reinterpret_cast<const uint32_t*>(codes),
                               reinterpret_cast<const __half*>(side) + (it.t0 / P.group_size) * 128, it.nvalid, lane);
    };

    Item cur = locate(0);
    Prefetch64 fcur;
    fetch(cur, fcur);
#pragma unroll 1
    for (int64_t k = 0; k < items; ++k) {
        Item nxt = cur;
        Prefetch64 fnxt = fcur;
        if (k + 1 < items) {
            nxt = locate(k + 1);
            fetch(nxt, fnxt);
        }
        const Plane64& P = p.plane[cur.pl];
        T* out = reinterpret_cast<T*>(P.out + cur.seg * P.out_seg_stride) + cur.t0 * 64;
        if (P.kind == 0)
            turbo64_decode_warp<T>(fcur, out, cur.nvalid, table, s_sign + cur.pl * 32, stage, lane);
        else
            channel64_decode_warp<T>(fcur, out, cur.nvalid, lane);
        cur = nxt;
        fcur = fnxt;
    }
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
