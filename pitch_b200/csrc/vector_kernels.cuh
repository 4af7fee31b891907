// Per-vector codecs (TurboQuant, PolarQuant variant), general path: every power-of-two
// dim 2...1024, every bit width 2...8, fp32 / fp16 / bf16 on the full-precision side.
//
// Mapping.  A warp owns a tile of 32 x E contiguous coordinates, E = min(dim, 32); each lane
// keeps its E contiguous coordinates in registers.  dim >= 32: dim/32 adjacent lanes share a
// vector (1024/dim vectors per warp tile), the low five Walsh-Hadamard stages run in registers
// and the remaining log2(dim/32) stages as lane-xor shuffles.  dim < 32: one vector per lane.
// Because 32 codes of b bits are exactly b words, every lane's slice of the packed stream is
// word aligned for any b, including the widths whose codes straddle words.
//
// Global traffic is staged through a warp-private, padded shared-memory tile so that every
// global access of the full-precision tensor is a contiguous 512-byte warp transaction
// while each lane still ends up with its own contiguous row.
#pragma once

#include "common.cuh"

namespace pitch {

constexpr int VEC_WARPS = 4;               // warps per CTA
constexpr int VEC_THREADS = VEC_WARPS * 32;

template <int BITS> struct Codebook { float c[1 << BITS]; };

// Geometry of a warp tile for a given dim.
// SMALL selects the dim < 32 variant (one vector per lane, dim coordinates in use); for dim >= 32
// the per-lane count is the compile-time constant 32, so all per-coordinate guards fold away.
template <bool SMALL> struct TileGeom {
    int e_small;  // coordinates per lane when SMALL
    int tpv;      // lanes per vector
    int vpw;      // vectors per warp tile
    int wpv;      // packed words per vector
    __device__ __forceinline__ TileGeom(int dim, int bits) {
        e_small = dim;
        tpv = SMALL ? 1 : dim >> 5;
        vpw = 32 / tpv;
        wpv = words_per_vector(dim, bits);
    }
    __device__ __forceinline__ int e() const { return SMALL ? e_small : 32; }
};

template <typename T, bool SMALL>
__device__ __forceinline__ void load_lane_coords(const T* __restrict__ in, int64_t v0, int64_t count, int dim,
                                                 const TileGeom<SMALL>& g, bool vec_ok, unsigned char* stage,
                                                 int lane, bool valid, int64_t v, float (&x)[32]) {
    if (!SMALL) {
        const int64_t left = count - v0;
        const int valid_elems = (int)(left < g.vpw ? left : g.vpw) * dim;
        WarpStage<T, 32>::load(in + v0 * dim, valid_elems, vec_ok, stage, lane, x);
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = (i < dim && valid) ? Elem<T>::to_f32(in[v * dim + i]) : 0.0f;
    }
}

template <typename T, bool SMALL>
__device__ __forceinline__ void store_lane_coords(T* __restrict__ out, int64_t v0, int64_t count, int dim,
                                                  const TileGeom<SMALL>& g, bool vec_ok, unsigned char* stage,
                                                  int lane, bool valid, int64_t v, const float (&x)[32]) {
    if (!SMALL) {
        const int64_t left = count - v0;
        const int valid_elems = (int)(left < g.vpw ? left : g.vpw) * dim;
        WarpStage<T, 32>::store(out + v0 * dim, valid_elems, vec_ok, stage, lane, x);
    } else if (valid) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < dim) out[v * dim + i] = Elem<T>::from_f32(x[i]);
    }
}

template <int BITS, bool SMALL>
__device__ __forceinline__ void load_lane_words(const uint32_t* __restrict__ codes, int64_t v, int sub, int dim,
                                                const TileGeom<SMALL>& g, bool valid, uint32_t (&w)[BITS]) {
#pragma unroll
    for (int k = 0; k < BITS; ++k) {
        w[k] = 0;
        if (valid && (!SMALL || k < g.wpv)) w[k] = ldg_stream32(codes + v * g.wpv + sub * BITS + k);
    }
}

template <int BITS, bool SMALL>
__device__ __forceinline__ void store_lane_words(uint32_t* __restrict__ codes, int64_t v, int sub, int dim,
                                                 const TileGeom<SMALL>& g, bool valid, const uint32_t (&w)[BITS]) {
#pragma unroll
    for (int k = 0; k < BITS; ++k)
        if (valid && (!SMALL || k < g.wpv)) codes[v * g.wpv + sub * BITS + k] = w[k];
}

__device__ __forceinline__ void init_negate_masks(uint32_t* s_neg, uint32_t seed, int dim, int tid, int nthreads) {
    const int nw = dim < 32 ? 1 : dim >> 5;
    for (int k = tid; k < nw; k += nthreads) s_neg[k] = negate_mask32(seed, 32u * (uint32_t)k);
}

// ------------------------------------------------------------------------------------------
// TurboQuant encode: norm, unit vector, sign flip, WHT, 1/sqrt(d), codebook search, pack.
// Follows reference/pitch_reference.py:92-102 in float32 (PITCHKernels.metal:114-152).
// A code is the number of decision boundaries strictly below the rotated coordinate.
// ------------------------------------------------------------------------------------------
template <int BITS, typename T, bool SMALL>
__global__ void __launch_bounds__(VEC_THREADS)
turbo_encode_kernel(const T* __restrict__ in, uint32_t* __restrict__ codes, float* __restrict__ norms,
                    int64_t count, int dim, uint32_t seed, float rs, int vec_ok, const Codebook<BITS> book) {
    __shared__ float s_edges[1 << BITS];
    __shared__ uint32_t s_neg[32];
    __shared__ __align__(16) unsigned char s_stage[VEC_WARPS][WarpStage<T, 32>::BYTES];
    for (int k = threadIdx.x; k < (1 << BITS) - 1; k += VEC_THREADS) s_edges[k] = 0.5f * (book.c[k] + book.c[k + 1]);
    init_negate_masks(s_neg, seed, dim, threadIdx.x, VEC_THREADS);
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const TileGeom<SMALL> g(dim, BITS);
    const int64_t v0 = ((int64_t)blockIdx.x * VEC_WARPS + warp) * g.vpw;
    if (v0 >= count) return;
    const int sub = lane & (g.tpv - 1);
    const int64_t v = v0 + lane / g.tpv;
    const bool valid = v < count;

    float x[32];
    load_lane_coords<T, SMALL>(in, v0, count, dim, g, vec_ok != 0, s_stage[warp], lane, valid, v, x);

    float t[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) t[i] = x[i] * x[i];
    const float norm = sqrtf(lanes_sum(tree_sum_regs(t), g.tpv));
    const float inv = norm > 0.0f ? 1.0f / norm : 0.0f;
    const uint32_t neg = s_neg[sub];
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = flip_if(x[i], neg, i) * inv;
    wht_regs(x, g.e());
    wht_lanes(x, g.tpv, lane);

    uint32_t w[BITS];
#pragma unroll
    for (int k = 0; k < BITS; ++k) w[k] = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        if (i < g.e()) {
            const float u = x[i] * rs;
            uint32_t code = 0;
#pragma unroll
            for (int step = (1 << BITS) >> 1; step > 0; step >>= 1) {
                const uint32_t cand = code + step;
                if (u > s_edges[cand - 1]) code = cand;
            }
            insert_code<BITS>(w, i, code);
        }
    }
    store_lane_words<BITS, SMALL>(codes, v, sub, dim, g, valid, w);
    if (valid && sub == 0) norms[v] = norm;
}

// ------------------------------------------------------------------------------------------
// TurboQuant encode, dim >= 32, table-driven quantiser.
//
// Same arithmetic as turbo_encode_kernel up to the rotated coordinate u; only the search differs.
// The code of u is the number of decision boundaries strictly below u.  A uniform grid of M
// cells over [-1.125, 1.125] is laid over the boundaries, fine enough that no cell holds two of
// them (the host checks this and picks M).  cell(u) is read from the mantissa of
// fma(u, 8M/2.25, 1.5*2^23 + 4M), a monotone function of u, so every boundary in an earlier
// cell is below u and every boundary in a later cell is above: code = base[cell] + (u > edge[cell])
// with base[cell] = boundaries in earlier cells and edge[cell] = the cell's own boundary or +inf.
// One 8-byte shared load and one compare replace the BITS-step binary search; the result is
// identical for every u, ties included.  CTAs loop over warp tiles so the table is built once.
// ------------------------------------------------------------------------------------------
struct QuantGrid {
    int cells;        // M, a power of two
    float scale8;     // 8 * M / 2.25
    float magic8;     // 1.5 * 2^23 + 4 * M
};

__host__ __device__ __forceinline__ uint32_t quant_cell8(float u, float scale8, float magic8, uint32_t mask8) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(__fmaf_rn(u, scale8, magic8)) & mask8;      // byte offset of the cell's entry
#else
    float t = fmaf(u, scale8, magic8);
    uint32_t b;
    memcpy(&b, &t, 4);
    return b & mask8;
#endif
}

template <int BITS, typename T>
__global__ void __launch_bounds__(VEC_THREADS)
turbo_encode_grid_kernel(const T* __restrict__ in, uint32_t* __restrict__ codes, float* __restrict__ norms,
                         int64_t count, int dim, uint32_t seed, float rs, int vec_ok, const QuantGrid grid,
                         const Codebook<BITS> book) {
    extern __shared__ __align__(16) unsigned char dyn[];            // [cells] x {float edge, uint base}
    __shared__ float s_edges[1 << BITS];
    __shared__ int s_cell_of_edge[1 << BITS];
    __shared__ uint32_t s_neg[32];
    __shared__ __align__(16) unsigned char s_stage[VEC_WARPS][2][WarpStage<T, 32>::BYTES];     // two tiles: one in flight
    constexpr int NEDGES = (1 << BITS) - 1;
    const uint32_t mask8 = (uint32_t)(grid.cells - 1) << 3;
    for (int k = threadIdx.x; k < NEDGES; k += VEC_THREADS) {
        const float e = 0.5f * (book.c[k] + book.c[k + 1]);
        s_edges[k] = e;
        s_cell_of_edge[k] = (int)(quant_cell8(e, grid.scale8, grid.magic8, mask8) >> 3);
    }
    init_negate_masks(s_neg, seed, dim, threadIdx.x, VEC_THREADS);
    __syncthreads();
    for (int j = threadIdx.x; j < grid.cells; j += VEC_THREADS) {
        int lo = 0, hi = NEDGES;                                    // first boundary whose cell is >= j
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (s_cell_of_edge[mid] < j) lo = mid + 1; else hi = mid;
        }
        const bool own = lo < NEDGES && s_cell_of_edge[lo] == j;
        *reinterpret_cast<float2*>(dyn + j * 8) =
            make_float2(own ? s_edges[lo] : __int_as_float(0x7F800000), __uint_as_float((uint32_t)lo));
    }
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const TileGeom<false> g(dim, BITS);
    const int sub = lane & (g.tpv - 1);
    const uint32_t neg = s_neg[sub];
    const float2 rs2 = make_float2(rs, rs), sc2 = make_float2(grid.scale8, grid.scale8), mg2 = make_float2(grid.magic8, grid.magic8);
    const int64_t tiles = (count + g.vpw - 1) / g.vpw;
    const int64_t stride = (int64_t)gridDim.x * VEC_WARPS;
    // With an aligned input the next tile is copied into the other staging buffer asynchronously
    // while this one is encoded.
    auto tile_elems = [&](int64_t tile) {
        const int64_t left = count - tile * g.vpw;
        return (int)(left < g.vpw ? left : g.vpw) * dim;
    };
    int cur = 0;
    const int64_t first = (int64_t)blockIdx.x * VEC_WARPS + warp;
    if (vec_ok && first < tiles) WarpStage<T, 32>::issue_async(in + first * g.vpw * dim, tile_elems(first), s_stage[warp][0], lane);
    for (int64_t tile = first; tile < tiles; tile += stride) {
        const int64_t v0 = tile * g.vpw;
        const int64_t v = v0 + lane / g.tpv;
        const bool valid = v < count;
        float x[32];
        if (vec_ok) {
            const int64_t next = tile + stride;
            if (next < tiles) {
                WarpStage<T, 32>::issue_async(in + next * g.vpw * dim, tile_elems(next), s_stage[warp][cur ^ 1], lane);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncwarp();
            WarpStage<T, 32>::read_rows(s_stage[warp][cur], lane, x);
            cur ^= 1;
        } else {
            load_lane_coords<T, false>(in, v0, count, dim, g, false, s_stage[warp][0], lane, valid, v, x);
        }

        // norm: squares, then the balanced adjacent-pair tree (same order as tree_sum_regs + lanes_sum)
        float t[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) t[i] = x[i] * x[i];
        const float norm = sqrtf(lanes_sum(tree_sum_regs(t), g.tpv));
        const float inv = norm > 0.0f ? 1.0f / norm : 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = flip_if(x[i], neg, i) * inv;
        wht_regs(x, 32);
        wht_lanes(x, g.tpv, lane);

        uint32_t w[BITS];
#pragma unroll
        for (int k = 0; k < BITS; ++k) w[k] = 0;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            const float2 u = __fmul2_rn(make_float2(x[i], x[i + 1]), rs2);
            const float2 tt = __ffma2_rn(u, sc2, mg2);
            const float2 e0 = *reinterpret_cast<const float2*>(dyn + (__float_as_uint(tt.x) & mask8));
            const float2 e1 = *reinterpret_cast<const float2*>(dyn + (__float_as_uint(tt.y) & mask8));
            insert_code<BITS>(w, i, __float_as_uint(e0.y) + (u.x > e0.x ? 1u : 0u));
            insert_code<BITS>(w, i + 1, __float_as_uint(e1.y) + (u.y > e1.x ? 1u : 0u));
        }
        store_lane_words<BITS, false>(codes, v, sub, dim, g, valid, w);
        if (valid && sub == 0) norms[v] = norm;
    }
}

// ------------------------------------------------------------------------------------------
// Decode tail for dim >= 256 (8, 16 or 32 lanes per vector): the Walsh-Hadamard stages above
// coordinate bit 4 go through shared memory instead of lane shuffles.  Each lane writes its 32
// contiguous coordinates as a row of a padded warp tile and reads the tile back transposed, so
// that it then holds coordinates j*32 + lane (j = 0...31): stages 32, 64, ... become register
// butterflies over j, in the same order as before.  In that layout every j is 32 consecutive
// coordinates across the warp, so the result is stored straight to global memory (128 contiguous
// bytes per instruction for float32) and the output staging of the general path is not needed.
// The float operations, and their order, are those of the general path.
// ------------------------------------------------------------------------------------------
template <typename T, bool WITH_NORM>
__device__ __forceinline__ void finish_decode_transposed(float (&x)[32], unsigned char* sm, int lane, int tpv,
                                                         uint32_t my_neg, float my_norm, float rs,
                                                         T* __restrict__ tile_out, int valid_elems) {
    typedef WarpStage<float, 32> Stage;
#pragma unroll
    for (int q = 0; q < 8; ++q)
        *reinterpret_cast<float4*>(sm + lane * Stage::PITCHB + q * 16) =
            make_float4(x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
    // the row's pad carries what the transposed side needs to know about the row: the norm of the
    // vector it belongs to and the sign word of its 32 coordinates
    *reinterpret_cast<uint2*>(sm + lane * Stage::PITCHB + Stage::ROWB) = make_uint2(__float_as_uint(my_norm), my_neg);
    __syncwarp();
    float y[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = *reinterpret_cast<const float*>(sm + j * Stage::PITCHB + lane * 4);
    wht_regs(y, tpv);                       // row index bit k is coordinate bit 5 + k
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const uint2 row = *reinterpret_cast<const uint2*>(sm + j * Stage::PITCHB + Stage::ROWB);   // broadcast
        float v = flip_if(y[j], row.y, lane) * rs;
        if (WITH_NORM) v = v * __uint_as_float(row.x);
        if (j * 32 + lane < valid_elems) tile_out[j * 32 + lane] = Elem<T>::from_f32(v);
    }
    __syncwarp();
}

// ------------------------------------------------------------------------------------------
// TurboQuant decode: centroid lookup, WHT, sign, 1/sqrt(d), norm.
// reference/pitch_reference.py:104-107, PITCHKernels.metal:154-174.
// ------------------------------------------------------------------------------------------
template <int BITS, typename T, bool SMALL>
__global__ void __launch_bounds__(VEC_THREADS)
turbo_decode_kernel(const uint32_t* __restrict__ codes, const float* __restrict__ norms, T* __restrict__ out,
                    int64_t count, int dim, uint32_t seed, float rs, int vec_ok, const Codebook<BITS> book) {
    __shared__ float s_book[1 << BITS];
    __shared__ uint32_t s_neg[32];
    __shared__ __align__(16) unsigned char s_stage[VEC_WARPS][WarpStage<float, 32>::BYTES];   // float rows: also used by the transposed tail
    for (int k = threadIdx.x; k < (1 << BITS); k += VEC_THREADS) s_book[k] = book.c[k];
    init_negate_masks(s_neg, seed, dim, threadIdx.x, VEC_THREADS);
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const TileGeom<SMALL> g(dim, BITS);
    const int sub = lane & (g.tpv - 1);
    const uint32_t neg = s_neg[sub];
    // CTAs loop over warp tiles; the code words and the norm of the next tile are fetched while
    // this one is decoded.
    const int64_t tiles = (count + g.vpw - 1) / g.vpw;
    const int64_t stride = (int64_t)gridDim.x * VEC_WARPS;
    uint32_t wn[BITS];
    float norm_n = 0.0f;
    auto fetch = [&](int64_t tile) {
        const int64_t vv = tile * g.vpw + lane / g.tpv;
        const bool ok = vv < count;
        load_lane_words<BITS, SMALL>(codes, vv, sub, dim, g, ok, wn);
        norm_n = ok ? __uint_as_float(ldg_stream32(reinterpret_cast<const uint32_t*>(norms + vv))) : 0.0f;
    };
    const int64_t first = (int64_t)blockIdx.x * VEC_WARPS + warp;
    if (first < tiles) fetch(first);
    for (int64_t tile = first; tile < tiles; tile += stride) {
        const int64_t v0 = tile * g.vpw;
        const int64_t v = v0 + lane / g.tpv;
        const bool valid = v < count;
        uint32_t w[BITS];
#pragma unroll
        for (int k = 0; k < BITS; ++k) w[k] = wn[k];
        const float norm = norm_n;
        if (tile + stride < tiles) fetch(tile + stride);

        float x[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = (i < g.e()) ? s_book[extract_code<BITS>(w, i)] : 0.0f;
        wht_regs(x, g.e());
        if (!SMALL && g.tpv >= 8) {
            const int64_t left = count - v0;
            const int valid_elems = (int)(left < g.vpw ? left : g.vpw) * dim;
            finish_decode_transposed<T, true>(x, s_stage[warp], lane, g.tpv, neg, norm, rs, out + v0 * dim, valid_elems);
            continue;
        }
        wht_lanes(x, g.tpv, lane);
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = flip_if(x[i], neg, i) * rs * norm;
        store_lane_coords<T, SMALL>(out, v0, count, dim, g, vec_ok != 0, s_stage[warp], lane, valid, v, x);
    }
}

// ------------------------------------------------------------------------------------------
// PolarQuant variant encode: sign flip, WHT, 1/sqrt(d); pairs (y[2p], y[2p+1]) -> (r, theta);
// radius code on 2^b - 1 steps of [0, rmax], angle code on 2^b circular bins.
// reference/pitch_reference.py:109-121, PITCHKernels.metal:178-222.
// ------------------------------------------------------------------------------------------
template <int BITS, typename T, bool SMALL>
__global__ void __launch_bounds__(VEC_THREADS)
polar_encode_kernel(const T* __restrict__ in, uint32_t* __restrict__ codes, float* __restrict__ scales,
                    int64_t count, int dim, uint32_t seed, float rs, int vec_ok) {
    __shared__ uint32_t s_neg[32];
    __shared__ __align__(16) unsigned char s_stage[VEC_WARPS][SMALL ? 1 : 2][WarpStage<T, 32>::BYTES];   // two tiles: one in flight
    init_negate_masks(s_neg, seed, dim, threadIdx.x, VEC_THREADS);
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const TileGeom<SMALL> g(dim, BITS);
    const int sub = lane & (g.tpv - 1);
    const uint32_t neg = s_neg[sub];
    // CTAs loop over warp tiles; with an aligned input (dim >= 32) the next tile is copied into the
    // other staging buffer asynchronously while this one is encoded.
    const int64_t tiles = (count + g.vpw - 1) / g.vpw;
    const int64_t stride = (int64_t)gridDim.x * VEC_WARPS;
    const bool async = !SMALL && vec_ok != 0;
    auto tile_elems = [&](int64_t tile) {
        const int64_t left = count - tile * g.vpw;
        return (int)(left < g.vpw ? left : g.vpw) * dim;
    };
    int cur = 0;
    const int64_t first = (int64_t)blockIdx.x * VEC_WARPS + warp;
    if (async && first < tiles) WarpStage<T, 32>::issue_async(in + first * g.vpw * dim, tile_elems(first), s_stage[warp][0], lane);
    for (int64_t tile = first; tile < tiles; tile += stride) {
    const int64_t v0 = tile * g.vpw;
    const int64_t v = v0 + lane / g.tpv;
    const bool valid = v < count;

    float x[32];
    if (async) {
        const int64_t next = tile + stride;
        if (next < tiles) {
            WarpStage<T, 32>::issue_async(in + next * g.vpw * dim, tile_elems(next), s_stage[warp][SMALL ? 0 : (cur ^ 1)], lane);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        WarpStage<T, 32>::read_rows(s_stage[warp][SMALL ? 0 : cur], lane, x);
        cur ^= 1;
    } else {
        load_lane_coords<T, SMALL>(in, v0, count, dim, g, false, s_stage[warp][0], lane, valid, v, x);
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = flip_if(x[i], neg, i);
    wht_regs(x, g.e());
    wht_lanes(x, g.tpv, lane);

    // Radii.  The scale of the vector is the largest pair radius: sqrt is monotone and correctly
    // rounded, so sqrt(max r^2) is exactly max sqrt(r^2) and only ONE correctly rounded square root
    // is needed per vector.  The radius of each pair, which is only ever compared with the
    // quantiser's steps, comes from the hardware's approximate square root (within an ulp of the
    // exact one): its code can differ from the exactly rounded radius's only when r * scale + 1/2
    // lies within rounding distance of an integer - the boundary ties the parity tests count.
    float r[16];
    float rmax2 = 0.0f;
#pragma unroll
    for (int p = 0; p < 16; ++p) {
        x[2 * p] = x[2 * p] * rs;
        x[2 * p + 1] = x[2 * p + 1] * rs;
        const float aa = x[2 * p] * x[2 * p], cc = x[2 * p + 1] * x[2 * p + 1];
        const float r2 = aa + cc;
        asm("sqrt.approx.f32 %0, %1;" : "=f"(r[p]) : "f"(r2));
        if (2 * p < g.e()) rmax2 = fmaxf(rmax2, r2);
    }
    const float rmax = sqrtf(lanes_max(rmax2, g.tpv));
    const float safe = rmax > 0.0f ? rmax : 1.0f;
    constexpr int RL = (1 << BITS) - 1;
    const float radius_scale = (float)RL / safe;                          // one division per vector

    uint32_t w[BITS];
#pragma unroll
    for (int k = 0; k < BITS; ++k) w[k] = 0;
#pragma unroll
    for (int p = 0; p < 16; ++p) {
        if (2 * p < g.e()) {
            // floor(r * scale + 1/2), never negative; r <= rmax * (1 + 2^-22) keeps it at most RL, the
            // minimum only guards the packing against non-finite input
            const int q = __float2int_rd(r[p] * radius_scale + 0.5f);
            insert_code<BITS>(w, 2 * p, (uint32_t)min(q, RL));
            insert_code<BITS>(w, 2 * p + 1, angle_bin(x[2 * p], x[2 * p + 1], BITS));
        }
    }
    store_lane_words<BITS, SMALL>(codes, v, sub, dim, g, valid, w);
    if (valid && sub == 0) scales[v] = rmax;
    }
}

// ------------------------------------------------------------------------------------------
// PolarQuant variant decode.  reference/pitch_reference.py:123-129, PITCHKernels.metal:224-246.
// The 2^b angles are tabulated once per CTA.
// ------------------------------------------------------------------------------------------
template <int BITS, typename T, bool SMALL>
__global__ void __launch_bounds__(VEC_THREADS)
polar_decode_kernel(const uint32_t* __restrict__ codes, const float* __restrict__ scales, T* __restrict__ out,
                    int64_t count, int dim, uint32_t seed, float rs, int vec_ok) {
    __shared__ float s_cos[1 << BITS], s_sin[1 << BITS], s_ratio[1 << BITS];
    __shared__ uint32_t s_neg[32];
    __shared__ __align__(16) unsigned char s_stage[VEC_WARPS][WarpStage<float, 32>::BYTES];   // float rows: also used by the transposed tail
    for (int k = threadIdx.x; k < (1 << BITS); k += VEC_THREADS) {
        const float theta = (float)k / (float)(1 << BITS) * TWO_PI_F;
        s_cos[k] = cosf(theta);
        s_sin[k] = sinf(theta);
        s_ratio[k] = (float)k / (float)((1 << BITS) - 1);                 // radius code / levels, the IEEE quotient
    }
    init_negate_masks(s_neg, seed, dim, threadIdx.x, VEC_THREADS);
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const TileGeom<SMALL> g(dim, BITS);
    const int sub = lane & (g.tpv - 1);
    const uint32_t neg = s_neg[sub];
    // CTAs loop over warp tiles (the angle tables are built once); the code words and the scale
    // of the next tile are fetched while this one is decoded.
    const int64_t tiles = (count + g.vpw - 1) / g.vpw;
    const int64_t stride = (int64_t)gridDim.x * VEC_WARPS;
    uint32_t wn[BITS];
    float scale_n = 0.0f;
    auto fetch = [&](int64_t tile) {
        const int64_t vv = tile * g.vpw + lane / g.tpv;
        const bool ok = vv < count;
        load_lane_words<BITS, SMALL>(codes, vv, sub, dim, g, ok, wn);
        scale_n = ok ? __uint_as_float(ldg_stream32(reinterpret_cast<const uint32_t*>(scales + vv))) : 0.0f;
    };
    const int64_t first = (int64_t)blockIdx.x * VEC_WARPS + warp;
    if (first < tiles) fetch(first);
    for (int64_t tile = first; tile < tiles; tile += stride) {
        const int64_t v0 = tile * g.vpw;
        const int64_t v = v0 + lane / g.tpv;
        const bool valid = v < count;
        uint32_t w[BITS];
#pragma unroll
        for (int k = 0; k < BITS; ++k) w[k] = wn[k];
        const float scale = scale_n;
        if (tile + stride < tiles) fetch(tile + stride);

        float x[32];
#pragma unroll
        for (int p = 0; p < 16; ++p) {
            if (2 * p < g.e()) {
                const float r = s_ratio[extract_code<BITS>(w, 2 * p)] * scale;
                const uint32_t tq = extract_code<BITS>(w, 2 * p + 1);
                x[2 * p] = r * s_cos[tq];
                x[2 * p + 1] = r * s_sin[tq];
            } else {
                x[2 * p] = 0.0f;
                x[2 * p + 1] = 0.0f;
            }
        }
        wht_regs(x, g.e());
        if (!SMALL && g.tpv >= 8) {
            const int64_t left = count - v0;
            const int valid_elems = (int)(left < g.vpw ? left : g.vpw) * dim;
            finish_decode_transposed<T, false>(x, s_stage[warp], lane, g.tpv, neg, 0.0f, rs, out + v0 * dim, valid_elems);
            continue;
        }
        wht_lanes(x, g.tpv, lane);
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = flip_if(x[i], neg, i) * rs;
        store_lane_coords<T, SMALL>(out, v0, count, dim, g, vec_ok != 0, s_stage[warp], lane, valid, v, x);
    }
}

// ------------------------------------------------------------------------------------------
// The rotation on its own (float32 in, float32 out).  mode 0: unnormalised WHT; mode 1:
// rotate = WHT(x * signs) / sqrt(d); mode 2: unrotate = WHT(y) * signs / sqrt(d).
// reference/pitch_reference.py:21-34.
// ------------------------------------------------------------------------------------------
template <bool SMALL>
__global__ void __launch_bounds__(VEC_THREADS)
rotate_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t count, int dim, uint32_t seed,
              float rs, int mode, int vec_in_ok, int vec_out_ok) {
    __shared__ uint32_t s_neg[32];
    __shared__ __align__(16) unsigned char s_stage[VEC_WARPS][WarpStage<float, 32>::BYTES];
    init_negate_masks(s_neg, seed, dim, threadIdx.x, VEC_THREADS);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const TileGeom<SMALL> g(dim, 8);
    const int64_t v0 = ((int64_t)blockIdx.x * VEC_WARPS + warp) * g.vpw;
    if (v0 >= count) return;
    const int sub = lane & (g.tpv - 1);
    const int64_t v = v0 + lane / g.tpv;
    const bool valid = v < count;
    float x[32];
    load_lane_coords<float, SMALL>(in, v0, count, dim, g, vec_in_ok != 0, s_stage[warp], lane, valid, v, x);
    const uint32_t neg = s_neg[sub];
    if (mode == 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = flip_if(x[i], neg, i);
    }
    wht_regs(x, g.e());
    wht_lanes(x, g.tpv, lane);
    if (mode == 2) {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = flip_if(x[i], neg, i);
    }
    if (mode != 0) {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = x[i] * rs;
    }
    store_lane_coords<float, SMALL>(out, v0, count, dim, g, vec_out_ok != 0, s_stage[warp], lane, valid, v, x);
}

}  // namespace pitch
