// Exact key-bias removal around the codecs (reference/mechanism_eval.py:4-7, 82-91; README.md:100
// lists it as not yet in the reference's kernels).  A model whose key projection has a bias b_k
// caches k_t = R_t W x_t + R_t b_k; R_t b_k is known exactly (b_k is a weight, R_t the rotary
// embedding of position t), so it is subtracted before quantisation and added back after decoding
// at no storage cost.  With the model's own rotary tables (full width, as it applies them):
//     R_t b = b * cos[t] + rotate_half(b) * sin[t],   rotate_half(b) = (-b[d/2:], b[:d/2])
// One element-wise, in-place pass: x[v][i] +/- fl(fl(b_i cos) + fl(rh_i sin)), float32 arithmetic
// with one rounding per operation, then one rounding to the element type.
#pragma once

#include "common.cuh"

namespace pitch {

constexpr int RB_THREADS = 256;
constexpr int RB_SMEM_BYTES = 48 * 1024;          // bias rows of one tile of segments

// Segments per CTA: up to 8 (table reads are then a quarter of the data traffic, and the launch
// still has many more CTAs than the GPU holds at once), fewer if their bias rows (two float rows
// per segment) would not fit the shared-memory budget.
__host__ __device__ inline int rope_bias_seg_tile(int dim, int64_t segments) {
    int64_t tile = RB_SMEM_BYTES / (2 * dim * (int)sizeof(float));
    if (tile > 8) tile = 8;
    if (tile > segments) tile = segments;
    return (int)(tile < 1 ? 1 : tile);
}

// grid = (chunk blocks, segment tiles).  A thread owns one 16-byte chunk position (vector v,
// coordinates i0 ...) and walks the segments of its tile with the chunk's table values in
// registers: the rotary tables are read once per tile of segments, not once per segment.
template <typename T>
__global__ void __launch_bounds__(RB_THREADS)
rope_bias_kernel(unsigned char* __restrict__ data, int64_t data_seg_stride, const unsigned char* __restrict__ bias,
                 int64_t bias_seg_stride, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                 int dim, int64_t segments, int seg_tile, int64_t first_position, int64_t count, int subtract) {
    constexpr int EPC = 16 / (int)sizeof(T);                  // elements per chunk
    extern __shared__ float s_bias[];                         // per segment of the tile: [dim] b, then [dim] rotate_half(b)
    const int64_t seg0 = (int64_t)blockIdx.y * seg_tile;
    const int nseg = (int)(segments - seg0 < seg_tile ? segments - seg0 : seg_tile);
    for (int idx = threadIdx.x; idx < nseg * dim; idx += RB_THREADS) {
        const int s = idx / dim, i = idx - s * dim;
        const float* b = reinterpret_cast<const float*>(bias + (seg0 + s) * bias_seg_stride);
        s_bias[2 * s * dim + i] = b[i];
        s_bias[(2 * s + 1) * dim + i] = i < dim / 2 ? -b[i + dim / 2] : b[i - dim / 2];
    }
    __syncthreads();
    const int cpv = dim / EPC;                                // chunks per vector
    const int64_t chunks = count * cpv;
    for (int64_t c = (int64_t)blockIdx.x * RB_THREADS + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * RB_THREADS) {
        const int64_t v = c / cpv;
        const int i0 = (int)(c - v * cpv) * EPC;
        const float* cs = cos_table + (first_position + v) * dim + i0;
        const float* sn = sin_table + (first_position + v) * dim + i0;
        float cc[EPC], ss[EPC];
#pragma unroll
        for (int j = 0; j < EPC; j += 4) {
            const float4 c4 = __ldg(reinterpret_cast<const float4*>(cs + j));
            const float4 s4 = __ldg(reinterpret_cast<const float4*>(sn + j));
            cc[j] = c4.x; cc[j + 1] = c4.y; cc[j + 2] = c4.z; cc[j + 3] = c4.w;
            ss[j] = s4.x; ss[j + 1] = s4.y; ss[j + 2] = s4.z; ss[j + 3] = s4.w;
        }
        uint4* p = reinterpret_cast<uint4*>(data + seg0 * data_seg_stride) + c;
        const float* sb = s_bias + i0;
#pragma unroll 4
        for (int s = 0; s < nseg; ++s) {
            const uint4 q = *p;
            uint32_t w[4] = {q.x, q.y, q.z, q.w};
            float x[EPC];
            Packer<T, EPC>::unpack(w, x);
#pragma unroll
            for (int e = 0; e < EPC; ++e) {
                const float rb = __fadd_rn(__fmul_rn(sb[e], cc[e]), __fmul_rn(sb[dim + e], ss[e]));
                x[e] = subtract ? __fsub_rn(x[e], rb) : __fadd_rn(x[e], rb);
            }
            Packer<T, EPC>::pack(x, w);
            *p = make_uint4(w[0], w[1], w[2], w[3]);
            p = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(p) + data_seg_stride);
            sb += 2 * dim;
        }
    }
}

}  // namespace pitch
