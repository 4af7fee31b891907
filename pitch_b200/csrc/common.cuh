// Shared device helpers: element types, the rotation's sign diagonal, bit packing,
// Walsh-Hadamard butterflies.  Compiled with -fmad=false: every float operation below is
// one IEEE-754 rounding unless written as an explicit fused call.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pitch {

constexpr unsigned FULL = 0xFFFFFFFFu;
constexpr float TWO_PI_F = 6.28318530717958647692f;
constexpr float INV_TWO_PI_F = 0.15915494309189533577f;

// ------------------------------------------------------------------------------------------
// Element types of the full-precision side
// ------------------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float to_f32(float v) { return v; }
    static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

// Converts `N` floats to T and returns them packed in 32-bit words (N*sizeof(T)/4 words).
template <typename T, int N> struct Packer;
template <int N> struct Packer<float, N> {
    static constexpr int WORDS = N;
    static __device__ __forceinline__ void pack(const float* v, uint32_t* w) {
#pragma unroll
        for (int i = 0; i < N; ++i) w[i] = __float_as_uint(v[i]);
    }
    static __device__ __forceinline__ void unpack(const uint32_t* w, float* v) {
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = __uint_as_float(w[i]);
    }
};
template <int N> struct Packer<__half, N> {
    static constexpr int WORDS = N / 2;
    static __device__ __forceinline__ void pack(const float* v, uint32_t* w) {
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
    static __device__ __forceinline__ void unpack(const uint32_t* w, float* v) {
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            float2 f = __half22float2(h);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
};
template <int N> struct Packer<__nv_bfloat16, N> {
    static constexpr int WORDS = N / 2;
    static __device__ __forceinline__ void pack(const float* v, uint32_t* w) {
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
    static __device__ __forceinline__ void unpack(const uint32_t* w, float* v) {
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            // bf16 -> f32 is a 16-bit shift
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
};

// ------------------------------------------------------------------------------------------
// Rotation diagonal.  PCG-style hash of (seed + i) mod 2^32; sign is +1 when the low bit is
// set.  Follows reference/pitch_reference.py:11-19 and PITCHKernels.metal:26-37.
// ------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint32_t pcg_hash(uint32_t v) {
    uint32_t state = v * 747796405u + 2891336453u;
    uint32_t word = ((state >> ((state >> 28u) + 4u)) ^ state) * 277803737u;
    return (word >> 22u) ^ word;
}

// Bit j of the result is 1 when coordinate (first + j) is NEGATED by the diagonal.
__host__ __device__ __forceinline__ uint32_t negate_mask32(uint32_t seed, uint32_t first) {
    uint32_t m = 0;
#pragma unroll 4
    for (uint32_t j = 0; j < 32; ++j) m |= ((pcg_hash(seed + first + j) & 1u) ^ 1u) << j;
    return m;
}

__device__ __forceinline__ float flip_if(float v, uint32_t mask, int bit) {
    return __uint_as_float(__float_as_uint(v) ^ (((mask >> bit) & 1u) << 31));
}

// ------------------------------------------------------------------------------------------
// Bit stream of b-bit codes, LSB first in little-endian 32-bit words; code i of a vector
// occupies bits [i*b, i*b+b).  reference/pitch_reference.py:65-90.
// ------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ int words_per_vector(int dim, int bits) { return (dim * bits + 31) >> 5; }

// Code `i` (compile-time after unrolling) out of a register array of words.
template <int BITS>
__device__ __forceinline__ uint32_t extract_code(const uint32_t* w, int i) {
    const int start = i * BITS, word = start >> 5, off = start & 31;
    uint32_t v = w[word] >> off;
    if (off + BITS > 32) v |= w[word + 1] << (32 - off);
    return v & ((1u << BITS) - 1u);
}

template <int BITS>
__device__ __forceinline__ void insert_code(uint32_t* w, int i, uint32_t code) {
    const int start = i * BITS, word = start >> 5, off = start & 31;
    w[word] |= code << off;
    if (off + BITS > 32) w[word + 1] |= code >> (32 - off);
}

// Runtime-indexed variant reading from memory (global or shared).
__device__ __forceinline__ uint32_t read_code(const uint32_t* buf, int i, int bits) {
    const int start = i * bits, word = start >> 5, off = start & 31;
    uint32_t v = buf[word] >> off;
    if (off + bits > 32) v |= buf[word + 1] << (32 - off);
    return v & ((1u << bits) - 1u);
}

// ------------------------------------------------------------------------------------------
// Walsh-Hadamard butterflies on N register-resident values: stages h = 1, 2, 4 ... < limit,
// (a, b) -> (a + b, a - b) on index bit h.  PITCHKernels.metal:46-55, pitch_reference.py:21-31.
// ------------------------------------------------------------------------------------------
template <int N>
__device__ __forceinline__ void wht_regs(float (&x)[N], int limit) {
#pragma unroll
    for (int h = 1; h < N; h <<= 1) {
        if (h < limit) {
            if (h == 1) {
#pragma unroll
                for (int i = 0; i < N; i += 2) {
                    const float a = x[i], b = x[i + 1];
                    x[i] = a + b;
                    x[i + 1] = a - b;
                }
            } else {
                // adjacent pairs (x[2j], x[2j+1]) go through the same butterfly: packed fp32x2 add, and
                // a - b as fma(b, -1, a), each component one IEEE rounding like the scalar form
#pragma unroll
                for (int i = 0; i < N; i += 2) {
                    if (!(i & h)) {
                        const float2 a = make_float2(x[i], x[i + 1]), b = make_float2(x[i | h], x[(i | h) + 1]);
                        const float2 sum = __fadd2_rn(a, b);
                        const float2 dif = __ffma2_rn(b, make_float2(-1.0f, -1.0f), a);
                        x[i] = sum.x; x[i + 1] = sum.y;
                        x[i | h] = dif.x; x[(i | h) + 1] = dif.y;
                    }
                }
            }
        }
    }
}

// Stages across lanes: lane bit m corresponds to element bit m * N.  The lane whose bit m is set
// holds the upper half: it needs (partner - own), the other (own + partner); both are
// fma(own, +-1, partner), one rounding.
template <int N>
__device__ __forceinline__ void wht_lanes(float (&x)[N], int lanes_per_vector, int lane) {
    for (int m = 1; m < lanes_per_vector; m <<= 1) {
        const float sg = (lane & m) ? -1.0f : 1.0f;
        const float2 s2 = make_float2(sg, sg);
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            float2 o;
            o.x = __shfl_xor_sync(FULL, x[i], m);
            o.y = __shfl_xor_sync(FULL, x[i + 1], m);
            const float2 r = __ffma2_rn(make_float2(x[i], x[i + 1]), s2, o);
            x[i] = r.x;
            x[i + 1] = r.y;
        }
    }
}

// Balanced pairwise sum over adjacent elements: level 1 adds t[2j] + t[2j+1], and so on.
// Values beyond `limit` must be zero.  Independent of how a vector is split over lanes as
// long as each lane owns a contiguous power-of-two block.
template <int N>
__device__ __forceinline__ float tree_sum_regs(float (&t)[N]) {
#pragma unroll
    for (int n = N; n > 1; n >>= 1) {
#pragma unroll
        for (int j = 0; j < n / 2; ++j) t[j] = t[2 * j] + t[2 * j + 1];
    }
    return t[0];
}

__device__ __forceinline__ float lanes_sum(float v, int lanes_per_vector) {
    for (int m = 1; m < lanes_per_vector; m <<= 1) v = v + __shfl_xor_sync(FULL, v, m);
    return v;
}

__device__ __forceinline__ float lanes_max(float v, int lanes_per_vector) {
    for (int m = 1; m < lanes_per_vector; m <<= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, m));
    return v;
}

// 128-bit global accesses.  Codes and side information are read once: bypass L1 allocation.
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream64(const uint2* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ void stg_stream(uint4* p, const uint4& v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// PolarQuant angle code of the pair (x, y): floor(atan2(y, x) * 2^bits / 2pi + 1/2) mod 2^bits
// (reference/pitch_reference.py:116-119).  For 2, 3 and 4 bits no arctangent is needed: the
// first-quadrant angle atan2(|y|, |x|) has reached bin j once |y| >= |x| * tan((j - 1/2) * 2pi/N), so j
// is a count of at most four comparisons, and the quadrant is restored from the two sign bits
// (atan2's own conventions for signed zeros included).  Decisions differ from the arctangent
// route only for angles within rounding distance of a bin boundary.  Wider codes use atan2f.
__device__ __forceinline__ uint32_t angle_bin(float x, float y, int bits) {
    const uint32_t n = 1u << bits;
    if (bits > 4) {
        const float theta = atan2f(y, x);                      // (-pi, pi]: a negative bin index wraps to theta + 2*pi
        return (uint32_t)(int)floorf(theta * ((float)n * INV_TWO_PI_F) + 0.5f) & (n - 1u);
    }
    const float a = fabsf(x), b = fabsf(y);
    uint32_t j;
    if (bits == 2) {
        j = b >= a ? 1u : 0u;
    } else if (bits == 3) {
        j = (b >= a * 0.4142135679721832f ? 1u : 0u) + (b >= a * 2.4142136573791504f ? 1u : 0u);
    } else {
        j = (b >= a * 0.1989123672246933f ? 1u : 0u) + (b >= a * 0.6681786179542542f ? 1u : 0u) +
            (b >= a * 1.4966057538986206f ? 1u : 0u) + (b >= a * 5.027339458465576f ? 1u : 0u);
    }
    if (b == 0.0f) j = 0u;                                     // also the pair (0, 0), where every comparison holds
    const uint32_t k = (__float_as_uint(x) >> 31) ? n / 2u - j : j;             // x < 0 or -0: pi - angle
    return (__float_as_uint(y) >> 31) ? (n - k) & (n - 1u) : k;                 // y < 0 or -0: negated angle
}

template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// ------------------------------------------------------------------------------------------
// Warp tile <-> registers.  The tile is 32 rows of E contiguous elements of T (32*E contiguous
// elements of global memory); lane r ends up with (or starts from) row r in registers while
// every global access is a contiguous 512-byte warp transaction.  Row r lives at r * PITCHB
// bytes of a warp-private shared buffer; the 16-byte pad keeps both the row-owner accesses
// and the transposed accesses free of bank conflicts.
// ------------------------------------------------------------------------------------------
template <typename T, int E> struct WarpStage {
    static constexpr int ROWB = E * (int)sizeof(T);
    static constexpr int PITCHB = ROWB + 16;
    static constexpr int BYTES = 32 * PITCHB;
    static constexpr int CPR = ROWB / 16;            // 16-byte chunks per row
    static constexpr int EPC = 16 / (int)sizeof(T);  // elements per chunk
    static constexpr int WORDS = ROWB / 4;

    static __device__ __forceinline__ void load(const T* __restrict__ g, int valid_elems, bool vec_ok,
                                                unsigned char* sm, int lane, float (&x)[E]) {
        if (vec_ok) {
#pragma unroll
            for (int k = 0; k < CPR; ++k) {
                const int c = k * 32 + lane;
                uint4 q = make_uint4(0, 0, 0, 0);
                if (c * EPC < valid_elems) q = ldg_stream(reinterpret_cast<const uint4*>(g) + c);
                *reinterpret_cast<uint4*>(sm + (c / CPR) * PITCHB + (c % CPR) * 16) = q;
            }
        } else {
#pragma unroll 4
            for (int k = 0; k < E; ++k) {
                const int e = k * 32 + lane;
                T v = Elem<T>::from_f32(0.0f);
                if (e < valid_elems) v = g[e];
                *reinterpret_cast<T*>(sm + (e / E) * PITCHB + (e % E) * (int)sizeof(T)) = v;
            }
        }
        __syncwarp();
        uint32_t w[WORDS];
#pragma unroll
        for (int j = 0; j < CPR; ++j) {
            const uint4 q = *reinterpret_cast<const uint4*>(sm + lane * PITCHB + j * 16);
            w[4 * j] = q.x; w[4 * j + 1] = q.y; w[4 * j + 2] = q.z; w[4 * j + 3] = q.w;
        }
        Packer<T, E>::unpack(w, x);
        __syncwarp();
    }

    // The same tile, fetched by asynchronous 16-byte copies straight into the staging buffer (no
    // registers, nothing waits): issue for the next tile, compute the current one, then
    // cp_async_wait + __syncwarp + read_rows.  Needs a 16-byte aligned `g`; chunks beyond
    // valid_elems are zero-filled without touching memory.
    static __device__ __forceinline__ void issue_async(const T* __restrict__ g, int valid_elems, unsigned char* sm, int lane) {
        const uint32_t base = (uint32_t)__cvta_generic_to_shared(sm);
#pragma unroll
        for (int k = 0; k < CPR; ++k) {
            const int c = k * 32 + lane;
            const bool live = c * EPC < valid_elems;
            const void* src = live ? static_cast<const void*>(reinterpret_cast<const uint4*>(g) + c) : static_cast<const void*>(g);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                         :: "r"(base + (c / CPR) * PITCHB + (c % CPR) * 16), "l"(src), "r"(live ? 16 : 0) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    static __device__ __forceinline__ void read_rows(const unsigned char* sm, int lane, float (&x)[E]) {
        uint32_t w[WORDS];
#pragma unroll
        for (int j = 0; j < CPR; ++j) {
            const uint4 q = *reinterpret_cast<const uint4*>(sm + lane * PITCHB + j * 16);
            w[4 * j] = q.x; w[4 * j + 1] = q.y; w[4 * j + 2] = q.z; w[4 * j + 3] = q.w;
        }
        Packer<T, E>::unpack(w, x);
        __syncwarp();
    }

    static __device__ __forceinline__ void store(T* __restrict__ g, int valid_elems, bool vec_ok,
                                                 unsigned char* sm, int lane, const float (&x)[E]) {
        uint32_t w[WORDS];
        Packer<T, E>::pack(x, w);
#pragma unroll
        for (int j = 0; j < CPR; ++j)
            *reinterpret_cast<uint4*>(sm + lane * PITCHB + j * 16) =
                make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        __syncwarp();
        if (vec_ok) {
#pragma unroll
            for (int k = 0; k < CPR; ++k) {
                const int c = k * 32 + lane;
                const uint4 q = *reinterpret_cast<const uint4*>(sm + (c / CPR) * PITCHB + (c % CPR) * 16);
                if (c * EPC < valid_elems) stg_stream(reinterpret_cast<uint4*>(g) + c, q);
            }
        } else {
#pragma unroll 4
            for (int k = 0; k < E; ++k) {
                const int e = k * 32 + lane;
                const T v = *reinterpret_cast<const T*>(sm + (e / E) * PITCHB + (e % E) * (int)sizeof(T));
                if (e < valid_elems) g[e] = v;
            }
        }
        __syncwarp();
    }
};

}  // namespace pitch
