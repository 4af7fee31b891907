/* CPU oracle #2: float32 restatement of the codec arithmetic, one IEEE
 * operation at a time (no FMA contraction, no fast-math).
 *
 * TEST INFRASTRUCTURE ONLY - never linked into or called by the product.
 *
 * The reference has two implementations of every operation: the float64
 * NumPy specification (oracle #1 restates it) and float32 Metal kernels.
 * This file restates the float32 side: it follows the bodies of the six
 * kernels in Sources/PITCH/Shaders/PITCHKernels.metal (cited per function)
 * in plain C, so that a float32 GPU kernel can be required to agree with it
 * bit for bit on codes, and so that the count of codes on which float32 and
 * float64 disagree ("boundary ties") can be predicted on the CPU.
 *
 * Deliberate, documented differences from the Metal text:
 *  - the sum of squares is a balanced pairwise tree over ADJACENT elements
 *    (level 1 adds s[2j]+s[2j+1], ...) where PITCHKernels.metal:58-69 pairs
 *    element i with i+dim/2.  Both are balanced binary trees with identical
 *    error bounds; adjacent-first does not depend on how a vector is split
 *    over GPU lanes.
 *  - 1/sqrt(dim) is the correctly rounded float32 of the exact value (Metal's
 *    rsqrt is approximate).
 *  - PolarQuant encode exists in two variants.  pitch_oracle_polar_encode scales
 *    the radius by levels/rmax (one division per vector) and the angle by
 *    bins/(2*pi) (one multiplication, a negative bin index wrapping around), the
 *    way a GPU kernel that avoids per-pair divisions does; the same real-number
 *    formula, two float roundings placed differently.  pitch_oracle_polar_encode_metal
 *    follows PITCHKernels.metal:207-214 to the letter (r / rmax * levels, theta made
 *    non-negative, theta / (2*pi) * bins).  Tests report a kernel's code mismatches
 *    against both, and against the float64 specification.
 *
 * Parity status: PINNED against the reference's golden fixtures within the
 * reference's own float32-vs-float64 tolerances (tests/test_oracle_golden.py):
 * codes differing on at most max(2, n/500) coordinates, scales to 1e-5,
 * decode of the golden codes to 1e-5 relative L2; per-channel codes, ranges
 * and reconstructions bit-identical.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define PITCH_MAX_DIM 1024
static const float TWO_PI_F = 6.28318530717958647692f;
static const float INV_TWO_PI_F = 0.15915494309189533577f;

/* PITCHKernels.metal:26-31 */
static inline uint32_t pcg_hash(uint32_t v) {
    uint32_t state = v * 747796405u + 2891336453u;
    uint32_t word = ((state >> ((state >> 28u) + 4u)) ^ state) * 277803737u;
    return (word >> 22u) ^ word;
}

/* PITCHKernels.metal:34-37 */
static inline float rand_sign(uint32_t seed, uint32_t i) {
    return (pcg_hash(seed + i) & 1u) ? 1.0f : -1.0f;
}

static inline int words_per_vector(int dim, int bits) { return (dim * bits + 31) >> 5; } /* :40-43 */

/* PITCHKernels.metal:46-55: stages len = 1, 2, 4 ...; element with bit `len` clear
 * becomes lo+hi, its partner lo-hi. */
static void wht_f32(float* s, int dim) {
    for (int len = 1; len < dim; len <<= 1)
        for (int i = 0; i < dim; ++i)
            if (!(i & len)) {
                float lo = s[i], hi = s[i | len];
                s[i] = lo + hi;
                s[i | len] = lo - hi;
            }
}

/* balanced adjacent-pair tree (see header) */
static float tree_sum(float* t, int n) {
    for (; n > 1; n >>= 1)
        for (int j = 0; j < n / 2; ++j) t[j] = t[2 * j] + t[2 * j + 1];
    return t[0];
}

static float rsqrt_dim(int dim) { return (float)(1.0 / sqrt((double)dim)); }

/* PITCHKernels.metal:86-100 / reference/pitch_reference.py:68-79 */
static void pack_vector(const uint32_t* codes, uint32_t* out, int dim, int bits) {
    int words = words_per_vector(dim, bits);
    memset(out, 0, (size_t)words * 4);
    for (int i = 0; i < dim; ++i) {
        int start = i * bits, w = start >> 5, off = start & 31;
        out[w] |= codes[i] << off;
        if (off + bits > 32) out[w + 1] |= codes[i] >> (32 - off);
    }
}

/* PITCHKernels.metal:103-111 */
static inline uint32_t unpack_code(const uint32_t* buf, int i, int bits) {
    int start = i * bits, w = start >> 5, off = start & 31;
    uint32_t v = buf[w] >> off;
    if (off + bits > 32) v |= buf[w + 1] << (32 - off);
    return v & ((1u << bits) - 1u);
}

/* float32 decision boundaries 0.5f*(c[i-1]+c[i])  (PITCHKernels.metal:145) */
void pitch_oracle_edges(const float* codebook, int bits, float* edges) {
    for (int i = 1; i < (1 << bits); ++i) edges[i - 1] = 0.5f * (codebook[i - 1] + codebook[i]);
}

/* PITCHKernels.metal:114-152 */
void pitch_oracle_turbo_encode(const float* in, int64_t count, int dim, int bits, uint32_t seed,
                               const float* codebook, uint32_t* codes, float* norms) {
    const int words = words_per_vector(dim, bits);
    const int levels = 1 << bits;
    const float rs = rsqrt_dim(dim);
    float edges[256];
    pitch_oracle_edges(codebook, bits, edges);
    for (int64_t v = 0; v < count; ++v) {
        float s[PITCH_MAX_DIM], t[PITCH_MAX_DIM];
        uint32_t c[PITCH_MAX_DIM];
        const float* x = in + v * dim;
        for (int i = 0; i < dim; ++i) t[i] = x[i] * x[i];
        const float norm = sqrtf(tree_sum(t, dim));
        const float inv = (norm > 0.0f) ? (1.0f / norm) : 0.0f;
        for (int i = 0; i < dim; ++i) s[i] = rand_sign(seed, (uint32_t)i) * x[i] * inv;
        wht_f32(s, dim);
        for (int i = 0; i < dim; ++i) {
            const float u = s[i] * rs;
            uint32_t code = 0;
            for (int step = levels >> 1; step > 0; step >>= 1) {
                uint32_t cand = code + (uint32_t)step;
                if (u > edges[cand - 1]) code = cand;
            }
            c[i] = code;
        }
        pack_vector(c, codes + v * words, dim, bits);
        norms[v] = norm;
    }
}

/* PITCHKernels.metal:154-174 */
void pitch_oracle_turbo_decode(const uint32_t* codes, const float* norms, int64_t count, int dim,
                               int bits, uint32_t seed, const float* codebook, float* out) {
    const int words = words_per_vector(dim, bits);
    const float rs = rsqrt_dim(dim);
    for (int64_t v = 0; v < count; ++v) {
        float s[PITCH_MAX_DIM];
        for (int i = 0; i < dim; ++i) s[i] = codebook[unpack_code(codes + v * words, i, bits)];
        wht_f32(s, dim);
        for (int i = 0; i < dim; ++i)
            out[v * dim + i] = rand_sign(seed, (uint32_t)i) * s[i] * rs * norms[v];
    }
}

/* PITCHKernels.metal:178-222 */
void pitch_oracle_polar_encode(const float* in, int64_t count, int dim, int bits, uint32_t seed,
                               uint32_t* codes, float* scales) {
    const int words = words_per_vector(dim, bits);
    const float rs = rsqrt_dim(dim);
    const uint32_t radius_levels = (1u << bits) - 1u, angle_bins = 1u << bits;
    for (int64_t v = 0; v < count; ++v) {
        float s[PITCH_MAX_DIM], r[PITCH_MAX_DIM / 2];
        uint32_t c[PITCH_MAX_DIM];
        for (int i = 0; i < dim; ++i) s[i] = rand_sign(seed, (uint32_t)i) * in[v * dim + i];
        wht_f32(s, dim);
        float rmax = 0.0f;
        for (int p = 0; p < dim / 2; ++p) {
            const float a = s[2 * p] * rs, b = s[2 * p + 1] * rs;
            const float aa = a * a, bb = b * b;
            r[p] = sqrtf(aa + bb);
            rmax = fmaxf(rmax, r[p]);
        }
        const float safe = (rmax > 0.0f) ? rmax : 1.0f;
        const float radius_scale = (float)radius_levels / safe;              /* one division per vector */
        const float angle_scale = (float)angle_bins * INV_TWO_PI_F;          /* bins per radian */
        for (int p = 0; p < dim / 2; ++p) {
            const float a = s[2 * p] * rs, b = s[2 * p + 1] * rs;
            const float scaled = r[p] * radius_scale;
            float q = floorf(scaled + 0.5f);
            q = fminf(fmaxf(q, 0.0f), (float)radius_levels);
            c[2 * p] = (uint32_t)q;
            /* theta in (-pi, pi]: a negative bin index wraps to the bin of theta + 2*pi */
            const float turns = atan2f(b, a) * angle_scale;
            c[2 * p + 1] = (uint32_t)(int32_t)floorf(turns + 0.5f) & (angle_bins - 1u);
        }
        pack_vector(c, codes + v * words, dim, bits);
        scales[v] = rmax;
    }
}

/* PITCHKernels.metal:178-222, operation for operation (lines 207-214 for the two codes) */
void pitch_oracle_polar_encode_metal(const float* in, int64_t count, int dim, int bits, uint32_t seed,
                                     uint32_t* codes, float* scales) {
    const int words = words_per_vector(dim, bits);
    const float rs = rsqrt_dim(dim);
    const uint32_t radius_levels = (1u << bits) - 1u, angle_bins = 1u << bits;
    for (int64_t v = 0; v < count; ++v) {
        float s[PITCH_MAX_DIM], r[PITCH_MAX_DIM / 2];
        uint32_t c[PITCH_MAX_DIM];
        for (int i = 0; i < dim; ++i) s[i] = rand_sign(seed, (uint32_t)i) * in[v * dim + i];
        wht_f32(s, dim);
        float rmax = 0.0f;
        for (int p = 0; p < dim / 2; ++p) {
            const float a = s[2 * p] * rs, b = s[2 * p + 1] * rs;
            const float aa = a * a, bb = b * b;
            r[p] = sqrtf(aa + bb);
            rmax = fmaxf(rmax, r[p]);
        }
        const float safe = (rmax > 0.0f) ? rmax : 1.0f;
        for (int p = 0; p < dim / 2; ++p) {
            const float a = s[2 * p] * rs, b = s[2 * p + 1] * rs;
            const float ratio = r[p] / safe;
            const float scaled = ratio * (float)radius_levels;
            float q = floorf(scaled + 0.5f);
            q = fminf(fmaxf(q, 0.0f), (float)radius_levels);
            c[2 * p] = (uint32_t)q;
            float theta = atan2f(b, a);
            if (theta < 0.0f) theta += TWO_PI_F;
            const float turns = theta / TWO_PI_F;
            const float bin = turns * (float)angle_bins;
            c[2 * p + 1] = (uint32_t)floorf(bin + 0.5f) & (angle_bins - 1u);
        }
        pack_vector(c, codes + v * words, dim, bits);
        scales[v] = rmax;
    }
}

/* PITCHKernels.metal:224-246 */
void pitch_oracle_polar_decode(const uint32_t* codes, const float* scales, int64_t count, int dim,
                               int bits, uint32_t seed, float* out) {
    const int words = words_per_vector(dim, bits);
    const float rs = rsqrt_dim(dim);
    for (int64_t v = 0; v < count; ++v) {
        float s[PITCH_MAX_DIM];
        const uint32_t* w = codes + v * words;
        for (int p = 0; p < dim / 2; ++p) {
            const float r = (float)unpack_code(w, 2 * p, bits) / (float)((1u << bits) - 1u) * scales[v];
            const float theta = (float)unpack_code(w, 2 * p + 1, bits) / (float)(1u << bits) * TWO_PI_F;
            s[2 * p] = r * cosf(theta);
            s[2 * p + 1] = r * sinf(theta);
        }
        wht_f32(s, dim);
        for (int i = 0; i < dim; ++i) out[v * dim + i] = rand_sign(seed, (uint32_t)i) * s[i] * rs;
    }
}

/* float <-> IEEE binary16, round to nearest even (what `half(x)` does, PITCHKernels.metal:283-284) */
static uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) return (uint16_t)(sign | (x > 0x7F800000u ? 0x7E00u : 0x7C00u));
    if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);          /* rounds to infinity */
    if (x < 0x33000001u) return (uint16_t)sign;                       /* rounds to zero */
    int exp = (int)(x >> 23) - 127;
    uint32_t man = (x & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (exp < -14) { shift = 13 + (-14 - exp); base = 0; }            /* subnormal half */
    else { shift = 13; base = (uint32_t)(exp + 15) << 10; man &= 0x7FFFFFu; }
    uint32_t q = man >> shift, rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    return (uint16_t)(sign | (base + q));                             /* carry into exponent is correct */
}

static float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, x;
    if (exp == 0) {
        if (man == 0) x = sign;
        else {
            int e = -1;
            do { ++e; man <<= 1; } while (!(man & 0x400u));
            x = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
        }
    } else if (exp == 31) x = sign | 0x7F800000u | man << 13;
    else x = sign | (exp + 112u) << 23 | man << 13;
    float f;
    memcpy(&f, &x, 4);
    return f;
}

uint16_t pitch_oracle_f32_to_f16(float f) { return f32_to_f16(f); }
float pitch_oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

/* PITCHKernels.metal:262-303 / reference/pitch_reference.py:145-162 */
void pitch_oracle_channel_encode(const float* in, int64_t count, int dim, int bits, int group_size,
                                 uint32_t* codes, uint16_t* ranges) {
    const int words = words_per_vector(dim, bits);
    const float levels = (float)((1u << bits) - 1u);
    const int64_t groups = (count + group_size - 1) / group_size;
    for (int64_t g = 0; g < groups; ++g) {
        const int64_t first = g * group_size;
        const int64_t n = (count - first < group_size) ? count - first : group_size;
        float base[PITCH_MAX_DIM], step[PITCH_MAX_DIM];
        uint32_t c[PITCH_MAX_DIM];
        for (int ch = 0; ch < dim; ++ch) {
            float lo = in[first * dim + ch], hi = lo;
            for (int64_t t = 1; t < n; ++t) {
                const float x = in[(first + t) * dim + ch];
                lo = fminf(lo, x);
                hi = fmaxf(hi, x);
            }
            const uint16_t lo16 = f32_to_f16(lo), hi16 = f32_to_f16(hi);
            ranges[g * 2 * dim + ch] = lo16;
            ranges[g * 2 * dim + dim + ch] = hi16;
            base[ch] = f16_to_f32(lo16);
            step[ch] = (f16_to_f32(hi16) - base[ch]) / levels;
            if (step[ch] == 0.0f) step[ch] = 1.0f;
        }
        for (int64_t t = 0; t < n; ++t) {
            for (int ch = 0; ch < dim; ++ch) {
                const float x = in[(first + t) * dim + ch];
                float q = floorf((x - base[ch]) / step[ch] + 0.5f);
                q = fminf(fmaxf(q, 0.0f), levels);
                c[ch] = (uint32_t)q;
            }
            pack_vector(c, codes + (first + t) * words, dim, bits);
        }
    }
}

/* PITCHKernels.metal:306-325 / reference/pitch_reference.py:165-174 */
void pitch_oracle_channel_decode(const uint32_t* codes, const uint16_t* ranges, int64_t count, int dim,
                                 int bits, int group_size, float* out) {
    const int words = words_per_vector(dim, bits);
    const float levels = (float)((1u << bits) - 1u);
    for (int64_t tok = 0; tok < count; ++tok) {
        const int64_t g = tok / group_size;
        for (int ch = 0; ch < dim; ++ch) {
            const float base = f16_to_f32(ranges[g * 2 * dim + ch]);
            float step = (f16_to_f32(ranges[g * 2 * dim + dim + ch]) - base) / levels;
            if (step == 0.0f) step = 1.0f;
            const float code = (float)unpack_code(codes + tok * words, ch, bits);
            const float prod = code * step;
            out[tok * dim + ch] = prod + base;
        }
    }
}
