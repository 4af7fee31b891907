// Single-token attention straight from the compressed cache (head dimension 64 with per-channel 4-bit
// or TurboQuant 4-bit keys, head dimension 128 with TurboQuant keys of 4 or 3 bits; TurboQuant values of
// the same width): the decoded cache is never written to memory.  The text below describes dimension
// 64; at 128 every row is twice as long (eight blocks of 16 channels / coordinates instead of four, four
// code words per lane instead of two, three with 3-bit codes, whose pairs are 6-bit fields cut out of
// the words by funnel shifts) and a CTA has 8 warps instead of 16, because the accumulators double.  This is the step
// the reference names as what has to come next for long contexts (README.md:96, "decoding needs
// to move inside the attention kernel").
//
// For one segment (layer x KV head) with up to eight query vectors q_r (grouped-query attention:
// the query heads that share this KV head) and T cached tokens:
//
//   scores   s_r,t = scale * sum_c q_r,c * K_t,c        with K_t,c = code_t,c * step_g,c + lo_g,c
//                  = sum_c (scale * q_r,c * step_g,c) * code_t,c  +  scale * sum_c q_r,c * lo_g,c
//            -> per group g of tokens the query is folded into the quantisation grid once; a
//               score is then a dot product with the 4-bit codes plus a bias.
//   output   o_r = sum_t p_r,t V_t / sum_t p_r,t        with V_t = norm_t/8 * D H cb[codes_t]
//                = D H ( sum_t p_r,t norm_t cb[codes_t] ) / (8 sum_t p_r,t)
//            -> centroids are accumulated in the rotated domain; the Walsh-Hadamard transform and
//               the sign diagonal are applied once per query at the very end, not once per token.
//
// Both contractions are small matrix products per tile of 32 tokens, and the eight queries of a
// KV head fill the N = 8 side of the m16n8k16 tensor-core shape exactly:
//   scores^T [tokens x queries] = codes [tokens x channels] . folded query^T [channels x queries]
//   out^T    [dims x queries]   = centroids^T [dims x tokens] . weights^T [tokens x queries]
// Operands are bf16 with float32 accumulation.  float32 quantities are split into bf16 parts
// (x = hi + mid + lo to 2^-25 for the folded query; hi + lo to 2^-17 for weights and centroids,
// accumulated as hi*hi + hi*lo + lo*hi), so the result keeps float32-like accuracy.
//  * key codes become bf16 without a conversion instruction: nibble n placed in the top mantissa
//    bits of 16.0 reads as 16 + n exactly (one shift and one logic operation per pair of codes);
//    the constant 16 * sum(folded query) goes into the bias, i.e. the accumulator's initial value;
//  * value codes of two adjacent tokens are interleaved into one byte per coordinate, and a
//    lane-replicated (bank-conflict free) table maps that byte to the hi and lo pairs of the two
//    centroids, already in A-fragment form;
//  * the score fragment (token rows, two queries per thread) becomes the weight operand of the
//    second product (token pairs per thread, one query) through movmatrix transposes.
// Free permutations make this cheap: the order of channels inside the first contraction and of
// output coordinates in the second is chosen to match how codes sit in their words.
// Thread (g, t) = (lane / 4, lane % 4).  Rows >= n_queries repeat query 0 and are discarded.
//
// TurboQuant keys (K_t = norm_t / 8 * D H cb[codes_t]) take the route of the values instead: the
// query is rotated once per run, q' = scale * H D q / 8, so that s_t = norm_t * <q', cb[codes_t]>;
// the centroids of a token's code bytes come from the same lane-replicated table as the values'
// (both planes use the codebook of (64, 4)), already in A-fragment form, and the key's norm scales
// the score row after the product.  No grouping, no folding.
//
// Kernel 1 (attention_partial_kernel): one CTA of 16 warps per SM, every warp on its own.  The
// tokens of a segment are cut into runs of whole tiles, about one run per resident warp of the
// GPU; a warp walks its run with online softmax (running maximum and sum per query, base-2
// exponentials), its next tile arriving by asynchronous copies in the second of two shared-memory
// buffers, and writes (max, sum, 64 accumulators) per query to a workspace.  Apart from the table
// build there is no barrier.
// Kernel 2 (attention_combine_kernel): merges the runs of a segment, normalises, un-rotates.
#pragma once

#include "cache_kernels.cuh"
#include "common.cuh"

namespace pitch {

constexpr int AT_MAX_QUERIES = 8;
constexpr int AT_COMBINE_WARPS = 8;
constexpr int AT_TABLE_ADDR = 0x10000;      // shared-memory address of the centroid table: byte 2 of every entry's address is 1
constexpr int AT_SMEM_RESERVED = 1024;      // start of a block's dynamic shared memory when it takes all there is
constexpr int AT_SMEM_BYTES = 232448;       // dynamic shared memory of a launch: the most a block may have (227 KB)

// Warps of a CTA (one CTA per multiprocessor): 16 at head dimension 64, 8 at 128 where the accumulators
// double - and 10 there for 4-bit codes with bf16 operands, the one variant that measured faster with
// more warps than that (20 warps at dimension 64 fit in 96 registers but ran slower: the shared-memory
// pipe, not the latency of a warp's own chain, is what the extra warps queue on).
__host__ __device__ constexpr int attn_warps(int dim, int bits, bool fast) {
    return dim == 64 ? 16 : (bits == 4 && fast ? 10 : 8);
}

// Sizes of a tile for head dimension D (64 or 128) and code width BITS (4; 3 at D = 128).
template <int D, int BITS = 4> struct AttnGeom {
    static constexpr int NKB = D / 16;                         // blocks of 16 channels / coordinates
    static constexpr int ROWB = D * BITS / 8;                  // bytes of codes per token
    static constexpr int VPITCH = ROWB + (BITS == 4 ? 16 : 8); // value rows padded (bank spread)
    static constexpr int PART_FLOATS = 2 + D;                  // per (segment, run, query): max, sum, D accumulators
    static constexpr int STAGE_K = 32 * ROWB;                  // a tile's key codes
    static constexpr int STAGE_V = 32 * VPITCH;                // a tile's value codes
};

// Layout of a CTA's shared memory for one kernel variant.
template <int D, int BITS, bool FAST, bool TK> struct AttnCta {
    typedef AttnGeom<D, BITS> G;
    static constexpr int WARPS = attn_warps(D, BITS, FAST);
    static constexpr int THREADS = WARPS * 32;
    static constexpr int QF_PARTS = FAST ? 2 : 3;                                   // bf16 parts of the query kept
    static constexpr int RANGE_BYTES = TK ? 0 : 512;                                // per-group steps and offsets of per-channel keys
    static constexpr int STAGE_BYTES = G::STAGE_K + G::STAGE_V + (TK ? 256 : 128);   // + 32 value norms (+ 32 key norms)
    // per warp: [steps, offsets;] query fragments; two tile buffers (one in flight)
    static constexpr int WARP_SMEM = RANGE_BYTES + QF_PARTS * G::NKB * 32 * 8 + 2 * STAGE_BYTES;
    // The centroid table sits at shared-memory address AT_TABLE_ADDR exactly (see table_word), the warps'
    // areas below and above it.  The kernel is launched with all the shared memory a block may have
    // (AT_SMEM_BYTES of dynamic memory), which pins the start of its dynamic memory to an address of
    // 0 ... AT_SMEM_RESERVED: a later start would not fit the multiprocessor and the launch would fail.
    static constexpr int LOW_FIT = (AT_TABLE_ADDR - AT_SMEM_RESERVED) / WARP_SMEM;
    static constexpr int LOW_WARPS = LOW_FIT < WARPS - 1 ? LOW_FIT : WARPS - 1;     // areas below the table
    static_assert(LOW_WARPS >= 1, "warps' areas on both sides of the table");
    static_assert(AT_TABLE_ADDR + CD_TABLE_BYTES + (WARPS - LOW_WARPS) * WARP_SMEM <= AT_SMEM_BYTES, "the areas above the table must fit");
};

struct AttentionParams {
    int segments, tokens, splits, tokens_per_split;    // a run: tokens_per_split tokens, a multiple of 32
    int n_queries, group_size;
    float scale_log2;                                  // softmax scale * log2(e)
    uint32_t neg[4];                                   // sign diagonal of the values' rotation (bit i of word j: coordinate 32j + i)
    uint32_t kneg[4];                                  // sign diagonal of the keys' rotation (TurboQuant keys)
    float rs;                                          // 1 / sqrt(dim)
    const unsigned char* k_codes; int64_t k_codes_seg;
    const unsigned char* k_ranges; int64_t k_ranges_seg;
    const unsigned char* v_codes; int64_t v_codes_seg;
    const unsigned char* v_norms; int64_t v_norms_seg;
    const float* q;                                    // [segments][n_queries][dim]
    float* work;                                       // [segments][splits][n_queries][2 + dim]
    float* out;                                        // [segments][n_queries][dim]
    Book16 book;                                       // TurboQuant centroids (dim, 4)
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t transpose8x8(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t bf16_pair(float x0, float x1) {     // lower half = x0
    const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// (x0, x1) -> bf16 pair of heads and bf16 pair of remainders
__device__ __forceinline__ void split_pair(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    hi = bf16_pair(x0, x1);
    lo = bf16_pair(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xFFFF0000u));
}
__device__ __forceinline__ void split_pair3(float x0, float x1, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
    hi = bf16_pair(x0, x1);
    const float r0 = x0 - __uint_as_float(hi << 16), r1 = x1 - __uint_as_float(hi & 0xFFFF0000u);
    mid = bf16_pair(r0, r1);
    lo = bf16_pair(r0 - __uint_as_float(mid << 16), r1 - __uint_as_float(mid & 0xFFFF0000u));
}
// nibbles KB and KB + 4 of a word as the bf16 pair (16 + n_KB, 16 + n_KB+4)
template <int KB>
__device__ __forceinline__ uint32_t key_pair(uint32_t w) {
    const uint32_t s = KB == 0 ? (w << 3) : (w >> (4 * KB - 3));
    return (s & 0x00780078u) | 0x41804180u;
}

// The centroid table: entry e (a byte of two 4-bit codes, or 6 bits of two 3-bit codes) holds the bf16 pair
// of its two centroids' heads in 32 lane slots of 4 bytes (every lane reads its own bank), the pair of
// remainders 128 bytes further.  Because the table starts at shared-memory address 0x10000, the address of
// (entry, lane) is the bytes (4 * lane, entry, 1, 0): one byte permutation of a code word and the lane's
// constant `slot` = AT_TABLE_ADDR | 4 * lane, with no addition.
__device__ __forceinline__ uint32_t table_word(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t table_word_lo(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1+128];" : "=r"(v) : "r"(addr));
    return v;
}
template <int B>
__device__ __forceinline__ uint32_t entry_of_byte(uint32_t w, uint32_t slot) { return __byte_perm(w, slot, 0x7604 | (B << 4)); }

// Starts the asynchronous copy of a tile (32 tokens from `tok`, `nvalid` of them existing) into a
// warp's tile buffer: key codes, value codes, norms.  Bytes of tokens that do not exist are
// zero-filled without touching memory.  k_norms: the keys' norms (TurboQuant keys) or null.
template <int D, int BITS>
__device__ __forceinline__ void issue_attn_tile(unsigned char* stage, const unsigned char* __restrict__ k_codes,
                                                const unsigned char* __restrict__ v_codes,
                                                const float* __restrict__ v_norms, const float* __restrict__ k_norms,
                                                int tok, int nvalid, int lane) {
    typedef AttnGeom<D, BITS> G;
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(stage);
    const unsigned char* ksrc = k_codes + (int64_t)tok * G::ROWB;
    const unsigned char* vsrc = v_codes + (int64_t)tok * G::ROWB;
    if (BITS == 4) {
        constexpr int CPR = G::ROWB / 16;                           // 16-byte chunks per token row
#pragma unroll
        for (int i = 0; i < CPR; ++i) {
            const int c = lane + 32 * i, token = c / CPR;            // chunk c of the tile's key bytes
            const int live = token < nvalid ? 16 : 0;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                         :: "r"(base + c * 16), "l"(live ? ksrc + c * 16 : ksrc), "r"(live) : "memory");
            // value rows are VPITCH apart (3 or 5 chunks): eight lanes that write the SAME chunk of eight
            // consecutive rows land in eight different bank groups, eight consecutive chunks do not
            const int idx = (lane >> 3) + 4 * i, vtoken = (idx / CPR) * 8 + (lane & 7), part = idx % CPR;
            const int vlive = vtoken < nvalid ? 16 : 0;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                         :: "r"(base + G::STAGE_K + vtoken * G::VPITCH + part * 16),
                            "l"(vlive ? vsrc + (vtoken * CPR + part) * 16 : vsrc), "r"(vlive) : "memory");
        }
    } else {
        // rows of 48 bytes: 8-byte pieces, so that a piece never straddles two rows
        constexpr int PPR = G::ROWB / 8;                            // pieces per token row
#pragma unroll
        for (int i = 0; i < PPR; ++i) {
            const int c = lane + 32 * i, token = c / PPR;
            const int live = token < nvalid ? 8 : 0;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;"
                         :: "r"(base + c * 8), "l"(live ? ksrc + c * 8 : ksrc), "r"(live) : "memory");
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;"
                         :: "r"(base + G::STAGE_K + token * G::VPITCH + (c % PPR) * 8), "l"(live ? vsrc + c * 8 : vsrc), "r"(live) : "memory");
        }
    }
    if (lane < 8 || (k_norms != nullptr && lane < 16)) {
        const int l8 = lane & 7;
        int live = nvalid * 4 - 16 * l8;
        live = live < 0 ? 0 : (live > 16 ? 16 : live);
        const float* nsrc = (lane < 8 ? v_norms : k_norms) + tok;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;"
                     :: "r"(base + G::STAGE_K + G::STAGE_V + lane * 16), "l"(live ? nsrc + 4 * l8 : nsrc), "r"(live) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// w[i], or w[0] where i lies beyond the array (only ever reached in code that is compiled but never run)
template <int N>
__device__ __forceinline__ uint32_t word_at(const uint32_t (&w)[N], int i) { return w[i < N ? i : 0]; }

// Table address of the pair of adjacent 3-bit codes number p (bits [6p, 6p + 6)) of a run of N code
// words, for the lane of `slot`.
template <int N>
__device__ __forceinline__ uint32_t pair3_offset(const uint32_t (&w)[N], int p, uint32_t slot) {
    const int bit = 6 * p, word = bit >> 5, off = bit & 31;
    uint32_t x;
    if (off + 6 <= 32) x = off >= 8 ? (w[word] >> (off - 8)) : (w[word] << (8 - off));
    else x = __funnelshift_r(w[word], w[word + 1 < N ? word + 1 : word], off - 8);
    return (x & 0x3F00u) | slot;
}

template <int D> struct AttnState {
    float m0, m1, l0, l1;         // running maximum and (per-thread partial) sum of queries 2t and 2t + 1
    float acc[D / 16][4];         // out^T fragments: [block of 16 coordinates][fragment register]
};

// One tile: scores, online softmax, value accumulation.  kb / vb / nb: this lane's places in the
// tile buffer (key row g words 2t, 2t+1; value row 2t word g; norm g); qf: its folded-query fragments
// in shared memory (stride 32 entries); bias0/1: score offsets of queries 2t and 2t + 1.
// FAST: operands as a bf16 pipeline would have them - the folded query in two bf16 parts instead of
// three (one part alone doubles the error of attention over a bf16 cache: the folded query multiplies
// 16 + code, the rotated query of TurboQuant keys has all its coordinates of one magnitude), weights and
// centroids in one instead of two - which halves the tensor-core products and the table look-ups; the
// result is then as accurate as attention over the cache decoded to bf16.
// TK: TurboQuant keys - the A operand of the score product is looked up in the centroid table and the
// key norms (128 bytes after the value norms) scale the score rows.
template <int D, int BITS, bool FAST, bool TK>
__device__ __forceinline__ void attn_tile(const unsigned char* kb, const unsigned char* vb, const unsigned char* nb,
                                          AttnState<D>& st, const uint2* qf,
                                          float bias0, float bias1, int nvalid, uint32_t slot, int g) {
    // ---- scores^T: two blocks of 16 tokens x 8 queries; one accumulator per part of the query, so
    //      that six short chains of products are in flight instead of two long ones
    typedef AttnGeom<D, BITS> G;
    constexpr int NKB = G::NKB, WPL = D * BITS / 128;             // code words per lane and row: 2 or 4 (3 at 3 bits)
    uint32_t kc[2][2][WPL];                                       // this lane's words of tokens 16m + g and 16m + g + 8
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (BITS == 3) {
#pragma unroll
                for (int i = 0; i < WPL; ++i) kc[m][h][i] = *reinterpret_cast<const uint32_t*>(kb + (16 * m + 8 * h) * G::ROWB + 4 * i);
            } else if (WPL == 2) {
                const uint2 v = *reinterpret_cast<const uint2*>(kb + (16 * m + 8 * h) * G::ROWB);
                kc[m][h][0] = v.x; kc[m][h][1] = v.y;
            } else {
                const uint4 v = *reinterpret_cast<const uint4*>(kb + (16 * m + 8 * h) * G::ROWB);
                kc[m][h][0] = v.x; kc[m][h][1] = v.y; kc[m][h][WPL - 2] = v.z; kc[m][h][WPL - 1] = v.w;
            }
        }
    float sc[2][4], sm[2][4], sl[2][4];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        sc[m][0] = bias0; sc[m][1] = bias1; sc[m][2] = bias0; sc[m][3] = bias1;
#pragma unroll
        for (int i = 0; i < 4; ++i) { sm[m][i] = 0.0f; sl[m][i] = 0.0f; }
    }
    // block KB of 16 channels: words 2*(KB/4), 2*(KB/4) + 1 of the lane's words, byte / nibble pair KB % 4
#define PITCH_QK(KB)                                                                                 \
    if (KB < NKB) {                                                                                  \
        constexpr int W = 2 * ((KB) >> 2) < D / 32 ? 2 * ((KB) >> 2) : 0, B = (KB) & 3;              \
        const uint2 qh = qf[(0 * NKB + KB) * 32], qm = qf[(1 * NKB + KB) * 32];                      \
        uint2 ql = make_uint2(0, 0);                                                                 \
        if (!FAST) ql = qf[(2 * NKB + KB) * 32];                                                     \
        _Pragma("unroll")                                                                            \
        for (int m = 0; m < 2; ++m) {                                                                \
            if (TK) {                                                                                \
                /* the pair of adjacent codes number 4W + B (and four pairs on) of rows g and g+8 */ \
                uint32_t e0, e1, e2, e3;                                                             \
                if (BITS == 4) {                                                                     \
                    e0 = entry_of_byte<B>(word_at(kc[m][0], W), slot);                               \
                    e1 = entry_of_byte<B>(word_at(kc[m][1], W), slot);                               \
                    e2 = entry_of_byte<B>(word_at(kc[m][0], W + 1), slot);                           \
                    e3 = entry_of_byte<B>(word_at(kc[m][1], W + 1), slot);                           \
                } else {                                                                             \
                    e0 = pair3_offset(kc[m][0], 4 * W + B, slot);                                    \
                    e1 = pair3_offset(kc[m][1], 4 * W + B, slot);                                    \
                    e2 = pair3_offset(kc[m][0], 4 * W + B + 4, slot);                                \
                    e3 = pair3_offset(kc[m][1], 4 * W + B + 4, slot);                                \
                }                                                                                    \
                const uint32_t a0 = table_word(e0), a1 = table_word(e1), a2 = table_word(e2), a3 = table_word(e3); \
                mma_bf16(sc[m], a0, a1, a2, a3, qh.x, qh.y);                                         \
                mma_bf16(sm[m], a0, a1, a2, a3, qm.x, qm.y);                                         \
                if (!FAST) {                                                                         \
                    const uint32_t l0 = table_word_lo(e0), l1 = table_word_lo(e1), l2 = table_word_lo(e2), l3 = table_word_lo(e3); \
                    mma_bf16(sl[m], a0, a1, a2, a3, ql.x, ql.y);                                     \
                    mma_bf16(sl[m], l0, l1, l2, l3, qh.x, qh.y);                                     \
                    mma_bf16(sl[m], l0, l1, l2, l3, qm.x, qm.y);                                     \
                }                                                                                    \
            } else {                                                                                 \
                const uint32_t a0 = key_pair<B>(word_at(kc[m][0], W)), a1 = key_pair<B>(word_at(kc[m][1], W)); \
                const uint32_t a2 = key_pair<B>(word_at(kc[m][0], W + 1)), a3 = key_pair<B>(word_at(kc[m][1], W + 1)); \
                mma_bf16(sc[m], a0, a1, a2, a3, qh.x, qh.y);                                         \
                mma_bf16(sm[m], a0, a1, a2, a3, qm.x, qm.y);                                         \
                if (!FAST) mma_bf16(sl[m], a0, a1, a2, a3, ql.x, ql.y);                              \
            }                                                                                        \
        }                                                                                            \
    }
    PITCH_QK(0) PITCH_QK(1) PITCH_QK(2) PITCH_QK(3) PITCH_QK(4) PITCH_QK(5) PITCH_QK(6) PITCH_QK(7)
#undef PITCH_QK
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[m][i] += FAST ? sm[m][i] : sm[m][i] + sl[m][i];
    if (TK) {
        // s_t = norm_t * <q', centroids>: rows g and g + 8 of each block of 16 tokens
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const float n0 = *reinterpret_cast<const float*>(nb + 128 + (16 * m) * 4);
            const float n1 = *reinterpret_cast<const float*>(nb + 128 + (16 * m + 8) * 4);
            sc[m][0] *= n0; sc[m][1] *= n0; sc[m][2] *= n1; sc[m][3] *= n1;
        }
    }
    if (nvalid < 32) {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            if (16 * m + g >= nvalid) { sc[m][0] = -INFINITY; sc[m][1] = -INFINITY; }
            if (16 * m + 8 + g >= nvalid) { sc[m][2] = -INFINITY; sc[m][3] = -INFINITY; }
        }
    }
    // ---- online softmax (base 2); sums over tokens stay per thread until the end of the run
    float x0 = fmaxf(fmaxf(sc[0][0], sc[0][2]), fmaxf(sc[1][0], sc[1][2]));
    float x1 = fmaxf(fmaxf(sc[0][1], sc[0][3]), fmaxf(sc[1][1], sc[1][3]));
#pragma unroll
    for (int s = 4; s < 32; s <<= 1) {
        x0 = fmaxf(x0, __shfl_xor_sync(0xFFFFFFFFu, x0, s));
        x1 = fmaxf(x1, __shfl_xor_sync(0xFFFFFFFFu, x1, s));
    }
    if (__any_sync(0xFFFFFFFFu, x0 > st.m0 || x1 > st.m1)) {
        const float n0 = fmaxf(st.m0, x0), n1 = fmaxf(st.m1, x1);
        const float c0 = fast_exp2(st.m0 - n0), c1 = fast_exp2(st.m1 - n1);     // 0 on the first tile
        st.l0 *= c0; st.l1 *= c1;
#pragma unroll
        for (int mb = 0; mb < NKB; ++mb) { st.acc[mb][0] *= c0; st.acc[mb][1] *= c1; st.acc[mb][2] *= c0; st.acc[mb][3] *= c1; }
        st.m0 = n0; st.m1 = n1;
    }
    uint32_t wh[2][2], wl[2][2];                                  // weights^T, B fragments per 16 tokens
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float p0 = fast_exp2(sc[m][2 * h] - st.m0), p1 = fast_exp2(sc[m][2 * h + 1] - st.m1);
            st.l0 += p0; st.l1 += p1;
            const float norm = *reinterpret_cast<const float*>(nb + (16 * m + 8 * h) * 4);
            if (FAST) {
                wh[m][h] = transpose8x8(bf16_pair(p0 * norm, p1 * norm));
                wl[m][h] = 0;
            } else {
                uint32_t hi, lo;
                split_pair(p0 * norm, p1 * norm, hi, lo);
                wh[m][h] = transpose8x8(hi);
                wl[m][h] = transpose8x8(lo);
            }
        }
    }
    // ---- out^T += centroids^T . weights^T
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int half = 0; half < D / 64; ++half) {
            uint32_t ch[4][4], cl[4][4];                               // [coordinate block][fragment register]
            uint32_t e[4][4];                                          // table addresses of the same
            if (BITS == 4) {
                // coordinate-wise interleave of the token pairs (2t, 2t+1) and (2t+8, 2t+9)
                // word g (+ 8 per half) of tokens 16m + {2t, 2t+1, 2t+8, 2t+9}: coordinates 64 * half + 8g ...
                const unsigned char* vrow = vb + 16 * m * G::VPITCH + half * 32;
                const uint32_t v0 = *reinterpret_cast<const uint32_t*>(vrow), v1 = *reinterpret_cast<const uint32_t*>(vrow + G::VPITCH);
                const uint32_t v2 = *reinterpret_cast<const uint32_t*>(vrow + 8 * G::VPITCH), v3 = *reinterpret_cast<const uint32_t*>(vrow + 9 * G::VPITCH);
                const uint32_t ea = (v0 & 0x0F0F0F0Fu) | ((v1 << 4) & 0xF0F0F0F0u);   // even coordinates
                const uint32_t oa = ((v0 >> 4) & 0x0F0F0F0Fu) | (v1 & 0xF0F0F0F0u);   // odd coordinates
                const uint32_t eb = (v2 & 0x0F0F0F0Fu) | ((v3 << 4) & 0xF0F0F0F0u);
                const uint32_t ob = ((v2 >> 4) & 0x0F0F0F0Fu) | (v3 & 0xF0F0F0F0u);
#pragma unroll
                for (int mb = 0; mb < 4; ++mb) {
                    e[mb][0] = __byte_perm(ea, slot, 0x7604 | (mb << 4));
                    e[mb][1] = __byte_perm(oa, slot, 0x7604 | (mb << 4));
                    e[mb][2] = __byte_perm(eb, slot, 0x7604 | (mb << 4));
                    e[mb][3] = __byte_perm(ob, slot, 0x7604 | (mb << 4));
                }
            } else {
                // 3-bit codes: the 8 coordinates 64 * half + 8g ... of a token are 24 bits at byte 3g + 24 * half
                // of its row (vb points 4g bytes into the row of token 2t, the place of the 4-bit word)
                const int byte0 = 3 * g + 24 * half;
                const unsigned char* vrow = vb - 4 * g + 16 * m * G::VPITCH + (byte0 & ~3);
                const int sh = 8 * (byte0 & 3);
                uint32_t x[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const unsigned char* row = vrow + ((r & 1) + 8 * (r >> 1)) * G::VPITCH;       // tokens 2t, 2t+1, 2t+8, 2t+9
                    x[r] = __funnelshift_r(*reinterpret_cast<const uint32_t*>(row), *reinterpret_cast<const uint32_t*>(row + 4), sh);
                }
#pragma unroll
                for (int mb = 0; mb < 4; ++mb) {
                    // coordinate j of tokens (A, B): entry (code_A | code_B << 3) at byte (entry << 8) + slot
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int j = 2 * mb + (k & 1);                                             // even, odd coordinate
                        const uint32_t xa = x[2 * (k >> 1)], xb = x[2 * (k >> 1) + 1];
                        const uint32_t lo3 = 3 * j >= 8 ? (xa >> (3 * j - 8)) : (xa << (8 - 3 * j));
                        const uint32_t hi3 = 3 * j >= 11 ? (xb >> (3 * j - 11)) : (xb << (11 - 3 * j));
                        e[mb][k] = (lo3 & 0x0700u) | (hi3 & 0x3800u) | slot;
                    }
                }
            }
#pragma unroll
            for (int mb = 0; mb < 4; ++mb) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    ch[mb][k] = table_word(e[mb][k]);
                    if (!FAST) cl[mb][k] = table_word_lo(e[mb][k]);
                }
            }
#pragma unroll
            for (int mb = 0; mb < 4; ++mb) mma_bf16(st.acc[4 * half + mb], ch[mb][0], ch[mb][1], ch[mb][2], ch[mb][3], wh[m][0], wh[m][1]);
            if (!FAST) {
#pragma unroll
                for (int mb = 0; mb < 4; ++mb) mma_bf16(st.acc[4 * half + mb], ch[mb][0], ch[mb][1], ch[mb][2], ch[mb][3], wl[m][0], wl[m][1]);
#pragma unroll
                for (int mb = 0; mb < 4; ++mb) mma_bf16(st.acc[4 * half + mb], cl[mb][0], cl[mb][1], cl[mb][2], cl[mb][3], wh[m][0], wh[m][1]);
            }
        }
    }
}

// Folds the queries of the run into the quantisation grid of one group of tokens: B fragments
// (three bf16 parts, left in shared memory: qf[(part * 4 + block of 16 channels) * 32 + lane])
// and the score bias of queries 2t and 2t + 1.  lo2 / hi2: this lane's two
// channels of the group's fp16 minima and maxima.
template <bool FAST>
__device__ __forceinline__ void fold_group(uint32_t lo2, uint32_t hi2, const float* __restrict__ qrow, float qscale, float* gstep, float* goff,
                                           uint2* qf, float& bias0, float& bias1, int lane, int g, int t) {
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&lo2));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&hi2));
    const float s0 = step15(lo.x, hi.x), s1 = step15(lo.y, hi.y);
    // Shared-memory layout of the per-channel rows (steps, offsets): the 16-byte chunk of channels
    // 16t + 4i ... + 3 sits at chunk index 4i + t, so that the lanes of a 128-bit load phase touch
    // different bank groups.
    const int chunk = 4 * ((lane >> 1) & 3) + (lane >> 3);            // of channels 2 * lane, 2 * lane + 1
    __syncwarp();
    // both already carry the softmax scale (base 2), so the query is used as it is
    *reinterpret_cast<float2*>(gstep + 4 * chunk + (2 * lane & 3)) = make_float2(s0 * qscale, s1 * qscale);
    *reinterpret_cast<float2*>(goff + 4 * chunk + (2 * lane & 3)) =
        make_float2(fmaf(-16.0f, s0, lo.x) * qscale, fmaf(-16.0f, s1, lo.y) * qscale);
    __syncwarp();
    float x[16];
    float b = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 qv = __ldg(reinterpret_cast<const float4*>(qrow + 16 * t + 4 * i));     // query g
        const float4 sv = *reinterpret_cast<const float4*>(gstep + 4 * (4 * i + t));
        const float4 ov = *reinterpret_cast<const float4*>(goff + 4 * (4 * i + t));
        x[4 * i] = qv.x * sv.x; x[4 * i + 1] = qv.y * sv.y; x[4 * i + 2] = qv.z * sv.z; x[4 * i + 3] = qv.w * sv.w;
        b = fmaf(qv.x, ov.x, b); b = fmaf(qv.y, ov.y, b); b = fmaf(qv.z, ov.z, b); b = fmaf(qv.w, ov.w, b);
    }
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
        uint2 h, m, l;
        if (FAST) {                                       // the third part is not used
            split_pair(x[kb], x[kb + 4], h.x, m.x);
            split_pair(x[8 + kb], x[12 + kb], h.y, m.y);
        } else {
            split_pair3(x[kb], x[kb + 4], h.x, m.x, l.x);
            split_pair3(x[8 + kb], x[12 + kb], h.y, m.y, l.y);
            qf[(2 * 4 + kb) * 32 + lane] = l;
        }
        qf[(0 * 4 + kb) * 32 + lane] = h;
        qf[(1 * 4 + kb) * 32 + lane] = m;
    }
    __syncwarp();
    b += __shfl_xor_sync(0xFFFFFFFFu, b, 1);
    b += __shfl_xor_sync(0xFFFFFFFFu, b, 2);              // bias of query g
    bias0 = __shfl_sync(0xFFFFFFFFu, b, 8 * t);           // of query 2t
    bias1 = __shfl_sync(0xFFFFFFFFu, b, 8 * t + 4);       // of query 2t + 1
}

// TurboQuant keys: the rotated query q' = qscale / sqrt(D) * H D q of query g as B fragments (three bf16
// parts, same places as fold_group's).  Lane (g, t) owns the D/4 channels from t * D/4 on: the
// Walsh-Hadamard stages of the low channel bits run in registers, those of the two top bits between the
// four lanes of a query.  Fragment slots follow the A side of the TurboQuant-key product: in block KB,
// slots (2t, 2t+1) are the lane's channels 16 (KB / 4) + 2 (KB % 4), + 1 (byte KB % 4 of its word
// 2 (KB / 4)), slots (2t+8, 2t+9) the same 8 channels further on (the next word).
template <int D, bool FAST>
__device__ __forceinline__ void rotate_query(const float* __restrict__ qrow, float qscale, float rs, const uint32_t (&kneg)[4],
                                             uint2* qf, int lane, int t) {
    constexpr int N = D / 4, NKB = D / 16;
    float x[N];
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
        const float4 qv = __ldg(reinterpret_cast<const float4*>(qrow + N * t + 4 * i));
        x[4 * i] = qv.x; x[4 * i + 1] = qv.y; x[4 * i + 2] = qv.z; x[4 * i + 3] = qv.w;
    }
    const uint32_t neg = kneg[(N * t) >> 5];
    const int shift = (N * t) & 31;
#pragma unroll
    for (int i = 0; i < N; ++i) x[i] = flip_if(x[i], neg, shift + i);
#pragma unroll
    for (int h = 1; h < N; h <<= 1)
#pragma unroll
        for (int i = 0; i < N; ++i)
            if (!(i & h)) {
                const float a = x[i], b = x[i | h];
                x[i] = a + b;
                x[i | h] = a - b;
            }
#pragma unroll
    for (int m = 1; m < 4; m <<= 1)
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const float o = __shfl_xor_sync(0xFFFFFFFFu, x[i], m);
            x[i] = (lane & m) ? o - x[i] : x[i] + o;
        }
    const float sc = qscale * rs;
    __syncwarp();
#pragma unroll
    for (int kb = 0; kb < NKB; ++kb) {
        const int i0 = 16 * (kb >> 2) + 2 * (kb & 3);
        uint2 h, m, l;
        if (FAST) {                                       // the third part is not used
            split_pair(x[i0] * sc, x[i0 + 1] * sc, h.x, m.x);
            split_pair(x[i0 + 8] * sc, x[i0 + 9] * sc, h.y, m.y);
        } else {
            split_pair3(x[i0] * sc, x[i0 + 1] * sc, h.x, m.x, l.x);
            split_pair3(x[i0 + 8] * sc, x[i0 + 9] * sc, h.y, m.y, l.y);
            qf[(2 * NKB + kb) * 32 + lane] = l;
        }
        qf[(0 * NKB + kb) * 32 + lane] = h;
        qf[(1 * NKB + kb) * 32 + lane] = m;
    }
    __syncwarp();
}

template <int D, int BITS, bool FAST, bool TK>
__global__ void __launch_bounds__(AttnCta<D, BITS, FAST, TK>::THREADS, 1)
attention_partial_kernel(const __grid_constant__ AttentionParams p) {
    static_assert(D == 64 || TK, "per-channel keys are handled at head dimension 64 only");
    static_assert(BITS == 4 || (BITS == 3 && D == 128 && TK), "3-bit codes are handled at head dimension 128 with TurboQuant keys");
    typedef AttnGeom<D, BITS> G;
    typedef AttnCta<D, BITS, FAST, TK> C;
    constexpr int AT_WARPS = C::WARPS, AT_STAGE_BYTES = C::STAGE_BYTES, AT_PART_FLOATS = G::PART_FLOATS;
    extern __shared__ __align__(1024) unsigned char smem[];
    // the table at shared address AT_TABLE_ADDR; warps 0 ... LOW_WARPS - 1 below it, the others above
    const uint32_t smem_addr = (uint32_t)__cvta_generic_to_shared(smem);            // <= AT_SMEM_RESERVED
    unsigned char* table = smem + (AT_TABLE_ADDR - smem_addr);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // (one base pointer plus an offset, so that every access stays a plain shared-memory access)
    const uint32_t area_offset = warp < C::LOW_WARPS ? (uint32_t)(warp * C::WARP_SMEM)
        : (uint32_t)(AT_TABLE_ADDR + CD_TABLE_BYTES + (warp - C::LOW_WARPS) * C::WARP_SMEM) - smem_addr;
    unsigned char* area = smem + area_offset;
    float* gstep = reinterpret_cast<float*>(area);                                          // [64] (per-channel keys only)
    float* goff = gstep + 64;                                                               // [64] lo - 16 * step
    uint2* qf = reinterpret_cast<uint2*>(area + C::RANGE_BYTES);                            // [parts][blocks][32 lanes]
    unsigned char* stage0 = reinterpret_cast<unsigned char*>(qf + C::QF_PARTS * G::NKB * 32);   // two tile buffers
    const int R = p.n_queries;
    const uint32_t slot = (uint32_t)AT_TABLE_ADDR | (uint32_t)lane * 4u;

    {
        // Before anything else: ask the L2 for the first tile of this warp's first run (its codes arrive while
        // the table is built and the grid waits for its predecessor).  A prefetch changes nothing that can be
        // observed; the addresses are inside the planes' buffers.
        const int run = blockIdx.x * C::WARPS + warp;
        if (run < p.segments * p.splits) {
            const int64_t seg = run / p.splits;
            const int64_t tok = (int64_t)(run - (int)seg * p.splits) * p.tokens_per_split;
            constexpr int LINES = G::STAGE_K / 128;                     // a tile's codes of one plane: 8, 16 or 12 lines
            const int64_t left = ((int64_t)p.tokens - tok) * G::ROWB;   // bytes of codes from the tile's first token on
            const unsigned char* src = lane < LINES ? p.k_codes + seg * p.k_codes_seg : p.v_codes + seg * p.v_codes_seg;
            const int line = lane < LINES ? lane : lane - LINES;
            if (lane < 2 * LINES && (int64_t)line * 128 < left)
                asm volatile("prefetch.global.L2 [%0];" :: "l"(src + tok * G::ROWB + line * 128));
        }
    }

    for (int e = threadIdx.x; e < (1 << (2 * BITS)); e += C::THREADS) {
        // one table entry per thread (all pairs of codes), written to its 32 lane slots
        uint32_t hi, lo;
        split_pair(p.book.c[e & ((1 << BITS) - 1)], p.book.c[e >> BITS], hi, lo);
        uint4* row = reinterpret_cast<uint4*>(table + e * 256);
#pragma unroll
        for (int i = 0; i < 16; ++i) {                   // rows are 256 bytes apart: rotate the chunk order per lane
            const int c = (i + threadIdx.x) & 15;        // so that a store phase spreads over the banks
            const uint32_t v = c < 8 ? hi : lo;
            row[c] = make_uint4(v, v, v, v);
        }
    }
    __syncthreads();
    // Everything above touched only kernel parameters and shared memory.  Under programmatic
    // dependent launch this grid may have started before the previous kernel of the stream ended:
    // wait for it before reading the cache, then let the combine kernel be scheduled early.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");

    const int n_runs = p.segments * p.splits;
    for (int run = blockIdx.x * AT_WARPS + warp; run < n_runs; run += gridDim.x * AT_WARPS) {
        const int64_t seg = run / p.splits;
        const int split = run - (int)seg * p.splits;
        const int w_begin = split * p.tokens_per_split;
        int w_end = w_begin + p.tokens_per_split;
        if (w_end > p.tokens) w_end = p.tokens;

        const __half* k_ranges = reinterpret_cast<const __half*>(p.k_ranges + seg * p.k_ranges_seg) + 2 * lane;
        const float* k_norms = TK ? reinterpret_cast<const float*>(p.k_ranges + seg * p.k_ranges_seg) : nullptr;
        const unsigned char* k_codes = p.k_codes + seg * p.k_codes_seg;
        const unsigned char* v_codes = p.v_codes + seg * p.v_codes_seg;
        const float* v_norms = reinterpret_cast<const float*>(p.v_norms + seg * p.v_norms_seg);
        // this lane's query row (query g); rows beyond n_queries repeat query 0 and are never written out
        const float* qrow = p.q + (seg * R + (g < R ? g : 0)) * D;
        const float qscale = p.scale_log2;

        AttnState<D> st;
        st.m0 = st.m1 = -INFINITY;
        st.l0 = st.l1 = 0.0f;
#pragma unroll
        for (int mb = 0; mb < G::NKB; ++mb)
#pragma unroll
            for (int i = 0; i < 4; ++i) st.acc[mb][i] = 0.0f;
        float bias0 = 0.0f, bias1 = 0.0f;

        // the first tile is on its way before anything else of the run is fetched
        __syncwarp();
        issue_attn_tile<D, BITS>(stage0, k_codes, v_codes, v_norms, k_norms, w_begin, w_end - w_begin, lane);

        // per-channel keys: the ranges of the first group; those of the following group are fetched a
        // group ahead.  TurboQuant keys: the query is rotated once, here.
        int group = TK ? 0 : w_begin / p.group_size;
        const int last_group = TK ? 0 : (w_end - 1) / p.group_size;
        int group_end = TK ? 0x7FFFFFFF : (group + 1) * p.group_size;   // first token of the next group
        uint32_t lo2 = 0, hi2 = 0;
        bool fold = !TK;
        if (TK) {
            rotate_query<D, FAST>(qrow, qscale, p.rs, p.kneg, qf, lane, t);
        } else {
            lo2 = ldg_stream32(reinterpret_cast<const uint32_t*>(k_ranges + (int64_t)group * 128));
            hi2 = ldg_stream32(reinterpret_cast<const uint32_t*>(k_ranges + (int64_t)group * 128 + 64));
        }

        // this lane's places in tile buffer 0; buffer 1 is AT_STAGE_BYTES further
        const unsigned char* kb = stage0 + g * G::ROWB + t * (G::ROWB / 4);
        const unsigned char* vb = stage0 + G::STAGE_K + 2 * t * G::VPITCH + g * 4;
        const unsigned char* nb = stage0 + G::STAGE_K + G::STAGE_V + g * 4;
#define PITCH_TILE(BUF)                                                                                  \
        {                                                                                               \
            const int nvalid = w_end - t0;                            /* >= 32 for a whole tile */      \
            if (nvalid > 32) {                                                                          \
                issue_attn_tile<D, BITS>(stage0 + (1 - BUF) * AT_STAGE_BYTES, k_codes, v_codes, v_norms, k_norms, t0 + 32, nvalid - 32, lane); \
                cp_async_wait<1>();                                                                     \
            } else {                                                                                    \
                cp_async_wait<0>();                                                                     \
            }                                                                                           \
            __syncwarp();                                                                               \
            if (!TK && t0 >= group_end) { ++group; group_end += p.group_size; fold = true; }           \
            if (!TK && fold) {                                                                          \
                fold = false;                                                                           \
                fold_group<FAST>(lo2, hi2, qrow, qscale, gstep, goff, qf, bias0, bias1, lane, g, t);          \
                if (group < last_group) {                                                               \
                    lo2 = ldg_stream32(reinterpret_cast<const uint32_t*>(k_ranges + (int64_t)(group + 1) * 128));      \
                    hi2 = ldg_stream32(reinterpret_cast<const uint32_t*>(k_ranges + (int64_t)(group + 1) * 128 + 64)); \
                }                                                                                       \
            }                                                                                           \
            attn_tile<D, BITS, FAST, TK>(kb + BUF * AT_STAGE_BYTES, vb + BUF * AT_STAGE_BYTES, nb + BUF * AT_STAGE_BYTES, st, qf + lane,  \
                      bias0, bias1, nvalid, slot, g);                                                   \
            __syncwarp();                                             /* this buffer is refilled two tiles on */ \
        }
        for (int t0 = w_begin; t0 < w_end; t0 += 32) {
            PITCH_TILE(0)
            t0 += 32;
            if (t0 >= w_end) break;
            PITCH_TILE(1)
        }
#undef PITCH_TILE

        // ---- finish the sums over tokens; this run's partial result
#pragma unroll
        for (int s = 4; s < 32; s <<= 1) {
            st.l0 += __shfl_xor_sync(0xFFFFFFFFu, st.l0, s);
            st.l1 += __shfl_xor_sync(0xFFFFFFFFu, st.l1, s);
        }
        float* d0 = p.work + ((seg * p.splits + split) * R + 2 * t) * AT_PART_FLOATS;   // query 2t
        float* d1 = d0 + AT_PART_FLOATS;                                                // query 2t + 1
        if (2 * t < R) {
            if (g == 0) { d0[0] = st.m0; d0[1] = st.l0; }
#pragma unroll
            for (int mb = 0; mb < G::NKB; ++mb)                       // coordinates 64 (mb / 4) + 8g + 2 (mb % 4) and the next
                *reinterpret_cast<float2*>(d0 + 2 + 64 * (mb >> 2) + 8 * g + 2 * (mb & 3)) = make_float2(st.acc[mb][0], st.acc[mb][2]);
        }
        if (2 * t + 1 < R) {
            if (g == 0) { d1[0] = st.m1; d1[1] = st.l1; }
#pragma unroll
            for (int mb = 0; mb < G::NKB; ++mb)
                *reinterpret_cast<float2*>(d1 + 2 + 64 * (mb >> 2) + 8 * g + 2 * (mb & 3)) = make_float2(st.acc[mb][1], st.acc[mb][3]);
        }
    }
}

// grid = (n_queries, segments), 8 warps: warp w merges runs w, w + 8, ... of its (segment, query),
// lane l owning coordinates l * D/32 ... ; warp 0 merges the eight, normalises and un-rotates.
template <int D>
__global__ void __launch_bounds__(32 * AT_COMBINE_WARPS)
attention_combine_kernel(const __grid_constant__ AttentionParams p) {
    constexpr int PF = AttnGeom<D>::PART_FLOATS, E = D / 32;       // coordinates per lane: 2 or 4
    __shared__ float part[AT_COMBINE_WARPS][PF];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x;
    const int64_t seg = blockIdx.y;
    const int R = p.n_queries;
    asm volatile("griddepcontrol.wait;" ::: "memory");       // the partial results of the kernel before this one
    const float* base = p.work + (seg * p.splits * R + r) * PF;
    const int64_t stride = (int64_t)R * PF;
    float mm = -INFINITY;
    float a[E];
#pragma unroll
    for (int e = 0; e < E; ++e) a[e] = 0.0f;
    float ll = 0.0f;
    for (int s0 = warp; s0 < p.splits; s0 += 4 * AT_COMBINE_WARPS) {
        // four runs in flight per warp
        float ms[4], ls[4];
        float v[4][E];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int s = s0 + k * AT_COMBINE_WARPS;
            ms[k] = -INFINITY; ls[k] = 0.0f;
#pragma unroll
            for (int e = 0; e < E; ++e) v[k][e] = 0.0f;
            if (s < p.splits) {
                const float* src = base + s * stride;
                ms[k] = src[0]; ls[k] = src[1];
#pragma unroll
                for (int e = 0; e < E; e += 2) {
                    const float2 f = *reinterpret_cast<const float2*>(src + 2 + E * lane + e);
                    v[k][e] = f.x; v[k][e + 1] = f.y;
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (ms[k] == -INFINITY) continue;                             // beyond the last run
            const float mn = fmaxf(mm, ms[k]);
            const float fo = fast_exp2(mm - mn), fn = fast_exp2(ms[k] - mn);
#pragma unroll
            for (int e = 0; e < E; ++e) a[e] = fmaf(v[k][e], fn, a[e] * fo);
            ll = fmaf(ls[k], fn, ll * fo);
            mm = mn;
        }
    }
    if (lane == 0) { part[warp][0] = mm; part[warp][1] = ll; }
#pragma unroll
    for (int e = 0; e < E; ++e) part[warp][2 + E * lane + e] = a[e];
    __syncthreads();
    if (warp != 0) return;
    mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < AT_COMBINE_WARPS; ++w) mm = fmaxf(mm, part[w][0]);
#pragma unroll
    for (int e = 0; e < E; ++e) a[e] = 0.0f;
    ll = 0.0f;
#pragma unroll
    for (int w = 0; w < AT_COMBINE_WARPS; ++w) {
        const float f = part[w][0] == -INFINITY ? 0.0f : fast_exp2(part[w][0] - mm);   // a warp without a run
#pragma unroll
        for (int e = 0; e < E; ++e) a[e] = fmaf(part[w][2 + E * lane + e], f, a[e]);
        ll = fmaf(part[w][1], f, ll);
    }
    // normalise, then rotate back once: H over D coordinates (E per lane), 1/sqrt(D), sign diagonal
    const float inv = p.rs / ll;
#pragma unroll
    for (int h = 1; h < E; h <<= 1)                          // stages inside the lane
#pragma unroll
        for (int i = 0; i < E; ++i)
            if (!(i & h)) {
                const float x = a[i], y = a[i | h];
                a[i] = x + y;
                a[i | h] = x - y;
            }
#pragma unroll
    for (int mbit = 1; mbit < 32; mbit <<= 1) {              // stages across lanes
        const bool upper = (lane & mbit) != 0;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float o = __shfl_xor_sync(0xFFFFFFFFu, a[e], mbit);
            a[e] = upper ? o - a[e] : a[e] + o;
        }
    }
    const uint32_t neg = p.neg[(E * lane) >> 5];
    const int bit = (E * lane) & 31;
#pragma unroll
    for (int e = 0; e < E; ++e) a[e] = flip_if(a[e] * inv, neg, bit + e);
#pragma unroll
    for (int e = 0; e < E; e += 2)
        *reinterpret_cast<float2*>(p.out + (seg * R + r) * D + E * lane + e) = make_float2(a[e], a[e + 1]);
}

}  // namespace pitch
