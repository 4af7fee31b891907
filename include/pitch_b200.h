/*
 * pitch_b200.h - C ABI of the B200 (sm_100a) KV-cache codec.
 *
 * Drop-in boundary for the codec hot path of SwiftCham/PITCH.  The reference
 * has no C interface: its kernels are reached through the Swift command
 * encoders `Codec` (Sources/PITCH/Core/Codec.swift) and `ChannelCodec`
 * (Sources/PITCH/PerChannel.swift:300-390), which validate the caller's
 * buffers and append one compute dispatch to the caller's command buffer.
 * Every entry point below replaces one of those methods; the comment on each
 * names it.  Translation of terms:
 *
 *   MTLBuffer + byte offset   ->  pitch_buffer { device pointer, length, offset }
 *   MTLCommandBuffer          ->  cudaStream_t (passed as void*)
 *   throws PITCHError.<case>  ->  returned pitch_status (never throws, never aborts)
 *
 * All enqueue functions are stream-ordered: they launch and return; outputs
 * are valid once the work queued on `stream` before them has completed.  They
 * allocate nothing, are re-entrant and thread-safe, write exactly the bytes
 * documented and leave every other byte of the output buffers untouched.
 * Inputs are not inspected on the device path (same contract as
 * Sources/PITCH/PITCH.swift:136-143).
 *
 * Plain C: no CUDA or torch types appear in any signature.
 */
#ifndef PITCH_B200_H
#define PITCH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PITCH_ABI_VERSION 2
#define PITCH_DEFAULT_SEED 0x50495443u /* Sources/PITCH/PITCH.swift:18 */
#define PITCH_MAX_DIM 1024             /* Sources/PITCH/Models/QuantConfig.swift:13 */
#define PITCH_MIN_BITS 2               /* Sources/PITCH/Models/QuantConfig.swift:12 */
#define PITCH_MAX_BITS 8
#define PITCH_MAX_GROUP 65536          /* Sources/PITCH/PerChannel.swift:18 */

/* One code per case of PITCHError (Sources/PITCH/Core/PITCHError.swift:10-19). */
typedef enum pitch_status {
    PITCH_OK = 0,
    PITCH_ERR_INVALID_INPUT = 1,          /* .invalidInput */
    PITCH_ERR_INVALID_BIT_WIDTH = 2,      /* .invalidBitWidth */
    PITCH_ERR_INVALID_DIMENSION = 3,      /* .invalidDimension */
    PITCH_ERR_CONFIGURATION_MISMATCH = 4, /* .configurationMismatch */
    PITCH_ERR_KERNEL_UNAVAILABLE = 5,     /* .shaderCompilationFailed: no kernel image for this GPU */
    PITCH_ERR_ENCODING_FAILED = 6,        /* .encodingFailed: launch error on an encode path */
    PITCH_ERR_DECODING_FAILED = 7,        /* .decodingFailed: launch error on a decode path */
    PITCH_ERR_DEVICE_NOT_SUPPORTED = 8    /* .metalNotSupported: no usable CUDA device */
} pitch_status;

/* Sources/PITCH/Models/QuantMethod.swift:8-11 */
typedef enum pitch_method { PITCH_TURBO_QUANT = 0, PITCH_POLAR_QUANT = 1 } pitch_method;

/* Element type of the full-precision side (encode input / decode output).  The reference is
 * float32 only (README.md "Limitations"); fp16 and bf16 are converted inside the kernels. */
typedef enum pitch_dtype { PITCH_F32 = 0, PITCH_F16 = 1, PITCH_BF16 = 2 } pitch_dtype;

/* A device allocation and a byte offset into it: the (MTLBuffer, offset) pair of the reference.
 * `offset` must be a non-negative multiple of 4 and `length - offset` must cover what the call
 * reads or writes (Codec.check, Sources/PITCH/Core/Codec.swift:37-47). */
typedef struct pitch_buffer {
    void*   base;    /* device pointer to the start of the allocation */
    int64_t length;  /* bytes in the allocation */
    int64_t offset;  /* byte offset at which this call starts */
} pitch_buffer;

int pitch_abi_version(void);
/* Static description of a status code. */
const char* pitch_status_string(int status);
/* Detail of the last failure on the calling thread (the associated String of PITCHError). */
const char* pitch_last_error(void);

/* Bytes of packed codes per vector / token: ceil(dim*bits/32)*4.
 * QuantConfig.codeStride, Sources/PITCH/Models/QuantConfig.swift:47. */
int pitch_code_stride(int dim, int bits);

/* Registers the 2^bits ascending float32 centroids TurboQuant uses for (dim, bits), copied into
 * a host-side table; kernels receive them by value at launch, as Codec.swift:93 does with
 * setBytes.  Replaces TurboCodebooks.codebook(dim:bits:) (Sources/PITCH/TurboCodebooks.swift),
 * whose values are reference/codebooks.json. */
int pitch_set_codebook(int dim, int bits, const float* centroids);
int pitch_has_codebook(int dim, int bits);

/* Codec.encodeCompress (Sources/PITCH/Core/Codec.swift:70-103), reached from
 * PITCH.enqueueEncode (Sources/PITCH/PITCH.swift:144-154).
 * Reads  count*dim elements of `dtype` from input.
 * Writes count*stride bytes of codes and count float32 scales (norm or rmax).
 * count*dim is not limited to 32 bits (the reference rejects more, Codec.swift:30-32). */
int pitch_enqueue_encode(int method, int dim, int bits, uint32_t seed, int dtype,
                         pitch_buffer input, pitch_buffer codes, pitch_buffer scales,
                         int64_t count, void* stream);

/* Codec.encodeDecompress (Sources/PITCH/Core/Codec.swift:107-140), reached from
 * PITCH.enqueueDecode (Sources/PITCH/PITCH.swift:156-165).
 * Writes count*dim elements of `dtype` to output. */
int pitch_enqueue_decode(int method, int dim, int bits, uint32_t seed, int dtype,
                         pitch_buffer codes, pitch_buffer scales, pitch_buffer output,
                         int64_t count, void* stream);

/* ChannelCodec.encode (Sources/PITCH/PerChannel.swift:338-363), reached from
 * PITCH.enqueuePerChannelEncode (PerChannel.swift:251-260).  Token-major input, groups of
 * `group_size` tokens (the last may be partial).  Writes count*stride code bytes and
 * ceil(count/group_size) * 2*dim fp16 values: dim minima then dim maxima per group. */
int pitch_enqueue_channel_encode(int dim, int bits, int group_size, int dtype,
                                 pitch_buffer input, pitch_buffer codes, pitch_buffer ranges,
                                 int64_t count, void* stream);

/* ChannelCodec.decode (Sources/PITCH/PerChannel.swift:365-389), reached from
 * PITCH.enqueuePerChannelDecode (PerChannel.swift:261-270). */
int pitch_enqueue_channel_decode(int dim, int bits, int group_size, int dtype,
                                 pitch_buffer codes, pitch_buffer ranges, pitch_buffer output,
                                 int64_t count, void* stream);

/* The rotation alone, float32 in and out: wht / rotate / unrotate of the specification
 * (reference/pitch_reference.py:21-34; wht_inplace and rand_sign in
 * Sources/PITCH/Shaders/PITCHKernels.metal:34-55).  mode 0: unnormalised Walsh-Hadamard
 * transform; 1: WHT(x * signs) / sqrt(dim); 2: WHT(y) * signs / sqrt(dim).  */
int pitch_enqueue_rotate(int mode, int dim, uint32_t seed, pitch_buffer input, pitch_buffer output,
                         int64_t count, void* stream);

/* pack_codes / unpack_codes of the specification (reference/pitch_reference.py:68-90;
 * pack_codes / unpack_code in Sources/PITCH/Shaders/PITCHKernels.metal:86-111): conversion
 * between one int32 per code, shape (count, dim), and the packed little-endian bit stream. */
int pitch_enqueue_pack_codes(int dim, int bits, pitch_buffer codes_i32, pitch_buffer packed,
                             int64_t count, void* stream);
int pitch_enqueue_unpack_codes(int dim, int bits, pitch_buffer packed, pitch_buffer codes_i32,
                               int64_t count, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Whole-cache decode: the per-step bottleneck named in README.md:96 and shown in the usage
 * pattern README.md:62-77 (one enqueueDecode per tensor over the whole cache).  One launch
 * decodes every plane (a K or V tensor of the cache) for every segment (layer x KV head held by
 * this GPU).  It computes exactly what one pitch_enqueue_decode / pitch_enqueue_channel_decode
 * per (plane, segment) would, with the same results.
 * ------------------------------------------------------------------------------------------- */
typedef enum pitch_plane_kind {
    PITCH_PLANE_TURBO = 0,   /* TurboQuant codes + float32 norms  */
    PITCH_PLANE_POLAR = 1,   /* PolarQuant codes + float32 rmax   */
    PITCH_PLANE_CHANNEL = 2  /* per-channel codes + fp16 ranges   */
} pitch_plane_kind;

/* Rotary tables and key-projection bias for exact key-bias removal (see pitch_enqueue_rope_bias). */
typedef struct pitch_rope_bias {
    const float* bias;          /* [segments][dim] */
    int64_t bias_seg_stride;    /* bytes */
    const float* cos_table;     /* [positions][dim] */
    const float* sin_table;     /* [positions][dim] */
    int64_t positions;
} pitch_rope_bias;

/* Every pointer of a plane comes with the number of bytes the caller's allocation holds from that
 * pointer on: the (MTLBuffer.length - offset) that Codec.check tests against the bytes a call
 * needs (Sources/PITCH/Core/Codec.swift:42-46).  A call fails with PITCH_ERR_INVALID_INPUT, before
 * anything is launched, when a plane's buffers are too small for the segments and tokens it
 * addresses, are not device memory, or live on different GPUs (Codec.swift:38-40). */
typedef struct pitch_plane {
    int32_t  kind;        /* pitch_plane_kind */
    int32_t  bits;
    int32_t  group_size;  /* PITCH_PLANE_CHANNEL only */
    uint32_t seed;        /* rotation seed (turbo / polar) */
    void*    codes;       /* segment s, token t at codes + s*codes_seg_stride + t*stride(dim,bits) */
    int64_t  codes_seg_stride;
    void*    side;        /* float32 [tokens] per segment, or fp16 [groups][2][dim] per segment */
    int64_t  side_seg_stride;
    void*    out;         /* [tokens][dim] of out_dtype per segment; may be NULL where it is not used */
    int64_t  out_seg_stride;
    int64_t  codes_bytes; /* bytes available from `codes` */
    int64_t  side_bytes;  /* bytes available from `side` */
    int64_t  out_bytes;   /* bytes available from `out` (0 with a NULL out) */
} pitch_plane;

typedef struct pitch_cache_desc {
    int32_t dim;
    int32_t out_dtype;   /* pitch_dtype */
    int64_t segments;    /* layers x KV heads on this GPU */
    int64_t tokens;      /* tokens currently held per segment */
    int32_t n_planes;    /* 1..4 */
    int32_t reserved;    /* 0 */
    pitch_plane planes[4];
    /* Exact key-bias removal for plane 0 (the keys), or NULL: the rotated bias of a token's position
     * is subtracted from plane 0's new tokens by pitch_enqueue_cache_step before they are encoded and
     * added back to plane 0's output by pitch_enqueue_cache_decode / _step, inside the same launch
     * (README.md:100 lists this as missing from the reference's kernels; arithmetic of
     * pitch_enqueue_rope_bias below).  positions must cover every token addressed. */
    const pitch_rope_bias* key_bias;
    /* Tokens per segment the buffers were sized for, or 0.  When set, buffer extents are checked
     * against it instead of against the tokens a call addresses (so the check can be made once
     * for the life of the cache), and no call may address more. */
    int64_t capacity;
} pitch_cache_desc;

/* All pointers must be 16-byte aligned and all segment strides multiples of 16. */
int pitch_enqueue_cache_decode(const pitch_cache_desc* desc, void* stream);

/* Appends n_new tokens per segment to every plane of a cache: the growing-cache pattern of
 * README.md:62-71 (enqueueEncode of the new token at codesOffset = t*h*codeStride) and, for
 * per-channel planes, README.md:85 ("the newest, partial group can be ... re-encoded as it
 * grows").  desc->tokens is the number of tokens held BEFORE the call; the codes and side
 * information of tokens [tokens, tokens + n_new) are written, for all segments and planes, by
 * one launch.  Per-channel planes keep the newest group of each segment in float32 in
 * `residual` ([segments][group_size + 2][dim]: the group's tokens, then the running per-channel
 * minimum and maximum); the new tokens are copied there and the whole group is re-encoded, so
 * codes and ranges always equal a bulk encode of the tokens seen so far.
 * All new tokens of a call must fall into one group: (tokens % group_size) + n_new <= group_size. */
typedef struct pitch_append_src {
    const void* input;            /* [segments][n_new][dim] elements of in_dtype */
    int64_t input_seg_stride;     /* bytes between segments */
    void*   residual;             /* per-channel planes only, else NULL */
    int64_t residual_seg_stride;  /* bytes between segments, >= (group_size+2)*dim*4 */
    int64_t input_bytes;          /* bytes available from `input` */
    int64_t residual_bytes;       /* bytes available from `residual` (0 with a NULL residual) */
} pitch_append_src;

int pitch_enqueue_cache_append(const pitch_cache_desc* desc, const pitch_append_src* src, int in_dtype,
                               int64_t n_new, void* stream);

/* One generation step of a compressed cache in ONE launch: appends one new token per segment to
 * every plane and decodes the whole cache, new token included - the per-step pattern of
 * README.md:62-77 (enqueueEncode of the new token, then enqueueDecode of the whole cache, in
 * one command buffer).  Results are those of pitch_enqueue_cache_append(desc, src, in_dtype, 1)
 * followed by pitch_enqueue_cache_decode at tokens + 1, bit for bit: codes, side information,
 * residual and outputs.  The planes' `out` buffers must hold tokens + 1 tokens per segment.
 *
 * `state` is NULL or points to a pitch_cache_state in device memory (16-byte aligned).
 *   NULL:     desc->tokens is the number of tokens held before the call.
 *   non-NULL: the kernel reads the token count from state->tokens instead (desc->tokens is
 *             ignored, desc->capacity must be set) and adds one to it when the step is done.  No
 *             launch parameter depends on the token count, so the same call - or a captured CUDA
 *             graph of it - can be replayed step after step with no host bookkeeping.  When the
 *             cache is full (state->tokens >= capacity) the step does nothing and sets
 *             state->status to 1.
 * Shapes off the fused path (see pitch_enqueue_cache_decode) run as the two stand-alone launches
 * and then require state == NULL. */
typedef struct pitch_cache_state {
    int64_t  tokens;    /* tokens held per segment; advanced by every step */
    int32_t  status;    /* 0, or 1 once a step was refused because the cache was full */
    uint32_t arrivals;  /* internal: must be 0 between launches */
} pitch_cache_state;

int pitch_enqueue_cache_step(const pitch_cache_desc* desc, const pitch_append_src* src, int in_dtype,
                             pitch_cache_state* state, void* stream);

/* The decoded token at the newest position (tokens - 1) of every plane and segment, gathered into
 * dst as [n_planes][segments][dim] elements of out_dtype: what a host reads back after a step
 * (README.md:73-76 reads the decoded buffer on the host) without knowing, on the host, where the
 * newest token sits.  `state` as for pitch_enqueue_cache_step: NULL -> desc->tokens tokens are held;
 * non-NULL -> the kernel reads the count from the device-side counter (desc->capacity must be set), so
 * a captured CUDA graph of (copy the new token in, step, this, copy dst out) can be replayed token
 * after token.  dst: device memory, 16-byte aligned, dst_bytes >= n_planes * segments * dim *
 * sizeof(element).  No counterpart in the reference. */
int pitch_enqueue_cache_newest(const pitch_cache_desc* desc, const pitch_cache_state* state, void* dst,
                               int64_t dst_bytes, void* stream);

/* Same as pitch_enqueue_cache_append for callers that cannot provide the residual buffer.
 * No counterpart in the reference.  Two kinds of caller are meant: a serving process that hands
 * all device memory to its own arena at start-up and forbids driver allocations afterwards
 * (cudaMalloc synchronises the whole device and can fail on a fragmented heap in the middle of
 * generation), and a host runtime that reaches this library through a foreign-function binding,
 * owns only the cache buffers it passes in, and has no device allocator with which to size a
 * residual buffer and keep it alive between steps.  For them the residual of the per-channel
 * planes lives in a fixed array inside the library image: src[i].residual and
 * src[i].residual_seg_stride are ignored, everything else is as in pitch_enqueue_cache_append.
 *   - Limit: the per-channel planes together may need at most PITCH_NOALLOC_RESIDUAL_FLOATS
 *     floats, counted as segments * (group_size + 2) * dim per plane (8 MiB; the 48-segment,
 *     dim 64, group 64 cache of the benchmark needs 0.8 MiB).  Larger requests fail with
 *     PITCH_ERR_INVALID_INPUT.  Every GPU that loads the library holds the array until exit.
 *   - The call itself allocates nothing: no cudaMalloc, cudaFree or allocating library routine.
 *     The first call on a GPU looks the array's device address up once (with that GPU current);
 *     make that first call before starting any stream capture.
 *   - One array serves every call.  It keeps the newest group of ONE cache per GPU: feed every
 *     token of that group through this entry point, and switch to another cache only when
 *     tokens is a multiple of the group size (otherwise PITCH_ERR_CONFIGURATION_MISMATCH).
 *     The cache is recognised by plane 0's `codes` pointer and its token count, nothing more: a
 *     cache that was freed and another one allocated at the same address and filled to the same
 *     count would be taken for it, so start a new cache on a group boundary (tokens = 0 is one).
 *     Nothing in it needs to start at zero: a group's running range and rows are written before
 *     they are read.  Two calls that overlap on the GPU (different streams, or two host threads)
 *     race on the array; keep calls on one GPU stream-ordered. */
#define PITCH_NOALLOC_RESIDUAL_FLOATS (2 * 1024 * 1024)
int pitch_enqueue_cache_append_noalloc(const pitch_cache_desc* desc, const pitch_append_src* src, int in_dtype,
                                       int64_t n_new, void* stream);

/* Single-token attention computed straight from the compressed cache, without writing the
 * decoded cache to memory: for every segment s and query r < n_queries
 *     out[s][r] = softmax_t(scale * <queries[s][r], K_s,t>) . V_s,t      (t < desc->tokens)
 * where K and V are what pitch_enqueue_cache_decode would reconstruct for plane 0 and plane 1
 * (before its final rounding to out_dtype).  n_queries (1...8) is the number of query heads that
 * share one KV head (grouped-query attention).  No counterpart in the reference: its README.md:96
 * names this fusion ("decoding needs to move inside the attention kernel") as the work that has
 * to follow the whole-cache decode.
 *   Supported cache shapes: dim 64 with plane 0 (keys) per-channel, 4 bits, group size a multiple
 *   of 32, or TurboQuant, 4 bits; dim 128 with TurboQuant keys of 4 or 3 bits (a Llama-3-70B-shaped
 *   cache); plane 1 (values) TurboQuant, 4 bits (3 bits where the keys have 3).  Anything else
 *   returns PITCH_ERR_INVALID_INPUT.  The
 *   planes' `out` pointers are not used and may be null.
 *   queries, out: float32 [segments][n_queries][dim], 16-byte aligned, device memory.
 *   workspace: device scratch of at least pitch_cache_attention_workspace(desc, n_queries)
 *   bytes, 16-byte aligned; its content on entry does not matter, and it may be reused by the
 *   next stream-ordered call.
 * Results agree with attention over the decoded float32 cache to about 1e-5 relative L2 (float32
 * accumulation in a different order, base-2 exponentials). */
typedef enum pitch_attention_precision {
    PITCH_ATTENTION_F32 = 0,   /* operands split into bf16 parts so that products are float32-accurate (about 1e-5) */
    PITCH_ATTENTION_BF16 = 1   /* operands as a bf16 pipeline has them: as accurate as attention over the cache
                                  decoded to bf16 (a few bf16 roundings: up to about 5e-3), half the tensor-core products and table look-ups */
} pitch_attention_precision;

typedef struct pitch_attention_args {
    const void* queries;
    void* out;
    void* workspace;
    int64_t workspace_bytes;
    int32_t n_queries;
    float scale;               /* softmax scale, usually 1/sqrt(dim) */
    int32_t precision;         /* pitch_attention_precision */
    int32_t reserved;          /* 0 */
} pitch_attention_args;
int64_t pitch_cache_attention_workspace(const pitch_cache_desc* desc, int n_queries);
int pitch_enqueue_cache_attention(const pitch_cache_desc* desc, const pitch_attention_args* args, void* stream);

/* Exact key-bias removal (reference/mechanism_eval.py:4-7 and rotated_bias, :82-91; README.md:100
 * lists it as not yet built into the reference's kernels).  A model whose key projection has a
 * bias b caches k_t = R_t W x_t + R_t b, and R_t b is known exactly, so it can be subtracted before
 * quantisation and added back after decoding at no storage cost.  In place, for every segment s,
 * vector v < count and coordinate i < dim of data (dtype elements, [segments][..][dim]):
 *     data[s][v][i] -/+= bias[s][i] * cos[p][i] + rotate_half(bias[s])[i] * sin[p][i],  p = first_position + v
 * with rotate_half(b) = (-b[dim/2:], b[:dim/2]) and cos / sin the model's own full-width rotary
 * tables (float32 [positions][dim]).  float32 arithmetic with one rounding per operation, one
 * rounding to dtype.  subtract != 0 before encoding, 0 after decoding.
 *   dim: even, a multiple of 8, at most PITCH_MAX_DIM; data 16-byte aligned, data_seg_stride a
 *   multiple of 16; first_position + count <= positions; segments <= 65535. */
int pitch_enqueue_rope_bias(int dim, int dtype, int subtract, void* data, int64_t data_seg_stride, int64_t segments,
                            int64_t first_position, int64_t count, const pitch_rope_bias* rope, void* stream);

/* 64-bit checksum of `bytes` bytes (multiple of 4) at buf: sum over 32-bit words w_i of
 * (w_i + 1) * (2*i + 1) mod 2^64, ADDED onto *result (a device uint64 the caller zeroes).
 * Used to compare shards across GPUs without moving them; no counterpart in the reference. */
int pitch_enqueue_checksum(pitch_buffer buf, int64_t bytes, uint64_t* result_device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PITCH_B200_H */
