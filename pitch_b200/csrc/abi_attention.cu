// C ABI, attention straight from the compressed cache: pitch_enqueue_cache_attention.
// Declarations: include/pitch_b200.h.
#include "abi_internal.h"

#include <atomic>
#include <cstring>

#include "attention_kernels.cuh"
#include "common.cuh"

using namespace pitch;
using namespace pitch_abi;

// Multiprocessors of the GPU that holds the cache (the one plane 0's codes live on); 148, a full
// B200, when that cannot be told.  The run layout, and with it the workspace size, follows it.
static int desc_sm_count(const pitch_cache_desc* d) {
    cudaPointerAttributes attr;
    if (d->planes[0].codes == nullptr || cudaPointerGetAttributes(&attr, d->planes[0].codes) != cudaSuccess ||
        attr.type != cudaMemoryTypeDevice) {
        cudaGetLastError();
        return 148;
    }
    DeviceGuard guard(attr.device);
    return sm_count();
}

static int64_t plane_side_bytes(const pitch_plane& pl, int dim, int64_t tokens) {
    if (pl.kind == PITCH_PLANE_CHANNEL) return ceil_div(tokens, pl.group_size) * 4 * dim;
    return tokens * 4;
}

extern "C" {

// -------------------------------------------------------------------------------- attention
// How a segment's tokens are cut into runs (one warp each).  Depends on the shape and on the GPU's
// multiprocessor count only, so that the workspace size can be computed ahead of the call: runs of
// whole 32-token tiles, about one run per warp that the GPU keeps resident (`warps` per multiprocessor:
// attn_warps), at least 4 tiles long.
static void attention_slices(int sms, int warps, int64_t segments, int64_t tokens, int* splits, int* tokens_per_split) {
    const int64_t tiles = ceil_div(tokens, 32), slots = (int64_t)sms * warps;
    int64_t run = ceil_div(segments * tiles, slots);
    if (run < 4) run = 4;
    // rounding the runs per segment up must not push the total past the resident warps: a few
    // left-over runs would cost a whole second round
    while (run < tiles && segments * ceil_div(tiles, run) > slots && segments <= slots) ++run;
    if (run > tiles) run = tiles;
    *tokens_per_split = (int)(run * 32);
    *splits = (int)ceil_div(tiles, run);
}

static int check_attention_shape(const pitch_cache_desc* d, int n_queries) {
    if (d == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "descriptor is null");
    if (n_queries < 1 || n_queries > AT_MAX_QUERIES)
        return fail(PITCH_ERR_INVALID_INPUT, "n_queries %d must be in 1...%d", n_queries, AT_MAX_QUERIES);
    if (d->segments < 1 || d->segments > 65535 || d->tokens < 1 || d->tokens > 0x7FFFFFFF - 1024)
        return fail(PITCH_ERR_INVALID_INPUT, "segments must be in 1...65535 and tokens in 1...2^31-1025");
    if ((d->dim != 64 && d->dim != 128) || d->n_planes != 2)
        return fail(PITCH_ERR_INVALID_INPUT, "cache attention needs dim 64 or 128 and two planes (keys, values)");
    const pitch_plane& k = d->planes[0];
    const pitch_plane& v = d->planes[1];
    if (k.kind == PITCH_PLANE_TURBO) {
        if (k.bits != 4 && !(k.bits == 3 && d->dim == 128))
            return fail(PITCH_ERR_INVALID_INPUT, "cache attention needs 4-bit keys (3-bit TurboQuant keys at dim 128 only)");
    } else if (d->dim != 64) {
        return fail(PITCH_ERR_INVALID_INPUT, "cache attention at dim 128 needs TurboQuant 4-bit keys");
    } else if (k.kind != PITCH_PLANE_CHANNEL || k.bits != 4 || k.group_size < 32 || k.group_size % 32 != 0 || k.group_size > PITCH_MAX_GROUP) {
        return fail(PITCH_ERR_INVALID_INPUT, "cache attention needs TurboQuant 4-bit keys, or per-channel 4-bit keys with a group size that is a multiple of 32");
    }
    if (v.kind != PITCH_PLANE_TURBO || (v.bits != 4 && !(v.bits == 3 && d->dim == 128 && k.kind == PITCH_PLANE_TURBO)))
        return fail(PITCH_ERR_INVALID_INPUT, "cache attention needs TurboQuant 4-bit values (3-bit at dim 128 with TurboQuant keys)");
    if (k.kind == PITCH_PLANE_TURBO && k.bits != v.bits)
        return fail(PITCH_ERR_INVALID_INPUT, "cache attention needs keys and values of one width");
    return PITCH_OK;
}

int64_t pitch_cache_attention_workspace(const pitch_cache_desc* d, int n_queries) {
    if (check_attention_shape(d, n_queries)) return -1;
    // the run layout can depend on the precision of the call (attn_warps): room for either
    const int sms = desc_sm_count(d);
    int splits = 0;
    for (int fast = 0; fast < 2; ++fast) {
        int sp, tps;
        attention_slices(sms, attn_warps(d->dim, d->planes[1].bits, fast != 0), d->segments, d->tokens, &sp, &tps);
        if (sp > splits) splits = sp;
    }
    return d->segments * splits * n_queries * (2 + d->dim) * (int64_t)sizeof(float);
}

int pitch_enqueue_cache_attention(const pitch_cache_desc* d, const pitch_attention_args* a, void* stream) {
    if (a == nullptr) return fail(PITCH_ERR_INVALID_INPUT, "arguments are null");
    int st;
    if ((st = check_attention_shape(d, a->n_queries))) return st;
    if (!(a->scale > 0.0f) || !std::isfinite(a->scale)) return fail(PITCH_ERR_INVALID_INPUT, "scale must be positive and finite");
    if (a->precision != PITCH_ATTENTION_F32 && a->precision != PITCH_ATTENTION_BF16)
        return fail(PITCH_ERR_INVALID_INPUT, "unknown attention precision %d", a->precision);
    if (!a->queries || !a->out || !a->workspace) return fail(PITCH_ERR_INVALID_INPUT, "queries, out or workspace is null");
    if (!aligned16(a->queries) || !aligned16(a->out) || !aligned16(a->workspace))
        return fail(PITCH_ERR_INVALID_INPUT, "queries, out and workspace must be 16-byte aligned");
    const int64_t need = pitch_cache_attention_workspace(d, a->n_queries);
    if (a->workspace_bytes < need)
        return fail(PITCH_ERR_INVALID_INPUT, "workspace has %lld bytes; needs %lld", (long long)a->workspace_bytes, (long long)need);
    for (int i = 0; i < 2; ++i) {
        const pitch_plane& pl = d->planes[i];
        if (!pl.codes || !pl.side) return fail(PITCH_ERR_INVALID_INPUT, "plane %d: null pointer", i);
        if (!aligned16(pl.codes) || !aligned16(pl.side) || (pl.codes_seg_stride & 15) || (pl.side_seg_stride & 15))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: pointers and segment strides must be multiples of 16", i);
        if (d->segments > 1 && (pl.codes_seg_stride < d->tokens * pitch_code_stride(d->dim, pl.bits) || pl.side_seg_stride < plane_side_bytes(pl, d->dim, d->tokens)))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: a segment stride is smaller than one segment", i);
        // Codec.check (Sources/PITCH/Core/Codec.swift:42-46): the buffers must hold what the call reads
        if (pl.codes_bytes < (d->segments - 1) * pl.codes_seg_stride + d->tokens * pitch_code_stride(d->dim, pl.bits))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: codes buffer has %lld bytes; needs %lld", i, (long long)pl.codes_bytes,
                        (long long)((d->segments - 1) * pl.codes_seg_stride + d->tokens * pitch_code_stride(d->dim, pl.bits)));
        if (pl.side_bytes < (d->segments - 1) * pl.side_seg_stride + plane_side_bytes(pl, d->dim, d->tokens))
            return fail(PITCH_ERR_INVALID_INPUT, "plane %d: side-information buffer has %lld bytes; needs %lld", i,
                        (long long)pl.side_bytes, (long long)((d->segments - 1) * pl.side_seg_stride + plane_side_bytes(pl, d->dim, d->tokens)));
    }
    const pitch_buffer bufs[5] = {{const_cast<void*>(a->queries), 0, 0}, {a->out, 0, 0}, {a->workspace, 0, 0},
                                  {d->planes[0].codes, 0, 0}, {d->planes[1].codes, 0, 0}};
    const char* const names[5] = {"queries", "out", "workspace", "key codes", "value codes"};
    int dev;
    if ((st = check_same_device(bufs, names, 5, &dev))) return st;
    DeviceGuard guard(dev);

    AttentionParams p;
    memset(&p, 0, sizeof p);
    p.segments = (int)d->segments;
    p.tokens = (int)d->tokens;
    const bool fast = a->precision == PITCH_ATTENTION_BF16;
    const int warps = attn_warps(d->dim, d->planes[1].bits, fast);
    attention_slices(sm_count(), warps, d->segments, d->tokens, &p.splits, &p.tokens_per_split);
    if ((int64_t)p.segments * p.splits > 0x7FFFFFFF) return fail(PITCH_ERR_INVALID_INPUT, "segments x runs exceeds 2^31 - 1");
    p.n_queries = a->n_queries;
    const bool turbo_keys = d->planes[0].kind == PITCH_PLANE_TURBO;
    p.group_size = turbo_keys ? 32 : d->planes[0].group_size;
    for (int j = 0; j < 4; ++j) {
        p.kneg[j] = negate_mask32(d->planes[0].seed, 32u * j);
        p.neg[j] = negate_mask32(d->planes[1].seed, 32u * j);
    }
    p.rs = rsqrt_dim(d->dim);
    p.scale_log2 = (float)((double)a->scale * 1.4426950408889634);
    p.k_codes = static_cast<const unsigned char*>(d->planes[0].codes);
    p.k_codes_seg = d->planes[0].codes_seg_stride;
    p.k_ranges = static_cast<const unsigned char*>(d->planes[0].side);
    p.k_ranges_seg = d->planes[0].side_seg_stride;
    p.v_codes = static_cast<const unsigned char*>(d->planes[1].codes);
    p.v_codes_seg = d->planes[1].codes_seg_stride;
    p.v_norms = static_cast<const unsigned char*>(d->planes[1].side);
    p.v_norms_seg = d->planes[1].side_seg_stride;
    p.q = static_cast<const float*>(a->queries);
    p.work = static_cast<float*>(a->workspace);
    p.out = static_cast<float*>(a->out);
    const int vbits = d->planes[1].bits;
    if (!book_get(d->dim, vbits, p.book.c)) return fail(PITCH_ERR_INVALID_INPUT, "no TurboQuant codebook for dim %d, bits %d", d->dim, vbits);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    {
        const bool wide = d->dim == 128;
        // all the shared memory a block may have: the kernel's table must sit at a fixed shared-memory address
        const int smem = AT_SMEM_BYTES;
        static std::atomic<bool> configured[64];
        if (dev >= 0 && dev < 64 && !configured[dev].load(std::memory_order_acquire)) {
            int optin = 0;
            if (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess || optin != AT_SMEM_BYTES)
                return fail(PITCH_ERR_KERNEL_UNAVAILABLE, "cache attention needs a device with %d bytes of shared memory per block (this one: %d)", AT_SMEM_BYTES, optin);
            const cudaFuncAttribute at = cudaFuncAttributeMaxDynamicSharedMemorySize;
            if (cudaFuncSetAttribute(attention_partial_kernel<64, 4, false, false>, at, smem) != cudaSuccess ||
                cudaFuncSetAttribute(attention_partial_kernel<64, 4, true, false>, at, smem) != cudaSuccess ||
                cudaFuncSetAttribute(attention_partial_kernel<64, 4, false, true>, at, smem) != cudaSuccess ||
                cudaFuncSetAttribute(attention_partial_kernel<64, 4, true, true>, at, smem) != cudaSuccess ||
                cudaFuncSetAttribute(attention_partial_kernel<128, 4, false, true>, at, smem) != cudaSuccess ||
                cudaFuncSetAttribute(attention_partial_kernel<128, 4, true, true>, at, smem) != cudaSuccess ||
                cudaFuncSetAttribute(attention_partial_kernel<128, 3, false, true>, at, smem) != cudaSuccess ||
                cudaFuncSetAttribute(attention_partial_kernel<128, 3, true, true>, at, smem) != cudaSuccess)
                return launch_status(false, "cache_attention (shared memory opt-in)");
            configured[dev].store(true, std::memory_order_release);
        }
        // one CTA per SM (attn_warps warps); a warp takes runs warp, warp + all warps, ...
        int64_t ctas = ceil_div((int64_t)p.segments * p.splits, warps);
        if (ctas > sm_count()) ctas = sm_count();
        // Both launches are programmatic dependent launches: each grid may be scheduled while the
        // kernel before it in the stream is still running, sets itself up, then waits for that
        // kernel to complete before it reads what it wrote.
        cudaLaunchAttribute pdl[1];
        pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        pdl[0].val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)ctas);
        cfg.blockDim = dim3(32 * warps);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cfg.attrs = pdl;
        cfg.numAttrs = 1;
        if (wide && vbits == 3) {
            if (fast) cudaLaunchKernelEx(&cfg, attention_partial_kernel<128, 3, true, true>, p);
            else cudaLaunchKernelEx(&cfg, attention_partial_kernel<128, 3, false, true>, p);
        } else if (wide) {
            if (fast) cudaLaunchKernelEx(&cfg, attention_partial_kernel<128, 4, true, true>, p);
            else cudaLaunchKernelEx(&cfg, attention_partial_kernel<128, 4, false, true>, p);
        } else if (turbo_keys) {
            if (fast) cudaLaunchKernelEx(&cfg, attention_partial_kernel<64, 4, true, true>, p);
            else cudaLaunchKernelEx(&cfg, attention_partial_kernel<64, 4, false, true>, p);
        } else {
            if (fast) cudaLaunchKernelEx(&cfg, attention_partial_kernel<64, 4, true, false>, p);
            else cudaLaunchKernelEx(&cfg, attention_partial_kernel<64, 4, false, false>, p);
        }
        if ((st = launch_status(false, "cache_attention"))) return st;
        cfg.gridDim = dim3((unsigned)p.n_queries, (unsigned)p.segments);
        cfg.blockDim = dim3(32 * AT_COMBINE_WARPS);
        cfg.dynamicSmemBytes = 0;
        if (wide) cudaLaunchKernelEx(&cfg, attention_combine_kernel<128>, p);
        else cudaLaunchKernelEx(&cfg, attention_combine_kernel<64>, p);
    }
    return launch_status(false, "cache_attention (combine)");
}

}  // extern "C"
