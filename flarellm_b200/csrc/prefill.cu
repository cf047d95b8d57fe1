// Causal (and sliding-window) prefill attention on the 5th-generation tensor cores.
//
// Replaces the reference's O(S^2) loop of per-position decode calls
// (ComputeBackend::prefill_attention_gpu, flare-core/src/model.rs:336-368) and its WGSL shader
// (flare-gpu/shaders/prefill_attention.wgsl).  Row t attends rows max(0, t-W+1)..=t; query head
// h reads kv head h / (num_heads / num_kv_heads), the CPU mapping.
//
// This file holds the dispatch: operand conversion to bf16, the TMA tensor maps, the tensor-core kernel
// of prefill_pp.cu for head_dim 64 / 128, and for every other shape the general decode kernel run with
// one causally masked query per prompt row.
#include "common.cuh"
#include "tma.cuh"
#include "tc5.cuh"
#include <math_constants.h>

namespace {

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __bfloat162float(in[i]);
}

// f32 -> f16 for the tensor cores.  f16 keeps 11 significant bits (bf16: 8) but spans only 6e-5 .. 65504 at
// full precision, so each tensor is first scaled by a power of two (exact) that puts its largest magnitude in
// [2^14, 2^15); the attention kernel undoes the scaling in its softmax scale and its final normalisation.
__global__ void amax3_kernel(const float* __restrict__ q, size_t qn, const float* __restrict__ k,
                             const float* __restrict__ v, size_t kn, unsigned* __restrict__ amax_bits) {
    __shared__ unsigned s_red[3][8];
    float m[3] = {0.0f, 0.0f, 0.0f};
    const size_t stride = (size_t)gridDim.x * blockDim.x, i0 = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    for (size_t i = i0; i < qn; i += stride) m[0] = fmaxf(m[0], fabsf(q[i]));
    for (size_t i = i0; i < kn; i += stride) { m[1] = fmaxf(m[1], fabsf(k[i])); m[2] = fmaxf(m[2], fabsf(v[i])); }
#pragma unroll
    for (int t = 0; t < 3; t++) {
#pragma unroll
        for (int off = 16; off; off >>= 1) m[t] = fmaxf(m[t], __shfl_xor_sync(0xffffffffu, m[t], off));
        if ((threadIdx.x & 31) == 0) s_red[t][threadIdx.x >> 5] = __float_as_uint(m[t]);
    }
    __syncthreads();
    if (threadIdx.x < 3) {
        unsigned r = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) r = max(r, s_red[threadIdx.x][w]);   // non-negative floats order as integers
        atomicMax(amax_bits + threadIdx.x, r);
    }
}
__device__ __forceinline__ float f16_fit_scale(unsigned amax_bits) {
    const float a = __uint_as_float(amax_bits);
    if (!(a > 0.0f) || a > 3.0e38f) return 1.0f;           // all zero, or not finite: nothing sensible to fit
    int e;
    frexpf(a, &e);                                          // a = m 2^e, m in [0.5, 1)
    return ldexpf(1.0f, max(-40, min(40, 15 - e)));         // a * scale in [2^14, 2^15) unless a is extreme
}
__global__ void f32_to_f16_scaled_kernel(const float* __restrict__ q, size_t qn, const float* __restrict__ k,
                                         const float* __restrict__ v, size_t kn, __half* __restrict__ wq,
                                         __half* __restrict__ wk, __half* __restrict__ wv,
                                         const unsigned* __restrict__ amax_bits, float* __restrict__ descale) {
    const float sq = f16_fit_scale(amax_bits[0]), sk = f16_fit_scale(amax_bits[1]), sv = f16_fit_scale(amax_bits[2]);
    if (blockIdx.x == 0 && threadIdx.x == 0) { descale[0] = 1.0f / (sq * sk); descale[1] = 1.0f / sv; }
    const size_t stride = (size_t)gridDim.x * blockDim.x, i0 = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    for (size_t i = i0; i < qn; i += stride) wq[i] = __float2half_rn(q[i] * sq);
    for (size_t i = i0; i < kn; i += stride) { wk[i] = __float2half_rn(k[i] * sk); wv[i] = __float2half_rn(v[i] * sv); }
}

int make_qkv_map(CUtensorMap* m, const void* base, int hd, int heads, int S, int batch, bool f16) {
    const uint64_t dims[4] = {(uint64_t)hd, (uint64_t)heads, (uint64_t)S, (uint64_t)batch};
    const uint64_t strides[3] = {(uint64_t)hd * 2, (uint64_t)heads * hd * 2, (uint64_t)S * heads * hd * 2};
    const uint32_t box[4] = {64, 1, 128, 1};
    return flare_make_tensor_map(m, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                                 const_cast<void*>(base), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

// Any-shape path: the prompt's K/V viewed as an f32 cache, every row a causally ordered query of
// the general decode kernel (query i of S reads rows max(0, i-W+1) .. i).
static int prefill_generic(flare_attn_ctx* ctx, const PrefillArgs& a, const float* q, const float* k, const float* v, float* out) {
    DecodeArgs d;
    KvLayerView& kvw = d.kv;
    memset(&kvw, 0, sizeof(kvw));
    kvw.dtype = FLARE_KV_F32; kvw.batch = a.batch; kvw.max_seq_len = a.seq_len; kvw.num_kv_heads = a.num_kv_heads;
    kvw.head_dim = a.head_dim; kvw.kv_dim = a.num_kv_heads * a.head_dim;
    kvw.plane[FLARE_PLANE_K] = (const char*)k; kvw.plane[FLARE_PLANE_V] = (const char*)v;
    kvw.stride[FLARE_PLANE_K] = kvw.stride[FLARE_PLANE_V] = (size_t)a.seq_len * kvw.kv_dim * 4;
    // per-sequence attend length = S, ring state unused by the f32 loader
    std::vector<int> small((size_t)a.batch * 3, 0);
    for (int b = 0; b < a.batch; b++) small[2 * (size_t)a.batch + b] = a.seq_len;
    FLARE_TRY(flare_ensure(ctx, &ctx->d_misc2, &ctx->misc2_bytes, small.size() * 4));
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(ctx->d_misc2, small.data(), small.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));     // `small` is pageable and about to go out of scope
    d.ring = (const int2*)ctx->d_misc2;
    d.attend_len = (const int*)ctx->d_misc2 + 2 * (size_t)a.batch;
    d.q = q; d.out = out; d.batch = a.batch; d.n_q = a.seq_len; d.num_heads = a.num_heads;
    d.slot_begin = 0; d.slot_end = -1; d.want_partial = 0; d.causal_q = 1; d.max_attend = a.seq_len;
    d.layer = 0; d.kmap = d.vmap = nullptr; d.whole_rows = 0; d.window = a.window; d.kv_obj = nullptr; d.h_attend = nullptr;
    return flare_launch_decode_generic(ctx, d);
}

int flare_launch_prefill(flare_attn_ctx* ctx, const PrefillArgs& a) {
    const size_t qn = (size_t)a.batch * a.seq_len * a.num_heads * a.head_dim;
    const size_t kn = (size_t)a.batch * a.seq_len * a.num_kv_heads * a.head_dim;
    const bool tc = (a.head_dim == 64 || a.head_dim == 128) && flare_get_encode_tiled() != nullptr;
    const int conv_threads = 256, conv_grid = 148 * 8;
    if (!tc) {
        // general shapes: f32 in and out
        const float *q = (const float*)a.q, *k = (const float*)a.k, *v = (const float*)a.v;
        float* out = (float*)a.out;
        size_t need = 0;
        if (a.in_dtype == FLARE_DT_BF16) need += (qn + 2 * kn) * 4;
        if (a.out_dtype == FLARE_DT_BF16) need += qn * 4;
        if (need) {
            FLARE_TRY(flare_ensure(ctx, &ctx->d_conv, &ctx->conv_bytes, need + 1024));
            float* w = (float*)ctx->d_conv;
            if (a.in_dtype == FLARE_DT_BF16) {
                bf16_to_f32_kernel<<<conv_grid, conv_threads, 0, ctx->stream>>>((const __nv_bfloat16*)a.q, w, qn);
                bf16_to_f32_kernel<<<conv_grid, conv_threads, 0, ctx->stream>>>((const __nv_bfloat16*)a.k, w + qn, kn);
                bf16_to_f32_kernel<<<conv_grid, conv_threads, 0, ctx->stream>>>((const __nv_bfloat16*)a.v, w + qn + kn, kn);
                FLARE_LAUNCH_CHECK(ctx);
                q = w; k = w + qn; v = w + qn + kn; w += qn + 2 * kn;
            }
            if (a.out_dtype == FLARE_DT_BF16) out = w;
        }
        ctx->last_path = FLARE_PATH_GENERAL;
        FLARE_TRY(prefill_generic(ctx, a, q, k, v, out));
        if (a.out_dtype == FLARE_DT_BF16) {
            f32_to_bf16_kernel<<<conv_grid, conv_threads, 0, ctx->stream>>>(out, (__nv_bfloat16*)a.out, qn);
            FLARE_LAUNCH_CHECK(ctx);
        }
        return FLARE_OK;
    }
    // tensor-core path: bf16 operands as given, f32 inputs as f16 operands (the trait hook's contract is the f32 CPU
    // loop within 2e-3 + 1e-3 |x|: a row that attends one key returns that key's value row, and bf16 would round it
    // by up to 2^-8 relative)
    const void *q = a.q, *k = a.k, *v = a.v;
    PrefillArgs a2 = a;
    if (a.in_dtype == FLARE_DT_F32) {
        const size_t halves = ((qn + 2 * kn) * 2 + 255) / 256 * 256;
        FLARE_TRY(flare_ensure(ctx, &ctx->d_conv, &ctx->conv_bytes, halves + 256));
        __half* w = (__half*)ctx->d_conv;
        unsigned* amax = (unsigned*)((char*)ctx->d_conv + halves);
        float* descale = (float*)(amax + 4);
        FLARE_CUDA_OK(ctx, cudaMemsetAsync(amax, 0, 16, ctx->stream));
        amax3_kernel<<<conv_grid, conv_threads, 0, ctx->stream>>>((const float*)a.q, qn, (const float*)a.k, (const float*)a.v, kn, amax);
        FLARE_LAUNCH_CHECK(ctx);
        f32_to_f16_scaled_kernel<<<conv_grid, conv_threads, 0, ctx->stream>>>((const float*)a.q, qn, (const float*)a.k,
                                                                              (const float*)a.v, kn, w, w + qn, w + qn + kn,
                                                                              amax, descale);
        FLARE_LAUNCH_CHECK(ctx);
        q = w; k = w + qn; v = w + qn + kn;
        a2.f16_ops = 1; a2.descale = descale;
    }
    CUtensorMap qm, km, vm;
    const bool f16 = a2.f16_ops != 0;
    if (make_qkv_map(&qm, q, a.head_dim, a.num_heads, a.seq_len, a.batch, f16) ||
        make_qkv_map(&km, k, a.head_dim, a.num_kv_heads, a.seq_len, a.batch, f16) ||
        make_qkv_map(&vm, v, a.head_dim, a.num_kv_heads, a.seq_len, a.batch, f16))
        return flare_set_error(ctx, FLARE_ERR_CUDA, "cuTensorMapEncodeTiled failed for the prefill operands (are they 16-byte aligned?)");
    a2.q = q; a2.k = k; a2.v = v;
    ctx->last_path = FLARE_PATH_PREFILL_TENSOR;
    return flare_launch_prefill_pp(ctx, qm, km, vm, a2);
}
