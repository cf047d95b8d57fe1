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

int make_qkv_map(CUtensorMap* m, const void* base, int hd, int heads, int S, int batch) {
    const uint64_t dims[4] = {(uint64_t)hd, (uint64_t)heads, (uint64_t)S, (uint64_t)batch};
    const uint64_t strides[3] = {(uint64_t)hd * 2, (uint64_t)heads * hd * 2, (uint64_t)S * heads * hd * 2};
    const uint32_t box[4] = {64, 1, 128, 1};
    return flare_make_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
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
        FLARE_TRY(prefill_generic(ctx, a, q, k, v, out));
        if (a.out_dtype == FLARE_DT_BF16) {
            f32_to_bf16_kernel<<<conv_grid, conv_threads, 0, ctx->stream>>>(out, (__nv_bfloat16*)a.out, qn);
            FLARE_LAUNCH_CHECK(ctx);
        }
        return FLARE_OK;
    }
    // tensor-core path: bf16 operands
    const void *q = a.q, *k = a.k, *v = a.v;
    if (a.in_dtype == FLARE_DT_F32) {
        FLARE_TRY(flare_ensure(ctx, &ctx->d_conv, &ctx->conv_bytes, (qn + 2 * kn) * 2 + 1024));
        __nv_bfloat16* w = (__nv_bfloat16*)ctx->d_conv;
        f32_to_bf16_kernel<<<conv_grid, conv_threads, 0, ctx->stream>>>((const float*)a.q, w, qn);
        f32_to_bf16_kernel<<<conv_grid, conv_threads, 0, ctx->stream>>>((const float*)a.k, w + qn, kn);
        f32_to_bf16_kernel<<<conv_grid, conv_threads, 0, ctx->stream>>>((const float*)a.v, w + qn + kn, kn);
        FLARE_LAUNCH_CHECK(ctx);
        q = w; k = w + qn; v = w + qn + kn;
    }
    CUtensorMap qm, km, vm;
    if (make_qkv_map(&qm, q, a.head_dim, a.num_heads, a.seq_len, a.batch) || make_qkv_map(&km, k, a.head_dim, a.num_kv_heads, a.seq_len, a.batch) ||
        make_qkv_map(&vm, v, a.head_dim, a.num_kv_heads, a.seq_len, a.batch))
        return flare_set_error(ctx, FLARE_ERR_CUDA, "cuTensorMapEncodeTiled failed for the prefill operands (are they 16-byte aligned?)");
    {
        PrefillArgs a2 = a;
        a2.q = q; a2.k = k; a2.v = v;
        return flare_launch_prefill_pp(ctx, qm, km, vm, a2);
    }
}
