// The whole single-token forward pass on the device: what WebGpuBackend::forward_single_token_gpu
// (flare-gpu/src/backend.rs:4010-4375, called from flare-core/src/model.rs:1697-1734) keeps resident — weights, KV
// cache, every intermediate — so that one token costs one upload of its embedding row and one download of its logits.
//
// The arithmetic follows the CPU's Q8_0 path (Model::forward_layers, flare-core/src/model.rs:2010-2548, the
// branch with use_q8_attn / use_q8_ffn / use_q8_output), because that is the path whose numbers a host can check:
//   x            = token embedding row
//   per layer:     normed_q8 = rmsnorm_quantize_q8_0(x, attn_norm)            model.rs:5610-5641
//                  qkv       = matvec_q8_0_preq(fused [wq; wk; wv], normed_q8)   model.rs:2018-2040, 8066-8100
//                  q, k      = apply_rope_with_table(.., pos)                  model.rs:2165-2180, 7256-7292
//                  cache    <- k, v at the ring position;  attn = GQA over min(len + 1, max_seq) slots
//                  x        += matvec_q8_0_preq(wo, quantize_input_q8_0(attn))     model.rs:2276-2287, 2307-2311
//                  gate_up   = matvec_q8_0_preq(fused [w_gate; w_up], rmsnorm_quantize_q8_0(x, ffn_norm))
//                  hidden    = silu(gate) * up = (g / (1 + exp(-g))) * up       model.rs:7091-7099
//                  x        += matvec_q8_0_preq(w_down, quantize_input_q8_0(hidden))
//   logits       = matvec_q8_0_preq(output, quantize_input_q8_0(rmsnorm(x, output_norm)))   model.rs:1759-1770
//                  or the f32 product when the output matrix is kept in f32     model.rs:1771-1779
// The integer dots, the block sums of a row, the rotation and the quantisation steps are the reference's operation
// for operation.  Two things are not: the sum of squares of a norm is a tree over the block's threads where the
// CPU adds left to right, and exp() is the device's expf; so a forward pass agrees with the CPU within a
// tolerance, not bit for bit.  Biases (Qwen2), post-norms and soft-caps (Gemma 2), MoE and LoRA are not handled.
#include "common.cuh"
#include "q8_input.cuh"

#include <vector>

struct flare_model {
    flare_attn_ctx* ctx = nullptr;
    flare_model_config cfg = {};
    struct Layer {
        float* attn_norm = nullptr;
        float* ffn_norm = nullptr;
        flare_weight *qkv = nullptr, *wo = nullptr, *gate_up = nullptr, *down = nullptr;
    };
    std::vector<Layer> layers;
    float* output_norm = nullptr;
    flare_weight* output_q8 = nullptr;
    float* output_f32 = nullptr;
    // activations for `buf_batch` sequences
    int buf_batch = 0;
    float *x = nullptr, *qkv = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *proj = nullptr,
          *gate_up = nullptr, *normed = nullptr, *logits = nullptr, *xs = nullptr;
    int8_t* xq = nullptr;
    long long* pos = nullptr;        // the token's absolute positions, uploaded once per call
};

namespace {

// rmsnorm_quantize_q8_0: one block per input vector
__global__ void __launch_bounds__(256) rmsnorm_quantize_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                                float eps, int dim, int8_t* __restrict__ xq,
                                                                float* __restrict__ xs) {
    flare_pdl_wait();
    flare_pdl_trigger();
    __shared__ float s_red[32];
    flare_quantize_vector(x + (size_t)blockIdx.x * dim, weight, eps, dim, xq + (size_t)blockIdx.x * dim,
                          xs + (size_t)blockIdx.x * (dim / 32), s_red);
}

__device__ __forceinline__ float block_sum_sq(const float* __restrict__ x, int dim, float* s_red) {
    float s = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) s = fmaf(x[i], x[i], s);
    return flare_block_sum(s, s_red);
}

// rmsnorm_into: out = (x * inv_rms) * weight
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ weight, float eps,
                                                      int dim, float* __restrict__ out) {
    flare_pdl_wait();
    flare_pdl_trigger();
    __shared__ float s_red[32];
    const float* row = x + (size_t)blockIdx.x * dim;
    const float sum_sq = block_sum_sq(row, dim, s_red);
    const float rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_sq, (float)dim), eps));
    const float inv_rms = __fdiv_rn(1.0f, rms);
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        out[(size_t)blockIdx.x * dim + i] = __fmul_rn(__fmul_rn(row[i], inv_rms), weight[i]);
}

// rows of [q | k | v] -> three dense buffers
__global__ void split_qkv_kernel(const float* __restrict__ qkv, int q_dim, int kv_dim, float* __restrict__ q,
                                 float* __restrict__ k, float* __restrict__ v) {
    flare_pdl_wait();
    flare_pdl_trigger();
    const int b = blockIdx.y, total = q_dim + 2 * kv_dim;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const float val = qkv[(size_t)b * total + i];
        if (i < q_dim) q[(size_t)b * q_dim + i] = val;
        else if (i < q_dim + kv_dim) k[(size_t)b * kv_dim + (i - q_dim)] = val;
        else v[(size_t)b * kv_dim + (i - q_dim - kv_dim)] = val;
    }
}

// hidden = silu(gate) * up out of rows of [gate | up], quantised per 32 as quantize_input_q8_0 does: a warp per block
__global__ void silu_mul_quantize_kernel(const float* __restrict__ gate_up, int inter, size_t n_blocks,
                                         int8_t* __restrict__ xq, float* __restrict__ xs) {
    flare_pdl_wait();
    flare_pdl_trigger();
    const int lane = threadIdx.x & 31, nb = inter / 32;
    for (size_t w = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5; w < n_blocks; w += ((size_t)gridDim.x * blockDim.x) >> 5) {
        const size_t b = w / nb, blk = w % nb;
        const float g = gate_up[b * 2 * inter + blk * 32 + lane];
        const float u = gate_up[b * 2 * inter + inter + blk * 32 + lane];
        const float h = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
        float amax = fabsf(h);
#pragma unroll
        for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = d != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
        xq[w * 32 + lane] = flare_to_i8_saturating(roundf(__fmul_rn(h, id)));
        if (lane == 0) xs[w] = d;
    }
}

// f32 output matrix: a warp per row, the input vectors of the batch one after the other
__global__ void __launch_bounds__(256) matvec_f32_kernel(const float* __restrict__ w, const float* __restrict__ x, int rows,
                                                         int cols, int batch, float* __restrict__ out) {
    flare_pdl_wait();
    flare_pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float4* wr = reinterpret_cast<const float4*>(w + (size_t)row * cols);
    for (int b = 0; b < batch; b++) {
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)b * cols);
        float s = 0.0f;
        for (int i = lane; i < cols / 4; i += 32) {
            const float4 a = __ldg(wr + i), c = __ldg(xr + i);
            s = fmaf(a.x, c.x, s); s = fmaf(a.y, c.y, s); s = fmaf(a.z, c.z, s); s = fmaf(a.w, c.w, s);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) out[(size_t)b * rows + row] = s;
    }
}

int upload_f32(flare_attn_ctx* ctx, const float* host, size_t n, float** dev) {
    cudaFree(*dev); *dev = nullptr;
    FLARE_CUDA_OK(ctx, cudaMalloc((void**)dev, n * sizeof(float)));
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(*dev, host, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return FLARE_OK;
}

int replace_weight(flare_attn_ctx* ctx, const void* blocks, int rows, int cols, flare_weight** slot) {
    if (*slot) { flare_weight_free(*slot); *slot = nullptr; }
    return flare_weight_upload_q8_0(ctx, blocks, rows, cols, slot);
}

void free_buffers(flare_model* m) {
    float** bufs[] = {&m->x, &m->qkv, &m->q, &m->k, &m->v, &m->attn, &m->proj, &m->gate_up, &m->normed, &m->logits, &m->xs};
    for (float** b : bufs) { cudaFree(*b); *b = nullptr; }
    cudaFree(m->xq); m->xq = nullptr;
    cudaFree(m->pos); m->pos = nullptr;
    m->buf_batch = 0;
}

int ensure_buffers(flare_model* m, int batch) {
    if (batch <= m->buf_batch) return FLARE_OK;
    flare_attn_ctx* ctx = m->ctx;
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    free_buffers(m);
    const flare_model_config& c = m->cfg;
    const size_t B = (size_t)batch, q_dim = (size_t)c.num_heads * c.head_dim, kv_dim = (size_t)c.num_kv_heads * c.head_dim;
    const size_t widest = (size_t)(c.intermediate_dim > c.hidden_dim ? c.intermediate_dim : c.hidden_dim) > q_dim
                              ? (size_t)(c.intermediate_dim > c.hidden_dim ? c.intermediate_dim : c.hidden_dim) : q_dim;
    struct { float** p; size_t n; } want[] = {
        {&m->x, B * c.hidden_dim}, {&m->qkv, B * (q_dim + 2 * kv_dim)}, {&m->q, B * q_dim}, {&m->k, B * kv_dim},
        {&m->v, B * kv_dim}, {&m->attn, B * q_dim}, {&m->proj, B * c.hidden_dim}, {&m->gate_up, B * 2 * c.intermediate_dim},
        {&m->normed, B * c.hidden_dim}, {&m->logits, B * c.vocab_size}, {&m->xs, B * widest / 32 + 8}};
    for (auto& w : want)
        if (cudaMalloc((void**)w.p, w.n * sizeof(float)) != cudaSuccess) { cudaGetLastError(); free_buffers(m); return flare_set_error(ctx, FLARE_ERR_OOM, "forward buffers for %d sequences", batch); }
    if (cudaMalloc((void**)&m->xq, B * widest) != cudaSuccess || cudaMalloc((void**)&m->pos, B * sizeof(long long)) != cudaSuccess) { cudaGetLastError(); free_buffers(m); return flare_set_error(ctx, FLARE_ERR_OOM, "forward buffers for %d sequences", batch); }
    m->buf_batch = batch;
    return FLARE_OK;
}

int grid_for(size_t threads_wanted) {
    size_t g = (threads_wanted + 255) / 256;
    if (g > 148 * 8) g = 148 * 8;
    return g < 1 ? 1 : (int)g;
}

}  // namespace

extern "C" {

int flare_model_create(flare_attn_ctx* ctx, const flare_model_config* cfg, flare_model** out_model) {
    if (!ctx) return FLARE_ERR_INVALID_ARG;
    if (!cfg || !out_model) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_model_create: null argument");
    *out_model = nullptr;
    const flare_model_config& c = *cfg;
    if (c.hidden_dim < 32 || c.hidden_dim % 32 || c.intermediate_dim < 32 || c.intermediate_dim % 32 || c.num_heads < 1 ||
        c.num_kv_heads < 1 || c.num_heads % c.num_kv_heads || c.head_dim < 2 || c.head_dim % 2 ||
        (c.num_heads * c.head_dim) % 32 || c.vocab_size < 1 || c.num_layers < 1 || !(c.rms_norm_eps >= 0.0f))
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_model_create: hidden %d, intermediate %d (multiples of 32), heads %d / %d x %d, "
                               "vocabulary %d, layers %d", c.hidden_dim, c.intermediate_dim, c.num_heads, c.num_kv_heads, c.head_dim,
                               c.vocab_size, c.num_layers);
    flare_model* m = new (std::nothrow) flare_model();
    if (!m) return FLARE_ERR_OOM;
    m->ctx = ctx; m->cfg = c;
    m->layers.resize(c.num_layers);
    *out_model = m;
    return FLARE_OK;
}

int flare_model_set_layer(flare_model* m, int layer, const float* attn_norm, const void* qkv_q8_0, const void* wo_q8_0,
                          const float* ffn_norm, const void* gate_up_q8_0, const void* down_q8_0) {
    if (!m) return FLARE_ERR_INVALID_ARG;
    flare_attn_ctx* ctx = m->ctx;
    if (layer < 0 || layer >= m->cfg.num_layers || !attn_norm || !qkv_q8_0 || !wo_q8_0 || !ffn_norm || !gate_up_q8_0 || !down_q8_0)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_model_set_layer: layer %d or a null matrix", layer);
    FLARE_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const flare_model_config& c = m->cfg;
    const int q_dim = c.num_heads * c.head_dim, kv_dim = c.num_kv_heads * c.head_dim;
    flare_model::Layer& L = m->layers[layer];
    FLARE_TRY(upload_f32(ctx, attn_norm, c.hidden_dim, &L.attn_norm));
    FLARE_TRY(upload_f32(ctx, ffn_norm, c.hidden_dim, &L.ffn_norm));
    FLARE_TRY(replace_weight(ctx, qkv_q8_0, q_dim + 2 * kv_dim, c.hidden_dim, &L.qkv));
    FLARE_TRY(replace_weight(ctx, wo_q8_0, c.hidden_dim, q_dim, &L.wo));
    FLARE_TRY(replace_weight(ctx, gate_up_q8_0, 2 * c.intermediate_dim, c.hidden_dim, &L.gate_up));
    FLARE_TRY(replace_weight(ctx, down_q8_0, c.hidden_dim, c.intermediate_dim, &L.down));
    return FLARE_OK;
}

int flare_model_set_output(flare_model* m, const float* output_norm, const void* output_q8_0, const float* output_f32) {
    if (!m) return FLARE_ERR_INVALID_ARG;
    flare_attn_ctx* ctx = m->ctx;
    if (!output_norm || (!output_q8_0) == (!output_f32))
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_model_set_output: the norm and exactly one of the two matrices");
    FLARE_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const flare_model_config& c = m->cfg;
    FLARE_TRY(upload_f32(ctx, output_norm, c.hidden_dim, &m->output_norm));
    if (m->output_q8) { flare_weight_free(m->output_q8); m->output_q8 = nullptr; }
    cudaFree(m->output_f32); m->output_f32 = nullptr;
    if (output_q8_0) return flare_weight_upload_q8_0(ctx, output_q8_0, c.vocab_size, c.hidden_dim, &m->output_q8);
    return upload_f32(ctx, output_f32, (size_t)c.vocab_size * c.hidden_dim, &m->output_f32);
}

int flare_model_free(flare_model* m) {
    if (!m) return FLARE_OK;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    for (auto& L : m->layers) {
        cudaFree(L.attn_norm); cudaFree(L.ffn_norm);
        flare_weight_free(L.qkv); flare_weight_free(L.wo); flare_weight_free(L.gate_up); flare_weight_free(L.down);
    }
    cudaFree(m->output_norm); cudaFree(m->output_f32);
    flare_weight_free(m->output_q8);
    free_buffers(m);
    delete m;
    return FLARE_OK;
}

int flare_forward_token(flare_attn_ctx* ctx, flare_model* m, flare_kv* kv, const float* token_embed, const int64_t* positions,
                        float* logits) {
    if (!ctx) return FLARE_ERR_INVALID_ARG;
    if (!m || m->ctx != ctx || !kv) return flare_set_error(ctx, FLARE_ERR_STATE, "the model or the cache does not belong to this context");
    if (!token_embed || !positions || !logits) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_forward_token: null buffer");
    const flare_model_config& c = m->cfg;
    if (kv->num_layers != c.num_layers || kv->num_kv_heads != c.num_kv_heads || kv->head_dim != c.head_dim)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "the cache (%d layers, %d kv heads x %d) does not fit the model (%d, %d x %d)",
                               kv->num_layers, kv->num_kv_heads, kv->head_dim, c.num_layers, c.num_kv_heads, c.head_dim);
    if (!m->output_norm) return flare_set_error(ctx, FLARE_ERR_STATE, "flare_model_set_output has not been called");
    for (auto& L : m->layers)
        if (!L.qkv) return flare_set_error(ctx, FLARE_ERR_STATE, "a layer has no weights yet");
    FLARE_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const int B = kv->batch;
    if (B > 256) return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "flare_forward_token: %d sequences (at most 256)", B);
    FLARE_TRY(ensure_buffers(m, B));
    const int dim = c.hidden_dim, inter = c.intermediate_dim, q_dim = c.num_heads * c.head_dim, kv_dim = c.num_kv_heads * c.head_dim;
    cudaStream_t st = ctx->stream;
    // 256 threads, like a CTA of the matrix-vector kernel: the fused and the standalone norm add in the same order
    const int norm_threads = dim >= 256 ? 256 : 32 * (dim / 32);
    if (!kv->rope_cos) return flare_set_error(ctx, FLARE_ERR_STATE, "no rotary table: call flare_kv_set_rope_table first");
    for (int b = 0; b < B; b++)
        if (positions[b] < 0 || positions[b] >= kv->rope_len)
            return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "positions[%d] = %lld is outside the rotary table of %d rows", b,
                                   (long long)positions[b], kv->rope_len);
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(m->x, token_embed, (size_t)B * dim * sizeof(float), cudaMemcpyHostToDevice, st));
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(m->pos, positions, (size_t)B * sizeof(long long), cudaMemcpyHostToDevice, st));
    ctx->last_launch_overlappable = false;
    // a single sequence needs no copy to take [q | k | v] apart
    float* q = B == 1 ? m->qkv : m->q;
    float* k = B == 1 ? m->qkv + q_dim : m->k;
    float* v = B == 1 ? m->qkv + q_dim + kv_dim : m->v;
    for (int layer = 0; layer < c.num_layers; layer++) {
        const flare_model::Layer& L = m->layers[layer];
        // attention block
        FLARE_CUDA_OK(ctx, flare_launch_pdl(rmsnorm_quantize_kernel, dim3(B), dim3(norm_threads), 0, st, m->x, L.attn_norm, c.rms_norm_eps, dim, m->xq, m->xs));
        FLARE_LAUNCH_CHECK(ctx);
        FLARE_TRY(flare_launch_matvec_q8_0_preq(ctx, L.qkv, m->xq, m->xs, B, m->qkv, 0));
        if (B > 1) {
            FLARE_CUDA_OK(ctx, flare_launch_pdl(split_qkv_kernel, dim3(grid_for((size_t)q_dim + 2 * kv_dim), B), dim3(256), 0, st, m->qkv, q_dim, kv_dim, m->q, m->k, m->v));
            FLARE_LAUNCH_CHECK(ctx);
        }
        FLARE_TRY(flare_kv_write_step_rope_device(kv, layer, k, v, m->pos, q, c.num_heads));     // rotates q as well
        FLARE_TRY(flare_decode_attn(ctx, kv, layer, c.num_heads, q, 1, nullptr, 0.0f, m->attn, 1));
        FLARE_TRY(flare_launch_quantize_input(ctx, m->attn, (size_t)B * q_dim / 32, m->xq, m->xs));
        FLARE_TRY(flare_launch_matvec_q8_0_preq(ctx, L.wo, m->xq, m->xs, B, m->x, 1));
        // feed-forward block
        FLARE_CUDA_OK(ctx, flare_launch_pdl(rmsnorm_quantize_kernel, dim3(B), dim3(norm_threads), 0, st, m->x, L.ffn_norm, c.rms_norm_eps, dim, m->xq, m->xs));
        FLARE_LAUNCH_CHECK(ctx);
        FLARE_TRY(flare_launch_matvec_q8_0_preq(ctx, L.gate_up, m->xq, m->xs, B, m->gate_up, 0));
        FLARE_CUDA_OK(ctx, flare_launch_pdl(silu_mul_quantize_kernel, dim3(grid_for((size_t)B * inter)), dim3(256), 0, st, m->gate_up, inter, (size_t)B * inter / 32, m->xq, m->xs));
        FLARE_LAUNCH_CHECK(ctx);
        FLARE_TRY(flare_launch_matvec_q8_0_preq(ctx, L.down, m->xq, m->xs, B, m->x, 1));
        ctx->last_launch_overlappable = false;
    }
    FLARE_CUDA_OK(ctx, flare_launch_pdl(rmsnorm_kernel, dim3(B), dim3(norm_threads), 0, st, m->x, m->output_norm, c.rms_norm_eps, dim, m->normed));
    FLARE_LAUNCH_CHECK(ctx);
    if (m->output_q8) {
        FLARE_TRY(flare_launch_quantize_input(ctx, m->normed, (size_t)B * dim / 32, m->xq, m->xs));
        FLARE_TRY(flare_launch_matvec_q8_0_preq(ctx, m->output_q8, m->xq, m->xs, B, m->logits, 0));
    } else {
        FLARE_CUDA_OK(ctx, flare_launch_pdl(matvec_f32_kernel, dim3((c.vocab_size + 7) / 8), dim3(256), 0, st, m->output_f32, m->normed, c.vocab_size, dim, B, m->logits));
        FLARE_LAUNCH_CHECK(ctx);
    }
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(logits, m->logits, (size_t)B * c.vocab_size * sizeof(float), cudaMemcpyDeviceToHost, st));
    FLARE_TRY(flare_check_device_error(ctx));      // waits for the stream
    return flare_kv_advance(kv, -1, 1);            // Model::forward advances the cache once per token (model.rs:2543)
}

}  // extern "C"
