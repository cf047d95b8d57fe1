// Q8_0-weight matrix-vector products next to attention: the QKV projections before it and the output projection
// after it (flare-core/src/model.rs:2016-2136, 2249-2291), for `batch` input vectors at once.
//
// The arithmetic is the reference's, operation for operation, so that the result is the CPU's bit for bit
// (flare-core/src/model.rs, the branch compiled on x86_64):
//   quantize_input_q8_0 (5507-5527)     per 32 inputs: amax, d = amax / 127, id = 127 / amax (0 when d == 0),
//                                       q = round(x * id) as i8; the block scale d stays f32
//   matvec_q8_0_preq_into (8066-8100)   per row, blocks in ascending order:
//                                       sum += (w_scale * x_scale[block]) * (int32 dot of the 32 int8 pairs) as f32
//                                       with w_scale the block's f16 scale widened exactly; separate multiplies and add
// The integer dot is exact in any order (dp4a); the f32 sum over a row's blocks is the only order-sensitive part and
// is kept sequential: the lanes of a warp each own one input vector of the batch for that sum, so 32 sums run side
// by side.  A weight row is read from HBM once for the whole batch.
#include "common.cuh"
#include <mutex>

struct flare_weight {
    flare_attn_ctx* ctx = nullptr;
    int rows = 0, cols = 0;
    unsigned char* blocks = nullptr;     // [rows][cols / 32] x 34 bytes: f16 LE scale, 32 x i8 (GGUF Q8_0)
};

namespace {

constexpr int CHUNK = 64;            // blocks of a row handled per pass: two per lane
constexpr int WARPS = 8;
constexpr int TS = CHUNK + 1;        // floats per input vector in the product buffer
constexpr int WARP_SMEM = CHUNK * 34 + 32 * TS * 4;      // 2176 + 8320 bytes, a multiple of 16

// quantize_input_q8_0: one warp per 32-value block, lane = element
__global__ void quantize_input_kernel(const float* __restrict__ x, size_t n_blocks, int8_t* __restrict__ xq,
                                      float* __restrict__ xs) {
    const int lane = threadIdx.x & 31;
    for (size_t w = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5; w < n_blocks; w += ((size_t)gridDim.x * blockDim.x) >> 5) {
        const float v = x[w * 32 + lane];
        float amax = fabsf(v);
#pragma unroll
        for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = (d != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
        const float r = roundf(__fmul_rn(v, id));
        const int qi = (r != r) ? 0 : (r >= 127.0f ? 127 : (r <= -128.0f ? -128 : (int)r));    // Rust `as i8` saturates
        xq[w * 32 + lane] = (int8_t)qi;
        if (lane == 0) xs[w] = d;
    }
}

struct MatvecParams {
    const unsigned char* w;      // weight blocks
    const int8_t* xq;            // [batch][cols]
    const float* xs;             // [batch][cols / 32]
    float* out;                  // [batch][rows]
    int rows, cols, batch;
};

__global__ void __launch_bounds__(32 * WARPS) matvec_q8_0_kernel(MatvecParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * WARPS + warp;
    if (row >= p.rows) return;
    const int nb = p.cols / 32;
    // per warp: the current chunk of the weight row (CHUNK x 34 = 2176 bytes) and the products
    // [input vector of the batch tile][block of the chunk], rows padded by one float against bank conflicts
    unsigned char* wrow = smem + (size_t)warp * WARP_SMEM;
    float* terms = reinterpret_cast<float*>(wrow + CHUNK * 34);
    const unsigned char* src = p.w + (size_t)row * nb * 34;
    const int n_tiles = (p.batch + 31) / 32;
    float sum[8];                                     // running sums of this lane's input vector in each batch tile (batch <= 256)
#pragma unroll
    for (int t = 0; t < 8; t++) sum[t] = 0.0f;
    for (int c0 = 0; c0 < nb; c0 += CHUNK) {
        const int cn = min(CHUNK, nb - c0);
        __syncwarp();
        // the chunk's bytes, as 16-bit units (a row of 34-byte blocks starts on a 2-byte boundary)
        const uint16_t* s16 = reinterpret_cast<const uint16_t*>(src + (size_t)c0 * 34);
        uint16_t* d16 = reinterpret_cast<uint16_t*>(wrow);
        for (int i = lane; i < cn * 17; i += 32) d16[i] = __ldg(s16 + i);
        __syncwarp();
        // this lane's (up to) two blocks of the chunk: scale and the 32 weights as eight 32-bit words
        float wsc[2];
        int wq[2][8];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int blk = lane + 32 * k;
            if (blk < cn) {
                const uint16_t* b16 = d16 + blk * 17;
                wsc[k] = __half2float(__ushort_as_half(b16[0]));
#pragma unroll
                for (int j = 0; j < 8; j++) wq[k][j] = (int)b16[1 + 2 * j] | ((int)b16[2 + 2 * j] << 16);
            } else {
                wsc[k] = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; j++) wq[k][j] = 0;
            }
        }
#pragma unroll 1
        for (int t = 0; t < n_tiles; t++) {
            const int bn = min(32, p.batch - 32 * t);
            // products of this lane's blocks with every input vector of the tile
            for (int b = 0; b < bn; b++) {
                const size_t vec = (size_t)(32 * t + b);
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const int blk = lane + 32 * k;
                    if (blk < cn) {
                        const int4* xp = reinterpret_cast<const int4*>(p.xq + vec * p.cols + (size_t)(c0 + blk) * 32);
                        const int4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
                        int acc = 0;
                        acc = __dp4a(wq[k][0], x0.x, acc); acc = __dp4a(wq[k][1], x0.y, acc);
                        acc = __dp4a(wq[k][2], x0.z, acc); acc = __dp4a(wq[k][3], x0.w, acc);
                        acc = __dp4a(wq[k][4], x1.x, acc); acc = __dp4a(wq[k][5], x1.y, acc);
                        acc = __dp4a(wq[k][6], x1.z, acc); acc = __dp4a(wq[k][7], x1.w, acc);
                        const float cs = __fmul_rn(wsc[k], __ldg(p.xs + vec * nb + c0 + blk));
                        terms[b * TS + blk] = __fmul_rn(cs, (float)acc);
                    }
                }
            }
            __syncwarp();
            // lane b adds the chunk's products of input vector b in block order
            if (lane < bn) {
                float s = sum[t];
                for (int blk = 0; blk < cn; blk++) s = __fadd_rn(s, terms[lane * TS + blk]);
                sum[t] = s;
            }
            __syncwarp();
        }
    }
#pragma unroll
    for (int t = 0; t < 8; t++)
        if (t < n_tiles && 32 * t + lane < p.batch) p.out[(size_t)(32 * t + lane) * p.rows + row] = sum[t];
}

}  // namespace

extern "C" {

int flare_weight_upload_q8_0(flare_attn_ctx* ctx, const void* blocks, int rows, int cols, flare_weight** out_w) {
    if (!ctx) return FLARE_ERR_INVALID_ARG;
    if (!out_w) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "out_w is null");
    *out_w = nullptr;
    if (!blocks || rows < 1 || cols < 32 || cols % 32)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_weight_upload_q8_0: %d x %d (cols must be a positive multiple of 32)", rows, cols);
    FLARE_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    flare_weight* w = new (std::nothrow) flare_weight();
    if (!w) return FLARE_ERR_OOM;
    w->ctx = ctx; w->rows = rows; w->cols = cols;
    const size_t bytes = (size_t)rows * (cols / 32) * 34;
    cudaError_t e = cudaMalloc(&w->blocks, bytes + 64);
    if (e == cudaSuccess) e = cudaMemcpyAsync(w->blocks, blocks, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        const int code = e == cudaErrorMemoryAllocation ? FLARE_ERR_OOM : FLARE_ERR_CUDA;
        flare_set_error(ctx, code, "flare_weight_upload_q8_0: %zu bytes: %s", bytes, cudaGetErrorString(e));
        cudaGetLastError();
        cudaFree(w->blocks);
        delete w;
        return code;
    }
    *out_w = w;
    return FLARE_OK;
}

int flare_weight_free(flare_weight* w) {
    if (!w) return FLARE_OK;
    cudaSetDevice(w->ctx->device);
    cudaStreamSynchronize(w->ctx->stream);
    cudaFree(w->blocks);
    delete w;
    return FLARE_OK;
}

int flare_matvec_q8_0(flare_attn_ctx* ctx, const flare_weight* w, const float* x, int batch, float* out, int on_device) {
    if (!ctx) return FLARE_ERR_INVALID_ARG;
    if (!w || w->ctx != ctx) return flare_set_error(ctx, FLARE_ERR_STATE, "the weight matrix does not belong to this context");
    if (!x || !out || batch < 1 || batch > 256)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_matvec_q8_0: null buffer or batch %d outside [1, 256]", batch);
    FLARE_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const size_t xn = (size_t)batch * w->cols, on = (size_t)batch * w->rows, nblk = xn / 32;
    // scratch: quantised inputs and their scales (and, with host buffers, x and out themselves)
    const size_t q_off = 0, s_off = (xn + 255) / 256 * 256, x_off = s_off + (nblk * 4 + 255) / 256 * 256;
    const size_t o_off = x_off + (on_device ? 0 : (xn * 4 + 255) / 256 * 256);
    const size_t need = o_off + (on_device ? 0 : on * 4);
    FLARE_TRY(flare_ensure(ctx, &ctx->d_conv, &ctx->conv_bytes, need + 256));
    char* d = (char*)ctx->d_conv;
    const float* dx = x;
    float* dout = out;
    if (!on_device) {
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d + x_off, x, xn * 4, cudaMemcpyHostToDevice, ctx->stream));
        dx = (const float*)(d + x_off); dout = (float*)(d + o_off);
    }
    FLARE_TRY(flare_launch_quantize_input(ctx, dx, nblk, (int8_t*)(d + q_off), (float*)(d + s_off)));
    FLARE_TRY(flare_launch_matvec_q8_0_preq(ctx, w, (const int8_t*)(d + q_off), (const float*)(d + s_off), batch, dout));
    if (!on_device) {
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(out, dout, on * 4, cudaMemcpyDeviceToHost, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return FLARE_OK;
}

}  // extern "C"

// quantize_input_q8_0 of n_blocks blocks of 32 values, all on the device
int flare_launch_quantize_input(flare_attn_ctx* ctx, const float* d_x, size_t n_blocks, int8_t* d_xq, float* d_xs) {
    const int threads = 256;
    size_t g = (n_blocks * 32 + threads - 1) / threads;
    if (g > 148 * 16) g = 148 * 16;
    if (g < 1) g = 1;
    ctx->last_launch_overlappable = false;
    quantize_input_kernel<<<(int)g, threads, 0, ctx->stream>>>(d_x, n_blocks, d_xq, d_xs);
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}

// matvec_q8_0_preq_into for `batch` quantised input vectors, all on the device
int flare_launch_matvec_q8_0_preq(flare_attn_ctx* ctx, const flare_weight* w, const int8_t* d_xq, const float* d_xs, int batch,
                                  float* d_out) {
    MatvecParams p;
    p.w = w->blocks; p.xq = d_xq; p.xs = d_xs; p.out = d_out;
    p.rows = w->rows; p.cols = w->cols; p.batch = batch;
    const int smem = WARPS * WARP_SMEM;
    {
        static std::mutex m;
        std::lock_guard<std::mutex> lock(m);
        static bool attr_done[64] = {};
        if (!attr_done[ctx->device & 63]) {
            FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(matvec_q8_0_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            attr_done[ctx->device & 63] = true;
        }
    }
    ctx->last_launch_overlappable = false;
    matvec_q8_0_kernel<<<(w->rows + WARPS - 1) / WARPS, 32 * WARPS, smem, ctx->stream>>>(p);
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}

void flare_weight_dims(const flare_weight* w, int* rows, int* cols) { *rows = w->rows; *cols = w->cols; }
