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
#include "q8_input.cuh"
#include "tma.cuh"
#include <mutex>

struct flare_weight {
    flare_attn_ctx* ctx = nullptr;
    int rows = 0, cols = 0;
    // the GGUF block stream (f16 LE scale + 32 x i8 per 34 bytes) taken apart at upload, so that the 32 weights
    // of a block start on a 32-byte boundary: same numbers, same bytes per block read
    int8_t* qs = nullptr;        // [rows][cols]
    __half* sc = nullptr;        // [rows][cols / 32]
};

namespace {

constexpr int CHUNK = 64;            // blocks of a row handled per pass: two per lane
constexpr int WARPS = 8;
constexpr int TS = CHUNK + 1;        // floats per input vector in the product buffer (odd: no bank conflicts in the sums)

// one thread per block: 34 bytes -> scale plane + weight plane
__global__ void repack_q8_0_kernel(const unsigned char* __restrict__ blocks, size_t n_blocks, int8_t* __restrict__ qs,
                                   __half* __restrict__ sc) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_blocks; i += (size_t)gridDim.x * blockDim.x) {
        const uint16_t* b16 = reinterpret_cast<const uint16_t*>(blocks + i * 34);
        sc[i] = __ushort_as_half(b16[0]);
        uint16_t* d16 = reinterpret_cast<uint16_t*>(qs + i * 32);
#pragma unroll
        for (int j = 0; j < 16; j++) d16[j] = b16[1 + j];
    }
}

// quantize_input_q8_0: one warp per 32-value block, lane = element
__global__ void quantize_input_kernel(const float* __restrict__ x, size_t n_blocks, int8_t* __restrict__ xq,
                                      float* __restrict__ xs) {
    flare_pdl_wait();
    flare_pdl_trigger();
    const int lane = threadIdx.x & 31;
    for (size_t w = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5; w < n_blocks; w += ((size_t)gridDim.x * blockDim.x) >> 5)
        flare_quantize_block_of_32(x[w * 32 + lane], lane, xq + w * 32, xs + w);
}

struct MatvecParams {
    const int8_t* wq;            // [rows][cols]
    const __half* ws;            // [rows][cols / 32]
    const int8_t* xq;            // [batch][cols]
    const float* xs;             // [batch][cols / 32]
    float* out;                  // [batch][rows]
    int rows, cols, batch;
    int bt;                      // input vectors per tile: min(batch, 32); sizes the product buffer
    int accumulate;              // out += product (the residual connection) instead of out = product
    int* err;                    // status word of the context (a bulk copy that never arrives)
};

// A warp owns one row at a time.  Per chunk of 64 blocks every lane holds two blocks of the row in registers
// (two 16-byte loads each, the warp reads 2 KB contiguous), multiplies them with every input vector of the tile
// and leaves the products in shared memory; then lane b adds the chunk's products of input vector b in block order.
__global__ void __launch_bounds__(32 * WARPS) matvec_q8_0_kernel(MatvecParams p) {
    extern __shared__ __align__(16) float terms_all[];
    flare_pdl_wait();
    flare_pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = p.cols / 32;
    float* terms = terms_all + (size_t)warp * p.bt * TS;
    const int n_tiles = (p.batch + 31) / 32;
    const int8_t* xq = p.xq;
    const float* xs = p.xs;
    for (int row = blockIdx.x * WARPS + warp; row < p.rows; row += gridDim.x * WARPS) {
        const int8_t* wrow = p.wq + (size_t)row * p.cols;
        const __half* srow = p.ws + (size_t)row * nb;
        float sum[8];                                 // running sums of this lane's input vector in each batch tile (batch <= 256)
#pragma unroll
        for (int t = 0; t < 8; t++) sum[t] = 0.0f;
        for (int c0 = 0; c0 < nb; c0 += CHUNK) {
            const int cn = min(CHUNK, nb - c0);
            // this lane's (up to) two blocks of the chunk
            float wsc[2];
            int4 w0[2], w1[2];
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int blk = lane + 32 * k;
                if (blk < cn) {
                    const int4* wp = reinterpret_cast<const int4*>(wrow + (size_t)(c0 + blk) * 32);
                    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(w0[k].x), "=r"(w0[k].y), "=r"(w0[k].z), "=r"(w0[k].w) : "l"(wp));
                    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(w1[k].x), "=r"(w1[k].y), "=r"(w1[k].z), "=r"(w1[k].w) : "l"(wp + 1));
                    wsc[k] = __half2float(srow[c0 + blk]);
                } else {
                    wsc[k] = 0.0f;
                    w0[k] = make_int4(0, 0, 0, 0); w1[k] = make_int4(0, 0, 0, 0);
                }
            }
#pragma unroll 1
            for (int t = 0; t < n_tiles; t++) {
                const int bn = min(32, p.batch - 32 * t);
                __syncwarp();                         // the sums of the previous pass have read the buffer
                for (int b = 0; b < bn; b++) {
                    const size_t vec = (size_t)(32 * t + b);
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        const int blk = lane + 32 * k;
                        if (blk < cn) {
                            const int4* xp = reinterpret_cast<const int4*>(xq + vec * p.cols + (size_t)(c0 + blk) * 32);
                            const int4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
                            int acc = 0;
                            acc = __dp4a(w0[k].x, x0.x, acc); acc = __dp4a(w0[k].y, x0.y, acc);
                            acc = __dp4a(w0[k].z, x0.z, acc); acc = __dp4a(w0[k].w, x0.w, acc);
                            acc = __dp4a(w1[k].x, x1.x, acc); acc = __dp4a(w1[k].y, x1.y, acc);
                            acc = __dp4a(w1[k].z, x1.z, acc); acc = __dp4a(w1[k].w, x1.w, acc);
                            const float cs = __fmul_rn(wsc[k], __ldg(xs + vec * nb + c0 + blk));
                            terms[b * TS + blk] = __fmul_rn(cs, (float)acc);
                        }
                    }
                }
                __syncwarp();
                // lane b adds the chunk's products of input vector b in block order
                if (lane < bn) {
                    float s = sum[t];
                    const float* tp = terms + lane * TS;
#pragma unroll 8
                    for (int blk = 0; blk < cn; blk++) s = __fadd_rn(s, tp[blk]);
                    sum[t] = s;
                }
            }
        }
#pragma unroll
        for (int t = 0; t < 8; t++)
            if (t < n_tiles && 32 * t + lane < p.batch) {
                float* o = p.out + (size_t)(32 * t + lane) * p.rows + row;
                *o = p.accumulate ? __fadd_rn(*o, sum[t]) : sum[t];
            }
    }
}

// The same product with the weights staged through shared memory by bulk copies: every warp keeps a ring of
// RING chunk buffers (64 blocks: 2 KB of weights + 128 B of scales) that lane 0 refills with cp.async.bulk as soon as
// the warp has taken a chunk into registers, so several chunks per warp are on their way from HBM at any time without
// costing registers.  Needs rows and chunks on 16-byte boundaries (cols % 256 == 0); used for one or two input vectors.
constexpr int RING = 4;
constexpr int RING_CHUNK_BYTES = CHUNK * 32 + CHUNK * 2;        // 2176

__global__ void __launch_bounds__(32 * WARPS) matvec_q8_0_ring_kernel(MatvecParams p) {
    extern __shared__ __align__(128) unsigned char ring_smem[];
    __shared__ uint64_t full_bar[WARPS][RING];
    flare_pdl_wait();
    flare_pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = p.cols / 32;
    const int chunks_per_row = (nb + CHUNK - 1) / CHUNK;
    unsigned char* my_ring = ring_smem + (size_t)warp * RING * RING_CHUNK_BYTES;
    float* terms = reinterpret_cast<float*>(ring_smem + (size_t)WARPS * RING * RING_CHUNK_BYTES) + (size_t)warp * p.bt * TS;
    uint64_t* bars = full_bar[warp];
    // this warp's rows: first_row, first_row + row_step, ...; its units are (row, chunk) pairs in that order
    const int first_row = blockIdx.x * WARPS + warp, row_step = gridDim.x * WARPS;
    const int my_rows = first_row < p.rows ? (p.rows - first_row + row_step - 1) / row_step : 0;
    const long long n_units = (long long)my_rows * chunks_per_row;
    auto issue = [&](long long u) {                    // lane 0 only
        const int s = (int)(u % RING);
        const int row = first_row + (int)(u / chunks_per_row) * row_step, c0 = (int)(u % chunks_per_row) * CHUNK;
        const int cn = min(CHUNK, nb - c0);
        unsigned char* dst = my_ring + (size_t)s * RING_CHUNK_BYTES;
        ptx::mbar_expect_tx(&bars[s], (uint32_t)cn * 34);
        ptx::bulk_load(dst, p.wq + (size_t)row * p.cols + (size_t)c0 * 32, (uint32_t)cn * 32, &bars[s]);
        ptx::bulk_load(dst + CHUNK * 32, p.ws + (size_t)row * nb + c0, (uint32_t)cn * 2, &bars[s]);
    };
    if (lane == 0) {
        for (int s = 0; s < RING; s++) ptx::mbar_init(&bars[s], 1);
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
        for (long long u = 0; u < RING && u < n_units; u++) issue(u);
    }
    __syncwarp();
    float sum = 0.0f;                                  // lane b: running sum of input vector b for the current row
    bool failed = false;
    for (long long u = 0; u < n_units; u++) {
        const int s = (int)(u % RING);
        const int row = first_row + (int)(u / chunks_per_row) * row_step, chunk = (int)(u % chunks_per_row), c0 = chunk * CHUNK;
        const int cn = min(CHUNK, nb - c0);
        if (!ptx::mbar_wait(&bars[s], (uint32_t)((u / RING) & 1))) { failed = true; break; }
        const unsigned char* buf = my_ring + (size_t)s * RING_CHUNK_BYTES;
        float wsc[2];
        int4 w0[2], w1[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int blk = lane + 32 * k;
            if (blk < cn) {
                const int4* wp = reinterpret_cast<const int4*>(buf + blk * 32);
                w0[k] = wp[0]; w1[k] = wp[1];
                wsc[k] = __half2float(*reinterpret_cast<const __half*>(buf + CHUNK * 32 + blk * 2));
            } else {
                wsc[k] = 0.0f; w0[k] = make_int4(0, 0, 0, 0); w1[k] = make_int4(0, 0, 0, 0);
            }
        }
        __syncwarp();                                  // every lane has its blocks: the buffer may be refilled
        if (lane == 0 && u + RING < n_units) { ptx::fence_proxy_async(); issue(u + RING); }
        for (int b = 0; b < p.batch; b++) {
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int blk = lane + 32 * k;
                if (blk < cn) {
                    const int4* xp = reinterpret_cast<const int4*>(p.xq + (size_t)b * p.cols + (size_t)(c0 + blk) * 32);
                    const int4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
                    int acc = 0;
                    acc = __dp4a(w0[k].x, x0.x, acc); acc = __dp4a(w0[k].y, x0.y, acc);
                    acc = __dp4a(w0[k].z, x0.z, acc); acc = __dp4a(w0[k].w, x0.w, acc);
                    acc = __dp4a(w1[k].x, x1.x, acc); acc = __dp4a(w1[k].y, x1.y, acc);
                    acc = __dp4a(w1[k].z, x1.z, acc); acc = __dp4a(w1[k].w, x1.w, acc);
                    const float cs = __fmul_rn(wsc[k], __ldg(p.xs + (size_t)b * nb + c0 + blk));
                    terms[b * TS + blk] = __fmul_rn(cs, (float)acc);
                }
            }
        }
        __syncwarp();
        if (lane < p.batch) {
            if (chunk == 0) sum = 0.0f;
            const float* tp = terms + lane * TS;
#pragma unroll 8
            for (int blk = 0; blk < cn; blk++) sum = __fadd_rn(sum, tp[blk]);
            if (chunk == chunks_per_row - 1) {
                float* o = p.out + (size_t)lane * p.rows + row;
                *o = p.accumulate ? __fadd_rn(*o, sum) : sum;
            }
        }
        __syncwarp();                                  // the sums have read the products before the next chunk writes them
    }
    if (failed && lane == 0) flare_report(p.err, FLARE_ERR_TIMEOUT);
}

// One input vector, rows of at most 64 blocks (cols <= 2048: the projections that read the hidden state): the case a
// single-token forward pass spends most of its bytes on.  Two things change against the kernel above.  The input's
// blocks of a lane are the same for every row, so they stay in registers for the whole kernel; and the ordered sum of
// a row, which one lane has to do alone, is done for GROUP rows at a time, a lane per row, so that its 64 dependent
// adds cost 8 instruction slots per row instead of 128.
constexpr int GROUP = 16;

__global__ void __launch_bounds__(32 * WARPS) matvec_q8_0_ring1_kernel(MatvecParams p) {
    extern __shared__ __align__(128) unsigned char ring_smem[];
    __shared__ uint64_t full_bar[WARPS][RING];
    flare_pdl_wait();
    flare_pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = p.cols / 32;                       // <= 64: one chunk per row
    unsigned char* my_ring = ring_smem + (size_t)warp * RING * RING_CHUNK_BYTES;
    float* terms = reinterpret_cast<float*>(ring_smem + (size_t)WARPS * RING * RING_CHUNK_BYTES) + (size_t)warp * GROUP * TS;
    uint64_t* bars = full_bar[warp];
    const int first_row = blockIdx.x * WARPS + warp, row_step = gridDim.x * WARPS;
    const int my_rows = first_row < p.rows ? (p.rows - first_row + row_step - 1) / row_step : 0;
    auto issue = [&](int k) {                          // lane 0 only: row number k of this warp -> stage k % RING
        const int s = k % RING;
        const int row = first_row + k * row_step;
        unsigned char* dst = my_ring + (size_t)s * RING_CHUNK_BYTES;
        ptx::mbar_expect_tx(&bars[s], (uint32_t)nb * 34);
        ptx::bulk_load(dst, p.wq + (size_t)row * p.cols, (uint32_t)nb * 32, &bars[s]);
        ptx::bulk_load(dst + CHUNK * 32, p.ws + (size_t)row * nb, (uint32_t)nb * 2, &bars[s]);
    };
    if (lane == 0) {
        for (int s = 0; s < RING; s++) ptx::mbar_init(&bars[s], 1);
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
        for (int k = 0; k < RING && k < my_rows; k++) issue(k);
    }
    // the input's blocks of this lane
    int4 x0[2], x1[2];
    float xsc[2];
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const int blk = lane + 32 * k;
        if (blk < nb) {
            const int4* xp = reinterpret_cast<const int4*>(p.xq + (size_t)blk * 32);
            x0[k] = __ldg(xp); x1[k] = __ldg(xp + 1);
            xsc[k] = __ldg(p.xs + blk);
        } else {
            x0[k] = make_int4(0, 0, 0, 0); x1[k] = make_int4(0, 0, 0, 0); xsc[k] = 0.0f;
        }
    }
    __syncwarp();
    bool failed = false;
    for (int k = 0; k < my_rows; k++) {
        const int s = k % RING, slot = k % GROUP;
        if (!ptx::mbar_wait(&bars[s], (uint32_t)((k / RING) & 1))) { failed = true; break; }
        const unsigned char* buf = my_ring + (size_t)s * RING_CHUNK_BYTES;
        float t[2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int blk = lane + 32 * j;
            if (blk < nb) {
                const int4* wp = reinterpret_cast<const int4*>(buf + blk * 32);
                const int4 w0 = wp[0], w1 = wp[1];
                const float wsc = __half2float(*reinterpret_cast<const __half*>(buf + CHUNK * 32 + blk * 2));
                int acc = 0;
                acc = __dp4a(w0.x, x0[j].x, acc); acc = __dp4a(w0.y, x0[j].y, acc);
                acc = __dp4a(w0.z, x0[j].z, acc); acc = __dp4a(w0.w, x0[j].w, acc);
                acc = __dp4a(w1.x, x1[j].x, acc); acc = __dp4a(w1.y, x1[j].y, acc);
                acc = __dp4a(w1.z, x1[j].z, acc); acc = __dp4a(w1.w, x1[j].w, acc);
                t[j] = __fmul_rn(__fmul_rn(wsc, xsc[j]), (float)acc);
            } else t[j] = 0.0f;
        }
        __syncwarp();                                  // every lane has read its blocks: the buffer may be refilled
        if (lane == 0 && k + RING < my_rows) { ptx::fence_proxy_async(); issue(k + RING); }
        if (lane < nb) terms[slot * TS + lane] = t[0];
        if (lane + 32 < nb) terms[slot * TS + lane + 32] = t[1];
        if (slot == GROUP - 1 || k == my_rows - 1) {
            __syncwarp();
            if (lane <= slot) {                        // lane r: the r-th row of this group, blocks in ascending order
                const float* tp = terms + lane * TS;
                float sum = 0.0f;
#pragma unroll 8
                for (int blk = 0; blk < nb; blk++) sum = __fadd_rn(sum, tp[blk]);
                float* o = p.out + (first_row + (k - slot + lane) * row_step);
                *o = p.accumulate ? __fadd_rn(*o, sum) : sum;
            }
            __syncwarp();
        }
    }
    if (failed && lane == 0) flare_report(p.err, FLARE_ERR_TIMEOUT);
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
    const size_t n_blocks = (size_t)rows * (cols / 32), bytes = n_blocks * 34;
    unsigned char* raw = nullptr;
    cudaError_t e = cudaMalloc(&raw, bytes + 64);
    if (e == cudaSuccess) e = cudaMalloc(&w->qs, n_blocks * 32);
    if (e == cudaSuccess) e = cudaMalloc(&w->sc, n_blocks * sizeof(__half));
    if (e == cudaSuccess) e = cudaMemcpyAsync(raw, blocks, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
        size_t g = (n_blocks + 255) / 256;
        if (g > 148 * 32) g = 148 * 32;
        repack_q8_0_kernel<<<(int)g, 256, 0, ctx->stream>>>(raw, n_blocks, w->qs, w->sc);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(raw);
    if (e != cudaSuccess) {
        const int code = e == cudaErrorMemoryAllocation ? FLARE_ERR_OOM : FLARE_ERR_CUDA;
        flare_set_error(ctx, code, "flare_weight_upload_q8_0: %zu bytes: %s", bytes, cudaGetErrorString(e));
        cudaGetLastError();
        cudaFree(w->qs); cudaFree(w->sc);
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
    cudaFree(w->qs); cudaFree(w->sc);
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
    FLARE_TRY(flare_launch_matvec_q8_0_preq(ctx, w, (const int8_t*)(d + q_off), (const float*)(d + s_off), batch, dout, 0));
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
    FLARE_CUDA_OK(ctx, flare_launch_pdl(quantize_input_kernel, dim3((unsigned)g), dim3(threads), 0, ctx->stream, d_x, n_blocks, d_xq, d_xs));
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}

// matvec_q8_0_preq_into for `batch` quantised input vectors, all on the device; accumulate: out += product (the
// residual connection) instead of out = product.  (Letting every CTA quantise the f32 input for itself, to save the
// quantiser's launch, was measured slower: 1.69 instead of 1.55 ms per token of the 1B-shaped forward pass.)
int flare_launch_matvec_q8_0_preq(flare_attn_ctx* ctx, const flare_weight* w, const int8_t* d_xq, const float* d_xs, int batch,
                                  float* d_out, int accumulate) {
    MatvecParams p;
    p.wq = w->qs; p.ws = w->sc; p.xq = d_xq; p.xs = d_xs; p.out = d_out;
    p.rows = w->rows; p.cols = w->cols; p.batch = batch;
    p.bt = batch < 32 ? batch : 32;
    p.accumulate = accumulate;
    const int smem = WARPS * p.bt * TS * (int)sizeof(float);
    {
        static std::mutex m;
        std::lock_guard<std::mutex> lock(m);
        static bool attr_done[64] = {};
        if (!attr_done[ctx->device & 63]) {
            FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(matvec_q8_0_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    WARPS * 32 * TS * (int)sizeof(float)));
            attr_done[ctx->device & 63] = true;
        }
    }
    p.err = ctx->d_err;
    ctx->last_launch_overlappable = false;
    if (w->cols % 256 == 0 && batch == 1 && w->cols <= CHUNK * 32) {
        const int ring1_smem = WARPS * RING * RING_CHUNK_BYTES + WARPS * GROUP * TS * (int)sizeof(float);
        {
            static std::mutex m3;
            std::lock_guard<std::mutex> lock(m3);
            static bool ring1_attr[64] = {};
            if (!ring1_attr[ctx->device & 63]) {
                FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(matvec_q8_0_ring1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ring1_smem));
                ring1_attr[ctx->device & 63] = true;
            }
        }
        int grid = (w->rows + WARPS - 1) / WARPS;
        const int max_grid = 148 * 2;                 // two CTAs per SM fit
        if (grid > max_grid) grid = max_grid;
        FLARE_CUDA_OK(ctx, flare_launch_pdl(matvec_q8_0_ring1_kernel, dim3(grid), dim3(32 * WARPS), (size_t)ring1_smem, ctx->stream, p));
        FLARE_LAUNCH_CHECK(ctx);
        return FLARE_OK;
    }
    if (w->cols % 256 == 0 && batch <= 2) {
        // One or two input vectors: the product is bound by memory, and rows and chunks start on 16-byte boundaries, so
        // the weights go through a ring of bulk copies.  (From 8 input vectors on the dots dominate and the direct-load
        // kernel with its many more warps is faster: 212 against 289 us for 128256 x 2048 at batch 8.)
        const int ring_smem = WARPS * RING * RING_CHUNK_BYTES + smem;
        {
            static std::mutex m2;
            std::lock_guard<std::mutex> lock(m2);
            static bool ring_attr[64] = {};
            if (!ring_attr[ctx->device & 63]) {
                FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(matvec_q8_0_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                        WARPS * RING * RING_CHUNK_BYTES + WARPS * 32 * TS * (int)sizeof(float)));
                ring_attr[ctx->device & 63] = true;
            }
        }
        // enough CTAs to fill the SMs (3 per SM at batch 1); each warp then walks its rows through the ring
        int grid = (w->rows + WARPS - 1) / WARPS;
        const int max_grid = 148 * 3;
        if (grid > max_grid) grid = max_grid;
        FLARE_CUDA_OK(ctx, flare_launch_pdl(matvec_q8_0_ring_kernel, dim3(grid), dim3(32 * WARPS), (size_t)ring_smem, ctx->stream, p));
        FLARE_LAUNCH_CHECK(ctx);
        return FLARE_OK;
    }
    // a row per warp; many more warps than the SMs hold at once are pointless, so large matrices loop
    int grid = (w->rows + WARPS - 1) / WARPS;
    const int max_grid = 148 * 8 * 4;
    if (grid > max_grid) grid = max_grid;
    FLARE_CUDA_OK(ctx, flare_launch_pdl(matvec_q8_0_kernel, dim3(grid), dim3(32 * WARPS), (size_t)smem, ctx->stream, p));
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}

void flare_weight_dims(const flare_weight* w, int* rows, int* cols) { *rows = w->rows; *cols = w->cols; }
