// Device pieces shared by the input quantisers (quantize_input_q8_0, rmsnorm_quantize_q8_0; flare-core/src/model.rs:
// 5507-5527, 5610-5641): used by the standalone kernels and by the matrix-vector kernel's prologue.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

__device__ __forceinline__ int8_t flare_to_i8_saturating(float r) {       // Rust `as i8`
    return (int8_t)((r != r) ? 0 : (r >= 127.0f ? 127 : (r <= -128.0f ? -128 : (int)r)));
}

// sum over the block of one value per thread; every thread gets the total (s_red: one float per warp)
__device__ __forceinline__ float flare_block_sum(float s, float* s_red) {
#pragma unroll
    for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    __syncthreads();                                  // s_red may still be read from an earlier call
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = s;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += s_red[w];
    return t;
}

// one warp, one block of 32 values (lane = element): amax, scale = amax / 127, q = round(n * (127 / amax)) as i8
__device__ __forceinline__ void flare_quantize_block_of_32(float n, int lane, int8_t* q_out, float* s_out) {
    float amax = fabsf(n);
#pragma unroll
    for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float scale = __fdiv_rn(amax, 127.0f);
    const float inv_scale = scale != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    q_out[lane] = flare_to_i8_saturating(roundf(__fmul_rn(n, inv_scale)));
    if (lane == 0) *s_out = scale;
}

// One input vector of `dim` values quantised by the whole block (any number of warps): plain (norm_weight ==
// nullptr) or after the RMS norm, n = x * weight * inv_rms.  Up to eight blocks per warp stay in registers between
// the sum of squares and the quantisation, so that all loads of a pass are in flight together.
__device__ __forceinline__ void flare_quantize_vector(const float* __restrict__ x, const float* __restrict__ norm_weight,
                                                      float eps, int dim, int8_t* q_out, float* s_out, float* s_red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5, nb = dim / 32;
    if (nb <= 8 * nw) {
        // the whole vector fits in registers: read once, all loads in flight together
        float xv[8], wv[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int blk = warp + k * nw;
            xv[k] = blk < nb ? x[blk * 32 + lane] : 0.0f;
            wv[k] = (norm_weight && blk < nb) ? norm_weight[blk * 32 + lane] : 1.0f;
        }
        float inv_rms = 1.0f;
        if (norm_weight) {
            float s = 0.0f;
#pragma unroll
            for (int k = 0; k < 8; k++) s = fmaf(xv[k], xv[k], s);
            const float sum_sq = flare_block_sum(s, s_red);
            inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_sq, (float)dim), eps)));
        }
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int blk = warp + k * nw;
            if (blk < nb) {
                const float n = norm_weight ? __fmul_rn(__fmul_rn(xv[k], wv[k]), inv_rms) : xv[k];
                flare_quantize_block_of_32(n, lane, q_out + blk * 32, s_out + blk);
            }
        }
        return;
    }
    float inv_rms = 1.0f;
    if (norm_weight) {
        float s = 0.0f;
        for (int i = threadIdx.x; i < dim; i += blockDim.x) s = fmaf(x[i], x[i], s);
        const float sum_sq = flare_block_sum(s, s_red);
        inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_sq, (float)dim), eps)));
    }
    for (int blk0 = 0; blk0 < nb; blk0 += 8 * nw) {
        float xv[8], wv[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int blk = blk0 + warp + k * nw;
            xv[k] = blk < nb ? x[blk * 32 + lane] : 0.0f;
            wv[k] = (norm_weight && blk < nb) ? norm_weight[blk * 32 + lane] : 1.0f;
        }
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int blk = blk0 + warp + k * nw;
            if (blk < nb) {
                const float n = norm_weight ? __fmul_rn(__fmul_rn(xv[k], wv[k]), inv_rms) : xv[k];
                flare_quantize_block_of_32(n, lane, q_out + blk * 32, s_out + blk);
            }
        }
    }
}
