// Causal (and sliding-window) prefill attention on the 5th-generation tensor cores.
//
// Replaces the reference's O(S^2) loop of per-position decode calls
// (ComputeBackend::prefill_attention_gpu, flare-core/src/model.rs:336-368) and its WGSL shader
// (flare-gpu/shaders/prefill_attention.wgsl).  Row t attends rows max(0, t-W+1)..=t; query head
// h reads kv head h / (num_heads / num_kv_heads), the CPU mapping.
//
// One CTA = 128 query rows of one (sequence, query head).  Warp roles:
//   warps 0-3  softmax: thread r owns row r; reads its S row from tensor memory, online softmax in
//              log2 units with lazy rescaling, writes P (bf16) to shared memory in the 128B-swizzled
//              K-major layout the MMA reads, rescales O in tensor memory when the row maximum
//              moved, and writes the normalised output at the end
//   warp 4     TMA producer: Q once, then K and V tiles of 128 rows through 2-stage rings
//              (cp.async.bulk.tensor, 128B swizzle, no multicast)
//   warp 5     MMA issuer (one thread): S = Q K^T and O += P V with tcgen05.mma kind::f16
//              (bf16 in, f32 accumulate in tensor memory: S double-buffered, O resident)
// All hand-offs are mbarriers; every wait is bounded and a give-up sets an error word, the CTA
// still frees its tensor memory and exits.
#include "common.cuh"
#include "tma.cuh"
#include "tc5.cuh"
#include <math_constants.h>

namespace {

constexpr int BN = 128;   // key/value rows per tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kWaitLimit = 1u << 20;

struct PrefillParams {
    void* out;
    int out_dtype, batch, seq_len, num_heads, num_kv_heads, window;
    float scale_log2;
    int* err;
};

using namespace tc5;

template <int HD>
struct Smem {
    static constexpr int PANELS = HD / 64;                 // 64-column panels per head row
    static constexpr int Q_BYTES = BM * HD * 2;
    static constexpr int KV_BYTES = BN * HD * 2;
    static constexpr int P_BYTES = BM * BN * 2;
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = Q_OFF + Q_BYTES;          // 2 stages
    static constexpr int V_OFF = K_OFF + 2 * KV_BYTES;     // 2 stages
    static constexpr int P_OFF = V_OFF + 2 * KV_BYTES;
    static constexpr int TOTAL = P_OFF + P_BYTES;
};

struct Barriers {
    uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], s_free[2], p_full, pv_done, o_final;
    uint32_t tmem_base;
    int abort_flag;
};

#define WAIT_OR_ABORT(barptr, parity)                                              \
    do {                                                                           \
        if (!ptx::mbar_wait((barptr), (parity), kWaitLimit)) { bars->abort_flag = 1; aborted = true; } \
    } while (0)

template <int HD>
__global__ void __launch_bounds__(192, 1) prefill_tc_kernel(const __grid_constant__ CUtensorMap qmap,
                                                            const __grid_constant__ CUtensorMap kmap,
                                                            const __grid_constant__ CUtensorMap vmap, PrefillParams p) {
    using L = Smem<HD>;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ Barriers bar_storage;
    Barriers* bars = &bar_storage;
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (p.num_heads / p.num_kv_heads);
    const int r0 = qt * BM;
    const int S = p.seq_len;
    // key/value tiles this query tile reads: columns [col_lo, col_hi)
    const int last_row = min(r0 + BM, S) - 1;
    const int col_hi = last_row + 1;
    const int col_lo = p.window > 0 ? max(0, r0 - p.window + 1) : 0;
    const int j0 = col_lo / BN, j1 = (col_hi + BN - 1) / BN;   // tile range [j0, j1)
    const int n_tiles = j1 - j0;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars->q_full, 1);
        for (int s = 0; s < 2; s++) {
            ptx::mbar_init(&bars->k_full[s], 1); ptx::mbar_init(&bars->v_full[s], 1);
            ptx::mbar_init(&bars->k_empty[s], 1); ptx::mbar_init(&bars->v_empty[s], 1);
            ptx::mbar_init(&bars->s_full[s], 1); ptx::mbar_init(&bars->s_free[s], 128);
        }
        ptx::mbar_init(&bars->p_full, 128);
        ptx::mbar_init(&bars->pv_done, 1);
        ptx::mbar_init(&bars->o_final, 1);
        bars->abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    if (warp == 5) {                       // one warp allocates all 512 columns (1 CTA per SM)
        tmem_alloc(&bars->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    const uint32_t tmem_S0 = tmem, tmem_S1 = tmem + 128, tmem_O = tmem + 256;
    bool aborted = false;

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::mbar_expect_tx(&bars->q_full, L::Q_BYTES);
            for (int pn = 0; pn < L::PANELS; pn++)
                ptx::tma_load_4d(sm + L::Q_OFF + pn * (BM * 128), &qmap, &bars->q_full, pn * 64, h, r0, b);
            for (int t = 0; t < n_tiles && !aborted; t++) {
                const int s = t & 1, row = (j0 + t) * BN;
                if (t >= 2) WAIT_OR_ABORT(&bars->k_empty[s], (uint32_t)(((t >> 1) - 1) & 1));
                if (aborted) break;
                ptx::mbar_expect_tx(&bars->k_full[s], L::KV_BYTES);
                for (int pn = 0; pn < L::PANELS; pn++)
                    ptx::tma_load_4d(sm + L::K_OFF + s * L::KV_BYTES + pn * (BN * 128), &kmap, &bars->k_full[s], pn * 64, kvh, row, b);
                if (t >= 2) WAIT_OR_ABORT(&bars->v_empty[s], (uint32_t)(((t >> 1) - 1) & 1));
                if (aborted) break;
                ptx::mbar_expect_tx(&bars->v_full[s], L::KV_BYTES);
                for (int pn = 0; pn < L::PANELS; pn++)
                    ptx::tma_load_4d(sm + L::V_OFF + s * L::KV_BYTES + pn * (BN * 128), &vmap, &bars->v_full[s], pn * 64, kvh, row, b);
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_qk = idesc_bf16(BN, false);
            const uint32_t idesc_pv = idesc_bf16(HD, true);
            const uint32_t q_addr = ptx::smem_u32(sm + L::Q_OFF), p_addr = ptx::smem_u32(sm + L::P_OFF);
            auto do_pv = [&](int t) {
                const int s = t & 1;
                WAIT_OR_ABORT(&bars->p_full, (uint32_t)(t & 1));
                if (aborted) return;
                WAIT_OR_ABORT(&bars->v_full[s], (uint32_t)((t >> 1) & 1));
                if (aborted) return;
                tc_fence_after();
                const uint32_t v_addr = ptx::smem_u32(sm + L::V_OFF + s * L::KV_BYTES);
#pragma unroll
                for (int k = 0; k < BN / 16; k++) {
                    // A = P[128 rows][16 slots]: K-major, slot panels of 64; B = V[16 slots][HD]: MN-major
                    const uint64_t ad = desc_kmajor(p_addr + (k >> 2) * (BM * 128) + (k & 3) * 32);
                    const uint64_t bd = desc_mnmajor(v_addr + k * 2048, BN * 128);
                    umma_bf16(tmem_O, ad, bd, idesc_pv, (t > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(&bars->v_empty[s]);
                tc_commit(&bars->pv_done);
            };
            WAIT_OR_ABORT(&bars->q_full, 0);
            for (int t = 0; t < n_tiles && !aborted; t++) {
                const int s = t & 1;
                WAIT_OR_ABORT(&bars->k_full[s], (uint32_t)((t >> 1) & 1));
                if (aborted) break;
                if (t >= 2) WAIT_OR_ABORT(&bars->s_free[s], (uint32_t)(((t >> 1) - 1) & 1));
                if (aborted) break;
                tc_fence_after();
                const uint32_t k_addr = ptx::smem_u32(sm + L::K_OFF + s * L::KV_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; k++) {
                    const uint64_t ad = desc_kmajor(q_addr + (k >> 2) * (BM * 128) + (k & 3) * 32);
                    const uint64_t bd = desc_kmajor(k_addr + (k >> 2) * (BN * 128) + (k & 3) * 32);
                    umma_bf16(s ? tmem_S1 : tmem_S0, ad, bd, idesc_qk, k > 0 ? 1u : 0u);
                }
                tc_commit(&bars->k_empty[s]);
                tc_commit(&bars->s_full[s]);
                if (t >= 1) do_pv(t - 1);
            }
            if (!aborted && n_tiles > 0) do_pv(n_tiles - 1);
            if (!aborted) tc_commit(&bars->o_final);
        }
    } else {
        // ------------------------------------------------------------------ softmax (thread = row)
        const int r = threadIdx.x;                      // 0..127
        const int grow = r0 + r;                        // global row
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        float m_ref = -CUDART_INF_F, l_sum = 0.0f;
        const int row_lo = p.window > 0 ? max(0, grow - p.window + 1) : 0;   // first column this row attends
        for (int t = 0; t < n_tiles && !aborted; t++) {
            const int s = t & 1;
            const int c0 = (j0 + t) * BN;               // first column of the tile
            const uint32_t ts = (s ? tmem_S1 : tmem_S0) + lane_base;
            WAIT_OR_ABORT(&bars->s_full[s], (uint32_t)((t >> 1) & 1));
            if (aborted) break;
            tc_fence_after();
            // a tile needs element masks only if it crosses the diagonal, the window edge or the end
            const bool need_mask = (c0 + BN - 1 > r0) || (p.window > 0 && c0 < r0 + BM - p.window) || (c0 + BN > S);
            // pass 1: row maximum
            float tmax = -CUDART_INF_F;
#pragma unroll 1
            for (int ch = 0; ch < 4; ch++) {
                uint32_t v[32];
                tmem_ld32(ts + ch * 32, v);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    float x = __uint_as_float(v[i]);
                    if (need_mask) {
                        const int col = c0 + ch * 32 + i;
                        if (col > grow || col < row_lo || col >= S) x = -CUDART_INF_F;
                    }
                    tmax = fmaxf(tmax, x);
                }
            }
            tmax *= p.scale_log2;
            // lazy rescale: move the reference maximum only when it is exceeded by more than 2^8
            float alpha = 1.0f;
            const bool bump = tmax > m_ref + 8.0f;
            if (bump) { alpha = fast_exp2(m_ref - tmax); m_ref = tmax; }
            const bool any_bump = __any_sync(0xffffffffu, bump);
            // P of the previous tile must have been consumed (and O updated) before we touch P or O
            if (t >= 1) { WAIT_OR_ABORT(&bars->pv_done, (uint32_t)((t - 1) & 1)); if (aborted) break; tc_fence_after(); }
            if (any_bump && t >= 1) {
                const uint32_t to = tmem_O + lane_base;
#pragma unroll 1
                for (int ch = 0; ch < HD / 32; ch++) {
                    uint32_t v[32];
                    tmem_ld32(to + ch * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st32(to + ch * 32, v);
                }
                tmem_wait_st();
            }
            l_sum *= alpha;
            // pass 2: p = exp2(s * scale - m), bf16, into the swizzled P tile
            const float neg_m = (m_ref == -CUDART_INF_F) ? 0.0f : -m_ref;   // fully masked so far: exp2(-inf) = 0
            unsigned char* prow = sm + L::P_OFF + r * 128;
#pragma unroll 1
            for (int ch = 0; ch < 4; ch++) {
                uint32_t v[32];
                tmem_ld32(ts + ch * 32, v);
                tmem_wait_ld();
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float x0 = __uint_as_float(v[i]), x1 = __uint_as_float(v[i + 1]);
                    if (need_mask) {
                        const int col = c0 + ch * 32 + i;
                        if (col > grow || col < row_lo || col >= S) x0 = -CUDART_INF_F;
                        if (col + 1 > grow || col + 1 < row_lo || col + 1 >= S) x1 = -CUDART_INF_F;
                    }
                    float p0 = fast_exp2(fmaf(x0, p.scale_log2, neg_m)), p1 = fast_exp2(fmaf(x1, p.scale_log2, neg_m));
                    __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
                    // the row sum uses the rounded weights, the values the tensor core will multiply
                    l_sum += __bfloat162float(pb.x) + __bfloat162float(pb.y);
                    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&pb);
                }
                // 32 columns = 64 bytes = 4 chunks of 16 B; panel = ch / 2, chunk index within the row = (ch & 1) * 4 + q
                unsigned char* pp = prow + (ch >> 1) * (BM * 128);
#pragma unroll
                for (int qd = 0; qd < 4; qd++) {
                    const int chunk = ((ch & 1) * 4 + qd) ^ (r & 7);
                    *reinterpret_cast<uint4*>(pp + chunk * 16) = make_uint4(packed[4 * qd], packed[4 * qd + 1], packed[4 * qd + 2], packed[4 * qd + 3]);
                }
            }
            // S buffer consumed; P written: make the generic-proxy writes visible to the tensor core
            tc_fence_before();
            ptx::mbar_arrive(&bars->s_free[s]);
            ptx::fence_proxy_async();
            ptx::mbar_arrive(&bars->p_full);
        }
        // epilogue: O / l
        if (!aborted) {
            WAIT_OR_ABORT(&bars->o_final, 0);
        }
        if (!aborted && n_tiles > 0) {
            tc_fence_after();
            const float inv = l_sum > 0.0f ? 1.0f / l_sum : 0.0f;
            const uint32_t to = tmem_O + lane_base;
            const size_t orow = (((size_t)b * S + grow) * p.num_heads + h) * HD;
#pragma unroll 1
            for (int ch = 0; ch < HD / 32; ch++) {
                uint32_t v[32];
                tmem_ld32(to + ch * 32, v);
                tmem_wait_ld();
                if (grow < S) {
                    if (p.out_dtype == FLARE_DT_F32) {
                        float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + orow + ch * 32);
#pragma unroll
                        for (int i = 0; i < 8; i++)
                            o[i] = make_float4(__uint_as_float(v[4 * i]) * inv, __uint_as_float(v[4 * i + 1]) * inv,
                                               __uint_as_float(v[4 * i + 2]) * inv, __uint_as_float(v[4 * i + 3]) * inv);
                    } else {
                        uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + orow + ch * 32);
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            uint32_t w[4];
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                __nv_bfloat162 pb = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * k]) * inv, __uint_as_float(v[8 * i + 2 * k + 1]) * inv);
                                w[k] = *reinterpret_cast<uint32_t*>(&pb);
                            }
                            o[i] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        }
    }
    // ---- teardown: everyone meets, tensor memory is returned -----------------------------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && bars->abort_flag) atomicExch(p.err, FLARE_ERR_TIMEOUT);
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

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
    d.layer = 0; d.kmap = d.vmap = nullptr; d.whole_rows = 0; d.window = a.window; d.kv_obj = nullptr;
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
    PrefillParams p;
    p.out = a.out; p.out_dtype = a.out_dtype; p.batch = a.batch; p.seq_len = a.seq_len; p.num_heads = a.num_heads;
    p.num_kv_heads = a.num_kv_heads; p.window = a.window;
    p.scale_log2 = (1.0f / sqrtf((float)a.head_dim)) * kLog2e;
    p.err = ctx->d_err;
    {
        PrefillArgs a2 = a;
        a2.q = q; a2.k = k; a2.v = v;
        return flare_launch_prefill_pp(ctx, qm, km, vm, a2);
    }
    dim3 grid((a.seq_len + BM - 1) / BM, a.num_heads, a.batch);
    if (a.head_dim == 128) {
        const int smem = Smem<128>::TOTAL + 1024;
        FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        prefill_tc_kernel<128><<<grid, 192, smem, ctx->stream>>>(qm, km, vm, p);
    } else {
        // at least 120 KB so that only one CTA (which takes all 512 tensor-memory columns) fits per SM
        const int smem = (Smem<64>::TOTAL + 1024) > 120 * 1024 ? (Smem<64>::TOTAL + 1024) : 120 * 1024;
        FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        prefill_tc_kernel<64><<<grid, 192, smem, ctx->stream>>>(qm, km, vm, p);
    }
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}
