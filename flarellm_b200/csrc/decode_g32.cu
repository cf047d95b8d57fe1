// Group-32 KIVI (2-bit) split-KV decode attention on tensor cores, for the quantised part of the
// cache (head_dim 64, up to 4 query heads per KV head, one query per sequence, ring not wrapped).
// The newest <= 159 tokens (the f16 residual ring and the group that is still filling) go through
// the general kernel; the two partial results are merged by log-sum-exp.
//
// Same skeleton as the Q8_0 path: one CTA per (sequence, slot range), one warp per KV head, 32-slot
// tiles (= one key group) streamed into a ring of shared-memory stages by TMA — the 2-bit K and V codes
// as [head][slot][16 B] through tensor maps, the group's key (scale, zero) pairs and the tile's value
// (scale, zero) pairs as plain bulk copies — each stage behind an mbarrier, refilled by the last
// warp that finishes with it.
//
// Dequantisation never happens per element.  With c the 2-bit code:
//   scores  S[h, t] = sum_ch q[h,ch] (c[t,ch] s[ch] + z[ch]) = sum_ch (q s)[h,ch] c[t,ch] + sum_ch q[h,ch] z[ch]
//           q*s is rebuilt per key group as f16 hi + lo (A operand rows g and g+8, m16n8k16), the codes
//           become exact f16 values with one shift, one mask-or and one subtract per pair;
//   output  O[h, ch] = sum_t (p[t] s[t,blk]) c[t,ch] + sum_t p[t] z[t,blk]
//           weights p*s in f16, codes transposed by ldmatrix.trans (16-bit units hold 8 codes of a slot)
//           and expanded the same way, the zero-point term is one scalar per (head, 32-channel block).
#include "common.cuh"
#include "tma.cuh"
#include <math_constants.h>

namespace {

constexpr int T = 32;
constexpr int STAGES = 4;
constexpr int HD = 64;
constexpr float kLog2e = 1.4426950408889634f;

struct G32Params {
    const float* q;
    float* work;
    const int* attend_len;
    const unsigned char* k_meta;     // layer base, sequence 0: [group][kv_dim] half2
    const unsigned char* v_meta;     // [slot][kv_dim/32] half2
    size_t k_meta_seq_stride, v_meta_seq_stride;   // bytes
    int layer_seq0, num_heads, nkv, G, n_split;
    int* err;
};

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    uint32_t u;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(u) : "f"(hi), "f"(lo));
    return u;
}
__device__ __forceinline__ float2 unpack_half2(uint32_t u) {
    float2 f;
    asm("{\n\t.reg .f16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.f32.f16 %0, lo;\n\tcvt.f32.f16 %1, hi;\n\t}"
        : "=f"(f.x), "=f"(f.y) : "r"(u));
    return f;
}
// two 2-bit codes that sit 16 bits apart in `w` (at bit `sh` of each half) -> half2 of their values
__device__ __forceinline__ uint32_t codes_to_half2(uint32_t w, int sh) {
    uint32_t u = ((w >> sh) & 0x00030003u) | 0x64006400u;      // 1024 + code in each half
    asm("sub.f16x2 %0, %0, %1;" : "+r"(u) : "r"(0x64006400u));   // exact
    return u;
}
__device__ __forceinline__ uint32_t codes_to_half2_biased(uint32_t w, int sh) {
    return ((w >> sh) & 0x00030003u) | 0x64006400u;             // 1024 + code; the bias is removed at the end
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__global__ void __launch_bounds__(256) decode_g32_kernel(const __grid_constant__ CUtensorMap kmap,
                                                         const __grid_constant__ CUtensorMap vmap, G32Params p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ uint64_t full_bar[STAGES];
    __shared__ int done_cnt[STAGES];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int split = blockIdx.x, b = blockIdx.y;
    const int nkv = p.nkv, kvh = warp;
    const int kv_dim = nkv * HD;
    // stage: K codes [nkv][T][16], V codes [nkv][T][16], K meta [kv_dim] half2, V meta [T][nkv*2] half2
    const int codes = nkv * T * 16;
    const int kmeta_bytes = kv_dim * 4, vmeta_bytes = T * nkv * 2 * 4;
    const int stage_bytes = 2 * codes + kmeta_bytes + vmeta_bytes;
    unsigned char* sbase = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

    // quantised slots of this sequence: everything older than the newest 128 tokens, in whole groups
    const int n = p.attend_len[b];
    const int lim_tiles = n > 128 ? (n - 128) / T : 0;
    const int t_begin = (int)(((long long)split * lim_tiles) / p.n_split);
    const int t_end = (int)(((long long)(split + 1) * lim_tiles) / p.n_split);
    const int n_tiles = t_end - t_begin;

    const unsigned char* kmg = p.k_meta + (size_t)b * p.k_meta_seq_stride;
    const unsigned char* vmg = p.v_meta + (size_t)b * p.v_meta_seq_stride;
    auto issue = [&](int i) {
        const int s = i % STAGES;
        unsigned char* st = sbase + (size_t)s * stage_bytes;
        const int tile = t_begin + i;
        ptx::mbar_expect_tx(&full_bar[s], stage_bytes);
        ptx::tma_load_4d(st, &kmap, &full_bar[s], 0, tile * T, 0, p.layer_seq0 + b);
        ptx::tma_load_4d(st + codes, &vmap, &full_bar[s], 0, tile * T, 0, p.layer_seq0 + b);
        ptx::bulk_load(st + 2 * codes, kmg + (size_t)tile * kmeta_bytes, kmeta_bytes, &full_bar[s]);
        ptx::bulk_load(st + 2 * codes + kmeta_bytes, vmg + (size_t)tile * vmeta_bytes, vmeta_bytes, &full_bar[s]);
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { ptx::mbar_init(&full_bar[s], 1); done_cnt[s] = 0; }
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
        for (int i = 0; i < STAGES && i < n_tiles; i++) issue(i);
    }
    __syncthreads();
    pdl_wait();

    // ---- this lane's 16 channels of q (scaled): channel(ks, u) = 16 ks + tig + 4 u ------------------
    const int hq = g & 3;
    const bool head_ok = hq < p.G;
    const size_t row = (size_t)b * p.num_heads + kvh * p.G + (head_ok ? hq : 0);
    float qv[4][4];
    {
        const float sc = rsqrtf((float)HD) * kLog2e;
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
#pragma unroll
            for (int u = 0; u < 4; u++) qv[ks][u] = head_ok ? __ldg(p.q + row * HD + 16 * ks + tig + 4 * u) * sc : 0.0f;
    }

    float acc[8][4];                      // n-tile cc: columns g <-> channel 8 g + cc
#pragma unroll
    for (int cc = 0; cc < 8; cc++)
#pragma unroll
        for (int k = 0; k < 4; k++) acc[cc][k] = 0.0f;
    float m_run = -CUDART_INF_F, l_run = 0.0f, lb = 0.0f, zacc = 0.0f;
    const int lane_blk = g >> 2;          // rows g < 4 weight channel block 0, rows 4..7 block 1

    bool failed = false;
    for (int i = 0; i < n_tiles; i++) {
        const int s = i % STAGES;
        if (!ptx::mbar_wait(&full_bar[s], (uint32_t)((i / STAGES) & 1))) { failed = true; break; }
        const unsigned char* st = sbase + (size_t)s * stage_bytes;
        const unsigned char* kc = st + kvh * (T * 16);
        const uint32_t vc = ptx::smem_u32(st + codes + kvh * (T * 16));
        const uint32_t* kmeta = reinterpret_cast<const uint32_t*>(st + 2 * codes) + kvh * HD;
        const uint32_t* vmeta = reinterpret_cast<const uint32_t*>(st + 2 * codes + kmeta_bytes);

        // ---- A operand of the score product: (q s) as f16 hi + lo, and the zero-point term ---------
        uint32_t qa[4][4];
        float bias = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            float qs[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float2 m = unpack_half2(kmeta[16 * ks + tig + 4 * u]);     // (scale, zero) of the channel
                qs[u] = qv[ks][u] * m.x;
                bias = fmaf(qv[ks][u], m.y, bias);
            }
            // logical k (2tig, 2tig+1) <-> channels (tig, tig+8) = u 0, 2;  k (2tig+8, +9) <-> (tig+4, tig+12) = u 1, 3
            const uint32_t h0 = pack_half2(qs[0], qs[2]), h1 = pack_half2(qs[1], qs[3]);
            const float2 f0 = unpack_half2(h0), f1 = unpack_half2(h1);
            qa[ks][0] = h0;                                          // row g,   k low half  (hi part)
            qa[ks][1] = pack_half2(qs[0] - f0.x, qs[2] - f0.y);      // row g+8              (lo part)
            qa[ks][2] = h1;                                          // row g,   k high half
            qa[ks][3] = pack_half2(qs[1] - f1.x, qs[3] - f1.y);
        }
        bias += __shfl_xor_sync(0xffffffffu, bias, 1);
        bias += __shfl_xor_sync(0xffffffffu, bias, 2);

        // ---- scores ---------------------------------------------------------------------------------
        float sc[4][2];
        float tmax = -CUDART_INF_F;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint4 w = *reinterpret_cast<const uint4*>(kc + (8 * j + g) * 16);   // 64 codes of slot 8j+g
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int ks = 0; ks < 4; ks++)
                mma_f16(d, qa[ks], codes_to_half2(ww[ks], 2 * tig), codes_to_half2(ww[ks], 2 * tig + 8));
            sc[j][0] = d[0] + d[2] + bias;        // slot 8j + 2tig
            sc[j][1] = d[1] + d[3] + bias;        // slot 8j + 2tig + 1
            tmax = fmaxf(tmax, fmaxf(sc[j][0], sc[j][1]));
        }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const bool bump = tmax > m_run + 8.0f;
        if (__any_sync(0xffffffffu, bump)) {
            const float alpha = bump ? fast_exp2(m_run - tmax) : 1.0f;
            if (bump) m_run = tmax;
            l_run *= alpha; lb *= alpha; zacc *= alpha;
#pragma unroll
            for (int cc = 0; cc < 8; cc++)
#pragma unroll
                for (int k = 0; k < 4; k++) acc[cc][k] *= alpha;
        }
        // ---- weights p * s[t, blk] (f16) and the zero-point sum ---------------------------------------
        uint32_t pa[2][4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float p0 = fast_exp2(sc[j][0] - m_run), p1 = fast_exp2(sc[j][1] - m_run);
            l_run += p0 + p1;
            const float2 m0 = unpack_half2(vmeta[(8 * j + 2 * tig) * (nkv * 2) + kvh * 2 + lane_blk]);
            const float2 m1 = unpack_half2(vmeta[(8 * j + 2 * tig + 1) * (nkv * 2) + kvh * 2 + lane_blk]);
            zacc = fmaf(p0, m0.y, fmaf(p1, m1.y, zacc));
            const uint32_t wb = pack_half2(p0 * m0.x, p1 * m1.x);
            const float2 wf = unpack_half2(wb);
            lb += wf.x + wf.y;
            pa[j >> 1][(j & 1) * 2] = wb;
            pa[j >> 1][(j & 1) * 2 + 1] = 0u;
        }
        // ---- output -------------------------------------------------------------------------------------
        uint32_t rr[4];
        ldmatrix_x4_trans(rr, vc + lane * 16);          // matrix m = slots 8m .. 8m+7, 16 bytes (64 codes) per slot
#pragma unroll
        for (int kstep = 0; kstep < 2; kstep++)
#pragma unroll
            for (int cc = 0; cc < 8; cc++)
                mma_f16(acc[cc], pa[kstep], codes_to_half2_biased(rr[2 * kstep], 2 * cc), codes_to_half2_biased(rr[2 * kstep + 1], 2 * cc));

        __syncwarp();
        if (lane == 0 && i + STAGES < n_tiles) {
            if (atomicAdd(&done_cnt[s], 1) == nkv - 1) {
                done_cnt[s] = 0;
                ptx::fence_proxy_async();
                issue(i + STAGES);
            }
        }
    }
    pdl_trigger();
    if (failed) {
        if (lane == 0) atomicExch(p.err, FLARE_ERR_TIMEOUT);
        return;
    }
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    lb += __shfl_xor_sync(0xffffffffu, lb, 1);
    lb += __shfl_xor_sync(0xffffffffu, lb, 2);
    zacc += __shfl_xor_sync(0xffffffffu, zacc, 1);
    zacc += __shfl_xor_sync(0xffffffffu, zacc, 2);
    if (!head_ok) return;
    // this lane's columns are channels 16 tig + cc (c0) and 16 tig + 8 + cc (c1): block tig >> 1; its rows
    // weight block g >> 2 -> the accumulators are meaningful where the two agree
    float* wrec = p.work + (row * p.n_split + split) * (HD + 2);
    if ((tig >> 1) == lane_blk) {
        const float fix = zacc - 1024.0f * lb;
#pragma unroll
        for (int cc = 0; cc < 8; cc++) {
            wrec[2 + 16 * tig + cc] = acc[cc][0] + fix;
            wrec[2 + 16 * tig + 8 + cc] = acc[cc][1] + fix;
        }
    }
    if (g < 4 && tig == 0) { wrec[0] = m_run; wrec[1] = l_run; }
}

// merge of this path's split partials into one [m (natural log units), l, o] record per row
__global__ void merge_g32_kernel(const float* __restrict__ work, int n_split, float* __restrict__ out) {
    pdl_wait();
    const int row = blockIdx.x, d = threadIdx.x;
    const float* base = work + (size_t)row * n_split * (HD + 2);
    float mm = -CUDART_INF_F;
    for (int r = 0; r < n_split; r++)
        if (base[r * (HD + 2) + 1] > 0.0f) mm = fmaxf(mm, base[r * (HD + 2)]);
    float ll = 0.0f, a = 0.0f;
    for (int r = 0; r < n_split; r++) {
        const float l_r = base[r * (HD + 2) + 1];
        const float w = l_r > 0.0f ? fast_exp2(base[r * (HD + 2)] - mm) : 0.0f;
        ll += l_r * w;
        a = fmaf(base[r * (HD + 2) + 2 + d], w, a);
    }
    out[(size_t)row * (HD + 2) + 2 + d] = a;
    if (d == 0) { out[(size_t)row * (HD + 2)] = mm * 0.6931471805599453f; out[(size_t)row * (HD + 2) + 1] = ll; }
}

}  // namespace

bool flare_decode_g32_supported(const DecodeArgs& a, const flare_kv* kv) {
    if (a.kv.dtype != FLARE_KV_KIVI_G32 || a.kv.head_dim != 64 || a.n_q != 1 || a.kv.num_kv_heads > 8 ||
        a.num_heads / a.kv.num_kv_heads > 4 || !kv->has_g32_maps || a.slot_end >= 0 || a.want_partial)
        return false;
    // the quantised slots form a prefix only while the ring has not wrapped; and it has to be worth it
    for (int b = 0; b < kv->batch; b++)
        if (kv->length[b] + a.n_q > kv->max_seq_len) return false;
    return a.max_attend >= 1024;
}

// records [2][rows][HD + 2]: part 0 from this kernel (quantised slots), part 1 from the general kernel
// (the newest slots); the caller merges them.
int flare_launch_decode_g32_part(flare_attn_ctx* ctx, const DecodeArgs& a, const flare_kv* kv, float* part0) {
    const int nkv = a.kv.num_kv_heads, rows = a.batch * a.num_heads;
    G32Params p;
    p.q = a.q; p.attend_len = a.attend_len;
    p.k_meta = reinterpret_cast<const unsigned char*>(a.kv.plane[FLARE_PLANE_K_SCALE]);
    p.v_meta = reinterpret_cast<const unsigned char*>(a.kv.plane[FLARE_PLANE_V_SCALE]);
    p.k_meta_seq_stride = a.kv.stride[FLARE_PLANE_K_SCALE];
    p.v_meta_seq_stride = a.kv.stride[FLARE_PLANE_V_SCALE];
    p.layer_seq0 = a.layer * a.batch;
    p.num_heads = a.num_heads; p.nkv = nkv; p.G = a.num_heads / nkv;
    p.err = ctx->d_err;
    const size_t stage = 2 * (size_t)nkv * T * 16 + (size_t)nkv * HD * 4 + (size_t)T * nkv * 2 * 4;
    const size_t smem = STAGES * stage + 128;
    int n_split = (ctx->sm_count * 2) / a.batch;
    const int max_split = (a.max_attend / T + 7) / 8;
    if (n_split > max_split) n_split = max_split;
    if (n_split < 1) n_split = 1;
    if (n_split > 256) n_split = 256;
    p.n_split = n_split;
    size_t need = ((size_t)rows * n_split * (HD + 2) * sizeof(float) + 255) / 256 * 256;
    FLARE_TRY(flare_ensure(ctx, &ctx->d_work, &ctx->work_bytes, 2 * need));
    ctx->work_phase ^= 1;
    p.work = (float*)((char*)ctx->d_work + (size_t)ctx->work_phase * need);
    static bool attr_done[64] = {};
    if (!attr_done[ctx->device & 63]) {
        FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(decode_g32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)(STAGES * (2 * 8 * T * 16 + 8 * HD * 4 + T * 8 * 2 * 4) + 128)));
        attr_done[ctx->device & 63] = true;
    }
    decode_g32_kernel<<<dim3(n_split, a.batch), 32 * nkv, smem, ctx->stream>>>(kv->g32_kmap, kv->g32_vmap, p);
    FLARE_LAUNCH_CHECK(ctx);
    merge_g32_kernel<<<rows, HD, 0, ctx->stream>>>(p.work, n_split, part0);
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}
