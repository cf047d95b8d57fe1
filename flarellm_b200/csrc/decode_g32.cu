// Group-32 KIVI (2-bit) split-KV decode attention on tensor cores, for the quantised part of the
// cache (head_dim 64, up to 4 query heads per KV head, one query per sequence, ring not wrapped).
// The newest <= 127 + tile tokens (the f16 residual ring and the group that is still filling) go through
// the general kernel; the two partial results are merged by log-sum-exp.
//
// Same skeleton as the Q8_0 path: one CTA per (sequence, slot range), one warp per KV head, 32-slot
// tiles (= one key group) streamed into a ring of shared-memory stages by TMA — the 2-bit K and V codes
// as [head][slot][16 B] through tensor maps, the group's key (scale, zero) pairs and the tile's value
// (scale, zero) pairs as plain bulk copies — each stage behind an mbarrier, refilled by the last
// warp that finishes with it.
//
// Dequantisation never happens per element, and both products run "transposed" so that the codes are
// the 16-row A operand and the 8 columns carry the (at most 4) query heads.  With c the 2-bit code:
//   scores  S[t, h] = sum_ch c[t,ch] (q s)[ch,h]  +  sum_ch z[ch] q[ch,h]
//           A = codes of 16 slots, used as they are: a code masked out at bit 2k of a 16-bit half IS the f16
//           subnormal c 4^k 2^-24 (one AND per pair of codes, nothing else), the factor 4^-k goes into B and 2^24
//           into the f32 result; lane tig works on word tig of a slot's 16 code bytes, i.e. channels
//           16 tig .. 16 tig + 15,
//           B = q*s rebuilt per key group with packed f16 arithmetic as an exact hi + lo pair
//           (column 2h = hi, 2h+1 = lo; q is pre-scaled by a power of two so q*s cannot overflow);
//           the zero-point term is one more MMA whose A holds z in row 0 and whose B is q itself.
//   output  O[ch, (h, blk)] = sum_t c[t,ch] (p[t,h] s_v[t,blk])  +  sum_t p[t,h] z_v[t,blk]
//           A = V codes transposed by ldmatrix.trans (16-bit units hold 8 codes of a slot), masked the same
//           way (here 4^k 2^-24 is a factor of the output ROW and is removed once, at the end),
//           B = the f16 weights p*s_v moved into operand layout by movmatrix; column
//           2h+blk serves channel block blk; the zero-point term is one f32 scalar per (head, block).
#include "common.cuh"
#include "tma.cuh"
#include <math_constants.h>
#include <mutex>

namespace {

constexpr int T = FLARE_G32_TILE;      // slots per tile: NG key groups
constexpr int NG = T / 32;
constexpr int STAGES = FLARE_G32_TILE == 64 ? 3 : 4;
constexpr int HD = 64;
constexpr float kLog2e = 1.4426950408889634f;

struct G32Params {
    const float* q;
    float* work;
    const int* attend_len;
    const unsigned char* k_meta;     // layer base, sequence 0: [group][kv_dim] half2
    const unsigned char* v_meta;     // [slot][kv_dim/32] half2
    size_t k_meta_seq_stride, v_meta_seq_stride;   // bytes
    // for the newest tokens: code planes [slot][kv_dim/4], f16 residual rings [128][kv_dim], ring state
    const unsigned char *k_codes, *v_codes, *k_res, *v_res;
    size_t codes_seq_stride, res_seq_stride;       // bytes
    const int2* ring;
    int layer_seq0, num_heads, nkv, G, n_split, max_seq;
    int* err;
    uint32_t mask3;         // 0x00030003: a 2-bit code at bit 0 of both 16-bit halves
};

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
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
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ uint32_t hneg2(uint32_t a) {
    uint32_t d; asm("neg.f16x2 %0, %1;" : "=r"(d) : "r"(a)); return d;
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// half2 (4^-k, 4^-k), k = 0..4: the factor that a code masked out at bit 2k of a 16-bit half carries too much
// (the half then reads as the f16 subnormal code * 4^k * 2^-24).
__device__ __forceinline__ constexpr uint32_t code_mul(int k) {
    return k == 0 ? 0x3c003c00u : k == 1 ? 0x34003400u : k == 2 ? 0x2c002c00u : k == 3 ? 0x24002400u : 0x1c001c00u;
}

// Scratch of one warp for its share of the newest tokens, kept until the end of the kernel.
struct NewestScratch {
    float qo[4 * HD];      // q of the warp's (up to) 4 heads, later their unnormalised outputs
    float p[4 * 32];       // weights of the current 32-slot chunk
    float m[4], l[4];      // running maximum (log2 units) and sum per head
};

// State of the newest-token routine across chunks.
struct NewestState {
    float m[4], l[4], acc[4][2];
};

// One chunk of up to 32 slots c0 .. c0+cn-1, all served by the f16 ring (RING) or all by 2-bit codes.
// Lanes own slots for the scores, then channels 2 lane, 2 lane + 1 for the output.  Every global load of
// the chunk is issued before the first use, so that they are in flight together.
template <bool RING>
__device__ __forceinline__ void g32_newest_chunk(const G32Params& p, int b, int kvh, int lane, int c0, int cn, bool& have_q,
                                                 NewestScratch* ws, NewestState& st) {
    const int kv_dim = p.nkv * HD, G = p.G;
    float* q_s = ws->qo;
    float* p_s = ws->p;
    const int t = c0 + lane;
    const bool mine = lane < cn;
    // values
    uint32_t va[32], vb[RING ? 1 : 32];
    if (RING) {
        const unsigned char* vres = p.v_res + (size_t)b * p.res_seq_stride + (size_t)kvh * HD * 2 + lane * 4;
#pragma unroll
        for (int u = 0; u < 32; u++)
            va[u] = u < cn ? __ldg(reinterpret_cast<const uint32_t*>(vres + (size_t)((c0 + u) % FLARE_G32_RESIDUAL) * kv_dim * 2)) : 0u;
    } else {
        const unsigned char* vcod = p.v_codes + (size_t)b * p.codes_seq_stride + kvh * (HD / 4) + ((lane >> 1) & ~3);
        const unsigned char* vmeta = p.v_meta + (size_t)b * p.v_meta_seq_stride + (size_t)(kvh * (HD / 32) + (lane >> 4)) * 4;
#pragma unroll
        for (int u = 0; u < 32; u++) {
            va[u] = u < cn ? __ldg(reinterpret_cast<const uint32_t*>(vcod + (size_t)(c0 + u) * (kv_dim / 4))) : 0u;
            vb[u] = u < cn ? __ldg(reinterpret_cast<const uint32_t*>(vmeta + (size_t)(c0 + u) * (kv_dim / 32) * 4)) : 0u;
        }
    }
    // keys of this lane's slot: the f16 row, or the 16 code bytes
    uint4 w[RING ? HD / 8 : 1];
    if (RING) {
        const uint4* row = reinterpret_cast<const uint4*>(p.k_res + (size_t)b * p.res_seq_stride + ((size_t)(t % FLARE_G32_RESIDUAL) * kv_dim + kvh * HD) * 2);
#pragma unroll
        for (int c8 = 0; c8 < HD / 8; c8++) w[c8] = mine ? __ldg(row + c8) : make_uint4(0u, 0u, 0u, 0u);
    } else {
        w[0] = mine ? __ldg(reinterpret_cast<const uint4*>(p.k_codes + (size_t)b * p.codes_seq_stride + (size_t)t * (kv_dim / 4) + kvh * (HD / 4)))
                    : make_uint4(0u, 0u, 0u, 0u);
    }
    if (!have_q) {
        const float sc = rsqrtf((float)HD) * kLog2e;
        float qr[4 * HD / 32];
#pragma unroll
        for (int k = 0; k < 4 * HD / 32; k++) {
            const int i = lane + 32 * k, h = i / HD;
            qr[k] = h < G ? __ldg(p.q + ((size_t)b * p.num_heads + kvh * G + h) * HD + (i % HD)) : 0.0f;
        }
#pragma unroll
        for (int k = 0; k < 4 * HD / 32; k++) q_s[lane + 32 * k] = qr[k] * sc;
        have_q = true;
    }
    __syncwarp();                                   // q is there; the previous chunk's weights have been consumed
    // ---- scores ----------------------------------------------------------------------------------------
    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (RING) {
#pragma unroll
        for (int c8 = 0; c8 < HD / 8; c8++) {
            const __half2* h2 = reinterpret_cast<const __half2*>(&w[c8]);
            float k[8];
#pragma unroll
            for (int j = 0; j < 4; j++) { const float2 f = __half22float2(h2[j]); k[2 * j] = f.x; k[2 * j + 1] = f.y; }
#pragma unroll
            for (int h = 0; h < 4; h++)
#pragma unroll
                for (int j = 0; j < 8; j++) s[h] = fmaf(q_s[h * HD + c8 * 8 + j], k[j], s[h]);
        }
    } else if (mine) {
        const uint32_t w4[4] = {w[0].x, w[0].y, w[0].z, w[0].w};
        // the group's metadata: per 16-channel block 16 scales then 16 zero points, pair (r, r+8) adjacent
        const uint4* mrow = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.k_meta + (size_t)b * p.k_meta_seq_stride) +
                                                           (size_t)(t >> 5) * kv_dim * 2 + (size_t)kvh * (HD / 16) * 32);
#pragma unroll
        for (int wi = 0; wi < 4; wi++) {
            const uint4 m4[4] = {__ldg(mrow + 4 * wi), __ldg(mrow + 4 * wi + 1), __ldg(mrow + 4 * wi + 2), __ldg(mrow + 4 * wi + 3)};
            const __half2* sp = reinterpret_cast<const __half2*>(&m4[0]);
            const __half2* zp = reinterpret_cast<const __half2*>(&m4[2]);
#pragma unroll
            for (int r = 0; r < 8; r++) {
                const float2 sf = __half22float2(sp[r]), zf = __half22float2(zp[r]);
                const float k0 = q2_dequant((float)((w4[wi] >> (2 * r)) & 3u), sf.x, zf.x);            // channel r
                const float k1 = q2_dequant((float)((w4[wi] >> (2 * r + 16)) & 3u), sf.y, zf.y);       // channel r + 8
#pragma unroll
                for (int h = 0; h < 4; h++)
                    s[h] = fmaf(q_s[h * HD + wi * 16 + r + 8], k1, fmaf(q_s[h * HD + wi * 16 + r], k0, s[h]));
            }
        }
    }
    // ---- online softmax over the chunk -------------------------------------------------------------
#pragma unroll
    for (int h = 0; h < 4; h++) {
        float v = mine ? s[h] : -CUDART_INF_F, cm = v;
#pragma unroll
        for (int o = 16; o; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
        const float m_new = fmaxf(st.m[h], cm);     // finite: the chunk is not empty
        const float alpha = fast_exp2(st.m[h] - m_new);
        const float e = mine ? fast_exp2(v - m_new) : 0.0f;
        float sum = e;
#pragma unroll
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        p_s[h * 32 + lane] = e;
        st.l[h] = st.l[h] * alpha + sum;
        st.acc[h][0] *= alpha; st.acc[h][1] *= alpha;
        st.m[h] = m_new;
    }
    __syncwarp();
    // ---- output --------------------------------------------------------------------------------------
#pragma unroll
    for (int u = 0; u < 32; u++) {
        float v0, v1;
        if (RING) {
            const float2 fr = __half22float2(*reinterpret_cast<const __half2*>(&va[u]));
            v0 = fr.x; v1 = fr.y;
        } else {
            const float2 mz = __half22float2(*reinterpret_cast<const __half2*>(&vb[u]));
            const uint32_t byte = va[u] >> (((lane >> 1) & 3) * 8);
            v0 = q2_dequant((float)((byte >> ((lane & 1) * 4)) & 3u), mz.x, mz.y);
            v1 = q2_dequant((float)((byte >> ((lane & 1) * 4 + 2)) & 3u), mz.x, mz.y);
        }
#pragma unroll
        for (int h = 0; h < 4; h++) {
            const float wgt = p_s[h * 32 + u];       // 0 beyond the chunk
            st.acc[h][0] = fmaf(wgt, v0, st.acc[h][0]);
            st.acc[h][1] = fmaf(wgt, v1, st.acc[h][1]);
        }
    }
}

// The slots of a sequence that the group-aligned tile loop does not cover: up to two runs of 2-bit codes
// [a0, a1) and [b0, b1) (physical slots: tokens that have left the residual ring but share a tile with ring
// tokens) and the run [r0, r1) served by the f16 ring (slot indices that are only ever used modulo 128, so a
// run that crosses the end of a wrapped ring needs no special case).  One warp per KV head on CUDA cores, 32
// slots at a time with an online softmax.  Leaves (m, l, o) per head in `ws`.
__device__ __noinline__ void g32_newest_tokens(const G32Params& p, int b, int kvh, int lane, int a0, int a1, int b0, int b1,
                                               int r0, int r1, NewestScratch* ws) {
    NewestState st;
#pragma unroll
    for (int h = 0; h < 4; h++) { st.m[h] = -CUDART_INF_F; st.l[h] = 0.0f; st.acc[h][0] = st.acc[h][1] = 0.0f; }
    bool have_q = false;
    for (int c0 = a0; c0 < a1; c0 += 32) g32_newest_chunk<false>(p, b, kvh, lane, c0, min(32, a1 - c0), have_q, ws, st);
    for (int c0 = b0; c0 < b1; c0 += 32) g32_newest_chunk<false>(p, b, kvh, lane, c0, min(32, b1 - c0), have_q, ws, st);
    for (int c0 = r0; c0 < r1; c0 += 32) g32_newest_chunk<true>(p, b, kvh, lane, c0, min(32, r1 - c0), have_q, ws, st);
    __syncwarp();                                       // q is dead: its place takes the outputs
#pragma unroll
    for (int h = 0; h < 4; h++) {
        *reinterpret_cast<float2*>(ws->qo + h * HD + 2 * lane) = make_float2(st.acc[h][0], st.acc[h][1]);
        if (lane == 0) { ws->m[h] = st.m[h]; ws->l[h] = st.l[h]; }
    }
    __syncwarp();
}

// WRAP: some sequence of the batch has a wrapped ring (the instantiation without it carries no ring arithmetic
// through the tile loop).
template <bool WRAP>
__global__ void __launch_bounds__(256, 2) decode_g32_kernel(const __grid_constant__ CUtensorMap kmap,
                                                            const __grid_constant__ CUtensorMap vmap, G32Params p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ uint64_t full_bar[STAGES];
    __shared__ int done_cnt[STAGES];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int split = blockIdx.x, b = blockIdx.y;
    const int nkv = p.nkv, kvh = warp;
    const int kv_dim = nkv * HD;
    // stage: K codes [nkv][T][16], V codes [nkv][T][16], K meta of NG groups [NG][kv_dim] x 4 B, V meta [T][nkv*2] half2
    const int codes = nkv * T * 16;
    const int kmeta_bytes = NG * kv_dim * 4, vmeta_bytes = T * nkv * 2 * 4;
    const int stage_bytes = 2 * codes + kmeta_bytes + vmeta_bytes;
    unsigned char* sbase = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

    // Which slots go through the tile loop (2-bit codes only, whole tiles) and which through the newest-token
    // routine.  Ring not wrapped: slot = token index; tiles 0 .. (n - 128) / T - 1 are all codes, the rest of the
    // n attended slots ends with the <= 128 tokens that the f16 ring serves.  Ring wrapped (every slot holds a
    // token, the newest one in slot ring.x): the 128 ring tokens are the slots ring.x - 127 .. ring.x cyclically;
    // the two or three tiles they touch go to the newest-token routine — ring tokens, the older codes before them
    // in their first tile, and the OLDEST codes after ring.x in its tile — and the tile loop walks the remaining
    // tiles starting behind that window.
    const int n = p.attend_len[b];
    const int2 ring = p.ring[b];
    const int TT = p.max_seq / T;
    const bool wrapped = WRAP && ring.y >= p.max_seq;
    int lim_tiles, tile0;              // tiles of the tile loop; the first one of them (physical)
    if (!wrapped) {
        lim_tiles = n > 128 ? (n - 128) / T : 0;
        tile0 = 0;
    } else {
        const int w0 = (ring.x - (FLARE_G32_RESIDUAL - 1) + p.max_seq) % p.max_seq;
        const int tile_sn = ring.x / T;
        lim_tiles = TT - (((tile_sn - w0 / T + TT) % TT) + 1);  // all but the tiles touched by the ring window
        tile0 = (tile_sn + 1) % TT;
    }
    if (split == p.n_split) {            // the CTA of the newest tokens: one more record per row
        int ca0, ca1, cb0, cb1, rr0, rr1;
        if (!wrapped) {
            int t_ring = ring.x - (FLARE_G32_RESIDUAL - 1);          // first slot that the ring serves
            t_ring = t_ring < lim_tiles * T ? lim_tiles * T : (t_ring > n ? n : t_ring);
            ca0 = lim_tiles * T; ca1 = t_ring; cb0 = cb1 = 0; rr0 = t_ring; rr1 = n;
        } else {
            const int s_n = ring.x, w0 = (s_n - (FLARE_G32_RESIDUAL - 1) + p.max_seq) % p.max_seq;
            ca0 = (w0 / T) * T; ca1 = w0; cb0 = s_n + 1; cb1 = (s_n / T + 1) * T; rr0 = w0; rr1 = w0 + FLARE_G32_RESIDUAL;
        }
        pdl_trigger();
        pdl_wait();
        NewestScratch* ws = reinterpret_cast<NewestScratch*>(sbase) + warp;
        g32_newest_tokens(p, b, kvh, lane, ca0, ca1, cb0, cb1, rr0, rr1, ws);
        for (int h = 0; h < p.G; h++) {
            const size_t row = (size_t)b * p.num_heads + kvh * p.G + h;
            float* wrec = p.work + (row * (p.n_split + 1) + split) * (HD + 2);
            *reinterpret_cast<float2*>(wrec + 2 + 2 * lane) = *reinterpret_cast<const float2*>(ws->qo + h * HD + 2 * lane);
            if (lane == 0) { wrec[0] = ws->l[h] > 0.0f ? ws->m[h] : 0.0f; wrec[1] = ws->l[h]; }
        }
        return;
    }
    const int t_begin = tile0 + (int)(((long long)split * lim_tiles) / p.n_split);     // may run past TT: wrapped below
    const int n_tiles = (int)(((long long)(split + 1) * lim_tiles) / p.n_split) - (int)(((long long)split * lim_tiles) / p.n_split);

    const unsigned char* kmg = p.k_meta + (size_t)b * p.k_meta_seq_stride;
    const unsigned char* vmg = p.v_meta + (size_t)b * p.v_meta_seq_stride;
    auto issue = [&](int i) {
        const int s = i % STAGES;
        unsigned char* st = sbase + (size_t)s * stage_bytes;
        int tile = t_begin + i;                             // physical tile: the walk starts behind the ring window
        if (WRAP && tile >= TT) tile -= TT;
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
    pdl_trigger();          // the next kernel may be scheduled: its CTAs take the places this grid's CTAs leave
    pdl_wait();

    // ---- the q side (B operand, column g): head g >> 1, hi part in even columns, lo part in odd ones.
    //      Lane tig owns channels 16 tig .. 16 tig + 15 (one 32-bit code word of a slot).  In k-step ks its
    //      logical k (2tig, 2tig+1 | 2tig+8, 2tig+9) are channels 16 tig + (ks, ks+8 | ks+4, ks+12): two codes
    //      16 bits apart in the word pair up, at bit 2 ks of the word or of the word shifted down by 8.
    const int hB = g >> 1;
    const bool lo_col = g & 1;
    uint32_t qx[4][2], qhz[4][2];          // qx: this column's part of q (hi or lo); qhz: hi part in lo columns, else 0
    float unscale, unscale24;              // 2^e that undoes the power-of-two pre-scaling of head `tig`; 2^(e + 24)
    {
        const bool ok = hB < p.G;
        const float* qrow = p.q + ((size_t)b * p.num_heads + kvh * p.G + (ok ? hB : 0)) * HD + 16 * tig;
        const float sc = rsqrtf((float)HD) * kLog2e;
        float qv[16], mx = 0.0f;
#pragma unroll
        for (int r = 0; r < 16; r++) {
            qv[r] = ok ? __ldg(qrow + r) * sc : 0.0f;
            mx = fmaxf(mx, fabsf(qv[r]));
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        // |q| * 2^-e <= 1/2, so q*s stays below the f16 maximum for every f16 scale
        int e = (mx > 0.0f && mx < CUDART_INF_F) ? ilogbf(mx) + 2 : 0;
        e = max(-100, min(100, e));
        const float down = exp2f((float)-e);
        const float up = exp2f((float)e);
        unscale = __shfl_sync(0xffffffffu, up, 8 * tig);          // lane with g = 2 tig holds head tig
        unscale24 = unscale * 16777216.0f;                        // and the 2^24 of the subnormal codes
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
#pragma unroll
            for (int bb = 0; bb < 2; bb++) {
                const float x0 = qv[ks + 4 * bb] * down, x1 = qv[ks + 4 * bb + 8] * down;
                const uint32_t h = pack_half2(x0, x1);
                const float2 hf = unpack_half2(h);
                const uint32_t l = pack_half2(x0 - hf.x, x1 - hf.y);
                qx[ks][bb] = lo_col ? l : h;
                qhz[ks][bb] = lo_col ? h : 0u;
            }
    }
    uint32_t cmask[5];                                             // a code at bit 0, 2, 4, 6, 8 of both halves
#pragma unroll
    for (int k = 0; k < 5; k++) cmask[k] = p.mask3 << (2 * k);

    float acc[4][4];                      // m-tile j: rows g, g+8 <-> channels 8g + 2j, 8g + 2j + 1; columns (head tig, blk 0 | 1)
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
        for (int k = 0; k < 4; k++) acc[j][k] = 0.0f;
    float m_run = -CUDART_INF_F, l_run = 0.0f, zacc0 = 0.0f, zacc1 = 0.0f;

    bool failed = false;
    for (int i = 0; i < n_tiles; i++) {
        const int s = i % STAGES;
        if (!ptx::mbar_wait(&full_bar[s], (uint32_t)((i / STAGES) & 1))) { failed = true; break; }
        const unsigned char* st = sbase + (size_t)s * stage_bytes;
        const unsigned char* kc = st + kvh * (T * 16);
        const uint32_t vc = ptx::smem_u32(st + codes + kvh * (T * 16));
        const unsigned char* kmeta0 = st + 2 * codes + (kvh * 4 + tig) * 64;                        // 16 scales, 16 zeros
        const uint2* vmeta = reinterpret_cast<const uint2*>(st + 2 * codes + kmeta_bytes) + kvh;

        float sc[4 * NG];                                   // sc[r]: slot 8 r + g of the tile, head tig
#pragma unroll
        for (int gi = 0; gi < NG; gi++) {
            // ---- B = (q s) hi/lo for this group; the zero-point term as row 0 of one more product ---------
            const uint4* kmeta = reinterpret_cast<const uint4*>(kmeta0 + FLARE_CK(gi * (kmeta_bytes / NG), 64, kmeta_bytes - (kvh * 4 + tig) * 64, p.err));
            uint32_t bq[4][2];
            float dz[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            {
                const uint4 sa = kmeta[0], sb = kmeta[1];
                uint4 za = make_uint4(0u, 0u, 0u, 0u), zb = za;
                if (g == 0) { za = kmeta[2]; zb = kmeta[3]; }
                const uint32_t s2[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};     // pair p: channels (p, p + 8)
                const uint32_t z2[8] = {za.x, za.y, za.z, za.w, zb.x, zb.y, zb.z, zb.w};
#pragma unroll
                for (int ks = 0; ks < 4; ks++) {
#pragma unroll
                    for (int bb = 0; bb < 2; bb++) {
                        // the scale of the pair, times the 4^-ks that the masked codes of k-step ks carry too much
                        const uint32_t sv = ks == 0 ? s2[4 * bb] : hmul2(s2[ks + 4 * bb], code_mul(ks));
                        const uint32_t ph = hmul2(qhz[ks][bb], sv);                  // lo columns: rounded hi product
                        const uint32_t er = hfma2(qhz[ks][bb], sv, hneg2(ph));       //             its exact rounding error
                        bq[ks][bb] = hfma2(qx[ks][bb], sv, er);                      // hi columns: round(q_hi s); lo: q_lo s + error
                    }
                    mma_f16(dz, z2[ks], 0u, z2[ks + 4], 0u, qx[ks][0], qx[ks][1]);
                }
            }
            const float zdu = __shfl_sync(0xffffffffu, dz[0] + dz[1], tig) * unscale;   // row 0 lives in lanes g = 0

            // ---- scores of slots 32 gi + 16 mt + g and + 8 for head tig -----------------------------------
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const uint32_t wa = *reinterpret_cast<const uint32_t*>(kc + FLARE_CK((32 * gi + 16 * mt + g) * 16 + 4 * tig, 4, T * 16, p.err));
                const uint32_t wb = *reinterpret_cast<const uint32_t*>(kc + FLARE_CK((32 * gi + 16 * mt + 8 + g) * 16 + 4 * tig, 4, T * 16, p.err));
                const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
                float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int ks = 0; ks < 4; ks++) {
                    // a code at bit 2 ks of a half, alone in the word, reads as the subnormal code * 4^ks * 2^-24
                    mma_f16(d, wa & cmask[ks], wb & cmask[ks], wa8 & cmask[ks], wb8 & cmask[ks], bq[ks][0], bq[ks][1]);
                }
                sc[4 * gi + 2 * mt] = fmaf(d[0] + d[1], unscale24, zdu);
                sc[4 * gi + 2 * mt + 1] = fmaf(d[2] + d[3], unscale24, zdu);
            }
        }
        float tmax = sc[0];
#pragma unroll
        for (int r = 1; r < 4 * NG; r++) tmax = fmaxf(tmax, sc[r]);
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
        const bool bump = tmax > m_run + 8.0f;
        if (__any_sync(0xffffffffu, bump)) {
            const float alpha = bump ? fast_exp2(m_run - tmax) : 1.0f;
            if (bump) m_run = tmax;
            l_run *= alpha; zacc0 *= alpha; zacc1 *= alpha;
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int k = 0; k < 4; k++) acc[j][k] *= alpha;
        }
        // ---- weights p * s_v[t, blk] as f16 (column 2 tig + blk of the 8x8 slot-by-column matrices) ----
        uint32_t bp[4 * NG];
#pragma unroll
        for (int r = 0; r < 4 * NG; r++) {                  // slot 8 r + g
            const float pr = fast_exp2(sc[r] - m_run);
            l_run += pr;
            const uint2 mv = vmeta[FLARE_CK((8 * r + g) * nkv, 1, T * nkv - kvh, p.err)];   // (scale, zero) of blocks 0 and 1
            const float2 m0 = unpack_half2(mv.x), m1 = unpack_half2(mv.y);
            zacc0 = fmaf(pr, m0.y, zacc0);
            zacc1 = fmaf(pr, m1.y, zacc1);
            bp[r] = movmatrix_trans(pack_half2(pr * m0.x, pr * m1.x));
        }
        // ---- output ----------------------------------------------------------------------------------------
#pragma unroll
        for (int gi = 0; gi < NG; gi++) {
            uint32_t rr[4];
            // matrix m = slots 32 gi + 8m .. +7, 16 bytes (64 codes) per slot
            ldmatrix_x4_trans(rr, vc + FLARE_CK(gi * 512 + lane * 16, 16, T * 16, p.err));
#pragma unroll
            for (int kstep = 0; kstep < 2; kstep++) {
                const uint32_t r0 = rr[2 * kstep], r1 = rr[2 * kstep + 1];
                const uint32_t r0s = r0 >> 6, r1s = r1 >> 6;
                const uint32_t b0 = bp[4 * gi + 2 * kstep], b1 = bp[4 * gi + 2 * kstep + 1];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    // channel 8g + c: its code sits at bit 2c of the 16-bit unit, or at bit 2c - 6 after the shift
                    const int c0 = 2 * j, c1 = 2 * j + 1;
                    const int k0 = c0 <= 4 ? c0 : c0 - 3, k1 = c1 <= 4 ? c1 : c1 - 3;
                    const uint32_t a0 = (c0 <= 4 ? r0 : r0s) & cmask[k0];
                    const uint32_t a1 = (c1 <= 4 ? r0 : r0s) & cmask[k1];
                    const uint32_t a2 = (c0 <= 4 ? r1 : r1s) & cmask[k0];
                    const uint32_t a3 = (c1 <= 4 ? r1 : r1s) & cmask[k1];
                    mma_f16(acc[j], a0, a1, a2, a3, b0, b1);
                }
            }
        }

        __syncwarp();
        if (lane == 0 && i + STAGES < n_tiles) {
            if (atomicAdd(&done_cnt[s], 1) == nkv - 1) {
                done_cnt[s] = 0;
                ptx::fence_proxy_async();
                issue(i + STAGES);
            }
        }
    }
    if (failed) {
        if (lane == 0) flare_report(p.err, FLARE_ERR_TIMEOUT);
        return;
    }
#pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
        l_run += __shfl_xor_sync(0xffffffffu, l_run, o);
        zacc0 += __shfl_xor_sync(0xffffffffu, zacc0, o);
        zacc1 += __shfl_xor_sync(0xffffffffu, zacc1, o);
    }
    const int blk = g >> 2;                                            // channels 8g .. 8g+7 lie in block g >> 2
    if (tig >= p.G) return;
    const float zp = blk ? zacc1 : zacc0;
    const size_t row = (size_t)b * p.num_heads + kvh * p.G + tig;
    float* wrec = p.work + (row * (p.n_split + 1) + split) * (HD + 2);
    float o8[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        // rows g / g + 8 of m-tile j used the codes at position k0 / k1: remove 4^k 2^-24
        const int c0 = 2 * j, c1 = 2 * j + 1;
        const int k0 = c0 <= 4 ? c0 : c0 - 3, k1 = c1 <= 4 ? c1 : c1 - 3;
        o8[2 * j] = fmaf(blk ? acc[j][1] : acc[j][0], 16777216.0f / (float)(1 << (2 * k0)), zp);
        o8[2 * j + 1] = fmaf(blk ? acc[j][3] : acc[j][2], 16777216.0f / (float)(1 << (2 * k1)), zp);
    }
#pragma unroll
    for (int k = 0; k < 8; k++) wrec[2 + 8 * g + k] = o8[k];
    if (g == 0) { wrec[0] = m_run; wrec[1] = l_run; }
}

}  // namespace

bool flare_decode_g32_supported(const DecodeArgs& a, const flare_kv* kv) {
    if (a.kv.dtype != FLARE_KV_KIVI_G32 || a.kv.head_dim != 64 || a.n_q != 1 || a.kv.num_kv_heads > 8 ||
        a.num_heads / a.kv.num_kv_heads > 4 || !kv->has_g32_maps || a.slot_end >= 0 || a.want_partial || a.window > 0)
        return false;
    // a wrapped ring is served when the whole ring is attended (what the ring state gives once it is full)
    for (int b = 0; b < kv->batch; b++)
        if (kv->length[b] >= kv->max_seq_len && (!a.h_attend || a.h_attend[b] != kv->max_seq_len)) return false;
    // and it has to be worth it
    return a.max_attend >= 1024;
}

// One CTA per (sequence, slot range of the quantised prefix) plus one per sequence for the newest tokens,
// then the merge of their records into a.out (the kernel shared with the other split paths, multi.cu).
int flare_launch_decode_g32(flare_attn_ctx* ctx, const DecodeArgs& a, const flare_kv* kv) {
    const int nkv = a.kv.num_kv_heads, rows = a.batch * a.num_heads;
    G32Params p;
    p.q = a.q; p.attend_len = a.attend_len; p.ring = a.ring;
    p.k_meta = reinterpret_cast<const unsigned char*>(a.kv.plane[FLARE_PLANE_K_SCALE]);
    p.v_meta = reinterpret_cast<const unsigned char*>(a.kv.plane[FLARE_PLANE_V_SCALE]);
    p.k_meta_seq_stride = a.kv.stride[FLARE_PLANE_K_SCALE];
    p.v_meta_seq_stride = a.kv.stride[FLARE_PLANE_V_SCALE];
    p.k_codes = reinterpret_cast<const unsigned char*>(a.kv.plane[FLARE_PLANE_K_Q]);
    p.v_codes = reinterpret_cast<const unsigned char*>(a.kv.plane[FLARE_PLANE_V_Q]);
    p.codes_seq_stride = a.kv.stride[FLARE_PLANE_K_Q];
    p.k_res = reinterpret_cast<const unsigned char*>(a.kv.plane[FLARE_PLANE_K_RES]);
    p.v_res = reinterpret_cast<const unsigned char*>(a.kv.plane[FLARE_PLANE_V_RES]);
    p.res_seq_stride = a.kv.stride[FLARE_PLANE_K_RES];
    p.layer_seq0 = a.layer * a.batch;
    p.num_heads = a.num_heads; p.nkv = nkv; p.G = a.num_heads / nkv; p.max_seq = a.kv.max_seq_len;
    p.err = ctx->d_err;
    p.mask3 = 0x00030003u;
    const size_t stage = 2 * (size_t)nkv * T * 16 + (size_t)NG * nkv * HD * 4 + (size_t)T * nkv * 2 * 4;
    size_t smem = STAGES * stage + 128;
    if (smem < (size_t)nkv * sizeof(NewestScratch) + 128) smem = (size_t)nkv * sizeof(NewestScratch) + 128;
    // all CTAs resident at once (two per SM): n_split slot ranges and one newest-token CTA per sequence
    int n_split = (ctx->sm_count * 2) / a.batch - 1;
    const int max_split = (a.max_attend / T + 7) / 8;
    if (n_split > max_split) n_split = max_split;
    if (n_split < 1) n_split = 1;
    if (n_split > 255) n_split = 255;
    p.n_split = n_split;
    size_t need = ((size_t)rows * (n_split + 1) * (HD + 2) * sizeof(float) + 255) / 256 * 256;
    FLARE_TRY(flare_ensure(ctx, &ctx->d_work, &ctx->work_bytes, 2 * need));
    ctx->work_phase ^= 1;
    p.work = (float*)((char*)ctx->d_work + (size_t)ctx->work_phase * need);
    {
        static std::mutex attr_mutex;          // two contexts on two host threads may get here at once
        std::lock_guard<std::mutex> lock(attr_mutex);
        static bool attr_done[64] = {};
        if (!attr_done[ctx->device & 63]) {
            const int max_smem = (int)(STAGES * (2 * 8 * T * 16 + NG * 8 * HD * 4 + T * 8 * 2 * 4) + 128);
            FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(decode_g32_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
            FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(decode_g32_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
            attr_done[ctx->device & 63] = true;
        }
    }
    // Programmatic dependent launch as in the Q8_0 path: after one of this library's own attention kernels
    // (which never write the cache) the next one may start early; both wait before touching q or records.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_split + 1, a.batch);
    cfg.blockDim = dim3(32 * nkv);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->last_launch_overlappable ? 1 : 0;
    bool any_wrapped = false;
    for (int b = 0; b < kv->batch; b++) any_wrapped = any_wrapped || kv->length[b] >= kv->max_seq_len;
    if (any_wrapped) FLARE_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, decode_g32_kernel<true>, kv->g32_kmap, kv->g32_vmap, p));
    else FLARE_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, decode_g32_kernel<false>, kv->g32_kmap, kv->g32_vmap, p));
    FLARE_LAUNCH_CHECK(ctx);
    // log-sum-exp merge of the slot ranges and the newest-token record, chained with programmatic dependent launch
    FLARE_TRY(flare_launch_merge_splits(ctx, p.work, n_split + 1, rows, HD, a.out, 0));
    ctx->last_launch_overlappable = true;
    return FLARE_OK;
}
