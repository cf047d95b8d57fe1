// Split-KV GQA decode attention over the ring-buffer cache, all cache formats, dequantised
// in the kernel.  This is the general CUDA-core path: every (kv head, group of <= 4 query
// heads, query, slot range) is one CTA that streams its K and V rows exactly once and keeps
// the running (max, sum, output) of flare-core's online softmax
// (flare-core/src/model.rs:9914-9966) in registers; ranges are combined by log-sum-exp.
//
// Work split inside a CTA (128 threads): a group of TPS = head_dim/8 lanes owns one slot at
// a time, each lane 8 consecutive channels of it, so a row is read with 16/32-byte vector
// loads; the 32/TPS lane groups of the 4 warps take interleaved slots and hold independent
// softmax states that are combined once at the end (shuffles, then shared memory).
#include "common.cuh"
#include <algorithm>
#include <math_constants.h>
#include <mutex>

namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct SeqKv {
    const char* p[FLARE_PLANE_COUNT];
    int max_seq, kv_dim, position, length, newest;
};

// ---- row loaders: channels [c0, c0+8) of ring slot `slot`, as the reference dequantises them
template <int DT, bool IS_V> struct Row;

template <bool IS_V> struct Row<FLARE_KV_F32, IS_V> {
    static __device__ __forceinline__ void load8(const SeqKv& s, int slot, int c0, float* o) {
        const float4* r = reinterpret_cast<const float4*>(s.p[IS_V ? FLARE_PLANE_V : FLARE_PLANE_K]) +
                          ((size_t)slot * s.kv_dim + c0) / 4;
        float4 a = __ldg(r), b = __ldg(r + 1);
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    }
};

template <bool IS_V> struct Row<FLARE_KV_Q8_0, IS_V> {
    static __device__ __forceinline__ void load8(const SeqKv& s, int slot, int c0, float* o) {
        const char* qp = s.p[IS_V ? FLARE_PLANE_V_Q : FLARE_PLANE_K_Q] + (size_t)slot * s.kv_dim + c0;
        int2 raw = __ldg(reinterpret_cast<const int2*>(qp));
        const __half* sp = reinterpret_cast<const __half*>(s.p[IS_V ? FLARE_PLANE_V_SCALE : FLARE_PLANE_K_SCALE]) +
                           (size_t)slot * (s.kv_dim / 32) + c0 / 32;
        float sc = __half2float(__ldg(sp));
        // (i8 as f32) * scale, one multiply (flare-loader/src/quantize.rs:188-197)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            o[i] = (float)(int8_t)((raw.x >> (8 * i)) & 0xFF) * sc;
            o[4 + i] = (float)(int8_t)((raw.y >> (8 * i)) & 0xFF) * sc;
        }
    }
};

// flare-core QuantizedKvCache::dequant_keys / dequant_values (kv_cache.rs:189-250) seen
// from a ring slot, including what the decode step observes between write and advance.
template <bool IS_V> struct Row<FLARE_KV_KIVI_REF, IS_V> {
    static __device__ __forceinline__ void load8(const SeqKv& s, int slot, int c0, float* o) {
        int R = s.max_seq < FLARE_REF_RESIDUAL ? s.max_seq : FLARE_REF_RESIDUAL;
        int t;
        if (s.length < s.max_seq) {
            if (slot >= s.length) {   // not yet part of the cache: dequant_* leaves zeros there
#pragma unroll
                for (int i = 0; i < 8; i++) o[i] = 0.0f;
                return;
            }
            t = slot;
        } else {
            t = slot - s.position;
            if (t < 0) t += s.max_seq;
        }
        bool in_res = (s.length <= R) || (t >= s.length - R);
        if (in_res) {
            const float* r = reinterpret_cast<const float*>(s.p[IS_V ? FLARE_PLANE_V_RES : FLARE_PLANE_K_RES]) +
                             (size_t)(slot % R) * s.kv_dim + c0;
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] = __ldg(r + i);
            return;
        }
        int ppt = s.kv_dim / 4;
        const uint8_t* pk = reinterpret_cast<const uint8_t*>(s.p[IS_V ? FLARE_PLANE_V_Q : FLARE_PLANE_K_Q]) +
                            (size_t)slot * ppt;
        if (IS_V) {
            float sc = __ldg(reinterpret_cast<const float*>(s.p[FLARE_PLANE_V_SCALE]) + slot);
            float mn = __ldg(reinterpret_cast<const float*>(s.p[FLARE_PLANE_V_MIN]) + slot);
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] = q2_dequant(q2_code(pk, c0 + i), sc, mn);
        } else {
            const float* sc = reinterpret_cast<const float*>(s.p[FLARE_PLANE_K_SCALE]) + c0;
            const float* mn = reinterpret_cast<const float*>(s.p[FLARE_PLANE_K_MIN]) + c0;
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] = q2_dequant(q2_code(pk, c0 + i), __ldg(sc + i), __ldg(mn + i));
        }
    }
};

template <bool IS_V> struct Row<FLARE_KV_KIVI_G32, IS_V> {
    static __device__ __forceinline__ void load8(const SeqKv& s, int slot, int c0, float* o) {
        int age = s.newest - slot;
        if (age < 0) age += s.max_seq;
        if (age < FLARE_G32_RESIDUAL) {
            const uint4* r = reinterpret_cast<const uint4*>(
                s.p[IS_V ? FLARE_PLANE_V_RES : FLARE_PLANE_K_RES] +
                ((size_t)(slot % FLARE_G32_RESIDUAL) * s.kv_dim + c0) * 2);
            uint4 w = __ldg(r);
            const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 f = __half22float2(h[i]);
                o[2 * i] = f.x; o[2 * i + 1] = f.y;
            }
            return;
        }
        if (IS_V) {
            const uint16_t* cp = reinterpret_cast<const uint16_t*>(s.p[FLARE_PLANE_V_Q] + (size_t)slot * (s.kv_dim / 4) + c0 / 4);
            uint32_t w = __ldg(cp);
            const __half2* mp = reinterpret_cast<const __half2*>(s.p[FLARE_PLANE_V_SCALE]) +
                                (size_t)slot * (s.kv_dim / 32) + c0 / 32;
            float2 m = __half22float2(__ldg(mp));
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] = q2_dequant((float)((w >> (2 * i)) & 3), m.x, m.y);
        } else {
            const int grp = slot >> 5;
            const uint16_t* cp = reinterpret_cast<const uint16_t*>(s.p[FLARE_PLANE_K_Q] + (size_t)slot * (s.kv_dim / 4) + c0 / 4);
            const uint32_t w = __ldg(cp);
            // channels c0 .. c0+7 are the even (or, for the upper 8 of a 16-block, odd) f16 entries of the
            // block's 16 scales and 16 zero points: 64 contiguous bytes
            const uint4* mp = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(s.p[FLARE_PLANE_K_SCALE]) +
                                                             (size_t)grp * s.kv_dim * 2 + (c0 >> 4) * 32);
            const uint4 s0 = __ldg(mp), s1 = __ldg(mp + 1), z0 = __ldg(mp + 2), z1 = __ldg(mp + 3);
            const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            const uint32_t zw[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
            const bool upper = (c0 >> 3) & 1;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sw[i]));
                const float2 zf = __half22float2(*reinterpret_cast<const __half2*>(&zw[i]));
                o[i] = q2_dequant((float)((w >> (2 * i)) & 3), upper ? sf.y : sf.x, upper ? zf.y : zf.x);
            }
        }
    }
};

constexpr long long kMaxGridZ = 65535;

struct DecodeParams {
    KvLayerView kv;
    const float* q;
    float* out;        // final output (n_split == 1 and !want_partial) ...
    float* work;       // ... else partials [row][n_split][hd+2], m in log2 units
    const int* attend_len;
    const int2* ring;
    int n_q, num_heads, n_chunks, slot_begin, slot_end, want_partial, range_max, causal_q, window;
    int bq0;           // (sequence, query) index of blockIdx.z == 0: more than 65535 of them take several launches
};

__device__ __forceinline__ SeqKv seq_view(const DecodeParams& p, int b, int n_q) {
    SeqKv s;
#pragma unroll
    for (int i = 0; i < FLARE_PLANE_COUNT; i++) s.p[i] = p.kv.plane[i] ? p.kv.plane[i] + (size_t)b * p.kv.stride[i] : nullptr;
    s.max_seq = p.kv.max_seq_len;
    s.kv_dim = p.kv.kv_dim;
    int2 r = p.ring[b];
    s.position = r.x;
    s.length = r.y;
    s.newest = (r.x + n_q - 1) % s.max_seq;
    return s;
}

template <int DT, int TPS, int GC>
__global__ void __launch_bounds__(128) decode_splitkv_kernel(DecodeParams p) {
    constexpr int HD = TPS * 8;
    constexpr int SPW = 32 / TPS;           // slots per warp per iteration
    const int split = blockIdx.x, n_split = gridDim.x;
    const int kvh = blockIdx.y / p.n_chunks, chunk = blockIdx.y % p.n_chunks;
    const int bq = p.bq0 + (int)blockIdx.z;
    const int b = bq / p.n_q, qi = bq % p.n_q;
    const int G = p.num_heads / p.kv.num_kv_heads;
    const int h0 = kvh * G + chunk * GC;
    const int heads_here = min(GC, G - chunk * GC);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / TPS, cl = lane % TPS;
    const int c0 = kvh * HD + cl * 8;

    const SeqKv s = seq_view(p, b, p.n_q);
    int n = p.attend_len[b] - (p.causal_q ? (p.n_q - 1 - qi) : 0);
    int lo = 0, hi = n;
    if (p.window > 0) lo = max(lo, n - p.window);
    if (p.slot_end >= 0) { lo = max(lo, p.slot_begin); hi = min(hi, p.slot_end); }
    const int base = p.slot_end >= 0 ? p.slot_begin : 0;
    const int per = (p.range_max + n_split - 1) / n_split;
    const int s0 = max(lo, base + split * per);
    const int s1 = min(hi, base + (split + 1) * per);

    const float scale_log2 = rsqrtf((float)HD) * kLog2e;
    float q[GC][8], o[GC][8], m[GC], l[GC];
    const size_t row0 = ((size_t)b * p.n_q + qi) * p.num_heads;
#pragma unroll
    for (int g = 0; g < GC; g++) {
        m[g] = -CUDART_INF_F;
        l[g] = 0.0f;
        const float* qp = p.q + (row0 + h0 + (g < heads_here ? g : 0)) * HD + cl * 8;
#pragma unroll
        for (int i = 0; i < 8; i++) { q[g][i] = qp[i] * scale_log2; o[g][i] = 0.0f; }
    }

    // U slots per lane group and iteration: their loads are issued together, and the online softmax is
    // updated once per block of U (one running-maximum step, U + 1 exponentials) instead of per slot.
    // The loop bound is the same for every lane of a warp, so the shuffles stay convergent; a lane group
    // whose slot falls past the end computes on zeros and gets weight 0.
    constexpr int U = 4;
    for (int tb = s0 + warp * SPW; tb < s1; tb += 4 * SPW * U) {
        float k[U][8], v[U][8];
        bool valid[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int t = tb + u * 4 * SPW + sub;
            valid[u] = t < s1;
            if (valid[u]) {
                Row<DT, false>::load8(s, t, c0, k[u]);
                Row<DT, true>::load8(s, t, c0, v[u]);
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) { k[u][i] = 0.0f; v[u][i] = 0.0f; }
            }
        }
#pragma unroll
        for (int g = 0; g < GC; g++) {
            float d[U], mn = m[g];
#pragma unroll
            for (int u = 0; u < U; u++) {
                float acc = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) acc = fmaf(q[g][i], k[u][i], acc);
#pragma unroll
                for (int off = 1; off < TPS; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
                d[u] = valid[u] ? acc : -CUDART_INF_F;
                mn = fmaxf(mn, d[u]);
            }
            if (mn != -CUDART_INF_F) {
                const float a = fast_exp2(m[g] - mn);          // 0 while m is still -inf
                float w[U], ws = 0.0f;
#pragma unroll
                for (int u = 0; u < U; u++) { w[u] = fast_exp2(d[u] - mn); ws += w[u]; }
                l[g] = l[g] * a + ws;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    float acc = o[g][i] * a;
#pragma unroll
                    for (int u = 0; u < U; u++) acc = fmaf(w[u], v[u][i], acc);
                    o[g][i] = acc;
                }
                m[g] = mn;
            }
        }
    }

    // combine the SPW lane groups of this warp
#pragma unroll
    for (int off = TPS; off < 32; off <<= 1) {
#pragma unroll
        for (int g = 0; g < GC; g++) {
            float m2 = __shfl_xor_sync(0xffffffffu, m[g], off);
            float l2 = __shfl_xor_sync(0xffffffffu, l[g], off);
            float mn = fmaxf(m[g], m2);
            float a1 = (m[g] == -CUDART_INF_F) ? 0.0f : fast_exp2(m[g] - mn);
            float a2 = (m2 == -CUDART_INF_F) ? 0.0f : fast_exp2(m2 - mn);
            l[g] = l[g] * a1 + l2 * a2;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float o2 = __shfl_xor_sync(0xffffffffu, o[g][i], off);
                o[g][i] = o[g][i] * a1 + o2 * a2;
            }
            m[g] = mn;
        }
    }
    __shared__ float sm_o[4][GC][HD];
    __shared__ float sm_m[4][GC], sm_l[4][GC];
    if (sub == 0) {
#pragma unroll
        for (int g = 0; g < GC; g++) {
#pragma unroll
            for (int i = 0; i < 8; i++) sm_o[warp][g][cl * 8 + i] = o[g][i];
            if (cl == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
        }
    }
    __syncthreads();
    const bool final_out = (n_split == 1) && !p.want_partial;
    for (int t = threadIdx.x; t < heads_here * HD; t += 128) {
        int g = t / HD, d = t % HD;
        float mm = fmaxf(fmaxf(sm_m[0][g], sm_m[1][g]), fmaxf(sm_m[2][g], sm_m[3][g]));
        float acc = 0.0f, ll = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            float a = (sm_m[w][g] == -CUDART_INF_F) ? 0.0f : fast_exp2(sm_m[w][g] - mm);
            acc += sm_o[w][g][d] * a;
            ll += sm_l[w][g] * a;
        }
        size_t row = row0 + h0 + g;
        if (final_out) {
            p.out[row * HD + d] = ll > 0.0f ? acc / ll : 0.0f;
        } else {
            float* w = p.work + (row * n_split + split) * (HD + 2);
            w[2 + d] = acc;
            if (d == 0) { w[0] = mm; w[1] = ll; }
        }
    }
}

// Any head_dim / any group size, f32 cache only: one warp per (sequence, query, head), lanes
// stride over channels.  Slow; exists so that the trait's shapes (head_dim 1, 2, 3, 4 ...
// flare-core/src/model.rs:10427-10435) run on the device as well.
__global__ void decode_f32_anyshape_kernel(DecodeParams p) {
    const int hd = p.kv.head_dim;
    const int bq = p.bq0 + (int)blockIdx.z;
    const int h = blockIdx.x, b = bq / p.n_q, qi = bq % p.n_q;
    const int lane = threadIdx.x;
    const int kvh = h / (p.num_heads / p.kv.num_kv_heads);
    int n = p.attend_len[b] - (p.causal_q ? (p.n_q - 1 - qi) : 0);
    int lo = 0, hi = n;
    if (p.window > 0) lo = max(lo, n - p.window);
    if (p.slot_end >= 0) { lo = max(lo, p.slot_begin); hi = min(hi, p.slot_end); }
    const float* K = reinterpret_cast<const float*>(p.kv.plane[FLARE_PLANE_K] + (size_t)b * p.kv.stride[FLARE_PLANE_K]);
    const float* V = reinterpret_cast<const float*>(p.kv.plane[FLARE_PLANE_V] + (size_t)b * p.kv.stride[FLARE_PLANE_V]);
    const size_t row = ((size_t)b * p.n_q + qi) * p.num_heads + h;
    const float* q = p.q + row * hd;
    const float scale_log2 = rsqrtf((float)hd) * kLog2e;
    constexpr int MAXD = 8;   // head_dim <= 256
    float o[MAXD], qq[MAXD];
#pragma unroll
    for (int i = 0; i < MAXD; i++) { o[i] = 0.0f; int d = lane + 32 * i; qq[i] = d < hd ? q[d] * scale_log2 : 0.0f; }
    float m = -CUDART_INF_F, l = 0.0f;
    for (int t = lo; t < hi; t++) {
        const float* kr = K + (size_t)t * p.kv.kv_dim + kvh * hd;
        const float* vr = V + (size_t)t * p.kv.kv_dim + kvh * hd;
        float d = 0.0f;
#pragma unroll
        for (int i = 0; i < MAXD; i++) { int c = lane + 32 * i; if (c < hd) d = fmaf(qq[i], kr[c], d); }
#pragma unroll
        for (int off = 16; off; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        float mn = fmaxf(m, d);
        float a = fast_exp2(m - mn), w = fast_exp2(d - mn);
        l = l * a + w;
#pragma unroll
        for (int i = 0; i < MAXD; i++) { int c = lane + 32 * i; if (c < hd) o[i] = o[i] * a + w * vr[c]; }
        m = mn;
    }
#pragma unroll
    for (int i = 0; i < MAXD; i++) {
        int c = lane + 32 * i;
        if (c >= hd) continue;
        if (p.want_partial) p.out[row * (hd + 2) + 2 + c] = o[i];
        else p.out[row * hd + c] = l > 0.0f ? o[i] / l : 0.0f;
    }
    if (p.want_partial && lane == 0) { p.out[row * (hd + 2)] = m * kLn2; p.out[row * (hd + 2) + 1] = l; }
}

// Log-sum-exp merge of n_parts partials per row.  in_log2: the stored max is in log2 units
// (the split kernel's workspace); otherwise natural units (partials exchanged between GPUs).
__global__ void merge_partials_kernel(const float* __restrict__ parts, size_t part_stride, size_t row_stride,
                                      int n_parts, int hd, float* __restrict__ out, int in_log2,
                                      int want_partial) {
    const int row = blockIdx.x;
    const float* base = parts + (size_t)row * row_stride;
    const float unit = in_log2 ? 1.0f : kLog2e;
    float mm = -CUDART_INF_F;
    for (int r = 0; r < n_parts; r++) {
        const float* pr = base + r * part_stride;
        if (pr[1] > 0.0f) mm = fmaxf(mm, pr[0] * unit);
    }
    float ll = 0.0f;
    for (int r = 0; r < n_parts; r++) {
        const float* pr = base + r * part_stride;
        if (pr[1] > 0.0f) ll += pr[1] * fast_exp2(pr[0] * unit - mm);
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.0f;
        for (int r = 0; r < n_parts; r++) {
            const float* pr = base + r * part_stride;
            if (pr[1] > 0.0f) acc += pr[2 + d] * fast_exp2(pr[0] * unit - mm);
        }
        if (want_partial) out[(size_t)row * (hd + 2) + 2 + d] = acc;
        else out[(size_t)row * hd + d] = ll > 0.0f ? acc / ll : 0.0f;
    }
    if (want_partial && threadIdx.x == 0) {
        out[(size_t)row * (hd + 2)] = mm * kLn2;
        out[(size_t)row * (hd + 2) + 1] = ll;
    }
}

template <int DT, int TPS>
void launch_gc(int gc, dim3 grid, cudaStream_t st, const DecodeParams& p) {
    switch (gc) {
        case 1: decode_splitkv_kernel<DT, TPS, 1><<<grid, 128, 0, st>>>(p); break;
        case 2: decode_splitkv_kernel<DT, TPS, 2><<<grid, 128, 0, st>>>(p); break;
        case 3: decode_splitkv_kernel<DT, TPS, 3><<<grid, 128, 0, st>>>(p); break;
        default: decode_splitkv_kernel<DT, TPS, 4><<<grid, 128, 0, st>>>(p); break;
    }
}
template <int DT>
bool launch_tps(int hd, int gc, dim3 grid, cudaStream_t st, const DecodeParams& p) {
    switch (hd) {
        case 64: launch_gc<DT, 8>(gc, grid, st, p); return true;
        case 128: launch_gc<DT, 16>(gc, grid, st, p); return true;
        default: return false;
    }
}
bool launch_f32_small(int hd, int gc, dim3 grid, cudaStream_t st, const DecodeParams& p) {
    switch (hd) {
        case 32: launch_gc<FLARE_KV_F32, 4>(gc, grid, st, p); return true;
        case 256: launch_gc<FLARE_KV_F32, 32>(gc, grid, st, p); return true;
        default: return false;
    }
}

}  // namespace

int flare_launch_merge(flare_attn_ctx* ctx, const float* partials, size_t part_stride_floats, int n_parts,
                       int rows, int head_dim, float* out, int want_partial) {
    if (rows <= 0) return FLARE_OK;
    int threads = head_dim < 128 ? ((head_dim + 31) / 32) * 32 : 128;
    merge_partials_kernel<<<rows, threads, 0, ctx->stream>>>(partials, part_stride_floats, (size_t)(head_dim + 2),
                                                             n_parts, head_dim, out, 0, want_partial);
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}

int flare_launch_merge_work(flare_attn_ctx* ctx, const float* work, int n_split, int rows, int hd, float* out,
                            int want_partial) {
    int threads = hd < 128 ? hd : 128;
    merge_partials_kernel<<<rows, threads, 0, ctx->stream>>>(work, (size_t)(hd + 2), (size_t)n_split * (hd + 2), n_split,
                                                             hd, out, 1, want_partial);
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}

int flare_launch_decode_generic(flare_attn_ctx* ctx, const DecodeArgs& a) {
    const int hd = a.kv.head_dim, nkv = a.kv.num_kv_heads;
    const int G = a.num_heads / nkv;
    const int rows = a.batch * a.n_q * a.num_heads;
    if (rows == 0) return FLARE_OK;
    DecodeParams p;
    p.kv = a.kv; p.q = a.q; p.out = a.out; p.work = nullptr;
    p.attend_len = a.attend_len; p.ring = a.ring;
    p.n_q = a.n_q; p.num_heads = a.num_heads;
    p.slot_begin = a.slot_begin; p.slot_end = a.slot_end; p.want_partial = a.want_partial; p.causal_q = a.causal_q;
    p.window = a.window;
    p.range_max = a.slot_end >= 0 ? (a.slot_end - a.slot_begin) : a.max_attend;
    if (p.range_max < 0) p.range_max = 0;

    const bool fast_hd = (hd == 64 || hd == 128) || (a.kv.dtype == FLARE_KV_F32 && (hd == 32 || hd == 256));
    if (!fast_hd) {
        if (a.kv.dtype != FLARE_KV_F32 || hd > 256)
            return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "head_dim %d is not supported for this cache format", hd);
        p.n_chunks = 1;
        for (long long z0 = 0; z0 < (long long)a.batch * a.n_q; z0 += kMaxGridZ) {
            p.bq0 = (int)z0;
            dim3 grid(a.num_heads, 1, (unsigned)std::min<long long>(kMaxGridZ, (long long)a.batch * a.n_q - z0));
            decode_f32_anyshape_kernel<<<grid, 32, 0, ctx->stream>>>(p);
            FLARE_LAUNCH_CHECK(ctx);
        }
        return FLARE_OK;
    }
    const int gc = G >= 4 ? 4 : G;
    p.n_chunks = (G + gc - 1) / gc;
    // enough CTAs to fill the machine several times over, but at least 256 slots per CTA
    const int units = a.batch * a.n_q * nkv * p.n_chunks;
    int want = (ctx->sm_count * 8 + units - 1) / units;
    int max_split = (p.range_max + 255) / 256;
    int n_split = want < max_split ? want : max_split;
    if (n_split < 1) n_split = 1;
    if (n_split > 256) n_split = 256;
    if (n_split > 1 || a.want_partial) {
        size_t need = (size_t)rows * n_split * (hd + 2) * sizeof(float);
        FLARE_TRY(flare_ensure(ctx, &ctx->d_work, &ctx->work_bytes, need));
        p.work = (float*)ctx->d_work;
    }
    // grid.z = (sequence, query) pairs, at most 65535 per launch: a long prompt through the general prefill path
    // (every row a query) takes several launches
    for (long long z0 = 0; z0 < (long long)a.batch * a.n_q; z0 += kMaxGridZ) {
        p.bq0 = (int)z0;
        dim3 grid(n_split, nkv * p.n_chunks, (unsigned)std::min<long long>(kMaxGridZ, (long long)a.batch * a.n_q - z0));
        bool ok = false;
        switch (a.kv.dtype) {
            case FLARE_KV_F32:
                ok = launch_tps<FLARE_KV_F32>(hd, gc, grid, ctx->stream, p) || launch_f32_small(hd, gc, grid, ctx->stream, p);
                break;
            case FLARE_KV_Q8_0: ok = launch_tps<FLARE_KV_Q8_0>(hd, gc, grid, ctx->stream, p); break;
            case FLARE_KV_KIVI_REF: ok = launch_tps<FLARE_KV_KIVI_REF>(hd, gc, grid, ctx->stream, p); break;
            case FLARE_KV_KIVI_G32: ok = launch_tps<FLARE_KV_KIVI_G32>(hd, gc, grid, ctx->stream, p); break;
        }
        if (!ok) return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "no decode kernel for dtype %d head_dim %d", a.kv.dtype, hd);
        FLARE_LAUNCH_CHECK(ctx);
    }
    if (a.defer_merge && a.want_partial) {          // the caller merges: tell it where the records are
        *a.work_out = p.work; *a.n_split_out = n_split;
        return FLARE_OK;
    }
    if (n_split > 1 || a.want_partial) {
        int threads = hd < 128 ? hd : 128;
        merge_partials_kernel<<<rows, threads, 0, ctx->stream>>>(p.work, (size_t)(hd + 2), (size_t)n_split * (hd + 2),
                                                                 n_split, hd, a.out, 1, a.want_partial);
        FLARE_LAUNCH_CHECK(ctx);
    }
    return FLARE_OK;
}

// ---------------------------------------------------------------------------------------
// Decode attention that allocates nothing (flare_decode_attn_noalloc).
//
// Who needs it: code that calls into this library at a point where device allocation is
// off the table — a serving loop that has handed the whole GPU memory to its own pool at
// start-up, a latency-critical callback that must not take the driver's allocation lock,
// a host that forbids cudaMalloc after initialisation.  The ordinary entry point grows a
// split-KV workspace and a few staging buffers with cudaMalloc on first use; this one keeps
// its workspace in the library image instead.
//
// The workspace is one file-scope __device__ array: every GPU that loads the library carries
// these bytes until the process exits, which is why the size is modest and fixed.  In host
// code the array's name is only a handle; the device address is obtained once per device
// with cudaGetSymbolAddress (while that device is current) and handed to the kernels.
//
// The first launch of each kernel instantiation (cache type x head_dim x heads per KV head) can also
// make the driver load code lazily; that is the driver's business, not an allocation made here.
//
// Layout of the array: [0, kSmallBytes) the per-sequence (position, length) records followed
// by the per-sequence attend lengths; [kSmallBytes, end) the split-KV partials
// [row][split][head_dim + 2].  Nothing has to start at zero: every (row, split) record and
// every small record that a call reads is written by that same call first.  All calls on a
// device share the array, so two calls that overlap on the GPU (different streams or
// contexts) race; callers serialise them.
// ---------------------------------------------------------------------------------------
#define FLARE_NOALLOC_SCRATCH_BYTES (8u << 20)      /* the stated maximum: 8 MiB per GPU */
#define FLARE_NOALLOC_MAX_BATCH 256
static __device__ __align__(256) unsigned char g_noalloc_scratch[FLARE_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr size_t kSmallBytes = 4096;   // 256 x (int2 + int) = 3072, rounded up
void* g_noalloc_ptr[64] = {};          // device address of the array, per device ordinal
}

size_t flare_noalloc_scratch_bytes() { return FLARE_NOALLOC_SCRATCH_BYTES; }

int flare_decode_noalloc(flare_attn_ctx* ctx, const flare_kv* kv, int layer, int num_heads, const float* q_dev,
                         int n_q, const int* attend_len, float* out_dev) {
    const int hd = kv->head_dim, nkv = kv->num_kv_heads, B = kv->batch;
    if (kv->dtype != FLARE_KV_F32 && kv->dtype != FLARE_KV_Q8_0)
        return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "the no-allocation entry point serves f32 and Q8_0 caches only");
    if (hd != 64 && hd != 128)
        return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "the no-allocation entry point needs head_dim 64 or 128, got %d", hd);
    if (B > FLARE_NOALLOC_MAX_BATCH)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "batch %d exceeds the no-allocation maximum of %d", B,
                               FLARE_NOALLOC_MAX_BATCH);
    if (ctx->device < 0 || ctx->device >= 64) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "device ordinal out of range");

    // set-up, once per device, with that device current (the caller has bound it)
    char* scratch;
    {
        static std::mutex setup_mutex;     // two contexts on two host threads may make their first call at once
        std::lock_guard<std::mutex> lock(setup_mutex);
        if (!g_noalloc_ptr[ctx->device]) {
            void* p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p)
                return flare_set_error(ctx, FLARE_ERR_CUDA, "cudaGetSymbolAddress(g_noalloc_scratch) failed: %s", cudaGetErrorString(e));
            g_noalloc_ptr[ctx->device] = p;
        }
        scratch = (char*)g_noalloc_ptr[ctx->device];
    }

    // small per-sequence records, built on the host stack
    struct { int2 ring[FLARE_NOALLOC_MAX_BATCH]; int att[FLARE_NOALLOC_MAX_BATCH]; } small;
    int max_attend = 0;
    for (int b = 0; b < B; b++) {
        int64_t a;
        if (attend_len) a = attend_len[b];
        else { a = kv->length[b] + n_q; if (a > kv->max_seq_len) a = kv->max_seq_len; }
        if (a < 0 || a > kv->max_seq_len)
            return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "attend_len[%d] = %lld outside [0, %d]", b, (long long)a, kv->max_seq_len);
        small.att[b] = (int)a;
        if (a > max_attend) max_attend = (int)a;
        small.ring[b] = make_int2((int)kv->position[b], (int)kv->length[b]);
    }
    int* d_att = (int*)(scratch + sizeof(small.ring));

    const int G = num_heads / nkv;
    const int rows = B * n_q * num_heads;
    DecodeParams p;
    p.kv = flare_layer_view(kv, layer);
    p.q = q_dev; p.out = out_dev; p.work = (float*)(scratch + kSmallBytes);
    p.attend_len = d_att; p.ring = (const int2*)scratch;
    p.n_q = n_q; p.num_heads = num_heads;
    p.slot_begin = 0; p.slot_end = -1; p.want_partial = 0; p.causal_q = 1; p.window = 0;
    p.range_max = max_attend;
    const int gc = G >= 4 ? 4 : G;
    p.n_chunks = (G + gc - 1) / gc;
    const int units = B * n_q * nkv * p.n_chunks;
    int want = (ctx->sm_count * 8 + units - 1) / units;
    int max_split = (p.range_max + 255) / 256;
    int n_split = want < max_split ? want : max_split;
    if (n_split < 1) n_split = 1;
    if (n_split > 256) n_split = 256;
    // refuse before anything is put on the stream
    const size_t need = n_split > 1 ? (size_t)rows * n_split * (hd + 2) * sizeof(float) : 0;
    if (need > FLARE_NOALLOC_SCRATCH_BYTES - kSmallBytes)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG,
                               "this call needs %zu bytes of split-KV workspace (%d rows x %d splits); the no-allocation "
                               "entry point has %zu", need, rows, n_split, (size_t)FLARE_NOALLOC_SCRATCH_BYTES - kSmallBytes);
    // The records go into the head of the array.  The source is pageable stack memory: the runtime has taken
    // its own copy of `small` by the time each of these calls returns.
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(scratch, small.ring, sizeof(int2) * B, cudaMemcpyHostToDevice, ctx->stream));
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d_att, small.att, sizeof(int) * B, cudaMemcpyHostToDevice, ctx->stream));
    p.bq0 = 0;
    dim3 grid(n_split, nkv * p.n_chunks, B * n_q);
    bool ok = kv->dtype == FLARE_KV_F32 ? launch_tps<FLARE_KV_F32>(hd, gc, grid, ctx->stream, p)
                                        : launch_tps<FLARE_KV_Q8_0>(hd, gc, grid, ctx->stream, p);
    if (!ok) return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "no decode kernel for head_dim %d", hd);
    FLARE_LAUNCH_CHECK(ctx);
    if (n_split > 1) {
        int threads = hd < 128 ? hd : 128;
        merge_partials_kernel<<<rows, threads, 0, ctx->stream>>>(p.work, (size_t)(hd + 2), (size_t)n_split * (hd + 2),
                                                                 n_split, hd, out_dev, 1, 0);
        FLARE_LAUNCH_CHECK(ctx);
    }
    return FLARE_OK;
}
