// KV-cache kernels: storing rows (with on-device quantisation), the bit-exact dequantised
// view, and the Q8_0 block-stream converters.  Every quantiser reproduces the reference
// arithmetic operation by operation (IEEE divide, separate multiply and add, round half
// away from zero) so that codes and scales are byte-identical to the CPU's.
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr float kF32Eps = 1.1920929e-07f;

__device__ __forceinline__ int ring_slot(int64_t abs_pos, int max_seq) { return (int)(abs_pos % max_seq); }

// ------------------------------------------------------------------ F32: plain row copy
__global__ void write_f32_kernel(float* __restrict__ K, float* __restrict__ V, const float* __restrict__ key,
                                 const float* __restrict__ value, int64_t first_pos, int n_rows, int kv_dim,
                                 int max_seq) {
    size_t total = (size_t)n_rows * kv_dim;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int r = (int)(i / kv_dim), c = (int)(i % kv_dim);
        // when n_rows > max_seq only the last max_seq rows survive, as with sequential writes
        if (n_rows - r > max_seq) continue;
        size_t dst = (size_t)ring_slot(first_pos + r, max_seq) * kv_dim + c;
        K[dst] = key[i];
        V[dst] = value[i];
    }
}

// ------------------------------------------------------------------ Q8_0
// flare-core/src/model.rs:5507-5527: amax, d = amax / 127, id = 127 / amax (0 when d == 0),
// q = round(x * id) as i8 (saturating); the block scale is d rounded to f16 (RNE).
// One warp per 32-value block, lane = element.
__global__ void write_q8_kernel(int8_t* __restrict__ Kq, __half* __restrict__ Ks, int8_t* __restrict__ Vq,
                                __half* __restrict__ Vs, const float* __restrict__ key, const float* __restrict__ value,
                                int64_t first_pos, int n_rows, int kv_dim, int max_seq) {
    const int lane = threadIdx.x & 31;
    const int bpr = kv_dim / 32;
    const size_t n_blocks = (size_t)n_rows * bpr * 2;   // K blocks then V blocks
    for (size_t w = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5; w < n_blocks; w += ((size_t)gridDim.x * blockDim.x) >> 5) {
        const bool is_v = w >= n_blocks / 2;
        const size_t bi = is_v ? w - n_blocks / 2 : w;
        const int r = (int)(bi / bpr), blk = (int)(bi % bpr);
        if (n_rows - r > max_seq) continue;
        const float x = (is_v ? value : key)[(size_t)r * kv_dim + blk * 32 + lane];
        float amax = fabsf(x);
#pragma unroll
        for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = (d != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
        float rr = roundf(__fmul_rn(x, id));
        int qi = (rr != rr) ? 0 : (rr >= 127.0f ? 127 : (rr <= -128.0f ? -128 : (int)rr));
        const int slot = ring_slot(first_pos + r, max_seq);
        (is_v ? Vq : Kq)[(size_t)slot * kv_dim + blk * 32 + lane] = (int8_t)qi;
        if (lane == 0) (is_v ? Vs : Ks)[(size_t)slot * bpr + blk] = __float2half_rn(d);
    }
}

// ------------------------------------------------------------------ rotary position embedding
// apply_rope_with_table (flare-core/src/model.rs:7256-7292, the branch compiled on x86_64): element i of a head
// pairs with element i + head_dim/2; (x0, x1) -> (x0 c - x1 s, x0 s + x1 c) with c, s from the caller's table row
// of the token's position; two multiplies and a subtract / an add, never fused, so that the rotated row is the
// CPU's bit for bit.
struct RopeArgs {
    const float* cos;            // null: no rotation
    const float* sin;
    const long long* positions;  // per row: absolute token position = row of the table
    int head_dim;
    float* q_rows;               // optional: [batch][q_heads][head_dim] query rows rotated in place by the same launch
    int q_heads;
};
// Channel c of the rotated key row `row` (kv_dim values) of a token at table row `pos`.
__device__ __forceinline__ float rope_channel(const float* __restrict__ row, int c, const RopeArgs& r, long long pos) {
    const int half = r.head_dim >> 1, e = c % r.head_dim, head0 = c - e;
    const float* cr = r.cos + (size_t)pos * half;
    const float* sr = r.sin + (size_t)pos * half;
    if (e < half) return __fsub_rn(__fmul_rn(row[head0 + e], cr[e]), __fmul_rn(row[head0 + e + half], sr[e]));
    const int i = e - half;
    return __fadd_rn(__fmul_rn(row[head0 + i], sr[i]), __fmul_rn(row[head0 + e], cr[i]));
}
// In-place rotation of [n_rows][num_heads][head_dim] (used for q, and for the key rows of the 2-bit caches).
__device__ __forceinline__ void rope_rows_in_place(float* __restrict__ rows, int n_rows, int num_heads, const RopeArgs& r) {
    const int half = r.head_dim >> 1;
    const size_t total = (size_t)n_rows * num_heads * half;
    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        const int i = (int)(t % half);
        const size_t rh = t / half;                   // (row, head)
        const int row = (int)(rh / num_heads);
        const long long pos = r.positions[row];
        float* x = rows + rh * r.head_dim;
        const float c = r.cos[(size_t)pos * half + i], s = r.sin[(size_t)pos * half + i];
        const float x0 = x[i], x1 = x[i + half];
        x[i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        x[i + half] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
}
__global__ void rope_rows_kernel(float* __restrict__ rows, int n_rows, int num_heads, RopeArgs r) {
    flare_pdl_wait();
    flare_pdl_trigger();
    rope_rows_in_place(rows, n_rows, num_heads, r);
}

// One new token per sequence (a decode step of the whole batch): row b -> ring slot position[b].
__global__ void write_step_f32_kernel(float* __restrict__ K, float* __restrict__ V, size_t seq_stride_floats,
                                      const float* __restrict__ key, const float* __restrict__ value,
                                      const int2* __restrict__ ring, int batch, int kv_dim, RopeArgs rope) {
    flare_pdl_wait();
    flare_pdl_trigger();
    size_t total = (size_t)batch * kv_dim;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int b = (int)(i / kv_dim), c = (int)(i % kv_dim);
        size_t dst = (size_t)b * seq_stride_floats + (size_t)ring[b].x * kv_dim + c;
        K[dst] = rope.cos ? rope_channel(key + (size_t)b * kv_dim, c, rope, rope.positions[b]) : key[i];
        V[dst] = value[i];
    }
    if (rope.cos && rope.q_rows) rope_rows_in_place(rope.q_rows, batch, rope.q_heads, rope);
}
__global__ void write_step_q8_kernel(int8_t* __restrict__ Kq, __half* __restrict__ Ks, int8_t* __restrict__ Vq,
                                     __half* __restrict__ Vs, size_t q_stride, size_t s_stride,
                                     const float* __restrict__ key, const float* __restrict__ value,
                                     const int2* __restrict__ ring, int batch, int kv_dim, RopeArgs rope) {
    flare_pdl_wait();
    flare_pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int bpr = kv_dim / 32;
    const size_t n_blocks = (size_t)batch * bpr * 2;
    for (size_t w = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5; w < n_blocks; w += ((size_t)gridDim.x * blockDim.x) >> 5) {
        const bool is_v = w >= n_blocks / 2;
        const size_t bi = is_v ? w - n_blocks / 2 : w;
        const int b = (int)(bi / bpr), blk = (int)(bi % bpr);
        // the key is rotated (when a table is given) before it is quantised, as the model does (model.rs:2168-2206)
        const float x = (!is_v && rope.cos) ? rope_channel(key + (size_t)b * kv_dim, blk * 32 + lane, rope, rope.positions[b])
                                            : (is_v ? value : key)[(size_t)b * kv_dim + blk * 32 + lane];
        float amax = fabsf(x);
#pragma unroll
        for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = (d != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
        float rr = roundf(__fmul_rn(x, id));
        int qi = (rr != rr) ? 0 : (rr >= 127.0f ? 127 : (rr <= -128.0f ? -128 : (int)rr));
        const int slot = ring[b].x;
        (is_v ? Vq : Kq)[(size_t)b * q_stride + (size_t)slot * kv_dim + blk * 32 + lane] = (int8_t)qi;
        if (lane == 0) (is_v ? Vs : Ks)[(size_t)b * s_stride + (size_t)slot * bpr + blk] = __float2half_rn(d);
    }
    if (rope.cos && rope.q_rows) rope_rows_in_place(rope.q_rows, batch, rope.q_heads, rope);
}

// ------------------------------------------------------------------ 2-bit group quantiser
// flare-core/src/kv_cache.rs:332-371 for one group handled by one warp: `n` values spread
// over the lanes (value i on lane i % 32, visited in ascending i).  Returns this lane's codes
// through `code_of(i)`.
struct Q2Stats { float scale, mn, inv_scale; };
__device__ __forceinline__ Q2Stats q2_stats_from_minmax(float mn, float mx) {
    Q2Stats s;
    float range = __fsub_rn(mx, mn);
    s.scale = (fabsf(range) < kF32Eps) ? 0.0f : __fdiv_rn(range, 3.0f);
    s.inv_scale = (fabsf(s.scale) < kF32Eps) ? 0.0f : __fdiv_rn(3.0f, range);
    s.mn = mn;
    return s;
}
__device__ __forceinline__ uint32_t q2_code_of(float v, const Q2Stats& s) {
    if (fabsf(s.scale) < kF32Eps) return 0u;
    float r = roundf(__fmul_rn(__fsub_rn(v, s.mn), s.inv_scale));
    if (r != r) return 0u;
    r = fminf(fmaxf(r, 0.0f), 3.0f);
    return (uint32_t)r;
}

// ------------------------------------------------------------------ KIVI reference-exact write
// QuantizedKvCache::write (kv_cache.rs:121-162).  Kernel A: one block per row computes the
// per-token min/max, the key and value codes and the value (scale, min).
__global__ void write_kivi_ref_codes_kernel(uint8_t* __restrict__ Kq, uint8_t* __restrict__ Vq,
                                            float* __restrict__ Vscale, float* __restrict__ Vmin,
                                            const float* __restrict__ key, const float* __restrict__ value,
                                            int64_t first_pos, int n_rows, int kv_dim, int max_seq) {
    const int r = blockIdx.x >> 1;
    const bool is_v = blockIdx.x & 1;
    if (n_rows - r > max_seq) return;
    const float* src = (is_v ? value : key) + (size_t)r * kv_dim;
    __shared__ float s_mn[32], s_mx[32];
    float mn = CUDART_INF_F, mx = -CUDART_INF_F;
    for (int i = threadIdx.x; i < kv_dim; i += blockDim.x) {
        float v = src[i];
        if (v < mn) mn = v;
        if (v > mx) mx = v;
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) {
        float a = __shfl_xor_sync(0xffffffffu, mn, off), b = __shfl_xor_sync(0xffffffffu, mx, off);
        if (a < mn) mn = a;
        if (b > mx) mx = b;
    }
    if ((threadIdx.x & 31) == 0) { s_mn[threadIdx.x >> 5] = mn; s_mx[threadIdx.x >> 5] = mx; }
    __syncthreads();
    const int nw = blockDim.x >> 5;
    mn = s_mn[0]; mx = s_mx[0];
    for (int w = 1; w < nw; w++) { if (s_mn[w] < mn) mn = s_mn[w]; if (s_mx[w] > mx) mx = s_mx[w]; }
    const Q2Stats st = q2_stats_from_minmax(mn, mx);
    const int slot = ring_slot(first_pos + r, max_seq);
    const int ppt = kv_dim / 4;
    uint8_t* dst = (is_v ? Vq : Kq) + (size_t)slot * ppt;
    for (int j = threadIdx.x; j < ppt; j += blockDim.x) {
        uint32_t byte = 0;
#pragma unroll
        for (int e = 0; e < 4; e++) byte |= q2_code_of(src[4 * j + e], st) << (2 * e);
        dst[j] = (uint8_t)byte;
    }
    if (is_v && threadIdx.x == 0) { Vscale[slot] = st.scale; Vmin[slot] = st.mn; }
}
// Kernel B: one thread per channel walks the rows in order: running per-channel key stats
// (update_per_channel_stats, kv_cache.rs:399-420) and the f32 residual ring (kv_cache.rs:158-161).
__global__ void write_kivi_ref_stats_kernel(float* __restrict__ Kscale, float* __restrict__ Kmin,
                                            float* __restrict__ Kres, float* __restrict__ Vres,
                                            const float* __restrict__ key, const float* __restrict__ value,
                                            int64_t first_pos, int64_t length_before, int n_rows, int kv_dim,
                                            int max_seq, int residual_len) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= kv_dim) return;
    float mn = Kmin[c], sc = Kscale[c];
    for (int r = 0; r < n_rows; r++) {
        const float v = key[(size_t)r * kv_dim + c];
        if (length_before + r == 0) {
            mn = v; sc = 0.0f;
        } else {
            float old_max = __fadd_rn(mn, __fmul_rn(sc, 3.0f));
            float new_min = fminf(mn, v), new_max = fmaxf(old_max, v);
            float range = __fsub_rn(new_max, new_min);
            mn = new_min;
            sc = (fabsf(range) < kF32Eps) ? 0.0f : __fdiv_rn(range, 3.0f);
        }
        const int slot = ring_slot(first_pos + r, max_seq);
        Kres[(size_t)(slot % residual_len) * kv_dim + c] = v;
        Vres[(size_t)(slot % residual_len) * kv_dim + c] = value[(size_t)r * kv_dim + c];
    }
    Kmin[c] = mn; Kscale[c] = sc;
}

// ------------------------------------------------------------------ KIVI group-32 write
// A token is quantised when it is about to leave the 128-row f16 residual ring: writing the
// token with absolute index p (p % 32 == 0, p >= 128) first quantises tokens p-128 .. p-97,
// one whole key group (32 consecutive ring slots), from their f16 values.  The value of such
// a token comes from the rows being appended if it is one of them, else from the ring.
// grid: (trigger, kv_dim/32); block 32x32: K part: thread (cx, t) ...
__device__ __forceinline__ float g32_token_value(const __half* ring, const float* rows, int64_t tok,
                                                 int64_t first_pos, int c, int kv_dim) {
    if (tok >= first_pos) return __half2float(__float2half_rn(rows[(size_t)(tok - first_pos) * kv_dim + c]));
    return __half2float(ring[(size_t)(tok % FLARE_G32_RESIDUAL) * kv_dim + c]);
}
__global__ void write_g32_groups_kernel(uint8_t* __restrict__ Kq, __half2* __restrict__ Kmeta,
                                        uint8_t* __restrict__ Vq, __half2* __restrict__ Vmeta,
                                        const __half* __restrict__ Kres, const __half* __restrict__ Vres,
                                        const float* __restrict__ key, const float* __restrict__ value,
                                        int64_t first_pos, int64_t first_trigger, int kv_dim, int max_seq) {
    // blockIdx.x: trigger index; blockIdx.y: block of 32 channels; 32 warps, warp = w, lane = l
    const int64_t p = first_trigger + 32 * (int64_t)blockIdx.x;
    const int64_t tok0 = p - FLARE_G32_RESIDUAL;
    const int cb = blockIdx.y * 32;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int grp = (int)((tok0 % max_seq) / 32);
    __shared__ uint8_t s_code[32][33];   // [token][channel of this 32-block]
    {   // keys: warp w handles channel cb + w, lane = token within the group
        const int c = cb + w;
        float v = g32_token_value(Kres, key, tok0 + lane, first_pos, c, kv_dim);
        float mn = v, mx = v;
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            float a = __shfl_xor_sync(0xffffffffu, mn, off), b = __shfl_xor_sync(0xffffffffu, mx, off);
            if (a < mn) mn = a;
            if (b > mx) mx = b;
        }
        const Q2Stats st = q2_stats_from_minmax(mn, mx);
        s_code[lane][w] = (uint8_t)q2_code_of(v, st);
        if (lane == 0) {
            __half* row = reinterpret_cast<__half*>(Kmeta + (size_t)grp * kv_dim);
            row[FLARE_G32_KMETA_INDEX(c)] = __float2half_rn(st.scale);
            row[FLARE_G32_KMETA_INDEX(c) + 16] = __float2half_rn(st.mn);
        }
    }
    __syncthreads();
    if (threadIdx.x < 256) {   // pack 4 channels per byte: token t = tid / 8, byte j = tid % 8 of this 32-channel block
        const int t = threadIdx.x >> 3, j = threadIdx.x & 7;
        const uint32_t byte = s_code[t][4 * j] | (s_code[t][4 * j + 1] << 2) | (s_code[t][4 * j + 2] << 4) | (s_code[t][4 * j + 3] << 6);
        const int slot = (int)((tok0 + t) % max_seq);
        Kq[(size_t)slot * (kv_dim / 4) + cb / 4 + j] = (uint8_t)byte;
    }
    {   // values: warp w handles token tok0 + w, lane = channel within the 32-channel group
        const int64_t tok = tok0 + w;
        const int slot = (int)(tok % max_seq);
        float v = g32_token_value(Vres, value, tok, first_pos, cb + lane, kv_dim);
        float mn = v, mx = v;
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            float a = __shfl_xor_sync(0xffffffffu, mn, off), b = __shfl_xor_sync(0xffffffffu, mx, off);
            if (a < mn) mn = a;
            if (b > mx) mx = b;
        }
        const Q2Stats st = q2_stats_from_minmax(mn, mx);
        uint32_t code = q2_code_of(v, st) << ((lane & 3) * 2);
        code |= __shfl_xor_sync(0xffffffffu, code, 1);
        code |= __shfl_xor_sync(0xffffffffu, code, 2);
        if ((lane & 3) == 0) Vq[(size_t)slot * (kv_dim / 4) + (cb + lane) / 4] = (uint8_t)code;
        if (lane == 0) Vmeta[(size_t)slot * (kv_dim / 32) + blockIdx.y] = __halves2half2(__float2half_rn(st.scale), __float2half_rn(st.mn));
    }
}
__global__ void write_g32_ring_kernel(__half* __restrict__ Kres, __half* __restrict__ Vres,
                                      const float* __restrict__ key, const float* __restrict__ value,
                                      int64_t first_pos, int n_rows, int kv_dim) {
    const int skip = n_rows > FLARE_G32_RESIDUAL ? n_rows - FLARE_G32_RESIDUAL : 0;
    const size_t total = (size_t)(n_rows - skip) * kv_dim;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int r = skip + (int)(i / kv_dim), c = (int)(i % kv_dim);
        size_t dst = (size_t)((first_pos + r) % FLARE_G32_RESIDUAL) * kv_dim + c;
        Kres[dst] = __float2half_rn(key[(size_t)r * kv_dim + c]);
        Vres[dst] = __float2half_rn(value[(size_t)r * kv_dim + c]);
    }
}

// ------------------------------------------------------------------ dequantised view
struct DqView {
    const char* p[FLARE_PLANE_COUNT];
    int dtype, max_seq, kv_dim, position, length, newest;
};
__device__ float dq_element(const DqView& s, bool is_v, int slot, int c) {
    switch (s.dtype) {
        case FLARE_KV_F32:
            return reinterpret_cast<const float*>(s.p[is_v ? FLARE_PLANE_V : FLARE_PLANE_K])[(size_t)slot * s.kv_dim + c];
        case FLARE_KV_Q8_0: {
            int8_t qv = reinterpret_cast<const int8_t*>(s.p[is_v ? FLARE_PLANE_V_Q : FLARE_PLANE_K_Q])[(size_t)slot * s.kv_dim + c];
            __half sc = reinterpret_cast<const __half*>(s.p[is_v ? FLARE_PLANE_V_SCALE : FLARE_PLANE_K_SCALE])[(size_t)slot * (s.kv_dim / 32) + c / 32];
            return __fmul_rn((float)qv, __half2float(sc));
        }
        case FLARE_KV_KIVI_REF: {
            // QuantizedKvCache::dequant_keys/_values (kv_cache.rs:189-250)
            int R = s.max_seq < FLARE_REF_RESIDUAL ? s.max_seq : FLARE_REF_RESIDUAL;
            int t;
            if (s.length < s.max_seq) { if (slot >= s.length) return 0.0f; t = slot; }
            else { t = slot - s.position; if (t < 0) t += s.max_seq; }
            if (s.length <= R || t >= s.length - R)
                return reinterpret_cast<const float*>(s.p[is_v ? FLARE_PLANE_V_RES : FLARE_PLANE_K_RES])[(size_t)(slot % R) * s.kv_dim + c];
            const uint8_t* pk = reinterpret_cast<const uint8_t*>(s.p[is_v ? FLARE_PLANE_V_Q : FLARE_PLANE_K_Q]) + (size_t)slot * (s.kv_dim / 4);
            float code = q2_code(pk, c);
            if (is_v) return q2_dequant(code, reinterpret_cast<const float*>(s.p[FLARE_PLANE_V_SCALE])[slot],
                                        reinterpret_cast<const float*>(s.p[FLARE_PLANE_V_MIN])[slot]);
            return q2_dequant(code, reinterpret_cast<const float*>(s.p[FLARE_PLANE_K_SCALE])[c],
                              reinterpret_cast<const float*>(s.p[FLARE_PLANE_K_MIN])[c]);
        }
        default: {  // FLARE_KV_KIVI_G32
            int n = s.length;   // tokens that exist (the caller has advanced past them)
            if (n == 0) return 0.0f;
            int age = s.newest - slot; if (age < 0) age += s.max_seq;
            if (age >= n) return 0.0f;
            if (age < FLARE_G32_RESIDUAL)
                return __half2float(reinterpret_cast<const __half*>(s.p[is_v ? FLARE_PLANE_V_RES : FLARE_PLANE_K_RES])[(size_t)(slot % FLARE_G32_RESIDUAL) * s.kv_dim + c]);
            if (is_v) {
                const uint8_t* pk = reinterpret_cast<const uint8_t*>(s.p[FLARE_PLANE_V_Q]) + (size_t)slot * (s.kv_dim / 4);
                float2 m = __half22float2(reinterpret_cast<const __half2*>(s.p[FLARE_PLANE_V_SCALE])[(size_t)slot * (s.kv_dim / 32) + c / 32]);
                return q2_dequant(q2_code(pk, c), m.x, m.y);
            }
            int grp = slot >> 5;
            const uint8_t* pk = reinterpret_cast<const uint8_t*>(s.p[FLARE_PLANE_K_Q]) + (size_t)slot * (s.kv_dim / 4);
            const __half* row = reinterpret_cast<const __half*>(s.p[FLARE_PLANE_K_SCALE]) + (size_t)grp * s.kv_dim * 2;
            return q2_dequant(q2_code(pk, c), __half2float(row[FLARE_G32_KMETA_INDEX(c)]), __half2float(row[FLARE_G32_KMETA_INDEX(c) + 16]));
        }
    }
}
__global__ void export_dequant_kernel(DqView s, float* __restrict__ k_out, float* __restrict__ v_out) {
    const size_t total = (size_t)s.max_seq * s.kv_dim;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int slot = (int)(i / s.kv_dim), c = (int)(i % s.kv_dim);
        if (k_out) k_out[i] = dq_element(s, false, slot, c);
        if (v_out) v_out[i] = dq_element(s, true, slot, c);
    }
}

// ------------------------------------------------------------------ Q8_0 block stream <-> planes
__global__ void q8_blocks_kernel(int8_t* __restrict__ q, __half* __restrict__ sc, uint8_t* __restrict__ blocks,
                                 int first_slot, int n_slots, int kv_dim, int to_blocks) {
    const int bpr = kv_dim / 32;
    const size_t total = (size_t)n_slots * bpr * 34;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t blk = i / 34;
        int byte = (int)(i % 34);
        int r = (int)(blk / bpr), b = (int)(blk % bpr);
        int slot = first_slot + r;
        if (byte < 2) {
            uint16_t* sp = reinterpret_cast<uint16_t*>(sc) + (size_t)slot * bpr + b;
            if (to_blocks) blocks[i] = (uint8_t)((*sp >> (8 * byte)) & 0xFF);
            else if (byte == 0) *sp = (uint16_t)(blocks[i] | (blocks[i + 1] << 8));
        } else {
            int8_t* qp = q + (size_t)slot * kv_dim + b * 32 + (byte - 2);
            if (to_blocks) blocks[i] = (uint8_t)*qp;
            else *qp = (int8_t)blocks[i];
        }
    }
}

int grid_for(size_t total, int threads) {
    size_t g = (total + threads - 1) / threads;
    if (g > 148 * 16) g = 148 * 16;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace

int flare_launch_kv_write(flare_kv* kv, int layer, int seq, int64_t first_pos, int64_t length_before, int n_rows,
                          const float* d_key, const float* d_value) {
    flare_attn_ctx* ctx = kv->ctx;
    if (n_rows <= 0) return FLARE_OK;
    cudaStream_t st = ctx->stream;
    const int kvd = kv->kv_dim, ms = kv->max_seq_len;
    switch (kv->dtype) {
        case FLARE_KV_F32:
            write_f32_kernel<<<grid_for((size_t)n_rows * kvd, 256), 256, 0, st>>>(
                (float*)kv->plane_ptr(FLARE_PLANE_K, layer, seq), (float*)kv->plane_ptr(FLARE_PLANE_V, layer, seq), d_key,
                d_value, first_pos, n_rows, kvd, ms);
            FLARE_LAUNCH_CHECK(ctx);
            break;
        case FLARE_KV_Q8_0:
            write_q8_kernel<<<grid_for((size_t)n_rows * kvd * 2, 256), 256, 0, st>>>(
                (int8_t*)kv->plane_ptr(FLARE_PLANE_K_Q, layer, seq), (__half*)kv->plane_ptr(FLARE_PLANE_K_SCALE, layer, seq),
                (int8_t*)kv->plane_ptr(FLARE_PLANE_V_Q, layer, seq), (__half*)kv->plane_ptr(FLARE_PLANE_V_SCALE, layer, seq),
                d_key, d_value, first_pos, n_rows, kvd, ms);
            FLARE_LAUNCH_CHECK(ctx);
            break;
        case FLARE_KV_KIVI_REF: {
            write_kivi_ref_codes_kernel<<<n_rows * 2, 128, 0, st>>>(
                (uint8_t*)kv->plane_ptr(FLARE_PLANE_K_Q, layer, seq), (uint8_t*)kv->plane_ptr(FLARE_PLANE_V_Q, layer, seq),
                (float*)kv->plane_ptr(FLARE_PLANE_V_SCALE, layer, seq), (float*)kv->plane_ptr(FLARE_PLANE_V_MIN, layer, seq),
                d_key, d_value, first_pos, n_rows, kvd, ms);
            FLARE_LAUNCH_CHECK(ctx);
            int R = ms < FLARE_REF_RESIDUAL ? ms : FLARE_REF_RESIDUAL;
            write_kivi_ref_stats_kernel<<<(kvd + 127) / 128, 128, 0, st>>>(
                (float*)kv->plane_ptr(FLARE_PLANE_K_SCALE, layer, seq), (float*)kv->plane_ptr(FLARE_PLANE_K_MIN, layer, seq),
                (float*)kv->plane_ptr(FLARE_PLANE_K_RES, layer, seq), (float*)kv->plane_ptr(FLARE_PLANE_V_RES, layer, seq),
                d_key, d_value, first_pos, length_before, n_rows, kvd, ms, R);
            FLARE_LAUNCH_CHECK(ctx);
            break;
        }
        case FLARE_KV_KIVI_G32: {
            // triggers: absolute positions p in [first_pos, first_pos + n_rows), p % 32 == 0, p >= 128
            int64_t t0 = ((first_pos + 31) / 32) * 32;
            if (t0 < FLARE_G32_RESIDUAL) t0 = FLARE_G32_RESIDUAL;
            int64_t last = first_pos + n_rows - 1;
            if (t0 <= last) {
                int n_trig = (int)((last - t0) / 32) + 1;
                dim3 grid(n_trig, kvd / 32);
                write_g32_groups_kernel<<<grid, 1024, 0, st>>>(
                    (uint8_t*)kv->plane_ptr(FLARE_PLANE_K_Q, layer, seq), (__half2*)kv->plane_ptr(FLARE_PLANE_K_SCALE, layer, seq),
                    (uint8_t*)kv->plane_ptr(FLARE_PLANE_V_Q, layer, seq), (__half2*)kv->plane_ptr(FLARE_PLANE_V_SCALE, layer, seq),
                    (const __half*)kv->plane_ptr(FLARE_PLANE_K_RES, layer, seq), (const __half*)kv->plane_ptr(FLARE_PLANE_V_RES, layer, seq),
                    d_key, d_value, first_pos, t0, kvd, ms);
                FLARE_LAUNCH_CHECK(ctx);
            }
            write_g32_ring_kernel<<<grid_for((size_t)(n_rows > 128 ? 128 : n_rows) * kvd, 256), 256, 0, st>>>(
                (__half*)kv->plane_ptr(FLARE_PLANE_K_RES, layer, seq), (__half*)kv->plane_ptr(FLARE_PLANE_V_RES, layer, seq),
                d_key, d_value, first_pos, n_rows, kvd);
            FLARE_LAUNCH_CHECK(ctx);
            break;
        }
        default:
            return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "unknown kv dtype %d", kv->dtype);
    }
    return FLARE_OK;
}

int flare_launch_rope_rows(flare_kv* kv, float* d_rows, int n_rows, int num_heads, const long long* d_positions) {
    flare_attn_ctx* ctx = kv->ctx;
    if (n_rows <= 0) return FLARE_OK;
    RopeArgs r = {kv->rope_cos, kv->rope_sin, d_positions, kv->head_dim, nullptr, 0};
    FLARE_CUDA_OK(ctx, flare_launch_pdl(rope_rows_kernel, dim3(grid_for((size_t)n_rows * num_heads * (kv->head_dim / 2), 256)), dim3(256), 0,
                                        ctx->stream, d_rows, n_rows, num_heads, r));
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}

int flare_launch_kv_write_step(flare_kv* kv, int layer, const int2* d_ring, const float* d_key, const float* d_value,
                               const long long* d_positions, float* d_q_rows, int q_heads) {
    flare_attn_ctx* ctx = kv->ctx;
    const int kvd = kv->kv_dim, B = kv->batch;
    // f32 and Q8_0 caches: the same launch rotates the step's query rows in place when they are given
    RopeArgs rope = {d_positions ? kv->rope_cos : nullptr, kv->rope_sin, d_positions, kv->head_dim,
                     (kv->dtype == FLARE_KV_F32 || kv->dtype == FLARE_KV_Q8_0) ? d_q_rows : nullptr, q_heads};
    switch (kv->dtype) {
        case FLARE_KV_F32:
            FLARE_CUDA_OK(ctx, flare_launch_pdl(write_step_f32_kernel, dim3(grid_for((size_t)B * kvd, 256)), dim3(256), 0, ctx->stream,
                                                (float*)kv->plane_ptr(FLARE_PLANE_K, layer, 0), (float*)kv->plane_ptr(FLARE_PLANE_V, layer, 0),
                                                kv->plane_bytes[FLARE_PLANE_K] / 4, d_key, d_value, d_ring, B, kvd, rope));
            FLARE_LAUNCH_CHECK(ctx);
            return FLARE_OK;
        case FLARE_KV_Q8_0:
#ifdef FLARE_TUNE
            if (const char* e = getenv("FLARE_STEP_PDL")) if (!atoi(e)) {
                write_step_q8_kernel<<<grid_for((size_t)B * kvd * 2, 256), 256, 0, ctx->stream>>>(
                    (int8_t*)kv->plane_ptr(FLARE_PLANE_K_Q, layer, 0), (__half*)kv->plane_ptr(FLARE_PLANE_K_SCALE, layer, 0),
                    (int8_t*)kv->plane_ptr(FLARE_PLANE_V_Q, layer, 0), (__half*)kv->plane_ptr(FLARE_PLANE_V_SCALE, layer, 0),
                    kv->plane_bytes[FLARE_PLANE_K_Q], kv->plane_bytes[FLARE_PLANE_K_SCALE] / 2, d_key, d_value, d_ring, B, kvd, rope);
                FLARE_LAUNCH_CHECK(ctx);
                return FLARE_OK;
            }
#endif
            FLARE_CUDA_OK(ctx, flare_launch_pdl(write_step_q8_kernel, dim3(grid_for((size_t)B * kvd * 2, 256)), dim3(256), 0, ctx->stream,
                                                (int8_t*)kv->plane_ptr(FLARE_PLANE_K_Q, layer, 0), (__half*)kv->plane_ptr(FLARE_PLANE_K_SCALE, layer, 0),
                                                (int8_t*)kv->plane_ptr(FLARE_PLANE_V_Q, layer, 0), (__half*)kv->plane_ptr(FLARE_PLANE_V_SCALE, layer, 0),
                                                kv->plane_bytes[FLARE_PLANE_K_Q], kv->plane_bytes[FLARE_PLANE_K_SCALE] / 2, d_key, d_value,
                                                d_ring, B, kvd, rope));
            FLARE_LAUNCH_CHECK(ctx);
            return FLARE_OK;
        default:
            // the 2-bit caches keep per-sequence running state: one sequence at a time (the caller has rotated the rows)
            for (int b = 0; b < B; b++) {
                int64_t abs_pos = kv->length[b] < kv->max_seq_len ? kv->length[b] : kv->max_seq_len + kv->position[b];
                FLARE_TRY(flare_launch_kv_write(kv, layer, b, abs_pos, kv->length[b], 1, d_key + (size_t)b * kvd,
                                                d_value + (size_t)b * kvd));
            }
            return FLARE_OK;
    }
}

int flare_launch_kv_export_dequant(flare_kv* kv, int layer, int seq, float* d_k, float* d_v) {
    flare_attn_ctx* ctx = kv->ctx;
    DqView s;
    for (int i = 0; i < FLARE_PLANE_COUNT; i++) s.p[i] = kv->plane[i] ? kv->plane_ptr(i, layer, seq) : nullptr;
    s.dtype = kv->dtype; s.max_seq = kv->max_seq_len; s.kv_dim = kv->kv_dim;
    s.position = (int)kv->position[seq]; s.length = (int)kv->length[seq];
    s.newest = (int)((kv->position[seq] + kv->max_seq_len - 1) % kv->max_seq_len);
    export_dequant_kernel<<<grid_for((size_t)kv->max_seq_len * kv->kv_dim, 256), 256, 0, ctx->stream>>>(s, d_k, d_v);
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}

int flare_launch_q8_blocks(flare_kv* kv, int layer, int seq, int first_slot, int n_slots, void* d_kb, void* d_vb,
                           int to_blocks) {
    flare_attn_ctx* ctx = kv->ctx;
    if (n_slots <= 0) return FLARE_OK;
    size_t total = (size_t)n_slots * (kv->kv_dim / 32) * 34;
    if (d_kb) {
        q8_blocks_kernel<<<grid_for(total, 256), 256, 0, ctx->stream>>>(
            (int8_t*)kv->plane_ptr(FLARE_PLANE_K_Q, layer, seq), (__half*)kv->plane_ptr(FLARE_PLANE_K_SCALE, layer, seq),
            (uint8_t*)d_kb, first_slot, n_slots, kv->kv_dim, to_blocks);
        FLARE_LAUNCH_CHECK(ctx);
    }
    if (d_vb) {
        q8_blocks_kernel<<<grid_for(total, 256), 256, 0, ctx->stream>>>(
            (int8_t*)kv->plane_ptr(FLARE_PLANE_V_Q, layer, seq), (__half*)kv->plane_ptr(FLARE_PLANE_V_SCALE, layer, seq),
            (uint8_t*)d_vb, first_slot, n_slots, kv->kv_dim, to_blocks);
        FLARE_LAUNCH_CHECK(ctx);
    }
    return FLARE_OK;
}
