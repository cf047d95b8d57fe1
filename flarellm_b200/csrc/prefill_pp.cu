// Prefill attention, the fast tensor-core kernel: two 128-row query tiles per CTA that take turns
// on the tensor core ("ping-pong"), with P kept in tensor memory.
//
//   warps 0-3   softmax of query tile A (thread r owns row r): S row out of tensor memory once for the
//               maximum (128 registers) and again, 64 columns at a time, for the exponentials, online
//               softmax in log2 units with lazy rescaling, P written back as
//               bf16 pairs into the first 64 columns of the same S buffer, O rescaled in place on
//               the rare occasions the row maximum moved by more than 2^8; final O / l to global
//   warps 4-7   the same for query tile B
//   warp 8      MMA issuer (one thread):  QK(A,0) QK(B,0) { PV(A,j) QK(A,j+1) PV(B,j) QK(B,j+1) }
//               S = Q K^T from shared-memory descriptors (K-major, 128B swizzle);
//               O += P V with P read from tensor memory and V from shared memory (MN-major)
//   warp 9      TMA producer: both Q tiles once, then K and V tiles through 2-stage rings
// Tensor memory (512 columns): S_A 0-127, S_B 128-255, O_A 256-383, O_B 384-511.  MMAs issued by
// one thread execute in order, so S_X(j+1) = QK cannot overwrite P_X(j) before PV(X,j) has read it,
// and when S_X(j+1) is signalled complete PV(X,j) has completed as well (O_X is stable).
// Measured and rejected (causal S 4096, 897 TFLOP/s as is): S and P in two 64-column halves with
// their own barriers (713: an N=64 SS-MMA re-reads Q from shared memory twice as often), P alone
// handed over in halves (848: the extra store-wait, fence and arrive in the exponential loop cost
// more than the earlier start of PV saves).
#include "common.cuh"
#include "tc5.cuh"
#include <math_constants.h>

using namespace tc5;

namespace {

constexpr int BN = 128;
#ifndef POLY_EVERY
#define POLY_EVERY 0      // one pair of exponentials in POLY_EVERY goes to the FMA-pipe polynomial (0: none; measured at
                          // S 4096 causal: none 907, every 4th pair 902, every 2nd 856 TFLOP/s)
#endif
constexpr uint32_t kWaitLimit = 1u << 20;

struct PPParams {
    void* out;
    int out_dtype, batch, seq_len, num_heads, num_kv_heads, window;
    float scale_log2;
    // f16 operands only: the power-of-two factors that undo the per-tensor scaling of the conversion,
    // [0] = 1 / (scale of q * scale of k), [1] = 1 / scale of v (null: both 1)
    const float* descale;
    int* err;
};

constexpr int KS = 2;      // stages of the K ring (3 measured no faster: 902 vs 907 TFLOP/s)

template <int HD>
struct SmemPP {
    static constexpr int PANELS = HD / 64;
    static constexpr int Q_BYTES = BM * HD * 2;        // one query tile
    static constexpr int KV_BYTES = BN * HD * 2;
    static constexpr int Q_OFF = 0;                     // 2 query tiles
    static constexpr int K_OFF = 2 * Q_BYTES;           // KS stages: K tiles are needed one step before the V tile of the same rows
    static constexpr int V_OFF = K_OFF + KS * KV_BYTES; // 2 stages
    static constexpr int TOTAL = V_OFF + 2 * KV_BYTES;  // 224 KB at head_dim 128
};

struct BarsPP {
    uint64_t q_full, k_full[KS], v_full[2], k_empty[KS], v_empty[2], s_full[2], p_full[2], o_final[2];
    uint32_t tmem_base;
    int abort_flag;
};

#define PP_WAIT(barptr, parity)                                                    \
    do {                                                                           \
        if (!ptx::mbar_wait((barptr), (parity), kWaitLimit)) { bars->abort_flag = 1; aborted = true; } \
    } while (0)

// columns [lo, hi) that query rows [r0, r0 + 128) may read, as a tile range
__device__ __forceinline__ void tile_range(int r0, int S, int window, int& j0, int& j1) {
    if (r0 >= S) { j0 = j1 = 0; return; }
    const int last_row = min(r0 + BM, S) - 1;
    const int col_lo = window > 0 ? max(0, r0 - window + 1) : 0;
    j0 = col_lo / BN;
    j1 = last_row / BN + 1;
}

// 2^x for x <= 0 on the FMA pipe (Cody-Waite split + cubic), used for part of the elements so that
// the MUFU is not the only unit computing exponentials.  Relative error < 1e-4, far below the bf16
// rounding of P (2^-9).
__device__ __forceinline__ float exp2_poly(float x) {
    x = fmaxf(x, -126.0f);                                   // also maps -inf (masked) to ~1e-38
    const float xr = x + 12582912.0f;                        // 1.5 * 2^23: integer part lands in the low mantissa bits
    const float f = x - (xr - 12582912.0f);                  // f in [-0.5, 0.5]
    float p = fmaf(f, 0.055170249f, 0.24260791f);            // minimax cubic of 2^f on [-0.5, 0.5], rel. error 7.5e-5
    p = fmaf(p, f, 0.69326091f);
    p = fmaf(p, f, 0.99992830f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(xr) << 23));
}

// The same for a pair, on packed f32x2 instructions: 2^x0, 2^x1 in 8 FMA-pipe instructions and 2 maxima.
__device__ __forceinline__ void exp2_poly2(float& y0, float& y1, float x0, float x1) {
    x0 = fmaxf(x0, -126.0f); x1 = fmaxf(x1, -126.0f);
    float p0, p1, r0, r1;
    asm("{\n\t.reg .b64 t, xr, fl, f, p, cm, cn, c3, c2, c1, c0, m1;\n\t"
        "mov.b64 t, {%4, %5};\n\t"
        "mov.b64 cm, {%6, %6};\n\tmov.b64 cn, {%7, %7};\n\tmov.b64 m1, {%8, %8};\n\t"
        "mov.b64 c3, {%9, %9};\n\tmov.b64 c2, {%10, %10};\n\tmov.b64 c1, {%11, %11};\n\tmov.b64 c0, {%12, %12};\n\t"
        "add.rn.f32x2 xr, t, cm;\n\t"          // integer part lands in the low mantissa bits
        "add.rn.f32x2 fl, xr, cn;\n\t"         // round(x)
        "fma.rn.f32x2 f, fl, m1, t;\n\t"       // f = x - round(x) in [-0.5, 0.5]
        "fma.rn.f32x2 p, f, c3, c2;\n\t"
        "fma.rn.f32x2 p, p, f, c1;\n\t"
        "fma.rn.f32x2 p, p, f, c0;\n\t"
        "mov.b64 {%0, %1}, p;\n\tmov.b64 {%2, %3}, xr;\n\t}"
        : "=f"(p0), "=f"(p1), "=f"(r0), "=f"(r1)
        : "f"(x0), "f"(x1), "f"(12582912.0f), "f"(-12582912.0f), "f"(-1.0f), "f"(0.055170249f), "f"(0.24260791f),
          "f"(0.69326091f), "f"(0.99992830f));
    y0 = __int_as_float(__float_as_int(p0) + (__float_as_int(r0) << 23));
    y1 = __int_as_float(__float_as_int(p1) + (__float_as_int(r1) << 23));
}

// packed-pair f32 arithmetic and the 3-input maximum of sm_100: half the issue slots per element
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b, float c) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// F16OPS: the operands (and P) are f16 instead of bf16.  f32 inputs take this form: 11 significant bits instead of 8
// keep a row that attends a single key within 2^-11 of the f32 result, which bf16 operands would not.
template <int HD, bool F16OPS>
// 10 warps are allocated as 12 (granularity 4): 12 x 32 x 168 registers is what one SM holds
__global__ void __launch_bounds__(320, 1) prefill_pp_kernel(const __grid_constant__ CUtensorMap qmap,
                                                            const __grid_constant__ CUtensorMap kmap,
                                                            const __grid_constant__ CUtensorMap vmap, PPParams p) {
    using L = SmemPP<HD>;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ BarsPP bar_storage;
    BarsPP* bars = &bar_storage;
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (p.num_heads / p.num_kv_heads);
    const int S = p.seq_len;
    // heavier (later) query tiles first: better tail behaviour under the causal mask
    const int pair = gridDim.x - 1 - blockIdx.x;
    const int rA = pair * 2 * BM, rB = rA + BM;
    int jA0, jA1, jB0, jB1;
    tile_range(rA, S, p.window, jA0, jA1);
    tile_range(rB, S, p.window, jB0, jB1);
    // the CTA walks tiles [j0, j1); a query tile takes part in tile j when its own range holds j
    const int j0 = (jB1 > jB0) ? min(jA0, jB0) : jA0;
    const int j1 = max(jA1, jB1);
    const int n_tiles = j1 - j0;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars->q_full, 1);
        for (int s = 0; s < 2; s++) {
            ptx::mbar_init(&bars->v_full[s], 1); ptx::mbar_init(&bars->v_empty[s], 1);
            ptx::mbar_init(&bars->s_full[s], 1); ptx::mbar_init(&bars->p_full[s], 128);
            ptx::mbar_init(&bars->o_final[s], 1);
        }
        for (int s = 0; s < KS; s++) { ptx::mbar_init(&bars->k_full[s], 1); ptx::mbar_init(&bars->k_empty[s], 1); }
        bars->abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    if (warp == 8) {
        tmem_alloc(&bars->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    bool aborted = false;

    if (warp == 9) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::mbar_expect_tx(&bars->q_full, 2 * L::Q_BYTES);
            for (int x = 0; x < 2; x++)
                for (int pn = 0; pn < L::PANELS; pn++)
                    ptx::tma_load_4d(sm + L::Q_OFF + x * L::Q_BYTES + pn * (BM * 128), &qmap, &bars->q_full, pn * 64, h, rA + x * BM, b);
            for (int t = 0; t < n_tiles && !aborted; t++) {
                const int s = t & 1, sk = t % KS, row = (j0 + t) * BN;
                if (t >= KS) PP_WAIT(&bars->k_empty[sk], (uint32_t)((t / KS - 1) & 1));
                if (aborted) break;
                ptx::mbar_expect_tx(&bars->k_full[sk], L::KV_BYTES);
                for (int pn = 0; pn < L::PANELS; pn++)
                    ptx::tma_load_4d(sm + FLARE_CK(L::K_OFF + sk * L::KV_BYTES + pn * (BN * 128), BN * 128, L::V_OFF, p.err), &kmap, &bars->k_full[sk], pn * 64, kvh, row, b);
                if (t >= 2) PP_WAIT(&bars->v_empty[s], (uint32_t)(((t >> 1) - 1) & 1));
                if (aborted) break;
                ptx::mbar_expect_tx(&bars->v_full[s], L::KV_BYTES);
                for (int pn = 0; pn < L::PANELS; pn++)
                    ptx::tma_load_4d(sm + FLARE_CK(L::V_OFF + s * L::KV_BYTES + pn * (BN * 128), BN * 128, L::TOTAL, p.err), &vmap, &bars->v_full[s], pn * 64, kvh, row, b);
            }
        }
    } else if (warp == 8) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_qk = F16OPS ? idesc_f16(BN, false) : idesc_bf16(BN, false);
            const uint32_t idesc_pv = F16OPS ? idesc_f16(HD, true) : idesc_bf16(HD, true);
            int n_done[2] = {0, 0};            // tiles issued so far per query tile (for barrier parities)
            auto in_range = [&](int x, int j) { return x == 0 ? (j >= jA0 && j < jA1) : (j >= jB0 && j < jB1); };
            auto qk = [&](int x, int t) {      // S_x = Q_x K_t^T
                const int s = t % KS;
                const uint32_t q_addr = ptx::smem_u32(sm + FLARE_CK(L::Q_OFF + x * L::Q_BYTES, L::Q_BYTES, L::K_OFF, p.err));
                const uint32_t k_addr = ptx::smem_u32(sm + FLARE_CK(L::K_OFF + s * L::KV_BYTES, L::KV_BYTES, L::V_OFF, p.err));
#pragma unroll
                for (int k = 0; k < HD / 16; k++) {
                    const uint64_t ad = desc_kmajor(q_addr + (k >> 2) * (BM * 128) + (k & 3) * 32);
                    const uint64_t bd = desc_kmajor(k_addr + (k >> 2) * (BN * 128) + (k & 3) * 32);
                    umma_bf16(tmem + x * 128, ad, bd, idesc_qk, k > 0 ? 1u : 0u);
                }
                tc_commit(&bars->s_full[x]);
            };
            auto pv = [&](int x, int t, bool first) {      // O_x (+)= P_x V_t, P_x in columns [0,64) of S_x
                const int s = t & 1;
                const uint32_t v_addr = ptx::smem_u32(sm + FLARE_CK(L::V_OFF + s * L::KV_BYTES, L::KV_BYTES, L::TOTAL, p.err));
#pragma unroll
                for (int k = 0; k < BN / 16; k++) {
                    const uint64_t bd = desc_mnmajor(v_addr + k * 2048, BN * 128);
                    umma_bf16_ts(tmem + 256 + x * 128, tmem + x * 128 + k * 8, bd, idesc_pv, (!first || k > 0) ? 1u : 0u);
                }
            };
            PP_WAIT(&bars->q_full, 0);
            // software pipeline over tiles: at step t issue QK(.,t) and PV(.,t-1)
            for (int t = 0; t <= n_tiles && !aborted; t++) {
                const int j = j0 + t;
                if (t < n_tiles) {
                    PP_WAIT(&bars->k_full[t % KS], (uint32_t)((t / KS) & 1));
                    if (aborted) break;
                    tc_fence_after();
                }
                for (int x = 0; x < 2 && !aborted; x++) {
                    // PV(x, t-1) first: it must read P_x before QK(x, t) overwrites the buffer (program order)
                    if (t >= 1 && in_range(x, j - 1)) {
                        const int nd = n_done[x] - 1;                       // index of that tile among x's tiles
                        PP_WAIT(&bars->p_full[x], (uint32_t)(nd & 1));
                        if (aborted) break;
                        if (x == 0 || !in_range(0, j - 1)) {                 // first PV of this step: V tile needed
                            PP_WAIT(&bars->v_full[(t - 1) & 1], (uint32_t)(((t - 1) >> 1) & 1));
                            if (aborted) break;
                        }
                        tc_fence_after();
                        pv(x, t - 1, nd == 0);
                        // last user of V_{t-1} in this step releases the stage
                        if (x == 1 || !in_range(1, j - 1)) tc_commit(&bars->v_empty[(t - 1) & 1]);
                        const bool last_tile_of_x = !(t < n_tiles && in_range(x, j));
                        if (last_tile_of_x) tc_commit(&bars->o_final[x]);
                    }
                    if (t < n_tiles && in_range(x, j)) { qk(x, t); n_done[x]++; }
                }
                if (t < n_tiles) tc_commit(&bars->k_empty[t % KS]);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax warps
        const int x = warp >> 2;                          // query tile
        const int r = threadIdx.x & 127;                  // row within the tile
        const int r0 = x ? rB : rA;
        const int grow = r0 + r;
        const int jx0 = x ? jB0 : jA0, jx1 = x ? jB1 : jA1;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + x * 128 + lane_base, tO = tmem + 256 + x * 128 + lane_base;
        const int row_lo = p.window > 0 ? max(0, grow - p.window + 1) : 0;
        float m_ref = -CUDART_INF_F, l_sum = 0.0f;
        const float scale_log2 = (F16OPS && p.descale) ? p.scale_log2 * __ldg(p.descale) : p.scale_log2;
        for (int j = jx0; j < jx1 && !aborted; j++) {
            const int nd = j - jx0;
            const int c0 = j * BN;
            PP_WAIT(&bars->s_full[x], (uint32_t)(nd & 1));
            if (aborted) break;
            tc_fence_after();
            // Pass 1: the whole S row (128 registers) only for the row maximum; the registers are free again after it.
            const bool need_mask = (c0 + BN - 1 > r0) || (p.window > 0 && c0 < r0 + BM - p.window) || (c0 + BN > S);
            float tmax;
            {
                uint32_t v[128];
                tmem_ld32(tS, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
                tmem_ld32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
                tmem_ld32(tS + 64, *reinterpret_cast<uint32_t(*)[32]>(&v[64]));
                tmem_ld32(tS + 96, *reinterpret_cast<uint32_t(*)[32]>(&v[96]));
                tmem_wait_ld();
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 128; i++) {
                        const int col = c0 + i;
                        if (col > grow || col < row_lo || col >= S) v[i] = 0xff800000u;   // -inf
                    }
                }
                // eight independent chains instead of one 128-long dependency chain
                float mx[8];
#pragma unroll
                for (int c = 0; c < 8; c++) mx[c] = __uint_as_float(v[c]);
#pragma unroll
                for (int i = 8; i < 120; i += 16)
#pragma unroll
                    for (int c = 0; c < 8; c++) mx[c] = fmax3(mx[c], __uint_as_float(v[i + c]), __uint_as_float(v[i + 8 + c]));
#pragma unroll
                for (int c = 0; c < 8; c++) mx[c] = fmaxf(mx[c], __uint_as_float(v[120 + c]));
                tmax = fmax3(fmax3(mx[0], mx[1], mx[2]), fmax3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7]));
            }
            tmax *= scale_log2;
            const bool bump = tmax > m_ref + 8.0f;
            float alpha = 1.0f;
            if (bump) { alpha = fast_exp2(m_ref - tmax); m_ref = tmax; }
            // O_x is stable here: S_x(j) complete implies PV(x, j-1) complete (in-order tensor pipe)
            if (nd >= 1 && __any_sync(0xffffffffu, bump)) {
#pragma unroll 1
                for (int ch = 0; ch < HD / 32; ch++) {
                    uint32_t o[32];
                    tmem_ld32(tO + ch * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(tO + ch * 32, o);
                }
                tmem_wait_st();
            }
            l_sum *= alpha;
            const float neg_m = (m_ref == -CUDART_INF_F) ? 0.0f : -m_ref;
            // p = exp2(s * scale - m) -> bf16 pairs, written over the first 64 columns of S_x.
            // Pass 2: the row again, 64 columns at a time (the second warp of the scheduler covers the load).
            float ls[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t u[64];
                tmem_ld32(tS + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&u[0]));
                tmem_ld32(tS + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&u[32]));
                tmem_wait_ld();
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 64; i++) {
                        const int col = c0 + half * 64 + i;
                        if (col > grow || col < row_lo || col >= S) u[i] = 0xff800000u;   // -inf
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    float x0, x1;
                    ffma2(x0, x1, __uint_as_float(u[2 * i]), __uint_as_float(u[2 * i + 1]), scale_log2, neg_m);
                    float p0, p1;
                    if (POLY_EVERY > 0 && (i % POLY_EVERY) == POLY_EVERY - 1) exp2_poly2(p0, p1, x0, x1);   // one pair in POLY_EVERY on the FMA pipe
                    else { p0 = fast_exp2(x0); p1 = fast_exp2(x1); }
                    fadd2(ls[(2 * i) & 3], ls[(2 * i + 1) & 3], ls[(2 * i) & 3], ls[(2 * i + 1) & 3], p0, p1);
                    uint32_t w;
                    if (F16OPS) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(p1), "f"(p0));
                    else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(p1), "f"(p0));
                    u[i] = w;                      // packed in place: slot i was consumed already
                }
                // this half's P goes over columns [32 half, 32 half + 32): S columns that pass 2 has already read
                tmem_st32(tS + half * 32, *reinterpret_cast<uint32_t(*)[32]>(&u[0]));
            }
            l_sum += (ls[0] + ls[1]) + (ls[2] + ls[3]);
            tmem_wait_st();
            tc_fence_before();
            ptx::mbar_arrive(&bars->p_full[x]);
        }
        // epilogue
        const int n_x = jx1 - jx0;
        if (!aborted && n_x > 0) PP_WAIT(&bars->o_final[x], 0);
        if (!aborted && n_x > 0) {
            tc_fence_after();
            float inv = l_sum > 0.0f ? 1.0f / l_sum : 0.0f;
            if (F16OPS && p.descale) inv *= __ldg(p.descale + 1);
            const size_t orow = (((size_t)b * S + grow) * p.num_heads + h) * HD;
#pragma unroll 1
            for (int ch = 0; ch < HD / 32; ch++) {
                uint32_t o[32];
                tmem_ld32(tO + ch * 32, o);
                tmem_wait_ld();
#ifdef FLARE_DEBUG_BOUNDS
                if (grow < S && (size_t)(orow + ch * 32 + 32) > (size_t)p.batch * S * p.num_heads * HD) flare_report(p.err, FLARE_ERR_BOUNDS);
#endif
                if (grow < S) {
                    if (p.out_dtype == FLARE_DT_F32) {
                        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + orow + ch * 32);
#pragma unroll
                        for (int i = 0; i < 8; i++)
                            dst[i] = make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                                                 __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
                    } else {
                        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + orow + ch * 32);
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            uint32_t w[4];
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                __nv_bfloat162 pb = __floats2bfloat162_rn(__uint_as_float(o[8 * i + 2 * k]) * inv, __uint_as_float(o[8 * i + 2 * k + 1]) * inv);
                                w[k] = *reinterpret_cast<uint32_t*>(&pb);
                            }
                            dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && bars->abort_flag) flare_report(p.err, FLARE_ERR_TIMEOUT);
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace

int flare_launch_prefill_pp(flare_attn_ctx* ctx, const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm,
                            const PrefillArgs& a) {
    PPParams p;
    p.out = a.out; p.out_dtype = a.out_dtype; p.batch = a.batch; p.seq_len = a.seq_len; p.num_heads = a.num_heads;
    p.num_kv_heads = a.num_kv_heads; p.window = a.window;
    p.scale_log2 = (1.0f / sqrtf((float)a.head_dim)) * 1.4426950408889634f;
    p.descale = a.descale;
    p.err = ctx->d_err;
    dim3 grid((a.seq_len + 2 * BM - 1) / (2 * BM), a.num_heads, a.batch);
    // one CTA per SM: it owns all 512 tensor-memory columns
    const int smem128 = SmemPP<128>::TOTAL + 1024;
    const int smem64 = (SmemPP<64>::TOTAL + 1024) > 120 * 1024 ? (SmemPP<64>::TOTAL + 1024) : 120 * 1024;
#define PP_LAUNCH(HD_, F16_, SMEM_)                                                                                     \
    do {                                                                                                                \
        FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(prefill_pp_kernel<HD_, F16_>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_)); \
        prefill_pp_kernel<HD_, F16_><<<grid, 320, SMEM_, ctx->stream>>>(qm, km, vm, p);                                  \
    } while (0)
    if (a.head_dim == 128) {
        if (a.f16_ops) PP_LAUNCH(128, true, smem128); else PP_LAUNCH(128, false, smem128);
    } else {
        if (a.f16_ops) PP_LAUNCH(64, true, smem64); else PP_LAUNCH(64, false, smem64);
    }
#undef PP_LAUNCH
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}
