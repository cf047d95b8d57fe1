// Q8_0 split-KV decode attention, the bandwidth-bound fast path (head_dim 64 / 128, up to 4
// query heads per KV head, one query per sequence).
//
// One CTA = one (sequence, slot range), one warp per KV head.  Whole 32-slot tiles — every
// head's int8 K and V payload and the f16 scales, i.e. contiguous 16 KB + 1 KB pieces of each
// plane, which keeps DRAM pages open — stream into a ring of shared-memory stages through
// cp.async.bulk.tensor (hardware 64B/128B swizzle, landing as [head][slot][head_dim]) and
// cp.async.bulk, each stage guarded by an mbarrier.  There is no producer warp and no wait for
// a free stage: the last warp to finish with a stage (a shared-memory ticket) refills it.
// K/V are read from HBM exactly once for the 4 query heads sharing them.
//
// Dequantise-then-FMA on CUDA cores costs ~10 instructions per KV byte and cannot keep up with
// HBM, so both contractions run on tensor cores with the Q8_0 scales hoisted out of the sums:
//   scores  S[head, slot] = qs_head * sum_blk ks[slot, blk] * (Qint[head, blk, :] . Kint[slot, blk, :])
//           as an exact int8 MMA (m16n8k32): Qint is q * log2e/sqrt(d) in 15-bit fixed point per head,
//           carried as two int8 limbs (rows g and g+8 of the A operand).
//   output  O[head, d] = sum_slot (p * vs[slot, blk(d)]) * Vint[slot, d]
//           as an f16 MMA (m16n8k16, f32 accumulate): the weight p*vs is rounded to f16, Vint bytes
//           become exact f16 values 1024 + (v + 128) with one xor and one byte-permute per pair,
//           and the constant 1152 * sum(weights) is subtracted at the end.  V is transposed for
//           the MMA by ldmatrix.trans on the swizzled tile.
// Softmax is the single-pass online recurrence of flare-core/src/model.rs:9914-9966, applied to
// 32 slots at a time; ranges are merged by log-sum-exp (merge_partials_kernel).
#include "common.cuh"
#include "tma.cuh"
#include <math_constants.h>
#include <mutex>

#ifdef FLARE_TIMELINE
// Tuning aid (not part of the product build): thread 0 of every CTA stamps the global timer at eight points of
// the kernel into a device array that flare_debug_timeline copies out.
__device__ unsigned long long g_timeline[8192 * 8];
#define TL_STAMP(k)                                                                                              \
    do {                                                                                                         \
        if (threadIdx.x == 0) {                                                                                  \
            unsigned long long _t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t));                        \
            const unsigned _c = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;                  \
            if (_c < 8192) g_timeline[_c * 8 + (k)] = _t;                                                        \
        }                                                                                                        \
    } while (0)
extern "C" __attribute__((visibility("default"))) int flare_debug_timeline(void* dst, size_t bytes) {
    return (int)cudaMemcpyFromSymbol(dst, g_timeline, bytes < sizeof(g_timeline) ? bytes : sizeof(g_timeline));
}
#else
#define TL_STAMP(k) do { } while (0)
#endif

namespace {

// Guards the per-device tables below: two contexts on two host threads may make their first call at once.
std::mutex g_table_mutex;

constexpr int T = 32;            // slots per tile
constexpr int STAGES = 3;
constexpr int MAX_CLUSTER = 16;       // 9 .. 16 CTAs per cluster are beyond the portable size: opted into per kernel
constexpr int L2_AHEAD = 0;      // tiles requested into L2 ahead of the shared-memory copy (0: off; measured slower)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kQFix = 16256.0f;     // 127 * 128: |Qint| <= 16256 = 128 * limb0 + limb1

struct Q8Params {
    const float* q;
    float* out;
    float* work;
    const int* attend_len;
    const __half* k_scale;      // layer base, sequence 0
    const __half* v_scale;
    size_t scale_seq_stride;    // halves between sequences
    int layer_seq0;             // layer * batch: TMA coordinate of sequence 0
    int num_heads, nkv, G, max_seq, n_split, slot_begin, slot_end, want_partial, range_max;
    int n_small;             // > 0: attend_small[] holds the lengths (no global load before the first TMA request)
    int attend_small[64];
    int n_q, causal_q, hgroups;   // grid.z = n_q * hgroups: one query and one group of up to 4 of its heads per kv head
    int cluster;             // the n_split CTAs of a sequence form one thread-block cluster and merge through shared memory
    int whole_rows;             // 1: the maps deliver all heads of a tile in one copy; 0: one copy per head
    int prefetch_q;             // ask L2 for q's lines before waiting for the previous kernel
    int early_trigger;          // let the next kernel be scheduled as soon as this CTA has requested its first tiles
    int wait_first;             // the previous kernel may write the cache (a step write): wait for it before the first tile request
    int* err;
};

template <int HD> __device__ __forceinline__ uint32_t swz(int row, int chunk) {
    uint32_t off = (uint32_t)(row * HD + chunk * 16);
    constexpr uint32_t MASK = (HD == 64) ? 3u : 7u;
    return off ^ (((off >> 7) & MASK) << 4);
}

__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// register-only conversions (no address is taken, so nothing is forced into local memory)
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

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute
// may start while its predecessor in the stream is still running; pdl_wait() blocks until the
// predecessor has completed and its writes are visible, pdl_trigger() lets the successor start.
// Both are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Thread-block cluster: hardware barrier over all threads of all CTAs of the cluster, and loads from a
// peer CTA's shared memory (distributed shared memory).
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t cta_rank) {
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank)); return r;
}
__device__ __forceinline__ float cluster_ld(uint32_t addr) {
    float v; asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory"); return v;
}

// TWOQ: a warp's 16 MMA rows carry two work items (a query, or a group of 4 heads of a query) instead of one item
// twice: rows 0-3 / 8-11 the two limbs of the first, rows 4-7 / 12-15 of the second; in the output product row g
// carries the weights scaled for the first 32-channel block of a 64-channel tile and row g + 8 those for the second.
// Calls with several items per sequence (speculative verify, more than 4 query heads per KV head) then read the
// cache once per pair of items at nearly the cost of one.
template <int HD, bool TWOQ>
__global__ void __launch_bounds__(256) decode_q8_kernel(const __grid_constant__ CUtensorMap kmap,
                                                        const __grid_constant__ CUtensorMap vmap, Q8Params p) {
    constexpr int NB = HD / 32;        // Q8_0 blocks per head row
    constexpr int MT = NB / 2;         // M-tiles of the PV product (two 32-channel blocks each)
    constexpr int TILE = T * HD;       // bytes of one K (or V) tile
    constexpr int SCALE_ROW = 8 * NB * 2;   // bytes of one slot's scale row when nkv == 8 (runtime: p.nkv * NB * 2)
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ uint64_t full_bar[STAGES];
    __shared__ int done_cnt[STAGES];        // warps that have finished with the stage's current tile

    TL_STAMP(0);            // CTA started
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int split = blockIdx.x, b = blockIdx.y;
    const int nkv = p.nkv;
    const int kvh = warp;
    // stage layout: K payload [nkv][T][HD], V payload [nkv][T][HD], K scales [T][nkv*NB] f16, V scales
    const int payload = nkv * TILE;
    const int scale_tile = T * nkv * NB * 2;
    const int stage_bytes = 2 * payload + 2 * scale_tile;     // a multiple of 1024 (checked on the host)
    unsigned char* sbase = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    (void)SCALE_ROW;

    // blockIdx.z: which query of the sequence (speculative verify: query i sees n_q-1-i slots fewer) and which
    // group of up to 4 query heads per KV head; each such chunk streams the cache on its own
    const int n_items = p.n_q * p.hgroups;
    const int item = TWOQ ? min(2 * (int)blockIdx.z + (g >> 2), n_items - 1) : (int)blockIdx.z;     // this lane's item
    const bool item_ok = !TWOQ || 2 * (int)blockIdx.z + (g >> 2) < n_items;
    const int qi = item / p.hgroups, hg = item % p.hgroups;
    // slot range of this (sequence, query, split), in whole tiles.  With two items the tiles cover the longer of the two
    // ranges (the later query's); a lane masks what lies beyond its own.
    const int attend_b = p.n_small ? p.attend_small[b] : p.attend_len[b];
    int lo = 0, hi = max(0, attend_b - (p.causal_q ? (p.n_q - 1 - qi) : 0));
    int hi_lane = hi, hi_short = hi;
    if (TWOQ) {
        const int q_hi = min(2 * (int)blockIdx.z + 1, n_items - 1) / p.hgroups, q_lo = (2 * (int)blockIdx.z) / p.hgroups;
        hi = max(0, attend_b - (p.causal_q ? (p.n_q - 1 - q_hi) : 0));
        hi_short = max(0, attend_b - (p.causal_q ? (p.n_q - 1 - q_lo) : 0));
    }
    if (p.slot_end >= 0) { lo = max(lo, p.slot_begin); hi = min(hi, p.slot_end); hi_lane = min(hi_lane, p.slot_end); hi_short = min(hi_short, p.slot_end); }
    int t_first = lo / T, t_last = hi > lo ? (hi + T - 1) / T : t_first;
    const int n_tiles_seq = t_last - t_first;
    const int t_begin = t_first + (int)(((long long)split * n_tiles_seq) / p.n_split);
    const int t_end = t_first + (int)(((long long)(split + 1) * n_tiles_seq) / p.n_split);
    const int n_tiles = t_end - t_begin;

    const int bpr = nkv * NB;       // scale entries per slot row
    const unsigned char* ksg = reinterpret_cast<const unsigned char*>(p.k_scale + (size_t)b * p.scale_seq_stride);
    const unsigned char* vsg = reinterpret_cast<const unsigned char*>(p.v_scale + (size_t)b * p.scale_seq_stride);
    auto issue = [&](int i) {       // one thread: tile i of this CTA -> stage i % STAGES
        const int s = i % STAGES;
        unsigned char* st = sbase + (size_t)s * stage_bytes;
        const int slot0 = (t_begin + i) * T;
        const int rows = min(T, p.max_seq - slot0);            // scale rows that exist in the plane
        const uint32_t sbytes = (uint32_t)rows * bpr * 2;
        ptx::mbar_expect_tx(&full_bar[s], 2 * payload + 2 * sbytes);
        if (p.whole_rows) {
            ptx::tma_load_4d(st, &kmap, &full_bar[s], 0, slot0, 0, p.layer_seq0 + b);
            ptx::tma_load_4d(st + payload, &vmap, &full_bar[s], 0, slot0, 0, p.layer_seq0 + b);
        } else {
            for (int h = 0; h < nkv; h++) {
                ptx::tma_load_4d(st + h * TILE, &kmap, &full_bar[s], 0, h, slot0, p.layer_seq0 + b);
                ptx::tma_load_4d(st + payload + h * TILE, &vmap, &full_bar[s], 0, h, slot0, p.layer_seq0 + b);
            }
        }
        ptx::bulk_load(st + 2 * payload, ksg + (size_t)slot0 * bpr * 2, sbytes, &full_bar[s]);
        ptx::bulk_load(st + 2 * payload + scale_tile, vsg + (size_t)slot0 * bpr * 2, sbytes, &full_bar[s]);
    };
    // Shared memory can hold only ~2 tiles in flight per CTA, too few bytes to cover DRAM latency at
    // full bandwidth; tiles further ahead are therefore pulled into L2 first.
    auto prefetch = [&](int i) {
        const int slot0 = (t_begin + i) * T;
        if (p.whole_rows) {
            ptx::tma_prefetch_l2_4d(&kmap, 0, slot0, 0, p.layer_seq0 + b);
            ptx::tma_prefetch_l2_4d(&vmap, 0, slot0, 0, p.layer_seq0 + b);
        } else {
            for (int h = 0; h < nkv; h++) {
                ptx::tma_prefetch_l2_4d(&kmap, 0, h, slot0, p.layer_seq0 + b);
                ptx::tma_prefetch_l2_4d(&vmap, 0, h, slot0, p.layer_seq0 + b);
            }
        }
    };
    // Launched as a programmatic dependent in every case: after one of this path's own kernels the first tiles are
    // requested while that kernel drains; after anything else (a step write into the cache, above all) only the launch
    // latency is hidden and the kernel waits here before it touches the cache.
    if (p.wait_first) pdl_wait();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { ptx::mbar_init(&full_bar[s], 1); done_cnt[s] = 0; }
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
        for (int i = 0; i < STAGES && i < n_tiles; i++) issue(i);
        for (int i = STAGES; i < STAGES + L2_AHEAD && i < n_tiles; i++) prefetch(i);
    }
    // q was written by an earlier kernel of the stream: asking L2 for its lines ahead of the wait below is harmless
    // (L2 stays coherent with later writes) and takes a DRAM round trip out of the path between the wait and the
    // first product when q has been pushed out of L2 by the cache stream of the previous call
    if (!TWOQ && p.prefetch_q && (lane & 3) < NB) {
        const int hq0 = (lane >> 2) & 3;
        const int heads_here = min(4, p.G - 4 * (int)(blockIdx.z % p.hgroups));
        const size_t row0 = ((size_t)b * p.n_q + blockIdx.z / p.hgroups) * p.num_heads + warp * p.G + 4 * (blockIdx.z % p.hgroups) +
                            (hq0 < heads_here ? hq0 : 0);
        if ((lane >> 4) == 0)       // rows g and g + 4 are the same head: once is enough
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q + row0 * HD + (lane & 3) * 32));
    }
    __syncthreads();
    TL_STAMP(1);            // first tiles requested
    // The next kernel of the stream may be scheduled from here on: its CTAs take the places this grid's CTAs leave one
    // by one (and the SMs' free places at once), request their first tiles and wait for this grid to complete.
    if (p.early_trigger) pdl_trigger();

    // The K/V tiles requested above do not depend on the previous kernel in the stream (the previous
    // layer's attention); q does.
    pdl_wait();
    TL_STAMP(2);            // predecessor complete

    // ---- q as two int8 limbs per head, laid out as the A operand of m16n8k32 --------------
    const int hq = g & 3;                          // query head of this lane within the group
    const bool head_ok = item_ok && hq < min(4, p.G - 4 * hg);
    const size_t row = ((size_t)b * p.n_q + qi) * p.num_heads + kvh * p.G + 4 * hg + (head_ok ? hq : 0);
    uint32_t qa[NB][4];
    float qs;                                       // score = qs * sum_blk ks * (int dot)
    {
        const float sc = rsqrtf((float)HD) * kLog2e;
        float qv[NB][8];
        float amax = 0.0f;
#pragma unroll
        for (int blk = 0; blk < NB; blk++) {
            const float4* qp = reinterpret_cast<const float4*>(p.q + row * HD + blk * 32 + tig * 8);
            float4 x = __ldg(qp), y = __ldg(qp + 1);
            qv[blk][0] = x.x * sc; qv[blk][1] = x.y * sc; qv[blk][2] = x.z * sc; qv[blk][3] = x.w * sc;
            qv[blk][4] = y.x * sc; qv[blk][5] = y.y * sc; qv[blk][6] = y.z * sc; qv[blk][7] = y.w * sc;
#pragma unroll
            for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(qv[blk][i]));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float inv = amax > 0.0f ? kQFix / amax : 0.0f;
        qs = amax / kQFix;
        // rows g and g+4 both carry limb 0 of head g & 3 (rows g+8, g+12: limb 1), so the lanes that
        // own the second channel block of the PV operand get the same scores without a shuffle
        const bool limb_rows = head_ok;
#pragma unroll
        for (int blk = 0; blk < NB; blk++) {
            uint32_t l0[2] = {0, 0}, l1[2] = {0, 0};
#pragma unroll
            for (int i = 0; i < 8; i++) {
                int Q = __float2int_rn(qv[blk][i] * inv);
                int lo_limb = ((Q + 64) & 127) - 64;          // [-64, 63]
                int hi_limb = (Q - lo_limb) >> 7;              // exact: Q = 128 * hi + lo
                l0[i >> 2] |= (uint32_t)(hi_limb & 0xFF) << (8 * (i & 3));
                l1[i >> 2] |= (uint32_t)(lo_limb & 0xFF) << (8 * (i & 3));
            }
            qa[blk][0] = limb_rows ? l0[0] : 0u;   // row g,   k 0..15 half
            qa[blk][1] = limb_rows ? l1[0] : 0u;   // row g+8
            qa[blk][2] = limb_rows ? l0[1] : 0u;   // row g,   k 16..31 half
            qa[blk][3] = limb_rows ? l1[1] : 0u;
        }
    }

    // ---- running state ---------------------------------------------------------------------
    float acc[MT][4][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
            for (int e = 0; e < 2; e++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[mt][c][e][i] = 0.0f;
    float m_run = -CUDART_INF_F, l_run = 0.0f, lb[MT], lb2[MT];      // lb2: TWOQ, the second channel block's bias sum
#pragma unroll
    for (int mt = 0; mt < MT; mt++) { lb[mt] = 0.0f; lb2[mt] = 0.0f; }

    const int lane_blk = g >> 2;    // which block of an M-tile this lane's rows belong to

    // lane-constant shared-memory offsets.  The swizzle XORs the 16-byte chunk index with row bits
    // that are the same for every 8-slot step (rows advance by 8), so each address is
    // base(lane) + constant.
    uint32_t koff[NB];              // K bytes of slot g, channels blk*32 + 8*tig .. +7
#pragma unroll
    for (int blk = 0; blk < NB; blk++) koff[blk] = kvh * TILE + swz<HD>(g, blk * 2 + (tig >> 1)) + (tig & 1) * 8;
    uint32_t voff[MT][2];           // ldmatrix row address: V slot (mi&1)*8 + r, chunk 4mt + 2cp + (mi>>1)
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int cp = 0; cp < 2; cp++)
            voff[mt][cp] = payload + kvh * TILE + swz<HD>(((lane >> 3) & 1) * 8 + (lane & 7), 4 * mt + 2 * cp + (lane >> 4));
    // scales of slot 2*tig (+1) of each 8-slot step, this head: [slot][nkv*NB] f16
    const uint32_t ksoff = 2 * payload + (2 * tig * bpr + kvh * NB) * 2;
    const uint32_t vsoff = ksoff + scale_tile + (TWOQ ? 0 : lane_blk * 2);

    bool failed = false;
    TL_STAMP(3);            // q ready
    for (int i = 0; i < n_tiles; i++) {
        const int s = i % STAGES;
        const int slot0 = (t_begin + i) * T;
        if (!ptx::mbar_wait(&full_bar[s], (uint32_t)((i / STAGES) & 1))) { failed = true; break; }
        if (i == 0) TL_STAMP(4);        // first tile arrived
        const unsigned char* kt = sbase + (size_t)s * stage_bytes;
        const uint32_t vt = ptx::smem_u32(kt);

        // ---- scores: int8 MMA per 8-slot column tile and 32-channel block ------------------
        float sc[4][2], vs[MT][4][2];    // sc: integer-domain scores (score = qs * sc, qs >= 0)
        float vs2[TWOQ ? MT : 1][4][2];  // TWOQ: the scales of the second 32-channel block (vs holds the first)
        float tmax = -CUDART_INF_F;
        const bool edge_tile = (slot0 < lo) || (slot0 + T > (TWOQ ? hi_short : hi));      // warp-uniform
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
            for (int h = 0; h < NB / 2; h++) {
                // (blk 2h, blk 2h+1) scales of slots 8j + 2tig and 8j + 2tig + 1
                const float2 kf0 = unpack_half2(*reinterpret_cast<const uint32_t*>(kt + FLARE_CK(ksoff + (8 * j * bpr + 2 * h) * 2, 4, stage_bytes, p.err)));
                const float2 kf1 = unpack_half2(*reinterpret_cast<const uint32_t*>(kt + FLARE_CK(ksoff + ((8 * j + 1) * bpr + 2 * h) * 2, 4, stage_bytes, p.err)));
                if (TWOQ) {
                    const float2 v0 = unpack_half2(*reinterpret_cast<const uint32_t*>(kt + FLARE_CK(vsoff + (8 * j * bpr + 2 * h) * 2, 4, stage_bytes, p.err)));
                    const float2 v1 = unpack_half2(*reinterpret_cast<const uint32_t*>(kt + FLARE_CK(vsoff + ((8 * j + 1) * bpr + 2 * h) * 2, 4, stage_bytes, p.err)));
                    vs[h][j][0] = v0.x; vs2[h][j][0] = v0.y;
                    vs[h][j][1] = v1.x; vs2[h][j][1] = v1.y;
                } else {
                    vs[h][j][0] = __half2float(*reinterpret_cast<const __half*>(kt + FLARE_CK(vsoff + (8 * j * bpr + 2 * h) * 2, 2, stage_bytes, p.err)));
                    vs[h][j][1] = __half2float(*reinterpret_cast<const __half*>(kt + FLARE_CK(vsoff + ((8 * j + 1) * bpr + 2 * h) * 2, 2, stage_bytes, p.err)));
                }
#pragma unroll
                for (int bb = 0; bb < 2; bb++) {
                    const int blk = 2 * h + bb;
                    // B fragment: 8 contiguous bytes of slot 8j+g, channels blk*32 + 8*tig .. +7
                    const uint2 kb = *reinterpret_cast<const uint2*>(kt + FLARE_CK(koff[blk] + j * 8 * HD, 8, payload, p.err));
                    int d[4] = {0, 0, 0, 0};
                    mma_s8(d, qa[blk], kb.x, kb.y);
                    // rows g / g+8 = limb 0 / limb 1 of head g & 3; columns = slots 2tig, 2tig+1
                    s0 = fmaf(bb ? kf0.y : kf0.x, (float)(d[0] * 128 + d[2]), s0);
                    s1 = fmaf(bb ? kf1.y : kf1.x, (float)(d[1] * 128 + d[3]), s1);
                }
            }
            if (edge_tile) {       // only the first and last tile of a range hold slots outside it
                // A slot outside the range gets weight exp2(-inf) = 0, but its V scale may be anything: rows past
                // the end of the plane are never copied, so that part of the stage keeps what an earlier kernel
                // left in shared memory (possibly Inf or NaN bit patterns, and 0 * NaN = NaN).  Zero it as well.
                const int slot = slot0 + 8 * j + 2 * tig;
                const int hi_mine = TWOQ ? hi_lane : hi;
                if (slot < lo || slot >= hi_mine) {
                    s0 = -CUDART_INF_F;
#pragma unroll
                    for (int h = 0; h < NB / 2; h++) { vs[h][j][0] = 0.0f; if (TWOQ) vs2[h][j][0] = 0.0f; }
                }
                if (slot + 1 < lo || slot + 1 >= hi_mine) {
                    s1 = -CUDART_INF_F;
#pragma unroll
                    for (int h = 0; h < NB / 2; h++) { vs[h][j][1] = 0.0f; if (TWOQ) vs2[h][j][1] = 0.0f; }
                }
            }
            sc[j][0] = s0; sc[j][1] = s1;
            tmax = fmaxf(tmax, fmaxf(s0, s1));
        }
        tmax *= qs;
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        // Lazy rescaling: the reference maximum m_run only moves when the tile maximum exceeds it by
        // more than 2^8, so exponentials stay below 256 and the accumulators are rarely rescaled.
        const bool bump = tmax > m_run + 8.0f;          // also true for the first valid tile (m_run = -inf)
        if (__any_sync(0xffffffffu, bump)) {
            const float alpha = bump ? fast_exp2(m_run - tmax) : 1.0f;     // m_run = -inf -> 0 (nothing accumulated yet)
            if (bump) m_run = tmax;
            l_run *= alpha;
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                lb[mt] *= alpha;
                lb2[mt] *= alpha;
#pragma unroll
                for (int c = 0; c < 4; c++)
#pragma unroll
                    for (int e = 0; e < 2; e++)
#pragma unroll
                        for (int k = 0; k < 4; k++) acc[mt][c][e][k] *= alpha;
            }
        }
        // every tile of a non-empty range holds at least one slot of it, so m_run is finite from the
        // first tile on and a masked slot gives exp2(-inf) = 0
        float pw[4][2];
        // two items: a lane whose own range ends before this CTA's first tile has seen nothing yet (m_run = -inf)
        const float neg_m = (TWOQ && m_run == -CUDART_INF_F) ? 0.0f : -m_run;
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                pw[j][e] = fast_exp2(fmaf(sc[j][e], qs, neg_m));
                l_run += pw[j][e];
            }

        // ---- output: f16 MMA, weights p * vs split into hi + lo -----------------------------
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            uint32_t pa[2][4];   // A fragments of the two 16-slot k-steps
#pragma unroll
            for (int j = 0; j < 4; j++) {
                // weights rounded to f16 (relative error 2^-12, well inside the output tolerance); the
                // bias term uses the rounded weights so that it cancels exactly
                const uint32_t wb = pack_half2(pw[j][0] * vs[mt][j][0], pw[j][1] * vs[mt][j][1]);
                const float2 wf = unpack_half2(wb);
                lb[mt] += wf.x + wf.y;
                pa[j >> 1][(j & 1) * 2] = wb;             // a0 / a2: row g
                if (TWOQ) {                               // a1 / a3: row g+8, the weights for the second channel block
                    const uint32_t wb2 = pack_half2(pw[j][0] * vs2[mt][j][0], pw[j][1] * vs2[mt][j][1]);
                    const float2 wf2 = unpack_half2(wb2);
                    lb2[mt] += wf2.x + wf2.y;
                    pa[j >> 1][(j & 1) * 2 + 1] = wb2;
                } else {
                    pa[j >> 1][(j & 1) * 2 + 1] = 0u;     // a1 / a3: row g+8 unused
                }
            }
#pragma unroll
            for (int kstep = 0; kstep < 2; kstep++) {
#pragma unroll
                for (int cp = 0; cp < 2; cp++) {          // chunk pairs of this M-tile's 64 channels
                    uint32_t rr[4];
                    // a row of 16 bytes per lane, inside this head's V tile
                    ldmatrix_x4_trans(rr, vt + FLARE_CK(voff[mt][cp] + kstep * 16 * HD, 16, 2 * payload, p.err));
#pragma unroll
                    for (int k = 0; k < 4; k++) rr[k] ^= 0x80808080u;     // int8 -> uint8 (v + 128)
                    // bytes (slot a, ch 0), (slot a, ch 1), (slot a+1, ch 0), (slot a+1, ch 1) ->
                    // half2 (1024 + u[a][ch], 1024 + u[a+1][ch]) for ch = even / odd
#pragma unroll
                    for (int cc = 0; cc < 2; cc++) {
                        uint32_t b0e = __byte_perm(rr[2 * cc], 0x64646464u, 0x4240);
                        uint32_t b1e = __byte_perm(rr[2 * cc + 1], 0x64646464u, 0x4240);
                        uint32_t b0o = __byte_perm(rr[2 * cc], 0x64646464u, 0x4341);
                        uint32_t b1o = __byte_perm(rr[2 * cc + 1], 0x64646464u, 0x4341);
                        mma_f16(acc[mt][2 * cp + cc][0], pa[kstep], b0e, b1e);
                        mma_f16(acc[mt][2 * cp + cc][1], pa[kstep], b0o, b1o);
                    }
                }
            }
        }

        // ---- the last warp to finish with this stage refills it -------------------------------
        __syncwarp();
        if (lane == 0 && i + STAGES < n_tiles) {
            if (atomicAdd(&done_cnt[s], 1) == nkv - 1) {
                done_cnt[s] = 0;
                ptx::fence_proxy_async();
                issue(i + STAGES);
                if (i + STAGES + L2_AHEAD < n_tiles) prefetch(i + STAGES + L2_AHEAD);
            }
        }
    }
    TL_STAMP(5);            // warp 0 done with its tiles
    if (!p.early_trigger) pdl_trigger();          // the next kernel in the stream may be scheduled; it waits for this grid to finish
    if (failed) {
        if (lane == 0) flare_report(p.err, FLARE_ERR_TIMEOUT);
        if (!p.cluster) return;     // in a cluster every CTA still has to reach the barriers
    }

    // ---- finish: sums over the 4 lanes that share a row, remove the 1152 bias, write --------
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        lb[mt] += __shfl_xor_sync(0xffffffffu, lb[mt], 1);
        lb[mt] += __shfl_xor_sync(0xffffffffu, lb[mt], 2);
        if (TWOQ) {
            lb2[mt] += __shfl_xor_sync(0xffffffffu, lb2[mt], 1);
            lb2[mt] += __shfl_xor_sync(0xffffffffu, lb2[mt], 2);
        }
    }
    if (!TWOQ && p.cluster) {
        // The splits of this sequence are the CTAs of one cluster: every CTA leaves its (m, l, o) records
        // in its own shared memory, then each merges a share of the rows by reading its peers' records.
        __syncthreads();                                    // all warps are done with the stage buffers
        float* rec = reinterpret_cast<float*>(sbase);       // [num_heads][HD + 2]
        if (head_ok) {
            float* r = rec + (kvh * p.G + hq) * (HD + 2);
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const float bias = 1152.0f * lb[mt];
#pragma unroll
                for (int lc = 0; lc < 2; lc++) {
                    const int d0 = 64 * mt + 16 * (2 * lane_blk + lc) + 4 * tig;
                    r[2 + d0] = (lane_blk ? acc[mt][2 + lc][0][0] : acc[mt][lc][0][0]) - bias;
                    r[2 + d0 + 1] = (lane_blk ? acc[mt][2 + lc][1][0] : acc[mt][lc][1][0]) - bias;
                    r[2 + d0 + 2] = (lane_blk ? acc[mt][2 + lc][0][1] : acc[mt][lc][0][1]) - bias;
                    r[2 + d0 + 3] = (lane_blk ? acc[mt][2 + lc][1][1] : acc[mt][lc][1][1]) - bias;
                }
            }
            if (g < 4 && tig == 0) { r[0] = m_run; r[1] = failed ? 0.0f : l_run; }
        }
        cluster_sync_all();
        const uint32_t rank = cluster_ctarank(), n = (uint32_t)p.n_split;
        const uint32_t rec0 = ptx::smem_u32(rec);
        for (int item = threadIdx.x;; item += blockDim.x) {
            const int r = (int)rank + (item / HD) * (int)n, d = item % HD;
            if (r >= p.num_heads) break;
            float mv[MAX_CLUSTER], lv[MAX_CLUSTER], ov[MAX_CLUSTER];
#pragma unroll
            for (uint32_t s2 = 0; s2 < MAX_CLUSTER; s2++) {
                if (s2 < n) {
                    const uint32_t a = cluster_map(rec0 + (uint32_t)r * (HD + 2) * 4, s2);
                    mv[s2] = cluster_ld(a); lv[s2] = cluster_ld(a + 4); ov[s2] = cluster_ld(a + (2 + d) * 4);
                } else { mv[s2] = 0.0f; lv[s2] = 0.0f; ov[s2] = 0.0f; }
            }
            float mm = -CUDART_INF_F;
#pragma unroll
            for (int s2 = 0; s2 < MAX_CLUSTER; s2++) if (lv[s2] > 0.0f) mm = fmaxf(mm, mv[s2]);
            float ll = 0.0f, o = 0.0f;
#pragma unroll
            for (int s2 = 0; s2 < MAX_CLUSTER; s2++) {
                const float w = lv[s2] > 0.0f ? fast_exp2(mv[s2] - mm) : 0.0f;
                ll = fmaf(lv[s2], w, ll);
                o = fmaf(ov[s2], w, o);
            }
            p.out[((size_t)b * p.num_heads + r) * HD + d] = ll > 0.0f ? o / ll : 0.0f;
        }
        cluster_sync_all();                                 // nobody leaves while a peer still reads its records
        return;
    }
    if (!head_ok) return;
    const bool final_out = (p.n_split == 1) && !p.want_partial;
    const float inv_l = l_run > 0.0f ? 1.0f / l_run : 0.0f;
    float* wrec = p.work + (row * p.n_split + split) * (HD + 2);
#ifdef FLARE_DEBUG_BOUNDS
    if (row >= (size_t)gridDim.y * p.n_q * p.num_heads || split >= p.n_split) { flare_report(p.err, FLARE_ERR_BOUNDS); return; }
#endif
    if (TWOQ) {
        // this lane's row: channels of the first block from row g (accumulator elements 0, 1), of the second from row g + 8
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
#pragma unroll
            for (int vb = 0; vb < 2; vb++) {
                const float bias = 1152.0f * (vb ? lb2[mt] : lb[mt]);
#pragma unroll
                for (int lc = 0; lc < 2; lc++) {
                    const int c = 2 * vb + lc, d0 = 64 * mt + 16 * c + 4 * tig;
                    const float o0 = acc[mt][c][0][2 * vb] - bias, o1 = acc[mt][c][1][2 * vb] - bias;
                    const float o2 = acc[mt][c][0][2 * vb + 1] - bias, o3 = acc[mt][c][1][2 * vb + 1] - bias;
                    if (final_out) {
                        *reinterpret_cast<float4*>(p.out + row * HD + d0) = make_float4(o0 * inv_l, o1 * inv_l, o2 * inv_l, o3 * inv_l);
                    } else {
                        *reinterpret_cast<float2*>(wrec + 2 + d0) = make_float2(o0, o1);
                        *reinterpret_cast<float2*>(wrec + 2 + d0 + 2) = make_float2(o2, o3);
                    }
                }
            }
        }
        if (!final_out && tig == 0) { wrec[0] = m_run; wrec[1] = l_run; }
    } else {
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const float bias = 1152.0f * lb[mt];
#pragma unroll
        for (int lc = 0; lc < 2; lc++) {
            // chunk 2*lane_blk + lc of the M-tile holds this lane's rows; select without a
            // lane-dependent array index (that would push the accumulators into local memory)
            const int d0 = 64 * mt + 16 * (2 * lane_blk + lc) + 4 * tig;
            float o0 = (lane_blk ? acc[mt][2 + lc][0][0] : acc[mt][lc][0][0]) - bias;   // channel d0
            float o1 = (lane_blk ? acc[mt][2 + lc][1][0] : acc[mt][lc][1][0]) - bias;   // d0 + 1
            float o2 = (lane_blk ? acc[mt][2 + lc][0][1] : acc[mt][lc][0][1]) - bias;   // d0 + 2
            float o3 = (lane_blk ? acc[mt][2 + lc][1][1] : acc[mt][lc][1][1]) - bias;   // d0 + 3
            if (final_out) {
                *reinterpret_cast<float4*>(p.out + row * HD + d0) = make_float4(o0 * inv_l, o1 * inv_l, o2 * inv_l, o3 * inv_l);
            } else {
                *reinterpret_cast<float2*>(wrec + 2 + d0) = make_float2(o0, o1);
                *reinterpret_cast<float2*>(wrec + 2 + d0 + 2) = make_float2(o2, o3);
            }
        }
    }
    if (!final_out && g < 4 && tig == 0) { wrec[0] = m_run; wrec[1] = l_run; }
    }
}

}  // namespace

bool flare_decode_q8_supported(const DecodeArgs& a) {
    const int hd = a.kv.head_dim, nkv = a.kv.num_kv_heads;
    // every stage must start on a 1024-byte boundary (swizzle) and the scale tile on 16 bytes
    const size_t stage = (size_t)nkv * 2 * T * hd + 2 * (size_t)T * nkv * (hd / 32) * 2;
    const int chunks = a.n_q * ((a.num_heads / nkv + 3) / 4);
    return a.kv.dtype == FLARE_KV_Q8_0 && (hd == 64 || hd == 128) && nkv <= 8 && chunks <= 64 && a.window == 0 &&
           a.kmap != nullptr && stage % 1024 == 0;
}

int flare_launch_decode_q8(flare_attn_ctx* ctx, const DecodeArgs& a) {
    const int hd = a.kv.head_dim, nkv = a.kv.num_kv_heads;
    const int rows = a.batch * a.n_q * a.num_heads;
    if (rows == 0) return FLARE_OK;
    Q8Params p;
    p.q = a.q; p.out = a.out; p.attend_len = a.attend_len;
    p.k_scale = reinterpret_cast<const __half*>(a.kv.plane[FLARE_PLANE_K_SCALE]);
    p.v_scale = reinterpret_cast<const __half*>(a.kv.plane[FLARE_PLANE_V_SCALE]);
    p.scale_seq_stride = a.kv.stride[FLARE_PLANE_K_SCALE] / 2;
    p.layer_seq0 = a.layer * a.batch;
    p.num_heads = a.num_heads; p.nkv = nkv; p.G = a.num_heads / nkv; p.max_seq = a.kv.max_seq_len;
    p.n_q = a.n_q; p.causal_q = a.causal_q; p.hgroups = (p.G + 3) / 4;
    p.n_small = 0;
    if (a.h_attend && a.batch <= 64) {
        p.n_small = a.batch;
        for (int b = 0; b < a.batch; b++) p.attend_small[b] = a.h_attend[b];
    }
    const int chunks = p.n_q * p.hgroups;
    p.slot_begin = a.slot_begin; p.slot_end = a.slot_end; p.want_partial = a.want_partial;
    p.range_max = a.slot_end >= 0 ? (a.slot_end - a.slot_begin) : a.max_attend;
    if (p.range_max < 0) p.range_max = 0;
    p.err = ctx->d_err;

    p.whole_rows = a.whole_rows;
    const size_t stage = (size_t)nkv * 2 * T * hd + 2 * (size_t)T * nkv * (hd / 32) * 2;
    const size_t smem = STAGES * stage + 1024;
    const int ctas_per_sm = smem <= 110 * 1024 ? 2 : 1;
    // one wave: as many splits as fit without a second, partly filled wave
    // several items (queries, groups of 4 heads) per sequence go two to a CTA
    const bool two_items = chunks >= 2;
    const int zdim = two_items ? (chunks + 1) / 2 : chunks;
    int n_split = (ctx->sm_count * ctas_per_sm) / (a.batch * zdim);
    // at least two tiles per CTA (four was the rule while a cluster held at most 8 CTAs; with 16 a short context at
    // a small batch is better served by more, shorter ranges: batch 4 x 4096 slots 11.7 -> 10.4 us per call, the
    // attention inside the single-token forward pass at 1024 slots 4 % of the whole token)
    // (slot-range calls and calls whose records another kernel merges keep four: twice the ranges are twice the
    // records for that kernel)
    int min_tiles = (a.defer_merge || a.want_partial || a.slot_end >= 0) ? 4 : 2;
#ifdef FLARE_TUNE
    if (const char* e = getenv("FLARE_Q8_MINTILES")) min_tiles = atoi(e);
#endif
    const int max_split = (p.range_max + min_tiles * T - 1) / (min_tiles * T);
    if (n_split > max_split) n_split = max_split;
    if (n_split < 1) n_split = 1;
    // Several queries (or head groups) per sequence and a wave filled to less than three quarters: two full waves of
    // shorter ranges keep every SM loaded twice (speculative verify, 6 queries x 32 sequences: 192 CTAs on 296 places
    // took 200 us per call, 576 CTAs take 158 us; 4, 8 and 16 ranges per query were slower)
    {
        const int units = a.batch * zdim, places = ctx->sm_count * ctas_per_sm;
        if (chunks > 1 && n_split * units * 4 < places * 3) {
            const int two_waves = (2 * places) / units;
            if (two_waves > n_split && two_waves <= max_split) n_split = two_waves;
        }
    }
    if (n_split > 256) n_split = 256;
    // Cluster mode: when a handful of splits per sequence fill the GPU anyway, the splits of a sequence become one
    // thread-block cluster (2 .. 16 CTAs; more than 8 is the non-portable size, opted into) and merge through distributed shared memory: no second kernel, no round
    // trip of the records through global memory.  The size is the largest one, not far below the number of splits
    // that would fit, for which every sequence's cluster is resident at once (a second wave costs more than the
    // merge kernel).  Measured and rejected: clusters of 9 for 32 sequences (only 30 are resident at once); records
    // pushed into the owner's shared memory with a single cluster barrier (warps that reach the cluster barrier
    // early poll it and slow the warps still streaming: 37.8 instead of 32.1 us per call).
    int cluster = 0;
    if (!a.want_partial && a.slot_end < 0 && n_split >= 2 && chunks == 1) {
        std::lock_guard<std::mutex> lock(g_table_mutex);
        // [device][hd == 128][size]: 0 = not asked yet.  Asked with the shapes of the first call (number of kv
        // heads); other shapes of the same head size have smaller or equal footprints
        static int max_clusters[64][2][MAX_CLUSTER + 1] = {};
        static bool attr_set[64][2] = {};
        bool& as = attr_set[ctx->device & 63][hd == 128];
        if (!as) {
            // the opt-in to large dynamic shared memory has to precede the occupancy queries
            const int max_smem = STAGES * (8 * 2 * T * hd + 2 * T * 8 * (hd / 32) * 2) + 1024;
            if (hd == 64) cudaFuncSetAttribute(decode_q8_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
            else cudaFuncSetAttribute(decode_q8_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
            if (hd == 64) cudaFuncSetAttribute(decode_q8_kernel<64, false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            else cudaFuncSetAttribute(decode_q8_kernel<128, false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            cudaGetLastError();
            as = true;
        }
        int c_max = MAX_CLUSTER;
#ifdef FLARE_TUNE
        if (const char* e = getenv("FLARE_Q8_CMAX")) c_max = atoi(e) > MAX_CLUSTER ? MAX_CLUSTER : atoi(e);
#endif
        int c_first = n_split > c_max ? c_max : n_split;
        bool forced = false;
#ifdef FLARE_TUNE
        if (const char* e = getenv("FLARE_Q8_CLUSTER")) { c_first = atoi(e) > MAX_CLUSTER ? MAX_CLUSTER : atoi(e); forced = true; }     // 0 or 1: no cluster
#endif
        for (int c = c_first; c >= 2 && !cluster; c--) {
            if (c * 5 < n_split * 4 && !forced) break;            // far fewer CTAs than places: the merge kernel is cheaper
            int& mc = max_clusters[ctx->device & 63][hd == 128][c];
            if (mc == 0) {
                cudaLaunchAttribute ca[1];
                ca[0].id = cudaLaunchAttributeClusterDimension;
                ca[0].val.clusterDim.x = c; ca[0].val.clusterDim.y = 1; ca[0].val.clusterDim.z = 1;
                cudaLaunchConfig_t qc = {};
                qc.gridDim = dim3(c, 1); qc.blockDim = dim3(32 * nkv); qc.dynamicSmemBytes = smem;
                qc.attrs = ca; qc.numAttrs = 1;
                int n = 0;
                cudaError_t e = hd == 64 ? cudaOccupancyMaxActiveClusters(&n, decode_q8_kernel<64, false>, &qc)
                                         : cudaOccupancyMaxActiveClusters(&n, decode_q8_kernel<128, false>, &qc);
                if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
                mc = n > 0 ? n : -1;
            }
            if (mc >= a.batch) cluster = c;
        }
    }
    if (cluster) n_split = cluster;
#ifdef FLARE_TUNE
    if (const char* e = getenv("FLARE_Q8_NSPLIT")) if (!cluster) n_split = atoi(e);
#endif
    p.n_split = n_split;
    p.cluster = cluster;
    // both measured on one GPU, 16 layer calls back to back: 31.3 -> 31.0 us at batch 32, 21.6 -> 20.7 at 16,
    // 56.7 -> 55.5 at 64 (13.95 -> 14.25 at batch 8)
    p.prefetch_q = 1;
    p.early_trigger = 1;
#ifdef FLARE_TUNE
    if (const char* e = getenv("FLARE_Q8_EARLYTRIG")) p.early_trigger = atoi(e);
    if (const char* e = getenv("FLARE_Q8_PREFQ")) p.prefetch_q = atoi(e);
#endif
    // two workspaces used alternately: the merge of one call may still be reading while the next
    // call's decode kernel (started early, see below) writes
    size_t need = ((size_t)rows * n_split * (hd + 2) * sizeof(float) + 255) / 256 * 256;
    FLARE_TRY(flare_ensure(ctx, &ctx->d_work, &ctx->work_bytes, 2 * need));
    ctx->work_phase ^= 1;
    p.work = (float*)((char*)ctx->d_work + (size_t)ctx->work_phase * need);

    // opt in to the large dynamic shared memory once per device
    {
        std::lock_guard<std::mutex> lock(g_table_mutex);
        static bool attr_done[64][2] = {};
        bool& done = attr_done[ctx->device & 63][hd == 128];
        if (!done) {
            const int max_smem = STAGES * (8 * 2 * T * hd + 2 * T * 8 * (hd / 32) * 2) + 1024;
            if (hd == 64) FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(decode_q8_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
            else FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(decode_q8_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
            done = true;
        }
    }
    // Programmatic dependent launch: when the previous kernel on this stream is one of this path's
    // own kernels (it never writes the cache), this kernel may start early and request its first
    // K/V tiles while the predecessor drains; it waits (pdl_wait) before touching q.
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster ? cluster : 1; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_split, a.batch, zdim);
    cfg.blockDim = dim3(32 * nkv);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    // the attributes in use are a contiguous run of attr[]: [PDL][cluster]
    p.wait_first = ctx->last_launch_overlappable ? 0 : 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1 + (cluster ? 1 : 0);
#ifdef FLARE_TUNE
    if (const char* e = getenv("FLARE_Q8_ALWAYS_PDL")) if (!atoi(e) && !ctx->last_launch_overlappable) { cfg.attrs = attr + 1; cfg.numAttrs = cluster ? 1 : 0; }
#endif
    if (two_items) {
        std::lock_guard<std::mutex> lock(g_table_mutex);
        static bool attr2_done[64][2] = {};
        bool& done2 = attr2_done[ctx->device & 63][hd == 128];
        if (!done2) {
            const int max_smem = STAGES * (8 * 2 * T * hd + 2 * T * 8 * (hd / 32) * 2) + 1024;
            if (hd == 64) FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(decode_q8_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
            else FLARE_CUDA_OK(ctx, cudaFuncSetAttribute(decode_q8_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
            done2 = true;
        }
    }
    if (two_items) {
        if (hd == 64) FLARE_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, decode_q8_kernel<64, true>, *a.kmap, *a.vmap, p));
        else FLARE_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, decode_q8_kernel<128, true>, *a.kmap, *a.vmap, p));
    } else {
        if (hd == 64) FLARE_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, decode_q8_kernel<64, false>, *a.kmap, *a.vmap, p));
        else FLARE_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, decode_q8_kernel<128, false>, *a.kmap, *a.vmap, p));
    }
    FLARE_LAUNCH_CHECK(ctx);
    ctx->last_launch_overlappable = true;
    if (a.defer_merge && a.want_partial) {          // the caller merges: tell it where the records are
        *a.work_out = p.work; *a.n_split_out = n_split;
        return FLARE_OK;
    }
    if (!cluster && (n_split > 1 || a.want_partial)) {
        // log-sum-exp merge of the slot ranges, chained with programmatic dependent launch (multi.cu)
        FLARE_TRY(flare_launch_merge_splits(ctx, p.work, n_split, rows, hd, a.out, a.want_partial));
        ctx->last_launch_overlappable = true;
    }
    return FLARE_OK;
}
