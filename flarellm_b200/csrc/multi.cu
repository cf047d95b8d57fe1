// One sequence whose KV cache is split along the slot axis over several GPUs (one process per GPU).
//
// The reference is single-device; this is the block form of its online-softmax recurrence
// (flare-core/src/model.rs:9945-9956): every rank attends its own slot range and holds, per query head, a
// record [m, l, o[head_dim]] (reference maximum, sum, unnormalised output); the records of all ranks are
// combined by log-sum-exp:   m* = max_r m_r,  l = sum_r l_r e^(m_r - m*),  o = sum_r o_r e^(m_r - m*) / l.
//
// Two ways to exchange the records (num_heads * (head_dim + 2) floats per rank, 16.6 KB at 32 x 128):
//   NCCL     ncclAllGather on the context's stream, then a merge kernel.  Always available after
//            flare_attn_comm_init.  NCCL is loaded at run time (libnccl.so.2); the library does not link it.
//   direct   after flare_attn_comm_enable_direct every rank owns a record buffer that its peers have mapped
//            (CUDA IPC).  The kernel that merges a rank's slot ranges STORES the rank's record into slot `rank`
//            of every peer's buffer as 8-byte words {value, sequence number of the call}: an aligned 8-byte store
//            arrives whole, so a word whose number matches carries its value — no fence, no separate flag.  It
//            then polls the words of all ranks in its OWN buffer, with a time limit, and merges.  Peer memory is
//            only ever written with plain stores, never read, and no bulk copy touches it.
//            One kernel instead of a kernel, a collective and another kernel.
// Every rank makes the same sequence of multi-GPU calls; a rank that does not show up makes the others' wait run
// out: they report FLARE_ERR_TIMEOUT and stay usable.
#include "common.cuh"
#include <dlfcn.h>
#include <math_constants.h>
#include <algorithm>
#include <mutex>
#include <nccl.h>

#ifdef FLARE_TIMELINE
// Tuning aid (not part of the product build): thread 0 of every CTA of the exchange kernel stamps the global timer.
__device__ unsigned long long g_timeline_x[1024 * 8];
#define TLX_STAMP(k)                                                                                             \
    do {                                                                                                         \
        if (threadIdx.x == 0 && blockIdx.x < 1024) {                                                             \
            unsigned long long _t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t));                        \
            g_timeline_x[blockIdx.x * 8 + (k)] = _t;                                                             \
        }                                                                                                        \
    } while (0)
extern "C" __attribute__((visibility("default"))) int flare_debug_timeline_x(void* dst, size_t bytes) {
    return (int)cudaMemcpyFromSymbol(dst, g_timeline_x, bytes < sizeof(g_timeline_x) ? bytes : sizeof(g_timeline_x));
}
#else
#define TLX_STAMP(k) do { } while (0)
#endif

namespace {

constexpr int kMaxWorld = 16;
constexpr float kLn2 = 0.6931471805599453f;

// ---- NCCL through dlopen ---------------------------------------------------------------------------------
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    std::string why;            // why loading failed
};

NcclApi* nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* env = getenv("FLARE_NCCL_LIB");
        const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            if (!n || !*n) continue;
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
            api.why = dlerror();
        }
        if (!api.handle) return;
#define FLARE_NCCL_SYM(field, name)                                                         \
        api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, name));          \
        if (!api.field) { api.why = std::string("symbol not found: ") + name; api.handle = nullptr; return; }
        FLARE_NCCL_SYM(GetUniqueId, "ncclGetUniqueId")
        FLARE_NCCL_SYM(CommInitRank, "ncclCommInitRank")
        FLARE_NCCL_SYM(CommDestroy, "ncclCommDestroy")
        FLARE_NCCL_SYM(CommAbort, "ncclCommAbort")
        FLARE_NCCL_SYM(AllGather, "ncclAllGather")
        FLARE_NCCL_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
        FLARE_NCCL_SYM(GetErrorString, "ncclGetErrorString")
#undef FLARE_NCCL_SYM
    });
    return api.handle ? &api : nullptr;
}

}  // namespace

struct FlareComm {
    int rank = 0, world = 1;
    ncclComm_t comm = nullptr;
    // NCCL exchange: this rank's records and the gathered ones
    float* part = nullptr;
    float* gathered = nullptr;
    size_t part_floats = 0;
    // direct exchange
    bool direct = false;
    int rows_max = 0, hd_max = 0;
    char* local_buf = nullptr;            // [2 phases][world][rows_max][hd_max / 32][34] words of {f32 value, u32 call number}
    size_t buf_bytes = 0;
    void* peer_buf[kMaxWorld] = {};       // the same buffer of every rank as mapped here; [rank] = local_buf
    uint32_t seq = 0;
    unsigned wait_ms = 2000;
    float probe_us = 0.0f;               // time of one exchange measured at set-up, the slowest rank's median
};

namespace {

#define FLARE_NCCL_OK(ctx, api, expr)                                                                          \
    do {                                                                                                       \
        ncclResult_t _r = (expr);                                                                              \
        if (_r != ncclSuccess)                                                                                 \
            return flare_set_error((ctx), FLARE_ERR_NCCL, "%s failed: %s (%s:%d)", #expr, (api)->GetErrorString(_r), \
                                   __FILE__, __LINE__);                                                        \
    } while (0)

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}
constexpr int CW = 32;               // channels per CTA of the merge kernel
constexpr int WORDS = CW + 2;        // 8-byte words of one (row, channel chunk) record: o[32], m, l

struct ExchangeParams {
    uint2* rec[kMaxWorld];          // record buffer of rank r (as mapped in this process): [2][world][rows_max][chunks][WORDS]
    int rank, world, rows_max, chunks_max;
    int phase;                      // which half of the record buffers this call uses
    int fence;                      // issue a system-scope fence after the stores
    uint32_t seq;                   // this call's sequence number
    unsigned long long wait_ns;
    int* err;                       // status word (mapped host memory): written once, by a wait that ran out
    int* gaveup;                    // device memory: non-zero once a wait has run out on this context
};

__device__ __forceinline__ void st_word(uint2* p, float v, uint32_t seq) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(seq) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* p) {
    uint2 v; asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory"); return v;
}
// The same with acquire semantics at system scope: a load that must observe what another GPU has stored.
__device__ __forceinline__ uint2 ld_word_acquire(const uint2* p) {
    uint2 v; asm volatile("ld.acquire.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory"); return v;
}

enum { MODE_FINAL = 0, MODE_RECORD = 1, MODE_EXCHANGE = 2 };

// One CTA per (row, chunk of 32 channels); a row is one (sequence, query, head).  Merges the row's n_split
// slot-range records (maximum in log2 units, n_split <= 256) into one record for its channels, then
//   MODE_FINAL     writes the normalised output (a world of one rank)
//   MODE_RECORD    writes the record with the maximum in natural units to `out` [row][hd + 2] (NCCL exchange)
//   MODE_EXCHANGE  stores the record into every rank's buffer, waits for all ranks' records in its own buffer and
//                  writes the normalised output over all ranks
// The split records of a long-context call are a few MB spread over L2: many small CTAs with several loads in
// flight per thread fetch them far faster than one CTA per row.
template <int MODE>
__global__ void __launch_bounds__(256) merge_exchange_kernel(const float* __restrict__ work, int n_split, int hd,
                                                             ExchangeParams mp, float* __restrict__ out) {
    __shared__ float s_w[256];          // weight of each slot range
    __shared__ float s_red[8];
    __shared__ float s_part[16][CW];
    __shared__ float s_send[WORDS];
    __shared__ float s_recv[kMaxWorld][WORDS];
    __shared__ int s_fail, s_gaveup;
    TLX_STAMP(0);
    pdl_trigger();          // the next call's attention kernel may begin its prologue (it never writes what is read here)
    pdl_wait();             // the attention kernel has written every slot-range record
    TLX_STAMP(1);
    const int row = blockIdx.x, chunk = blockIdx.y, tid = threadIdx.x;
    const int rs = hd + 2;
    const float* base = work + (size_t)row * n_split * rs;
    // ---- weights of the slot ranges: one range per thread ------------------------------------------------
    float m_r = -CUDART_INF_F, l_r = 0.0f;
    if (tid < n_split) { l_r = base[tid * rs + 1]; if (l_r > 0.0f) m_r = base[tid * rs]; }
    float mm = m_r;
#pragma unroll
    for (int off = 16; off; off >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
    if ((tid & 31) == 0) s_red[tid >> 5] = mm;
    if (tid == 0) {
        s_fail = 0;
        if (MODE == MODE_EXCHANGE) s_gaveup = *reinterpret_cast<volatile int*>(mp.gaveup);
    }
    __syncthreads();
    mm = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; w++) mm = fmaxf(mm, s_red[w]);
    __syncthreads();
    const float w_r = l_r > 0.0f ? fast_exp2(m_r - mm) : 0.0f;
    s_w[tid] = w_r;
    float ll = l_r * w_r;
#pragma unroll
    for (int off = 16; off; off >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, off);
    if ((tid & 31) == 0) s_red[tid >> 5] = ll;
    __syncthreads();
    ll = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) ll += s_red[w];
    // ---- weighted sum of the ranges' outputs: 16 groups of 16 threads, a thread owns 2 channels ------------
    {
        const int grp = tid >> 4, c2 = (tid & 15) * 2;
        const float* src = base + 2 + chunk * CW + c2;
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 4
        for (int r = grp; r < n_split; r += 16) {
            const float2 v = *reinterpret_cast<const float2*>(src + (size_t)r * rs);
            const float w = s_w[r];
            a0 = fmaf(v.x, w, a0); a1 = fmaf(v.y, w, a1);
        }
        s_part[grp][c2] = a0; s_part[grp][c2 + 1] = a1;
    }
    __syncthreads();
    float val = 0.0f;
    if (tid < CW) {
#pragma unroll
        for (int k = 0; k < 16; k++) val += s_part[k][tid];
    }
    TLX_STAMP(2);
    const int d = chunk * CW + tid;         // channel of thread tid < CW
    if (MODE == MODE_FINAL) {
        if (tid < CW) out[(size_t)row * hd + d] = ll > 0.0f ? val / ll : 0.0f;
        return;
    }
    if (MODE == MODE_RECORD) {
        if (tid < CW) out[(size_t)row * rs + 2 + d] = val;
        if (chunk == 0 && tid == 0) { out[(size_t)row * rs] = ll > 0.0f ? mm * kLn2 : 0.0f; out[(size_t)row * rs + 1] = ll; }
        return;
    }
    if (tid < CW) s_send[tid] = val;
    if (tid == 0) { s_send[CW] = ll > 0.0f ? mm : 0.0f; s_send[CW + 1] = ll; }
    __syncthreads();
    // ---- this rank's record into slot `rank` of every rank's buffer: {value, call number} words ------------
    const size_t slot_words = (size_t)WORDS;
    const size_t my_slot = ((((size_t)mp.phase * mp.world + mp.rank) * mp.rows_max + row) * mp.chunks_max + chunk) * slot_words;
    // one destination GPU per store instruction: warp w serves ranks w, w + 8, ...
    for (int r = tid >> 5; r < mp.world; r += (int)(blockDim.x >> 5)) {
        uint2* dst = mp.rec[r] + my_slot;
        for (int i = tid & 31; i < WORDS; i += 32) st_word(dst + i, s_send[i], mp.seq);
    }
    if (mp.fence) __threadfence_system();
    TLX_STAMP(3);
    // ---- every rank's record of this (row, chunk) out of the own buffer: a word is there when its number matches.
    // Once a wait has run out on this context (flag in device memory set, not yet cleared by the host) the ranks are
    // out of step: the calls still queued behind it do not wait their full limit again, they give up at once.
    const unsigned long long t0 = global_ns();
    const unsigned long long limit = s_gaveup ? 0ull : mp.wait_ns;
    const size_t in_base = (((size_t)mp.phase * mp.world) * mp.rows_max + row) * mp.chunks_max + chunk;   // + r * rows_max * chunks_max
    const size_t in_rank_stride = (size_t)mp.rows_max * mp.chunks_max;
    // First one thread per rank waits for the LAST word of that rank's record, pausing between looks, so that the
    // wait costs a few loads per CTA rather than a poll by every thread.
    if (tid < mp.world) {
        const uint2* src = mp.rec[mp.rank] + (in_base + (size_t)tid * in_rank_stride) * slot_words + (WORDS - 1);
        for (;;) {
            if ((mp.fence & 2 ? ld_word_acquire(src) : ld_word(src)).y == mp.seq) break;
            if (global_ns() - t0 > limit) { s_fail = 1; break; }
            __nanosleep(200);
        }
    }
    __syncthreads();
    // Then every word is checked for itself (stores of different threads may arrive in any order), which now
    // almost always succeeds at the first look.
    for (int t = tid; t < WORDS * mp.world && !s_fail; t += blockDim.x) {
        const int r = t / WORDS, i = t % WORDS;
        const uint2* src = mp.rec[mp.rank] + (in_base + (size_t)r * in_rank_stride) * slot_words + i;
        bool ok = false;
        for (;;) {
            const uint2 v = (mp.fence & 2) ? ld_word_acquire(src) : ld_word(src);
            if (v.y == mp.seq) { s_recv[r][i] = __uint_as_float(v.x); ok = true; break; }
            if (global_ns() - t0 > limit) break;
            __nanosleep(100);
        }
        if (!ok) s_fail = 1;
    }
    __syncthreads();
    TLX_STAMP(5);
    if (s_fail) {       // a rank did not show up in time: report, leave zeros, return (the context stays usable)
        if (tid == 0) { *reinterpret_cast<volatile int*>(mp.gaveup) = 1; flare_report(mp.err, FLARE_ERR_TIMEOUT); }
        if (tid < CW) out[(size_t)row * hd + d] = 0.0f;
        return;
    }
    if (tid < CW) {
        float gm = -CUDART_INF_F;
        for (int r = 0; r < mp.world; r++)
            if (s_recv[r][CW + 1] > 0.0f) gm = fmaxf(gm, s_recv[r][CW]);
        float gl = 0.0f, go = 0.0f;
        for (int r = 0; r < mp.world; r++) {
            const float l2 = s_recv[r][CW + 1];
            const float w = l2 > 0.0f ? fast_exp2(s_recv[r][CW] - gm) : 0.0f;
            gl = fmaf(l2, w, gl);
            go = fmaf(s_recv[r][tid], w, go);
        }
        out[(size_t)row * hd + d] = gl > 0.0f ? go / gl : 0.0f;
    }
    TLX_STAMP(6);
}

template <int MODE>
int launch_merge_exchange(flare_attn_ctx* ctx, const float* work, int n_split, int rows, int hd, const ExchangeParams& mp,
                          float* out) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows, hd / CW);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
#ifdef FLARE_TUNE
    if (const char* e = getenv("FLARE_MX_NOPDL")) if (atoi(e)) cfg.numAttrs = 0;
#endif
    FLARE_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, merge_exchange_kernel<MODE>, work, n_split, hd, mp, out));
    FLARE_LAUNCH_CHECK(ctx);
    return FLARE_OK;
}

int ensure_nccl_buffers(flare_attn_ctx* ctx, FlareComm* c, size_t part_floats) {
    if (part_floats <= c->part_floats) return FLARE_OK;
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    cudaFree(c->part); cudaFree(c->gathered);
    c->part = c->gathered = nullptr; c->part_floats = 0;
    FLARE_CUDA_OK(ctx, cudaMalloc(&c->part, part_floats * sizeof(float)));
    FLARE_CUDA_OK(ctx, cudaMalloc(&c->gathered, part_floats * sizeof(float) * c->world));
    c->part_floats = part_floats;
    return FLARE_OK;
}

void fill_exchange_params(const FlareComm* c, ExchangeParams* mp, int* err, int* gaveup) {
    memset(mp, 0, sizeof(*mp));
    for (int r = 0; r < c->world; r++) mp->rec[r] = reinterpret_cast<uint2*>(c->peer_buf[r]);
    mp->rank = c->rank; mp->world = c->world; mp->rows_max = c->rows_max; mp->chunks_max = c->hd_max / CW;
    mp->wait_ns = (unsigned long long)c->wait_ms * 1000000ull;
    mp->err = err;
    mp->gaveup = gaveup;
    mp->fence = 0;
#ifdef FLARE_TUNE
    if (const char* e = getenv("FLARE_MX_FENCE")) mp->fence = atoi(e);
#endif
}

}  // namespace

void flare_comm_free(flare_attn_ctx* ctx) {
    FlareComm* c = ctx->comm;
    if (!c) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int r = 0; r < c->world; r++)
        if (r != c->rank && c->peer_buf[r]) cudaIpcCloseMemHandle(c->peer_buf[r]);
    cudaFree(c->local_buf);
    cudaFree(c->part); cudaFree(c->gathered);
    NcclApi* api = nccl_api();
    if (c->comm && api) api->CommDestroy(c->comm);
    delete c;
    ctx->comm = nullptr;
}

int flare_launch_merge_splits(flare_attn_ctx* ctx, const float* work, int n_split, int rows, int head_dim, float* out,
                              int want_partial) {
    ExchangeParams mp;
    memset(&mp, 0, sizeof(mp));
    return want_partial ? launch_merge_exchange<MODE_RECORD>(ctx, work, n_split, rows, head_dim, mp, out)
                        : launch_merge_exchange<MODE_FINAL>(ctx, work, n_split, rows, head_dim, mp, out);
}

int flare_multi_tail(flare_attn_ctx* ctx, const float* work, int n_split, int rows, int head_dim, float* out) {
    FlareComm* c = ctx->comm;
    ExchangeParams mp;
    memset(&mp, 0, sizeof(mp));
    if (!c || c->world == 1) {
        FLARE_TRY(launch_merge_exchange<MODE_FINAL>(ctx, work, n_split, rows, head_dim, mp, out));
        ctx->last_launch_overlappable = true;
        return FLARE_OK;
    }
    if (c->direct && rows <= c->rows_max && head_dim <= c->hd_max) {
        fill_exchange_params(c, &mp, ctx->d_err, ctx->d_gaveup);
        c->seq++;
        mp.seq = c->seq; mp.phase = (int)(c->seq & 1u);
        FLARE_TRY(launch_merge_exchange<MODE_EXCHANGE>(ctx, work, n_split, rows, head_dim, mp, out));
        ctx->last_launch_overlappable = true;
#ifdef FLARE_TUNE
        if (const char* e = getenv("FLARE_MX_NOPDL")) if (atoi(e)) ctx->last_launch_overlappable = false;
#endif
        return FLARE_OK;
    }
    NcclApi* api = nccl_api();
    if (!api) return flare_set_error(ctx, FLARE_ERR_NCCL, "NCCL is not loaded");
    const size_t part_floats = (size_t)rows * (head_dim + 2);
    FLARE_TRY(ensure_nccl_buffers(ctx, c, part_floats));
    FLARE_TRY(launch_merge_exchange<MODE_RECORD>(ctx, work, n_split, rows, head_dim, mp, c->part));
    FLARE_NCCL_OK(ctx, api, api->AllGather(c->part, c->gathered, part_floats, ncclFloat, c->comm, ctx->stream));
    ctx->last_launch_overlappable = false;
    return flare_launch_merge(ctx, c->gathered, part_floats, c->world, rows, head_dim, out, 0);
}

extern "C" {

int flare_attn_comm_unique_id(void* id_out) {
    if (!id_out) return FLARE_ERR_INVALID_ARG;
    NcclApi* api = nccl_api();
    if (!api) return FLARE_ERR_NCCL;
    static_assert(sizeof(ncclUniqueId) == FLARE_COMM_ID_BYTES, "FLARE_COMM_ID_BYTES must match ncclUniqueId");
    ncclUniqueId id;
    if (api->GetUniqueId(&id) != ncclSuccess) return FLARE_ERR_NCCL;
    memcpy(id_out, &id, sizeof(id));
    return FLARE_OK;
}

int flare_attn_comm_init(flare_attn_ctx* ctx, const void* id, int rank, int world) {
    if (!ctx) return FLARE_ERR_INVALID_ARG;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || (world > 1 && !id))
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_attn_comm_init: rank %d of %d (at most %d ranks)", rank, world, kMaxWorld);
    if (ctx->comm) return flare_set_error(ctx, FLARE_ERR_STATE, "this context already has a communicator");
    FLARE_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    FlareComm* c = new (std::nothrow) FlareComm();
    if (!c) return FLARE_ERR_OOM;
    c->rank = rank; c->world = world;
    if (world > 1) {
        NcclApi* api = nccl_api();
        if (!api) {
            delete c;
            return flare_set_error(ctx, FLARE_ERR_NCCL, "cannot load libnccl.so.2 (set FLARE_NCCL_LIB to its path)");
        }
        ncclUniqueId uid;
        memcpy(&uid, id, sizeof(uid));
        ncclResult_t r = api->CommInitRank(&c->comm, world, uid, rank);
        if (r != ncclSuccess) {
            delete c;
            return flare_set_error(ctx, FLARE_ERR_NCCL, "ncclCommInitRank failed: %s", api->GetErrorString(r));
        }
    }
    ctx->comm = c;
    return FLARE_OK;
}

int flare_attn_comm_destroy(flare_attn_ctx* ctx) {
    if (!ctx) return FLARE_ERR_INVALID_ARG;
    flare_comm_free(ctx);
    return FLARE_OK;
}

int flare_attn_comm_set_wait_ms(flare_attn_ctx* ctx, unsigned wait_ms) {
    if (!ctx || !ctx->comm) return FLARE_ERR_INVALID_ARG;
    if (wait_ms < 1 || wait_ms > 60000) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "wait limit %u ms outside [1, 60000]", wait_ms);
    ctx->comm->wait_ms = wait_ms;
    return FLARE_OK;
}

int flare_attn_comm_enable_direct(flare_attn_ctx* ctx, int max_rows, int head_dim) {
    if (!ctx || !ctx->comm) return FLARE_ERR_INVALID_ARG;
    FlareComm* c = ctx->comm;
    if (max_rows < 1 || max_rows > 65536 || (head_dim != 64 && head_dim != 128))
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_attn_comm_enable_direct: %d rows, head_dim %d", max_rows, head_dim);
    if (c->direct) return flare_set_error(ctx, FLARE_ERR_STATE, "the direct exchange is already set up");
    if (c->world == 1) return FLARE_OK;
    NcclApi* api = nccl_api();
    if (!api) return flare_set_error(ctx, FLARE_ERR_NCCL, "NCCL is not loaded");
    FLARE_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    c->buf_bytes = (size_t)2 * c->world * max_rows * (head_dim / CW) * WORDS * sizeof(uint2);
    FLARE_CUDA_OK(ctx, cudaMalloc(&c->local_buf, c->buf_bytes));
    FLARE_CUDA_OK(ctx, cudaMemsetAsync(c->local_buf, 0, c->buf_bytes, ctx->stream));
    // every rank's IPC handle to every rank (an all-gather of 64 bytes through device memory)
    cudaIpcMemHandle_t mine;
    FLARE_CUDA_OK(ctx, cudaIpcGetMemHandle(&mine, c->local_buf));
    char* d_tmp = nullptr;
    FLARE_CUDA_OK(ctx, cudaMalloc(&d_tmp, sizeof(mine) * (c->world + 1)));
    std::vector<cudaIpcMemHandle_t> all(c->world);
    int st = FLARE_OK;
    do {
        if (cudaMemcpyAsync(d_tmp, &mine, sizeof(mine), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) { st = FLARE_ERR_CUDA; break; }
        if (api->AllGather(d_tmp, d_tmp + sizeof(mine), sizeof(mine), ncclChar, c->comm, ctx->stream) != ncclSuccess) { st = FLARE_ERR_NCCL; break; }
        if (cudaMemcpyAsync(all.data(), d_tmp + sizeof(mine), sizeof(mine) * c->world, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess ||
            cudaStreamSynchronize(ctx->stream) != cudaSuccess) { st = FLARE_ERR_CUDA; break; }
    } while (0);
    cudaFree(d_tmp);
    if (st != FLARE_OK) {
        cudaGetLastError();
        cudaFree(c->local_buf); c->local_buf = nullptr;
        return flare_set_error(ctx, st, "exchange of the buffer handles failed");
    }
    for (int r = 0; r < c->world; r++) {
        if (r == c->rank) { c->peer_buf[r] = c->local_buf; continue; }
        cudaError_t e = cudaIpcOpenMemHandle(&c->peer_buf[r], all[r], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            for (int k = 0; k < r; k++)
                if (k != c->rank && c->peer_buf[k]) { cudaIpcCloseMemHandle(c->peer_buf[k]); c->peer_buf[k] = nullptr; }
            cudaFree(c->local_buf); c->local_buf = nullptr;
            return flare_set_error(ctx, FLARE_ERR_CUDA, "cudaIpcOpenMemHandle for rank %d failed: %s (one process per GPU, "
                                   "peer access between the GPUs, a shared IPC namespace are needed)", r, cudaGetErrorString(e));
        }
    }
    c->rows_max = max_rows; c->hd_max = head_dim; c->seq = 0;
    c->direct = true;
    // Probe: a few exchanges of one small record, timed on the device.  Peer stores normally arrive within a
    // microsecond or two; a machine on which they do not (peer access through the host bridge, a fabric in a
    // degraded state) is better served by NCCL's all-gather.  The slowest rank decides for everybody: above
    // 100 us per exchange the direct mode is switched off again and the calls use ncclAllGather.
    {
        const int probe_rounds = 12;
        float* work = nullptr;
        cudaEvent_t ev[2] = {nullptr, nullptr};
        float worst_us = 0.0f;
        int st = FLARE_OK;
        do {
            if (cudaMalloc(&work, (size_t)(head_dim + 2) * 4 + head_dim * 4 + 2 * sizeof(float)) != cudaSuccess ||
                cudaMemsetAsync(work, 0, (size_t)(head_dim + 2) * 4 + head_dim * 4, ctx->stream) != cudaSuccess ||
                cudaEventCreate(&ev[0]) != cudaSuccess || cudaEventCreate(&ev[1]) != cudaSuccess) { st = FLARE_ERR_CUDA; break; }
            // line the ranks up first (opening the peers' handles takes them different times)
            float* d_bar = nullptr;
            if (cudaMalloc(&d_bar, sizeof(float) * (c->world + 1)) != cudaSuccess) { st = FLARE_ERR_CUDA; break; }
            const bool lined_up = cudaMemsetAsync(d_bar, 0, sizeof(float) * (c->world + 1), ctx->stream) == cudaSuccess &&
                                  api->AllGather(d_bar, d_bar + 1, 1, ncclFloat, c->comm, ctx->stream) == ncclSuccess &&
                                  cudaStreamSynchronize(ctx->stream) == cudaSuccess;
            cudaFree(d_bar);
            if (!lined_up) { st = FLARE_ERR_NCCL; break; }
            std::vector<float> us;
            int probe_st = FLARE_OK;
            for (int i = 0; i < probe_rounds && probe_st == FLARE_OK; i++) {
                ExchangeParams mp;
                fill_exchange_params(c, &mp, ctx->d_err, ctx->d_gaveup);
                c->seq++;
                mp.seq = c->seq; mp.phase = (int)(c->seq & 1u);
                mp.wait_ns = 200ull * 1000000ull;
                ctx->last_launch_overlappable = false;
                cudaEventRecord(ev[0], ctx->stream);
                probe_st = launch_merge_exchange<MODE_EXCHANGE>(ctx, work, 1, 1, head_dim, mp, work + head_dim + 2);
                cudaEventRecord(ev[1], ctx->stream);
                if (probe_st == FLARE_OK && cudaEventSynchronize(ev[1]) != cudaSuccess) probe_st = FLARE_ERR_CUDA;
                if (probe_st != FLARE_OK) break;
                if (*reinterpret_cast<volatile int*>(ctx->h_err) != 0) { probe_st = FLARE_ERR_TIMEOUT; break; }
                float ms = 0.0f;
                cudaEventElapsedTime(&ms, ev[0], ev[1]);
                if (i >= 2) us.push_back(ms * 1e3f);           // the first rounds include what skew is left
            }
            // a rank whose probe failed still takes part in the vote below, with a time nobody accepts
            float median_us = 1.0e9f;
            if (probe_st == FLARE_OK && !us.empty()) {
                std::sort(us.begin(), us.end());
                median_us = us[us.size() / 2];
            }
            float* d_all = nullptr;
            if (cudaMalloc(&d_all, sizeof(float) * (c->world + 1)) != cudaSuccess) { st = FLARE_ERR_CUDA; break; }
            std::vector<float> all_med(c->world, 0.0f);
            bool ok = cudaMemcpyAsync(d_all, &median_us, sizeof(float), cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess &&
                      api->AllGather(d_all, d_all + 1, 1, ncclFloat, c->comm, ctx->stream) == ncclSuccess &&
                      cudaMemcpyAsync(all_med.data(), d_all + 1, sizeof(float) * c->world, cudaMemcpyDeviceToHost, ctx->stream) == cudaSuccess &&
                      cudaStreamSynchronize(ctx->stream) == cudaSuccess;
            cudaFree(d_all);
            if (!ok) { st = FLARE_ERR_NCCL; break; }
            for (float m : all_med) worst_us = m > worst_us ? m : worst_us;
        } while (0);
        cudaFree(work);
        if (ev[0]) cudaEventDestroy(ev[0]);
        if (ev[1]) cudaEventDestroy(ev[1]);
        // a probe that timed out has left a status behind: take it off the context
        if (*reinterpret_cast<volatile int*>(ctx->h_err) != 0) {
            *reinterpret_cast<volatile int*>(ctx->h_err) = 0;
            cudaMemsetAsync(ctx->d_gaveup, 0, sizeof(int), ctx->stream);
            if (st == FLARE_OK) st = FLARE_ERR_TIMEOUT;
        }
        c->probe_us = worst_us;
        if (st != FLARE_OK || worst_us > 100.0f) {
            c->direct = false;        // the buffers stay mapped until the communicator goes; the calls use ncclAllGather
            if (st != FLARE_OK) flare_set_error(ctx, FLARE_OK, "direct exchange probe failed (status %d): using ncclAllGather", st);
            else flare_set_error(ctx, FLARE_OK, "direct exchange probe: %.0f us per exchange on the slowest rank: using ncclAllGather", (double)worst_us);
        }
    }
    return FLARE_OK;
}

int flare_attn_comm_info(const flare_attn_ctx* ctx, int* rank, int* world, int* direct) {
    if (!ctx || !ctx->comm) return FLARE_ERR_INVALID_ARG;
    if (rank) *rank = ctx->comm->rank;
    if (world) *world = ctx->comm->world;
    if (direct) *direct = ctx->comm->direct ? 1 : 0;
    return FLARE_OK;
}

double flare_attn_comm_probe_us(const flare_attn_ctx* ctx) { return ctx && ctx->comm ? (double)ctx->comm->probe_us : 0.0; }

int flare_decode_attn_splitkv_multi(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads, const float* q,
                                    int n_local_slots, float* out, int on_device) {
    if (!ctx) return FLARE_ERR_INVALID_ARG;
    if (!kv) return flare_set_error(ctx, FLARE_ERR_STATE, "no KV cache");
    if (n_local_slots < 0 || n_local_slots > kv->max_seq_len)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "n_local_slots %d outside [0, %d]", n_local_slots, kv->max_seq_len);
    if (ctx->comm && ctx->comm->comm) {          // surface an asynchronous NCCL failure before queueing more work
        NcclApi* api = nccl_api();
        ncclResult_t ar = ncclSuccess;
        if (api && api->CommGetAsyncError(ctx->comm->comm, &ar) == ncclSuccess && ar != ncclSuccess && ar != ncclInProgress)
            return flare_set_error(ctx, FLARE_ERR_NCCL, "the communicator reported an asynchronous error: %s", api->GetErrorString(ar));
    }
    if (ctx->comm && ctx->comm->world > 1 && *reinterpret_cast<volatile int*>(ctx->h_err) != 0)
        return flare_set_error(ctx, *reinterpret_cast<volatile int*>(ctx->h_err),
                               "an earlier multi-GPU call on this context gave up waiting for a peer rank; read the status "
                               "(flare_attn_sync) and re-create the communicator on every rank before calling again");
    std::vector<int> att(kv->batch, n_local_slots);
    return flare_decode_common(ctx, kv, layer, num_heads, q, 1, att.data(), 0.0f, 0, n_local_slots, 1, 0, out, on_device,
                               nullptr, 1);
}

// Exercises the give-up path of the direct exchange on one GPU without a second rank and without a fault:
// a two-rank exchange is laid out in this device's own memory, rank 1 never publishes, the wait (50 ms) runs
// out.  Expected return value: FLARE_ERR_TIMEOUT; the context stays usable.
int flare_attn_comm_selftest_missing_peer(flare_attn_ctx* ctx) {
    if (!ctx) return FLARE_ERR_INVALID_ARG;
    FLARE_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const int hd = 64, rows = 2, world = 2;
    const size_t buf_bytes = ((size_t)2 * world * rows * (hd / CW) * WORDS * sizeof(uint2) + 255) / 256 * 256;
    char* bufs = nullptr;
    float* work = nullptr;
    FLARE_CUDA_OK(ctx, cudaMalloc(&bufs, 2 * buf_bytes));
    if (cudaMalloc(&work, (size_t)rows * (hd + 2) * 4 + rows * hd * 4) != cudaSuccess) { cudaFree(bufs); cudaGetLastError(); return FLARE_ERR_OOM; }
    cudaMemsetAsync(bufs, 0, 2 * buf_bytes, ctx->stream);
    cudaMemsetAsync(work, 0, (size_t)rows * (hd + 2) * 4 + rows * hd * 4, ctx->stream);
    ExchangeParams mp;
    memset(&mp, 0, sizeof(mp));
    for (int r = 0; r < world; r++) mp.rec[r] = reinterpret_cast<uint2*>(bufs + r * buf_bytes);
    mp.rank = 0; mp.world = world; mp.rows_max = rows; mp.chunks_max = hd / CW; mp.phase = 1; mp.seq = 1;
    mp.wait_ns = 50ull * 1000000ull;
    mp.err = ctx->d_err;
    mp.gaveup = ctx->d_gaveup;
    ctx->last_launch_overlappable = false;
    int st = launch_merge_exchange<MODE_EXCHANGE>(ctx, work, 1, rows, hd, mp, work + (size_t)rows * (hd + 2));
    if (st == FLARE_OK) st = flare_check_device_error(ctx);
    else cudaStreamSynchronize(ctx->stream);
    cudaFree(bufs); cudaFree(work);
    return st;
}

}  // extern "C"
