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
//            of every peer's buffer, publishes a sequence number per (rank, row) with a system-scope release
//            store, waits — with a time limit — until the numbers of all ranks have arrived in its OWN buffer,
//            and merges.  Peer memory is only ever written, never read, and no bulk or multicast copy touches it.
//            One kernel instead of a kernel, a collective and another kernel.
// Every rank makes the same sequence of multi-GPU calls; a rank that does not show up makes the others' wait run
// out: they report FLARE_ERR_TIMEOUT and stay usable.
#include "common.cuh"
#include <dlfcn.h>
#include <math_constants.h>
#include <mutex>
#include <nccl.h>

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
    char* local_buf = nullptr;            // [2 phases][world][rows_max][hd_max + 2] f32, then flags [world][rows_max] u32
    size_t flags_off = 0, buf_bytes = 0;
    void* peer_buf[kMaxWorld] = {};       // the same buffer of every rank as mapped here; [rank] = local_buf
    uint32_t seq = 0;
    unsigned wait_ms = 2000;
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
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}

struct ExchangeParams {
    float* rec[kMaxWorld];          // record buffer of rank r (as mapped in this process)
    uint32_t* flags[kMaxWorld];     // flag array of rank r
    int rank, world, rows_max, rec_stride;   // rec_stride: floats per record slot (hd_max + 2)
    int phase;                      // which half of the record buffers this call uses
    uint32_t seq;                   // this call's sequence number
    unsigned long long wait_ns;
    int* err;
};

enum { MODE_FINAL = 0, MODE_RECORD = 1, MODE_EXCHANGE = 2 };

// One CTA per (sequence, query, head) row.  Merges the row's n_split slot-range records (maximum in log2
// units) into one record, then
//   MODE_FINAL     writes the normalised output (a world of one rank)
//   MODE_RECORD    writes the record with the maximum in natural units to `out` [row][hd + 2] (NCCL exchange)
//   MODE_EXCHANGE  stores the record into every rank's buffer, publishes, waits for all ranks' records in its own
//                  buffer and writes the normalised output over all ranks
template <int MODE>
__global__ void __launch_bounds__(256) merge_exchange_kernel(const float* __restrict__ work, int n_split, int hd,
                                                             ExchangeParams mp, float* __restrict__ out) {
    __shared__ float s_w[256];          // weight of each slot range (n_split <= 256)
    __shared__ float s_red[8];
    __shared__ float s_part[256];
    __shared__ float s_rec[258];        // this rank's record of the row
    __shared__ int s_fail;
    pdl_trigger();          // the next call's attention kernel may begin its prologue (it never writes what is read here)
    pdl_wait();             // the attention kernel has written every slot-range record
    const int row = blockIdx.x, tid = threadIdx.x, nthr = blockDim.x;
    const float* base = work + (size_t)row * n_split * (hd + 2);
    float mm = -CUDART_INF_F;
    for (int r = tid; r < n_split; r += nthr)
        if (base[r * (hd + 2) + 1] > 0.0f) mm = fmaxf(mm, base[r * (hd + 2)]);
#pragma unroll
    for (int off = 16; off; off >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
    if ((tid & 31) == 0) s_red[tid >> 5] = mm;
    if (tid == 0) s_fail = 0;
    __syncthreads();
    mm = s_red[0];
    for (int w = 1; w < (nthr + 31) / 32; w++) mm = fmaxf(mm, s_red[w]);
    __syncthreads();
    float ll = 0.0f;
    for (int r = tid; r < n_split; r += nthr) {
        const float l_r = base[r * (hd + 2) + 1];
        const float w = l_r > 0.0f ? fast_exp2(base[r * (hd + 2)] - mm) : 0.0f;
        s_w[r] = w;
        ll += l_r * w;
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, off);
    if ((tid & 31) == 0) s_red[tid >> 5] = ll;
    __syncthreads();
    ll = 0.0f;
    for (int w = 0; w < (nthr + 31) / 32; w++) ll += s_red[w];
    const int groups = nthr / hd, grp = tid / hd, d = tid % hd;
    float acc = 0.0f;
    if (grp < groups) {
#pragma unroll 4
        for (int r = grp; r < n_split; r += groups) acc = fmaf(base[r * (hd + 2) + 2 + d], s_w[r], acc);
    }
    s_part[tid] = acc;
    __syncthreads();
    if (tid < hd) {
        for (int k = 1; k < groups; k++) acc += s_part[k * hd + tid];
        if (MODE == MODE_FINAL) out[(size_t)row * hd + tid] = ll > 0.0f ? acc / ll : 0.0f;
        else if (MODE == MODE_RECORD) out[(size_t)row * (hd + 2) + 2 + tid] = acc;
        else s_rec[2 + tid] = acc;
    }
    if (MODE == MODE_FINAL) return;
    if (MODE == MODE_RECORD) {
        if (tid == 0) {
            out[(size_t)row * (hd + 2)] = ll > 0.0f ? mm * kLn2 : 0.0f;
            out[(size_t)row * (hd + 2) + 1] = ll;
        }
        return;
    }
    if (tid == 0) { s_rec[0] = ll > 0.0f ? mm : 0.0f; s_rec[1] = ll; }
    __syncthreads();

    // ---- this rank's record into slot `rank` of every rank's buffer (plain stores; the own buffer included) ----
    const size_t slot_off = ((size_t)(mp.phase * mp.world + mp.rank) * mp.rows_max + row) * mp.rec_stride;
    for (int r = 0; r < mp.world; r++) {
        float* dst = mp.rec[r] + slot_off;
        for (int i = tid; i < hd + 2; i += nthr) dst[i] = s_rec[i];
    }
    __threadfence_system();             // each thread's stores are ordered before what follows, system-wide
    __syncthreads();
    if (tid < mp.world) st_release_sys(mp.flags[tid] + (size_t)mp.rank * mp.rows_max + row, mp.seq);
    // ---- wait until every rank's record of this row has arrived here (own memory, bounded) -----------------
    if (tid < mp.world) {
        const uint32_t* f = mp.flags[mp.rank] + (size_t)tid * mp.rows_max + row;
        const unsigned long long t0 = global_ns();
        bool ok = false;
        for (;;) {
            if (ld_acquire_sys(f) == mp.seq) { ok = true; break; }
            if (global_ns() - t0 > mp.wait_ns) break;
            __nanosleep(100);
        }
        if (!ok) s_fail = 1;
    }
    __syncthreads();
    if (s_fail) {       // a rank did not show up in time: report, leave zeros, return (the context stays usable)
        if (tid == 0) atomicExch(mp.err, FLARE_ERR_TIMEOUT);
        if (tid < hd) out[(size_t)row * hd + tid] = 0.0f;
        return;
    }
    // ---- merge the ranks' records (read past L1: they were written by other GPUs) ---------------------------
    if (tid < hd) {
        const float* mine = mp.rec[mp.rank] + ((size_t)(mp.phase * mp.world) * mp.rows_max + row) * mp.rec_stride;
        const size_t rank_stride = (size_t)mp.rows_max * mp.rec_stride;
        float gm = -CUDART_INF_F;
        for (int r = 0; r < mp.world; r++)
            if (__ldcg(mine + r * rank_stride + 1) > 0.0f) gm = fmaxf(gm, __ldcg(mine + r * rank_stride));
        float gl = 0.0f, go = 0.0f;
        for (int r = 0; r < mp.world; r++) {
            const float l_r = __ldcg(mine + r * rank_stride + 1);
            const float w = l_r > 0.0f ? fast_exp2(__ldcg(mine + r * rank_stride) - gm) : 0.0f;
            gl = fmaf(l_r, w, gl);
            go = fmaf(__ldcg(mine + r * rank_stride + 2 + tid), w, go);
        }
        out[(size_t)row * hd + tid] = gl > 0.0f ? go / gl : 0.0f;
    }
}

template <int MODE>
int launch_merge_exchange(flare_attn_ctx* ctx, const float* work, int n_split, int rows, int hd, const ExchangeParams& mp,
                          float* out) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows);
    cfg.blockDim = dim3(256);           // a multiple of head_dim 64 / 128
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
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

void fill_exchange_params(const FlareComm* c, ExchangeParams* mp, int* err) {
    memset(mp, 0, sizeof(*mp));
    for (int r = 0; r < c->world; r++) {
        mp->rec[r] = reinterpret_cast<float*>(c->peer_buf[r]);
        mp->flags[r] = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(c->peer_buf[r]) + c->flags_off);
    }
    mp->rank = c->rank; mp->world = c->world; mp->rows_max = c->rows_max; mp->rec_stride = c->hd_max + 2;
    mp->wait_ns = (unsigned long long)c->wait_ms * 1000000ull;
    mp->err = err;
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
        fill_exchange_params(c, &mp, ctx->d_err);
        c->seq++;
        mp.seq = c->seq; mp.phase = (int)(c->seq & 1u);
        FLARE_TRY(launch_merge_exchange<MODE_EXCHANGE>(ctx, work, n_split, rows, head_dim, mp, out));
        ctx->last_launch_overlappable = true;
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
    const size_t rec_bytes = (size_t)2 * c->world * max_rows * (head_dim + 2) * sizeof(float);
    c->flags_off = (rec_bytes + 255) / 256 * 256;
    c->buf_bytes = c->flags_off + (size_t)c->world * max_rows * sizeof(uint32_t);
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
    return FLARE_OK;
}

int flare_attn_comm_info(const flare_attn_ctx* ctx, int* rank, int* world, int* direct) {
    if (!ctx || !ctx->comm) return FLARE_ERR_INVALID_ARG;
    if (rank) *rank = ctx->comm->rank;
    if (world) *world = ctx->comm->world;
    if (direct) *direct = ctx->comm->direct ? 1 : 0;
    return FLARE_OK;
}

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
    const size_t rec_floats = (size_t)2 * world * rows * (hd + 2);
    const size_t flags_off = (rec_floats * 4 + 255) / 256 * 256;
    const size_t buf_bytes = flags_off + world * rows * 4;
    char* bufs = nullptr;
    float* work = nullptr;
    FLARE_CUDA_OK(ctx, cudaMalloc(&bufs, 2 * buf_bytes + 256));
    if (cudaMalloc(&work, (size_t)rows * (hd + 2) * 4 + rows * hd * 4) != cudaSuccess) { cudaFree(bufs); cudaGetLastError(); return FLARE_ERR_OOM; }
    cudaMemsetAsync(bufs, 0, 2 * buf_bytes + 256, ctx->stream);
    cudaMemsetAsync(work, 0, (size_t)rows * (hd + 2) * 4 + rows * hd * 4, ctx->stream);
    ExchangeParams mp;
    memset(&mp, 0, sizeof(mp));
    for (int r = 0; r < world; r++) {
        mp.rec[r] = reinterpret_cast<float*>(bufs + r * ((buf_bytes + 255) / 256 * 256));
        mp.flags[r] = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(mp.rec[r]) + flags_off);
    }
    mp.rank = 0; mp.world = world; mp.rows_max = rows; mp.rec_stride = hd + 2; mp.phase = 1; mp.seq = 1;
    mp.wait_ns = 50ull * 1000000ull;
    mp.err = ctx->d_err;
    ctx->last_launch_overlappable = false;
    int st = launch_merge_exchange<MODE_EXCHANGE>(ctx, work, 1, rows, hd, mp, work + (size_t)rows * (hd + 2));
    if (st == FLARE_OK) st = flare_check_device_error(ctx);
    else cudaStreamSynchronize(ctx->stream);
    cudaFree(bufs); cudaFree(work);
    return st;
}

}  // extern "C"
