// The C ABI of libflare_attn.so: contexts, caches, argument checks, staging of host
// buffers, and dispatch to the kernels.  Declarations and reference citations are in
// include/flare_attn.h.
#include "common.cuh"
#include "tma.cuh"
#include <stdarg.h>
#include <new>

int flare_set_error(flare_attn_ctx* ctx, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) ctx->last_error = buf;
    return code;
}

int flare_ensure(flare_attn_ctx* ctx, void** buf, size_t* have, size_t need) {
    if (need <= *have) return FLARE_OK;
    // the old buffer may still be in use by queued work on the stream
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    if (*buf) FLARE_CUDA_OK(ctx, cudaFree(*buf));
    *buf = nullptr; *have = 0;
    size_t sz = need + need / 4 + 256;
    FLARE_CUDA_OK(ctx, cudaMalloc(buf, sz));
    *have = sz;
    return FLARE_OK;
}

int flare_ensure_pinned(flare_attn_ctx* ctx, size_t need) {
    if (need <= ctx->pinned_bytes) return FLARE_OK;
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->h_pinned) FLARE_CUDA_OK(ctx, cudaFreeHost(ctx->h_pinned));
    ctx->h_pinned = nullptr; ctx->pinned_bytes = 0;
    size_t sz = need + need / 4 + 4096;
    FLARE_CUDA_OK(ctx, cudaMallocHost(&ctx->h_pinned, sz));
    ctx->pinned_bytes = sz;
    return FLARE_OK;
}

KvLayerView flare_layer_view(const flare_kv* kv, int layer) {
    KvLayerView v;
    v.dtype = kv->dtype; v.batch = kv->batch; v.max_seq_len = kv->max_seq_len;
    v.num_kv_heads = kv->num_kv_heads; v.head_dim = kv->head_dim; v.kv_dim = kv->kv_dim;
    for (int i = 0; i < FLARE_PLANE_COUNT; i++) {
        v.plane[i] = kv->plane[i] ? kv->plane_ptr(i, layer, 0) : nullptr;
        v.stride[i] = kv->plane_bytes[i];
    }
    return v;
}

int flare_launch_decode(flare_attn_ctx* ctx, const DecodeArgs& a) {
    if (flare_decode_q8_supported(a)) { ctx->last_path = FLARE_PATH_Q8_TENSOR; return flare_launch_decode_q8(ctx, a); }
    if (a.kv_obj && flare_decode_g32_supported(a, a.kv_obj)) {
        ctx->last_path = FLARE_PATH_KIVI_TENSOR;
        return flare_launch_decode_g32(ctx, a, a.kv_obj);
    }
    ctx->last_path = FLARE_PATH_GENERAL;
    return flare_launch_decode_generic(ctx, a);
}

// A kernel whose bounded wait gave up leaves a status in the context's status word (mapped host memory);
// wait for the stream, read and clear it.
int flare_check_device_error(flare_attn_ctx* ctx) {
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    const int h = *reinterpret_cast<volatile int*>(ctx->h_err);
    if (h != 0) {
        *reinterpret_cast<volatile int*>(ctx->h_err) = 0;      // nothing is running on the stream
        cudaMemsetAsync(ctx->d_gaveup, 0, sizeof(int), ctx->stream);
        return flare_set_error(ctx, h, h == FLARE_ERR_TIMEOUT ? "a kernel gave up waiting (for its own memory copies, or for a peer rank's records): status %d"
                                                              : "a kernel reported status %d", h);
    }
    return FLARE_OK;
}

// One warp waits, with the same bounded helper the attention kernels use, on a barrier that nothing completes.
__global__ void selftest_wait_kernel(int* err, uint32_t limit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        ptx::fence_barrier_init();
        if (!ptx::mbar_wait(&bar, 0, limit)) flare_report(err, FLARE_ERR_TIMEOUT);
    }
}

// ---- per-call measurements -------------------------------------------------------------------
static int stats_fold(flare_attn_ctx* ctx) {       // bring the last measured call into the totals
    if (!ctx->stats_pending) return FLARE_OK;
    FLARE_CUDA_OK(ctx, cudaEventSynchronize(ctx->stats_ev[1]));
    float ms = 0.0f;
    FLARE_CUDA_OK(ctx, cudaEventElapsedTime(&ms, ctx->stats_ev[0], ctx->stats_ev[1]));
    flare_attn_stats& st = ctx->stats;
    const double us = (double)ms * 1e3, sec = (double)ms * 1e-3;
    st.calls++;
    st.last_op = ctx->stats_op;
    st.last_elapsed_us = us; st.last_bytes = ctx->stats_bytes; st.last_flops = ctx->stats_flops;
    st.last_gbs = sec > 0.0 ? ctx->stats_bytes / sec / 1e9 : 0.0;
    st.last_tflops = sec > 0.0 ? ctx->stats_flops / sec / 1e12 : 0.0;
    st.last_frac_of_peak = ctx->stats_op == FLARE_OP_PREFILL ? st.last_tflops / ctx->peak_tflops : st.last_gbs / ctx->peak_hbm_gbs;
    st.total_elapsed_us += us; st.total_bytes += ctx->stats_bytes; st.total_flops += ctx->stats_flops;
    ctx->stats_pending = false;
    return FLARE_OK;
}
static int stats_begin(flare_attn_ctx* ctx) {
    if (!ctx->stats_on) return FLARE_OK;
    FLARE_TRY(stats_fold(ctx));
    ctx->last_launch_overlappable = false;      // a measured call does not start inside its predecessor
    FLARE_CUDA_OK(ctx, cudaEventRecord(ctx->stats_ev[0], ctx->stream));
    return FLARE_OK;
}
static int stats_end(flare_attn_ctx* ctx, int op, double bytes, double flops) {
    if (!ctx->stats_on) return FLARE_OK;
    FLARE_CUDA_OK(ctx, cudaEventRecord(ctx->stats_ev[1], ctx->stream));
    ctx->stats_op = op; ctx->stats_bytes = bytes; ctx->stats_flops = flops;
    ctx->stats_pending = true;
    ctx->last_launch_overlappable = false;      // nor does its successor start inside it
    return FLARE_OK;
}
// K/V bytes that `slots` attended slots of one sequence occupy in the cache's storage format.
static double kv_bytes_of(const flare_kv* kv, double slots) {
    const double kvd = kv->kv_dim;
    switch (kv->dtype) {
        case FLARE_KV_F32: return slots * 2.0 * kvd * 4.0;
        case FLARE_KV_Q8_0: return slots * 2.0 * (kvd + kvd / 16.0);
        case FLARE_KV_KIVI_REF: return slots * (kvd / 2.0 + 8.0);
        default: {       // group-32 KIVI: the newest 128 tokens are f16 rows, the rest 0.75 bytes per value
            const double ring = slots < FLARE_G32_RESIDUAL ? slots : FLARE_G32_RESIDUAL;
            return (slots - ring) * 0.75 * kvd + ring * 2.0 * kvd * 2.0;
        }
    }
}

// The device's address of a page-locked host buffer, or null when the buffer is pageable.
static const float* device_view_of_host(const void* p) {
    cudaPointerAttributes pa;
    if (cudaPointerGetAttributes(&pa, p) == cudaSuccess && pa.type == cudaMemoryTypeHost && pa.devicePointer)
        return (const float*)pa.devicePointer;
    cudaGetLastError();
    return nullptr;
}

// The same question for an INPUT buffer, remembered per address: a wrong answer (memory freed and reused as pageable at
// the same address) only costs the copy its speed, never its correctness, which is why outputs are always asked anew.
static bool input_is_locked(flare_attn_ctx* ctx, const void* p) {
    for (auto& e : ctx->lock_cache)
        if (e.p == p) return e.locked;
    const bool locked = device_view_of_host(p) != nullptr;
    auto& slot = ctx->lock_cache[ctx->lock_cache_next++ % 64];
    slot.p = p; slot.locked = locked;
    return locked;
}

#define CHECK_CTX(ctx) do { if (!(ctx)) return FLARE_ERR_INVALID_ARG; } while (0)
#define BIND(ctx) FLARE_CUDA_OK(ctx, cudaSetDevice((ctx)->device))

// ---------------------------------------------------------------- context
extern "C" {

int flare_attn_create(int device, flare_attn_ctx** out_ctx) {
    if (!out_ctx) return FLARE_ERR_INVALID_ARG;
    *out_ctx = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0 || device < 0 || device >= n) return FLARE_ERR_CUDA;
    flare_attn_ctx* ctx = new (std::nothrow) flare_attn_ctx();
    if (!ctx) return FLARE_ERR_OOM;
    ctx->device = device;
    if (cudaSetDevice(device) != cudaSuccess ||
        cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return FLARE_ERR_CUDA;
    }
    ctx->stream = ctx->own_stream;
    if (cudaHostAlloc((void**)&ctx->h_err, 64, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void**)&ctx->d_err, ctx->h_err, 0) != cudaSuccess ||
        cudaMalloc((void**)&ctx->d_gaveup, 256) != cudaSuccess || cudaMemset(ctx->d_gaveup, 0, 256) != cudaSuccess) {
        cudaFree(ctx->d_gaveup);
        if (ctx->h_err) cudaFreeHost(ctx->h_err);
        cudaStreamDestroy(ctx->own_stream);
        delete ctx;
        return FLARE_ERR_CUDA;
    }
    cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device);
    *ctx->h_err = 0;
    *out_ctx = ctx;
    return FLARE_OK;
}

int flare_attn_destroy(flare_attn_ctx* ctx) {
    if (!ctx) return FLARE_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->backend_kv) flare_kv_free(ctx->backend_kv);
    flare_comm_free(ctx);
    if (ctx->h_err) cudaFreeHost(ctx->h_err);
    cudaFree(ctx->d_gaveup);
    cudaFree(ctx->d_misc2); cudaFree(ctx->d_conv);
    cudaFree(ctx->d_work); cudaFree(ctx->d_stage_in); cudaFree(ctx->d_stage_out); cudaFree(ctx->d_misc);
    if (ctx->h_pinned) cudaFreeHost(ctx->h_pinned);
    if (ctx->h_rows) cudaFreeHost(ctx->h_rows);
    for (int i = 0; i < FLARE_ROW_SLOTS; i++) if (ctx->rows_events[i]) cudaEventDestroy(ctx->rows_events[i]);
    for (int i = 0; i < FLARE_SMALL_SLOTS; i++) if (ctx->small_events[i]) cudaEventDestroy(ctx->small_events[i]);
    for (int i = 0; i < 2; i++) if (ctx->stats_ev[i]) cudaEventDestroy(ctx->stats_ev[i]);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return FLARE_OK;
}

int flare_attn_enable_stats(flare_attn_ctx* ctx, int on) {
    CHECK_CTX(ctx);
    BIND(ctx);
    if (on) {
        for (int i = 0; i < 2; i++)
            if (!ctx->stats_ev[i]) FLARE_CUDA_OK(ctx, cudaEventCreate(&ctx->stats_ev[i]));
    } else {
        FLARE_TRY(stats_fold(ctx));
    }
    ctx->stats_on = on != 0;
    return FLARE_OK;
}

int flare_attn_set_peaks(flare_attn_ctx* ctx, double hbm_gbs, double tensor_tflops) {
    CHECK_CTX(ctx);
    if (!(hbm_gbs > 0.0) || !(tensor_tflops > 0.0)) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "peaks must be positive");
    ctx->peak_hbm_gbs = hbm_gbs; ctx->peak_tflops = tensor_tflops;
    return FLARE_OK;
}

int flare_attn_get_stats(flare_attn_ctx* ctx, flare_attn_stats* out) {
    CHECK_CTX(ctx);
    if (!out) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_attn_get_stats: out is null");
    BIND(ctx);
    FLARE_TRY(stats_fold(ctx));
    *out = ctx->stats;
    out->last_path = ctx->last_path;
    return FLARE_OK;
}

int flare_attn_set_stream(flare_attn_ctx* ctx, void* cuda_stream) {
    CHECK_CTX(ctx);
    BIND(ctx);
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->stream = cuda_stream ? (cudaStream_t)cuda_stream : ctx->own_stream;
    ctx->last_launch_overlappable = false;
    return FLARE_OK;
}

int flare_attn_sync(flare_attn_ctx* ctx) {
    CHECK_CTX(ctx);
    BIND(ctx);
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return flare_check_device_error(ctx);
}

int flare_attn_selftest_wait_timeout(flare_attn_ctx* ctx) {
    CHECK_CTX(ctx);
    BIND(ctx);
    selftest_wait_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_err, 1u << 12);
    FLARE_LAUNCH_CHECK(ctx);
    return flare_check_device_error(ctx);
}

const char* flare_attn_last_error(const flare_attn_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }
uint64_t flare_attn_launch_count(const flare_attn_ctx* ctx) { return ctx ? ctx->launches : 0; }
const char* flare_attn_backend_name(void) { return "cuda"; }

// ---------------------------------------------------------------- KV cache
int flare_kv_alloc(flare_attn_ctx* ctx, int num_layers, int batch, int max_seq_len, int num_kv_heads, int head_dim,
                   int kv_dtype, flare_kv** out_kv) {
    CHECK_CTX(ctx);
    if (!out_kv) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "out_kv is null");
    *out_kv = nullptr;
    if (num_layers <= 0 || batch <= 0 || max_seq_len <= 0 || num_kv_heads <= 0 || head_dim <= 0)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_kv_alloc: non-positive dimension");
    const size_t kvd = (size_t)num_kv_heads * head_dim, ms = (size_t)max_seq_len;
    size_t pb[FLARE_PLANE_COUNT] = {};
    switch (kv_dtype) {
        case FLARE_KV_F32:
            pb[FLARE_PLANE_K] = pb[FLARE_PLANE_V] = ms * kvd * 4;
            break;
        case FLARE_KV_Q8_0:
            if (head_dim % 32) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "Q8_0 cache needs head_dim %% 32 == 0");
            pb[FLARE_PLANE_K_Q] = pb[FLARE_PLANE_V_Q] = ms * kvd;
            pb[FLARE_PLANE_K_SCALE] = pb[FLARE_PLANE_V_SCALE] = ms * (kvd / 32) * 2;
            break;
        case FLARE_KV_KIVI_REF: {
            if (kvd % 4) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "KIVI_REF cache needs kv_dim %% 4 == 0");
            size_t R = ms < FLARE_REF_RESIDUAL ? ms : FLARE_REF_RESIDUAL;
            pb[FLARE_PLANE_K_Q] = pb[FLARE_PLANE_V_Q] = ms * (kvd / 4);
            pb[FLARE_PLANE_K_SCALE] = pb[FLARE_PLANE_K_MIN] = kvd * 4;
            pb[FLARE_PLANE_V_SCALE] = pb[FLARE_PLANE_V_MIN] = ms * 4;
            pb[FLARE_PLANE_K_RES] = pb[FLARE_PLANE_V_RES] = R * kvd * 4;
            break;
        }
        case FLARE_KV_KIVI_G32:
            if (head_dim % 32 || max_seq_len % FLARE_G32_RESIDUAL)
                return flare_set_error(ctx, FLARE_ERR_INVALID_ARG,
                                       "KIVI_G32 cache needs head_dim %% 32 == 0 and max_seq_len %% 128 == 0");
            pb[FLARE_PLANE_K_Q] = ms * (kvd / 4);
            pb[FLARE_PLANE_K_SCALE] = (ms / 32) * kvd * 4;
            pb[FLARE_PLANE_V_Q] = ms * (kvd / 4);
            pb[FLARE_PLANE_V_SCALE] = ms * (kvd / 32) * 4;
            pb[FLARE_PLANE_K_RES] = pb[FLARE_PLANE_V_RES] = (size_t)FLARE_G32_RESIDUAL * kvd * 2;
            break;
        default:
            return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "unknown kv_dtype %d", kv_dtype);
    }
    BIND(ctx);
    flare_kv* kv = new (std::nothrow) flare_kv();
    if (!kv) return FLARE_ERR_OOM;
    kv->ctx = ctx; kv->num_layers = num_layers; kv->batch = batch; kv->max_seq_len = max_seq_len;
    kv->num_kv_heads = num_kv_heads; kv->head_dim = head_dim; kv->kv_dim = (int)kvd; kv->dtype = kv_dtype;
    kv->position.assign(batch, 0); kv->length.assign(batch, 0);
    for (int i = 0; i < FLARE_PLANE_COUNT; i++) {
        kv->plane_bytes[i] = pb[i];
        if (!pb[i]) continue;
        // every (layer, sequence) plane starts on a 256-byte boundary when its size allows
        size_t total = pb[i] * (size_t)num_layers * batch;
        cudaError_t e = cudaMalloc(&kv->plane[i], total);
        if (e == cudaSuccess) e = cudaMemsetAsync(kv->plane[i], 0, total, ctx->stream);
        if (e != cudaSuccess) {
            int code = e == cudaErrorMemoryAllocation ? FLARE_ERR_OOM : FLARE_ERR_CUDA;
            flare_set_error(ctx, code, "flare_kv_alloc: %zu bytes for plane %d: %s", total, i, cudaGetErrorString(e));
            cudaGetLastError();
            flare_kv_free(kv);
            return code;
        }
    }
    if (kv_dtype == FLARE_KV_Q8_0 && (head_dim == 64 || head_dim == 128) && num_kv_heads <= 8) {
        CUtensorMapSwizzle swz = head_dim == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
        // preferred: (head_dim bytes, slot, kv head, layer*batch + seq) with a box of 32 slots x all heads,
        // which lands in shared memory as [head][slot][head_dim] from one contiguous stretch of the plane
        const uint64_t dims_w[4] = {(uint64_t)head_dim, (uint64_t)max_seq_len, (uint64_t)num_kv_heads, (uint64_t)num_layers * batch};
        const uint64_t strides_w[3] = {(uint64_t)kvd, (uint64_t)head_dim, (uint64_t)max_seq_len * kvd};
        const uint32_t box_w[4] = {(uint32_t)head_dim, 32, (uint32_t)num_kv_heads, 1};
        int r1 = flare_make_tensor_map(&kv->kq_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, kv->plane[FLARE_PLANE_K_Q], dims_w, strides_w, box_w, swz);
        int r2 = flare_make_tensor_map(&kv->vq_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, kv->plane[FLARE_PLANE_V_Q], dims_w, strides_w, box_w, swz);
        kv->maps_whole_rows = (r1 == 0 && r2 == 0);
        if (!kv->maps_whole_rows) {
            // fallback: natural dimension order, one box per head
            const uint64_t dims[4] = {(uint64_t)head_dim, (uint64_t)num_kv_heads, (uint64_t)max_seq_len, (uint64_t)num_layers * batch};
            const uint64_t strides[3] = {(uint64_t)head_dim, (uint64_t)kvd, (uint64_t)max_seq_len * kvd};
            const uint32_t box[4] = {(uint32_t)head_dim, 1, 32, 1};
            r1 = flare_make_tensor_map(&kv->kq_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, kv->plane[FLARE_PLANE_K_Q], dims, strides, box, swz);
            r2 = flare_make_tensor_map(&kv->vq_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, kv->plane[FLARE_PLANE_V_Q], dims, strides, box, swz);
        }
        if (r1 != 0 || r2 != 0) {
            flare_set_error(ctx, FLARE_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d, %d)", r1, r2);
            flare_kv_free(kv);
            return FLARE_ERR_CUDA;
        }
        kv->has_maps = true;
    }
    if (kv_dtype == FLARE_KV_KIVI_G32 && head_dim == 64 && num_kv_heads <= 8) {
        const uint64_t dims[4] = {16, (uint64_t)max_seq_len, (uint64_t)num_kv_heads, (uint64_t)num_layers * batch};
        const uint64_t strides[3] = {(uint64_t)kvd / 4, 16, (uint64_t)max_seq_len * (kvd / 4)};
        const uint32_t box[4] = {16, FLARE_G32_TILE, (uint32_t)num_kv_heads, 1};
        int r1 = flare_make_tensor_map(&kv->g32_kmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, kv->plane[FLARE_PLANE_K_Q], dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        int r2 = flare_make_tensor_map(&kv->g32_vmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, kv->plane[FLARE_PLANE_V_Q], dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        kv->has_g32_maps = (r1 == 0 && r2 == 0);     // without them the general kernel serves the cache
    }
    *out_kv = kv;
    return FLARE_OK;
}

int flare_kv_free(flare_kv* kv) {
    if (!kv) return FLARE_OK;
    cudaSetDevice(kv->ctx->device);
    cudaStreamSynchronize(kv->ctx->stream);
    for (int i = 0; i < FLARE_PLANE_COUNT; i++) if (kv->plane[i]) cudaFree(kv->plane[i]);
    cudaFree(kv->rope_cos); cudaFree(kv->rope_sin);
    if (kv->ctx->backend_kv == kv) kv->ctx->backend_kv = nullptr;
    delete kv;
    return FLARE_OK;
}

static int check_layer_seq(const flare_kv* kv, int layer, int seq) {
    if (!kv) return FLARE_ERR_INVALID_ARG;
    if (layer < 0 || layer >= kv->num_layers || seq < 0 || seq >= kv->batch)
        return flare_set_error(kv->ctx, FLARE_ERR_INVALID_ARG, "layer %d / sequence %d out of range (%d layers, batch %d)",
                               layer, seq, kv->num_layers, kv->batch);
    return FLARE_OK;
}

// stage two host row blocks on the device; returns device pointers
// *synced is set when the host buffers have NOT been fully consumed yet and the caller must
// synchronise the stream before returning.
static int stage_rows(flare_attn_ctx* ctx, const float* key, const float* value, size_t n_floats, int on_device,
                      const float** dk, const float** dv, bool* must_sync) {
    *must_sync = false;
    if (on_device) { *dk = key; *dv = value; return FLARE_OK; }
    size_t bytes = n_floats * sizeof(float);
    FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_in, &ctx->stage_in_bytes, 2 * bytes));
    float* d = (float*)ctx->d_stage_in;
    *dk = d; *dv = d + n_floats;
    if (2 * bytes <= (1u << 20)) {
        // small: CPU copy into a page-locked slot, then a truly asynchronous transfer; nothing to wait for
        const size_t slot_bytes = 1u << 20;
        if (!ctx->h_rows) {
            FLARE_CUDA_OK(ctx, cudaMallocHost(&ctx->h_rows, slot_bytes * FLARE_ROW_SLOTS));
            ctx->rows_slot_bytes = slot_bytes;
        }
        const int slot = (int)(ctx->rows_counter++ % FLARE_ROW_SLOTS);
        if (!ctx->rows_events[slot]) FLARE_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->rows_events[slot], cudaEventDisableTiming));
        else FLARE_CUDA_OK(ctx, cudaEventSynchronize(ctx->rows_events[slot]));
        char* h = (char*)ctx->h_rows + (size_t)slot * slot_bytes;
        memcpy(h, key, bytes);
        memcpy(h + bytes, value, bytes);
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d, h, 2 * bytes, cudaMemcpyHostToDevice, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaEventRecord(ctx->rows_events[slot], ctx->stream));
        ctx->last_launch_overlappable = false;
        return FLARE_OK;
    }
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d, key, bytes, cudaMemcpyHostToDevice, ctx->stream));
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d + n_floats, value, bytes, cudaMemcpyHostToDevice, ctx->stream));
    *must_sync = true;      // the caller's (possibly pageable) buffers are still being read
    return FLARE_OK;
}

int flare_kv_write_f32(flare_kv* kv, int layer, int seq, int64_t abs_position, const float* key, const float* value,
                       int on_device) {
    FLARE_TRY(check_layer_seq(kv, layer, seq));
    flare_attn_ctx* ctx = kv->ctx;
    if (!key || !value || abs_position < 0) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_kv_write_f32: bad argument");
    BIND(ctx);
    const float *dk, *dv;
    bool must_sync;
    FLARE_TRY(stage_rows(ctx, key, value, kv->kv_dim, on_device, &dk, &dv, &must_sync));
    // how many tokens are pending (written, not yet advanced) before this one
    int64_t slot = abs_position % kv->max_seq_len;
    int64_t pending = slot - kv->position[seq];
    if (pending < 0) pending += kv->max_seq_len;
    int64_t len_before = kv->length[seq] + pending;
    if (len_before > kv->max_seq_len) len_before = kv->max_seq_len;
    FLARE_TRY(flare_launch_kv_write(kv, layer, seq, abs_position, len_before, 1, dk, dv));
    if (must_sync) FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return FLARE_OK;
}

int flare_kv_append_f32(flare_kv* kv, int layer, int seq, int n_rows, const float* key, const float* value,
                        int on_device) {
    FLARE_TRY(check_layer_seq(kv, layer, seq));
    flare_attn_ctx* ctx = kv->ctx;
    if (n_rows < 0 || (n_rows > 0 && (!key || !value))) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_kv_append_f32: bad argument");
    if (n_rows == 0) return FLARE_OK;
    BIND(ctx);
    const float *dk, *dv;
    bool must_sync;
    FLARE_TRY(stage_rows(ctx, key, value, (size_t)n_rows * kv->kv_dim, on_device, &dk, &dv, &must_sync));
    // an absolute index congruent to the ring position (and to the token count before the wrap)
    int64_t first = kv->length[seq] < kv->max_seq_len ? kv->length[seq] : kv->max_seq_len + kv->position[seq];
    FLARE_TRY(flare_launch_kv_write(kv, layer, seq, first, kv->length[seq], n_rows, dk, dv));
    if (must_sync) FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return FLARE_OK;
}

static int upload_small(flare_attn_ctx* ctx, const flare_kv* kv, int n_q, const int* attend_len, const int** d_attend,
                        const int2** d_ring, int* max_attend);

int flare_kv_write_step_f32(flare_kv* kv, int layer, const float* key, const float* value, int on_device) {
    FLARE_TRY(check_layer_seq(kv, layer, 0));
    flare_attn_ctx* ctx = kv->ctx;
    if (!key || !value) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_kv_write_step_f32: null rows");
    BIND(ctx);
    const int* d_att; const int2* d_ring; int mx;
    FLARE_TRY(upload_small(ctx, kv, 1, nullptr, &d_att, &d_ring, &mx));
    const float *dk, *dv;
    bool must_sync;
    FLARE_TRY(stage_rows(ctx, key, value, (size_t)kv->batch * kv->kv_dim, on_device, &dk, &dv, &must_sync));
    FLARE_TRY(flare_launch_kv_write_step(kv, layer, d_ring, dk, dv));
    if (must_sync) FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return FLARE_OK;
}

int flare_kv_set_rope_table(flare_kv* kv, const float* cos, const float* sin, int table_len) {
    if (!kv) return FLARE_ERR_INVALID_ARG;
    flare_attn_ctx* ctx = kv->ctx;
    if (!cos || !sin || table_len < 1 || kv->head_dim % 2)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_kv_set_rope_table: null table, no rows, or an odd head_dim");
    BIND(ctx);
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    cudaFree(kv->rope_cos); cudaFree(kv->rope_sin);
    kv->rope_cos = kv->rope_sin = nullptr; kv->rope_len = 0;
    const size_t bytes = (size_t)table_len * (kv->head_dim / 2) * sizeof(float);
    FLARE_CUDA_OK(ctx, cudaMalloc(&kv->rope_cos, bytes));
    FLARE_CUDA_OK(ctx, cudaMalloc(&kv->rope_sin, bytes));
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(kv->rope_cos, cos, bytes, cudaMemcpyHostToDevice, ctx->stream));
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(kv->rope_sin, sin, bytes, cudaMemcpyHostToDevice, ctx->stream));
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    kv->rope_len = table_len;
    return FLARE_OK;
}

// positions of a step on the device (checked against the table on the host first)
static int upload_positions(flare_kv* kv, const int64_t* positions, int n, const long long** d_pos) {
    flare_attn_ctx* ctx = kv->ctx;
    if (!kv->rope_cos) return flare_set_error(ctx, FLARE_ERR_STATE, "no rotary table: call flare_kv_set_rope_table first");
    if (!positions) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "positions is null");
    for (int i = 0; i < n; i++)
        if (positions[i] < 0 || positions[i] >= kv->rope_len)
            return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "positions[%d] = %lld is outside the rotary table of %d rows", i,
                                   (long long)positions[i], kv->rope_len);
    FLARE_TRY(flare_ensure(ctx, &ctx->d_misc2, &ctx->misc2_bytes, (size_t)n * sizeof(long long)));
    // pageable source: the runtime has taken its own copy by the time this returns
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(ctx->d_misc2, positions, (size_t)n * sizeof(long long), cudaMemcpyHostToDevice, ctx->stream));
    ctx->last_launch_overlappable = false;
    *d_pos = (const long long*)ctx->d_misc2;
    return FLARE_OK;
}

int flare_kv_write_step_rope_f32(flare_kv* kv, int layer, const float* key, const float* value, const int64_t* positions,
                                 int on_device) {
    FLARE_TRY(check_layer_seq(kv, layer, 0));
    flare_attn_ctx* ctx = kv->ctx;
    if (!key || !value) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_kv_write_step_rope_f32: null rows");
    BIND(ctx);
    const long long* d_pos = nullptr;
    FLARE_TRY(upload_positions(kv, positions, kv->batch, &d_pos));
    const int* d_att; const int2* d_ring; int mx;
    FLARE_TRY(upload_small(ctx, kv, 1, nullptr, &d_att, &d_ring, &mx));
    const float *dk, *dv;
    bool must_sync;
    FLARE_TRY(stage_rows(ctx, key, value, (size_t)kv->batch * kv->kv_dim, on_device, &dk, &dv, &must_sync));
    if (kv->dtype == FLARE_KV_KIVI_REF || kv->dtype == FLARE_KV_KIVI_G32) {
        // the 2-bit caches take one sequence at a time through the general row writer: rotate a copy of the rows first
        const size_t bytes = (size_t)kv->batch * kv->kv_dim * sizeof(float);
        FLARE_TRY(flare_ensure(ctx, &ctx->d_conv, &ctx->conv_bytes, bytes));
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(ctx->d_conv, dk, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        FLARE_TRY(flare_launch_rope_rows(kv, (float*)ctx->d_conv, kv->batch, kv->num_kv_heads, d_pos));
        FLARE_TRY(flare_launch_kv_write_step(kv, layer, d_ring, (const float*)ctx->d_conv, dv));
    } else {
        FLARE_TRY(flare_launch_kv_write_step(kv, layer, d_ring, dk, dv, d_pos));
    }
    if (must_sync) FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return FLARE_OK;
}

// The same on device buffers with the positions already on the device (one upload per token, not per layer); the
// step's query rows [batch][q_heads][head_dim], when given, are rotated in place by the same launch.
int flare_kv_write_step_rope_device(flare_kv* kv, int layer, const float* d_key, const float* d_value, const long long* d_pos,
                                    float* d_q_rows, int q_heads) {
    FLARE_TRY(check_layer_seq(kv, layer, 0));
    flare_attn_ctx* ctx = kv->ctx;
    BIND(ctx);
    const int* d_att; const int2* d_ring; int mx;
    FLARE_TRY(upload_small(ctx, kv, 1, nullptr, &d_att, &d_ring, &mx));
    if (kv->dtype == FLARE_KV_KIVI_REF || kv->dtype == FLARE_KV_KIVI_G32) {
        const size_t bytes = (size_t)kv->batch * kv->kv_dim * sizeof(float);
        FLARE_TRY(flare_ensure(ctx, &ctx->d_conv, &ctx->conv_bytes, bytes));
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(ctx->d_conv, d_key, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        FLARE_TRY(flare_launch_rope_rows(kv, (float*)ctx->d_conv, kv->batch, kv->num_kv_heads, d_pos));
        if (d_q_rows) FLARE_TRY(flare_launch_rope_rows(kv, d_q_rows, kv->batch, q_heads, d_pos));
        return flare_launch_kv_write_step(kv, layer, d_ring, (const float*)ctx->d_conv, d_value);
    }
    return flare_launch_kv_write_step(kv, layer, d_ring, d_key, d_value, d_pos, d_q_rows, q_heads);
}

int flare_rope_rows_f32(flare_kv* kv, float* rows, int n_rows, int num_heads, const int64_t* positions, int on_device) {
    if (!kv) return FLARE_ERR_INVALID_ARG;
    flare_attn_ctx* ctx = kv->ctx;
    if (!rows || n_rows < 0 || num_heads < 1) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_rope_rows_f32: bad argument");
    if (n_rows == 0) return FLARE_OK;
    BIND(ctx);
    const long long* d_pos = nullptr;
    FLARE_TRY(upload_positions(kv, positions, n_rows, &d_pos));
    if (on_device) return flare_launch_rope_rows(kv, rows, n_rows, num_heads, d_pos);
    const size_t bytes = (size_t)n_rows * num_heads * kv->head_dim * sizeof(float);
    FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_in, &ctx->stage_in_bytes, bytes));
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(ctx->d_stage_in, rows, bytes, cudaMemcpyHostToDevice, ctx->stream));
    FLARE_TRY(flare_launch_rope_rows(kv, (float*)ctx->d_stage_in, n_rows, num_heads, d_pos));
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(rows, ctx->d_stage_in, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return FLARE_OK;
}

int flare_kv_advance(flare_kv* kv, int seq, int n) {
    if (!kv || n < 0 || seq >= kv->batch) return FLARE_ERR_INVALID_ARG;
    int lo = seq < 0 ? 0 : seq, hi = seq < 0 ? kv->batch : seq + 1;
    for (int s = lo; s < hi; s++) {
        kv->position[s] = (kv->position[s] + n) % kv->max_seq_len;
        kv->length[s] = kv->length[s] + n < kv->max_seq_len ? kv->length[s] + n : kv->max_seq_len;
    }
    return FLARE_OK;
}

int flare_kv_get_state(const flare_kv* kv, int seq, int64_t* position, int64_t* length) {
    if (!kv || seq < 0 || seq >= kv->batch) return FLARE_ERR_INVALID_ARG;
    if (position) *position = kv->position[seq];
    if (length) *length = kv->length[seq];
    return FLARE_OK;
}

int flare_kv_set_state(flare_kv* kv, int seq, int64_t position, int64_t length) {
    if (!kv || seq < 0 || seq >= kv->batch) return FLARE_ERR_INVALID_ARG;
    if (position < 0 || position >= kv->max_seq_len || length < 0 || length > kv->max_seq_len)
        return flare_set_error(kv->ctx, FLARE_ERR_INVALID_ARG, "flare_kv_set_state: position %lld / length %lld out of range",
                               (long long)position, (long long)length);
    kv->position[seq] = position; kv->length[seq] = length;
    return FLARE_OK;
}

int flare_kv_truncate(flare_kv* kv, int seq, int64_t target_len) {
    if (!kv || seq < 0 || seq >= kv->batch || target_len < 0) return FLARE_ERR_INVALID_ARG;
    if (target_len >= kv->length[seq]) return FLARE_OK;
    if (kv->dtype == FLARE_KV_KIVI_G32 && kv->length[seq] > FLARE_G32_RESIDUAL)
        return flare_set_error(kv->ctx, FLARE_ERR_UNSUPPORTED,
                               "a group-32 KIVI cache cannot be rolled back once tokens have left the residual ring");
    if (kv->length[seq] < kv->max_seq_len) { kv->position[seq] = target_len; kv->length[seq] = target_len; }
    return FLARE_OK;
}

int flare_kv_clear(flare_kv* kv, int seq) {
    if (!kv || seq >= kv->batch) return FLARE_ERR_INVALID_ARG;
    flare_attn_ctx* ctx = kv->ctx;
    BIND(ctx);
    int lo = seq < 0 ? 0 : seq, hi = seq < 0 ? kv->batch : seq + 1;
    for (int s = lo; s < hi; s++) {
        kv->position[s] = 0; kv->length[s] = 0;
        for (int p = 0; p < FLARE_PLANE_COUNT; p++) {
            if (!kv->plane[p]) continue;
            for (int l = 0; l < kv->num_layers; l++)
                FLARE_CUDA_OK(ctx, cudaMemsetAsync(kv->plane_ptr(p, l, s), 0, kv->plane_bytes[p], ctx->stream));
        }
    }
    return FLARE_OK;
}

size_t flare_kv_plane_bytes(const flare_kv* kv, int plane) {
    if (!kv || plane < 0 || plane >= FLARE_PLANE_COUNT) return 0;
    return kv->plane_bytes[plane];
}

static int plane_copy(flare_kv* kv, int layer, int seq, int plane, void* host_or_dev, size_t bytes, int on_device, bool to_cache) {
    FLARE_TRY(check_layer_seq(kv, layer, seq));
    flare_attn_ctx* ctx = kv->ctx;
    if (plane < 0 || plane >= FLARE_PLANE_COUNT || !kv->plane[plane])
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "this cache has no plane %d", plane);
    if (!host_or_dev || bytes != kv->plane_bytes[plane])
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "plane %d is %zu bytes, got %zu", plane, kv->plane_bytes[plane], bytes);
    BIND(ctx);
    ctx->last_launch_overlappable = false;
    char* p = kv->plane_ptr(plane, layer, seq);
    cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : (to_cache ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost);
    if (to_cache) FLARE_CUDA_OK(ctx, cudaMemcpyAsync(p, host_or_dev, bytes, kind, ctx->stream));
    else FLARE_CUDA_OK(ctx, cudaMemcpyAsync(host_or_dev, p, bytes, kind, ctx->stream));
    if (!on_device) FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return FLARE_OK;
}
int flare_kv_export_plane(flare_kv* kv, int layer, int seq, int plane, void* dst, size_t bytes, int on_device) {
    return plane_copy(kv, layer, seq, plane, dst, bytes, on_device, false);
}
int flare_kv_import_plane(flare_kv* kv, int layer, int seq, int plane, const void* src, size_t bytes, int on_device) {
    return plane_copy(kv, layer, seq, plane, const_cast<void*>(src), bytes, on_device, true);
}

static int q8_blocks(flare_kv* kv, int layer, int seq, int first_slot, int n_slots, void* kb, void* vb, int on_device, int to_blocks) {
    FLARE_TRY(check_layer_seq(kv, layer, seq));
    flare_attn_ctx* ctx = kv->ctx;
    if (kv->dtype != FLARE_KV_Q8_0) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "not a Q8_0 cache");
    if (first_slot < 0 || n_slots < 0 || first_slot + n_slots > kv->max_seq_len)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "slots [%d, %d) outside the ring of %d", first_slot, first_slot + n_slots, kv->max_seq_len);
    if (n_slots == 0) return FLARE_OK;
    BIND(ctx);
    size_t bytes = (size_t)n_slots * (kv->kv_dim / 32) * 34;
    void *dkb = kb, *dvb = vb;
    if (!on_device) {
        FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_in, &ctx->stage_in_bytes, 2 * bytes));
        dkb = kb ? ctx->d_stage_in : nullptr;
        dvb = vb ? (char*)ctx->d_stage_in + bytes : nullptr;
        if (!to_blocks) {
            if (kb) FLARE_CUDA_OK(ctx, cudaMemcpyAsync(dkb, kb, bytes, cudaMemcpyHostToDevice, ctx->stream));
            if (vb) FLARE_CUDA_OK(ctx, cudaMemcpyAsync(dvb, vb, bytes, cudaMemcpyHostToDevice, ctx->stream));
        }
    }
    FLARE_TRY(flare_launch_q8_blocks(kv, layer, seq, first_slot, n_slots, dkb, dvb, to_blocks));
    if (!on_device) {
        if (to_blocks) {
            if (kb) FLARE_CUDA_OK(ctx, cudaMemcpyAsync(kb, dkb, bytes, cudaMemcpyDeviceToHost, ctx->stream));
            if (vb) FLARE_CUDA_OK(ctx, cudaMemcpyAsync(vb, dvb, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        }
        FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return FLARE_OK;
}
int flare_kv_import_q8_0_blocks(flare_kv* kv, int layer, int seq, int first_slot, int n_slots, const void* k_blocks,
                                const void* v_blocks, int on_device) {
    return q8_blocks(kv, layer, seq, first_slot, n_slots, const_cast<void*>(k_blocks), const_cast<void*>(v_blocks), on_device, 0);
}
int flare_kv_export_q8_0_blocks(flare_kv* kv, int layer, int seq, int first_slot, int n_slots, void* k_blocks,
                                void* v_blocks, int on_device) {
    return q8_blocks(kv, layer, seq, first_slot, n_slots, k_blocks, v_blocks, on_device, 1);
}

int flare_kv_export_dequant(flare_kv* kv, int layer, int seq, float* k_out, float* v_out, int on_device) {
    FLARE_TRY(check_layer_seq(kv, layer, seq));
    flare_attn_ctx* ctx = kv->ctx;
    if (!k_out && !v_out) return FLARE_OK;
    BIND(ctx);
    size_t n = (size_t)kv->max_seq_len * kv->kv_dim, bytes = n * 4;
    float *dk = k_out, *dv = v_out;
    if (!on_device) {
        FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_out, &ctx->stage_out_bytes, 2 * bytes));
        dk = k_out ? (float*)ctx->d_stage_out : nullptr;
        dv = v_out ? (float*)ctx->d_stage_out + n : nullptr;
    }
    FLARE_TRY(flare_launch_kv_export_dequant(kv, layer, seq, dk, dv));
    if (!on_device) {
        if (k_out) FLARE_CUDA_OK(ctx, cudaMemcpyAsync(k_out, dk, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        if (v_out) FLARE_CUDA_OK(ctx, cudaMemcpyAsync(v_out, dv, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return FLARE_OK;
}

// ---------------------------------------------------------------- attention
// Small per-call integer arrays (attend_len, ring state) go through pinned memory.
static int upload_small(flare_attn_ctx* ctx, const flare_kv* kv, int n_q, const int* attend_len, const int** d_attend,
                        const int2** d_ring, int* max_attend) {
    const int B = kv->batch;
    size_t bytes = (size_t)B * (sizeof(int) + sizeof(int2));
    // a ring of pinned/device slots so that back-to-back calls do not overwrite in-flight data
    const int kSlots = FLARE_SMALL_SLOTS;
    size_t slot_bytes = (bytes + 255) / 256 * 256;
    // build the arrays first; a decode step makes one call per layer with identical contents,
    // in which case the device copy of the previous call is reused and nothing is uploaded
    std::vector<int> cur((size_t)B * 3);
    int2* c_ring = (int2*)cur.data();
    int* c_att = cur.data() + 2 * (size_t)B;
    int mx = 0;
    for (int b = 0; b < B; b++) {
        int64_t a;
        if (attend_len) a = attend_len[b];
        else { a = kv->length[b] + n_q; if (a > kv->max_seq_len) a = kv->max_seq_len; }
        if (a < 0 || a > kv->max_seq_len)
            return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "attend_len[%d] = %lld outside [0, %d]", b, (long long)a, kv->max_seq_len);
        c_att[b] = (int)a;
        if (a > mx) mx = (int)a;
        c_ring[b] = make_int2((int)kv->position[b], (int)kv->length[b]);
    }
    *max_attend = mx;
    if (ctx->small_last_dev && cur == ctx->small_last) {
        *d_ring = (const int2*)ctx->small_last_dev;
        *d_attend = (const int*)((const char*)ctx->small_last_dev + (size_t)B * sizeof(int2));
        return FLARE_OK;
    }
    if (slot_bytes * kSlots > ctx->pinned_bytes || slot_bytes * kSlots > ctx->misc_bytes) {
        FLARE_TRY(flare_ensure_pinned(ctx, slot_bytes * kSlots));
        FLARE_TRY(flare_ensure(ctx, &ctx->d_misc, &ctx->misc_bytes, slot_bytes * kSlots));
    }
    const int slot = (int)(ctx->small_counter++ % kSlots);
    size_t off = (size_t)slot * slot_bytes;
    if (!ctx->small_events[slot]) FLARE_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->small_events[slot], cudaEventDisableTiming));
    else FLARE_CUDA_OK(ctx, cudaEventSynchronize(ctx->small_events[slot]));   // the copy that last used this slot is done
    memcpy((char*)ctx->h_pinned + off, cur.data(), bytes);
    char* d = (char*)ctx->d_misc + off;
    FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d, (char*)ctx->h_pinned + off, bytes, cudaMemcpyHostToDevice, ctx->stream));
    FLARE_CUDA_OK(ctx, cudaEventRecord(ctx->small_events[slot], ctx->stream));
    *d_ring = (const int2*)d;
    *d_attend = (const int*)(d + (size_t)B * sizeof(int2));
    ctx->small_last.swap(cur);
    ctx->small_last_dev = d;
    *max_attend = mx;
    return FLARE_OK;
}

// q_staged: when non-null, q is already on the device there although `out` is a host buffer (on_device = 0).
// multi: the slot range is this rank's share of one sequence; the records of all ranks are exchanged and merged
// (flare_multi_tail) and `out` receives the attention output over the whole sequence.
int flare_decode_common(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads, const float* q, int n_q,
                        const int* attend_len, float softcap, int slot_begin, int slot_end, int want_partial,
                        int causal_q, float* out, int on_device, const float* q_staged, int multi) {
    CHECK_CTX(ctx);
    if (!kv || kv->ctx != ctx) return flare_set_error(ctx, FLARE_ERR_STATE, "no KV cache bound to this context");
    if (layer < 0 || layer >= kv->num_layers) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "layer %d out of range", layer);
    if (!q || !out || n_q < 1 || num_heads < 1 || num_heads % kv->num_kv_heads)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "decode: bad q/out/n_q or num_heads %d not a multiple of %d kv heads",
                               num_heads, kv->num_kv_heads);
    if (softcap != 0.0f)
        return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "attention logit soft-capping is not implemented on the GPU path");
    if (slot_end >= 0 && (slot_begin < 0 || slot_begin > slot_end || slot_end > kv->max_seq_len))
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "slot range [%d, %d) invalid", slot_begin, slot_end);
    BIND(ctx);
    DecodeArgs a;
    a.kv = flare_layer_view(kv, layer);
    a.layer = layer;
    a.window = 0;
    a.kmap = kv->has_maps ? &kv->kq_map : nullptr;
    a.vmap = kv->has_maps ? &kv->vq_map : nullptr;
    a.whole_rows = kv->maps_whole_rows ? 1 : 0;
    a.kv_obj = kv;
    a.batch = kv->batch; a.n_q = n_q; a.num_heads = num_heads;
    a.slot_begin = slot_begin; a.slot_end = slot_end; a.want_partial = want_partial; a.causal_q = causal_q;
    FLARE_TRY(upload_small(ctx, kv, n_q, attend_len, &a.attend_len, &a.ring, &a.max_attend));
    a.h_attend = ctx->small_last.size() == (size_t)kv->batch * 3 ? ctx->small_last.data() + 2 * (size_t)kv->batch : nullptr;
    const size_t rows = (size_t)kv->batch * n_q * num_heads;
    const size_t q_bytes = rows * kv->head_dim * 4;
    const size_t o_bytes = rows * (kv->head_dim + ((want_partial && !multi) ? 2 : 0)) * 4;
    const float* work = nullptr;
    int n_split = 0;
    if (multi) {
        if (kv->head_dim != 64 && kv->head_dim != 128)
            return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "the multi-GPU split needs head_dim 64 or 128, got %d", kv->head_dim);
        a.defer_merge = 1; a.work_out = &work; a.n_split_out = &n_split;
    }
    bool copy_out = false;
    if (on_device) { a.q = q; a.out = out; }
    else {
        if (q_staged) a.q = q_staged;
        else {
            FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_in, &ctx->stage_in_bytes, q_bytes));
            FLARE_CUDA_OK(ctx, cudaMemcpyAsync(ctx->d_stage_in, q, q_bytes, cudaMemcpyHostToDevice, ctx->stream));
            a.q = (const float*)ctx->d_stage_in;
        }
        // A page-locked output buffer is written by the kernel itself over the bus (each element once, at the
        // end of the kernel) instead of by a separate device-to-host copy after it.
        cudaPointerAttributes pa;
        if (cudaPointerGetAttributes(&pa, out) == cudaSuccess && pa.type == cudaMemoryTypeHost && pa.devicePointer) {
            a.out = (float*)pa.devicePointer;
        } else {
            cudaGetLastError();
            FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_out, &ctx->stage_out_bytes, o_bytes));
            a.out = (float*)ctx->d_stage_out;
            copy_out = true;
        }
    }
    FLARE_TRY(stats_begin(ctx));
    FLARE_TRY(flare_launch_decode(ctx, a));
    if (multi) FLARE_TRY(flare_multi_tail(ctx, work, n_split, (int)rows, kv->head_dim, a.out));
    if (ctx->stats_on) {
        double bytes = 0.0, pairs = 0.0;
        for (int b = 0; b < kv->batch && a.h_attend; b++) {
            for (int i = 0; i < n_q; i++) {
                int lo = 0, hi = a.h_attend[b] - (causal_q ? (n_q - 1 - i) : 0);
                if (slot_end >= 0) { lo = slot_begin; if (hi > slot_end) hi = slot_end; }
                const double n = hi > lo ? hi - lo : 0;
                pairs += n;
                if (i == n_q - 1) bytes += kv_bytes_of(kv, n);
            }
        }
        FLARE_TRY(stats_end(ctx, FLARE_OP_DECODE, bytes, 4.0 * num_heads * kv->head_dim * pairs));
    }
    if (!on_device) {
        if (copy_out) FLARE_CUDA_OK(ctx, cudaMemcpyAsync(out, a.out, o_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        FLARE_TRY(flare_check_device_error(ctx));    // synchronises the stream
    }
    return FLARE_OK;
}

int flare_decode_attn(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads, const float* q, int n_q,
                      const int* attend_len, float softcap, float* out, int on_device) {
    return flare_decode_common(ctx, kv, layer, num_heads, q, n_q, attend_len, softcap, 0, -1, 0, 1, out, on_device);
}


int flare_decode_step(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads, const float* key, const float* value,
                      const float* q, float* out, int on_device) {
    CHECK_CTX(ctx);
    if (!kv || kv->ctx != ctx) return flare_set_error(ctx, FLARE_ERR_STATE, "no KV cache bound to this context");
    if (!key || !value || !q || !out) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_decode_step: null buffer");
    if (layer < 0 || layer >= kv->num_layers) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "layer %d out of range", layer);
    if (num_heads < 1 || num_heads % kv->num_kv_heads)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "num_heads %d is not a multiple of %d kv heads", num_heads, kv->num_kv_heads);
    BIND(ctx);
    const int* d_att; const int2* d_ring; int mx;
    FLARE_TRY(upload_small(ctx, kv, 1, nullptr, &d_att, &d_ring, &mx));
    if (on_device) {
        FLARE_TRY(flare_launch_kv_write_step(kv, layer, d_ring, key, value));
        return flare_decode_common(ctx, kv, layer, num_heads, q, 1, nullptr, 0.0f, 0, -1, 0, 1, out, 1);
    }
    const size_t row_fl = (size_t)kv->batch * kv->kv_dim, q_fl = (size_t)kv->batch * num_heads * kv->head_dim;
    const size_t bytes = (2 * row_fl + q_fl) * sizeof(float);
    FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_in, &ctx->stage_in_bytes, bytes));
    float* d = (float*)ctx->d_stage_in;
    const float *dk = d, *dv = d + row_fl, *dq = d + 2 * row_fl;
    const bool locked = input_is_locked(ctx, key) && input_is_locked(ctx, value) && input_is_locked(ctx, q);
    const size_t slot_bytes = 1u << 20;
    if (locked && value == key + row_fl && q == value + row_fl) {
        // page-locked and laid out [K rows][V rows][q] in one piece (a host that keeps its per-layer forward
        // buffers in one allocation): one transfer straight from the caller's memory
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d, key, bytes, cudaMemcpyHostToDevice, ctx->stream));
    } else if (locked) {
        // page-locked: the copy engine reads the caller's buffers as they are.  (Letting the kernels read them in
        // place over the bus was measured slower: 1.73 ms instead of 1.22 ms per 16-layer step.)
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d, key, row_fl * 4, cudaMemcpyHostToDevice, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d + row_fl, value, row_fl * 4, cudaMemcpyHostToDevice, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d + 2 * row_fl, q, q_fl * 4, cudaMemcpyHostToDevice, ctx->stream));
    } else if (bytes <= slot_bytes) {
        // pageable and small: pack the three inputs into one page-locked slot, one transfer
        if (!ctx->h_rows) {
            FLARE_CUDA_OK(ctx, cudaMallocHost(&ctx->h_rows, slot_bytes * FLARE_ROW_SLOTS));
            ctx->rows_slot_bytes = slot_bytes;
        }
        const int slot = (int)(ctx->rows_counter++ % FLARE_ROW_SLOTS);
        if (!ctx->rows_events[slot]) FLARE_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->rows_events[slot], cudaEventDisableTiming));
        else FLARE_CUDA_OK(ctx, cudaEventSynchronize(ctx->rows_events[slot]));
        float* h = (float*)((char*)ctx->h_rows + (size_t)slot * slot_bytes);
        memcpy(h, key, row_fl * 4);
        memcpy(h + row_fl, value, row_fl * 4);
        memcpy(h + 2 * row_fl, q, q_fl * 4);
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaEventRecord(ctx->rows_events[slot], ctx->stream));
    } else {
        // pageable and large: the call synchronises before it returns, so the buffers stay valid long enough
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d, key, row_fl * 4, cudaMemcpyHostToDevice, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d + row_fl, value, row_fl * 4, cudaMemcpyHostToDevice, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d + 2 * row_fl, q, q_fl * 4, cudaMemcpyHostToDevice, ctx->stream));
    }
    ctx->last_launch_overlappable = false;
    FLARE_TRY(flare_launch_kv_write_step(kv, layer, d_ring, dk, dv));
    // attention on the staged q; the output goes to the caller's host buffer; one synchronisation at the end
    return flare_decode_common(ctx, kv, layer, num_heads, q, 1, nullptr, 0.0f, 0, -1, 0, 1, out, 0, dq);
}

int flare_decode_attn_noalloc(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads, const float* q_dev, int n_q,
                              const int* attend_len, float* out_dev) {
    CHECK_CTX(ctx);
    if (!kv || kv->ctx != ctx) return flare_set_error(ctx, FLARE_ERR_STATE, "no KV cache bound to this context");
    if (layer < 0 || layer >= kv->num_layers) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "layer %d out of range", layer);
    if (!q_dev || !out_dev || n_q < 1 || num_heads < 1 || num_heads % kv->num_kv_heads)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "decode: bad q/out/n_q or num_heads %d not a multiple of %d kv heads",
                               num_heads, kv->num_kv_heads);
    BIND(ctx);
    return flare_decode_noalloc(ctx, kv, layer, num_heads, q_dev, n_q, attend_len, out_dev);
}
size_t flare_decode_attn_noalloc_scratch_bytes(void) { return flare_noalloc_scratch_bytes(); }

int flare_decode_attn_partial(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads, const float* q, int n_q,
                              int slot_begin, int slot_end, float* partial, int on_device) {
    CHECK_CTX(ctx);
    if (!kv) return flare_set_error(ctx, FLARE_ERR_STATE, "no KV cache");
    if (slot_end < 0) return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "slot_end must be >= 0");
    // every query reads the whole range: the range itself is the mask
    std::vector<int> att(kv->batch, slot_end > kv->max_seq_len ? kv->max_seq_len : slot_end);
    return flare_decode_common(ctx, kv, layer, num_heads, q, n_q, att.data(), 0.0f, slot_begin, slot_end, 1, 0, partial, on_device);
}

int flare_merge_partials(flare_attn_ctx* ctx, const float* partials, int n_parts, int rows, int head_dim, float* out,
                         int on_device) {
    CHECK_CTX(ctx);
    if (!partials || !out || n_parts < 1 || rows < 0 || head_dim < 1)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_merge_partials: bad argument");
    BIND(ctx);
    size_t in_bytes = (size_t)n_parts * rows * (head_dim + 2) * 4, out_bytes = (size_t)rows * head_dim * 4;
    const float* dp = partials; float* dout = out;
    if (!on_device) {
        FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_in, &ctx->stage_in_bytes, in_bytes));
        FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_out, &ctx->stage_out_bytes, out_bytes));
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(ctx->d_stage_in, partials, in_bytes, cudaMemcpyHostToDevice, ctx->stream));
        dp = (const float*)ctx->d_stage_in; dout = (float*)ctx->d_stage_out;
    }
    FLARE_TRY(flare_launch_merge(ctx, dp, (size_t)rows * (head_dim + 2), n_parts, rows, head_dim, dout, 0));
    if (!on_device) {
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(out, dout, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return FLARE_OK;
}

int flare_gqa_attention_host(flare_attn_ctx* ctx, const float* q, const float* k_cache, const float* v_cache,
                             int num_heads, int num_kv_heads, int head_dim, int seq_len, float softcap, float* out) {
    CHECK_CTX(ctx);
    if (!q || !out || num_heads < 1 || num_kv_heads < 1 || head_dim < 1 || seq_len < 0 || (seq_len > 0 && (!k_cache || !v_cache)))
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_gqa_attention_host: bad argument");
    if (softcap != 0.0f)
        return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "attention logit soft-capping is not implemented on the GPU path");
    if (seq_len == 0) {   // cpu_grouped_query_attention_into leaves zeros (model.rs:9929-9931)
        memset(out, 0, (size_t)num_heads * head_dim * 4);
        return FLARE_OK;
    }
    flare_kv* tmp = nullptr;
    FLARE_TRY(flare_kv_alloc(ctx, 1, 1, seq_len, num_kv_heads, head_dim, FLARE_KV_F32, &tmp));
    size_t bytes = (size_t)seq_len * num_kv_heads * head_dim * 4;
    int s = flare_kv_import_plane(tmp, 0, 0, FLARE_PLANE_K, k_cache, bytes, 0);
    if (s == FLARE_OK) s = flare_kv_import_plane(tmp, 0, 0, FLARE_PLANE_V, v_cache, bytes, 0);
    int att = seq_len;
    if (s == FLARE_OK) s = flare_decode_attn(ctx, tmp, 0, num_heads, q, 1, &att, 0.0f, out, 0);
    flare_kv_free(tmp);
    return s;
}

int flare_prefill_attn(flare_attn_ctx* ctx, const void* q, const void* k, const void* v, int in_dtype, int batch,
                       int seq_len, int num_heads, int num_kv_heads, int head_dim, int window, float softcap, void* out,
                       int out_dtype, int on_device) {
    CHECK_CTX(ctx);
    if (!q || !k || !v || !out || batch < 1 || seq_len < 1 || num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads ||
        window < 0 || (in_dtype != FLARE_DT_F32 && in_dtype != FLARE_DT_BF16) || (out_dtype != FLARE_DT_F32 && out_dtype != FLARE_DT_BF16))
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "flare_prefill_attn: bad argument");
    if (softcap != 0.0f)
        return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "attention logit soft-capping is not implemented on the GPU path");
    BIND(ctx);
    PrefillArgs a;
    a.in_dtype = in_dtype; a.out_dtype = out_dtype; a.batch = batch; a.seq_len = seq_len; a.num_heads = num_heads;
    a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.window = window;
    const size_t esz_in = in_dtype == FLARE_DT_F32 ? 4 : 2, esz_out = out_dtype == FLARE_DT_F32 ? 4 : 2;
    const size_t qn = (size_t)batch * seq_len * num_heads * head_dim, kn = (size_t)batch * seq_len * num_kv_heads * head_dim;
    if (on_device) { a.q = q; a.k = k; a.v = v; a.out = out; }
    else {
        size_t qb = (qn * esz_in + 255) / 256 * 256, kb = (kn * esz_in + 255) / 256 * 256;
        FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_in, &ctx->stage_in_bytes, qb + 2 * kb));
        FLARE_TRY(flare_ensure(ctx, &ctx->d_stage_out, &ctx->stage_out_bytes, qn * esz_out));
        char* d = (char*)ctx->d_stage_in;
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d, q, qn * esz_in, cudaMemcpyHostToDevice, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d + qb, k, kn * esz_in, cudaMemcpyHostToDevice, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(d + qb + kb, v, kn * esz_in, cudaMemcpyHostToDevice, ctx->stream));
        a.q = d; a.k = d + qb; a.v = d + qb + kb; a.out = ctx->d_stage_out;
    }
    FLARE_TRY(stats_begin(ctx));
    FLARE_TRY(flare_launch_prefill(ctx, a));
    if (ctx->stats_on) {
        double pairs = 0.0;
        for (int t = 0; t < seq_len; t++) pairs += (window > 0 && t + 1 > window) ? window : t + 1;
        const double io = ((double)qn * (esz_in + esz_out) + 2.0 * (double)kn * esz_in);
        FLARE_TRY(stats_end(ctx, FLARE_OP_PREFILL, io, 4.0 * batch * num_heads * head_dim * pairs));
    }
    if (!on_device) {
        FLARE_CUDA_OK(ctx, cudaMemcpyAsync(out, a.out, qn * esz_out, cudaMemcpyDeviceToHost, ctx->stream));
        FLARE_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return FLARE_OK;
}

// ---------------------------------------------------------------- trait-shaped shims
int flare_backend_init_gpu_kv_cache_dtype(flare_attn_ctx* ctx, int num_layers, int max_seq_len, int num_kv_heads,
                                          int head_dim, int kv_dtype) {
    CHECK_CTX(ctx);
    if (ctx->backend_kv) { flare_kv_free(ctx->backend_kv); ctx->backend_kv = nullptr; }
    flare_kv* kv = nullptr;
    FLARE_TRY(flare_kv_alloc(ctx, num_layers, 1, max_seq_len, num_kv_heads, head_dim, kv_dtype, &kv));
    ctx->backend_kv = kv;
    return FLARE_OK;
}
int flare_backend_init_gpu_kv_cache(flare_attn_ctx* ctx, int num_layers, int max_seq_len, int num_kv_heads, int head_dim) {
    return flare_backend_init_gpu_kv_cache_dtype(ctx, num_layers, max_seq_len, num_kv_heads, head_dim, FLARE_KV_F32);
}
int flare_backend_gpu_kv_write(flare_attn_ctx* ctx, int layer, int64_t position, int num_kv_heads, int head_dim,
                               const float* key, const float* value) {
    CHECK_CTX(ctx);
    flare_kv* kv = ctx->backend_kv;
    if (!kv) return flare_set_error(ctx, FLARE_ERR_STATE, "GPU KV cache is not initialized - call init_gpu_kv_cache first");
    if (num_kv_heads != kv->num_kv_heads || head_dim != kv->head_dim)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "gpu_kv_write: %d kv heads x %d, cache has %d x %d", num_kv_heads,
                               head_dim, kv->num_kv_heads, kv->head_dim);
    return flare_kv_write_f32(kv, layer, 0, position, key, value, 0);
}
int flare_backend_has_gpu_kv_cache(const flare_attn_ctx* ctx) { return ctx && ctx->backend_kv ? 1 : 0; }
int flare_backend_gqa_from_gpu_cache(flare_attn_ctx* ctx, const float* q, int layer, int num_heads, int num_kv_heads,
                                     int head_dim, int seq_len, float softcap, float* out) {
    CHECK_CTX(ctx);
    flare_kv* kv = ctx->backend_kv;
    if (!kv) return flare_set_error(ctx, FLARE_ERR_STATE, "GPU KV cache is not initialized - call init_gpu_kv_cache first");
    if (num_kv_heads != kv->num_kv_heads || head_dim != kv->head_dim || seq_len < 0)
        return flare_set_error(ctx, FLARE_ERR_INVALID_ARG, "gqa_from_gpu_cache: shape does not match the cache");
    int att = seq_len < kv->max_seq_len ? seq_len : kv->max_seq_len;
    return flare_decode_attn(ctx, kv, layer, num_heads, q, 1, &att, softcap, out, 0);
}
flare_kv* flare_backend_kv(flare_attn_ctx* ctx) { return ctx ? ctx->backend_kv : nullptr; }

}  // extern "C"
