/*
 * flare_attn.h — C ABI of the B200 attention engine for Flare.
 *
 * This is the boundary a Rust crate `flare-cuda` (beside flare-gpu) binds with
 * `extern "C"`; it replaces the attention / KV-cache hooks of flare-core's
 * `ComputeBackend` trait (flare-core/src/model.rs:176-618) and the attention / KV
 * shaders of flare-gpu.  Paths in comments are relative to the reference project.
 *
 * Conventions
 *  - every function returns a flare_status (0 = OK); nothing aborts or throws;
 *    flare_attn_last_error() gives the text of the last failure on a context.
 *  - one context = one CUDA device + one stream.  Calls on one context must be
 *    serialised by the caller (the Rust side keeps it behind a Mutex, as
 *    flare-gpu/src/backend.rs:183-188 does for its own state).
 *  - a pointer argument is host memory unless the function has an `on_device`
 *    flag and it is non-zero; host buffers are fully consumed / produced before
 *    the call returns, device buffers are used asynchronously on the context's
 *    stream and must stay alive until flare_attn_sync().
 *  - there is no CPU fallback: without a CUDA device every call fails with
 *    FLARE_ERR_CUDA.
 *
 * Layouts (row-major, last index fastest)
 *  - q   [batch][n_q][num_heads][head_dim]            f32
 *  - out [batch][n_q][num_heads][head_dim]            f32
 *  - a K or V row is [num_kv_heads][head_dim] = kv_dim values, exactly the row of
 *    flare-core's KvCache tensor [max_seq_len, num_kv_heads, head_dim]
 *    (flare-core/src/kv_cache.rs:431-446); a ring slot is position % max_seq_len.
 *  - query head h reads kv head h / (num_heads / num_kv_heads)
 *    (flare-core/src/model.rs:9877-9882).
 */
#ifndef FLARE_ATTN_H
#define FLARE_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define FLARE_API
#else
#define FLARE_API __attribute__((visibility("default")))
#endif

typedef struct flare_attn_ctx flare_attn_ctx;
typedef struct flare_kv flare_kv;

typedef enum {
    FLARE_OK = 0,
    FLARE_ERR_INVALID_ARG = 1,
    FLARE_ERR_UNSUPPORTED = 2,   /* softcap != 0 on the GPU path, head_dim outside the kernels' range ... */
    FLARE_ERR_OOM = 3,
    FLARE_ERR_CUDA = 4,
    FLARE_ERR_TIMEOUT = 5,
    FLARE_ERR_STATE = 6,         /* e.g. attention before any KV cache exists */
    FLARE_ERR_NCCL = 7,          /* the collective library failed or is missing (multi-GPU calls only) */
    FLARE_ERR_BOUNDS = 8         /* range-checked build only: a kernel computed an index outside its buffer */
} flare_status;

/* How a cache stores its rows. */
typedef enum {
    FLARE_KV_F32 = 0,       /* flare-core KvCache: f32 rows (kv_cache.rs:431-546) */
    FLARE_KV_Q8_0 = 1,      /* Q8_0 codec (flare-loader/src/quantize.rs:188-197): 32 int8 + one f16 scale */
    FLARE_KV_KIVI_REF = 2,  /* flare-core QuantizedKvCache, bit for bit (kv_cache.rs:35-420) */
    FLARE_KV_KIVI_G32 = 3   /* 2-bit, groups of 32, f16 scale+zero, 128-token f16 residual ring */
} flare_kv_dtype;

typedef enum { FLARE_DT_F32 = 0, FLARE_DT_BF16 = 1 } flare_dtype;

/* Raw planes of a cache, for flare_kv_export_plane / flare_kv_import_plane.
 * Sizes are per (layer, sequence); kv_dim = num_kv_heads * head_dim.
 *   F32       K, V                 f32  [max_seq][kv_dim]
 *   Q8_0      K_Q, V_Q             i8   [max_seq][kv_dim]
 *             K_SCALE, V_SCALE     f16  [max_seq][kv_dim/32]
 *   KIVI_REF  K_Q, V_Q             u8   [max_seq][kv_dim/4]     (kv_cache.rs:27-29)
 *             K_SCALE, K_MIN       f32  [kv_dim]                 running per-channel stats
 *             V_SCALE, V_MIN       f32  [max_seq]                per-token
 *             K_RES, V_RES         f32  [32][kv_dim]             residual window
 *   KIVI_G32  K_Q                  u8   [max_seq][kv_dim/4]      byte j of a slot holds channels 4j..4j+3
 *             K_SCALE              f16  [max_seq/32][kv_dim/16][2][16]  per 32-slot group and block of 16
 *                                       channels: 16 scales, then 16 zero points; channel r of the block at
 *                                       position 2 (r mod 8) + r div 8
 *             V_Q                  u8   [max_seq][kv_dim/4]
 *             V_SCALE              f16x2 [max_seq][kv_dim/32]    (scale, zero)
 *             K_RES, V_RES         f16  [128][kv_dim]            residual ring, slot % 128
 */
typedef enum {
    FLARE_PLANE_K = 0, FLARE_PLANE_V = 1,
    FLARE_PLANE_K_Q = 2, FLARE_PLANE_V_Q = 3,
    FLARE_PLANE_K_SCALE = 4, FLARE_PLANE_V_SCALE = 5,
    FLARE_PLANE_K_MIN = 6, FLARE_PLANE_V_MIN = 7,
    FLARE_PLANE_K_RES = 8, FLARE_PLANE_V_RES = 9,
    FLARE_PLANE_COUNT = 10
} flare_kv_plane;

/* ---------------------------------------------------------------- context */

/* Replaces WebGpuBackend::new (flare-gpu/src/backend.rs:219-228): binds CUDA device
 * `device` and creates the stream all work of this context runs on. */
FLARE_API int flare_attn_create(int device, flare_attn_ctx** out_ctx);
FLARE_API int flare_attn_destroy(flare_attn_ctx* ctx);
/* Run on a caller-owned cudaStream_t instead.  NULL restores the context's own stream; to run
 * on CUDA's legacy default stream pass cudaStreamLegacy, not 0. */
FLARE_API int flare_attn_set_stream(flare_attn_ctx* ctx, void* cuda_stream);
/* Replaces the blocking readback device.poll(Maintain::Wait) (flare-gpu/src/backend.rs:417). */
FLARE_API int flare_attn_sync(flare_attn_ctx* ctx);
FLARE_API const char* flare_attn_last_error(const flare_attn_ctx* ctx);
/* Kernels launched by this context so far (replaces nothing; for measurement). */
FLARE_API uint64_t flare_attn_launch_count(const flare_attn_ctx* ctx);
/* ComputeBackend::name (flare-core/src/model.rs:615-617): "cuda". */
FLARE_API const char* flare_attn_backend_name(void);

/* Per-call measurements, the counterpart of the reference's PrefillProfile / attention_ms
 * (flare-core/src/model.rs:1198-1236, 2784-2795), taken on the device instead of with a host clock.
 * While enabled, every attention call (decode, partial, step, prefill) is bracketed by two CUDA events on
 * the context's stream and is not overlapped with its predecessor.  flare_attn_get_stats waits for
 * the last measured call to finish.
 *   bytes   algorithmic K/V bytes of the attended slots in the cache's storage format
 *   flops   4 * query rows * head_dim * attended (query, key) pairs
 *   frac    achieved / peak: bytes per second over the HBM peak for decode, flops per second over the
 *           tensor peak for prefill; peaks are the caller's (flare_attn_set_peaks), default 7700 GB/s
 *           and 2250 TFLOP/s (nominal B200). */
typedef enum { FLARE_OP_NONE = 0, FLARE_OP_DECODE = 1, FLARE_OP_PREFILL = 2 } flare_stat_op;
/* Which kernel family served the last attention call of the context (whether or not stats are enabled). */
typedef enum {
    FLARE_PATH_NONE = 0,
    FLARE_PATH_GENERAL = 1,        /* CUDA-core split-KV kernel: every cache type and shape */
    FLARE_PATH_Q8_TENSOR = 2,      /* Q8_0, head_dim 64 / 128: TMA-staged tiles, int8 / f16 tensor-core products */
    FLARE_PATH_KIVI_TENSOR = 3,    /* group-32 2-bit cache, head_dim 64: TMA-staged code tiles, f16 tensor-core products */
    FLARE_PATH_PREFILL_TENSOR = 4  /* prefill, head_dim 64 / 128: tcgen05 / tensor-memory kernel */
} flare_kernel_path;
typedef struct {
    uint64_t calls;                /* measured calls so far */
    int32_t last_op;               /* flare_stat_op */
    int32_t last_path;             /* flare_kernel_path of the most recent attention call */
    double last_elapsed_us, last_bytes, last_flops, last_gbs, last_tflops, last_frac_of_peak;
    double total_elapsed_us, total_bytes, total_flops;
} flare_attn_stats;
FLARE_API int flare_attn_enable_stats(flare_attn_ctx* ctx, int on);
FLARE_API int flare_attn_set_peaks(flare_attn_ctx* ctx, double hbm_gbs, double tensor_tflops);
FLARE_API int flare_attn_get_stats(flare_attn_ctx* ctx, flare_attn_stats* out);

/* No counterpart in the reference.  Every wait inside the kernels of this library (on a tile's
 * mbarrier) is bounded: when it runs out the kernel records FLARE_ERR_TIMEOUT in the context's status
 * word and returns, and the next host call that reads results reports it.  This call exercises that
 * path without touching a cache: one warp waits on a barrier that nothing will ever complete, with a
 * limit of a few milliseconds.  Expected return value: FLARE_ERR_TIMEOUT; the context stays usable. */
FLARE_API int flare_attn_selftest_wait_timeout(flare_attn_ctx* ctx);

/* ---------------------------------------------------------------- KV cache */

/* Replaces KvCache::new / QuantizedKvCache::new / GpuKvCache::new
 * (flare-core/src/kv_cache.rs:448-473, 62-114; flare-gpu/src/kv_cache.rs:16-98) with a
 * batch dimension: `batch` independent sequences, each with its own ring state.
 * Q8_0 and KIVI_G32 need head_dim % 32 == 0; KIVI_G32 needs max_seq_len % 128 == 0;
 * KIVI_REF needs kv_dim % 4 == 0. */
FLARE_API int flare_kv_alloc(flare_attn_ctx* ctx, int num_layers, int batch, int max_seq_len,
                             int num_kv_heads, int head_dim, int kv_dtype, flare_kv** out_kv);
FLARE_API int flare_kv_free(flare_kv* kv);

/* Replaces KvCache::write + ComputeBackend::gpu_kv_write (flare-core/src/kv_cache.rs:475-481,
 * model.rs:287-296; GpuKvCache::write flare-gpu/src/kv_cache.rs:116-160): store the post-RoPE
 * row of one token of sequence `seq` at ring slot abs_position % max_seq_len of `layer`.
 * Quantised caches quantise on the device (QuantizedKvCache::write, kv_cache.rs:121-162).
 * The ring state is NOT advanced (flare_kv_advance does that once per token, after all
 * layers, as model.rs:2547 does). */
FLARE_API int flare_kv_write_f32(flare_kv* kv, int layer, int seq, int64_t abs_position,
                                 const float* key, const float* value, int on_device);

/* n_rows consecutive tokens, as if written and advanced one by one starting from the
 * current state of `seq` (replaces the bulk write after prefill, model.rs:2956-2979).
 * key/value are [n_rows][kv_dim].  Does not advance; call flare_kv_advance(kv, seq, n_rows)
 * after every layer has been written. */
FLARE_API int flare_kv_append_f32(flare_kv* kv, int layer, int seq, int n_rows,
                                  const float* key, const float* value, int on_device);

/* One decode step of the whole batch: row b of key/value ([batch][kv_dim]) is the new token
 * of sequence b and goes to that sequence's current ring position (the batched form of the
 * gpu_kv_write call at model.rs:2199-2206).  Does not advance. */
FLARE_API int flare_kv_write_step_f32(flare_kv* kv, int layer, const float* key, const float* value,
                                      int on_device);

/* Rotary position embedding fused into the step write (the reference rotates on the CPU right before the
 * write: apply_rope_with_table at flare-core/src/model.rs:2168-2183, then gpu_kv_write at 2199-2206).
 *
 * flare_kv_set_rope_table   the caller's RopeTable (model.rs:7184-7213): cos and sin, each
 *                           [table_len][head_dim / 2] f32, copied to the device.  The library never evaluates
 *                           sin / cos itself, so the rotation uses the caller's values bit for bit; a caller with
 *                           positions beyond the reference's 8192-row cap passes a longer table (every entry is
 *                           the expression the reference's inline fallback, model.rs:7299-7332, evaluates).
 * flare_kv_write_step_rope_f32   flare_kv_write_step_f32 on key rows that have NOT been rotated yet: row b is
 *                           rotated for absolute position positions[b] (half-split pairs, model.rs:7280-7289:
 *                           two multiplies and a subtract / an add, not fused) and quantised / stored in the same
 *                           kernel (f32 and Q8_0 caches; the 2-bit caches rotate in a kernel of their own first).
 *                           Values are stored as given.  positions is a host array of `batch` entries.
 * flare_rope_rows_f32       the same rotation in place on [n_rows][num_heads][head_dim] rows (for q). */
FLARE_API int flare_kv_set_rope_table(flare_kv* kv, const float* cos, const float* sin, int table_len);
FLARE_API int flare_kv_write_step_rope_f32(flare_kv* kv, int layer, const float* key, const float* value,
                                           const int64_t* positions, int on_device);
FLARE_API int flare_rope_rows_f32(flare_kv* kv, float* rows, int n_rows, int num_heads, const int64_t* positions,
                                  int on_device);

/* KvCache::advance (kv_cache.rs:484-489) applied n times; seq < 0 = every sequence. */
FLARE_API int flare_kv_advance(flare_kv* kv, int seq, int n);
/* KvCache::len / position (kv_cache.rs:502-513). */
FLARE_API int flare_kv_get_state(const flare_kv* kv, int seq, int64_t* position, int64_t* length);
/* Restore a state previously read with flare_kv_get_state (checkpoint / resume). */
FLARE_API int flare_kv_set_state(flare_kv* kv, int seq, int64_t position, int64_t length);
/* KvCache::truncate_to (kv_cache.rs:521-531): ignored once the ring has wrapped. */
FLARE_API int flare_kv_truncate(flare_kv* kv, int seq, int64_t target_len);
/* KvCache::clear (kv_cache.rs:534-545): zero-fill and reset; seq < 0 = every sequence. */
FLARE_API int flare_kv_clear(flare_kv* kv, int seq);

/* Byte size of one plane for one (layer, sequence); 0 if the cache has no such plane. */
FLARE_API size_t flare_kv_plane_bytes(const flare_kv* kv, int plane);
FLARE_API int flare_kv_export_plane(flare_kv* kv, int layer, int seq, int plane, void* dst,
                                    size_t bytes, int on_device);
FLARE_API int flare_kv_import_plane(flare_kv* kv, int layer, int seq, int plane, const void* src,
                                    size_t bytes, int on_device);
/* Q8_0 rows as the GGUF block stream [n_slots][kv_dim/32] x 34 bytes (f16 LE scale, 32 i8),
 * the format of flare-loader/src/quantize.rs:188-197. */
FLARE_API int flare_kv_import_q8_0_blocks(flare_kv* kv, int layer, int seq, int first_slot, int n_slots,
                                          const void* k_blocks, const void* v_blocks, int on_device);
FLARE_API int flare_kv_export_q8_0_blocks(flare_kv* kv, int layer, int seq, int first_slot, int n_slots,
                                          void* k_blocks, void* v_blocks, int on_device);

/* The f32 view attention reads: [max_seq_len][kv_dim] indexed by ring slot, computed with
 * the literal reference formulae so that it is bit-identical to the CPU:
 *   Q8_0      (i8 as f32) * f16_to_f32(scale)             (quantize.rs:188-197)
 *   KIVI_REF  QuantizedKvCache::dequant_keys/_values        (kv_cache.rs:189-250, 374-391)
 *   KIVI_G32  code * scale + zero, residual ring for the newest 128 tokens
 * Either output may be NULL. */
FLARE_API int flare_kv_export_dequant(flare_kv* kv, int layer, int seq, float* k_out, float* v_out,
                                      int on_device);

/* ---------------------------------------------------------------- attention */

/* Replaces ComputeBackend::grouped_query_attention_from_gpu_cache (model.rs:311-322;
 * flare-gpu/src/backend.rs:4885-4979) and the CPU routine it stands for
 * (cpu_grouped_query_attention_into, model.rs:9849-9905), for `batch` sequences and
 * n_q causally ordered queries per sequence (n_q = 1: plain decode; n_q = 1 + drafts:
 * speculative verify, flare-core/src/generate.rs:258-303 done in one call).
 *   attend_len[b]  slots 0..attend_len[b]-1 of sequence b are read by the LAST query;
 *                  query i reads attend_len[b] - (n_q-1-i) slots.  NULL = ring state:
 *                  min(length + 1, max_seq_len)  (model.rs:2209; clamped once the ring is full).
 *   softcap        must be 0 (the wgpu backend asserts the same, backend.rs:4907-4910).
 * K/V are streamed once per kv head for up to 4 query heads that share it and one query; with several queries
 * (or more than 4 heads per kv head) a Q8_0 cache with head_dim 64 / 128 is streamed once per pair of them.  With host buffers
 * (on_device = 0) the call returns when `out` is filled; an `out` in page-locked memory
 * (cudaHostAlloc / cudaHostRegister) is written by the kernels directly, with no copy after them. */
FLARE_API int flare_decode_attn(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads,
                                const float* q, int n_q, const int* attend_len, float softcap,
                                float* out, int on_device);

/* One decode step of one layer for a host that batches sequences: what ComputeBackend::gpu_kv_write
 * followed by grouped_query_attention_from_gpu_cache (model.rs:2199-2224) collapse to.  Row b of
 * key/value ([batch][kv_dim], post-RoPE) is stored at sequence b's current ring position exactly as
 * flare_kv_write_step_f32 does, then q ([batch][1][num_heads][head_dim]) attends min(length + 1,
 * max_seq_len) slots exactly as flare_decode_attn does.  The ring state is not advanced.  With host
 * buffers the call synchronises once, when `out` is filled, and the inputs cross the bus in as few
 * transfers as their memory allows: one, straight from the caller's memory, when they are page-locked
 * and contiguous as [K rows][V rows][q]; three when page-locked but apart; one through a page-locked
 * staging slot of the library when pageable.  A page-locked `out` is written by the kernel itself. */
FLARE_API int flare_decode_step(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads,
                                const float* key, const float* value, const float* q, float* out,
                                int on_device);

/* No counterpart in the reference.  flare_decode_attn for callers that must not allocate
 * device memory when they call in: an inference server that gave all GPU memory to its own
 * pool at start-up, a real-time callback that may not wait on the driver's allocator, a host
 * whose policy forbids cudaMalloc after initialisation.  This entry point calls no cudaMalloc,
 * cudaFree or other allocating routine: the split-KV workspace is a fixed 8 MiB __device__
 * array inside the library (flare_decode_attn_noalloc_scratch_bytes()), which every GPU that
 * loads the library carries until the process exits.
 *   - q_dev and out_dev are DEVICE pointers owned by the caller ([batch][n_q][num_heads][head_dim]
 *     f32); attend_len is a host array as in flare_decode_attn (NULL = ring state).
 *   - f32 and Q8_0 caches, head_dim 64 or 128, batch <= 256 (more is refused with
 *     FLARE_ERR_INVALID_ARG).  A call whose partial results (rows x splits x (head_dim + 2)
 *     floats) would not fit in the array is refused the same way, with a message that names both
 *     sizes, before anything is put on the stream; with the split rule in use and batch <= 256
 *     the partials stay below 5 MiB, so that refusal is a guard, not a limit callers meet.
 *   - it always runs the general CUDA-core split-KV kernel.  For a Q8_0 cache flare_decode_attn
 *     picks the faster tensor-core kernel instead, so the two entry points agree within the
 *     output tolerance (2e-3 + 1e-3 |x|), not bit for bit, and this one is the slower of the two.
 *   - the first call on a device is the set-up call: it looks up the array's device address
 *     (cudaGetSymbolAddress), and the driver may load the library's device image, array
 *     included, at that moment.  This first call should come before any stream capture begins.
 *     The first launch of each kernel variant (cache type x head_dim x heads per KV head) may
 *     likewise make the driver load code.  The per-sequence lengths travel to the device through
 *     a copy from the host stack on every call.
 *   - every call on a device shares the one array and leaves its partial results in it; a
 *     call overwrites what it reads, so nothing needs clearing, but two calls that overlap on
 *     the GPU (different streams or contexts) race: serialise them. */
FLARE_API int flare_decode_attn_noalloc(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads,
                                        const float* q_dev, int n_q, const int* attend_len,
                                        float* out_dev);
FLARE_API size_t flare_decode_attn_noalloc_scratch_bytes(void);

/* Split-KV building blocks for one sequence spread over several GPUs (no counterpart in
 * the reference, which is single-device).  Attends slots [slot_begin, slot_end) only and
 * returns, per (sequence, query, head), [m, l, o[head_dim]] with o unnormalised:
 * partial is [batch][n_q][num_heads][head_dim + 2]. */
FLARE_API int flare_decode_attn_partial(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads,
                                        const float* q, int n_q, int slot_begin, int slot_end,
                                        float* partial, int on_device);
/* Log-sum-exp merge of n_parts partials, each [rows][head_dim + 2], into out [rows][head_dim]. */
FLARE_API int flare_merge_partials(flare_attn_ctx* ctx, const float* partials, int n_parts, int rows,
                                   int head_dim, float* out, int on_device);

/* ---------------------------------------------------------------- projections either side of attention
 * The Q8_0-weight matrix-vector products that feed attention (the Q, K and V projections,
 * flare-core/src/model.rs:2016-2136) and follow it (the output projection, model.rs:2249-2291), for `batch`
 * input vectors; replaces matvec_q8_0_preq_into + quantize_input_q8_0 (model.rs:7976-8100, 5507-5527) and
 * flare-gpu/shaders/dequant_matvec_q8_0.wgsl.
 *
 * flare_weight_upload_q8_0   a weight matrix [rows][cols] as the GGUF Q8_0 block stream the loader hands out
 *                            (rows * cols / 32 blocks of 34 bytes, flare-loader/src/quantize.rs:188-197), copied
 *                            to the device once and kept there as an int8 plane and an f16 scale plane (the same
 *                            numbers; a block's weights then start on a 32-byte boundary).  cols % 32 == 0.
 * flare_matvec_q8_0          out[b][r] = row r of the matrix . x[b], computed the reference's way so that the
 *                            result is bit-identical to the CPU (x86_64 branch): x is quantised per block of 32
 *                            (scale kept in f32), the int8 dot of a block is exact, and a row's blocks are added
 *                            in ascending order as sum += (w_scale * x_scale) * dot with separate multiplies
 *                            and add.  x [batch][cols], out [batch][rows], batch <= 256; a weight row is read
 *                            from device memory once for the whole batch. */
typedef struct flare_weight flare_weight;
FLARE_API int flare_weight_upload_q8_0(flare_attn_ctx* ctx, const void* blocks, int rows, int cols, flare_weight** out_w);
FLARE_API int flare_weight_free(flare_weight* w);
FLARE_API int flare_matvec_q8_0(flare_attn_ctx* ctx, const flare_weight* w, const float* x, int batch, float* out,
                                int on_device);

/* ---------------------------------------------------------------- the whole token on the device
 * Replaces ComputeBackend::forward_single_token_gpu (flare-core/src/model.rs:1697-1734;
 * flare-gpu/src/backend.rs:4010-4375): weights, cache and every intermediate stay on the device, a token costs one
 * upload of its embedding row and one download of its logits.  The arithmetic is the CPU's Q8_0 path
 * (Model::forward_layers, model.rs:2010-2548, with use_q8_attn / use_q8_ffn): rmsnorm_quantize_q8_0 -> fused
 * [wq; wk; wv] -> RoPE -> cache write -> attention -> wo -> residual -> rmsnorm_quantize_q8_0 -> fused
 * [w_gate; w_up] -> silu(gate) * up -> w_down -> residual; then the final norm and the output matrix (Q8_0 as at
 * model.rs:1759-1770, or f32 as at 1771-1779).  Integer dots, block sums, the rotation and every quantisation step
 * are the reference's operation for operation; the sum of squares of a norm is a tree where the CPU adds left to
 * right and exp() is the device's, so logits agree with the CPU within a tolerance, not bit for bit.
 * Not handled: biases (Qwen2), post-norms and soft-caps (Gemma 2), MoE, LoRA.
 *
 * flare_model_set_layer   host pointers: the norms are [hidden_dim] f32; the matrices are GGUF Q8_0 block streams,
 *                         qkv [(num_heads + 2 num_kv_heads) * head_dim][hidden_dim] = wq, wk, wv stacked by rows
 *                         (FusedLayerWeights::qkv), wo [hidden_dim][num_heads * head_dim], gate_up
 *                         [2 * intermediate_dim][hidden_dim] = w_gate, w_up stacked, down [hidden_dim][intermediate_dim].
 * flare_model_set_output  output_norm [hidden_dim] and exactly one of the output matrix as Q8_0 blocks or as f32,
 *                         [vocab_size][hidden_dim].
 * flare_forward_token     one token for each of the cache's `batch` sequences: token_embed [batch][hidden_dim] and
 *                         positions[batch] (absolute, for the rotary table set with flare_kv_set_rope_table) from the
 *                         host, logits [batch][vocab_size] to the host.  Every layer's K/V row is written at the
 *                         ring position and the cache is advanced by one at the end, as Model::forward does. */
typedef struct flare_model flare_model;
typedef struct flare_model_config {
    int hidden_dim, num_heads, num_kv_heads, head_dim, intermediate_dim, vocab_size, num_layers;
    float rms_norm_eps;
} flare_model_config;
FLARE_API int flare_model_create(flare_attn_ctx* ctx, const flare_model_config* cfg, flare_model** out_model);
FLARE_API int flare_model_set_layer(flare_model* m, int layer, const float* attn_norm, const void* qkv_q8_0,
                                    const void* wo_q8_0, const float* ffn_norm, const void* gate_up_q8_0,
                                    const void* down_q8_0);
FLARE_API int flare_model_set_output(flare_model* m, const float* output_norm, const void* output_q8_0,
                                     const float* output_f32);
FLARE_API int flare_model_free(flare_model* m);
FLARE_API int flare_forward_token(flare_attn_ctx* ctx, flare_model* m, flare_kv* kv, const float* token_embed,
                                  const int64_t* positions, float* logits);

/* ---------------------------------------------------------------- one sequence over several GPUs
 * No counterpart in the reference (single device).  One process per GPU; every process creates its context,
 * then all of them make the same sequence of calls below.  The recurrence merged across GPUs is the block
 * form of flare-core/src/model.rs:9945-9956.
 *
 * flare_attn_comm_unique_id   rank 0 obtains a 128-byte id and hands it to the other ranks over any host
 *                             channel (the Rust side: whatever already connects its workers).
 * flare_attn_comm_init        collective: joins the NCCL communicator (libnccl.so.2 is loaded at run time, or
 *                             the file named by FLARE_NCCL_LIB).  world = 1 needs no id and no NCCL.
 * flare_attn_comm_enable_direct  collective, optional: sets up the exchange without a collective call — every
 *                             rank allocates a record buffer for up to max_rows = batch * num_heads rows of
 *                             head_dim (64 or 128) floats and maps its peers' buffers (CUDA IPC: one process per
 *                             GPU with peer access).  Afterwards the kernel that finishes a rank's attention
 *                             stores its records straight into the peers' buffers and merges as soon as theirs
 *                             have arrived, waiting at most the limit of flare_attn_comm_set_wait_ms (default
 *                             2000 ms); when the wait runs out the call reports FLARE_ERR_TIMEOUT and the
 *                             context stays usable.  Without it the records travel by ncclAllGather.
 *                             The set-up ends with a timed probe of a few exchanges; if the slowest rank needs
 *                             more than 100 us per exchange the mode is switched off again on every rank (the
 *                             call still returns FLARE_OK; flare_attn_comm_info tells, flare_attn_comm_probe_us
 *                             gives the measured time, flare_attn_last_error the reason).
 * flare_attn_comm_destroy     frees the buffers and the communicator; make sure no rank is still inside a
 *                             multi-GPU call (a host barrier) before any rank destroys.
 *
 * flare_decode_attn_splitkv_multi   `kv` holds this rank's share of the sequence in its slots
 *                             0 .. n_local_slots-1 (a contiguous range of the whole sequence; which range does
 *                             not matter to the result).  q [batch][1][num_heads][head_dim] is the same on every
 *                             rank; every rank receives the attention output over the whole sequence in `out`
 *                             [batch][1][num_heads][head_dim].  head_dim 64 or 128.  Without a communicator, or in
 *                             a world of one, it is flare_decode_attn over the slots given.
 * NCCL failures are reported as FLARE_ERR_NCCL with NCCL's own message in flare_attn_last_error. */
#define FLARE_COMM_ID_BYTES 128
FLARE_API int flare_attn_comm_unique_id(void* id_out);
FLARE_API int flare_attn_comm_init(flare_attn_ctx* ctx, const void* id, int rank, int world);
FLARE_API int flare_attn_comm_enable_direct(flare_attn_ctx* ctx, int max_rows, int head_dim);
FLARE_API int flare_attn_comm_set_wait_ms(flare_attn_ctx* ctx, unsigned wait_ms);
FLARE_API int flare_attn_comm_info(const flare_attn_ctx* ctx, int* rank, int* world, int* direct);
FLARE_API double flare_attn_comm_probe_us(const flare_attn_ctx* ctx);
FLARE_API int flare_attn_comm_destroy(flare_attn_ctx* ctx);
FLARE_API int flare_decode_attn_splitkv_multi(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads,
                                              const float* q, int n_local_slots, float* out, int on_device);
/* Runs the give-up path of the direct exchange on one GPU, without a second rank and without a fault: a
 * two-rank exchange laid out in this device's own memory in which rank 1 never publishes; the 50 ms wait
 * runs out.  Expected return value: FLARE_ERR_TIMEOUT; the context stays usable. */
FLARE_API int flare_attn_comm_selftest_missing_peer(flare_attn_ctx* ctx);

/* Replaces ComputeBackend::grouped_query_attention (model.rs:246-267;
 * flare-gpu/src/backend.rs:4701-4811): K/V given as host f32 [seq_len][kv_dim]. */
FLARE_API int flare_gqa_attention_host(flare_attn_ctx* ctx, const float* q, const float* k_cache,
                                       const float* v_cache, int num_heads, int num_kv_heads,
                                       int head_dim, int seq_len, float softcap, float* out);

/* Replaces ComputeBackend::prefill_attention_gpu (model.rs:336-368;
 * flare-gpu/src/backend.rs:4981-5022, 2461-2533): causal self-attention of `batch`
 * prompts of seq_len tokens; row t attends rows max(0, t-window+1)..=t (window 0 = all).
 * q [batch][seq_len][num_heads][head_dim]; k, v [batch][seq_len][num_kv_heads][head_dim];
 * in_dtype / out_dtype are flare_dtype.  Accumulation is f32.  At head_dim 64 / 128 the products run
 * on the tensor cores: bf16 inputs as they are; f32 inputs (the trait hook's type) rounded to f16
 * (11 significant bits; a tensor whose largest magnitude exceeds 2^15 is scaled by a power of two
 * first, exactly), which keeps the result within 2e-3 + 1e-3 |x| of the f32 CPU loop.  Other
 * head sizes run in f32 on the general kernel. */
FLARE_API int flare_prefill_attn(flare_attn_ctx* ctx, const void* q, const void* k, const void* v,
                                 int in_dtype, int batch, int seq_len, int num_heads, int num_kv_heads,
                                 int head_dim, int window, float softcap, void* out, int out_dtype,
                                 int on_device);

/* ---------------------------------------------------------------- trait-shaped shims
 * The exact ComputeBackend attention hooks, batch 1, host f32 in and out. */

/* ComputeBackend::init_gpu_kv_cache (model.rs:274-281): f32 cache owned by the context. */
FLARE_API int flare_backend_init_gpu_kv_cache(flare_attn_ctx* ctx, int num_layers, int max_seq_len,
                                              int num_kv_heads, int head_dim);
/* Same, choosing the storage (no counterpart: the trait has no quantised-cache notion). */
FLARE_API int flare_backend_init_gpu_kv_cache_dtype(flare_attn_ctx* ctx, int num_layers, int max_seq_len,
                                                    int num_kv_heads, int head_dim, int kv_dtype);
/* ComputeBackend::gpu_kv_write (model.rs:287-296). */
FLARE_API int flare_backend_gpu_kv_write(flare_attn_ctx* ctx, int layer, int64_t position,
                                         int num_kv_heads, int head_dim, const float* key,
                                         const float* value);
/* ComputeBackend::has_gpu_kv_cache (model.rs:299-301): 1 or 0. */
FLARE_API int flare_backend_has_gpu_kv_cache(const flare_attn_ctx* ctx);
/* ComputeBackend::grouped_query_attention_from_gpu_cache (model.rs:311-322): attends ring
 * slots 0..seq_len-1 (seq_len is clamped to max_seq_len). */
FLARE_API int flare_backend_gqa_from_gpu_cache(flare_attn_ctx* ctx, const float* q, int layer,
                                               int num_heads, int num_kv_heads, int head_dim,
                                               int seq_len, float softcap, float* out);
/* The context-owned cache, e.g. to advance or truncate it (Model::truncate_kv_cache,
 * model.rs:4835-4840); NULL before init. */
FLARE_API flare_kv* flare_backend_kv(flare_attn_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* FLARE_ATTN_H */
