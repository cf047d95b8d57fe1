// Internal declarations shared by the .cu files of libflare_attn.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <string>
#include <vector>

#include "../../include/flare_attn.h"

#define FLARE_G32_RESIDUAL 128
#define FLARE_G32_TILE 64          // slots per tile of the group-32 tensor-core decode kernel (TMA box)
// Group-32 KIVI key metadata: per 32-slot group a row of kv_dim (scale, zero) f16 pairs stored per block of
// 16 channels as 16 scales then 16 zero points, channel r of the block at position 2 (r mod 8) + r div 8 —
// the pair (r, r + 8), whose 2-bit codes sit 16 bits apart in a code word, is adjacent.  Index of the scale
// in f16 units; the zero point is 16 entries further.
#define FLARE_G32_KMETA_INDEX(c) ((((c) >> 4) << 5) + (((c) & 7) << 1) + (((c) >> 3) & 1))
#define FLARE_REF_RESIDUAL 32
#define FLARE_SMALL_SLOTS 64
#define FLARE_ROW_SLOTS 8

struct FlareComm;        // collective state of a context (multi.cu)

struct flare_attn_ctx {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    std::string last_error;
    uint64_t launches = 0;
    // scratch owned by the context (grown on demand, never shrunk)
    void* d_work = nullptr;      size_t work_bytes = 0;     // split-KV partials
    void* d_stage_in = nullptr;  size_t stage_in_bytes = 0; // device copy of host q / K / V
    void* d_stage_out = nullptr; size_t stage_out_bytes = 0;
    void* d_misc = nullptr;      size_t misc_bytes = 0;     // attend_len and other small arrays
    void* d_misc2 = nullptr;     size_t misc2_bytes = 0;    // small arrays of the prefill path
    void* d_conv = nullptr;      size_t conv_bytes = 0;     // dtype-converted prefill operands
    void* h_pinned = nullptr;    size_t pinned_bytes = 0;
    // ring of page-locked staging slots for small host inputs (new K/V rows): the caller's buffer is
    // copied here by the CPU, the transfer to the device is then asynchronous and the call need not wait
    void* h_rows = nullptr;      size_t rows_slot_bytes = 0;
    cudaEvent_t rows_events[FLARE_ROW_SLOTS] = {};
    uint64_t rows_counter = 0;
    // inputs of flare_decode_step already classified as page-locked or pageable (a decode loop passes the same
    // buffers every token; the driver query costs about a microsecond per pointer)
    struct { const void* p; bool locked; } lock_cache[64] = {};
    unsigned lock_cache_next = 0;
    uint64_t small_counter = 0;
    std::vector<int> small_last;       // host copy of the last uploaded (ring, attend) arrays
    const void* small_last_dev = nullptr;
    cudaEvent_t small_events[FLARE_SMALL_SLOTS] = {};
    int work_phase = 0;              // which half of d_work the last split-KV launch used
    // true while the last kernel put on the stream is one that never writes a cache or q, so that the
    // next decode kernel may overlap its prologue with it (programmatic dependent launch)
    bool last_launch_overlappable = false;
    int* h_err = nullptr;            // status word in page-locked, device-mapped host memory: a kernel whose bounded wait gives up stores a code here
    int* d_err = nullptr;            // the device's address of the same word (what kernels are given)
    int* d_gaveup = nullptr;         // device memory: set by an exchange whose wait ran out, so that the calls queued behind
                                     // it give up at once; looked at by every CTA, hence not in host memory (a read of
                                     // the mapped word crosses PCIe: 1024 warps doing so cost a call a millisecond)
    int sm_count = 148;
    flare_kv* backend_kv = nullptr;  // cache created by flare_backend_init_gpu_kv_cache
    FlareComm* comm = nullptr;       // set by flare_attn_comm_init
    // per-call measurements (flare_attn_enable_stats): two events around the kernels of a call
    bool stats_on = false, stats_pending = false;
    cudaEvent_t stats_ev[2] = {};
    int stats_op = 0;
    int last_path = 0;               // flare_kernel_path of the most recent attention call
    double stats_bytes = 0.0, stats_flops = 0.0;
    double peak_hbm_gbs = 7700.0, peak_tflops = 2250.0;
    flare_attn_stats stats = {};
};

struct flare_kv {
    flare_attn_ctx* ctx = nullptr;
    int num_layers = 0, batch = 0, max_seq_len = 0, num_kv_heads = 0, head_dim = 0, kv_dim = 0;
    int dtype = 0;
    void* plane[FLARE_PLANE_COUNT] = {};
    size_t plane_bytes[FLARE_PLANE_COUNT] = {};   // per (layer, sequence)
    std::vector<int64_t> position, length;       // per sequence
    // TMA maps of the Q8_0 payload planes: (head_dim bytes, kv head, slot, layer*batch + seq), box 32 slots of one head
    CUtensorMap kq_map, vq_map;
    bool has_maps = false;
    bool maps_whole_rows = false;
    // TMA maps of the group-32 KIVI code planes: (16 bytes = 64 codes of one head, slot, kv head, layer*batch + seq)
    CUtensorMap g32_kmap, g32_vmap;
    bool has_g32_maps = false;
    // rotary table of the caller (RopeTable, flare-core/src/model.rs:7184-7213): cos and sin, [rope_len][head_dim / 2]
    float* rope_cos = nullptr;
    float* rope_sin = nullptr;
    int rope_len = 0;
    inline char* plane_ptr(int p, int layer, int seq) const {
        return (char*)plane[p] + ((size_t)layer * batch + seq) * plane_bytes[p];
    }
};

int flare_set_error(flare_attn_ctx* ctx, int code, const char* fmt, ...);

#define FLARE_CUDA_OK(ctx, expr)                                                           \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess)                                                             \
            return flare_set_error((ctx), _e == cudaErrorMemoryAllocation ? FLARE_ERR_OOM : FLARE_ERR_CUDA, \
                                   "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
    } while (0)

#define FLARE_TRY(expr)                 \
    do {                                \
        int _s = (expr);                \
        if (_s != FLARE_OK) return _s;  \
    } while (0)

#define FLARE_LAUNCH_CHECK(ctx)                                                            \
    do {                                                                                   \
        (ctx)->launches++;                                                                 \
        (ctx)->last_launch_overlappable = false;                                                                 \
        cudaError_t _e = cudaGetLastError();                                               \
        if (_e != cudaSuccess)                                                             \
            return flare_set_error((ctx), FLARE_ERR_CUDA, "kernel launch failed: %s (%s:%d)", \
                                   cudaGetErrorString(_e), __FILE__, __LINE__);            \
    } while (0)

int flare_ensure(flare_attn_ctx* ctx, void** buf, size_t* have, size_t need);
int flare_ensure_pinned(flare_attn_ctx* ctx, size_t need);

// ---- device views of one (layer) of a cache, handed to kernels by value -------------------
struct KvLayerView {
    int dtype, batch, max_seq_len, num_kv_heads, head_dim, kv_dim;
    const char* plane[FLARE_PLANE_COUNT];     // base of (layer, seq 0)
    size_t stride[FLARE_PLANE_COUNT];         // bytes between sequences
};
KvLayerView flare_layer_view(const flare_kv* kv, int layer);

// ---- kernels-in-other-files entry points (host launchers) ----------------------------------
struct DecodeArgs {
    KvLayerView kv;
    const float* q;        // device [batch][n_q][nh][hd]
    float* out;            // device: final [batch][n_q][nh][hd] or partial [..][hd+2]
    const int* attend_len; // device [batch]  (slots seen by the last query)
    const int2* ring;      // device [batch]  (position, length) — KIVI caches need it
    int batch, n_q, num_heads;
    int slot_begin, slot_end;  // restrict to [slot_begin, slot_end) (slot_end < 0: no restriction)
    int want_partial;          // 1: write [m, l, o] unnormalised
    int causal_q;              // 1: query i of n_q reads attend_len - (n_q-1-i) slots; 0: all read attend_len
    int max_attend;            // max over batch of attend_len (host-known upper bound)
    int window;                // > 0: every query reads at most its newest `window` slots (sliding-window prefill)
    int layer;
    const CUtensorMap *kmap, *vmap;   // Q8_0 payload maps (null when the cache has none)
    int whole_rows;                   // maps deliver [head][32 slots][head_dim] in one copy
    const flare_kv* kv_obj;           // the cache itself (tensor maps, ring state)
    const int* h_attend;              // host copy of attend_len (valid during the call), or null
    // defer_merge (with want_partial): the launcher leaves the per-range records unmerged and reports where they
    // are — [row][n_split][head_dim + 2], maximum in log2 units — so that the caller's own kernel merges them
    // (the multi-GPU exchange does, together with the records of the other ranks)
    int defer_merge = 0;
    const float** work_out = nullptr;
    int* n_split_out = nullptr;
};
int flare_launch_decode(flare_attn_ctx* ctx, const DecodeArgs& a);
int flare_launch_decode_generic(flare_attn_ctx* ctx, const DecodeArgs& a);
bool flare_decode_q8_supported(const DecodeArgs& a);
int flare_launch_decode_q8(flare_attn_ctx* ctx, const DecodeArgs& a);
int flare_check_device_error(flare_attn_ctx* ctx);
bool flare_decode_g32_supported(const DecodeArgs& a, const flare_kv* kv);
int flare_launch_decode_g32(flare_attn_ctx* ctx, const DecodeArgs& a, const flare_kv* kv);
int flare_decode_noalloc(flare_attn_ctx* ctx, const flare_kv* kv, int layer, int num_heads, const float* q_dev,
                         int n_q, const int* attend_len, float* out_dev);
size_t flare_noalloc_scratch_bytes();
int flare_launch_merge(flare_attn_ctx* ctx, const float* partials, size_t part_stride_floats, int n_parts,
                       int rows, int head_dim, float* out, int want_partial);

// ---- one sequence split over several GPUs (multi.cu) --------------------------------------------
void flare_comm_free(flare_attn_ctx* ctx);
// Called by the decode path after its kernels when the call is a multi-GPU one: exchanges this rank's records
// with the other ranks and writes the merged attention output.
int flare_multi_tail(flare_attn_ctx* ctx, const float* work, int n_split, int rows, int head_dim, float* out);
// Log-sum-exp merge of per-row slot-range records [row][n_split][head_dim + 2] (maximum in log2 units, n_split <= 256,
// head_dim a multiple of 32) into the attention output [row][head_dim], or (want_partial) into one record per row
// with the maximum in natural units.  Launched with programmatic stream serialisation: it waits for its predecessor.
int flare_launch_merge_splits(flare_attn_ctx* ctx, const float* work, int n_split, int rows, int head_dim, float* out,
                              int want_partial);
extern "C" int flare_decode_common(flare_attn_ctx* ctx, flare_kv* kv, int layer, int num_heads, const float* q, int n_q,
                        const int* attend_len, float softcap, int slot_begin, int slot_end, int want_partial,
                        int causal_q, float* out, int on_device, const float* q_staged = nullptr, int multi = 0);

struct PrefillArgs {
    const void *q, *k, *v; void* out;   // device
    int in_dtype, out_dtype, batch, seq_len, num_heads, num_kv_heads, head_dim, window;
    int f16_ops = 0;                    // tensor-core operands are f16 (converted f32 inputs) instead of bf16
    const float* descale = nullptr;     // device [2]: undoes the conversion's power-of-two scaling (f16_ops only)
};
int flare_launch_prefill(flare_attn_ctx* ctx, const PrefillArgs& a);
int flare_launch_prefill_pp(flare_attn_ctx* ctx, const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm,
                            const PrefillArgs& a);

int flare_launch_kv_write(flare_kv* kv, int layer, int seq, int64_t first_abs_position, int64_t length_before,
                          int n_rows, const float* d_key, const float* d_value);
// d_positions (with the cache's rotary table): the key rows are rotated for these absolute positions on their way
// into the cache; null = stored as given
int flare_launch_kv_write_step(flare_kv* kv, int layer, const int2* d_ring, const float* d_key, const float* d_value,
                               const long long* d_positions = nullptr, float* d_q_rows = nullptr, int q_heads = 0);
int flare_launch_rope_rows(flare_kv* kv, float* d_rows, int n_rows, int num_heads, const long long* d_positions);
extern "C" int flare_kv_write_step_rope_device(flare_kv* kv, int layer, const float* d_key, const float* d_value, const long long* d_pos,
                                               float* d_q_rows, int q_heads);
// Programmatic dependent launch for chains of small kernels (the forward pass): a kernel launched with
// flare_launch_pdl may be scheduled while its predecessor in the stream still runs; it begins with
// flare_pdl_wait(), which returns once the predecessor has completed and its writes are visible, and then lets its
// own successor be scheduled with flare_pdl_trigger().  Nothing is read or written before the wait, so the only
// effect is that the launch latency of a kernel hides behind the kernel before it.
#ifdef __CUDACC__
__device__ __forceinline__ void flare_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void flare_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename... KArgs, typename... Args>
inline cudaError_t flare_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif
// matvec.cu: the two halves of flare_matvec_q8_0 on device buffers
struct flare_weight;
int flare_launch_quantize_input(flare_attn_ctx* ctx, const float* d_x, size_t n_blocks, int8_t* d_xq, float* d_xs);
int flare_launch_matvec_q8_0_preq(flare_attn_ctx* ctx, const flare_weight* w, const int8_t* d_xq, const float* d_xs, int batch,
                                  float* d_out, int accumulate);
void flare_weight_dims(const flare_weight* w, int* rows, int* cols);
int flare_launch_kv_export_dequant(flare_kv* kv, int layer, int seq, float* d_k, float* d_v);
int flare_launch_q8_blocks(flare_kv* kv, int layer, int seq, int first_slot, int n_slots, void* d_kb, void* d_vb,
                           int to_blocks);

// ---- device codecs ---------------------------------------------------------------------------
#ifdef __CUDACC__
// 2-bit code i of a packed stream (flare-core/src/kv_cache.rs:374-391).
__device__ __forceinline__ float q2_code(const uint8_t* packed, int i) {
    return (float)((packed[i >> 2] >> ((i & 3) * 2)) & 3);
}
// code * scale + min as a separate multiply and add, never fused.
__device__ __forceinline__ float q2_dequant(float code, float scale, float mn) {
    return __fadd_rn(__fmul_rn(code, scale), mn);
}
// A kernel reports a status (FLARE_ERR_TIMEOUT ...) by storing it into the context's status word, which lives in
// page-locked host memory mapped into the device: the host reads it after synchronising, with no copy.  A plain
// store: the word only ever goes from 0 to a code, and every writer writes the same kind of code.
__device__ __forceinline__ void flare_report(int* status_word, int code) {
    *reinterpret_cast<volatile int*>(status_word) = code;
}
// Range-checked build (-DFLARE_DEBUG_BOUNDS, `python -m flarellm_b200.build --variant _dbg -DFLARE_DEBUG_BOUNDS`):
// the kernels that compute shared-memory offsets by hand (swizzled tiles, ldmatrix rows, stage rings) and the
// records they write to global memory verify every such offset against the extent of its buffer.  A violation
// stores FLARE_ERR_BOUNDS in the context's status word and the access is redirected to offset 0 — nothing traps,
// nothing is read or written out of range — so the next host call that reads results reports it.  In the
// product build the macro is the identity and costs nothing.
#ifdef FLARE_DEBUG_BOUNDS
__device__ __forceinline__ uint32_t flare_checked(uint32_t off, uint32_t bytes, uint32_t limit, int* status_word) {
    if (off + bytes > limit || off + bytes < off) { flare_report(status_word, FLARE_ERR_BOUNDS); return 0u; }
    return off;
}
#define FLARE_CK(off, bytes, limit, err) flare_checked((uint32_t)(off), (uint32_t)(bytes), (uint32_t)(limit), (err))
#else
#define FLARE_CK(off, bytes, limit, err) (off)
#endif
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
#endif
