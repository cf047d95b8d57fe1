/*
 * flare_oracle.c — CPU restatement of flare-core's attention / KV-cache path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA kernels are
 * compared against (and the timed CPU baseline).  Nothing in the product path
 * (flarellm_b200/) may link, load or call it.
 *
 * Every routine restates, in plain C, one routine of the Rust reference and
 * names it.  Paths are relative to the reference project root.  Build with
 *   gcc -O2 -ffp-contract=off -fno-fast-math
 * so that no multiply-add is contracted: the reference's scalar x86_64 code
 * performs a separate multiply and add for every accumulate.
 *
 * Pinning status.  The reference is Rust and there is no Rust toolchain on the
 * build machine, so the reference itself was never executed.  The restatement
 * is pinned against the reference's own known-answer tests, restated in
 * tests/test_oracle_*.py:
 *   - flare-core/src/model.rs:10369-10463  online-softmax vs 3-pass attention
 *   - flare-core/src/kv_cache.rs:552-940   ring buffer + KIVI 2-bit tests
 *   - flare-loader/src/quantize.rs:886-960, 1259-1353, 1694  f16 and Q8_0 blocks
 * Pieces with NO counterpart in the reference ("parity unpinned"; they are
 * compositions of pinned primitives): Q8_0 used as a KV cache, the group-32
 * KIVI mode, the sliding window, the batched multi-query verify, bf16 inputs,
 * batch > 1, the wrapped-ring clamp and the multi-GPU partial merge.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

#define ORC_API __attribute__((visibility("default")))


/* ------------------------------------------------------------------------ */
/* a minimal pthread parallel-for (the build machine has no OpenMP runtime)  */
/* ------------------------------------------------------------------------ */
typedef void (*orc_task_fn)(long index, void* arg);
typedef struct { orc_task_fn fn; void* arg; long total; long next; pthread_mutex_t mu; } orc_pool;
static void* orc_pool_worker(void* p_) {
    orc_pool* p = (orc_pool*)p_;
    for (;;) {
        pthread_mutex_lock(&p->mu);
        long i = p->next++;
        pthread_mutex_unlock(&p->mu);
        if (i >= p->total) return NULL;
        p->fn(i, p->arg);
    }
}
static void orc_parallel_for(long total, int threads, orc_task_fn fn, void* arg) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    if (threads == 1 || total <= 1) { for (long i = 0; i < total; i++) fn(i, arg); return; }
    orc_pool p; p.fn = fn; p.arg = arg; p.total = total; p.next = 0;
    pthread_mutex_init(&p.mu, NULL);
    pthread_t th[256];
    int started = 0;
    for (int t = 0; t < threads; t++) if (pthread_create(&th[started], NULL, orc_pool_worker, &p) == 0) started++;
    if (started == 0) orc_pool_worker(&p);
    for (int t = 0; t < started; t++) pthread_join(th[t], NULL);
    pthread_mutex_destroy(&p.mu);
}

/* ------------------------------------------------------------------------ */
/* scalar codecs                                                            */
/* ------------------------------------------------------------------------ */

static inline float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* flare-loader/src/quantize.rs:505-534 (f16_to_f32) and the identical
 * flare-core/src/model.rs:5302-5329 (f16_to_f32_inline): exact binary16 ->
 * binary32, subnormals renormalised by a shift loop, NaN payload = mant<<13. */
ORC_API uint32_t orc_f16_to_f32_bits(uint16_t bits) {
    uint32_t sign = (bits >> 15) & 1u;
    uint32_t exp = (bits >> 10) & 0x1Fu;
    uint32_t mant = bits & 0x3FFu;
    if (exp == 0) {
        if (mant == 0) return sign << 31;
        uint32_t e = 0, m = mant;
        while ((m & 0x400u) == 0) { m <<= 1; e -= 1; }   /* wrapping_sub */
        m &= 0x3FFu;
        uint32_t f32_exp = (113u + e) & 0xFFu;            /* 127-15+1 + e */
        return (sign << 31) | (f32_exp << 23) | (m << 13);
    }
    if (exp == 0x1F) return (sign << 31) | (0xFFu << 23) | (mant << 13);
    return (sign << 31) | ((exp + 112u) << 23) | (mant << 13);
}
ORC_API float orc_f16_to_f32(uint16_t bits) { return bits_to_f32(orc_f16_to_f32_bits(bits)); }

/* flare-loader/src/quantize.rs:540-542 (bf16_to_f32). */
ORC_API float orc_bf16_to_f32(uint16_t bits) { return bits_to_f32((uint32_t)bits << 16); }

/* binary32 -> binary16, round to nearest even.  The reference obtains this
 * from the third-party crate `half` 2.7.1 (Cargo.lock:765-766, source not in
 * the tree) at flare-gpu/src/kv_cache.rs:132-133 (`f16::from_f32`); IEEE-754
 * round-to-nearest-even is that crate's documented behaviour and is restated
 * here.  tests/test_oracle_codecs.py checks it against numpy's float16 cast on
 * every interesting binade. */
ORC_API uint16_t orc_f32_to_f16(float f) {
    uint32_t x = f32_to_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 0xFF) {                       /* inf / nan */
        if (man == 0) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | 0x7E00u | (man >> 13));
    }
    int32_t e = (int32_t)exp - 127 + 15;
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);       /* overflow */
    if (e <= 0) {                            /* subnormal or zero */
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);  /* 14..24 */
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;   /* may carry into exp: correct */
    return (uint16_t)(sign | half);
}

/* binary32 -> bfloat16 (RNE), used only to prepare the bf16 prefill inputs. */
ORC_API uint16_t orc_f32_to_bf16(float f) {
    uint32_t x = f32_to_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

ORC_API void orc_f32_to_f16_n(const float* x, size_t n, uint16_t* out) { for (size_t i = 0; i < n; i++) out[i] = orc_f32_to_f16(x[i]); }
ORC_API void orc_f16_to_f32_n(const uint16_t* x, size_t n, float* out) { for (size_t i = 0; i < n; i++) out[i] = orc_f16_to_f32(x[i]); }
ORC_API void orc_f32_to_bf16_n(const float* x, size_t n, uint16_t* out) { for (size_t i = 0; i < n; i++) out[i] = orc_f32_to_bf16(x[i]); }

/* ------------------------------------------------------------------------ */
/* Q8_0 blocks                                                              */
/* ------------------------------------------------------------------------ */

#define Q8_BLOCK 32
#define Q8_BYTES 34

/* flare-loader/src/quantize.rs:188-197 (dequant_q8_0_block): a block shorter
 * than 34 bytes leaves the output untouched. */
ORC_API void orc_dequant_q8_0_block(const uint8_t* block, size_t block_len, float* out32) {
    if (block_len < Q8_BYTES) return;
    float scale = orc_f16_to_f32((uint16_t)(block[0] | (block[1] << 8)));
    for (int i = 0; i < 32; i++) out32[i] = (float)(int8_t)block[2 + i] * scale;
}

static inline int8_t sat_i8(float r) {      /* Rust `as i8`: saturating, NaN -> 0 */
    if (r != r) return 0;
    if (r >= 127.0f) return 127;
    if (r <= -128.0f) return -128;
    return (int8_t)r;
}

/* flare-core/src/model.rs:5507-5527 (quantize_input_q8_0, the branch compiled
 * on x86_64): amax, d = amax/127, id = 127/amax, q = round(x*id) as i8.  The
 * reference keeps d as f32; a Q8_0 *block* stores it as f16, rounded the way
 * flare-gpu/src/kv_cache.rs:132 rounds (RNE).  n must be a multiple of 32. */
ORC_API void orc_quantize_q8_0(const float* x, size_t n, uint8_t* blocks) {
    for (size_t b = 0; b < n / Q8_BLOCK; b++) {
        const float* blk = x + b * Q8_BLOCK;
        float amax = 0.0f;
        for (int j = 0; j < Q8_BLOCK; j++) amax = fmaxf(amax, fabsf(blk[j]));
        float d = amax / 127.0f;
        float id = (d != 0.0f) ? 127.0f / amax : 0.0f;
        uint16_t h = orc_f32_to_f16(d);
        uint8_t* o = blocks + b * Q8_BYTES;
        o[0] = (uint8_t)(h & 0xFF);
        o[1] = (uint8_t)(h >> 8);
        for (int j = 0; j < Q8_BLOCK; j++) o[2 + j] = (uint8_t)sat_i8(roundf(blk[j] * id));
    }
}

ORC_API void orc_dequant_q8_0(const uint8_t* blocks, size_t n_values, float* out) {
    for (size_t b = 0; b < n_values / Q8_BLOCK; b++)
        orc_dequant_q8_0_block(blocks + b * Q8_BYTES, Q8_BYTES, out + b * Q8_BLOCK);
}
/* The same block by block, spread over host threads in chunks of 4096 blocks (for the timed
 * all-cores baseline only; the arithmetic per block is orc_dequant_q8_0_block). */
typedef struct { const uint8_t* blocks; float* out; size_t n_blocks; } orc_dq_args;
static void orc_dq_task(long c, void* a_) {
    orc_dq_args* a = (orc_dq_args*)a_;
    size_t b0 = (size_t)c * 4096, b1 = b0 + 4096 < a->n_blocks ? b0 + 4096 : a->n_blocks;
    for (size_t b = b0; b < b1; b++) orc_dequant_q8_0_block(a->blocks + b * Q8_BYTES, Q8_BYTES, a->out + b * Q8_BLOCK);
}
ORC_API void orc_dequant_q8_0_mt(const uint8_t* blocks, size_t n_values, float* out, int threads) {
    orc_dq_args a = {blocks, out, n_values / Q8_BLOCK};
    orc_parallel_for((long)((a.n_blocks + 4095) / 4096), threads, orc_dq_task, &a);
}

/* ------------------------------------------------------------------------ */
/* 2-bit pack / unpack                                                      */
/* ------------------------------------------------------------------------ */

#define Q2_MAX 3.0f
#define F32_EPS 1.1920929e-07f

static inline uint8_t sat_u8_code(float r) {   /* .round().clamp(0,3) as u8 */
    r = roundf(r);
    if (r != r) return 0;          /* clamp keeps NaN; `as u8` maps NaN to 0 */
    if (r < 0.0f) r = 0.0f;
    if (r > Q2_MAX) r = Q2_MAX;
    return (uint8_t)r;
}

/* flare-core/src/kv_cache.rs:332-371 (quantize_to_packed). */
ORC_API void orc_q2_quantize_to_packed(const float* values, size_t n, uint8_t* packed,
                                       float* scale_out, float* min_out) {
    float min_val = INFINITY, max_val = -INFINITY;
    for (size_t i = 0; i < n; i++) {
        if (values[i] < min_val) min_val = values[i];
        if (values[i] > max_val) max_val = values[i];
    }
    float range = max_val - min_val;
    float scale = (fabsf(range) < F32_EPS) ? 0.0f : range / Q2_MAX;
    float inv_scale = (fabsf(scale) < F32_EPS) ? 0.0f : Q2_MAX / range;
    size_t nbytes = (n + 3) / 4;
    memset(packed, 0, nbytes);
    for (size_t i = 0; i < n; i++) {
        uint8_t q = (fabsf(scale) < F32_EPS) ? 0 : sat_u8_code((values[i] - min_val) * inv_scale);
        packed[i / 4] |= (uint8_t)(q << ((i % 4) * 2));
    }
    *scale_out = scale;
    *min_out = min_val;
}

/* flare-core/src/kv_cache.rs:374-381 (dequant_from_packed_per_channel). */
ORC_API void orc_q2_dequant_per_channel(const uint8_t* packed, const float* mins,
                                        const float* scales, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float q = (float)((packed[i / 4] >> ((i % 4) * 2)) & 3);
        out[i] = q * scales[i] + mins[i];
    }
}

/* flare-core/src/kv_cache.rs:384-391 (dequant_from_packed_per_token). */
ORC_API void orc_q2_dequant_per_token(const uint8_t* packed, float scale, float min_val,
                                      float* out, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float q = (float)((packed[i / 4] >> ((i % 4) * 2)) & 3);
        out[i] = q * scale + min_val;
    }
}

/* flare-core/src/kv_cache.rs:399-420 (update_per_channel_stats). */
ORC_API void orc_q2_update_per_channel_stats(const float* values, float* mins, float* scales,
                                             size_t n, int first) {
    if (first) {
        for (size_t i = 0; i < n; i++) { mins[i] = values[i]; scales[i] = 0.0f; }
        return;
    }
    for (size_t i = 0; i < n; i++) {
        float v = values[i];
        float old_min = mins[i];
        float old_max = old_min + scales[i] * Q2_MAX;
        float new_min = fminf(old_min, v);
        float new_max = fmaxf(old_max, v);
        float range = new_max - new_min;
        mins[i] = new_min;
        scales[i] = (fabsf(range) < F32_EPS) ? 0.0f : range / Q2_MAX;
    }
}

/* ------------------------------------------------------------------------ */
/* attention                                                                */
/* ------------------------------------------------------------------------ */

/* flare-core/src/model.rs:9914-9966 (fused_attention_head_scalar): one query
 * head, slots visited in ascending order, single-pass online softmax. */
static void fused_attention_head_scalar(const float* q, size_t q_offset, const float* k_cache,
                                        const float* v_cache, float* output, size_t out_offset,
                                        size_t head_dim, size_t seq_len, size_t kv_stride,
                                        size_t kv_head, float scale) {
    for (size_t d = 0; d < head_dim; d++) output[out_offset + d] = 0.0f;
    float max_score = -INFINITY;
    float sum_exp = 0.0f;
    for (size_t t = 0; t < seq_len; t++) {
        size_t k_offset = t * kv_stride + kv_head * head_dim;
        float dot = 0.0f;
        for (size_t d = 0; d < head_dim; d++) dot += q[q_offset + d] * k_cache[k_offset + d];
        float score = dot * scale;
        float new_max = fmaxf(max_score, score);
        float old_scale = expf(max_score - new_max);
        float new_weight = expf(score - new_max);
        sum_exp = sum_exp * old_scale + new_weight;
        size_t v_offset = k_offset;
        for (size_t d = 0; d < head_dim; d++)
            output[out_offset + d] = output[out_offset + d] * old_scale + new_weight * v_cache[v_offset + d];
        max_score = new_max;
    }
    if (sum_exp > 0.0f) {
        float inv_sum = 1.0f / sum_exp;
        for (size_t d = 0; d < head_dim; d++) output[out_offset + d] *= inv_sum;
    }
}

/* flare-core/src/model.rs:10119-10212 (cpu_gqa_softcap), x86_64 branch. */
static void cpu_gqa_softcap(const float* q, const float* k_cache, const float* v_cache,
                            size_t num_heads, size_t num_kv_heads, size_t head_dim,
                            size_t seq_len, float attn_softcap, float* output) {
    size_t heads_per_kv = num_heads / num_kv_heads;
    size_t kv_stride = num_kv_heads * head_dim;
    float scale = 1.0f / sqrtf((float)head_dim);
    for (size_t i = 0; i < num_heads * head_dim; i++) output[i] = 0.0f;
    float* scores = (float*)calloc(seq_len ? seq_len : 1, sizeof(float));
    for (size_t h = 0; h < num_heads; h++) {
        size_t kv_head = h / heads_per_kv;
        size_t q_offset = h * head_dim;
        for (size_t t = 0; t < seq_len; t++) {
            size_t k_offset = t * kv_stride + kv_head * head_dim;
            float dot = 0.0f;
            for (size_t d = 0; d < head_dim; d++) dot += q[q_offset + d] * k_cache[k_offset + d];
            scores[t] = dot * scale;
        }
        for (size_t t = 0; t < seq_len; t++) scores[t] = tanhf(scores[t] / attn_softcap) * attn_softcap;
        float max_score = -INFINITY;
        for (size_t t = 0; t < seq_len; t++) max_score = fmaxf(max_score, scores[t]);
        float sum = 0.0f;
        for (size_t t = 0; t < seq_len; t++) { scores[t] = expf(scores[t] - max_score); sum += scores[t]; }
        float inv_sum = 1.0f / sum;
        for (size_t t = 0; t < seq_len; t++) scores[t] *= inv_sum;
        size_t out_offset = h * head_dim;
        for (size_t t = 0; t < seq_len; t++) {
            float weight = scores[t];
            if (weight < 1e-8f) continue;
            size_t v_offset = t * kv_stride + kv_head * head_dim;
            for (size_t d = 0; d < head_dim; d++) output[out_offset + d] += weight * v_cache[v_offset + d];
        }
        for (size_t t = 0; t < seq_len; t++) scores[t] = 0.0f;
    }
    free(scores);
}

/* flare-core/src/model.rs:9849-9905 (cpu_grouped_query_attention_into);
 * kv_head = h / (num_heads / num_kv_heads). */
ORC_API void orc_gqa_decode(const float* q, const float* k_cache, const float* v_cache,
                            size_t num_heads, size_t num_kv_heads, size_t head_dim,
                            size_t seq_len, float attn_softcap, float* output) {
    if (attn_softcap > 0.0f) {
        cpu_gqa_softcap(q, k_cache, v_cache, num_heads, num_kv_heads, head_dim, seq_len, attn_softcap, output);
        return;
    }
    size_t heads_per_kv = num_heads / num_kv_heads;
    size_t kv_stride = num_kv_heads * head_dim;
    float scale = 1.0f / sqrtf((float)head_dim);
    for (size_t h = 0; h < num_heads; h++) {
        size_t kv_head = h / heads_per_kv;
        fused_attention_head_scalar(q, h * head_dim, k_cache, v_cache, output, h * head_dim,
                                    head_dim, seq_len, kv_stride, kv_head, scale);
    }
}

/* The independent 3-pass formulation that the reference's own test compares
 * its online-softmax routine with: flare-core/src/model.rs:10371-10425
 * (reference_attention inside test_fused_attention_matches_reference). */
ORC_API void orc_gqa_decode_three_pass(const float* q, const float* k_cache, const float* v_cache,
                                       size_t num_heads, size_t num_kv_heads, size_t head_dim,
                                       size_t seq_len, float* output) {
    size_t heads_per_kv = num_heads / num_kv_heads;
    size_t kv_stride = num_kv_heads * head_dim;
    float scale = 1.0f / sqrtf((float)head_dim);
    for (size_t i = 0; i < num_heads * head_dim; i++) output[i] = 0.0f;
    float* scores = (float*)calloc(seq_len ? seq_len : 1, sizeof(float));
    for (size_t h = 0; h < num_heads; h++) {
        size_t kv_head = h / heads_per_kv;
        for (size_t t = 0; t < seq_len; t++) {
            size_t k_offset = t * kv_stride + kv_head * head_dim;
            float dot = 0.0f;
            for (size_t d = 0; d < head_dim; d++) dot += q[h * head_dim + d] * k_cache[k_offset + d];
            scores[t] = dot * scale;
        }
        float max_s = -INFINITY;
        for (size_t t = 0; t < seq_len; t++) max_s = fmaxf(max_s, scores[t]);
        float sum = 0.0f;
        for (size_t t = 0; t < seq_len; t++) { scores[t] = expf(scores[t] - max_s); sum += scores[t]; }
        float inv = 1.0f / sum;
        for (size_t t = 0; t < seq_len; t++) scores[t] *= inv;
        for (size_t t = 0; t < seq_len; t++) {
            float w = scores[t];
            size_t v_off = t * kv_stride + kv_head * head_dim;
            for (size_t d = 0; d < head_dim; d++) output[h * head_dim + d] += w * v_cache[v_off + d];
        }
    }
    free(scores);
}

/* Independent sequences and several causally ordered queries per sequence.
 * The reference has neither: its speculative verify runs one full forward per
 * draft token (flare-core/src/generate.rs:258-303), so query i of n_q sees
 * attend_len[b] - (n_q-1-i) slots; a batch is b independent calls.  K/V of
 * sequence b start at k + b*seq_stride (floats).  Threaded over (b, i) when
 * threads > 1; the per-head arithmetic is untouched. */
typedef struct {
    const float *q, *k, *v; const int* attend_len; float* out;
    size_t n_q, seq_stride, nh, nkv, hd; float softcap;
} orc_batched_args;
static void orc_batched_task(long u, void* a_) {
    orc_batched_args* a = (orc_batched_args*)a_;
    size_t qd = a->nh * a->hd;
    size_t b = (size_t)u / a->n_q, i = (size_t)u % a->n_q;
    size_t len = (size_t)a->attend_len[b] - (a->n_q - 1 - i);
    orc_gqa_decode(a->q + (b * a->n_q + i) * qd, a->k + b * a->seq_stride, a->v + b * a->seq_stride,
                   a->nh, a->nkv, a->hd, len, a->softcap, a->out + (b * a->n_q + i) * qd);
}
ORC_API void orc_gqa_decode_batched(const float* q, const float* k, const float* v, size_t batch,
                                    size_t n_q, size_t seq_stride, const int* attend_len,
                                    size_t num_heads, size_t num_kv_heads, size_t head_dim,
                                    float attn_softcap, float* out, int threads) {
    orc_batched_args a = {q, k, v, attend_len, out, n_q, seq_stride, num_heads, num_kv_heads, head_dim, attn_softcap};
    orc_parallel_for((long)(batch * n_q), threads, orc_batched_task, &a);
}

/* Same, but threaded over (b, head): used for the timed "all host threads"
 * baseline when batch*n_q is smaller than the core count.  softcap == 0 only. */
static void orc_heads_task(long u, void* a_) {
    orc_batched_args* a = (orc_batched_args*)a_;
    size_t qd = a->nh * a->hd;
    size_t b = (size_t)u / a->nh, h = (size_t)u % a->nh;
    fused_attention_head_scalar(a->q + b * qd, h * a->hd, a->k + b * a->seq_stride, a->v + b * a->seq_stride,
                                a->out + b * qd, h * a->hd, a->hd, (size_t)a->attend_len[b],
                                a->nkv * a->hd, h / (a->nh / a->nkv), 1.0f / sqrtf((float)a->hd));
}
ORC_API void orc_gqa_decode_heads_mt(const float* q, const float* k, const float* v, size_t batch,
                                     size_t seq_stride, const int* attend_len, size_t num_heads,
                                     size_t num_kv_heads, size_t head_dim, float* out, int threads) {
    orc_batched_args a = {q, k, v, attend_len, out, 1, seq_stride, num_heads, num_kv_heads, head_dim, 0.0f};
    orc_parallel_for((long)(batch * num_heads), threads, orc_heads_task, &a);
}

/* flare-core/src/model.rs:336-368 (default ComputeBackend::prefill_attention_gpu):
 * row t attends rows 0..=t.  `window` > 0 restricts row t to rows
 * max(0,t-window+1)..=t — the reference has no sliding window (only a doc
 * comment, flare-core/src/kv_cache.rs:430), so that variant is unpinned.
 * Only rows row_start, row_start+row_step, ... are computed (others untouched)
 * so that long prompts can be spot-checked.  Threaded over rows. */
typedef struct {
    const float *q, *k, *v; float* out;
    size_t nh, nkv, hd, window, row_start, row_step; float softcap;
} orc_prefill_args;
static void orc_prefill_task(long r, void* a_) {
    orc_prefill_args* a = (orc_prefill_args*)a_;
    size_t q_dim = a->nh * a->hd, kv_dim = a->nkv * a->hd;
    size_t t = a->row_start + (size_t)r * a->row_step;
    size_t lo = 0;
    if (a->window > 0 && t + 1 > a->window) lo = t + 1 - a->window;
    orc_gqa_decode(a->q + t * q_dim, a->k + lo * kv_dim, a->v + lo * kv_dim, a->nh, a->nkv, a->hd,
                   t + 1 - lo, a->softcap, a->out + t * q_dim);
}
ORC_API void orc_prefill(const float* q, const float* k, const float* v, size_t seq_len,
                         size_t num_heads, size_t num_kv_heads, size_t head_dim,
                         float attn_softcap, size_t window, size_t row_start, size_t row_step,
                         float* out, int threads) {
    if (row_step == 0) row_step = 1;
    long n_rows = seq_len > row_start ? (long)((seq_len - row_start + row_step - 1) / row_step) : 0;
    orc_prefill_args a = {q, k, v, out, num_heads, num_kv_heads, head_dim, window, row_start, row_step, attn_softcap};
    orc_parallel_for(n_rows, threads, orc_prefill_task, &a);
}

/* Partial attention over a slot range and the log-sum-exp merge of partials.
 * No counterpart in the reference (it has no multi-device path); the recurrence
 * is the block form of flare-core/src/model.rs:9945-9956.  partial layout per
 * head: [m, l, o[head_dim]] with o unnormalised. */
ORC_API void orc_gqa_decode_partial(const float* q, const float* k_cache, const float* v_cache,
                                    size_t num_heads, size_t num_kv_heads, size_t head_dim,
                                    size_t slot_begin, size_t slot_end, float* partial) {
    size_t heads_per_kv = num_heads / num_kv_heads;
    size_t kv_stride = num_kv_heads * head_dim;
    float scale = 1.0f / sqrtf((float)head_dim);
    for (size_t h = 0; h < num_heads; h++) {
        float* p = partial + h * (head_dim + 2);
        float* o = p + 2;
        size_t kv_head = h / heads_per_kv;
        float m = -INFINITY, l = 0.0f;
        for (size_t d = 0; d < head_dim; d++) o[d] = 0.0f;
        for (size_t t = slot_begin; t < slot_end; t++) {
            size_t off = t * kv_stride + kv_head * head_dim;
            float dot = 0.0f;
            for (size_t d = 0; d < head_dim; d++) dot += q[h * head_dim + d] * k_cache[off + d];
            float s = dot * scale;
            float nm = fmaxf(m, s);
            float a = expf(m - nm), w = expf(s - nm);
            l = l * a + w;
            for (size_t d = 0; d < head_dim; d++) o[d] = o[d] * a + w * v_cache[off + d];
            m = nm;
        }
        p[0] = m; p[1] = l;
    }
}

ORC_API void orc_merge_partials(const float* partials, size_t n_parts, size_t num_heads,
                                size_t head_dim, float* out) {
    size_t stride = num_heads * (head_dim + 2);
    for (size_t h = 0; h < num_heads; h++) {
        float m = -INFINITY;
        for (size_t r = 0; r < n_parts; r++) m = fmaxf(m, partials[r * stride + h * (head_dim + 2)]);
        float l = 0.0f;
        for (size_t d = 0; d < head_dim; d++) out[h * head_dim + d] = 0.0f;
        for (size_t r = 0; r < n_parts; r++) {
            const float* p = partials + r * stride + h * (head_dim + 2);
            if (p[1] == 0.0f) continue;
            float w = expf(p[0] - m);
            l += p[1] * w;
            for (size_t d = 0; d < head_dim; d++) out[h * head_dim + d] += p[2 + d] * w;
        }
        if (l > 0.0f) {
            float inv = 1.0f / l;
            for (size_t d = 0; d < head_dim; d++) out[h * head_dim + d] *= inv;
        }
    }
}

/* ------------------------------------------------------------------------ */
/* KvCache — flare-core/src/kv_cache.rs:431-546                             */
/* ------------------------------------------------------------------------ */

typedef struct {
    float* keys;      /* [num_layers][max_seq_len][kv_size] */
    float* values;
    size_t position, length, max_seq_len, num_layers, num_kv_heads, head_dim;
} orc_kv_cache;

ORC_API orc_kv_cache* orc_kv_new(size_t num_layers, size_t max_seq_len, size_t num_kv_heads, size_t head_dim) {
    orc_kv_cache* c = (orc_kv_cache*)calloc(1, sizeof(*c));
    size_t n = num_layers * max_seq_len * num_kv_heads * head_dim;
    c->keys = (float*)calloc(n ? n : 1, sizeof(float));
    c->values = (float*)calloc(n ? n : 1, sizeof(float));
    c->max_seq_len = max_seq_len; c->num_layers = num_layers;
    c->num_kv_heads = num_kv_heads; c->head_dim = head_dim;
    return c;
}
ORC_API void orc_kv_free(orc_kv_cache* c) { if (c) { free(c->keys); free(c->values); free(c); } }
/* kv_cache.rs:475-481 (write at the current position) */
ORC_API void orc_kv_write(orc_kv_cache* c, size_t layer, const float* key, const float* value) {
    size_t kv = c->num_kv_heads * c->head_dim;
    size_t off = (layer * c->max_seq_len + c->position) * kv;
    memcpy(c->keys + off, key, kv * sizeof(float));
    memcpy(c->values + off, value, kv * sizeof(float));
}
/* kv_cache.rs:484-489 */
ORC_API void orc_kv_advance(orc_kv_cache* c) {
    c->position = (c->position + 1) % c->max_seq_len;
    if (c->length < c->max_seq_len) c->length += 1;
}
ORC_API size_t orc_kv_len(const orc_kv_cache* c) { return c->length; }
ORC_API size_t orc_kv_position(const orc_kv_cache* c) { return c->position; }
ORC_API float* orc_kv_keys(orc_kv_cache* c, size_t layer) {
    return c->keys + layer * c->max_seq_len * c->num_kv_heads * c->head_dim;
}
ORC_API float* orc_kv_values(orc_kv_cache* c, size_t layer) {
    return c->values + layer * c->max_seq_len * c->num_kv_heads * c->head_dim;
}
/* kv_cache.rs:521-531: only a cache that has not wrapped can be rolled back */
ORC_API void orc_kv_truncate_to(orc_kv_cache* c, size_t target_len) {
    if (target_len >= c->length) return;
    if (c->length < c->max_seq_len) { c->position = target_len; c->length = target_len; }
}
/* kv_cache.rs:534-545 */
ORC_API void orc_kv_clear(orc_kv_cache* c) {
    size_t n = c->num_layers * c->max_seq_len * c->num_kv_heads * c->head_dim;
    c->position = 0; c->length = 0;
    memset(c->keys, 0, n * sizeof(float));
    memset(c->values, 0, n * sizeof(float));
}

/* The decode step's ordering contract, flare-core/src/model.rs:2186-2247 and
 * 2547: the caller has written the new token with orc_kv_write (slot =
 * position); seq_len = len + 1; attend; advance happens after all layers.
 * Once the ring is full the reference's seq_len would be max_seq_len + 1 and
 * its scalar loop would index past the buffer (model.rs:9937); this engine
 * defines that case as min(len + 1, max_seq_len) physical slots. */
ORC_API size_t orc_kv_attend_len(const orc_kv_cache* c) {
    size_t n = c->length + 1;
    return n < c->max_seq_len ? n : c->max_seq_len;
}

/* ------------------------------------------------------------------------ */
/* QuantizedKvCache — flare-core/src/kv_cache.rs:35-323 (reference-exact)    */
/* ------------------------------------------------------------------------ */

#define RESIDUAL_WINDOW 32

typedef struct {
    uint8_t *key_packed, *value_packed;             /* [L][max_seq][packed_per_token] */
    float *key_scales, *key_mins;                   /* [L][kv_size] */
    float *value_scales, *value_mins;               /* [L][max_seq] */
    float *residual_keys, *residual_values;         /* [L][residual_len][kv_size] */
    size_t position, length, max_seq_len, num_layers, num_kv_heads, head_dim, residual_len;
} orc_qkv_cache;

ORC_API orc_qkv_cache* orc_qkv_new(size_t num_layers, size_t max_seq_len, size_t num_kv_heads, size_t head_dim) {
    orc_qkv_cache* c = (orc_qkv_cache*)calloc(1, sizeof(*c));
    size_t kv = num_kv_heads * head_dim, ppt = (kv + 3) / 4;
    c->residual_len = RESIDUAL_WINDOW < max_seq_len ? RESIDUAL_WINDOW : max_seq_len;
    c->key_packed = (uint8_t*)calloc(num_layers * max_seq_len * ppt + 1, 1);
    c->value_packed = (uint8_t*)calloc(num_layers * max_seq_len * ppt + 1, 1);
    c->key_scales = (float*)calloc(num_layers * kv + 1, 4);
    c->key_mins = (float*)calloc(num_layers * kv + 1, 4);
    c->value_scales = (float*)calloc(num_layers * max_seq_len + 1, 4);
    c->value_mins = (float*)calloc(num_layers * max_seq_len + 1, 4);
    c->residual_keys = (float*)calloc(num_layers * c->residual_len * kv + 1, 4);
    c->residual_values = (float*)calloc(num_layers * c->residual_len * kv + 1, 4);
    c->max_seq_len = max_seq_len; c->num_layers = num_layers;
    c->num_kv_heads = num_kv_heads; c->head_dim = head_dim;
    return c;
}
ORC_API void orc_qkv_free(orc_qkv_cache* c) {
    if (!c) return;
    free(c->key_packed); free(c->value_packed); free(c->key_scales); free(c->key_mins);
    free(c->value_scales); free(c->value_mins); free(c->residual_keys); free(c->residual_values);
    free(c);
}
/* kv_cache.rs:121-162 */
ORC_API void orc_qkv_write(orc_qkv_cache* c, size_t layer, const float* key, const float* value) {
    size_t kv = c->num_kv_heads * c->head_dim, ppt = (kv + 3) / 4;
    size_t pos = c->position;
    size_t poff = (layer * c->max_seq_len + pos) * ppt;
    float s, m;
    orc_q2_quantize_to_packed(key, kv, c->key_packed + poff, &s, &m);   /* (scale,min) discarded */
    orc_q2_update_per_channel_stats(key, c->key_mins + layer * kv, c->key_scales + layer * kv, kv,
                                    c->length == 0);
    orc_q2_quantize_to_packed(value, kv, c->value_packed + poff, &s, &m);
    c->value_scales[layer * c->max_seq_len + pos] = s;
    c->value_mins[layer * c->max_seq_len + pos] = m;
    size_t res_off = (layer * c->residual_len + pos % c->residual_len) * kv;
    memcpy(c->residual_keys + res_off, key, kv * 4);
    memcpy(c->residual_values + res_off, value, kv * 4);
}
ORC_API void orc_qkv_advance(orc_qkv_cache* c) {
    c->position = (c->position + 1) % c->max_seq_len;
    if (c->length < c->max_seq_len) c->length += 1;
}
ORC_API size_t orc_qkv_len(const orc_qkv_cache* c) { return c->length; }
ORC_API size_t orc_qkv_position(const orc_qkv_cache* c) { return c->position; }
/* kv_cache.rs:306-312 */
static size_t qkv_ring_pos(const orc_qkv_cache* c, size_t t) {
    return c->length < c->max_seq_len ? t : (c->position + t) % c->max_seq_len;
}
/* kv_cache.rs:315-322 */
static int qkv_is_in_residual(const orc_qkv_cache* c, size_t t) {
    size_t n = c->length;
    if (n <= c->residual_len) return 1;
    return t >= n - c->residual_len;
}
/* kv_cache.rs:189-250 (dequant_keys / dequant_values): out is
 * [max_seq_len][kv_size] indexed by ring slot, zero where nothing is valid. */
ORC_API void orc_qkv_dequant(const orc_qkv_cache* c, size_t layer, int want_values, float* out) {
    size_t kv = c->num_kv_heads * c->head_dim, ppt = (kv + 3) / 4;
    memset(out, 0, c->max_seq_len * kv * 4);
    const float* residual = want_values ? c->residual_values : c->residual_keys;
    const uint8_t* packed = want_values ? c->value_packed : c->key_packed;
    for (size_t t = 0; t < c->length; t++) {
        size_t rp = qkv_ring_pos(c, t);
        float* dst = out + rp * kv;
        if (qkv_is_in_residual(c, t)) {
            memcpy(dst, residual + (layer * c->residual_len + rp % c->residual_len) * kv, kv * 4);
        } else {
            const uint8_t* p = packed + (layer * c->max_seq_len + rp) * ppt;
            if (want_values)
                orc_q2_dequant_per_token(p, c->value_scales[layer * c->max_seq_len + rp],
                                         c->value_mins[layer * c->max_seq_len + rp], dst, kv);
            else
                orc_q2_dequant_per_channel(p, c->key_mins + layer * kv, c->key_scales + layer * kv, dst, kv);
        }
    }
}
/* kv_cache.rs:258-268 */
ORC_API void orc_qkv_truncate_to(orc_qkv_cache* c, size_t target_len) {
    if (target_len >= c->length) return;
    if (c->length < c->max_seq_len) { c->position = target_len; c->length = target_len; }
}
/* kv_cache.rs:270-300 */
ORC_API void orc_qkv_clear(orc_qkv_cache* c) {
    size_t kv = c->num_kv_heads * c->head_dim, ppt = (kv + 3) / 4, L = c->num_layers;
    c->position = 0; c->length = 0;
    memset(c->key_packed, 0, L * c->max_seq_len * ppt);
    memset(c->value_packed, 0, L * c->max_seq_len * ppt);
    memset(c->key_scales, 0, L * kv * 4); memset(c->key_mins, 0, L * kv * 4);
    memset(c->value_scales, 0, L * c->max_seq_len * 4); memset(c->value_mins, 0, L * c->max_seq_len * 4);
    memset(c->residual_keys, 0, L * c->residual_len * kv * 4);
    memset(c->residual_values, 0, L * c->residual_len * kv * 4);
}
/* raw plane access so that the device cache can be compared byte for byte */
ORC_API const uint8_t* orc_qkv_key_packed(const orc_qkv_cache* c, size_t layer) {
    return c->key_packed + layer * c->max_seq_len * ((c->num_kv_heads * c->head_dim + 3) / 4);
}
ORC_API const uint8_t* orc_qkv_value_packed(const orc_qkv_cache* c, size_t layer) {
    return c->value_packed + layer * c->max_seq_len * ((c->num_kv_heads * c->head_dim + 3) / 4);
}
ORC_API const float* orc_qkv_key_scales(const orc_qkv_cache* c, size_t l) { return c->key_scales + l * c->num_kv_heads * c->head_dim; }
ORC_API const float* orc_qkv_key_mins(const orc_qkv_cache* c, size_t l) { return c->key_mins + l * c->num_kv_heads * c->head_dim; }
ORC_API const float* orc_qkv_value_scales(const orc_qkv_cache* c, size_t l) { return c->value_scales + l * c->max_seq_len; }
ORC_API const float* orc_qkv_value_mins(const orc_qkv_cache* c, size_t l) { return c->value_mins + l * c->max_seq_len; }
ORC_API const float* orc_qkv_residual_keys(const orc_qkv_cache* c, size_t l) { return c->residual_keys + l * c->residual_len * c->num_kv_heads * c->head_dim; }
ORC_API const float* orc_qkv_residual_values(const orc_qkv_cache* c, size_t l) { return c->residual_values + l * c->residual_len * c->num_kv_heads * c->head_dim; }

/* ------------------------------------------------------------------------ */
/* KIVI group-32 mode (no counterpart in the reference; unpinned)            */
/* ------------------------------------------------------------------------ */
/* The 2-bit quantiser and dequantiser above (kv_cache.rs:332-391) applied to
 * groups of 32: a key group is 32 consecutive ring slots of one channel, a
 * value group is 32 consecutive channels of one slot.  Codes are computed from
 * the f32 group statistics exactly as quantize_to_packed does; the stored scale
 * and zero (= group minimum) are then rounded to f16 (RNE) and dequantisation
 * is  code * f16_to_f32(scale) + f16_to_f32(zero)  as a separate multiply and
 * add.  Inputs are first rounded to f16, because a token is quantised only
 * when it leaves the 128-token f16 residual ring.
 *
 * Planes for one layer of one sequence (max_seq_len a multiple of 32):
 *   k_codes [max_seq][kv_dim/4]          byte j of a slot holds channels 4j..4j+3 (as v_codes);
 *                                        the 32 slots of a group share one (scale, zero) per channel
 *   k_meta  [max_seq/32][kv_dim][2] u16  (scale, zero) as f16 bits
 *   v_codes [max_seq][kv_dim/4]          byte j of a slot holds channels 4j..4j+3
 *   v_meta  [max_seq][kv_dim/32][2] u16
 *   res_k, res_v [128][kv_dim] u16       f16 bits, ring slot = position % 128
 */
#define G32 32
#define G32_RESIDUAL 128

static void g32_quant_group(const float* vals, uint8_t* codes8, uint16_t* meta2) {
    float s, m;
    orc_q2_quantize_to_packed(vals, G32, codes8, &s, &m);
    meta2[0] = orc_f32_to_f16(s);
    meta2[1] = orc_f32_to_f16(m);
}

/* Index (in f16 units) of channel c's scale inside a group's key metadata row: per block of 16
 * channels 16 scales then 16 zero points, channel r of the block at position 2 (r mod 8) + r div 8
 * (so the pair (r, r+8), whose codes sit 16 bits apart in a code word, is adjacent).  The zero
 * point is 16 entries further. */
static size_t g32_kmeta_index(size_t c) { return (c >> 4) * 32 + 2 * (c & 7) + ((c >> 3) & 1); }

/* Quantise key group `group` (ring slots 32*group .. +31) from f16-rounded rows
 * rows_f16[32][kv_dim] (as f32 values). */
ORC_API void orc_g32_quant_key_group(const float* rows, size_t kv_dim, uint8_t* k_codes_group,
                                     uint16_t* k_meta_group) {
    /* k_codes_group: the 32 slot rows of the group, [32][kv_dim/4] */
    float col[G32];
    uint8_t codes8[8];
    memset(k_codes_group, 0, G32 * kv_dim / 4);
    for (size_t c = 0; c < kv_dim; c++) {
        for (int t = 0; t < G32; t++) col[t] = rows[(size_t)t * kv_dim + c];
        uint16_t meta[2];
        g32_quant_group(col, codes8, meta);                          /* codes8: slot t at byte t/4, bits (t%4)*2 */
        k_meta_group[g32_kmeta_index(c)] = meta[0];
        k_meta_group[g32_kmeta_index(c) + 16] = meta[1];
        for (int t = 0; t < G32; t++) {
            uint8_t q = (uint8_t)((codes8[t / 4] >> ((t % 4) * 2)) & 3);
            k_codes_group[(size_t)t * (kv_dim / 4) + c / 4] |= (uint8_t)(q << ((c % 4) * 2));
        }
    }
}
/* Quantise one value row. */
ORC_API void orc_g32_quant_value_row(const float* row, size_t kv_dim, uint8_t* v_codes_row,
                                     uint16_t* v_meta_row) {
    for (size_t g = 0; g < kv_dim / G32; g++)
        g32_quant_group(row + g * G32, v_codes_row + g * 8, v_meta_row + g * 2);
}
ORC_API void orc_g32_dequant_key_group(const uint8_t* k_codes_group, const uint16_t* k_meta_group,
                                       size_t kv_dim, float* rows_out) {
    for (size_t c = 0; c < kv_dim; c++) {
        float s = orc_f16_to_f32(k_meta_group[g32_kmeta_index(c)]), z = orc_f16_to_f32(k_meta_group[g32_kmeta_index(c) + 16]);
        for (int t = 0; t < G32; t++) {
            float q = (float)((k_codes_group[(size_t)t * (kv_dim / 4) + c / 4] >> ((c % 4) * 2)) & 3);
            rows_out[(size_t)t * kv_dim + c] = q * s + z;
        }
    }
}
ORC_API void orc_g32_dequant_value_row(const uint8_t* v_codes_row, const uint16_t* v_meta_row,
                                       size_t kv_dim, float* row_out) {
    for (size_t g = 0; g < kv_dim / G32; g++)
        orc_q2_dequant_per_token(v_codes_row + g * 8, orc_f16_to_f32(v_meta_row[g * 2]),
                                 orc_f16_to_f32(v_meta_row[g * 2 + 1]), row_out + g * G32, G32);
}

typedef struct {
    uint8_t *k_codes, *v_codes;
    uint16_t *k_meta, *v_meta, *res_k, *res_v;
    size_t position, length, written;   /* written = absolute index of the next token */
    size_t max_seq_len, kv_dim;
} orc_g32_cache;   /* one layer, one sequence */

ORC_API orc_g32_cache* orc_g32_new(size_t max_seq_len, size_t kv_dim) {
    orc_g32_cache* c = (orc_g32_cache*)calloc(1, sizeof(*c));
    c->max_seq_len = max_seq_len; c->kv_dim = kv_dim;
    c->k_codes = (uint8_t*)calloc(max_seq_len * kv_dim / 4 + 1, 1);
    c->k_meta = (uint16_t*)calloc(max_seq_len / G32 * kv_dim * 2 + 1, 2);
    c->v_codes = (uint8_t*)calloc(max_seq_len * kv_dim / 4 + 1, 1);
    c->v_meta = (uint16_t*)calloc(max_seq_len * kv_dim / G32 * 2 + 1, 2);
    c->res_k = (uint16_t*)calloc(G32_RESIDUAL * kv_dim + 1, 2);
    c->res_v = (uint16_t*)calloc(G32_RESIDUAL * kv_dim + 1, 2);
    return c;
}
ORC_API void orc_g32_free(orc_g32_cache* c) {
    if (!c) return;
    free(c->k_codes); free(c->v_codes); free(c->k_meta); free(c->v_meta); free(c->res_k); free(c->res_v);
    free(c);
}
/* Write the token with absolute index p = c->written.  Before its residual
 * slot (p % 128) is overwritten, and whenever p is a multiple of 32 with
 * p >= 128, tokens p-128 .. p-97 (one whole key group, still in the ring) are
 * quantised into ring slots (p-128) % max_seq_len ..  Then advance. */
ORC_API void orc_g32_write_advance(orc_g32_cache* c, const float* key, const float* value) {
    size_t kv = c->kv_dim, p = c->written;
    if (p >= G32_RESIDUAL && p % G32 == 0) {
        float* rows = (float*)malloc(G32 * kv * 4);
        size_t first = p - G32_RESIDUAL;
        size_t group = (first % c->max_seq_len) / G32;
        for (int t = 0; t < G32; t++)
            for (size_t i = 0; i < kv; i++)
                rows[(size_t)t * kv + i] = orc_f16_to_f32(c->res_k[((first + t) % G32_RESIDUAL) * kv + i]);
        orc_g32_quant_key_group(rows, kv, c->k_codes + group * G32 * kv / 4, c->k_meta + group * kv * 2);
        for (int t = 0; t < G32; t++) {
            size_t slot = (first + t) % c->max_seq_len;
            for (size_t i = 0; i < kv; i++)
                rows[i] = orc_f16_to_f32(c->res_v[((first + t) % G32_RESIDUAL) * kv + i]);
            orc_g32_quant_value_row(rows, kv, c->v_codes + slot * kv / 4, c->v_meta + slot * kv / G32 * 2);
        }
        free(rows);
    }
    size_t rs = p % G32_RESIDUAL;
    for (size_t i = 0; i < kv; i++) {
        c->res_k[rs * kv + i] = orc_f32_to_f16(key[i]);
        c->res_v[rs * kv + i] = orc_f32_to_f16(value[i]);
    }
    c->written = p + 1;
    c->position = c->written % c->max_seq_len;
    if (c->length < c->max_seq_len) c->length += 1;
}
/* Dequantised view used for attention: for every one of the n_attend =
 * min(written, max_seq_len) live tokens, ring slot -> f32 row; a token among
 * the newest 128 comes from the f16 residual ring, any older one from codes.
 * out_k/out_v are [max_seq_len][kv_dim]; dead slots are zero. */
ORC_API void orc_g32_dequant(const orc_g32_cache* c, float* out_k, float* out_v) {
    size_t kv = c->kv_dim, n = c->written < c->max_seq_len ? c->written : c->max_seq_len;
    memset(out_k, 0, c->max_seq_len * kv * 4);
    memset(out_v, 0, c->max_seq_len * kv * 4);
    float* rows = (float*)malloc(G32 * kv * 4);
    for (size_t g = 0; g < c->max_seq_len / G32; g++) {
        orc_g32_dequant_key_group(c->k_codes + g * G32 * kv / 4, c->k_meta + g * kv * 2, kv, rows);
        for (int t = 0; t < G32; t++) memcpy(out_k + (g * G32 + t) * kv, rows + (size_t)t * kv, kv * 4);
    }
    free(rows);
    for (size_t s = 0; s < c->max_seq_len; s++)
        orc_g32_dequant_value_row(c->v_codes + s * kv / 4, c->v_meta + s * kv / G32 * 2, kv, out_v + s * kv);
    /* overlay residual tokens, blank dead slots */
    for (size_t s = 0; s < c->max_seq_len; s++) {
        /* newest token with ring slot s */
        if (c->written == 0) { memset(out_k + s * kv, 0, kv * 4); memset(out_v + s * kv, 0, kv * 4); continue; }
        size_t last = c->written - 1;
        size_t back = (last % c->max_seq_len + c->max_seq_len - s) % c->max_seq_len;  /* age of slot s */
        if (back >= n) { memset(out_k + s * kv, 0, kv * 4); memset(out_v + s * kv, 0, kv * 4); continue; }
        if (back < G32_RESIDUAL) {
            size_t tok = last - back;
            for (size_t i = 0; i < kv; i++) {
                out_k[s * kv + i] = orc_f16_to_f32(c->res_k[(tok % G32_RESIDUAL) * kv + i]);
                out_v[s * kv + i] = orc_f16_to_f32(c->res_v[(tok % G32_RESIDUAL) * kv + i]);
            }
        }
    }
}
ORC_API const uint8_t* orc_g32_k_codes(const orc_g32_cache* c) { return c->k_codes; }
ORC_API const uint8_t* orc_g32_v_codes(const orc_g32_cache* c) { return c->v_codes; }
ORC_API const uint16_t* orc_g32_k_meta(const orc_g32_cache* c) { return c->k_meta; }
ORC_API const uint16_t* orc_g32_v_meta(const orc_g32_cache* c) { return c->v_meta; }
ORC_API const uint16_t* orc_g32_res_k(const orc_g32_cache* c) { return c->res_k; }
ORC_API const uint16_t* orc_g32_res_v(const orc_g32_cache* c) { return c->res_v; }
ORC_API size_t orc_g32_written(const orc_g32_cache* c) { return c->written; }

/* ------------------------------------------------------------------------ */
/* rotary position embedding (the step before the KV write)                 */
/* ------------------------------------------------------------------------ */

/* flare-core/src/model.rs:7171 (ROPE_TABLE_MAX_SEQ_LEN) and 7190-7213 (RopeTable::new):
 * cos/sin of pos * freq for every (pos, d), d < head_dim / 2, flattened [positions][head_dim / 2];
 * freq = 1 / theta^(2 d / head_dim), everything in f32.  The number of positions is capped at
 * `cap` (the reference's constant is 8192; a caller that wants exact rows for later positions
 * passes a larger cap — the expression per entry is the one the inline fallback evaluates).
 * Returns the number of positions written. */
ORC_API size_t orc_rope_table(size_t head_dim, size_t max_seq_len, float rope_theta, size_t cap,
                              float* cos_out, float* sin_out) {
    size_t capped = max_seq_len < cap ? max_seq_len : cap;
    size_t half = head_dim / 2;
    for (size_t pos = 0; pos < capped; pos++) {
        for (size_t d = 0; d < half; d++) {
            float freq = 1.0f / powf(rope_theta, 2.0f * (float)d / (float)head_dim);
            float angle = (float)pos * freq;
            cos_out[pos * half + d] = cosf(angle);
            sin_out[pos * half + d] = sinf(angle);
        }
    }
    return capped;
}

/* model.rs:7280-7289 (the branch compiled on x86_64): half-split pairs (i, i + half) of every head,
 * two multiplies and a subtract / an add per element, no fused multiply-add. */
static void rope_rotate(float* data, size_t num_heads, size_t head_dim, const float* cos_row, const float* sin_row) {
    size_t half = head_dim / 2;
    for (size_t h = 0; h < num_heads; h++) {
        size_t offset = h * head_dim;
        for (size_t i = 0; i < half; i++) {
            float c = cos_row[i], s = sin_row[i];
            float x0 = data[offset + i], x1 = data[offset + i + half];
            data[offset + i] = x0 * c - x1 * s;
            data[offset + i + half] = x0 * s + x1 * c;
        }
    }
}

/* model.rs:7299-7332 (apply_rope): cos/sin computed inline for one position. */
ORC_API void orc_apply_rope(float* data, size_t num_heads, size_t head_dim, size_t pos, float theta) {
    size_t half = head_dim / 2;
    float* cs = (float*)malloc(2 * half * sizeof(float) + 8);
    for (size_t i = 0; i < half; i++) {
        float freq = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
        float angle = (float)pos * freq;
        cs[half + i] = sinf(angle);
        cs[i] = cosf(angle);
    }
    rope_rotate(data, num_heads, head_dim, cs, cs + half);
    free(cs);
}

/* model.rs:7256-7292 (apply_rope_with_table): table rows for positions inside the table and a
 * matching head size, the inline computation otherwise. */
ORC_API void orc_apply_rope_with_table(float* data, size_t num_heads, size_t head_dim, size_t pos, float theta,
                                       const float* cos_tab, const float* sin_tab, size_t table_len,
                                       size_t table_head_dim) {
    if (pos >= table_len || head_dim != table_head_dim) { orc_apply_rope(data, num_heads, head_dim, pos, theta); return; }
    size_t half = head_dim / 2;
    rope_rotate(data, num_heads, head_dim, cos_tab + pos * half, sin_tab + pos * half);
}


/* ------------------------------------------------------------------------ */
/* Q8_0-weight matrix-vector product (the projections either side of attention) */
/* ------------------------------------------------------------------------ */

/* flare-core/src/model.rs:5507-5527 (quantize_input_q8_0, the branch compiled on x86_64): per
 * block of 32: amax, d = amax / 127, id = 127 / amax (0 when d == 0), q = round(x * id) as i8;
 * the scale stays f32.  n must be a multiple of 32. */
ORC_API void orc_quantize_input_q8_0(const float* input, size_t n, float* scales, int8_t* quants) {
    for (size_t b = 0; b < n / Q8_BLOCK; b++) {
        const float* blk = input + b * Q8_BLOCK;
        float amax = 0.0f;
        for (int j = 0; j < Q8_BLOCK; j++) amax = fmaxf(amax, fabsf(blk[j]));
        float d = amax / 127.0f;
        float id = (d != 0.0f) ? 127.0f / amax : 0.0f;
        scales[b] = d;
        for (int j = 0; j < Q8_BLOCK; j++) quants[b * Q8_BLOCK + j] = sat_i8(roundf(blk[j] * id));
    }
}

/* flare-core/src/model.rs:8066-8100 (matvec_q8_0_preq_into, the scalar branch): per row, blocks in
 * ascending order, sum += (w_scale * x_scale[block]) * (s0 + s1 + s2 + s3) as f32 with four
 * interleaved int32 partial sums. */
ORC_API void orc_matvec_q8_0_preq(const uint8_t* weight_data, const float* in_scales, const int8_t* in_quants,
                                  size_t rows, size_t blocks_per_row, float* output) {
    size_t bytes_per_row = blocks_per_row * Q8_BYTES;
    for (size_t i = 0; i < rows; i++) {
        const uint8_t* row_bytes = weight_data + i * bytes_per_row;
        float sum = 0.0f;
        for (size_t block = 0; block < blocks_per_row; block++) {
            size_t block_start = block * Q8_BYTES;
            float w_scale = orc_f16_to_f32((uint16_t)(row_bytes[block_start] | (row_bytes[block_start + 1] << 8)));
            const uint8_t* w_quants = row_bytes + block_start + 2;
            size_t input_offset = block * Q8_BLOCK;
            float combined_scale = w_scale * in_scales[block];
            int32_t s0 = 0, s1 = 0, s2 = 0, s3 = 0;
            for (int j = 0; j < 32; j += 4) {
                s0 += (int32_t)(int8_t)w_quants[j] * (int32_t)in_quants[input_offset + j];
                s1 += (int32_t)(int8_t)w_quants[j + 1] * (int32_t)in_quants[input_offset + j + 1];
                s2 += (int32_t)(int8_t)w_quants[j + 2] * (int32_t)in_quants[input_offset + j + 2];
                s3 += (int32_t)(int8_t)w_quants[j + 3] * (int32_t)in_quants[input_offset + j + 3];
            }
            sum += combined_scale * (float)(s0 + s1 + s2 + s3);
        }
        output[i] = sum;
    }
}


/* flare-core/src/model.rs:5610-5641 (rmsnorm_quantize_q8_0_scalar): rms over the vector (squares added left to
 * right in f32), then per block of 32: n = x * weight * inv_rms, amax, scale = amax / 127,
 * inv_scale = 127 / amax (0 when scale == 0), q = round(n * inv_scale) as i8. */
ORC_API void orc_rmsnorm_quantize_q8_0(const float* x, const float* weight, float eps, size_t dim, float* scales,
                                       int8_t* quants) {
    float sum_sq = 0.0f;
    for (size_t i = 0; i < dim; i++) sum_sq += x[i] * x[i];
    float rms = sqrtf(sum_sq / (float)dim + eps);
    float inv_rms = 1.0f / rms;
    for (size_t b = 0; b < dim / Q8_BLOCK; b++) {
        float normed[Q8_BLOCK];
        float amax = 0.0f;
        for (int j = 0; j < Q8_BLOCK; j++) {
            float n = x[b * Q8_BLOCK + j] * weight[b * Q8_BLOCK + j] * inv_rms;
            normed[j] = n;
            amax = fmaxf(amax, fabsf(n));
        }
        float scale = amax / 127.0f;
        scales[b] = scale;
        float inv_scale = (scale != 0.0f) ? 127.0f / amax : 0.0f;
        for (int j = 0; j < Q8_BLOCK; j++) quants[b * Q8_BLOCK + j] = sat_i8(roundf(normed[j] * inv_scale));
    }
}

/* flare-core/src/model.rs:7469-7478 (rmsnorm_scalar_into): out = (x * inv_rms) * weight. */
ORC_API void orc_rmsnorm_into(const float* x, const float* weight, float eps, size_t dim, float* out) {
    float sum_sq = 0.0f;
    for (size_t i = 0; i < dim; i++) sum_sq += x[i] * x[i];
    float rms = sqrtf(sum_sq / (float)dim + eps);
    float inv_rms = 1.0f / rms;
    for (size_t i = 0; i < dim; i++) out[i] = (x[i] * inv_rms) * weight[i];
}

/* flare-core/src/model.rs:7091-7099 (silu_mul_scalar): (g / (1 + exp(-g))) * up. */
ORC_API void orc_silu_mul(const float* gate, const float* up, size_t n, float* out) {
    for (size_t i = 0; i < n; i++) {
        float g = gate[i];
        out[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

/* The f32 product of the output matrix (matvec, flare-core/src/model.rs:4968-5016, dispatches by platform: AVX2,
 * NEON, Accelerate or matvec_scalar); restated as the plain left-to-right sum of a row.  The platform kernels add
 * in other orders, so this one is compared within a tolerance on either side. */
ORC_API void orc_matvec_f32(const float* mat, const float* vec, size_t rows, size_t cols, float* out) {
    for (size_t r = 0; r < rows; r++) {
        float s = 0.0f;
        for (size_t c = 0; c < cols; c++) s += mat[r * cols + c] * vec[c];
        out[r] = s;
    }
}

ORC_API int orc_max_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}
