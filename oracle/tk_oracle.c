/*
 * tk_oracle.c — CPU oracle for the paged KV-cache hot path (see tk_oracle.h).
 *
 * TEST INFRASTRUCTURE ONLY: the checker and the reported CPU baseline, never
 * part of the shipped library.  Build with -ffp-contract=off and without
 * -ffast-math so that every FP32 operation rounds once, as written.
 */
#include "tk_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ======================================================================== */
/* scalar conversions                                                        */
/* ======================================================================== */

/* E4M3 -> float.  Restates f8e4m3_to_float, src/compute/cuda/fp4.cu:173-185:
 * codes 0x7F/0xFF (NaN) decode to 0, bias 7, subnormals exact. */
float tko_e4m3_decode(uint8_t v) {
    if ((v & 0x7F) == 0x7F) return 0.0f;
    int sign = (v >> 7) & 1;
    int exp = (v >> 3) & 0xF;
    int mant = v & 0x7;
    float mag;
    if (exp == 0) mag = ldexpf((float)mant * (1.0f / 8.0f), 1 - 7);
    else          mag = ldexpf(1.0f + (float)mant * (1.0f / 8.0f), exp - 7);
    return sign ? -mag : mag;
}

/* float -> E4M3, round-to-nearest-even, saturate to +-448 (0x7E), NaN -> 0x7F.
 * The reference has no E4M3 encoder; this is the published OCP FP8 E4M3
 * rounding, the behaviour of the GPU's cvt.rn.satfinite.e4m3x2.f32. */
uint8_t tko_e4m3_encode(float x) {
    if (x != x) return 0x7F;
    uint8_t sign = signbit(x) ? 0x80 : 0x00;
    float a = fabsf(x);
    if (a >= 448.0f) return sign | 0x7E;
    if (a < 0.015625f) {                       /* below 2^-6: subnormal grid, step 2^-9 */
        int q = (int)nearbyintf(a * 512.0f);   /* exact scaling, ties to even; q==8 is the first normal */
        return sign | (uint8_t)q;
    }
    int e;
    float f = frexpf(a, &e);                   /* a = f * 2^e, f in [0.5,1) */
    float mant = f * 2.0f; e -= 1;             /* mant in [1,2) */
    int q = (int)nearbyintf((mant - 1.0f) * 8.0f);
    if (q == 8) { q = 0; e += 1; }
    int code = ((e + 7) << 3) | q;
    if (code > 0x7E) code = 0x7E;
    return sign | (uint8_t)code;
}

uint16_t tko_f32_to_bf16(float x) {
    uint32_t u; memcpy(&u, &x, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    u += 0x7FFFu + ((u >> 16) & 1u);           /* round to nearest even */
    return (uint16_t)(u >> 16);
}
float tko_bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f;
}
uint16_t tko_f32_to_f16(float x) {
    _Float16 h = (_Float16)x; uint16_t u; memcpy(&u, &h, 2); return u;
}
float tko_f16_to_f32(uint16_t u) {
    _Float16 h; memcpy(&h, &u, 2); return (float)h;
}
static inline float to_f32(uint16_t h, int dtype) {
    return dtype == TKO_BF16 ? tko_bf16_to_f32(h) : tko_f16_to_f32(h);
}
void tko_f32_to_16(const float* src, uint16_t* dst, size_t n, int dtype) {
    for (size_t i = 0; i < n; i++)
        dst[i] = dtype == TKO_BF16 ? tko_f32_to_bf16(src[i]) : tko_f32_to_f16(src[i]);
}
void tko_16_to_f32(const uint16_t* src, float* dst, size_t n, int dtype) {
    for (size_t i = 0; i < n; i++) dst[i] = to_f32(src[i], dtype);
}

/* ======================================================================== */
/* tier (1): the reference's contiguous FP32 path                            */
/* ======================================================================== */

/* KVCache::update, src/inference/kv_cache.cpp:121-151: silent no-op on a bad
 * layer/position (:124-126), exact copy of Hkv*D floats to row `position`
 * (:128-140), seq_len bumped when position >= seq_len (:148-150). */
int tko_kv_update_f32(float* k_data, float* v_data, int num_layers, int max_seq_len,
                      int num_kv_heads, int head_dim, int layer, int position,
                      const float* key, const float* value, int seq_len) {
    if (!k_data || !v_data) return seq_len;
    if (position < 0) return seq_len;
    if (layer < 0 || layer >= num_layers || position >= max_seq_len) return seq_len;
    size_t row = (size_t)num_kv_heads * head_dim;
    size_t layer_stride = (size_t)max_seq_len * row;
    size_t off = (size_t)layer * layer_stride + (size_t)position * row;
    memcpy(k_data + off, key, row * sizeof(float));
    memcpy(v_data + off, value, row * sizeof(float));
    if (position >= seq_len) seq_len = position + 1;
    return seq_len;
}

/* One query head over rows with stride `row_stride` floats.
 * attention_decode_kernel, src/compute/cuda/attention.cu:58-157:
 *   score = dot * scale (:85-92), max from -1e30f (:97), expf (:122),
 *   inv = 1/(sum + 1e-8f) (:142), out = sum_p w[p]*V[p] in position order (:149-156).
 * `scores` is scratch of seq_len floats. */
static void attn_head_kv(const float* qh, const float* k_rows, const float* v_rows,
                         size_t k_stride, size_t v_stride, int k_dim, int v_dim, int seq_len, float scale,
                         float* scores, float* out) {
    const int head_dim = v_dim;
    const size_t row_stride = v_stride;
    for (int p = 0; p < seq_len; p++) {
        const float* kh = k_rows + (size_t)p * k_stride;
        float dot = 0.0f;
        for (int d = 0; d < k_dim; d++) dot += qh[d] * kh[d];
        scores[p] = dot * scale;
    }
    float max_val = -1e30f;
    for (int p = 0; p < seq_len; p++) max_val = fmaxf(max_val, scores[p]);
    float sum_exp = 0.0f;
    for (int p = 0; p < seq_len; p++) { scores[p] = expf(scores[p] - max_val); sum_exp += scores[p]; }
    float inv_sum = 1.0f / (sum_exp + 1e-8f);
    for (int p = 0; p < seq_len; p++) scores[p] *= inv_sum;
    for (int d = 0; d < head_dim; d++) out[d] = 0.0f;
    for (int p = 0; p < seq_len; p++) {
        const float* vh = v_rows + (size_t)p * row_stride;
        float w = scores[p];
        for (int d = 0; d < head_dim; d++) out[d] += w * vh[d];
    }
}

static void attn_head_f32(const float* qh, const float* k_rows, const float* v_rows,
                          size_t row_stride, int head_dim, int seq_len, float scale,
                          float* scores, float* out) {
    attn_head_kv(qh, k_rows, v_rows, row_stride, row_stride, head_dim, head_dim, seq_len, scale, scores, out);
}

/* cuda::attention_decode_mla, src/compute/cuda/attention.cu:168-253,332-349: K rows of k_head_dim
 * (scores, scale = 1/sqrtf(k_head_dim)), V rows and output of v_head_dim; otherwise the same
 * three-pass softmax as attention_decode. */
void tko_attention_decode_mla_f32(const float* q, const float* k_cache, const float* v_cache, float* out,
                                  int num_heads, int num_kv_heads, int k_head_dim, int v_head_dim, int seq_len) {
    float scale = 1.0f / sqrtf((float)k_head_dim);
    float* scores = (float*)malloc(sizeof(float) * (size_t)(seq_len > 0 ? seq_len : 1));
    for (int h = 0; h < num_heads; h++) {
        int kvh = h / (num_heads / num_kv_heads);
        attn_head_kv(q + (size_t)h * k_head_dim, k_cache + (size_t)kvh * k_head_dim, v_cache + (size_t)kvh * v_head_dim,
                     (size_t)num_kv_heads * k_head_dim, (size_t)num_kv_heads * v_head_dim, k_head_dim, v_head_dim,
                     seq_len, scale, scores, out + (size_t)h * v_head_dim);
    }
    free(scores);
}

/* cuda::attention_decode, src/compute/cuda/attention.cu:315-330 (scale = 1/sqrtf(D));
 * GQA map kv_head = head / (H/Hkv), :70. */
void tko_attention_decode_f32(const float* q, const float* k_cache, const float* v_cache,
                              float* out, int num_heads, int num_kv_heads, int head_dim,
                              int seq_len) {
    float scale = 1.0f / sqrtf((float)head_dim);
    size_t row = (size_t)num_kv_heads * head_dim;
    float* scores = (float*)malloc(sizeof(float) * (size_t)(seq_len > 0 ? seq_len : 1));
    for (int h = 0; h < num_heads; h++) {
        int kvh = h / (num_heads / num_kv_heads);
        attn_head_f32(q + (size_t)h * head_dim, k_cache + (size_t)kvh * head_dim,
                      v_cache + (size_t)kvh * head_dim, row, head_dim, seq_len, scale,
                      scores, out + (size_t)h * head_dim);
    }
    free(scores);
}

/* rope_mla_kernel, src/compute/cuda/attention.cu:259-294: the same rotation on the rope dims only
 * (the last rope_hd dims of rows of nope_hd + rope_hd), freq = 1/powf(theta, d/rope_hd), no scaling. */
void tko_rope_mla_f32(float* q, float* k, int num_heads, int num_kv_heads, int nope_hd, int rope_hd,
                      int position, float theta_base) {
    int max_heads = num_heads > num_kv_heads ? num_heads : num_kv_heads;
    int head_dim = nope_hd + rope_hd;
    for (int head = 0; head < max_heads; head++) {
        for (int d = 0; d < rope_hd; d += 2) {
            float freq = 1.0f / powf(theta_base, (float)d / rope_hd);
            float angle = position * freq;
            float c = cosf(angle), s = sinf(angle);
            if (head < num_heads) {
                float* qh = q + (size_t)head * head_dim + nope_hd;
                float a = qh[d], b = qh[d + 1];
                qh[d] = a * c - b * s; qh[d + 1] = a * s + b * c;
            }
            if (head < num_kv_heads) {
                float* kh = k + (size_t)head * head_dim + nope_hd;
                float a = kh[d], b = kh[d + 1];
                kh[d] = a * c - b * s; kh[d + 1] = a * s + b * c;
            }
        }
    }
}

/* rope_kernel, src/compute/cuda/attention.cu:15-48: interleaved pairs (d, d+1),
 * freq = (1/powf(theta, d/D)) * scaling, angle = position * freq. */
void tko_rope_f32(float* q, float* k, int num_heads, int num_kv_heads, int head_dim,
                  int position, float theta_base, float rope_scaling) {
    int max_heads = num_heads > num_kv_heads ? num_heads : num_kv_heads;
    for (int head = 0; head < max_heads; head++) {
        for (int d = 0; d < head_dim; d += 2) {
            float freq = 1.0f / powf(theta_base, (float)d / head_dim);
            freq *= rope_scaling;
            float angle = position * freq;
            float c = cosf(angle), s = sinf(angle);
            if (head < num_heads) {
                float* qh = q + (size_t)head * head_dim;
                float a = qh[d], b = qh[d + 1];
                qh[d] = a * c - b * s; qh[d + 1] = a * s + b * c;
            }
            if (head < num_kv_heads) {
                float* kh = k + (size_t)head * head_dim;
                float a = kh[d], b = kh[d + 1];
                kh[d] = a * c - b * s; kh[d + 1] = a * s + b * c;
            }
        }
    }
}

/* ======================================================================== */
/* tier (2): page manager                                                    */
/* ======================================================================== */
/* Defined here (the reference has no paging):
 *  - free list = LIFO stack of page ids, initialised so that pops yield 0,1,2,...
 *  - sequence slots = lowest free index (idiom of BatchScheduler::allocate_slot,
 *    src/inference/batch.cpp:86-96)
 *  - reserve() takes pages one at a time as ceil(len/page_size) grows; on
 *    shortage it fails with no state change
 *  - free() pushes the sequence's pages in logical order 0..n-1, so the last
 *    logical page is the first one reused. */
struct tko_mgr {
    int num_pages, max_seqs, max_pages_per_seq, page_size;
    int32_t* free_stack; int free_top;
    int32_t* page_table; int32_t* seq_len; int32_t* seq_pages;
    /* cold tier (off unless tko_mgr_enable_cold): host-resident pages, ids from their own LIFO stack;
     * a cold page is recorded in the table as -2 - cold_id */
    int hot_window, num_cold_pages; int32_t* cold_stack; int cold_top;
    int32_t* refcount;   /* per page: sequences whose table names it (prefix sharing after a fork) */
    int32_t* seq_tail;   /* tokens of the logical sequence held AFTER this cache's last one (other ranks) */
};

tko_mgr* tko_mgr_create(int num_pages, int max_seqs, int max_pages_per_seq, int page_size) {
    if (num_pages <= 0 || max_seqs <= 0 || max_pages_per_seq <= 0 || page_size <= 0) return NULL;
    tko_mgr* m = (tko_mgr*)calloc(1, sizeof(*m));
    m->num_pages = num_pages; m->max_seqs = max_seqs;
    m->max_pages_per_seq = max_pages_per_seq; m->page_size = page_size;
    m->free_stack = (int32_t*)malloc(sizeof(int32_t) * (size_t)num_pages);
    for (int i = 0; i < num_pages; i++) m->free_stack[i] = num_pages - 1 - i;
    m->free_top = num_pages;
    size_t n = (size_t)max_seqs * max_pages_per_seq;
    m->page_table = (int32_t*)malloc(sizeof(int32_t) * n);
    for (size_t i = 0; i < n; i++) m->page_table[i] = -1;
    m->seq_len = (int32_t*)malloc(sizeof(int32_t) * (size_t)max_seqs);
    m->seq_pages = (int32_t*)calloc((size_t)max_seqs, sizeof(int32_t));
    m->seq_tail = (int32_t*)calloc((size_t)max_seqs, sizeof(int32_t));
    m->refcount = (int32_t*)calloc((size_t)num_pages, sizeof(int32_t));
    for (int i = 0; i < max_seqs; i++) m->seq_len[i] = -1;
    return m;
}
void tko_mgr_destroy(tko_mgr* m) {
    if (!m) return;
    free(m->refcount); free(m->seq_tail); free(m->cold_stack); free(m->free_stack); free(m->page_table); free(m->seq_len); free(m->seq_pages); free(m);
}
int tko_seq_alloc(tko_mgr* m) {
    for (int i = 0; i < m->max_seqs; i++)
        if (m->seq_len[i] < 0) { m->seq_len[i] = 0; m->seq_pages[i] = 0; m->seq_tail[i] = 0; return i; }
    return -1;
}
/* A sequence lets go of a device page: back to the free stack when nobody else names it. */
static void release_page(tko_mgr* m, int32_t page) {
    if (--m->refcount[page] <= 0) { m->refcount[page] = 0; m->free_stack[m->free_top++] = page; }
}
static int live(const tko_mgr* m, int seq) { return seq >= 0 && seq < m->max_seqs && m->seq_len[seq] >= 0; }
int tko_seq_free(tko_mgr* m, int seq) {
    if (!live(m, seq)) return TKO_INVALID_ARG;
    int32_t* row = m->page_table + (size_t)seq * m->max_pages_per_seq;
    for (int i = 0; i < m->seq_pages[seq]; i++) {
        if (row[i] <= -2) m->cold_stack[m->cold_top++] = -2 - row[i];
        else              release_page(m, row[i]);
        row[i] = -1;
    }
    m->seq_pages[seq] = 0; m->seq_len[seq] = -1;
    return TKO_OK;
}
/* Cold tier.  A page is cold iff its last token index < seq_len - hot_window.  Cold ids come from
 * a LIFO stack that pops 0,1,2,... on a fresh pool; the hot page goes back to the free stack. */
int tko_mgr_enable_cold(tko_mgr* m, int hot_window, int num_cold_pages) {
    if (hot_window < m->page_size || num_cold_pages <= 0 || m->cold_stack) return TKO_INVALID_ARG;
    m->hot_window = hot_window; m->num_cold_pages = num_cold_pages;
    m->cold_stack = (int32_t*)malloc(sizeof(int32_t) * (size_t)num_cold_pages);
    for (int i = 0; i < num_cold_pages; i++) m->cold_stack[i] = num_cold_pages - 1 - i;
    m->cold_top = num_cold_pages;
    return TKO_OK;
}
/* Move every newly cold page of `seq` (ascending logical order) to the cold tier; stable_len is
 * the sequence length before the current step (its tokens are already stored).  Returns the
 * number moved, or -1 when the cold pool is exhausted (nothing is moved then). */
int tko_evict_cold(tko_mgr* m, int seq, int stable_len) {
    if (!live(m, seq) || !m->cold_stack) return 0;
    int32_t* row = m->page_table + (size_t)seq * m->max_pages_per_seq;
    int limit = m->seq_len[seq] + m->seq_tail[seq] - m->hot_window;   /* tokens below this index are cold */
    if (limit > stable_len) limit = stable_len;            /* but never a page the current step still writes */
    int n_cold = limit > 0 ? limit / m->page_size : 0;     /* pages entirely below the limit */
    int need = 0;
    for (int i = 0; i < n_cold; i++) need += row[i] >= 0;
    if (need > m->cold_top) return -1;
    for (int i = 0; i < n_cold; i++) {
        if (row[i] < 0) continue;
        release_page(m, row[i]);
        row[i] = -2 - m->cold_stack[--m->cold_top];
    }
    return need;
}
/* For a sequence split over several caches: `tail` tokens of it follow this cache's last token. */
int tko_set_tail(tko_mgr* m, int seq, int tail) {
    if (!live(m, seq) || tail < 0) return TKO_INVALID_ARG;
    m->seq_tail[seq] = tail;
    return TKO_OK;
}
int tko_num_cold_used(const tko_mgr* m) { return m->cold_stack ? m->num_cold_pages - m->cold_top : 0; }
int tko_reserve(tko_mgr* m, int seq, int n_tokens) {
    if (!live(m, seq) || n_tokens < 0) return TKO_INVALID_ARG;
    int64_t new_len = (int64_t)m->seq_len[seq] + n_tokens;
    int64_t need_pages = (new_len + m->page_size - 1) / m->page_size;
    if (need_pages > m->max_pages_per_seq) return TKO_INVALID_ARG;
    int extra = (int)need_pages - m->seq_pages[seq];
    if (extra > m->free_top) return TKO_OUT_OF_PAGES;
    int32_t* row = m->page_table + (size_t)seq * m->max_pages_per_seq;
    for (int i = 0; i < extra; i++) { int32_t pg = m->free_stack[--m->free_top]; m->refcount[pg] = 1; row[m->seq_pages[seq]++] = pg; }
    m->seq_len[seq] = (int32_t)new_len;
    return TKO_OK;
}
/* Drop tokens past new_len; pages no longer needed go back in logical order. */
int tko_truncate(tko_mgr* m, int seq, int new_len) {
    if (!live(m, seq) || new_len < 0 || new_len > m->seq_len[seq]) return TKO_INVALID_ARG;
    int keep = (new_len + m->page_size - 1) / m->page_size;
    int32_t* row = m->page_table + (size_t)seq * m->max_pages_per_seq;
    /* a page in the host pool cannot become the page that later appends write */
    if (new_len % m->page_size != 0 && keep > 0 && row[keep - 1] <= -2) return TKO_UNSUPPORTED;
    for (int i = keep; i < m->seq_pages[seq]; i++) {
        if (row[i] <= -2) m->cold_stack[m->cold_top++] = -2 - row[i];
        else              release_page(m, row[i]);
        row[i] = -1;
    }
    m->seq_pages[seq] = keep; m->seq_len[seq] = new_len;
    return TKO_OK;
}
/* Install a caller-chosen page list on an empty live sequence; the pages leave the free
 * stack, whose remaining order is kept. */
int tko_adopt(tko_mgr* m, int seq, const int32_t* pages, int n_pages, int seq_len) {
    if (!live(m, seq) || m->seq_pages[seq] != 0 || n_pages < 0 || n_pages > m->max_pages_per_seq) return TKO_INVALID_ARG;
    if (seq_len < 0 || (seq_len + m->page_size - 1) / m->page_size != n_pages) return TKO_INVALID_ARG;
    uint8_t* want = (uint8_t*)calloc((size_t)m->num_pages, 1);
    int ok = 1, found = 0;
    for (int i = 0; i < n_pages && ok; i++) {
        if (pages[i] < 0 || pages[i] >= m->num_pages || want[pages[i]]) ok = 0; else want[pages[i]] = 1;
    }
    for (int i = 0; i < m->free_top && ok; i++) found += want[m->free_stack[i]];
    if (!ok || found != n_pages) { free(want); return TKO_INVALID_ARG; }
    int w = 0;
    for (int i = 0; i < m->free_top; i++) if (!want[m->free_stack[i]]) m->free_stack[w++] = m->free_stack[i];
    m->free_top = w;
    int32_t* row = m->page_table + (size_t)seq * m->max_pages_per_seq;
    for (int i = 0; i < n_pages; i++) { row[i] = pages[i]; m->refcount[pages[i]] = 1; }
    m->seq_pages[seq] = n_pages; m->seq_len[seq] = seq_len;
    free(want);
    return TKO_OK;
}
/* Prefix sharing: a new sequence (lowest free slot) with the same tokens as `parent`.  Full pages
 * are shared (reference-counted); a partly filled last page is copied into a fresh page taken
 * from the free stack (*copy_src / *copy_dst name it, -1 when there is none).  Returns the child
 * slot, -1 when no slot is free, -2 when no page is free (nothing changes in either case). */
int tko_fork(tko_mgr* m, int parent, int32_t* copy_src, int32_t* copy_dst) {
    if (copy_src) *copy_src = -1;
    if (copy_dst) *copy_dst = -1;
    if (!live(m, parent) || m->cold_stack) return -3;
    const int len = m->seq_len[parent], n_pg = m->seq_pages[parent];
    const int partial = len % m->page_size != 0;
    int child = -1;
    for (int i = 0; i < m->max_seqs; i++) if (m->seq_len[i] < 0) { child = i; break; }
    if (child < 0) return -1;
    if (partial && m->free_top < 1) return -2;
    const int32_t* prow = m->page_table + (size_t)parent * m->max_pages_per_seq;
    int32_t* crow = m->page_table + (size_t)child * m->max_pages_per_seq;
    for (int i = 0; i < n_pg; i++) {
        if (partial && i == n_pg - 1) {
            int32_t pg = m->free_stack[--m->free_top];
            m->refcount[pg] = 1;
            crow[i] = pg;
            if (copy_src) *copy_src = prow[i];
            if (copy_dst) *copy_dst = pg;
        } else {
            crow[i] = prow[i];
            m->refcount[prow[i]]++;
        }
    }
    m->seq_len[child] = len; m->seq_pages[child] = n_pg; m->seq_tail[child] = 0;
    return child;
}
int tko_seq_len(const tko_mgr* m, int seq) { return live(m, seq) ? m->seq_len[seq] : -1; }
int tko_seq_num_pages(const tko_mgr* m, int seq) { return live(m, seq) ? m->seq_pages[seq] : -1; }
int tko_num_free_pages(const tko_mgr* m) { return m->free_top; }
const int32_t* tko_page_table(const tko_mgr* m) { return m->page_table; }
const int32_t* tko_seq_lens(const tko_mgr* m) { return m->seq_len; }
int64_t tko_slot(const tko_mgr* m, int seq, int pos) {
    if (!live(m, seq) || pos < 0 || pos >= m->seq_len[seq]) return -1;
    int32_t page = m->page_table[(size_t)seq * m->max_pages_per_seq + pos / m->page_size];
    return (int64_t)page * m->page_size + pos % m->page_size;
}
static uint64_t fnv(uint64_t h, const void* p, size_t n) {
    const uint8_t* b = (const uint8_t*)p;
    for (size_t i = 0; i < n; i++) { h ^= b[i]; h *= 0x100000001B3ull; }
    return h;
}
uint64_t tko_state_digest(const tko_mgr* m) {
    uint64_t h = 0xCBF29CE484222325ull;
    h = fnv(h, m->seq_len, sizeof(int32_t) * (size_t)m->max_seqs);
    h = fnv(h, m->page_table, sizeof(int32_t) * (size_t)m->max_seqs * m->max_pages_per_seq);
    int32_t top = m->free_top;
    h = fnv(h, &top, sizeof(top));
    h = fnv(h, m->free_stack, sizeof(int32_t) * (size_t)m->free_top);
    if (m->cold_stack) {
        int32_t ct = m->cold_top;
        h = fnv(h, &ct, sizeof(ct));
        h = fnv(h, m->cold_stack, sizeof(int32_t) * (size_t)m->cold_top);
    }
    return h;
}

/* ======================================================================== */
/* tier (2): append                                                          */
/* ======================================================================== */
/* tile of (page, kv head): page_size rows of K (D elements) then page_size rows of V (Dv elements) */
static inline size_t tile_off2(int page, int kvh, int kv, int Hkv, int page_size, int D, int Dv) {
    return ((size_t)page * Hkv + kvh) * (size_t)page_size * (D + Dv) + (kv ? (size_t)page_size * D : 0);
}
static inline size_t tile_off(int page, int kvh, int kv, int Hkv, int page_size, int D) {
    return tile_off2(page, kvh, kv, Hkv, page_size, D, D);
}

/* Page-table scatter of 16-bit rows: an exact copy, like the reference's
 * cudaMemcpy of each token row (src/inference/kv_cache.cpp:136-140). */
void tko_append_16(uint16_t* pool, int Hkv, int D, int page_size,
                   const int32_t* page_table, int max_pages_per_seq,
                   int n_tokens, const int32_t* tok_seq, const int32_t* tok_pos,
                   const uint16_t* k, const uint16_t* v, int64_t* slots_out) {
    tko_append_16_kv(pool, Hkv, D, D, page_size, page_table, max_pages_per_seq, n_tokens, tok_seq, tok_pos, k, v, slots_out);
}

/* Same with K rows of D and V rows of Dv elements (the MLA cache: src/inference/kv_cache.cpp:83-108). */
void tko_append_16_kv(uint16_t* pool, int Hkv, int D, int Dv, int page_size,
                      const int32_t* page_table, int max_pages_per_seq,
                      int n_tokens, const int32_t* tok_seq, const int32_t* tok_pos,
                      const uint16_t* k, const uint16_t* v, int64_t* slots_out) {
    for (int t = 0; t < n_tokens; t++) {
        int pos = tok_pos[t];
        int page = page_table[(size_t)tok_seq[t] * max_pages_per_seq + pos / page_size];
        int r = pos % page_size;
        if (slots_out) slots_out[t] = (int64_t)page * page_size + r;
        for (int h = 0; h < Hkv; h++) {
            memcpy(pool + tile_off2(page, h, 0, Hkv, page_size, D, Dv) + (size_t)r * D,
                   k + ((size_t)t * Hkv + h) * D, sizeof(uint16_t) * (size_t)D);
            memcpy(pool + tile_off2(page, h, 1, Hkv, page_size, D, Dv) + (size_t)r * Dv,
                   v + ((size_t)t * Hkv + h) * Dv, sizeof(uint16_t) * (size_t)Dv);
        }
    }
}

/* Seal one (page, kv head, K|V) tile.  Recipe of quantize_fp4_kernel,
 * src/compute/cuda/fp4.cu:102-113, with 448 (E4M3 max) in place of 6:
 * amax -> scale = amax/448, clamped to >= 1e-10 -> multiply by 1/scale. */
static void seal_tile(const uint16_t* src, int n, int carrier, uint8_t* codes, float* scale_out) {
    float amax = 0.0f;
    for (int i = 0; i < n; i++) { float a = fabsf(to_f32(src[i], carrier)); if (a > amax) amax = a; }
    float scale = amax / 448.0f;
    if (scale < 1e-10f) scale = 1e-10f;
    float inv_scale = 1.0f / scale;
    *scale_out = scale;
    for (int i = 0; i < n; i++) codes[i] = tko_e4m3_encode(to_f32(src[i], carrier) * inv_scale);
}

void tko_append_fp8(uint8_t* codes, float* scales, uint16_t* open_pages, int carrier,
                    int Hkv, int D, int page_size,
                    const int32_t* page_table, int max_pages_per_seq,
                    int n_tokens, const int32_t* tok_seq, const int32_t* tok_pos,
                    const uint16_t* k, const uint16_t* v, int64_t* slots_out) {
    size_t tile = (size_t)page_size * D;
    for (int t = 0; t < n_tokens; t++) {
        int seq = tok_seq[t], pos = tok_pos[t];
        int page = page_table[(size_t)seq * max_pages_per_seq + pos / page_size];
        int r = pos % page_size;
        if (slots_out) slots_out[t] = (int64_t)page * page_size + r;
        for (int h = 0; h < Hkv; h++)
            for (int kv = 0; kv < 2; kv++) {
                uint16_t* open = open_pages + (((size_t)seq * Hkv + h) * 2 + kv) * tile;
                const uint16_t* src = (kv ? v : k) + ((size_t)t * Hkv + h) * D;
                memcpy(open + (size_t)r * D, src, sizeof(uint16_t) * (size_t)D);
                if (r == page_size - 1)
                    seal_tile(open, (int)tile, carrier,
                              codes + tile_off(page, h, kv, Hkv, page_size, D),
                              scales + ((size_t)page * Hkv + h) * 2 + kv);
            }
    }
}

/* ======================================================================== */
/* tier (2): paged decode attention                                          */
/* ======================================================================== */
void tko_gather_f32(const tko_view* vw, int seq, int seq_len, int kvh, int t0, int t1,
                    float* k_rows, float* v_rows) {
    int D = vw->head_dim, ps = vw->page_size, Hkv = vw->num_kv_heads;
    int Dv = vw->v_head_dim > 0 ? vw->v_head_dim : D;
    const int32_t* row = vw->page_table + (size_t)seq * vw->max_pages_per_seq;
    int sealed_end = (seq_len / ps) * ps;      /* FP8: tokens >= sealed_end sit in the open page */
    for (int t = t0; t < t1; t++) {
        int page = row[t / ps], r = t % ps;
        for (int kv = 0; kv < 2; kv++) {
            int Dx = kv ? Dv : D;
            float* dst = (kv ? v_rows : k_rows) + (size_t)(t - t0) * Dx;
            if (vw->dtype == TKO_FP8_E4M3) {
                if (t < sealed_end) {
                    const uint8_t* c = (const uint8_t*)vw->pool + tile_off(page, kvh, kv, Hkv, ps, D) + (size_t)r * D;
                    float s = vw->scales[((size_t)page * Hkv + kvh) * 2 + kv];
                    for (int d = 0; d < D; d++) dst[d] = tko_e4m3_decode(c[d]) * s;
                } else {
                    const uint16_t* o = vw->open_pages + (((size_t)seq * Hkv + kvh) * 2 + kv) * (size_t)ps * D + (size_t)r * D;
                    for (int d = 0; d < D; d++) dst[d] = to_f32(o[d], vw->carrier_dtype);
                }
            } else {
                const uint16_t* p = (const uint16_t*)vw->pool + tile_off2(page, kvh, kv, Hkv, ps, D, Dv) + (size_t)r * Dx;
                for (int d = 0; d < Dx; d++) dst[d] = to_f32(p[d], vw->dtype);
            }
        }
    }
}

void tko_decode_paged(const tko_view* vw, int n_seqs, const int32_t* seq_ids,
                      const int32_t* seq_lens, const uint16_t* q, float* out) {
    int H = vw->num_heads, Hkv = vw->num_kv_heads, D = vw->head_dim, G = H / Hkv;
    int Dv = vw->v_head_dim > 0 ? vw->v_head_dim : D;
    float scale = 1.0f / sqrtf((float)D);
    int n_units = n_seqs * Hkv;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1)
#endif
    for (int u = 0; u < n_units; u++) {
        int b = u / Hkv, kvh = u % Hkv;
        int len = seq_lens[b];
        size_t n = (size_t)(len > 0 ? len : 1);
        float* kr = (float*)malloc(sizeof(float) * n * D);
        float* vr = (float*)malloc(sizeof(float) * n * Dv);
        float* sc = (float*)malloc(sizeof(float) * n);
        float* qf = (float*)malloc(sizeof(float) * (size_t)D);
        tko_gather_f32(vw, seq_ids[b], len, kvh, 0, len, kr, vr);
        for (int g = 0; g < G; g++) {
            int h = kvh * G + g;           /* inverse of kv_head = h / (H/Hkv) */
            tko_16_to_f32(q + ((size_t)b * H + h) * D, qf, (size_t)D, vw->carrier_dtype);
            attn_head_kv(qf, kr, vr, (size_t)D, (size_t)Dv, D, Dv, len, scale, sc, out + ((size_t)b * H + h) * Dv);
        }
        free(kr); free(vr); free(sc); free(qf);
    }
}

void tko_decode_partial(const tko_view* vw, int seq, int seq_len, int t0, int t1,
                        const uint16_t* q, float* m, float* l, float* o) {
    int H = vw->num_heads, Hkv = vw->num_kv_heads, D = vw->head_dim, G = H / Hkv;
    int Dv = vw->v_head_dim > 0 ? vw->v_head_dim : D;
    float scale = 1.0f / sqrtf((float)D);
    int n = t1 - t0;
    float* kr = (float*)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1) * D);
    float* vr = (float*)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1) * Dv);
    float* sc = (float*)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
    float* qf = (float*)malloc(sizeof(float) * (size_t)D);
    for (int kvh = 0; kvh < Hkv; kvh++) {
        tko_gather_f32(vw, seq, seq_len, kvh, t0, t1, kr, vr);
        for (int g = 0; g < G; g++) {
            int h = kvh * G + g;
            tko_16_to_f32(q + (size_t)h * D, qf, (size_t)D, vw->carrier_dtype);
            float mx = -1e30f;
            for (int p = 0; p < n; p++) {
                float dot = 0.0f;
                for (int d = 0; d < D; d++) dot += qf[d] * kr[(size_t)p * D + d];
                sc[p] = dot * scale; mx = fmaxf(mx, sc[p]);
            }
            float sum = 0.0f;
            float* oh = o + (size_t)h * Dv;
            for (int d = 0; d < Dv; d++) oh[d] = 0.0f;
            for (int p = 0; p < n; p++) {
                float e = expf(sc[p] - mx); sum += e;
                for (int d = 0; d < Dv; d++) oh[d] += e * vr[(size_t)p * Dv + d];
            }
            m[h] = mx; l[h] = sum;
        }
    }
    free(kr); free(vr); free(sc); free(qf);
}

void tko_combine(int n_parts, const float* m, const float* l, const float* o, int D, float* out) {
    float M = -1e30f;
    for (int i = 0; i < n_parts; i++) M = fmaxf(M, m[i]);
    float L = 0.0f;
    for (int d = 0; d < D; d++) out[d] = 0.0f;
    for (int i = 0; i < n_parts; i++) {
        float w = expf(m[i] - M);
        L += l[i] * w;
        for (int d = 0; d < D; d++) out[d] += o[(size_t)i * D + d] * w;
    }
    float inv = 1.0f / (L + 1e-8f);
    for (int d = 0; d < D; d++) out[d] *= inv;
}

/* The launcher of multi-process jobs pins OMP_NUM_THREADS to 1; a timed CPU arm that is alone on the
 * host asks for its threads explicitly. */
void tko_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int tko_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
