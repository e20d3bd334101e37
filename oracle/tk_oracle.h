/*
 * tk_oracle.h — CPU oracle for the paged KV-cache hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is the checker the CUDA path is compared
 * against and the CPU baseline that the benchmark reports; the product
 * library never links, loads or calls anything declared here.
 *
 * Two tiers of pinning:
 *   (1) tko_attention_decode_f32 / tko_kv_update_f32 restate the reference's
 *       own contiguous-FP32 code (src/compute/cuda/attention.cu:58-157,315-330;
 *       src/inference/kv_cache.cpp:121-151).  They are pinned against the
 *       reference kernels themselves (golden vectors under tests/golden made by
 *       running the unmodified reference sources on a GPU).
 *   (2) Paging, the free list, FP8-E4M3 sealing and split-KV/LSE-combine do
 *       not exist in the reference: for those this oracle DEFINES the
 *       semantics ("parity unpinned" by the reference).  The paged attention
 *       is a gather followed by exactly the tier-(1) arithmetic.
 */
#ifndef TK_ORACLE_H
#define TK_ORACLE_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes: same numbering as the product C ABI (include/titan_kv.h) */
enum { TKO_OK = 0, TKO_INVALID_ARG = 1, TKO_OUT_OF_PAGES = 2, TKO_OUT_OF_SEQS = 5, TKO_UNSUPPORTED = 6 };
/* storage dtypes: numbering of the reference's titan::DType (src/core/types.h:17-21) */
enum { TKO_FP16 = 1, TKO_BF16 = 2, TKO_FP8_E4M3 = 3 };

/* ---- scalar conversions ------------------------------------------------ */
float    tko_e4m3_decode(uint8_t code);      /* src/compute/cuda/fp4.cu:173-185 */
uint8_t  tko_e4m3_encode(float x);           /* round-to-nearest-even, saturate-to-finite */
uint16_t tko_f32_to_f16(float x);
uint16_t tko_f32_to_bf16(float x);
float    tko_f16_to_f32(uint16_t h);
float    tko_bf16_to_f32(uint16_t h);
void     tko_f32_to_16(const float* src, uint16_t* dst, size_t n, int dtype);
void     tko_16_to_f32(const uint16_t* src, float* dst, size_t n, int dtype);

/* ---- tier (1): the reference's contiguous FP32 path ------------------- */
/* KVCache::update, src/inference/kv_cache.cpp:121-151.  Returns the new seq_len. */
int tko_kv_update_f32(float* k_data, float* v_data, int num_layers, int max_seq_len,
                      int num_kv_heads, int head_dim, int layer, int position,
                      const float* key, const float* value, int seq_len);
/* cuda::attention_decode, src/compute/cuda/attention.cu:58-157,315-330 */
void tko_attention_decode_f32(const float* q, const float* k_cache, const float* v_cache,
                              float* out, int num_heads, int num_kv_heads, int head_dim,
                              int seq_len);

/* cuda::attention_decode_mla, src/compute/cuda/attention.cu:168-253,332-349 */
void tko_attention_decode_mla_f32(const float* q, const float* k_cache, const float* v_cache, float* out,
                                  int num_heads, int num_kv_heads, int k_head_dim, int v_head_dim, int seq_len);

/* ---- tier (2): page manager (semantics defined here) ------------------- */
typedef struct tko_mgr tko_mgr;
tko_mgr* tko_mgr_create(int num_pages, int max_seqs, int max_pages_per_seq, int page_size);
void     tko_mgr_destroy(tko_mgr* m);
int      tko_seq_alloc(tko_mgr* m);                    /* lowest free slot, or -1 */
int      tko_seq_free(tko_mgr* m, int seq);
int      tko_reserve(tko_mgr* m, int seq, int n_tokens);
int      tko_truncate(tko_mgr* m, int seq, int new_len);
int      tko_adopt(tko_mgr* m, int seq, const int32_t* pages, int n_pages, int seq_len);
int      tko_mgr_enable_cold(tko_mgr* m, int hot_window, int num_cold_pages);
int      tko_evict_cold(tko_mgr* m, int seq, int stable_len);   /* pages moved, -1 if the cold pool is full */
int      tko_num_cold_used(const tko_mgr* m);
int      tko_set_tail(tko_mgr* m, int seq, int tail);
int      tko_fork(tko_mgr* m, int parent, int32_t* copy_src, int32_t* copy_dst);  /* child slot; -1 no slot, -2 no page */
int      tko_seq_len(const tko_mgr* m, int seq);       /* -1 if seq not live */
int      tko_seq_num_pages(const tko_mgr* m, int seq);
int      tko_num_free_pages(const tko_mgr* m);
const int32_t* tko_page_table(const tko_mgr* m);       /* [max_seqs][max_pages_per_seq], -1 unmapped */
const int32_t* tko_seq_lens(const tko_mgr* m);         /* [max_seqs], -1 = slot free */
int64_t  tko_slot(const tko_mgr* m, int seq, int pos); /* page*page_size + pos%page_size */
/* FNV-1a 64 over (seq lens, page tables, free stack): one number per step for churn parity */
uint64_t tko_state_digest(const tko_mgr* m);

/* ---- tier (2): append -------------------------------------------------- */
/* 16-bit pool layout per layer: [num_pages][Hkv][2 (K,V)][page_size][D].
 * k, v: [n_tokens][Hkv][D] 16-bit.  slots_out (nullable): slot of every token. */
void tko_append_16(uint16_t* pool, int num_kv_heads, int head_dim, int page_size,
                   const int32_t* page_table, int max_pages_per_seq,
                   int n_tokens, const int32_t* tok_seq, const int32_t* tok_pos,
                   const uint16_t* k, const uint16_t* v, int64_t* slots_out);
void tko_append_16_kv(uint16_t* pool, int num_kv_heads, int head_dim, int v_head_dim, int page_size,
                      const int32_t* page_table, int max_pages_per_seq,
                      int n_tokens, const int32_t* tok_seq, const int32_t* tok_pos,
                      const uint16_t* k, const uint16_t* v, int64_t* slots_out);
/* FP8 pool: codes [num_pages][Hkv][2][page_size][D] bytes, scales [num_pages][Hkv][2] f32,
 * open pages [max_seqs][Hkv][2][page_size][D] in the 16-bit carrier type.  Tokens are
 * processed in order; a token landing on the last row of a page seals that page:
 * amax over page_size*D values -> scale = max(amax/448, 1e-10) -> code = e4m3(x * (1/scale))
 * (recipe of src/compute/cuda/fp4.cu:102-113 with the E4M3 maximum). */
void tko_append_fp8(uint8_t* codes, float* scales, uint16_t* open_pages, int carrier_dtype,
                    int num_kv_heads, int head_dim, int page_size,
                    const int32_t* page_table, int max_pages_per_seq,
                    int n_tokens, const int32_t* tok_seq, const int32_t* tok_pos,
                    const uint16_t* k, const uint16_t* v, int64_t* slots_out);

/* ---- tier (2): paged decode attention ---------------------------------- */
typedef struct {
    int dtype;                 /* TKO_FP16 / TKO_BF16 / TKO_FP8_E4M3 */
    int carrier_dtype;         /* 16-bit type of q and of open pages (== dtype unless FP8) */
    int num_heads, num_kv_heads, head_dim, page_size;
    const void*     pool;      /* 16-bit pool or FP8 codes */
    const float*    scales;    /* FP8 only */
    const uint16_t* open_pages;/* FP8 only */
    const int32_t*  page_table; int max_pages_per_seq;
    int v_head_dim;            /* V rows / output width when it differs from head_dim (MLA); 0 = head_dim */
} tko_view;
/* Gather kv head `kvh` of tokens [t0,t1) of sequence `seq` (length seq_len) to FP32 rows. */
void tko_gather_f32(const tko_view* v, int seq, int seq_len, int kvh, int t0, int t1,
                    float* k_rows, float* v_rows);
/* out[n_seqs][H][D] FP32 = reference arithmetic on the gathered rows; q is 16-bit [n_seqs][H][D].
 * Parallel over (sequence, kv head) when built with OpenMP. */
void tko_decode_paged(const tko_view* v, int n_seqs, const int32_t* seq_ids,
                      const int32_t* seq_lens, const uint16_t* q, float* out);
/* Split-KV partial over tokens [t0,t1): m from -1e30, l = sum exp(s-m), o = sum exp(s-m)*V (unnormalised). */
void tko_decode_partial(const tko_view* v, int seq, int seq_len, int t0, int t1,
                        const uint16_t* q /*[H][D]*/, float* m /*[H]*/, float* l /*[H]*/, float* o /*[H][D]*/);
/* LSE merge of n_parts partials of one head: M=max m_i, L=sum l_i e^{m_i-M}, O=sum o_i e^{m_i-M}, out=O/(L+1e-8). */
void tko_combine(int n_parts, const float* m, const float* l, const float* o, int head_dim, float* out);

/* ---- "next" row: RoPE exactly as rope_kernel, src/compute/cuda/attention.cu:15-48 */
void tko_rope_f32(float* q, float* k, int num_heads, int num_kv_heads, int head_dim,
                  int position, float theta_base, float rope_scaling);
/* ... and as rope_mla_kernel, src/compute/cuda/attention.cu:259-294 (rope dims of MLA rows only) */
void tko_rope_mla_f32(float* q, float* k, int num_heads, int num_kv_heads, int nope_hd, int rope_hd,
                      int position, float theta_base);

int tko_num_threads(void);
void tko_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
