/*
 * titan_kv.h — C ABI of the B200 (sm_100a) paged KV-cache hot path.
 *
 * The reference (titan-engine) has no FFI seam for this path: callers link
 * straight against class titan::KVCache (src/inference/kv_cache.h:15-81) and the
 * free function titan::cuda::attention_decode (src/compute/dispatch.h:73-75).
 * Every entry point below names the reference interface it stands in for.  The
 * C++ classes with the reference's own names that sit on top of this ABI are in
 * titan_engine_b200/csrc/compat/.
 *
 * Conventions
 *  - plain pointers and sizes only; `stream` is a cudaStream_t passed as void*
 *    (NULL = default stream, as the reference passes nullptr: src/inference/engine.cpp:191)
 *  - every call returns a tk_status and never throws; tk_kv_last_error() gives text
 *  - one caller thread per handle (the reference serialises the path under one
 *    mutex, src/api/server.cpp:33); all device work is stream-ordered and no entry
 *    point other than create/destroy and the *_host variants synchronises the device
 *  - no device allocation after tk_kv_create* (reference invariant: no cudaMalloc
 *    during generation, src/model/moe.cpp:49-108); the two exceptions are one-off:
 *    the first tk_kv_decode_exchange of a handle, and a tk_kv_decode_multi step that
 *    needs more split-KV workspace than any step before it
 *  - there is no CPU fallback: without a CUDA device every compute call fails.
 */
#ifndef TITAN_KV_H
#define TITAN_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tk_status {
    TK_OK = 0,
    TK_INVALID_ARG = 1,
    TK_OUT_OF_PAGES = 2,
    TK_CUDA_ERROR = 3,
    TK_TIMEOUT = 4,
    TK_OUT_OF_SEQS = 5,
    TK_UNSUPPORTED = 6
} tk_status;

/* dtype numbering = titan::DType (src/core/types.h:17-21) */
enum { TK_FP32 = 0, TK_FP16 = 1, TK_BF16 = 2, TK_FP8_E4M3 = 3 };

/* which decode kernel tk_kv_decode launches */
enum { TK_DECODE_AUTO = 0, TK_DECODE_SIMT = 1, TK_DECODE_MMA = 2 };
/* who merges the split-KV partial rows: the attention kernel's last CTA per (sequence, kv head), or a
 * combine launch of its own after it */
enum { TK_MERGE_IN_KERNEL = 0, TK_MERGE_SEPARATE = 1 };
/* back-to-back attention launches of different layers: the later one may start (programmatic dependent
 * launch) while the earlier one drains, or every launch waits for the one before it */
enum { TK_OVERLAP_AUTO = 0, TK_OVERLAP_OFF = 1 };
/* attention of prefill chunks (tk_kv_decode_multi with many tokens per sequence): the tcgen05 kernel (tiles of
 * 128 rows, accumulators in tensor memory) where the shape allows it (16-bit pool, head_dim 128), or always the
 * mma.sync kernel (tiles of 64 rows) */
enum { TK_PREFILL_AUTO = 0, TK_PREFILL_MMA_SYNC = 1 };

/* Stands in for the (L, Hkv, D, max_seq_len, dtype) argument list of
 * KVCache::initialize (src/inference/kv_cache.h:21-23) plus the fields of
 * RuntimeConfig the reference declares for this path but never reads
 * (max_context_len, kv_cache_dtype: src/core/types.h:243-248). */
typedef struct tk_kv_config {
    int32_t num_layers;
    int32_t num_heads;          /* query heads */
    int32_t num_kv_heads;
    int32_t head_dim;           /* 64 or 128; 192 with v_head_dim 128 for the MLA cache */
    int32_t page_size;          /* tokens per page: 16 */
    int32_t dtype;              /* storage: TK_FP16 / TK_BF16 / TK_FP8_E4M3 */
    int32_t io_dtype;           /* type of q, k, v, out and of FP8 open pages: TK_FP16 / TK_BF16; 0 = dtype */
    int32_t num_pages;          /* physical pages per layer */
    int32_t max_seqs;           /* sequence slots */
    int32_t max_pages_per_seq;  /* page-table row length */
    int32_t max_step_tokens;    /* most tokens one step may append (all sequences together) */
    int32_t chunk_tokens;       /* split-KV chunk, multiple of page_size; 0 = choose per step */
    int32_t decode_impl;        /* TK_DECODE_* */
    int32_t device;             /* CUDA ordinal, -1 = current, -2 = none: page bookkeeping only,
                                   every compute call fails (there is no CPU compute path) */
    int32_t hot_window;         /* most recent tokens of a sequence kept in HBM; 0 = everything (no cold
                                   tier).  A page whose last token index < seq_len - hot_window is moved
                                   to pinned host memory and staged back one layer ahead of its use. */
    int32_t cold_pages;         /* capacity of the host pool, pages per layer (needed when hot_window > 0) */
    int32_t v_head_dim;         /* width of V rows and of the output; 0 = head_dim.  192/128 is the MLA cache
                                   (KVCache::initialize_external_mla, src/inference/kv_cache.cpp:83-108;
                                   attention_decode_mla, src/compute/cuda/attention.cu:168-253): K rows and q
                                   have head_dim, scale = 1/sqrtf(head_dim); 16-bit storage, generic kernel */
    int32_t merge_impl;         /* TK_MERGE_* */
    int32_t launch_overlap;     /* TK_OVERLAP_* */
    int32_t prefill_impl;       /* TK_PREFILL_* */
} tk_kv_config;

typedef struct tk_kv_stats {    /* in the style of CacheStats, src/memory/memory_manager.h:211-220 */
    int64_t pages_total, pages_free, pages_cold;
    int64_t page_allocs, page_frees, seq_allocs, seq_frees;
    int64_t evictions, prefetch_hits, prefetch_misses;
    int64_t bytes_h2d, bytes_d2h;
    int64_t steps, tokens_appended, pages_sealed;
    int64_t evictions_refused;  /* (sequence, step) pairs whose old pages stayed in HBM because the host pool was
                                   full; the step still succeeds, later steps end in TK_OUT_OF_PAGES once HBM fills */
} tk_kv_stats;

typedef struct tk_kv tk_kv;

const char* tk_status_str(int status);
const char* tk_kv_last_error(const tk_kv* h);          /* h may be NULL: last create error */

/* ---- lifetime: KVCache::initialize / initialize_external / ~KVCache ----------
 * (src/inference/kv_cache.cpp:16-57, :59-81, :9-14).  The pool is zero-filled like
 * the reference's slabs (:49-50). */
void   tk_kv_config_default(tk_kv_config* cfg);
size_t tk_kv_arena_bytes(const tk_kv_config* cfg);     /* device bytes create_external needs */
int    tk_kv_create(const tk_kv_config* cfg, tk_kv** out);
/* Adopts caller-owned device memory (e.g. carved from the reference's VramPool,
 * src/model/moe.cpp:549-595); it is never freed by the handle (kv_cache.cpp:71).  All arena_bytes
 * belong to the handle: when they exceed tk_kv_arena_bytes by 4 KiB or more, the 4 KiB behind the
 * pool hold guard bytes (tk_kv_check_canaries). */
int    tk_kv_create_external(const tk_kv_config* cfg, void* arena, size_t arena_bytes, tk_kv** out);
int    tk_kv_destroy(tk_kv* h);
int    tk_kv_get_config(const tk_kv* h, tk_kv_config* out);
/* KVCache::memory_bytes (kv_cache.cpp:153-156) */
size_t tk_kv_memory_bytes(const tk_kv* h);
/* Device address of layer `layer`'s pool: [num_pages][Hkv][2][page_size][D] (parity dumps).
 * FP8: `codes`, plus scales f32 [num_pages][Hkv][2] and open pages [max_seqs][Hkv][2][page_size][D]. */
int    tk_kv_layer_ptrs(const tk_kv* h, int layer, void** pool, float** scales, void** open_pages);

/* ---- sequences and pages ------------------------------------------------------
 * The reference's closest analogues: BatchScheduler::allocate_slot / free_slot
 * (src/inference/batch.cpp:86-101; lowest free index) and KVCache::clear /
 * set_seq_len (kv_cache.cpp:158-167, kv_cache.h:51).  Host-only; no device work. */
int tk_kv_seq_alloc(tk_kv* h, int32_t* seq_out);
int tk_kv_seq_free(tk_kv* h, int32_t seq);
/* Grow `seq` by n_tokens, taking pages from the LIFO free list (pops 0,1,2,... on a
 * fresh pool).  TK_OUT_OF_PAGES leaves all state unchanged. */
int tk_kv_reserve(tk_kv* h, int32_t seq, int32_t n_tokens);
/* Drop tokens past new_len (speculative rollback; the reference has none:
 * src/inference/speculative.cpp:306-307).  TK_UNSUPPORTED when new_len ends inside a page that is
 * shared with a forked sequence or lives in the host (cold) pool: later appends would have to write it. */
int tk_kv_truncate(tk_kv* h, int32_t seq, int32_t new_len);
/* Install a caller-chosen page list (e.g. a shuffled pool) as the table of `seq`;
 * the pages must be free. */
int tk_kv_seq_adopt(tk_kv* h, int32_t seq, const int32_t* pages, int32_t n_pages, int32_t seq_len);
/* Prefix sharing: a new sequence (lowest free slot) with the same tokens as `parent`.  Full pages
 * are shared between the two (reference-counted, freed when the last owner lets go); a partly
 * filled last page is copied on `stream` into a fresh page, so that both can go on appending.
 * TK_OUT_OF_SEQS / TK_OUT_OF_PAGES change nothing.  Not available with a cold tier.
 * (The reference has neither prefix sharing nor rollback: src/inference/speculative.cpp:306-307.) */
int tk_kv_seq_fork(tk_kv* h, int32_t parent, int32_t* child_out, void* stream);
/* For a sequence whose tokens are split over several caches (one per GPU): tail_tokens of it
 * follow this cache's last token, so the hot window is measured from seq_len + tail_tokens. */
int tk_kv_seq_set_tail(tk_kv* h, int32_t seq, int32_t tail_tokens);
/* KVCache::seq_len (kv_cache.h:50), per sequence here; -1 if the slot is free */
int tk_kv_seq_len(const tk_kv* h, int32_t seq);
int tk_kv_num_free_pages(const tk_kv* h);
/* Copies the page-table row of `seq` (n_out pages). */
int tk_kv_page_table(const tk_kv* h, int32_t seq, int32_t* out, int32_t cap, int32_t* n_out);
/* Slot index page*page_size + pos%page_size of token `pos`, or -1. */
int64_t  tk_kv_slot(const tk_kv* h, int32_t seq, int32_t pos);
/* FNV-1a over (sequence lengths, page tables, free stack). */
uint64_t tk_kv_state_digest(const tk_kv* h);
int tk_kv_get_stats(const tk_kv* h, tk_kv_stats* out);
/* Snapshot / restore of the allocator and page-table state (sequence lengths, page tables, free list,
 * reference counts, cold ids) as a flat int32 image, for replaying a churn run from the step where it went
 * wrong; the reference has no counterpart (its slots are whole-sequence, src/inference/batch.cpp:86-101).
 * save: *n_out = image length; image may be NULL to ask for it.  load: a handle of the same geometry takes
 * the state over (the K/V bytes of the pool are the caller's to restore); the device copy of the page table
 * is rewritten by the next tk_kv_step_begin.  TK_INVALID_ARG for a foreign or damaged image. */
int tk_kv_state_save(const tk_kv* h, int32_t* image, int64_t cap, int64_t* n_out);
int tk_kv_state_load(tk_kv* h, const int32_t* image, int64_t n);

/* ---- one decode/prefill step ---------------------------------------------------
 * tk_kv_step_begin reserves n_new[i] tokens for seq_ids[i] (all or nothing), lays
 * out this step's token list (sequence order of the call, then position) and the
 * split-KV work list, and uploads the page-table delta: one pinned-buffer copy and
 * one small kernel on `stream`.  n_new may be NULL (decode without append).
 * Sequence lengths advance once per step, not once per layer as the reference's
 * single counter does (kv_cache.cpp:148-150). */
int tk_kv_step_begin(tk_kv* h, int32_t n_seqs, const int32_t* seq_ids, const int32_t* n_new,
                     void* stream);
/* Same, with len_cap[i] limiting how many leading tokens of seq_ids[i] attention covers
 * (cuda::attention_decode takes seq_len as an argument, src/compute/dispatch.h:73-75, so a
 * caller may attend to a prefix).  16-bit storage only. */
int tk_kv_step_begin_capped(tk_kv* h, int32_t n_seqs, const int32_t* seq_ids, const int32_t* n_new,
                            const int32_t* len_cap, void* stream);
/* The query-head count is an argument of cuda::attention_decode, not of KVCache::initialize
 * (src/inference/kv_cache.h:21-23): a handle sized for cfg.num_heads may be told a smaller
 * head count (same kv heads) before a step. */
int tk_kv_set_num_heads(tk_kv* h, int32_t num_heads);
int tk_kv_step_num_tokens(const tk_kv* h);
int tk_kv_step_num_work_items(const tk_kv* h);
int tk_kv_step_chunk_tokens(const tk_kv* h);
/* Work list of the prefill attention kernel for the current step (inspection and tests): *n_items items of
 * four int32 (index into the step's sequences, split-KV chunk, kv head, tile of 64 (token, head) rows), the
 * split-KV chunk in tokens of each of the step's sequences, and how many (sequence, chunk, kv head) items
 * stay with the decode kernel.  *n_items is 0 for a step that tk_kv_decode_multi serves without that kernel. */
int tk_kv_step_prefill_plan(const tk_kv* h, int32_t cap, int32_t* items, int32_t* n_items, int32_t* chunk_tokens,
                            int32_t* n_decode_items);

/* KVCache::update (src/inference/kv_cache.cpp:121-151) for every token of the step:
 * k, v device [n_tokens][Hkv][D] in io_dtype.  Page-table scatter; with FP8 storage,
 * pages completed by this step are sealed (absmax scale + E4M3 codes).
 * slots_out (device int64[n_tokens], may be NULL) receives each token's slot index. */
int tk_kv_append(tk_kv* h, int32_t layer, const void* k, const void* v, int64_t* slots_out,
                 void* stream);
/* cuda::attention_decode (src/compute/cuda/attention.cu:315-330) for every sequence
 * of the step: q, out device [n_seqs][H][D] in io_dtype.  Paged GQA attention,
 * online softmax, split-KV partials and log-sum-exp combine. */
int tk_kv_decode(tk_kv* h, int32_t layer, const void* q, void* out, void* stream);
/* update + attention_decode of one layer in one call (the pair at src/model/dense.cpp:388-398).
 * On a decode step (at most one new token per sequence) with 16-bit storage this is ONE kernel:
 * the attention kernel writes the new token's K/V rows into the page it is about to read.
 * In every other case it does tk_kv_append then tk_kv_decode. */
int tk_kv_append_decode(tk_kv* h, int32_t layer, const void* k, const void* v, const void* q, void* out,
                        void* stream);
/* apply_rope + update + attention_decode of one layer: the three calls of the reference's layer
 * loop (src/model/dense.cpp:382-398; rope_kernel, src/compute/cuda/attention.cu:15-48).  q and k are
 * the rows BEFORE rotation and are not modified; a q row takes the position of its sequence's
 * newest token, a k row its own.  On a decode step with 16-bit storage everything is ONE kernel:
 * q is rotated as it is loaded, the new K row as it is stored. */
int tk_kv_rope_append_decode(tk_kv* h, int32_t layer, const void* k, const void* v, const void* q, void* out,
                             float theta, float scaling, void* stream);
/* tk_kv_decode with explicit types: q_dtype and out_dtype are each TK_FP32 (the reference's
 * float* interface) or the handle's io dtype. */
int tk_kv_decode_ex(tk_kv* h, int32_t layer, const void* q, int32_t q_dtype, void* out, int32_t out_dtype,
                    void* stream);
/* Attention for EVERY token the step appended, several per sequence: q and out are
 * [n_tokens][H][D] (the order of tk_kv_append's rows), token j of a sequence attends to positions
 * <= its own - causal among the step's tokens - and 16 / (num_heads / num_kv_heads) tokens of a
 * sequence share one pass over its pages (more tokens take further passes, up to 8).  Call after
 * tk_kv_append of the layer.  This is the batched verification of drafted tokens
 * that the reference's speculative decoder runs as one layer pass per token
 * (src/inference/speculative.cpp:262-272); rejected tokens are dropped with tk_kv_truncate.
 * It is also the attention of a prefill chunk: the reference runs update + attention_decode once per
 * prompt token (src/inference/engine.cpp:182-193, src/inference/batch.cpp:169-198).  When a sequence
 * appends more than 128 / (num_heads / num_kv_heads) tokens, the sequences with many tokens go to a kernel
 * that works on tiles of 64 (token, head) rows sharing each K/V page tile; the others stay with the decode
 * kernel.  16-bit pools with the tensor-core kernels, every sequence of the step appending at least one
 * token, no cold pages; the MLA shape up to 64 / (num_heads / num_kv_heads) tokens per sequence;
 * TK_UNSUPPORTED otherwise. */
int tk_kv_decode_multi(tk_kv* h, int32_t layer, const void* q, void* out, void* stream);
/* tk_kv_decode_multi with the output type given: TK_FP32 (the reference's float* interface,
 * src/compute/dispatch.h:73-75) or the handle's io dtype. */
int tk_kv_decode_multi_ex(tk_kv* h, int32_t layer, const void* q, void* out, int32_t out_dtype, void* stream);
/* tk_kv_append of the step's rows followed by tk_kv_decode_multi, in one call. */
int tk_kv_append_decode_multi(tk_kv* h, int32_t layer, const void* k, const void* v, const void* q, void* out,
                              void* stream);
/* Same, but stops before normalisation: partial[n_seqs][H][D+2] f32 =
 * (o unnormalised [D], m, l), for a cross-GPU combine. */
int tk_kv_decode_partial(tk_kv* h, int32_t layer, const void* q, float* partial, void* stream);
/* Log-sum-exp merge of n_parts partial sets: parts [n_parts][n_rows][D+2] f32 ->
 * out [n_rows][D] in out_dtype (TK_FP16 / TK_BF16 / TK_FP32). */
int tk_combine_partials(const float* parts, int32_t n_parts, int32_t n_rows, int32_t head_dim,
                        void* out, int32_t out_dtype, void* stream);

/* ---- cross-GPU exchange of partials over peer memory, fused with the combine -----------------
 * One process per GPU.  Every rank owns a mailbox in its device memory; tk_peer_export gives the
 * CUDA IPC handle of it, the ranks swap handles over whatever transport they have, and
 * tk_peer_connect maps the peers' mailboxes.  tk_peer_exchange_combine then is ONE kernel that
 * stores this rank's partial rows [n_rows][dv+2] into every rank's mailbox (plain NVLink peer
 * stores of 8-byte cells that carry the value and the exchange's epoch together, so no flag and no
 * fence follows the rows), waits - with a limit - until the cells of every rank's rows show the epoch,
 * and writes the log-sum-exp combine of all ranks' rows (rank order, same arithmetic as
 * tk_combine_partials) to out [n_rows][dv].  Calls of one tk_peer must be ordered on one stream and made
 * by every rank the same number of times.  A row for which some peer's cells do not arrive within the
 * limit (default 2 s) stays unwritten and tk_peer_status returns TK_TIMEOUT.  The reference runs on one
 * GPU (src/memory/memory_manager.cpp:15) and has no counterpart. */
typedef struct tk_peer tk_peer;
#define TK_PEER_HANDLE_BYTES 64
int tk_peer_create(int32_t rank, int32_t world, int32_t max_rows, int32_t row_floats, int32_t device,
                   tk_peer** out);                        /* row_floats = dv + 2; world <= 16 */
void tk_peer_destroy(tk_peer* p);
const char* tk_peer_last_error(const tk_peer* p);
int tk_peer_export(tk_peer* p, void* handle_out);         /* TK_PEER_HANDLE_BYTES bytes */
int tk_peer_connect(tk_peer* p, const void* handles);     /* world x TK_PEER_HANDLE_BYTES, indexed by rank */
/* Ranks that live in one process (or a test) connect with the mailbox addresses themselves. */
void* tk_peer_mailbox(const tk_peer* p);
size_t tk_peer_mailbox_bytes(const tk_peer* p);
int tk_peer_connect_ptrs(tk_peer* p, void* const* mailboxes);
int tk_peer_set_wait_limit_ms(tk_peer* p, int32_t ms);
int tk_peer_exchange_combine(tk_peer* p, const float* partial, int32_t n_rows, int32_t dv, void* out,
                             int32_t out_dtype, void* stream);
/* The two halves as launches of their own (send early, combine later; also how ranks that share
 * a GPU must be driven: all sends first, so that no kernel waits for a later launch). */
int tk_peer_send(tk_peer* p, const float* partial, int32_t n_rows, int32_t dv, void* stream);
int tk_peer_recv_combine(tk_peer* p, const float* partial, int32_t n_rows, int32_t dv, void* out,
                         int32_t out_dtype, void* stream);
int tk_peer_status(tk_peer* p, void* stream);
/* Attention of one layer over the tokens of EVERY rank: out [n_seqs][H][v_head_dim] in the handle's io
 * dtype.  Where the step allows it this is ONE launch: the attention kernel's merging CTAs store their
 * rows into the peers' mailboxes, await the peers' rows of their (sequence, kv head) and write the
 * combine.  Otherwise tk_kv_decode_partial followed by the exchange kernel, on the same mailbox cells. */
int tk_kv_decode_exchange(tk_kv* h, int32_t layer, const void* q, tk_peer* peer, void* out, void* stream);

/* update + attention_decode of one layer with HOST buffers (pageable or pinned):
 * copies k, v, q in, runs append and decode, copies out back, and waits for it. */
int tk_kv_append_decode_host(tk_kv* h, int32_t layer, const void* k_host, const void* v_host,
                             const void* q_host, void* out_host, void* stream);

/* Same without the final wait.  Copies run on the handle's own copy streams so that they
 * overlap the kernels of neighbouring calls; before reading out_host the caller calls
 * tk_kv_host_wait(h, stream) and synchronises `stream`.  The host buffers must be pinned and
 * stay untouched until then.  The copy-in starts at the call; the kernel launches of up to four
 * consecutive calls (decode-sized steps) are held back and issued together - by the fourth call,
 * by tk_kv_host_wait, or by any other launching entry point of the handle - so that the launches
 * of neighbouring layers sit next to each other in the stream and overlap. */
int tk_kv_append_decode_host_async(tk_kv* h, int32_t layer, const void* k_host, const void* v_host,
                                   const void* q_host, void* out_host, void* stream);

/* Issues the launches the *_host_async calls still hold back and makes `stream` wait for every
 * device-to-host copy the *_host calls have queued. */
int tk_kv_host_wait(tk_kv* h, void* stream);

/* Timing of the dominant decode kernel on its own stream: after enable(n), each of the next
 * n tk_kv_decode calls brackets its main attention kernel with a CUDA event pair;
 * read() waits for them and returns the summed kernel time and the number of launches.
 * enable(0) turns it off.  (The reference times only with std::chrono around whole
 * phases, src/inference/engine.cpp:179-201.) */
int tk_kv_profile_enable(tk_kv* h, int32_t max_launches);
int tk_kv_profile_read(tk_kv* h, double* total_ms, int64_t* launches);
/* The same, one duration per launch: writes up to `cap` kernel times (milliseconds, in launch
 * order) to ms_out and the number of timed launches to *launches. */
int tk_kv_profile_read_each(tk_kv* h, float* ms_out, int32_t cap, int32_t* launches);

/* Paged decode attention for callers that cannot allocate device memory (a plugin inside a
 * process whose allocator belongs to someone else, a serving loop that has handed all of
 * HBM to its own arena, a caller that wants a step guaranteed not to reach the driver's
 * allocator).  No counterpart in the reference.  No handle, no workspace: the split-KV
 * scratch is one fixed 4 MiB array inside the library image (held by every GPU that loads
 * the library), so the call allocates nothing on the device and is refused — not truncated —
 * beyond n_seqs 256, 4096 (sequence, split-KV chunk, kv head) work items or 4 MiB of
 * partial rows.  All calls on a device share that array: calls whose kernels may overlap
 * race, keep them on one stream.  A device's first call looks the array's address up.  Every
 * call uploads its work list from host memory that lives only until the call returns, so a call
 * made while `stream` is being captured into a graph is refused (TK_INVALID_ARG).
 *   pool        device, one layer: [num_pages][Hkv][2][16][D] in dtype (TK_FP16 / TK_BF16)
 *   page_table  device int32 [n_seqs][max_pages_per_seq]
 *   seq_lens    HOST int32 [n_seqs]
 *   q, out      device [n_seqs][H][D] in dtype */
int tk_paged_decode_static(const void* pool, int32_t dtype, int32_t num_pages,
                           const int32_t* page_table, int32_t max_pages_per_seq,
                           const int32_t* seq_lens, int32_t n_seqs, int32_t num_heads,
                           int32_t num_kv_heads, int32_t head_dim, const void* q, void* out,
                           void* stream);

/* Reads the device status word after draining `stream`: TK_OK, or TK_TIMEOUT when a
 * bounded device-side wait gave up (the word is cleared). */
int tk_kv_device_status(tk_kv* h, void* stream);

/* ---- continuous batching over the paged cache -------------------------------------------
 * Stands for BatchScheduler (src/inference/batch.h:75-140): submit / cancel / one
 * schedule_iteration at a time (src/inference/batch.cpp:103-167), with pages instead of
 * whole-sequence KV slots, chunked prefill and preemption when the pool runs dry.  Host only. */
typedef struct tk_sched tk_sched;
typedef struct tk_sched_config {        /* BatchSchedulerConfig, batch.h:68-73 */
    int32_t max_batch_size;             /* concurrent requests */
    int32_t max_prefill_tokens;         /* prompt tokens appended per iteration, all requests together */
    int32_t reserved[6];
} tk_sched_config;
typedef struct tk_sched_stats {         /* BatchScheduler::Stats, batch.h:99-108 */
    int32_t active_requests, queued_requests, completed_requests, cancelled_requests;
    int64_t total_tokens_generated, total_prompt_tokens, iterations, preemptions;
    float avg_ttft_ms, avg_tps, batch_utilization;
} tk_sched_stats;
int tk_sched_create(tk_kv* kv, const tk_sched_config* cfg, tk_sched** out);      /* BatchScheduler::initialize */
int tk_sched_destroy(tk_sched* s);
int tk_sched_submit(tk_sched* s, int32_t prompt_tokens, int32_t max_output_tokens, int32_t* request_id);
int tk_sched_cancel(tk_sched* s, int32_t request_id);
/* One iteration: retire finished/cancelled (ascending slot), admit FIFO, lay out the step
 * (decoding requests 1 token, prefilling requests their next chunk), tk_kv_step_begin on `stream`
 * (preempting the most recently admitted request while pages are short).  Row i of the step:
 * request, sequence slot, tokens appended, and whether its attention output is sampled from. */
int tk_sched_next(tk_sched* s, int32_t cap, int32_t* req_ids, int32_t* seq_ids, int32_t* n_new, int32_t* samples,
                  int32_t* n_out, void* stream);
/* After sampling: finished[i] != 0 when row i's request produced its last token (EOS). */
int tk_sched_commit(tk_sched* s, int32_t n, const int32_t* finished);
/* state: 0 queued, 1 prefilling, 2 decoding, 3 finished, 4 cancelled (RequestState, batch.h:31-37) */
int tk_sched_request_state(const tk_sched* s, int32_t request_id, int32_t* state, int32_t* seq, int32_t* prefill_pos,
                           int32_t* output_tokens);
/* Sequence slots touched by the last tk_sched_next: which = 0 retired, 1 admitted, 2 preempted. */
int tk_sched_last_events(const tk_sched* s, int32_t which, int32_t cap, int32_t* seqs, int32_t* n_out);
int tk_sched_get_stats(const tk_sched* s, tk_sched_stats* out);

/* Failure-detection self-test.  Every device-side wait in this library is bounded; this launches
 * one warp that waits limit_ms (1..2000) on a barrier nothing completes, so the wait runs out and
 * the kernel returns normally with the status word set: the next tk_kv_device_status reports
 * TK_TIMEOUT and the context stays usable.  (The reference reports failures as bool / log lines
 * only, src/inference/kv_cache.cpp:34-47.) */
int tk_kv_selftest_bounded_wait(tk_kv* h, int32_t limit_ms, void* stream);

/* Test hook for the fail-closed rule: sets the handle's device status word (TK_OK or TK_TIMEOUT) from the
 * host, as a timed-out device wait would.  While the word is set, attention launches on the handle write no
 * output; tk_kv_device_status reports and clears it. */
int tk_kv_selftest_set_status(tk_kv* h, int32_t value, void* stream);
/* Stray-write check (the reference relies on external memory checkers; this is built in): 4 KiB of guard
 * bytes sit behind the pool arena (when the handle allocated it, or an external arena is 4 KiB larger than
 * tk_kv_arena_bytes), the page table, the split-KV workspace and the step metadata.  Drains `stream`,
 * compares them, and returns TK_CUDA_ERROR naming the buffer when any byte changed. */
int tk_kv_check_canaries(tk_kv* h, void* stream);
/* The same for an exchange mailbox (guard bytes behind its last slot). */
int tk_peer_check_canaries(tk_peer* p, void* stream);

/* Number of kernels this library has launched on this handle so far. */
int64_t tk_kv_launch_count(const tk_kv* h);

#ifdef __cplusplus
}
#endif
#endif /* TITAN_KV_H */
