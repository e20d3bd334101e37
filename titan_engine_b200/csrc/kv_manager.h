// kv_manager.h — host-side page manager of the paged KV cache (no CUDA here).
//
// Stands where the reference keeps its per-request KV bookkeeping: whole-sequence
// slots handed out lowest-index-first (BatchScheduler::allocate_slot/free_slot,
// src/inference/batch.cpp:86-101) and one length counter (KVCache::seq_len,
// src/inference/kv_cache.h:50-51).  The reference has no pages; the page rules are:
//   * free list = LIFO stack of page ids, a fresh pool pops 0,1,2,...
//   * reserve() takes pages one at a time as ceil(len/page_size) grows and
//     changes nothing when the pool cannot cover the request
//   * free() returns a sequence's pages in logical order 0..n-1 (the last
//     logical page is reused first)
// Every change to a page-table entry is also logged as an (index, value) pair so
// the device copy can be patched with one small upload per step.
#pragma once

#include <cstdint>
#include <utility>
#include <vector>

namespace tk {

struct WorkItem {      // one CTA's worth of decode work; mirrors the device int4
    int32_t b;         // index into the step's sequence list
    int32_t chunk;     // split-KV chunk index inside the sequence
    int32_t kvh;       // kv head
    int32_t kind;      // 0 = pool pages, 1 = FP8 open page (16-bit tail)
};

struct SealItem {      // FP8: one logical page completed by this step
    int32_t seq;       // sequence slot (its open page holds the rows that predate the step)
    int32_t page;      // physical page that receives the codes
    int32_t n_old;     // rows [0, n_old) come from the open page, the rest from this step's input
    int32_t tok0;      // index in the step's token list of the token that is row n_old
};

struct Eviction {      // a page that moved from the device pool to the host (cold) pool
    int32_t hot_page;
    int32_t cold_id;
};

struct StepPlan {
    int32_t chunk_tokens = 0;
    std::vector<int32_t> seq;        // [n_seqs] sequence slot ids
    std::vector<int32_t> len;        // [n_seqs] lengths after the step's appends
    std::vector<int32_t> chunk_base; // [n_seqs+1] prefix sum of partial rows per sequence
    std::vector<int32_t> tok_b;      // [n_tokens] index into seq[]
    std::vector<int32_t> tok_pos;    // [n_tokens] position inside the sequence
    std::vector<int32_t> tok_dst;    // [n_tokens] destination row: pool slot, FP8: open-page slot or -1 (sealed)
    std::vector<int32_t> tok_open;   // FP8: the tokens (indices into the lists above) that stay in an open page
    std::vector<int32_t> new_tok;    // [n_seqs] row of the sequence's single new token, or -1
    std::vector<int32_t> q_base;     // [n_seqs] index of the sequence's first new token in the token lists
    std::vector<int32_t> nq;         // [n_seqs] tokens the sequence appends in this step
    int32_t nq_max = 0, nq_min = 0;  // over the step's sequences
    bool one_token_steps = false;    // every sequence appends at most one token (a decode step)
    bool has_empty_seq = false;      // some sequence attends to zero tokens
    std::vector<WorkItem> items;
    std::vector<SealItem> seals;
    std::vector<Eviction> evictions; // pages that went cold in this step (copy out before reuse)
    int32_t evictions_refused = 0;   // sequences whose pages stayed hot because the host pool was full

    // Prefill-sized multi-token steps (16-bit storage, some sequence appending more tokens than the decode
    // kernel's token groups hold).  Sequences whose (tokens x heads per kv head) rows fit one 16-row tile keep
    // the decode kernel (pf_small_items, chunked by chunk_tokens); the others are cut into tiles of kPrefillRows rows
    // and, where a sequence has too few tiles to fill the GPU, into split-KV chunks of pf_ct[b] tokens.
    bool pf_built = false;
    std::vector<WorkItem> pf_items;        // (b, chunk, kvh, tile)
    std::vector<WorkItem> pf_small_items;  // (b, chunk, kvh, 0)
    std::vector<int32_t> pf_ct;            // [n_seqs] split-KV chunk of the sequence in the prefill kernel (tokens)
    std::vector<int32_t> pf_poff;          // [n_seqs] first token row of the sequence's split region (rows of H x (Dv+2) floats)
    std::vector<int32_t> pf_cbase;         // [n_seqs] first arrival counter of the sequence: + kvh * tiles + tile
    int32_t pf_small_nq_max = 0;           // most tokens a sequence of pf_small_items appends
    int32_t pf_partial_rows = 0;           // token rows the split regions take
    int32_t pf_groups = 0;                 // (sequence, kv head, tile) groups = arrival counters in use
    int32_t pf_rows = 0;                   // (token, head) rows per tile the lists were laid out for
};

// Geometry of the prefill kernel's work list, shared by the planner and the kernel.
constexpr int kPrefillRows = 64;           // (token, head) rows per tile of the mma.sync prefill kernel
constexpr int kPrefillRowsTc = 128;        // ... of the tcgen05 prefill kernel
constexpr int kPrefillMaxPages = 2048;     // pages per item: a split-KV chunk holds at most 32768 tokens
constexpr int kDecodeTileRows = 16;        // rows of the decode kernel's tile
constexpr int kDecodeMaxTokenGroups = 8;   // token groups per sequence the decode kernel's multi-token form takes

class PageManager {
public:
    PageManager(int num_pages, int max_seqs, int max_pages_per_seq, int page_size);

    int  seq_alloc();                              // lowest free slot or -1
    int  seq_free(int seq);                        // status
    int  reserve(int seq, int n_tokens);           // status
    int  truncate(int seq, int new_len);           // status
    int  adopt(int seq, const int32_t* pages, int n_pages, int seq_len);  // status
    // Prefix sharing: a new sequence (lowest free slot) holding the same tokens as `parent`.  Full
    // pages are shared and reference-counted; a partly filled last page gets a fresh page whose
    // contents the caller must copy (*copy_src -> *copy_dst, -1 when there is none).  On
    // ST_OUT_OF_SEQS / ST_OUT_OF_PAGES nothing changes.  Not available with a cold tier.
    int  fork(int parent, int* child, int32_t* copy_src, int32_t* copy_dst);
    int  refcount(int page) const { return page >= 0 && page < num_pages_ ? refcount_[page] : 0; }
    // Cold tier: a page is cold iff its last token index < seq_len - hot_window.  Cold pages
    // live in a host pool with its own LIFO id stack; the table holds -2 - cold_id for them.
    // The idiom is the reference's expert cache (evict, count, keep a host copy:
    // src/memory/memory_manager.cpp:266-278) with the eviction order fixed by the window.
    int  enable_cold(int hot_window, int num_cold_pages);                  // status
    int  evict_cold(int seq, int stable_len, std::vector<Eviction>* moved); // pages moved, -1 = cold pool full;
                                                                           // stable_len = length before the current step
    // A sequence split over several caches: `tail` tokens of it follow this cache's last token,
    // so the window is measured from seq_len + tail.
    int  set_tail(int seq, int tail);
    bool cold_enabled() const { return hot_window_ > 0; }
    int  num_cold_used() const { return num_cold_pages_ - (int)cold_stack_.size(); }
    int  cold_high_water() const { return cold_high_water_; }
    bool live(int seq) const { return seq >= 0 && seq < max_seqs_ && seq_len_[seq] >= 0; }
    int  seq_len(int seq) const { return live(seq) ? seq_len_[seq] : -1; }
    int  seq_pages(int seq) const { return live(seq) ? seq_pages_[seq] : -1; }
    int  num_free_pages() const { return (int)free_stack_.size(); }
    int64_t slot(int seq, int pos) const;
    uint64_t digest() const;

    const int32_t* page_table() const { return table_.data(); }
    const int32_t* row(int seq) const { return table_.data() + (size_t)seq * max_pages_per_seq_; }
    int num_pages() const { return num_pages_; }
    int max_seqs() const { return max_seqs_; }
    int max_pages_per_seq() const { return max_pages_per_seq_; }
    int page_size() const { return page_size_; }

    // (flat index into the table, new value) pairs since the last take_delta()
    std::vector<std::pair<int32_t, int32_t>>& delta() { return delta_; }
    // Keep only the last write to each index: the device applies the patches in
    // parallel, so an index must not appear twice (free then re-map of a slot's row).
    void compact_delta();

    // Reserve n_new[i] tokens for seqs[i] (all or nothing), then lay out the step:
    // token list in call order then position, FP8 seal list, split-KV work list.
    // chunk_tokens == 0 picks a chunk so that about `target_items` items exist.
    // len_cap (optional, 16-bit storage only) limits the attended prefix of each sequence.
    // heads_per_kv > 0 (16-bit storage): also lay out the prefill work lists when a sequence appends
    // more tokens than the decode kernel's token groups hold, in tiles of prefill_rows (token, head) rows.
    int plan_step(int n_seqs, const int32_t* seqs, const int32_t* n_new, int num_kv_heads,
                  bool fp8, int chunk_tokens, int target_items, int max_step_tokens,
                  int max_partial_rows, StepPlan* plan, const int32_t* len_cap = nullptr, int heads_per_kv = 0,
                  int prefill_rows = kPrefillRows);

    // Snapshot of the whole bookkeeping state (lengths, page tables, free lists, reference counts, cold ids)
    // as a flat int32 image, and its restore into a manager of the same geometry: a failing churn run can be
    // saved at step N and replayed from there.  load() marks every table entry as changed.
    std::vector<int32_t> save() const;
    int load(const int32_t* image, size_t n);              // status; ST_INVALID_ARG on a foreign or damaged image
    bool take_full_upload() { const bool f = full_upload_; full_upload_ = false; return f; }

    struct Counters { int64_t page_allocs = 0, page_frees = 0, seq_allocs = 0, seq_frees = 0, evictions = 0; } counters;

private:
    void set_entry(int seq, int idx, int32_t value);
    void release_page(int32_t page);      // free stack once no sequence names it
    std::vector<int32_t> refcount_;
    int num_pages_, max_seqs_, max_pages_per_seq_, page_size_;
    std::vector<int32_t> free_stack_;   // back() is the next page handed out
    std::vector<int32_t> table_;        // [max_seqs][max_pages_per_seq], -1 = unmapped
    std::vector<int32_t> seq_len_;      // -1 = slot free
    std::vector<int32_t> seq_pages_;
    std::vector<int32_t> seq_tail_;
    int hot_window_ = 0, num_cold_pages_ = 0, cold_high_water_ = 0;
    std::vector<int32_t> cold_stack_;   // back() is the next cold id handed out
    std::vector<std::pair<int32_t, int32_t>> delta_;
    std::vector<uint32_t> delta_stamp_;  // per table index: generation of the last compaction that saw it
    bool full_upload_ = false;           // the device copy of the table must be rewritten whole (after load())
    uint32_t delta_gen_ = 0;
};

// status codes shared with include/titan_kv.h
enum { ST_OK = 0, ST_INVALID_ARG = 1, ST_OUT_OF_PAGES = 2, ST_CUDA_ERROR = 3, ST_TIMEOUT = 4,
       ST_OUT_OF_SEQS = 5, ST_UNSUPPORTED = 6 };

}  // namespace tk
