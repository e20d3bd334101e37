// kv_manager.cpp — host-side page manager (see kv_manager.h).  No CUDA.
#include "kv_manager.h"

#include <cstdint>

#include <algorithm>
#include <cstring>

namespace tk {

PageManager::PageManager(int num_pages, int max_seqs, int max_pages_per_seq, int page_size)
    : num_pages_(num_pages), max_seqs_(max_seqs), max_pages_per_seq_(max_pages_per_seq),
      page_size_(page_size) {
    free_stack_.resize(num_pages);
    for (int i = 0; i < num_pages; i++) free_stack_[i] = num_pages - 1 - i;  // pops give 0,1,2,...
    table_.assign((size_t)max_seqs * max_pages_per_seq, -1);
    seq_len_.assign(max_seqs, -1);
    seq_pages_.assign(max_seqs, 0);
    seq_tail_.assign(max_seqs, 0);
    refcount_.assign(num_pages, 0);
}

void PageManager::release_page(int32_t page) {
    if (--refcount_[page] <= 0) { refcount_[page] = 0; free_stack_.push_back(page); }
}

void PageManager::set_entry(int seq, int idx, int32_t value) {
    int32_t flat = seq * max_pages_per_seq_ + idx;
    table_[flat] = value;
    delta_.emplace_back(flat, value);
}

void PageManager::compact_delta() {
    if (delta_.size() < 2) return;
    if (delta_stamp_.size() != table_.size()) delta_stamp_.assign(table_.size(), 0);
    if (++delta_gen_ == 0) { std::fill(delta_stamp_.begin(), delta_stamp_.end(), 0u); delta_gen_ = 1; }
    size_t w = delta_.size();
    for (size_t i = delta_.size(); i-- > 0;) {            // newest first; keep the first sighting
        uint32_t& st = delta_stamp_[delta_[i].first];
        if (st == delta_gen_) continue;
        st = delta_gen_;
        delta_[--w] = delta_[i];
    }
    delta_.erase(delta_.begin(), delta_.begin() + (ptrdiff_t)w);
}

// Lowest free index, like BatchScheduler::allocate_slot (src/inference/batch.cpp:86-96).
int PageManager::seq_alloc() {
    for (int i = 0; i < max_seqs_; i++)
        if (seq_len_[i] < 0) { seq_len_[i] = 0; seq_pages_[i] = 0; seq_tail_[i] = 0; counters.seq_allocs++; return i; }
    return -1;
}

int PageManager::seq_free(int seq) {
    if (!live(seq)) return ST_INVALID_ARG;
    const int32_t* r = row(seq);
    for (int i = 0; i < seq_pages_[seq]; i++) {
        if (r[i] <= -2) cold_stack_.push_back(-2 - r[i]);
        else            release_page(r[i]);
        set_entry(seq, i, -1);
    }
    counters.page_frees += seq_pages_[seq];
    counters.seq_frees++;
    seq_pages_[seq] = 0;
    seq_len_[seq] = -1;
    return ST_OK;
}

int PageManager::reserve(int seq, int n_tokens) {
    if (!live(seq) || n_tokens < 0) return ST_INVALID_ARG;
    int64_t new_len = (int64_t)seq_len_[seq] + n_tokens;
    int64_t need = (new_len + page_size_ - 1) / page_size_;
    if (need > max_pages_per_seq_) return ST_INVALID_ARG;
    int extra = (int)need - seq_pages_[seq];
    if (extra > (int)free_stack_.size()) return ST_OUT_OF_PAGES;
    for (int i = 0; i < extra; i++) {
        int32_t page = free_stack_.back();
        free_stack_.pop_back();
        refcount_[page] = 1;
        set_entry(seq, seq_pages_[seq]++, page);
    }
    counters.page_allocs += extra > 0 ? extra : 0;
    seq_len_[seq] = (int32_t)new_len;
    return ST_OK;
}

int PageManager::truncate(int seq, int new_len) {
    if (!live(seq) || new_len < 0 || new_len > seq_len_[seq]) return ST_INVALID_ARG;
    int keep = (new_len + page_size_ - 1) / page_size_;
    const int32_t* r = row(seq);
    // the new last page would be appended to later: it must not be shared with another sequence
    if (new_len % page_size_ != 0 && keep > 0 && r[keep - 1] >= 0 && refcount_[r[keep - 1]] > 1) return ST_UNSUPPORTED;
    // ... nor live in the host pool: a cold page has no device row a later append could write
    if (new_len % page_size_ != 0 && keep > 0 && r[keep - 1] <= -2) return ST_UNSUPPORTED;
    for (int i = keep; i < seq_pages_[seq]; i++) {
        if (r[i] <= -2) cold_stack_.push_back(-2 - r[i]);
        else            release_page(r[i]);
        set_entry(seq, i, -1);
        counters.page_frees++;
    }
    seq_pages_[seq] = keep;
    seq_len_[seq] = new_len;
    return ST_OK;
}

int PageManager::adopt(int seq, const int32_t* pages, int n_pages, int seq_len) {
    if (!live(seq) || seq_pages_[seq] != 0 || n_pages < 0 || n_pages > max_pages_per_seq_) return ST_INVALID_ARG;
    if (seq_len < 0 || (seq_len + page_size_ - 1) / page_size_ != n_pages) return ST_INVALID_ARG;
    std::vector<uint8_t> want(num_pages_, 0);
    for (int i = 0; i < n_pages; i++) {
        if (pages[i] < 0 || pages[i] >= num_pages_ || want[pages[i]]) return ST_INVALID_ARG;
        want[pages[i]] = 1;
    }
    int found = 0;
    for (int32_t p : free_stack_) found += want[p];
    if (found != n_pages) return ST_INVALID_ARG;                 // some page is not free
    free_stack_.erase(std::remove_if(free_stack_.begin(), free_stack_.end(),
                                     [&](int32_t p) { return want[p] != 0; }),
                      free_stack_.end());
    for (int i = 0; i < n_pages; i++) { set_entry(seq, i, pages[i]); refcount_[pages[i]] = 1; }
    seq_pages_[seq] = n_pages;
    seq_len_[seq] = seq_len;
    counters.page_allocs += n_pages;
    return ST_OK;
}

int PageManager::fork(int parent, int* child_out, int32_t* copy_src, int32_t* copy_dst) {
    if (copy_src) *copy_src = -1;
    if (copy_dst) *copy_dst = -1;
    if (!live(parent) || !child_out) return ST_INVALID_ARG;
    if (cold_enabled()) return ST_UNSUPPORTED;
    const int len = seq_len_[parent], n_pg = seq_pages_[parent];
    const bool partial = len % page_size_ != 0;
    int child = -1;
    for (int i = 0; i < max_seqs_; i++) if (seq_len_[i] < 0) { child = i; break; }
    if (child < 0) return ST_OUT_OF_SEQS;
    if (partial && free_stack_.empty()) return ST_OUT_OF_PAGES;
    seq_len_[child] = len; seq_pages_[child] = n_pg; seq_tail_[child] = 0;
    counters.seq_allocs++;
    for (int i = 0; i < n_pg; i++) {
        const int32_t src = row(parent)[i];
        if (partial && i == n_pg - 1) {
            const int32_t page = free_stack_.back();
            free_stack_.pop_back();
            refcount_[page] = 1;
            set_entry(child, i, page);
            counters.page_allocs++;
            if (copy_src) *copy_src = src;
            if (copy_dst) *copy_dst = page;
        } else {
            set_entry(child, i, src);
            refcount_[src]++;
        }
    }
    *child_out = child;
    return ST_OK;
}

int PageManager::enable_cold(int hot_window, int num_cold_pages) {
    if (hot_window < page_size_ || num_cold_pages <= 0 || cold_enabled()) return ST_INVALID_ARG;
    hot_window_ = hot_window;
    num_cold_pages_ = num_cold_pages;
    cold_stack_.resize(num_cold_pages);
    for (int i = 0; i < num_cold_pages; i++) cold_stack_[i] = num_cold_pages - 1 - i;   // pops give 0,1,2,...
    return ST_OK;
}

int PageManager::set_tail(int seq, int tail) {
    if (!live(seq) || tail < 0) return ST_INVALID_ARG;
    seq_tail_[seq] = tail;
    return ST_OK;
}

int PageManager::evict_cold(int seq, int stable_len, std::vector<Eviction>* moved) {
    if (!live(seq) || !cold_enabled()) return 0;
    const int32_t* r = row(seq);
    int limit = seq_len_[seq] + seq_tail_[seq] - hot_window_;   // tokens below this index are cold ...
    if (limit > stable_len) limit = stable_len;             // ... but never a page this step still writes
    const int n_cold = limit > 0 ? limit / page_size_ : 0;  // pages that lie entirely below it
    int need = 0;
    for (int i = 0; i < n_cold; i++) need += r[i] >= 0;
    if (need > (int)cold_stack_.size()) return -1;
    for (int i = 0; i < n_cold; i++) {
        if (r[i] < 0) continue;
        const int32_t hot = r[i], cold = cold_stack_.back();
        cold_stack_.pop_back();
        release_page(hot);
        set_entry(seq, i, -2 - cold);
        if (cold + 1 > cold_high_water_) cold_high_water_ = cold + 1;
        if (moved) moved->push_back({hot, cold});
    }
    counters.evictions += need;
    return need;
}

int64_t PageManager::slot(int seq, int pos) const {
    if (!live(seq) || pos < 0 || pos >= seq_len_[seq]) return -1;
    const int32_t page = row(seq)[pos / page_size_];
    if (page < 0) return -1;                               // cold pages have no device slot
    return (int64_t)page * page_size_ + pos % page_size_;
}

static uint64_t fnv(uint64_t h, const void* p, size_t n) {
    const uint8_t* b = (const uint8_t*)p;
    for (size_t i = 0; i < n; i++) { h ^= b[i]; h *= 0x100000001B3ull; }
    return h;
}

uint64_t PageManager::digest() const {
    uint64_t h = 0xCBF29CE484222325ull;
    h = fnv(h, seq_len_.data(), sizeof(int32_t) * seq_len_.size());
    h = fnv(h, table_.data(), sizeof(int32_t) * table_.size());
    int32_t top = (int32_t)free_stack_.size();
    h = fnv(h, &top, sizeof(top));
    h = fnv(h, free_stack_.data(), sizeof(int32_t) * free_stack_.size());
    if (cold_enabled()) {
        int32_t ct = (int32_t)cold_stack_.size();
        h = fnv(h, &ct, sizeof(ct));
        h = fnv(h, cold_stack_.data(), sizeof(int32_t) * cold_stack_.size());
    }
    return h;
}

namespace { constexpr int32_t kImageMagic = 0x544B5631; }      // "TKV1"

std::vector<int32_t> PageManager::save() const {
    std::vector<int32_t> im = {kImageMagic, num_pages_, max_seqs_, max_pages_per_seq_, page_size_, hot_window_,
                               num_cold_pages_, cold_high_water_, (int32_t)free_stack_.size(), (int32_t)cold_stack_.size()};
    im.insert(im.end(), seq_len_.begin(), seq_len_.end());
    im.insert(im.end(), seq_pages_.begin(), seq_pages_.end());
    im.insert(im.end(), seq_tail_.begin(), seq_tail_.end());
    im.insert(im.end(), refcount_.begin(), refcount_.end());
    im.insert(im.end(), free_stack_.begin(), free_stack_.end());
    im.insert(im.end(), cold_stack_.begin(), cold_stack_.end());
    for (int s = 0; s < max_seqs_; s++)                       // only the rows in use: live sequences, their pages
        if (seq_len_[s] >= 0) im.insert(im.end(), row(s), row(s) + seq_pages_[s]);
    return im;
}

int PageManager::load(const int32_t* im, size_t n) {
    if (!im || n < 10 || im[0] != kImageMagic) return ST_INVALID_ARG;
    if (im[1] != num_pages_ || im[2] != max_seqs_ || im[3] != max_pages_per_seq_ || im[4] != page_size_ ||
        im[5] != hot_window_ || im[6] != num_cold_pages_) return ST_INVALID_ARG;
    const int n_free = im[8], n_cold = im[9];
    if (n_free < 0 || n_free > num_pages_ || n_cold < 0 || n_cold > num_cold_pages_) return ST_INVALID_ARG;
    size_t at = 10;
    const size_t fixed = at + 3 * (size_t)max_seqs_ + num_pages_ + n_free + n_cold;
    if (n < fixed) return ST_INVALID_ARG;
    const int32_t *len = im + at, *pages = len + max_seqs_, *tail = pages + max_seqs_, *ref = tail + max_seqs_;
    const int32_t *fs = ref + num_pages_, *cs = fs + n_free, *rows = cs + n_cold;
    size_t need = fixed;
    for (int s = 0; s < max_seqs_; s++) {
        if (len[s] < -1 || pages[s] < 0 || pages[s] > max_pages_per_seq_) return ST_INVALID_ARG;
        if (len[s] >= 0 && ((int64_t)len[s] + page_size_ - 1) / page_size_ != pages[s]) return ST_INVALID_ARG;
        if (len[s] >= 0) need += pages[s];
    }
    if (n != need) return ST_INVALID_ARG;
    for (int i = 0; i < n_free; i++) if (fs[i] < 0 || fs[i] >= num_pages_) return ST_INVALID_ARG;
    for (size_t i = fixed; i < need; i++) if (im[i] >= num_pages_ || im[i] < -2 - num_cold_pages_ || im[i] == -1) return ST_INVALID_ARG;
    seq_len_.assign(len, len + max_seqs_);
    seq_pages_.assign(pages, pages + max_seqs_);
    seq_tail_.assign(tail, tail + max_seqs_);
    refcount_.assign(ref, ref + num_pages_);
    free_stack_.assign(fs, fs + n_free);
    cold_stack_.assign(cs, cs + n_cold);
    cold_high_water_ = im[7];
    table_.assign(table_.size(), -1);
    for (int s = 0; s < max_seqs_; s++) {
        if (seq_len_[s] < 0) { seq_pages_[s] = 0; continue; }
        std::copy(rows, rows + seq_pages_[s], table_.begin() + (size_t)s * max_pages_per_seq_);
        rows += seq_pages_[s];
    }
    delta_.clear();
    full_upload_ = true;
    return ST_OK;
}

namespace {
// One stable counting pass of an index permutation by 11 bits of a 32-bit key (LSD radix sort: call it for
// the low digit first).  The step plans sort a few thousand to a few ten thousand items per step; a
// comparison sort of that many took longer than everything else in the plan.
void radix_pass(const std::vector<uint32_t>& key, std::vector<int32_t>& idx, std::vector<int32_t>& tmp, int shift) {
    uint32_t count[2049] = {};
    for (int32_t i : idx) count[((key[(size_t)i] >> shift) & 2047u) + 1]++;
    for (int d = 0; d < 2048; d++) count[d + 1] += count[d];
    tmp.resize(idx.size());
    for (int32_t i : idx) tmp[count[(key[(size_t)i] >> shift) & 2047u]++] = i;
    idx.swap(tmp);
}
}  // namespace

int PageManager::plan_step(int n_seqs, const int32_t* seqs, const int32_t* n_new, int num_kv_heads,
                           bool fp8, int chunk_tokens, int target_items, int max_step_tokens,
                           int max_partial_rows, StepPlan* plan, const int32_t* len_cap, int heads_per_kv,
                           int prefill_rows) {
    if (n_seqs < 0 || (n_seqs > 0 && !seqs) || !plan) return ST_INVALID_ARG;
    const int ps = page_size_;
    if (chunk_tokens < 0 || chunk_tokens % ps != 0) return ST_INVALID_ARG;

    // validate; count pages needed (all or nothing)
    std::vector<uint8_t> seen(max_seqs_, 0);
    int64_t total_new = 0, extra_pages = 0;
    for (int i = 0; i < n_seqs; i++) {
        int s = seqs[i];
        if (!live(s) || seen[s]) return ST_INVALID_ARG;
        seen[s] = 1;
        int add = n_new ? n_new[i] : 0;
        if (add < 0) return ST_INVALID_ARG;
        int64_t new_len = (int64_t)seq_len_[s] + add;
        int64_t need = (new_len + ps - 1) / ps;
        if (need > max_pages_per_seq_) return ST_INVALID_ARG;
        // the partly filled last page receives this step's first rows: it must have a device row
        if (add > 0 && seq_len_[s] % ps != 0 && row(s)[seq_len_[s] / ps] < 0) return ST_UNSUPPORTED;
        extra_pages += need - seq_pages_[s];
        total_new += add;
    }
    if (total_new > max_step_tokens) return ST_INVALID_ARG;
    if (extra_pages > (int64_t)free_stack_.size()) return ST_OUT_OF_PAGES;

    // pick the split-KV chunk before touching state (rows must fit the workspace)
    auto rows_for = [&](int chunk, int64_t* items_out) {
        int64_t rows = 0, items = 0;
        for (int i = 0; i < n_seqs; i++) {
            int64_t len = (int64_t)seq_len_[seqs[i]] + (n_new ? n_new[i] : 0);
            if (len_cap && len_cap[i] < len) len = len_cap[i] < 0 ? 0 : len_cap[i];
            int64_t pool_tokens = fp8 ? (len / ps) * ps : len;
            int64_t r = (pool_tokens + chunk - 1) / chunk + ((fp8 && len > pool_tokens) ? 1 : 0);
            rows += r;
            items += r * num_kv_heads;
        }
        if (items_out) *items_out = items;
        return rows;
    };
    int chunk = chunk_tokens;
    if (chunk == 0) {
        // Measured on B200 (8B head shape, 3 resident CTAs per SM): an item costs a few microseconds
        // beyond its bytes, the CTA that finishes last merges one row per chunk, and a little more than
        // one wave of equal items is the worst schedule.  So: the largest chunk, unless that leaves
        // between 0.9 and 1.5 waves (then the largest chunk of at least 1024 tokens that gives 1.5
        // waves) or fewer than 128 items (then the largest chunk, down to 256 tokens, that gives 128).
        const int64_t slots = std::max<int64_t>(1, (int64_t)target_items * 3 / 8);   // target = 8 per SM, 3 CTAs per SM
        std::vector<int> cands;                         // descending, multiples of the page size
        for (int c : {2048, 1792, 1536, 1280, 1024, 896, 768, 640, 512, 384, 256, 128}) {
            const int r = c / ps * ps;
            if (r > 0 && (cands.empty() || cands.back() != r)) cands.push_back(r);
        }
        auto fits = [&](int c, int64_t* items) { return rows_for(c, items) <= max_partial_rows; };
        int64_t items_max = 0;
        size_t first = cands.size();                    // index of the largest admissible chunk
        for (size_t i = 0; i < cands.size(); i++)
            if (fits(cands[i], &items_max)) { first = i; break; }
        if (first == cands.size()) return ST_INVALID_ARG;
        chunk = cands[first];
        if (items_max * 10 > slots * 9 && items_max * 2 < slots * 3) {
            for (size_t i = first + 1; i < cands.size() && cands[i] >= 1024; i++) {
                int64_t items = 0;
                if (fits(cands[i], &items) && items * 2 >= slots * 3) { chunk = cands[i]; break; }
            }
        } else if (items_max < 128) {
            int64_t items = items_max;
            for (size_t i = first + 1; i < cands.size() && cands[i] >= 256 && items < 128; i++)
                if (fits(cands[i], &items)) chunk = cands[i];
        }
    } else if (rows_for(chunk, nullptr) > max_partial_rows) {
        return ST_INVALID_ARG;
    }

    plan->chunk_tokens = chunk;
    plan->seq.assign(seqs, seqs + n_seqs);
    plan->len.resize(n_seqs);
    plan->chunk_base.assign(n_seqs + 1, 0);
    plan->tok_b.clear(); plan->tok_pos.clear(); plan->tok_dst.clear(); plan->tok_open.clear(); plan->items.clear(); plan->seals.clear();
    plan->evictions.clear();
    plan->new_tok.assign(n_seqs, -1);
    plan->q_base.assign(n_seqs, 0);
    plan->nq.assign(n_seqs, 0);
    plan->nq_max = 0;
    plan->nq_min = n_seqs > 0 ? INT32_MAX : 0;
    plan->one_token_steps = true;
    plan->has_empty_seq = false;

    std::vector<int32_t> item_tokens;
    std::vector<int32_t> old_lens(n_seqs);
    for (int i = 0; i < n_seqs; i++) old_lens[i] = seq_len_[seqs[i]];
    for (int i = 0; i < n_seqs; i++) {
        int s = seqs[i];
        int add = n_new ? n_new[i] : 0;
        int old_len = seq_len_[s];
        int st = reserve(s, add);
        if (st != ST_OK) return st;                     // cannot happen after the checks above
        int len = seq_len_[s];
        const int full_len = len;
        if (len_cap && len_cap[i] < len) len = len_cap[i] < 0 ? 0 : len_cap[i];   // attend to a prefix only
        plan->len[i] = len;
        int tok_base = (int)plan->tok_b.size();
        plan->q_base[i] = tok_base;
        plan->nq[i] = add;
        plan->nq_max = std::max(plan->nq_max, add);
        plan->nq_min = std::min(plan->nq_min, add);
        if (add == 1) plan->new_tok[i] = tok_base;
        if (add > 1) plan->one_token_steps = false;
        if (len == 0) plan->has_empty_seq = true;
        const int sealed_end = (full_len / ps) * ps;    // FP8: rows below it are in sealed pages after this step
        {   // the step's token list: (sequence index, position, destination row) - filled in place, page by page
            const size_t at = plan->tok_b.size();
            plan->tok_b.resize(at + add, i);
            plan->tok_pos.resize(at + add);
            plan->tok_dst.resize(at + add);
            int32_t* pos = plan->tok_pos.data() + at;
            int32_t* dst = plan->tok_dst.data() + at;
            const int32_t* row_s = table_.data() + (size_t)s * max_pages_per_seq_;
            for (int p = old_len; p < full_len;) {
                const int r0 = p % ps, n = std::min(ps - r0, full_len - p);
                const int32_t base = fp8 ? (p >= sealed_end ? s * ps : -1) : row_s[p / ps] * ps;
                for (int r = 0; r < n; r++) {
                    pos[p - old_len + r] = p + r;
                    dst[p - old_len + r] = (fp8 && base < 0) ? -1 : base + r0 + r;
                }
                if (fp8 && base >= 0)
                    for (int r = 0; r < n; r++) plan->tok_open.push_back((int32_t)(at + (p - old_len) + r));
                p += n;
            }
        }
        if (fp8)
            for (int lp = old_len / ps; (lp + 1) * ps <= full_len; lp++)
            {
                const int n_old = std::min(ps, std::max(0, old_len - lp * ps));
                plan->seals.push_back({s, table_[(size_t)s * max_pages_per_seq_ + lp], n_old,
                                       tok_base + lp * ps + n_old - old_len});
            }
        int pool_tokens = fp8 ? (len / ps) * ps : len;
        int n_chunks = (pool_tokens + chunk - 1) / chunk;
        for (int c = 0; c < n_chunks; c++)
            for (int h = 0; h < num_kv_heads; h++) {
                plan->items.push_back({i, c, h, 0});
                item_tokens.push_back(std::min(chunk, pool_tokens - c * chunk));
            }
        int rows = n_chunks;
        if (fp8 && len > pool_tokens) {
            for (int h = 0; h < num_kv_heads; h++) {
                plan->items.push_back({i, n_chunks, h, 1});
                item_tokens.push_back(len - pool_tokens);
            }
            rows++;
        }
        plan->chunk_base[i + 1] = plan->chunk_base[i] + rows;
    }
    // after every reservation of the step: pages that fell out of the hot window go cold
    // (a full host pool moves nothing for that sequence: its pages stay hot and the step still
    // succeeds; the caller sees it in evictions_refused and, later, as ST_OUT_OF_PAGES)
    plan->evictions_refused = 0;
    if (cold_enabled())
        for (int i = 0; i < n_seqs; i++)
            if (evict_cold(seqs[i], old_lens[i], &plan->evictions) < 0) plan->evictions_refused++;
    // biggest items first, so the short tails fill the end of the schedule
    {
        std::vector<uint32_t> key(plan->items.size());       // descending size: a chunk holds at most 2^22 tokens
        std::vector<int32_t> order(key.size()), tmp;
        for (size_t i = 0; i < key.size(); i++) { key[i] = 0x3FFFFFu - (uint32_t)std::min(item_tokens[i], 0x3FFFFF); order[i] = (int32_t)i; }
        radix_pass(key, order, tmp, 0);
        radix_pass(key, order, tmp, 11);
        std::vector<WorkItem> sorted(order.size());
        for (size_t i = 0; i < order.size(); i++) sorted[i] = plan->items[(size_t)order[i]];
        plan->items.swap(sorted);
    }

    // ---- prefill-sized steps: tiles of kPrefillRows rows for the sequences that append many tokens ----
    plan->pf_built = false;
    plan->pf_items.clear(); plan->pf_small_items.clear();
    plan->pf_small_nq_max = 0; plan->pf_partial_rows = 0; plan->pf_groups = 0;
    const int G = heads_per_kv;
    if (!fp8 && !len_cap && G > 0 && G <= kDecodeTileRows && prefill_rows % G == 0 && plan->nq_min >= 1 &&
        (int64_t)plan->nq_max * G > (int64_t)kDecodeTileRows * kDecodeMaxTokenGroups) {
        const int tpt = prefill_rows / G;                      // query tokens per tile
        plan->pf_rows = prefill_rows;
        const int max_ct = kPrefillMaxPages * ps;
        plan->pf_ct.assign(n_seqs, 0); plan->pf_poff.assign(n_seqs, 0); plan->pf_cbase.assign(n_seqs, 0);
        auto is_small = [&](int i) { return plan->nq[i] * G <= kDecodeTileRows; };
        for (int i = 0; i < n_seqs; i++)
            if (is_small(i)) plan->pf_small_nq_max = std::max(plan->pf_small_nq_max, plan->nq[i]);
        // rows of the workspace the decode kernel's share of the step uses; the split regions lie behind them
        const int64_t small_rows = (int64_t)plan->chunk_base[n_seqs] * plan->pf_small_nq_max;
        // split-KV chunk per sequence: about 48 items per sequence where its tiles alone give fewer; halve
        // the number of chunks (shrink) until the split regions fit the workspace
        for (int shrink = 0;; shrink++) {
            int64_t rows = 0;
            for (int i = 0; i < n_seqs; i++) {
                if (is_small(i)) continue;
                const int nq = plan->nq[i], len = plan->len[i];
                const int tiles = (nq + tpt - 1) / tpt;
                int want = (48 + tiles * num_kv_heads - 1) / (tiles * num_kv_heads);
                want = std::max(1, want >> shrink);
                int64_t ct = ((int64_t)len + want - 1) / want;
                ct = (ct + 511) / 512 * 512;
                ct = std::min<int64_t>(std::max<int64_t>(ct, 1024), max_ct);
                plan->pf_ct[i] = (int32_t)ct;
                const int n_chunks = (int)((len + ct - 1) / ct);
                plan->pf_poff[i] = (int32_t)rows;
                if (n_chunks > 1) rows += (int64_t)n_chunks * nq;
            }
            // (past the last shrink every sequence has as few chunks as 32768-token items allow: the caller
            // then finds room for the rows elsewhere)
            if (small_rows + rows <= max_partial_rows || shrink > 8) { plan->pf_partial_rows = (int32_t)std::min<int64_t>(rows, INT32_MAX); break; }
        }
        std::vector<int64_t> weight;
        weight.reserve(plan->pf_items.capacity());
        for (int i = 0; i < n_seqs; i++) {
            if (is_small(i)) continue;
            const int nq = plan->nq[i], len = plan->len[i], ct = plan->pf_ct[i];
            const int tiles = (nq + tpt - 1) / tpt;
            plan->pf_cbase[i] = plan->pf_groups;
            plan->pf_groups += tiles * num_kv_heads;
            for (int t = 0; t < tiles; t++) {
                const int tok_cnt = std::min(nq - t * tpt, tpt);
                const int p_last = len - nq + t * tpt + tok_cnt - 1;
                for (int c = 0; c <= p_last / ct; c++)
                    for (int h = 0; h < num_kv_heads; h++) {
                        plan->pf_items.push_back({i, c, h, t});
                        weight.push_back((int64_t)(std::min(ct, p_last + 1 - c * ct)) * (tok_cnt * G));
                    }
            }
        }
        for (const WorkItem& w : plan->items)
            if (is_small(w.b)) plan->pf_small_items.push_back(w);     // already big-first
        // Launch order: the tiles and chunks of one (sequence, kv head) walk the same K/V pages, so they go out
        // together and the pages stay in L2 (with a plain big-first order every group of the step was in flight at
        // once and each page came from DRAM ~9 times).  Groups by total work, big first, are cut into sets of about
        // 48 MB of K/V; inside a set the items go big first, which keeps the load balance of the plain order when
        // contexts are short.
        std::vector<int32_t> ord(plan->pf_items.size());
        for (size_t i = 0; i < ord.size(); i++) ord[i] = (int32_t)i;
        const size_t n_groups = (size_t)n_seqs * num_kv_heads;
        std::vector<int64_t> group_weight(n_groups, 0);
        std::vector<int32_t> group_items(n_groups, 0), group_set(n_groups, 0), gord;
        auto group_of = [&](int32_t k) { return (size_t)plan->pf_items[k].b * num_kv_heads + plan->pf_items[k].kvh; };
        for (size_t k = 0; k < ord.size(); k++) { group_weight[group_of((int32_t)k)] += weight[k]; group_items[group_of((int32_t)k)]++; }
        for (size_t gi = 0; gi < n_groups; gi++) if (group_items[gi]) gord.push_back((int32_t)gi);
        std::stable_sort(gord.begin(), gord.end(), [&](int32_t a, int32_t b) { return group_weight[a] > group_weight[b]; });
        {
            constexpr int64_t kSetBytes = (int64_t)48 << 20;
            int64_t bytes_in = 0;
            int32_t set = 0;
            for (int32_t gi : gord) {
                const int64_t kv_bytes = (int64_t)plan->len[gi / num_kv_heads] * 512;   // K and V rows of 128 16-bit dims
                if (bytes_in > 0 && bytes_in + kv_bytes > kSetBytes) { set++; bytes_in = 0; }
                group_set[gi] = set;
                bytes_in += kv_bytes;
            }
        }
        {   // by set, inside a set by descending weight (at most 32768 tokens x 128 rows: 22 bits), then the order of
            // generation: three stable passes, least significant first (sets beyond 2047 share the last one)
            std::vector<uint32_t> kw(ord.size()), ks(ord.size());
            std::vector<int32_t> tmp;
            for (size_t k = 0; k < ord.size(); k++) {
                kw[k] = 0x3FFFFFu - (uint32_t)std::min<int64_t>(weight[k], 0x3FFFFF);
                ks[k] = (uint32_t)std::min(group_set[group_of((int32_t)k)], 2047);
            }
            radix_pass(kw, ord, tmp, 0);
            radix_pass(kw, ord, tmp, 11);
            radix_pass(ks, ord, tmp, 0);
        }
        std::vector<WorkItem> pf_sorted(ord.size());
        for (size_t i = 0; i < ord.size(); i++) pf_sorted[i] = plan->pf_items[ord[i]];
        plan->pf_items.swap(pf_sorted);
        plan->pf_built = true;
    }
    return ST_OK;
}

}  // namespace tk
