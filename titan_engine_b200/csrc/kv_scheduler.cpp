// kv_scheduler.cpp — continuous batching over the paged KV cache (see kv_scheduler.h).
#include "kv_scheduler.h"

#include "../../include/titan_kv.h"

#include <algorithm>

namespace tk {

int PagedScheduler::submit(int32_t prompt_tokens, int32_t max_output_tokens) {
    tk_kv_config cfg;
    if (tk_kv_get_config(kv_, &cfg) != TK_OK) return -1;
    const int64_t capacity = (int64_t)cfg.max_pages_per_seq * cfg.page_size;
    if (prompt_tokens <= 0 || max_output_tokens <= 0 || (int64_t)prompt_tokens + max_output_tokens > capacity) return -1;
    Request r;
    r.id = next_id_++;
    r.prompt_tokens = prompt_tokens;
    r.max_output_tokens = max_output_tokens;
    r.submit_time = std::chrono::steady_clock::now();
    pending_.push_back(r);
    return r.id;
}

bool PagedScheduler::cancel(int32_t id) {
    for (auto it = pending_.begin(); it != pending_.end(); ++it)
        if (it->id == id) {
            it->state = ReqState::CANCELLED;
            it->finish_time = std::chrono::steady_clock::now();
            done_.push_back(*it);
            pending_.erase(it);
            return true;
        }
    for (auto& r : active_)
        if (r.id == id && r.state != ReqState::FINISHED) { r.state = ReqState::CANCELLED; return true; }   // retired by next()
    return false;
}

// Finished and cancelled requests give their pages back, ascending sequence slot.
void PagedScheduler::retire() {
    std::vector<Request*> out;
    for (auto& r : active_)
        if (r.state == ReqState::FINISHED || r.state == ReqState::CANCELLED) out.push_back(&r);
    std::sort(out.begin(), out.end(), [](const Request* a, const Request* b) { return a->seq < b->seq; });
    for (Request* r : out) {
        tk_kv_seq_free(kv_, r->seq);
        retired_.push_back(r->seq);
        r->finish_time = std::chrono::steady_clock::now();
        done_.push_back(*r);
    }
    active_.erase(std::remove_if(active_.begin(), active_.end(),
                                 [](const Request& r) { return r.state == ReqState::FINISHED || r.state == ReqState::CANCELLED; }),
                  active_.end());
}

// FIFO admission while a batch slot, a sequence slot and pages for the first chunk are there.
void PagedScheduler::admit() {
    tk_kv_config cfg;
    tk_kv_get_config(kv_, &cfg);
    int64_t pages_spoken_for = 0;
    while (!pending_.empty() && (int)active_.size() < cfg_.max_batch_size) {
        Request& head = pending_.front();
        const int first_chunk = std::min(head.prompt_tokens, cfg_.max_prefill_tokens);
        const int64_t need = (first_chunk + cfg.page_size - 1) / cfg.page_size;
        // keep one page per running request in hand so that admitting never starves decoding
        if (pages_spoken_for + need + (int64_t)active_.size() > tk_kv_num_free_pages(kv_)) break;
        int32_t seq = -1;
        if (tk_kv_seq_alloc(kv_, &seq) != TK_OK) break;       // no sequence slot: leave it queued (batch.cpp:112-116)
        Request r = head;
        pending_.pop_front();
        r.seq = seq;
        r.state = ReqState::PREFILLING;
        r.admit_order = admit_counter_++;
        pages_spoken_for += need;
        admitted_.push_back(seq);
        active_.push_back(r);
    }
}

// Out of pages: the most recently admitted request loses its pages and goes back to the head of
// the queue; its prompt (and the tokens it had generated) are recomputed when it is readmitted.
void PagedScheduler::preempt_youngest() {
    auto it = std::max_element(active_.begin(), active_.end(),
                               [](const Request& a, const Request& b) { return a.admit_order < b.admit_order; });
    Request r = *it;
    active_.erase(it);
    tk_kv_seq_free(kv_, r.seq);
    preempted_.push_back(r.seq);
    r.prompt_tokens += r.output_tokens;       // what it had generated becomes part of what must be prefilled again
    r.max_output_tokens -= r.output_tokens;
    r.generated_prior += r.output_tokens;
    r.output_tokens = 0;
    r.prefill_pos = 0;
    r.seq = -1;
    r.state = ReqState::QUEUED;
    r.preemptions++;
    preemptions_++;
    pending_.push_front(r);
}

int PagedScheduler::next(std::vector<StepRow>* rows, void* stream) {
    retired_.clear(); admitted_.clear(); preempted_.clear();
    rows_.clear();
    retire();
    admit();
    for (;;) {
        std::vector<Request*> order;
        for (auto& r : active_) order.push_back(&r);
        std::sort(order.begin(), order.end(), [](const Request* a, const Request* b) { return a->seq < b->seq; });
        rows_.clear();
        int budget = cfg_.max_prefill_tokens;
        for (Request* r : order) {
            if (r->state == ReqState::DECODING) {
                rows_.push_back({r->id, r->seq, 1, 1});
            } else if (r->state == ReqState::PREFILLING) {
                const int n = std::min(r->prompt_tokens - r->prefill_pos, budget);
                if (n <= 0) continue;                         // no budget left this iteration
                budget -= n;
                rows_.push_back({r->id, r->seq, n, r->prefill_pos + n == r->prompt_tokens ? 1 : 0});
            }
        }
        std::vector<int32_t> seqs, n_new;
        for (const StepRow& row : rows_) { seqs.push_back(row.seq); n_new.push_back(row.n_new); }
        const int st = tk_kv_step_begin(kv_, (int32_t)rows_.size(), seqs.data(), n_new.data(), stream);
        if (st == TK_OUT_OF_PAGES && active_.size() > 1) { preempt_youngest(); continue; }
        if (st != TK_OK) { rows_.clear(); return st; }
        break;
    }
    for (const StepRow& row : rows_)
        for (auto& r : active_)
            if (r.id == row.req_id && r.state == ReqState::PREFILLING) r.prefill_pos += row.n_new;
    iterations_++;
    batch_rows_total_ += (int64_t)rows_.size();
    if (rows) *rows = rows_;
    return TK_OK;
}

int PagedScheduler::commit(int n, const int32_t* finished) {
    if (n != (int)rows_.size() || (n > 0 && !finished)) return TK_INVALID_ARG;
    const auto now = std::chrono::steady_clock::now();
    for (int i = 0; i < n; i++) {
        if (!rows_[i].samples) continue;
        for (auto& r : active_) {
            if (r.id != rows_[i].req_id || r.state == ReqState::CANCELLED) continue;
            if (r.state == ReqState::PREFILLING) { r.state = ReqState::DECODING; r.first_token_time = now; }   // batch.cpp:171-176
            r.output_tokens++;
            if (finished[i] || r.output_tokens >= r.max_output_tokens) r.state = ReqState::FINISHED;
        }
    }
    rows_.clear();
    return TK_OK;
}

SchedStats PagedScheduler::stats() const {
    SchedStats s;
    s.active_requests = (int32_t)active_.size();
    s.queued_requests = (int32_t)pending_.size();
    s.iterations = iterations_;
    s.preemptions = preemptions_;
    double ttft = 0, tps = 0;
    int n_ttft = 0;
    for (const Request& r : done_) {
        if (r.state == ReqState::CANCELLED) { s.cancelled_requests++; continue; }
        s.completed_requests++;
        s.total_tokens_generated += r.output_tokens + r.generated_prior;
        s.total_prompt_tokens += r.prompt_tokens - r.generated_prior;
        ttft += std::chrono::duration<double, std::milli>(r.first_token_time - r.submit_time).count();
        const double secs = std::chrono::duration<double>(r.finish_time - r.first_token_time).count();
        if (secs > 0) tps += (r.output_tokens + r.generated_prior) / secs;
        n_ttft++;
    }
    for (const Request& r : active_) s.total_tokens_generated += r.output_tokens + r.generated_prior;
    if (n_ttft) { s.avg_ttft_ms = (float)(ttft / n_ttft); s.avg_tps = (float)(tps / n_ttft); }
    if (iterations_ && cfg_.max_batch_size)
        s.batch_utilization = (float)((double)batch_rows_total_ / iterations_ / cfg_.max_batch_size);
    return s;
}

const Request* PagedScheduler::find(int32_t id) const {
    for (const Request& r : active_) if (r.id == id) return &r;
    for (const Request& r : pending_) if (r.id == id) return &r;
    for (const Request& r : done_) if (r.id == id) return &r;
    return nullptr;
}

}  // namespace tk
