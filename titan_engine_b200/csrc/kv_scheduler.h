// kv_scheduler.h — continuous batching over the paged KV cache (host only).
//
// Stands where the reference has BatchScheduler (src/inference/batch.h:75-140,
// src/inference/batch.cpp:86-167): a request queue, admit-while-capacity, retire-when-done.
// The reference gives every request a whole KVCache of max_context_len/kv_cache_slots positions
// (batch.cpp:39-50) and never wires those slots into the model; here a request is a sequence of
// the paged cache, capacity is counted in pages, prompts are prefilled in chunks through the same
// append path as decode tokens, and a request can be preempted (pages freed, recomputed later)
// when the pool runs dry.
//
// One iteration = schedule_iteration (batch.cpp:103-167) in this order:
//   1. retire FINISHED / CANCELLED requests, ascending sequence slot  (free_slot, :97-101)
//   2. admit pending requests FIFO while batch slots, sequence slots and pages allow (:107-121)
//   3. lay out the step: decoding requests append 1 token, prefilling requests the next chunk of
//      their prompt (shared token budget), in ascending sequence-slot order
//   4. reserve the pages (all or nothing); on shortage preempt the most recently admitted
//      request and retry
// The model's forward pass is the caller's: it gets the rows of the step, runs
// tk_kv_append / tk_kv_decode per layer, samples, and reports which requests ended.
#pragma once

#include <chrono>
#include <cstdint>
#include <deque>
#include <vector>

struct tk_kv;

namespace tk {

enum class ReqState : int32_t { QUEUED = 0, PREFILLING = 1, DECODING = 2, FINISHED = 3, CANCELLED = 4 };  // batch.h:31-37

struct Request {
    int32_t id = -1;
    ReqState state = ReqState::QUEUED;
    int32_t prompt_tokens = 0;
    int32_t prefill_pos = 0;        // prompt tokens already in the cache
    int32_t output_tokens = 0;      // generated since the last (re)admission
    int32_t generated_prior = 0;    // generated before preemptions (recomputed as prompt afterwards)
    int32_t max_output_tokens = 0;
    int32_t seq = -1;               // sequence slot of the paged cache (kv_slot, batch.h:53)
    int64_t admit_order = -1;
    int32_t preemptions = 0;
    std::chrono::steady_clock::time_point submit_time, first_token_time, finish_time;
};

struct StepRow {
    int32_t req_id, seq, n_new;
    int32_t samples;                // 1 if this row's attention output leads to a sampled token
};

struct SchedConfig {
    int32_t max_batch_size = 8;         // batch.h:69
    int32_t max_prefill_tokens = 2048;  // prompt tokens appended per iteration, all requests together
};

struct SchedStats {                     // batch.h:99-108
    int32_t active_requests = 0, queued_requests = 0, completed_requests = 0, cancelled_requests = 0;
    int64_t total_tokens_generated = 0, total_prompt_tokens = 0, iterations = 0, preemptions = 0;
    float avg_ttft_ms = 0, avg_tps = 0, batch_utilization = 0;
};

class PagedScheduler {
public:
    PagedScheduler(tk_kv* kv, const SchedConfig& cfg) : kv_(kv), cfg_(cfg) {}

    int submit(int32_t prompt_tokens, int32_t max_output_tokens);      // request id, or -1
    bool cancel(int32_t request_id);
    // Lays out and begins the next step on `stream`; rows come back in step order.
    int next(std::vector<StepRow>* rows, void* stream);                // tk_status
    // finished[i] != 0: the request of row i (of the last next()) produced its final token.
    int commit(int n, const int32_t* finished);
    SchedStats stats() const;
    const Request* find(int32_t request_id) const;
    // sequence slots retired / admitted by the last next(), in the order it happened
    const std::vector<int32_t>& last_retired() const { return retired_; }
    const std::vector<int32_t>& last_admitted() const { return admitted_; }
    const std::vector<int32_t>& last_preempted() const { return preempted_; }

private:
    void retire();
    void admit();
    void preempt_youngest();
    tk_kv* kv_;
    SchedConfig cfg_;
    std::deque<Request> pending_;
    std::vector<Request> active_;
    std::vector<Request> done_;         // finished or cancelled, kept for lookup and stats
    std::vector<StepRow> rows_;
    std::vector<int32_t> retired_, admitted_, preempted_;
    int32_t next_id_ = 0;
    int64_t admit_counter_ = 0, iterations_ = 0, batch_rows_total_ = 0, preemptions_ = 0;
};

}  // namespace tk
