// sched_abi.cpp — C ABI of the continuous-batching scheduler (declared in include/titan_kv.h).
#include "../../include/titan_kv.h"

#include "kv_scheduler.h"

#include <new>

struct tk_sched {
    tk::PagedScheduler impl;
    std::vector<tk::StepRow> rows;
    tk_sched(tk_kv* kv, const tk::SchedConfig& c) : impl(kv, c) {}
};

extern "C" {

int tk_sched_create(tk_kv* kv, const tk_sched_config* cfg, tk_sched** out) {
    if (!kv || !out) return TK_INVALID_ARG;
    tk::SchedConfig c;
    if (cfg) {
        if (cfg->max_batch_size <= 0 || cfg->max_prefill_tokens <= 0) return TK_INVALID_ARG;
        c.max_batch_size = cfg->max_batch_size;
        c.max_prefill_tokens = cfg->max_prefill_tokens;
    }
    tk_kv_config kc;
    if (tk_kv_get_config(kv, &kc) != TK_OK) return TK_INVALID_ARG;
    // a step appends at most max_prefill_tokens prompt tokens plus one token per decoding request
    if (c.max_prefill_tokens + c.max_batch_size > kc.max_step_tokens) return TK_INVALID_ARG;
    *out = new (std::nothrow) tk_sched(kv, c);
    return *out ? TK_OK : TK_INVALID_ARG;
}

int tk_sched_destroy(tk_sched* s) {
    if (!s) return TK_INVALID_ARG;
    delete s;
    return TK_OK;
}

int tk_sched_submit(tk_sched* s, int32_t prompt_tokens, int32_t max_output_tokens, int32_t* request_id) {
    if (!s || !request_id) return TK_INVALID_ARG;
    const int id = s->impl.submit(prompt_tokens, max_output_tokens);
    if (id < 0) return TK_INVALID_ARG;
    *request_id = id;
    return TK_OK;
}

int tk_sched_cancel(tk_sched* s, int32_t request_id) {
    if (!s) return TK_INVALID_ARG;
    return s->impl.cancel(request_id) ? TK_OK : TK_INVALID_ARG;
}

int tk_sched_next(tk_sched* s, int32_t cap, int32_t* req_ids, int32_t* seq_ids, int32_t* n_new, int32_t* samples,
                  int32_t* n_out, void* stream) {
    if (!s || !n_out) return TK_INVALID_ARG;
    const int st = s->impl.next(&s->rows, stream);
    if (st != TK_OK) { *n_out = 0; return st; }
    const int n = (int)s->rows.size();
    *n_out = n;
    if (n > cap) return TK_INVALID_ARG;
    for (int i = 0; i < n; i++) {
        if (req_ids) req_ids[i] = s->rows[i].req_id;
        if (seq_ids) seq_ids[i] = s->rows[i].seq;
        if (n_new) n_new[i] = s->rows[i].n_new;
        if (samples) samples[i] = s->rows[i].samples;
    }
    return TK_OK;
}

int tk_sched_commit(tk_sched* s, int32_t n, const int32_t* finished) {
    if (!s) return TK_INVALID_ARG;
    return s->impl.commit(n, finished);
}

int tk_sched_request_state(const tk_sched* s, int32_t request_id, int32_t* state, int32_t* seq, int32_t* prefill_pos,
                           int32_t* output_tokens) {
    if (!s) return TK_INVALID_ARG;
    const tk::Request* r = s->impl.find(request_id);
    if (!r) return TK_INVALID_ARG;
    if (state) *state = (int32_t)r->state;
    if (seq) *seq = r->seq;
    if (prefill_pos) *prefill_pos = r->prefill_pos;
    if (output_tokens) *output_tokens = r->output_tokens + r->generated_prior;
    return TK_OK;
}

int tk_sched_last_events(const tk_sched* s, int32_t which, int32_t cap, int32_t* seqs, int32_t* n_out) {
    if (!s || !n_out || which < 0 || which > 2) return TK_INVALID_ARG;
    const std::vector<int32_t>& v = which == 0 ? s->impl.last_retired() : which == 1 ? s->impl.last_admitted() : s->impl.last_preempted();
    *n_out = (int32_t)v.size();
    if ((int)v.size() > cap) return TK_INVALID_ARG;
    for (size_t i = 0; i < v.size(); i++) seqs[i] = v[i];
    return TK_OK;
}

int tk_sched_get_stats(const tk_sched* s, tk_sched_stats* out) {
    if (!s || !out) return TK_INVALID_ARG;
    const tk::SchedStats st = s->impl.stats();
    out->active_requests = st.active_requests; out->queued_requests = st.queued_requests;
    out->completed_requests = st.completed_requests; out->cancelled_requests = st.cancelled_requests;
    out->total_tokens_generated = st.total_tokens_generated; out->total_prompt_tokens = st.total_prompt_tokens;
    out->iterations = st.iterations; out->preemptions = st.preemptions;
    out->avg_ttft_ms = st.avg_ttft_ms; out->avg_tps = st.avg_tps; out->batch_utilization = st.batch_utilization;
    return TK_OK;
}

}  // extern "C"
