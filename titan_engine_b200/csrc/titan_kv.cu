// titan_kv.cu — the C ABI (include/titan_kv.h): handle, device memory, per-step
// metadata upload and kernel launches.  Host bookkeeping lives in kv_manager.cpp.
#include "../../include/titan_kv.h"

#include "kv_manager.h"
#include "tk_kernels.cuh"
#include "tk_peer.cuh"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

namespace {

constexpr int kRing = 4;                 // pinned staging buffers in rotation
constexpr int kHostSetsMax = 8;          // device staging sets of the host-buffer entry points
constexpr int kMaxDelta = 1 << 16;       // page-table patches per upload; more -> full table copy
constexpr int TK_DEVICE_NONE = -2;       // bookkeeping only: no device memory, compute calls fail
// Guard bytes behind every buffer that kernels write at host-computed rows (the pool arena, the split-KV
// workspace, the step metadata, the page table): filled with kCanaryByte at creation and compared by
// tk_kv_check_canaries, which stands in for a memory checker on stray writes past a buffer's end.
constexpr size_t kCanaryBytes = 4096;
constexpr int kCanaryByte = 0xA5;

std::string g_create_error;

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct ArenaLayout {
    size_t pool_layer, scales_layer, open_layer;   // bytes per layer
    size_t pool_off, scales_off, open_off, total;
};

ArenaLayout arena_layout(const tk_kv_config& c) {
    ArenaLayout a{};
    const size_t esize = c.dtype == TK_FP8_E4M3 ? 1 : 2;
    const size_t tile = (size_t)c.num_kv_heads * c.page_size * (c.head_dim + c.v_head_dim);   // K rows + V rows
    a.pool_layer = align_up((size_t)c.num_pages * tile * esize, 1024);
    if (c.dtype == TK_FP8_E4M3) {
        a.scales_layer = align_up((size_t)c.num_pages * c.num_kv_heads * 2 * sizeof(float), 1024);
        a.open_layer = align_up((size_t)c.max_seqs * tile * 2, 1024);
    }
    a.pool_off = 0;
    a.scales_off = a.pool_off + a.pool_layer * c.num_layers;
    a.open_off = a.scales_off + a.scales_layer * c.num_layers;
    a.total = a.open_off + a.open_layer * c.num_layers;
    return a;
}

const char* validate(const tk_kv_config& c) {
    if (c.num_layers <= 0 || c.num_heads <= 0 || c.num_kv_heads <= 0) return "layers/heads must be positive";
    if (c.num_heads % c.num_kv_heads != 0) return "num_heads must be a multiple of num_kv_heads";
    const int G = c.num_heads / c.num_kv_heads;
    if (G != 1 && G != 2 && G != 4 && G != 8 && G != 16) return "heads per kv head must be 1, 2, 4, 8 or 16";
    const bool mla = c.head_dim == 192 && c.v_head_dim == 128;      // K = nope + rope dims, V = nope dims
    if (!mla && ((c.head_dim != 64 && c.head_dim != 128) || c.v_head_dim != c.head_dim))
        return "head_dim must be 64 or 128 (v_head_dim equal), or 192 with v_head_dim 128 (MLA)";
    if (mla && c.dtype == TK_FP8_E4M3) return "the MLA shape needs 16-bit storage";
    if (c.page_size <= 0 || c.page_size % 8 != 0) return "page_size must be a positive multiple of 8";
    if (c.dtype != TK_FP16 && c.dtype != TK_BF16 && c.dtype != TK_FP8_E4M3) return "dtype must be FP16, BF16 or FP8_E4M3";
    if (c.io_dtype != TK_FP16 && c.io_dtype != TK_BF16) return "io_dtype must be FP16 or BF16";
    if (c.dtype != TK_FP8_E4M3 && c.io_dtype != c.dtype) return "io_dtype must equal dtype for 16-bit storage";
    if (c.num_pages <= 0 || c.max_seqs <= 0 || c.max_pages_per_seq <= 0) return "num_pages/max_seqs/max_pages_per_seq must be positive";
    if ((int64_t)c.max_seqs * c.max_pages_per_seq > (int64_t)1 << 30) return "page table too large";
    if ((int64_t)c.num_pages * c.page_size >= (int64_t)1 << 31 || (int64_t)c.max_seqs * c.page_size >= (int64_t)1 << 31)
        return "num_pages * page_size must stay below 2^31 (row indices are 32-bit)";
    if (c.max_step_tokens <= 0) return "max_step_tokens must be positive";
    if (c.chunk_tokens < 0 || c.chunk_tokens % c.page_size != 0) return "chunk_tokens must be a multiple of page_size";
    if (c.decode_impl < TK_DECODE_AUTO || c.decode_impl > TK_DECODE_MMA) return "bad decode_impl";
    if (c.merge_impl != TK_MERGE_IN_KERNEL && c.merge_impl != TK_MERGE_SEPARATE) return "bad merge_impl";
    if (c.launch_overlap != TK_OVERLAP_AUTO && c.launch_overlap != TK_OVERLAP_OFF) return "bad launch_overlap";
    if (c.prefill_impl != TK_PREFILL_AUTO && c.prefill_impl != TK_PREFILL_MMA_SYNC) return "bad prefill_impl";
    if (c.hot_window < 0 || c.cold_pages < 0) return "hot_window and cold_pages must not be negative";
    if (c.hot_window > 0) {
        if (c.hot_window < c.page_size) return "hot_window must cover at least one page";
        if (c.cold_pages == 0) return "hot_window needs cold_pages > 0";
        if (c.dtype == TK_FP8_E4M3) return "the cold tier needs 16-bit storage";
    }
    return nullptr;
}

}  // namespace

struct tk_kv {
    tk_kv_config cfg{};
    tk::Geometry geo{};
    tk::PageManager* mgr = nullptr;
    bool host_only = false;
    int device = 0, num_sms = 148;
    bool use_mma = false;
    bool separate_combine = false;           // cfg.merge_impl == TK_MERGE_SEPARATE: combine launch instead of the in-kernel merge

    uint8_t* arena = nullptr;
    bool owns_arena = false;
    ArenaLayout lay{};

    int32_t* d_table = nullptr;
    float* d_partials = nullptr;
    int max_partial_rows = 0, max_items = 0, max_seals = 0;
    int* d_status = nullptr;
    int* d_counters = nullptr;           // [8 token groups][max_seqs * Hkv] arrival counters of the in-kernel merge
    int* d_pf_counters = nullptr;        // prefill kernel: one per (sequence, kv head, tile) group
    int max_pf_groups = 0, max_pf_items = 0;
    // programmatic dependent launch of back-to-back attention kernels: the launch count right after the last
    // attention launch, its layer and stream (another launch of this library in between breaks the chain)
    int64_t chain_launches = -1;
    int chain_layer = -1;
    cudaStream_t chain_stream = nullptr;
    tk::PrefillDev pf_dev{};             // device view of the step's prefill work list
    tk::StepDev small_dev{};             // ... and of the decode-kernel share of such a step

    size_t step_bytes = 0;
    uint8_t* d_step = nullptr;
    uint8_t* h_step[kRing] = {};
    cudaEvent_t ev[kRing] = {};
    bool ev_pending[kRing] = {};
    int ring_pos = 0;

    // staging for the *_host entry point
    void* d_q = nullptr;                 // FP32 callers: q narrowed to the io type
    void *d_rq = nullptr, *d_rk = nullptr;   // rotated q / k when RoPE cannot ride inside the attention kernel
    float2* d_rope_tab = nullptr;        // [max_seqs][D/2] (cos, sin) of each sequence's newest position
    int64_t rope_tab_step = -1;          // step the table was filled for, with which parameters
    float rope_tab_theta = 0, rope_tab_scaling = 0;
    // the *_host entry points: staging sets in rotation, so that the copies of one layer overlap the
    // kernel of another on the copy engines (copy-in stream, caller's stream, copy-out stream); the
    // asynchronous form launches its kernels in groups (see append_decode_host_impl)
    void *hs_k[kHostSetsMax] = {}, *hs_v[kHostSetsMax] = {}, *hs_q[kHostSetsMax] = {}, *hs_out[kHostSetsMax] = {};
    cudaStream_t st_in = nullptr, st_out = nullptr;
    cudaEvent_t ev_in[kHostSetsMax] = {}, ev_free[kHostSetsMax] = {}, ev_group = nullptr, ev_out_all = nullptr;
    uint64_t host_calls = 0;
    int host_calls_in_step = 0;          // groups start small so that a step's first kernel does not wait for four layers' copies
    int host_sets = 2, host_group = 1;   // sets in rotation; calls whose kernels are launched back to back
    struct HostPending { int layer, set; bool kv, q; void* out_host; size_t o_bytes; };
    std::vector<HostPending> host_pending;
    cudaStream_t host_pending_stream = nullptr;
    bool host_flushing = false;

    std::vector<CUtensorMap> maps;       // one per layer (MMA path); MLA shape: the K-row view
    std::vector<CUtensorMap> maps_v;     // MLA shape: the V-row view
    std::vector<CUtensorMap> maps16;     // boxes of 16 rows (the K or V rows of a page): tcgen05 prefill kernel
    bool prefill_tc = false;             // prefill chunks go to the tcgen05 kernel (128-row tiles)
    float* d_xpartial = nullptr;         // this rank's merged partial rows for tk_kv_decode_exchange
    float* d_multi_partials = nullptr;   // split-KV rows of multi-token steps that outgrow d_partials
    size_t multi_partials_floats = 0;
    bool mla_mma = false;

    // cold tier (hot_window > 0): pages older than the window live in pinned host memory and are
    // staged back, one layer ahead of use, into a two-slot device ring indexed by cold id
    uint8_t* h_cold = nullptr;           // pinned [L][cold_pages][page_bytes]
    uint8_t* d_stage[2] = {};            // device [cold_pages][page_bytes]
    size_t page_bytes = 0;
    cudaStream_t st_pf = nullptr, st_ev = nullptr;
    cudaEvent_t ev_pf[2] = {}, ev_used[2] = {}, ev_user = nullptr, ev_evict = nullptr;
    int staged_layer[2] = {-1, -1};
    CUtensorMap stage_maps[2];

    tk::StepPlan plan;
    tk::StepDev dev{};
    bool have_step = false;
    int n_pool_items = 0;                // items of kind 0 come first

    // optional timing of the dominant decode kernel: one event pair per launch
    bool profiling = false;
    std::vector<cudaEvent_t> prof_ev;    // start/stop pairs
    size_t prof_used = 0;

    // guards the page manager: allocator calls may come from another thread than the stepping one
    // (the reference's pools are mutex-guarded the same way: src/memory/vram_pool.cpp:47)
    std::mutex mgr_mu;

    tk_kv_stats stats{};
    int64_t launches = 0;
    std::string err;

    struct Canary { const char* name; uint8_t* at; };
    std::vector<Canary> canaries;

    tk::LayerPtrs layer(int l) const {
        tk::LayerPtrs p{};
        p.pool = arena + lay.pool_off + lay.pool_layer * l;
        p.scales = lay.scales_layer ? (float*)(arena + lay.scales_off + lay.scales_layer * l) : nullptr;
        p.open_pages = lay.open_layer ? (void*)(arena + lay.open_off + lay.open_layer * l) : nullptr;
        return p;
    }
};

extern "C" {
static int host_flush(tk_kv* h);       // launches what the host-buffer calls hold back (defined with them)
}

namespace {

int fail(tk_kv* h, int status, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (h) h->err = buf; else g_create_error = buf;
    return status;
}

#define TK_CUDA(h, call)                                                                         \
    do {                                                                                         \
        cudaError_t e_ = (call);                                                                 \
        if (e_ != cudaSuccess)                                                                   \
            return fail(h, TK_CUDA_ERROR, "%s failed: %s", #call, cudaGetErrorString(e_));       \
    } while (0)

void release(tk_kv* h) {
    if (!h) return;
    if (!h->host_only) {
        cudaSetDevice(h->device);
        if (h->owns_arena && h->arena) cudaFree(h->arena);
        if (h->d_table) cudaFree(h->d_table);
        if (h->d_partials) cudaFree(h->d_partials);
        if (h->d_xpartial) cudaFree(h->d_xpartial);
        if (h->d_multi_partials) cudaFree(h->d_multi_partials);
        if (h->d_status) cudaFree(h->d_status);
        if (h->d_counters) cudaFree(h->d_counters);
        if (h->d_pf_counters) cudaFree(h->d_pf_counters);
        if (h->d_step) cudaFree(h->d_step);
        if (h->d_q) cudaFree(h->d_q);
        if (h->d_rq) cudaFree(h->d_rq);
        if (h->d_rope_tab) cudaFree(h->d_rope_tab);
        if (h->d_rk) cudaFree(h->d_rk);
        for (int i = 0; i < kHostSetsMax; i++) {
            if (h->hs_k[i]) cudaFree(h->hs_k[i]);
            if (h->hs_v[i]) cudaFree(h->hs_v[i]);
            if (h->hs_q[i]) cudaFree(h->hs_q[i]);
            if (h->hs_out[i]) cudaFree(h->hs_out[i]);
            if (h->ev_in[i]) cudaEventDestroy(h->ev_in[i]);
            if (h->ev_free[i]) cudaEventDestroy(h->ev_free[i]);
        }
        if (h->ev_group) cudaEventDestroy(h->ev_group);
        if (h->ev_out_all) cudaEventDestroy(h->ev_out_all);
        if (h->st_in) cudaStreamDestroy(h->st_in);
        if (h->st_out) cudaStreamDestroy(h->st_out);
        for (int i = 0; i < kRing; i++) {
            if (h->h_step[i]) cudaFreeHost(h->h_step[i]);
            if (h->ev[i]) cudaEventDestroy(h->ev[i]);
        }
        for (cudaEvent_t e : h->prof_ev) cudaEventDestroy(e);
        if (h->h_cold) cudaFreeHost(h->h_cold);
        for (int i = 0; i < 2; i++) {
            if (h->d_stage[i]) cudaFree(h->d_stage[i]);
            if (h->ev_pf[i]) cudaEventDestroy(h->ev_pf[i]);
            if (h->ev_used[i]) cudaEventDestroy(h->ev_used[i]);
        }
        if (h->ev_user) cudaEventDestroy(h->ev_user);
        if (h->ev_evict) cudaEventDestroy(h->ev_evict);
        if (h->st_pf) cudaStreamDestroy(h->st_pf);
        if (h->st_ev) cudaStreamDestroy(h->st_ev);
    }
    delete h->mgr;
    delete h;
}

int create_impl(const tk_kv_config* cfg_in, void* arena, size_t arena_bytes, bool external, tk_kv** out) {
    if (!cfg_in || !out) return fail(nullptr, TK_INVALID_ARG, "null argument");
    *out = nullptr;
    tk_kv_config c = *cfg_in;
    if (c.io_dtype == 0) c.io_dtype = c.dtype == TK_FP8_E4M3 ? TK_BF16 : c.dtype;
    if (c.max_step_tokens == 0) c.max_step_tokens = c.max_seqs;
    if (c.v_head_dim == 0) c.v_head_dim = c.head_dim;
    if (const char* why = validate(c)) return fail(nullptr, TK_INVALID_ARG, "config: %s", why);

    tk_kv* h = new (std::nothrow) tk_kv();
    if (!h) return fail(nullptr, TK_INVALID_ARG, "out of host memory");
    h->cfg = c;
    h->geo = tk::Geometry{c.num_heads, c.num_kv_heads, c.head_dim, c.page_size, c.dtype, c.io_dtype,
                          c.num_pages, c.max_seqs, c.max_pages_per_seq, c.v_head_dim};
    h->mgr = new tk::PageManager(c.num_pages, c.max_seqs, c.max_pages_per_seq, c.page_size);
    h->separate_combine = c.merge_impl == TK_MERGE_SEPARATE;
    h->lay = arena_layout(c);
    h->host_only = c.device == TK_DEVICE_NONE;
    h->page_bytes = (size_t)c.num_kv_heads * c.page_size * (c.head_dim + c.v_head_dim) * (c.dtype == TK_FP8_E4M3 ? 1 : 2);
    if (c.hot_window > 0) h->mgr->enable_cold(c.hot_window, c.cold_pages);
    h->stats.pages_total = c.num_pages;

    const int min_chunk = c.chunk_tokens ? c.chunk_tokens : 128;
    int64_t rows = ((int64_t)c.num_pages * c.page_size + min_chunk - 1) / min_chunk + 2 * (int64_t)c.max_seqs;
    if (rows > (1 << 24)) rows = 1 << 24;
    h->max_partial_rows = (int)rows;
    h->max_items = h->max_partial_rows * c.num_kv_heads;
    h->max_seals = c.max_step_tokens / c.page_size + c.max_seqs;
    {   // prefill work list: tiles of 64 rows per (sequence, kv head), times the split-KV chunks a tile may see
        const int G = c.num_heads / c.num_kv_heads;
        const int64_t tiles = (int64_t)c.max_step_tokens * G / tk::kPrefillRows + c.max_seqs;      // the smaller tile: the upper bound
        const int64_t long_chunks = ((int64_t)c.max_pages_per_seq + tk::kPrefillMaxPages - 1) / tk::kPrefillMaxPages;
        h->max_pf_groups = (int)std::min<int64_t>(tiles * c.num_kv_heads, 1 << 24);
        h->max_pf_items = (int)std::min<int64_t>(tiles * c.num_kv_heads * long_chunks + 128 * (int64_t)c.max_seqs, 1 << 24);
    }

    // one buffer holds every per-step array; sections are 16-byte aligned
    size_t ints = 9 * (size_t)c.max_seqs + 4 + 32 + 4 * (size_t)c.max_step_tokens + 16 +
                  8 * (size_t)h->max_items + 12 * (size_t)h->max_pf_items + 4 * (size_t)h->max_seals +
                  2 * (size_t)kMaxDelta + 32;
    h->step_bytes = align_up(ints * 4, 256);

    if (h->host_only) { *out = h; return TK_OK; }

    if (c.device >= 0) h->device = c.device;
    else if (cudaGetDevice(&h->device) != cudaSuccess) { release(h); return fail(nullptr, TK_CUDA_ERROR, "no CUDA device"); }
#define CREATE_CUDA(call)                                                                        \
    do {                                                                                         \
        cudaError_t e_ = (call);                                                                 \
        if (e_ != cudaSuccess) {                                                                 \
            release(h);                                                                          \
            return fail(nullptr, TK_CUDA_ERROR, "%s failed: %s", #call, cudaGetErrorString(e_)); \
        }                                                                                        \
    } while (0)
    CREATE_CUDA(cudaSetDevice(h->device));
    cudaDeviceProp prop;
    CREATE_CUDA(cudaGetDeviceProperties(&prop, h->device));
    h->num_sms = prop.multiProcessorCount;
    if (prop.major != 10) {
        release(h);
        return fail(nullptr, TK_UNSUPPORTED, "built for sm_100a only; device is sm_%d%d", prop.major, prop.minor);
    }
    if (external) {
        if (!arena || arena_bytes < h->lay.total || ((uintptr_t)arena & 1023)) {
            release(h);
            return fail(nullptr, TK_INVALID_ARG, "external arena must be 1024-byte aligned and >= %zu bytes", h->lay.total);
        }
        h->arena = (uint8_t*)arena;
        // a caller that hands over kCanaryBytes more than the arena needs gets guard bytes there too
        if (arena_bytes >= h->lay.total + kCanaryBytes) h->canaries.push_back({"pool arena", h->arena + h->lay.total});
    } else {
        CREATE_CUDA(cudaMalloc((void**)&h->arena, h->lay.total + kCanaryBytes));
        h->owns_arena = true;
        h->canaries.push_back({"pool arena", h->arena + h->lay.total});
    }
    CREATE_CUDA(cudaMemset(h->arena, 0, h->lay.total));     // like KVCache::initialize, kv_cache.cpp:49-50
    const size_t table_bytes = (size_t)c.max_seqs * c.max_pages_per_seq * sizeof(int32_t);
    CREATE_CUDA(cudaMalloc((void**)&h->d_table, table_bytes + kCanaryBytes));
    CREATE_CUDA(cudaMemset(h->d_table, 0xFF, table_bytes));
    h->canaries.push_back({"page table", (uint8_t*)h->d_table + table_bytes});
    const size_t partial_bytes = (size_t)h->max_partial_rows * c.num_heads * (c.v_head_dim + 2) * sizeof(float);
    CREATE_CUDA(cudaMalloc((void**)&h->d_partials, partial_bytes + kCanaryBytes));
    h->canaries.push_back({"split-KV workspace", (uint8_t*)h->d_partials + partial_bytes});
    CREATE_CUDA(cudaMalloc((void**)&h->d_status, 256));
    CREATE_CUDA(cudaMemset(h->d_status, 0, 256));
    CREATE_CUDA(cudaMalloc((void**)&h->d_counters, sizeof(int) * 8 * (size_t)c.max_seqs * c.num_kv_heads));
    CREATE_CUDA(cudaMemset(h->d_counters, 0, sizeof(int) * 8 * (size_t)c.max_seqs * c.num_kv_heads));
    CREATE_CUDA(cudaMalloc((void**)&h->d_pf_counters, sizeof(int) * (size_t)h->max_pf_groups));
    CREATE_CUDA(cudaMemset(h->d_pf_counters, 0, sizeof(int) * (size_t)h->max_pf_groups));
    CREATE_CUDA(cudaMalloc((void**)&h->d_step, h->step_bytes + kCanaryBytes));
    h->canaries.push_back({"step metadata", h->d_step + h->step_bytes});
    for (const auto& cn : h->canaries) CREATE_CUDA(cudaMemset(cn.at, kCanaryByte, kCanaryBytes));
    for (int i = 0; i < kRing; i++) {
        CREATE_CUDA(cudaHostAlloc((void**)&h->h_step[i], h->step_bytes, cudaHostAllocDefault));
        CREATE_CUDA(cudaEventCreateWithFlags(&h->ev[i], cudaEventDisableTiming));
    }
    const size_t kv_bytes = (size_t)c.max_step_tokens * c.num_kv_heads * c.head_dim * 2;   // sized for K rows (>= V rows)
    const size_t q_bytes = (size_t)c.max_seqs * c.num_heads * c.head_dim * 2;              // q rows (>= out rows)
    CREATE_CUDA(cudaMalloc(&h->d_q, q_bytes));
    CREATE_CUDA(cudaMalloc(&h->d_rq, q_bytes));
    CREATE_CUDA(cudaMalloc((void**)&h->d_rope_tab, sizeof(float2) * (size_t)c.max_seqs * (c.head_dim / 2)));
    CREATE_CUDA(cudaMalloc(&h->d_rk, kv_bytes));
    // decode-sized steps: 8 sets, kernels launched up to four calls at a time; prefill-sized steps keep two sets
    h->host_group = 2 * (kv_bytes + q_bytes) * kHostSetsMax <= ((size_t)64 << 20) ? kHostSetsMax / 2 : 1;
    h->host_sets = 2 * h->host_group;
    for (int i = 0; i < h->host_sets; i++) {
        CREATE_CUDA(cudaMalloc(&h->hs_k[i], kv_bytes));
        CREATE_CUDA(cudaMalloc(&h->hs_v[i], kv_bytes));
        CREATE_CUDA(cudaMalloc(&h->hs_q[i], q_bytes));
        CREATE_CUDA(cudaMalloc(&h->hs_out[i], q_bytes));
        CREATE_CUDA(cudaEventCreateWithFlags(&h->ev_in[i], cudaEventDisableTiming));
        CREATE_CUDA(cudaEventCreateWithFlags(&h->ev_free[i], cudaEventDisableTiming));
    }
    CREATE_CUDA(cudaEventCreateWithFlags(&h->ev_group, cudaEventDisableTiming));
    CREATE_CUDA(cudaEventCreateWithFlags(&h->ev_out_all, cudaEventDisableTiming));
    CREATE_CUDA(cudaStreamCreateWithFlags(&h->st_in, cudaStreamNonBlocking));
    CREATE_CUDA(cudaStreamCreateWithFlags(&h->st_out, cudaStreamNonBlocking));

    // MLA shape: tensor-core kernel of its own; cold pages stay on the generic kernel
    h->mla_mma = tk::decode_mma_mla_supported(h->geo) && c.hot_window == 0;
    const bool mma_ok = tk::decode_mma_supported(h->geo) || h->mla_mma;
    if (c.decode_impl == TK_DECODE_MMA && !mma_ok) {
        release(h);
        return fail(nullptr, TK_UNSUPPORTED, "decode_impl=MMA needs page_size 16 and head_dim 64/128 (128 for FP8), or the "
                                             "192/128 shape with 16-bit storage, groups of <= 8 heads and no cold tier");
    }
    h->use_mma = mma_ok && c.decode_impl != TK_DECODE_SIMT;
    h->mla_mma = h->mla_mma && h->use_mma;
    if (h->use_mma) {
        h->maps.resize(c.num_layers);
        if (h->mla_mma) h->maps_v.resize(c.num_layers);
        for (int l = 0; l < c.num_layers; l++) {
            if (h->mla_mma) CREATE_CUDA(tk::make_mla_tensor_maps(h->geo, h->layer(l).pool, &h->maps[l], &h->maps_v[l]));
            else CREATE_CUDA(tk::make_pool_tensor_map(h->geo, h->layer(l).pool, &h->maps[l]));
        }
        h->prefill_tc = !h->mla_mma && c.prefill_impl != TK_PREFILL_MMA_SYNC && c.hot_window == 0 && tk::prefill_tc_supported(h->geo);
        if (h->prefill_tc) {
            h->maps16.resize(c.num_layers);
            for (int l = 0; l < c.num_layers; l++)
                CREATE_CUDA(tk::make_pool_tensor_map(h->geo, h->layer(l).pool, &h->maps16[l], 16));
        }
    }
    if (c.hot_window > 0) {
        const size_t layer_bytes = (size_t)c.cold_pages * h->page_bytes;
        CREATE_CUDA(cudaHostAlloc((void**)&h->h_cold, layer_bytes * c.num_layers, cudaHostAllocDefault));
        tk::Geometry cold_geo = h->geo;
        cold_geo.num_pages = c.cold_pages;
        for (int i = 0; i < 2; i++) {
            CREATE_CUDA(cudaMalloc((void**)&h->d_stage[i], layer_bytes));
            CREATE_CUDA(cudaMemset(h->d_stage[i], 0, layer_bytes));
            CREATE_CUDA(cudaEventCreateWithFlags(&h->ev_pf[i], cudaEventDisableTiming));
            CREATE_CUDA(cudaEventCreateWithFlags(&h->ev_used[i], cudaEventDisableTiming));
            if (h->use_mma) CREATE_CUDA(tk::make_pool_tensor_map(cold_geo, h->d_stage[i], &h->stage_maps[i]));
        }
        CREATE_CUDA(cudaEventCreateWithFlags(&h->ev_user, cudaEventDisableTiming));
        CREATE_CUDA(cudaEventCreateWithFlags(&h->ev_evict, cudaEventDisableTiming));
        CREATE_CUDA(cudaStreamCreateWithFlags(&h->st_pf, cudaStreamNonBlocking));
        CREATE_CUDA(cudaStreamCreateWithFlags(&h->st_ev, cudaStreamNonBlocking));
    }
    CREATE_CUDA(cudaDeviceSynchronize());
#undef CREATE_CUDA
    *out = h;
    return TK_OK;
}

// device encoding of a host page-table entry: cold pages (-2 - id on the host) carry kColdBit
inline int32_t dev_entry(int32_t v) { return v <= -2 ? (tk::kColdBit | (-2 - v)) : v; }

// Copy pages that just went cold, for every layer, device pool -> pinned host pool.  Runs on the
// eviction stream after the caller's stream has finished with the pages; the caller's stream
// (whose later appends may reuse them) and the prefetch stream then wait for the copies.
int run_evictions(tk_kv* h, const std::vector<tk::Eviction>& ev, cudaStream_t s) {
    if (ev.empty()) return TK_OK;
    TK_CUDA(h, cudaEventRecord(h->ev_user, s));
    TK_CUDA(h, cudaStreamWaitEvent(h->st_ev, h->ev_user, 0));
    const size_t pb = h->page_bytes, cold_layer = (size_t)h->cfg.cold_pages * pb;
    for (size_t i = 0; i < ev.size();) {
        size_t j = i + 1;                                   // runs with consecutive ids on both sides: one copy
        while (j < ev.size() && ev[j].hot_page == ev[j - 1].hot_page + 1 && ev[j].cold_id == ev[j - 1].cold_id + 1) j++;
        for (int l = 0; l < h->cfg.num_layers; l++)
            TK_CUDA(h, cudaMemcpyAsync(h->h_cold + cold_layer * l + (size_t)ev[i].cold_id * pb,
                                       (const uint8_t*)h->layer(l).pool + (size_t)ev[i].hot_page * pb, (j - i) * pb,
                                       cudaMemcpyDeviceToHost, h->st_ev));
        i = j;
    }
    TK_CUDA(h, cudaEventRecord(h->ev_evict, h->st_ev));
    TK_CUDA(h, cudaStreamWaitEvent(s, h->ev_evict, 0));
    TK_CUDA(h, cudaStreamWaitEvent(h->st_pf, h->ev_evict, 0));
    h->stats.bytes_d2h += (int64_t)ev.size() * (int64_t)pb * h->cfg.num_layers;
    return TK_OK;
}

// Stage layer `layer`'s cold pages into ring slot layer&1 on the prefetch stream.
int prefetch_layer(tk_kv* h, int layer, bool ahead) {
    const int n = h->mgr->cold_high_water();
    if (n == 0 || layer < 0 || layer >= h->cfg.num_layers) return TK_OK;
    const int slot = layer & 1;
    if (h->staged_layer[slot] == layer) return TK_OK;
    const size_t bytes = (size_t)n * h->page_bytes;
    TK_CUDA(h, cudaStreamWaitEvent(h->st_pf, h->ev_used[slot], 0));     // the kernel that last read this slot
    TK_CUDA(h, cudaMemcpyAsync(h->d_stage[slot], h->h_cold + (size_t)h->cfg.cold_pages * h->page_bytes * layer, bytes,
                               cudaMemcpyHostToDevice, h->st_pf));
    TK_CUDA(h, cudaEventRecord(h->ev_pf[slot], h->st_pf));
    h->staged_layer[slot] = layer;
    (ahead ? h->stats.prefetch_hits : h->stats.prefetch_misses) += n;
    h->stats.bytes_h2d += (int64_t)bytes;
    return TK_OK;
}

struct Sections {       // offsets (in int32 units) of the arrays inside a step buffer
    size_t seq, len, chunk_base, new_tok, q_base, nq, tok_b, tok_pos, tok_dst, tok_open, items, seals, delta,
           pf_ct, pf_poff, pf_cbase, pf_items, pf_info, pf_small, end;
};
Sections sections(int n_seqs, int n_tokens, int n_open, int n_items, int n_seals, int n_delta, int n_pf, int n_pf_small) {
    auto a4 = [](size_t x) { return (x + 3) / 4 * 4; };
    Sections s{};
    size_t o = 0;
    s.seq = o;        o = a4(o + n_seqs);
    s.len = o;        o = a4(o + n_seqs);
    s.chunk_base = o; o = a4(o + n_seqs + 1);
    s.new_tok = o;    o = a4(o + n_seqs);
    s.q_base = o;     o = a4(o + n_seqs);
    s.nq = o;         o = a4(o + n_seqs);
    s.tok_b = o;      o = a4(o + n_tokens);
    s.tok_pos = o;    o = a4(o + n_tokens);
    s.tok_dst = o;    o = a4(o + n_tokens);
    s.tok_open = o;   o = a4(o + n_open);
    s.items = o;      o = a4(o + 4 * (size_t)n_items);
    s.seals = o;      o = a4(o + 4 * (size_t)n_seals);
    s.delta = o;      o = a4(o + 2 * (size_t)n_delta);
    if (n_pf || n_pf_small) {
        s.pf_ct = o;    o = a4(o + n_seqs);
        s.pf_poff = o;  o = a4(o + n_seqs);
        s.pf_cbase = o; o = a4(o + n_seqs);
        s.pf_items = o; o = a4(o + 4 * (size_t)n_pf);
        s.pf_info = o;  o = a4(o + 8 * (size_t)n_pf);
        s.pf_small = o; o = a4(o + 4 * (size_t)n_pf_small);
    }
    s.end = o;
    return s;
}

}  // namespace

extern "C" {

const char* tk_status_str(int s) {
    switch (s) {
        case TK_OK: return "ok";
        case TK_INVALID_ARG: return "invalid argument";
        case TK_OUT_OF_PAGES: return "out of pages";
        case TK_CUDA_ERROR: return "CUDA error";
        case TK_TIMEOUT: return "device wait timed out";
        case TK_OUT_OF_SEQS: return "out of sequence slots";
        case TK_UNSUPPORTED: return "unsupported";
        default: return "unknown status";
    }
}

const char* tk_kv_last_error(const tk_kv* h) { return h ? h->err.c_str() : g_create_error.c_str(); }

void tk_kv_config_default(tk_kv_config* c) {
    if (!c) return;
    memset(c, 0, sizeof(*c));
    c->page_size = 16;
    c->dtype = TK_BF16;
    c->device = -1;
}

size_t tk_kv_arena_bytes(const tk_kv_config* cfg) {
    if (!cfg) return 0;
    tk_kv_config c = *cfg;
    if (c.io_dtype == 0) c.io_dtype = c.dtype == TK_FP8_E4M3 ? TK_BF16 : c.dtype;
    if (c.max_step_tokens == 0) c.max_step_tokens = c.max_seqs;
    if (c.v_head_dim == 0) c.v_head_dim = c.head_dim;
    if (validate(c)) return 0;
    return arena_layout(c).total;
}

int tk_kv_create(const tk_kv_config* cfg, tk_kv** out) { return create_impl(cfg, nullptr, 0, false, out); }
int tk_kv_create_external(const tk_kv_config* cfg, void* arena, size_t bytes, tk_kv** out) {
    return create_impl(cfg, arena, bytes, true, out);
}
int tk_kv_destroy(tk_kv* h) {
    if (!h) return TK_INVALID_ARG;
    if (!h->host_only) { cudaSetDevice(h->device); cudaDeviceSynchronize(); }
    release(h);
    return TK_OK;
}
int tk_kv_get_config(const tk_kv* h, tk_kv_config* out) {
    if (!h || !out) return TK_INVALID_ARG;
    *out = h->cfg;
    return TK_OK;
}
size_t tk_kv_memory_bytes(const tk_kv* h) { return h ? h->lay.total : 0; }

int tk_kv_layer_ptrs(const tk_kv* h, int layer, void** pool, float** scales, void** open_pages) {
    if (!h || layer < 0 || layer >= h->cfg.num_layers || h->host_only) return TK_INVALID_ARG;
    tk::LayerPtrs p = h->layer(layer);
    if (pool) *pool = p.pool;
    if (scales) *scales = p.scales;
    if (open_pages) *open_pages = p.open_pages;
    return TK_OK;
}

// ---- sequences and pages -------------------------------------------------------------
int tk_kv_seq_alloc(tk_kv* h, int32_t* seq_out) {
    if (!h || !seq_out) return TK_INVALID_ARG;
    std::lock_guard<std::mutex> lock(h->mgr_mu);
    int s = h->mgr->seq_alloc();
    if (s < 0) return fail(h, TK_OUT_OF_SEQS, "all %d sequence slots are in use", h->cfg.max_seqs);
    *seq_out = s;
    return TK_OK;
}
int tk_kv_seq_free(tk_kv* h, int32_t seq) {
    if (!h) return TK_INVALID_ARG;
    std::lock_guard<std::mutex> lock(h->mgr_mu);
    int st = h->mgr->seq_free(seq);
    return st == TK_OK ? TK_OK : fail(h, st, "seq_free(%d): sequence is not live", seq);
}
int tk_kv_reserve(tk_kv* h, int32_t seq, int32_t n) {
    if (!h) return TK_INVALID_ARG;
    std::lock_guard<std::mutex> lock(h->mgr_mu);
    int st = h->mgr->reserve(seq, n);
    return st == TK_OK ? TK_OK : fail(h, st, "reserve(%d, %d): %s", seq, n, tk_status_str(st));
}
int tk_kv_truncate(tk_kv* h, int32_t seq, int32_t new_len) {
    if (!h) return TK_INVALID_ARG;
    std::lock_guard<std::mutex> lock(h->mgr_mu);
    if (h->cfg.dtype == TK_FP8_E4M3 && h->mgr->live(seq) && new_len % h->cfg.page_size != 0 &&
        new_len / h->cfg.page_size < h->mgr->seq_len(seq) / h->cfg.page_size)
        return fail(h, TK_UNSUPPORTED, "FP8: cannot truncate into a sealed page (length must stay page-aligned there)");
    int st = h->mgr->truncate(seq, new_len);
    return st == TK_OK ? TK_OK : fail(h, st, "truncate(%d, %d): %s", seq, new_len, tk_status_str(st));
}
int tk_kv_seq_adopt(tk_kv* h, int32_t seq, const int32_t* pages, int32_t n_pages, int32_t seq_len) {
    if (!h || (n_pages > 0 && !pages)) return TK_INVALID_ARG;
    std::lock_guard<std::mutex> lock(h->mgr_mu);
    if (h->cfg.dtype == TK_FP8_E4M3 && seq_len % h->cfg.page_size != 0)
        return fail(h, TK_UNSUPPORTED, "FP8: adopted length must be page-aligned (no open page to adopt)");
    int st = h->mgr->adopt(seq, pages, n_pages, seq_len);
    return st == TK_OK ? TK_OK : fail(h, st, "seq_adopt(%d): pages must be distinct, in range and free", seq);
}
int tk_kv_seq_fork(tk_kv* h, int32_t parent, int32_t* child_out, void* stream) {
    if (!h || !child_out) return TK_INVALID_ARG;
    std::lock_guard<std::mutex> lock(h->mgr_mu);
    int child = -1;
    int32_t src = -1, dst = -1;
    const int st = h->mgr->fork(parent, &child, &src, &dst);
    if (st != TK_OK) return fail(h, st, "seq_fork(%d): %s", parent, tk_status_str(st));
    *child_out = child;
    if (h->host_only || dst < 0) return TK_OK;
    // the partly filled last page is private: copy it for every layer (FP8: it is the open page)
    cudaError_t e;
    if (h->cfg.dtype == TK_FP8_E4M3) {
        const size_t open_tile = h->page_bytes * 2;       // 16-bit rows
        e = tk::launch_copy_layers(h->arena + h->lay.open_off + (size_t)parent * open_tile, h->lay.open_layer,
                                   h->arena + h->lay.open_off + (size_t)child * open_tile, h->lay.open_layer, open_tile,
                                   h->cfg.num_layers, (cudaStream_t)stream);
    } else {
        e = tk::launch_copy_layers(h->arena + h->lay.pool_off + (size_t)src * h->page_bytes, h->lay.pool_layer,
                                   h->arena + h->lay.pool_off + (size_t)dst * h->page_bytes, h->lay.pool_layer,
                                   h->page_bytes, h->cfg.num_layers, (cudaStream_t)stream);
    }
    h->launches++;
    return e == cudaSuccess ? TK_OK : fail(h, TK_CUDA_ERROR, "seq_fork copy: %s", cudaGetErrorString(e));
}
int tk_kv_seq_set_tail(tk_kv* h, int32_t seq, int32_t tail_tokens) {
    if (!h) return TK_INVALID_ARG;
    std::lock_guard<std::mutex> lock(h->mgr_mu);
    int st = h->mgr->set_tail(seq, tail_tokens);
    return st == TK_OK ? TK_OK : fail(h, st, "seq_set_tail(%d, %d): sequence not live or negative tail", seq, tail_tokens);
}
int tk_kv_seq_len(const tk_kv* h, int32_t seq) { return h ? h->mgr->seq_len(seq) : -1; }
int tk_kv_num_free_pages(const tk_kv* h) { return h ? h->mgr->num_free_pages() : -1; }
int tk_kv_page_table(const tk_kv* h, int32_t seq, int32_t* out, int32_t cap, int32_t* n_out) {
    if (!h || !h->mgr->live(seq)) return TK_INVALID_ARG;
    int n = h->mgr->seq_pages(seq);
    if (n_out) *n_out = n;
    if (out) {
        if (cap < n) return TK_INVALID_ARG;
        memcpy(out, h->mgr->row(seq), sizeof(int32_t) * (size_t)n);
    }
    return TK_OK;
}
int64_t tk_kv_slot(const tk_kv* h, int32_t seq, int32_t pos) { return h ? h->mgr->slot(seq, pos) : -1; }
uint64_t tk_kv_state_digest(const tk_kv* h) { return h ? h->mgr->digest() : 0; }
int tk_kv_state_save(const tk_kv* h, int32_t* image, int64_t cap, int64_t* n_out) {
    if (!h || !n_out) return TK_INVALID_ARG;
    std::lock_guard<std::mutex> lock(const_cast<tk_kv*>(h)->mgr_mu);
    const std::vector<int32_t> im = h->mgr->save();
    *n_out = (int64_t)im.size();
    if (!image) return TK_OK;
    if (cap < (int64_t)im.size()) return TK_INVALID_ARG;
    memcpy(image, im.data(), im.size() * sizeof(int32_t));
    return TK_OK;
}
int tk_kv_state_load(tk_kv* h, const int32_t* image, int64_t n) {
    if (!h || !image || n <= 0) return TK_INVALID_ARG;
    std::lock_guard<std::mutex> lock(h->mgr_mu);
    if (h->mgr->cold_enabled() && !h->host_only)
        return fail(h, TK_UNSUPPORTED, "state_load: a device handle with a cold tier cannot take an image (the host pool's contents are not part of it)");
    const int st = h->mgr->load(image, (size_t)n);
    if (st != TK_OK) return fail(h, st, "state_load: the image does not belong to a cache of this geometry, or is damaged");
    h->have_step = false;
    return TK_OK;
}

int tk_kv_get_stats(const tk_kv* h, tk_kv_stats* out) {
    if (!h || !out) return TK_INVALID_ARG;
    *out = h->stats;
    out->pages_free = h->mgr->num_free_pages();
    out->pages_cold = h->mgr->num_cold_used();
    out->evictions = h->mgr->counters.evictions;
    out->page_allocs = h->mgr->counters.page_allocs;
    out->page_frees = h->mgr->counters.page_frees;
    out->seq_allocs = h->mgr->counters.seq_allocs;
    out->seq_frees = h->mgr->counters.seq_frees;
    return TK_OK;
}

// ---- step ----------------------------------------------------------------------------------
static int step_begin_impl(tk_kv* h, int32_t n_seqs, const int32_t* seq_ids, const int32_t* n_new,
                           const int32_t* len_cap, void* stream) {
    if (!h) return TK_INVALID_ARG;
    if (const int fs = host_flush(h)) return fs;               // launches the host-buffer calls still hold back come first
    h->host_calls_in_step = 0;
    if (len_cap && h->cfg.dtype == TK_FP8_E4M3)
        return fail(h, TK_UNSUPPORTED, "step_begin: an attended-length cap needs 16-bit storage");
    std::lock_guard<std::mutex> lock(h->mgr_mu);
    h->have_step = false;
    const int chunk = h->cfg.chunk_tokens;
    const int target = 8 * h->num_sms;       // work items the planner aims for when it picks the chunk itself
    // the tensor-core kernel keeps one page id per lane per warp: chunk <= 16*4*32 tokens
    int st = h->mgr->plan_step(n_seqs, seq_ids, n_new, h->cfg.num_kv_heads, h->cfg.dtype == TK_FP8_E4M3,
                               chunk, target, h->cfg.max_step_tokens, h->max_partial_rows, &h->plan, len_cap,
                               h->geo.H / h->geo.Hkv, h->prefill_tc ? tk::kPrefillRowsTc : tk::kPrefillRows);
    if (st != TK_OK) return fail(h, st, "step_begin: %s", tk_status_str(st));
    tk::StepPlan& p = h->plan;
    if (chunk == 0 && p.chunk_tokens > 2048) {
        return fail(h, TK_INVALID_ARG, "internal: chunk %d too large", p.chunk_tokens);
    }
    // kind-0 items first (already size-sorted), FP8 open-page items after them
    std::stable_partition(p.items.begin(), p.items.end(), [](const tk::WorkItem& w) { return w.kind == 0; });
    h->n_pool_items = 0;
    for (const auto& w : p.items) h->n_pool_items += w.kind == 0;

    h->stats.steps++;
    h->stats.tokens_appended += (int64_t)p.tok_b.size();
    h->stats.pages_sealed += (int64_t)p.seals.size();
    if (p.evictions_refused > 0) {
        h->stats.evictions_refused += p.evictions_refused;
        fail(h, TK_OK, "step_begin: host (cold) pool is full, %d sequence(s) kept their old pages in HBM", p.evictions_refused);
    }
    if (h->host_only) { h->mgr->delta().clear(); h->have_step = true; return TK_OK; }

    cudaStream_t s = (cudaStream_t)stream;
    TK_CUDA(h, cudaSetDevice(h->device));
    h->mgr->compact_delta();
    auto& delta = h->mgr->delta();
    int n_delta = (int)delta.size();
    if (n_delta > kMaxDelta || h->mgr->take_full_upload()) {
        // rare (bulk adopt / huge prefill): copy the whole table from pageable memory
        const size_t n_entries = (size_t)h->cfg.max_seqs * h->cfg.max_pages_per_seq;
        std::vector<int32_t> full(n_entries);
        for (size_t i = 0; i < n_entries; i++) full[i] = dev_entry(h->mgr->page_table()[i]);
        TK_CUDA(h, cudaMemcpyAsync(h->d_table, full.data(), n_entries * sizeof(int32_t), cudaMemcpyHostToDevice, s));
        TK_CUDA(h, cudaStreamSynchronize(s));
        h->stats.bytes_h2d += (int64_t)h->cfg.max_seqs * h->cfg.max_pages_per_seq * 4;
        delta.clear();
        n_delta = 0;
    }
    const int n_tok = (int)p.tok_b.size(), n_items = (int)p.items.size(), n_seals = (int)p.seals.size();
    if (n_items > h->max_items || n_seals > h->max_seals)
        return fail(h, TK_INVALID_ARG, "step_begin: work list exceeds the workspace (%d items, %d seals)", n_items, n_seals);
    const int n_open = (int)p.tok_open.size();
    const int n_pf = p.pf_built ? (int)p.pf_items.size() : 0, n_pf_small = p.pf_built ? (int)p.pf_small_items.size() : 0;
    if (n_pf > h->max_pf_items || p.pf_groups > h->max_pf_groups)
        return fail(h, TK_INVALID_ARG, "step_begin: prefill work list exceeds the workspace (%d items, %d groups)", n_pf, p.pf_groups);
    Sections sec = sections(n_seqs, n_tok, n_open, n_items, n_seals, n_delta, n_pf, n_pf_small);
    if (sec.end * 4 > h->step_bytes) return fail(h, TK_INVALID_ARG, "step_begin: step metadata exceeds its buffer");

    const int r = h->ring_pos;
    h->ring_pos = (r + 1) % kRing;
    if (h->ev_pending[r]) { TK_CUDA(h, cudaEventSynchronize(h->ev[r])); h->ev_pending[r] = false; }
    int32_t* w = (int32_t*)h->h_step[r];
    if (n_seqs) {
        memcpy(w + sec.seq, p.seq.data(), 4 * (size_t)n_seqs);
        memcpy(w + sec.len, p.len.data(), 4 * (size_t)n_seqs);
        memcpy(w + sec.new_tok, p.new_tok.data(), 4 * (size_t)n_seqs);
        memcpy(w + sec.q_base, p.q_base.data(), 4 * (size_t)n_seqs);
        memcpy(w + sec.nq, p.nq.data(), 4 * (size_t)n_seqs);
    }
    memcpy(w + sec.chunk_base, p.chunk_base.data(), 4 * (size_t)(n_seqs + 1));
    if (n_tok) {
        memcpy(w + sec.tok_b, p.tok_b.data(), 4 * (size_t)n_tok);
        memcpy(w + sec.tok_pos, p.tok_pos.data(), 4 * (size_t)n_tok);
        memcpy(w + sec.tok_dst, p.tok_dst.data(), 4 * (size_t)n_tok);
        if (n_open) memcpy(w + sec.tok_open, p.tok_open.data(), 4 * (size_t)n_open);
    }
    if (n_items) memcpy(w + sec.items, p.items.data(), 16 * (size_t)n_items);
    if (n_seals) memcpy(w + sec.seals, p.seals.data(), 16 * (size_t)n_seals);
    for (int i = 0; i < n_delta; i++) { w[sec.delta + 2 * i] = delta[i].first; w[sec.delta + 2 * i + 1] = dev_entry(delta[i].second); }
    delta.clear();
    if (p.pf_built) {
        memcpy(w + sec.pf_ct, p.pf_ct.data(), 4 * (size_t)n_seqs);
        memcpy(w + sec.pf_poff, p.pf_poff.data(), 4 * (size_t)n_seqs);
        memcpy(w + sec.pf_cbase, p.pf_cbase.data(), 4 * (size_t)n_seqs);
        if (n_pf) memcpy(w + sec.pf_items, p.pf_items.data(), 16 * (size_t)n_pf);
        for (int i = 0; i < n_pf; i++) {                     // what the item's CTA needs of its sequence, next to the item:
            const int b = p.pf_items[i].b;                   // one dependent load less before its first copy can go out
            int32_t* o = w + sec.pf_info + 8 * (size_t)i;
            o[0] = p.seq[b]; o[1] = p.len[b]; o[2] = p.nq[b]; o[3] = p.pf_ct[b];
            o[4] = p.q_base[b]; o[5] = p.pf_poff[b]; o[6] = p.pf_cbase[b]; o[7] = 0;
        }
        if (n_pf_small) memcpy(w + sec.pf_small, p.pf_small_items.data(), 16 * (size_t)n_pf_small);
    }
    TK_CUDA(h, cudaMemcpyAsync(h->d_step, w, sec.end * 4, cudaMemcpyHostToDevice, s));
    TK_CUDA(h, cudaEventRecord(h->ev[r], s));
    h->ev_pending[r] = true;
    h->stats.bytes_h2d += (int64_t)sec.end * 4;

    const int32_t* d = (const int32_t*)h->d_step;
    tk::StepDev& dv = h->dev;
    dv.seq = d + sec.seq; dv.len = d + sec.len; dv.chunk_base = d + sec.chunk_base;
    dv.new_tok = d + sec.new_tok; dv.q_base = d + sec.q_base; dv.nq = d + sec.nq; dv.nq_max = p.nq_max;
    dv.tok_b = d + sec.tok_b; dv.tok_pos = d + sec.tok_pos; dv.tok_dst = d + sec.tok_dst; dv.tok_open = d + sec.tok_open;
    dv.items = (const int4*)(d + sec.items); dv.seals = (const int4*)(d + sec.seals);
    dv.n_seqs = n_seqs; dv.n_tokens = n_tok; dv.n_items = n_items; dv.n_seals = n_seals;
    dv.chunk_tokens = p.chunk_tokens; dv.n_open = n_open;
    h->pf_dev = tk::PrefillDev{};
    if (p.pf_built) {
        h->pf_dev = tk::PrefillDev{(const int4*)(d + sec.pf_items), d + sec.pf_ct, d + sec.pf_poff, d + sec.pf_cbase, n_pf,
                                   (const int4*)(d + sec.pf_info)};
        h->small_dev = dv;                                  // the decode kernel's share: the short sequences only
        h->small_dev.items = (const int4*)(d + sec.pf_small);
        h->small_dev.n_items = n_pf_small;
        h->small_dev.nq_max = p.pf_small_nq_max;
    }
    if (n_delta) {
        TK_CUDA(h, tk::launch_apply_delta(h->d_table, (const int2*)(d + sec.delta), n_delta, s));
        h->launches++;
    }
    if (h->mgr->cold_enabled()) {
        int est = run_evictions(h, p.evictions, s);
        if (est != TK_OK) return est;
        h->staged_layer[0] = h->staged_layer[1] = -1;       // cold contents may have changed
        est = prefetch_layer(h, 0, /*ahead=*/false);
        if (est != TK_OK) return est;
    }
    h->have_step = true;
    return TK_OK;
}

int tk_kv_step_begin(tk_kv* h, int32_t n_seqs, const int32_t* seq_ids, const int32_t* n_new, void* stream) {
    return step_begin_impl(h, n_seqs, seq_ids, n_new, nullptr, stream);
}
int tk_kv_step_begin_capped(tk_kv* h, int32_t n_seqs, const int32_t* seq_ids, const int32_t* n_new,
                            const int32_t* len_cap, void* stream) {
    return step_begin_impl(h, n_seqs, seq_ids, n_new, len_cap, stream);
}

int tk_kv_set_num_heads(tk_kv* h, int32_t num_heads) {
    if (!h) return TK_INVALID_ARG;
    const int hkv = h->cfg.num_kv_heads;
    const int g = num_heads > 0 && num_heads % hkv == 0 ? num_heads / hkv : 0;
    if (g != 1 && g != 2 && g != 4 && g != 8 && g != 16) return fail(h, TK_INVALID_ARG, "set_num_heads(%d): heads per kv head must be 1, 2, 4, 8 or 16", num_heads);
    if (num_heads > h->cfg.num_heads) return fail(h, TK_INVALID_ARG, "set_num_heads(%d): above the %d the handle was sized for", num_heads, h->cfg.num_heads);
    h->geo.H = num_heads;
    return TK_OK;
}

int tk_kv_step_num_tokens(const tk_kv* h) { return h && h->have_step ? (int)h->plan.tok_b.size() : -1; }
int tk_kv_step_num_work_items(const tk_kv* h) { return h && h->have_step ? (int)h->plan.items.size() : -1; }
int tk_kv_step_chunk_tokens(const tk_kv* h) { return h && h->have_step ? h->plan.chunk_tokens : -1; }
int tk_kv_step_prefill_plan(const tk_kv* h, int32_t cap, int32_t* items, int32_t* n_items, int32_t* chunk_tokens,
                            int32_t* n_decode_items) {
    if (!h || !h->have_step || !n_items) return TK_INVALID_ARG;
    const tk::StepPlan& p = h->plan;
    *n_items = p.pf_built ? (int32_t)p.pf_items.size() : 0;
    if (n_decode_items) *n_decode_items = p.pf_built ? (int32_t)p.pf_small_items.size() : 0;
    if (!p.pf_built) return TK_OK;
    if (items) {
        if (cap < *n_items) return TK_INVALID_ARG;
        memcpy(items, p.pf_items.data(), 16 * p.pf_items.size());
    }
    if (chunk_tokens) memcpy(chunk_tokens, p.pf_ct.data(), 4 * p.pf_ct.size());
    return TK_OK;
}

int tk_kv_append(tk_kv* h, int32_t layer, const void* k, const void* v, int64_t* slots_out, void* stream) {
    if (!h || layer < 0 || layer >= h->cfg.num_layers) return TK_INVALID_ARG;
    if (const int fs = host_flush(h)) return fs;               // launches the host-buffer calls still hold back come first
    if (h->host_only) return fail(h, TK_CUDA_ERROR, "append: handle has no device (bookkeeping only)");
    if (!h->have_step) return fail(h, TK_INVALID_ARG, "append: no step in progress (call tk_kv_step_begin)");
    if (h->dev.n_tokens == 0) return TK_OK;
    if (!k || !v) return fail(h, TK_INVALID_ARG, "append: null k/v");
    int n = 0;
    cudaError_t e = tk::launch_append(h->geo, h->layer(layer), h->dev, h->d_table, k, v, slots_out,
                                      (cudaStream_t)stream, &n);
    h->launches += n;
    if (e != cudaSuccess) return fail(h, TK_CUDA_ERROR, "append launch: %s", cudaGetErrorString(e));
    return TK_OK;
}

static int decode_impl(tk_kv* h, int layer, const void* q, void* out, float* partial_out, cudaStream_t s,
                       int q_dtype = -1, int out_dtype = -1, const void* fuse_k = nullptr,
                       const void* fuse_v = nullptr, const float* rope = nullptr,
                       const tk::PeerCtx* peer_ctx = nullptr) {
    if (!h || layer < 0 || layer >= h->cfg.num_layers) return TK_INVALID_ARG;
    if (const int fs = host_flush(h)) return fs;               // launches the host-buffer calls still hold back come first
    if (h->host_only) return fail(h, TK_CUDA_ERROR, "decode: handle has no device (bookkeeping only)");
    if (!h->have_step) return fail(h, TK_INVALID_ARG, "decode: no step in progress (call tk_kv_step_begin)");
    if (h->dev.n_seqs == 0) return TK_OK;
    if (!q || (!out && !partial_out)) return fail(h, TK_INVALID_ARG, "decode: null q/out");
    tk::LayerPtrs lp = h->layer(layer);
    cudaError_t e = cudaSuccess;
    const bool cold = h->mgr->cold_enabled() && h->mgr->cold_high_water() > 0;
    const int slot = layer & 1;
    if (cold) {
        int pst = prefetch_layer(h, layer, /*ahead=*/false);   // no-op when it was staged ahead
        if (pst != TK_OK) return pst;
        TK_CUDA(h, cudaStreamWaitEvent(s, h->ev_pf[slot], 0));
        lp.cold_stage = h->d_stage[slot];
    }
    if (q_dtype == TK_FP32) {                               // FP32 callers: narrow q into the staging buffer
        e = tk::launch_f32_to_16((const float*)q, h->d_q, (size_t)h->dev.n_seqs * h->geo.H * h->geo.D,
                                 h->cfg.io_dtype, s);
        h->launches++;
        if (e != cudaSuccess) return fail(h, TK_CUDA_ERROR, "q conversion launch: %s", cudaGetErrorString(e));
        q = h->d_q;
    } else if (q_dtype >= 0 && q_dtype != h->cfg.io_dtype) {
        return fail(h, TK_INVALID_ARG, "decode: q dtype must be FP32 or the handle's io dtype");
    }
    if (out_dtype < 0) out_dtype = h->cfg.io_dtype;
    if (out_dtype != TK_FP32 && out_dtype != h->cfg.io_dtype)
        return fail(h, TK_INVALID_ARG, "decode: out dtype must be FP32 or the handle's io dtype");
    const bool mma = h->use_mma && h->dev.chunk_tokens <= 2048;
    // the last CTA of each (sequence, kv head) merges the split-KV rows itself; a sequence that
    // attends to nothing has no CTA, so such steps keep the separate combine kernel
    const bool fused_merge = !h->plan.has_empty_seq && !h->separate_combine;
    if (peer_ctx && !fused_merge) return fail(h, TK_INVALID_ARG, "decode: the in-kernel exchange needs the in-kernel merge");
    const tk::MergeOut mo{fused_merge ? h->d_counters : nullptr, out, partial_out, out_dtype, peer_ctx, h->d_status};
    const tk::FuseAppend fa{fuse_k, fuse_v, rope ? h->d_rope_tab : nullptr};
    const bool timed = h->profiling && h->prof_used + 2 <= h->prof_ev.size();
    if (timed) cudaEventRecord(h->prof_ev[h->prof_used], s);
    if (mma) {
        // FP8: the 16-bit open pages are items of kind 1 of the same launch
        if (h->dev.n_items > 0) {
            // A launch of ANOTHER layer that directly follows an attention launch of this handle on the same
            // stream may overlap that launch's tail: its page tiles belong to a pool the earlier kernel does
            // not touch, and it waits for the earlier kernel before it writes split-KV rows or `out`.
            const bool overlap = h->cfg.launch_overlap == TK_OVERLAP_AUTO && !cold && !timed &&
                                 h->chain_launches == h->launches && h->chain_stream == s && h->chain_layer != layer;
            if (h->mla_mma)
                e = tk::launch_decode_mma_mla(h->geo, lp, &h->maps[layer], &h->maps_v[layer], h->dev, h->d_table, q,
                                              h->d_partials, h->d_status, s, &mo, &fa, overlap);
            else
                e = tk::launch_decode_mma(h->geo, lp, &h->maps[layer], cold ? &h->stage_maps[slot] : nullptr, h->dev,
                                          h->d_table, q, h->d_partials, h->d_status, s, &mo, &fa, overlap);
            h->chain_launches = h->launches + 1; h->chain_layer = layer; h->chain_stream = s;
            h->launches++;
        }
        if (timed) { cudaEventRecord(h->prof_ev[h->prof_used + 1], s); h->prof_used += 2; }
    } else {
        if (h->dev.n_items > 0) {
            e = tk::launch_decode_simt(h->geo, lp, h->dev, h->d_table, q, h->d_partials, s, &mo);
            h->launches++;
        }
        if (timed) { cudaEventRecord(h->prof_ev[h->prof_used + 1], s); h->prof_used += 2; }
    }
    if (e != cudaSuccess) return fail(h, TK_CUDA_ERROR, "decode launch: %s", cudaGetErrorString(e));
    if (cold) {
        TK_CUDA(h, cudaEventRecord(h->ev_used[slot], s));
        int pst = prefetch_layer(h, layer + 1, /*ahead=*/true);   // next layer's pages ride PCIe under this kernel
        if (pst != TK_OK) return pst;
    }
    if (!fused_merge) {
        e = tk::launch_combine_step(h->geo, h->dev, h->d_partials, out, out_dtype, partial_out, s, h->d_status);
        h->launches++;
        if (e != cudaSuccess) return fail(h, TK_CUDA_ERROR, "combine launch: %s", cudaGetErrorString(e));
    }
    return TK_OK;
}

int tk_kv_decode(tk_kv* h, int32_t layer, const void* q, void* out, void* stream) {
    return decode_impl(h, layer, q, out, nullptr, (cudaStream_t)stream);
}
// Decode step in one launch where the shape allows it: the attention kernel writes the new
// token's rows itself.  Otherwise the two calls it stands for.
int tk_kv_append_decode(tk_kv* h, int32_t layer, const void* k, const void* v, const void* q, void* out,
                        void* stream) {
    if (!h || layer < 0 || layer >= h->cfg.num_layers) return TK_INVALID_ARG;
    if (const int fs = host_flush(h)) return fs;               // launches the host-buffer calls still hold back come first
    if (h->host_only) return fail(h, TK_CUDA_ERROR, "append_decode: handle has no device (bookkeeping only)");
    if (!h->have_step) return fail(h, TK_INVALID_ARG, "append_decode: no step in progress (call tk_kv_step_begin)");
    // 16-bit storage: the new row goes into the page the kernel is about to read.  FP8 storage: it
    // goes into the sequence's 16-bit open page, unless this step completes (seals) a page.
    const bool fusable = h->use_mma && h->plan.one_token_steps && h->dev.chunk_tokens <= 2048 &&
                         h->dev.n_tokens > 0 && h->dev.n_seqs > 0 && !h->plan.has_empty_seq &&
                         (h->cfg.dtype != TK_FP8_E4M3 || h->plan.seals.empty());
    if (!fusable) {
        int st = tk_kv_append(h, layer, k, v, nullptr, stream);
        if (st != TK_OK) return st;
        return tk_kv_decode(h, layer, q, out, stream);
    }
    if (!k || !v) return fail(h, TK_INVALID_ARG, "append_decode: null k/v");
    return decode_impl(h, layer, q, out, nullptr, (cudaStream_t)stream, -1, -1, k, v);
}

// rope_kernel + update + attention_decode of one layer (src/model/dense.cpp:382-398).
int tk_kv_rope_append_decode(tk_kv* h, int32_t layer, const void* k, const void* v, const void* q, void* out,
                             float theta, float scaling, void* stream) {
    if (!h || layer < 0 || layer >= h->cfg.num_layers) return TK_INVALID_ARG;
    if (h->host_only) return fail(h, TK_CUDA_ERROR, "rope_append_decode: handle has no device (bookkeeping only)");
    if (!h->have_step) return fail(h, TK_INVALID_ARG, "rope_append_decode: no step in progress (call tk_kv_step_begin)");
    if (!q || !out || (h->dev.n_tokens > 0 && (!k || !v))) return fail(h, TK_INVALID_ARG, "rope_append_decode: null argument");
    const bool fusable = h->use_mma && h->cfg.dtype != TK_FP8_E4M3 && h->plan.one_token_steps &&
                         h->dev.chunk_tokens <= 2048 && h->dev.n_tokens > 0 && h->dev.n_seqs > 0 &&
                         !h->plan.has_empty_seq;
    if (fusable) {
        const float rope[2] = {theta, scaling};
        // cos/sin of each sequence's newest position: computed once per step, shared by all layers
        if (h->rope_tab_step != h->stats.steps || h->rope_tab_theta != theta || h->rope_tab_scaling != scaling) {
            cudaError_t te = tk::launch_rope_table(h->geo, h->dev, h->d_rope_tab, theta, scaling, (cudaStream_t)stream);
            h->launches++;
            if (te != cudaSuccess) return fail(h, TK_CUDA_ERROR, "rope table launch: %s", cudaGetErrorString(te));
            h->rope_tab_step = h->stats.steps; h->rope_tab_theta = theta; h->rope_tab_scaling = scaling;
        }
        return decode_impl(h, layer, q, out, nullptr, (cudaStream_t)stream, -1, -1, k, v, rope);
    }
    cudaError_t e = tk::launch_rope16(h->geo, h->dev, q, k, h->d_rq, h->d_rk, theta, scaling, (cudaStream_t)stream);
    h->launches++;
    if (e != cudaSuccess) return fail(h, TK_CUDA_ERROR, "rope launch: %s", cudaGetErrorString(e));
    return tk_kv_append_decode(h, layer, h->d_rk, v, h->d_rq, out, stream);
}

int tk_kv_decode_ex(tk_kv* h, int32_t layer, const void* q, int32_t q_dtype, void* out, int32_t out_dtype,
                    void* stream) {
    return decode_impl(h, layer, q, out, nullptr, (cudaStream_t)stream, q_dtype, out_dtype);
}
int tk_kv_decode_partial(tk_kv* h, int32_t layer, const void* q, float* partial, void* stream) {
    return decode_impl(h, layer, q, nullptr, partial, (cudaStream_t)stream);
}

// Split-KV workspace of a multi-token step: the handle's own when `floats` fit it, else a buffer that is
// allocated (and grown) on demand - the one device allocation a step may make after creation.
static float* multi_workspace(tk_kv* h, size_t floats, cudaStream_t stream) {
    if (floats <= (size_t)h->max_partial_rows * h->cfg.num_heads * (h->cfg.v_head_dim + 2)) return h->d_partials;
    if (floats > h->multi_partials_floats) {
        if (cudaSetDevice(h->device) != cudaSuccess) { fail(h, TK_CUDA_ERROR, "cudaSetDevice failed"); return nullptr; }
        if (h->d_multi_partials) { cudaStreamSynchronize(stream); cudaFree(h->d_multi_partials); }
        h->d_multi_partials = nullptr; h->multi_partials_floats = 0;
        cudaError_t e = cudaMalloc((void**)&h->d_multi_partials, floats * sizeof(float));
        if (e != cudaSuccess) { fail(h, TK_CUDA_ERROR, "split-KV workspace of %zu bytes: %s", floats * sizeof(float), cudaGetErrorString(e)); return nullptr; }
        h->multi_partials_floats = floats;
    }
    return h->d_multi_partials;
}

// Attention for every token the step appended (several per sequence), causal among themselves, in one
// pass over the pages: what the verification of drafted tokens needs.
static int decode_multi_impl(tk_kv* h, int32_t layer, const void* q, void* out, int out_dtype, void* stream) {
    if (!h || layer < 0 || layer >= h->cfg.num_layers) return TK_INVALID_ARG;
    if (const int fs = host_flush(h)) return fs;               // launches the host-buffer calls still hold back come first
    if (out_dtype != TK_FP32 && out_dtype != h->cfg.io_dtype)
        return fail(h, TK_INVALID_ARG, "decode_multi: out dtype must be FP32 or the handle's io dtype");
    if (h->host_only) return fail(h, TK_CUDA_ERROR, "decode_multi: handle has no device (bookkeeping only)");
    if (!h->have_step) return fail(h, TK_INVALID_ARG, "decode_multi: no step in progress (call tk_kv_step_begin)");
    if (h->dev.n_seqs == 0) return TK_OK;
    if (!q || !out) return fail(h, TK_INVALID_ARG, "decode_multi: null q/out");
    const tk::StepPlan& p = h->plan;
    if (p.nq_min < 1) return fail(h, TK_INVALID_ARG, "decode_multi: every sequence of the step must append at least one token");
    if (p.pf_built && h->use_mma && !h->mla_mma && tk::prefill_mma_supported(h->geo)) {
        // a prefill-sized step: the sequences with one tile of rows keep the decode kernel, the prefill
        // kernel takes the others; the two write disjoint rows of `out`
        if (h->mgr->cold_enabled() && h->mgr->cold_high_water() > 0)
            return fail(h, TK_UNSUPPORTED, "decode_multi: not available while pages are cold");
        // split-KV rows: the decode kernel's share first, the prefill kernel's split regions behind it; steps that
        // outgrow the handle's workspace get one of their own, grown when a step needs a larger one
        const size_t row_floats = (size_t)h->cfg.num_heads * (h->cfg.v_head_dim + 2);
        const size_t small_rows = h->small_dev.n_items > 0 ? (size_t)p.chunk_base[h->dev.n_seqs] * p.pf_small_nq_max : 0;
        float* ws = multi_workspace(h, (small_rows + (size_t)p.pf_partial_rows) * row_floats, (cudaStream_t)stream);
        if (!ws) return TK_CUDA_ERROR;
        cudaError_t e = cudaSuccess;
        if (h->small_dev.n_items > 0) {
            if (p.has_empty_seq || h->separate_combine || h->dev.chunk_tokens > 2048)
                return fail(h, TK_UNSUPPORTED, "decode_multi: needs the in-kernel merge");
            const tk::MergeOut mo{h->d_counters, out, nullptr, out_dtype, nullptr, h->d_status};
            e = tk::launch_decode_mma_multi(h->geo, h->layer(layer), &h->maps[layer], h->small_dev, h->d_table, q,
                                            ws, h->d_status, (cudaStream_t)stream, mo);
            h->launches++;
            if (e != cudaSuccess) return fail(h, TK_CUDA_ERROR, "decode_multi launch: %s", cudaGetErrorString(e));
        }
        float* pf_partials = ws + small_rows * row_floats;
        if (h->prefill_tc && p.pf_rows == tk::kPrefillRowsTc)
            e = tk::launch_prefill_tc(h->geo, &h->maps16[layer], h->dev, h->pf_dev, h->d_table, q, out, out_dtype, pf_partials,
                                      h->d_pf_counters, h->d_status, (cudaStream_t)stream);
        else
            e = tk::launch_prefill_mma(h->geo, &h->maps[layer], h->dev, h->pf_dev, h->d_table, q, out, out_dtype, pf_partials,
                                       h->d_pf_counters, h->d_status, (cudaStream_t)stream);
        if (h->pf_dev.n_items > 0) h->launches++;
        if (e != cudaSuccess) return fail(h, TK_CUDA_ERROR, "prefill attention launch: %s", cudaGetErrorString(e));
        return TK_OK;
    }
    const bool ok = h->use_mma && (h->mla_mma ? tk::decode_mma_mla_multi_supported(h->geo, p.nq_max)
                                              : tk::decode_mma_multi_supported(h->geo, p.nq_max));
    if (!ok)
        return fail(h, TK_UNSUPPORTED, "decode_multi: needs the tensor-core kernels on a 16-bit pool (MLA shape: (heads per kv "
                                       "head) x (tokens per sequence) <= 64; here %d x %d)", h->geo.H / h->geo.Hkv, p.nq_max);
    if (h->mgr->cold_enabled() && h->mgr->cold_high_water() > 0)
        return fail(h, TK_UNSUPPORTED, "decode_multi: not available while pages are cold");
    if (p.has_empty_seq || h->separate_combine || h->dev.chunk_tokens > 2048)
        return fail(h, TK_UNSUPPORTED, "decode_multi: needs the in-kernel merge");
    // partial rows hold H * nq_max columns here; the handle's workspace was sized for H columns
    float* partials = multi_workspace(h, (size_t)p.chunk_base[h->dev.n_seqs] * h->geo.H * p.nq_max * (h->geo.Dv + 2),
                                      (cudaStream_t)stream);
    if (!partials) return TK_CUDA_ERROR;
    const tk::MergeOut mo{h->d_counters, out, nullptr, out_dtype, nullptr, h->d_status};
    cudaError_t e = h->mla_mma
        ? tk::launch_decode_mma_mla_multi(h->geo, h->layer(layer), &h->maps[layer], &h->maps_v[layer], h->dev, h->d_table, q,
                                          partials, h->d_status, (cudaStream_t)stream, mo)
        : tk::launch_decode_mma_multi(h->geo, h->layer(layer), &h->maps[layer], h->dev, h->d_table, q,
                                      partials, h->d_status, (cudaStream_t)stream, mo);
    h->launches++;
    if (e != cudaSuccess) return fail(h, TK_CUDA_ERROR, "decode_multi launch: %s", cudaGetErrorString(e));
    return TK_OK;
}

int tk_kv_decode_multi(tk_kv* h, int32_t layer, const void* q, void* out, void* stream) {
    return decode_multi_impl(h, layer, q, out, h ? h->cfg.io_dtype : 0, stream);
}
int tk_kv_decode_multi_ex(tk_kv* h, int32_t layer, const void* q, void* out, int32_t out_dtype, void* stream) {
    return decode_multi_impl(h, layer, q, out, out_dtype, stream);
}

int tk_kv_append_decode_multi(tk_kv* h, int32_t layer, const void* k, const void* v, const void* q, void* out,
                              void* stream) {
    int st = tk_kv_append(h, layer, k, v, nullptr, stream);
    if (st != TK_OK) return st;
    return tk_kv_decode_multi(h, layer, q, out, stream);
}

// Attention over a sequence whose tokens are spread over the ranks of `peer`.  One launch where the
// step allows it: the attention kernel's merging CTAs store their merged rows into every rank's
// mailbox, await every rank's rows of their (sequence, kv head) and write the combine themselves.
// Otherwise two launches: this rank's merged rows, then the exchange kernel, which fills and reads the
// same cells - so ranks that take different routes for the same layer still meet.
int tk_kv_decode_exchange(tk_kv* h, int32_t layer, const void* q, tk_peer* peer, void* out, void* stream) {
    if (!h || !peer || !out) return TK_INVALID_ARG;
    if (const int fs = host_flush(h)) return fs;               // launches the host-buffer calls still hold back come first
    if (h->host_only) return fail(h, TK_CUDA_ERROR, "decode_exchange: handle has no device (bookkeeping only)");
    if (!h->have_step) return fail(h, TK_INVALID_ARG, "decode_exchange: no step in progress (call tk_kv_step_begin)");
    const tk::PeerCtx* ctx = tk::peer_device_ctx(peer);
    if (!ctx) return fail(h, TK_INVALID_ARG, "decode_exchange: peers are not connected");
    const int n_rows = h->dev.n_seqs * h->geo.H, dv = h->cfg.v_head_dim;
    if (tk::peer_row_floats(peer) != dv + 2 || n_rows > tk::peer_max_rows(peer))
        return fail(h, TK_INVALID_ARG, "decode_exchange: %d rows of %d floats do not fit the mailbox", n_rows, dv + 2);
    if (h->dev.n_seqs == 0) return TK_OK;
    // a merging CTA waits for its peers while it holds a CTA slot: keep those few against the slots of a
    // launch, or ranks could fill their GPUs with CTAs that wait for CTAs the other ranks cannot start
    const bool in_kernel = !h->plan.has_empty_seq && !h->separate_combine && h->dev.n_items > 0 &&
                           h->dev.n_seqs * h->geo.Hkv <= h->num_sms / 2;
    if (in_kernel) {
        int st = decode_impl(h, layer, q, out, nullptr, (cudaStream_t)stream, -1, -1, nullptr, nullptr, nullptr, ctx);
        if (st == TK_OK) tk::peer_note_fused_send(peer);
        return st;
    }
    const size_t need = (size_t)h->cfg.max_seqs * h->cfg.num_heads * (h->cfg.v_head_dim + 2) * sizeof(float);
    if (!h->d_xpartial) {                                   // first use only
        TK_CUDA(h, cudaSetDevice(h->device));
        TK_CUDA(h, cudaMalloc((void**)&h->d_xpartial, need));
    }
    int st = decode_impl(h, layer, q, nullptr, h->d_xpartial, (cudaStream_t)stream);
    if (st != TK_OK) return st;
    st = tk::peer_exchange(peer, h->d_xpartial, n_rows, dv, out, h->cfg.io_dtype, stream);
    h->launches++;
    if (st != TK_OK) return fail(h, st, "decode_exchange: %s", tk_peer_last_error(peer));
    return TK_OK;
}

int tk_combine_partials(const float* parts, int32_t n_parts, int32_t n_rows, int32_t head_dim, void* out,
                        int32_t out_dtype, void* stream) {
    if (!parts || !out || n_parts <= 0 || n_rows < 0 || head_dim <= 0) return TK_INVALID_ARG;
    if (out_dtype != TK_FP32 && out_dtype != TK_FP16 && out_dtype != TK_BF16) return TK_INVALID_ARG;
    cudaError_t e = tk::launch_combine_parts(parts, n_parts, n_rows, head_dim, out, out_dtype, (cudaStream_t)stream);
    return e == cudaSuccess ? TK_OK : TK_CUDA_ERROR;
}

// Host-buffer path.  Call n uses staging set n % host_sets:
//   copy-in stream : (wait: this set's last use is over)            H2D k, v, q        - at the call
//   caller's stream: (wait: H2D of the group's last call done)      append + decode    - one group of calls at a time
//   copy-out stream: (wait: the group's kernels done)               D2H out of each call of the group
// so the copies of neighbouring layers ride the copy engines while a kernel runs.  The asynchronous form
// holds its kernel launches back until host_group calls are in (or until tk_kv_host_wait, a new step, or any
// other launching entry point): an event wait or record BETWEEN two attention launches keeps the later one
// from starting while the earlier one drains (programmatic dependent launch needs them adjacent in the
// stream), so the waits and records go around a group of launches, not around each.
// tk_kv_host_wait() launches what is held back and makes the caller's stream wait for the outstanding D2H copies.
static int host_flush(tk_kv* h) {
    if (h->host_flushing || h->host_pending.empty()) return TK_OK;
    h->host_flushing = true;
    std::vector<tk_kv::HostPending> pend;
    pend.swap(h->host_pending);
    cudaStream_t s = h->host_pending_stream;
    int st = TK_OK;
    cudaError_t e = cudaStreamWaitEvent(s, h->ev_in[pend.back().set], 0);   // the copy-in stream is in order: all of them are in
    for (size_t i = 0; i < pend.size() && st == TK_OK && e == cudaSuccess; i++) {
        const auto& p = pend[i];
        if (p.kv && p.q)  st = tk_kv_append_decode(h, p.layer, h->hs_k[p.set], h->hs_v[p.set], h->hs_q[p.set], h->hs_out[p.set], s);
        else if (p.kv)    st = tk_kv_append(h, p.layer, h->hs_k[p.set], h->hs_v[p.set], nullptr, s);
        else if (p.q)     st = tk_kv_decode(h, p.layer, h->hs_q[p.set], h->hs_out[p.set], s);
    }
    if (e == cudaSuccess) e = cudaEventRecord(h->ev_group, s);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(h->st_out, h->ev_group, 0);
    for (size_t i = 0; i < pend.size() && e == cudaSuccess; i++) {
        const auto& p = pend[i];
        if (p.q && st == TK_OK) {
            e = cudaMemcpyAsync(p.out_host, h->hs_out[p.set], p.o_bytes, cudaMemcpyDeviceToHost, h->st_out);
            h->stats.bytes_d2h += (int64_t)p.o_bytes;
        }
        if (e == cudaSuccess) e = cudaEventRecord(h->ev_free[p.set], h->st_out);
    }
    if (e == cudaSuccess) e = cudaEventRecord(h->ev_out_all, h->st_out);
    h->host_flushing = false;
    if (st != TK_OK) return st;
    if (e != cudaSuccess) return fail(h, TK_CUDA_ERROR, cudaGetErrorString(e));
    return TK_OK;
}

static int append_decode_host_impl(tk_kv* h, int32_t layer, const void* k_host, const void* v_host,
                                   const void* q_host, void* out_host, void* stream, bool wait) {
    if (!h || layer < 0 || layer >= h->cfg.num_layers) return TK_INVALID_ARG;
    if (h->host_only) return fail(h, TK_CUDA_ERROR, "append_decode_host: handle has no device");
    if (!h->have_step) return fail(h, TK_INVALID_ARG, "append_decode_host: no step in progress");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t kv_bytes = (size_t)h->dev.n_tokens * h->cfg.num_kv_heads * h->cfg.head_dim * 2;
    const size_t vv_bytes = (size_t)h->dev.n_tokens * h->cfg.num_kv_heads * h->cfg.v_head_dim * 2;
    const size_t q_bytes = (size_t)h->dev.n_seqs * h->cfg.num_heads * h->cfg.head_dim * 2;
    const size_t o_bytes = (size_t)h->dev.n_seqs * h->cfg.num_heads * h->cfg.v_head_dim * 2;
    if (kv_bytes && (!k_host || !v_host)) return fail(h, TK_INVALID_ARG, "append_decode_host: null k/v");
    if (q_bytes && (!q_host || !out_host)) return fail(h, TK_INVALID_ARG, "append_decode_host: null q/out");
    if (!h->host_pending.empty() && h->host_pending_stream != s) {      // one group, one stream
        const int st = host_flush(h);
        if (st != TK_OK) return st;
    }
    const int set = (int)(h->host_calls++ % (uint64_t)h->host_sets);
    TK_CUDA(h, cudaStreamWaitEvent(h->st_in, h->ev_free[set], 0));
    if (kv_bytes) {
        TK_CUDA(h, cudaMemcpyAsync(h->hs_k[set], k_host, kv_bytes, cudaMemcpyHostToDevice, h->st_in));
        TK_CUDA(h, cudaMemcpyAsync(h->hs_v[set], v_host, vv_bytes, cudaMemcpyHostToDevice, h->st_in));
        h->stats.bytes_h2d += (int64_t)kv_bytes + (int64_t)vv_bytes;
    }
    if (q_bytes) {
        TK_CUDA(h, cudaMemcpyAsync(h->hs_q[set], q_host, q_bytes, cudaMemcpyHostToDevice, h->st_in));
        h->stats.bytes_h2d += (int64_t)q_bytes;
    }
    TK_CUDA(h, cudaEventRecord(h->ev_in[set], h->st_in));
    h->host_pending.push_back({layer, set, kv_bytes != 0, q_bytes != 0, out_host, o_bytes});
    h->host_pending_stream = s;
    const int c = h->host_calls_in_step++;
    const int group = std::min(h->host_group, c < 2 ? 1 : (c < 6 ? 2 : 4));   // 1, 1, 2, 2, 4, 4, ...
    if (wait || (int)h->host_pending.size() >= group) {
        const int st = host_flush(h);
        if (st != TK_OK) return st;
    }
    if (wait) {
        TK_CUDA(h, cudaStreamSynchronize(s));
        TK_CUDA(h, cudaStreamSynchronize(h->st_out));
    }
    return TK_OK;
}

int tk_kv_host_wait(tk_kv* h, void* stream) {
    if (!h || h->host_only) return TK_INVALID_ARG;
    const int st = host_flush(h);
    if (st != TK_OK) return st;
    TK_CUDA(h, cudaStreamWaitEvent((cudaStream_t)stream, h->ev_out_all, 0));
    return TK_OK;
}

int tk_kv_append_decode_host(tk_kv* h, int32_t layer, const void* k_host, const void* v_host,
                             const void* q_host, void* out_host, void* stream) {
    return append_decode_host_impl(h, layer, k_host, v_host, q_host, out_host, stream, true);
}
int tk_kv_append_decode_host_async(tk_kv* h, int32_t layer, const void* k_host, const void* v_host,
                                   const void* q_host, void* out_host, void* stream) {
    return append_decode_host_impl(h, layer, k_host, v_host, q_host, out_host, stream, false);
}

int tk_kv_profile_enable(tk_kv* h, int32_t max_launches) {
    if (!h || h->host_only || max_launches < 0) return TK_INVALID_ARG;
    TK_CUDA(h, cudaSetDevice(h->device));
    while (h->prof_ev.size() < 2 * (size_t)max_launches) {
        cudaEvent_t e;
        TK_CUDA(h, cudaEventCreate(&e));
        h->prof_ev.push_back(e);
    }
    h->prof_used = 0;
    h->profiling = max_launches > 0;
    return TK_OK;
}
int tk_kv_profile_read(tk_kv* h, double* total_ms, int64_t* launches) {
    if (!h || h->host_only || !total_ms || !launches) return TK_INVALID_ARG;
    double sum = 0.0;
    for (size_t i = 0; i + 1 < h->prof_used; i += 2) {
        TK_CUDA(h, cudaEventSynchronize(h->prof_ev[i + 1]));
        float ms = 0.0f;
        TK_CUDA(h, cudaEventElapsedTime(&ms, h->prof_ev[i], h->prof_ev[i + 1]));
        sum += ms;
    }
    *total_ms = sum;
    *launches = (int64_t)(h->prof_used / 2);
    h->prof_used = 0;
    return TK_OK;
}

int tk_kv_profile_read_each(tk_kv* h, float* ms_out, int32_t cap, int32_t* launches) {
    if (!h || h->host_only || !launches || cap < 0 || (cap > 0 && !ms_out)) return TK_INVALID_ARG;
    int32_t n = 0;
    for (size_t i = 0; i + 1 < h->prof_used; i += 2, n++) {
        TK_CUDA(h, cudaEventSynchronize(h->prof_ev[i + 1]));
        float ms = 0.0f;
        TK_CUDA(h, cudaEventElapsedTime(&ms, h->prof_ev[i], h->prof_ev[i + 1]));
        if (n < cap) ms_out[n] = ms;
    }
    *launches = n;
    h->prof_used = 0;
    return TK_OK;
}

int tk_kv_device_status(tk_kv* h, void* stream) {
    if (!h || h->host_only) return TK_INVALID_ARG;
    if (const int fs = host_flush(h)) return fs;               // launches the host-buffer calls still hold back come first
    int st = 0;
    TK_CUDA(h, cudaMemcpyAsync(&st, h->d_status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    TK_CUDA(h, cudaStreamSynchronize((cudaStream_t)stream));
    if (st != 0) {
        cudaMemsetAsync(h->d_status, 0, sizeof(int), (cudaStream_t)stream);
        // CTAs that gave up may have left arrival counters of the in-kernel merges half counted
        cudaMemsetAsync(h->d_counters, 0, sizeof(int) * 8 * (size_t)h->cfg.max_seqs * h->cfg.num_kv_heads, (cudaStream_t)stream);
        cudaMemsetAsync(h->d_pf_counters, 0, sizeof(int) * (size_t)h->max_pf_groups, (cudaStream_t)stream);
        return fail(h, st, "a device-side wait gave up (status %d)", st);
    }
    return TK_OK;
}

int tk_kv_selftest_bounded_wait(tk_kv* h, int32_t limit_ms, void* stream) {
    if (!h || h->host_only || limit_ms <= 0 || limit_ms > 2000) return TK_INVALID_ARG;
    cudaError_t e = tk::launch_bounded_wait_selftest(h->d_status, (unsigned long long)limit_ms * 1000000ull,
                                                     (cudaStream_t)stream);
    h->launches++;
    return e == cudaSuccess ? TK_OK : fail(h, TK_CUDA_ERROR, "selftest launch: %s", cudaGetErrorString(e));
}

int tk_kv_selftest_set_status(tk_kv* h, int32_t value, void* stream) {
    if (!h || h->host_only) return TK_INVALID_ARG;
    if (value != TK_OK && value != TK_TIMEOUT) return fail(h, TK_INVALID_ARG, "selftest_set_status: value must be TK_OK or TK_TIMEOUT");
    TK_CUDA(h, cudaMemcpyAsync(h->d_status, &value, sizeof(int), cudaMemcpyHostToDevice, (cudaStream_t)stream));
    TK_CUDA(h, cudaStreamSynchronize((cudaStream_t)stream));      // `value` lives on this call's stack
    return TK_OK;
}

int tk_kv_check_canaries(tk_kv* h, void* stream) {
    if (!h || h->host_only) return TK_INVALID_ARG;
    TK_CUDA(h, cudaSetDevice(h->device));
    TK_CUDA(h, cudaStreamSynchronize((cudaStream_t)stream));
    std::vector<uint8_t> buf(kCanaryBytes);
    for (const auto& cn : h->canaries) {
        TK_CUDA(h, cudaMemcpy(buf.data(), cn.at, kCanaryBytes, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < kCanaryBytes; i++)
            if (buf[i] != (uint8_t)kCanaryByte)
                return fail(h, TK_CUDA_ERROR, "guard bytes behind the %s were overwritten (first at +%zu): a kernel wrote past its buffer",
                            cn.name, i);
    }
    return TK_OK;
}

int64_t tk_kv_launch_count(const tk_kv* h) { return h ? h->launches : 0; }

}  // extern "C"
