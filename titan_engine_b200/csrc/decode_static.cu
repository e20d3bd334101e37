// decode_static.cu — paged decode attention for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc where they need attention: code that
// runs inside a serving loop which has handed all device memory to its own arena, a plugin
// loaded into a process whose allocator is owned by someone else, or a caller that wants a
// hard guarantee that a decode step never touches the driver's allocator.  For them
// tk_paged_decode_static() runs the same tensor-core split-KV decode + log-sum-exp combine as
// tk_kv_decode(), but needs no handle and no workspace: the caller passes the pool, the
// page table, the lengths, q and out, and the split-KV partials (plus the small work list)
// live in ONE fixed array that is part of the library image.
//
// Consequences of that choice, all of which the caller has to know:
//   * the array has a fixed size (kMaxSeqs sequences, kMaxItems work items, kMaxPartialFloats
//     floats of partials = 4 MiB); larger requests are refused, never truncated;
//   * every GPU that loads the library carries the array until the process exits;
//   * all calls on a device share it: two calls whose kernels can overlap on the GPU (different
//     streams, or different host threads) race on it.  Serialise them on one stream;
//   * the array keeps whatever the previous call left.  Each call rewrites the work list and every
//     partial row it later reads, and clears the one word that must start at zero (the status word a
//     timed-out device wait sets) with a stream-ordered memset;
//   * the device address of the array is looked up once per device, on that device's first
//     call;
//   * every call uploads its work list from host memory that lives only until the call returns,
//     so a call is refused while its stream is being captured into a graph.
#include "../../include/titan_kv.h"

#include "tk_kernels.cuh"

#include <algorithm>
#include <cstdio>
#include <mutex>
#include <vector>

namespace {

constexpr int kMaxSeqs = 256;
constexpr int kMaxItems = 4096;
constexpr size_t kMaxPartialFloats = (size_t)1 << 20;          // 4 MiB of (o, m, l) partial rows
constexpr int kPage = 16;

struct StaticScratch {
    int32_t status[4];                                             // [0]: set when a bounded device wait gives up
    int32_t seq[kMaxSeqs];
    int32_t len[kMaxSeqs];
    int32_t chunk_base[kMaxSeqs + 4];
    int4    items[kMaxItems];
    float   partials[kMaxPartialFloats];
};

// The scratch itself.  In host code this name is only a stand-in for the symbol; the
// address kernels can use comes from cudaGetSymbolAddress (scratch_for_current_device).
static __device__ __align__(256) unsigned char g_static_scratch[sizeof(StaticScratch)];

StaticScratch* g_scratch_addr[64] = {};
std::mutex g_scratch_mu;        // first calls on a device may come from several host threads

// Device address of the array on the current device; looked up on the first call per device.
cudaError_t scratch_for_current_device(StaticScratch** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_addr[dev] = (StaticScratch*)p;
    }
    *out = g_scratch_addr[dev];
    return cudaSuccess;
}

int refuse(const char* why) {
    fprintf(stderr, "[titan-kv] tk_paged_decode_static: %s\n", why);
    return TK_INVALID_ARG;
}

}  // namespace

extern "C" int tk_paged_decode_static(const void* pool, int32_t dtype, int32_t num_pages,
                                      const int32_t* page_table, int32_t max_pages_per_seq,
                                      const int32_t* seq_lens_host, int32_t n_seqs, int32_t num_heads,
                                      int32_t num_kv_heads, int32_t head_dim, const void* q, void* out,
                                      void* stream) {
    if (!pool || !page_table || !seq_lens_host || !q || !out) return refuse("null pointer argument");
    if (dtype != TK_FP16 && dtype != TK_BF16) return refuse("dtype must be TK_FP16 or TK_BF16");
    if (n_seqs <= 0 || n_seqs > kMaxSeqs) return refuse("n_seqs must be in 1..256");
    if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return refuse("num_heads must be a multiple of num_kv_heads");
    const int G = num_heads / num_kv_heads;
    if (G != 1 && G != 2 && G != 4 && G != 8 && G != 16) return refuse("heads per kv head must be 1, 2, 4, 8 or 16");
    if (head_dim != 64 && head_dim != 128) return refuse("head_dim must be 64 or 128");
    if (num_pages <= 0 || max_pages_per_seq <= 0) return refuse("num_pages and max_pages_per_seq must be positive");

    cudaStream_t s = (cudaStream_t)stream;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone)
        return refuse("the stream is being captured: this call uploads per-call host data and cannot be recorded");

    // split-KV chunk: the largest of 2048 .. 256 tokens that still gives the GPU a few hundred work items
    auto chunks_at = [&](int chunk) {
        int64_t total = 0;
        for (int b = 0; b < n_seqs; b++) total += ((int64_t)std::max(seq_lens_host[b], 0) + chunk - 1) / chunk;
        return total;
    };
    for (int b = 0; b < n_seqs; b++) {
        const int n = seq_lens_host[b];
        if (n < 0 || ((int64_t)n + kPage - 1) / kPage > max_pages_per_seq) return refuse("a sequence length does not fit its page-table row");
    }
    int chunk_tokens = 2048;
    while (chunk_tokens > 256 && chunks_at(chunk_tokens) * num_kv_heads < 592) chunk_tokens /= 2;
    // size check first, by arithmetic: nothing is built for a request that will be refused
    const int64_t total_chunks = chunks_at(chunk_tokens);
    if (total_chunks * num_kv_heads > kMaxItems)
        return refuse("too much work for the fixed scratch: more than 4096 (sequence, chunk, kv head) items");
    if ((size_t)total_chunks * num_heads * (head_dim + 2) > kMaxPartialFloats)
        return refuse("too much work for the fixed scratch: partial rows exceed 4 MiB (use tk_kv_decode with a handle)");

    // work list: one item per (sequence, chunk, kv head), built on the host
    std::vector<int32_t> seq(n_seqs), len(n_seqs), chunk_base(n_seqs + 1, 0);
    std::vector<int4> items;
    items.reserve((size_t)total_chunks * num_kv_heads);
    for (int b = 0; b < n_seqs; b++) {
        const int n = seq_lens_host[b];
        seq[b] = b;
        len[b] = n;
        const int chunks = (n + chunk_tokens - 1) / chunk_tokens;
        chunk_base[b + 1] = chunk_base[b] + chunks;
        for (int c = 0; c < chunks; c++)
            for (int h = 0; h < num_kv_heads; h++) items.push_back(make_int4(b, c, h, 0));
    }
    StaticScratch* sc = nullptr;
    cudaError_t e = scratch_for_current_device(&sc);
    if (e != cudaSuccess) {
        fprintf(stderr, "[titan-kv] tk_paged_decode_static: cudaGetSymbolAddress: %s\n", cudaGetErrorString(e));
        return TK_CUDA_ERROR;
    }
    // pageable sources: each copy is staged by the driver before the call returns
    if ((e = cudaMemcpyAsync(sc->seq, seq.data(), sizeof(int32_t) * n_seqs, cudaMemcpyHostToDevice, s)) != cudaSuccess ||
        (e = cudaMemcpyAsync(sc->len, len.data(), sizeof(int32_t) * n_seqs, cudaMemcpyHostToDevice, s)) != cudaSuccess ||
        (e = cudaMemcpyAsync(sc->chunk_base, chunk_base.data(), sizeof(int32_t) * (n_seqs + 1), cudaMemcpyHostToDevice, s)) != cudaSuccess ||
        (!items.empty() &&
         (e = cudaMemcpyAsync(sc->items, items.data(), sizeof(int4) * items.size(), cudaMemcpyHostToDevice, s)) != cudaSuccess)) {
        fprintf(stderr, "[titan-kv] tk_paged_decode_static: metadata copy: %s\n", cudaGetErrorString(e));
        return TK_CUDA_ERROR;
    }

    tk::Geometry g{num_heads, num_kv_heads, head_dim, kPage, dtype, dtype, num_pages, n_seqs, max_pages_per_seq, head_dim};
    tk::LayerPtrs lp{const_cast<void*>(pool), nullptr, nullptr, nullptr};
    // the pool as the TMA sees it: a descriptor built on the host and passed by value, nothing on the device
    CUtensorMap map;
    if ((e = tk::make_pool_tensor_map(g, const_cast<void*>(pool), &map)) != cudaSuccess ||
        (e = cudaMemsetAsync(sc->status, 0, sizeof(sc->status), s)) != cudaSuccess) {
        fprintf(stderr, "[titan-kv] tk_paged_decode_static: set-up: %s\n", cudaGetErrorString(e));
        return TK_CUDA_ERROR;
    }
    tk::StepDev st{};
    st.seq = sc->seq; st.len = sc->len; st.chunk_base = sc->chunk_base;
    st.items = sc->items;
    st.n_seqs = n_seqs; st.n_items = (int)items.size(); st.chunk_tokens = chunk_tokens;
    // the tensor-core decode kernel leaves (o, m, l) rows; the combine launch merges them and writes nothing
    // if a bounded wait inside the kernel gave up
    if ((st.n_items > 0 &&
         (e = tk::launch_decode_mma(g, lp, &map, nullptr, st, page_table, q, sc->partials, sc->status, s)) != cudaSuccess) ||
        (e = tk::launch_combine_step(g, st, sc->partials, out, dtype, nullptr, s, sc->status)) != cudaSuccess) {
        fprintf(stderr, "[titan-kv] tk_paged_decode_static: launch: %s\n", cudaGetErrorString(e));
        return TK_CUDA_ERROR;
    }
    return TK_OK;
}
