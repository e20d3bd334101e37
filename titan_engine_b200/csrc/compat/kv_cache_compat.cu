// kv_cache_compat.cu — titan::KVCache and titan::cuda::attention_decode / apply_rope with the
// reference's signatures, implemented over the paged KV cache's C ABI (include/titan_kv.h).
//
// Call sites this serves unchanged (reference): src/model/dense.cpp:382-398,
// src/model/moe.cpp:832-838, src/inference/engine.cpp:137-142.
#include "inference/kv_cache.h"
#include "compute/dispatch.h"

#include "../../../include/titan_kv.h"
#include "../tk_kernels.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <mutex>
#include <vector>

namespace titan {

namespace {

constexpr int kPage = 16;

#define KV_LOG(fmt, ...) fprintf(stderr, "[titan-kv] " fmt "\n", ##__VA_ARGS__)

// k_cache() tokens -> owning cache, so that attention_decode(float* k_cache, ...) can find it
struct Registry {
    std::mutex mu;
    std::vector<KVCache*> caches;
} g_registry;

// One token's K and V rows: FP32 -> 16-bit while scattering to the page slot.
// grid covers Hkv*D elements; dst rows are D contiguous 16-bit values.
// grid covers Hkv*(D + Dv) elements: first the K row elements, then the V row elements.
__global__ void compat_update_kernel(void* __restrict__ pool, const float* __restrict__ key,
                                     const float* __restrict__ value, int Hkv, int D, int Dv, int page, int r,
                                     int bf16) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= Hkv * (D + Dv)) return;
    const bool is_v = i >= Hkv * D;
    if (is_v) i -= Hkv * D;
    const int dim = is_v ? Dv : D;
    const int h = i / dim, d = i % dim;
    // tile of (page, head): kPage K rows of D, then kPage V rows of Dv
    const size_t off = ((size_t)page * Hkv + h) * kPage * (D + Dv) + (is_v ? (size_t)kPage * D : 0) + (size_t)r * dim + d;
    const float x = is_v ? value[i] : key[i];
    if (bf16) ((__nv_bfloat16*)pool)[off] = __float2bfloat16_rn(x);
    else      ((__half*)pool)[off] = __float2half_rn(x);
}

}  // namespace

KVCache::~KVCache() { release(); }

void KVCache::release() {
    {
        std::lock_guard<std::mutex> lock(g_registry.mu);
        auto& v = g_registry.caches;
        for (size_t i = 0; i < v.size(); i++)
            if (v[i] == this) { v.erase(v.begin() + (ptrdiff_t)i); break; }
    }
    if (h_) { tk_kv_destroy(h_); h_ = nullptr; }
    if (owns_memory_) {
        if (k_base_) cudaFree(k_base_);
        if (v_base_) cudaFree(v_base_);
    }
    k_base_ = v_base_ = nullptr;
    arena_ = nullptr;
}

bool KVCache::setup(uint32_t L, uint32_t Hkv, uint32_t D, uint32_t Dv, uint32_t max_seq, DType dtype, float* k_buf,
                    float* v_buf) {
    release();
    num_layers_ = L; num_kv_heads_ = Hkv; head_dim_ = D; v_head_dim_ = Dv == D ? 0 : Dv; max_seq_len_ = max_seq;
    seq_len_ = 0; planned_len_ = planned_heads_ = -1;
    if (dtype != DType::FP32 && dtype != DType::FP16 && dtype != DType::BF16) {
        // FP8 pools need the step interface (open pages, sealing); this class appends row by row
        KV_LOG("KV cache: storage dtype %d is not served through titan::KVCache (FP32/FP16 -> fp16 pool, BF16 -> bf16 "
               "pool); FP8-E4M3 pools are behind the C ABI (tk_kv_create with dtype TK_FP8_E4M3)", (int)dtype);
        return false;
    }
    store_dtype_ = dtype == DType::BF16 ? TK_BF16 : TK_FP16;    // FP32 / FP16 requests are stored as FP16
    const size_t ref_stride = (size_t)max_seq * Hkv * D;        // floats per layer in the reference's K slab
    const size_t ref_vstride = (size_t)max_seq * Hkv * Dv;      // ... and in its V slab
    const size_t tile = (size_t)Hkv * kPage * (D + Dv) * 2;      // bytes of one page of one layer
    int pages = (int)((max_seq + kPage - 1) / kPage);
    if (L == 0 || Hkv == 0 || tile == 0 || pages == 0) { KV_LOG("KV cache: bad dimensions"); return false; }

    owns_memory_ = k_buf == nullptr;
    if (owns_memory_) {
        k_bytes_ = (size_t)L * pages * tile + 1024;
        if (k_bytes_ < (size_t)L * ref_stride * sizeof(float)) k_bytes_ = (size_t)L * ref_stride * sizeof(float);
        v_bytes_ = (size_t)L * 256;
        cudaError_t e = cudaMalloc((void**)&k_base_, k_bytes_);
        if (e != cudaSuccess) {
            KV_LOG("KV cache: failed to allocate the pool (%.1f MB): %s", k_bytes_ / 1e6, cudaGetErrorString(e));
            k_base_ = nullptr;
            return false;
        }
        e = cudaMalloc((void**)&v_base_, v_bytes_);
        if (e != cudaSuccess) {
            KV_LOG("KV cache: failed to allocate (%zu B): %s", v_bytes_, cudaGetErrorString(e));
            cudaFree(k_base_); k_base_ = nullptr; v_base_ = nullptr;
            return false;
        }
        v_layer_stride_ = 64;
    } else {
        k_base_ = k_buf; v_base_ = v_buf;
        k_bytes_ = (size_t)L * ref_stride * sizeof(float);
        v_bytes_ = (size_t)L * ref_vstride * sizeof(float);
        v_layer_stride_ = ref_vstride;
    }
    k_layer_stride_ = ref_stride;
    const size_t shift = (1024 - ((uintptr_t)k_base_ & 1023)) & 1023;
    arena_ = (char*)k_base_ + shift;
    const size_t avail = k_bytes_ - shift;
    if ((size_t)L * pages * tile > avail) pages = (int)(avail / ((size_t)L * tile));
    if (pages <= 0) { KV_LOG("KV cache: buffer too small for one page per layer"); return false; }
    capacity_ = pages * kPage;

    tk_kv_config cfg;
    tk_kv_config_default(&cfg);
    cfg.num_layers = (int)L; cfg.num_kv_heads = (int)Hkv; cfg.num_heads = (int)Hkv * 16;  // real count comes with attention_decode
    cfg.head_dim = (int)D; cfg.v_head_dim = Dv == D ? 0 : (int)Dv; cfg.page_size = kPage; cfg.dtype = store_dtype_; cfg.io_dtype = store_dtype_;
    cfg.num_pages = pages; cfg.max_seqs = 1; cfg.max_pages_per_seq = pages; cfg.max_step_tokens = kPage;
    int st = tk_kv_create_external(&cfg, arena_, avail, &h_);
    if (st != TK_OK) {
        KV_LOG("KV cache: %s", tk_kv_last_error(nullptr));
        h_ = nullptr;
        if (owns_memory_) { cudaFree(k_base_); cudaFree(v_base_); }
        k_base_ = v_base_ = nullptr;
        return false;
    }
    int32_t s = -1;
    tk_kv_seq_alloc(h_, &s);
    seq_ = s;
    {
        std::lock_guard<std::mutex> lock(g_registry.mu);
        g_registry.caches.push_back(this);
    }
    fprintf(stderr, "[titan-kv] KV cache: %u layers, %u heads, dim=%u, max_seq=%u (paged %s, %.1f MB%s)\n", L, Hkv, D,
            max_seq, store_dtype_ == TK_BF16 ? "bf16" : "fp16", tk_kv_memory_bytes(h_) / 1e6,
            owns_memory_ ? "" : ", pool-backed");
    return true;
}

bool KVCache::initialize(uint32_t num_layers, uint32_t num_kv_heads, uint32_t head_dim, uint32_t max_seq_len,
                         DType dtype) {
    return setup(num_layers, num_kv_heads, head_dim, head_dim, max_seq_len, dtype, nullptr, nullptr);
}

bool KVCache::initialize_external(uint32_t num_layers, uint32_t num_kv_heads, uint32_t head_dim,
                                  uint32_t max_seq_len, float* k_buf, float* v_buf) {
    if (!k_buf || !v_buf) return false;                       // reference: kv_cache.cpp:62
    return setup(num_layers, num_kv_heads, head_dim, head_dim, max_seq_len, DType::FP32, k_buf, v_buf);
}

bool KVCache::initialize_external_mla(uint32_t num_layers, uint32_t num_kv_heads, uint32_t k_head_dim,
                                      uint32_t v_head_dim, uint32_t max_seq_len, float* k_buf, float* v_buf) {
    if (!k_buf || !v_buf) return false;                       // reference: kv_cache.cpp:87
    return setup(num_layers, num_kv_heads, k_head_dim, v_head_dim, max_seq_len, DType::FP32, k_buf, v_buf);
}

float* KVCache::k_cache(uint32_t layer) const {
    if (!k_base_ || layer >= num_layers_) return nullptr;
    return k_base_ + layer * k_layer_stride_;
}

float* KVCache::v_cache(uint32_t layer) const {
    if (!v_base_ || layer >= num_layers_) return nullptr;
    return v_base_ + layer * v_layer_stride_;
}

void KVCache::update(uint32_t layer, int position, const float* key, const float* value, cudaStream_t stream) {
    if (!h_ || !key || !value) return;
    if (position < 0) return;
    if (layer >= num_layers_ || position >= (int)max_seq_len_ || position >= capacity_) return;
    const int cur = tk_kv_seq_len(h_, seq_);
    if (position >= cur && tk_kv_reserve(h_, seq_, position + 1 - cur) != TK_OK) return;
    const int64_t slot = tk_kv_slot(h_, seq_, position);
    if (slot < 0) return;
    void* pool = nullptr;
    if (tk_kv_layer_ptrs(h_, (int)layer, &pool, nullptr, nullptr) != TK_OK) return;
    const int n = (int)(num_kv_heads_ * (head_dim_ + v_head_dim()));
    compat_update_kernel<<<(n + 255) / 256, 256, 0, stream>>>(pool, key, value, (int)num_kv_heads_, (int)head_dim_,
                                                              (int)v_head_dim(), (int)(slot / kPage),
                                                              (int)(slot % kPage), store_dtype_ == TK_BF16);
    if (position >= seq_len_) seq_len_ = position + 1;         // reference: kv_cache.cpp:148-150
}

void KVCache::set_seq_len(int len) {
    if (len < 0) len = 0;
    if (h_) {
        const int cur = tk_kv_seq_len(h_, seq_);
        if (len < cur) tk_kv_truncate(h_, seq_, len);
        else if (len > cur && len <= capacity_) tk_kv_reserve(h_, seq_, len - cur);
    }
    seq_len_ = len;
    planned_len_ = -1;
}

size_t KVCache::memory_bytes() const { return k_bytes_ + v_bytes_; }

void KVCache::clear() {
    seq_len_ = 0;
    planned_len_ = -1;
    if (!h_) return;
    tk_kv_seq_free(h_, seq_);
    int32_t s = -1;
    tk_kv_seq_alloc(h_, &s);
    seq_ = s;
    cudaMemset(arena_, 0, tk_kv_memory_bytes(h_));              // the reference zeroes its slabs too (:160-166)
}

bool KVCache::attend(int layer, const float* q, float* out, int num_heads, int seq_len, cudaStream_t stream) {
    if (!h_ || layer < 0 || layer >= (int)num_layers_ || !q || !out) return false;
    if (num_heads != planned_heads_) {
        if (tk_kv_set_num_heads(h_, num_heads) != TK_OK) { KV_LOG("attention_decode: %s", tk_kv_last_error(h_)); return false; }
    }
    int32_t cap = seq_len < 0 ? 0 : seq_len;
    const int cur = tk_kv_seq_len(h_, seq_);
    if (cap > cur) cap = cur;
    if (cap != planned_len_ || num_heads != planned_heads_) {
        int32_t seq = seq_;
        if (tk_kv_step_begin_capped(h_, 1, &seq, nullptr, &cap, stream) != TK_OK) {
            KV_LOG("attention_decode: %s", tk_kv_last_error(h_));
            return false;
        }
        planned_len_ = cap;
        planned_heads_ = num_heads;
    }
    if (tk_kv_decode_ex(h_, layer, q, TK_FP32, out, TK_FP32, stream) != TK_OK) {
        KV_LOG("attention_decode: %s", tk_kv_last_error(h_));
        return false;
    }
    return true;
}

namespace cuda {

static void attend_impl(const char* what, const float* q, const float* k_cache, float* output, int num_heads,
                        int num_kv_heads, int head_dim, int v_head_dim, int seq_len, cudaStream_t stream) {
    KVCache* owner = nullptr;
    int layer = -1;
    {
        std::lock_guard<std::mutex> lock(g_registry.mu);
        for (KVCache* c : g_registry.caches) {
            const float* base = c->k_cache(0);
            if (!base || k_cache < base) continue;
            const size_t stride = c->num_layers() > 1 ? (size_t)(c->k_cache(1) - base) : 1;
            const size_t off = (size_t)(k_cache - base);
            if (off % stride == 0 && off / stride < c->num_layers()) { owner = c; layer = (int)(off / stride); break; }
        }
    }
    if (!owner) {
        KV_LOG("%s: k_cache %p was not returned by a KVCache::k_cache(); nothing launched", what, (const void*)k_cache);
        return;
    }
    if ((int)owner->num_kv_heads() != num_kv_heads || (int)owner->k_head_dim() != head_dim ||
        (int)owner->v_head_dim() != v_head_dim) {
        KV_LOG("%s: shape (%d kv heads, dims %d/%d) does not match the cache (%u, %u/%u)", what, num_kv_heads, head_dim,
               v_head_dim, owner->num_kv_heads(), owner->k_head_dim(), owner->v_head_dim());
        return;
    }
    owner->attend(layer, q, output, num_heads, seq_len, stream);
}

void attention_decode(const float* q, const float* k_cache, const float* v_cache, float* output, int num_heads,
                      int num_kv_heads, int head_dim, int seq_len, cudaStream_t stream) {
    (void)v_cache;
    attend_impl("attention_decode", q, k_cache, output, num_heads, num_kv_heads, head_dim, head_dim, seq_len, stream);
}

void attention_decode_mla(const float* q, const float* k_cache, const float* v_cache, float* output, int num_heads,
                          int num_kv_heads, int k_head_dim, int v_head_dim, int seq_len, cudaStream_t stream) {
    (void)v_cache;
    attend_impl("attention_decode_mla", q, k_cache, output, num_heads, num_kv_heads, k_head_dim, v_head_dim, seq_len, stream);
}

// Both run the library's own FP32 rotation kernel (rope_append.cu).
void apply_rope(float* q, float* k, int num_heads, int num_kv_heads, int head_dim, int position, float theta,
                float scaling, cudaStream_t stream) {
    if (head_dim < 2 || num_heads < 0 || num_kv_heads < 0) return;
    tk::launch_rope_f32(q, k, num_heads, num_kv_heads, head_dim, 0, head_dim, position, theta, scaling, stream);
}

void apply_rope_mla(float* q, float* k, int num_heads, int num_kv_heads, int nope_hd, int rope_hd, int position,
                    float theta, cudaStream_t stream) {
    if (rope_hd < 2 || nope_hd < 0 || num_heads < 0 || num_kv_heads < 0) return;
    tk::launch_rope_f32(q, k, num_heads, num_kv_heads, nope_hd + rope_hd, nope_hd, rope_hd, position, theta, 1.0f, stream);
}

}  // namespace cuda
}  // namespace titan
