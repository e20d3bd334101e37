// inference/kv_cache.h — titan::KVCache over the paged B200 KV cache.
//
// Same class name, method names, argument meaning and error behaviour as the reference's
// KVCache (reference: src/inference/kv_cache.h:15-81, src/inference/kv_cache.cpp), so that
// its callers (DenseExecutor::forward_layer, src/model/dense.cpp:388-398;
// MoEExecutor::forward_layer, src/model/moe.cpp:832-838) compile unchanged against this
// header and link against libtitan_kv.so instead of the reference's kv_cache.o.
//
// What is different underneath:
//   * storage is a paged 16-bit pool (FP16 unless BF16 is asked for), not an FP32 slab:
//     update() narrows the FP32 row while scattering it to its page slot (one kernel instead
//     of two device-to-device copies), attention widens on the fly;
//   * k_cache(layer) / v_cache(layer) return addresses inside the cache's own device slabs
//     that identify (cache, layer) to cuda::attention_decode; they are tokens for that call,
//     not FP32 rows to be read directly;
//   * the MLA variant (initialize_external_mla: K rows of nope+rope dims, V rows of nope dims)
//     is served for the 192 / 128 shape.
#pragma once

#include "core/types.h"

#include <cuda_runtime.h>

struct tk_kv;

namespace titan {

class KVCache {
public:
    KVCache() = default;
    ~KVCache();
    KVCache(const KVCache&) = delete;
    KVCache& operator=(const KVCache&) = delete;

    // Allocates its own device memory.  false + a log line on failure, like the reference.
    bool initialize(uint32_t num_layers, uint32_t num_kv_heads, uint32_t head_dim,
                    uint32_t max_seq_len, DType dtype = DType::FP32);

    // Adopts caller-owned buffers sized as the reference sizes them
    // (num_layers * max_seq_len * num_kv_heads * head_dim floats each); never frees them.
    // k_buf holds the paged pool (16-bit K and V fit in the bytes of the FP32 K slab).
    bool initialize_external(uint32_t num_layers, uint32_t num_kv_heads, uint32_t head_dim,
                             uint32_t max_seq_len, float* k_buf, float* v_buf);

    bool initialize_external_mla(uint32_t num_layers, uint32_t num_kv_heads, uint32_t k_head_dim,
                                 uint32_t v_head_dim, uint32_t max_seq_len, float* k_buf, float* v_buf);

    float* k_cache(uint32_t layer) const;      // nullptr on a bad layer, like the reference
    float* v_cache(uint32_t layer) const;

    // key, value: device float[num_kv_heads * head_dim].  Silently ignores a bad layer or
    // position (reference: kv_cache.cpp:124-126); position >= seq_len() extends the sequence.
    void update(uint32_t layer, int position, const float* key, const float* value,
                cudaStream_t stream = nullptr);

    int  seq_len() const { return seq_len_; }
    void set_seq_len(int len);

    uint32_t num_layers() const { return num_layers_; }
    uint32_t num_kv_heads() const { return num_kv_heads_; }
    uint32_t head_dim() const { return head_dim_; }
    uint32_t k_head_dim() const { return head_dim_; }
    uint32_t v_head_dim() const { return v_head_dim_ > 0 ? v_head_dim_ : head_dim_; }
    uint32_t max_seq_len() const { return max_seq_len_; }

    size_t memory_bytes() const;
    void   clear();

    // ---- beyond the reference interface ---------------------------------------------
    tk_kv* handle() const { return h_; }       // the C-ABI handle underneath (include/titan_kv.h)

    // used by cuda::attention_decode
    bool attend(int layer, const float* q, float* out, int num_heads, int seq_len, cudaStream_t stream);

private:
    bool setup(uint32_t L, uint32_t Hkv, uint32_t D, uint32_t Dv, uint32_t max_seq, DType dtype, float* k_buf, float* v_buf);
    void release();

    tk_kv*   h_ = nullptr;
    float*   k_base_ = nullptr;        // slab holding the paged pool
    float*   v_base_ = nullptr;        // slab whose addresses only serve as v_cache() tokens
    void*    arena_ = nullptr;         // 1024-byte aligned start of the pool inside k_base_
    bool     owns_memory_ = true;
    uint32_t num_layers_ = 0, num_kv_heads_ = 0, head_dim_ = 0, v_head_dim_ = 0, max_seq_len_ = 0;
    int      seq_len_ = 0;
    int      capacity_ = 0;            // tokens the pool can hold (multiple of the page size)
    int      seq_ = -1;                // sequence slot inside the handle
    size_t   k_layer_stride_ = 0, v_layer_stride_ = 0;   // floats between consecutive k_cache()/v_cache() tokens
    size_t   k_bytes_ = 0, v_bytes_ = 0;
    int      store_dtype_ = 1;
    int      planned_len_ = -1, planned_heads_ = -1;     // what the uploaded decode plan was made for
};

}  // namespace titan
