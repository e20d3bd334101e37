// standalone/compute/dispatch.h — the attention operators of the reference's operator header
// (reference: src/compute/dispatch.h:68-79), served by the paged B200 KV cache.  For builds outside
// the reference tree; inside it the reference's own dispatch.h declares the same four functions.
#pragma once

#include <cuda_runtime.h>

namespace titan {
namespace cuda {

// softmax(q K^T / sqrt(D)) V for one query token over the first seq_len cached tokens, GQA.
// q, output: device float[num_heads * head_dim].  k_cache / v_cache must be the values
// KVCache::k_cache(layer) / v_cache(layer) returned: they name the cache and the layer.
// Like the reference's launcher it returns void and reports problems on stderr only.
void attention_decode(const float* q, const float* k_cache, const float* v_cache, float* output,
                      int num_heads, int num_kv_heads, int head_dim, int seq_len, cudaStream_t stream);

// The same with K rows (and q) of k_head_dim and V rows / output of v_head_dim
// (reference: attention_decode_mla, src/compute/cuda/attention.cu:168-253,332-349).
void attention_decode_mla(const float* q, const float* k_cache, const float* v_cache, float* output,
                          int num_heads, int num_kv_heads, int k_head_dim, int v_head_dim, int seq_len,
                          cudaStream_t stream);

// Interleaved-pair RoPE on q [num_heads, head_dim] and k [num_kv_heads, head_dim] in place
// (reference: rope_kernel, src/compute/cuda/attention.cu:15-48).
void apply_rope(float* q, float* k, int num_heads, int num_kv_heads, int head_dim, int position,
                float theta, float scaling, cudaStream_t stream);
// The same on the rope dims only: the last rope_hd dims of rows of nope_hd + rope_hd
// (reference: rope_mla_kernel, src/compute/cuda/attention.cu:259-294,351-366).
void apply_rope_mla(float* q, float* k, int num_heads, int num_kv_heads, int nope_hd, int rope_hd, int position,
                    float theta, cudaStream_t stream);

}  // namespace cuda
}  // namespace titan
