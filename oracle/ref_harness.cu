// ref_harness.cu — drives the UNMODIFIED reference sources (compiled from where
// they lie by oracle/Makefile, target `ref`) so that the CPU oracle can be
// pinned against the reference's real kernels.  TEST INFRASTRUCTURE ONLY.
//
// All pointers are HOST pointers; the harness owns the device round trip, so a
// test needs nothing but ctypes + numpy.
#include "inference/kv_cache.h"      // titan::KVCache   (reference: src/inference/kv_cache.h:15-81)
#include "compute/dispatch.h"        // titan::cuda::attention_decode / apply_rope (src/compute/dispatch.h:68-75)

#include <cuda_runtime.h>
#include <vector>

#define TKREF_CHECK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) return (int)e_; } while (0)

extern "C" {

// Append `seq_len` tokens one by one through KVCache::update for every layer,
// then run cuda::attention_decode on layer `layer`.
//   k, v : [num_layers][seq_len][Hkv][D] FP32 (host)     q : [H][D]     out : [H][D]
// Returns 0, or the cudaError_t of the first failing call (the Release build of
// the reference does not report a failed launch itself: cuda_check.h:8-18).
int tkref_update_and_decode(const float* k, const float* v, const float* q, float* out,
                            int num_layers, int layer, int H, int Hkv, int D,
                            int seq_len, int max_seq_len, int* seq_len_out) {
    titan::KVCache cache;
    if (!cache.initialize(num_layers, Hkv, D, max_seq_len)) return -1;
    size_t row = (size_t)Hkv * D;
    float *dk = nullptr, *dv = nullptr, *dq = nullptr, *dout = nullptr;
    TKREF_CHECK(cudaMalloc(&dk, row * sizeof(float)));
    TKREF_CHECK(cudaMalloc(&dv, row * sizeof(float)));
    TKREF_CHECK(cudaMalloc(&dq, (size_t)H * D * sizeof(float)));
    TKREF_CHECK(cudaMalloc(&dout, (size_t)H * D * sizeof(float)));
    cudaStream_t stream;
    TKREF_CHECK(cudaStreamCreate(&stream));
    for (int pos = 0; pos < seq_len; pos++) {
        for (int l = 0; l < num_layers; l++) {
            size_t off = ((size_t)l * seq_len + pos) * row;
            TKREF_CHECK(cudaMemcpyAsync(dk, k + off, row * sizeof(float), cudaMemcpyHostToDevice, stream));
            TKREF_CHECK(cudaMemcpyAsync(dv, v + off, row * sizeof(float), cudaMemcpyHostToDevice, stream));
            cache.update(l, pos, dk, dv, stream);
            TKREF_CHECK(cudaStreamSynchronize(stream));
        }
    }
    if (seq_len_out) *seq_len_out = cache.seq_len();
    TKREF_CHECK(cudaMemcpyAsync(dq, q, (size_t)H * D * sizeof(float), cudaMemcpyHostToDevice, stream));
    titan::cuda::attention_decode(dq, cache.k_cache(layer), cache.v_cache(layer), dout,
                                  H, Hkv, D, cache.seq_len(), stream);
    TKREF_CHECK(cudaGetLastError());
    TKREF_CHECK(cudaMemcpyAsync(out, dout, (size_t)H * D * sizeof(float), cudaMemcpyDeviceToHost, stream));
    TKREF_CHECK(cudaStreamSynchronize(stream));
    cudaStreamDestroy(stream);
    cudaFree(dk); cudaFree(dv); cudaFree(dq); cudaFree(dout);
    return 0;
}

// cuda::attention_decode alone on contiguous host arrays k,v: [seq_len][Hkv][D].
int tkref_attention_decode(const float* q, const float* k, const float* v, float* out,
                           int H, int Hkv, int D, int seq_len) {
    size_t kv_bytes = (size_t)seq_len * Hkv * D * sizeof(float), q_bytes = (size_t)H * D * sizeof(float);
    float *dk = nullptr, *dv = nullptr, *dq = nullptr, *dout = nullptr;
    TKREF_CHECK(cudaMalloc(&dk, kv_bytes));
    TKREF_CHECK(cudaMalloc(&dv, kv_bytes));
    TKREF_CHECK(cudaMalloc(&dq, q_bytes));
    TKREF_CHECK(cudaMalloc(&dout, q_bytes));
    TKREF_CHECK(cudaMemcpy(dk, k, kv_bytes, cudaMemcpyHostToDevice));
    TKREF_CHECK(cudaMemcpy(dv, v, kv_bytes, cudaMemcpyHostToDevice));
    TKREF_CHECK(cudaMemcpy(dq, q, q_bytes, cudaMemcpyHostToDevice));
    titan::cuda::attention_decode(dq, dk, dv, dout, H, Hkv, D, seq_len, nullptr);
    TKREF_CHECK(cudaGetLastError());
    TKREF_CHECK(cudaDeviceSynchronize());
    TKREF_CHECK(cudaMemcpy(out, dout, q_bytes, cudaMemcpyDeviceToHost));
    cudaFree(dk); cudaFree(dv); cudaFree(dq); cudaFree(dout);
    return 0;
}

// cuda::attention_decode_mla on contiguous host arrays k: [seq_len][Hkv][Dk], v: [seq_len][Hkv][Dv].
int tkref_attention_decode_mla(const float* q, const float* k, const float* v, float* out,
                               int H, int Hkv, int Dk, int Dv, int seq_len) {
    size_t k_bytes = (size_t)seq_len * Hkv * Dk * sizeof(float), v_bytes = (size_t)seq_len * Hkv * Dv * sizeof(float);
    size_t q_bytes = (size_t)H * Dk * sizeof(float), o_bytes = (size_t)H * Dv * sizeof(float);
    float *dk = nullptr, *dv = nullptr, *dq = nullptr, *dout = nullptr;
    TKREF_CHECK(cudaMalloc(&dk, k_bytes));
    TKREF_CHECK(cudaMalloc(&dv, v_bytes));
    TKREF_CHECK(cudaMalloc(&dq, q_bytes));
    TKREF_CHECK(cudaMalloc(&dout, o_bytes));
    TKREF_CHECK(cudaMemcpy(dk, k, k_bytes, cudaMemcpyHostToDevice));
    TKREF_CHECK(cudaMemcpy(dv, v, v_bytes, cudaMemcpyHostToDevice));
    TKREF_CHECK(cudaMemcpy(dq, q, q_bytes, cudaMemcpyHostToDevice));
    titan::cuda::attention_decode_mla(dq, dk, dv, dout, H, Hkv, Dk, Dv, seq_len, nullptr);
    TKREF_CHECK(cudaGetLastError());
    TKREF_CHECK(cudaDeviceSynchronize());
    TKREF_CHECK(cudaMemcpy(out, dout, o_bytes, cudaMemcpyDeviceToHost));
    cudaFree(dk); cudaFree(dv); cudaFree(dq); cudaFree(dout);
    return 0;
}

// cuda::apply_rope in place on host arrays q: [H][D], k: [Hkv][D].
int tkref_apply_rope(float* q, float* k, int H, int Hkv, int D, int position,
                     float theta, float scaling) {
    size_t qb = (size_t)H * D * sizeof(float), kb = (size_t)Hkv * D * sizeof(float);
    float *dq = nullptr, *dk = nullptr;
    TKREF_CHECK(cudaMalloc(&dq, qb));
    TKREF_CHECK(cudaMalloc(&dk, kb));
    TKREF_CHECK(cudaMemcpy(dq, q, qb, cudaMemcpyHostToDevice));
    TKREF_CHECK(cudaMemcpy(dk, k, kb, cudaMemcpyHostToDevice));
    titan::cuda::apply_rope(dq, dk, H, Hkv, D, position, theta, scaling, nullptr);
    TKREF_CHECK(cudaGetLastError());
    TKREF_CHECK(cudaDeviceSynchronize());
    TKREF_CHECK(cudaMemcpy(q, dq, qb, cudaMemcpyDeviceToHost));
    TKREF_CHECK(cudaMemcpy(k, dk, kb, cudaMemcpyDeviceToHost));
    cudaFree(dq); cudaFree(dk);
    return 0;
}

// cuda::apply_rope_mla in place on host arrays q: [H][nope+rope], k: [Hkv][nope+rope].
int tkref_apply_rope_mla(float* q, float* k, int H, int Hkv, int nope_hd, int rope_hd, int position, float theta) {
    size_t qb = (size_t)H * (nope_hd + rope_hd) * sizeof(float), kb = (size_t)Hkv * (nope_hd + rope_hd) * sizeof(float);
    float *dq = nullptr, *dk = nullptr;
    TKREF_CHECK(cudaMalloc(&dq, qb));
    TKREF_CHECK(cudaMalloc(&dk, kb));
    TKREF_CHECK(cudaMemcpy(dq, q, qb, cudaMemcpyHostToDevice));
    TKREF_CHECK(cudaMemcpy(dk, k, kb, cudaMemcpyHostToDevice));
    titan::cuda::apply_rope_mla(dq, dk, H, Hkv, nope_hd, rope_hd, position, theta, nullptr);
    TKREF_CHECK(cudaGetLastError());
    TKREF_CHECK(cudaDeviceSynchronize());
    TKREF_CHECK(cudaMemcpy(q, dq, qb, cudaMemcpyDeviceToHost));
    TKREF_CHECK(cudaMemcpy(k, dk, kb, cudaMemcpyDeviceToHost));
    cudaFree(dq); cudaFree(dk);
    return 0;
}

}  // extern "C"
