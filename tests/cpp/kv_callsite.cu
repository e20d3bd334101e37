// kv_callsite.cu — one source, two builds.  It uses titan::KVCache and the attention
// operators exactly the way the reference's layer loop does (rope -> update -> seq_len ->
// attention_decode; reference: src/model/dense.cpp:382-398) and dumps the attention outputs.
//   build A: reference headers + the reference's own objects (oracle/_ref/libtitan_ref.so)
//   build B: titan_engine_b200/csrc/compat headers + libtitan_kv.so
// tests/test_gpu_compat.py runs both and compares the dumps.
#include "inference/kv_cache.h"
#include "compute/dispatch.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#define CHECK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); return 2; } } while (0)

static uint32_t lcg(uint32_t& s) { s = s * 1664525u + 1013904223u; return s >> 8; }
// values with <= 10 significant bits: exactly representable in fp16 and in fp32
static float val(uint32_t& s) { return ((int)(lcg(s) % 1025) - 512) / 256.0f; }

// The MLA layer loop (reference: src/model/moe.cpp:832-838): K rows of nope+rope dims, V rows of
// nope dims, the cache placed in caller memory by initialize_external_mla.
static int run_mla(const char* path, int n_tokens) {
    const uint32_t L = 2, H = 8, Hkv = 8, Dk = 192, Dv = 128, max_seq = 256;
    titan::KVCache cache;
    float *kbuf = nullptr, *vbuf = nullptr;
    CHECK(cudaMalloc(&kbuf, (size_t)L * max_seq * Hkv * Dk * sizeof(float)));
    CHECK(cudaMalloc(&vbuf, (size_t)L * max_seq * Hkv * Dv * sizeof(float)));
    if (!cache.initialize_external_mla(L, Hkv, Dk, Dv, max_seq, kbuf, vbuf)) { fprintf(stderr, "initialize_external_mla failed\n"); return 3; }
    if (cache.k_head_dim() != Dk || cache.v_head_dim() != Dv || cache.seq_len() != 0) return 4;
    float *dq, *dk, *dv, *dout;
    CHECK(cudaMalloc(&dq, H * Dk * sizeof(float)));
    CHECK(cudaMalloc(&dk, Hkv * Dk * sizeof(float)));
    CHECK(cudaMalloc(&dv, Hkv * Dv * sizeof(float)));
    CHECK(cudaMalloc(&dout, H * Dv * sizeof(float)));
    cudaStream_t stream;
    CHECK(cudaStreamCreate(&stream));
    std::vector<float> q(H * Dk), k(Hkv * Dk), v(Hkv * Dv), out(H * Dv);
    FILE* f = fopen(path, "wb");
    if (!f) return 5;
    uint32_t seed = 777;
    for (int pos = 0; pos < n_tokens; pos++) {
        for (uint32_t l = 0; l < L; l++) {
            for (auto& x : q) x = val(seed);
            for (auto& x : k) x = val(seed);
            for (auto& x : v) x = val(seed);
            CHECK(cudaMemcpyAsync(dq, q.data(), q.size() * 4, cudaMemcpyHostToDevice, stream));
            CHECK(cudaMemcpyAsync(dk, k.data(), k.size() * 4, cudaMemcpyHostToDevice, stream));
            CHECK(cudaMemcpyAsync(dv, v.data(), v.size() * 4, cudaMemcpyHostToDevice, stream));
            titan::cuda::apply_rope_mla(dq, dk, H, Hkv, Dk - 64, 64, pos, 10000.0f, stream);
            cache.update(l, pos, dk, dv, stream);
            const int seq_len = cache.seq_len();
            if (seq_len != pos + 1) { fprintf(stderr, "seq_len %d at pos %d\n", seq_len, pos); return 6; }
            titan::cuda::attention_decode_mla(dq, cache.k_cache(l), cache.v_cache(l), dout, H, Hkv, Dk, Dv, seq_len, stream);
            CHECK(cudaGetLastError());
            CHECK(cudaMemcpyAsync(out.data(), dout, out.size() * 4, cudaMemcpyDeviceToHost, stream));
            CHECK(cudaStreamSynchronize(stream));
            fwrite(out.data(), 4, out.size(), f);
        }
    }
    fclose(f);
    printf("ok %d tokens (MLA), memory_bytes %zu\n", n_tokens, cache.memory_bytes());
    return 0;
}

int main(int argc, char** argv) {
    if (argc < 2) { fprintf(stderr, "usage: %s out.bin [n_tokens] [0 owned | 1 external | 2 external MLA | 3 storage types]\n", argv[0]); return 2; }
    const int n_tokens = argc > 2 ? atoi(argv[2]) : 150;
    const int mode = argc > 3 ? atoi(argv[3]) : 0;
    if (mode == 2) return run_mla(argv[1], n_tokens);
    if (mode == 3) {
        // storage types (RuntimeConfig::kv_cache_dtype, src/core/types.h:243-248): the reference ignores the argument;
        // the paged cache stores FP32/FP16 requests as fp16, BF16 as bf16 and refuses FP8 (that pool is behind the C ABI)
        titan::KVCache a, b, c;
        const bool f16 = a.initialize(2, 2, 64, 64, titan::DType::FP16), bf = b.initialize(2, 2, 64, 64, titan::DType::BF16);
        const bool f8 = c.initialize(2, 2, 64, 64, titan::DType::FP8_E4M3);
        printf("dtype fp16 %d bf16 %d fp8_e4m3 %d\n", (int)f16, (int)bf, (int)f8);
        return 0;
    }
    const bool external = mode != 0;
    const uint32_t L = 2, H = 8, Hkv = 2, D = 64, max_seq = 256;
    const float theta = 10000.0f;

    titan::KVCache cache;
    float *kbuf = nullptr, *vbuf = nullptr;
    if (external) {
        const size_t bytes = (size_t)L * max_seq * Hkv * D * sizeof(float);
        CHECK(cudaMalloc(&kbuf, bytes));
        CHECK(cudaMalloc(&vbuf, bytes));
        if (!cache.initialize_external(L, Hkv, D, max_seq, kbuf, vbuf)) { fprintf(stderr, "initialize_external failed\n"); return 3; }
    } else if (!cache.initialize(L, Hkv, D, max_seq)) { fprintf(stderr, "initialize failed\n"); return 3; }
    if (cache.seq_len() != 0 || cache.num_layers() != L || cache.k_cache(L) != nullptr || cache.k_cache(0) == nullptr) return 4;

    float *dq, *dk, *dv, *dout;
    CHECK(cudaMalloc(&dq, H * D * sizeof(float)));
    CHECK(cudaMalloc(&dk, Hkv * D * sizeof(float)));
    CHECK(cudaMalloc(&dv, Hkv * D * sizeof(float)));
    CHECK(cudaMalloc(&dout, H * D * sizeof(float)));
    cudaStream_t stream;
    CHECK(cudaStreamCreate(&stream));
    std::vector<float> q(H * D), k(Hkv * D), v(Hkv * D), out(H * D);
    FILE* f = fopen(argv[1], "wb");
    if (!f) return 5;
    uint32_t seed = 12345;
    for (int pos = 0; pos < n_tokens; pos++) {
        for (uint32_t l = 0; l < L; l++) {
            for (auto& x : q) x = val(seed);
            for (auto& x : k) x = val(seed);
            for (auto& x : v) x = val(seed);
            CHECK(cudaMemcpyAsync(dq, q.data(), q.size() * 4, cudaMemcpyHostToDevice, stream));
            CHECK(cudaMemcpyAsync(dk, k.data(), k.size() * 4, cudaMemcpyHostToDevice, stream));
            CHECK(cudaMemcpyAsync(dv, v.data(), v.size() * 4, cudaMemcpyHostToDevice, stream));
            titan::cuda::apply_rope(dq, dk, H, Hkv, D, pos, theta, 1.0f, stream);
            cache.update(l, pos, dk, dv, stream);
            const int seq_len = cache.seq_len();
            if (seq_len != pos + 1) { fprintf(stderr, "seq_len %d at pos %d\n", seq_len, pos); return 6; }
            titan::cuda::attention_decode(dq, cache.k_cache(l), cache.v_cache(l), dout, H, Hkv, D, seq_len, stream);
            CHECK(cudaGetLastError());
            CHECK(cudaMemcpyAsync(out.data(), dout, out.size() * 4, cudaMemcpyDeviceToHost, stream));
            CHECK(cudaStreamSynchronize(stream));
            fwrite(out.data(), 4, out.size(), f);
        }
    }
    // bad arguments are silent no-ops; clear() resets the length
    cache.update(L, 0, dk, dv, stream);
    cache.update(0, -1, dk, dv, stream);
    cache.update(0, (int)max_seq, dk, dv, stream);
    if (cache.seq_len() != n_tokens) return 7;
    // attend to a prefix: seq_len is an argument of the operator
    titan::cuda::attention_decode(dq, cache.k_cache(1), cache.v_cache(1), dout, H, Hkv, D, n_tokens / 2, stream);
    CHECK(cudaMemcpyAsync(out.data(), dout, out.size() * 4, cudaMemcpyDeviceToHost, stream));
    CHECK(cudaStreamSynchronize(stream));
    fwrite(out.data(), 4, out.size(), f);
    cache.clear();
    if (cache.seq_len() != 0) return 8;
    cache.update(0, 0, dk, dv, stream);
    titan::cuda::attention_decode(dq, cache.k_cache(0), cache.v_cache(0), dout, H, Hkv, D, cache.seq_len(), stream);
    CHECK(cudaMemcpyAsync(out.data(), dout, out.size() * 4, cudaMemcpyDeviceToHost, stream));
    CHECK(cudaStreamSynchronize(stream));
    fwrite(out.data(), 4, out.size(), f);
    fclose(f);
    printf("ok %d tokens, memory_bytes %zu\n", n_tokens, cache.memory_bytes());
    return 0;
}
