// append.cu — per-step K/V append: page-table scatter, FP8-E4M3 page sealing, and
// the page-table delta patch.
//
// Replaces the two cudaMemcpyAsync D2D copies per layer per token of
// KVCache::update (reference: src/inference/kv_cache.cpp:121-151) with one launch
// per layer for all tokens of all sequences of the step.  HBM-bound byte movement:
// every thread moves 16 bytes, rows are 128- or 256-byte contiguous runs.
#include "tk_kernels.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace tk {

__global__ void apply_delta_kernel(int32_t* __restrict__ table, const int2* __restrict__ delta, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) table[delta[i].x] = delta[i].y;
}

cudaError_t launch_apply_delta(int32_t* table, const int2* delta, int n, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    apply_delta_kernel<<<(n + 255) / 256, 256, 0, s>>>(table, delta, n);
    return cudaGetLastError();
}

__global__ void copy_layers_kernel(const uint8_t* __restrict__ src, size_t src_stride, uint8_t* __restrict__ dst,
                                   size_t dst_stride, size_t bytes) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src + (size_t)blockIdx.y * src_stride);
    uint4* d4 = reinterpret_cast<uint4*>(dst + (size_t)blockIdx.y * dst_stride);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < bytes / 16; i += (size_t)gridDim.x * blockDim.x)
        d4[i] = s4[i];
}

cudaError_t launch_copy_layers(const void* src, size_t src_stride, void* dst, size_t dst_stride, size_t bytes,
                               int n_layers, cudaStream_t s) {
    if (bytes == 0 || n_layers <= 0) return cudaSuccess;
    dim3 grid((unsigned)((bytes / 16 + 255) / 256), n_layers);
    if (grid.x > 64) grid.x = 64;
    copy_layers_kernel<<<grid, 256, 0, s>>>((const uint8_t*)src, src_stride, (uint8_t*)dst, dst_stride, bytes);
    return cudaGetLastError();
}

__device__ __forceinline__ size_t tile_off(int page, int kvh, int kv, int Hkv, int ps, int D) {
    return (((size_t)page * Hkv + kvh) * 2 + kv) * (size_t)ps * D;
}

// One CTA per token.  16-bit storage: rows go to the pool page the table names.
// FP8 storage: rows that stay in a still-open page go to the sequence's open page;
// rows of pages sealed by this step were already consumed by seal_kernel.
__global__ void __launch_bounds__(256)
append_rows_kernel(Geometry g, LayerPtrs lp, StepDev st, const int32_t* __restrict__ page_table,
                   const uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                   int64_t* __restrict__ slots_out) {
    const int t = blockIdx.x;
    const int b = st.tok_b[t], pos = st.tok_pos[t];
    const int seq = st.seq[b];
    const int page = page_table[(size_t)seq * g.max_pages_per_seq + pos / g.ps];
    const int r = pos % g.ps;
    if (threadIdx.x == 0 && slots_out) slots_out[t] = (int64_t)page * g.ps + r;

    uint16_t* base;
    int tile_page;
    if (g.dtype == DT_FP8) {
        const int sealed_end = (st.len[b] / g.ps) * g.ps;
        if (pos < sealed_end) return;
        base = (uint16_t*)lp.open_pages;
        tile_page = seq;                       // open pages are indexed by sequence slot
    } else {
        base = (uint16_t*)lp.pool;
        tile_page = page;
    }
    const int vk = g.D / 8, vv = g.Dv / 8;     // 16-byte vectors per K row / per V row
    const int n_k = g.Hkv * vk, n_vec = n_k + g.Hkv * vv;
    for (int i = threadIdx.x; i < n_vec; i += blockDim.x) {
        const int kv = i >= n_k;
        const int per = kv ? vv : vk, dim = kv ? g.Dv : g.D;
        const int ii = kv ? i - n_k : i;
        const int h = ii / per, c = ii % per;
        const uint16_t* src = (kv ? v : k) + ((size_t)t * g.Hkv + h) * dim + c * 8;
        uint16_t* dst = base + tile_offset(g, tile_page, h, kv) + (size_t)r * dim + c * 8;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    }
}

template <bool BF16>
__device__ __forceinline__ float cvt16(uint16_t x) {
    if (BF16) return __uint_as_float((uint32_t)x << 16);
    return __half2float(__ushort_as_half(x));
}

// FP8 seal: one CTA per (completed page, kv head, K|V).  absmax over the ps*D values,
// scale = max(amax/448, 1e-10), code = e4m3_rn_satfinite(x * (1/scale)): the recipe of
// quantize_fp4_kernel (reference: src/compute/cuda/fp4.cu:102-113) with the E4M3 maximum.
// Rows older than the step come from the open page, newer rows from this step's input.
// Every float op is a single IEEE-rounded operation so codes and scales are bit-exact
// against a plain C restatement.
template <bool BF16>
__global__ void __launch_bounds__(256)
seal_kernel(Geometry g, LayerPtrs lp, StepDev st, const int32_t* __restrict__ page_table,
            const uint16_t* __restrict__ k, const uint16_t* __restrict__ v) {
    const int4 it = st.seals[blockIdx.x];
    const int b = it.x, lpage = it.y, old_len = it.z, tok_base = it.w;
    const int kvh = blockIdx.y >> 1, kv = blockIdx.y & 1;
    const int seq = st.seq[b];
    const int page = page_table[(size_t)seq * g.max_pages_per_seq + lpage];
    const int vec_per_row = g.D / 8;
    const int n_vec = g.ps * vec_per_row;
    const uint16_t* open = (const uint16_t*)lp.open_pages + tile_off(seq, kvh, kv, g.Hkv, g.ps, g.D);
    const uint16_t* in = kv ? v : k;

    auto row_src = [&](int r) -> const uint16_t* {
        const int pos = lpage * g.ps + r;
        if (pos < old_len) return open + (size_t)r * g.D;
        return in + ((size_t)(tok_base + pos - old_len) * g.Hkv + kvh) * g.D;
    };

    float amax = 0.0f;
    for (int i = threadIdx.x; i < n_vec; i += blockDim.x) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row_src(i / vec_per_row) + (i % vec_per_row) * 8);
        const uint16_t* e = reinterpret_cast<const uint16_t*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(cvt16<BF16>(e[j])));
    }
    __shared__ float red[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int w = 1; w < 8; w++) amax = fmaxf(amax, red[w]);

    float scale = __fdiv_rn(amax, 448.0f);
    if (scale < 1e-10f) scale = 1e-10f;
    const float inv_scale = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0) lp.scales[((size_t)page * g.Hkv + kvh) * 2 + kv] = scale;

    uint8_t* codes = (uint8_t*)lp.pool + tile_off(page, kvh, kv, g.Hkv, g.ps, g.D);
    for (int i = threadIdx.x; i < n_vec; i += blockDim.x) {
        const int r = i / vec_per_row, c = i % vec_per_row;
        const uint4 raw = *reinterpret_cast<const uint4*>(row_src(r) + c * 8);
        const uint16_t* e = reinterpret_cast<const uint16_t*>(&raw);
        uint8_t out[8];
#pragma unroll
        for (int j = 0; j < 8; j++)
            out[j] = (uint8_t)__nv_cvt_float_to_fp8(__fmul_rn(cvt16<BF16>(e[j]), inv_scale),
                                                    __NV_SATFINITE, __NV_E4M3);
        *reinterpret_cast<uint2*>(codes + (size_t)r * g.D + c * 8) = *reinterpret_cast<const uint2*>(out);
    }
}

cudaError_t launch_append(const Geometry& g, const LayerPtrs& lp, const StepDev& st,
                          const int32_t* page_table, const void* k, const void* v,
                          int64_t* slots_out, cudaStream_t s, int* n_launches) {
    *n_launches = 0;
    if (st.n_tokens <= 0) return cudaSuccess;
    if (g.dtype == DT_FP8 && st.n_seals > 0) {
        dim3 grid(st.n_seals, g.Hkv * 2);
        if (g.io_dtype == DT_BF16)
            seal_kernel<true><<<grid, 256, 0, s>>>(g, lp, st, page_table, (const uint16_t*)k, (const uint16_t*)v);
        else
            seal_kernel<false><<<grid, 256, 0, s>>>(g, lp, st, page_table, (const uint16_t*)k, (const uint16_t*)v);
        (*n_launches)++;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    append_rows_kernel<<<st.n_tokens, 256, 0, s>>>(g, lp, st, page_table, (const uint16_t*)k,
                                                   (const uint16_t*)v, slots_out);
    (*n_launches)++;
    return cudaGetLastError();
}

}  // namespace tk
