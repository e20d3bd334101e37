// decode_simt.cu — generic paged GQA decode attention (SIMT) and the LSE combine.
//
// The arithmetic is that of attention_decode_kernel (reference:
// src/compute/cuda/attention.cu:58-157): score = (q.k) * 1/sqrtf(D), running max
// from -1e30f, expf, FP32 accumulation, normaliser 1/(sum + 1e-8f), GQA map
// kv_head = head / (H/Hkv).  What differs is the schedule: one CTA per
// (sequence, kv head, split-KV chunk) serves all G query heads of the group from
// one pass over the pages (the reference re-reads K/V once per query head), softmax
// is online, and each CTA leaves an (o, m, l) partial that combine_step_kernel merges.
//
// This kernel covers every supported shape and storage type, including the 16-bit
// open page of an FP8 cache; the TMA + tensor-core kernel in decode_mma.cu is the
// fast path for full pool pages.
#include "tk_kernels.cuh"
#include "tk_merge.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace tk {

namespace {

constexpr int kWarps = 4;

template <bool BF16>
__device__ __forceinline__ float cvt16(uint16_t x) {
    if (BF16) return __uint_as_float((uint32_t)x << 16);
    return __half2float(__ushort_as_half(x));
}

__device__ __forceinline__ float cvt_e4m3(uint8_t c) {
    __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&hr));
}

// Load EPL consecutive elements of a row (lane's slice) as floats.
template <int EPL, bool BF16>
__device__ __forceinline__ void load16(const uint16_t* row, int lane, float (&out)[EPL]) {
    const uint16_t* p = row + lane * EPL;
    if constexpr (EPL == 2) {
        uint32_t w = *reinterpret_cast<const uint32_t*>(p);
        out[0] = cvt16<BF16>((uint16_t)(w & 0xFFFF)); out[1] = cvt16<BF16>((uint16_t)(w >> 16));
    } else if constexpr (EPL == 6) {
        const uint32_t* pw = reinterpret_cast<const uint32_t*>(p);
#pragma unroll
        for (int i = 0; i < 3; i++) {
            const uint32_t w = pw[i];
            out[2 * i] = cvt16<BF16>((uint16_t)(w & 0xFFFF)); out[2 * i + 1] = cvt16<BF16>((uint16_t)(w >> 16));
        }
    } else if constexpr (EPL == 4) {
        uint2 w = *reinterpret_cast<const uint2*>(p);
        out[0] = cvt16<BF16>((uint16_t)(w.x & 0xFFFF)); out[1] = cvt16<BF16>((uint16_t)(w.x >> 16));
        out[2] = cvt16<BF16>((uint16_t)(w.y & 0xFFFF)); out[3] = cvt16<BF16>((uint16_t)(w.y >> 16));
    } else {
        uint4 w = *reinterpret_cast<const uint4*>(p);
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            out[2 * i] = cvt16<BF16>((uint16_t)(ws[i] & 0xFFFF));
            out[2 * i + 1] = cvt16<BF16>((uint16_t)(ws[i] >> 16));
        }
    }
}

template <int EPL>
__device__ __forceinline__ void load8(const uint8_t* row, int lane, float scale, float (&out)[EPL]) {
    const uint8_t* p = row + lane * EPL;
#pragma unroll
    for (int i = 0; i < EPL; i++) out[i] = cvt_e4m3(p[i]) * scale;
}

// G = query heads per kv head, EPL = D/32 and EPLV = Dv/32 elements per lane (they differ only for
// the MLA cache, 192/128), FP8 = pool holds E4M3 codes, BF16 = 16-bit type is bf16 (else fp16).
template <int G, int EPL, int EPLV, bool FP8, bool BF16>
__global__ void __launch_bounds__(kWarps * 32)
decode_simt_kernel(Geometry g, LayerPtrs lp, StepDev st, const int32_t* __restrict__ page_table,
                   const uint16_t* __restrict__ q, float* __restrict__ partials, MergeOut mo) {
    constexpr int D = EPL * 32, DV = EPLV * 32;
    __shared__ float qs[G][D];
    __shared__ float red[kWarps][G][DV + 2];
    __shared__ int s_flag;

    const int4 it = st.items[blockIdx.x];
    const int b = it.x, chunk = it.y, kvh = it.z, kind = it.w;
    const int seq = st.seq[b], len = st.len[b];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ps = g.ps;

    int t0, t1;
    if (kind == 1) {                                  // FP8 open page: the 16-bit tail
        t0 = (len / ps) * ps; t1 = len;
    } else {
        const int pool_tokens = FP8 ? (len / ps) * ps : len;
        t0 = chunk * st.chunk_tokens;
        t1 = min(pool_tokens, t0 + st.chunk_tokens);
    }

    for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
        const int gq = i / D, d = i % D;
        qs[gq][d] = cvt16<BF16>(q[((size_t)b * g.H + kvh * G + gq) * D + d]);
    }
    __syncthreads();

    const float scale = 1.0f / sqrtf((float)D);
    float m[G], l[G], o[G][EPLV];
#pragma unroll
    for (int gq = 0; gq < G; gq++) {
        m[gq] = -1e30f; l[gq] = 0.0f;
#pragma unroll
        for (int i = 0; i < EPLV; i++) o[gq][i] = 0.0f;
    }

    const int32_t* prow = page_table + (size_t)seq * g.max_pages_per_seq;
    for (int t = t0 + warp; t < t1; t += kWarps) {
        const int r = t % ps;
        float kf[EPL], vf[EPLV];
        if (FP8 && kind == 0) {
            const int page = prow[t / ps];
            const size_t tile = ((size_t)page * g.Hkv + kvh) * 2;
            const uint8_t* kt = (const uint8_t*)lp.pool + tile * ps * D + (size_t)r * D;
            const float ks = lp.scales[tile], vs = lp.scales[tile + 1];
            load8<EPL>(kt, lane, ks, kf);
            load8<EPLV>(kt + (size_t)ps * D, lane, vs, vf);
        } else {
            const uint16_t* tile;                       // K rows (D wide), then V rows (DV wide)
            if (FP8) tile = (const uint16_t*)lp.open_pages + ((size_t)seq * g.Hkv + kvh) * ps * (D + DV);
            else {
                const int pg = prow[t / ps];
                const uint16_t* base = (const uint16_t*)((pg & kColdBit) ? lp.cold_stage : lp.pool);
                tile = base + ((size_t)(pg & ~kColdBit) * g.Hkv + kvh) * ps * (D + DV);
            }
            load16<EPL, BF16>(tile + (size_t)r * D, lane, kf);
            load16<EPLV, BF16>(tile + (size_t)ps * D + (size_t)r * DV, lane, vf);
        }
#pragma unroll
        for (int gq = 0; gq < G; gq++) {
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < EPL; i++) dot += qs[gq][lane * EPL + i] * kf[i];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, off);
            const float s = dot * scale;
            const float m_new = fmaxf(m[gq], s);
            const float alpha = expf(m[gq] - m_new);
            const float p = expf(s - m_new);
            l[gq] = l[gq] * alpha + p;
#pragma unroll
            for (int i = 0; i < EPLV; i++) o[gq][i] = o[gq][i] * alpha + p * vf[i];
            m[gq] = m_new;
        }
    }

#pragma unroll
    for (int gq = 0; gq < G; gq++) {
#pragma unroll
        for (int i = 0; i < EPLV; i++) red[warp][gq][lane * EPLV + i] = o[gq][i];
        if (lane == 0) { red[warp][gq][DV] = m[gq]; red[warp][gq][DV + 1] = l[gq]; }
    }
    __syncthreads();

    const int row = st.chunk_base[b] + chunk;
    for (int i = threadIdx.x; i < G * (DV + 2); i += blockDim.x) {
        const int gq = i / (DV + 2), d = i % (DV + 2);
        float M = -1e30f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, red[w][gq][DV]);
        float val;
        if (d == DV) {
            val = M;
        } else {
            val = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) val += red[w][gq][d] * expf(red[w][gq][DV] - M);
        }
        partials[partial_off(row, kvh * G + gq, g.H, DV) + d] = val;
    }
    merge_if_last(g, st, mo, b, kvh, G, partials, &s_flag);
}

template <int G, int EPL, int EPLV = EPL>
cudaError_t launch_simt_ge(const Geometry& g, const LayerPtrs& lp, const StepDev& st,
                           const int32_t* page_table, const void* q, float* partials, cudaStream_t s,
                           const MergeOut& mo) {
    const bool fp8 = g.dtype == DT_FP8, bf16 = g.io_dtype == DT_BF16;
    dim3 grid(st.n_items), block(kWarps * 32);
    const uint16_t* qq = (const uint16_t*)q;
    if (fp8) {
        if constexpr (EPLV != EPL) {
            return cudaErrorNotSupported;                   // the MLA shape is stored in 16 bits only
        } else {
            if (bf16) decode_simt_kernel<G, EPL, EPLV, true, true><<<grid, block, 0, s>>>(g, lp, st, page_table, qq, partials, mo);
            else      decode_simt_kernel<G, EPL, EPLV, true, false><<<grid, block, 0, s>>>(g, lp, st, page_table, qq, partials, mo);
        }
    }
    else if (bf16)         decode_simt_kernel<G, EPL, EPLV, false, true><<<grid, block, 0, s>>>(g, lp, st, page_table, qq, partials, mo);
    else                   decode_simt_kernel<G, EPL, EPLV, false, false><<<grid, block, 0, s>>>(g, lp, st, page_table, qq, partials, mo);
    return cudaGetLastError();
}

template <int G>
cudaError_t launch_simt_g(const Geometry& g, const LayerPtrs& lp, const StepDev& st,
                          const int32_t* page_table, const void* q, float* partials, cudaStream_t s,
                          const MergeOut& mo) {
    if (g.D == 192 && g.Dv == 128) return launch_simt_ge<G, 6, 4>(g, lp, st, page_table, q, partials, s, mo);
    if (g.Dv != g.D) return cudaErrorNotSupported;
    switch (g.D) {
        case 64:  return launch_simt_ge<G, 2>(g, lp, st, page_table, q, partials, s, mo);
        case 128: return launch_simt_ge<G, 4>(g, lp, st, page_table, q, partials, s, mo);
        default:  return cudaErrorNotSupported;
    }
}

}  // namespace

cudaError_t launch_decode_simt(const Geometry& g, const LayerPtrs& lp, const StepDev& st,
                               const int32_t* page_table, const void* q, float* partials,
                               cudaStream_t s, const MergeOut* merge) {
    if (st.n_items <= 0) return cudaSuccess;
    if (g.Hkv <= 0 || g.H % g.Hkv != 0) return cudaErrorNotSupported;
    const MergeOut mo = merge ? *merge : MergeOut{nullptr, nullptr, nullptr, 0};
    switch (g.H / g.Hkv) {
        case 1:  return launch_simt_g<1>(g, lp, st, page_table, q, partials, s, mo);
        case 2:  return launch_simt_g<2>(g, lp, st, page_table, q, partials, s, mo);
        case 4:  return launch_simt_g<4>(g, lp, st, page_table, q, partials, s, mo);
        case 8:  return launch_simt_g<8>(g, lp, st, page_table, q, partials, s, mo);
        case 16: return launch_simt_g<16>(g, lp, st, page_table, q, partials, s, mo);
        default: return cudaErrorNotSupported;
    }
}

// ---------------------------------------------------------------------------------
// LSE combine.  M = max m_i, L = sum l_i e^{m_i-M}, O = sum o_i e^{m_i-M},
// out = O * 1/(L + 1e-8f)  (the reference's normaliser, attention.cu:142).
// ---------------------------------------------------------------------------------
// grid = (H, n_seqs); block = 128 threads striding over D
__global__ void combine_step_kernel(Geometry g, StepDev st, const float* __restrict__ partials,
                                    void* __restrict__ out, int out_dtype,
                                    float* __restrict__ partial_out, const int* __restrict__ status) {
    if (status && __ldcg(status) != 0) return;       // a device wait gave up on this handle: write nothing
    const int h = blockIdx.x, b = blockIdx.y, D = g.Dv;
    const int r0 = st.chunk_base[b], r1 = st.chunk_base[b + 1];
    float M = -1e30f;
    for (int r = r0; r < r1; r++) M = fmaxf(M, partials[partial_off(r, h, g.H, D) + D]);
    float L = 0.0f;
    for (int r = r0; r < r1; r++) {
        const float* p = partials + partial_off(r, h, g.H, D);
        L += p[D + 1] * expf(p[D] - M);
    }
    const float inv = 1.0f / (L + 1e-8f);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int r = r0; r < r1; r++) {
            const float* p = partials + partial_off(r, h, g.H, D);
            acc += p[d] * expf(p[D] - M);
        }
        if (out) store_out(out, ((size_t)b * g.H + h) * D + d, acc * inv, out_dtype);
        if (partial_out) partial_out[partial_off(b, h, g.H, D) + d] = acc;
    }
    if (partial_out && threadIdx.x == 0) {
        partial_out[partial_off(b, h, g.H, D) + D] = M;
        partial_out[partial_off(b, h, g.H, D) + D + 1] = L;
    }
}

cudaError_t launch_combine_step(const Geometry& g, const StepDev& st, const float* partials,
                                void* out, int out_dtype, float* partial_out, cudaStream_t s, const int* status) {
    if (st.n_seqs <= 0) return cudaSuccess;
    dim3 grid(g.H, st.n_seqs);
    combine_step_kernel<<<grid, 128, 0, s>>>(g, st, partials, out, out_dtype, partial_out, status);
    return cudaGetLastError();
}

__global__ void f32_to_16_kernel(const float* __restrict__ src, void* __restrict__ dst, size_t n, int dtype) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) store_out(dst, i, src[i], dtype);
}

cudaError_t launch_f32_to_16(const float* src, void* dst, size_t n, int dtype, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    f32_to_16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, dst, n, dtype);
    return cudaGetLastError();
}

// parts [n_parts][n_rows][D+2]; grid = n_rows
__global__ void combine_parts_kernel(const float* __restrict__ parts, int n_parts, int n_rows, int D,
                                     void* __restrict__ out, int out_dtype) {
    const int row = blockIdx.x;
    const size_t stride = (size_t)n_rows * (D + 2);
    const float* base = parts + (size_t)row * (D + 2);
    float M = -1e30f;
    for (int i = 0; i < n_parts; i++) M = fmaxf(M, base[i * stride + D]);
    float L = 0.0f;
    for (int i = 0; i < n_parts; i++) L += base[i * stride + D + 1] * expf(base[i * stride + D] - M);
    const float inv = 1.0f / (L + 1e-8f);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int i = 0; i < n_parts; i++) acc += base[i * stride + d] * expf(base[i * stride + D] - M);
        store_out(out, (size_t)row * D + d, acc * inv, out_dtype);
    }
}

cudaError_t launch_combine_parts(const float* parts, int n_parts, int n_rows, int D, void* out,
                                 int out_dtype, cudaStream_t s) {
    if (n_rows <= 0) return cudaSuccess;
    combine_parts_kernel<<<n_rows, 128, 0, s>>>(parts, n_parts, n_rows, D, out, out_dtype);
    return cudaGetLastError();
}

}  // namespace tk
