// append.cu — per-step K/V append: page-table scatter, FP8-E4M3 page sealing, and
// the page-table delta patch.
//
// Replaces the two cudaMemcpyAsync D2D copies per layer per token of
// KVCache::update (reference: src/inference/kv_cache.cpp:121-151) with one launch
// per layer for all tokens of all sequences of the step.  HBM-bound byte movement:
// every lane moves 16-byte vectors, rows are 128- to 384-byte contiguous runs.
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

// One warp per token.  The destination row comes from the step plan (tok_dst): 16-bit storage:
// pool slot page*ps + r; FP8 storage: slot seq*ps + r of the sequence's 16-bit open page, or -1 for
// rows of pages sealed by this step, which seal_*_kernel consumes.  No dependent page-table lookups
// stand between a warp and its copies.
constexpr int kAppendWarps = 8;
constexpr int kAppendInFlight = 4;     // 16-byte copies in flight per lane (measured at 64 x 512 tokens: 2 -> 5.86, 4 -> 5.98, 8 -> 5.63 TB/s)
__global__ void __launch_bounds__(kAppendWarps * 32)
append_rows_kernel(Geometry g, LayerPtrs lp, StepDev st, const int32_t* __restrict__ page_table,
                   const uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                   int64_t* __restrict__ slots_out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // with slots_out every token is visited; otherwise FP8 visits only the rows that stay open
    const bool listed = g.dtype == DT_FP8 && !slots_out;
    const int i_tok = blockIdx.x * kAppendWarps + warp;
    if (i_tok >= (listed ? st.n_open : st.n_tokens)) return;
    const int t = listed ? st.tok_open[i_tok] : i_tok;
    if (slots_out && lane == 0) {                       // pool slot of the token (what a caller would index)
        const int b = st.tok_b[t], pos = st.tok_pos[t];
        const int page = page_table[(size_t)st.seq[b] * g.max_pages_per_seq + pos / g.ps];
        slots_out[t] = (int64_t)page * g.ps + pos % g.ps;
    }
    const int dst_slot = st.tok_dst[t];
    if (dst_slot < 0) return;
    const int tile_page = dst_slot / g.ps, r = dst_slot % g.ps;
    uint16_t* base = g.dtype == DT_FP8 ? (uint16_t*)lp.open_pages : (uint16_t*)lp.pool;
    const int vk = g.D / 8, vv = g.Dv / 8;     // 16-byte vectors per K row / per V row
    const int n_k = g.Hkv * vk, n_vec = n_k + g.Hkv * vv;
    auto addr = [&](int i, const uint16_t*& src, uint16_t*& dst) {
        const int kv = i >= n_k;
        const int per = kv ? vv : vk, dim = kv ? g.Dv : g.D;
        const int ii = kv ? i - n_k : i;
        const int h = ii / per, c = ii % per;
        src = (kv ? v : k) + ((size_t)t * g.Hkv + h) * dim + c * 8;
        dst = base + tile_offset(g, tile_page, h, kv) + (size_t)r * dim + c * 8;
    };
    for (int i0 = lane; i0 < n_vec; i0 += kAppendInFlight * 32) {   // copies in flight per lane
        uint4 val[kAppendInFlight];
        uint16_t* dst[kAppendInFlight];
#pragma unroll
        for (int u = 0; u < kAppendInFlight; u++) {
            const int i = i0 + 32 * u;
            dst[u] = nullptr;
            if (i < n_vec) {
                const uint16_t* src;
                addr(i, src, dst[u]);
                val[u] = *reinterpret_cast<const uint4*>(src);
            }
        }
#pragma unroll
        for (int u = 0; u < kAppendInFlight; u++)
            if (dst[u]) *reinterpret_cast<uint4*>(dst[u]) = val[u];
    }
}

template <bool BF16>
__device__ __forceinline__ float cvt16(uint16_t x) {
    if (BF16) return __uint_as_float((uint32_t)x << 16);
    return __half2float(__ushort_as_half(x));
}

// FP8 seal of the tiles (completed page, kv head, K|V): absmax over the ps*D values,
// scale = max(amax/448, 1e-10), code = e4m3_rn_satfinite(x * (1/scale)): the recipe of
// quantize_fp4_kernel (reference: src/compute/cuda/fp4.cu:102-113) with the E4M3 maximum.
// Rows older than the step come from the open page, newer rows from this step's input; which rows,
// which physical page and which input token are in the seal item, so nothing is looked up on the
// way to the loads.  Every float op is a single IEEE-rounded operation (the absmax is taken on the
// 16-bit values, where a maximum is exact), so codes and scales are bit-exact against a plain C
// restatement.
template <bool BF16>
__device__ __forceinline__ uint32_t abs16x2(uint32_t w) { return w & 0x7FFF7FFFu; }
// maximum of two packed non-negative 16-bit floats (NaN patterns lose, as with fmaxf)
template <bool BF16>
__device__ __forceinline__ uint32_t max16x2(uint32_t a, uint32_t b) {
    if (BF16) {
        const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
    const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
// two 16-bit values (low half first) times inv_scale -> two E4M3 codes (low byte first)
template <bool BF16>
__device__ __forceinline__ uint32_t quant2(uint32_t w, float inv_scale) {
    const float lo = __fmul_rn(cvt16<BF16>((uint16_t)w), inv_scale);
    const float hi = __fmul_rn(cvt16<BF16>((uint16_t)(w >> 16)), inv_scale);
    return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}

// One warp per tile, the tile held in registers, one read of the rows, no shared memory; 8 tiles per CTA.
// D (row width) and the page size of 16 are compile-time constants: every index below is a shift or a
// mask, which matters - the kernel issues a few hundred instructions per tile and is bound by issue slots,
// not by HBM, when the addressing costs integer divisions.
template <bool BF16, int D>
__global__ void __launch_bounds__(256, 4)
seal_warp_kernel(Geometry g, LayerPtrs lp, StepDev st, const uint16_t* __restrict__ k, const uint16_t* __restrict__ v) {
    constexpr int PS = 16;
    constexpr int VPR = D / 8;                  // 16-byte vectors per row
    constexpr int N_VEC = PS * VPR;             // vectors per tile
    constexpr int VPL = N_VEC / 32;             // vectors per lane: 8 (D = 128) or 4 (D = 64)
    constexpr int RPI = 32 / VPR;               // rows one warp-wide load covers: 2 or 4
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_seal = g.Hkv * 2;
    const long long tile = (long long)blockIdx.x * 8 + warp;
    if (tile >= (long long)st.n_seals * per_seal) return;
    const int seal = (int)(tile / per_seal);
    const int rem = (int)(tile - (long long)seal * per_seal);
    const int4 it = st.seals[seal];
    const int seq = it.x, page = it.y, n_old = it.z, tok0 = it.w;
    const int kvh = rem >> 1, kv = rem & 1;
    const int r_lane = lane / VPR, c = lane % VPR;          // this lane's row within a load, its vector within the row
    const uint16_t* open = (const uint16_t*)lp.open_pages + tile_off(seq, kvh, kv, g.Hkv, PS, D) + c * 8;
    const size_t in_stride = (size_t)g.Hkv * D;             // elements between two tokens' rows of the input
    const uint16_t* in = (kv ? v : k) + ((ptrdiff_t)(tok0 - n_old) * g.Hkv + kvh) * D + c * 8;

    uint4 raw[VPL];
#pragma unroll
    for (int u = 0; u < VPL; u++) {
        const int r = r_lane + RPI * u;
        const uint16_t* src = r < n_old ? open + (size_t)r * D : in + (size_t)r * in_stride;
        raw[u] = *reinterpret_cast<const uint4*>(src);
    }
    uint32_t mx = 0u;
#pragma unroll
    for (int u = 0; u < VPL; u++) {
        mx = max16x2<BF16>(mx, abs16x2<BF16>(raw[u].x));
        mx = max16x2<BF16>(mx, abs16x2<BF16>(raw[u].y));
        mx = max16x2<BF16>(mx, abs16x2<BF16>(raw[u].z));
        mx = max16x2<BF16>(mx, abs16x2<BF16>(raw[u].w));
    }
    float amax = fmaxf(cvt16<BF16>((uint16_t)mx), cvt16<BF16>((uint16_t)(mx >> 16)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));

    float scale = __fdiv_rn(amax, 448.0f);
    if (scale < 1e-10f) scale = 1e-10f;
    const float inv_scale = __fdiv_rn(1.0f, scale);
    if (lane == 0) lp.scales[((size_t)page * g.Hkv + kvh) * 2 + kv] = scale;

    // vector i = lane + 32 u of the tile (row r, vector c of the row) is 8 codes at byte 8 i
    uint8_t* codes = (uint8_t*)lp.pool + tile_off(page, kvh, kv, g.Hkv, PS, D) + (size_t)lane * 8;
#pragma unroll
    for (int u = 0; u < VPL; u++) {
        uint2 out;
        out.x = quant2<BF16>(raw[u].x, inv_scale) | (quant2<BF16>(raw[u].y, inv_scale) << 16);
        out.y = quant2<BF16>(raw[u].z, inv_scale) | (quant2<BF16>(raw[u].w, inv_scale) << 16);
        *reinterpret_cast<uint2*>(codes + (size_t)u * 256) = out;
    }
}

// Tiles too large for a warp's registers: one CTA per tile, two passes over the rows.
template <bool BF16>
__global__ void __launch_bounds__(256)
seal_kernel(Geometry g, LayerPtrs lp, StepDev st, const uint16_t* __restrict__ k, const uint16_t* __restrict__ v) {
    const int4 it = st.seals[blockIdx.x];
    const int seq = it.x, page = it.y, n_old = it.z, tok0 = it.w;
    const int kvh = blockIdx.y >> 1, kv = blockIdx.y & 1;
    const int vec_per_row = g.D / 8;
    const int n_vec = g.ps * vec_per_row;
    const uint16_t* open = (const uint16_t*)lp.open_pages + tile_off(seq, kvh, kv, g.Hkv, g.ps, g.D);
    const uint16_t* in = (kv ? v : k) + ((ptrdiff_t)(tok0 - n_old) * g.Hkv + kvh) * g.D;
    auto row_src = [&](int r) -> const uint16_t* {
        return r < n_old ? open + (size_t)r * g.D : in + (size_t)r * g.Hkv * g.D;
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
        const uint4 raw = *reinterpret_cast<const uint4*>(row_src(i / vec_per_row) + (i % vec_per_row) * 8);
        uint2 out;
        out.x = quant2<BF16>(raw.x, inv_scale) | (quant2<BF16>(raw.y, inv_scale) << 16);
        out.y = quant2<BF16>(raw.z, inv_scale) | (quant2<BF16>(raw.w, inv_scale) << 16);
        *reinterpret_cast<uint2*>(codes + (size_t)i * 8) = out;
    }
}

template <bool BF16>
cudaError_t launch_seal(const Geometry& g, const LayerPtrs& lp, const StepDev& st, const uint16_t* k,
                        const uint16_t* v, cudaStream_t s) {
    const long long tiles = (long long)st.n_seals * g.Hkv * 2;
    const unsigned grid = (unsigned)((tiles + 7) / 8);
    if (g.ps == 16 && g.D == 128)     seal_warp_kernel<BF16, 128><<<grid, 256, 0, s>>>(g, lp, st, k, v);
    else if (g.ps == 16 && g.D == 64) seal_warp_kernel<BF16, 64><<<grid, 256, 0, s>>>(g, lp, st, k, v);
    else                              seal_kernel<BF16><<<dim3(st.n_seals, g.Hkv * 2), 256, 0, s>>>(g, lp, st, k, v);
    return cudaGetLastError();
}

cudaError_t launch_append(const Geometry& g, const LayerPtrs& lp, const StepDev& st,
                          const int32_t* page_table, const void* k, const void* v,
                          int64_t* slots_out, cudaStream_t s, int* n_launches) {
    *n_launches = 0;
    if (st.n_tokens <= 0) return cudaSuccess;
    if (g.dtype == DT_FP8 && st.n_seals > 0) {
        cudaError_t e = g.io_dtype == DT_BF16
            ? launch_seal<true>(g, lp, st, (const uint16_t*)k, (const uint16_t*)v, s)
            : launch_seal<false>(g, lp, st, (const uint16_t*)k, (const uint16_t*)v, s);
        (*n_launches)++;
        if (e != cudaSuccess) return e;
    }
    const int n_rows = (g.dtype == DT_FP8 && !slots_out) ? st.n_open : st.n_tokens;
    if (n_rows <= 0) return cudaSuccess;                    // FP8: every row of the step went into a sealed page
    append_rows_kernel<<<(n_rows + kAppendWarps - 1) / kAppendWarps, kAppendWarps * 32, 0, s>>>(
        g, lp, st, page_table, (const uint16_t*)k, (const uint16_t*)v, slots_out);
    (*n_launches)++;
    return cudaGetLastError();
}

}  // namespace tk
