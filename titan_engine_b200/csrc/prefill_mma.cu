// prefill_mma.cu — paged attention for EVERY token of a prefill chunk (sm_100a).
//
// The reference runs its whole layer — KVCache::update + attention_decode — once per prompt token
// (src/inference/engine.cpp:182-193, src/inference/batch.cpp:169-198): layer l+1 needs token t's
// attention output of layer l.  Here a step appends a chunk of T tokens per sequence in one call
// (tk_kv_append) and this kernel computes the T attention outputs at once, token t attending to
// positions <= its own (causal inside the chunk, everything before the chunk visible).
//
// Arithmetic contract: that of attention_decode_kernel (src/compute/cuda/attention.cu:58-157) per
// token — score = (q.k)/sqrtf(D), max from -1e30f, FP32 accumulation, out = O/(L + 1e-8f),
// kv_head = head/(H/Hkv) — evaluated as an online softmax.
//
// Schedule.  The rows of a (sequence, kv head) are its (query token, head of the group) pairs:
// T * G rows, G = H/Hkv.  One CTA takes a tile of 64 rows (64/G whole tokens) and a range of the
// context (the whole visible context, or one split-KV chunk of it when the sequence has too few
// tiles to fill the GPU).  Its 4 warps own 16 rows each — the M rows of m16n8k16 MMAs — and all
// consume the SAME K/V page tiles: a CTA-wide ring of TMA stages (one elected thread issues
// cp.async.bulk.tensor.2d per page tile; `full` mbarriers carry the byte count, `empty`
// mbarriers collect one arrival per warp), so a page is fetched once per 64 rows instead of once
// per 16 as in the decode kernel's multi-token form.  With T * G >= 64 this is a contraction in
// its own right (64 flop per K/V byte at D = 128), bounded by the tensor pipe, not by HBM.
// Tiles that see the whole visible context write normalised outputs directly; split ones leave
// (o, m, l) partials and the CTA that arrives last for the tile merges them (tk_merge.cuh).
// Every wait is bounded; a wait that gives up sets the status word and nothing is written.
//
// Measured alternatives (16 fresh sequences growing by 1024 tokens per step, 8B head shape, B200): this form
// 235 TFLOP/s; four instead of two accumulator chains in QK^T 214; 32 rows per warp (128-row tiles, every
// shared-memory fragment feeding two MMAs, 255 registers, 2 CTAs/SM) 200; 6 instead of 4 stages and the L2
// eviction hint of the tile loads: no difference.  ncu: tensor pipe 42 % active, issue slots 44 %: the
// kernel sits at what the warp-level mma.sync path delivers on this part, not at a memory limit.
#include "tk_kernels.cuh"
#include "tk_merge.cuh"
#include "tk_mma.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cudaTypedefs.h>

namespace tk {

namespace {

constexpr int kPfStages = 4;              // page tiles in flight per CTA

template <int D>
struct PfCfg {
    static constexpr int NBOX = D * 2 / 128;                 // TMA boxes per (page, kv head) tile
    static constexpr int STAGE_BYTES = NBOX * kBoxBytes;
    static constexpr int BAR_BYTES = 2 * kPfStages * 8 + 16;  // full + empty barriers, merge flag
    static constexpr int SMEM_BYTES = kPfStages * STAGE_BYTES + BAR_BYTES + kPrefillMaxPages * 4 + 1024;
};

template <bool BF, int D>
__global__ void __launch_bounds__(kWarps * 32, 3)
prefill_mma_kernel(const __grid_constant__ CUtensorMap tmap, Geometry g, StepDev st, PrefillDev pf,
                   const int32_t* __restrict__ page_table, const uint16_t* __restrict__ q, void* __restrict__ out,
                   int out_dtype, float* __restrict__ partials, int* __restrict__ counters, int* __restrict__ status) {
    using C = PfCfg<D>;
    constexpr int KS = D / 16, NT = D / 8;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + kPfStages * C::STAGE_BYTES);
    uint64_t* empty = full + kPfStages;
    int* s_flag = (int*)(empty + kPfStages);
    int32_t* s_pages = (int32_t*)(smem + kPfStages * C::STAGE_BYTES + C::BAR_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gr = lane >> 2, j = lane & 3;                 // fragment row / column-pair index
    const int G = g.H / g.Hkv;

    const int4 it = pf.items[blockIdx.x];
    const int b = it.x, chunk = it.y, kvh = it.z, tile = it.w;
    const int seq = st.seq[b], len = st.len[b], nq = st.nq[b];
    const int ct = pf.ct[b];                                // tokens per split-KV chunk of this sequence
    const int tpt = kPrefillRows / G;                       // query tokens per tile
    const int tok_first = tile * tpt;                       // first query token of the tile
    const int tok_cnt = min(nq - tok_first, tpt);           // its query tokens (>= 1)
    const int base_pos = len - nq;                          // position of the sequence's first query token
    const int p_last = base_pos + tok_first + tok_cnt - 1;  // last position the tile may see
    const int t0 = chunk * ct;
    const int t1 = min(t0 + ct, p_last + 1);                // > t0: the host emits no empty item
    const int n_pages = (t1 - t0 + kPage - 1) / kPage;
    const int lp0 = t0 / kPage;
    const int n_chunks = p_last / ct + 1;                   // items of this (sequence, kv head, tile)

    if (threadIdx.x == 0) {
        for (int i = 0; i < kPfStages; i++) { mbar_init(smem_u32(&full[i]), 1); mbar_init(smem_u32(&empty[i]), kWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < n_pages; i += blockDim.x)
        s_pages[i] = page_table[(size_t)seq * g.max_pages_per_seq + lp0 + i];
    __syncthreads();

    auto issue = [&](int i) {                               // thread 0 only
        const int s = i % kPfStages;
        const uint32_t bar = smem_u32(&full[s]);
        const uint32_t dst = smem_u32(smem + (size_t)s * C::STAGE_BYTES);
        mbar_expect_tx(bar, C::STAGE_BYTES);
        const int row = (s_pages[i] * g.Hkv + kvh) * 32;
#pragma unroll
        for (int h = 0; h < C::NBOX; h++) tma_load_2d_shared_tile(dst + h * kBoxBytes, &tmap, h * 64, row, bar);
    };
    if (threadIdx.x == 0)
        for (int i = 0; i < kPfStages && i < n_pages; i++) issue(i);

    // ---- this warp's 16 rows: row r is query token (16*warp + r) / G of the tile, head (16*warp + r) % G
    const int r0 = 16 * warp + gr, r1 = r0 + 8;
    const bool v0 = r0 / G < tok_cnt, v1 = r1 / G < tok_cnt;
    const int lim0 = base_pos + tok_first + r0 / G + 1;     // positions row r0 attends to: [0, lim0)
    const int lim1 = base_pos + tok_first + r1 / G + 1;
    // last position any row of this warp sees (0: the warp has no row)
    const int warp_lim = (16 * warp) / G < tok_cnt ? base_pos + tok_first + min(tok_cnt - 1, (16 * warp + 15) / G) + 1 : 0;

    uint32_t qa[KS][4];
    {
        const uint16_t* qrow0 = q + ((size_t)(st.q_base[b] + tok_first + r0 / G) * g.H + (size_t)kvh * G + r0 % G) * D;
        const uint16_t* qrow1 = q + ((size_t)(st.q_base[b] + tok_first + r1 / G) * g.H + (size_t)kvh * G + r1 % G) * D;
#pragma unroll
        for (int kk = 0; kk < KS; kk++) {
            qa[kk][0] = v0 ? *reinterpret_cast<const uint32_t*>(qrow0 + 16 * kk + 2 * j) : 0u;
            qa[kk][2] = v0 ? *reinterpret_cast<const uint32_t*>(qrow0 + 16 * kk + 8 + 2 * j) : 0u;
            qa[kk][1] = v1 ? *reinterpret_cast<const uint32_t*>(qrow1 + 16 * kk + 2 * j) : 0u;
            qa[kk][3] = v1 ? *reinterpret_cast<const uint32_t*>(qrow1 + 16 * kk + 8 + 2 * j) : 0u;
        }
    }

    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f; }
    float m0 = -1e30f, m1 = -1e30f, l0 = 0.0f, l1 = 0.0f;  // rows r0 and r1
    const float sm_scale = 1.0f / sqrtf((float)D);
    bool alive = true;

    for (int i = 0; i < n_pages; i++) {
        const int s = i % kPfStages;
        if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded(smem_u32(&full[s]), (uint32_t)((i / kPfStages) & 1), status))) {
            alive = false;
            break;
        }
        uint8_t* stg = smem + (size_t)s * C::STAGE_BYTES;
        const uint32_t stg_u = smem_u32(stg);
        const int tok_base = t0 + i * kPage;
        bool wrote = false;

        if (tok_base < warp_lim) {
            const int n_live = min(kPage, len - tok_base);      // rows of the page that hold tokens of the sequence
            if (n_live < kPage) {
                // rows past the sequence's end hold whatever the page's last owner left: zero the V rows,
                // so that probability 0 times garbage cannot make NaN.  Every warp does it for itself
                // before it reads (the same zeros, whoever writes them).
                for (int idx = lane; idx < (kPage - n_live) * 8 * C::NBOX; idx += 32) {
                    const int h = idx / ((kPage - n_live) * 8), rem = idx % ((kPage - n_live) * 8);
                    const int r = 16 + n_live + rem / 8, c = rem % 8;
                    *reinterpret_cast<uint4*>(stg + h * kBoxBytes + r * 128 + c * 16) = make_uint4(0, 0, 0, 0);
                }
                wrote = true;
                __syncwarp();
            }
            const int n_valid = min(kPage, t1 - tok_base);
            const int nv0 = v0 ? max(0, min(n_valid, lim0 - tok_base)) : 0;
            const int nv1 = v1 ? max(0, min(n_valid, lim1 - tok_base)) : 0;

            // ---- S = Q K^T over the page's 16 tokens ----
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
            {
                const int row = ((lane >> 4) << 3) + (lane & 7);
#pragma unroll
                for (int kk = 0; kk < KS; kk++) {
                    const int cc = 2 * kk + ((lane >> 3) & 1);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(stg_u + (cc >> 3) * kBoxBytes + swz(row, cc & 7), b0, b1, b2, b3);
                    mma16816<BF>(s0, qa[kk], b0, b1);
                    mma16816<BF>(s1, qa[kk], b2, b3);
                }
            }

            // ---- online softmax: row r0 in [0],[1]; row r1 in [2],[3]; token columns 2j, 2j+1, 2j+8, 2j+9 ----
            float p0[4], p1[4];
            const int c0 = 2 * j;
            {
                float a0 = s0[0] * sm_scale, a1 = s0[1] * sm_scale, a2 = s1[0] * sm_scale, a3 = s1[1] * sm_scale;
                if (c0 >= nv0) a0 = -1e30f;
                if (c0 + 1 >= nv0) a1 = -1e30f;
                if (c0 + 8 >= nv0) a2 = -1e30f;
                if (c0 + 9 >= nv0) a3 = -1e30f;
                float mx = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
                mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
                const float mn = fmaxf(m0, mx);
                const float alpha = ex2((m0 - mn) * kLog2e);
                const float nb = -mn * kLog2e;
                // a row may see nothing of a page: exp(-1e30 + 1e30) is 1, not 0
                p0[0] = c0 < nv0 ? ex2(fmaf(a0, kLog2e, nb)) : 0.0f;
                p0[1] = c0 + 1 < nv0 ? ex2(fmaf(a1, kLog2e, nb)) : 0.0f;
                p1[0] = c0 + 8 < nv0 ? ex2(fmaf(a2, kLog2e, nb)) : 0.0f;
                p1[1] = c0 + 9 < nv0 ? ex2(fmaf(a3, kLog2e, nb)) : 0.0f;
                l0 = l0 * alpha + (p0[0] + p0[1] + p1[0] + p1[1]);
                if (!__all_sync(0xFFFFFFFFu, mn == m0)) {
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) { o[nt][0] *= alpha; o[nt][1] *= alpha; }
                }
                m0 = mn;
            }
            {
                float a0 = s0[2] * sm_scale, a1 = s0[3] * sm_scale, a2 = s1[2] * sm_scale, a3 = s1[3] * sm_scale;
                if (c0 >= nv1) a0 = -1e30f;
                if (c0 + 1 >= nv1) a1 = -1e30f;
                if (c0 + 8 >= nv1) a2 = -1e30f;
                if (c0 + 9 >= nv1) a3 = -1e30f;
                float mx = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
                mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
                const float mn = fmaxf(m1, mx);
                const float alpha = ex2((m1 - mn) * kLog2e);
                const float nb = -mn * kLog2e;
                p0[2] = c0 < nv1 ? ex2(fmaf(a0, kLog2e, nb)) : 0.0f;
                p0[3] = c0 + 1 < nv1 ? ex2(fmaf(a1, kLog2e, nb)) : 0.0f;
                p1[2] = c0 + 8 < nv1 ? ex2(fmaf(a2, kLog2e, nb)) : 0.0f;
                p1[3] = c0 + 9 < nv1 ? ex2(fmaf(a3, kLog2e, nb)) : 0.0f;
                l1 = l1 * alpha + (p0[2] + p0[3] + p1[2] + p1[3]);
                if (!__all_sync(0xFFFFFFFFu, mn == m1)) {
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) { o[nt][2] *= alpha; o[nt][3] *= alpha; }
                }
                m1 = mn;
            }

            // ---- O += P V ----
            uint32_t pa[4];
            pa[0] = pack2<BF>(p0[0], p0[1]);
            pa[1] = pack2<BF>(p0[2], p0[3]);
            pa[2] = pack2<BF>(p1[0], p1[1]);
            pa[3] = pack2<BF>(p1[2], p1[3]);
            {
                const int row = 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
                for (int np = 0; np < NT / 2; np++) {
                    const int cc = 2 * np + (lane >> 4);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(stg_u + (cc >> 3) * kBoxBytes + swz(row, cc & 7), b0, b1, b2, b3);
                    mma16816<BF>(o[2 * np], pa, b0, b1);
                    mma16816<BF>(o[2 * np + 1], pa, b2, b3);
                }
            }
        }

        // ---- this warp is done with the stage; the producer refills one stage behind ----
        __syncwarp();
        if (wrote) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (lane == 0) mbar_arrive(smem_u32(&empty[s]));
        if (warp == 0 && i >= 1 && i - 1 + kPfStages < n_pages) {
            const int prev = i - 1, ps = prev % kPfStages;
            bool ok = true;
            if (lane == 0) {
                ok = mbar_wait_bounded(smem_u32(&empty[ps]), (uint32_t)((prev / kPfStages) & 1), status);
                if (ok) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    issue(prev + kPfStages);
                }
            }
            if (!__all_sync(0xFFFFFFFFu, ok)) { alive = false; break; }
        }
    }

    // quad-reduce the row sums
    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 1); l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 2);
    l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 1); l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 2);
    // fail closed: a wait that gave up (here or anywhere on this handle) means no output
    const bool poisoned = !alive || __ldcg(status) != 0;

    if (n_chunks == 1) {
        // the tile saw its whole visible context: normalised rows straight to `out`
        if (poisoned) return;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            if (!(half ? v1 : v0)) continue;
            const int r = half ? r1 : r0;
            const float inv = 1.0f / ((half ? l1 : l0) + 1e-8f);
            const size_t base = ((size_t)(st.q_base[b] + tok_first + r / G) * g.H + (size_t)kvh * G + r % G) * D + 2 * j;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const float x = o[nt][2 * half] * inv, y = o[nt][2 * half + 1] * inv;
                if (out_dtype == DT_FP32) *reinterpret_cast<float2*>((float*)out + base + 8 * nt) = make_float2(x, y);
                else *reinterpret_cast<uint32_t*>((uint16_t*)out + base + 8 * nt) = pack2<BF>(x, y);
            }
        }
        return;
    }

    // ---- split context: (o, m, l) of this chunk, then the CTA that arrives last merges the tile's chunks ----
    // region of the sequence: [chunk][nq * H columns][D + 2]; column = query token * H + head
    float* region = partials + (size_t)pf.poff[b] * g.H * (D + 2);
    const int HP = nq * g.H;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        if (!(half ? v1 : v0)) continue;
        const int r = half ? r1 : r0;
        float* prow = region + partial_off(chunk, (tok_first + r / G) * g.H + kvh * G + r % G, HP, D);
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
            *reinterpret_cast<float2*>(prow + 8 * nt + 2 * j) = make_float2(o[nt][2 * half], o[nt][2 * half + 1]);
        if (j == 0) *reinterpret_cast<float2*>(prow + D) = make_float2(half ? m1 : m0, half ? l1 : l0);
    }
    __syncthreads();                                        // the CTA's rows are complete ...
    if (threadIdx.x == 0) {
        __threadfence();                                    // ... and ordered before the ticket, device-wide
        const int tiles = (nq + tpt - 1) / tpt;
        int* c = counters + pf.cbase[b] + kvh * tiles + tile;
        const int ticket = atomicAdd(c, 1);
        const int last = ticket == n_chunks - 1;
        if (last) *c = 0;                                   // nobody else touches it again in this launch
        *s_flag = last;
    }
    __syncthreads();
    if (*s_flag) {
        const MergeOut mo{nullptr, out, nullptr, out_dtype, nullptr, status};
        merge_rows(g, mo, b, kvh, G, 0, n_chunks, region, MergeMap{G * tok_cnt, HP, st.q_base[b] + tok_first, tok_first, 0});
    }
}

template <bool BF, int D>
cudaError_t launch_pf(const Geometry& g, const CUtensorMap* map, const StepDev& st, const PrefillDev& pf,
                      const int32_t* page_table, const void* q, void* out, int out_dtype, float* partials,
                      int* counters, int* status, cudaStream_t s) {
    using C = PfCfg<D>;
    auto kern = prefill_mma_kernel<BF, D>;
    static bool attr_done[64] = {};                         // per instantiation and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    kern<<<pf.n_items, kWarps * 32, C::SMEM_BYTES, s>>>(*map, g, st, pf, page_table, (const uint16_t*)q, out, out_dtype,
                                                        partials, counters, status);
    return cudaGetLastError();
}

}  // namespace

bool prefill_mma_supported(const Geometry& g) {
    return decode_mma_supported(g) && g.dtype != DT_FP8;
}

// Attention for the query tokens of the sequences the prefill work list covers (pf.items): q and out are
// [n_tokens][H][D] (the order of the step's appended rows); 16-bit pools, page size 16, no cold pages.
// `counters` holds one zeroed int per (sequence, kv head, tile) group (pf.cbase); `partials` the split
// regions (pf.poff).
cudaError_t launch_prefill_mma(const Geometry& g, const CUtensorMap* map, const StepDev& st, const PrefillDev& pf,
                               const int32_t* page_table, const void* q, void* out, int out_dtype, float* partials,
                               int* counters, int* status, cudaStream_t s) {
    if (pf.n_items <= 0) return cudaSuccess;
    if (!prefill_mma_supported(g) || !counters || !status) return cudaErrorNotSupported;
    if (out_dtype != DT_FP32 && out_dtype != g.io_dtype) return cudaErrorInvalidValue;
    if (g.dtype == DT_BF16)
        return g.D == 128 ? launch_pf<true, 128>(g, map, st, pf, page_table, q, out, out_dtype, partials, counters, status, s)
                          : launch_pf<true, 64>(g, map, st, pf, page_table, q, out, out_dtype, partials, counters, status, s);
    return g.D == 128 ? launch_pf<false, 128>(g, map, st, pf, page_table, q, out, out_dtype, partials, counters, status, s)
                      : launch_pf<false, 64>(g, map, st, pf, page_table, q, out, out_dtype, partials, counters, status, s);
}

}  // namespace tk
