// decode_mma.cu — paged GQA decode attention for sm_100a: TMA-staged pages,
// tensor-core QK^T / PV tiles, online softmax, split-KV partials.
//
// Arithmetic contract: that of attention_decode_kernel (reference:
// src/compute/cuda/attention.cu:58-157) — score = (q.k)/sqrtf(D), running max from
// -1e30f, FP32 accumulation, GQA map kv_head = head/(H/Hkv) — evaluated as an online
// softmax whose (o, m, l) partials are merged by the LSE combine (decode_simt.cu).
//
// Schedule.  One CTA per work item (sequence, kv head, chunk of pages).  A pool tile
// (page, kv head) is [K: 16 tokens x D][V: 16 tokens x D], contiguous in HBM, so one
// TMA box of 32 rows x 128 bytes (two boxes when a row is 256 bytes) brings K and V of a
// page into shared memory with the 128-byte swizzle that makes ldmatrix conflict-free.
// Each of the 4 warps owns every 4th page of the chunk and runs a private ring of
// 2-3 TMA stages (own mbarriers, no CTA-wide barrier in the loop), so a CTA keeps up to 8-12
// page tiles in flight and three CTAs share an SM.  The G query heads of the group are the M rows of
// m16n8k16 MMAs (rows >= G are zero padding): S = Q K^T over one page (2 n-tiles x D/16
// k-steps), softmax in registers, O += P V (D/8 n-tiles).  FP8 pools are expanded to
// fp16 in registers (cvt.rn.f16x2.e4m3x2, exact) with the per-page K scale folded into
// the score scale and the V scale folded into P.
//
// The path is HBM-bound: 4 flop/B (bf16, G=4) to 16 flop/B (fp8, G=8); the tensor pipe
// is used because FP32 SIMT FMAs cannot keep up with 6.5 TB/s at those intensities, not
// because the op is a large contraction.  tcgen05 needs M >= 64 rows; with 4-16 query
// rows mma.sync is the fitting instruction.
#include "tk_kernels.cuh"
#include "tk_merge.cuh"
#include "tk_mma.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cudaTypedefs.h>

#include <algorithm>

namespace tk {

namespace {

// Measured on B200, 8B-shape bf16: 2 stages x 3 CTAs/SM beats 3 x 2 (fewer idle slots while a CTA
// ramps up or merges) and 4 x 1.
constexpr int kStagesBig = 2;       // tiles of 8 KB (16-bit, D=128)
constexpr int kStagesSmall = 3;     // tiles of 4 KB (FP8, or D=64)
constexpr int kMinCtas = 3;
// FP8 caches keep each sequence's last, partly filled page in the 16-bit io type ("open page").
// Its 1..15 tokens are one work item of kind 1: plain SIMT arithmetic (reference form: score =
// q.k/sqrtf(D), expf, FP32), one token per warp at a time, all MAXG query heads of the group.
// With fa.k set the item first stores this step's new token into the open page (decode steps
// that do not complete a page), so that such a step needs no separate append launch.
template <bool IO_BF16, int MAXG>
__device__ __forceinline__ void open_page_item(uint8_t* smem, const Geometry& g, const LayerPtrs& lp, const StepDev& st,
                                               const int4 it, const uint16_t* __restrict__ q, float* __restrict__ partials,
                                               const MergeOut& mo, const FuseAppend& fa, int* s_flag) {
    constexpr int D = 128, EPL = 4;
    const int b = it.x, row_idx = it.y, kvh = it.z;
    const int seq = st.seq[b], len = st.len[b];
    const int G = g.H / g.Hkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = len - (len / kPage) * kPage;              // tokens in the open page (>= 1 for this item)
    uint16_t* open_k = (uint16_t*)lp.open_pages + (((size_t)seq * g.Hkv + kvh) * 2) * kPage * D;
    uint16_t* open_v = open_k + (size_t)kPage * D;
    float* qs = reinterpret_cast<float*>(smem);             // [G][D]
    float* red = qs + MAXG * D;                             // [kWarps][G][D+2]
    auto cvt = [](uint16_t x) -> float {
        return IO_BF16 ? __uint_as_float((uint32_t)x << 16) : __half2float(__ushort_as_half(x));
    };
    const int new_tok = fa.k != nullptr ? st.new_tok[b] : -1;
    if (new_tok >= 0 && warp == 0) {                        // the new token is the page's last row
        const int kv = lane >> 4, c = lane & 15;
        const uint16_t* src = (const uint16_t*)(kv ? fa.v : fa.k) + ((size_t)new_tok * g.Hkv + kvh) * D + c * 8;
        *reinterpret_cast<uint4*>((kv ? open_v : open_k) + (size_t)(n - 1) * D + c * 8) = *reinterpret_cast<const uint4*>(src);
    }
    for (int i = threadIdx.x; i < G * D; i += blockDim.x)
        qs[i] = cvt(q[((size_t)b * g.H + (size_t)kvh * G) * D + i]);
    __syncthreads();

    const float scale = 1.0f / sqrtf((float)D);
    float m[MAXG], l[MAXG], o[MAXG][EPL];
#pragma unroll
    for (int gq = 0; gq < MAXG; gq++) { m[gq] = -1e30f; l[gq] = 0.0f; o[gq][0] = o[gq][1] = o[gq][2] = o[gq][3] = 0.0f; }
    for (int r = warp; r < n; r += kWarps) {
        const uint2 kw = *reinterpret_cast<const uint2*>(open_k + (size_t)r * D + lane * EPL);
        const uint2 vw = *reinterpret_cast<const uint2*>(open_v + (size_t)r * D + lane * EPL);
        const float kf[4] = {cvt((uint16_t)kw.x), cvt((uint16_t)(kw.x >> 16)), cvt((uint16_t)kw.y), cvt((uint16_t)(kw.y >> 16))};
        const float vf[4] = {cvt((uint16_t)vw.x), cvt((uint16_t)(vw.x >> 16)), cvt((uint16_t)vw.y), cvt((uint16_t)(vw.y >> 16))};
#pragma unroll
        for (int gq = 0; gq < MAXG; gq++) {
            if (gq < G) {
                float dot = 0.0f;
#pragma unroll
                for (int e = 0; e < EPL; e++) dot += qs[gq * D + lane * EPL + e] * kf[e];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, off);
                const float sc = dot * scale;
                const float mn = fmaxf(m[gq], sc);
                const float alpha = expf(m[gq] - mn), p = expf(sc - mn);
                l[gq] = l[gq] * alpha + p;
#pragma unroll
                for (int e = 0; e < EPL; e++) o[gq][e] = o[gq][e] * alpha + p * vf[e];
                m[gq] = mn;
            }
        }
    }
    auto red_at = [&](int w, int row, int d) -> float& { return red[((size_t)w * G + row) * (D + 2) + d]; };
#pragma unroll
    for (int gq = 0; gq < MAXG; gq++) {
        if (gq < G) {
#pragma unroll
            for (int e = 0; e < EPL; e++) red_at(warp, gq, lane * EPL + e) = o[gq][e];
            if (lane == 0) { red_at(warp, gq, D) = m[gq]; red_at(warp, gq, D + 1) = l[gq]; }
        }
    }
    __syncthreads();
    pdl_wait();                                             // the split-KV rows and counters are shared with the launch before
    const int prow = st.chunk_base[b] + row_idx;
    for (int idx = threadIdx.x; idx < G * (D + 2); idx += blockDim.x) {
        const int row = idx / (D + 2), d = idx % (D + 2);
        float M = -1e30f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, red_at(w, row, D));
        float val = M;
        if (d != D) {
            val = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) val += red_at(w, row, d) * expf(red_at(w, row, D) - M);
        }
        partials[partial_off(prow, kvh * G + row, g.H, D) + d] = val;
    }
    merge_if_last(g, st, mo, b, kvh, G, partials, s_flag);
}

template <int KIND, int D>
struct Cfg {
    static constexpr int ESIZE = KIND == K_FP8 ? 1 : 2;
    static constexpr int ROW_BYTES = D * ESIZE;
    static constexpr int NBOX = ROW_BYTES / 128;            // TMA boxes per (page, kv head) tile
    static constexpr int STAGE_BYTES = NBOX * kBoxBytes;
    static constexpr int BOX_W = 128 / ESIZE;               // box width in elements
    static constexpr bool MMA_BF16 = KIND == K_BF16;        // FP8 computes in fp16
    static constexpr int STAGES = STAGE_BYTES >= 8192 ? kStagesBig : kStagesSmall;
    static constexpr int SMEM_BYTES = kWarps * STAGES * STAGE_BYTES + 1024 + 128;
};

// IO_BF16: type of q (relevant for FP8, where the MMA type is fp16 regardless).
// GHI: more than 8 rows of the M tile carry data (a group of more than 8 query heads, or several tokens).
// MULTI (16-bit pools): every sequence brings nq query tokens - the tokens the step appended, already in
// the pool - and token j attends causally to positions <= len - nq + j.  Row j*G + gg of the M tile is
// token j, head gg of the group (G * nq <= 16), so the tokens share one pass over the pages: what a
// speculative decoder's verification of nq drafted tokens needs (the reference runs the layer once per
// token there: src/inference/speculative.cpp:262-272).
// FP8 pools with a group of at most 8 query heads run the products transposed: S^T = K Q^T and
// O^T = V^T P^T, tokens (dims) as the 16 rows of the MMA and the 8 heads as its 8 columns, so that no row of
// a tile is padding: half the MMAs per page, half the accumulator registers (4 CTAs per SM instead of 3).
template <int KIND, bool GHI, bool MULTI>
constexpr bool kTransposed = KIND == K_FP8 && !GHI && !MULTI;

template <int KIND, int D, bool IO_BF16, bool GHI, bool MULTI>
__global__ void __launch_bounds__(kWarps * 32, kTransposed<KIND, GHI, MULTI> ? kMinCtas + 1 : kMinCtas)
decode_mma_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_cold, Geometry g, LayerPtrs lp, StepDev st,
                  const int32_t* __restrict__ page_table, const uint16_t* __restrict__ q,
                  float* __restrict__ partials, int* __restrict__ status, MergeOut mo, FuseAppend fa) {
    using C = Cfg<KIND, D>;
    constexpr int kStages = C::STAGES;
    constexpr bool BF = C::MMA_BF16;
    constexpr int KS = D / 16;                              // k-steps of QK^T
    constexpr bool SWAP = kTransposed<KIND, GHI, MULTI>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + kWarps * kStages * C::STAGE_BYTES);
    int* s_flag = (int*)(bars + kWarps * kStages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gr = lane >> 2, j = lane & 3;                 // fragment row / column-pair index
    const int G = g.H / g.Hkv;

    // A launch of the next layer may begin as soon as every CTA of this one has STARTED (the hardware hands the
    // dependent grid only the slots this grid no longer needs): its CTAs read what kernels of other layers leave
    // alone - their own layer's pool, q, the step's metadata - write only their own layer's pool row, and wait
    // (pdl_wait below) before they touch what is shared with this launch: split-KV rows, arrival counters, `out`.
    // So the last, ragged wave of one layer runs beside the first wave of the next.
    pdl_launch_dependents();
    const int4 it = st.items[blockIdx.x];
    if (KIND == K_FP8 && it.w == 1) {                       // the 16-bit open page of an FP8 cache
        open_page_item<IO_BF16, GHI ? 16 : 8>(smem, g, lp, st, it, q, partials, mo, fa, s_flag);
        return;
    }
    const int b = it.x, chunk = it.y, kvh = it.z;
    const int seq = st.seq[b], len = st.len[b];
    const int nq = MULTI ? st.nq[b] : 1;                    // query tokens of this sequence
    const int tok0 = MULTI ? (int)blockIdx.y * (16 / G) : 0;  // first query token of this CTA's token group
    const int nq_g = MULTI ? min(nq - tok0, 16 / G) : 1;    // query tokens of the group
    if (MULTI && nq_g <= 0) return;                         // this sequence has no such group
    const int rows = G * nq_g;                              // rows of the M tile that carry data
    const int q_row0 = MULTI ? st.q_base[b] + tok0 : b;     // row of q / out of the group's first query token
    const int pool_tokens = KIND == K_FP8 ? (len / kPage) * kPage : len;
    const int t0 = chunk * st.chunk_tokens;
    // the group's last token sees len - nq + tok0 + nq_g positions: nothing beyond is fetched
    const int t1 = min(MULTI ? len - nq + tok0 + nq_g : pool_tokens, t0 + st.chunk_tokens);
    const int n_pages = t1 > t0 ? (t1 - t0 + kPage - 1) / kPage : 0;
    const int lp0 = t0 / kPage;
    const int n_w = n_pages > warp ? (n_pages - warp + kWarps - 1) / kWarps : 0;   // pages of this warp (<= 32)
    // fused append (decode steps, 16-bit pools): row of this sequence's new token in fa.k / fa.v
    const int new_tok = (KIND != K_FP8 && fa.k != nullptr) ? st.new_tok[b] : -1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kWarps * kStages; i++) mbar_init(smem_u32(&bars[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // lane i keeps the physical page (and FP8 scales) of this warp's i-th page
    int my_page = 0;
    float my_ks = 1.0f, my_vs = 1.0f;
    if (lane < n_w) {
        my_page = page_table[(size_t)seq * g.max_pages_per_seq + lp0 + warp + kWarps * lane];
        if (KIND == K_FP8) {
            const float2 sc = *reinterpret_cast<const float2*>(lp.scales + ((size_t)my_page * g.Hkv + kvh) * 2);
            my_ks = sc.x; my_vs = sc.y;
        }
    }

    uint8_t* wstage = smem + (size_t)warp * kStages * C::STAGE_BYTES;
    auto issue = [&](int i) {                               // called by lane 0 only
        const int page = __shfl_sync(0xFFFFFFFFu, my_page, i);
        if (lane == 0) {
            const int s = i % kStages;
            const uint32_t bar = smem_u32(&bars[warp * kStages + s]);
            const uint32_t dst = smem_u32(wstage + (size_t)s * C::STAGE_BYTES);
            mbar_expect_tx(bar, C::STAGE_BYTES);
            const CUtensorMap* src = (page & kColdBit) ? &tmap_cold : &tmap;   // cold pages come from the staged copy
            const int row = ((page & ~kColdBit) * g.Hkv + kvh) * 32;
#pragma unroll
            for (int h = 0; h < C::NBOX; h++) tma_load_2d(dst + h * kBoxBytes, src, h * C::BOX_W, row, bar);
        }
    };
    for (int i = 0; i < kStages && i < n_w; i++) issue(i);

    // ---- Q fragments (A operand), rows >= G are zero -------------------------------
    uint32_t qa[SWAP ? 1 : KS][4];
    uint32_t qb[SWAP ? KS : 1][2];                          // transposed form: Q^T as the B operand, column gr = head gr
    if constexpr (SWAP) {
        // k index (2j,2j+1) <-> dims 16kk+4j,+1 ; (2j+8,2j+9) <-> dims 16kk+4j+2,+3 (the order the K codes arrive in)
        const uint16_t* qrow = q + ((size_t)q_row0 * g.H + (size_t)kvh * G + gr) * D;
#pragma unroll
        for (int kk = 0; kk < KS; kk++) {
            const uint2 x = gr < rows ? *reinterpret_cast<const uint2*>(qrow + 16 * kk + 4 * j) : make_uint2(0, 0);
            uint32_t w[2] = {x.x, x.y};
            if (IO_BF16) {                                  // bf16 -> fp16 (exact in fp16's normal range)
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);
                    w[i] = pack2<false>(lo, hi);
                }
            }
            qb[kk][0] = w[0]; qb[kk][1] = w[1];
        }
    } else {
        // row r of the tile: token r / G of the sequence, head r % G of the group
        const uint16_t* qrow0 = q + ((size_t)(q_row0 + (MULTI ? gr / G : 0)) * g.H + (size_t)kvh * G + (MULTI ? gr % G : gr)) * D;
        const uint16_t* qrow1 = MULTI ? q + ((size_t)(q_row0 + (gr + 8) / G) * g.H + (size_t)kvh * G + (gr + 8) % G) * D
                                      : qrow0 + (size_t)8 * D;
        const bool v0 = gr < rows, v1 = GHI && (gr + 8 < rows);
#pragma unroll
        for (int kk = 0; kk < KS; kk++) {
            uint32_t w[4];
            if (KIND == K_FP8) {
                // k index (2j,2j+1) <-> dims 16kk+4j,+1 ; (2j+8,2j+9) <-> dims 16kk+4j+2,+3
                const uint2 x0 = v0 ? *reinterpret_cast<const uint2*>(qrow0 + 16 * kk + 4 * j) : make_uint2(0, 0);
                const uint2 x1 = v1 ? *reinterpret_cast<const uint2*>(qrow1 + 16 * kk + 4 * j) : make_uint2(0, 0);
                w[0] = x0.x; w[2] = x0.y; w[1] = x1.x; w[3] = x1.y;
                if (IO_BF16) {                              // bf16 -> fp16 (exact in fp16's normal range)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);
                        w[i] = pack2<false>(lo, hi);
                    }
                }
            } else {
                w[0] = v0 ? *reinterpret_cast<const uint32_t*>(qrow0 + 16 * kk + 2 * j) : 0u;
                w[2] = v0 ? *reinterpret_cast<const uint32_t*>(qrow0 + 16 * kk + 8 + 2 * j) : 0u;
                w[1] = v1 ? *reinterpret_cast<const uint32_t*>(qrow1 + 16 * kk + 2 * j) : 0u;
                w[3] = v1 ? *reinterpret_cast<const uint32_t*>(qrow1 + 16 * kk + 8 + 2 * j) : 0u;
                if (fa.rope_tab) {                          // the query is the token at position len-1
                    const float2* tab = fa.rope_tab + (size_t)b * (D / 2);
                    w[0] = rope_pair<BF>(w[0], tab, 16 * kk + 2 * j);
                    w[2] = rope_pair<BF>(w[2], tab, 16 * kk + 8 + 2 * j);
                    if (GHI) {
                        w[1] = rope_pair<BF>(w[1], tab, 16 * kk + 2 * j);
                        w[3] = rope_pair<BF>(w[3], tab, 16 * kk + 8 + 2 * j);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) qa[kk][i] = w[i];
        }
    }

    // ---- running state -------------------------------------------------------------
    // 16-bit: o[nt] is the C fragment of n-tile nt (dims 8nt..8nt+7).
    // FP8:    o[2c] / o[2c+1] are the even-dim / odd-dim tiles of 16-dim chunk c.
    // Transposed (FP8, group <= 8): o[2c] / o[2c+1] hold the even / odd dims of 32-dim chunk c: element [0],[1] =
    //         (dim 32c + 2gr (+1), heads 2j, 2j+1), [2],[3] = (dim 32c + 16 + 2gr (+1), heads 2j, 2j+1);
    //         m0/l0 belong to head 2j, m1/l1 to head 2j+1, m in base-2 units, l summed over this lane's tokens only.
    constexpr int NT = SWAP ? D / 16 : D / 8;
    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f; }
    float m0 = -1e30f, m1 = -1e30f, l0 = 0.0f, l1 = 0.0f;  // rows gr and gr+8
    const float sm_scale = 1.0f / sqrtf((float)D);
    bool alive = true;

    for (int i = 0; i < n_w; i++) {
        const int s = i % kStages;
        const uint32_t bar = smem_u32(&bars[warp * kStages + s]);
        // warp-uniform verdict, so that a give-up never splits the warp before a shuffle
        if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded(bar, (uint32_t)((i / kStages) & 1), status))) { alive = false; break; }
        uint8_t* stg = wstage + (size_t)s * C::STAGE_BYTES;
        const uint32_t stg_u = smem_u32(stg);
        const int tok_base = (lp0 + warp + kWarps * i) * kPage;
        const int n_valid = min(kPage, t1 - tok_base);     // < 16 only on a sequence's last page
        // tokens of this page that rows gr / gr+8 may attend to (causal limit of their query token)
        const int nv0 = MULTI ? max(0, min(n_valid, len - nq + tok0 + gr / G + 1 - tok_base)) : n_valid;
        const int nv1 = MULTI ? max(0, min(n_valid, len - nq + tok0 + (gr + 8) / G + 1 - tok_base)) : n_valid;

        float sc_k = sm_scale, sc_v = 1.0f;
        if (KIND == K_FP8) {
            sc_k *= __shfl_sync(0xFFFFFFFFu, my_ks, i);
            sc_v = __shfl_sync(0xFFFFFFFFu, my_vs, i);
        }

        if (KIND != K_FP8 && new_tok >= 0 && tok_base == ((len - 1) & ~(kPage - 1))) {
            // This page holds the token appended by this step.  The TMA tile has the stale row:
            // put the new K/V row into shared memory for the MMAs and into the pool for later steps.
            const int r = (len - 1) & (kPage - 1);
            const int page = __shfl_sync(0xFFFFFFFFu, my_page, i);
            const int kv = lane >> 4;
            const uint16_t* src = (const uint16_t*)(kv ? fa.v : fa.k) + ((size_t)new_tok * g.Hkv + kvh) * D;
            uint16_t* dst = (uint16_t*)lp.pool + ((((size_t)page * g.Hkv + kvh) * 2 + kv) * kPage + r) * D;
            for (int c = lane & 15; c < D / 8; c += 16) {
                uint4 val = *reinterpret_cast<const uint4*>(src + c * 8);
                if (fa.rope_tab && kv == 0) {               // K row: rotate its 4 pairs before it is stored
                    const float2* tab = fa.rope_tab + (size_t)b * (D / 2);
                    val.x = rope_pair<BF>(val.x, tab, c * 8 + 0);
                    val.y = rope_pair<BF>(val.y, tab, c * 8 + 2);
                    val.z = rope_pair<BF>(val.z, tab, c * 8 + 4);
                    val.w = rope_pair<BF>(val.w, tab, c * 8 + 6);
                }
                *reinterpret_cast<uint4*>(stg + (c >> 3) * kBoxBytes + swz(kv * 16 + r, c & 7)) = val;
                *reinterpret_cast<uint4*>(dst + c * 8) = val;
            }
            __syncwarp();
        }
        if (KIND != K_FP8 && n_valid < kPage) {
            // stale rows of a partly filled page: zero the V rows so 0 * garbage cannot make NaN
            for (int idx = lane; idx < (kPage - n_valid) * 8 * C::NBOX; idx += 32) {
                const int h = idx / ((kPage - n_valid) * 8), rem = idx % ((kPage - n_valid) * 8);
                const int r = 16 + n_valid + rem / 8, c = rem % 8;
                *reinterpret_cast<uint4*>(stg + h * kBoxBytes + r * 128 + c * 16) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }

        if constexpr (SWAP) {
            // ---- S^T = K Q^T: rows = the page's 16 tokens, columns = heads ----
            float sT[4] = {0.f, 0.f, 0.f, 0.f}, uT[4] = {0.f, 0.f, 0.f, 0.f};
            const int mi = lane >> 3;                       // matrix this lane addresses: token half mi & 1, 16-dim chunk mi >> 1
            {
                const int row = ((mi & 1) << 3) + (lane & 7);
#pragma unroll
                for (int cp = 0; cp < D / 32; cp++) {
                    uint32_t r0, r1, r2, r3;                // (tokens 0-7 | 8-15) x (chunk 2cp | 2cp+1), 4 codes of one token each
                    ldsm_x4(stg_u + swz(row, 2 * cp + (mi >> 1)), r0, r1, r2, r3);
                    const uint32_t a0[4] = {e4m3x2_to_f16x2(r0), e4m3x2_to_f16x2(r1), e4m3x2_to_f16x2(r0 >> 16), e4m3x2_to_f16x2(r1 >> 16)};
                    mma16816<false>(sT, a0, qb[2 * cp][0], qb[2 * cp][1]);
                    const uint32_t a1[4] = {e4m3x2_to_f16x2(r2), e4m3x2_to_f16x2(r3), e4m3x2_to_f16x2(r2 >> 16), e4m3x2_to_f16x2(r3 >> 16)};
                    mma16816<false>(uT, a1, qb[2 * cp + 1][0], qb[2 * cp + 1][1]);
                }
            }
            // ---- softmax down the columns: this lane has tokens gr, gr+8 of heads 2j ([0],[2]) and 2j+1 ([1],[3]) ----
            // (sealed pages are always full, so nothing is masked).  The reference maximum of a head moves only when a
            // score exceeds it by 2^4: one vote per page instead of a shuffle reduction; probabilities stay below 16.
            const float k2 = sc_k * kLog2e;
            const float a0 = (sT[0] + uT[0]) * k2, a1 = (sT[1] + uT[1]) * k2, a2 = (sT[2] + uT[2]) * k2, a3 = (sT[3] + uT[3]) * k2;
            float xa = fmaxf(a0, a2), xb = fmaxf(a1, a3);
            if (__any_sync(0xFFFFFFFFu, xa > m0 + 4.0f || xb > m1 + 4.0f)) {
#pragma unroll
                for (int off = 4; off < 32; off <<= 1) {
                    xa = fmaxf(xa, __shfl_xor_sync(0xFFFFFFFFu, xa, off));
                    xb = fmaxf(xb, __shfl_xor_sync(0xFFFFFFFFu, xb, off));
                }
                const float na = fmaxf(m0, xa), nb = fmaxf(m1, xb);
                const float al0 = ex2(m0 - na), al1 = ex2(m1 - nb);
                l0 *= al0; l1 *= al1;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) { o[nt][0] *= al0; o[nt][2] *= al0; o[nt][1] *= al1; o[nt][3] *= al1; }
                m0 = na; m1 = nb;
            }
            const float p0 = ex2(a0 - m0), p1 = ex2(a1 - m1), p2 = ex2(a2 - m0), p3 = ex2(a3 - m1);
            l0 += p0 + p2; l1 += p1 + p3;
            // ---- O^T += V^T P^T: P^T (tokens x heads as the B operand) is the transpose of what this lane holds ----
            uint32_t b0, b1;
            {
                const uint32_t t0 = pack2<false>(p0 * sc_v, p1 * sc_v), t1 = pack2<false>(p2 * sc_v, p3 * sc_v);
                asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(b0) : "r"(t0));
                asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(b1) : "r"(t1));
            }
            {
                const int row = 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
                for (int cp = 0; cp < D / 32; cp++) {
                    uint32_t r0, r1, r2, r3;                // dims pair gr of (chunk 2cp | 2cp+1) for tokens (2j,2j+1 | 2j+8,2j+9)
                    ldsm_x4_t(stg_u + swz(row, 2 * cp + (mi >> 1)), r0, r1, r2, r3);
                    // bytes (even dim tok 2j, even dim tok 2j+1, odd dim tok 2j, odd dim tok 2j+1)
                    r0 = __byte_perm(r0, 0, 0x3120); r1 = __byte_perm(r1, 0, 0x3120);
                    r2 = __byte_perm(r2, 0, 0x3120); r3 = __byte_perm(r3, 0, 0x3120);
                    const uint32_t ae[4] = {e4m3x2_to_f16x2(r0), e4m3x2_to_f16x2(r2), e4m3x2_to_f16x2(r1), e4m3x2_to_f16x2(r3)};
                    mma16816<false>(o[2 * cp], ae, b0, b1);
                    const uint32_t ao[4] = {e4m3x2_to_f16x2(r0 >> 16), e4m3x2_to_f16x2(r2 >> 16), e4m3x2_to_f16x2(r1 >> 16), e4m3x2_to_f16x2(r3 >> 16)};
                    mma16816<false>(o[2 * cp + 1], ao, b0, b1);
                }
            }
        } else {
        // ---- S = Q K^T over the page's 16 tokens ----
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        if (KIND == K_FP8) {
            // the kernel is close to its issue limit here, and a chain of eight dependent MMAs per accumulator
            // leaves the warp waiting on fixed latencies: four accumulators (even / odd k-steps), summed at the end
            float u0[4] = {0.f, 0.f, 0.f, 0.f}, u1[4] = {0.f, 0.f, 0.f, 0.f};
            const int row = ((lane >> 4) << 3) + (lane & 7);
#pragma unroll
            for (int cp = 0; cp < D / 32; cp++) {
                uint32_t r0, r1, r2, r3;
                ldsm_x4(stg_u + swz(row, 2 * cp + ((lane >> 3) & 1)), r0, r1, r2, r3);
                mma16816<BF>(s0, qa[2 * cp],     e4m3x2_to_f16x2(r0), e4m3x2_to_f16x2(r0 >> 16));
                mma16816<BF>(s1, qa[2 * cp],     e4m3x2_to_f16x2(r2), e4m3x2_to_f16x2(r2 >> 16));
                mma16816<BF>(u0, qa[2 * cp + 1], e4m3x2_to_f16x2(r1), e4m3x2_to_f16x2(r1 >> 16));
                mma16816<BF>(u1, qa[2 * cp + 1], e4m3x2_to_f16x2(r3), e4m3x2_to_f16x2(r3 >> 16));
            }
#pragma unroll
            for (int e = 0; e < 4; e++) { s0[e] += u0[e]; s1[e] += u1[e]; }
        } else {
            const int row = ((lane >> 4) << 3) + (lane & 7);
#pragma unroll
            for (int kk = 0; kk < KS; kk++) {
                const int cc = 2 * kk + ((lane >> 3) & 1);
                uint32_t r0, r1, r2, r3;
                ldsm_x4(stg_u + (cc >> 3) * kBoxBytes + swz(row, cc & 7), r0, r1, r2, r3);
                mma16816<BF>(s0, qa[kk], r0, r1);
                mma16816<BF>(s1, qa[kk], r2, r3);
            }
        }

        // ---- online softmax (row gr in [0],[1]; row gr+8 in [2],[3]) ----
        float p0[4], p1[4];
        {
            const int c0 = 2 * j;                           // token columns of this thread: c0, c0+1, c0+8, c0+9
            float a0 = s0[0] * sc_k, a1 = s0[1] * sc_k, a2 = s1[0] * sc_k, a3 = s1[1] * sc_k;
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
            p0[0] = ex2(fmaf(a0, kLog2e, nb)); p0[1] = ex2(fmaf(a1, kLog2e, nb));
            p1[0] = ex2(fmaf(a2, kLog2e, nb)); p1[1] = ex2(fmaf(a3, kLog2e, nb));
            if (MULTI) {                                    // a row may see nothing of a page: exp(-1e30 + 1e30) is 1, not 0
                if (c0 >= nv0) p0[0] = 0.0f;
                if (c0 + 1 >= nv0) p0[1] = 0.0f;
                if (c0 + 8 >= nv0) p1[0] = 0.0f;
                if (c0 + 9 >= nv0) p1[1] = 0.0f;
            }
            l0 = l0 * alpha + (p0[0] + p0[1] + p1[0] + p1[1]);
            // the running maximum rarely moves after the first pages: skip the 2*NT multiplies then
            if (!__all_sync(0xFFFFFFFFu, mn == m0)) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++) { o[nt][0] *= alpha; o[nt][1] *= alpha; }
            }
            m0 = mn;
        }
        if (GHI) {
            const int c0 = 2 * j;
            float a0 = s0[2] * sc_k, a1 = s0[3] * sc_k, a2 = s1[2] * sc_k, a3 = s1[3] * sc_k;
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
            p0[2] = ex2(fmaf(a0, kLog2e, nb)); p0[3] = ex2(fmaf(a1, kLog2e, nb));
            p1[2] = ex2(fmaf(a2, kLog2e, nb)); p1[3] = ex2(fmaf(a3, kLog2e, nb));
            if (MULTI) {
                if (c0 >= nv1) p0[2] = 0.0f;
                if (c0 + 1 >= nv1) p0[3] = 0.0f;
                if (c0 + 8 >= nv1) p1[2] = 0.0f;
                if (c0 + 9 >= nv1) p1[3] = 0.0f;
            }
            l1 = l1 * alpha + (p0[2] + p0[3] + p1[2] + p1[3]);
            if (!__all_sync(0xFFFFFFFFu, mn == m1)) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++) { o[nt][2] *= alpha; o[nt][3] *= alpha; }
            }
            m1 = mn;
        } else {
            p0[2] = p0[3] = p1[2] = p1[3] = 0.0f;
        }

        // ---- O += P V ----
        uint32_t pa[4];
        pa[0] = pack2<BF>(p0[0] * sc_v, p0[1] * sc_v);
        pa[1] = pack2<BF>(p0[2] * sc_v, p0[3] * sc_v);
        pa[2] = pack2<BF>(p1[0] * sc_v, p1[1] * sc_v);
        pa[3] = pack2<BF>(p1[2] * sc_v, p1[3] * sc_v);
        if (KIND == K_FP8) {
            const int row = 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
            for (int cp = 0; cp < D / 32; cp++) {
                uint32_t r0, r1, r2, r3;
                ldsm_x4_t(stg_u + swz(row, 2 * cp + (lane >> 4)), r0, r1, r2, r3);
                const uint32_t e0 = __byte_perm(r0, r1, 0x6420), d0 = __byte_perm(r0, r1, 0x7531);
                const uint32_t e1 = __byte_perm(r2, r3, 0x6420), d1 = __byte_perm(r2, r3, 0x7531);
                mma16816<BF>(o[4 * cp + 0], pa, e4m3x2_to_f16x2(e0), e4m3x2_to_f16x2(e0 >> 16));
                mma16816<BF>(o[4 * cp + 1], pa, e4m3x2_to_f16x2(d0), e4m3x2_to_f16x2(d0 >> 16));
                mma16816<BF>(o[4 * cp + 2], pa, e4m3x2_to_f16x2(e1), e4m3x2_to_f16x2(e1 >> 16));
                mma16816<BF>(o[4 * cp + 3], pa, e4m3x2_to_f16x2(d1), e4m3x2_to_f16x2(d1 >> 16));
            }
        } else {
            const int row = 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {
                const int cc = 2 * np + (lane >> 4);
                uint32_t r0, r1, r2, r3;
                ldsm_x4_t(stg_u + (cc >> 3) * kBoxBytes + swz(row, cc & 7), r0, r1, r2, r3);
                mma16816<BF>(o[2 * np], pa, r0, r1);
                mma16816<BF>(o[2 * np + 1], pa, r2, r3);
            }
        }

        }

        // ---- refill this stage ----
        __syncwarp();
        if (i + kStages < n_w) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(i + kStages);
        }
    }
    // a wait that gave up has set the status word: the merging CTA sees it and writes no output
    (void)alive;
    // ---- merge the 4 warps through shared memory (stage memory is idle now) ----------
    if constexpr (SWAP) {
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, off);
            l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, off);
        }
    } else {
        l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 1); l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 2);
        l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 1); l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 2);
    }
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem);            // [kWarps][rows][D+2]
    auto red_at = [&](int w, int row, int d) -> float& { return red[((size_t)w * rows + row) * (D + 2) + d]; };
    if constexpr (SWAP) {
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {                    // heads 2j and 2j+1
            const int row = 2 * j + hh;
            if (row < rows) {
#pragma unroll
                for (int c = 0; c < D / 32; c++) {
                    red_at(warp, row, 32 * c + 2 * gr + 0) = o[2 * c][hh];
                    red_at(warp, row, 32 * c + 2 * gr + 1) = o[2 * c + 1][hh];
                    red_at(warp, row, 32 * c + 16 + 2 * gr + 0) = o[2 * c][2 + hh];
                    red_at(warp, row, 32 * c + 16 + 2 * gr + 1) = o[2 * c + 1][2 + hh];
                }
                if (gr == 0) {                              // the merge below works in natural-log units
                    red_at(warp, row, D) = (hh ? m1 : m0) * 0.6931471805599453f;
                    red_at(warp, row, D + 1) = hh ? l1 : l0;
                }
            }
        }
    } else {
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int row = gr + 8 * half;
        if (row < rows && (half == 0 || GHI)) {
            if (KIND == K_FP8) {
#pragma unroll
                for (int c = 0; c < D / 16; c++) {
                    red_at(warp, row, 16 * c + 4 * j + 0) = o[2 * c][2 * half + 0];
                    red_at(warp, row, 16 * c + 4 * j + 1) = o[2 * c + 1][2 * half + 0];
                    red_at(warp, row, 16 * c + 4 * j + 2) = o[2 * c][2 * half + 1];
                    red_at(warp, row, 16 * c + 4 * j + 3) = o[2 * c + 1][2 * half + 1];
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    red_at(warp, row, 8 * nt + 2 * j + 0) = o[nt][2 * half + 0];
                    red_at(warp, row, 8 * nt + 2 * j + 1) = o[nt][2 * half + 1];
                }
            }
            if (j == 0) {
                red_at(warp, row, D) = half ? m1 : m0;
                red_at(warp, row, D + 1) = half ? l1 : l0;
            }
        }
    }
    }
    __syncthreads();
    pdl_wait();
    const int prow = st.chunk_base[b] + chunk;
    const int heads_per_row = MULTI ? g.H * st.nq_max : g.H;   // columns of a partial row
    for (int idx = threadIdx.x; idx < rows * (D + 2); idx += blockDim.x) {
        const int row = idx / (D + 2), d = idx % (D + 2);
        float M = -1e30f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, red_at(w, row, D));
        float val;
        if (d == D) {
            val = M;
        } else {
            val = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) val += red_at(w, row, d) * ex2((red_at(w, row, D) - M) * kLog2e);
        }
        const int col = MULTI ? (tok0 + row / G) * g.H + kvh * G + row % G : kvh * G + row;
        partials[partial_off(prow, col, heads_per_row, D) + d] = val;
    }
    merge_if_last(g, st, mo, b, kvh, G, partials, s_flag,
                  MergeMap{rows, heads_per_row, q_row0, MULTI ? tok0 : 0, MULTI ? (int)blockIdx.y * st.n_seqs * g.Hkv : 0});
}

// One warp waits, with the same bounded wait the decode kernel uses, on a barrier that nothing
// ever completes: the wait runs out, the status word is set, the kernel returns normally.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    (void)__all_sync(0xFFFFFFFFu, mbar_wait_bounded(smem_u32(&bar), 0u, status, limit_ns));
}

template <int KIND, int D, bool IO_BF16, bool GHI, bool MULTI = false>
cudaError_t launch_one(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* map,
                       const CUtensorMap* map_cold, const StepDev& st,
                       const int32_t* page_table, const void* q, float* partials, int* status,
                       cudaStream_t s, const MergeOut& mo, const FuseAppend& fa, bool overlap_prev = false) {
    using C = Cfg<KIND, D>;
    auto kern = decode_mma_kernel<KIND, D, IO_BF16, GHI, MULTI>;
    static bool attr_done[64] = {};                         // per instantiation and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    // multi-token attention: one grid row per group of 16/G query tokens
    const int tpg = 16 / (g.H / g.Hkv);
    const dim3 grid(st.n_items, MULTI ? (st.nq_max + tpg - 1) / tpg : 1);
    if (!overlap_prev) {
        kern<<<grid, kWarps * 32, C::SMEM_BYTES, s>>>(*map, *map_cold, g, lp, st, page_table, (const uint16_t*)q,
                                                      partials, status, mo, fa);
        return cudaGetLastError();
    }
    // may start while the kernel before it in the stream drains (see pdl_wait in the kernel)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(kWarps * 32); cfg.dynamicSmemBytes = C::SMEM_BYTES; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, *map, *map_cold, g, lp, st, page_table, (const uint16_t*)q, partials, status, mo, fa);
}

template <int KIND, int D>
cudaError_t launch_kd(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* map,
                      const CUtensorMap* map_cold, const StepDev& st,
                      const int32_t* page_table, const void* q, float* partials, int* status,
                      cudaStream_t s, const MergeOut& mo, const FuseAppend& fa, bool ov) {
    const bool io_bf16 = g.io_dtype == DT_BF16;
    const bool ghi = g.H / g.Hkv > 8;
    if (io_bf16 && ghi)  return launch_one<KIND, D, true, true>(g, lp, map, map_cold, st, page_table, q, partials, status, s, mo, fa, ov);
    if (io_bf16)         return launch_one<KIND, D, true, false>(g, lp, map, map_cold, st, page_table, q, partials, status, s, mo, fa, ov);
    if (ghi)             return launch_one<KIND, D, false, true>(g, lp, map, map_cold, st, page_table, q, partials, status, s, mo, fa, ov);
    return launch_one<KIND, D, false, false>(g, lp, map, map_cold, st, page_table, q, partials, status, s, mo, fa, ov);
}

template <int KIND, int D>
cudaError_t launch_kd_multi(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* map, const StepDev& st,
                            const int32_t* page_table, const void* q, float* partials, int* status,
                            cudaStream_t s, const MergeOut& mo) {
    const FuseAppend fa{nullptr, nullptr, nullptr};
    if ((g.H / g.Hkv) * std::min(st.nq_max, 16 / (g.H / g.Hkv)) > 8)
        return launch_one<KIND, D, KIND == K_BF16, true, true>(g, lp, map, map, st, page_table, q, partials, status, s, mo, fa);
    return launch_one<KIND, D, KIND == K_BF16, false, true>(g, lp, map, map, st, page_table, q, partials, status, s, mo, fa);
}

}  // namespace

// Token groups per sequence are grid rows; each is a pass of its own over the pages it may see.
constexpr int kMaxTokenGroups = 8;
bool decode_mma_multi_supported(const Geometry& g, int nq_max) {
    return decode_mma_supported(g) && g.dtype != DT_FP8 && nq_max >= 1 &&
           (g.H / g.Hkv) * nq_max <= 16 * kMaxTokenGroups;
}
int decode_mma_multi_groups(const Geometry& g, int nq_max) {
    const int tpg = 16 / (g.H / g.Hkv);
    return (nq_max + tpg - 1) / tpg;
}

// Multi-token attention (st.nq / st.q_base / st.nq_max set): q and out are [n_tokens][H][D]; partial rows
// hold H * nq_max columns.  16-bit pools without cold pages; the step's rows are already appended.
cudaError_t launch_decode_mma_multi(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* map, const StepDev& st,
                                    const int32_t* page_table, const void* q, float* partials, int* status,
                                    cudaStream_t s, const MergeOut& mo) {
    if (st.n_items <= 0) return cudaSuccess;
    if (!decode_mma_multi_supported(g, st.nq_max) || st.chunk_tokens > kPage * kWarps * 32 || !mo.counters || mo.peer)
        return cudaErrorNotSupported;
    if (g.dtype == DT_BF16) return g.D == 128 ? launch_kd_multi<K_BF16, 128>(g, lp, map, st, page_table, q, partials, status, s, mo)
                                              : launch_kd_multi<K_BF16, 64>(g, lp, map, st, page_table, q, partials, status, s, mo);
    return g.D == 128 ? launch_kd_multi<K_F16, 128>(g, lp, map, st, page_table, q, partials, status, s, mo)
                      : launch_kd_multi<K_F16, 64>(g, lp, map, st, page_table, q, partials, status, s, mo);
}

cudaError_t launch_bounded_wait_selftest(int* status, unsigned long long limit_ns, cudaStream_t s) {
    bounded_wait_selftest_kernel<<<1, 32, 0, s>>>(status, limit_ns);
    return cudaGetLastError();
}

bool decode_mma_supported(const Geometry& g) {
    if (g.ps != kPage || g.Hkv <= 0 || g.H % g.Hkv != 0 || g.H / g.Hkv > 16 || g.Dv != g.D) return false;
    if (g.dtype == DT_FP8) return g.D == 128;
    if (g.dtype == DT_FP16 || g.dtype == DT_BF16) return (g.D == 64 || g.D == 128) && g.io_dtype == g.dtype;
    return false;
}

// The layer's pool as a 2-D tensor: rows = num_pages*Hkv*2*16 token rows of D elements.
// Box = box_rows rows x 128 bytes, 128-byte swizzle: 32 rows = one tile (K rows then V rows) for the
// mma.sync kernels, 16 rows = the K or the V rows of a page for the tcgen05 prefill kernel.
cudaError_t make_pool_tensor_map(const Geometry& g, void* layer_pool, CUtensorMap* out, int box_rows) {
    static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return e;
        if (qres != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
        encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    }
    const int esize = g.dtype == DT_FP8 ? 1 : 2;
    cuuint64_t dims[2] = {(cuuint64_t)g.D, (cuuint64_t)g.num_pages * g.Hkv * 2 * g.ps};
    cuuint64_t strides[1] = {(cuuint64_t)g.D * esize};
    cuuint32_t box[2] = {(cuuint32_t)(128 / esize), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(out, esize == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                        layer_pool, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t launch_decode_mma(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* map,
                              const CUtensorMap* map_cold, const StepDev& st, const int32_t* page_table, const void* q,
                              float* partials, int* status, cudaStream_t s, const MergeOut* merge,
                              const FuseAppend* fuse, bool overlap_prev) {
    if (st.n_items <= 0) return cudaSuccess;
    const MergeOut mo = merge ? *merge : MergeOut{nullptr, nullptr, nullptr, 0};
    const FuseAppend fa = fuse ? *fuse : FuseAppend{nullptr, nullptr, nullptr};
    if (!map_cold) map_cold = map;
    if (!decode_mma_supported(g) || st.chunk_tokens > kPage * kWarps * 32) return cudaErrorNotSupported;
    const bool ov = overlap_prev;
    if (g.dtype == DT_FP8)  return launch_kd<K_FP8, 128>(g, lp, map, map_cold, st, page_table, q, partials, status, s, mo, fa, ov);
    if (g.dtype == DT_BF16) return g.D == 128 ? launch_kd<K_BF16, 128>(g, lp, map, map_cold, st, page_table, q, partials, status, s, mo, fa, ov)
                                              : launch_kd<K_BF16, 64>(g, lp, map, map_cold, st, page_table, q, partials, status, s, mo, fa, ov);
    return g.D == 128 ? launch_kd<K_F16, 128>(g, lp, map, map_cold, st, page_table, q, partials, status, s, mo, fa, ov)
                      : launch_kd<K_F16, 64>(g, lp, map, map_cold, st, page_table, q, partials, status, s, mo, fa, ov);
}

}  // namespace tk
