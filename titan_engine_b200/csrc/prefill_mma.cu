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
// T * G rows, G = H/Hkv.  One CTA takes a tile of 128 rows (128/G whole tokens) and a range of the
// context (the whole visible context, or one split-KV chunk of it when the sequence has too few
// tiles to fill the GPU).  Its 4 warps own 32 rows each — two sets of the M rows of m16n8k16 MMAs,
// so that every K/V fragment read from shared memory feeds two MMAs — and all consume the SAME K/V
// page tiles: a CTA-wide ring of TMA stages (one elected thread issues cp.async.bulk.tensor.2d per
// page tile; `full` mbarriers carry the byte count, `empty` mbarriers collect one arrival per
// warp), so a page is fetched once per 128 rows instead of once per 16 as in the decode kernel's
// multi-token form.  With T * G >= 128 this is a contraction in its own right (128 flop per K/V
// byte at D = 128), bounded by the tensor pipe, not by HBM.
// Tiles that see the whole visible context write normalised outputs directly; split ones leave
// (o, m, l) partials and the CTA that arrives last for the tile merges them (tk_merge.cuh).
// Every wait is bounded; a wait that gives up sets the status word and nothing is written.
#include "tk_kernels.cuh"
#include "tk_merge.cuh"
#include "tk_mma.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cudaTypedefs.h>

namespace tk {

namespace {

constexpr int kPfStages = 4;              // page tiles in flight per CTA
constexpr int kMT = 2;                    // 16-row MMA tiles per warp: kPrefillRows = 4 warps x kMT x 16
static_assert(kPrefillRows == kWarps * kMT * 16, "tile rows");

template <int D>
struct PfCfg {
    static constexpr int NBOX = D * 2 / 128;                 // TMA boxes per (page, kv head) tile
    static constexpr int STAGE_BYTES = NBOX * kBoxBytes;
    static constexpr int BAR_BYTES = 2 * kPfStages * 8 + 16;  // full + empty barriers, merge flag
    static constexpr int SMEM_BYTES = kPfStages * STAGE_BYTES + BAR_BYTES + kPrefillMaxPages * 4 + 1024;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <bool BF, int D>
__global__ void __launch_bounds__(kWarps * 32, 2)
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

    // ---- this warp's kMT x 16 rows: row r of the CTA tile is query token r / G of the tile, head r % G.
    // Each B fragment (K or V page rows from shared memory) feeds kMT MMAs: half the shared-memory traffic
    // per flop of a 16-row warp tile, which is what bounds a 16-row tile on this path.
    int rr[kMT][2], lim[kMT][2];
    bool vv[kMT][2];
#pragma unroll
    for (int mt = 0; mt < kMT; mt++)
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            rr[mt][hf] = kMT * 16 * warp + 16 * mt + gr + 8 * hf;
            vv[mt][hf] = rr[mt][hf] / G < tok_cnt;
            lim[mt][hf] = base_pos + tok_first + rr[mt][hf] / G + 1;      // positions the row attends to: [0, lim)
        }
    // last position any row of this warp sees (0: the warp has no row)
    const int warp_lim = (kMT * 16 * warp) / G < tok_cnt
                             ? base_pos + tok_first + min(tok_cnt - 1, (kMT * 16 * warp + kMT * 16 - 1) / G) + 1 : 0;

    uint32_t qa[kMT][KS][4];
#pragma unroll
    for (int mt = 0; mt < kMT; mt++) {
        const uint16_t* qrow0 = q + ((size_t)(st.q_base[b] + tok_first + rr[mt][0] / G) * g.H + (size_t)kvh * G + rr[mt][0] % G) * D;
        const uint16_t* qrow1 = q + ((size_t)(st.q_base[b] + tok_first + rr[mt][1] / G) * g.H + (size_t)kvh * G + rr[mt][1] % G) * D;
#pragma unroll
        for (int kk = 0; kk < KS; kk++) {
            qa[mt][kk][0] = vv[mt][0] ? *reinterpret_cast<const uint32_t*>(qrow0 + 16 * kk + 2 * j) : 0u;
            qa[mt][kk][2] = vv[mt][0] ? *reinterpret_cast<const uint32_t*>(qrow0 + 16 * kk + 8 + 2 * j) : 0u;
            qa[mt][kk][1] = vv[mt][1] ? *reinterpret_cast<const uint32_t*>(qrow1 + 16 * kk + 2 * j) : 0u;
            qa[mt][kk][3] = vv[mt][1] ? *reinterpret_cast<const uint32_t*>(qrow1 + 16 * kk + 8 + 2 * j) : 0u;
        }
    }

    float o[kMT][NT][4];
    float mrow[kMT][2], lrow[kMT][2];
#pragma unroll
    for (int mt = 0; mt < kMT; mt++) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++) { o[mt][nt][0] = o[mt][nt][1] = o[mt][nt][2] = o[mt][nt][3] = 0.0f; }
        mrow[mt][0] = mrow[mt][1] = -1e30f;
        lrow[mt][0] = lrow[mt][1] = 0.0f;
    }
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

            // ---- S = Q K^T over the page's 16 tokens: s[mt][0] tokens 0-7, s[mt][1] tokens 8-15 ----
            float sacc[kMT][2][4];
#pragma unroll
            for (int mt = 0; mt < kMT; mt++)
#pragma unroll
                for (int e = 0; e < 4; e++) sacc[mt][0][e] = sacc[mt][1][e] = 0.0f;
            {
                const int row = ((lane >> 4) << 3) + (lane & 7);
#pragma unroll
                for (int kk = 0; kk < KS; kk++) {
                    const int cc = 2 * kk + ((lane >> 3) & 1);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(stg_u + (cc >> 3) * kBoxBytes + swz(row, cc & 7), b0, b1, b2, b3);
#pragma unroll
                    for (int mt = 0; mt < kMT; mt++) {
                        mma16816<BF>(sacc[mt][0], qa[mt][kk], b0, b1);
                        mma16816<BF>(sacc[mt][1], qa[mt][kk], b2, b3);
                    }
                }
            }

            // ---- online softmax per row; a thread holds token columns 2j, 2j+1, 2j+8, 2j+9 of its rows ----
            uint32_t pa[kMT][4];
            const int c0 = 2 * j;
#pragma unroll
            for (int mt = 0; mt < kMT; mt++) {
                float p[2][4];                                  // [half][col]: cols 2j, 2j+1, 2j+8, 2j+9
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    const int nv = vv[mt][hf] ? max(0, min(n_valid, lim[mt][hf] - tok_base)) : 0;
                    float a0 = sacc[mt][0][2 * hf] * sm_scale, a1 = sacc[mt][0][2 * hf + 1] * sm_scale;
                    float a2 = sacc[mt][1][2 * hf] * sm_scale, a3 = sacc[mt][1][2 * hf + 1] * sm_scale;
                    if (c0 >= nv) a0 = -1e30f;
                    if (c0 + 1 >= nv) a1 = -1e30f;
                    if (c0 + 8 >= nv) a2 = -1e30f;
                    if (c0 + 9 >= nv) a3 = -1e30f;
                    float mx = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
                    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
                    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
                    const float mo_ = mrow[mt][hf];
                    const float mn = fmaxf(mo_, mx);
                    const float alpha = ex2((mo_ - mn) * kLog2e);
                    const float nb = -mn * kLog2e;
                    // a row may see nothing of a page: exp(-1e30 + 1e30) is 1, not 0
                    p[hf][0] = c0 < nv ? ex2(fmaf(a0, kLog2e, nb)) : 0.0f;
                    p[hf][1] = c0 + 1 < nv ? ex2(fmaf(a1, kLog2e, nb)) : 0.0f;
                    p[hf][2] = c0 + 8 < nv ? ex2(fmaf(a2, kLog2e, nb)) : 0.0f;
                    p[hf][3] = c0 + 9 < nv ? ex2(fmaf(a3, kLog2e, nb)) : 0.0f;
                    lrow[mt][hf] = lrow[mt][hf] * alpha + (p[hf][0] + p[hf][1] + p[hf][2] + p[hf][3]);
                    // the running maximum rarely moves after the first pages: skip the 2*NT multiplies then
                    if (!__all_sync(0xFFFFFFFFu, mn == mo_)) {
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) { o[mt][nt][2 * hf] *= alpha; o[mt][nt][2 * hf + 1] *= alpha; }
                    }
                    mrow[mt][hf] = mn;
                }
                pa[mt][0] = pack2<BF>(p[0][0], p[0][1]);        // row gr,   tokens 2j, 2j+1
                pa[mt][1] = pack2<BF>(p[1][0], p[1][1]);        // row gr+8, tokens 2j, 2j+1
                pa[mt][2] = pack2<BF>(p[0][2], p[0][3]);        // row gr,   tokens 2j+8, 2j+9
                pa[mt][3] = pack2<BF>(p[1][2], p[1][3]);        // row gr+8, tokens 2j+8, 2j+9
            }

            // ---- O += P V ----
            {
                const int row = 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
                for (int np = 0; np < NT / 2; np++) {
                    const int cc = 2 * np + (lane >> 4);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(stg_u + (cc >> 3) * kBoxBytes + swz(row, cc & 7), b0, b1, b2, b3);
#pragma unroll
                    for (int mt = 0; mt < kMT; mt++) {
                        mma16816<BF>(o[mt][2 * np], pa[mt], b0, b1);
                        mma16816<BF>(o[mt][2 * np + 1], pa[mt], b2, b3);
                    }
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
#pragma unroll
    for (int mt = 0; mt < kMT; mt++)
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            lrow[mt][hf] += __shfl_xor_sync(0xFFFFFFFFu, lrow[mt][hf], 1);
            lrow[mt][hf] += __shfl_xor_sync(0xFFFFFFFFu, lrow[mt][hf], 2);
        }
    // fail closed: a wait that gave up (here or anywhere on this handle) means no output
    const bool poisoned = !alive || __ldcg(status) != 0;

    if (n_chunks == 1) {
        // the tile saw its whole visible context: normalised rows straight to `out`
        if (poisoned) return;
#pragma unroll
        for (int mt = 0; mt < kMT; mt++)
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                if (!vv[mt][hf]) continue;
                const int r = rr[mt][hf];
                const float inv = 1.0f / (lrow[mt][hf] + 1e-8f);
                const size_t base = ((size_t)(st.q_base[b] + tok_first + r / G) * g.H + (size_t)kvh * G + r % G) * D + 2 * j;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const float x = o[mt][nt][2 * hf] * inv, y = o[mt][nt][2 * hf + 1] * inv;
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
    for (int mt = 0; mt < kMT; mt++)
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            if (!vv[mt][hf]) continue;
            const int r = rr[mt][hf];
            float* prow = region + partial_off(chunk, (tok_first + r / G) * g.H + kvh * G + r % G, HP, D);
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
                *reinterpret_cast<float2*>(prow + 8 * nt + 2 * j) = make_float2(o[mt][nt][2 * hf], o[mt][nt][2 * hf + 1]);
            if (j == 0) *reinterpret_cast<float2*>(prow + D) = make_float2(mrow[mt][hf], lrow[mt][hf]);
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
