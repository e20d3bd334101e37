// decode_mma_mla.cu — paged decode attention for the MLA cache shape (K rows of 192 =
// nope 128 + rope 64 dims, V rows of 128 dims) on sm_100a: TMA-staged pages, tensor-core
// QK^T / PV tiles, online softmax, split-KV partials.
//
// Arithmetic contract: that of attention_decode_mla_kernel (reference:
// src/compute/cuda/attention.cu:168-253) — score = (q.k)/sqrtf(k_head_dim) over all 192
// dims, running max from -1e30f, FP32 accumulation, output over the 128 V dims, GQA map
// kv_head = head/(H/Hkv) — evaluated as an online softmax whose (o, m, l) partials are
// merged by the LSE combine.
//
// A pool tile (page, kv head) is [K: 16 tokens x 192][V: 16 tokens x 128] = 10 KB,
// contiguous in HBM.  Three TMA boxes bring it into shared memory, all with the 128-byte
// swizzle:
//   K : one box of 48 lines of 128 bytes through a 4-D view (128-byte third, token, tile):
//       line 3t+h = third h of token t's K row; the 8 tokens of an ldmatrix phase sit on
//       lines whose low 3 bits are all different, so the swizzle spreads them over all banks;
//   V : two boxes of 16 lines through a 4-D view (128-byte half, token, tile), one per
//       half of the V rows, so that the 8 tokens of a transposed ldmatrix phase are 8
//       consecutive lines (a single 32-line box would put tokens t and t+4 on the same
//       banks).
// Schedule and warp roles are those of decode_mma.cu: one CTA per work item, each of the 4
// warps owns every 4th page of the chunk with a private 2-stage ring; two CTAs per SM.
#include "tk_kernels.cuh"
#include "tk_merge.cuh"
#include "tk_mma.cuh"

namespace tk {

namespace {

constexpr int kDk = 192, kDv = 128;
constexpr int kKBytes = kPage * kDk * 2;                    // 6144: K rows of a tile
constexpr int kVHalfBytes = kPage * 128;                    // 2048: one 128-byte half of the V rows
constexpr int kTileBytes = kKBytes + 2 * kVHalfBytes;       // 10240
constexpr int kMlaStages = 2;
constexpr int kMlaSmem = kWarps * kMlaStages * kTileBytes + 1024 + 128;

// byte offset of 16-byte chunk cc (0..23) of token t's K row inside a staged tile
__device__ __forceinline__ uint32_t k_off(int t, int cc) {
    const int line = 3 * t + (cc >> 3);
    return (uint32_t)(line * 128 + (((cc & 7) ^ (line & 7)) << 4));
}
// byte offset of 16-byte chunk cc (0..15) of token t's V row inside a staged tile
__device__ __forceinline__ uint32_t v_off(int t, int cc) {
    return (uint32_t)(kKBytes + (cc >> 3) * kVHalfBytes + t * 128 + (((cc & 7) ^ (t & 7)) << 4));
}

// MULTI: every sequence brings nq query tokens (the tokens the step appended, already in the pool), token j
// attending causally to positions <= len - nq + j; row j*G + gg of the tile is token j, head gg of the
// group, 8/G tokens per pass, further token groups as grid rows (as in decode_mma.cu).
template <bool BF, bool MULTI>
__global__ void __launch_bounds__(kWarps * 32, 2)
decode_mma_mla_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                      Geometry g, LayerPtrs lp, StepDev st, const int32_t* __restrict__ page_table,
                      const uint16_t* __restrict__ q, float* __restrict__ partials, int* __restrict__ status,
                      MergeOut mo, FuseAppend fa) {
    constexpr int KS = kDk / 16;                            // 12 k-steps of QK^T
    constexpr int NT = kDv / 8;                             // 16 n-tiles of PV
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + kWarps * kMlaStages * kTileBytes);
    int* s_flag = (int*)(bars + kWarps * kMlaStages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gr = lane >> 2, j = lane & 3;                 // fragment row / column-pair index
    const int G = g.H / g.Hkv;                              // <= 8: rows 8..15 of the M tile are padding

    pdl_launch_dependents();                                // a launch of another layer may fill the slots this one leaves (see decode_mma.cu)
    const int4 it = st.items[blockIdx.x];
    const int b = it.x, chunk = it.y, kvh = it.z;
    const int seq = st.seq[b], len = st.len[b];
    const int nq = MULTI ? st.nq[b] : 1;                    // query tokens of this sequence
    const int tok0 = MULTI ? (int)blockIdx.y * (8 / G) : 0; // first query token of this CTA's token group
    const int nq_g = MULTI ? min(nq - tok0, 8 / G) : 1;
    if (MULTI && nq_g <= 0) return;                         // this sequence has no such group
    const int rows = G * nq_g;                              // rows of the M tile that carry data (<= 8)
    const int q_row0 = MULTI ? st.q_base[b] + tok0 : b;     // row of q / out of the group's first query token
    const int t0 = chunk * st.chunk_tokens;
    // the group's last token sees len - nq + tok0 + nq_g positions: nothing beyond is fetched
    const int t1 = min(MULTI ? len - nq + tok0 + nq_g : len, t0 + st.chunk_tokens);
    const int n_pages = t1 > t0 ? (t1 - t0 + kPage - 1) / kPage : 0;
    const int lp0 = t0 / kPage;
    const int n_w = n_pages > warp ? (n_pages - warp + kWarps - 1) / kWarps : 0;   // pages of this warp (<= 32)
    const int new_tok = fa.k != nullptr ? st.new_tok[b] : -1;                       // fused append (decode steps)

    if (threadIdx.x == 0) {
        for (int i = 0; i < kWarps * kMlaStages; i++) mbar_init(smem_u32(&bars[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    int my_page = 0;                                        // lane i: physical page of this warp's i-th page
    if (lane < n_w) my_page = page_table[(size_t)seq * g.max_pages_per_seq + lp0 + warp + kWarps * lane];

    uint8_t* wstage = smem + (size_t)warp * kMlaStages * kTileBytes;
    auto issue = [&](int i) {
        const int page = __shfl_sync(0xFFFFFFFFu, my_page, i);
        if (lane == 0) {
            const int s = i % kMlaStages;
            const uint32_t bar = smem_u32(&bars[warp * kMlaStages + s]);
            const uint32_t dst = smem_u32(wstage + (size_t)s * kTileBytes);
            const int tile = page * g.Hkv + kvh;
            mbar_expect_tx(bar, kTileBytes);
            tma_load_4d(dst, &tmap_k, 0, 0, 0, tile, bar);
            tma_load_4d(dst + kKBytes, &tmap_v, 0, 0, 0, tile, bar);
            tma_load_4d(dst + kKBytes + kVHalfBytes, &tmap_v, 0, 1, 0, tile, bar);
        }
    };
    for (int i = 0; i < kMlaStages && i < n_w; i++) issue(i);

    // ---- Q fragments (A operand): row gr of the group, rows >= G and 8..15 are zero ----
    uint32_t qa[KS][2];
    {
        const uint16_t* qrow = q + ((size_t)(q_row0 + (MULTI ? gr / G : 0)) * g.H + (size_t)kvh * G + (MULTI ? gr % G : gr)) * kDk;
        const bool valid = gr < rows;
        // fused RoPE: the query is the token at position len-1; only dims kDv.. (the rope dims) rotate
        const float2* tab = fa.rope_tab ? fa.rope_tab + (size_t)b * ((kDk - kDv) / 2) : nullptr;
#pragma unroll
        for (int kk = 0; kk < KS; kk++) {
            qa[kk][0] = valid ? *reinterpret_cast<const uint32_t*>(qrow + 16 * kk + 2 * j) : 0u;
            qa[kk][1] = valid ? *reinterpret_cast<const uint32_t*>(qrow + 16 * kk + 8 + 2 * j) : 0u;
            if (16 * kk >= kDv && tab) {
                qa[kk][0] = rope_pair<BF>(qa[kk][0], tab, 16 * kk - kDv + 2 * j);
                qa[kk][1] = rope_pair<BF>(qa[kk][1], tab, 16 * kk - kDv + 8 + 2 * j);
            }
        }
    }

    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f; }
    float m0 = -1e30f, l0 = 0.0f;
    const float sm_scale = 1.0f / sqrtf((float)kDk);

    for (int i = 0; i < n_w; i++) {
        const int s = i % kMlaStages;
        const uint32_t bar = smem_u32(&bars[warp * kMlaStages + s]);
        // warp-uniform verdict, so that a give-up never splits the warp before a shuffle
        if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded(bar, (uint32_t)((i / kMlaStages) & 1), status))) break;
        uint8_t* stg = wstage + (size_t)s * kTileBytes;
        const uint32_t stg_u = smem_u32(stg);
        const int tok_base = (lp0 + warp + kWarps * i) * kPage;
        const int n_valid = min(kPage, t1 - tok_base);     // < 16 only on a sequence's last page
        // tokens of this page that row gr may attend to (causal limit of its query token)
        const int nv0 = MULTI ? max(0, min(n_valid, len - nq + tok0 + gr / G + 1 - tok_base)) : n_valid;

        if (new_tok >= 0 && tok_base == ((len - 1) & ~(kPage - 1))) {
            // This page holds the token appended by this step.  The TMA tile has the stale row:
            // put the new K/V row into shared memory for the MMAs and into the pool for later steps.
            const int r = (len - 1) & (kPage - 1);
            const int page = __shfl_sync(0xFFFFFFFFu, my_page, i);
            if (lane < kDk / 8) {
                uint4 val = *reinterpret_cast<const uint4*>((const uint16_t*)fa.k + ((size_t)new_tok * g.Hkv + kvh) * kDk + lane * 8);
                if (fa.rope_tab && lane >= kDv / 8) {           // rope dims of the K row: rotate its 4 pairs before it is stored
                    const float2* tab = fa.rope_tab + (size_t)b * ((kDk - kDv) / 2);
                    const int d = lane * 8 - kDv;
                    val.x = rope_pair<BF>(val.x, tab, d + 0);
                    val.y = rope_pair<BF>(val.y, tab, d + 2);
                    val.z = rope_pair<BF>(val.z, tab, d + 4);
                    val.w = rope_pair<BF>(val.w, tab, d + 6);
                }
                *reinterpret_cast<uint4*>(stg + k_off(r, lane)) = val;
                *reinterpret_cast<uint4*>((uint16_t*)lp.pool + tile_offset(g, page, kvh, 0) + (size_t)r * kDk + lane * 8) = val;
            }
            if (lane < kDv / 8) {
                const uint4 val = *reinterpret_cast<const uint4*>((const uint16_t*)fa.v + ((size_t)new_tok * g.Hkv + kvh) * kDv + lane * 8);
                *reinterpret_cast<uint4*>(stg + v_off(r, lane)) = val;
                *reinterpret_cast<uint4*>((uint16_t*)lp.pool + tile_offset(g, page, kvh, 1) + (size_t)r * kDv + lane * 8) = val;
            }
            __syncwarp();
        }
        if (n_valid < kPage) {
            // stale rows of a partly filled page: zero the V rows so 0 * garbage cannot make NaN
            for (int idx = lane; idx < (kPage - n_valid) * 16; idx += 32) {
                const int t = n_valid + idx / 16, cc = idx % 16;
                *reinterpret_cast<uint4*>(stg + v_off(t, cc)) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }

        // ---- S = Q K^T over the page's 16 tokens ----
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const int t = ((lane >> 4) << 3) + (lane & 7);
#pragma unroll
            for (int kk = 0; kk < KS; kk++) {
                uint32_t r0, r1, r2, r3;
                ldsm_x4(stg_u + k_off(t, 2 * kk + ((lane >> 3) & 1)), r0, r1, r2, r3);
                const uint32_t a[4] = {qa[kk][0], 0u, qa[kk][1], 0u};
                mma16816<BF>(s0, a, r0, r1);
                mma16816<BF>(s1, a, r2, r3);
            }
        }

        // ---- online softmax of row gr (token columns 2j, 2j+1, 2j+8, 2j+9) ----
        float p[4];
        {
            const int c0 = 2 * j;
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
            p[0] = ex2(fmaf(a0, kLog2e, nb)); p[1] = ex2(fmaf(a1, kLog2e, nb));
            p[2] = ex2(fmaf(a2, kLog2e, nb)); p[3] = ex2(fmaf(a3, kLog2e, nb));
            if (MULTI) {                                    // a row may see nothing of a page: exp(-1e30 + 1e30) is 1, not 0
                if (c0 >= nv0) p[0] = 0.0f;
                if (c0 + 1 >= nv0) p[1] = 0.0f;
                if (c0 + 8 >= nv0) p[2] = 0.0f;
                if (c0 + 9 >= nv0) p[3] = 0.0f;
            }
            l0 = l0 * alpha + (p[0] + p[1] + p[2] + p[3]);
            // the running maximum rarely moves after the first pages: skip the multiplies then
            if (!__all_sync(0xFFFFFFFFu, mn == m0)) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++) { o[nt][0] *= alpha; o[nt][1] *= alpha; }
            }
            m0 = mn;
        }

        // ---- O += P V ----
        {
            const uint32_t pa[4] = {pack2<BF>(p[0], p[1]), 0u, pack2<BF>(p[2], p[3]), 0u};
            const int t = (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {
                uint32_t r0, r1, r2, r3;
                ldsm_x4_t(stg_u + v_off(t, 2 * np + (lane >> 4)), r0, r1, r2, r3);
                mma16816<BF>(o[2 * np], pa, r0, r1);
                mma16816<BF>(o[2 * np + 1], pa, r2, r3);
            }
        }

        // ---- refill this stage ----
        __syncwarp();
        if (i + kMlaStages < n_w) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(i + kMlaStages);
        }
    }

    // ---- merge the 4 warps through shared memory (stage memory is idle now) ----------
    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 1); l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 2);
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem);            // [kWarps][G][kDv+2]
    auto red_at = [&](int w, int row, int d) -> float& { return red[((size_t)w * rows + row) * (kDv + 2) + d]; };
    if (gr < rows) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            red_at(warp, gr, 8 * nt + 2 * j + 0) = o[nt][0];
            red_at(warp, gr, 8 * nt + 2 * j + 1) = o[nt][1];
        }
        if (j == 0) { red_at(warp, gr, kDv) = m0; red_at(warp, gr, kDv + 1) = l0; }
    }
    __syncthreads();
    pdl_wait();                                             // split-KV rows, counters and `out` are shared with the launch before
    const int prow = st.chunk_base[b] + chunk;
    const int heads_per_row = MULTI ? g.H * st.nq_max : g.H;   // columns of a partial row
    for (int idx = threadIdx.x; idx < rows * (kDv + 2); idx += blockDim.x) {
        const int row = idx / (kDv + 2), d = idx % (kDv + 2);
        float M = -1e30f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, red_at(w, row, kDv));
        float val;
        if (d == kDv) {
            val = M;
        } else {
            val = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) val += red_at(w, row, d) * ex2((red_at(w, row, kDv) - M) * kLog2e);
        }
        const int col = MULTI ? (tok0 + row / G) * g.H + kvh * G + row % G : kvh * G + row;
        partials[partial_off(prow, col, heads_per_row, kDv) + d] = val;
    }
    merge_if_last(g, st, mo, b, kvh, G, partials, s_flag,
                  MergeMap{rows, heads_per_row, q_row0, MULTI ? tok0 : 0, MULTI ? (int)blockIdx.y * st.n_seqs * g.Hkv : 0});
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
        if (qres != cudaDriverEntryPointSuccess || !fn) return nullptr;
        encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    }
    return encode;
}

}  // namespace

bool decode_mma_mla_supported(const Geometry& g) {
    return g.ps == kPage && g.D == kDk && g.Dv == kDv && g.Hkv > 0 && g.H % g.Hkv == 0 && g.H / g.Hkv <= 8 &&
           (g.dtype == DT_FP16 || g.dtype == DT_BF16) && g.io_dtype == g.dtype;
}

// Two 4-D views of the layer's pool (tiles of 10240 bytes), innermost dimension 64 elements = 128 bytes:
//   k_map: (64 elements, 3 thirds of a K row, 16 tokens, tiles); box = all 48 lines of a tile's K rows
//   v_map: base 6144 bytes into the pool: (64 elements, 2 halves of a V row, 16 tokens, tiles);
//          box = one half of all 16 rows
cudaError_t make_mla_tensor_maps(const Geometry& g, void* layer_pool, CUtensorMap* k_map, CUtensorMap* v_map) {
    auto encode = encode_fn();
    if (!encode) return cudaErrorNotSupported;
    const cuuint64_t n_tiles = (cuuint64_t)g.num_pages * g.Hkv;
    cuuint32_t estr[4] = {1, 1, 1, 1};
    {
        cuuint64_t dims[4] = {64, 3, (cuuint64_t)kPage, n_tiles};
        cuuint64_t strides[3] = {128, 384, (cuuint64_t)kTileBytes};
        cuuint32_t box[4] = {64, 3, (cuuint32_t)kPage, 1};
        CUresult r = encode(k_map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, layer_pool, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    {
        cuuint64_t dims[4] = {64, 2, (cuuint64_t)kPage, n_tiles};
        cuuint64_t strides[3] = {128, 256, (cuuint64_t)kTileBytes};
        cuuint32_t box[4] = {64, 1, (cuuint32_t)kPage, 1};
        CUresult r = encode(v_map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, (uint8_t*)layer_pool + kKBytes, dims, strides,
                            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    return cudaSuccess;
}

template <bool BF, bool MULTI>
static cudaError_t launch_mla_cfg(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* k_map, const CUtensorMap* v_map,
                                  const StepDev& st, const int32_t* page_table, const void* q, float* partials, int* status,
                                  cudaStream_t s, const MergeOut& mo, const FuseAppend& fa, bool overlap_prev = false) {
    static bool attr_done[64] = {};                         // per instantiation and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(decode_mma_mla_kernel<BF, MULTI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    const int tpg = 8 / (g.H / g.Hkv);                      // multi-token attention: tokens per pass
    const dim3 grid(st.n_items, MULTI ? (st.nq_max + tpg - 1) / tpg : 1);
    if (!overlap_prev) {
        decode_mma_mla_kernel<BF, MULTI><<<grid, kWarps * 32, kMlaSmem, s>>>(*k_map, *v_map, g, lp, st, page_table,
                                                                             (const uint16_t*)q, partials, status, mo, fa);
        return cudaGetLastError();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(kWarps * 32); cfg.dynamicSmemBytes = kMlaSmem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_mma_mla_kernel<BF, MULTI>, *k_map, *v_map, g, lp, st, page_table,
                              (const uint16_t*)q, partials, status, mo, fa);
}

bool decode_mma_mla_multi_supported(const Geometry& g, int nq_max) {
    return decode_mma_mla_supported(g) && nq_max >= 1 && (g.H / g.Hkv) * nq_max <= 8 * 8;   // up to 8 token groups
}

// Multi-token attention for the MLA shape (st.nq / st.q_base / st.nq_max set): q [n_tokens][H][192],
// out [n_tokens][H][128]; `mo.counters` needs n_groups * n_seqs * Hkv zeroed counters.
cudaError_t launch_decode_mma_mla_multi(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* k_map,
                                        const CUtensorMap* v_map, const StepDev& st, const int32_t* page_table,
                                        const void* q, float* partials, int* status, cudaStream_t s, const MergeOut& mo) {
    if (st.n_items <= 0) return cudaSuccess;
    if (!decode_mma_mla_multi_supported(g, st.nq_max) || st.chunk_tokens > kPage * kWarps * 32 || !mo.counters || mo.peer)
        return cudaErrorNotSupported;
    const FuseAppend fa{nullptr, nullptr, nullptr};
    return g.dtype == DT_BF16 ? launch_mla_cfg<true, true>(g, lp, k_map, v_map, st, page_table, q, partials, status, s, mo, fa)
                              : launch_mla_cfg<false, true>(g, lp, k_map, v_map, st, page_table, q, partials, status, s, mo, fa);
}

cudaError_t launch_decode_mma_mla(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* k_map,
                                  const CUtensorMap* v_map, const StepDev& st, const int32_t* page_table,
                                  const void* q, float* partials, int* status, cudaStream_t s,
                                  const MergeOut* merge, const FuseAppend* fuse, bool overlap_prev) {
    if (st.n_items <= 0) return cudaSuccess;
    if (!decode_mma_mla_supported(g) || st.chunk_tokens > kPage * kWarps * 32) return cudaErrorNotSupported;
    const MergeOut mo = merge ? *merge : MergeOut{nullptr, nullptr, nullptr, 0};
    const FuseAppend fa = fuse ? *fuse : FuseAppend{nullptr, nullptr, nullptr};
    return g.dtype == DT_BF16 ? launch_mla_cfg<true, false>(g, lp, k_map, v_map, st, page_table, q, partials, status, s, mo, fa, overlap_prev)
                              : launch_mla_cfg<false, false>(g, lp, k_map, v_map, st, page_table, q, partials, status, s, mo, fa, overlap_prev);
}

}  // namespace tk
