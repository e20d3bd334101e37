// prefill_tc.cu — attention for every token of a prefill chunk on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory), head_dim 128, 16-bit pools.
//
// Same work and arithmetic contract as prefill_mma.cu (the reference runs its layer once per prompt token:
// src/inference/engine.cpp:182-193; per token: attention_decode_kernel, src/compute/cuda/attention.cu:58-157),
// same work list; what changes is the engine.  With T * G >= 128 (token, head) rows per kv head the tile
// is a contraction the tcgen05 instruction takes whole: M = 128 rows = the 128 lanes of tensor memory.
//
// One CTA = one tile of 128 rows x a range of the context: 4 softmax warps, thread t owns row t (TMEM lane t:
// no shuffles in the softmax), an MMA warp whose one elected thread issues every tcgen05.mma, and a loader warp
// whose lanes issue the TMA copies; the roles meet on mbarriers only (no CTA-wide barrier inside the loop).
// (Measured with clock64 around each phase: with one thread issuing both the 16 copies and the 12 MMAs of a
// block, that thread was busy 80 % of the kernel and the softmax warps waited for it 60 % of theirs.)
// Per block of 64 context tokens (4 pages):
//   TMA      K rows and V rows of the 4 pages land as [64 tokens][128 B] slabs per 64-dim half (128-byte
//            swizzle): separate boxes of 16 rows, so that the K rows of consecutive pages are consecutive;
//            eight boxes leave in one instruction of the loader warp, two stages for K and two for V
//   S = Q K^T  one thread issues 8 tcgen05.mma (M 128, N 64, K 16) with Q and K from shared memory (K-major
//            descriptors), S in one of two TMEM buffers (columns [0, 64) and [64, 128)); tcgen05.commit -> mbarrier.
//            S of block i+2 is issued right behind P V of block i, S of block i+1 is already there: the tensor
//            pipe works while the threads do the softmax of block i
//   softmax  every thread tcgen05.ld's its row of S (the second half while it works on the first).  Blocks that no
//            row of the warp sees cut (causal limit of its token, end of the sequence) take ONE pass: maximum,
//            exp2 against the current reference maximum, sum, P rounded to the 16-bit type - speculating that the
//            reference stays, which it does unless a score exceeds it by 2^8; only then (and on cut blocks) the
//            careful pass recomputes against the new reference and the warp rescales its rows of O in TMEM (ld,
//            multiply, st), for which alone it waits for the previous P V.  P goes over the first 32 columns of
//            the S buffer it came from (tcgen05.st); an mbarrier with one arrival per row tells the MMA thread
//   O += P V   4 tcgen05.mma (M 128, N 128, K 16) with P from TMEM and V from shared memory (MN-major
//            descriptor: V rows are tokens), O in TMEM columns [128, 256)
// Two CTAs share an SM (256 TMEM columns and 108 KB of shared memory each), so one CTA's softmax overlaps the
// other's MMAs.  No cluster, no multicast, cta_group::1 only, this GPU's memory only.
// Measured and left out: computing a share of the exponentials as a cubic on the FMA pipe (0 / 12.5 / 25 / 50 % of
// them: 916 / 887 / 856 / 793 TFLOP/s) - the softmax warps are short of issue slots and latency cover, not of
// special-function throughput.  Nor did more softmax warps help: two threads per row (8 softmax warps per CTA, 32
// columns each, the halves' maxima exchanged through shared memory on a named barrier per warp pair) ran at 771
// against 930 TFLOP/s; nor the pass written out in batches of 16 exponentials with four chains each (895).
// Nor blocks of 128 tokens with ONE S buffer of 128 columns (8 + 8 MMAs per block, half the barrier traffic and
// TMA instructions per token, but S of the next block cannot start before P V of this one): 857 against 935.
// Every mbarrier wait is bounded; on expiry the status word is set, nothing is written, and the CTA still
// frees its tensor memory before it returns.
#include "tk_kernels.cuh"
#include "tk_merge.cuh"
#include "tk_mma.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cudaTypedefs.h>

namespace tk {

namespace {

constexpr int kTcRows = 128;                    // rows per tile = TMEM lanes
constexpr int kTcBlock = 64;                    // context tokens per block (4 pages)
constexpr int kTcD = 128;
constexpr int kTcStages = 2;
constexpr int kTcThreads = kTcRows + 64;        // 4 softmax warps (a row per thread), the MMA warp, the loader warp
constexpr int kQBytes = 2 * kTcRows * 128;      // two 64-dim halves of [128 rows][128 B]
constexpr int kSlabBytes = 2 * kTcBlock * 128;  // K (or V) of one block: two halves of [64 tokens][128 B]
constexpr int kHalfBytes = kTcBlock * 128;      // one 64-dim half of a slab
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128;       // S buffers at columns 0 and 64 (P over their first 32), O at 128
constexpr int kTcSmem = kQBytes + 2 * kTcStages * kSlabBytes + 256 + kPrefillMaxPages * 4 + 1024;

// ---- tcgen05 / TMEM primitives -------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: register i of thread t = column i of lane (warp's base lane + t)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
// The same wait with the 32 registers of a load as in/out operands: nothing that reads them can be scheduled above it.
__device__ __forceinline__ void tc_wait_ld(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                   "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                   "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :: "memory");
}
// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// Two FP32 lanes per instruction (sm_100): (a0, a1) * b + c and (s0, s1) += (p0, p1)
__device__ __forceinline__ void fma2(float& r0, float& r1, float a0, float a1, float b, float c) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}" : "=f"(r0), "=f"(r1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float& s0, float& s1, float p0, float p1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%0, %1};\n\tmov.b64 rb, {%2, %3};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}" : "+f"(s0), "+f"(s1) : "f"(p0), "f"(p1));
}

// Shared-memory matrix descriptor, 128-byte swizzle, 8-row groups 1024 bytes apart (sm_100 format:
// address, leading and stride byte offsets in 16-byte units, descriptor version 1, layout type 2).
//   K-major operand (Q, K: rows of 128 B hold 64 consecutive dims): lbo is not used by the swizzled form
//   MN-major operand (V: rows are tokens, the MMA's N runs along the row): lbo = bytes between the two
//   64-dim halves of the slab
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((1024u >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;                                 // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                                 // SWIZZLE_128B
    return d;
}
// Instruction descriptor of kind::f16: F32 accumulate, A/B format (0 f16, 1 bf16), B major, N, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(bool bf16, bool b_mn_major, int n) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
}

template <bool BF>
__global__ void __launch_bounds__(kTcThreads, 2)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap, Geometry g, StepDev st, PrefillDev pf,
                  const int32_t* __restrict__ page_table, const uint16_t* __restrict__ q, void* __restrict__ out,
                  int out_dtype, float* __restrict__ partials, int* __restrict__ counters, int* __restrict__ status) {
    constexpr int D = kTcD;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* s_q = smem;                                     // [2 halves][128 rows][128 B]
    uint8_t* s_k = s_q + kQBytes;                            // [stages][2 halves][64 tokens][128 B]
    uint8_t* s_v = s_k + kTcStages * kSlabBytes;
    uint64_t* bars = (uint64_t*)(s_v + kTcStages * kSlabBytes);
    uint64_t* kfull = bars;                                  // [stages]
    uint64_t* vfull = bars + kTcStages;                      // [stages]
    uint64_t* bar_s = bars + 2 * kTcStages;                  // [2] S of a block is in TMEM (one barrier per S buffer)
    uint64_t* bar_o = bar_s + 2;                             // O += P V of a block is done
    uint64_t* p_ready = bar_o + 1;                           // [2] all 128 rows of P of a block are in TMEM (one per S buffer); + the loader
    uint32_t* s_tmem = (uint32_t*)(p_ready + 2);             // TMEM base address from the allocator
    int* s_flag = (int*)(s_tmem + 1);
    int32_t* s_pages = (int32_t*)((uint8_t*)bars + 256);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = g.H / g.Hkv;
    // item and the facts about its sequence in three independent loads (not item -> sequence index -> facts)
    const int4 it = pf.items[blockIdx.x], i0 = pf.info[2 * blockIdx.x], i1 = pf.info[2 * blockIdx.x + 1];
    const int b = it.x, chunk = it.y, kvh = it.z, tile = it.w;
    const int seq = i0.x, len = i0.y, nq = i0.z, ct = i0.w;
    const int q_base = i1.x, poff = i1.y, cbase = i1.z;
    const int tpt = kTcRows / G;                            // query tokens per tile
    const int tok_first = tile * tpt;
    const int tok_cnt = min(nq - tok_first, tpt);
    const int base_pos = len - nq;
    const int p_last = base_pos + tok_first + tok_cnt - 1;
    const int t0 = chunk * ct;
    const int t1 = min(t0 + ct, p_last + 1);
    const int n_pages = (t1 - t0 + kPage - 1) / kPage;
    const int n_blocks = (n_pages + 3) / 4;
    const int lp0 = t0 / kPage;
    const int n_chunks = p_last / ct + 1;

    // this thread's row: query token tid / G of the tile, head tid % G of the group
    const bool valid = tid < kTcRows && tid / G < tok_cnt;
    const int lim = base_pos + tok_first + tid / G + 1;     // positions the row attends to: [0, lim)
    const size_t qo_row = (size_t)(q_base + tok_first + tid / G) * g.H + (size_t)kvh * G + tid % G;

    // Q tile of the CTA: 128 rows of 256 B.  The loads go out first, so that their latency runs beside the rest of the
    // prologue (barriers, tensor-memory allocation, page ids, the first K/V copies), and each warp instruction reads
    // two whole rows: vector i of thread t is 16-byte chunk (i * 128 + t) % 16 of row (i * 128 + t) / 16.
    uint4 qv[16];
    if (tid < kTcRows) {
        const int sh = __ffs(G) - 1;                        // G divides 128: a power of two
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int r = (i * kTcRows + tid) >> 4, c = tid & 15;
            const bool ok = (r >> sh) < tok_cnt;
            const size_t row = (size_t)(q_base + tok_first + (r >> sh)) * g.H + (size_t)kvh * G + (r & (G - 1));
            qv[i] = ok ? __ldg(reinterpret_cast<const uint4*>(q + row * D) + c) : make_uint4(0, 0, 0, 0);
        }
    }
    if (tid == 0) {
        for (int i = 2 * kTcStages; i < 2 * kTcStages + 3; i++) mbar_init(smem_u32(&bars[i]), 1);
        mbar_init(smem_u32(&p_ready[0]), kTcRows + 1);
        mbar_init(smem_u32(&p_ready[1]), kTcRows + 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTcRows / 32) {                             // the MMA warp allocates the CTA's tensor memory
        tmem_alloc(smem_u32(s_tmem), kTmemCols);
        tmem_relinquish();
    }
    const int32_t* pt_row = page_table + (size_t)seq * g.max_pages_per_seq + lp0;
    for (int i = tid; i < n_pages; i += blockDim.x) s_pages[i] = pt_row[i];
    // The loader warp does not wait for the rest of the prologue: it sets up the K/V barriers itself and sends the
    // copies of the first two blocks off with page ids read straight from the table.
    auto load_rows = [&](int blk, bool is_v, const int32_t* pages_of) {
        const int s = blk % kTcStages;
        const int pages = min(4, n_pages - 4 * blk);
        const uint32_t bar = smem_u32(is_v ? &vfull[s] : &kfull[s]);
        if (lane == 0) mbar_expect_tx(bar, pages * 2 * 2048);
        __syncwarp();
        const int p = lane >> 1, h = lane & 1;
        if (lane < 8 && p < pages) {
            const int row = (pages_of[4 * blk + p] * g.Hkv + kvh) * 32 + (is_v ? 16 : 0);
            tma_load_2d_shared_tile(smem_u32((is_v ? s_v : s_k) + s * kSlabBytes + h * kHalfBytes + p * 2048), &tmap, h * 64, row, bar);
        }
    };
    if (warp == kTcRows / 32 + 1) {
        if (lane == 0) {
            for (int i = 0; i < 2 * kTcStages; i++) mbar_init(smem_u32(&bars[i]), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        load_rows(0, false, pt_row); load_rows(0, true, pt_row);
        if (n_blocks > 1) { load_rows(1, false, pt_row); load_rows(1, true, pt_row); }
    }
    // Q rows -> shared memory in the 128-byte-swizzled K-major form the MMA reads (16-byte chunk c of a row
    // sits at chunk c ^ (row & 7)); rows without a token are zero
    if (tid < kTcRows) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int r = (i * kTcRows + tid) >> 4, c = tid & 15;
            *reinterpret_cast<uint4*>(s_q + (c >> 3) * (kTcRows * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = qv[i];
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic writes above -> visible to TMA / MMA
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;  // this warp's 32 TMEM lanes

    constexpr uint32_t kIdescS = instr_desc(BF, false, kTcBlock);
    constexpr uint32_t kIdescO = instr_desc(BF, true, D);
    // MMA thread: the descriptors of a stage differ from those of stage 0 by the stage's byte offset / 16 in the
    // address field (the field cannot carry: shared memory addresses stay below 2^18)
    const uint64_t desc_q = smem_desc(smem_u32(s_q), 16), desc_k = smem_desc(smem_u32(s_k), 16),
                   desc_v = smem_desc(smem_u32(s_v), kHalfBytes);
    // S = Q K^T of block `blk` (8 k-steps of 16 dims: 4 per 64-dim half, 32 bytes apart inside the swizzled row)
    auto issue_s = [&](int blk) {
        const uint64_t dk = desc_k + (uint64_t)((blk % kTcStages) * (kSlabBytes >> 4));
        const uint32_t d_s = tmem + kColS + 64u * (blk & 1);
#pragma unroll
        for (int ks = 0; ks < 8; ks++)
            tc_mma_ss(d_s, desc_q + (uint64_t)(((ks >> 2) * (kTcRows * 128) + (ks & 3) * 32) >> 4),
                      dk + (uint64_t)(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4), kIdescS, ks > 0);
        tc_commit(smem_u32(&bar_s[blk & 1]));
    };

    // Softmax state of this thread's row, in base-2 units: scores are s * (log2e / sqrt(D)), m2 is the reference
    // maximum the probabilities are taken against.  The reference moves only when a block's maximum exceeds it by
    // more than kLazy (then O is rescaled); until then probabilities may reach 2^kLazy, which the 16-bit P and
    // the FP32 sums hold easily, and O / l is unchanged by the choice of reference.
    constexpr float kLazy = 8.0f;
    float m2 = -1e30f, l_run = 0.0f;
    const float sc2 = kLog2e / sqrtf((float)D);
    bool alive = true;

    if (warp == kTcRows / 32) {
        // ===== MMA warp: one thread feeds the tensor pipe; nobody else waits for its instruction stream =====
        if (lane == 0) {
            bool ok = mbar_wait_bounded_idle(smem_u32(&kfull[0]), 0u, status);
            if (ok) issue_s(0);
            if (ok && n_blocks > 1 && (ok = mbar_wait_bounded_idle(smem_u32(&kfull[1]), 0u, status))) issue_s(1);
            for (int blk = 0; blk < n_blocks && ok; blk++) {
                const int s = blk % kTcStages, buf = blk & 1;
                // every row's P of this block is in TMEM (and O rescaled): O += P V, then S of the block after next
                ok = mbar_wait_bounded_idle(smem_u32(&p_ready[buf]), (uint32_t)((blk >> 1) & 1), status) &&
                     mbar_wait_bounded_idle(smem_u32(&vfull[s]), (uint32_t)((blk / kTcStages) & 1), status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_p = tmem + kColS + 64u * buf;
                const uint64_t dv = desc_v + (uint64_t)(s * (kSlabBytes >> 4));
#pragma unroll
                for (int ks = 0; ks < 4; ks++)               // 16 tokens per MMA: 8 TMEM columns of P, 16 rows of the V slab
                    tc_mma_ts(tmem + kColO, a_p + 8 * ks, dv + (uint64_t)((ks * 2048) >> 4), kIdescO, (blk > 0 || ks > 0) ? 1u : 0u);
                tc_commit(smem_u32(bar_o));
                // the tensor pipe runs its MMAs in issue order: S(blk+2) overwrites these columns after P V has read them
                if (blk + 2 < n_blocks) {
                    ok = mbar_wait_bounded_idle(smem_u32(&kfull[s]), (uint32_t)(((blk + 2) / kTcStages) & 1), status);
                    if (ok) issue_s(blk + 2);
                }
            }
        }
        __syncwarp();
    } else if (warp == kTcRows / 32 + 1) {
        // ===== loader warp: keeps the two K stages and the two V stages full =====
        // (the copies of blocks 0 and 1 left in the prologue)
        for (int blk = 0; blk < n_blocks; blk++) {
            // S(blk) is done with its K stage: K of the block after next goes there
            if (blk + 2 < n_blocks) {
                if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded_idle(smem_u32(&bar_s[blk & 1]), (uint32_t)((blk >> 1) & 1), status))) break;
                load_rows(blk + 2, false, s_pages);
            }
            // P V (blk-1) is done with its V stage: V of the next block goes there
            if (blk > 0 && blk + 1 < n_blocks) {
                if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded_idle(smem_u32(bar_o), (uint32_t)((blk - 1) & 1), status))) break;
                load_rows(blk + 1, true, s_pages);
            }
            // P V (blk) may not complete before this warp has seen P V (blk-1) complete (a parity wait cannot tell
            // a phase that is two ahead from one that has not happened): the MMA thread waits for this arrival too
            if (lane == 0) mbar_arrive(smem_u32(&p_ready[blk & 1]));
        }
    } else {
        // ===== softmax warps: thread t owns row t =====
        for (int blk = 0; blk < n_blocks; blk++) {
            const int s = blk % kTcStages, buf = blk & 1;
            const uint32_t col_s = kColS + 64u * buf;        // S of this block; its first 32 columns become P
            const int tok_base = t0 + blk * kTcBlock;
            // ---- S of this block (issued one block ahead: the tensor pipe worked on it during the last softmax) ----
            if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded(smem_u32(&bar_s[buf]), (uint32_t)((blk >> 1) & 1), status))) { alive = false; break; }
            tc_fence_after();
            uint32_t sr[2][32];                              // the second half of the row arrives while the first is worked on
            tmem_ld32(tmem + lane_base + col_s, sr[0]);
            tc_wait_ld(sr[0]);
            tmem_ld32(tmem + lane_base + col_s + 32, sr[1]);

            // ---- online softmax of the row ----
            const int nv = valid ? max(0, min(min(kTcBlock, t1 - tok_base), lim - tok_base)) : 0;
            // no row of the warp is cut by the diagonal or the end, and every row has a reference already (on its first
            // block a row has none: speculating against -1e30 would be a pass thrown away)
            const bool full = __all_sync(0xFFFFFFFFu, nv == kTcBlock && m2 > -1e29f);
            float alpha = 1.0f;
            bool moved = false;
            uint32_t pr[32];                                 // P of the row: 64 values, two 16-bit per register
            bool settled = false;
            // Speculate that the reference maximum stays: maximum, probabilities and sum in ONE pass, so that the
            // maximum's compare chain and the sum's add chain issue in the shadow of the exponentials (the
            // special-function unit, 4 lanes per clock and scheduler, is the scarce pipe of this loop).
            float smx = -1e30f, ssum0 = 0.0f, ssum1 = 0.0f;
            if (full) {
                const float nb = -m2;
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    const float a0 = __uint_as_float(sr[0][2 * c]), a1 = __uint_as_float(sr[0][2 * c + 1]);
                    smx = fmaxf(smx, fmaxf(a0, a1));
                    float x0, x1;
                    fma2(x0, x1, a0, a1, sc2, nb);
                    const float p0 = ex2(x0), p1 = ex2(x1);
                    add2(ssum0, ssum1, p0, p1);
                    pr[c] = pack2<BF>(p0, p1);
                }
                tmem_st16(tmem + lane_base + col_s, pr);     // these columns of S are in registers already
            }
            tc_wait_ld(sr[1]);
            if (full) {
                const float nb = -m2;
#pragma unroll
                for (int c = 16; c < 32; c++) {
                    const float a0 = __uint_as_float(sr[1][2 * c - 32]), a1 = __uint_as_float(sr[1][2 * c - 31]);
                    smx = fmaxf(smx, fmaxf(a0, a1));
                    float x0, x1;
                    fma2(x0, x1, a0, a1, sc2, nb);
                    const float p0 = ex2(x0), p1 = ex2(x1);
                    add2(ssum0, ssum1, p0, p1);
                    pr[c] = pack2<BF>(p0, p1);
                }
                moved = smx * sc2 > m2 + kLazy;              // always on a row's first block (m2 = -1e30)
                if (!__any_sync(0xFFFFFFFFu, moved)) {
                    l_run += ssum0 + ssum1;
                    tmem_st16(tmem + lane_base + col_s + 16, pr + 16);
                    settled = true;
                }
            }
            if (!settled) {
                // the careful pass: masks, the new reference of every row that moved, and its probabilities again
                float mx = -1e30f;
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int c = 0; c < 32; c++) {
                        if (32 * h + c >= nv) sr[h][c] = __float_as_uint(-1e30f / sc2);  // masked: far below any score
                        mx = fmaxf(mx, __uint_as_float(sr[h][c]));
                    }
                mx *= sc2;                                   // sc2 > 0: the maximum of the scaled scores
                moved = mx > m2 + kLazy;
                const float m_new = moved ? mx : m2;
                alpha = moved ? ex2(m2 - m_new) : 1.0f;      // first block: ex2(-1e30 - mx) = 0
                const float nb = -m_new;
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
                for (int c = 0; c < 32; c++) {
                    float p0 = ex2(fmaf(__uint_as_float(sr[c >> 4][(2 * c) & 31]), sc2, nb));
                    float p1 = ex2(fmaf(__uint_as_float(sr[c >> 4][(2 * c + 1) & 31]), sc2, nb));
                    if (2 * c >= nv) p0 = 0.0f;              // a row that sees nothing: exp2(-1e30 + 1e30) is 1, not 0
                    if (2 * c + 1 >= nv) p1 = 0.0f;
                    sum0 += p0; sum1 += p1;
                    pr[c] = pack2<BF>(p0, p1);
                }
                l_run = l_run * alpha + (sum0 + sum1);
                m2 = m_new;
            }
            const bool p_stored = settled;

            // ---- O += P V of the previous block must be done before O is rescaled ----
            // S of this block was committed behind P V of block blk-2, so the barrier's current phase is blk-1 or
            // later and its parity cannot be mistaken for an older one; blocks that rescale nothing do not wait at all
            // (the last block waits in any case: once its P is handed over, P V of it may complete at any time, and
            // the wait for the last phase after the loop must not meet a barrier that is two phases ahead of it)
            const bool rescale = __any_sync(0xFFFFFFFFu, moved);
            if (blk > 0 && (rescale || blk == n_blocks - 1)) {
                if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded(smem_u32(bar_o), (uint32_t)((blk - 1) & 1), status))) { alive = false; break; }
                tc_fence_after();
                if (rescale) {                               // this warp's rows of O *= alpha
#pragma unroll
                    for (int part = 0; part < 4; part++) {
                        uint32_t orow[32];
                        tmem_ld32(tmem + lane_base + kColO + 32 * part, orow);
                        tc_wait_ld(orow);
#pragma unroll
                        for (int c = 0; c < 32; c++) orow[c] = __float_as_uint(__uint_as_float(orow[c]) * alpha);
                        tmem_st32(tmem + lane_base + kColO + 32 * part, orow);
                    }
                }
            }
            if (!p_stored) tmem_st32(tmem + lane_base + col_s, pr);   // P over the columns S was read from
            tc_wait_st();

            // V rows of the slab that no copy of this block wrote (pages this tile does not need: whatever the stage
            // held before, at first whatever the SM's last CTA left) or that lie past the sequence's end (whatever the
            // page's last owner left) meet P = 0, and 0 * NaN is NaN: zero them.  Last block(s) of a tile only.
            const int n_good = min(len - tok_base, 16 * min(4, n_pages - 4 * blk));   // rows that hold tokens of the sequence
            if (n_good < kTcBlock) {
                if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded(smem_u32(&vfull[s]), (uint32_t)((blk / kTcStages) & 1), status))) { alive = false; break; }
                const int r0 = max(n_good, 0), n_rows = kTcBlock - r0;
                for (int i = tid; i < n_rows * 16; i += kTcRows) {
                    const int r = r0 + (i >> 4), c = i & 15;
                    *reinterpret_cast<uint4*>(s_v + s * kSlabBytes + (c >> 3) * kHalfBytes + r * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&p_ready[buf]));            // this row's P (and O) are ready for the tensor pipe
        }
        // ---- the last block's O ----
        if (alive && !__all_sync(0xFFFFFFFFu, mbar_wait_bounded(smem_u32(bar_o), (uint32_t)((n_blocks - 1) & 1), status))) alive = false;
        tc_fence_after();
    }
    const float m_run = m2 * 0.6931471805599453f;            // natural-log units, as the split-KV rows carry it

    const bool poisoned = __any_sync(0xFFFFFFFFu, !alive || __ldcg(status) != 0);   // fail closed, whole warps at a time

    if (!poisoned && warp < kTcRows / 32) {
        float* prow = nullptr;
        if (n_chunks > 1)                                    // split context: (o, m, l) of this chunk into the sequence's region
            prow = partials + (size_t)poff * g.H * (D + 2) +
                   partial_off(chunk, (tok_first + tid / G) * g.H + kvh * G + tid % G, nq * g.H, D);
        const float inv = 1.0f / (l_run + 1e-8f);
#pragma unroll
        for (int part = 0; part < 4; part++) {
            uint32_t orow[32];
            tmem_ld32(tmem + lane_base + kColO + 32 * part, orow);
            tc_wait_ld(orow);
            if (!valid) continue;
            if (n_chunks > 1) {
#pragma unroll
                for (int c = 0; c < 32; c += 2)
                    *reinterpret_cast<float2*>(prow + 32 * part + c) = make_float2(__uint_as_float(orow[c]), __uint_as_float(orow[c + 1]));
            } else if (out_dtype == DT_FP32) {
#pragma unroll
                for (int c = 0; c < 32; c += 4)
                    *reinterpret_cast<float4*>((float*)out + qo_row * D + 32 * part + c) =
                        make_float4(__uint_as_float(orow[c]) * inv, __uint_as_float(orow[c + 1]) * inv,
                                    __uint_as_float(orow[c + 2]) * inv, __uint_as_float(orow[c + 3]) * inv);
            } else {
#pragma unroll
                for (int c = 0; c < 32; c += 8) {
                    uint4 w;
                    w.x = pack2<BF>(__uint_as_float(orow[c]) * inv, __uint_as_float(orow[c + 1]) * inv);
                    w.y = pack2<BF>(__uint_as_float(orow[c + 2]) * inv, __uint_as_float(orow[c + 3]) * inv);
                    w.z = pack2<BF>(__uint_as_float(orow[c + 4]) * inv, __uint_as_float(orow[c + 5]) * inv);
                    w.w = pack2<BF>(__uint_as_float(orow[c + 6]) * inv, __uint_as_float(orow[c + 7]) * inv);
                    *reinterpret_cast<uint4*>((uint16_t*)out + qo_row * D + 32 * part + c) = w;
                }
            }
        }
        if (n_chunks > 1 && valid) *reinterpret_cast<float2*>(prow + D) = make_float2(m_run, l_run);
    }

    // ---- tensor memory goes back on every path ----
    tc_fence_before();
    __syncthreads();
    if (warp == kTcRows / 32) tmem_dealloc(tmem, kTmemCols);
    if (n_chunks == 1) return;

    // the CTA that arrives last for the tile merges its chunks (nothing is written while the status word is set)
    if (tid == 0) {
        __threadfence();
        const int tiles = (nq + tpt - 1) / tpt;
        int* c = counters + cbase + kvh * tiles + tile;
        const int ticket = atomicAdd(c, 1);
        const int last = ticket == n_chunks - 1;
        if (last) *c = 0;
        *s_flag = last;
    }
    __syncthreads();
    if (*s_flag) {
        const MergeOut mo{nullptr, out, nullptr, out_dtype, nullptr, status};
        merge_rows(g, mo, b, kvh, G, 0, n_chunks, partials + (size_t)poff * g.H * (D + 2),
                   MergeMap{G * tok_cnt, nq * g.H, q_base + tok_first, tok_first, 0});
    }
}

}  // namespace

// 128-row tiles on tcgen05: 16-bit pools, head_dim 128, page size 16, groups that divide 128.
bool prefill_tc_supported(const Geometry& g) {
    return decode_mma_supported(g) && g.dtype != DT_FP8 && g.D == kTcD && g.Hkv > 0 && kTcRows % (g.H / g.Hkv) == 0;
}

// `map16`: the layer's pool as rows of D elements with a box of 16 rows x 64 elements (make_pool_tensor_map
// with box_rows = 16).  Work list, counters and split regions as for launch_prefill_mma, with tiles of 128 rows.
cudaError_t launch_prefill_tc(const Geometry& g, const CUtensorMap* map16, const StepDev& st, const PrefillDev& pf,
                              const int32_t* page_table, const void* q, void* out, int out_dtype, float* partials,
                              int* counters, int* status, cudaStream_t s) {
    if (pf.n_items <= 0) return cudaSuccess;
    if (!prefill_tc_supported(g) || !counters || !status) return cudaErrorNotSupported;
    if (out_dtype != DT_FP32 && out_dtype != g.io_dtype) return cudaErrorInvalidValue;
    static bool attr_done[2][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int bf = g.dtype == DT_BF16;
    if (dev < 0 || dev >= 64 || !attr_done[bf][dev]) {
        cudaError_t e = bf ? cudaFuncSetAttribute(prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem)
                           : cudaFuncSetAttribute(prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[bf][dev] = true;
    }
    if (bf) prefill_tc_kernel<true><<<pf.n_items, kTcThreads, kTcSmem, s>>>(*map16, g, st, pf, page_table, (const uint16_t*)q, out,
                                                                     out_dtype, partials, counters, status);
    else    prefill_tc_kernel<false><<<pf.n_items, kTcThreads, kTcSmem, s>>>(*map16, g, st, pf, page_table, (const uint16_t*)q, out,
                                                                      out_dtype, partials, counters, status);
    return cudaGetLastError();
}

}  // namespace tk
