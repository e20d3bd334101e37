// tk_merge.cuh — log-sum-exp merge of split-KV partial rows, done inside the decode kernels by
// whichever CTA finishes last for a (sequence, kv head): no separate combine launch, no tail.
//
// Merge rule: M = max m_i, L = sum l_i e^{m_i-M}, O = sum o_i e^{m_i-M}, out = O * 1/(L + 1e-8f)
// — the normaliser of the reference's kernel (src/compute/cuda/attention.cu:142) applied to the
// merged sums.
#pragma once

#include "tk_kernels.cuh"
#include "tk_peer.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tk {

__device__ __forceinline__ void store_out(void* out, size_t idx, float v, int dt) {
    if (dt == DT_BF16)      ((__nv_bfloat16*)out)[idx] = __float2bfloat16_rn(v);
    else if (dt == DT_FP16) ((__half*)out)[idx] = __float2half_rn(v);
    else                    ((float*)out)[idx] = v;
}

// Which partial columns a (sequence, kv head) group owns and where its outputs go.  One query token
// per sequence: the G heads of the kv head, out row = the sequence's index in the step.  Several query
// tokens per sequence (multi-token attention): G * nq columns, column j*G + gg = token j, head gg of the
// group; a partial row then holds heads_per_row = H * nq_max columns, token-major.
struct MergeMap {
    int cols;            // G * (query tokens of the group)
    int heads_per_row;   // H, or H * nq_max
    int out_row0;        // row of `out` that the group's first token writes
    int tok0;            // index, within the sequence's query tokens, of the group's first token
    int counter_off;     // this token group's block of arrival counters
};

// The merge itself, by every thread of the CTA that arrived last for (b, kvh): rows r0 .. r0+n-1.
__device__ __forceinline__ void merge_rows(const Geometry& g, const MergeOut& mo, int b, int kvh, int G, int r0, int n,
                                           const float* partials, const MergeMap& mm) {
    __threadfence();                                   // see the other CTAs' rows
    if (mo.status && __ldcg(mo.status) != 0) return;   // fail closed: a wait timed out, leave `out` alone
    const int D = g.Dv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int epl = D >> 5;                            // dims per lane: 2 (D=64) or 4 (D=128)
    const PeerCtx* pc = mo.peer;
    const uint32_t epoch = pc ? __ldcg(pc->epoch) + 1u : 0u;
    const int parity = (int)(epoch & 1u);
    for (int gq = warp; gq < mm.cols; gq += n_warps) {
        const int tq = gq / G;                         // query token of the sequence (0 unless multi-token)
        const int h = kvh * G + gq % G;                // query head
        const int col = (mm.tok0 + tq) * g.H + h;      // column of the partial rows
        const int HP = mm.heads_per_row;
        float M = -1e30f;
        for (int r = lane; r < n; r += 32) M = fmaxf(M, __ldcg(partials + partial_off(r0 + r, col, HP, D) + D));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
        float L = 0.0f;
        for (int r = lane; r < n; r += 32) {
            const float* p = partials + partial_off(r0 + r, col, HP, D);
            L += __ldcg(p + D + 1) * expf(__ldcg(p + D) - M);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xFFFFFFFFu, L, o);
        // rows are added in ascending order; eight rows' loads are in flight at a time (the merge of a
        // long single sequence is a chain of L2 round trips otherwise)
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        constexpr int U = 8;
        for (int rb = 0; rb < n; rb += U) {
            float m[U], x[U][4];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const bool live = rb + u < n;
                const float* p = partials + partial_off(r0 + (live ? rb + u : rb), col, HP, D);
                m[u] = live ? __ldcg(p + D) : -1e30f;
                if (epl == 4) {                         // rows start on 8-byte, not 16-byte, boundaries
                    const float2 v0 = __ldcg(reinterpret_cast<const float2*>(p) + 2 * lane);
                    const float2 v1 = __ldcg(reinterpret_cast<const float2*>(p) + 2 * lane + 1);
                    x[u][0] = v0.x; x[u][1] = v0.y; x[u][2] = v1.x; x[u][3] = v1.y;
                } else {
                    const float2 v = __ldcg(reinterpret_cast<const float2*>(p) + lane);
                    x[u][0] = v.x; x[u][1] = v.y; x[u][2] = 0.f; x[u][3] = 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (rb + u >= n) break;
                const float w = expf(m[u] - M);
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (e < epl) acc[e] += x[u][e] * w;
            }
        }
        if (pc) {                                      // this rank's merged row goes to every rank's mailbox (its own too)
            for (int p = 0; p < pc->world; p++) {
                uint64_t* row = peer_cells(*pc, p, parity, pc->rank) + partial_off(b, h, g.H, D);
                st_cells2(row + lane * epl, make_cell(acc[0], epoch), make_cell(acc[1], epoch));
                if (epl == 4) st_cells2(row + lane * 4 + 2, make_cell(acc[2], epoch), make_cell(acc[3], epoch));
                if (lane == 0) st_cells2(row + D, make_cell(M, epoch), make_cell(L, epoch));
            }
            continue;
        }
        const float inv = 1.0f / (L + 1e-8f);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (e >= epl) break;
            const int d = lane * epl + e;
            if (mo.out) store_out(mo.out, ((size_t)(mm.out_row0 + tq) * g.H + h) * D + d, acc[e] * inv, mo.out_dtype);
            if (mo.partial_out) mo.partial_out[partial_off(b, h, g.H, D) + d] = acc[e];
        }
        if (mo.partial_out && lane == 0) {
            mo.partial_out[partial_off(b, h, g.H, D) + D] = M;
            mo.partial_out[partial_off(b, h, g.H, D) + D + 1] = L;
        }
    }
    if (!pc) return;

    // Wait for every rank's rows of this (sequence, kv head) group by polling the cells themselves - each
    // carries the epoch next to its value, so there is no flag and no fence behind the rows - then combine
    // in rank order.  A rank whose rows do not arrive within the limit: report, leave `out` alone.
    const PeerCtx& c = *pc;
    const size_t src_stride_pairs = c.slot_bytes / 16;             // cell pairs between the slots of two sources
    bool ok = true;
    for (int gq = warp; gq < G && ok; gq += n_warps) {
        const uint64_t* base = peer_cells(c, c.rank, parity, 0) + partial_off(b, kvh * G + gq, g.H, D);
        for (int s0 = 0; s0 < c.world && ok; s0 += 8) {            // eight sources' loads in flight at a time
            const int n = min(8, c.world - s0);
            const uint64_t* p0 = base + (size_t)s0 * 2 * src_stride_pairs;
            ok = peer_wait_pairs(p0 + lane * epl, src_stride_pairs, n, epoch, c.limit_ns);
            if (ok && epl == 4) ok = peer_wait_pairs(p0 + lane * 4 + 2, src_stride_pairs, n, epoch, c.limit_ns);
            if (ok && lane == 0) ok = peer_wait_pairs(p0 + D, src_stride_pairs, n, epoch, c.limit_ns);
        }
    }
    if (!__syncthreads_and(ok)) {
        if (threadIdx.x == 0) atomicExch(c.status, 4 /* TK_TIMEOUT */);
        return;
    }
    auto cell = [](const uint64_t* p) { return cell_value(__ldcg(reinterpret_cast<const unsigned long long*>(p))); };
    for (int gq = warp; gq < G; gq += n_warps) {
        const int h = kvh * G + gq;
        const size_t off = partial_off(b, h, g.H, D);
        float M = -1e30f;
        for (int r = 0; r < c.world; r++) M = fmaxf(M, cell(peer_cells(c, c.rank, parity, r) + off + D));
        float L = 0.0f;
        for (int r = 0; r < c.world; r++) {
            const uint64_t* row = peer_cells(c, c.rank, parity, r) + off;
            L += cell(row + D + 1) * expf(cell(row + D) - M);
        }
        const float inv = 1.0f / (L + 1e-8f);
        for (int d = lane; d < D; d += 32) {
            float acc = 0.0f;
            for (int r = 0; r < c.world; r++) {
                const uint64_t* row = peer_cells(c, c.rank, parity, r) + off;
                acc += cell(row + d) * expf(cell(row + D) - M);
            }
            store_out(mo.out, ((size_t)b * g.H + h) * D + d, acc * inv, mo.out_dtype);
        }
    }
}


// Every thread of the CTA calls this after the CTA's partial row for heads [kvh*G, kvh*G+G)
// of step-sequence b is in global memory.  The CTA that arrives last for (b, kvh) merges all
// of that sequence's rows for those heads and writes the result; it also re-arms the counter.
// `s_flag` is one int of shared memory.  Returns without merging when mo.counters is null.
__device__ __forceinline__ void merge_if_last(const Geometry& g, const StepDev& st, const MergeOut& mo,
                                              int b, int kvh, int G, const float* partials, int* s_flag,
                                              const MergeMap& mm) {
    if (!mo.counters) return;
    const int r0 = st.chunk_base[b], n = st.chunk_base[b + 1] - r0;
    __syncthreads();                                   // the CTA's partial row is complete ...
    if (threadIdx.x == 0) {
        __threadfence();                               // ... and ordered before the ticket, device-wide
        int* c = mo.counters + mm.counter_off + (size_t)b * g.Hkv + kvh;
        const int ticket = atomicAdd(c, 1);
        const int last = ticket == n - 1;
        if (last) *c = 0;                              // nobody else touches it again in this launch
        *s_flag = last;
    }
    __syncthreads();
    if (*s_flag) merge_rows(g, mo, b, kvh, G, r0, n, partials, mm);
    if (mo.peer) {                                     // the CTA that leaves last closes this exchange
        const PeerCtx& c = *mo.peer;
        __syncthreads();
        if (threadIdx.x == 0 && atomicAdd(c.tickets + 2, 1u) == gridDim.x - 1) {
            atomicExch(c.tickets + 2, 0u);
            atomicExch(c.epoch, __ldcg(c.epoch) + 1u);
        }
    }
}

// One query token per sequence.
__device__ __forceinline__ void merge_if_last(const Geometry& g, const StepDev& st, const MergeOut& mo,
                                              int b, int kvh, int G, const float* partials, int* s_flag) {
    merge_if_last(g, st, mo, b, kvh, G, partials, s_flag, MergeMap{G, g.H, b, 0, 0});
}

}  // namespace tk
