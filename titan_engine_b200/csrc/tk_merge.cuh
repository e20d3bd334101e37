// tk_merge.cuh — log-sum-exp merge of split-KV partial rows, done inside the decode kernels by
// whichever CTA finishes last for a (sequence, kv head): no separate combine launch, no tail.
//
// Merge rule: M = max m_i, L = sum l_i e^{m_i-M}, O = sum o_i e^{m_i-M}, out = O * 1/(L + 1e-8f)
// — the normaliser of the reference's kernel (src/compute/cuda/attention.cu:142) applied to the
// merged sums.
#pragma once

#include "tk_kernels.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tk {

__device__ __forceinline__ void store_out(void* out, size_t idx, float v, int dt) {
    if (dt == DT_BF16)      ((__nv_bfloat16*)out)[idx] = __float2bfloat16_rn(v);
    else if (dt == DT_FP16) ((__half*)out)[idx] = __float2half_rn(v);
    else                    ((float*)out)[idx] = v;
}

// Every thread of the CTA calls this after the CTA's partial row for heads [kvh*G, kvh*G+G)
// of step-sequence b is in global memory.  The CTA that arrives last for (b, kvh) merges all
// of that sequence's rows for those heads and writes the result; it also re-arms the counter.
// `s_flag` is one int of shared memory.  Returns without merging when mo.counters is null.
__device__ __forceinline__ void merge_if_last(const Geometry& g, const StepDev& st, const MergeOut& mo,
                                              int b, int kvh, int G, const float* partials, int* s_flag) {
    if (!mo.counters) return;
    const int D = g.Dv;                                // width of a partial / output row
    const int r0 = st.chunk_base[b], n = st.chunk_base[b + 1] - r0;
    __syncthreads();                                   // the CTA's partial row is complete ...
    if (threadIdx.x == 0) {
        __threadfence();                               // ... and ordered before the ticket, device-wide
        int* c = mo.counters + (size_t)b * g.Hkv + kvh;
        const int ticket = atomicAdd(c, 1);
        const int last = ticket == n - 1;
        if (last) *c = 0;                              // nobody else touches it again in this launch
        *s_flag = last;
    }
    __syncthreads();
    if (!*s_flag) return;
    __threadfence();                                   // see the other CTAs' rows

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int epl = D >> 5;                            // dims per lane: 2 (D=64) or 4 (D=128)
    for (int gq = warp; gq < G; gq += n_warps) {
        const int h = kvh * G + gq;
        float M = -1e30f;
        for (int r = lane; r < n; r += 32) M = fmaxf(M, __ldcg(partials + partial_off(r0 + r, h, g.H, D) + D));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
        float L = 0.0f;
        for (int r = lane; r < n; r += 32) {
            const float* p = partials + partial_off(r0 + r, h, g.H, D);
            L += __ldcg(p + D + 1) * expf(__ldcg(p + D) - M);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xFFFFFFFFu, L, o);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < n; r++) {
            const float* p = partials + partial_off(r0 + r, h, g.H, D);
            const float w = expf(__ldcg(p + D) - M);
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (e < epl) acc[e] += __ldcg(p + lane * epl + e) * w;
        }
        const float inv = 1.0f / (L + 1e-8f);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (e >= epl) break;
            const int d = lane * epl + e;
            if (mo.out) store_out(mo.out, ((size_t)b * g.H + h) * D + d, acc[e] * inv, mo.out_dtype);
            if (mo.partial_out) mo.partial_out[partial_off(b, h, g.H, D) + d] = acc[e];
        }
        if (mo.partial_out && lane == 0) {
            mo.partial_out[partial_off(b, h, g.H, D) + D] = M;
            mo.partial_out[partial_off(b, h, g.H, D) + D + 1] = L;
        }
    }
}

}  // namespace tk
