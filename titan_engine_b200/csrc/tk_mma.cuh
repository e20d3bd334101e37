// tk_mma.cuh — device primitives shared by the tensor-core decode kernels (decode_mma.cu,
// decode_mma_mla.cu): bounded mbarrier waits, tiled TMA loads, ldmatrix, m16n8k16 MMAs,
// the 128-byte-swizzle address, exp2 and 16-bit packing.
#pragma once

#include "tk_kernels.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cudaTypedefs.h>

namespace tk {

namespace {

constexpr int kWarps = 4;
constexpr int kPage = 16;               // tokens per page on this path
constexpr int kBoxBytes = 32 * 128;     // one TMA box: 32 rows (K 0-15, V 16-31) x 128 B
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // bounded mbarrier wait

enum Kind { K_F16 = 0, K_BF16 = 1, K_FP8 = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// The same test, but the thread may stay suspended in hardware for up to `hint_ns` while the phase is not complete
// (it is woken when it completes): a waiting thread then costs its scheduler almost no issue slots.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Wait with a wall-clock bound: on expiry record it and give up instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status,
                                                  unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    while (!mbar_try_wait(bar, parity)) {
        if (globaltimer_ns() - t0 > limit_ns) {
            if (status) atomicExch(status, 4 /* TK_TIMEOUT */);
            return false;
        }
    }
    return true;
}
// For threads that do nothing but wait (a producer role between two pieces of work): suspended waits.
__device__ __forceinline__ bool mbar_wait_bounded_idle(uint32_t bar, uint32_t parity, int* status,
                                                       unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    while (!mbar_try_wait_suspend(bar, parity, 100000u)) {
        if (globaltimer_ns() - t0 > limit_ns) {
            if (status) atomicExch(status, 4 /* TK_TIMEOUT */);
            return false;
        }
    }
    return true;
}
// 2-D tiled TMA load, global -> this CTA's shared memory, completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    // K/V pages are read once per step: mark them evict-first so they do not push q, the page
    // table and the split-KV partials out of L2 (measured +1.5 % on the 8B-shape batch)
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar), "l"(policy) : "memory");
}
// The same load for tiles that many CTAs read (the prefill kernel: every 64-row tile of a sequence walks the
// same pages): no evict-first hint, the tile should stay in L2 for the other CTAs.
__device__ __forceinline__ void tma_load_2d_shared_tile(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar), "l"(policy) : "memory");
}
// 4-D tiled TMA load (same completion and L2 hint as the 2-D form).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4, %5}], [%6], %7;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if (BF16) { __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&v); }
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// two E4M3 codes (low byte first) -> f16x2, exact
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_codes) {
    uint32_t r;
    const unsigned short a = (unsigned short)two_codes;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(a));
    return r;
}
// RoPE of one (d, d+1) pair held as two 16-bit values in one register; same arithmetic as the
// reference's rope_kernel (src/compute/cuda/attention.cu:22-37), result rounded to the storage type.
template <bool BF16>
__device__ __forceinline__ uint32_t rope_pair(uint32_t w, const float2* __restrict__ tab, int d) {
    float x0, x1;
    if (BF16) { x0 = __uint_as_float(w << 16); x1 = __uint_as_float(w & 0xFFFF0000u); }
    else { const __half2 h = *reinterpret_cast<const __half2*>(&w); x0 = __low2float(h); x1 = __high2float(h); }
    const float2 cs = tab[d >> 1];                          // (cos, sin) of this sequence's newest position
    return pack2<BF16>(x0 * cs.x - x1 * cs.y, x0 * cs.y + x1 * cs.x);
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute may
// start while the kernel before it in the stream is still running, once every CTA of that kernel has
// executed pdl_launch_dependents() or exited; it must call pdl_wait() - which returns when the earlier
// kernel has finished and its writes are visible - before it touches anything that kernel reads or
// writes.  Both are no-ops in a launch without the attribute.  The decode kernels signal as their first
// instruction: the dependent grid then gets exactly the SM slots the earlier grid has stopped needing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// swizzled byte offset of 16-byte chunk `c` of row `r` inside a 32x128-byte box
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

constexpr float kLog2e = 1.4426950408889634f;

}  // namespace

}  // namespace tk
