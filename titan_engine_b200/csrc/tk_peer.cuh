// tk_peer.cuh — device-side view of a peer exchange (peer_exchange.cu) for the kernels that take
// part in it: the mailboxes of all ranks, this rank's place among them, and the words the kernels
// synchronise on.  One PeerCtx lives in device memory per tk_peer and never changes after connect.
#pragma once

#include <cstddef>
#include <cstdint>

namespace tk {

constexpr int kPeerMaxWorld = 16;

// Mailbox of a rank (device memory of that rank):
//   payload[2 parities][world sources][max_rows * row_floats] float   (slots 256-byte aligned)
//   flags  [2 parities][world sources][max_rows] uint32: flag g of a source = epoch of its rows of
//          group g (a group = the rows one CTA publishes together)
struct PeerCtx {
    uint8_t* box[kPeerMaxWorld];
    int rank, world, max_rows, row_floats;
    size_t slot_bytes, flags_off;
    uint32_t* epoch;              // exchanges completed by this rank
    unsigned* tickets;            // [0]: CTAs that have sent, [1]: CTAs that have left (exchange kernel);
                                  // [2]: CTAs that have left (attention kernel with the exchange inside)
    int* status;                  // becomes TK_TIMEOUT when a wait gives up
    unsigned long long limit_ns;
};

__device__ __forceinline__ uint32_t* peer_flag(const PeerCtx& c, int box, int parity, int src, int group) {
    return reinterpret_cast<uint32_t*>(c.box[box] + c.flags_off) + ((size_t)(parity * c.world + src) * c.max_rows + group);
}
__device__ __forceinline__ float* peer_rows(const PeerCtx& c, int box, int parity, int src) {
    return reinterpret_cast<float*>(c.box[box] + ((size_t)parity * c.world + src) * c.slot_bytes);
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long peer_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Spin until *flag == epoch or the limit runs out; false on expiry.
__device__ __forceinline__ bool peer_wait_flag(const uint32_t* flag, uint32_t epoch, unsigned long long limit_ns) {
    if (ld_acquire_sys(flag) == epoch) return true;
    const unsigned long long t0 = peer_now_ns();
    while (ld_acquire_sys(flag) != epoch)
        if (peer_now_ns() - t0 > limit_ns) return false;
    return true;
}

}  // namespace tk

struct tk_peer;
namespace tk {
// Host side, for the library's own callers: the device context of a connected exchange (nullptr
// until connected) and one exchange launch whose rows are published in groups of `group_rows`
// (the grouping the attention kernels use when they carry the exchange themselves).
const PeerCtx* peer_device_ctx(const tk_peer* p);
int peer_max_rows(const tk_peer* p);
int peer_row_floats(const tk_peer* p);
int peer_exchange_grouped(tk_peer* p, const float* partial, int n_rows, int dv, int group_rows, void* out,
                          int out_dtype, void* stream);
void peer_note_fused_send(tk_peer* p);
}  // namespace tk
