// tk_peer.cuh — device-side view of a peer exchange (peer_exchange.cu) for the kernels that take
// part in it: the mailboxes of all ranks, this rank's place among them, and the words the kernels
// synchronise on.  One PeerCtx lives in device memory per tk_peer and never changes after connect.
#pragma once

#include <cstddef>
#include <cstdint>

namespace tk {

constexpr int kPeerMaxWorld = 16;

// Mailbox of a rank (device memory of that rank):
//   cells[2 parities][world sources][max_rows * row_floats]   (slots 256-byte aligned)
// A cell is 8 bytes: the float's bits in the low word, the epoch of the exchange it belongs to in the
// high word.  A cell is written with ONE 64-bit store and read with ONE 64-bit load, both single-copy
// atomic, so value and epoch always travel together: the receiver polls the data itself and needs
// neither a flag nor a fence behind the sender's rows (one NVLink crossing instead of two in a row).
struct PeerCtx {
    uint8_t* box[kPeerMaxWorld];
    int rank, world, max_rows, row_floats;
    size_t slot_bytes;
    uint32_t* epoch;              // exchanges completed by this rank
    unsigned* tickets;            // [1]: CTAs that have left (exchange kernel); [2]: CTAs that have left
                                  // (attention kernel with the exchange inside)
    int* status;                  // becomes TK_TIMEOUT when a wait gives up
    unsigned long long limit_ns;
};

__device__ __forceinline__ uint64_t* peer_cells(const PeerCtx& c, int box, int parity, int src) {
    return reinterpret_cast<uint64_t*>(c.box[box] + ((size_t)parity * c.world + src) * c.slot_bytes);
}
__device__ __forceinline__ uint64_t make_cell(float v, uint32_t epoch) {
    return (uint64_t)__float_as_uint(v) | ((uint64_t)epoch << 32);
}
__device__ __forceinline__ float cell_value(uint64_t cell) { return __uint_as_float((uint32_t)cell); }
__device__ __forceinline__ uint32_t cell_epoch(uint64_t cell) { return (uint32_t)(cell >> 32); }
// two neighbouring cells (16-byte aligned) in one instruction; each 64-bit element is its own atom
__device__ __forceinline__ void st_cells2(uint64_t* p, uint64_t a, uint64_t b) {
    asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_cells2(const uint64_t* p, uint64_t& a, uint64_t& b) {
    asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long peer_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Spin until the `n_pairs` cell pairs at p[2 * stride * i], i < n_pairs (n_pairs <= 8), all carry `epoch`,
// or the limit runs out; false on expiry.  All loads of a round are in flight together.
__device__ __forceinline__ bool peer_wait_pairs(const uint64_t* p, size_t stride_pairs, int n_pairs, uint32_t epoch,
                                                unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (;;) {
        uint64_t a[8], b[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (i < n_pairs) ld_cells2(p + 2 * stride_pairs * i, a[i], b[i]);
        bool ok = true;
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (i < n_pairs) ok = ok && cell_epoch(a[i]) == epoch && cell_epoch(b[i]) == epoch;
        if (ok) return true;
        if (t0 == 0) t0 = peer_now_ns();
        else if (peer_now_ns() - t0 > limit_ns) return false;
    }
}

}  // namespace tk

struct tk_peer;
namespace tk {
// Host side, for the library's own callers: the device context of a connected exchange (nullptr
// until connected) and one whole exchange launch.
const PeerCtx* peer_device_ctx(const tk_peer* p);
int peer_max_rows(const tk_peer* p);
int peer_row_floats(const tk_peer* p);
int peer_exchange(tk_peer* p, const float* partial, int n_rows, int dv, void* out, int out_dtype, void* stream);
void peer_note_fused_send(tk_peer* p);
}  // namespace tk
