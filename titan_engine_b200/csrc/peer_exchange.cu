// peer_exchange.cu — cross-GPU exchange of split-KV partials fused with the log-sum-exp
// combine, over NVLink peer memory (one process per GPU, CUDA IPC mappings).
//
// A sequence whose tokens are spread over several GPUs needs, per layer, every rank's merged
// (o, m, l) rows on every rank.  Instead of a library all-gather followed by a combine launch,
// ONE kernel per rank stores its rows straight into a mailbox in every peer's memory (plain
// peer stores), publishes a flag per peer, waits (bounded) for the peers' flags in its own
// mailbox and combines what arrived.  The reference is single-GPU (GPU 0 only:
// src/memory/memory_manager.cpp:15) and has no counterpart.
//
// Mailbox of a rank (device memory of that rank):
//   payload[2 parities][world sources][max_rows * row_floats] float   (slots 256-byte aligned)
//   flags  [2 parities][world sources][max_rows] uint32; value = epoch of that source's rows of one group
// The epoch counts exchanges (1, 2, ...), parity = epoch & 1.  Two parities are enough: a rank can
// only start sending epoch e+2 after it finished e+1, which needed every peer's e+1 flag, which a
// peer sends only after its own epoch-e kernel (the reader of that parity) has finished.
// The epoch lives in device memory and is advanced by the kernel itself (by the CTA that leaves
// last), so a launch carries no per-call host state.
//
// No multicast, no multimem: plain stores and loads, system-scope release/acquire on the flags.
#include "../../include/titan_kv.h"
#include "tk_kernels.cuh"
#include "tk_merge.cuh"
#include "tk_peer.cuh"

#include <cstdio>
#include <cstring>
#include <string>

namespace {

using tk::PeerCtx;
constexpr int kMaxWorld = tk::kPeerMaxWorld;
constexpr size_t kCanaryBytes = 4096;      // guard bytes behind the mailbox (tk_peer_check_canaries)
constexpr int kCanaryByte = 0xA5;

// mode bit 0: send this rank's rows to every peer and publish the flags;
// mode bit 1: wait for the peers' rows and combine.  Both: one launch does the whole exchange.
// Rows are published in groups of group_rows rows (one flag per group), the granularity at which the
// attention kernels publish when they carry the exchange themselves.
__global__ void __launch_bounds__(512)
peer_exchange_combine_kernel(const PeerCtx* __restrict__ ctx_p, const float* __restrict__ partial, int n_rows, int dv,
                             int group_rows, void* __restrict__ out, int out_dtype, int mode) {
    const PeerCtx& c = *ctx_p;
    const int rank = c.rank, world = c.world;
    const uint32_t epoch = __ldcg(c.epoch) + ((mode & 1) ? 1u : 0u);   // a send opens the next exchange
    // called by the whole CTA on every way out: the last CTA to leave stores the epoch for the next
    // launch (by then every CTA of this launch has read the old value)
    auto leave = [&]() {
        __syncthreads();
        if ((mode & 1) && threadIdx.x == 0 && atomicAdd(c.tickets + 1, 1u) == gridDim.x - 1) {
            atomicExch(c.tickets + 1, 0u);
            atomicExch(c.epoch, epoch);
        }
    };
    const int parity = (int)(epoch & 1u);
    const int row_floats = dv + 2;
    const int n_groups = (n_rows + group_rows - 1) / group_rows;
    __shared__ int s_flag;

    if (mode & 1) {
        const size_t n2 = (size_t)n_rows * row_floats / 2;                 // row_floats is even
        const float2* src = reinterpret_cast<const float2*>(partial);
        for (int p = 0; p < world; p++) {
            if (p == rank) continue;
            float2* dst = reinterpret_cast<float2*>(tk::peer_rows(c, p, parity, rank));
            for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += (size_t)gridDim.x * blockDim.x)
                dst[i] = src[i];
        }
        __threadfence_system();                                            // this thread's rows are out ...
        if (threadIdx.x == 0) s_flag = 0;
        __syncthreads();
        if (threadIdx.x == 0 && atomicAdd(c.tickets, 1u) == gridDim.x - 1) {   // ... and so are every CTA's
            atomicExch(c.tickets, 0u);
            __threadfence_system();
            s_flag = 1;
        }
        __syncthreads();
        if (s_flag)
            for (int i = threadIdx.x; i < world * n_groups; i += blockDim.x) {
                const int p = i / n_groups, g = i % n_groups;
                if (p != rank) tk::st_release_sys(tk::peer_flag(c, p, parity, rank, g), epoch);
            }
    }
    if (!(mode & 2)) { leave(); return; }

    bool ok = true;
    for (int i = threadIdx.x; i < world * n_groups; i += blockDim.x) {
        const int src = i / n_groups, g = i % n_groups;
        if (src != rank && ok) ok = tk::peer_wait_flag(tk::peer_flag(c, rank, parity, src, g), epoch, c.limit_ns);
    }
    if (!__syncthreads_and(ok)) {                                          // give up: a peer never published
        if (threadIdx.x == 0) atomicExch(c.status, (int)TK_TIMEOUT);
        leave();
        return;
    }

    // log-sum-exp combine over the sources in rank order (own rows from `partial`, the others from
    // the mailbox, read past L1): same arithmetic as the combine of stacked partials
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    for (int row = blockIdx.x * n_warps + warp; row < n_rows; row += gridDim.x * n_warps) {
        const float* src[kMaxWorld];
#pragma unroll
        for (int r = 0; r < kMaxWorld; r++)
            if (r < world) src[r] = (r == rank ? partial : tk::peer_rows(c, rank, parity, r)) + (size_t)row * row_floats;
        float M = -1e30f;
        for (int r = 0; r < world; r++) M = fmaxf(M, __ldcg(src[r] + dv));
        float L = 0.0f;
        for (int r = 0; r < world; r++) L += __ldcg(src[r] + dv + 1) * expf(__ldcg(src[r] + dv) - M);
        const float inv = 1.0f / (L + 1e-8f);
        for (int d = lane; d < dv; d += 32) {
            float acc = 0.0f;
            for (int r = 0; r < world; r++) acc += __ldcg(src[r] + d) * expf(__ldcg(src[r] + dv) - M);
            tk::store_out(out, (size_t)row * dv + d, acc * inv, out_dtype);
        }
    }
    leave();
}

}  // namespace

struct tk_peer {
    int rank = 0, world = 1, max_rows = 0, row_floats = 0, device = 0;
    size_t slot_bytes = 0, flags_off = 0, total = 0;
    uint8_t* local = nullptr;
    uint8_t* peers[kMaxWorld] = {};
    bool opened[kMaxWorld] = {};           // mapped through CUDA IPC (to be closed)
    bool connected = false;
    bool sent_once = false;
    int group_rows = 0;                    // rows per published group for the plain entry points; 0 = all rows
    uint32_t* d_epoch = nullptr;
    unsigned* d_ticket = nullptr;          // three counters
    tk::PeerCtx* d_ctx = nullptr;          // device copy of the context, written at connect
    int* d_status = nullptr;
    unsigned long long limit_ns = 2000000000ull;
    int num_sms = 148;
    std::string err;
};

namespace {

// (re)writes the device copy of the context; synchronous, used at connect time only
cudaError_t upload_ctx(tk_peer* p) {
    tk::PeerCtx c{};
    for (int r = 0; r < kMaxWorld; r++) c.box[r] = r < p->world ? p->peers[r] : nullptr;
    c.rank = p->rank; c.world = p->world; c.max_rows = p->max_rows; c.row_floats = p->row_floats;
    c.slot_bytes = p->slot_bytes; c.flags_off = p->flags_off;
    c.epoch = p->d_epoch; c.tickets = p->d_ticket; c.status = p->d_status; c.limit_ns = p->limit_ns;
    cudaError_t e = cudaSetDevice(p->device);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();      // no kernel may be reading the old copy
    if (e == cudaSuccess) e = cudaMemcpy(p->d_ctx, &c, sizeof(c), cudaMemcpyHostToDevice);
    return e;
}

int pfail(tk_peer* p, int st, const char* what, cudaError_t e = cudaSuccess) {
    if (p) {
        p->err = what;
        if (e != cudaSuccess) { p->err += ": "; p->err += cudaGetErrorString(e); }
    }
    return st;
}

}  // namespace

extern "C" {

int tk_peer_create(int32_t rank, int32_t world, int32_t max_rows, int32_t row_floats, int32_t device, tk_peer** out) {
    if (!out) return TK_INVALID_ARG;
    *out = nullptr;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || max_rows <= 0 || row_floats < 4 || (row_floats & 1))
        return TK_INVALID_ARG;
    tk_peer* p = new tk_peer;
    p->rank = rank; p->world = world; p->max_rows = max_rows; p->row_floats = row_floats;
    if (device < 0 && cudaGetDevice(&device) != cudaSuccess) { delete p; return TK_CUDA_ERROR; }
    p->device = device;
    p->slot_bytes = ((size_t)max_rows * row_floats * sizeof(float) + 255) / 256 * 256;
    p->flags_off = 2 * p->slot_bytes * world;
    p->total = p->flags_off + 2 * (size_t)world * max_rows * sizeof(uint32_t);
    cudaDeviceProp prop;
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete p; return TK_CUDA_ERROR; }
    p->num_sms = prop.multiProcessorCount;
    cudaError_t e = cudaMalloc((void**)&p->local, p->total + kCanaryBytes);
    if (e == cudaSuccess) e = cudaMemset(p->local, 0, p->total);
    if (e == cudaSuccess) e = cudaMemset(p->local + p->total, kCanaryByte, kCanaryBytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_ticket, 4 * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(p->d_ticket, 0, 4 * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_ctx, sizeof(tk::PeerCtx));
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_epoch, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(p->d_epoch, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(p->d_status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        fprintf(stderr, "[titan-kv] tk_peer_create: %s\n", cudaGetErrorString(e));
        if (p->local) cudaFree(p->local);
        if (p->d_ticket) cudaFree(p->d_ticket);
        if (p->d_epoch) cudaFree(p->d_epoch);
        if (p->d_status) cudaFree(p->d_status);
        if (p->d_ctx) cudaFree(p->d_ctx);
        delete p;
        return TK_CUDA_ERROR;
    }
    p->peers[rank] = p->local;
    p->connected = world == 1;
    if (p->connected && upload_ctx(p) != cudaSuccess) { tk_peer_destroy(p); return TK_CUDA_ERROR; }
    *out = p;
    return TK_OK;
}

void tk_peer_destroy(tk_peer* p) {
    if (!p) return;
    cudaSetDevice(p->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < p->world; r++)
        if (p->opened[r] && p->peers[r]) cudaIpcCloseMemHandle(p->peers[r]);
    if (p->local) cudaFree(p->local);
    if (p->d_ticket) cudaFree(p->d_ticket);
    if (p->d_epoch) cudaFree(p->d_epoch);
    if (p->d_status) cudaFree(p->d_status);
    if (p->d_ctx) cudaFree(p->d_ctx);
    delete p;
}

const char* tk_peer_last_error(const tk_peer* p) { return p ? p->err.c_str() : "null handle"; }

size_t tk_peer_mailbox_bytes(const tk_peer* p) { return p ? p->total : 0; }
void* tk_peer_mailbox(const tk_peer* p) { return p ? p->local : nullptr; }

int tk_peer_export(tk_peer* p, void* handle_out) {
    if (!p || !handle_out) return TK_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) <= TK_PEER_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaSetDevice(p->device);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p->local);
    if (e != cudaSuccess) return pfail(p, TK_CUDA_ERROR, "cudaIpcGetMemHandle", e);
    memset(handle_out, 0, TK_PEER_HANDLE_BYTES);
    memcpy(handle_out, &h, sizeof(h));
    return TK_OK;
}

int tk_peer_connect(tk_peer* p, const void* handles) {
    if (!p || !handles) return TK_INVALID_ARG;
    cudaError_t e = cudaSetDevice(p->device);
    if (e != cudaSuccess) return pfail(p, TK_CUDA_ERROR, "cudaSetDevice", e);
    for (int r = 0; r < p->world; r++) {
        if (r == p->rank || p->peers[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t*)handles + (size_t)r * TK_PEER_HANDLE_BYTES, sizeof(h));
        void* ptr = nullptr;
        e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return pfail(p, TK_CUDA_ERROR, "cudaIpcOpenMemHandle", e);
        p->peers[r] = (uint8_t*)ptr;
        p->opened[r] = true;
    }
    e = upload_ctx(p);
    if (e != cudaSuccess) return pfail(p, TK_CUDA_ERROR, "context upload", e);
    p->connected = true;
    return TK_OK;
}

int tk_peer_connect_ptrs(tk_peer* p, void* const* mailboxes) {
    if (!p || !mailboxes) return TK_INVALID_ARG;
    for (int r = 0; r < p->world; r++) {
        if (r == p->rank) continue;
        if (!mailboxes[r]) return pfail(p, TK_INVALID_ARG, "connect_ptrs: null mailbox");
        p->peers[r] = (uint8_t*)mailboxes[r];
    }
    cudaError_t e = upload_ctx(p);
    if (e != cudaSuccess) return pfail(p, TK_CUDA_ERROR, "context upload", e);
    p->connected = true;
    return TK_OK;
}

int tk_peer_set_group_rows(tk_peer* p, int32_t rows) {
    if (!p || rows < 0) return TK_INVALID_ARG;
    p->group_rows = rows;
    return TK_OK;
}

int tk_peer_set_wait_limit_ms(tk_peer* p, int32_t ms) {
    if (!p || ms <= 0) return TK_INVALID_ARG;
    p->limit_ns = (unsigned long long)ms * 1000000ull;
    if (p->connected) {
        cudaError_t e = upload_ctx(p);
        if (e != cudaSuccess) return pfail(p, TK_CUDA_ERROR, "context upload", e);
    }
    return TK_OK;
}

static int peer_launch(tk_peer* p, const float* partial, int32_t n_rows, int32_t dv, void* out, int32_t out_dtype,
                       void* stream, int mode, int group_rows = 0) {
    if (!p || n_rows < 0 || dv <= 0 || group_rows < 0) return TK_INVALID_ARG;
    if (group_rows == 0) group_rows = p ? p->group_rows : 0;
    if (group_rows == 0) group_rows = n_rows > 0 ? n_rows : 1;   // one group: one flag per source
    if (!p->connected) return pfail(p, TK_INVALID_ARG, "peers are not connected");
    if (dv + 2 != p->row_floats || n_rows > p->max_rows) return pfail(p, TK_INVALID_ARG, "rows do not fit the mailbox");
    if ((mode & 1) && !partial) return pfail(p, TK_INVALID_ARG, "null partial");
    if ((mode & 2) && (!partial || !out)) return pfail(p, TK_INVALID_ARG, "null partial/out");
    if ((mode & 2) && out_dtype != TK_FP32 && out_dtype != TK_FP16 && out_dtype != TK_BF16) return pfail(p, TK_INVALID_ARG, "bad out dtype");
    if (mode & 1) p->sent_once = true;
    if (!p->sent_once) return pfail(p, TK_INVALID_ARG, "recv_combine before any send");
    const size_t work = (size_t)n_rows * p->row_floats / 2;
    int grid = (int)((work + 4095) / 4096);
    if (grid < 1) grid = 1;
    if (grid > p->num_sms) grid = p->num_sms;
    peer_exchange_combine_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(p->d_ctx, partial, n_rows, dv, group_rows, out,
                                                                         out_dtype, mode);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return pfail(p, TK_CUDA_ERROR, "exchange launch", e);
    return TK_OK;
}

int tk_peer_exchange_combine(tk_peer* p, const float* partial, int32_t n_rows, int32_t dv, void* out,
                             int32_t out_dtype, void* stream) {
    return peer_launch(p, partial, n_rows, dv, out, out_dtype, stream, 3);
}
int tk_peer_send(tk_peer* p, const float* partial, int32_t n_rows, int32_t dv, void* stream) {
    return peer_launch(p, partial, n_rows, dv, nullptr, TK_FP32, stream, 1);
}
int tk_peer_recv_combine(tk_peer* p, const float* partial, int32_t n_rows, int32_t dv, void* out, int32_t out_dtype,
                         void* stream) {
    return peer_launch(p, partial, n_rows, dv, out, out_dtype, stream, 2);
}

int tk_peer_status(tk_peer* p, void* stream) {
    if (!p) return TK_INVALID_ARG;
    int st = 0;
    cudaError_t e = cudaMemcpyAsync(&st, p->d_status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return pfail(p, TK_CUDA_ERROR, "status read", e);
    if (st != 0) {
        cudaMemsetAsync(p->d_status, 0, sizeof(int), (cudaStream_t)stream);
        return pfail(p, st, "a peer's rows did not arrive within the wait limit");
    }
    return TK_OK;
}

int tk_peer_check_canaries(tk_peer* p, void* stream) {
    if (!p) return TK_INVALID_ARG;
    cudaError_t e = cudaSetDevice(p->device);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    uint8_t buf[kCanaryBytes];
    if (e == cudaSuccess) e = cudaMemcpy(buf, p->local + p->total, kCanaryBytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return pfail(p, TK_CUDA_ERROR, "canary read", e);
    for (size_t i = 0; i < kCanaryBytes; i++)
        if (buf[i] != (uint8_t)kCanaryByte) return pfail(p, TK_CUDA_ERROR, "guard bytes behind the mailbox were overwritten");
    return TK_OK;
}

}  // extern "C"

namespace tk {

const PeerCtx* peer_device_ctx(const tk_peer* p) { return p && p->connected ? p->d_ctx : nullptr; }
int peer_max_rows(const tk_peer* p) { return p ? p->max_rows : 0; }
int peer_row_floats(const tk_peer* p) { return p ? p->row_floats : 0; }
int peer_exchange_grouped(tk_peer* p, const float* partial, int n_rows, int dv, int group_rows, void* out, int out_dtype,
                          void* stream) {
    return peer_launch(p, partial, n_rows, dv, out, out_dtype, stream, 3, group_rows);
}
// An attention launch that carries the exchange itself counts as this exchange's send.
void peer_note_fused_send(tk_peer* p) { if (p) p->sent_once = true; }

}  // namespace tk
