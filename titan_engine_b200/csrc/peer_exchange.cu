// peer_exchange.cu — cross-GPU exchange of split-KV partials fused with the log-sum-exp
// combine, over NVLink peer memory (one process per GPU, CUDA IPC mappings).
//
// A sequence whose tokens are spread over several GPUs needs, per layer, every rank's merged
// (o, m, l) rows on every rank.  Instead of a library all-gather followed by a combine launch,
// ONE kernel per rank stores its rows straight into a mailbox in every peer's memory (plain
// peer stores), waits (bounded) for the peers' rows in its own
// mailbox and combines what arrived.  The reference is single-GPU (GPU 0 only:
// src/memory/memory_manager.cpp:15) and has no counterpart.
//
// Mailbox of a rank (device memory of that rank):
//   cells[2 parities][world sources][max_rows * row_floats], 8 bytes each: (float bits, epoch)
// A cell is stored and loaded as one 64-bit atom, so a receiver that finds the epoch it waits for has the
// value of that epoch with it: it polls the data itself, and a sender needs neither a flag nor a fence
// behind its rows.  The epoch counts exchanges (1, 2, ...), parity = epoch & 1.  Two parities are enough:
// a rank can only start sending epoch e+2 after it finished e+1, which needed every peer's e+1 rows,
// which a peer sends only after its own epoch-e kernel (the reader of that parity) has finished.
// The epoch lives in device memory and is advanced by the kernel itself (by the CTA that leaves
// last), so a launch carries no per-call host state.
//
// No multicast, no multimem: plain 64-bit stores and loads at system scope.
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

// mode bit 0: send this rank's rows to every rank's mailbox (its own included);
// mode bit 1: wait for every rank's rows and combine.  Both: one launch does the whole exchange.
__global__ void __launch_bounds__(512)
peer_exchange_combine_kernel(const PeerCtx* __restrict__ ctx_p, const float* __restrict__ partial, int n_rows, int dv,
                             void* __restrict__ out, int out_dtype, int mode) {
    const PeerCtx& c = *ctx_p;
    const int world = c.world;
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

    if (mode & 1) {
        const size_t n2 = (size_t)n_rows * row_floats / 2;                 // row_floats is even
        const float2* src = reinterpret_cast<const float2*>(partial);
        for (int p = 0; p < world; p++) {
            uint64_t* dst = tk::peer_cells(c, p, parity, c.rank);
            for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += (size_t)gridDim.x * blockDim.x) {
                const float2 v = src[i];
                tk::st_cells2(dst + 2 * i, tk::make_cell(v.x, epoch), tk::make_cell(v.y, epoch));
            }
        }
    }
    if (!(mode & 2)) { leave(); return; }

    // one warp per row: poll the row's cells of every source (they carry the epoch), then the
    // log-sum-exp combine over the sources in rank order: same arithmetic as the combine of stacked partials.
    // A row some source never sent stays unwritten and the status word says TK_TIMEOUT.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const size_t src_stride_pairs = c.slot_bytes / 16;
    auto cell = [](const uint64_t* p) { return tk::cell_value(__ldcg(reinterpret_cast<const unsigned long long*>(p))); };
    for (int row = blockIdx.x * n_warps + warp; row < n_rows; row += gridDim.x * n_warps) {
        const uint64_t* base = tk::peer_cells(c, c.rank, parity, 0) + (size_t)row * row_floats;
        bool ok = true;
        for (int pi = lane; pi < row_floats / 2 && ok; pi += 32)
            for (int s0 = 0; s0 < world && ok; s0 += 8)
                ok = tk::peer_wait_pairs(base + (size_t)s0 * 2 * src_stride_pairs + 2 * pi, src_stride_pairs,
                                         min(8, world - s0), epoch, c.limit_ns);
        if (!__all_sync(0xFFFFFFFFu, ok)) {
            if (lane == 0) atomicExch(c.status, (int)TK_TIMEOUT);
            continue;
        }
        const uint64_t* src[kMaxWorld];
#pragma unroll
        for (int r = 0; r < kMaxWorld; r++)
            if (r < world) src[r] = tk::peer_cells(c, c.rank, parity, r) + (size_t)row * row_floats;
        float M = -1e30f;
        for (int r = 0; r < world; r++) M = fmaxf(M, cell(src[r] + dv));
        float L = 0.0f;
        for (int r = 0; r < world; r++) L += cell(src[r] + dv + 1) * expf(cell(src[r] + dv) - M);
        const float inv = 1.0f / (L + 1e-8f);
        for (int d = lane; d < dv; d += 32) {
            float acc = 0.0f;
            for (int r = 0; r < world; r++) acc += cell(src[r] + d) * expf(cell(src[r] + dv) - M);
            tk::store_out(out, (size_t)row * dv + d, acc * inv, out_dtype);
        }
    }
    leave();
}

}  // namespace

struct tk_peer {
    int rank = 0, world = 1, max_rows = 0, row_floats = 0, device = 0;
    size_t slot_bytes = 0, total = 0;
    uint8_t* local = nullptr;
    uint8_t* peers[kMaxWorld] = {};
    bool opened[kMaxWorld] = {};           // mapped through CUDA IPC (to be closed)
    bool connected = false;
    bool sent_once = false;
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
    c.slot_bytes = p->slot_bytes;
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
    p->slot_bytes = ((size_t)max_rows * row_floats * sizeof(uint64_t) + 255) / 256 * 256;    // 8-byte cells
    p->total = 2 * p->slot_bytes * world;
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
                       void* stream, int mode) {
    if (!p || n_rows < 0 || dv <= 0) return TK_INVALID_ARG;
    if (!p->connected) return pfail(p, TK_INVALID_ARG, "peers are not connected");
    if (dv + 2 != p->row_floats || n_rows > p->max_rows) return pfail(p, TK_INVALID_ARG, "rows do not fit the mailbox");
    if ((mode & 1) && !partial) return pfail(p, TK_INVALID_ARG, "null partial");
    if ((mode & 2) && (!partial || !out)) return pfail(p, TK_INVALID_ARG, "null partial/out");
    if ((mode & 2) && out_dtype != TK_FP32 && out_dtype != TK_FP16 && out_dtype != TK_BF16) return pfail(p, TK_INVALID_ARG, "bad out dtype");
    if (mode & 1) p->sent_once = true;
    if (!p->sent_once) return pfail(p, TK_INVALID_ARG, "recv_combine before any send");
    const size_t work = (size_t)n_rows * p->row_floats / 2;
    int grid = (int)((work + 4095) / 4096);
    if ((mode & 2) && grid < (n_rows + 15) / 16) grid = (n_rows + 15) / 16;      // combine: one warp per row
    if (grid < 1) grid = 1;
    if (grid > p->num_sms) grid = p->num_sms;
    peer_exchange_combine_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(p->d_ctx, partial, n_rows, dv, out, out_dtype, mode);
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
int peer_exchange(tk_peer* p, const float* partial, int n_rows, int dv, void* out, int out_dtype, void* stream) {
    return peer_launch(p, partial, n_rows, dv, out, out_dtype, stream, 3);
}
// An attention launch that carries the exchange itself counts as this exchange's send.
void peer_note_fused_send(tk_peer* p) { if (p) p->sent_once = true; }

}  // namespace tk
