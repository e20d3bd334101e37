// tk_kernels.cuh — device-side views and launcher declarations shared by the
// kernels of the paged KV-cache path and the C ABI (titan_kv.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "kv_manager.h"

namespace tk {

// Storage numbering = titan::DType (reference: src/core/types.h:17-21).
enum : int { DT_FP32 = 0, DT_FP16 = 1, DT_BF16 = 2, DT_FP8 = 3 };

struct Geometry {
    int H, Hkv, D, ps;          // query heads, kv heads, head dim, tokens per page
    int dtype, io_dtype;        // storage type; type of q/k/v/out and of FP8 open pages
    int num_pages, max_seqs, max_pages_per_seq;
    int Dv;                     // V rows / output width; == D except for the MLA cache (D = 192, Dv = 128)
};

// Element offset of the K (kv = 0) or V (kv = 1) rows of tile (page, kv head): a tile is ps rows
// of K (D elements each) followed by ps rows of V (Dv elements each).
__host__ __device__ inline size_t tile_offset(const Geometry& g, int page, int kvh, int kv) {
    return ((size_t)page * g.Hkv + kvh) * (size_t)g.ps * (g.D + g.Dv) + (kv ? (size_t)g.ps * g.D : 0);
}

// Rotary embedding covers the whole row, except for the MLA cache shape (D != Dv), whose q / K rows
// are [nope dims = Dv][rope dims = D - Dv] and only the rope dims rotate.
__host__ __device__ inline int rope_off(const Geometry& g) { return g.D != g.Dv ? g.Dv : 0; }
__host__ __device__ inline int rope_dims(const Geometry& g) { return g.D - rope_off(g); }

// One layer of the pool.  16-bit / FP8 codes: [num_pages][Hkv][2 (K,V)][ps][D];
// scales f32 [num_pages][Hkv][2]; open pages [max_seqs][Hkv][2][ps][D] in io_dtype.
struct LayerPtrs {
    void*  pool;
    float* scales;
    void*  open_pages;
    void*  cold_stage;          // this layer's cold pages staged from host memory, indexed by cold id
};

// Page-table entries with this bit set name a cold page: low bits = cold id = index into cold_stage.
constexpr int kColdBit = 1 << 30;

// Device view of one step's metadata (all arrays live in one uploaded buffer).
struct StepDev {
    const int32_t* seq;         // [n_seqs] sequence slot
    const int32_t* len;         // [n_seqs] length after this step's appends
    const int32_t* chunk_base;  // [n_seqs+1] first partial row of each sequence
    const int32_t* tok_b;       // [n_tokens] index into seq[]
    const int32_t* tok_pos;     // [n_tokens]
    const int32_t* tok_dst;     // [n_tokens] row the token is stored to: page*ps + r of the pool (16-bit
                                //   storage), seq*ps + r of the open pages (FP8), -1 = sealed by this step
    const int32_t* tok_open;    // FP8: [n_open] tokens that stay in an open page (the only rows the row kernel copies)
    const int4*    items;       // [n_items] (b, chunk, kvh, kind)
    const int4*    seals;       // [n_seals] (seq slot, physical page, rows from the open page, token of the next row)
    const int32_t* new_tok;     // [n_seqs] row of the sequence's single new token in k/v, or -1
    const int32_t* q_base;      // [n_seqs] multi-token attention: row of the sequence's first new token in q / out
    const int32_t* nq;          // [n_seqs] multi-token attention: query tokens of the sequence (its new tokens)
    int n_seqs, n_tokens, n_items, n_seals, chunk_tokens;
    int n_open;
    int nq_max;                 // multi-token attention: largest nq of the step (row stride of the partials)
};

// Work list of the prefill kernel (prefill_mma.cu): tiles of kPrefillRows (token, head) rows per
// (sequence, kv head), each over the whole visible context or over split-KV chunks of ct[b] tokens.
// (kPrefillRows, kPrefillMaxPages: kv_manager.h, shared with the planner)
struct PrefillDev {
    const int4*    items;       // [n_items] (b, chunk, kvh, tile)
    const int32_t* ct;          // [n_seqs] split-KV chunk of the sequence, tokens
    const int32_t* poff;        // [n_seqs] first token row of the sequence's split region in the workspace
    const int32_t* cbase;       // [n_seqs] first arrival counter of the sequence (+ kvh * tiles + tile)
    int n_items;
    const int4*    info;        // [n_items][2]: (seq, len, nq, ct), (q_base, poff, cbase, 0) of the item's sequence
};

// partial row layout: [row][H][D+2] f32 = o[0..D) unnormalised, m at [D], l at [D+1]
__host__ __device__ inline size_t partial_off(int row, int h, int H, int D) {
    return ((size_t)row * H + h) * (size_t)(D + 2);
}

// Where the last CTA of each (sequence, kv head) puts the merged result (tk_merge.cuh).
// counters == nullptr: no in-kernel merge; partial rows are left for launch_combine_step.
struct MergeOut {
    int*   counters;            // [n_seqs * Hkv] arrival counters, zero between launches
    void*  out;                 // normalised [n_seqs][H][D] in out_dtype, or null
    float* partial_out;         // merged, unnormalised [n_seqs][H][D+2], or null
    int    out_dtype;
    // != null: the sequences' other tokens live on other GPUs.  The merging CTA stores its merged rows
    // into every rank's mailbox, publishes and awaits the per-(sequence, kv head) flags and writes the
    // combine over all ranks to `out` (tk_peer.cuh); partial_out is not used then.
    const struct PeerCtx* peer;
    // != null: the handle's status word.  A merging CTA that finds it set (a bounded wait gave up
    // somewhere on this handle and the host has not read it yet) writes nothing: no output is
    // better than one computed from a tile that never arrived.
    const int* status;
};

// Decode steps (at most one new token per sequence): the decode kernel itself writes the
// new token's K/V rows into the page it is about to read.  k == nullptr: nothing fused.
struct FuseAppend {
    const void* k;              // [n_tokens][Hkv][D] 16-bit
    const void* v;
    // rope_tab != null: q and the new K row are rotated on the fly (interleaved pairs (d, d+1))
    // before they are used/stored; rope_tab[b][d/2] = (cos, sin) of position len_b - 1, filled once
    // per step by launch_rope_table with freq = (1/powf(theta, d/rope_dims)) * scaling, angle = pos * freq,
    // d counted from the first rotated dim (rope_off)
    const float2* rope_tab;
};

cudaError_t launch_rope_table(const Geometry& g, const StepDev& st, float2* tab, float theta, float scaling,
                              cudaStream_t s);

// RoPE of a step's rows into separate buffers (used when the rotation cannot ride inside the
// attention kernel): q rows take position len-1 of their sequence, k rows their token position.
cudaError_t launch_rope16(const Geometry& g, const StepDev& st, const void* q, const void* k, void* q_out,
                          void* k_out, float theta, float scaling, cudaStream_t s);

// RoPE of FP32 rows in place at one position: q [n_q_rows][row_dim], k [n_k_rows][row_dim]; the rope_dims
// dims from rope_off on rotate (the whole row: rope_off 0, rope_dims = row_dim).
cudaError_t launch_rope_f32(float* q, float* k, int n_q_rows, int n_k_rows, int row_dim, int rope_off, int rope_dims,
                            int position, float theta, float scaling, cudaStream_t s);

// Copies `bytes` (multiple of 16) from src + l*src_stride to dst + l*dst_stride for l in [0, n_layers):
// one page (or open page) of every layer after a fork.
cudaError_t launch_copy_layers(const void* src, size_t src_stride, void* dst, size_t dst_stride, size_t bytes,
                               int n_layers, cudaStream_t s);

cudaError_t launch_apply_delta(int32_t* table, const int2* delta, int n, cudaStream_t s);

cudaError_t launch_append(const Geometry& g, const LayerPtrs& lp, const StepDev& st,
                          const int32_t* page_table, const void* k, const void* v,
                          int64_t* slots_out, cudaStream_t s, int* n_launches);

// Generic SIMT decode: one CTA per work item, any supported shape.  Returns
// cudaErrorNotSupported for shapes it has no instantiation for.
cudaError_t launch_decode_simt(const Geometry& g, const LayerPtrs& lp, const StepDev& st,
                               const int32_t* page_table, const void* q, float* partials,
                               cudaStream_t s, const MergeOut* merge = nullptr);

// TMA + mma.sync decode (16-bit and FP8 pools, page size 16, D in {64,128}).
bool        decode_mma_supported(const Geometry& g);
cudaError_t make_pool_tensor_map(const Geometry& g, void* layer_pool, CUtensorMap* out, int box_rows = 32);
cudaError_t launch_decode_mma(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* map,
                              const CUtensorMap* map_cold, const StepDev& st, const int32_t* page_table, const void* q,
                              float* partials, int* status, cudaStream_t s,
                              const MergeOut* merge = nullptr, const FuseAppend* fuse = nullptr,
                              bool overlap_prev = false);   // launch may start while the stream's previous kernel drains

// Several query tokens per sequence, causal among themselves (16-bit pools): 16/G tokens per pass over the
// pages, up to 8 such token groups.  `mo.counters` needs n_groups * n_seqs * Hkv zeroed counters.
bool        decode_mma_multi_supported(const Geometry& g, int nq_max);
int         decode_mma_multi_groups(const Geometry& g, int nq_max);
cudaError_t launch_decode_mma_multi(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* map, const StepDev& st,
                                    const int32_t* page_table, const void* q, float* partials, int* status,
                                    cudaStream_t s, const MergeOut& mo);

// Attention for every token of a prefill chunk (16-bit pools, page size 16, D in {64,128}, no cold pages).
bool        prefill_mma_supported(const Geometry& g);
cudaError_t launch_prefill_mma(const Geometry& g, const CUtensorMap* map, const StepDev& st, const PrefillDev& pf,
                               const int32_t* page_table, const void* q, void* out, int out_dtype, float* partials,
                               int* counters, int* status, cudaStream_t s);

// The same on tcgen05 / tensor memory: tiles of 128 rows (pf.items laid out for 128-row tiles), head_dim 128;
// `map16` is make_pool_tensor_map(..., box_rows = 16).
bool        prefill_tc_supported(const Geometry& g);
cudaError_t launch_prefill_tc(const Geometry& g, const CUtensorMap* map16, const StepDev& st, const PrefillDev& pf,
                              const int32_t* page_table, const void* q, void* out, int out_dtype, float* partials,
                              int* counters, int* status, cudaStream_t s);

// The same for the MLA cache shape (K rows 192, V rows 128; 16-bit pools, groups of <= 8 heads).
bool        decode_mma_mla_supported(const Geometry& g);
cudaError_t make_mla_tensor_maps(const Geometry& g, void* layer_pool, CUtensorMap* k_map, CUtensorMap* v_map);
cudaError_t launch_decode_mma_mla(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* k_map,
                                  const CUtensorMap* v_map, const StepDev& st, const int32_t* page_table,
                                  const void* q, float* partials, int* status, cudaStream_t s,
                                  const MergeOut* merge = nullptr, const FuseAppend* fuse = nullptr,
                                  bool overlap_prev = false);

// ... and its multi-token form: 8/G tokens per pass, up to 8 token groups.
bool        decode_mma_mla_multi_supported(const Geometry& g, int nq_max);
cudaError_t launch_decode_mma_mla_multi(const Geometry& g, const LayerPtrs& lp, const CUtensorMap* k_map,
                                        const CUtensorMap* v_map, const StepDev& st, const int32_t* page_table,
                                        const void* q, float* partials, int* status, cudaStream_t s, const MergeOut& mo);

// n FP32 values -> the 16-bit type `dtype` (round to nearest even).
cudaError_t launch_f32_to_16(const float* src, void* dst, size_t n, int dtype, cudaStream_t s);

// Failure-detection self-test: a bounded device wait that is made to run out (nothing completes
// the barrier); sets *status to TK_TIMEOUT after limit_ns and returns.
cudaError_t launch_bounded_wait_selftest(int* status, unsigned long long limit_ns, cudaStream_t s);

// LSE merge over each sequence's partial rows.
//   out != null     : normalised [n_seqs][H][D] in out_dtype
//   partial_out!=null: merged but unnormalised [n_seqs][H][D+2]
//   status != null  : the handle's status word; nothing is written while it is set
cudaError_t launch_combine_step(const Geometry& g, const StepDev& st, const float* partials,
                                void* out, int out_dtype, float* partial_out, cudaStream_t s,
                                const int* status = nullptr);
// LSE merge of n_parts stacked partial sets [n_parts][n_rows][D+2] -> out [n_rows][D].
cudaError_t launch_combine_parts(const float* parts, int n_parts, int n_rows, int D, void* out,
                                 int out_dtype, cudaStream_t s);

}  // namespace tk
