// rope_append.cu — rotary position embedding of a step's q and k rows (16-bit in, 16-bit out).
//
// Same arithmetic as the reference's rope_kernel (src/compute/cuda/attention.cu:15-48), which its
// layer loop runs immediately before KVCache::update (src/model/dense.cpp:382-388): interleaved
// pairs (d, d+1), freq = (1/powf(theta, d/D)) * scaling, angle = position * freq, in FP32.
// Positions come from the step plan: a q row belongs to the newest token of its sequence
// (len-1), a k row to its own token.  On decode steps with 16-bit storage this kernel is not
// launched at all — the rotation rides inside the attention kernel (decode_mma.cu).
// The MLA cache shape rotates only the rope dims at the end of each q / K row, with
// freq = 1/powf(theta, d/rope_dims) (rope_mla_kernel, src/compute/cuda/attention.cu:259-294):
// rope_off(g) dims are copied, the remaining rope_dims(g) rotated.
#include "tk_kernels.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tk {

namespace {

// src / dst point at the first rotated dim of the row; d counts from there, D = number of rotated dims
template <bool BF16>
__device__ __forceinline__ void rotate_store(const uint16_t* src, uint16_t* dst, int d, int D, int position,
                                             float theta, float scaling) {
    float x0, x1;
    if (BF16) { x0 = __uint_as_float((uint32_t)src[d] << 16); x1 = __uint_as_float((uint32_t)src[d + 1] << 16); }
    else      { x0 = __half2float(__ushort_as_half(src[d])); x1 = __half2float(__ushort_as_half(src[d + 1])); }
    float freq = 1.0f / powf(theta, (float)d / D);
    freq *= scaling;
    const float angle = position * freq;
    const float c = cosf(angle), s = sinf(angle);
    const float y0 = x0 * c - x1 * s, y1 = x0 * s + x1 * c;
    if (BF16) {
        dst[d] = __bfloat16_as_ushort(__float2bfloat16_rn(y0));
        dst[d + 1] = __bfloat16_as_ushort(__float2bfloat16_rn(y1));
    } else {
        dst[d] = __half_as_ushort(__float2half_rn(y0));
        dst[d + 1] = __half_as_ushort(__float2half_rn(y1));
    }
}

// blocks [0, n_seqs): q rows of one sequence (H heads); blocks [n_seqs, n_seqs + n_tokens): k rows
// of one token (Hkv heads).  Threads stride over (head, pair).
template <bool BF16>
__global__ void rope16_kernel(Geometry g, StepDev st, const uint16_t* __restrict__ q, const uint16_t* __restrict__ k,
                              uint16_t* __restrict__ q_out, uint16_t* __restrict__ k_out, float theta, float scaling) {
    const int half = g.D / 2, off = rope_off(g), rd = rope_dims(g);
    const bool is_q = (int)blockIdx.x < st.n_seqs;
    const int unit = is_q ? blockIdx.x : blockIdx.x - st.n_seqs;         // sequence of the step, or token
    const int heads = is_q ? g.H : g.Hkv;
    int pos = is_q ? st.len[unit] - 1 : st.tok_pos[unit];
    if (pos < 0) pos = 0;
    const uint16_t* src = is_q ? q : k;
    uint16_t* dst = is_q ? q_out : k_out;
    for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
        const size_t row = ((size_t)unit * heads + i / half) * g.D;
        const int d = (i % half) * 2;
        if (d < off) { dst[row + d] = src[row + d]; dst[row + d + 1] = src[row + d + 1]; }
        else rotate_store<BF16>(src + row + off, dst + row + off, d - off, rd, pos, theta, scaling);
    }
}

// FP32 rows in place, one position for all of them (the reference's operator interface:
// apply_rope / apply_rope_mla, src/compute/dispatch.h:68-72).  The q heads and the k heads form one
// flat list of (row, pair) units; a thread takes one unit.  Rows are row_dim floats, of which the
// last rope_dims, starting at rope_off, rotate; freq = (1/powf(theta, d/rope_dims)) * scaling with d
// counted from rope_off, angle = position * freq (rope_kernel / rope_mla_kernel,
// src/compute/cuda/attention.cu:22-37,266-283).
__global__ void rope_f32_kernel(float* __restrict__ q, float* __restrict__ k, int n_q_rows, int n_k_rows, int row_dim,
                                int rope_off, int rope_dims, int position, float theta, float scaling) {
    const int half = rope_dims / 2;
    const int unit = blockIdx.x * blockDim.x + threadIdx.x;
    if (unit >= (n_q_rows + n_k_rows) * half) return;
    const int row = unit / half, d = (unit % half) * 2;
    float* p = (row < n_q_rows ? q + (size_t)row * row_dim : k + (size_t)(row - n_q_rows) * row_dim) + rope_off;
    float freq = 1.0f / powf(theta, (float)d / rope_dims);
    freq *= scaling;
    const float angle = position * freq;
    const float c = cosf(angle), s = sinf(angle);
    const float x0 = p[d], x1 = p[d + 1];
    p[d] = x0 * c - x1 * s;
    p[d + 1] = x0 * s + x1 * c;
}

// (cos, sin) of every sequence's newest position, one entry per pair: tab[b][d/2].
__global__ void rope_table_kernel(Geometry g, StepDev st, float2* __restrict__ tab, float theta, float scaling) {
    const int rd = rope_dims(g), half = rd / 2;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= st.n_seqs * half) return;
    const int b = i / half, d = (i % half) * 2;
    const int pos = st.len[b] > 0 ? st.len[b] - 1 : 0;
    float freq = 1.0f / powf(theta, (float)d / rd);
    freq *= scaling;
    const float angle = pos * freq;
    tab[i] = make_float2(cosf(angle), sinf(angle));
}

}  // namespace

cudaError_t launch_rope_table(const Geometry& g, const StepDev& st, float2* tab, float theta, float scaling,
                              cudaStream_t s) {
    const int n = st.n_seqs * (rope_dims(g) / 2);
    if (n <= 0) return cudaSuccess;
    rope_table_kernel<<<(n + 255) / 256, 256, 0, s>>>(g, st, tab, theta, scaling);
    return cudaGetLastError();
}

cudaError_t launch_rope_f32(float* q, float* k, int n_q_rows, int n_k_rows, int row_dim, int rope_off, int rope_dims,
                            int position, float theta, float scaling, cudaStream_t s) {
    const int units = (n_q_rows + n_k_rows) * (rope_dims / 2);
    if (units <= 0) return cudaSuccess;
    rope_f32_kernel<<<(units + 127) / 128, 128, 0, s>>>(q, k, n_q_rows, n_k_rows, row_dim, rope_off, rope_dims, position,
                                                        theta, scaling);
    return cudaGetLastError();
}

cudaError_t launch_rope16(const Geometry& g, const StepDev& st, const void* q, const void* k, void* q_out,
                          void* k_out, float theta, float scaling, cudaStream_t s) {
    const int blocks = st.n_seqs + st.n_tokens;
    if (blocks <= 0) return cudaSuccess;
    if (g.io_dtype == DT_BF16)
        rope16_kernel<true><<<blocks, 256, 0, s>>>(g, st, (const uint16_t*)q, (const uint16_t*)k, (uint16_t*)q_out,
                                                   (uint16_t*)k_out, theta, scaling);
    else
        rope16_kernel<false><<<blocks, 256, 0, s>>>(g, st, (const uint16_t*)q, (const uint16_t*)k, (uint16_t*)q_out,
                                                    (uint16_t*)k_out, theta, scaling);
    return cudaGetLastError();
}

}  // namespace tk
