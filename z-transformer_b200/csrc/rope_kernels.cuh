// Rotary position embedding on the input side of attention (src/rope.zig:21-55) and its transpose on
// the gradient side (ropeBackward, src/autograd.zig:851-874).
//
// Row r of a [T, heads * head_dim] tensor sits at absolute position pos + r; element i of a head pairs
// with element i + head_dim/2 of the same head; the angle (pos + r) / theta^(2i / head_dim), its cosine
// and sine and both multiply-adds are f64, with one narrowing to f32 -- the reference's arithmetic.
//
// The (cos, sin) pairs depend on (row, i) only, so they are computed once per call -- angle, cosine
// and sine in f64 -- into a table of T x head_dim/2 float2 (kept in both orders) and read by whoever rotates: the pre-pass of
// the tensor-core kernels, which rotates q and k on their way into the f16 operand planes (the rotated
// f32 tensors are never written), or rope_apply_kernel for the CUDA-core path and for the gradients.
// Departure from the reference's arithmetic: the two multiply-adds are f32 (one fused) on f32-rounded
// cosines and sines, not f64 on f64 ones.  The result differs from the reference's by at most a few
// units in the last place of max(|lo|, |hi|) (2e-7 relative), three orders below the parity bar; what
// must be f64 -- the angle, which reaches thousands of radians -- is.  f64 multiply-adds on a 16-byte
// table entry per element made the rotation cost more than the HBM round trip it is there to save.
#pragma once

#include "zt_common.cuh"

namespace zt {

// table[r * half + i] = table_t[i * rows + r] = (cos, sin) of (pos + r) / theta^(2 i / head_dim)
__global__ void __launch_bounds__(256) rope_table_kernel(float2 *__restrict__ table, float2 *__restrict__ table_t, int rows,
                                                         int half, int pos, double theta) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)rows * half) return;
    const int r = (int)(idx / half), i = (int)(idx - (long long)r * half);
    const double exponent = (double)(2 * i) / (double)(2 * half);
    const double angle = (double)(pos + r) / pow(theta, exponent);
    double s, c;
    sincos(angle, &s, &c);
    const float2 cs = make_float2((float)c, (float)s);
    table[idx] = cs;
    table_t[(long long)i * rows + r] = cs;
}

// One element of a rotated row: `mine` at index w of its head, `other` its partner (w +- half).
// Forward: lo' = lo c - hi s, hi' = hi c + lo s.  Transpose: lo' = lo c + hi s, hi' = hi c - lo s.
__device__ __forceinline__ float rope_elem(float mine, float other, float2 cs, bool upper, bool transpose) {
    const float s = (upper != transpose) ? cs.y : -cs.y;
    return fmaf(mine, cs.x, other * s);
}

// out = R x (transpose = 0) or R^T x (transpose = 1) for x [batch][rows][width]; may run in place: a thread
// owns both elements of a pair.  grid over batch * rows * width / 2 pairs.
__global__ void __launch_bounds__(256) rope_apply_kernel(const float *x, float *out, const float2 *__restrict__ table,
                                                         int batch, int rows, int width, int head_dim, int transpose) {
    const int half = head_dim / 2;
    const long long pairs_per_row = width / 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)batch * rows * pairs_per_row) return;
    const long long row = idx / pairs_per_row;  // batch * rows + r
    const int pr = (int)(idx - row * pairs_per_row);
    const int r = (int)(row % rows);
    const int head = pr / half, i = pr - head * half;
    const long long lo_at = row * width + (long long)head * head_dim + i;
    const float lo = x[lo_at], hi = x[lo_at + half];
    const float2 cs = __ldg(table + (long long)r * half + i);
    out[lo_at] = rope_elem(lo, hi, cs, false, transpose != 0);
    out[lo_at + half] = rope_elem(hi, lo, cs, true, transpose != 0);
}

inline int launch_rope_table(float2 *table, float2 *table_t, int rows, int head_dim, int pos, double theta,
                             cudaStream_t stream) {
    const long long n = (long long)rows * (head_dim / 2);
    return ZT_LAUNCH("rope_table_kernel", stream,
                     (rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(table, table_t, rows, head_dim / 2, pos, theta)));
}
inline int launch_rope_apply(const float *x, float *out, const float2 *table, int batch, int rows, int width, int head_dim,
                             bool transpose, cudaStream_t stream) {
    const long long n = (long long)batch * rows * (width / 2);
    return ZT_LAUNCH("rope_apply_kernel", stream,
                     (rope_apply_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, out, table, batch, rows, width,
                                                                                         head_dim, transpose ? 1 : 0)));
}

}  // namespace zt
