// SIMT (CUDA-core) attention kernels: forward, and the two-kernel backward.
//
// These serve every shape the C ABI admits -- any even head_dim in [32, 256], any
// T, any q_offset/n_keys -- and are what the tensor-core kernels fall back to for
// shapes they are not specialised for (odd widths, ragged tails through the
// reference ABI).  They are flash-style: scores are never written to memory, the
// softmax is carried online in f32 with the running maximum in the log2 domain.
//
// Common geometry: a block is 256 threads and works on a 32 x 32 tile of
// (query rows) x (keys).  Thread `tid` owns tile row  r = tid / 8  and the four
// tile columns  c = tid % 8 + 8 i;  for the row-times-matrix products that follow
// it owns the same row and output columns  j = tid % 8 + 8 i  of the head.  The
// eight threads of a row are consecutive lanes of one warp, so a row's
// reductions are three xor-shuffles and its hand-off of P needs only __syncwarp.
//
// What they must match: attention.forward (src/attention.zig:60-153) and
// autograd.attentionBackward (src/autograd.zig:636-842) of the reference.
#pragma once

#include "zt_common.cuh"

namespace zt {

constexpr int kTile = 32;          // rows and keys per tile
constexpr int kSimtThreads = 256;  // 8 warps
constexpr int kMaxColsPerThread = 32;  // head_dim 256 / 8

struct SimtFwdParams {
    const float *q, *k, *v;
    float *out, *lse;  // lse may be null
    int T, n_heads, n_kv_heads, dim, q_offset, n_keys;
    long long q_batch_stride, kv_batch_stride, lse_batch_stride;  // in elements
    float scale_log2;  // log2(e) / sqrt(dim)
    // Decode form (T == 1): per-sequence key counts on the device.  When set, sequence b
    // uses n_keys = n_keys_dev[b], q_offset = n_keys - 1, and `n_keys` above is the cache
    // capacity; a count outside [1, capacity] yields a NaN row and bumps *bad_count.
    const int *n_keys_dev;
    int *bad_count;
};

struct SimtBwdParams {
    const float *q, *k, *v, *dout, *lse, *delta;
    float *dq, *dk, *dv;
    int T, n_heads, n_kv_heads, dim;
    long long q_batch_stride, kv_batch_stride, lse_batch_stride;
    float scale, scale_log2;
};

// Rows [row0, row0 + 32) of a [rows, ld_g] matrix, columns [col0, col0 + dim),
// into shared memory with leading dimension dim + 1 (odd, so that the 32 rows
// start in 32 different banks).  Rows past `rows - 1` repeat the last valid row:
// their products are computed and then discarded by the masks, which keeps every
// shared-memory read initialised.
__device__ __forceinline__ void load_tile(float *dst, const float *src, int row0, int rows,
                                          long long ld_g, int col0, int dim) {
    const int ld = dim + 1;
    for (int idx = threadIdx.x; idx < kTile * dim; idx += kSimtThreads) {
        const int rr = idx / dim, dd = idx - rr * dim;
        int gr = row0 + rr;
        gr = gr < rows ? gr : rows - 1;
        dst[rr * ld + dd] = __ldg(src + (long long)gr * ld_g + col0 + dd);
    }
}

// acc[i] = A[r, :] . B[c0 + 8 i, :]
__device__ __forceinline__ void dots4(const float *A, const float *B, int dim, int r, int c0,
                                      float acc[4]) {
    const int ld = dim + 1;
    const float *a = A + r * ld;
    const float *b0 = B + c0 * ld, *b1 = b0 + 8 * ld, *b2 = b0 + 16 * ld, *b3 = b0 + 24 * ld;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 4
    for (int d = 0; d < dim; ++d) {
        const float av = a[d];
        s0 = fmaf(av, b0[d], s0);
        s1 = fmaf(av, b1[d], s1);
        s2 = fmaf(av, b2[d], s2);
        s3 = fmaf(av, b3[d], s3);
    }
    acc[0] = s0, acc[1] = s1, acc[2] = s2, acc[3] = s3;
}

__device__ __forceinline__ float row_max8(float x) {
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 4));
    return x;
}
__device__ __forceinline__ float row_sum8(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    x += __shfl_xor_sync(0xffffffffu, x, 4);
    return x;
}

// ---------------------------------------------------------------------------
// Forward.  grid (ceil(T / 32), n_heads, batch).
// Key j is visible to query row t iff j <= q_offset + t and j < n_keys
// (src/cuda/attn_kernels.cu:276-321 for the semantics of the two arguments).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kSimtThreads) attn_fwd_simt(const SimtFwdParams p) {
    extern __shared__ float smem[];
    const int dim = p.dim, ld = dim + 1;
    float *sQ = smem, *sK = sQ + kTile * ld, *sV = sK + kTile * ld, *sP = sV + kTile * ld;
    const int b = blockIdx.z, h = blockIdx.y, t0 = blockIdx.x * kTile;
    const int kvh = h / (p.n_heads / p.n_kv_heads);
    const int r = threadIdx.x >> 3, cg = threadIdx.x & 7;
    const long long qld = (long long)p.n_heads * dim, kld = (long long)p.n_kv_heads * dim;
    const float *q = p.q + b * p.q_batch_stride;
    const float *k = p.k + b * p.kv_batch_stride;
    const float *v = p.v + b * p.kv_batch_stride;

    int n_keys = p.n_keys, q_offset = p.q_offset;
    if (p.n_keys_dev) {
        const int nk = p.n_keys_dev[b];
        if (nk < 1 || nk > p.n_keys) {
            float *orow = p.out + b * p.q_batch_stride + h * dim;
            for (int j = threadIdx.x; j < dim; j += kSimtThreads) orow[j] = __int_as_float(0x7fc00000);
            if (threadIdx.x == 0) {
                if (p.lse) p.lse[b * p.lse_batch_stride + h] = __int_as_float(0x7fc00000);
                if (h == 0 && p.bad_count) atomicAdd(p.bad_count, 1);
            }
            return;
        }
        n_keys = nk, q_offset = nk - 1;
    }

    load_tile(sQ, q, t0, p.T, qld, h * dim, dim);

    const int t = t0 + r;
    const int pos = q_offset + t;  // absolute position of this thread's query row
    int t_last = t0 + kTile < p.T ? t0 + kTile : p.T;
    int last_key = q_offset + t_last;  // exclusive bound on visible keys for the tile
    last_key = last_key < n_keys ? last_key : n_keys;

    float m = -INFINITY, l = 0.f;
    float o[kMaxColsPerThread];
#pragma unroll
    for (int i = 0; i < kMaxColsPerThread; ++i) o[i] = 0.f;

    for (int s0 = 0; s0 < last_key; s0 += kTile) {
        __syncthreads();  // previous tile's readers are done (also orders the Q load)
        load_tile(sK, k, s0, n_keys, kld, kvh * dim, dim);
        load_tile(sV, v, s0, n_keys, kld, kvh * dim, dim);
        __syncthreads();

        float s[4];
        dots4(sQ, sK, dim, r, cg, s);
        float tmax = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = s0 + cg + 8 * i;
            s[i] = ((key <= pos || ZT_DEFECT(1)) && key < n_keys) ? s[i] * p.scale_log2 : -INFINITY;
            tmax = fmaxf(tmax, s[i]);
        }
        tmax = row_max8(tmax);
        const float m_new = fmaxf(m, tmax);
        // A row with nothing visible yet keeps m = -inf; exp2(-inf - -inf) is NaN, so
        // both factors are forced to zero in that case.
        const float corr = (m_new == -INFINITY) ? 0.f : ((ZT_DEFECT(3) && m != -INFINITY) ? 1.f : ex2(m - m_new));
        float psum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float pe = (s[i] == -INFINITY) ? 0.f : ex2(s[i] - m_new);
            sP[r * (kTile + 1) + cg + 8 * i] = pe;
            psum += pe;
        }
        psum = row_sum8(psum);
        l = l * corr + psum;
        m = m_new;
        __syncwarp();  // this row's P is written and read by lanes of one warp
        const float *pr = sP + r * (kTile + 1);
#pragma unroll
        for (int i = 0; i < kMaxColsPerThread; ++i) {
            const int j = cg + 8 * i;
            if (j < dim) {
                float acc = o[i] * corr;
#pragma unroll 8
                for (int c = 0; c < kTile; ++c) acc = fmaf(pr[c], sV[c * ld + j], acc);
                o[i] = acc;
            }
        }
        __syncwarp();
    }

    if (t < p.T) {
        const float inv = 1.f / l;
        float *orow = p.out + b * p.q_batch_stride + (long long)t * qld + h * dim;
#pragma unroll
        for (int i = 0; i < kMaxColsPerThread; ++i) {
            const int j = cg + 8 * i;
            if (j < dim) orow[j] = o[i] * inv;
        }
        if (p.lse && cg == 0)
            p.lse[b * p.lse_batch_stride + (long long)t * p.n_heads + h] = (m + log2f(l)) * kLn2;
    }
}

// ---------------------------------------------------------------------------
// delta[b, t, h] = sum_j dout[b, t, h, j] * out[b, t, h, j]   (one warp per (t, h)).
// This is the softmax Jacobian's sum_s p[s] dp[s] (src/autograd.zig:774-797),
// obtained from the forward's output instead of a second pass over the keys.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_delta_kernel(const float *__restrict__ out,
                                                         const float *__restrict__ dout,
                                                         float *__restrict__ delta,
                                                         float *__restrict__ rnorm,
                                                         long long n_rows, int dim) {
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const float *o = out + row * dim, *g = dout + row * dim;
    float acc = 0.f, sq = 0.f;
    for (int j = lane; j < dim; j += 32) {
        const float gj = __ldg(g + j);
        acc = fmaf(__ldg(o + j), gj, acc);
        sq = fmaf(gj, gj, sq);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, off);
        sq += __shfl_xor_sync(0xffffffffu, sq, off);
    }
    if (lane == 0) {
        delta[row] = acc;
        // |dout row| for the tensor-core backward's per-row scale of dS (null when nobody wants it)
        if (rnorm) rnorm[row] = sqrtf(sq);
    }
}

// Fill a float buffer (row_den of the reference ABI is documented as 1).
__global__ void fill_kernel(float *dst, long long n, float value) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = value;
}

// ---------------------------------------------------------------------------
// Backward, query-outer: dq.  grid (ceil(T / 32), n_heads, batch).
//   p  = exp(score - lse),  dp = dout . v,  ds = p (dp - delta),  dq = scale * ds K
// (src/autograd.zig:799-820).  Assigns dq.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kSimtThreads) attn_bwd_dq_simt(const SimtBwdParams p) {
    extern __shared__ float smem[];
    const int dim = p.dim, ld = dim + 1;
    float *sQ = smem, *sG = sQ + kTile * ld, *sK = sG + kTile * ld, *sV = sK + kTile * ld,
          *sS = sV + kTile * ld;
    const int b = blockIdx.z, h = blockIdx.y, t0 = blockIdx.x * kTile;
    const int kvh = h / (p.n_heads / p.n_kv_heads);
    const int r = threadIdx.x >> 3, cg = threadIdx.x & 7;
    const long long qld = (long long)p.n_heads * dim, kld = (long long)p.n_kv_heads * dim;
    const float *q = p.q + b * p.q_batch_stride, *g = p.dout + b * p.q_batch_stride;
    const float *k = p.k + b * p.kv_batch_stride, *v = p.v + b * p.kv_batch_stride;

    load_tile(sQ, q, t0, p.T, qld, h * dim, dim);
    load_tile(sG, g, t0, p.T, qld, h * dim, dim);

    const int t = t0 + r;
    const int tc = t < p.T ? t : p.T - 1;
    const float lse2 = p.lse[b * p.lse_batch_stride + (long long)tc * p.n_heads + h] * kLog2e;
    const float del = ZT_DEFECT(13) ? 0.f : p.delta[b * p.lse_batch_stride + (long long)tc * p.n_heads + h];
    const int last_key = t0 + kTile < p.T ? t0 + kTile : p.T;

    float acc[kMaxColsPerThread];
#pragma unroll
    for (int i = 0; i < kMaxColsPerThread; ++i) acc[i] = 0.f;

    for (int s0 = 0; s0 < last_key; s0 += kTile) {
        __syncthreads();
        load_tile(sK, k, s0, p.T, kld, kvh * dim, dim);
        load_tile(sV, v, s0, p.T, kld, kvh * dim, dim);
        __syncthreads();
        float s[4], dp[4];
        dots4(sQ, sK, dim, r, cg, s);
        dots4(sG, sV, dim, r, cg, dp);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = s0 + cg + 8 * i;
            const float pe = ((key <= t || ZT_DEFECT(11)) && key < p.T) ? ex2(s[i] * p.scale_log2 - lse2) : 0.f;
            sS[r * (kTile + 1) + cg + 8 * i] = pe * (dp[i] - del);
        }
        __syncwarp();
        const float *sr = sS + r * (kTile + 1);
#pragma unroll
        for (int i = 0; i < kMaxColsPerThread; ++i) {
            const int j = cg + 8 * i;
            if (j < dim) {
                float a = acc[i];
#pragma unroll 8
                for (int c = 0; c < kTile; ++c) a = fmaf(sr[c], sK[c * ld + j], a);
                acc[i] = a;
            }
        }
        __syncwarp();
    }
    if (t < p.T) {
        float *row = p.dq + b * p.q_batch_stride + (long long)t * qld + h * dim;
#pragma unroll
        for (int i = 0; i < kMaxColsPerThread; ++i) {
            const int j = cg + 8 * i;
            if (j < dim) row[j] = acc[i] * p.scale;
        }
    }
}

// ---------------------------------------------------------------------------
// Backward, key-outer: dk and dv.  grid (ceil(T / 32), n_kv_heads, batch).
// One block owns 32 keys of one KV head and walks every query head of that
// head's group and every query tile at or after its keys, so dk/dv are complete
// when it ends: assigned, never accumulated across blocks, no atomics
// (src/autograd.zig:821-838 gives the sums; the reference's own device kernel
// makes the same ownership choice, src/cuda/attn_kernels.cu:557-634).
// Thread owns key  kk = tid / 8  and query rows  rr = tid % 8 + 8 i  of the tile.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kSimtThreads) attn_bwd_dkdv_simt(const SimtBwdParams p) {
    extern __shared__ float smem[];
    const int dim = p.dim, ld = dim + 1;
    float *sK = smem, *sV = sK + kTile * ld, *sQ = sV + kTile * ld, *sG = sQ + kTile * ld,
          *sP = sG + kTile * ld, *sS = sP + kTile * (kTile + 1), *sL = sS + kTile * (kTile + 1),
          *sD = sL + kTile;
    const int b = blockIdx.z, kvh = blockIdx.y, s0 = blockIdx.x * kTile;
    const int group = p.n_heads / p.n_kv_heads;
    const int kk = threadIdx.x >> 3, cg = threadIdx.x & 7;
    const long long qld = (long long)p.n_heads * dim, kld = (long long)p.n_kv_heads * dim;
    const float *q = p.q + b * p.q_batch_stride, *g = p.dout + b * p.q_batch_stride;
    const float *k = p.k + b * p.kv_batch_stride, *v = p.v + b * p.kv_batch_stride;
    const float *lse = p.lse + b * p.lse_batch_stride, *delta = p.delta + b * p.lse_batch_stride;

    load_tile(sK, k, s0, p.T, kld, kvh * dim, dim);
    load_tile(sV, v, s0, p.T, kld, kvh * dim, dim);
    const int key = s0 + kk;

    float dk[kMaxColsPerThread], dv[kMaxColsPerThread];
#pragma unroll
    for (int i = 0; i < kMaxColsPerThread; ++i) dk[i] = 0.f, dv[i] = 0.f;

    for (int hh = 0; hh < group; ++hh) {
        const int h = kvh * group + hh;
        for (int t0 = s0; t0 < p.T; t0 += kTile) {  // s0 is a multiple of 32, so tiles align
            __syncthreads();
            load_tile(sQ, q, t0, p.T, qld, h * dim, dim);
            load_tile(sG, g, t0, p.T, qld, h * dim, dim);
            if (threadIdx.x < kTile) {
                int t = t0 + threadIdx.x;
                t = t < p.T ? t : p.T - 1;
                sL[threadIdx.x] = lse[(long long)t * p.n_heads + h] * kLog2e;
                sD[threadIdx.x] = ZT_DEFECT(13) ? 0.f : delta[(long long)t * p.n_heads + h];
            }
            __syncthreads();
            float st[4], dpt[4];
            dots4(sK, sQ, dim, kk, cg, st);
            dots4(sV, sG, dim, kk, cg, dpt);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int rr = cg + 8 * i, t = t0 + rr;
                const float pe =
                    ((key <= t || ZT_DEFECT(11)) && t < p.T && key < p.T) ? ex2(st[i] * p.scale_log2 - sL[rr]) : 0.f;
                sP[kk * (kTile + 1) + rr] = pe;
                sS[kk * (kTile + 1) + rr] = pe * (dpt[i] - sD[rr]);
            }
            __syncwarp();
            const float *pr = sP + kk * (kTile + 1), *sr = sS + kk * (kTile + 1);
#pragma unroll
            for (int i = 0; i < kMaxColsPerThread; ++i) {
                const int j = cg + 8 * i;
                if (j < dim) {
                    float av = dv[i], ak = dk[i];
#pragma unroll 8
                    for (int c = 0; c < kTile; ++c) {
                        av = fmaf(pr[c], sG[c * ld + j], av);
                        ak = fmaf(sr[c], sQ[c * ld + j], ak);
                    }
                    dv[i] = av, dk[i] = ak;
                }
            }
            __syncwarp();
        }
    }
    if (key < p.T) {
        float *dkr = p.dk + b * p.kv_batch_stride + (long long)key * kld + kvh * dim;
        float *dvr = p.dv + b * p.kv_batch_stride + (long long)key * kld + kvh * dim;
#pragma unroll
        for (int i = 0; i < kMaxColsPerThread; ++i) {
            const int j = cg + 8 * i;
            if (j < dim) {
                dkr[j] = dk[i] * p.scale;
                dvr[j] = dv[i];
            }
        }
    }
}

inline size_t simt_fwd_smem(int dim) {
    return (size_t)(3 * kTile * (dim + 1) + kTile * (kTile + 1)) * sizeof(float);
}
inline size_t simt_bwd_dq_smem(int dim) {
    return (size_t)(4 * kTile * (dim + 1) + kTile * (kTile + 1)) * sizeof(float);
}
inline size_t simt_bwd_dkdv_smem(int dim) {
    return (size_t)(4 * kTile * (dim + 1) + 2 * kTile * (kTile + 1) + 2 * kTile) * sizeof(float);
}

// ---- host launchers ---------------------------------------------------------

inline int launch_fwd_simt(const SimtFwdParams &p, int batch, cudaStream_t stream) {
    const size_t smem = simt_fwd_smem(p.dim);
    if (optin_smem((const void *)attn_fwd_simt, smem)) return 1;
    dim3 grid((unsigned)((p.T + kTile - 1) / kTile), (unsigned)p.n_heads, (unsigned)batch);
    g_last_path = "simt";
    return ZT_LAUNCH("attn_fwd_simt", stream, attn_fwd_simt<<<grid, kSimtThreads, smem, stream>>>(p));
}

inline int launch_delta(const float *out, const float *dout, float *delta, float *rnorm, long long n_rows,
                        int dim, cudaStream_t stream) {
    const long long blocks = (n_rows + 7) / 8;
    return ZT_LAUNCH("attn_delta_kernel", stream,
                     attn_delta_kernel<<<(unsigned)blocks, 256, 0, stream>>>(out, dout, delta, rnorm, n_rows, dim));
}

inline int launch_bwd_simt(const SimtBwdParams &p, int batch, cudaStream_t stream) {
    const size_t smem_a = simt_bwd_dq_smem(p.dim), smem_b = simt_bwd_dkdv_smem(p.dim);
    if (optin_smem((const void *)attn_bwd_dq_simt, smem_a)) return 1;
    if (optin_smem((const void *)attn_bwd_dkdv_simt, smem_b)) return 1;
    const unsigned tiles = (unsigned)((p.T + kTile - 1) / kTile);
    const dim3 grid_a(tiles, (unsigned)p.n_heads, (unsigned)batch);
    const dim3 grid_b(tiles, (unsigned)p.n_kv_heads, (unsigned)batch);
    if (ZT_LAUNCH("attn_bwd_dq_simt", stream,
                  attn_bwd_dq_simt<<<grid_a, kSimtThreads, smem_a, stream>>>(p)))
        return 1;
    g_last_path = "simt";
    return ZT_LAUNCH("attn_bwd_dkdv_simt", stream,
                     attn_bwd_dkdv_simt<<<grid_b, kSimtThreads, smem_b, stream>>>(p));
}

}  // namespace zt
