// KV-cache decode attention: one new query row per sequence over that sequence's
// filled cache prefix (decode.attnStep, src/decode.zig:326-392, for a whole batch).
//
// The work is a stream over the cache -- every K and V row of every KV head is
// read exactly once and used by all query heads of its group -- so the kernel is
// bound by HBM bandwidth and everything here is arranged around that:
//   * split-K over the context: block (chunk, kv head, sequence) reads a fixed-size
//     chunk of keys, so ragged lengths balance by themselves and a short batch
//     still fills the machine;
//   * a K/V row is read by a group of LPK lanes as 128-bit, fully coalesced,
//     no-L1-allocate loads, several keys in flight per lane before any is used;
//   * a row is read once and dotted against every query head of the group held
//     in registers; lane-group shuffles finish each dot;
//   * online softmax in the log2 domain per lane group, merged across lane
//     groups by shuffles, across warps through shared memory, and across chunks
//     by a second small kernel (log-sum-exp combine).
//
// Algorithmic bytes per sequence step: n_keys * 2 * n_kv_heads * dim * 4 (K and V
// once each) plus q and out.
#pragma once

#include "zt_common.cuh"

namespace zt {

constexpr int kDecodeThreads = 256;
constexpr int kDecodeHeaderBytes = 256;  // workspace header: bad-sequence counter

struct DecodeParams {
    const float *q, *k_cache, *v_cache;
    const int *n_keys;  // per sequence; when null, n_keys_all applies to every sequence
    int n_keys_all;
    float *out, *lse;  // lse may be null
    float2 *part_ml;   // [batch, n_heads, max_chunks]  (running max (log2), denominator)
    float *part_acc;   // [batch, n_heads, max_chunks, dim]
    int *bad_count;    // in the workspace header
    int batch, n_ctx, n_heads, n_kv_heads, dim, chunk, max_chunks, n_sub;
    long long cache_batch_stride;  // elements between two sequences' caches
    float scale_log2;
};

__device__ __forceinline__ float4 ldg_stream(const float *ptr) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(ptr));
    return v;
}

template <int NCH, int GP>
struct DecodeCfg {
    // Keys in flight per lane group, and blocks per SM, from a register estimate:
    // K and V staging (8 floats per chunk per key) + q and accumulators (8 per chunk per head).
    static constexpr int kUnroll = (NCH >= 3 || NCH * GP >= 8) ? 2 : 4;
    static constexpr int kRegEstimate = kUnroll * NCH * 8 + GP * NCH * 8 + 28;
    static constexpr int kMinBlocks = kRegEstimate > 124 ? 1 : 2;
};

// LPK lanes share one key row; each lane holds NCH float4 chunks of it (chunk index
// li + LPK * c); GP query heads are processed per pass.
template <int LPK, int NCH, int GP>
__global__ void __launch_bounds__(kDecodeThreads, DecodeCfg<NCH, GP>::kMinBlocks)
    decode_splitk_kernel(const DecodeParams p) {
    constexpr int U = DecodeCfg<NCH, GP>::kUnroll;
    constexpr int GPW = 32 / LPK;                          // lane groups per warp
    constexpr int NG = (kDecodeThreads / 32) * GPW;        // lane groups per block
    extern __shared__ float smem[];

    const int b = blockIdx.z;
    const int nk = p.n_keys ? p.n_keys[b] : p.n_keys_all;
    if (nk < 1 || nk > p.n_ctx) return;  // reported by the combine kernel
    const int c0 = blockIdx.x * p.chunk;
    if (c0 >= nk) return;
    const int c1 = (c0 + p.chunk < nk) ? c0 + p.chunk : nk;
    const int group = p.n_heads / p.n_kv_heads;
    const int g = blockIdx.y / p.n_sub, sub = blockIdx.y - g * p.n_sub;
    const int h0 = g * group + sub * GP;
    const int nh = (group - sub * GP) < GP ? (group - sub * GP) : GP;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int li = lane % LPK;
    const int gi = warp * GPW + lane / LPK;
    const int dim = p.dim, n_chunks4 = dim >> 2;
    const long long kvw = (long long)p.n_kv_heads * dim;

    // This lane's slices of the group's query rows, pre-multiplied by log2(e)/sqrt(dim).
    float4 qr[GP][NCH];
#pragma unroll
    for (int hh = 0; hh < GP; ++hh)
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int ch = li + LPK * c;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (hh < nh && ch < n_chunks4) {
                x = *reinterpret_cast<const float4 *>(p.q + ((long long)b * p.n_heads + h0 + hh) * dim +
                                                      ch * 4);
                x.x *= p.scale_log2, x.y *= p.scale_log2, x.z *= p.scale_log2, x.w *= p.scale_log2;
            }
            qr[hh][c] = x;
        }

    float m[GP], l[GP];
    float4 acc[GP][NCH];
#pragma unroll
    for (int hh = 0; hh < GP; ++hh) {
        m[hh] = -INFINITY, l[hh] = 0.f;
#pragma unroll
        for (int c = 0; c < NCH; ++c) acc[hh][c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    const float *kb = p.k_cache + b * p.cache_batch_stride + (long long)g * dim;
    const float *vb = p.v_cache + b * p.cache_batch_stride + (long long)g * dim;

    // The trip count is the same for every lane of the block (the shuffles below name the
    // whole warp); a lane group whose keys run out early carries -inf scores instead.
    for (int base = c0; base < c1; base += NG * U) {
        const int s = base + gi;
        float4 kf[U][NCH], vf[U][NCH];
        // all loads of this step are issued before any is consumed
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int key = s + u * NG;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int ch = li + LPK * c;
                if (key < c1 && ch < n_chunks4) {
                    kf[u][c] = ldg_stream(kb + (long long)key * kvw + ch * 4);
                    vf[u][c] = ldg_stream(vb + (long long)key * kvw + ch * 4);
                } else {
                    kf[u][c] = make_float4(0.f, 0.f, 0.f, 0.f);
                    vf[u][c] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
        float sc[U][GP];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int hh = 0; hh < GP; ++hh) {
                float d = 0.f;
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    d = fmaf(kf[u][c].x, qr[hh][c].x, d);
                    d = fmaf(kf[u][c].y, qr[hh][c].y, d);
                    d = fmaf(kf[u][c].z, qr[hh][c].z, d);
                    d = fmaf(kf[u][c].w, qr[hh][c].w, d);
                }
#pragma unroll
                for (int off = LPK / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
                sc[u][hh] = (s + u * NG < c1) ? d : -INFINITY;
            }
#pragma unroll
        for (int hh = 0; hh < GP; ++hh) {
            float mx = m[hh];
#pragma unroll
            for (int u = 0; u < U; ++u) mx = fmaxf(mx, sc[u][hh]);
            // With no real key so far mx is -inf; subtracting 0 instead keeps every
            // exponent at -inf (factor 0) rather than -inf - -inf (NaN).
            const float mxs = (mx == -INFINITY) ? 0.f : mx;
            const float corr = ex2(m[hh] - mxs);
            m[hh] = mx;
            float ls = l[hh] * corr;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                acc[hh][c].x *= corr, acc[hh][c].y *= corr, acc[hh][c].z *= corr, acc[hh][c].w *= corr;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float pe = ex2(sc[u][hh] - mxs);  // exp2(-inf) = 0 for absent keys
                ls += pe;
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    acc[hh][c].x = fmaf(pe, vf[u][c].x, acc[hh][c].x);
                    acc[hh][c].y = fmaf(pe, vf[u][c].y, acc[hh][c].y);
                    acc[hh][c].z = fmaf(pe, vf[u][c].z, acc[hh][c].z);
                    acc[hh][c].w = fmaf(pe, vf[u][c].w, acc[hh][c].w);
                }
            }
            l[hh] = ls;
        }
    }

    // Merge the lane groups of a warp.  A group that saw no key has m = -inf, l = 0.
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
        for (int hh = 0; hh < GP; ++hh) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[hh], off);
            const float lo = __shfl_xor_sync(0xffffffffu, l[hh], off);
            const float mx = fmaxf(m[hh], mo);
            const float cs = (m[hh] == -INFINITY) ? 0.f : ex2(m[hh] - mx);
            const float co = (mo == -INFINITY) ? 0.f : ex2(mo - mx);
            l[hh] = l[hh] * cs + lo * co;
            m[hh] = mx;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                float4 o;
                o.x = __shfl_xor_sync(0xffffffffu, acc[hh][c].x, off);
                o.y = __shfl_xor_sync(0xffffffffu, acc[hh][c].y, off);
                o.z = __shfl_xor_sync(0xffffffffu, acc[hh][c].z, off);
                o.w = __shfl_xor_sync(0xffffffffu, acc[hh][c].w, off);
                acc[hh][c].x = acc[hh][c].x * cs + o.x * co;
                acc[hh][c].y = acc[hh][c].y * cs + o.y * co;
                acc[hh][c].z = acc[hh][c].z * cs + o.z * co;
                acc[hh][c].w = acc[hh][c].w * cs + o.w * co;
            }
        }
    }

    // Merge the warps through shared memory: [warp][head][dim + 4].
    constexpr int NW = kDecodeThreads / 32;
    const int rec = dim + 4;  // [0] max, [1] denominator, [4 ..] accumulators (16-byte aligned)
    if (lane < LPK) {
#pragma unroll
        for (int hh = 0; hh < GP; ++hh) {
            float *dst = smem + (warp * GP + hh) * rec;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int ch = li + LPK * c;
                if (ch < n_chunks4) *reinterpret_cast<float4 *>(dst + 4 + ch * 4) = acc[hh][c];
            }
            if (lane == 0) dst[0] = m[hh], dst[1] = l[hh];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nh * dim; idx += kDecodeThreads) {
        const int hh = idx / dim, j = idx - hh * dim;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) mx = fmaxf(mx, smem[(w * GP + hh) * rec]);
        float lsum = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float *src = smem + (w * GP + hh) * rec;
            const float cw = (src[0] == -INFINITY) ? 0.f : ex2(src[0] - mx);
            lsum = fmaf(src[1], cw, lsum);
            a = fmaf(src[4 + j], cw, a);
        }
        const long long slot = ((long long)b * p.n_heads + h0 + hh) * p.max_chunks + blockIdx.x;
        p.part_acc[slot * dim + j] = a;
        if (j == 0) p.part_ml[slot] = make_float2(mx, lsum);
    }
}

// Log-sum-exp combine of a sequence's chunks.  grid (n_heads, batch), block 128.
__global__ void __launch_bounds__(128) decode_combine_kernel(const DecodeParams p) {
    const int h = blockIdx.x, b = blockIdx.y;
    const int nk = p.n_keys ? p.n_keys[b] : p.n_keys_all;
    float *orow = p.out + ((long long)b * p.n_heads + h) * p.dim;
    if (nk < 1 || nk > p.n_ctx) {
        // decode.attnStep refuses an empty prefix (src/decode.zig:350); on the device the
        // refusal is a NaN row plus a count the host can read.
        for (int j = threadIdx.x; j < p.dim; j += blockDim.x) orow[j] = __int_as_float(0x7fc00000);
        if (threadIdx.x == 0) {
            if (p.lse) p.lse[(long long)b * p.n_heads + h] = __int_as_float(0x7fc00000);
            if (h == 0) atomicAdd(p.bad_count, 1);
        }
        return;
    }
    const int nchunks = (nk + p.chunk - 1) / p.chunk;
    const long long slot0 = ((long long)b * p.n_heads + h) * p.max_chunks;
    float mx = -INFINITY;
    for (int c = 0; c < nchunks; ++c) mx = fmaxf(mx, p.part_ml[slot0 + c].x);
    float lsum = 0.f;
    for (int c = 0; c < nchunks; ++c) {
        const float2 ml = p.part_ml[slot0 + c];
        lsum = fmaf(ml.y, ex2(ml.x - mx), lsum);
    }
    const float inv = 1.f / lsum;
    for (int j = threadIdx.x; j < p.dim; j += blockDim.x) {
        float a = 0.f;
        for (int c = 0; c < nchunks; ++c)
            a = fmaf(p.part_acc[(slot0 + c) * p.dim + j], ex2(p.part_ml[slot0 + c].x - mx), a);
        orow[j] = a * inv;
    }
    if (p.lse && threadIdx.x == 0)
        p.lse[(long long)b * p.n_heads + h] = (mx + log2f(lsum)) * kLn2;
}

// kv_cache.Layer.append for a batch (src/kv_cache.zig:88-95).  grid (batch), block 256.
__global__ void kv_append_kernel(float *k_cache, float *v_cache, int *n_keys, const float *k_new,
                                 const float *v_new, int *full_count, int n_ctx, int width) {
    const int b = blockIdx.x;
    const int len = n_keys[b];
    if (len < 0 || len >= n_ctx) {  // Error.Full: nothing is written, nothing advances
        if (threadIdx.x == 0 && full_count) atomicAdd(full_count, 1);
        return;
    }
    float *kd = k_cache + ((long long)b * n_ctx + len) * width;
    float *vd = v_cache + ((long long)b * n_ctx + len) * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        kd[j] = k_new[(long long)b * width + j];
        vd[j] = v_new[(long long)b * width + j];
    }
    __syncthreads();
    if (threadIdx.x == 0) n_keys[b] = len + 1;
}

// ---- host side ---------------------------------------------------------------

struct DecodePlan {
    int lpk, nch, gp, n_sub, chunk, max_chunks;
    size_t ml_bytes, acc_bytes, total_bytes;
};

// The split is a pure function of the shape and of the current device's SM count, so the
// workspace-size query and the launch agree (both made with the same device current).  The
// chunk is as large as keeps roughly four waves of blocks in flight (two blocks per SM),
// between 128 and 1024 keys.  Without a device (a size query on a machine with none) the
// count of a B200, 148, stands in.
inline DecodePlan decode_plan(int batch, int n_ctx, int n_heads, int n_kv_heads, int dim) {
    DecodePlan pl{};
    const int group = n_heads / n_kv_heads;
    pl.gp = group >= 3 ? 4 : group;
    pl.n_sub = (group + pl.gp - 1) / pl.gp;
    const int chunks4 = dim / 4;
    pl.lpk = chunks4 <= 8 ? 8 : 16;
    pl.nch = (chunks4 + pl.lpk - 1) / pl.lpk;
    const long long units = (long long)batch * n_kv_heads * pl.n_sub;
    const DeviceInfo *di = device_info();
    const long long target_blocks = 4LL * 2 * (di && di->sm_count > 0 ? di->sm_count : 148);
    long long want = (target_blocks + units - 1) / units;
    if (want < 1) want = 1;
    long long chunk = (n_ctx + want - 1) / want;
    chunk = (chunk + 63) / 64 * 64;
    if (chunk < 128) chunk = 128;
    if (chunk > 1024) chunk = 1024;
    pl.chunk = (int)chunk;
    pl.max_chunks = (n_ctx + pl.chunk - 1) / pl.chunk;
    pl.ml_bytes = (size_t)batch * n_heads * pl.max_chunks * sizeof(float2);
    pl.ml_bytes = (pl.ml_bytes + 255) / 256 * 256;
    pl.acc_bytes = (size_t)batch * n_heads * pl.max_chunks * dim * sizeof(float);
    pl.total_bytes = kDecodeHeaderBytes + pl.ml_bytes + pl.acc_bytes;
    return pl;
}

template <int LPK, int NCH, int GP>
inline int launch_decode_inst(const DecodeParams &p, cudaStream_t stream) {
    const size_t smem = (size_t)(kDecodeThreads / 32) * GP * (p.dim + 4) * sizeof(float);
    if (optin_smem((const void *)decode_splitk_kernel<LPK, NCH, GP>, smem)) return 1;
    dim3 grid((unsigned)p.max_chunks, (unsigned)(p.n_kv_heads * p.n_sub), (unsigned)p.batch);
    return ZT_LAUNCH("decode_splitk_kernel", stream,
                     (decode_splitk_kernel<LPK, NCH, GP><<<grid, kDecodeThreads, smem, stream>>>(p)));
}

template <int LPK, int NCH>
inline int launch_decode_gp(const DecodeParams &p, int gp, cudaStream_t stream) {
    switch (gp) {
        case 1: return launch_decode_inst<LPK, NCH, 1>(p, stream);
        case 2: return launch_decode_inst<LPK, NCH, 2>(p, stream);
        default: return launch_decode_inst<LPK, NCH, 4>(p, stream);
    }
}

// Split-K pass followed by the combine, both on `stream`.
inline int launch_decode(DecodeParams p, const DecodePlan &pl, void *workspace, cudaStream_t stream) {
    char *ws = static_cast<char *>(workspace);
    p.bad_count = reinterpret_cast<int *>(ws);
    p.part_ml = reinterpret_cast<float2 *>(ws + kDecodeHeaderBytes);
    p.part_acc = reinterpret_cast<float *>(ws + kDecodeHeaderBytes + pl.ml_bytes);
    p.chunk = pl.chunk, p.max_chunks = pl.max_chunks, p.n_sub = pl.n_sub;
    if (cudaMemsetAsync(ws, 0, kDecodeHeaderBytes, stream) != cudaSuccess) {
        cudaGetLastError();
        return refuse("could not clear the decode workspace header");
    }
    int rc;
    if (pl.lpk == 8) rc = launch_decode_gp<8, 1>(p, pl.gp, stream);
    else if (pl.nch == 1) rc = launch_decode_gp<16, 1>(p, pl.gp, stream);
    else if (pl.nch == 2) rc = launch_decode_gp<16, 2>(p, pl.gp, stream);
    else if (pl.nch == 3) rc = launch_decode_gp<16, 3>(p, pl.gp, stream);
    else rc = launch_decode_gp<16, 4>(p, pl.gp, stream);
    if (rc) return rc;
    g_last_path = "decode-splitk";
    const dim3 cgrid((unsigned)p.n_heads, (unsigned)p.batch);
    return ZT_LAUNCH("decode_combine_kernel", stream,
                     decode_combine_kernel<<<cgrid, 128, 0, stream>>>(p));
}

}  // namespace zt
