// Causal GQA attention backward on the Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
// What it computes: autograd.attentionBackward (src/autograd.zig:636-842) for a batch, from the
// forward's out (through delta = sum_j dout*out) and log-sum-exp:
//     P  = exp(S - lse),  dP = dO V^T,  dS = P (dP - delta)
//     dV = P^T dO,   dK = scale dS^T Q,   dQ = scale dS K
//
// Arithmetic.  A head_dim-128 backward needs Q, dO, K, V and P, dS as tensor-core operands at
// once; as f32 hi/lo pairs (8 bytes per element) they do not fit in shared memory plus TMEM.
// So the backward uses the same three-term split idea on 16-bit pieces instead of TF32 ones:
//     x * m = h + l,   h = f16(x m),  l = f16(x m - h),   a.b ~ (ha hb + ha lb + la hb) / (ma mb)
// with m a power of two per (sequence, KV group) that puts the block's largest |x| just under
// 2^15.  h + l carries 22 mantissa bits of x (what 3xTF32 carries is 21), products accumulate
// in f32 in TMEM, and each term is one kind::f16 MMA at twice the TF32 rate: half the operand
// bytes and half the tensor time of 3xTF32.  Elements more than 2^25 below their block's
// maximum lose relative (not absolute) precision; the parity tests bound the effect.
//
// Kernels:
//   bwd_absmax / bwd_split   per-(sequence, KV group) max |x| of q, k, v, dout; then the h and l
//                            planes of each tensor ([2][B][T][W] halves) in the workspace.  One
//                            launch of each for all tensors.
//   attn_bwd_dkdv_tc         one CTA per (128 keys, KV head, sequence): S^T = K Q^T and
//                            dP^T = V dO^T per 64-row query tile of every head of the group,
//                            P^T and dS^T written back to TMEM as packed halves,
//                            dV += P^T dO and dK += dS^T Q accumulated in TMEM for the whole walk:
//                            dk/dv are assigned by their one owner, no atomics.
//   attn_bwd_dq_tc           one CTA per (128 query rows, head, sequence): S = Q K^T, dP = dO V^T,
//                            dS, dQ += dS K over the causal key tiles of 64; dq assigned.
// Both kernels issue S (and dP) one or two tiles ahead into TMEM buffers of their own and spread
// the row work of a tile over four warp sets; see the comment above each.
// These two are the backward's first form: today's default folds dQ into the dK/dV kernel (tc_bwd_fused.cuh,
// which also holds launch_bwd_tc, the host side of both forms); they run when the two-kernel form is asked
// for, and for the call that also stores dq into peers' memory.  The pre-pass kernels and the walk (Walk)
// below serve both forms.
// Every wait is bounded (see tc_common.cuh); a wait that gives up raises g_tc_status.
#pragma once

#include <cuda_fp16.h>

#include "rope_kernels.cuh"
#include "tc_common.cuh"
#include "tc_fwd.cuh"
#include "zt_common.cuh"

namespace zt {
namespace tcb {

using namespace tc;

// ---- scaling --------------------------------------------------------------------------------------
// The power of two that moves a block's largest magnitude into [2^14, 2^15).  `bits` is the f32
// bit pattern of max |x| (non-negative, so it orders like an integer).
__host__ __device__ inline float block_mult(uint32_t bits) {
    const int ex = (int)((bits >> 23) & 0xff);  // biased exponent: |x| in [2^(ex-127), 2^(ex-126))
    if (ex == 0 || ex == 0xff) return 1.0f;      // zero/subnormal block, or inf/nan: leave alone
    int e = 14 - (ex - 127);                     // |x| * 2^e in [2^14, 2^15)
    if (e > 126) e = 126;
    if (e < -126) e = -126;
    uint32_t out = (uint32_t)(e + 127) << 23;
#if defined(__CUDA_ARCH__)
    return __uint_as_float(out);
#else
    float f;
    memcpy(&f, &out, 4);
    return f;
#endif
}

// The pre-pass over up to four tensors in one launch each: max |x| per (sequence, column group), then
// the 16-bit planes.  Tensor z is [batch][T][width] floats; its groups are `cols_per_group` columns wide.
struct PrepassTensor {
    const float *x;
    uint32_t *amax;   // [batch][width / cols_per_group] bit patterns of max |x|, zeroed by the caller
    __half *planes;   // [2][batch][T][width / src_head * dst_head]
    int width, cols_per_group;
    int src_head, dst_head;  // a head's columns in x and in the planes: 32 -> 64 pads each head with zeros
    const float2 *rope;      // null, or the (cos, sin) table [T][src_head / 2]: x is rotated on its way in
};

// Four consecutive elements of row r starting at column c of tensor t, rotated if the tensor asks for it.
// A head's halves are multiples of four wide, so the four partners are one float4 too.
__device__ __forceinline__ float4 prepass_load(const PrepassTensor &t, const float4 *row4, int r, int c) {
    const float4 v = __ldg(row4 + c / 4);
    if (t.rope == nullptr) return v;
    const int half = t.src_head / 2;
    const int w = c % t.src_head;
    const bool upper = w >= half;
    const float4 o = __ldg(row4 + (upper ? c - half : c + half) / 4);
    const float4 *cs = reinterpret_cast<const float4 *>(t.rope + (long long)r * half + (upper ? w - half : w));
    const float4 a = __ldg(cs), b = __ldg(cs + 1);  // four (cos, sin) pairs
    float4 out;
    out.x = rope_elem(v.x, o.x, make_float2(a.x, a.y), upper, false), out.y = rope_elem(v.y, o.y, make_float2(a.z, a.w), upper, false);
    out.z = rope_elem(v.z, o.z, make_float2(b.x, b.y), upper, false), out.w = rope_elem(v.w, o.w, make_float2(b.z, b.w), upper, false);
    return out;
}
struct PrepassArgs {
    PrepassTensor t[4];
    int n, batch, T;
};
constexpr int kPrepassRows = 32;      // rows of one sequence per absmax CTA
constexpr int kPrepassMaxGroups = 256;

// grid (ceil(T / kPrepassRows), batch, n tensors).  A thread keeps to its columns, so its group is fixed
// and the row loop is nothing but independent loads.
__global__ void __launch_bounds__(256) bwd_absmax_kernel(const PrepassArgs a) {
    __shared__ uint32_t gmax[kPrepassMaxGroups];
    const PrepassTensor t = a.t[blockIdx.z];
    const int b = blockIdx.y, r0 = blockIdx.x * kPrepassRows;
    const int w4 = t.width / 4, n_groups = t.width / t.cols_per_group;
    for (int i = threadIdx.x; i < n_groups; i += 256) gmax[i] = 0u;
    __syncthreads();
    const int r1 = min(r0 + kPrepassRows, a.T);
    const float4 *base = reinterpret_cast<const float4 *>(t.x + (long long)b * a.T * t.width);
    for (int c4 = threadIdx.x; c4 < w4; c4 += 256) {
        float m = 0.f;
#pragma unroll 8
        for (int r = r0; r < r1; ++r) {
            // (a tensor that will be rotated is measured unrotated: a rotated pair is at most sqrt(2) times its
            // larger element, and the scale leaves a factor of two below the f16 range)
            const float4 v = __ldg(base + (long long)r * w4 + c4);
            m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        atomicMax(&gmax[(c4 * 4) / t.cols_per_group], __float_as_uint(m));
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_groups; i += 256)
        if (gmax[i]) atomicMax(t.amax + b * n_groups + i, gmax[i]);
}

// x -> planes h = f16(x m), l = f16(x m - h).  grid (ceil(T width / 4 / 2048), batch, n tensors): a CTA
// converts 2048 consecutive float4 of one sequence, eight per thread.
constexpr int kSplitPerCta = 2048;
__global__ void __launch_bounds__(256) bwd_split_kernel(const PrepassArgs a) {
    const PrepassTensor t = a.t[blockIdx.z];
    const int b = blockIdx.y;
    const int n_groups = t.width / t.cols_per_group;
    if (t.src_head != t.dst_head) {
        // zero-padded heads: walk the planes' float4s, fetch the source's where there is one
        const int w4s = t.width / 4, w4d = t.width / t.src_head * t.dst_head / 4;
        const long long seq4d = (long long)a.T * w4d;
        const long long first = (long long)blockIdx.x * kSplitPerCta;
        if (first >= seq4d) return;
        const float4 *src = reinterpret_cast<const float4 *>(t.x) + (long long)b * a.T * w4s;
        uint2 *hp = reinterpret_cast<uint2 *>(t.planes) + b * seq4d;
        uint2 *lp = hp + (long long)a.batch * seq4d;
        const uint32_t *amax = t.amax + b * n_groups;
#pragma unroll
        for (int k = 0; k < kSplitPerCta / 256; ++k) {
            const long long i = first + k * 256 + threadIdx.x;
            if (i >= seq4d) break;
            const int r = (int)(i / w4d);
            const int cd = (int)(i - (long long)r * w4d) * 4;      // column in the planes
            const int head = cd / t.dst_head, within = cd - head * t.dst_head;
            uint2 hw = make_uint2(0u, 0u), lw = make_uint2(0u, 0u);
            if (within < t.src_head) {
                const int cs = head * t.src_head + within;          // column in x
                const float m = block_mult(amax[cs / t.cols_per_group]);
                const float4 v = prepass_load(t, src + (long long)r * w4s, r, cs);
                const float s[4] = {v.x * m, v.y * m, v.z * m, v.w * m};
                __half h[4], l[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    h[e] = __float2half_rn(s[e]);
                    l[e] = __float2half_rn(s[e] - __half2float(h[e]));
                }
                hw = *reinterpret_cast<const uint2 *>(h), lw = *reinterpret_cast<const uint2 *>(l);
            }
            hp[i] = hw, lp[i] = lw;
        }
        return;
    }
    const int w4 = t.width / 4;
    const long long seq4 = (long long)a.T * w4;  // float4 per sequence
    const long long first = (long long)blockIdx.x * kSplitPerCta;
    if (first >= seq4) return;
    const float4 *src = reinterpret_cast<const float4 *>(t.x) + b * seq4;
    uint2 *hp = reinterpret_cast<uint2 *>(t.planes) + b * seq4;
    uint2 *lp = hp + (long long)a.batch * seq4;
    const uint32_t *amax = t.amax + b * n_groups;
    const unsigned col0 = (unsigned)(first % w4);
#pragma unroll
    for (int k = 0; k < kSplitPerCta / 256; ++k) {
        const int o = k * 256 + threadIdx.x;
        const long long i = first + o;
        if (i >= seq4) break;
        const unsigned c4 = (col0 + (unsigned)o) % (unsigned)w4;
        const float m = block_mult(amax[(c4 * 4u) / (unsigned)t.cols_per_group]);
        const float4 v = t.rope ? prepass_load(t, src + (i - c4), (int)((i - c4) / w4), (int)(c4 * 4u)) : __ldg(src + i);
        const float s[4] = {v.x * m, v.y * m, v.z * m, v.w * m};
        __half h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            h[e] = __float2half_rn(s[e]);
            l[e] = __float2half_rn(s[e] - __half2float(h[e]));
        }
        hp[i] = *reinterpret_cast<const uint2 *>(h);
        lp[i] = *reinterpret_cast<const uint2 *>(l);
    }
}

// Both passes for the tensors in `a` (amax already zeroed).
inline int launch_prepass(const PrepassArgs &a, cudaStream_t stream) {
    int wmax = 0, wmax_src = 0;
    for (int i = 0; i < a.n; ++i) {
        const int wd = a.t[i].width / a.t[i].src_head * a.t[i].dst_head;
        wmax = wd > wmax ? wd : wmax;
        wmax_src = a.t[i].width > wmax_src ? a.t[i].width : wmax_src;
    }
    (void)wmax_src;
    const dim3 ga((unsigned)((a.T + kPrepassRows - 1) / kPrepassRows), (unsigned)a.batch, (unsigned)a.n);
    if (ZT_LAUNCH("bwd_absmax_kernel", stream, (bwd_absmax_kernel<<<ga, 256, 0, stream>>>(a)))) return 1;
    const long long seq4 = (long long)a.T * (wmax / 4);
    const dim3 gs((unsigned)((seq4 + kSplitPerCta - 1) / kSplitPerCta), (unsigned)a.batch, (unsigned)a.n);
    return ZT_LAUNCH("bwd_split_kernel", stream, (bwd_split_kernel<<<gs, 256, 0, stream>>>(a)));
}

// max over the rows s of |v[b, s, kv, :]| (Euclidean), per (sequence, KV head).  grid (ceil(T / 256), n_kv_heads,
// batch), 8 warps; a warp walks 32 rows of the block's 256 and keeps a running maximum, the block then makes ONE
// atomic: thousands of atomics on the same word serialise in L2 (a warp per row took 0.2 ms at the headline shape).
// vnmax holds f32 bit patterns (non-negative, so they order like integers), zeroed by the caller.
__global__ void __launch_bounds__(256) bwd_vnorm_kernel(const float *__restrict__ v, uint32_t *__restrict__ vnmax,
                                                        int T, int n_kv_heads, int dim) {
    __shared__ float wmax[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, kv = blockIdx.y, b = blockIdx.z;
    const int r0 = blockIdx.x * 256 + warp * 32;
    float best = 0.f;
    for (int r = r0; r < r0 + 32 && r < T; ++r) {
        const float *x = v + (((long long)b * T + r) * n_kv_heads + kv) * dim;
        float acc = 0.f;
        for (int j = lane; j < dim; j += 32) {
            const float e = __ldg(x + j);
            acc = fmaf(e, e, acc);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        best = fmaxf(best, acc);
    }
    if (lane == 0) wmax[warp] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = wmax[0];
        for (int i = 1; i < 8; ++i) m = fmaxf(m, wmax[i]);
        // (an Inf or NaN row: sqrt keeps it, and the scale built from it falls back to 1)
        atomicMax(vnmax + b * n_kv_heads + kv, __float_as_uint(sqrtf(m)));
    }
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}
// (a, b) -> packed h pair and packed l pair: one paired conversion each way instead of two single ones
__device__ __forceinline__ void split_pack(float a, float b, uint32_t &hw, uint32_t &lw) {
    const __half2 hh = __floats2half2_rn(a, b);
    const float2 back = __half22float2(hh);
    hw = *reinterpret_cast<const uint32_t *>(&hh);
    lw = pack_half2(a - back.x, b - back.y);
}

__device__ __forceinline__ void red_add_v4(float *addr, float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}


struct BwdParams {
    const float *lse, *delta;        // [B, T, H]
    const __half *k_planes, *v_planes;   // dkdv kernel: the hi planes of K and V are read straight into TMEM
    const __half *q_planes, *do_planes;  // dq kernel: Q, dO planes read straight into TMEM
    const uint32_t *amax_q, *amax_k, *amax_v, *amax_do;  // [B, Hkv] bit patterns of max |x|
    const float *rnorm;      // [B, T, H] Euclidean norm of each row of dout (bwd_rownorm_kernel)
    const uint32_t *vnmax;   // [B, Hkv] bit pattern of the largest Euclidean norm of a row of v
    uint32_t *dsmax;         // [B, Hkv] bit pattern of max |dS| (true units): written by the dQ kernel, read by dK/dV;
                             // for the fused kernel the same words hold the largest row norm of dout instead
    float *dq, *dk, *dv;
    PeerList dq_peers;       // dq is also stored here (same element index), see zt_common.cuh
    int batch, T, n_heads, n_kv_heads;
    int dim_out;     // the tensors' head_dim: the tile's D, or 32 under a tile padded to 64
    const float2 *rope_t;  // null, or the (cos, sin) table transposed, [dim_out / 2][T]: dq leaves as R^T of what was computed
    float scale, scale_log2;
    float p_scale;  // P is multiplied by this power of two before its 16-bit split
};

// The scale of dS.  dS = P (dP - delta) leaves the row threads as a pair of f16 pieces, so it must sit inside the
// f16 range, and as high in it as possible: a value 2^11 below the top of the range still has both pieces as
// normal numbers, one 2^26 below it has lost its low piece and half of the high one.  A single worst-case scale
// for a whole (sequence, KV group) -- |dP| <= head_dim max|dout| max|v| -- wastes the width of the head, the
// flatness of P and, worst, every outlier: with 0.1 % of dout and v a hundred times the rest, most of dq and a
// third of dk fell outside the tolerance.  So each kernel scales by what it can know:
//  * the dQ kernel owns whole rows of dS, so every query row has a scale of its own, from a bound that holds for
//    that row alone: |dP[t, s]| <= |dout[t]| |v[s]| (Euclidean norms), |delta[t]| is at most the largest |dP| of
//    its row and P <= 1, so |dS[t, s]| <= 2 |dout[t]| max_s |v[s]|.  Rows are independent of each other's
//    magnitude, and the scale only moves the accumulator of its own row, which is divided by it on the way out;
//  * the dK/dV kernel sums dS over query rows, so there one scale must serve a CTA.  It is calibrated, not
//    bounded: the dQ kernel, which runs first, records the largest |dS| it formed in each (sequence, KV group),
//    and the dK/dV kernel places that value an eighth below the top of the range (its own dS differs from the
//    dQ kernel's by rounding only).
// pow2_below_top(x, top): the power of two c with x c in [2^(top-1), 2^top); 1 when x is zero or not finite.
__device__ __forceinline__ float pow2_for(float x, int top) {
    if (!(x > 0.f) || !(x < 3.0e38f)) return 1.0f;
    int e;
    frexpf(x, &e);  // x = m 2^e, m in [0.5, 1)
    int k = top - e;
    k = k > 120 ? 120 : (k < -120 ? -120 : k);
    return __uint_as_float((uint32_t)(k + 127) << 23);
}

// The dK/dV kernel's walk over (query tile, head of the group), and where its TMEM accumulators
// are flushed to memory.
//
// The tensor core adds into its f32 accumulator with truncation, so every add made while the
// accumulator is already large shaves a little off it, always toward zero.  Two measures keep
// that below the f32 rounding noise of the answer:
//  * order: a key's terms grow as the query position falls (p ~ 1/t), so the walk starts at
//    the last query tile -- for each tile, all heads of the group -- and the accumulator stays
//    small until the end;
//  * flushes: the two query tiles that overlap the key tile carry the largest terms; they are
//    walked head by head, and after each head the accumulators are added to dk/dv in memory
//    (a rounded f32 add by the row threads) and restarted from zero, so no large partial sum
//    sits in TMEM while further terms arrive.  The tiles beyond them are flushed every
//    kFlushTiles query tiles for the same reason, which keeps the error flat in T.
//    (Before the periodic flushes, with a flush only per head: 12-26 of 524288 dk/dv elements
//    outside the tolerance at T = 4096; with them: none.)
// The bound on dS.  dS leaves the row threads as a pair of f16 pieces, so it must stay inside the f16 range;
// the scale c1 (launch_bwd_tc) is chosen from the worst case so that it does, with a factor of two to spare.
// Values are clamped to the bound all the same -- it costs two instructions and keeps an Inf or NaN that
// arrived in dout from spreading through the accumulators of a whole CTA -- and a clamp that fires is counted
// in g_tc_saturated (zt_attn_tc_saturated), which every test asserts to be zero.
constexpr float kDsBound = 65000.f;
constexpr int kFlushTiles = 8;  // query tiles of 64 rows between flushes (512 rows)
constexpr int kDiagTiles = 2;   // query tiles that overlap a 128-key tile
// An iterator: step `it` is (head hh of the group, query tile qi); `flush` says the accumulators are
// flushed after it, `fresh` that they restart from zero at it.  No divisions per step: every role of
// the kernel walks it in lockstep.
struct Walk {
    int group, qi0, nd, na;  // nd diagonal tiles (<= kDiagTiles); na steps over the tiles beyond them
    int it, hh, qi, cnt;     // cnt: steps since the last flush, while it < na
    bool flush, fresh;
    __device__ __forceinline__ Walk(int group_, int per_head, int qi0_, int n_q) : group(group_), qi0(qi0_) {
        nd = per_head < kDiagTiles ? per_head : kDiagTiles;
        na = (per_head - nd) * group;
        it = 0, hh = 0, cnt = 0;
        qi = na > 0 ? n_q - 1 : qi0 + nd - 1;
        fresh = true;
        set_flush();
    }
    __device__ __forceinline__ void set_flush() {
        flush = it < na ? (it == na - 1 || cnt + 1 == kFlushTiles * group) : (qi == qi0);
    }
    __device__ __forceinline__ void next() {
        fresh = flush;
        ++it;
        if (it < na) {
            // region A: tiles from the last one down, every head of the group on each
            cnt = (cnt + 1 == kFlushTiles * group) ? 0 : cnt + 1;
            if (++hh == group) hh = 0, --qi;
        } else if (it == na) {
            hh = 0, qi = qi0 + nd - 1;
        } else {
            // region B: the diagonal tiles, head by head
            if (qi == qi0) qi = qi0 + nd - 1, ++hh;
            else --qi;
        }
        set_flush();
    }
};

// One row of `words` packed-half words from global memory into TMEM columns [col, col + words).
template <int WORDS>
__device__ __forceinline__ void row_to_tmem(const __half *src, bool valid, uint32_t taddr) {
#pragma unroll 1
    for (int c = 0; c < WORDS; c += 32) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (valid) v = __ldg(reinterpret_cast<const uint4 *>(src) + (c + i) / 4);
            r[i] = v.x, r[i + 1] = v.y, r[i + 2] = v.z, r[i + 3] = v.w;
        }
        tmem_st32(taddr + c, r);
    }
}

// ---------------------------------------------------------------------------------------------------
// dK, dV.  grid (ceil(T / 128), n_kv_heads, batch), 576 threads: 16 row warps, a TMA warp, an MMA warp.
//
// Query tiles of 64 rows.  tcgen05.mma has a floor of about 50 clocks per instruction whatever its N
// (measured: M = 128, K = 16 takes 49-54 clocks at N = 32 and at N = 64, 64 at N = 128), so S^T and
// dP^T want the widest tile the 512 TMEM columns allow: 64 rows with S^T in two buffers and dP^T in
// one, beside the two D-column accumulators and V's hi plane.  The tensor core's order per step is
//     dK(it), dP^T(it+1), dV(it), S^T(it+2)
// so the row threads' exp of step it+1 runs under the MMAs of step it, and their dS part, which has
// to wait for dP^T(it+1), runs under dV(it) and S^T(it+2).  The row warps are four sets of four; a
// set handles 16 of the step's 64 query columns (one 16-deep MMA step of dV / dK), which keeps the
// serial part of the hand-off short.
// ---------------------------------------------------------------------------------------------------
constexpr int kKvRowWarps = 16;
constexpr int kKvThreads = (kKvRowWarps + 2) * 32;

struct KvShared {
    uint64_t full_q[4], full_g[4], free_q[4], free_g[4];  // a stage's Q planes and dO planes have lives of their own
    uint64_t k_full, a_ready, st_full[2], dp_full, p_full, ld_ready, flush_ready, flush_done;
    uint32_t tmem_base;
    volatile int abort;
    float lse2[2][64], dels[2][64];  // [buffer][query row of the tile]
};
__device__ __forceinline__ bool kwait(uint64_t *bar, uint32_t parity, KvShared *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void kgive_up(KvShared *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}
template <int D>
__host__ __device__ constexpr int kv_stages() { return D == 128 ? 2 : 4; }
template <int D>
__host__ __device__ constexpr size_t kv_smem_bytes() {
    return 3 * (size_t)(128 * D * 2) + kv_stages<D>() * 4 * (size_t)(64 * D * 2) + sizeof(KvShared) + 1024;
}

// 16 packed-half words of one row from global memory into TMEM columns [taddr, taddr + 16).
__device__ __forceinline__ void row_to_tmem16(const __half *src, bool valid, uint32_t taddr) {
    uint32_t r[16];
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (valid) v = __ldg(reinterpret_cast<const uint4 *>(src) + i / 4);
        r[i] = v.x, r[i + 1] = v.y, r[i + 2] = v.z, r[i + 3] = v.w;
    }
    tmem_st16(taddr, r);
}

template <int D>
__global__ void __launch_bounds__(kKvThreads, 1)
    attn_bwd_dkdv_tc(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                     const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap gmap,
                     const BwdParams p) {
    constexpr int NB = D / 64, W2 = D / 2, BQ = 64, NS = kv_stages<D>();
    constexpr int KP = 128 * D * 2, QP = BQ * D * 2;  // bytes of one plane of a K tile / a query tile
    constexpr int cVh = 0, cST = 64, cDPT = 192, cDV = 256, cDK = 256 + D;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sKh = smem, *sKl = smem + KP, *sVl = smem + 2 * KP;  // V's hi plane sits in TMEM
    uint8_t *stage0 = smem + 3 * KP;  // stage s: Qh, Ql, dOh, dOl at stage0 + s * 4 QP + {0,1,2,3} QP
    KvShared *sh = reinterpret_cast<KvShared *>(smem + 3 * KP + NS * 4 * QP);

    const int warp = threadIdx.x >> 5;
    // Launch order (x fastest): the KV groups of one sequence, key tile by key tile.  Early key tiles see the
    // most query rows, so within a sequence the longest walks start first and the shortest last, which keeps
    // the kernel's tail (SMs idle while the last long CTA finishes) to a fraction of one walk.
    const int g = blockIdx.x, kt = (int)blockIdx.y, b = blockIdx.z;
    const int group = p.n_heads / p.n_kv_heads;
    const int s0 = kt * 128;
    const int n_q = (p.T + BQ - 1) / BQ, qi0 = s0 / BQ;
    const int per_head = n_q - qi0;
    const int n_it = group * per_head;
    const int B = p.batch;
    Walk walk(group, per_head, qi0, n_q);

    if (threadIdx.x == 0) {
        for (int i = 0; i < NS; ++i) {
            mbar_init(&sh->full_q[i], 1), mbar_init(&sh->full_g[i], 1);
            mbar_init(&sh->free_q[i], 1), mbar_init(&sh->free_g[i], 1);
        }
        mbar_init(&sh->k_full, 1);
        mbar_init(&sh->a_ready, kKvRowWarps);
        mbar_init(&sh->st_full[0], 1);
        mbar_init(&sh->st_full[1], 1);
        mbar_init(&sh->dp_full, 1);
        mbar_init(&sh->p_full, kKvRowWarps);
        mbar_init(&sh->ld_ready, kKvRowWarps);
        mbar_init(&sh->flush_ready, 1);
        mbar_init(&sh->flush_done, kKvRowWarps);
        sh->abort = 0;
        mbar_fence_init();
    }
    if (warp == kKvRowWarps + 1) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    const float mq = block_mult(p.amax_q[b * p.n_kv_heads + g]), mk = block_mult(p.amax_k[b * p.n_kv_heads + g]);
    const float mv = block_mult(p.amax_v[b * p.n_kv_heads + g]), mdo = block_mult(p.amax_do[b * p.n_kv_heads + g]);
    // dS in this CTA's units: the largest |dS| of the (sequence, KV group), as the dQ kernel met it, goes to
    // [2^12, 2^13); c1 turns dP of the scaled planes into those units
    const float c1 = pow2_for(__uint_as_float(p.dsmax[b * p.n_kv_heads + g]), 13) / (mdo * mv);

    if (warp == kKvRowWarps) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            tma_prefetch_desc(&kmap), tma_prefetch_desc(&vmap), tma_prefetch_desc(&qmap), tma_prefetch_desc(&gmap);
            mbar_arrive_expect_tx(&sh->k_full, 3 * KP);
            tma_load_4d(sKh, &kmap, &sh->k_full, 0, s0, g * NB, b);
            tma_load_4d(sKl, &kmap, &sh->k_full, 0, s0, g * NB, B + b);
            tma_load_4d(sVl, &vmap, &sh->k_full, 0, s0, g * NB, B + b);
            int issued = 0;
            for (int it = 0; it < n_it; ++it, walk.next()) {
                const int s = it % NS;
                const uint32_t free_par = (uint32_t)(((it / NS) & 1) ^ 1);
                const int h = g * group + walk.hh, row = walk.qi * BQ;
                uint8_t *st = stage0 + s * 4 * QP;
                // Q's planes are released by dK(it - NS), early in that step, and wanted first (S^T runs
                // two steps ahead); dO's are released by dV and wanted a step later
                if (it >= NS && !kwait(&sh->free_q[s], free_par, sh)) { kgive_up(sh, 21); break; }
                mbar_arrive_expect_tx(&sh->full_q[s], 2 * QP);
                tma_load_4d(st, &qmap, &sh->full_q[s], 0, row, h * NB, b);
                tma_load_4d(st + QP, &qmap, &sh->full_q[s], 0, row, h * NB, B + b);
                ++issued;
                if (it >= NS && !kwait(&sh->free_g[s], free_par, sh)) { kgive_up(sh, 21); break; }
                mbar_arrive_expect_tx(&sh->full_g[s], 2 * QP);
                tma_load_4d(st + 2 * QP, &gmap, &sh->full_g[s], 0, row, h * NB, b);
                tma_load_4d(st + 3 * QP, &gmap, &sh->full_g[s], 0, row, h * NB, B + b);
                ++issued;
            }
            if (sh->abort) {
                // let the copies in flight land before the CTA's shared memory goes away: `issued` counts
                // half-stages, Q's then dO's of step issued / 2
                mbar_wait(&sh->k_full, 0);
                for (int c = (issued > 2 * NS ? issued - 2 * NS : 0); c < issued; ++c) {
                    const int it = c >> 1;
                    mbar_wait((c & 1) ? &sh->full_g[it % NS] : &sh->full_q[it % NS], (uint32_t)((it / NS) & 1));
                }
            }
        }
        __syncwarp();
    } else if (warp == kKvRowWarps + 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t id_s = idesc_f16(128, BQ, false, false);
            constexpr uint32_t id_a = idesc_f16(128, D, false, true);
            bool ok = kwait(&sh->k_full, 0, sh) && kwait(&sh->a_ready, 0, sh);
            if (!ok) kgive_up(sh, 22);
            tc_fence_after();
            const uint64_t bkh = desc_kmajor(smem_u32(sKh)), bkl = desc_kmajor(smem_u32(sKl));
            const uint64_t bvl = desc_kmajor(smem_u32(sVl));
            const uint32_t stage_u32 = smem_u32(stage0);
            // S^T(it) = K Q^T into buffer it & 1
            auto issue_st = [&](int it) {
                const uint32_t qh = stage_u32 + (uint32_t)((it % NS) * 4 * QP);
                const uint64_t bqh = desc_kmajor(qh), bql = desc_kmajor(qh + QP);
                const uint32_t oS = cST + (it & 1) * BQ;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t ao = (uint32_t)((kk >> 2) * (128 * 128) + (kk & 3) * 32);
                    const uint32_t bo = (uint32_t)((kk >> 2) * (BQ * 128) + (kk & 3) * 32);
                    const uint64_t dkh = desc_advance(bkh, ao), dkl = desc_advance(bkl, ao);
                    const uint64_t dqh = desc_advance(bqh, bo), dql = desc_advance(bql, bo);
                    mma_ss_f16(tmem + oS, dkh, dqh, id_s, kk > 0);
                    mma_ss_f16(tmem + oS, dkh, dql, id_s, 1);
                    mma_ss_f16(tmem + oS, dkl, dqh, id_s, 1);
                }
                mma_commit(&sh->st_full[it & 1]);
            };
            // dP^T(it) = V dO^T
            auto issue_dp = [&](int it) {
                const uint32_t qh = stage_u32 + (uint32_t)((it % NS) * 4 * QP);
                const uint64_t bgh = desc_kmajor(qh + 2 * QP), bgl = desc_kmajor(qh + 3 * QP);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t ao = (uint32_t)((kk >> 2) * (128 * 128) + (kk & 3) * 32);
                    const uint32_t bo = (uint32_t)((kk >> 2) * (BQ * 128) + (kk & 3) * 32);
                    const uint64_t dvl = desc_advance(bvl, ao);
                    const uint64_t dgh = desc_advance(bgh, bo), dgl = desc_advance(bgl, bo);
                    mma_ts_f16(tmem + cDPT, tmem + cVh + kk * 8, dgh, id_s, kk > 0);
                    mma_ts_f16(tmem + cDPT, tmem + cVh + kk * 8, dgl, id_s, 1);
                    mma_ss_f16(tmem + cDPT, dvl, dgh, id_s, 1);
                }
                mma_commit(&sh->dp_full);
            };
            auto stage_ready = [&](int it) -> bool {  // Q's planes of step `it`
                return mbar_try_wait(&sh->full_q[it % NS], (uint32_t)((it / NS) & 1));
            };
            auto stage_wait = [&](int it) -> bool {
                if (!kwait(&sh->full_q[it % NS], (uint32_t)((it / NS) & 1), sh)) return false;
                tc_fence_after();
                return true;
            };
            auto stage_wait_g = [&](int it) -> bool {  // dO's planes
                if (!kwait(&sh->full_g[it % NS], (uint32_t)((it / NS) & 1), sh)) return false;
                tc_fence_after();
                return true;
            };
            int n_flush = 0;
            int pending_st = -1;  // an S^T whose operands had not landed when its turn came
            if (ok) {
                if (!stage_wait(0) || !stage_wait_g(0)) { kgive_up(sh, 23); ok = false; }
                else {
                    issue_st(0), issue_dp(0);
                    if (n_it > 1) {
                        if (!stage_wait(1)) { kgive_up(sh, 23); ok = false; }
                        else issue_st(1);
                    }
                }
            }
            for (int it = 0; ok && it < n_it; ++it, walk.next()) {
                // wait for P^T(it) and dS^T(it); a pending S^T goes out as soon as its operands land,
                // so that the row threads' exp of that step is not left for after the next dV/dK
                {
                    bool got = false;
                    for (uint32_t i = 0; i < (1u << 20); ++i) {
                        if (mbar_try_wait(&sh->p_full, (uint32_t)(it & 1))) { got = true; break; }
                        if (pending_st >= 0 && stage_ready(pending_st)) {
                            tc_fence_after();
                            issue_st(pending_st);
                            pending_st = -1;
                        }
                        if ((i & 255u) == 255u && sh->abort) break;
                    }
                    if (!got) { kgive_up(sh, 24); break; }
                }
                if (walk.fresh && it > 0) {
                    // the row threads are adding the accumulators to memory; restart them only after that
                    if (!kwait(&sh->flush_done, (uint32_t)((n_flush - 1) & 1), sh)) { kgive_up(sh, 27); break; }
                }
                tc_fence_after();
                const int s = it % NS;
                const uint32_t qh = stage_u32 + (uint32_t)(s * 4 * QP);
                const uint64_t mqh = desc_mnmajor_16b(qh, BQ * 128), mql = desc_mnmajor_16b(qh + QP, BQ * 128);
                const uint64_t mgh = desc_mnmajor_16b(qh + 2 * QP, BQ * 128), mgl = desc_mnmajor_16b(qh + 3 * QP, BQ * 128);
                const uint32_t oS = cST + (it & 1) * BQ;
                const uint32_t acc0 = walk.fresh ? 0u : 1u;
                // P^T / dS^T: the set of query columns [16 c, 16 c + 16), one MMA step deep, left its hi
                // halves in the first 8 columns of its 16-column window and its lo halves in the last 8.
                // dK first: it frees dS^T's columns for dP^T(it+1), which the row threads wait for.
#pragma unroll
                for (int kk = 0; kk < BQ / 16; ++kk) {
                    const uint64_t dqh = desc_advance(mqh, kk * 2048), dql = desc_advance(mql, kk * 2048);
                    mma_ts_f16(tmem + cDK, tmem + cDPT + kk * 16, dqh, id_a, kk > 0 ? 1u : acc0);
                    mma_ts_f16(tmem + cDK, tmem + cDPT + kk * 16, dql, id_a, 1);
                    mma_ts_f16(tmem + cDK, tmem + cDPT + kk * 16 + 8, dqh, id_a, 1);
                }
                mma_commit(&sh->free_q[s]);
                if (it + 1 < n_it) {
                    if (pending_st == it + 1) {  // (its S^T has not gone out either: operands still in flight)
                        if (!stage_wait(it + 1)) { kgive_up(sh, 23); break; }
                        issue_st(it + 1);
                        pending_st = -1;
                    }
                    if (!stage_wait_g(it + 1)) { kgive_up(sh, 23); break; }
                    issue_dp(it + 1);
                }
#pragma unroll
                for (int kk = 0; kk < BQ / 16; ++kk) {
                    const uint64_t dgh = desc_advance(mgh, kk * 2048), dgl = desc_advance(mgl, kk * 2048);
                    mma_ts_f16(tmem + cDV, tmem + oS + kk * 16, dgh, id_a, kk > 0 ? 1u : acc0);
                    mma_ts_f16(tmem + cDV, tmem + oS + kk * 16, dgl, id_a, 1);
                    mma_ts_f16(tmem + cDV, tmem + oS + kk * 16 + 8, dgh, id_a, 1);
                }
                mma_commit(&sh->free_g[s]);
                if (walk.flush) {
                    // the row threads wait for every flush in turn, so one barrier's parity is enough
                    mma_commit(&sh->flush_ready);
                    ++n_flush;
                }
                if (it + 2 < n_it) {
                    // S^T(it+2) overwrites the buffer dV(it) has just read.  With two stages its operands
                    // have been on their way since dK(it) retired: if they have not landed yet, it goes
                    // out from the wait loop of the next step.
                    if (NS > 2) {
                        if (!stage_wait(it + 2)) { kgive_up(sh, 23); break; }
                        issue_st(it + 2);
                    } else if (stage_ready(it + 2)) {
                        tc_fence_after();
                        issue_st(it + 2);
                    } else {
                        pending_st = it + 2;
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ one thread per key row and
        // 16 of the step's query columns: set `set` handles columns [16 set, 16 set + 16)
        const int tid = threadIdx.x & 127, set = threadIdx.x >> 7;
        const int key = s0 + tid;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const long long wkv = (long long)p.n_kv_heads * D;
        {
            // V's hi plane -> TMEM, 16 words of the row per set
            const long long off = ((long long)b * p.T + (key < p.T ? key : 0)) * wkv + (long long)g * D;
            if (set * 16 < W2) row_to_tmem16(p.v_planes + off + set * 32, key < p.T, tmem + lane_base + cVh + set * 16);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->a_ready);
        }
        const float cs = p.scale_log2 / (mq * mk);
        // P is wanted times p_scale (for its 16-bit split) and dS without it: the scale rides in the exponent
        // (lse minus log2 p_scale) and leaves through dP's and delta's factors
        const float lse_shift = log2f(p.p_scale);
        const float c1p = c1 / p.p_scale;
        const float dfac = mdo * mv * c1p;
        // lse (set 0's first 64 threads) and delta (set 1's) of a step's 64 query rows, fetched one step
        // ahead into a register and published through shared memory
        auto fetch = [&](const Walk &w, int it) -> float {
            if (threadIdx.x >= 256 || tid >= 64 || it >= n_it) return 0.f;
            const int t = w.qi * BQ + tid;
            if (t >= p.T) return 0.f;
            const long long idx = ((long long)b * p.T + t) * p.n_heads + g * group + w.hh;
            return set == 0 ? __ldg(p.lse + idx) * kLog2e - lse_shift : (ZT_DEFECT(13) ? 0.f : __ldg(p.delta + idx) * dfac);
        };
        auto publish = [&](int it, float v) {
            if (threadIdx.x < 256 && tid < 64) (set == 0 ? sh->lse2 : sh->dels)[it & 1][tid] = v;
            mbar_arrive_warp(&sh->ld_ready);
        };
        Walk ahead = walk;  // one step ahead of `walk`
        publish(0, fetch(ahead, 0));
        ahead.next();
        int n_flush = 0;
        bool ok = true;
        bool saturated = false;  // a dS value of this thread met kDsBound (or was not a number)
        // The accumulators go to memory one step late: after a flush step's dS the row threads would only wait
        // for its dV and dK to retire, and the next step's exp and dS need neither the accumulators nor that
        // wait, so they come first and the tensor core finds them done when the flush ends.
        auto flush_now = [&]() -> bool {
            if (!__all_sync(0xffffffffu, kwait(&sh->flush_ready, (uint32_t)(n_flush & 1), sh))) {
                kgive_up(sh, 26);
                return false;
            }
            tc_fence_after();
            // sets 0, 1 add the halves of dV's columns to memory, sets 2, 3 those of dK's.  A thread owns a key
            // row; written as they are, the 32 rows of a warp would cost 32 memory transactions per
            // instruction.  Eight lanes first transpose their 8 x 8 blocks of float4 among themselves, so that
            // lane j holds the j-th float4 of eight rows and an instruction covers four rows' 128-byte runs.
            const int c0 = (set & 1) * (D / 2);
            const uint32_t acc = tmem + lane_base + (set < 2 ? cDV : cDK) + c0;
            const int lane = threadIdx.x & 31, j8 = lane & 7;
            const long long wo = (long long)p.n_kv_heads * p.dim_out;
            float *dst = (set < 2 ? p.dv : p.dk) + ((long long)b * p.T + (key - j8)) * wo + (long long)g * p.dim_out + c0 + 4 * j8;
            const float f = set < 2 ? 1.0f / (p.p_scale * mdo) : p.scale / (mdo * mv * c1 * mq);
#pragma unroll 1
            for (int c = 0; c < D / 2; c += 32) {
                uint32_t r[32];
                tmem_ld32(acc + c, r);
                tmem_wait_ld();
#pragma unroll
                for (int M = 4; M >= 1; M >>= 1) {
                    const bool up = (lane & M) != 0;
#pragma unroll
                    for (int m = 0; m < 8; ++m) {
                        if (m & M) continue;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t send = up ? r[4 * m + e] : r[4 * (m ^ M) + e];
                            const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, M);
                            if (up) r[4 * m + e] = recv;
                            else r[4 * (m ^ M) + e] = recv;
                        }
                    }
                }
                if (c0 + c < p.dim_out) {  // (a padded tile's upper columns are not the tensor's)
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (key - j8 + i >= p.T) continue;
                        float4 a;
                        a.x = __uint_as_float(r[4 * i]) * f, a.y = __uint_as_float(r[4 * i + 1]) * f;
                        a.z = __uint_as_float(r[4 * i + 2]) * f, a.w = __uint_as_float(r[4 * i + 3]) * f;
                        // the first flush assigns (dk/dv need no zeroing by the caller); later ones
                        // add in memory: a rounded f32 add with no reply to wait for
                        if (n_flush == 0) *reinterpret_cast<float4 *>(dst + i * wo + c) = a;
                        else red_add_v4(dst + i * wo + c, a);
                    }
                }
            }
            ++n_flush;
            // (no fence: the tensor core only needs the accumulators read, and nobody else adds to these rows)
            tc_fence_before();
            mbar_arrive_warp(&sh->flush_done);
            return true;
        };
        bool flush_pending = false;
        for (int it = 0; it < n_it; ++it, walk.next(), ahead.next()) {
            const int t0 = walk.qi * BQ + set * 16;
            const uint32_t par = (uint32_t)(it & 1);
            const float nxt = fetch(ahead, it + 1);
            if (!__all_sync(0xffffffffu, kwait(&sh->ld_ready, par, sh) && kwait(&sh->st_full[it & 1], (uint32_t)((it >> 1) & 1), sh))) {
                kgive_up(sh, 25);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t wS = tmem + lane_base + cST + (it & 1) * BQ + set * 16;
            const uint32_t wP = tmem + lane_base + cDPT + set * 16;
            float pr[16];
            {
                uint32_t rs[16];
                tmem_ld16(wS, rs);
                tmem_wait_ld();
                uint32_t ph[8], pl[8];
                // a step whose 64 query rows all lie past the tile's last key and inside the sequence needs no
                // mask (most steps of a long sequence); the test is the same for every thread of the CTA
                const int q_first = walk.qi * BQ;
                if ((q_first >= s0 + 127 || ZT_DEFECT(11)) && q_first + BQ <= p.T && s0 + 128 <= p.T) {
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
#pragma unroll
                        for (int e = 0; e < 2; ++e)
                            pr[i + e] = ex2(__uint_as_float(rs[i + e]) * cs - sh->lse2[it & 1][set * 16 + i + e]);
                        split_pack(pr[i], pr[i + 1], ph[i >> 1], pl[i >> 1]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int t = t0 + i + e;
                            const bool vis = (key <= t || ZT_DEFECT(11)) && (t < p.T) && (key < p.T);
                            const float pe = ex2(__uint_as_float(rs[i + e]) * cs - sh->lse2[it & 1][set * 16 + i + e]);
                            pr[i + e] = vis ? pe : 0.f;
                        }
                        split_pack(pr[i], pr[i + 1], ph[i >> 1], pl[i >> 1]);
                    }
                }
                tmem_st8(wS, ph);
                tmem_st8(wS + 8, pl);
            }
            if (!__all_sync(0xffffffffu, kwait(&sh->dp_full, par, sh))) {
                kgive_up(sh, 28);
                ok = false;
                break;
            }
            tc_fence_after();
            // dP^T(it) is issued only after every row warp has finished step it-1, so the staging
            // buffer of step it+1 (last read in step it-1) is free now
            if (it + 1 < n_it) publish(it + 1, nxt);
            {
                uint32_t rd[16];
                tmem_ld16(wP, rd);
                tmem_wait_ld();
                uint32_t dh[8], dl[8];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    float dv[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float x = pr[i + e] * (__uint_as_float(rd[i + e]) * c1p - sh->dels[it & 1][set * 16 + i + e]);
                        saturated |= !(fabsf(x) <= kDsBound);
                        dv[e] = fminf(fmaxf(x, -kDsBound), kDsBound);
                    }
                    split_pack(dv[0], dv[1], dh[i >> 1], dl[i >> 1]);
                }
                tmem_st8(wP, dh);
                tmem_st8(wP + 8, dl);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->p_full);
            if (flush_pending) {
                flush_pending = false;
                if (!flush_now()) { ok = false; break; }
            }
            if (walk.flush) {
                if (it + 1 < n_it) flush_pending = true;
                else if (!flush_now()) { ok = false; break; }
            }
        }
        (void)ok;
        if (__any_sync(0xffffffffu, saturated) && (threadIdx.x & 31) == 0) atomicAdd(&g_tc_saturated, 1u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kKvRowWarps + 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------------
// dQ.  grid (ceil(T / 128), n_heads, batch), 576 threads: 16 row warps, a TMA warp, an MMA warp.
//
// Key tiles of 64, S and dP in two TMEM buffers each: while the row threads turn S and dP of tile j
// into dS, the tensor core computes dQ of tile j-1 and S, dP of tile j+1.  The hi planes of the Q and
// dO tiles are TMEM operands, their lo planes (used by one of the three split terms) stay in shared
// memory.  K tiles live from S(j), issued two tiles ahead, to dQ(j): a ring of three; V tiles only for
// dP(j): a ring of two.  The row warps are four sets of four; a set handles 16 of the tile's 64 keys
// (one 16-deep MMA step of dQ).
// ---------------------------------------------------------------------------------------------------
constexpr int kDqKSlots = 3, kDqVSlots = 2;

struct DqShared {
    uint64_t full_k[kDqKSlots], free_k[kDqKSlots], full_v[kDqVSlots], free_v[kDqVSlots];
    uint64_t ql_full, qh_full, a_ready, sdp_full[2], p_full[2], all_done;
    uint32_t tmem_base;
    volatile int abort;
};
__device__ __forceinline__ bool dwait(uint64_t *bar, uint32_t parity, DqShared *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void dgive_up(DqShared *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}
template <int D>
__host__ __device__ constexpr size_t dq_smem_bytes() {
    return 2 * (size_t)(128 * D * 2) + (kDqKSlots + kDqVSlots) * 2 * (size_t)(64 * D * 2) + sizeof(DqShared) + 1024;
}

template <int D>
__global__ void __launch_bounds__(kKvThreads, 1)
    attn_bwd_dq_tc(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                   const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap gmap,
                   const BwdParams p) {
    constexpr int NB = D / 64, W2 = D / 2, BN = 64;
    constexpr int QP = 128 * D * 2;  // bytes of one plane of the 128-row Q / dO tile
    constexpr int KP = BN * D * 2;   // bytes of one plane of a 64-key tile
    constexpr int cQh = 0, cGh = 64, cS = 128, cDP = 256, cDQ = 384;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sQl = smem, *sGl = smem + QP;
    uint8_t *sK = smem + 2 * QP;               // slot s: Kh, Kl at sK + s * 2 KP + {0, 1} KP
    uint8_t *sV = sK + kDqKSlots * 2 * KP;     // slot s: Vh, Vl
    DqShared *sh = reinterpret_cast<DqShared *>(sV + kDqVSlots * 2 * KP);

    const int warp = threadIdx.x >> 5;
    // launch order (x fastest): a head's query tiles, late (long) ones first.  (Starting the heads of a sequence
    // tile by tile instead, which would shorten the tail, measured 1 % slower.)
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int g = h / (p.n_heads / p.n_kv_heads);
    const int t0 = qt * 128;
    const int rows_end = (t0 + 128 < p.T) ? t0 + 128 : p.T;
    const int n_tiles = (rows_end + BN - 1) / BN;
    const int B = p.batch;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kDqKSlots; ++i) mbar_init(&sh->full_k[i], 1), mbar_init(&sh->free_k[i], 1);
        for (int i = 0; i < kDqVSlots; ++i) mbar_init(&sh->full_v[i], 1), mbar_init(&sh->free_v[i], 1);
        mbar_init(&sh->ql_full, 1);
        mbar_init(&sh->qh_full, 1);
        mbar_init(&sh->a_ready, kKvRowWarps);
        for (int i = 0; i < 2; ++i) mbar_init(&sh->sdp_full[i], 1), mbar_init(&sh->p_full[i], kKvRowWarps);
        mbar_init(&sh->all_done, 1);
        sh->abort = 0;
        mbar_fence_init();
    }
    if (warp == kKvRowWarps + 1) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    const float mq = block_mult(p.amax_q[b * p.n_kv_heads + g]), mk = block_mult(p.amax_k[b * p.n_kv_heads + g]);
    const float mv = block_mult(p.amax_v[b * p.n_kv_heads + g]), mdo = block_mult(p.amax_do[b * p.n_kv_heads + g]);

    if (warp == kKvRowWarps) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            tma_prefetch_desc(&kmap), tma_prefetch_desc(&vmap), tma_prefetch_desc(&qmap), tma_prefetch_desc(&gmap);
            mbar_arrive_expect_tx(&sh->ql_full, 2 * QP);
            tma_load_4d(sQl, &qmap, &sh->ql_full, 0, t0, h * NB, B + b);
            tma_load_4d(sGl, &gmap, &sh->ql_full, 0, t0, h * NB, B + b);
            // the hi planes, bound for TMEM, are staged in K's slots 1 and 2 until the row threads have moved them:
            // one bulk copy each instead of a strided read per thread
            mbar_arrive_expect_tx(&sh->qh_full, 2 * QP);
            tma_load_4d(sK + 2 * KP, &qmap, &sh->qh_full, 0, t0, h * NB, b);
            tma_load_4d(sK + 4 * KP, &gmap, &sh->qh_full, 0, t0, h * NB, b);
            int n_k = 0, n_v = 0;  // tiles issued
            bool live = true;
            auto load_k = [&](int j) {
                const int ks = j % kDqKSlots;
                if (j >= kDqKSlots && !dwait(&sh->free_k[ks], (uint32_t)(((j / kDqKSlots) & 1) ^ 1), sh)) { dgive_up(sh, 31), live = false; return; }
                mbar_arrive_expect_tx(&sh->full_k[ks], 2 * KP);
                tma_load_4d(sK + ks * 2 * KP, &kmap, &sh->full_k[ks], 0, j * BN, g * NB, b);
                tma_load_4d(sK + ks * 2 * KP + KP, &kmap, &sh->full_k[ks], 0, j * BN, g * NB, B + b);
                ++n_k;
            };
            auto load_v = [&](int j) {
                const int vs = j % kDqVSlots;
                if (j >= kDqVSlots && !dwait(&sh->free_v[vs], (uint32_t)(((j / kDqVSlots) & 1) ^ 1), sh)) { dgive_up(sh, 31), live = false; return; }
                mbar_arrive_expect_tx(&sh->full_v[vs], 2 * KP);
                tma_load_4d(sV + vs * 2 * KP, &vmap, &sh->full_v[vs], 0, j * BN, g * NB, b);
                tma_load_4d(sV + vs * 2 * KP + KP, &vmap, &sh->full_v[vs], 0, j * BN, g * NB, B + b);
                ++n_v;
            };
            load_k(0), load_v(0);
            if (n_tiles > 1) load_v(1);
            // K's slots 1 and 2 are the hi planes' until every row thread has its part of them in TMEM
            if (!dwait(&sh->a_ready, 0, sh)) dgive_up(sh, 31), live = false;
            if (live && n_tiles > 1) load_k(1);
            if (live && n_tiles > 2) load_k(2);
            for (int j = 2; live && j < n_tiles; ++j) {
                if (j >= kDqKSlots) load_k(j);
                if (live) load_v(j);
            }
            if (sh->abort) {
                // let the copies in flight land before the CTA's shared memory goes away
                mbar_wait(&sh->ql_full, 0);
                mbar_wait(&sh->qh_full, 0);
                for (int j = (n_k > kDqKSlots ? n_k - kDqKSlots : 0); j < n_k; ++j)
                    mbar_wait(&sh->full_k[j % kDqKSlots], (uint32_t)((j / kDqKSlots) & 1));
                for (int j = (n_v > kDqVSlots ? n_v - kDqVSlots : 0); j < n_v; ++j)
                    mbar_wait(&sh->full_v[j % kDqVSlots], (uint32_t)((j / kDqVSlots) & 1));
            }
        }
        __syncwarp();
    } else if (warp == kKvRowWarps + 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t id_s = idesc_f16(128, BN, false, false);
            constexpr uint32_t id_a = idesc_f16(128, D, false, true);
            bool ok = dwait(&sh->ql_full, 0, sh) && dwait(&sh->a_ready, 0, sh);
            if (!ok) dgive_up(sh, 32);
            tc_fence_after();
            const uint64_t bql = desc_kmajor(smem_u32(sQl)), bgl = desc_kmajor(smem_u32(sGl));
            const uint32_t k_u32 = smem_u32(sK), v_u32 = smem_u32(sV);
            // S(j) = Q K^T and dP(j) = dO V^T into buffers j & 1
            auto issue_sdp = [&](int j) -> bool {
                const int ks = j % kDqKSlots, vs = j % kDqVSlots;
                if (!dwait(&sh->full_k[ks], (uint32_t)((j / kDqKSlots) & 1), sh)) return false;
                tc_fence_after();
                const uint32_t kh = k_u32 + (uint32_t)(ks * 2 * KP);
                const uint64_t bkh = desc_kmajor(kh), bkl = desc_kmajor(kh + KP);
                const uint32_t oS = cS + (j & 1) * BN, oP = cDP + (j & 1) * BN;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t ao = (uint32_t)((kk >> 2) * (128 * 128) + (kk & 3) * 32);
                    const uint32_t bo = (uint32_t)((kk >> 2) * (BN * 128) + (kk & 3) * 32);
                    const uint64_t dkh = desc_advance(bkh, bo), dkl = desc_advance(bkl, bo);
                    mma_ts_f16(tmem + oS, tmem + cQh + kk * 8, dkh, id_s, kk > 0);
                    mma_ts_f16(tmem + oS, tmem + cQh + kk * 8, dkl, id_s, 1);
                    mma_ss_f16(tmem + oS, desc_advance(bql, ao), dkh, id_s, 1);
                }
                if (!dwait(&sh->full_v[vs], (uint32_t)((j / kDqVSlots) & 1), sh)) return false;
                tc_fence_after();
                const uint32_t vh = v_u32 + (uint32_t)(vs * 2 * KP);
                const uint64_t bvh = desc_kmajor(vh), bvl = desc_kmajor(vh + KP);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t ao = (uint32_t)((kk >> 2) * (128 * 128) + (kk & 3) * 32);
                    const uint32_t bo = (uint32_t)((kk >> 2) * (BN * 128) + (kk & 3) * 32);
                    const uint64_t dvh = desc_advance(bvh, bo), dvl = desc_advance(bvl, bo);
                    mma_ts_f16(tmem + oP, tmem + cGh + kk * 8, dvh, id_s, kk > 0);
                    mma_ts_f16(tmem + oP, tmem + cGh + kk * 8, dvl, id_s, 1);
                    mma_ss_f16(tmem + oP, desc_advance(bgl, ao), dvh, id_s, 1);
                }
                mma_commit(&sh->free_v[vs]);
                mma_commit(&sh->sdp_full[j & 1]);
                return true;
            };
            if (ok && !issue_sdp(0)) { dgive_up(sh, 33); ok = false; }
            if (ok && n_tiles > 1 && !issue_sdp(1)) { dgive_up(sh, 33); ok = false; }
            for (int j = 0; ok && j < n_tiles; ++j) {
                if (!dwait(&sh->p_full[j & 1], (uint32_t)((j >> 1) & 1), sh)) { dgive_up(sh, 34); break; }
                tc_fence_after();
                const int ks = j % kDqKSlots;
                const uint32_t kh = k_u32 + (uint32_t)(ks * 2 * KP);
                const uint64_t mkh = desc_mnmajor_16b(kh, BN * 128), mkl = desc_mnmajor_16b(kh + KP, BN * 128);
                const uint32_t oP = cDP + (j & 1) * BN;
                // dS: the set of keys [16 c, 16 c + 16), one MMA step deep, left its hi halves in the first
                // 8 columns of its 16-column window and its lo halves in the last 8
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint64_t dkh = desc_advance(mkh, kk * 2048), dkl = desc_advance(mkl, kk * 2048);
                    mma_ts_f16(tmem + cDQ, tmem + oP + kk * 16, dkh, id_a, (j > 0 || kk > 0) ? 1 : 0);
                    mma_ts_f16(tmem + cDQ, tmem + oP + kk * 16, dkl, id_a, 1);
                    mma_ts_f16(tmem + cDQ, tmem + oP + kk * 16 + 8, dkh, id_a, 1);
                }
                mma_commit(&sh->free_k[ks]);
                // completes once, when every MMA of this CTA has retired: a barrier that counted
                // tiles could be several phases ahead of a waiting row set, and a parity wait can
                // only tell the current phase from the one before it
                if (j == n_tiles - 1) mma_commit(&sh->all_done);
                if (j + 2 < n_tiles && !issue_sdp(j + 2)) { dgive_up(sh, 33); break; }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ one thread per query row and
        // 16 of the tile's keys: set `set` handles keys [16 set, 16 set + 16) of every tile
        const int tid = threadIdx.x & 127, set = threadIdx.x >> 7;
        const int t = t0 + tid;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        bool ok = true;
        {
            // the hi planes of the Q and dO rows -> TMEM, 16 words (four 16-byte chunks of the 128-byte-swizzled
            // staging tiles) of each per set
            if (!__all_sync(0xffffffffu, dwait(&sh->qh_full, 0, sh))) dgive_up(sh, 37), ok = false;
            if (set * 16 < W2) {
                const uint8_t *src = sK + 2 * KP + (set >> 1) * (128 * 128) + tid * 128;
                uint32_t rq[16], rg[16];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int at = (((set & 1) * 4 + c) ^ (tid & 7)) << 4;
                    const uint4 a = *reinterpret_cast<const uint4 *>(src + at);
                    const uint4 g4 = *reinterpret_cast<const uint4 *>(src + 2 * KP + at);
                    rq[4 * c] = a.x, rq[4 * c + 1] = a.y, rq[4 * c + 2] = a.z, rq[4 * c + 3] = a.w;
                    rg[4 * c] = g4.x, rg[4 * c + 1] = g4.y, rg[4 * c + 2] = g4.z, rg[4 * c + 3] = g4.w;
                }
                tmem_st16(tmem + lane_base + cQh + set * 16, rq);
                tmem_st16(tmem + lane_base + cGh + set * 16, rg);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->a_ready);
        }
        const float cs = p.scale_log2 / (mq * mk);
        const long long ridx = ((long long)b * p.T + (t < p.T ? t : 0)) * p.n_heads + h;
        const float lse2 = (t < p.T) ? __ldg(p.lse + ridx) * kLog2e : 0.f;
        // this row's scale: |dS| <= 2 |dout[t]| max |v[s]| (a shade more: P may round to just above 1) goes below 2^14
        const float cq = (t < p.T) ? pow2_for(2.02f * __ldg(p.rnorm + ridx) * __uint_as_float(p.vnmax[b * p.n_kv_heads + g]), 14) : 1.0f;
        const float c1 = cq / (mdo * mv);
        const float dels = (t < p.T && !ZT_DEFECT(13)) ? __ldg(p.delta + ridx) * cq : 0.f;
        float ds_top = 0.f;  // largest |dS| of this thread, in the row's units
        bool saturated = false;  // a dS value of this thread met kDsBound (or was not a number)
        for (int j = 0; ok && j < n_tiles; ++j) {
            if (!__all_sync(0xffffffffu, dwait(&sh->sdp_full[j & 1], (uint32_t)((j >> 1) & 1), sh))) {
                dgive_up(sh, 35);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t wS = tmem + lane_base + cS + (j & 1) * BN + set * 16;
            const uint32_t wP = tmem + lane_base + cDP + (j & 1) * BN + set * 16;
            uint32_t rs[16], rd[16];
            tmem_ld16(wS, rs);
            tmem_ld16(wP, rd);
            tmem_wait_ld();
            uint32_t dh[8], dl[8];
            const int key0 = j * BN + set * 16;
            // a key tile that ends before the query tile begins needs no mask; the same test for the whole CTA
            if ((j * BN + BN - 1 <= t0 || ZT_DEFECT(11)) && j * BN + BN <= p.T) {
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    float dv[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float pe = ex2(__uint_as_float(rs[i + e]) * cs - lse2);
                        const float x = pe * (__uint_as_float(rd[i + e]) * c1 - dels);
                        const float ax = fabsf(x);
                        saturated |= !(ax <= kDsBound);
                        ds_top = fmaxf(ds_top, ax);
                        dv[e] = fminf(fmaxf(x, -kDsBound), kDsBound);
                    }
                    split_pack(dv[0], dv[1], dh[i >> 1], dl[i >> 1]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    float dv[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = key0 + i + e;
                        const bool vis = (key <= t || ZT_DEFECT(11)) && (key < p.T);
                        const float pe = ex2(__uint_as_float(rs[i + e]) * cs - lse2);
                        const float x = vis ? pe * (__uint_as_float(rd[i + e]) * c1 - dels) : 0.f;
                        const float ax = fabsf(x);
                        saturated |= !(ax <= kDsBound);
                        ds_top = fmaxf(ds_top, ax);
                        dv[e] = fminf(fmaxf(x, -kDsBound), kDsBound);
                    }
                    split_pack(dv[0], dv[1], dh[i >> 1], dl[i >> 1]);
                }
            }
            tmem_st8(wP, dh);
            tmem_st8(wP + 8, dl);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->p_full[j & 1]);
        }
        if (__any_sync(0xffffffffu, saturated) && (threadIdx.x & 31) == 0) atomicAdd(&g_tc_saturated, 1u);
        {
            // the largest |dS| of the (sequence, KV group), in true units, for the dK/dV kernel's scale (a clamped or
            // non-finite value counts as the bound: the flag above has already reported it)
            float top = fminf(ds_top, kDsBound) / cq;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
            // (most warps find a larger value already there and make no atomic)
            uint32_t *cell = p.dsmax + b * p.n_kv_heads + g;
            if ((threadIdx.x & 31) == 0 && __float_as_uint(top) > *reinterpret_cast<volatile uint32_t *>(cell))
                atomicMax(cell, __float_as_uint(top));
        }
        if (ok && !__all_sync(0xffffffffu, dwait(&sh->all_done, 0, sh))) {
            dgive_up(sh, 36);
            ok = false;
        }
        if (ok) {
            tc_fence_after();
            // each set writes a quarter of the row's columns
            constexpr int CW = D / 4;  // 32 or 16
            const float fq = p.scale / (cq * mk);
            // mine: this set's CW columns; other: their rotation partners (i +- dim_out / 2, another set's
            // chunk of this row's accumulator), read only when dQ leaves as the gradient of the unrotated q
            const bool rot = p.rope_t != nullptr && set * CW < p.dim_out;
            const int half = p.dim_out / 2, col = set * CW;
            const bool upper = col >= half;
            const uint32_t other_at = tmem + lane_base + cDQ + (upper ? col - half : col + half);
            uint32_t r[32], o[32];
            if (CW == 32) {
                tmem_ld32(tmem + lane_base + cDQ + col, r);
                if (rot) tmem_ld32(other_at, o);
                tmem_wait_ld();
            } else {
                uint32_t r16[16], o16[16];
                tmem_ld16(tmem + lane_base + cDQ + col, r16);
                if (rot) tmem_ld16(other_at, o16);
                tmem_wait_ld();  // the registers hold the values only from here on
#pragma unroll
                for (int i = 0; i < 16; ++i) r[i] = r16[i], o[i] = o16[i];
            }
            if (rot) {
                // the table is read transposed: the threads of a warp are consecutive rows, so entry i of 32 rows
                // is one 256-byte run
                const float2 *cs = p.rope_t + (long long)(upper ? col - half : col) * p.T + (t < p.T ? t : 0);
#pragma unroll
                for (int i = 0; i < CW; ++i)
                    r[i] = __float_as_uint(rope_elem(__uint_as_float(r[i]), __uint_as_float(o[i]), __ldg(cs + (long long)i * p.T), upper, true));
            }
            // to global memory through shared memory (K's slots, free once all_done completes): a thread owns a
            // row in TMEM, and a store of 32 rows costs 32 memory transactions; a row per instruction costs four
            uint8_t *srow = sK + tid * (D * 4);
#pragma unroll
            for (int i = 0; i < CW; i += 4) {
                float4 a;
                a.x = __uint_as_float(r[i]) * fq, a.y = __uint_as_float(r[i + 1]) * fq;
                a.z = __uint_as_float(r[i + 2]) * fq, a.w = __uint_as_float(r[i + 3]) * fq;
                const int ch = (col + i) >> 2;  // chunk c of row r sits at chunk c ^ (r & (CW - 1)): D / 4 chunks a row
                *reinterpret_cast<float4 *>(srow + ((ch ^ (tid & (CW - 1))) << 4)) = a;
            }
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");  // the 512 row threads
        if (!sh->abort) {
            constexpr int CH = D / 4, RPI = 32 / CH;  // 16-byte chunks per row, rows per store instruction
            const int lane = threadIdx.x & 31;
            const int ch = lane & (CH - 1);
            const long long wo = (long long)p.n_heads * p.dim_out;
#pragma unroll
            for (int i = 0; i < 8; i += RPI) {
                const int r = warp * 8 + i + lane / CH;
                const float4 a = *reinterpret_cast<const float4 *>(sK + r * (D * 4) + ((ch ^ (r & (CH - 1))) << 4));
                if (t0 + r < p.T && ch * 4 < p.dim_out) {  // (a padded tile's upper columns are not the tensor's)
                    const long long idx = ((long long)b * p.T + t0 + r) * wo + (long long)h * p.dim_out + ch * 4;
                    *reinterpret_cast<float4 *>(p.dq + idx) = a;
                    for (int pr = 0; pr < p.dq_peers.n; ++pr) *reinterpret_cast<float4 *>(p.dq_peers.ptr[pr] + idx) = a;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kKvRowWarps + 1) tmem_dealloc(tmem, 512);
}

// ---- host side ----------------------------------------------------------------------------------------

struct BwdWorkspace {
    uint32_t *amax_q, *amax_k, *amax_v, *amax_do, *vnmax, *dsmax;  // six [batch, n_kv_heads] arrays, in this order
    __half *q_planes, *do_planes, *k_planes, *v_planes;
    float *rnorm;  // [batch, T, n_heads]
    __half *qs_planes;  // the row-scaled copy of q's planes (the fused and the wide-head backward read it for dK)
    size_t total_bytes, amax_bytes;
};

inline BwdWorkspace bwd_workspace(void *base, int batch, int T, int n_heads, int n_kv_heads, int dim) {
    BwdWorkspace w{};
    const size_t n_amax = (size_t)batch * n_kv_heads;
    w.amax_bytes = (6 * n_amax * sizeof(uint32_t) + 1023) / 1024 * 1024;
    const size_t qh = (size_t)2 * batch * T * n_heads * dim * sizeof(__half);
    const size_t kh = (size_t)2 * batch * T * n_kv_heads * dim * sizeof(__half);
    auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
    char *c = static_cast<char *>(base);
    w.amax_q = reinterpret_cast<uint32_t *>(c);
    w.amax_k = w.amax_q + n_amax, w.amax_v = w.amax_k + n_amax, w.amax_do = w.amax_v + n_amax;
    w.vnmax = w.amax_do + n_amax, w.dsmax = w.vnmax + n_amax;
    size_t off = w.amax_bytes;
    w.q_planes = reinterpret_cast<__half *>(c + off), off += up(qh);
    w.do_planes = reinterpret_cast<__half *>(c + off), off += up(qh);
    w.k_planes = reinterpret_cast<__half *>(c + off), off += up(kh);
    w.v_planes = reinterpret_cast<__half *>(c + off), off += up(kh);
    w.rnorm = reinterpret_cast<float *>(c + off), off += up((size_t)batch * T * n_heads * sizeof(float));
    w.qs_planes = reinterpret_cast<__half *>(c + off), off += up(qh);
    w.total_bytes = off;
    return w;
}

inline bool tc_bwd_supported(int batch, int T, int dim, const void *q, const void *k, const void *v,
                             const void *dout, const void *dq, const void *dk, const void *dv) {
    if (!(dim == 32 || dim == 64 || dim == 96 || dim == 128) || T < 128 || batch < 1) return false;
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!al(q) || !al(k) || !al(v) || !al(dout) || !al(dq) || !al(dk) || !al(dv)) return false;
    const DeviceInfo *d = device_info();
    return d && d->cc_major == 10 && get_encode_tiled() != nullptr;
}

struct BwdMaps {
    CUtensorMap k128, v128, q64, g64;   // dK/dV kernel: 128-key K and V tiles, 64-row Q and dO tiles
    CUtensorMap k64, v64, q128, g128;   // dQ kernel: 64-key K and V tiles, 128-row Q and dO tiles
};

template <int D>
inline int launch_bwd_tc_d(const BwdMaps &m, const BwdParams &p, cudaStream_t stream) {
    const size_t floor_ = 120 * 1024;  // one CTA per SM: each wants all 512 TMEM columns
    const size_t sa = kv_smem_bytes<D>() > floor_ ? kv_smem_bytes<D>() : floor_;
    const size_t sb = dq_smem_bytes<D>() > floor_ ? dq_smem_bytes<D>() : floor_;
    if (optin_smem((const void *)attn_bwd_dkdv_tc<D>, sa)) return 1;
    if (optin_smem((const void *)attn_bwd_dq_tc<D>, sb)) return 1;
    const dim3 grid_a((unsigned)p.n_kv_heads, (unsigned)((p.T + 127) / 128), (unsigned)p.batch);
    const dim3 grid_b((unsigned)((p.T + 127) / 128), (unsigned)p.n_heads, (unsigned)p.batch);
    // dQ first: it records the largest |dS| of every (sequence, KV group), which scales dS in the dK/dV kernel
    if (ZT_LAUNCH("attn_bwd_dq_tc", stream,
                  (attn_bwd_dq_tc<D><<<grid_b, kKvThreads, sb, stream>>>(m.k64, m.v64, m.q128, m.g128, p))))
        return 1;
    return ZT_LAUNCH("attn_bwd_dkdv_tc", stream,
                     (attn_bwd_dkdv_tc<D><<<grid_a, kKvThreads, sa, stream>>>(m.k128, m.v128, m.q64, m.g64, p)));
}

}  // namespace tcb

// head_dim 32 runs on the 64-wide tiles and head_dim 96 on the 128-wide ones: the planes carry every head
// zero-padded to the tile's width (at 32 the MMAs would cost the same at half the width, see the clock floor
// above; at 96 a quarter of the tensor work is padding), outputs keep their own width.  The kernels write
// their outputs in 32-column (128-wide tiles) or 16/32-column (64-wide) pieces, which is why only these two.
inline int tc_tile_dim(int dim) { return dim == 32 ? 64 : (dim == 96 ? 128 : (dim == 192 ? 256 : dim)); }

inline size_t tc_bwd_workspace_bytes(int batch, int T, int n_heads, int n_kv_heads, int dim) {
    return tcb::bwd_workspace(nullptr, batch, T, n_heads, n_kv_heads, tc_tile_dim(dim)).total_bytes;
}

}  // namespace zt
