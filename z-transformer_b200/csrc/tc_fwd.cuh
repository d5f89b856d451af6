// Causal GQA attention forward on the Blackwell tensor cores (tcgen05 + TMEM + TMA), with
// 3xTF32 split arithmetic so that the result keeps f32 accuracy.
//
// What it computes: attention.forward (src/attention.zig:60-153) for a batch, plus the
// log-sum-exp of every row.  What it replaces: the reference's SIMT kernel
// (src/cuda/attn_kernels.cu:197-369), whose design it does not share.
//
// One CTA owns one tile of 128 query rows of one head and walks the key/value tiles of its
// causal prefix.  Per key tile (BN keys):
//
//   TMA warp        K tile and V tile, f32, into shared memory as column blocks of 32 floats
//                   (K with the 16-byte-atom 128B swizzle, V with the 32-byte-atom one that an
//                   MN-major tf32 operand needs); two buffers each.
//   split warps     lo = tf32(x - trunc_tf32(x)) for the tile, into a second buffer.  The tensor
//                   core itself ignores the low 13 mantissa bits of a 32-bit operand, so the
//                   raw tile already serves as the hi part.
//   MMA warp        S  = Qhi.Khi + Qhi.Klo + Qlo.Khi      (A = Q from TMEM, B = K from smem)
//                   O += Phi.Vhi + Phi.Vlo + Plo.Vhi      (A = P from TMEM, B = V from smem)
//                   f32 accumulators in TMEM; each product of two f32 numbers is reproduced
//                   to about 2^-21 relative.
//   softmax warps   one thread per query row: read S from TMEM, causal mask, running max
//                   (log2 domain; Q was pre-multiplied by log2(e)/sqrt(D)), P = exp2(S - m),
//                   split P into hi/lo and write both back to TMEM.  The running max is only
//                   moved when it grows by more than 2^8, so O in TMEM is rescaled rarely.
//
// TMEM columns: [0,D) Qhi, [D,2D) Qlo, [2D,3D) O, [3D,3D+BN) S then Phi, [3D+BN,3D+2BN) Plo.
// Every wait is bounded; a wait that gives up raises g_tc_status and the CTA leaves normally.
#pragma once

#include "tc_common.cuh"
#include "zt_common.cuh"

namespace zt {

// Non-zero after a tensor-core kernel gave up on a wait (code = which one).  Read by
// zt_attn_tc_status(); never set in a correct run.
static __device__ int g_tc_status;
// Number of CTAs of the backward kernels in which a dS value met the bound of its 16-bit split (see
// tc_bwd.cuh, "the bound on dS"); read and cleared by zt_attn_tc_saturated.  A correct run never raises it.
static __device__ unsigned int g_tc_saturated;

namespace tcf {

using namespace tc;

constexpr int kBM = 128;
constexpr int kThreads = 320;  // 4 softmax warps, 4 split warps, 1 TMA warp, 1 MMA warp
constexpr float kRescaleThreshold = 8.0f;

template <int D>
struct Cfg {
    static constexpr int BN = (D == 128) ? 64 : 128;
    static constexpr int kTileBytes = BN * D * 4;
    static constexpr int kTmemCols = 512;
    static constexpr int kQhi = 0, kQlo = D, kO = 2 * D, kS = 3 * D, kPlo = 3 * D + BN;
    static_assert(3 * D + 2 * BN <= 512, "TMEM budget");
    // Six tiles + alignment slack + barriers; never less than 120 KiB so that two CTAs (each
    // wanting all 512 TMEM columns) are never resident on one SM.
    static constexpr size_t kNeeded = 6 * (size_t)kTileBytes + 1024 + 512;
    static constexpr size_t kSmemBytes = kNeeded > 120 * 1024 ? kNeeded : 120 * 1024;
};

struct Shared {
    uint64_t kx_full[2], kx_free[2], vx_full[2], vx_free[2];
    uint64_t klo_ready, klo_free, vlo_ready, vlo_free;
    uint64_t q_ready, s_full, p_full, pv_done;
    uint32_t tmem_base;
    volatile int abort;
};

struct Params {
    const float *q;
    float *out, *lse;  // lse may be null
    int T, n_heads, n_kv_heads;
    float scale_log2;
};

// A wait that also gives up as soon as another role has given up.
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, Shared *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void give_up(Shared *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}


template <int D>
__global__ void __launch_bounds__(kThreads, 1)
    attn_fwd_tc(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, const Params p) {
    using C = Cfg<D>;
    constexpr int BN = C::BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *kx[2] = {smem, smem + C::kTileBytes};
    uint8_t *vx[2] = {smem + 2 * C::kTileBytes, smem + 3 * C::kTileBytes};
    uint8_t *klo = smem + 4 * C::kTileBytes;
    uint8_t *vlo = smem + 5 * C::kTileBytes;
    Shared *sh = reinterpret_cast<Shared *>(smem + 6 * C::kTileBytes);

    const int warp = threadIdx.x >> 5;
    // heavy (late) query tiles first: their causal prefix is the longest
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (p.n_heads / p.n_kv_heads);
    const int t0 = qt * kBM;
    const int rows_end = (t0 + kBM < p.T) ? t0 + kBM : p.T;  // one past the last valid query row
    const int n_tiles = (rows_end + BN - 1) / BN;            // key tiles of the causal prefix

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh->kx_full[i], 1);
            mbar_init(&sh->kx_free[i], 1);
            mbar_init(&sh->vx_full[i], 1);
            mbar_init(&sh->vx_free[i], 1);
        }
        mbar_init(&sh->klo_ready, 4);
        mbar_init(&sh->klo_free, 1);
        mbar_init(&sh->vlo_ready, 4);
        mbar_init(&sh->vlo_free, 1);
        mbar_init(&sh->q_ready, 4);
        mbar_init(&sh->s_full, 1);
        mbar_init(&sh->p_full, 4);
        mbar_init(&sh->pv_done, 1);
        sh->abort = 0;
        mbar_fence_init();
    }
    if (warp == 9) tmem_alloc(&sh->tmem_base, C::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 8) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            tma_prefetch_desc(&kmap);
            tma_prefetch_desc(&vmap);
            int issued_k = 0, issued_v = 0;
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                if (j >= 2 && !wait_or_abort(&sh->kx_free[s], ph ^ 1u, sh)) { give_up(sh, 1); break; }
                mbar_arrive_expect_tx(&sh->kx_full[s], C::kTileBytes);
                tma_load_4d(kx[s], &kmap, &sh->kx_full[s], 0, j * BN, kvh * (D / 32), b);
                ++issued_k;
                if (j >= 2 && !wait_or_abort(&sh->vx_free[s], ph ^ 1u, sh)) { give_up(sh, 2); break; }
                mbar_arrive_expect_tx(&sh->vx_full[s], C::kTileBytes);
                tma_load_4d(vx[s], &vmap, &sh->vx_full[s], 0, j * BN, kvh * (D / 32), b);
                ++issued_v;
            }
            if (sh->abort) {
                // Leave no copy in flight into this CTA's shared memory: wait (bounded) for the
                // loads already issued.
                for (int j = (issued_k > 2 ? issued_k - 2 : 0); j < issued_k; ++j)
                    mbar_wait(&sh->kx_full[j & 1], (uint32_t)((j >> 1) & 1));
                for (int j = (issued_v > 2 ? issued_v - 2 : 0); j < issued_v; ++j)
                    mbar_wait(&sh->vx_full[j & 1], (uint32_t)((j >> 1) & 1));
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc_s = idesc_tf32(kBM, BN, false);
            constexpr uint32_t idesc_o = idesc_tf32(kBM, D, true);
            bool ok = wait_or_abort(&sh->q_ready, 0, sh);
            if (!ok) give_up(sh, 3);
            for (int j = 0; ok && j < n_tiles; ++j) {
                const int s = j & 1;
                const uint32_t ph2 = (uint32_t)((j >> 1) & 1), ph1 = (uint32_t)(j & 1);
                // ---- S = Q K^T (three terms)
                if (!wait_or_abort(&sh->kx_full[s], ph2, sh) || !wait_or_abort(&sh->klo_ready, ph1, sh)) {
                    give_up(sh, 4);
                    break;
                }
                tc_fence_after();
                const uint64_t bkhi = desc_kmajor(smem_u32(kx[s])), bklo = desc_kmajor(smem_u32(klo));
#pragma unroll
                for (int kk = 0; kk < D / 8; ++kk) {
                    const uint32_t off = (uint32_t)((kk >> 2) * (BN * 128) + (kk & 3) * 32);
                    const uint64_t dhi = desc_advance(bkhi, off), dlo = desc_advance(bklo, off);
                    mma_ts_tf32(tmem + C::kS, tmem + C::kQhi + kk * 8, dhi, idesc_s, kk > 0);
                    mma_ts_tf32(tmem + C::kS, tmem + C::kQhi + kk * 8, dlo, idesc_s, 1);
                    mma_ts_tf32(tmem + C::kS, tmem + C::kQlo + kk * 8, dhi, idesc_s, 1);
                }
                mma_commit(&sh->s_full);
                mma_commit(&sh->kx_free[s]);
                mma_commit(&sh->klo_free);
                // ---- O += P V (three terms)
                if (!wait_or_abort(&sh->p_full, ph1, sh) || !wait_or_abort(&sh->vx_full[s], ph2, sh) ||
                    !wait_or_abort(&sh->vlo_ready, ph1, sh)) {
                    give_up(sh, 5);
                    break;
                }
                tc_fence_after();
                const uint64_t bvhi = desc_mnmajor(smem_u32(vx[s]), BN * 128), bvlo = desc_mnmajor(smem_u32(vlo), BN * 128);
#pragma unroll
                for (int kk = 0; kk < BN / 8; ++kk) {
                    const uint64_t dhi = desc_advance(bvhi, kk * 1024), dlo = desc_advance(bvlo, kk * 1024);
                    mma_ts_tf32(tmem + C::kO, tmem + C::kS + kk * 8, dhi, idesc_o, (j > 0 || kk > 0) ? 1 : 0);
                    mma_ts_tf32(tmem + C::kO, tmem + C::kS + kk * 8, dlo, idesc_o, 1);
                    mma_ts_tf32(tmem + C::kO, tmem + C::kPlo + kk * 8, dhi, idesc_o, 1);
                }
                mma_commit(&sh->pv_done);
                mma_commit(&sh->vx_free[s]);
                mma_commit(&sh->vlo_free);
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ hi/lo split
        const int tid = threadIdx.x - 128;
        constexpr int kVec = C::kTileBytes / 16 / 128;  // float4 per thread per tile
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            const uint32_t ph2 = (uint32_t)((j >> 1) & 1), ph1 = (uint32_t)(j & 1);
            for (int which = 0; which < 2; ++which) {
                uint64_t *full = which ? &sh->vx_full[s] : &sh->kx_full[s];
                uint64_t *free_ = which ? &sh->vlo_free : &sh->klo_free;
                uint64_t *ready = which ? &sh->vlo_ready : &sh->klo_ready;
                const float4 *src = reinterpret_cast<const float4 *>(which ? vx[s] : kx[s]);
                float4 *dst = reinterpret_cast<float4 *>(which ? vlo : klo);
                bool ok = wait_or_abort(full, ph2, sh);
                if (ok && j >= 1) ok = wait_or_abort(free_, ph1 ^ 1u, sh);
                if (!ok) {
                    give_up(sh, 6);
                    j = n_tiles;
                    break;
                }
#pragma unroll 4
                for (int i = 0; i < kVec; ++i) {
                    const float4 x = src[tid + i * 128];
                    float4 lo;
                    lo.x = tf32_round(x.x - tf32_trunc(x.x)), lo.y = tf32_round(x.y - tf32_trunc(x.y));
                    lo.z = tf32_round(x.z - tf32_trunc(x.z)), lo.w = tf32_round(x.w - tf32_trunc(x.w));
                    dst[tid + i * 128] = lo;
                }
                fence_async_smem();
                mbar_arrive_warp(ready);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax rows
        const int row = threadIdx.x;      // tile row == TMEM lane
        const int t = t0 + row;           // query position
        const uint32_t lane_base = (uint32_t)(warp * 32);
        const long long qld = (long long)p.n_heads * D;
        {
            // Q row, pre-scaled, split, into TMEM
            const float *qrow = p.q + ((long long)b * p.T + (t < p.T ? t : p.T - 1)) * qld + (long long)h * D;
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                uint32_t hi[32], lo[32];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 x = __ldg(reinterpret_cast<const float4 *>(qrow + c + i));
                    if (t >= p.T) x = make_float4(0.f, 0.f, 0.f, 0.f);
                    const float xs[4] = {x.x * p.scale_log2, x.y * p.scale_log2, x.z * p.scale_log2,
                                         x.w * p.scale_log2};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float hv = tf32_round(xs[e]);
                        hi[i + e] = __float_as_uint(hv);
                        lo[i + e] = __float_as_uint(tf32_round(xs[e] - hv));
                    }
                }
                tmem_st32(tmem_addr(tmem, lane_base, C::kQhi + c), hi);
                tmem_st32(tmem_addr(tmem, lane_base, C::kQlo + c), lo);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->q_ready);
        }
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const uint32_t ph1 = (uint32_t)(j & 1);
            // every branch below holds warp-wide tcgen05 instructions, so `ok` is made warp-uniform
            if (!__all_sync(0xffffffffu, wait_or_abort(&sh->s_full, ph1, sh))) {
                give_up(sh, 7);
                ok = false;
                break;
            }
            tc_fence_after();
            const int s0 = j * BN;
            const bool diag = (s0 + BN - 1 > t0);  // some (row, key) pair of this tile is masked
            // pass 1: the row maximum of the visible scores
            float mt = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_addr(tmem, lane_base, C::kS + c), r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float sv = __uint_as_float(r[i]);
                    if (!diag || s0 + c + i <= t) mt = fmaxf(mt, sv);
                }
            }
            // Move the reference maximum only when it would grow by more than 2^8: P stays below
            // 2^8 in between and O in TMEM needs no rescale.
            float factor = 1.f;
            if (mt > m_ref + kRescaleThreshold || m_ref == -INFINITY) {
                if (mt != -INFINITY) {
                    factor = (m_ref == -INFINITY) ? 0.f : ex2(m_ref - mt);
                    m_ref = mt;
                }
            }
            l *= factor;
            if (j > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
                // s_full(j) already implies P.V of tile j-1 is complete (MMAs retire in order);
                // the explicit wait keeps that independent of issue order.
                if (!__all_sync(0xffffffffu, wait_or_abort(&sh->pv_done, ph1 ^ 1u, sh))) {
                    give_up(sh, 8);
                    ok = false;
                    break;
                }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_addr(tmem, lane_base, C::kO + c), r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
                    tmem_st32(tmem_addr(tmem, lane_base, C::kO + c), r);
                }
            }
            // pass 2: P = exp2(S - m), split, back into TMEM (hi over S, lo beside it)
            const float mref_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
            float psum = 0.f;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32], lo[32];
                tmem_ld32(tmem_addr(tmem, lane_base, C::kS + c), r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float pe = ex2(__uint_as_float(r[i]) - mref_safe);
                    if (diag && s0 + c + i > t) pe = 0.f;
                    psum += pe;
                    const float hv = tf32_round(pe);
                    r[i] = __float_as_uint(hv);
                    lo[i] = __float_as_uint(tf32_round(pe - hv));
                }
                tmem_st32(tmem_addr(tmem, lane_base, C::kS + c), r);
                tmem_st32(tmem_addr(tmem, lane_base, C::kPlo + c), lo);
            }
            l += psum;
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->p_full);
        }
        if (ok) {
            if (!__all_sync(0xffffffffu, wait_or_abort(&sh->pv_done, (uint32_t)((n_tiles - 1) & 1), sh))) {
                give_up(sh, 9);
                ok = false;
            }
        }
        if (ok) {
            tc_fence_after();
            const float inv = 1.f / l;
            float *orow = p.out + ((long long)b * p.T + t) * qld + (long long)h * D;
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_addr(tmem, lane_base, C::kO + c), r);
                tmem_wait_ld();
                if (t < p.T) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float4 o4;
                        o4.x = __uint_as_float(r[i]) * inv, o4.y = __uint_as_float(r[i + 1]) * inv;
                        o4.z = __uint_as_float(r[i + 2]) * inv, o4.w = __uint_as_float(r[i + 3]) * inv;
                        *reinterpret_cast<float4 *>(orow + c + i) = o4;
                    }
                }
            }
            if (p.lse && t < p.T)
                p.lse[((long long)b * p.T + t) * p.n_heads + h] = (m_ref + log2f(l)) * kLn2;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, C::kTmemCols);
}

// ---- host side ------------------------------------------------------------------------------------

inline bool tc_fwd_supported(int batch, int T, int n_heads, int n_kv_heads, int dim, int q_offset, int n_keys,
                             const float *q, const float *k, const float *v, const float *out) {
    (void)n_heads, (void)n_kv_heads;
    if (!(dim == 32 || dim == 64 || dim == 128)) return false;
    if (q_offset != 0 || n_keys != T || T < 128 || batch < 1) return false;
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!al(q) || !al(k) || !al(v) || !al(out)) return false;
    const DeviceInfo *d = device_info();
    return d && d->cc_major == 10 && get_encode_tiled() != nullptr;
}

template <int D>
inline int launch_fwd_tc_d(const CUtensorMap &kmap, const CUtensorMap &vmap, const Params &p, int batch,
                           cudaStream_t stream) {
    const size_t smem = Cfg<D>::kSmemBytes;
    if (optin_smem((const void *)attn_fwd_tc<D>, smem)) return 1;
    dim3 grid((unsigned)((p.T + kBM - 1) / kBM), (unsigned)p.n_heads, (unsigned)batch);
    return ZT_LAUNCH("attn_fwd_tc", stream, (attn_fwd_tc<D><<<grid, kThreads, smem, stream>>>(kmap, vmap, p)));
}

}  // namespace tcf

inline bool tc_fwd_supported(int batch, int T, int n_heads, int n_kv_heads, int dim, int q_offset, int n_keys,
                             const float *q, const float *k, const float *v, const float *out) {
    return tcf::tc_fwd_supported(batch, T, n_heads, n_kv_heads, dim, q_offset, n_keys, q, k, v, out);
}

inline int launch_fwd_tc(const float *q, const float *k, const float *v, float *out, float *lse, int batch, int T,
                         int n_heads, int n_kv_heads, int dim, cudaStream_t stream) {
    CUtensorMap kmap, vmap;
    const int bn = (dim == 128) ? 64 : 128;
    if (!make_head_tile_map(&kmap, k, batch, T, n_kv_heads * dim, dim, bn, false) ||
        !make_head_tile_map(&vmap, v, batch, T, n_kv_heads * dim, dim, bn, true))
        return refuse("the TMA tensor maps for K/V could not be encoded.");
    tcf::Params p{};
    p.q = q, p.out = out, p.lse = lse;
    p.T = T, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads;
    p.scale_log2 = kLog2e / sqrtf((float)dim);
    g_last_path = "tcgen05";
    switch (dim) {
        case 32: return tcf::launch_fwd_tc_d<32>(kmap, vmap, p, batch, stream);
        case 64: return tcf::launch_fwd_tc_d<64>(kmap, vmap, p, batch, stream);
        default: return tcf::launch_fwd_tc_d<128>(kmap, vmap, p, batch, stream);
    }
}

// 0 when no tensor-core kernel has ever given up on a wait on the current device.
inline int tc_status_read(int *host_value) {
    return cudaMemcpyFromSymbol(host_value, g_tc_status, sizeof(int)) == cudaSuccess ? 0 : 1;
}
// The count of backward CTAs that saturated a dS value since the last read; cleared by the read.
inline int tc_saturated_read(unsigned int *host_value) {
    if (cudaMemcpyFromSymbol(host_value, g_tc_saturated, sizeof(unsigned int)) != cudaSuccess) return 1;
    const unsigned int zero = 0;
    return cudaMemcpyToSymbol(g_tc_saturated, &zero, sizeof(unsigned int)) == cudaSuccess ? 0 : 1;
}

}  // namespace zt
