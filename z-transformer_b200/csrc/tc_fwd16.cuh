// Causal GQA attention forward on the tensor cores with the three-term split on f16 pieces
// (the arithmetic of tc_bwd.cuh) and a two-deep pipeline over the key tiles.
//
// Same result as attn_fwd_tc (tc_fwd.cuh, 3xTF32) and the same role -- attention.forward
// (src/attention.zig:60-153) for a batch plus each row's log-sum-exp -- at 2.4 times the speed:
// an f16 term is half a TF32 MMA, operands take half the bytes (three K and three V tiles, hi and
// lo, fit in shared memory), and two S tiles and two O accumulators fit in TMEM.
//
//   bwd_absmax / bwd_split   (tc_bwd.cuh) q, k, v -> f16 hi/lo planes with a power-of-two scale
//                            per (sequence, KV group), in a workspace.
//   TMA warp        K and V hi/lo tiles of 64 keys, a ring of three slots each: a K tile is free
//                   once its S has retired, two tiles before its V.
//   MMA warp        S[j+2] = Qh.Kh + Qh.Kl + Ql.Kh  (A = Q from TMEM) into buffer j & 1 as soon as
//                   P.V of tile j has been issued; once P[j] is in TMEM,
//                   O[j & 1] += Ph.Vh + Ph.Vl + Pl.Vh   (A = P from TMEM, V tile as MN-major B).
//   softmax warps   two sets of four, one thread per query row; set j & 1 owns tile j, with a
//                   reference maximum (moved only when it grows by > 2^8), a sum and an O accumulator
//                   of its own, so neither set waits on the other's tile.  P is scaled by 2^7 and
//                   split into packed f16 pairs written over S.  The two partial softmaxes are merged
//                   when the row is written.
// TMEM columns: [0,D/2) Qh, [D/2,D) Ql, [D,2D) O of set 0, [2D,3D) O of set 1, then two S/P tiles of
// 64 columns.
#pragma once

#include "tc_bwd.cuh"

namespace zt {
namespace tcf16 {

using namespace tc;
using tcb::block_mult;
using tcb::row_to_tmem;
using tcb::split_pack;

constexpr int kThreads = 320;  // 8 softmax warps (two sets of four), 1 TMA warp, 1 MMA warp
constexpr float kPScale = 128.0f;  // 2^7: P is multiplied by it before its 16-bit split (the 7.0f in the kernels)
constexpr float kRescaleThreshold = 8.0f;

struct Shared {
    uint64_t full_k[3], free_k[3], full_v[3], free_v[3];
    uint64_t a_ready, s_full[2], p_full[2], pv_done[2], all_done, q_full;
    uint32_t tmem_base;
    volatile int abort;
    float fin_m[2][128], fin_l[2][128];  // each set's reference maximum and sum, for the final merge
};

struct Params {
    const __half *q_planes;                     // [2][B][T][H*D]
    const uint32_t *amax_q, *amax_k, *amax_v;   // [B, Hkv]
    float *out, *lse;                           // lse may be null
    int batch, T, n_heads, n_kv_heads;
    int dim_out;  // the tensors' head_dim: the tile's D, or 32 under a tile padded to 64
    int ahead;    // attn_fwd_tc16 prefetches the query tile of the block this many places on in launch order; 0: none
    float scale_log2;
    // When set, the epilogue also leaves out as f16 hi/lo planes ([2][B][T][H * dim_out], one power-of-two scale per
    // sequence) for the projection that follows (tc_gemm.cuh): the GEMM then needs no pass of its own over out.
    __half *o_planes;
    long long o_plane_stride;  // elements from the hi plane to the lo plane
    PeerList out_peers;        // out is also stored here (same element index), see zt_common.cuh
};

// The scale of a sequence's out planes.  An output row is a convex combination of rows of v, so |out| <= max |v|
// over the sequence's KV heads: the power of two that puts that maximum just under 2^15 fits out as well.
__device__ __forceinline__ float out_plane_mult(const Params &p, int b) {
    uint32_t top = 0;
    for (int g = 0; g < p.n_kv_heads; ++g) top = max(top, p.amax_v[b * p.n_kv_heads + g]);
    return block_mult(top);
}
// Four consecutive elements of out at element index idx, and their planes when asked for.
__device__ __forceinline__ void store_out4(const Params &p, long long idx, float4 o4, float mo) {
    *reinterpret_cast<float4 *>(p.out + idx) = o4;
    for (int r = 0; r < p.out_peers.n; ++r) *reinterpret_cast<float4 *>(p.out_peers.ptr[r] + idx) = o4;
    if (p.o_planes) {
        uint2 hw, lw;
        split_pack(o4.x * mo, o4.y * mo, hw.x, lw.x);
        split_pack(o4.z * mo, o4.w * mo, hw.y, lw.y);
        *reinterpret_cast<uint2 *>(p.o_planes + idx) = hw;
        *reinterpret_cast<uint2 *>(p.o_planes + p.o_plane_stride + idx) = lw;
    }
}

__device__ __forceinline__ bool fwait(uint64_t *bar, uint32_t parity, Shared *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void fgive_up(Shared *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}

// The row work on 32 score columns, in two forms chosen per tile (the same for every thread of the CTA): a tile
// that ends before the query tile begins needs no mask.  P comes out already multiplied by kPScale (the scale
// rides in the exponent: `off` is the reference maximum minus log2 kPScale), split into packed f16 pairs.
template <bool MASK>
__device__ __forceinline__ float row_max32(const uint32_t (&r)[32], int key0, int t, float m) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
        if (!MASK || key0 + i <= t) m = fmaxf(m, __uint_as_float(r[i]));
    return m;
}
template <bool MASK>
__device__ __forceinline__ float row_exp32(const uint32_t (&r)[32], int key0, int t, float cs, float off,
                                           uint32_t (&ph)[16], uint32_t (&pl)[16]) {
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        float pe[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            pe[e] = ex2(__uint_as_float(r[i + e]) * cs - off);
            if (MASK && key0 + i + e > t) pe[e] = 0.f;
            sum += pe[e];
        }
        split_pack(pe[0], pe[1], ph[i >> 1], pl[i >> 1]);
    }
    return sum;
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
    attn_fwd_tc16(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  const __grid_constant__ CUtensorMap qmap, const Params p) {
    constexpr int NB = D / 64, W2 = D / 2, BN = 64;
    constexpr int KP = BN * D * 2;  // bytes of one plane of a key tile
    constexpr int cQh = 0, cQl = W2, cO0 = D, cS0 = 3 * D;  // O of set s at cO0 + s D, S/P of buffer i at cS0 + 64 i
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem, *sV = smem + 6 * KP;  // three slots of (hi, lo) each
    Shared *sh = reinterpret_cast<Shared *>(smem + 12 * KP);

    const int warp = threadIdx.x >> 5;
    // launch order (x fastest): a head's query tiles, late (long) ones first.  (Starting the heads of a sequence
    // tile by tile instead, which would shorten the tail, measured 3 % slower.)
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int g = h / (p.n_heads / p.n_kv_heads);
    const int t0 = qt * 128;
    const int rows_end = (t0 + 128 < p.T) ? t0 + 128 : p.T;
    const int n_tiles = (rows_end + BN - 1) / BN;
    const int B = p.batch;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 3; ++i) {
            mbar_init(&sh->full_k[i], 1), mbar_init(&sh->free_k[i], 1);
            mbar_init(&sh->full_v[i], 1), mbar_init(&sh->free_v[i], 1);
        }
        mbar_init(&sh->a_ready, 8);
        for (int i = 0; i < 2; ++i) mbar_init(&sh->s_full[i], 1), mbar_init(&sh->p_full[i], 4), mbar_init(&sh->pv_done[i], 1);
        mbar_init(&sh->all_done, 1);
        mbar_init(&sh->q_full, 1);
        sh->abort = 0;
        mbar_fence_init();
    }
    if (warp == 9) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    const float mq = block_mult(p.amax_q[b * p.n_kv_heads + g]), mk = block_mult(p.amax_k[b * p.n_kv_heads + g]);
    const float mv = block_mult(p.amax_v[b * p.n_kv_heads + g]);

    if (warp == 8) {
        // ------------------------------------------------------------------ TMA producer
        // K of tile j is free again once S(j) has retired, two tiles before its V: rings of their own
        if (elect_one()) {
            tma_prefetch_desc(&qmap), tma_prefetch_desc(&kmap), tma_prefetch_desc(&vmap);
            // the query tile's two planes, staged in V's first two slots until the row threads have moved
            // them into TMEM: one bulk copy each instead of a strided read per thread
            mbar_arrive_expect_tx(&sh->q_full, 4 * KP);
            tma_load_4d(sV, &qmap, &sh->q_full, 0, t0, h * NB, b);
            tma_load_4d(sV + 2 * KP, &qmap, &sh->q_full, 0, t0, h * NB, B + b);
            int n_k = 0, n_v = 0;  // tiles issued
            bool live = true;
            const auto prefetch_next_q = [&]() {
                // The query tile of the CTA that will start when one of the running ones ends (`ahead` blocks on in
                // launch order, about the number of SMs), into L2: its planes were written once by the pre-pass and
                // would otherwise come from DRAM, under load, before that CTA's first MMA can go out.
                const long long gx = gridDim.x, gy = gridDim.y;
                const long long lin = blockIdx.x + gx * (blockIdx.y + gy * blockIdx.z) + p.ahead;
                if (p.ahead <= 0 || lin >= gx * gy * gridDim.z) return;
                const int nx = (int)(lin % gx), ny = (int)((lin / gx) % gy), nz = (int)(lin / (gx * gy));
                const int nt0 = ((int)gx - 1 - nx) * 128;
                tma_prefetch_l2_4d(&qmap, 0, nt0, ny * NB, nz);
                tma_prefetch_l2_4d(&qmap, 0, nt0, ny * NB, B + nz);
            };
            auto load_k = [&](int j) {
                const int s = j % 3;
                if (j >= 3 && !fwait(&sh->free_k[s], (uint32_t)(((j / 3) & 1) ^ 1), sh)) { fgive_up(sh, 41), live = false; return; }
                mbar_arrive_expect_tx(&sh->full_k[s], 2 * KP);
                tma_load_4d(sK + s * 2 * KP, &kmap, &sh->full_k[s], 0, j * BN, g * NB, b);
                tma_load_4d(sK + s * 2 * KP + KP, &kmap, &sh->full_k[s], 0, j * BN, g * NB, B + b);
                ++n_k;
            };
            auto load_v = [&](int j) {
                const int s = j % 3;
                if (j >= 3 && !fwait(&sh->free_v[s], (uint32_t)(((j / 3) & 1) ^ 1), sh)) { fgive_up(sh, 41), live = false; return; }
                mbar_arrive_expect_tx(&sh->full_v[s], 2 * KP);
                tma_load_4d(sV + s * 2 * KP, &vmap, &sh->full_v[s], 0, j * BN, g * NB, b);
                tma_load_4d(sV + s * 2 * KP + KP, &vmap, &sh->full_v[s], 0, j * BN, g * NB, B + b);
                ++n_v;
            };
            const int first = n_tiles < 3 ? n_tiles : 3;
            for (int j = 0; j < first; ++j) load_k(j);
            // V's slots are the query tile's until every row thread has its row in TMEM
            if (!fwait(&sh->a_ready, 0, sh)) fgive_up(sh, 41), live = false;
            for (int j = 0; live && j < first; ++j) load_v(j);
            prefetch_next_q();
            for (int j = 3; live && j < n_tiles; ++j) {
                load_k(j);
                if (live) load_v(j);
            }
            if (sh->abort) {
                // let the copies in flight land before the CTA's shared memory goes away
                mbar_wait(&sh->q_full, 0);
                for (int j = (n_k > 3 ? n_k - 3 : 0); j < n_k; ++j) mbar_wait(&sh->full_k[j % 3], (uint32_t)((j / 3) & 1));
                for (int j = (n_v > 3 ? n_v - 3 : 0); j < n_v; ++j) mbar_wait(&sh->full_v[j % 3], (uint32_t)((j / 3) & 1));
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t id_s = idesc_f16(128, BN, false, false);
            constexpr uint32_t id_o = idesc_f16(128, D, false, true);
            bool ok = fwait(&sh->a_ready, 0, sh);
            if (!ok) fgive_up(sh, 42);
            tc_fence_after();
            const uint32_t k_u32 = smem_u32(sK), v_u32 = smem_u32(sV);
            // S of tile j into buffer j & 1
            auto issue_qk = [&](int j) -> bool {
                const int s = j % 3;
                if (!fwait(&sh->full_k[s], (uint32_t)((j / 3) & 1), sh)) return false;
                tc_fence_after();
                const uint32_t kh = k_u32 + (uint32_t)(s * 2 * KP);
                const uint64_t bkh = desc_kmajor(kh), bkl = desc_kmajor(kh + KP);
                const uint32_t cS = cS0 + (j & 1) * BN;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t bo = (uint32_t)((kk >> 2) * (BN * 128) + (kk & 3) * 32);
                    const uint64_t dkh = desc_advance(bkh, bo), dkl = desc_advance(bkl, bo);
                    mma_ts_f16(tmem + cS, tmem + cQh + kk * 8, dkh, id_s, kk > 0);
                    mma_ts_f16(tmem + cS, tmem + cQh + kk * 8, dkl, id_s, 1);
                    mma_ts_f16(tmem + cS, tmem + cQl + kk * 8, dkh, id_s, 1);
                }
                mma_commit(&sh->free_k[s]);
                mma_commit(&sh->s_full[j & 1]);
                return true;
            };
            if (ok && !issue_qk(0)) { fgive_up(sh, 43); ok = false; }
            if (ok && n_tiles > 1 && !issue_qk(1)) { fgive_up(sh, 43); ok = false; }
            for (int j = 0; ok && j < n_tiles; ++j) {
                const int s = j % 3, set = j & 1;
                if (!fwait(&sh->p_full[set], (uint32_t)((j >> 1) & 1), sh) ||
                    !fwait(&sh->full_v[s], (uint32_t)((j / 3) & 1), sh)) { fgive_up(sh, 44); break; }
                tc_fence_after();
                const uint32_t vh = v_u32 + (uint32_t)(s * 2 * KP);
                const uint64_t mvh = desc_mnmajor_16b(vh, BN * 128), mvl = desc_mnmajor_16b(vh + KP, BN * 128);
                const uint32_t cS = cS0 + set * BN, cO = cO0 + set * D;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint32_t ac = (uint32_t)(32 * (kk >> 1) + (kk & 1) * 8);
                    const uint64_t dvh = desc_advance(mvh, kk * 2048), dvl = desc_advance(mvl, kk * 2048);
                    mma_ts_f16(tmem + cO, tmem + cS + ac, dvh, id_o, (j > 1 || kk > 0) ? 1 : 0);
                    mma_ts_f16(tmem + cO, tmem + cS + ac, dvl, id_o, 1);
                    mma_ts_f16(tmem + cO, tmem + cS + ac + 16, dvh, id_o, 1);
                }
                mma_commit(&sh->free_v[s]);
                mma_commit(&sh->pv_done[set]);
                // completes once, after the last P.V: a barrier that counts tiles may be two phases ahead
                // of a row thread by the time it gets there, which a parity wait cannot tell apart
                if (j == n_tiles - 1) mma_commit(&sh->all_done);
                // S(j+2) overwrites the P tile this P.V has just read
                if (j + 2 < n_tiles && !issue_qk(j + 2)) { fgive_up(sh, 43); break; }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ softmax rows: set `set` owns
        // the key tiles of its parity, with a reference maximum, a sum and an O accumulator of its own;
        // the two partial softmaxes are merged at the end.  Nothing a set does waits on the other's tile.
        const int tid = threadIdx.x & 127, set = threadIdx.x >> 7;
        const int t = t0 + tid;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        bool ok = true;
        {
            // this thread's row of Q's hi (set 0) or lo (set 1) plane, out of the 128-byte-swizzled staging tile
            if (!__all_sync(0xffffffffu, fwait(&sh->q_full, 0, sh))) fgive_up(sh, 49), ok = false;
            const uint8_t *src = sV + set * 2 * KP + tid * 128;
#pragma unroll
            for (int kb = 0; kb < NB; ++kb) {
                uint32_t r[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v4 = *reinterpret_cast<const uint4 *>(src + kb * (128 * 128) + ((c ^ (tid & 7)) << 4));
                    r[4 * c] = v4.x, r[4 * c + 1] = v4.y, r[4 * c + 2] = v4.z, r[4 * c + 3] = v4.w;
                }
                tmem_st32(tmem + lane_base + (set == 0 ? cQh : cQl) + kb * 32, r);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->a_ready);
        }
        const float cs = p.scale_log2 / (mq * mk);
        const uint32_t cS = cS0 + set * BN, cO = cO0 + set * D;
        float m_ref = -INFINITY, l = 0.f;
        for (int j = set; ok && j < n_tiles; j += 2) {
            if (!__all_sync(0xffffffffu, fwait(&sh->s_full[set], (uint32_t)((j >> 1) & 1), sh))) {
                fgive_up(sh, 45);
                ok = false;
                break;
            }
            tc_fence_after();
            const int s0 = j * BN;
            const bool diag = (s0 + BN - 1 > t0) && !ZT_DEFECT(1);
            uint32_t r0[32], r1[32];
            tmem_ld32(tmem + lane_base + cS, r0);
            tmem_ld32(tmem + lane_base + cS + 32, r1);
            tmem_wait_ld();
            float mt = -INFINITY;
            if (diag) mt = row_max32<true>(r1, s0 + 32, t, row_max32<true>(r0, s0, t, mt));
            else mt = row_max32<false>(r1, s0 + 32, t, row_max32<false>(r0, s0, t, mt));
            mt *= cs;  // cs > 0
            float factor = 1.f;
            if ((mt > m_ref + kRescaleThreshold || m_ref == -INFINITY) && mt != -INFINITY) {
                factor = (m_ref == -INFINITY) ? 0.f : ex2(m_ref - mt);
                m_ref = mt;
            }
            if (ZT_DEFECT(3) && j > 0) factor = 1.f;
            l *= factor;
            if (j > 1 && __any_sync(0xffffffffu, factor != 1.f)) {
                // this set's O may only be touched once its previous P.V (tile j-2) has retired
                if (!__all_sync(0xffffffffu, fwait(&sh->pv_done[set], (uint32_t)(((j >> 1) - 1) & 1), sh))) {
                    fgive_up(sh, 46);
                    ok = false;
                    break;
                }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem + lane_base + cO + c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
                    tmem_st32(tmem + lane_base + cO + c, r);
                }
            }
            // l is kept in P's units (times kPScale), like O
            const float off = ((m_ref == -INFINITY) ? 0.f : m_ref) - 7.0f;  // log2 kPScale
            float psum;
            {
                uint32_t ph[16], pl[16];
                psum = diag ? row_exp32<true>(r0, s0, t, cs, off, ph, pl) : row_exp32<false>(r0, s0, t, cs, off, ph, pl);
                tmem_st16(tmem + lane_base + cS, ph);
                tmem_st16(tmem + lane_base + cS + 16, pl);
                psum += diag ? row_exp32<true>(r1, s0 + 32, t, cs, off, ph, pl) : row_exp32<false>(r1, s0 + 32, t, cs, off, ph, pl);
                tmem_st16(tmem + lane_base + cS + 32, ph);
                tmem_st16(tmem + lane_base + cS + 48, pl);
            }
            l += psum;
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->p_full[set]);
        }
        // ---- merge the two partial softmaxes
        sh->fin_m[set][tid] = m_ref;
        sh->fin_l[set][tid] = l;
        asm volatile("bar.sync 1, 256;" ::: "memory");  // the 256 softmax threads
        if (ok && !__all_sync(0xffffffffu, fwait(&sh->all_done, 0, sh))) {
            fgive_up(sh, 48);
            ok = false;
        }
        // The merged rows go to global memory through shared memory (K's slots: every tile has been consumed
        // once all_done completes): a thread owns a row in TMEM, and 32 rows per store instruction would cost
        // 32 memory transactions each; written back a row (or two) per instruction they cost four.
        constexpr int CH = D / 4;  // 16-byte chunks per row; chunk c of row r sits at chunk c ^ (r & (CH - 1))
        if (ok) {
            tc_fence_after();
            const bool two = n_tiles > 1;  // set 1 has an accumulator only then
            const float m0 = sh->fin_m[0][tid], l0 = sh->fin_l[0][tid];
            const float m1 = two ? sh->fin_m[1][tid] : -INFINITY, l1 = two ? sh->fin_l[1][tid] : 0.f;
            const float mm = fmaxf(m0, m1);  // m0 is finite: key 0 is visible to every row
            const float w0 = ex2(m0 - mm), w1 = (m1 == -INFINITY) ? 0.f : ex2(m1 - mm);
            const float lsum = w0 * l0 + w1 * l1;
            const float inv = 1.f / (lsum * mv);  // lsum, like O, carries kPScale
            const float f0 = w0 * inv, f1 = w1 * inv;
            // set s merges columns [s D/2, (s+1) D/2) of the row
            uint8_t *srow = sK + tid * (D * 4);
#pragma unroll 1
            for (int c = 0; c < D / 2; c += 32) {
                uint32_t ra[32], rb[32];
                tmem_ld32(tmem + lane_base + cO0 + set * (D / 2) + c, ra);
                if (two) tmem_ld32(tmem + lane_base + cO0 + D + set * (D / 2) + c, rb);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 o4;
                    o4.x = __uint_as_float(ra[i]) * f0, o4.y = __uint_as_float(ra[i + 1]) * f0;
                    o4.z = __uint_as_float(ra[i + 2]) * f0, o4.w = __uint_as_float(ra[i + 3]) * f0;
                    if (two && w1 != 0.f) {
                        o4.x += __uint_as_float(rb[i]) * f1, o4.y += __uint_as_float(rb[i + 1]) * f1;
                        o4.z += __uint_as_float(rb[i + 2]) * f1, o4.w += __uint_as_float(rb[i + 3]) * f1;
                    }
                    const int ch = (set * (D / 2) + c + i) >> 2;
                    *reinterpret_cast<float4 *>(srow + ((ch ^ (tid & (CH - 1))) << 4)) = o4;
                }
            }
            if (set == 0 && p.lse && t < p.T)
                p.lse[((long long)b * p.T + t) * p.n_heads + h] = (mm + log2f(lsum) - 7.0f) * kLn2;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (!sh->abort) {
            constexpr int RPI = 32 / CH;  // rows per store instruction
            const int lane = threadIdx.x & 31;
            const int ch = lane & (CH - 1);
            const long long wo = (long long)p.n_heads * p.dim_out;
            const float mo = p.o_planes ? out_plane_mult(p, b) : 1.f;
#pragma unroll 4
            for (int i = 0; i < 16; i += RPI) {
                const int r = warp * 16 + i + lane / CH;
                const float4 o4 = *reinterpret_cast<const float4 *>(sK + r * (D * 4) + ((ch ^ (r & (CH - 1))) << 4));
                if (t0 + r < p.T && ch * 4 < p.dim_out)  // (a padded tile's upper columns are not the tensor's)
                    store_out4(p, ((long long)b * p.T + t0 + r) * wo + (long long)h * p.dim_out + ch * 4, o4, mo);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, 512);
}


struct Workspace {
    uint32_t *amax_q, *amax_k, *amax_v;
    __half *q_planes, *k_planes, *v_planes;
    size_t total_bytes, amax_bytes;
};

inline Workspace workspace(void *base, int batch, int T, int n_heads, int n_kv_heads, int dim) {
    Workspace w{};
    const size_t n_amax = (size_t)batch * n_kv_heads;
    w.amax_bytes = (3 * n_amax * sizeof(uint32_t) + 1023) / 1024 * 1024;
    auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
    const size_t qh = (size_t)2 * batch * T * n_heads * dim * sizeof(__half);
    const size_t kh = (size_t)2 * batch * T * n_kv_heads * dim * sizeof(__half);
    char *c = static_cast<char *>(base);
    w.amax_q = reinterpret_cast<uint32_t *>(c), w.amax_k = w.amax_q + n_amax, w.amax_v = w.amax_k + n_amax;
    size_t off = w.amax_bytes;
    w.q_planes = reinterpret_cast<__half *>(c + off), off += up(qh);
    w.k_planes = reinterpret_cast<__half *>(c + off), off += up(kh);
    w.v_planes = reinterpret_cast<__half *>(c + off), off += up(kh);
    w.total_bytes = off;
    return w;
}

template <int D>
inline int launch_d(const CUtensorMap &kmap, const CUtensorMap &vmap, const CUtensorMap &qmap, const Params &p,
                    cudaStream_t stream) {
    size_t smem = 12 * (size_t)(64 * D * 2) + sizeof(Shared) + 1024;
    if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: it allocates all of TMEM
    if (optin_smem((const void *)attn_fwd_tc16<D>, smem)) return 1;
    const dim3 grid((unsigned)((p.T + 127) / 128), (unsigned)p.n_heads, (unsigned)p.batch);
    return ZT_LAUNCH("attn_fwd_tc16", stream, (attn_fwd_tc16<D><<<grid, kThreads, smem, stream>>>(kmap, vmap, qmap, p)));
}

// (tc_fwd16x.cuh)
inline int launch_x(const CUtensorMap &kmap, const CUtensorMap &vmap, const CUtensorMap &qmap, const Params &p,
                    cudaStream_t stream);
// (tc_fwd16g.cuh)
template <int D>
inline int launch_g_d(const CUtensorMap &kmap, const CUtensorMap &vmap, const CUtensorMap &qmap, const Params &p,
                      cudaStream_t stream);

}  // namespace tcf16

inline size_t tc_fwd16_workspace_bytes(int batch, int T, int n_heads, int n_kv_heads, int dim) {
    return tcf16::workspace(nullptr, batch, T, n_heads, n_kv_heads, tc_tile_dim(dim)).total_bytes;
}

inline bool tc_fwd16_supported(int batch, int T, int dim, int q_offset, int n_keys, const void *q, const void *k,
                               const void *v, const void *out) {
    if (!(dim == 32 || dim == 64 || dim == 96 || dim == 128 || dim == 192 || dim == 256) || q_offset != 0 || n_keys != T ||
        T < 128 || batch < 1)
        return false;
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!al(q) || !al(k) || !al(v) || !al(out)) return false;
    const DeviceInfo *d = device_info();
    return d && d->cc_major == 10 && get_encode_tiled() != nullptr;
}

// `in_backward_workspace`: lay the planes out where the backward's workspace keeps them (tc_bwd.cuh
// bwd_workspace), so that a backward given the same workspace can use them as they are.
// out_planes (optional): where the kernel also leaves out as f16 hi/lo planes, [2][batch][T][n_heads * dim] halves.
inline int launch_fwd_tc16(const float *q, const float *k, const float *v, float *out, float *lse, void *ws,
                           int batch, int T, int n_heads, int n_kv_heads, int dim, cudaStream_t stream,
                           const float2 *rope = nullptr, bool in_backward_workspace = false, int variant = 0,
                           __half *out_planes = nullptr, const PeerList *out_peers = nullptr) {
    using namespace tcb;
    const int td = tc_tile_dim(dim);  // the kernel's D; the planes' head width (head_dim 32 is zero-padded to 64)
    tcf16::Workspace w = tcf16::workspace(ws, batch, T, n_heads, n_kv_heads, td);
    if (in_backward_workspace) {
        const BwdWorkspace bw = bwd_workspace(ws, batch, T, n_heads, n_kv_heads, td);
        w.amax_q = bw.amax_q, w.amax_k = bw.amax_k, w.amax_v = bw.amax_v;  // contiguous; amax_do follows
        w.amax_bytes = 3 * (size_t)batch * n_kv_heads * sizeof(uint32_t);
        w.q_planes = bw.q_planes, w.k_planes = bw.k_planes, w.v_planes = bw.v_planes;
    }
    const int group = n_heads / n_kv_heads;
    const int wq_src = n_heads * dim, wkv_src = n_kv_heads * dim;
    const int wkv = n_kv_heads * td;
    if (cudaMemsetAsync(w.amax_q, 0, w.amax_bytes, stream) != cudaSuccess) {
        cudaGetLastError();
        return refuse("could not clear the forward workspace header");
    }
    PrepassArgs pa{};
    pa.n = 3, pa.batch = batch, pa.T = T;
    pa.t[0] = {q, w.amax_q, w.q_planes, wq_src, group * dim, dim, td, rope};
    pa.t[1] = {k, w.amax_k, w.k_planes, wkv_src, dim, dim, td, rope};
    pa.t[2] = {v, w.amax_v, w.v_planes, wkv_src, dim, dim, td, nullptr};
    if (launch_prepass(pa, stream)) return 1;
    if (td == 256) {
        // head_dim 256 (and 192 padded to it): one head per CTA, K fetched block by block (attn_fwd_tc16x)
        CUtensorMap kmap, vmap, qmap;
        if (!make_half_tile_map(&kmap, w.k_planes, 2 * batch, T, wkv, 64, 64) ||
            !make_half_tile_map(&vmap, w.v_planes, 2 * batch, T, wkv, td, 64) ||
            !make_half_tile_map(&qmap, w.q_planes, 2 * batch, T, n_heads * td, td, 128))
            return refuse("the TMA tensor maps for the forward could not be encoded.");
        tcf16::Params p{};
        p.q_planes = w.q_planes, p.amax_q = w.amax_q, p.amax_k = w.amax_k, p.amax_v = w.amax_v;
        p.out = out, p.lse = lse;
        p.batch = batch, p.T = T, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads;
        p.dim_out = dim;
        p.o_planes = out_planes, p.o_plane_stride = (long long)batch * T * n_heads * dim;
        if (out_peers) p.out_peers = *out_peers;
        p.scale_log2 = kLog2e / sqrtf((float)dim);
        g_last_path = "tcgen05";
        return tcf16::launch_x(kmap, vmap, qmap, p, stream);
    }
    // variant 0: two heads of a KV group per CTA (attn_fwd_tc16g) when the group has an even number of query heads
    // and that still gives every SM a CTA, one head per CTA (attn_fwd_tc16) otherwise; 1: one head per CTA;
    // 2: two heads per CTA whatever the number of CTAs (the group must be even).
    CUtensorMap kmap, vmap, qmap;
    if (!make_half_tile_map(&kmap, w.k_planes, 2 * batch, T, wkv, td, 64) ||
        !make_half_tile_map(&vmap, w.v_planes, 2 * batch, T, wkv, td, 64) ||
        !make_half_tile_map(&qmap, w.q_planes, 2 * batch, T, n_heads * td, td, 128))
        return refuse("the TMA tensor maps for the forward could not be encoded.");
    tcf16::Params p{};
    p.q_planes = w.q_planes, p.amax_q = w.amax_q, p.amax_k = w.amax_k, p.amax_v = w.amax_v;
    p.out = out, p.lse = lse;
    p.batch = batch, p.T = T, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads;
    p.dim_out = dim;
    p.o_planes = out_planes, p.o_plane_stride = (long long)batch * T * n_heads * dim;
    if (out_peers) p.out_peers = *out_peers;
    p.ahead = device_info() ? device_info()->sm_count : 0;  // one CTA per SM
    p.scale_log2 = kLog2e / sqrtf((float)dim);
    g_last_path = "tcgen05";
    // two heads per CTA halve the number of CTAs: not when that leaves SMs without one
    const long long pair_ctas = (long long)((T + 127) / 128) * (n_heads / 2) * batch;
    if ((variant == 0 || variant == 2) && (n_heads / n_kv_heads) % 2 == 0 &&
        (variant == 2 || (device_info() && pair_ctas >= device_info()->sm_count)))
        return td == 64 ? tcf16::launch_g_d<64>(kmap, vmap, qmap, p, stream) : tcf16::launch_g_d<128>(kmap, vmap, qmap, p, stream);
    return td == 64 ? tcf16::launch_d<64>(kmap, vmap, qmap, p, stream) : tcf16::launch_d<128>(kmap, vmap, qmap, p, stream);
}

}  // namespace zt
