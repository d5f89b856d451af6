// The backward at head_dim 64 and 128 (and 32, 96 padded to them) as ONE tensor-core kernel: dK, dV and dQ from one
// computation of S^T and dP^T.
//
// tc_bwd.cuh computes S and dP twice: once in the dK/dV kernel (a CTA per 128 keys, query tiles walked) and
// once in the dQ kernel (a CTA per 128 query rows, key tiles walked) -- 7 products issued for 5 credited.  Here
// the dK/dV kernel also forms, per step, the partial product dQ^T[d, t] = sum_s K[s, d] dS^T[s, t] over its own
// 128 keys and adds it to dq in memory (red.global.add.v4.f32; dq is zeroed first): 5 products issued.
//
// What had to give, against attn_bwd_dkdv_tc:
//  * TMEM: dQ^T's 64 columns come from S^T's second buffer.  S^T is single-buffered; the tensor core's order per
//    step is  dK(it), first half of dQ^T(it), dP^T(it+1), second half of dQ^T(it), dV(it+1), S^T(it+2): after
//    dP^T(it+1) there are 2400 clocks of issued work for the row threads' dS of step it+1 to hide behind, and
//    3000 between S^T(it+1) and dV(it+1) for their exp.
//  * shared memory: dS^T goes to the tensor core twice -- as the TMEM A operand of dK, and as the B operand of
//    dQ^T, which has to be in shared memory (32 KB, hi and lo); dO's tiles have one slot instead of two.
//  * dq is a sum over key tiles made in memory: its additions come in no fixed order, so dq is reproducible run to
//    run to rounding only (dk, dv bit for bit, as before).  zt_attn_set_path(8) brings the two kernels back.
// Where its time goes (clock stamps of one CTA, 256 steps): 6030 clocks a step, 5200 of them the tensor pipe's own
// (its N = 64 products are bound by operand bandwidth from shared memory, 6 KB per 48 clocks), 830 waits (flushes
// 290, exp 220).  Two things found on the way: an mbarrier arrival AFTER global reductions waits for their round
// trip (1200 clocks a step until the arrival moved ahead of them), and one thread issues a kind::f16 MMA of N <= 64
// with A in TMEM every 52 clocks where two threads together reach the pipe's 32.
//  * the scale of dS: no dQ kernel runs first to measure the largest |dS| of a KV group.  dS is scaled per
//    query row (column of dS^T), as the dQ kernel did, and the row's factor is moved onto Q for dK: the Q tiles
//    this kernel reads are the row-scaled copy (tc_bwd_wide.cuh: wide_qscaled_kernel), row t divided by a power
//    of two rel(t) in [1, 2^12].  S^T = K Q~^T is multiplied back per column by the row threads (exact), dK is
//    sum_t (dS cq(t)) (Q / rel(t)) with one scale, dQ^T's column t leaves times 1 / cq(t).
#pragma once

#include "tc_bwd_wide.cuh"

namespace zt {
namespace tcf {

using namespace tc;
using namespace tcb;
using tcw::wide_group_scale;
using tcw::wide_row_scale;

struct FusedShared {
    uint64_t full_q[2], free_q[2], full_g, free_g;
    uint64_t k_full, a_ready, st_full, dp_full, p_ready, ds_ready, dq_done, dq_free, ld_ready, flush_ready, flush_done, all_done;
    uint32_t tmem_base;
    volatile int abort;
    float lse2[2][64], dels[2][64], csc[2][64], c1c[2][64];  // [buffer][query row of the step]
};
__device__ __forceinline__ bool fwait(uint64_t *bar, uint32_t parity, FusedShared *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void fgive_up(FusedShared *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}
// K hi, K lo, V lo; dS hi + lo (32 KB); two Q slots and one dO slot (each 32 KB at head_dim 128)
template <int D>
__host__ __device__ constexpr size_t fused_smem_bytes() {
    return 3 * (size_t)(128 * D * 2) + 2 * (size_t)(128 * 128) + 6 * (size_t)(64 * D * 2) + sizeof(FusedShared);
}

// grid (n_kv_heads, ceil(T / 128), batch), 608 threads: 16 row warps, a TMA warp, two MMA warps.
constexpr int kFusedThreads = (kKvRowWarps + 3) * 32;
template <int D>
__global__ void __launch_bounds__(kFusedThreads, 1)
    attn_bwd_fused_tc(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                      const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap gmap,
                      const BwdParams p) {
    static_assert(D == 64 || D == 128, "tile widths of this kernel");
    constexpr int NB = D / 64, W2 = D / 2, BQ = 64;
    constexpr int KP = 128 * D * 2, QP = BQ * D * 2;  // bytes of one plane of a K tile / a query tile
    constexpr int cVh = 0, cST = 64, cDPT = 128, cDQT = 192, cDV = 256, cDK = 256 + D;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sKh = smem, *sKl = smem + KP, *sVl = smem + 2 * KP;  // V's hi plane sits in TMEM
    constexpr int DSP = 128 * 128;  // bytes of one plane of dS^T: 128 key rows of 64 halves
    uint8_t *sDS = smem + 3 * KP;                                 // dS^T hi (16 KB), lo (16 KB): rows are keys
    uint8_t *sQ = sDS + 2 * DSP;                                  // slot s: Qh, Ql at sQ + s * 2 QP + {0, 1} QP
    uint8_t *sG = sQ + 2 * 2 * QP;                                // dOh, dOl
    FusedShared *sh = reinterpret_cast<FusedShared *>(sG + 2 * QP);

    const int warp = threadIdx.x >> 5;
    const int g = blockIdx.x, kt = (int)blockIdx.y, b = blockIdx.z;
    const int group = p.n_heads / p.n_kv_heads;
    const int s0 = kt * 128;
    const int n_q = (p.T + BQ - 1) / BQ, qi0 = s0 / BQ;
    const int per_head = n_q - qi0;
    const int n_it = group * per_head;
    const int B = p.batch;
    Walk walk(group, per_head, qi0, n_q);

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) mbar_init(&sh->full_q[i], 1), mbar_init(&sh->free_q[i], 1);
        mbar_init(&sh->full_g, 1), mbar_init(&sh->free_g, 2);  // (freed by two readers: dP^T and dV)
        mbar_init(&sh->k_full, 1);
        mbar_init(&sh->a_ready, kKvRowWarps);
        mbar_init(&sh->st_full, 1);
        mbar_init(&sh->dp_full, 1);
        mbar_init(&sh->p_ready, kKvRowWarps);
        mbar_init(&sh->ds_ready, kKvRowWarps);
        mbar_init(&sh->dq_done, 1);
        mbar_init(&sh->dq_free, kKvRowWarps);
        mbar_init(&sh->ld_ready, kKvRowWarps);
        mbar_init(&sh->flush_ready, 2);  // (dK's issuer and dV's)
        mbar_init(&sh->flush_done, kKvRowWarps);
        mbar_init(&sh->all_done, 2);
        sh->abort = (smem_u32(smem) & 1023u) ? 60 : 0;
        if (sh->abort) atomicMax(&g_tc_status, 60);
        mbar_fence_init();
    }
    if (warp == kKvRowWarps + 1) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    const int bg = b * p.n_kv_heads + g;
    const float mq = block_mult(p.amax_q[bg]), mk = block_mult(p.amax_k[bg]);
    const float mv = block_mult(p.amax_v[bg]), mdo = block_mult(p.amax_do[bg]);
    const uint32_t rn_bits = p.dsmax[bg], vn_bits = p.vnmax[bg];  // (the header's last array holds max |dout row| here)
    const float cmin = wide_group_scale(rn_bits, vn_bits);

    if (warp == kKvRowWarps) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one() && !sh->abort) {
            tma_prefetch_desc(&kmap), tma_prefetch_desc(&vmap), tma_prefetch_desc(&qmap), tma_prefetch_desc(&gmap);
            mbar_arrive_expect_tx(&sh->k_full, 3 * KP);
            tma_load_4d(sKh, &kmap, &sh->k_full, 0, s0, g * NB, b);
            tma_load_4d(sKl, &kmap, &sh->k_full, 0, s0, g * NB, B + b);
            tma_load_4d(sVl, &vmap, &sh->k_full, 0, s0, g * NB, B + b);
            int n_ql = 0, n_gl = 0;  // tiles issued
            bool live = true;
            Walk wq = walk, wg = walk;
            auto load_q = [&]() {  // Q tile of step n_ql
                const int j = n_ql, s = j & 1;
                // (its slot was last read by dK(j - 2))
                if (j >= 2 && !fwait(&sh->free_q[s], (uint32_t)((((j >> 1) - 1) & 1)), sh)) { fgive_up(sh, 61), live = false; return; }
                const int h = g * group + wq.hh, row = wq.qi * BQ;
                mbar_arrive_expect_tx(&sh->full_q[s], 2 * QP);
                tma_load_4d(sQ + s * 2 * QP, &qmap, &sh->full_q[s], 0, row, h * NB, b);
                tma_load_4d(sQ + s * 2 * QP + QP, &qmap, &sh->full_q[s], 0, row, h * NB, B + b);
                ++n_ql, wq.next();
            };
            auto load_g = [&]() {  // dO tile of step n_gl
                const int j = n_gl;
                // (the one slot was last read by dV(j - 1))
                if (j >= 1 && !fwait(&sh->free_g, (uint32_t)((j - 1) & 1), sh)) { fgive_up(sh, 61), live = false; return; }
                const int h = g * group + wg.hh, row = wg.qi * BQ;
                mbar_arrive_expect_tx(&sh->full_g, 2 * QP);
                tma_load_4d(sG, &gmap, &sh->full_g, 0, row, h * NB, b);
                tma_load_4d(sG + QP, &gmap, &sh->full_g, 0, row, h * NB, B + b);
                ++n_gl, wg.next();
            };
            // the tensor core frees dO's slot (dV) before Q's (dK of the next step): ask in that order
            load_q(), load_g();
            if (n_it > 1) load_q();
            for (int it = 0; live && it < n_it; ++it) {
                if (it + 1 < n_it) load_g();
                if (live && it + 2 < n_it) load_q();
            }
            if (sh->abort) {
                // let the copies in flight land before the CTA's shared memory goes away
                mbar_wait(&sh->k_full, 0);
                for (int j = (n_ql > 2 ? n_ql - 2 : 0); j < n_ql; ++j) mbar_wait(&sh->full_q[j & 1], (uint32_t)((j >> 1) & 1));
                if (n_gl > 0) mbar_wait(&sh->full_g, (uint32_t)((n_gl - 1) & 1));
            }
        }
        __syncwarp();
    } else if (warp == kKvRowWarps + 1) {
        // ------------------------------------------------------------------ MMA issuer of the P side: S^T and dV.
        // Two threads issue this kernel's MMAs.  One thread issues a kind::f16 MMA of N <= 64 every ~50 clocks,
        // which for the 96 MMAs of a step is as long as the tensor pipe needs to execute them; two threads
        // together keep the pipe fed.  The split follows the TMEM buffers, so that every overwrite of a buffer
        // is ordered by one thread's issue order: this one owns S^T / P^T (S^T(it+2) after dV(it+1)), the other
        // dP^T / dS^T and dQ^T.  What crosses between them goes through the row threads' barriers.
        if (elect_one()) {
            constexpr uint32_t id_s = idesc_f16(128, BQ, false, false);   // S^T: A = K, B = the query tile, both K-major
            constexpr uint32_t id_a = idesc_f16(128, D, false, true);     // dV: A in TMEM, B the dO tile N-major
            bool ok = !sh->abort && fwait(&sh->k_full, 0, sh);
            if (!ok) fgive_up(sh, 62);
            tc_fence_after();
            const uint64_t bkh = desc_kmajor(smem_u32(sKh)), bkl = desc_kmajor(smem_u32(sKl));
            const uint32_t q_u32 = smem_u32(sQ), g_u32 = smem_u32(sG);
            auto wait_q = [&](int j) -> bool {
                if (!fwait(&sh->full_q[j & 1], (uint32_t)((j >> 1) & 1), sh)) return false;
                tc_fence_after();
                return true;
            };
            // S^T(j) = K Q~^T
            auto issue_st = [&](int j) {
                const uint32_t qh = q_u32 + (uint32_t)((j & 1) * 2 * QP);
                const uint64_t bqh = desc_kmajor(qh), bql = desc_kmajor(qh + QP);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t ao = (uint32_t)((kk >> 2) * (128 * 128) + (kk & 3) * 32);
                    const uint32_t bo = (uint32_t)((kk >> 2) * (BQ * 128) + (kk & 3) * 32);
                    const uint64_t dkh = desc_advance(bkh, ao), dkl = desc_advance(bkl, ao);
                    const uint64_t dqh = desc_advance(bqh, bo), dql = desc_advance(bql, bo);
                    mma_ss_f16(tmem + cST, dkh, dqh, id_s, kk > 0);
                    mma_ss_f16(tmem + cST, dkh, dql, id_s, 1);
                    mma_ss_f16(tmem + cST, dkl, dqh, id_s, 1);
                }
                mma_commit(&sh->st_full);
            };
            // dV(j) += P^T dO: P^T's 16-column windows hold hi halves in their first 8 columns, lo in the last 8.
            // Waits for P^T(j) and for dO(j); `restart`: the accumulators were flushed after step j-1.
            int n_flush = 0;
            auto issue_dv = [&](int j, bool restart, bool flush_after) -> bool {
                if (!fwait(&sh->p_ready, (uint32_t)(j & 1), sh) || !fwait(&sh->full_g, (uint32_t)(j & 1), sh)) return false;
                if (restart && j > 0 && !fwait(&sh->flush_done, (uint32_t)((n_flush - 1) & 1), sh)) return false;
                tc_fence_after();
                const uint64_t mgh = desc_mnmajor_16b(g_u32, BQ * 128), mgl = desc_mnmajor_16b(g_u32 + QP, BQ * 128);
#pragma unroll
                for (int kk = 0; kk < BQ / 16; ++kk) {
                    const uint64_t dgh = desc_advance(mgh, kk * 2048), dgl = desc_advance(mgl, kk * 2048);
                    mma_ts_f16(tmem + cDV, tmem + cST + kk * 16, dgh, id_a, (kk > 0 || !restart) ? 1u : 0u);
                    mma_ts_f16(tmem + cDV, tmem + cST + kk * 16, dgl, id_a, 1);
                    mma_ts_f16(tmem + cDV, tmem + cST + kk * 16 + 8, dgh, id_a, 1);
                }
                mma_commit(&sh->free_g);  // (one of two arrivals: the other issuer's dP^T(j) reads the same tile)
                if (flush_after) {
                    mma_commit(&sh->flush_ready);  // (one of two: the other issuer's dK(j))
                    ++n_flush;
                }
                return true;
            };
            // walk.* describe step `it`; step it+1's restart flag is step it's flush flag
            if (ok) {
                if (!wait_q(0)) { fgive_up(sh, 63); ok = false; }
                else {
                    issue_st(0);
                    if (!issue_dv(0, true, walk.flush)) { fgive_up(sh, 64); ok = false; }
                    else if (n_it > 1) {
                        if (!wait_q(1)) { fgive_up(sh, 63); ok = false; }
                        else issue_st(1);
                    }
                }
            }
            for (int it = 0; ok && it + 1 < n_it; ++it) {
                const bool restart = walk.flush;
                walk.next();  // now step it+1
                if (!issue_dv(it + 1, restart, walk.flush)) { fgive_up(sh, 64); break; }
                if (it + 2 < n_it) {
                    if (!wait_q(it + 2)) { fgive_up(sh, 63); break; }
                    issue_st(it + 2);
                }
            }
            mma_commit(&sh->all_done);  // (one of two)
        }
        __syncwarp();
    } else if (warp == kKvRowWarps + 2) {
        // ------------------------------------------------------------------ MMA issuer of the dS side: dP^T, dK, dQ^T
        if (elect_one()) {
            constexpr uint32_t id_s = idesc_f16(128, BQ, false, false);   // dP^T: A = V (TMEM hi, shared lo), B = the dO tile K-major
            constexpr uint32_t id_a = idesc_f16(128, D, false, true);     // dK: A in TMEM, B the query tile N-major
            constexpr uint32_t id_q = idesc_f16(128, BQ, true, true);     // dQ^T: A = K read M-major, B = dS^T N-major
            bool ok = !sh->abort && fwait(&sh->k_full, 0, sh) && fwait(&sh->a_ready, 0, sh);
            if (!ok) fgive_up(sh, 62);
            tc_fence_after();
            const uint64_t bvl = desc_kmajor(smem_u32(sVl));
            // dQ^T's A operand is the K tile read M-major: M = the head's columns.  At 128 columns that is the two
            // 64-column blocks of one plane (16 KB apart), and a product is the usual three terms.  At 64 columns M
            // would be 64, half a tensor-core tile: instead the hi plane and the lo plane (KP apart) are read as ONE
            // 128-row operand, so that accumulator rows 0..63 hold Kh^T dS and rows 64..127 Kl^T dS; with dS hi and
            // dS lo as the two B operands that is all four terms in two MMAs, and the read-out adds the two halves.
            const uint64_t mkh = desc_mnmajor_16b(smem_u32(sKh), D == 128 ? 128 * 128 : KP);
            const uint64_t mkl = desc_mnmajor_16b(smem_u32(sKl), 128 * 128);
            const uint64_t mdh = desc_mnmajor_16b(smem_u32(sDS), DSP), mdl = desc_mnmajor_16b(smem_u32(sDS) + DSP, DSP);
            const uint32_t q_u32 = smem_u32(sQ), g_u32 = smem_u32(sG);
            // dP^T(j) = V dO^T (waits for dO(j))
            auto issue_dp = [&](int j) -> bool {
                if (!fwait(&sh->full_g, (uint32_t)(j & 1), sh)) return false;
                tc_fence_after();
                const uint64_t bgh = desc_kmajor(g_u32), bgl = desc_kmajor(g_u32 + QP);
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
                mma_commit(&sh->free_g);  // (one of two arrivals: dV(j) reads the same tile)
                mma_commit(&sh->dp_full);
                return true;
            };
            auto issue_dq = [&](int kk0) {
#pragma unroll
                for (int kk = kk0; kk < kk0 + 4; ++kk) {
                    const uint64_t dkh = desc_advance(mkh, kk * 2048), dkl = desc_advance(mkl, kk * 2048);
                    const uint64_t ddh = desc_advance(mdh, kk * 2048), ddl = desc_advance(mdl, kk * 2048);
                    mma_ss_f16(tmem + cDQT, dkh, ddh, id_q, kk > 0);
                    mma_ss_f16(tmem + cDQT, dkh, ddl, id_q, 1);
                    if (D == 128) mma_ss_f16(tmem + cDQT, dkl, ddh, id_q, 1);
                }
            };
            int n_flush = 0;
            if (ok && !issue_dp(0)) { fgive_up(sh, 63); ok = false; }
            for (int it = 0; ok && it < n_it; ++it, walk.next()) {
                if (!fwait(&sh->ds_ready, (uint32_t)(it & 1), sh)) { fgive_up(sh, 64); break; }
                // the accumulators restart at a step after a flush: the row threads must have added them to memory
                if (walk.fresh && it > 0 && !fwait(&sh->flush_done, (uint32_t)((n_flush - 1) & 1), sh)) { fgive_up(sh, 67); break; }
                tc_fence_after();
                {
                    // dK += dS^T Q~
                    const uint32_t qh = q_u32 + (uint32_t)((it & 1) * 2 * QP);
                    const uint64_t mqh = desc_mnmajor_16b(qh, BQ * 128), mql = desc_mnmajor_16b(qh + QP, BQ * 128);
                    const uint32_t acc0 = walk.fresh ? 0u : 1u;
#pragma unroll
                    for (int kk = 0; kk < BQ / 16; ++kk) {
                        const uint64_t dqh = desc_advance(mqh, kk * 2048), dql = desc_advance(mql, kk * 2048);
                        mma_ts_f16(tmem + cDK, tmem + cDPT + kk * 16, dqh, id_a, kk > 0 ? 1u : acc0);
                        mma_ts_f16(tmem + cDK, tmem + cDPT + kk * 16, dql, id_a, 1);
                        mma_ts_f16(tmem + cDK, tmem + cDPT + kk * 16 + 8, dqh, id_a, 1);
                    }
                    mma_commit(&sh->free_q[it & 1]);  // (S^T(it), the tile's other reader, retired before dS(it) could be formed)
                    if (walk.flush) {
                        mma_commit(&sh->flush_ready);  // (one of two: the other issuer's dV(it))
                        ++n_flush;
                    }
                }
                // dQ^T(it) = K^T dS^T over this CTA's 128 keys, in two halves with dP^T(it+1) between them: after
                // dP^T(it+1) this thread still has half of dQ^T(it) to issue while the row threads form dS of step
                // it+1 (the longest hand-off of a step); before it, the first half gives dO's one slot -- released
                // by dV(it) -- the time to fill.  dQ^T's columns must have been read out first.
                if (it >= 1 && !fwait(&sh->dq_free, (uint32_t)((it - 1) & 1), sh)) { fgive_up(sh, 65); break; }
                tc_fence_after();
                issue_dq(0);
                if (it + 1 < n_it && !issue_dp(it + 1)) { fgive_up(sh, 63); break; }
                issue_dq(4);
                mma_commit(&sh->dq_done);  // dS^T(it) in shared memory has been read; dQ^T(it) can be read out
            }
            mma_commit(&sh->all_done);  // (one of two)
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ one thread per key row and
        // 16 of the step's query columns: set `set` handles columns [16 set, 16 set + 16)
        const int tid = threadIdx.x & 127, set = threadIdx.x >> 7;
        const int lane = threadIdx.x & 31;
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
        const float cs_over_cmin = p.scale_log2 / (mq * mk * cmin);
        const float lse_shift = log2f(p.p_scale);
        const float inv_dov = 1.0f / (mdo * mv * p.p_scale);
        // Per query row of a step (fetched one step ahead by the first 64 threads of each set, published
        // through shared memory): set 0 lse, set 1 delta cq / p_scale, set 2 the factor that turns K Q~^T into
        // log2-domain scores (scale_log2 cq / (mq mk cmin)), set 3 the factor of dP^T (cq / (mdo mv p_scale)).
        auto fetch = [&](const Walk &w, int it) -> float {
            if (tid >= 64 || it >= n_it) return 0.f;
            const int t = w.qi * BQ + tid;
            if (t >= p.T) return 0.f;
            const long long idx = ((long long)b * p.T + t) * p.n_heads + g * group + w.hh;
            if (set == 0) return __ldg(p.lse + idx) * kLog2e - lse_shift;
            float cq, rel;
            wide_row_scale(__ldg(p.rnorm + idx), rn_bits, vn_bits, cq, rel);
            if (set == 1) return ZT_DEFECT(13) ? 0.f : __ldg(p.delta + idx) * cq / p.p_scale;
            if (set == 2) return cs_over_cmin * cq;
            return cq * inv_dov;
        };
        auto publish = [&](int it, float v) {
            if (tid < 64) (set == 0 ? sh->lse2 : set == 1 ? sh->dels : set == 2 ? sh->csc : sh->c1c)[it & 1][tid] = v;
            mbar_arrive_warp(&sh->ld_ready);
        };
        Walk ahead = walk;  // one step ahead of `walk`
        publish(0, fetch(ahead, 0));
        ahead.next();
        int n_flush = 0;
        bool ok = true;
        bool saturated = false;
        auto flush_now = [&]() -> bool {
            if (!__all_sync(0xffffffffu, fwait(&sh->flush_ready, (uint32_t)(n_flush & 1), sh))) {
                fgive_up(sh, 66);
                return false;
            }
            tc_fence_after();
            // sets 0, 1 add the halves of dV's columns to memory, sets 2, 3 those of dK's (see attn_bwd_dkdv_tc)
            const int c0 = (set & 1) * (D / 2);
            const uint32_t acc = tmem + lane_base + (set < 2 ? cDV : cDK) + c0;
            const int j8 = lane & 7;
            const long long wo = (long long)p.n_kv_heads * p.dim_out;
            float *dst = (set < 2 ? p.dv : p.dk) + ((long long)b * p.T + (key - j8)) * wo + (long long)g * p.dim_out + c0 + 4 * j8;
            const float f = set < 2 ? 1.0f / (p.p_scale * mdo) : p.scale / (mq * cmin);
#pragma unroll 1
            for (int c = 0; c < D / 2; c += 32) {
                uint32_t r[32];
                tmem_ld32(acc + c, r);
                tmem_wait_ld();
                if (c + 32 >= D / 2) {
                    // the accumulators have been read: the tensor core may restart them while the last columns
                    // are still on their way to memory (an arrival after the stores would wait for them)
                    tc_fence_before();
                    mbar_arrive_warp_relaxed(&sh->flush_done);
                }
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
                if (c0 + c < p.dim_out) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (key - j8 + i >= p.T) continue;
                        float4 a;
                        a.x = __uint_as_float(r[4 * i]) * f, a.y = __uint_as_float(r[4 * i + 1]) * f;
                        a.z = __uint_as_float(r[4 * i + 2]) * f, a.w = __uint_as_float(r[4 * i + 3]) * f;
                        if (n_flush == 0) *reinterpret_cast<float4 *>(dst + i * wo + c) = a;
                        else red_add_v4(dst + i * wo + c, a);
                    }
                }
            }
            ++n_flush;
            return true;
        };
        // dQ^T of the step before: this warp's 32 head columns (TMEM lanes) x this set's 16 query rows.  Four
        // lanes exchange 4 x 4 blocks so that a lane holds four consecutive head columns of ONE query row and
        // adds them with one 16-byte reduction: an instruction covers four query rows' 128-byte runs.
        float fq[4] = {0.f, 0.f, 0.f, 0.f};  // 1 / (the scale of dS) of the previous step's rows 16 set + 4 i + (lane & 3)
        int prev_qi = 0, prev_hh = 0;
        auto drain = [&]() {
            uint32_t r[16];
            tmem_ld16(tmem + lane_base + cDQT + set * 16, r);
            tmem_wait_ld();
            // the columns are free from here on.  (Arriving AFTER the reductions below held the tensor core back
            // for their round trip to L2, 1200 clocks a step.)
            tc_fence_before();
            mbar_arrive_warp_relaxed(&sh->dq_free);
#pragma unroll
            for (int M = 2; M >= 1; M >>= 1) {
                const bool up = (lane & M) != 0;
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    if (m & M) continue;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {  // the four blocks of four query rows
                        const uint32_t send = up ? r[4 * q4 + m] : r[4 * q4 + (m ^ M)];
                        const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, M);
                        if (up) r[4 * q4 + m] = recv;
                        else r[4 * q4 + (m ^ M)] = recv;
                    }
                }
            }
            // now r[4 q4 + e] = dQ^T[head column 4 (lane / 4) + e of this warp's 32][query row 16 set + 4 q4 + (lane & 3)]
            // (at 64 columns the accumulator's rows 64..127 are the K lo half of the same columns: both halves add)
            const int d0 = ((warp & 3) * 32 + (lane & ~3)) & (D - 1);
            if (d0 < p.dim_out) {
                const long long wq = (long long)p.n_heads * p.dim_out;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int t = prev_qi * BQ + set * 16 + 4 * q4 + (lane & 3);
                    if (t >= p.T) continue;
                    float4 a;
                    a.x = __uint_as_float(r[4 * q4]) * fq[q4], a.y = __uint_as_float(r[4 * q4 + 1]) * fq[q4];
                    a.z = __uint_as_float(r[4 * q4 + 2]) * fq[q4], a.w = __uint_as_float(r[4 * q4 + 3]) * fq[q4];
                    red_add_v4(p.dq + ((long long)b * p.T + t) * wq + (long long)(g * group + prev_hh) * p.dim_out + d0, a);
                }
            }
        };
        bool flush_pending = false;
        for (int it = 0; it < n_it; ++it, walk.next(), ahead.next()) {
            const int t0 = walk.qi * BQ + set * 16;
            const uint32_t par = (uint32_t)(it & 1);
            const float nxt = fetch(ahead, it + 1);
            if (!__all_sync(0xffffffffu, fwait(&sh->ld_ready, par, sh) && fwait(&sh->st_full, par, sh))) {
                fgive_up(sh, 68);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t wS = tmem + lane_base + cST + set * 16;
            const uint32_t wP = tmem + lane_base + cDPT + set * 16;
            const float *lse2 = sh->lse2[it & 1] + set * 16, *csc = sh->csc[it & 1] + set * 16;
            float pr[16];
            {
                uint32_t rs[16];
                tmem_ld16(wS, rs);
                tmem_wait_ld();
                uint32_t ph[8], pl[8];
                const int q_first = walk.qi * BQ;
                if ((q_first >= s0 + 127 || ZT_DEFECT(11)) && q_first + BQ <= p.T && s0 + 128 <= p.T) {
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) pr[i + e] = ex2(__uint_as_float(rs[i + e]) * csc[i + e] - lse2[i + e]);
                        split_pack(pr[i], pr[i + 1], ph[i >> 1], pl[i >> 1]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int t = t0 + i + e;
                            const bool vis = (key <= t || ZT_DEFECT(11)) && (t < p.T) && (key < p.T);
                            const float pe = ex2(__uint_as_float(rs[i + e]) * csc[i + e] - lse2[i + e]);
                            pr[i + e] = vis ? pe : 0.f;
                        }
                        split_pack(pr[i], pr[i + 1], ph[i >> 1], pl[i >> 1]);
                    }
                }
                tmem_st8(wS, ph);
                tmem_st8(wS + 8, pl);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp_relaxed(&sh->p_ready);
            // this step's rows for the next iteration's read-out of dQ^T, while dP^T is awaited (the staging buffers
            // of this step stay as they are until every warp has arrived on ds_ready)
            float fq_next[4];
            {
                const float *c1c = sh->c1c[it & 1] + set * 16 + (lane & 3);
                const float kq = p.scale * inv_dov / mk;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const float c = c1c[4 * q4];  // cq / (mdo mv p_scale), a power of two; 0 for rows past the sequence
                    // (the reciprocal of a power of two: its exponent mirrored)
                    fq_next[q4] = c > 0.f ? kq * __uint_as_float(0x7f000000u - __float_as_uint(c)) : 0.f;
                }
            }
            if (!__all_sync(0xffffffffu, fwait(&sh->dp_full, par, sh))) {
                fgive_up(sh, 69);
                ok = false;
                break;
            }
            tc_fence_after();
            {
                const float *c1c = sh->c1c[it & 1] + set * 16, *dels = sh->dels[it & 1] + set * 16;
                uint32_t rd[16];
                tmem_ld16(wP, rd);
                tmem_wait_ld();
                uint32_t dh[8], dl[8];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    float dv[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float x = pr[i + e] * (__uint_as_float(rd[i + e]) * c1c[i + e] - dels[i + e]);
                        saturated |= !(fabsf(x) <= kDsBound);
                        dv[e] = fminf(fmaxf(x, -kDsBound), kDsBound);
                    }
                    split_pack(dv[0], dv[1], dh[i >> 1], dl[i >> 1]);
                }
                tmem_st8(wP, dh);
                tmem_st8(wP + 8, dl);
                // the same 16 values as a row of the B operand of dQ^T: key row `tid`, 16-byte chunks 2 set and
                // 2 set + 1 of its 128 bytes, 128-byte swizzled
                uint8_t *row_h = sDS + tid * 128, *row_l = row_h + DSP;
                const int c0 = ((2 * set) ^ (tid & 7)) << 4, c1 = ((2 * set + 1) ^ (tid & 7)) << 4;
                // (dQ^T(it-1), issued after dP^T(it), may still be reading dS^T(it-1) there)
                if (it >= 1 && !__all_sync(0xffffffffu, fwait(&sh->dq_done, (uint32_t)((it - 1) & 1), sh))) {
                    fgive_up(sh, 59);
                    ok = false;
                    break;
                }
                *reinterpret_cast<uint4 *>(row_h + c0) = make_uint4(dh[0], dh[1], dh[2], dh[3]);
                *reinterpret_cast<uint4 *>(row_h + c1) = make_uint4(dh[4], dh[5], dh[6], dh[7]);
                *reinterpret_cast<uint4 *>(row_l + c0) = make_uint4(dl[0], dl[1], dl[2], dl[3]);
                *reinterpret_cast<uint4 *>(row_l + c1) = make_uint4(dl[4], dl[5], dl[6], dl[7]);
            }
            tmem_wait_st();
            fence_async_smem();
            tc_fence_before();
            mbar_arrive_warp(&sh->ds_ready);
            // dP^T(it) was issued after dK(it-1), which waited for every row warp's dS of step it-1: the staging buffers
            // of step it+1 (last read in step it-1) are free
            if (it + 1 < n_it) publish(it + 1, nxt);
            if (it >= 1) {
                tc_fence_after();  // (dq_done(it-1) was awaited above: dQ^T(it-1) is complete)
                drain();
            }
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) fq[q4] = fq_next[q4];
            prev_qi = walk.qi, prev_hh = walk.hh;
            if (flush_pending) {
                flush_pending = false;
                if (!flush_now()) { ok = false; break; }
            }
            if (walk.flush && it + 1 < n_it) flush_pending = true;
        }
        if (ok && n_it > 0) {
            // the last step: its dQ^T and the final flush wait for the tensor core's last instruction
            if (!__all_sync(0xffffffffu, fwait(&sh->all_done, 0, sh))) fgive_up(sh, 66);
            else {
                tc_fence_after();
                drain();
                flush_now();
            }
        }
        if (__any_sync(0xffffffffu, saturated) && lane == 0) atomicAdd(&g_tc_saturated, 1u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kKvRowWarps + 1) tmem_dealloc(tmem, 512);
}

template <int D>
inline int launch_bwd_fused_d(const CUtensorMap &k128, const CUtensorMap &v128, const CUtensorMap &qs64, const CUtensorMap &g64,
                              const BwdParams &p, cudaStream_t stream) {
    size_t smem = fused_smem_bytes<D>();
    if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: it allocates all of TMEM
    if (optin_smem((const void *)attn_bwd_fused_tc<D>, smem)) return 1;
    const dim3 grid((unsigned)p.n_kv_heads, (unsigned)((p.T + 127) / 128), (unsigned)p.batch);
    return ZT_LAUNCH("attn_bwd_fused_tc", stream, (attn_bwd_fused_tc<D><<<grid, kFusedThreads, smem, stream>>>(k128, v128, qs64, g64, p)));
}
inline int launch_bwd_fused(int td, const CUtensorMap &k128, const CUtensorMap &v128, const CUtensorMap &qs64, const CUtensorMap &g64,
                            const BwdParams &p, cudaStream_t stream) {
    return td == 64 ? launch_bwd_fused_d<64>(k128, v128, qs64, g64, p, stream)
                    : launch_bwd_fused_d<128>(k128, v128, qs64, g64, p, stream);
}

}  // namespace tcf

// Which backward a head_dim-`dim` call takes: the fused kernel at tile widths 64 and 128 (head_dim 32 ... 128) unless the
// two-kernel form is asked for (zt_attn_set_path(8)) or dq must also be stored into peers' memory (the fused
// kernel adds partial sums into dq, which a plain peer store cannot follow).
inline bool tc_bwd_takes_fused(int dim, bool two_kernels, const PeerList *dq_peers) {
    const int td = tc_tile_dim(dim);
    return (td == 64 || td == 128) && !two_kernels && !(dq_peers && dq_peers->n > 0);
}

// delta and the row norms of dout (workspace rnorm) must already be there.  dq, dk, dv are assigned.
// rope_t: only with the two-kernel form (the fused kernel's dq takes its rotation in a pass of its own, by the caller).
inline int launch_bwd_tc(const float *q, const float *k, const float *v, const float *dout, const float *lse,
                         const float *delta, float *dq, float *dk, float *dv, void *workspace, int batch, int T,
                         int n_heads, int n_kv_heads, int dim, cudaStream_t stream, const float2 *rope = nullptr,
                         const float2 *rope_t = nullptr, bool qkv_planes_kept = false, const PeerList *dq_peers = nullptr,
                         bool two_kernels = false) {
    using namespace tcb;
    const int td = tc_tile_dim(dim);  // the kernels' D; the planes' head width
    const bool fused = tc_bwd_takes_fused(dim, two_kernels, dq_peers);
    if (fused && rope_t) return refuse("internal: the fused backward does not rotate dq.");
    const BwdWorkspace w = bwd_workspace(workspace, batch, T, n_heads, n_kv_heads, td);
    const int group = n_heads / n_kv_heads;
    const int wq_src = n_heads * dim, wkv_src = n_kv_heads * dim;
    const int wq = n_heads * td, wkv = n_kv_heads * td;
    // With the planes of q, k, v kept by the forward (and their maxima beside them), only dout is converted.
    const size_t n_amax = (size_t)batch * n_kv_heads;
    // (with kept planes the maxima of q, k, v stay; those of dout, the row norms of v and the header's last array --
    // max |dS| for the two kernels, the largest row norm of dout for the fused one -- start from zero)
    if (cudaMemsetAsync(qkv_planes_kept ? w.amax_do : w.amax_q, 0,
                        qkv_planes_kept ? 3 * n_amax * sizeof(uint32_t) : w.amax_bytes, stream) != cudaSuccess ||
        (fused && cudaMemsetAsync(dq, 0, (size_t)batch * T * wq_src * sizeof(float), stream) != cudaSuccess)) {
        cudaGetLastError();
        return refuse("could not clear the backward workspace header");
    }
    PrepassArgs pa{};
    pa.batch = batch, pa.T = T;
    pa.t[0] = {dout, w.amax_do, w.do_planes, wq_src, group * dim, dim, td, nullptr};
    pa.n = 1;
    if (!qkv_planes_kept) {
        pa.t[1] = {q, w.amax_q, w.q_planes, wq_src, group * dim, dim, td, rope};
        pa.t[2] = {k, w.amax_k, w.k_planes, wkv_src, dim, dim, td, rope};
        pa.t[3] = {v, w.amax_v, w.v_planes, wkv_src, dim, dim, td, nullptr};
        pa.n = 4;
    }
    if (launch_prepass(pa, stream)) return 1;
    {
        const dim3 gv((unsigned)((T + 255) / 256), (unsigned)n_kv_heads, (unsigned)batch);
        if (ZT_LAUNCH("bwd_vnorm_kernel", stream, (bwd_vnorm_kernel<<<gv, 256, 0, stream>>>(v, w.vnmax, T, n_kv_heads, dim))))
            return 1;
    }
    if (fused) {
        // the largest row norm of dout per KV group, then Q's planes with every row divided by its share of the scale of dS
        const dim3 gr((unsigned)((T + 63) / 64), (unsigned)batch);
        if (ZT_LAUNCH("wide_rnmax_kernel", stream, (tcw::wide_rnmax_kernel<<<gr, 256, 0, stream>>>(w.rnorm, w.dsmax, T, n_heads, n_kv_heads))))
            return 1;
        const long long n8 = (long long)batch * T * wq / 8;
        if (ZT_LAUNCH("wide_qscaled_kernel", stream,
                      (tcw::wide_qscaled_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(w.q_planes, w.qs_planes, w.rnorm, w.dsmax,
                                                                                                  w.vnmax, batch, T, n_heads, n_kv_heads, td))))
            return 1;
    }
    BwdMaps m;
    if (!make_half_tile_map(&m.k128, w.k_planes, 2 * batch, T, wkv, td, 128) ||
        !make_half_tile_map(&m.v128, w.v_planes, 2 * batch, T, wkv, td, 128) ||
        !make_half_tile_map(&m.q64, fused ? w.qs_planes : w.q_planes, 2 * batch, T, wq, td, 64) ||
        !make_half_tile_map(&m.g64, w.do_planes, 2 * batch, T, wq, td, 64) ||
        !make_half_tile_map(&m.k64, w.k_planes, 2 * batch, T, wkv, td, 64) ||
        !make_half_tile_map(&m.v64, w.v_planes, 2 * batch, T, wkv, td, 64) ||
        !make_half_tile_map(&m.q128, w.q_planes, 2 * batch, T, wq, td, 128) ||
        !make_half_tile_map(&m.g128, w.do_planes, 2 * batch, T, wq, td, 128))
        return refuse("the TMA tensor maps for the backward could not be encoded.");
    BwdParams p{};
    p.lse = lse, p.delta = delta;
    p.k_planes = w.k_planes, p.v_planes = w.v_planes, p.q_planes = w.q_planes, p.do_planes = w.do_planes;
    p.amax_q = w.amax_q, p.amax_k = w.amax_k, p.amax_v = w.amax_v, p.amax_do = w.amax_do;
    p.rnorm = w.rnorm, p.vnmax = w.vnmax, p.dsmax = w.dsmax;
    p.dq = dq, p.dk = dk, p.dv = dv;
    if (dq_peers) p.dq_peers = *dq_peers;
    p.batch = batch, p.T = T, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads;
    p.dim_out = dim;
    p.rope_t = rope_t;
    p.scale = 1.0f / sqrtf((float)dim), p.scale_log2 = kLog2e / sqrtf((float)dim);
    // P in [0, 1] is split after a multiplication by 2^10 (its low piece then stays a normal f16 down to p ~ 2^-14).
    // dS is scaled inside the kernels (see "The scale of dS" in tc_bwd.cuh and the head of this file).
    p.p_scale = ldexpf(1.0f, 10);
    g_last_path = "tcgen05";
    if (fused) return tcf::launch_bwd_fused(td, m.k128, m.v128, m.q64, m.g64, p, stream);
    return td == 64 ? launch_bwd_tc_d<64>(m, p, stream) : launch_bwd_tc_d<128>(m, p, stream);
}

}  // namespace zt
