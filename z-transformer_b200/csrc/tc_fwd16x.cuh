// attn_fwd_tc16x: the f16-split forward for head widths up to 256 (head_dim 256, and 192 zero-padded to it).
//
// At 256 columns a head no longer fits the layout of attn_fwd_tc16 / tc16g: one O accumulator alone is 256 of
// the 512 TMEM columns, and a 64-key K or V tile (hi and lo planes) is 64 KB.  This kernel keeps their
// arithmetic (S = Qh.Kh + Qh.Kl + Ql.Kh on kind::f16, P scaled by 2^7 and split into f16 pairs written over S,
// O += Ph.Vh + Ph.Vl + Pl.Vh, online softmax in the log2 domain with a lazily moved maximum) and changes
// what the sizes force:
//   CTA    128 query rows of ONE head; 6 warps: four softmax warps (a thread per row, every key tile), TMA, MMA.
//   TMEM   [0, 128) Q hi as the A operand, [128, 384) O, [384, 512) two S/P tiles of 64 columns.
//   smem   Q lo (64 KB; an SS MMA for the Ql.Kh term), ONE K tile and ONE V tile (64 KB each) = 192 KB.
//   K      is a ring of its four 64-column blocks rather than of whole tiles: S contracts over the blocks one
//          after the other, a block is free as soon as its twelve MMAs have retired and the same block of the
//          next tile is fetched into it while the later blocks are still being read.  So S(j+1) can follow
//          S(j) at once although there is room for one K tile only.
//   MMA    S(0) S(1) | P.V(0) S(2) | P.V(1) S(3) | ...: the softmax of tile j+1 runs under P.V(j) and S(j+2).
//          V(j+1) is fetched while S(j+2) runs.
// Per 64-key tile the tensor core issues 48 MMAs of N = 64 for S and 12 of N = 256 for P.V.
// The Q hi tile reaches TMEM through V's slot (TMA, then the row threads); the rows leave through the K and V
// slots (128 KB), a row per store instruction.  Every wait is bounded; a wait that gives up raises g_tc_status.
//
// The backward at these widths has no tensor-core form: dK and dV are two 256-column accumulators, and K, V, Q and
// dO tiles of 64 rows are 64 KB each with their lo planes -- neither fits beside the other.  It stays on the
// CUDA-core kernels.
#pragma once

#include "tc_fwd16.cuh"

namespace zt {
namespace tcf16 {

constexpr int kThreadsX = 6 * 32;

struct SharedX {
    uint64_t full_k[4], free_k[4], full_v, free_v;
    uint64_t a_ready, q_full, ql_full, s_full[2], p_full[2], pv_done, staged, all_done;
    uint32_t tmem_base;
    volatile int abort;
};
__device__ __forceinline__ bool xwait(uint64_t *bar, uint32_t parity, SharedX *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void xgive_up(SharedX *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}

// kmap: K planes with a box of ONE 64-column block x 64 keys; vmap: V planes, four blocks x 64 keys; qmap: Q planes,
// four blocks x 128 rows.
__global__ void __launch_bounds__(kThreadsX, 1)
    attn_fwd_tc16x(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                   const __grid_constant__ CUtensorMap qmap, const Params p) {
    constexpr int D = 256, NB = 4, BN = 64;
    constexpr int KB = BN * 128;        // bytes of one 64-column block of one plane of a key tile (8 KB)
    constexpr int KP = NB * KB;         // one plane of a key tile (32 KB); a K or V tile is 2 KP
    constexpr int QB = 128 * 128;       // one block of one plane of the 128-row query tile (16 KB)
    constexpr int cQh = 0, cO = 128, cS0 = 384;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // K: block c of the tile at sK + c * 2 KB (hi, then lo); V: hi plane, lo plane; Q lo: four blocks
    uint8_t *sK = smem_raw, *sV = sK + 2 * KP, *sQl = sV + 2 * KP;
    SharedX *sh = reinterpret_cast<SharedX *>(sQl + NB * QB);

    const int warp = threadIdx.x >> 5;
    // launch order (x fastest): a head's query tiles, late (long) ones first
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int g = h / (p.n_heads / p.n_kv_heads);
    const int t0 = qt * 128;
    const int rows_end = (t0 + 128 < p.T) ? t0 + 128 : p.T;
    const int n_tiles = (rows_end + BN - 1) / BN;
    const int B = p.batch;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; ++i) mbar_init(&sh->full_k[i], 1), mbar_init(&sh->free_k[i], 1);
        mbar_init(&sh->full_v, 1), mbar_init(&sh->free_v, 1);
        mbar_init(&sh->a_ready, 4);
        mbar_init(&sh->q_full, 1), mbar_init(&sh->ql_full, 1);
        for (int i = 0; i < 2; ++i) mbar_init(&sh->s_full[i], 1), mbar_init(&sh->p_full[i], 4);
        mbar_init(&sh->pv_done, 1);
        mbar_init(&sh->staged, 4);
        mbar_init(&sh->all_done, 1);
        sh->abort = (smem_u32(smem_raw) & 1023u) ? 60 : 0;
        if (sh->abort) atomicMax(&g_tc_status, 60);
        mbar_fence_init();
    }
    if (warp == 5) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    const float mq = block_mult(p.amax_q[b * p.n_kv_heads + g]), mk = block_mult(p.amax_k[b * p.n_kv_heads + g]);
    const float mv = block_mult(p.amax_v[b * p.n_kv_heads + g]);

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one() && !sh->abort) {
            tma_prefetch_desc(&qmap), tma_prefetch_desc(&kmap), tma_prefetch_desc(&vmap);
            // the Q hi plane waits in V's slot until the row threads have moved it into TMEM
            mbar_arrive_expect_tx(&sh->q_full, NB * QB);
            tma_load_4d(sV, &qmap, &sh->q_full, 0, t0, h * NB, b);
            mbar_arrive_expect_tx(&sh->ql_full, NB * QB);
            tma_load_4d(sQl, &qmap, &sh->ql_full, 0, t0, h * NB, B + b);
            int n_k = 0, n_v = 0;  // K blocks and V tiles issued
            bool live = true;
            auto load_k_block = [&](int j, int c) {
                if (j >= 1 && !xwait(&sh->free_k[c], (uint32_t)((j - 1) & 1), sh)) { xgive_up(sh, 61), live = false; return; }
                mbar_arrive_expect_tx(&sh->full_k[c], 2 * KB);
                tma_load_4d(sK + c * 2 * KB, &kmap, &sh->full_k[c], 0, j * BN, g * NB + c, b);
                tma_load_4d(sK + c * 2 * KB + KB, &kmap, &sh->full_k[c], 0, j * BN, g * NB + c, B + b);
                ++n_k;
            };
            auto load_v = [&](int j) {
                if (j >= 1 && !xwait(&sh->free_v, (uint32_t)((j - 1) & 1), sh)) { xgive_up(sh, 61), live = false; return; }
                mbar_arrive_expect_tx(&sh->full_v, 2 * KP);
                tma_load_4d(sV, &vmap, &sh->full_v, 0, j * BN, g * NB, b);
                tma_load_4d(sV + KP, &vmap, &sh->full_v, 0, j * BN, g * NB, B + b);
                ++n_v;
            };
            for (int c = 0; c < NB; ++c) load_k_block(0, c);
            if (!xwait(&sh->a_ready, 0, sh)) xgive_up(sh, 61), live = false;  // V's slot holds Q hi until then
            if (live) load_v(0);
            for (int j = 1; live && j < n_tiles; ++j) {
                for (int c = 0; live && c < NB; ++c) load_k_block(j, c);
                if (live) load_v(j);
            }
            if (sh->abort) {
                // let the copies in flight land before the CTA's shared memory goes away
                mbar_wait(&sh->q_full, 0), mbar_wait(&sh->ql_full, 0);
                for (int i = (n_k > NB ? n_k - NB : 0); i < n_k; ++i) mbar_wait(&sh->full_k[i % NB], (uint32_t)((i / NB) & 1));
                if (n_v > 0) mbar_wait(&sh->full_v, (uint32_t)((n_v - 1) & 1));
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t id_s = idesc_f16(128, BN, false, false);
            constexpr uint32_t id_o = idesc_f16(128, D, false, true);
            bool ok = xwait(&sh->a_ready, 0, sh) && xwait(&sh->ql_full, 0, sh);
            if (!ok) xgive_up(sh, 62);
            tc_fence_after();
            const uint32_t k_u32 = smem_u32(sK), v_u32 = smem_u32(sV), ql_u32 = smem_u32(sQl);
            // S(j) into buffer j & 1, block by block of the contraction
            auto issue_qk = [&](int j) -> bool {
                const uint32_t cS = cS0 + (j & 1) * BN;
#pragma unroll
                for (int c = 0; c < NB; ++c) {
                    if (!xwait(&sh->full_k[c], (uint32_t)(j & 1), sh)) return false;
                    tc_fence_after();
                    const uint64_t bkh = desc_kmajor(k_u32 + (uint32_t)(c * 2 * KB));
                    const uint64_t bkl = desc_kmajor(k_u32 + (uint32_t)(c * 2 * KB + KB));
                    const uint64_t bql = desc_kmajor(ql_u32 + (uint32_t)(c * QB));
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const int kk = c * 4 + ks;
                        const uint64_t dkh = desc_advance(bkh, ks * 32), dkl = desc_advance(bkl, ks * 32);
                        mma_ts_f16(tmem + cS, tmem + cQh + kk * 8, dkh, id_s, kk > 0);
                        mma_ts_f16(tmem + cS, tmem + cQh + kk * 8, dkl, id_s, 1);
                        mma_ss_f16(tmem + cS, desc_advance(bql, ks * 32), dkh, id_s, 1);
                    }
                    mma_commit(&sh->free_k[c]);
                }
                mma_commit(&sh->s_full[j & 1]);
                return true;
            };
            // P.V of tile j
            auto issue_pv = [&](int j) {
                const uint64_t mvh = desc_mnmajor_16b(v_u32, BN * 128), mvl = desc_mnmajor_16b(v_u32 + KP, BN * 128);
                const uint32_t cS = cS0 + (j & 1) * BN;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint32_t ac = (uint32_t)(32 * (kk >> 1) + (kk & 1) * 8);
                    const uint64_t dvh = desc_advance(mvh, kk * 2048), dvl = desc_advance(mvl, kk * 2048);
                    mma_ts_f16(tmem + cO, tmem + cS + ac, dvh, id_o, (j > 0 || kk > 0) ? 1 : 0);
                    mma_ts_f16(tmem + cO, tmem + cS + ac, dvl, id_o, 1);
                    mma_ts_f16(tmem + cO, tmem + cS + ac + 16, dvh, id_o, 1);
                }
                mma_commit(&sh->free_v);
                mma_commit(&sh->pv_done);
            };
            if (ok && !issue_qk(0)) { xgive_up(sh, 63); ok = false; }
            if (ok && n_tiles > 1 && !issue_qk(1)) { xgive_up(sh, 63); ok = false; }
            for (int j = 0; ok && j < n_tiles; ++j) {
                if (!xwait(&sh->p_full[j & 1], (uint32_t)((j >> 1) & 1), sh) || !xwait(&sh->full_v, (uint32_t)(j & 1), sh)) {
                    xgive_up(sh, 64);
                    break;
                }
                tc_fence_after();
                issue_pv(j);
                if (j == n_tiles - 1) mma_commit(&sh->all_done);  // once, after the last P.V
                if (j + 2 < n_tiles && !issue_qk(j + 2)) { xgive_up(sh, 63); break; }  // over the P tile P.V(j) has just read
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ softmax rows: a thread per query row
        const int tid = threadIdx.x, lane = threadIdx.x & 31;
        const int t = t0 + tid;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        bool ok = true;
        {
            // this thread's row of the Q hi plane, out of the 128-byte-swizzled staging tile
            if (!__all_sync(0xffffffffu, xwait(&sh->q_full, 0, sh))) xgive_up(sh, 69), ok = false;
            const uint8_t *src = sV + tid * 128;
#pragma unroll 1
            for (int kb = 0; kb < NB; ++kb) {
                uint32_t r[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v4 = *reinterpret_cast<const uint4 *>(src + kb * QB + ((c ^ (tid & 7)) << 4));
                    r[4 * c] = v4.x, r[4 * c + 1] = v4.y, r[4 * c + 2] = v4.z, r[4 * c + 3] = v4.w;
                }
                tmem_st32(tmem + lane_base + cQh + kb * 32, r);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->a_ready);
        }
        const float cs = p.scale_log2 / (mq * mk);
        float m_ref = -INFINITY, l = 0.f;
        for (int j = 0; ok && j < n_tiles; ++j) {
            if (!__all_sync(0xffffffffu, xwait(&sh->s_full[j & 1], (uint32_t)((j >> 1) & 1), sh))) {
                xgive_up(sh, 65);
                ok = false;
                break;
            }
            tc_fence_after();
            const int s0 = j * BN;
            const uint32_t cS = cS0 + (j & 1) * BN;
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
            if (j > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
                // O may only be touched once the previous P.V has retired
                if (!__all_sync(0xffffffffu, xwait(&sh->pv_done, (uint32_t)((j - 1) & 1), sh))) {
                    xgive_up(sh, 66);
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
            mbar_arrive_warp(&sh->p_full[j & 1]);
        }
        if (ok && !__all_sync(0xffffffffu, xwait(&sh->all_done, 0, sh))) {
            xgive_up(sh, 68);
            ok = false;
        }
        // The rows go to global memory through shared memory (the K and V slots are idle once all_done completes):
        // 128 rows x 1 KB; a row per store instruction instead of 32.
        constexpr int CH = D / 4;  // 16-byte chunks per row (64); chunk c of row r sits at chunk c ^ (r & 31)
        uint8_t *stage = smem_raw;
        if (ok) {
            tc_fence_after();
            const float inv = 1.f / (l * mv);  // l, like O, carries kPScale
            uint8_t *srow = stage + tid * (D * 4);
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                uint32_t ra[32];
                tmem_ld32(tmem + lane_base + cO + c, ra);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 o4;
                    o4.x = __uint_as_float(ra[i]) * inv, o4.y = __uint_as_float(ra[i + 1]) * inv;
                    o4.z = __uint_as_float(ra[i + 2]) * inv, o4.w = __uint_as_float(ra[i + 3]) * inv;
                    const int ch = (c + i) >> 2;
                    *reinterpret_cast<float4 *>(srow + ((ch ^ (tid & 31)) << 4)) = o4;
                }
            }
            if (p.lse && t < p.T) p.lse[((long long)b * p.T + t) * p.n_heads + h] = (m_ref + log2f(l) - 7.0f) * kLn2;
        }
        mbar_arrive_warp(&sh->staged);
        if (__all_sync(0xffffffffu, xwait(&sh->staged, 0, sh)) && !sh->abort) {
            const long long wo = (long long)p.n_heads * p.dim_out;
            const float mo = p.o_planes ? out_plane_mult(p, b) : 1.f;
            // a warp stores its 32 rows; a row is 64 chunks: two instructions of 32 lanes each
#pragma unroll 4
            for (int i = 0; i < 32; ++i) {
                const int r = warp * 32 + i;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int ch = half * 32 + lane;
                    const float4 o4 = *reinterpret_cast<const float4 *>(stage + r * (D * 4) + ((ch ^ (r & 31)) << 4));
                    if (t0 + r < p.T && ch * 4 < p.dim_out)  // (a padded tile's upper columns are not the tensor's)
                        store_out4(p, ((long long)b * p.T + t0 + r) * wo + (long long)h * p.dim_out + ch * 4, o4, mo);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem, 512);
}

inline int launch_x(const CUtensorMap &kmap, const CUtensorMap &vmap, const CUtensorMap &qmap, const Params &p,
                    cudaStream_t stream) {
    const size_t smem = 3 * (size_t)(2 * 64 * 256 * 2) + sizeof(SharedX);  // K tile, V tile, Q lo
    if (optin_smem((const void *)attn_fwd_tc16x, smem)) return 1;
    const dim3 grid((unsigned)((p.T + 127) / 128), (unsigned)p.n_heads, (unsigned)p.batch);
    return ZT_LAUNCH("attn_fwd_tc16x", stream, (attn_fwd_tc16x<<<grid, kThreadsX, smem, stream>>>(kmap, vmap, qmap, p)));
}

}  // namespace tcf16
}  // namespace zt
