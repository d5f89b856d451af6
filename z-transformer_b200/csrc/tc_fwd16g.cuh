// attn_fwd_tc16 for two query heads of one KV group per CTA.
//
// The forward moves 64 KB of K and V (hi and lo planes) from L2 into an SM per 64-key tile and 128 query
// rows, 7 TB/s over the whole chip at the headline shape, and that traffic bounds it as much as its MMAs do.
// The heads of a KV group read the same K and V: here a CTA takes the same 128 query rows of two of them and
// uses every K/V tile it loads twice, which halves the traffic.  The two softmax warp sets, which in
// attn_fwd_tc16 split one head's key tiles between them by parity, take one head each and walk every tile:
//   TMEM  [0, D/2) Qh of head A, [D/2, D) Qh of head B, [D, 2D) O of A, [2D, 3D) O of B, then S/P of A and of B
//         (64 columns each): the Q lo planes, needed by one of the three split terms, stay in shared memory
//         (an SS MMA), which is what makes room for the second head;
//   MMA   S_A(0) S_B(0) | P.V_A(j) S_A(j+1) P.V_B(j) S_B(j+1) | ...: a head's next S goes out behind its P.V,
//         so its softmax runs under the other head's MMAs, as with the parity split;
//   smem  K ring of three slots, V ring of two, two Q lo planes (224 KB at head_dim 128).
// One accumulator per head: no merge at the end.  Needs an even number of query heads per KV group.
#pragma once

#include "tc_fwd16.cuh"

namespace zt {
namespace tcf16 {

struct SharedG {
    uint64_t full_k[3], free_k[3], full_v[2], free_v[2];
    uint64_t a_ready, q_full, ql_full, s_full[2], p_full[2], pv_done[2], staged[2], all_done;
    uint32_t tmem_base;
    volatile int abort;
};
__device__ __forceinline__ bool gwait(uint64_t *bar, uint32_t parity, SharedG *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void ggive_up(SharedG *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
    attn_fwd_tc16g(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                   const __grid_constant__ CUtensorMap qmap, const Params p) {
    constexpr int NB = D / 64, W2 = D / 2, BN = 64;
    constexpr int KP = BN * D * 2;  // bytes of one plane of a key tile; a ring slot is 2 KP (hi, lo)
    constexpr int cQh = 0, cO0 = D, cS0 = 3 * D;  // head s: Qh at cQh + s W2, O at cO0 + s D, S/P at cS0 + 64 s
    extern __shared__ __align__(1024) uint8_t smem_raw[];  // (the swizzled tiles need the alignment; checked below)
    uint8_t *sK = smem_raw, *sV = sK + 6 * KP, *sQl = sV + 4 * KP;  // sQl: Q lo of head A, of head B (2 KP each)
    SharedG *sh = reinterpret_cast<SharedG *>(sQl + 4 * KP);

    const int warp = threadIdx.x >> 5;
    // launch order (x fastest): the head pairs of a sequence, query tile by query tile, late (long) tiles first, so
    // that the last CTAs to start are the shortest (1.5 % faster than a head pair's tiles together)
    const int qt = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int h0 = 2 * (int)blockIdx.x, b = blockIdx.z;
    const int g = h0 / (p.n_heads / p.n_kv_heads);
    const int t0 = qt * 128;
    const int rows_end = (t0 + 128 < p.T) ? t0 + 128 : p.T;
    const int n_tiles = (rows_end + BN - 1) / BN;
    const int B = p.batch;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 3; ++i) mbar_init(&sh->full_k[i], 1), mbar_init(&sh->free_k[i], 1);
        for (int i = 0; i < 2; ++i) mbar_init(&sh->full_v[i], 1), mbar_init(&sh->free_v[i], 1);
        mbar_init(&sh->a_ready, 8);
        mbar_init(&sh->q_full, 1), mbar_init(&sh->ql_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh->s_full[i], 1), mbar_init(&sh->p_full[i], 4), mbar_init(&sh->pv_done[i], 1);
            mbar_init(&sh->staged[i], 4);
        }
        mbar_init(&sh->all_done, 1);
        sh->abort = (smem_u32(smem_raw) & 1023u) ? 40 : 0;
        if (sh->abort) atomicMax(&g_tc_status, 40);
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
        if (elect_one() && !sh->abort) {
            tma_prefetch_desc(&qmap), tma_prefetch_desc(&kmap), tma_prefetch_desc(&vmap);
            // the Q hi planes wait in V's two slots until the row threads have moved them into TMEM
            mbar_arrive_expect_tx(&sh->q_full, 4 * KP);
            tma_load_4d(sV, &qmap, &sh->q_full, 0, t0, h0 * NB, b);
            tma_load_4d(sV + 2 * KP, &qmap, &sh->q_full, 0, t0, (h0 + 1) * NB, b);
            mbar_arrive_expect_tx(&sh->ql_full, 4 * KP);
            tma_load_4d(sQl, &qmap, &sh->ql_full, 0, t0, h0 * NB, B + b);
            tma_load_4d(sQl + 2 * KP, &qmap, &sh->ql_full, 0, t0, (h0 + 1) * NB, B + b);
            int n_k = 0, n_v = 0;  // tiles issued
            bool live = true;
            auto load_k = [&](int j) {
                const int s = j % 3;
                if (j >= 3 && !gwait(&sh->free_k[s], (uint32_t)(((j / 3) & 1) ^ 1), sh)) { ggive_up(sh, 41), live = false; return; }
                mbar_arrive_expect_tx(&sh->full_k[s], 2 * KP);
                tma_load_4d(sK + s * 2 * KP, &kmap, &sh->full_k[s], 0, j * BN, g * NB, b);
                tma_load_4d(sK + s * 2 * KP + KP, &kmap, &sh->full_k[s], 0, j * BN, g * NB, B + b);
                ++n_k;
            };
            auto load_v = [&](int j) {
                const int s = j & 1;
                if (j >= 2 && !gwait(&sh->free_v[s], (uint32_t)(((j >> 1) & 1) ^ 1), sh)) { ggive_up(sh, 41), live = false; return; }
                mbar_arrive_expect_tx(&sh->full_v[s], 2 * KP);
                tma_load_4d(sV + s * 2 * KP, &vmap, &sh->full_v[s], 0, j * BN, g * NB, b);
                tma_load_4d(sV + s * 2 * KP + KP, &vmap, &sh->full_v[s], 0, j * BN, g * NB, B + b);
                ++n_v;
            };
            for (int j = 0; j < 3 && j < n_tiles; ++j) load_k(j);
            if (!gwait(&sh->a_ready, 0, sh)) ggive_up(sh, 41), live = false;
            for (int j = 0; live && j < 2 && j < n_tiles; ++j) load_v(j);
            for (int j = 2; live && j < n_tiles; ++j) {
                if (j + 1 < n_tiles) load_k(j + 1);
                if (live) load_v(j);
            }
            if (sh->abort) {
                // let the copies in flight land before the CTA's shared memory goes away
                mbar_wait(&sh->q_full, 0), mbar_wait(&sh->ql_full, 0);
                for (int j = (n_k > 3 ? n_k - 3 : 0); j < n_k; ++j) mbar_wait(&sh->full_k[j % 3], (uint32_t)((j / 3) & 1));
                for (int j = (n_v > 2 ? n_v - 2 : 0); j < n_v; ++j) mbar_wait(&sh->full_v[j & 1], (uint32_t)((j >> 1) & 1));
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t id_s = idesc_f16(128, BN, false, false);
            constexpr uint32_t id_o = idesc_f16(128, D, false, true);
            bool ok = gwait(&sh->a_ready, 0, sh) && gwait(&sh->ql_full, 0, sh);
            if (!ok) ggive_up(sh, 42);
            tc_fence_after();
            const uint32_t k_u32 = smem_u32(sK), v_u32 = smem_u32(sV);
            // S of head `hd`, tile j (K tile j has landed: the caller waited)
            auto issue_qk = [&](int hd, int j) {
                const uint32_t kh = k_u32 + (uint32_t)((j % 3) * 2 * KP);
                const uint64_t bkh = desc_kmajor(kh), bkl = desc_kmajor(kh + KP);
                const uint64_t bql = desc_kmajor(smem_u32(sQl) + (uint32_t)(hd * 2 * KP));
                const uint32_t cS = cS0 + hd * BN, cQ = cQh + hd * W2;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t ao = (uint32_t)((kk >> 2) * (128 * 128) + (kk & 3) * 32);
                    const uint32_t bo = (uint32_t)((kk >> 2) * (BN * 128) + (kk & 3) * 32);
                    const uint64_t dkh = desc_advance(bkh, bo), dkl = desc_advance(bkl, bo);
                    mma_ts_f16(tmem + cS, tmem + cQ + kk * 8, dkh, id_s, kk > 0);
                    mma_ts_f16(tmem + cS, tmem + cQ + kk * 8, dkl, id_s, 1);
                    mma_ss_f16(tmem + cS, desc_advance(bql, ao), dkh, id_s, 1);
                }
                if (hd == 1) mma_commit(&sh->free_k[j % 3]);
                mma_commit(&sh->s_full[hd]);
            };
            auto k_landed = [&](int j) -> bool {
                if (!gwait(&sh->full_k[j % 3], (uint32_t)((j / 3) & 1), sh)) return false;
                tc_fence_after();
                return true;
            };
            // P.V of head `hd`, tile j (V tile j has landed)
            auto issue_pv = [&](int hd, int j) {
                const uint32_t vh = v_u32 + (uint32_t)((j & 1) * 2 * KP);
                const uint64_t mvh = desc_mnmajor_16b(vh, BN * 128), mvl = desc_mnmajor_16b(vh + KP, BN * 128);
                const uint32_t cS = cS0 + hd * BN, cO = cO0 + hd * D;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint32_t ac = (uint32_t)(32 * (kk >> 1) + (kk & 1) * 8);
                    const uint64_t dvh = desc_advance(mvh, kk * 2048), dvl = desc_advance(mvl, kk * 2048);
                    mma_ts_f16(tmem + cO, tmem + cS + ac, dvh, id_o, (j > 0 || kk > 0) ? 1 : 0);
                    mma_ts_f16(tmem + cO, tmem + cS + ac, dvl, id_o, 1);
                    mma_ts_f16(tmem + cO, tmem + cS + ac + 16, dvh, id_o, 1);
                }
                if (hd == 1) mma_commit(&sh->free_v[j & 1]);
                mma_commit(&sh->pv_done[hd]);
            };
            if (ok && !k_landed(0)) { ggive_up(sh, 43); ok = false; }
            if (ok) issue_qk(0, 0), issue_qk(1, 0);
            for (int j = 0; ok && j < n_tiles; ++j) {
                const uint32_t par = (uint32_t)(j & 1);
                if (!gwait(&sh->p_full[0], par, sh) || !gwait(&sh->full_v[j & 1], (uint32_t)((j >> 1) & 1), sh)) { ggive_up(sh, 44); break; }
                tc_fence_after();
                issue_pv(0, j);
                if (j + 1 < n_tiles) {
                    if (!k_landed(j + 1)) { ggive_up(sh, 43); break; }
                    issue_qk(0, j + 1);  // overwrites the P tile that P.V_A(j) has just read
                }
                if (!gwait(&sh->p_full[1], par, sh)) { ggive_up(sh, 44); break; }
                tc_fence_after();
                issue_pv(1, j);
                if (j == n_tiles - 1) mma_commit(&sh->all_done);  // once, after the last P.V
                if (j + 1 < n_tiles) issue_qk(1, j + 1);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ softmax rows: set `set` owns
        // head h0 + set, every key tile of it
        const int tid = threadIdx.x & 127, set = threadIdx.x >> 7;
        const int lane = threadIdx.x & 31;
        const int h = h0 + set;
        const int t = t0 + tid;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        bool ok = true;
        {
            // this thread's row of its head's Q hi plane, out of the 128-byte-swizzled staging tile
            if (!__all_sync(0xffffffffu, gwait(&sh->q_full, 0, sh))) ggive_up(sh, 49), ok = false;
            const uint8_t *src = sV + set * 2 * KP + tid * 128;
#pragma unroll
            for (int kb = 0; kb < NB; ++kb) {
                uint32_t r[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v4 = *reinterpret_cast<const uint4 *>(src + kb * (128 * 128) + ((c ^ (tid & 7)) << 4));
                    r[4 * c] = v4.x, r[4 * c + 1] = v4.y, r[4 * c + 2] = v4.z, r[4 * c + 3] = v4.w;
                }
                tmem_st32(tmem + lane_base + cQh + set * W2 + kb * 32, r);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->a_ready);
        }
        const float cs = p.scale_log2 / (mq * mk);
        const uint32_t cS = cS0 + set * BN, cO = cO0 + set * D;
        float m_ref = -INFINITY, l = 0.f;
        for (int j = 0; ok && j < n_tiles; ++j) {
            if (!__all_sync(0xffffffffu, gwait(&sh->s_full[set], (uint32_t)(j & 1), sh))) {
                ggive_up(sh, 45);
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
            if (j > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
                // this head's O may only be touched once its previous P.V has retired
                if (!__all_sync(0xffffffffu, gwait(&sh->pv_done[set], (uint32_t)((j - 1) & 1), sh))) {
                    ggive_up(sh, 46);
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
        if (ok && !__all_sync(0xffffffffu, gwait(&sh->all_done, 0, sh))) {
            ggive_up(sh, 48);
            ok = false;
        }
        // The head's rows go to global memory through shared memory (the rings are idle once all_done completes):
        // head A's in the first 4 KP bytes, head B's in the next; a row per store instruction instead of 32.
        constexpr int CH = D / 4;  // 16-byte chunks per row; chunk c of row r sits at chunk c ^ (r & (CH - 1))
        uint8_t *stage = smem_raw + set * 4 * KP;
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
                    *reinterpret_cast<float4 *>(srow + ((ch ^ (tid & (CH - 1))) << 4)) = o4;
                }
            }
            if (p.lse && t < p.T) p.lse[((long long)b * p.T + t) * p.n_heads + h] = (m_ref + log2f(l) - 7.0f) * kLn2;
        }
        mbar_arrive_warp(&sh->staged[set]);
        if (__all_sync(0xffffffffu, gwait(&sh->staged[set], 0, sh)) && !sh->abort) {
            constexpr int RPI = 32 / CH;  // rows per store instruction
            const int ch = lane & (CH - 1);
            const long long wo = (long long)p.n_heads * p.dim_out;
            const float mo = p.o_planes ? out_plane_mult(p, b) : 1.f;
#pragma unroll 4
            for (int i = 0; i < 32; i += RPI) {
                const int r = (warp & 3) * 32 + i + lane / CH;
                const float4 o4 = *reinterpret_cast<const float4 *>(stage + r * (D * 4) + ((ch ^ (r & (CH - 1))) << 4));
                if (t0 + r < p.T && ch * 4 < p.dim_out)  // (a padded tile's upper columns are not the tensor's)
                    store_out4(p, ((long long)b * p.T + t0 + r) * wo + (long long)h * p.dim_out + ch * 4, o4, mo);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, 512);
}

template <int D>
inline int launch_g_d(const CUtensorMap &kmap, const CUtensorMap &vmap, const CUtensorMap &qmap, const Params &p,
                      cudaStream_t stream) {
    size_t smem = 14 * (size_t)(64 * D * 2) + sizeof(SharedG);
    if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: it allocates all of TMEM
    if (optin_smem((const void *)attn_fwd_tc16g<D>, smem)) return 1;
    const dim3 grid((unsigned)(p.n_heads / 2), (unsigned)((p.T + 127) / 128), (unsigned)p.batch);
    return ZT_LAUNCH("attn_fwd_tc16g", stream, (attn_fwd_tc16g<D><<<grid, kThreads, smem, stream>>>(kmap, vmap, qmap, p)));
}

}  // namespace tcf16
}  // namespace zt
