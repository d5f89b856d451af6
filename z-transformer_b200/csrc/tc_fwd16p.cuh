// attn_fwd_tc16 with CTAs that outlive a query tile.
//
// One CTA per SM walks a list of query tiles.  What a CTA of attn_fwd_tc16 pays per query tile besides its
// MMAs -- the wait for its first operands (7-8 K clocks inside a loaded chip), the write-back of its rows and
// the launch of its successor -- is here overlapped with the neighbouring tiles' work:
//   * the K and V rings stream on across query tiles: the next tile's first key tiles are fetched as the
//     current tile's last ones retire;
//   * a staging buffer of its own holds the next tile's Q planes, fetched a whole query tile ahead; at the
//     boundary the row threads move them into TMEM first (the tensor core then computes S(0), S(1) of the next
//     tile), merge the finished tile's rows into the same buffer and write them to memory from there, after
//     which the buffer takes the Q planes of the tile after next.  (At head_dim 128 the buffer's 64 KB come
//     out of V's ring: two slots instead of three.)
// The list: item w is a pair of query tiles (the i-th from the end, then the i-th from the start) of one
// (head, sequence), so every item is the same amount of work and a static round-robin over the CTAs balances.
// Arithmetic, barriers within a tile and TMEM layout are attn_fwd_tc16's; every ring and hand-off barrier runs
// on counters that continue across tiles.
#pragma once

#include "tc_fwd16.cuh"

namespace zt {
namespace tcf16 {

struct SharedP {
    uint64_t full_k[3], free_k[3], full_v[3], free_v[3];
    uint64_t a_ready, s_full[2], p_full[2], pv_done[2], all_done, q_full;
    uint64_t fin_ready, staged, stage_free;  // per tile: both sets' (m, l) published; rows staged; staging read back
    uint32_t tmem_base;
    volatile int abort;
    float fin_m[2][128], fin_l[2][128];
};
__device__ __forceinline__ bool pwait(uint64_t *bar, uint32_t parity, SharedP *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void pgive_up(SharedP *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}

// The CTA's walk over its query tiles; every role steps it in lockstep.
struct TileWalk {
    int n_qt, n_pairs, n_heads, n_items, stride;
    int w, half;          // item, and which tile of its pair
    int qt, h, b;         // the current tile
    bool valid;
    __device__ __forceinline__ TileWalk(int n_qt_, int n_heads_, int n_items_, int first, int stride_)
        : n_qt(n_qt_), n_pairs((n_qt_ + 1) / 2), n_heads(n_heads_), n_items(n_items_), stride(stride_), w(first), half(0) {
        set();
    }
    __device__ __forceinline__ void set() {
        valid = w < n_items;
        if (!valid) return;
        const int i = w % n_pairs, hb = w / n_pairs;
        h = hb % n_heads, b = hb / n_heads;
        qt = half == 0 ? n_qt - 1 - i : i;
    }
    __device__ __forceinline__ void next() {
        const int i = w % n_pairs;
        if (half == 0 && i < n_qt - 1 - i) half = 1;  // (the middle tile of an odd count has no partner)
        else half = 0, w += stride;
        set();
    }
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
    attn_fwd_tc16p(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                   const __grid_constant__ CUtensorMap qmap, const Params p) {
    constexpr int NB = D / 64, BN = 64;
    constexpr int KP = BN * D * 2;  // bytes of one plane of a key tile; a ring slot is 2 KP (hi, lo)
    constexpr int W2 = D / 2;
    constexpr int cQh = 0, cQl = W2, cO0 = D, cS0 = 3 * D;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int NV = D == 128 ? 2 : 3;  // V's ring
    uint8_t *smem = smem_raw;  // 1024-byte aligned by declaration (the swizzled tiles need it); checked below
    uint8_t *sK = smem, *sV = smem + 6 * KP, *sQ = sV + NV * 2 * KP;  // sQ: Q hi, Q lo planes; later the tile's rows
    SharedP *sh = reinterpret_cast<SharedP *>(sQ + 4 * KP);

    const int warp = threadIdx.x >> 5;
    const int B = p.batch;
    const int group = p.n_heads / p.n_kv_heads;
    const int n_qt = (p.T + 127) / 128;
    TileWalk walk(n_qt, p.n_heads, p.n_items, (int)blockIdx.x, (int)gridDim.x);
    auto tiles_of = [&](int qt) {
        const int rows_end = (qt * 128 + 128 < p.T) ? qt * 128 + 128 : p.T;
        return (rows_end + BN - 1) / BN;
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < 3; ++i) {
            mbar_init(&sh->full_k[i], 1), mbar_init(&sh->free_k[i], 1);
            mbar_init(&sh->full_v[i], 1), mbar_init(&sh->free_v[i], 1);
        }
        mbar_init(&sh->a_ready, 8);
        for (int i = 0; i < 2; ++i) mbar_init(&sh->s_full[i], 1), mbar_init(&sh->p_full[i], 4), mbar_init(&sh->pv_done[i], 1);
        mbar_init(&sh->all_done, 1);
        mbar_init(&sh->q_full, 1);
        mbar_init(&sh->fin_ready, 8), mbar_init(&sh->staged, 8), mbar_init(&sh->stage_free, 8);
        sh->abort = (smem_u32(smem_raw) & 1023u) ? 40 : 0;
        if (sh->abort) atomicMax(&g_tc_status, 40);
        mbar_fence_init();
    }
    if (warp == 9) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 8) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            tma_prefetch_desc(&qmap), tma_prefetch_desc(&kmap), tma_prefetch_desc(&vmap);
            int kc = 0, vc = 0;  // K and V tiles issued so far, over all query tiles: load x goes to slot x % ring
            int q_issued = 0;    // query tiles whose Q planes have been requested
            bool live = !sh->abort;
            // a slot is free for load x once the MMAs that read load x - ring have retired
            auto k_slot_free = [&](int x) { return x < 3 || pwait(&sh->free_k[x % 3], (uint32_t)(((x / 3) & 1) ^ 1), sh); };
            auto v_slot_free = [&](int x) { return x < NV || pwait(&sh->free_v[x % NV], (uint32_t)(((x / NV) & 1) ^ 1), sh); };
            auto load_q = [&](const TileWalk &w) {
                mbar_arrive_expect_tx(&sh->q_full, 4 * KP);
                tma_load_4d(sQ, &qmap, &sh->q_full, 0, w.qt * 128, w.h * NB, w.b);
                tma_load_4d(sQ + 2 * KP, &qmap, &sh->q_full, 0, w.qt * 128, w.h * NB, B + w.b);
                ++q_issued;
            };
            // the staging buffer is free for tile n + 1's Q once tile n's Q has left it (a_ready) and, from the second
            // tile on, the rows of tile n - 1 have been written out of it (stage_free, which comes later)
            auto stage_is_free = [&](int n, bool block) -> bool {
                uint64_t *bar = n == 0 ? &sh->a_ready : &sh->stage_free;
                const uint32_t par = (uint32_t)((n == 0 ? 0 : n - 1) & 1);
                return block ? pwait(bar, par, sh) : mbar_try_wait(bar, par);
            };
            if (live && walk.valid) load_q(walk);
            for (int n = 0; live && walk.valid; ++n) {
                const int b = walk.b, g = walk.h / group;
                const int n_tiles = tiles_of(walk.qt);
                TileWalk nxt = walk;
                nxt.next();
                for (int j = 0; live && j < n_tiles; ++j) {
                    if (nxt.valid && q_issued == n + 1 && stage_is_free(n, false)) load_q(nxt);
                    if (!k_slot_free(kc)) { pgive_up(sh, 41), live = false; break; }
                    {
                        const int s = kc % 3;
                        mbar_arrive_expect_tx(&sh->full_k[s], 2 * KP);
                        tma_load_4d(sK + s * 2 * KP, &kmap, &sh->full_k[s], 0, j * BN, g * NB, b);
                        tma_load_4d(sK + s * 2 * KP + KP, &kmap, &sh->full_k[s], 0, j * BN, g * NB, B + b);
                        ++kc;
                    }
                    if (!v_slot_free(vc)) { pgive_up(sh, 41), live = false; break; }
                    {
                        const int s = vc % NV;
                        mbar_arrive_expect_tx(&sh->full_v[s], 2 * KP);
                        tma_load_4d(sV + s * 2 * KP, &vmap, &sh->full_v[s], 0, j * BN, g * NB, b);
                        tma_load_4d(sV + s * 2 * KP + KP, &vmap, &sh->full_v[s], 0, j * BN, g * NB, B + b);
                        ++vc;
                    }
                }
                if (live && nxt.valid && q_issued == n + 1) {
                    if (!stage_is_free(n, true)) pgive_up(sh, 41), live = false;
                    else load_q(nxt);
                }
                walk = nxt;
            }
            if (sh->abort) {
                // let the copies in flight land before the CTA's shared memory goes away
                if (q_issued > 0) mbar_wait(&sh->q_full, (uint32_t)((q_issued - 1) & 1));
                for (int x = (kc > 3 ? kc - 3 : 0); x < kc; ++x) mbar_wait(&sh->full_k[x % 3], (uint32_t)((x / 3) & 1));
                for (int x = (vc > NV ? vc - NV : 0); x < vc; ++x) mbar_wait(&sh->full_v[x % NV], (uint32_t)((x / NV) & 1));
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t id_s = idesc_f16(128, BN, false, false);
            constexpr uint32_t id_o = idesc_f16(128, D, false, true);
            const uint32_t k_u32 = smem_u32(sK), v_u32 = smem_u32(sV);
            int kc = 0, vc = 0;     // K, V tiles consumed before this query tile
            int u0 = 0, u1 = 0;     // uses of each S/P buffer (and O accumulator) before this query tile
            bool ok = true;
            for (int n = 0; ok && walk.valid; ++n, walk.next()) {
                const int n_tiles = tiles_of(walk.qt);
                if (!pwait(&sh->a_ready, (uint32_t)(n & 1), sh)) { pgive_up(sh, 42); break; }
                tc_fence_after();
                auto issue_qk = [&](int j) -> bool {
                    const int x = kc + j, s = x % 3;
                    if (!pwait(&sh->full_k[s], (uint32_t)((x / 3) & 1), sh)) return false;
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
                if (!issue_qk(0)) { pgive_up(sh, 43); break; }
                if (n_tiles > 1 && !issue_qk(1)) { pgive_up(sh, 43); break; }
                for (int j = 0; j < n_tiles; ++j) {
                    const int set = j & 1, x = vc + j, s = x % NV;
                    if (!pwait(&sh->p_full[set], (uint32_t)(((set ? u1 : u0) + (j >> 1)) & 1), sh) ||
                        !pwait(&sh->full_v[s], (uint32_t)((x / NV) & 1), sh)) { pgive_up(sh, 44), ok = false; break; }
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
                    if (j == n_tiles - 1) mma_commit(&sh->all_done);  // once per query tile
                    if (j + 2 < n_tiles && !issue_qk(j + 2)) { pgive_up(sh, 43), ok = false; break; }
                }
                kc += n_tiles, vc += n_tiles;
                u0 += (n_tiles + 1) >> 1, u1 += n_tiles >> 1;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ softmax rows
        const int tid = threadIdx.x & 127, set = threadIdx.x >> 7;
        const int lane = threadIdx.x & 31;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t cS = cS0 + set * BN, cO = cO0 + set * D;
        int uset = 0;  // this set's S/P buffer uses before this query tile, as the MMA warp counts them
        bool ok = true;
        // this thread's row of Q's hi (set 0) or lo (set 1) plane of query tile n, out of its staging slot
        auto q_to_tmem = [&](int n) -> bool {
            if (!__all_sync(0xffffffffu, pwait(&sh->q_full, (uint32_t)(n & 1), sh))) { pgive_up(sh, 49); return false; }
            const uint8_t *src = sQ + set * 2 * KP + tid * 128;
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
            return true;
        };
        if (walk.valid) ok = q_to_tmem(0);
        for (int n = 0; ok && walk.valid; ++n) {
            const int h = walk.h, b = walk.b, g = h / group, t0 = walk.qt * 128;
            const int n_tiles = tiles_of(walk.qt);
            const int t = t0 + tid;
            const float mq = block_mult(p.amax_q[b * p.n_kv_heads + g]), mk = block_mult(p.amax_k[b * p.n_kv_heads + g]);
            const float mv = block_mult(p.amax_v[b * p.n_kv_heads + g]);
            const float cs = p.scale_log2 / (mq * mk);
            float m_ref = -INFINITY, l = 0.f;
            for (int j = set; ok && j < n_tiles; j += 2) {
                const int use = uset + (j >> 1);
                if (!__all_sync(0xffffffffu, pwait(&sh->s_full[set], (uint32_t)(use & 1), sh))) {
                    pgive_up(sh, 45);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const int s0 = j * BN;
                const bool diag = (s0 + BN - 1 > t0);
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
                l *= factor;
                if (j > 1 && __any_sync(0xffffffffu, factor != 1.f)) {
                    // this set's O may only be touched once its previous P.V (tile j-2) has retired
                    if (!__all_sync(0xffffffffu, pwait(&sh->pv_done[set], (uint32_t)((use - 1) & 1), sh))) {
                        pgive_up(sh, 46);
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
            if (!ok) break;
            // ---- merge the two partial softmaxes
            sh->fin_m[set][tid] = m_ref;
            sh->fin_l[set][tid] = l;
            mbar_arrive_warp(&sh->fin_ready);
            if (!__all_sync(0xffffffffu, pwait(&sh->fin_ready, (uint32_t)(n & 1), sh) && pwait(&sh->all_done, (uint32_t)(n & 1), sh))) {
                pgive_up(sh, 48);
                ok = false;
                break;
            }
            tc_fence_after();
            uset += (n_tiles + 1 - set) >> 1;
            constexpr int CH = D / 4;  // 16-byte chunks per row; chunk c of row r sits at chunk c ^ (r & (CH - 1))
            auto stage_row = [&](int r) { return sQ + r * (D * 4); };
            // the next tile's Q goes into TMEM first, so that its S(0), S(1) run while this tile's rows leave; the
            // staging buffer is the finished tile's only after every warp has taken its Q rows out of it
            const float keep_m0 = sh->fin_m[0][tid], keep_l0 = sh->fin_l[0][tid];
            const float keep_m1 = sh->fin_m[1][tid], keep_l1 = sh->fin_l[1][tid];
            walk.next();
            if (walk.valid) {
                if (!q_to_tmem(n + 1)) { ok = false; break; }
                if (!__all_sync(0xffffffffu, pwait(&sh->a_ready, (uint32_t)((n + 1) & 1), sh))) {
                    pgive_up(sh, 48);
                    ok = false;
                    break;
                }
            }
            {
                const float m0 = keep_m0, l0 = keep_l0;
                const float m1 = keep_m1, l1 = keep_l1;  // (every query tile has two key tiles or more)
                const float mm = fmaxf(m0, m1);  // m0 is finite: key 0 is visible to every row
                const float w0 = ex2(m0 - mm), w1 = (m1 == -INFINITY) ? 0.f : ex2(m1 - mm);
                const float lsum = w0 * l0 + w1 * l1;
                const float inv = 1.f / (lsum * mv);  // lsum, like O, carries kPScale
                const float f0 = w0 * inv, f1 = w1 * inv;
                uint8_t *srow = stage_row(tid);
#pragma unroll 1
                for (int c = 0; c < D / 2; c += 32) {
                    uint32_t ra[32], rb[32];
                    tmem_ld32(tmem + lane_base + cO0 + set * (D / 2) + c, ra);
                    tmem_ld32(tmem + lane_base + cO0 + D + set * (D / 2) + c, rb);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float4 o4;
                        o4.x = __uint_as_float(ra[i]) * f0, o4.y = __uint_as_float(ra[i + 1]) * f0;
                        o4.z = __uint_as_float(ra[i + 2]) * f0, o4.w = __uint_as_float(ra[i + 3]) * f0;
                        if (w1 != 0.f) {
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
            tc_fence_before();  // the accumulators have been read: the next tile's P.V may overwrite them
            mbar_arrive_warp(&sh->staged);
            if (!__all_sync(0xffffffffu, pwait(&sh->staged, (uint32_t)(n & 1), sh))) {
                pgive_up(sh, 48);
                ok = false;
                break;
            }
            {
                constexpr int RPI = 32 / CH;  // rows per store instruction
                const int ch = lane & (CH - 1);
                const long long wo = (long long)p.n_heads * p.dim_out;
#pragma unroll 4
                for (int i = 0; i < 16; i += RPI) {
                    const int r = warp * 16 + i + lane / CH;
                    const float4 o4 = *reinterpret_cast<const float4 *>(stage_row(r) + ((ch ^ (r & (CH - 1))) << 4));
                    if (t0 + r < p.T && ch * 4 < p.dim_out)  // (a padded tile's upper columns are not the tensor's)
                        *reinterpret_cast<float4 *>(p.out + ((long long)b * p.T + t0 + r) * wo + (long long)h * p.dim_out + ch * 4) = o4;
                }
            }
            fence_async_smem();  // the staging buffer is next written by TMA
            mbar_arrive_warp(&sh->stage_free);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, 512);
}

template <int D>
inline int launch_p_d(const CUtensorMap &kmap, const CUtensorMap &vmap, const CUtensorMap &qmap, const Params &p,
                      cudaStream_t stream) {
    size_t smem = (size_t)(6 + (D == 128 ? 4 : 6) + 4) * (64 * D * 2) + sizeof(SharedP);
    if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: it allocates all of TMEM
    if (optin_smem((const void *)attn_fwd_tc16p<D>, smem)) return 1;
    const DeviceInfo *d = device_info();
    int ctas = d ? d->sm_count : 1;
    if (ctas > p.n_items) ctas = p.n_items;
    return ZT_LAUNCH("attn_fwd_tc16p", stream, (attn_fwd_tc16p<D><<<dim3((unsigned)ctas), kThreads, smem, stream>>>(kmap, vmap, qmap, p)));
}

}  // namespace tcf16
}  // namespace zt
