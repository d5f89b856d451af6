// Causal GQA attention backward at head_dim 256 (and 192 zero-padded to it) on the tensor cores.
//
// What it computes: autograd.attentionBackward (src/autograd.zig:636-842) for a batch, as tc_bwd.cuh does:
//     P = exp(S - lse),  dP = dO V^T,  dS = P (dP - delta),  dV = P^T dO,  dK = scale dS^T Q,  dQ = scale dS K
// with the same arithmetic (f32 operands as f16 hi/lo planes times a power of two, three kind::f16 MMAs per
// product, f32 accumulation in TMEM).
//
// Why another form.  The fused kernels of tc_bwd.cuh keep a CTA's K, V, Q, dO tiles and the dK, dV (or dQ)
// accumulators on chip at once.  At head_dim 256 that is two 256-column accumulators -- all 512 TMEM columns
// before S and dP have any -- and four 64 KB operand tiles beside them.  Here the products are separate
// launches and P and dS travel through memory, as f16 hi/lo planes laid out as the next launch's operand:
//   bwd_wide_scores   one CTA per (128 query rows, 128 keys) tile at or below the diagonal of one (sequence,
//                     head): S = Q K^T and dP = dO V^T over the head's 256 columns into two TMEM accumulators,
//                     then P and dS, split, into the scratch planes [T, T] of that head;
//   gemm_tri<0>       dQ = scale dS K: 128 x 256 output tiles (the whole head), contraction over the keys a query tile sees;
//   gemm_tri<1>       dK = scale sum_h dS^T Q and dV = sum_h P^T dO: contraction over the query rows at or after
//                     the key tile, every head of the KV group adding into the same output.
// Contractions longer than 1024 are cut into pieces that separate CTAs add with red.global.add.f32 (the tensor
// core adds into its accumulator with truncation; see tc_gemm.cuh), so dq, dk, dv are zeroed first.
// The planes of P and dS cost 8 bytes per (query, key) pair written and 12 read -- independent of head_dim,
// which is why this form is for the wide heads only: at 256 columns the products above are 2.5 times the flops
// per byte they are at 128.  A scratch of a few GiB holds the planes of a chunk of heads; chunks run in turn.
//
// The scale of dS.  Every query row has its own, from the bound the fused dQ kernel uses (|dS[t, s]| <=
// 2 |dout[t]| max_s |v[s]|): dQ's contraction runs along a row, so the row's factor leaves with the row.  dK's
// contraction runs ACROSS rows, so there the factor is moved to the other operand: the Q planes it reads are a
// second copy whose row t is divided by (row t's scale / the smallest scale of the KV group), a power of two
// between 1 and 2^12, and the product dS Q has one scale again.
#pragma once

#include "tc_gemm.cuh"

namespace zt {
namespace tcw {

using namespace tc;
using tcb::block_mult;
using tcb::kDsBound;
using tcb::pow2_for;
using tcb::split_pack;

constexpr int kStages = 3;
constexpr int kTB = 128 * 64 * 2;  // bytes of one plane of an operand tile
constexpr int kSB = 4 * kTB;       // a stage: A hi, A lo, B hi, B lo
constexpr int kScoreThreads = 10 * 32;  // TMA producer, MMA issuer, eight epilogue warps
constexpr int kTriThreads = 6 * 32;     // TMA producer, MMA issuer, four epilogue warps
constexpr int kPiece = 1024;            // contraction depth of one CTA of gemm_tri
constexpr float kRowBoostMax = 4096.f;  // a row's scale is at most this many times the group's smallest

struct WideShared {
    uint64_t full[kStages], freed[kStages], all_done, staged;
    uint32_t tmem_base;
    volatile int abort;
};
__device__ __forceinline__ bool wwait(uint64_t *bar, uint32_t parity, WideShared *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void wgive_up(WideShared *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}

struct WideParams {
    const float *lse, *delta, *rnorm;  // [B, T, H]
    const uint32_t *amax_q, *amax_k, *amax_v, *amax_do;  // [B, Hkv] bit patterns of max |x|
    const uint32_t *vnmax, *rnmax;     // [B, Hkv] bit patterns: largest row norm of v, of dout (over the group's heads)
    __half *p_planes, *ds_planes;      // [2][unit_cap][Tp][Tp]: hi planes of the chunk's units, then lo planes
    float *out;                        // gemm_tri: dq, dk or dv
    int batch, T, Tp, n_heads, n_kv_heads;
    int dim_out, td;                   // the tensors' head_dim, the planes' (256)
    int unit0, unit_cap;               // the chunk: units (b * n_heads + h) from unit0; planes allocated for unit_cap
    int pieces;                        // gemm_tri: pieces of kPiece along one head's contraction
    int which;                         // gemm_tri<1>: 0 dK (dS and the row-scaled Q), 1 dV (P and dO)
    float scale, scale_log2, p_scale;
};

// Row t's scale of dS (cq) and what divides row t of the second copy of Q (1 / rel): both powers of two.
__device__ __forceinline__ float wide_group_scale(uint32_t rnmax_bits, uint32_t vnmax_bits) {
    return pow2_for(2.02f * __uint_as_float(rnmax_bits) * __uint_as_float(vnmax_bits), 14);
}
__device__ __forceinline__ void wide_row_scale(float rnorm_t, uint32_t rnmax_bits, uint32_t vnmax_bits, float &cq, float &rel) {
    const float cmin = wide_group_scale(rnmax_bits, vnmax_bits);
    const float x = 2.02f * rnorm_t * __uint_as_float(vnmax_bits);
    float c = (x > 0.f && x < 3.0e38f) ? pow2_for(x, 14) : cmin;
    c = fminf(fmaxf(c, cmin), cmin * kRowBoostMax);
    if (!(c < 3.0e38f)) c = cmin;
    cq = c;
    rel = cmin / c;
}

// rnmax[b, g] = the largest row norm of dout over the rows and the heads of KV group g.  grid (ceil(T / 64), B).
__global__ void __launch_bounds__(256) wide_rnmax_kernel(const float *__restrict__ rnorm, uint32_t *__restrict__ rnmax,
                                                         int T, int n_heads, int n_kv_heads) {
    __shared__ uint32_t gmax[tcb::kPrepassMaxGroups];
    const int b = blockIdx.y, group = n_heads / n_kv_heads;
    for (int i = threadIdx.x; i < n_kv_heads; i += 256) gmax[i] = 0u;
    __syncthreads();
    const long long r0 = (long long)blockIdx.x * 64, r1 = r0 + 64 < T ? r0 + 64 : T;
    const long long n = (r1 - r0) * n_heads;
    const float *base = rnorm + ((long long)b * T + r0) * n_heads;
    for (long long i = threadIdx.x; i < n; i += 256) {
        const float x = __ldg(base + i);
        if (x > 0.f) atomicMax(&gmax[(int)(i % n_heads) / group], __float_as_uint(x));
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_kv_heads; i += 256)
        if (gmax[i]) atomicMax(rnmax + b * n_kv_heads + i, gmax[i]);
}

// The second copy of Q's planes: row t of head h times rel(t, h).  A thread converts eight elements.
__global__ void __launch_bounds__(256) wide_qscaled_kernel(const __half *__restrict__ q_planes, __half *__restrict__ qs_planes,
                                                           const float *__restrict__ rnorm, const uint32_t *__restrict__ rnmax,
                                                           const uint32_t *__restrict__ vnmax, int batch, int T, int n_heads,
                                                           int n_kv_heads, int td) {
    const long long per_plane = (long long)batch * T * n_heads * td;
    const long long i8 = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i8 * 8 >= per_plane) return;
    const long long e = i8 * 8;
    const long long rowhead = e / td;  // (b * T + t) * n_heads + h
    const int h = (int)(rowhead % n_heads);
    const int b = (int)(rowhead / ((long long)T * n_heads));
    const int g = h / (n_heads / n_kv_heads);
    float cq, rel;
    wide_row_scale(__ldg(rnorm + rowhead), rnmax[b * n_kv_heads + g], vnmax[b * n_kv_heads + g], cq, rel);
    const uint4 hw = __ldg(reinterpret_cast<const uint4 *>(q_planes + e));
    const uint4 lw = __ldg(reinterpret_cast<const uint4 *>(q_planes + per_plane + e));
    const uint32_t hs[4] = {hw.x, hw.y, hw.z, hw.w}, ls[4] = {lw.x, lw.y, lw.z, lw.w};
    uint32_t ho[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&hs[j]));
        const float2 c = __half22float2(*reinterpret_cast<const __half2 *>(&ls[j]));
        split_pack((a.x + c.x) * rel, (a.y + c.y) * rel, ho[j], lo[j]);
    }
    *reinterpret_cast<uint4 *>(qs_planes + e) = make_uint4(ho[0], ho[1], ho[2], ho[3]);
    *reinterpret_cast<uint4 *>(qs_planes + per_plane + e) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
}

// ---------------------------------------------------------------------------------------------------
// P and dS of one 128 x 128 tile.  grid (tiles at or below the diagonal, units of the chunk), 320 threads.
// Eight 64-deep steps through a ring of three stages: four for S (Q and K tiles), four for dP (dO and V tiles).
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kScoreThreads, 1)
    bwd_wide_scores(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                    const __grid_constant__ CUtensorMap gmap, const __grid_constant__ CUtensorMap vmap, const WideParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    WideShared *sh = reinterpret_cast<WideShared *>(smem_raw + kStages * kSB);
    const int warp = threadIdx.x >> 5;
    // tile (m, n), n <= m, from the index along the triangle
    const int ti = (int)blockIdx.x;
    int m = (int)((sqrtf(8.f * (float)ti + 1.f) - 1.f) * 0.5f);
    while ((m + 1) * (m + 2) / 2 <= ti) ++m;
    while (m * (m + 1) / 2 > ti) --m;
    const int n = ti - m * (m + 1) / 2;
    const int m0 = m * 128, n0 = n * 128;
    const int u = (int)blockIdx.y, ug = p.unit0 + u;
    const int b = ug / p.n_heads, h = ug % p.n_heads;
    const int group = p.n_heads / p.n_kv_heads, g = h / group;
    const int B = p.batch;
    const int nbk = p.td / 64;       // 64-column blocks of a head: steps per product
    const int n_steps = 2 * nbk;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) mbar_init(&sh->full[i], 1), mbar_init(&sh->freed[i], 1);
        mbar_init(&sh->all_done, 1);
        mbar_init(&sh->staged, 8);
        sh->abort = (smem_u32(smem_raw) & 1023u) ? 80 : 0;
        if (sh->abort) atomicMax(&g_tc_status, 80);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&sh->tmem_base, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one() && !sh->abort) {
            tma_prefetch_desc(&qmap), tma_prefetch_desc(&kmap), tma_prefetch_desc(&gmap), tma_prefetch_desc(&vmap);
            int issued = 0;
            for (int s = 0; s < n_steps; ++s) {
                const int st = s % kStages;
                if (s >= kStages && !wwait(&sh->freed[st], (uint32_t)(((s / kStages) & 1) ^ 1), sh)) { wgive_up(sh, 81); break; }
                uint8_t *base = smem_raw + st * kSB;
                mbar_arrive_expect_tx(&sh->full[st], 4 * kTB);
                const bool first = s < nbk;
                const int blk = first ? s : s - nbk;
                const CUtensorMap *am = first ? &qmap : &gmap, *bm = first ? &kmap : &vmap;
                tma_load_4d(base, am, &sh->full[st], 0, m0, h * nbk + blk, b);
                tma_load_4d(base + kTB, am, &sh->full[st], 0, m0, h * nbk + blk, B + b);
                tma_load_4d(base + 2 * kTB, bm, &sh->full[st], 0, n0, g * nbk + blk, b);
                tma_load_4d(base + 3 * kTB, bm, &sh->full[st], 0, n0, g * nbk + blk, B + b);
                ++issued;
            }
            if (sh->abort)  // let the copies in flight land before the CTA's shared memory goes away
                for (int s = (issued > kStages ? issued - kStages : 0); s < issued; ++s)
                    mbar_wait(&sh->full[s % kStages], (uint32_t)((s / kStages) & 1));
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc = idesc_f16(128, 128, false, false);
            const uint32_t s_u32 = smem_u32(smem_raw);
            bool ok = !sh->abort;
            for (int s = 0; ok && s < n_steps; ++s) {
                const int st = s % kStages;
                if (!wwait(&sh->full[st], (uint32_t)((s / kStages) & 1), sh)) { wgive_up(sh, 82); ok = false; break; }
                tc_fence_after();
                const uint32_t base = s_u32 + (uint32_t)(st * kSB);
                const uint64_t ah = desc_kmajor(base), al = desc_kmajor(base + kTB);
                const uint64_t bh = desc_kmajor(base + 2 * kTB), bl = desc_kmajor(base + 3 * kTB);
                const uint32_t acc = tmem + (s < nbk ? 0u : 128u);
                const bool fresh = (s == 0 || s == nbk);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t dah = desc_advance(ah, kk * 32), dal = desc_advance(al, kk * 32);
                    const uint64_t dbh = desc_advance(bh, kk * 32), dbl = desc_advance(bl, kk * 32);
                    mma_ss_f16(acc, dah, dbh, idesc, (fresh && kk == 0) ? 0 : 1);
                    mma_ss_f16(acc, dah, dbl, idesc, 1);
                    mma_ss_f16(acc, dal, dbh, idesc, 1);
                }
                mma_commit(&sh->freed[st]);
            }
            if (ok) mma_commit(&sh->all_done);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ a thread per query row and 64 of the
        // tile's 128 keys: warps 2..5 the first 64, warps 6..9 the others
        const int lane = threadIdx.x & 31;
        const int lane_grp = warp & 3;  // the TMEM lanes a warp may read are those of its index modulo 4
        const int half = (warp - 2) >> 2;
        const int row = lane_grp * 32 + lane;
        const uint32_t lane_base = (uint32_t)(lane_grp * 32) << 16;
        const int t = m0 + row;
        const float mq = block_mult(p.amax_q[b * p.n_kv_heads + g]), mk = block_mult(p.amax_k[b * p.n_kv_heads + g]);
        const float mv = block_mult(p.amax_v[b * p.n_kv_heads + g]), mdo = block_mult(p.amax_do[b * p.n_kv_heads + g]);
        const long long ridx = ((long long)b * p.T + (t < p.T ? t : 0)) * p.n_heads + h;
        float cq = 1.f, rel = 1.f;
        if (t < p.T) wide_row_scale(__ldg(p.rnorm + ridx), p.rnmax[b * p.n_kv_heads + g], p.vnmax[b * p.n_kv_heads + g], cq, rel);
        const float cs = p.scale_log2 / (mq * mk);
        // P leaves times p_scale: the factor rides in the exponent
        const float lse2 = (t < p.T) ? __ldg(p.lse + ridx) * kLog2e - log2f(p.p_scale) : 0.f;
        const float c1 = cq / (mdo * mv * p.p_scale);  // (P carries p_scale; dS must not)
        const float dels = (t < p.T && !ZT_DEFECT(13)) ? __ldg(p.delta + ridx) * cq / p.p_scale : 0.f;
        bool ok = __all_sync(0xffffffffu, wwait(&sh->all_done, 0, sh));
        if (!ok) wgive_up(sh, 83);
        bool saturated = false;
        // the four output tiles (P hi, P lo, dS hi, dS lo: 128 rows x 256 bytes each) are put together in the
        // stages, idle by now: 16-byte chunk c of row r at chunk c ^ (r & 15)
        if (ok) {
            tc_fence_after();
            const bool diag = (m == n) || (m0 + 128 > p.T);  // tiles that need the mask
#pragma unroll 1
            for (int c = 0; c < 64; c += 32) {
                uint32_t rs[32], rd[32];
                tmem_ld32(tmem + lane_base + half * 64 + c, rs);
                tmem_ld32(tmem + lane_base + 128 + half * 64 + c, rd);
                tmem_wait_ld();
                const int key0 = n0 + half * 64 + c;
                uint32_t ph[16], pl[16], dh[16], dl[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float pv[2], dv[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = key0 + i + e;
                        const bool vis = !diag || ((key <= t || ZT_DEFECT(11)) && key < p.T && t < p.T);
                        const float pe = vis ? ex2(__uint_as_float(rs[i + e]) * cs - lse2) : 0.f;
                        const float x = vis ? pe * (__uint_as_float(rd[i + e]) * c1 - dels) : 0.f;
                        saturated |= !(fabsf(x) <= kDsBound);
                        pv[e] = pe;
                        dv[e] = fminf(fmaxf(x, -kDsBound), kDsBound);
                    }
                    split_pack(pv[0], pv[1], ph[i >> 1], pl[i >> 1]);
                    split_pack(dv[0], dv[1], dh[i >> 1], dl[i >> 1]);
                }
                uint8_t *srow = smem_raw + row * 256;
                const int ch0 = (half * 64 + c) >> 3;  // 8 halves per chunk
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int at = ((ch0 + j) ^ (row & 15)) << 4;
                    *reinterpret_cast<uint4 *>(srow + at) = make_uint4(ph[4 * j], ph[4 * j + 1], ph[4 * j + 2], ph[4 * j + 3]);
                    *reinterpret_cast<uint4 *>(srow + 32768 + at) = make_uint4(pl[4 * j], pl[4 * j + 1], pl[4 * j + 2], pl[4 * j + 3]);
                    *reinterpret_cast<uint4 *>(srow + 65536 + at) = make_uint4(dh[4 * j], dh[4 * j + 1], dh[4 * j + 2], dh[4 * j + 3]);
                    *reinterpret_cast<uint4 *>(srow + 98304 + at) = make_uint4(dl[4 * j], dl[4 * j + 1], dl[4 * j + 2], dl[4 * j + 3]);
                }
            }
        }
        if (__any_sync(0xffffffffu, saturated) && lane == 0) atomicAdd(&g_tc_saturated, 1u);
        mbar_arrive_warp(&sh->staged);
        if (__all_sync(0xffffffffu, wwait(&sh->staged, 0, sh)) && !sh->abort) {
            // warp w writes rows [16 w, 16 w + 16) of each of the four tiles, two rows (512 bytes) per instruction
            const int w8 = warp - 2;
            const long long plane = (long long)p.Tp * p.Tp;
            const int ch = lane & 15;
#pragma unroll
            for (int pl4 = 0; pl4 < 4; ++pl4) {
                __half *dst = (pl4 < 2 ? p.p_planes : p.ds_planes) + ((long long)((pl4 & 1) * p.unit_cap + u)) * plane;
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    const int r = w8 * 16 + i + (lane >> 4);
                    const uint4 x = *reinterpret_cast<const uint4 *>(smem_raw + pl4 * 32768 + r * 256 + ((ch ^ (r & 15)) << 4));
                    *reinterpret_cast<uint4 *>(dst + (long long)(m0 + r) * p.Tp + n0 + ch * 8) = x;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------------
// The same P and dS with the query side resident.  One CTA per (128 query rows, head): the hi planes of its Q and
// dO rows live in TMEM (128 columns each, A operands), their lo planes in shared memory (64 KB each), and the CTA
// walks the key tiles at or below its diagonal, 128 keys at a time.  K and V arrive as 64-column blocks (128 keys x
// 64 columns, hi and lo: 32 KB) through a ring of three; per key tile, S (4 blocks x 12 MMAs of N = 128) into one
// 128-column accumulator, then dP into the other.  Against bwd_wide_scores every operand byte of the query side
// is loaded once per CTA instead of once per tile: half the traffic from L2, which is what bounds both.
// The eight epilogue warps read S as soon as it is complete (P, kept in registers, goes to memory while dP's
// MMAs run), then dP (dS goes out while the next tile's S runs): the accumulators are single, and free again as
// soon as they have been read.  No shared memory is left for staging rows, so a tile's rows reach memory from
// registers: four lanes exchange 4 x 4 blocks of 16-byte chunks, and an instruction writes 64-byte runs of 8 rows.
// grid (units of the chunk, query tiles), 320 threads.
// ---------------------------------------------------------------------------------------------------
struct ResShared {
    uint64_t full[3], freed[3], qh_full, ql_full, a_ready, s_full, s_free, dp_full, dp_free;
    uint32_t tmem_base;
    volatile int abort;
};
__device__ __forceinline__ bool rwait(uint64_t *bar, uint32_t parity, ResShared *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void rgive_up(ResShared *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}
// 16 packed words (32 halves, four 16-byte chunks) of this thread's row -> global memory: the four lanes of a quad
// exchange chunks so that lane j holds chunk j of the quad's four rows, and each of the four stores below writes
// 64 contiguous bytes of 8 rows.  `dst` points at the chunk-0 position of the quad's FIRST row; rows are `ld`
// halves apart.
__device__ __forceinline__ void store_rows_quad(__half *dst, long long ld, const uint32_t (&w)[16], int lane) {
    uint32_t r[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = w[i];
#pragma unroll
    for (int M = 2; M >= 1; M >>= 1) {
        const bool up = (lane & M) != 0;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
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
    // r[4 i .. 4 i + 3] = chunk (lane & 3) of the quad's row i
    const int j = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        *reinterpret_cast<uint4 *>(dst + i * ld + j * 8) = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
}

__global__ void __launch_bounds__(kScoreThreads, 1)
    bwd_wide_scores_res(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                        const __grid_constant__ CUtensorMap gmap, const __grid_constant__ CUtensorMap vmap, const WideParams p) {
    constexpr int BT = 128 * 64 * 2;          // one 64-column block of a 128-row tile, one plane: 16 KB
    constexpr int cQh = 0, cGh = 128, cS = 256, cDP = 384;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *sQl = smem_raw, *sGl = smem_raw + 4 * BT;   // lo planes of Q and dO: four blocks each (hi planes first, staged)
    uint8_t *ring = smem_raw + 8 * BT;                   // slot s: block hi, block lo at ring + s * 2 BT + {0, 1} BT
    ResShared *sh = reinterpret_cast<ResShared *>(ring + 3 * 2 * BT);
    const int warp = threadIdx.x >> 5;
    // launch order (x fastest): every unit's last query tile, then every unit's last but one, ...: the longest
    // walks of the whole launch start first, so its tail is a fraction of a short walk
    const int m = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int m0 = m * 128;
    const int u = (int)blockIdx.x, ug = p.unit0 + u;
    const int b = ug / p.n_heads, h = ug % p.n_heads;
    const int group = p.n_heads / p.n_kv_heads, g = h / group;
    const int B = p.batch;
    const int n_tiles = m + 1;
    const int n_blocks = 8 * n_tiles;  // per tile: K's four blocks, then V's

    if (threadIdx.x == 0) {
        for (int i = 0; i < 3; ++i) mbar_init(&sh->full[i], 1), mbar_init(&sh->freed[i], 1);
        mbar_init(&sh->qh_full, 1), mbar_init(&sh->ql_full, 1);
        mbar_init(&sh->a_ready, 8);
        mbar_init(&sh->s_full, 1), mbar_init(&sh->s_free, 8);
        mbar_init(&sh->dp_full, 1), mbar_init(&sh->dp_free, 8);
        sh->abort = (smem_u32(smem_raw) & 1023u) ? 90 : 0;
        if (sh->abort) atomicMax(&g_tc_status, 90);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one() && !sh->abort) {
            tma_prefetch_desc(&qmap), tma_prefetch_desc(&kmap), tma_prefetch_desc(&gmap), tma_prefetch_desc(&vmap);
            // the hi planes first, into the lo planes' place, until the row threads have moved them to TMEM
            mbar_arrive_expect_tx(&sh->qh_full, 8 * BT);
            for (int blk = 0; blk < 4; ++blk) {
                tma_load_4d(sQl + blk * BT, &qmap, &sh->qh_full, 0, m0, h * 4 + blk, b);
                tma_load_4d(sGl + blk * BT, &gmap, &sh->qh_full, 0, m0, h * 4 + blk, b);
            }
            int issued = 0;
            bool live = true;
            auto load_block = [&](int j) {
                const int st = j % 3;
                if (j >= 3 && !rwait(&sh->freed[st], (uint32_t)(((j / 3) & 1) ^ 1), sh)) { rgive_up(sh, 91), live = false; return; }
                const int n = j >> 3, blk = j & 3;
                const bool is_v = (j & 4) != 0;
                const CUtensorMap *mp = is_v ? &vmap : &kmap;
                uint8_t *base = ring + st * 2 * BT;
                mbar_arrive_expect_tx(&sh->full[st], 2 * BT);
                tma_load_4d(base, mp, &sh->full[st], 0, n * 128, g * 4 + blk, b);
                tma_load_4d(base + BT, mp, &sh->full[st], 0, n * 128, g * 4 + blk, B + b);
                ++issued;
            };
            for (int j = 0; j < 3 && j < n_blocks; ++j) load_block(j);
            if (!rwait(&sh->a_ready, 0, sh)) rgive_up(sh, 91), live = false;
            if (live) {
                mbar_arrive_expect_tx(&sh->ql_full, 8 * BT);
                for (int blk = 0; blk < 4; ++blk) {
                    tma_load_4d(sQl + blk * BT, &qmap, &sh->ql_full, 0, m0, h * 4 + blk, B + b);
                    tma_load_4d(sGl + blk * BT, &gmap, &sh->ql_full, 0, m0, h * 4 + blk, B + b);
                }
            }
            for (int j = 3; live && j < n_blocks; ++j) load_block(j);
            if (sh->abort) {
                mbar_wait(&sh->qh_full, 0);
                if (live) mbar_wait(&sh->ql_full, 0);
                for (int j = (issued > 3 ? issued - 3 : 0); j < issued; ++j) mbar_wait(&sh->full[j % 3], (uint32_t)((j / 3) & 1));
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc = idesc_f16(128, 128, false, false);
            bool ok = !sh->abort && rwait(&sh->a_ready, 0, sh) && rwait(&sh->ql_full, 0, sh);
            if (!ok) rgive_up(sh, 92);
            tc_fence_after();
            const uint32_t ring_u32 = smem_u32(ring);
            const uint32_t ql_u32 = smem_u32(sQl), gl_u32 = smem_u32(sGl);
            int j = 0;  // ring block counter
            for (int n = 0; ok && n < n_tiles; ++n) {
                for (int prod = 0; ok && prod < 2; ++prod) {  // 0: S = Q K^T, 1: dP = dO V^T
                    // the accumulator must have been read by the row threads (tile n-1)
                    if (n >= 1 && !rwait(prod ? &sh->dp_free : &sh->s_free, (uint32_t)((n - 1) & 1), sh)) { rgive_up(sh, 93); ok = false; break; }
                    tc_fence_after();
                    const uint32_t acc = tmem + (prod ? cDP : cS), a_hi = tmem + (prod ? cGh : cQh);
                    const uint32_t a_lo = prod ? gl_u32 : ql_u32;
                    for (int blk = 0; blk < 4; ++blk, ++j) {
                        const int st = j % 3;
                        if (!rwait(&sh->full[st], (uint32_t)((j / 3) & 1), sh)) { rgive_up(sh, 94); ok = false; break; }
                        tc_fence_after();
                        const uint32_t base = ring_u32 + (uint32_t)(st * 2 * BT);
                        const uint64_t bh = desc_kmajor(base), bl = desc_kmajor(base + BT);
                        const uint64_t al = desc_kmajor(a_lo + (uint32_t)(blk * BT));
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint64_t dbh = desc_advance(bh, kk * 32), dbl = desc_advance(bl, kk * 32);
                            const uint32_t at = a_hi + (uint32_t)((blk * 4 + kk) * 8);
                            mma_ts_f16(acc, at, dbh, idesc, (blk > 0 || kk > 0) ? 1 : 0);
                            mma_ts_f16(acc, at, dbl, idesc, 1);
                            mma_ss_f16(acc, desc_advance(al, kk * 32), dbh, idesc, 1);
                        }
                        mma_commit(&sh->freed[st]);
                    }
                    if (ok) mma_commit(prod ? &sh->dp_full : &sh->s_full);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ a thread per query row and 64 of a
        // tile's 128 keys: warps 2..5 the first 64, warps 6..9 the others
        const int lane = threadIdx.x & 31;
        const int lane_grp = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row = lane_grp * 32 + lane;
        const uint32_t lane_base = (uint32_t)(lane_grp * 32) << 16;
        const int t = m0 + row;
        bool ok = true;
        {
            // this row's hi plane of Q (warps 2..5) or of dO (warps 6..9) -> TMEM, out of the 128-byte-swizzled staging tiles
            if (!__all_sync(0xffffffffu, rwait(&sh->qh_full, 0, sh))) rgive_up(sh, 95), ok = false;
            const uint8_t *src = (half ? sGl : sQl) + row * 128;
#pragma unroll 1
            for (int blk = 0; blk < 4; ++blk) {
                uint32_t r[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v4 = *reinterpret_cast<const uint4 *>(src + blk * BT + ((c ^ (row & 7)) << 4));
                    r[4 * c] = v4.x, r[4 * c + 1] = v4.y, r[4 * c + 2] = v4.z, r[4 * c + 3] = v4.w;
                }
                tmem_st32(tmem + lane_base + (half ? cGh : cQh) + blk * 32, r);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&sh->a_ready);
        }
        const int bg = b * p.n_kv_heads + g;
        const float mq = block_mult(p.amax_q[bg]), mk = block_mult(p.amax_k[bg]);
        const float mv = block_mult(p.amax_v[bg]), mdo = block_mult(p.amax_do[bg]);
        const long long ridx = ((long long)b * p.T + (t < p.T ? t : 0)) * p.n_heads + h;
        float cq = 1.f, rel = 1.f;
        if (t < p.T) wide_row_scale(__ldg(p.rnorm + ridx), p.rnmax[bg], p.vnmax[bg], cq, rel);
        const float cs = p.scale_log2 / (mq * mk);
        const float lse2 = (t < p.T) ? __ldg(p.lse + ridx) * kLog2e - log2f(p.p_scale) : 0.f;
        const float c1 = cq / (mdo * mv * p.p_scale);
        const float dels = (t < p.T && !ZT_DEFECT(13)) ? __ldg(p.delta + ridx) * cq / p.p_scale : 0.f;
        bool saturated = false;
        const long long plane = (long long)p.Tp * p.Tp;
        // the quad's first row, this thread's 64 columns, of the unit's hi planes (lo: unit_cap planes further)
        __half *p_hi = p.p_planes + (long long)u * plane + (long long)(m0 + (row & ~3)) * p.Tp + half * 64;
        __half *d_hi = p.ds_planes + (long long)u * plane + (long long)(m0 + (row & ~3)) * p.Tp + half * 64;
        const long long lo_off = (long long)p.unit_cap * plane;
        for (int n = 0; ok && n < n_tiles; ++n) {
            const int n0 = n * 128;
            const bool diag = (n == m) || (m0 + 128 > p.T);
            float pr[64];
            if (!__all_sync(0xffffffffu, rwait(&sh->s_full, (uint32_t)(n & 1), sh))) { rgive_up(sh, 96); ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 64; c += 32) {
                uint32_t rs[32];
                tmem_ld32(tmem + lane_base + cS + half * 64 + c, rs);
                tmem_wait_ld();
                if (c == 32) {  // S has been read: the next tile's may overwrite it
                    tc_fence_before();
                    mbar_arrive_warp_relaxed(&sh->s_free);
                }
                const int key0 = n0 + half * 64 + c;
                uint32_t ph[16], pl[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = key0 + i + e;
                        const bool vis = !diag || ((key <= t || ZT_DEFECT(11)) && key < p.T && t < p.T);
                        pr[c + i + e] = vis ? ex2(__uint_as_float(rs[i + e]) * cs - lse2) : 0.f;
                    }
                    split_pack(pr[c + i], pr[c + i + 1], ph[i >> 1], pl[i >> 1]);
                }
                store_rows_quad(p_hi + n0 + c, p.Tp, ph, lane);
                store_rows_quad(p_hi + lo_off + n0 + c, p.Tp, pl, lane);
            }
            if (!__all_sync(0xffffffffu, rwait(&sh->dp_full, (uint32_t)(n & 1), sh))) { rgive_up(sh, 97); ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 64; c += 32) {
                uint32_t rd[32];
                tmem_ld32(tmem + lane_base + cDP + half * 64 + c, rd);
                tmem_wait_ld();
                if (c == 32) {
                    tc_fence_before();
                    mbar_arrive_warp_relaxed(&sh->dp_free);
                }
                uint32_t dh[16], dl[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float dv[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float x = pr[c + i + e] * (__uint_as_float(rd[i + e]) * c1 - dels);  // (pr is zero where masked)
                        saturated |= !(fabsf(x) <= kDsBound);
                        dv[e] = fminf(fmaxf(x, -kDsBound), kDsBound);
                    }
                    split_pack(dv[0], dv[1], dh[i >> 1], dl[i >> 1]);
                }
                store_rows_quad(d_hi + n0 + c, p.Tp, dh, lane);
                store_rows_quad(d_hi + lo_off + n0 + c, p.Tp, dl, lane);
            }
        }
        if (__any_sync(0xffffffffu, saturated) && lane == 0) atomicAdd(&g_tc_saturated, 1u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}
inline size_t res_smem_bytes() { return (size_t)14 * (128 * 64 * 2) + sizeof(ResShared); }

// ---------------------------------------------------------------------------------------------------
// The three products that read the planes.  128 x 256 output tiles (a head's whole width, so that a tile of the
// planes is read once), 64-deep steps, B always the tensor whose rows are the contraction index ([T, width] planes
// read as N-major tiles).
//   MODE 0: dQ.  grid (query tiles, units x pieces).  A = dS planes, K-major; contraction over keys
//           [piece * 1024, min((m + 1) * 128, (piece + 1) * 1024)); row t leaves times scale / (cq(t) mk).
//   MODE 1: dK (which 0) or dV (which 1).  grid (key tiles, KV groups of the chunk x heads of a group x pieces).  A = dS or P planes read M-major (rows are the contraction index: query rows); contraction
//           over query rows [max(m * 128, piece * 1024), min(Tp, (piece + 1) * 1024)).
// Every tile is added to the output (red.global.add.v4.f32), which the host has zeroed.
// ---------------------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(kTriThreads, 1)
    gemm_tri(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, const WideParams p) {
    constexpr bool A_MN = MODE == 1;
    // a stage: A hi, A lo (128 x 64 halves each) and B hi, B lo (64 contraction rows x 256 columns each, as four
    // 64-column blocks of 8 KB): 96 KB; two stages.  The whole head width per CTA: an A tile is read once for it.
    constexpr int kBT = 64 * 256 * 2, kStage = 2 * kTB + 2 * kBT, kSt = 2;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    WideShared *sh = reinterpret_cast<WideShared *>(smem_raw + kSt * kStage);
    const int warp = threadIdx.x >> 5;
    const int m0 = blockIdx.x * 128;
    const int group = p.n_heads / p.n_kv_heads;
    int u, piece;
    if (MODE == 0) {
        u = (int)blockIdx.y / p.pieces, piece = (int)blockIdx.y % p.pieces;
    } else {
        const int cg = (int)blockIdx.y / (group * p.pieces), rem = (int)blockIdx.y % (group * p.pieces);
        u = cg * group + rem / p.pieces, piece = rem % p.pieces;
    }
    const int ug = p.unit0 + u;
    const int b = ug / p.n_heads, h = ug % p.n_heads, g = h / group;
    const int B = p.batch;
    int k_begin = piece * kPiece, k_end = k_begin + kPiece;
    if (MODE == 0) {
        if (k_end > m0 + 128) k_end = m0 + 128;
    } else {
        if (k_begin < m0) k_begin = m0;
    }
    if (k_end > p.Tp) k_end = p.Tp;
    if (k_begin >= k_end || m0 >= p.T) return;  // (the whole CTA: nothing has been set up yet)
    const int n_steps = (k_end - k_begin) / 64;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kSt; ++i) mbar_init(&sh->full[i], 1), mbar_init(&sh->freed[i], 1);
        mbar_init(&sh->all_done, 1);
        mbar_init(&sh->staged, 4);
        sh->abort = (smem_u32(smem_raw) & 1023u) ? 84 : 0;
        if (sh->abort) atomicMax(&g_tc_status, 84);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&sh->tmem_base, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one() && !sh->abort) {
            tma_prefetch_desc(&amap), tma_prefetch_desc(&bmap);
            // B's column blocks: the head's (MODE 0: the KV head's) 256 columns
            const int bblk = ((MODE == 0 ? g : h) * p.td) / 64;
            int issued = 0;
            for (int s = 0; s < n_steps; ++s) {
                const int st = s % kSt, k0 = k_begin + s * 64;
                if (s >= kSt && !wwait(&sh->freed[st], (uint32_t)(((s / kSt) & 1) ^ 1), sh)) { wgive_up(sh, 85); break; }
                uint8_t *base = smem_raw + st * kStage;
                mbar_arrive_expect_tx(&sh->full[st], kStage);
                if (A_MN) {  // rows = query rows (contraction), columns = keys (M): 64 rows x two 64-column blocks
                    tma_load_4d(base, &amap, &sh->full[st], 0, k0, m0 / 64, u);
                    tma_load_4d(base + kTB, &amap, &sh->full[st], 0, k0, m0 / 64, p.unit_cap + u);
                } else {     // rows = query rows (M), columns = keys (contraction): 128 rows x one block
                    tma_load_4d(base, &amap, &sh->full[st], 0, m0, k0 / 64, u);
                    tma_load_4d(base + kTB, &amap, &sh->full[st], 0, m0, k0 / 64, p.unit_cap + u);
                }
                tma_load_4d(base + 2 * kTB, &bmap, &sh->full[st], 0, k0, bblk, b);
                tma_load_4d(base + 2 * kTB + kBT, &bmap, &sh->full[st], 0, k0, bblk, B + b);
                ++issued;
            }
            if (sh->abort)
                for (int s = (issued > kSt ? issued - kSt : 0); s < issued; ++s)
                    mbar_wait(&sh->full[s % kSt], (uint32_t)((s / kSt) & 1));
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc = idesc_f16(128, 256, A_MN, true);
            const uint32_t s_u32 = smem_u32(smem_raw);
            bool ok = !sh->abort;
            for (int s = 0; ok && s < n_steps; ++s) {
                const int st = s % kSt;
                if (!wwait(&sh->full[st], (uint32_t)((s / kSt) & 1), sh)) { wgive_up(sh, 86); ok = false; break; }
                tc_fence_after();
                const uint32_t base = s_u32 + (uint32_t)(st * kStage);
                const uint64_t ah = A_MN ? desc_mnmajor_16b(base, 64 * 128) : desc_kmajor(base);
                const uint64_t al = A_MN ? desc_mnmajor_16b(base + kTB, 64 * 128) : desc_kmajor(base + kTB);
                const uint64_t bh = desc_mnmajor_16b(base + 2 * kTB, 64 * 128);
                const uint64_t bl = desc_mnmajor_16b(base + 2 * kTB + kBT, 64 * 128);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint32_t ao = A_MN ? kk * 2048 : kk * 32, bo = kk * 2048;
                    const uint64_t dah = desc_advance(ah, ao), dal = desc_advance(al, ao);
                    const uint64_t dbh = desc_advance(bh, bo), dbl = desc_advance(bl, bo);
                    mma_ss_f16(tmem, dah, dbh, idesc, (s > 0 || kk > 0) ? 1 : 0);
                    mma_ss_f16(tmem, dah, dbl, idesc, 1);
                    mma_ss_f16(tmem, dal, dbh, idesc, 1);
                }
                mma_commit(&sh->freed[st]);
            }
            if (ok) mma_commit(&sh->all_done);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue: a thread per output row
        const int lane = threadIdx.x & 31;
        const int lane_grp = warp & 3;
        const int row = lane_grp * 32 + lane;
        const uint32_t lane_base = (uint32_t)(lane_grp * 32) << 16;
        const int t = m0 + row;  // MODE 0: the query row; MODE 1: the key
        float f;
        if (MODE == 0) {
            float cq = 1.f, rel = 1.f;
            if (t < p.T)
                wide_row_scale(__ldg(p.rnorm + ((long long)b * p.T + t) * p.n_heads + h), p.rnmax[b * p.n_kv_heads + g],
                               p.vnmax[b * p.n_kv_heads + g], cq, rel);
            f = p.scale / (cq * block_mult(p.amax_k[b * p.n_kv_heads + g]));
        } else if (p.which == 0) {
            f = p.scale / (wide_group_scale(p.rnmax[b * p.n_kv_heads + g], p.vnmax[b * p.n_kv_heads + g]) *
                           block_mult(p.amax_q[b * p.n_kv_heads + g]));
        } else {
            f = 1.0f / (p.p_scale * block_mult(p.amax_do[b * p.n_kv_heads + g]));
        }
        bool ok = __all_sync(0xffffffffu, wwait(&sh->all_done, 0, sh));
        if (!ok) wgive_up(sh, 87);
        uint8_t *stage = smem_raw;  // rows go through shared memory: 128 rows x 1024 bytes, chunk c of row r at c ^ (r & 31)
        if (ok) {
            tc_fence_after();
            uint8_t *srow = stage + row * 1024;
#pragma unroll 1
            for (int c = 0; c < 256; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem + lane_base + c, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 o4;
                    o4.x = __uint_as_float(r[i]) * f, o4.y = __uint_as_float(r[i + 1]) * f;
                    o4.z = __uint_as_float(r[i + 2]) * f, o4.w = __uint_as_float(r[i + 3]) * f;
                    const int ch = (c + i) >> 2;
                    *reinterpret_cast<float4 *>(srow + ((ch ^ (row & 31)) << 4)) = o4;
                }
            }
        }
        mbar_arrive_warp(&sh->staged);
        if (__all_sync(0xffffffffu, wwait(&sh->staged, 0, sh)) && !sh->abort) {
            const int heads_out = MODE == 0 ? p.n_heads : p.n_kv_heads, head_out = MODE == 0 ? h : g;
            const long long ld = (long long)heads_out * p.dim_out;
            const int wrow0 = (warp - 2) * 32;
#pragma unroll 4
            for (int i = 0; i < 32; ++i) {
                const int r = wrow0 + i;
                if (m0 + r >= p.T) continue;
                float *dst = p.out + ((long long)b * p.T + m0 + r) * ld + (long long)head_out * p.dim_out;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int ch = half * 32 + lane;
                    const float4 o4 = *reinterpret_cast<const float4 *>(stage + r * 1024 + ((ch ^ (r & 31)) << 4));
                    if (ch * 4 < p.dim_out) tcb::red_add_v4(dst + ch * 4, o4);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 256);
}

inline size_t tri_smem_bytes() { return (size_t)2 * (2 * kTB + 2 * 64 * 256 * 2) + sizeof(WideShared); }

// ---- host side ----------------------------------------------------------------------------------------

constexpr size_t kScratchBudget = (size_t)2 << 30;   // planes of P and dS held at once, unless one KV group needs more
constexpr size_t kScratchLimit = (size_t)16 << 30;   // one KV group's planes beyond this: the shape is not taken

struct WideWorkspace {
    tcb::BwdWorkspace base;   // the fused backward's layout first: the forward may have left q, k, v planes there
    __half *p_planes, *ds_planes;
    int Tp, unit_cap;
    size_t total_bytes;
};

inline int wide_unit_cap(int batch, int T, int n_heads, int n_kv_heads) {
    const long long Tp = (T + 127) / 128 * 128;
    const size_t unit = (size_t)8 * Tp * Tp;  // four planes of Tp x Tp halves
    const int group = n_heads / n_kv_heads;
    if (unit * group > kScratchLimit) return 0;
    long long cap = (long long)(kScratchBudget / unit) / group * group;
    if (cap < group) cap = group;
    const long long all = (long long)batch * n_heads;
    return (int)(cap < all ? cap : all);
}

inline WideWorkspace wide_workspace(void *ws, int batch, int T, int n_heads, int n_kv_heads, int td) {
    WideWorkspace w{};
    w.base = tcb::bwd_workspace(ws, batch, T, n_heads, n_kv_heads, td);
    auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
    w.Tp = (T + 127) / 128 * 128;
    w.unit_cap = wide_unit_cap(batch, T, n_heads, n_kv_heads);
    char *c = static_cast<char *>(ws);
    size_t off = w.base.total_bytes;
    const size_t planes = (size_t)2 * w.unit_cap * w.Tp * w.Tp * sizeof(__half);
    w.p_planes = reinterpret_cast<__half *>(c + off), off += up(planes);
    w.ds_planes = reinterpret_cast<__half *>(c + off), off += up(planes);
    w.total_bytes = off;
    return w;
}

inline bool tc_bwd_wide_supported(int batch, int T, int n_heads, int n_kv_heads, int dim, const void *q, const void *k,
                                  const void *v, const void *dout, const void *dq, const void *dk, const void *dv) {
    if (!(dim == 192 || dim == 256) || T < 128 || batch < 1) return false;
    if (wide_unit_cap(batch, T, n_heads, n_kv_heads) == 0) return false;
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!al(q) || !al(k) || !al(v) || !al(dout) || !al(dq) || !al(dk) || !al(dv)) return false;
    const DeviceInfo *d = device_info();
    return d && d->cc_major == 10 && get_encode_tiled() != nullptr;
}

inline size_t wide_smem_bytes() { return (size_t)kStages * kSB + sizeof(WideShared); }

}  // namespace tcw

inline size_t tc_bwd_wide_workspace_bytes(int batch, int T, int n_heads, int n_kv_heads, int dim) {
    if (tcw::wide_unit_cap(batch, T, n_heads, n_kv_heads) == 0) return 0;
    return tcw::wide_workspace(nullptr, batch, T, n_heads, n_kv_heads, tc_tile_dim(dim)).total_bytes;
}

// delta and the row norms of dout (workspace .base.rnorm) must already be there.  dq, dk, dv are assigned.
inline int launch_bwd_wide(const float *q, const float *k, const float *v, const float *dout, const float *lse,
                           const float *delta, float *dq, float *dk, float *dv, void *workspace, int batch, int T,
                           int n_heads, int n_kv_heads, int dim, cudaStream_t stream, bool qkv_planes_kept = false,
                           bool tile_scores = false) {
    using namespace tcb;
    using namespace tcw;
    const int td = tc_tile_dim(dim);
    const WideWorkspace ww = wide_workspace(workspace, batch, T, n_heads, n_kv_heads, td);
    const BwdWorkspace &w = ww.base;
    const int group = n_heads / n_kv_heads;
    const int wq_src = n_heads * dim, wkv_src = n_kv_heads * dim;
    const int wq = n_heads * td, wkv = n_kv_heads * td;
    const size_t n_amax = (size_t)batch * n_kv_heads;
    // (with kept planes the maxima of q, k, v stay; those of dout and the two norms start from zero.  The header's
    // last array holds the largest row norm of dout here.)
    if (cudaMemsetAsync(qkv_planes_kept ? w.amax_do : w.amax_q, 0,
                        qkv_planes_kept ? 3 * n_amax * sizeof(uint32_t) : w.amax_bytes, stream) != cudaSuccess ||
        cudaMemsetAsync(dq, 0, (size_t)batch * T * wq_src * sizeof(float), stream) != cudaSuccess ||
        cudaMemsetAsync(dk, 0, (size_t)batch * T * wkv_src * sizeof(float), stream) != cudaSuccess ||
        cudaMemsetAsync(dv, 0, (size_t)batch * T * wkv_src * sizeof(float), stream) != cudaSuccess) {
        cudaGetLastError();
        return refuse("could not clear the backward's outputs and workspace header");
    }
    PrepassArgs pa{};
    pa.batch = batch, pa.T = T;
    pa.t[0] = {dout, w.amax_do, w.do_planes, wq_src, group * dim, dim, td, nullptr};
    pa.n = 1;
    if (!qkv_planes_kept) {
        pa.t[1] = {q, w.amax_q, w.q_planes, wq_src, group * dim, dim, td, nullptr};
        pa.t[2] = {k, w.amax_k, w.k_planes, wkv_src, dim, dim, td, nullptr};
        pa.t[3] = {v, w.amax_v, w.v_planes, wkv_src, dim, dim, td, nullptr};
        pa.n = 4;
    }
    if (launch_prepass(pa, stream)) return 1;
    uint32_t *rnmax = w.dsmax;
    {
        const dim3 gv((unsigned)((T + 255) / 256), (unsigned)n_kv_heads, (unsigned)batch);
        if (ZT_LAUNCH("bwd_vnorm_kernel", stream, (bwd_vnorm_kernel<<<gv, 256, 0, stream>>>(v, w.vnmax, T, n_kv_heads, dim))))
            return 1;
        const dim3 gr((unsigned)((T + 63) / 64), (unsigned)batch);
        if (ZT_LAUNCH("wide_rnmax_kernel", stream, (wide_rnmax_kernel<<<gr, 256, 0, stream>>>(w.rnorm, rnmax, T, n_heads, n_kv_heads))))
            return 1;
        const long long n8 = (long long)batch * T * wq / 8;
        if (ZT_LAUNCH("wide_qscaled_kernel", stream,
                      (wide_qscaled_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(w.q_planes, w.qs_planes, w.rnorm, rnmax,
                                                                                             w.vnmax, batch, T, n_heads, n_kv_heads, td))))
            return 1;
    }
    const int Tp = ww.Tp, cap = ww.unit_cap;
    CUtensorMap q_k, k_k, g_k, v_k;      // K-major 128-row tiles of one 64-column block: the scores' operands
    CUtensorMap k_n, qs_n, g_n;          // N-major tiles (64 contraction rows x the head's 256 columns): B of the three products
    CUtensorMap ds_k, ds_m, p_m;         // the planes: K-major A (dQ), M-major A (dK, dV)
    if (!make_half_tile_map(&q_k, w.q_planes, 2 * batch, T, wq, 64, 128) ||
        !make_half_tile_map(&k_k, w.k_planes, 2 * batch, T, wkv, 64, 128) ||
        !make_half_tile_map(&g_k, w.do_planes, 2 * batch, T, wq, 64, 128) ||
        !make_half_tile_map(&v_k, w.v_planes, 2 * batch, T, wkv, 64, 128) ||
        !make_half_tile_map(&k_n, w.k_planes, 2 * batch, T, wkv, 256, 64) ||
        !make_half_tile_map(&qs_n, w.qs_planes, 2 * batch, T, wq, 256, 64) ||
        !make_half_tile_map(&g_n, w.do_planes, 2 * batch, T, wq, 256, 64) ||
        !make_half_tile_map(&ds_k, ww.ds_planes, 2 * cap, Tp, Tp, 64, 128) ||
        !make_half_tile_map(&ds_m, ww.ds_planes, 2 * cap, Tp, Tp, 128, 64) ||
        !make_half_tile_map(&p_m, ww.p_planes, 2 * cap, Tp, Tp, 128, 64))
        return refuse("the TMA tensor maps for the wide-head backward could not be encoded.");
    const size_t smem = wide_smem_bytes();
    const size_t smem_t = tri_smem_bytes(), smem_r = res_smem_bytes();
    if (optin_smem((const void *)bwd_wide_scores, smem) || optin_smem((const void *)bwd_wide_scores_res, smem_r) ||
        optin_smem((const void *)gemm_tri<0>, smem_t) || optin_smem((const void *)gemm_tri<1>, smem_t))
        return 1;
    WideParams p{};
    p.lse = lse, p.delta = delta, p.rnorm = w.rnorm;
    p.amax_q = w.amax_q, p.amax_k = w.amax_k, p.amax_v = w.amax_v, p.amax_do = w.amax_do;
    p.vnmax = w.vnmax, p.rnmax = rnmax;
    p.p_planes = ww.p_planes, p.ds_planes = ww.ds_planes;
    p.batch = batch, p.T = T, p.Tp = Tp, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads;
    p.dim_out = dim, p.td = td;
    p.unit_cap = cap;
    p.pieces = (Tp + kPiece - 1) / kPiece;
    p.scale = 1.0f / sqrtf((float)dim), p.scale_log2 = kLog2e / sqrtf((float)dim);
    p.p_scale = ldexpf(1.0f, 10);
    g_last_path = "tcgen05";
    const int nt = Tp / 128;
    const int all = batch * n_heads;
    for (int unit0 = 0; unit0 < all; unit0 += cap) {
        const int units = all - unit0 < cap ? all - unit0 : cap;
        p.unit0 = unit0;
        if (tile_scores) {
            const dim3 gs((unsigned)(nt * (nt + 1) / 2), (unsigned)units);
            if (ZT_LAUNCH("bwd_wide_scores", stream, (bwd_wide_scores<<<gs, kScoreThreads, smem, stream>>>(q_k, k_k, g_k, v_k, p))))
                return 1;
        } else {
            const dim3 gs((unsigned)units, (unsigned)nt);
            if (ZT_LAUNCH("bwd_wide_scores_res", stream,
                          (bwd_wide_scores_res<<<gs, kScoreThreads, smem_r, stream>>>(q_k, k_k, g_k, v_k, p))))
                return 1;
        }
        p.out = dq, p.which = 0;
        const dim3 gq((unsigned)nt, (unsigned)(units * p.pieces));
        if (ZT_LAUNCH("gemm_tri_dq", stream, (gemm_tri<0><<<gq, kTriThreads, smem_t, stream>>>(ds_k, k_n, p)))) return 1;
        const dim3 gk((unsigned)nt, (unsigned)(units * p.pieces));  // (units = KV groups x heads of a group)
        p.out = dk, p.which = 0;
        if (ZT_LAUNCH("gemm_tri_dk", stream, (gemm_tri<1><<<gk, kTriThreads, smem_t, stream>>>(ds_m, qs_n, p)))) return 1;
        p.out = dv, p.which = 1;
        if (ZT_LAUNCH("gemm_tri_dv", stream, (gemm_tri<1><<<gk, kTriThreads, smem_t, stream>>>(p_m, g_n, p)))) return 1;
    }
    return 0;
}

}  // namespace zt
