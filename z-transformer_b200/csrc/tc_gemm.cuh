// The projection beside the attention path on the tensor cores: tensor.matmul(ctx, wo) (src/model.zig:396,
// src/tensor.zig:78-106) and its two gradients, inputGrad and weightGrad (src/autograd.zig:553-557,958-1022),
// with the arithmetic of the attention kernels: f32 operands as f16 hi/lo planes times a power of two, every
// product as three kind::f16 MMAs (hi.hi + hi.lo + lo.hi), f32 accumulation in TMEM.
//
// One kernel, gemm_f16split_tc<A_MN, B_MN>, C[M, N] = A . B over a contraction range, 128 x 128 output tiles,
// 64-deep steps through a ring of three shared-memory stages (A and B tiles, hi and lo: 64 KB a stage):
//   forward     y    = ctx . w        A = ctx planes, rows x K, K-major;      B = w planes, K x N, N-major
//   inputGrad   dctx = dy . w^T       A = dy planes, rows x N, K-major;       B = w planes read as N x K^T, K-major
//   weightGrad  dw  += ctx^T . dy     A = ctx planes read as K x rows^T, M-major; B = dy planes, rows x N, N-major
// Activations are scaled per sequence (one power of two per batch item), the weight by one power of two, so the
// contraction index always sees one scale and the output's factor is per row tile (or per CTA) -- applied when
// the tile leaves TMEM.  A contraction longer than 1024 is cut into pieces that separate CTAs add into the
// output (red.global.add.f32): the tensor core adds into its accumulator with truncation, and a piece of 1024
// keeps that drift below the f32 rounding of the answer; weightGrad's contraction runs over the rows of ONE
// sequence per piece, which is also what makes its scale uniform.
// 6 warps: TMA producer, MMA issuer, four epilogue warps (a thread per output row; rows leave through shared
// memory, a row per store instruction).  Every wait is bounded and raises g_tc_status when it gives up.
#pragma once

#include "tc_bwd.cuh"

namespace zt {
namespace tcg {

using namespace tc;
using tcb::block_mult;

constexpr int kStages = 3;
constexpr int kGemmThreads = 6 * 32;
constexpr int kPiece = 1024;  // contraction depth of one CTA

struct GemmShared {
    uint64_t full[kStages], freed[kStages], all_done, staged;
    uint32_t tmem_base;
    volatile int abort;
};
__device__ __forceinline__ bool gmwait(uint64_t *bar, uint32_t parity, GemmShared *sh) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && sh->abort) return false;
    }
    return false;
}
__device__ __forceinline__ void gmgive_up(GemmShared *sh, int code) {
    sh->abort = code;
    atomicMax(&g_tc_status, code);
}

struct GemmParams {
    float *c;            // output, row-major, leading dimension ldc
    long long ldc;
    long long c_batch_stride;  // elements between the outputs of consecutive batch items (0: one output for all)
    int m_rows, n_cols;  // extent of one batch item's output
    int depth;           // contraction extent of one batch item
    int pieces;          // CTAs along the contraction (1: the tile is assigned; more: added with red.global)
    int batch;           // planes per operand: [2][batch][rows][width]
    const uint32_t *amax_a, *amax_b;  // bit patterns of max |x|: per batch item, or one word when *_shared
    int a_shared, b_shared;           // the operand is one matrix for every batch item (the weight)
};

// Tiles in shared memory.  K-major operand (rows are the M or N index, the contraction runs along the 128-byte
// rows): one 64-column block of 128 rows.  M/N-major operand (rows are contraction indices, the 128 M or N indices
// lie along the rows): two 64-column blocks of 64 rows, 8 KB apart.
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_f16split_tc(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, const GemmParams p) {
    constexpr int TB = 128 * 64 * 2;   // bytes of one plane of an operand tile (16 KB in either layout)
    constexpr int SB = 4 * TB;         // a stage: A hi, A lo, B hi, B lo
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    GemmShared *sh = reinterpret_cast<GemmShared *>(smem_raw + kStages * SB);

    const int warp = threadIdx.x >> 5;
    const int m0 = blockIdx.x * 128, n0 = blockIdx.y * 128;
    const int b = (int)blockIdx.z / p.pieces, piece = (int)blockIdx.z % p.pieces;
    const int k_begin = piece * kPiece;
    const int k_end = (k_begin + kPiece < p.depth) ? k_begin + kPiece : p.depth;
    const int n_steps = (k_end - k_begin + 63) / 64;
    const int pa = p.a_shared ? 0 : b, pb = p.b_shared ? 0 : b;          // plane index of the hi plane
    const int la = p.a_shared ? 1 : p.batch, lb = p.b_shared ? 1 : p.batch;  // hi -> lo plane distance

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) mbar_init(&sh->full[i], 1), mbar_init(&sh->freed[i], 1);
        mbar_init(&sh->all_done, 1);
        mbar_init(&sh->staged, 4);
        sh->abort = (smem_u32(smem_raw) & 1023u) ? 70 : 0;
        if (sh->abort) atomicMax(&g_tc_status, 70);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&sh->tmem_base, 128);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one() && !sh->abort) {
            tma_prefetch_desc(&amap), tma_prefetch_desc(&bmap);
            int issued = 0;
            for (int s = 0; s < n_steps; ++s) {
                const int st = s % kStages, k0 = k_begin + s * 64;
                if (s >= kStages && !gmwait(&sh->freed[st], (uint32_t)(((s / kStages) & 1) ^ 1), sh)) { gmgive_up(sh, 71); break; }
                uint8_t *base = smem_raw + st * SB;
                mbar_arrive_expect_tx(&sh->full[st], 4 * TB);
                // tensor maps: dims (64 columns, rows, column blocks, planes)
                if (A_MN) {  // rows = contraction, columns = M: 64 rows x two blocks
                    tma_load_4d(base, &amap, &sh->full[st], 0, k0, m0 / 64, pa);
                    tma_load_4d(base + TB, &amap, &sh->full[st], 0, k0, m0 / 64, pa + la);
                } else {     // rows = M, columns = contraction: 128 rows x one block
                    tma_load_4d(base, &amap, &sh->full[st], 0, m0, k0 / 64, pa);
                    tma_load_4d(base + TB, &amap, &sh->full[st], 0, m0, k0 / 64, pa + la);
                }
                if (B_MN) {
                    tma_load_4d(base + 2 * TB, &bmap, &sh->full[st], 0, k0, n0 / 64, pb);
                    tma_load_4d(base + 3 * TB, &bmap, &sh->full[st], 0, k0, n0 / 64, pb + lb);
                } else {
                    tma_load_4d(base + 2 * TB, &bmap, &sh->full[st], 0, n0, k0 / 64, pb);
                    tma_load_4d(base + 3 * TB, &bmap, &sh->full[st], 0, n0, k0 / 64, pb + lb);
                }
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
            constexpr uint32_t idesc = idesc_f16(128, 128, A_MN, B_MN);
            const uint32_t s_u32 = smem_u32(smem_raw);
            bool ok = !sh->abort;
            for (int s = 0; ok && s < n_steps; ++s) {
                const int st = s % kStages;
                if (!gmwait(&sh->full[st], (uint32_t)((s / kStages) & 1), sh)) { gmgive_up(sh, 72); ok = false; break; }
                tc_fence_after();
                const uint32_t base = s_u32 + (uint32_t)(st * SB);
                const uint64_t ah = A_MN ? desc_mnmajor_16b(base, 64 * 128) : desc_kmajor(base);
                const uint64_t al = A_MN ? desc_mnmajor_16b(base + TB, 64 * 128) : desc_kmajor(base + TB);
                const uint64_t bh = B_MN ? desc_mnmajor_16b(base + 2 * TB, 64 * 128) : desc_kmajor(base + 2 * TB);
                const uint64_t bl = B_MN ? desc_mnmajor_16b(base + 3 * TB, 64 * 128) : desc_kmajor(base + 3 * TB);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    // a 16-deep step: 32 bytes along a K-major row, two 8-row atoms (2048 bytes) down an M/N-major tile
                    const uint32_t ao = A_MN ? kk * 2048 : kk * 32, bo = B_MN ? kk * 2048 : kk * 32;
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
        // TMEM lanes are reachable by the warp whose index modulo 4 owns them: warps 2..5 own lanes of (warp % 4)
        const int lane_grp = warp & 3;
        const int row = lane_grp * 32 + lane;  // the output row of the tile this thread reads
        const uint32_t lane_base = (uint32_t)(lane_grp * 32) << 16;
        bool ok = __all_sync(0xffffffffu, gmwait(&sh->all_done, 0, sh));
        if (!ok) gmgive_up(sh, 73);
        const float ma = block_mult(p.amax_a[p.a_shared ? 0 : b]), mb = block_mult(p.amax_b[p.b_shared ? 0 : b]);
        const float f = 1.0f / (ma * mb);
        // rows go through shared memory (the stages are idle now): 128 rows x 512 bytes, chunk c of row r at c ^ (r & 31)
        uint8_t *stage = smem_raw;
        if (ok) {
            tc_fence_after();
            uint8_t *srow = stage + row * 512;
#pragma unroll 1
            for (int c = 0; c < 128; c += 32) {
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
        if (__all_sync(0xffffffffu, gmwait(&sh->staged, 0, sh)) && !sh->abort) {
            float *cb = p.c + (long long)b * p.c_batch_stride;
            const int wrow0 = (warp - 2) * 32;
#pragma unroll 4
            for (int i = 0; i < 32; ++i) {
                const int r = wrow0 + i;
                const float4 o4 = *reinterpret_cast<const float4 *>(stage + r * 512 + ((lane ^ (r & 31)) << 4));
                const int gr = m0 + r, gc = n0 + lane * 4;
                if (gr < p.m_rows && gc < p.n_cols) {
                    float *dst = cb + (long long)gr * p.ldc + gc;
                    if (p.pieces == 1 && p.c_batch_stride != 0) *reinterpret_cast<float4 *>(dst) = o4;
                    else tcb::red_add_v4(dst, o4);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 128);
}

inline size_t gemm_smem_bytes() { return (size_t)kStages * 4 * (128 * 64 * 2) + sizeof(GemmShared); }

// Tensor map over [planes][rows][width] halves with a box of (64, box_rows, blocks, 1).
inline bool make_plane_map(CUtensorMap *map, const void *base, int planes, long long rows, int width, int blocks, int box_rows) {
    return make_half_tile_map(map, base, planes, rows, width, blocks * 64, box_rows);
}

template <bool A_MN, bool B_MN>
inline int launch_gemm(const CUtensorMap &amap, const CUtensorMap &bmap, const GemmParams &p, cudaStream_t stream) {
    const size_t smem = gemm_smem_bytes();
    if (optin_smem((const void *)gemm_f16split_tc<A_MN, B_MN>, smem)) return 1;
    const dim3 grid((unsigned)((p.m_rows + 127) / 128), (unsigned)((p.n_cols + 127) / 128), (unsigned)(p.batch * p.pieces));
    return ZT_LAUNCH("gemm_f16split_tc", stream, (gemm_f16split_tc<A_MN, B_MN><<<grid, kGemmThreads, smem, stream>>>(amap, bmap, p)));
}

}  // namespace tcg
}  // namespace zt
