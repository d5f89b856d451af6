// Blackwell (sm_100a) building blocks for the tensor-core kernels, as inline PTX:
// mbarriers with bounded waits, TMA tile loads, tensor-memory (TMEM) allocation and
// register<->TMEM moves, shared-memory matrix descriptors and tcgen05.mma issue.
//
// Every wait in this file is bounded: it gives up after a fixed number of polls, and the
// caller then raises the kernel's error flag and leaves through its normal epilogue, so a
// protocol mistake costs a wrong answer and a status word, never a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace zt {
namespace tc {

// ---- addresses ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival for a whole warp: every lane's earlier writes are ordered before the elected
// arrival by the warp barrier.  Hundreds of per-thread arrivals on one barrier word serialise
// (each is a shared-memory atomic); per-warp arrival keeps a hand-off to a few of them.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t *bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
// The same without the release: for hand-offs of TMEM contents only, which tcgen05.wait and the tcgen05 fences
// order by themselves.  A releasing arrival also waits for the thread's earlier global stores and reductions
// to be performed -- a round trip to L2 that the waiting tensor core has no use for.
__device__ __forceinline__ void mbar_arrive_warp_relaxed(uint64_t *bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0)
        asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Polls at most kWaitPolls times (each poll may itself block for a hardware-defined short
// time).  Returns false when the phase never completed.
constexpr uint32_t kWaitPolls = 4u << 20;
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitPolls; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// ---- proxies and tcgen05 fences ------------------------------------------------------------
// Generic-proxy writes to shared memory (st.shared) become visible to the async proxy
// (TMA, tcgen05.mma operand reads) only after this fence.
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMA -------------------------------------------------------------------------------------
// 4-D tiled load (no multicast) into this CTA's shared memory, completion on `bar`.
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0,
                                            int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// The same tile into L2 only: nothing lands in shared memory and nothing is signalled.
__device__ __forceinline__ void tma_prefetch_l2_4d(const CUtensorMap *map, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(map), "r"(c0), "r"(c1),
                 "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tensor memory ----------------------------------------------------------------------------
// Whole-warp calls.  `slot` is a shared-memory word that receives the base address.
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(ncols) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp moves row (lane base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 8 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// TMEM address: lane in bits [31:16], column in bits [15:0].
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
    return base + (lane << 16) + col;
}

// ---- descriptors --------------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bits): start address >> 4 in [0,14), leading byte offset >> 4
// in [16,30), stride byte offset >> 4 in [32,46), version 1 in [46,48), layout type in [61,64)
// (2 = 128-byte swizzle).  All operand tiles here are stored as column blocks of 32 floats:
// block c holds rows x 128 bytes, 128-byte swizzled in 8-row (1024-byte) atoms -- exactly what a
// TMA box with a 32-float inner extent and CU_TENSOR_MAP_SWIZZLE_128B writes.
constexpr uint64_t kDescSw128 = (uint64_t)1 << 46 | (uint64_t)2 << 61;

// Operand whose contraction index runs along the 128-byte rows ("K-major"): rows are the M or N
// index; 8-row atoms are 1024 bytes apart.  `addr` may be advanced by 32 bytes per 8-float K step
// inside a 1024-byte-aligned tile.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return kDescSw128 | (uint64_t)((addr >> 4) & 0x3fff) | (uint64_t)1 << 16 | (uint64_t)(1024 >> 4) << 32;
}
// Operand whose contraction index runs down the rows ("MN-major", e.g. V as the B operand of
// P.V): the 32 floats of a row are N indices and the rows are contraction indices.  For 32-bit
// operands the only MN-major layout the tensor core reads is the 128-byte swizzle with 32-byte
// atoms (layout type 1): 32-byte chunks of a row are permuted by the row index modulo 4, in
// 4-row (512-byte) atoms -- what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.  Column
// blocks (N index + 32) are `block_bytes` apart (leading offset); the next 4 contraction rows
// are 512 bytes on (stride offset).  One 8-deep MMA step spans two such atoms; the next step
// starts 1024 bytes further.
constexpr uint64_t kDescSw128Atom32 = (uint64_t)1 << 46 | (uint64_t)1 << 61;
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t block_bytes) {
    return kDescSw128Atom32 | (uint64_t)((addr >> 4) & 0x3fff) | (uint64_t)((block_bytes >> 4) & 0x3fff) << 16 |
           (uint64_t)(512 >> 4) << 32;
}

// A descriptor `bytes` further into the same tile (start-address field only; tiles sit below 256 KB,
// so the 14-bit field cannot carry).  With a compile-time `bytes` this is one integer add per MMA,
// which matters: one thread issues every MMA of a CTA, and an MMA of N = 64 executes in ~34 cycles.
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) { return desc + (uint64_t)(bytes >> 4); }

// Instruction descriptor for kind::tf32, f32 accumulate, M x N, A K-major (or in TMEM).
// c_format f32 = 1 at [4,6); a/b format tf32 = 2 at [7,10)/[10,13); b_major at 16; N >> 3 at
// [17,23); M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t idesc_tf32(int m, int n, bool b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// 16-bit operands (kind::f16, f16 inputs, f32 accumulate): both K-major and MN-major tiles use the
// plain 128-byte swizzle; a row is 64 halves, a column block is rows x 128 bytes.  MN-major:
// column blocks `block_bytes` apart (leading offset), 8 contraction rows per 1024-byte atom
// (stride offset); one 16-deep MMA step covers two atoms, the next step starts 2048 bytes on.
__device__ __forceinline__ uint64_t desc_mnmajor_16b(uint32_t addr, uint32_t block_bytes) {
    return kDescSw128 | (uint64_t)((addr >> 4) & 0x3fff) | (uint64_t)((block_bytes >> 4) & 0x3fff) << 16 |
           (uint64_t)(1024 >> 4) << 32;
}
// a/b format f16 = 0, c format f32 = 1.
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_ss_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] . B[smem]; issued by one thread.
__device__ __forceinline__ void mma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[smem] . B[smem]
__device__ __forceinline__ void mma_ss_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Make `bar` complete (one arrival) when every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---- 3xTF32 split --------------------------------------------------------------------------------
// kind::tf32 reads the sign, exponent and top 10 mantissa bits of a 32-bit operand and ignores
// the low 13 bits (truncation, measured).  Two splits x = hi + lo are used:
//  * operands that pass through registers (Q, P): hi = round-to-nearest tf32(x), so lo is
//    zero-mean with |lo| <= 2^-12 |x|;
//  * operands that TMA lands in shared memory (K, V): the raw f32 tile IS the hi operand (the
//    tensor core truncates it), lo = x - trunc(x) in [0, 2^-10 |x|).
// Either lo is itself rounded to tf32 before use, so the hardware's truncation of it adds no
// one-sided error.  The dropped lo.lo term is then a zero-mean ~2^-24 relative quantity.
__device__ __forceinline__ float tf32_trunc(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
__device__ __forceinline__ float tf32_round(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}

}  // namespace tc

// ---- host: tensor maps through the driver entry point (no link-time libcuda dependency) ---------
typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_tiled() {
    static PFN_encodeTiled fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiled>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

// Tensor map over a [batch, rows, heads*dim] f32 tensor seen as column blocks of 32 floats:
// dims (fastest first) = (32, rows, heads*dim/32, batch); box = (32, box_rows, dim/32, 1), 128-byte
// swizzle, zero fill out of bounds.  One load brings a (box_rows x dim) head tile in as dim/32
// column blocks of box_rows x 128 bytes each.
// `mn_major` selects the 32-byte-atom swizzle that an MN-major tf32 operand needs.
inline bool make_head_tile_map(CUtensorMap *map, const float *base, int batch, long long rows, int width,
                               int dim, int box_rows, bool mn_major) {
    PFN_encodeTiled enc = get_encode_tiled();
    if (!enc) return false;
    const cuuint64_t dims[4] = {32, (cuuint64_t)rows, (cuuint64_t)(width / 32), (cuuint64_t)batch};
    const cuuint64_t strides[3] = {(cuuint64_t)width * 4, 128, (cuuint64_t)rows * width * 4};
    const cuuint32_t box[4] = {32, (cuuint32_t)box_rows, (cuuint32_t)(dim / 32), 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE,
               mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor map over a [planes, rows, width] f16 tensor (planes = hi/lo x batch) seen as column
// blocks of 64 halves: dims (64, rows, width/64, planes); box (64, box_rows, dim/64, 1); plain
// 128-byte swizzle.
inline bool make_half_tile_map(CUtensorMap *map, const void *base, int planes, long long rows, int width,
                               int dim, int box_rows) {
    PFN_encodeTiled enc = get_encode_tiled();
    if (!enc) return false;
    const cuuint64_t dims[4] = {64, (cuuint64_t)rows, (cuuint64_t)(width / 64), (cuuint64_t)planes};
    const cuuint64_t strides[3] = {(cuuint64_t)width * 2, 128, (cuuint64_t)rows * width * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, (cuuint32_t)(dim / 64), 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace zt
