// libztattn: the C ABI declared in include/zt_attn.h.
//
// This file holds only argument checking and dispatch; the kernels live in
// simt_kernels.cuh (CUDA-core, any admissible shape), decode_kernels.cuh
// (bandwidth-bound split-K decode) and tc_fwd.cuh (tcgen05/TMEM forward).
// There is no CPU path: every launching entry point needs a CUDA device.
//
// The refusal order and wording follow the reference's launchers
// (src/cuda/attn_kernels.cu:843-929 forward, :962-1011 backward) so that a caller
// probing the boundary sees the same answers from either library.
#include "../../include/zt_attn.h"

#include "decode_kernels.cuh"
#include "simt_kernels.cuh"
#include "zt_common.cuh"
#ifndef ZT_NO_TC
#include "tc_bwd.cuh"
#include "tc_fwd.cuh"
#include "tc_fwd16.cuh"
#include "tc_fwd16g.cuh"
#include "tc_fwd16x.cuh"
#include "tc_gemm.cuh"
#include "tc_bwd_wide.cuh"
#include "tc_bwd_fused.cuh"
#endif

#include <mutex>

namespace zt {

constexpr int kMinDim = 32, kMaxDim = 256;  // src/cuda/attn_kernels.cu:147-148
constexpr size_t kArenaBytes = 16u << 20;

// One arena per device for the entry points that take no workspace argument (the reference's own two, and
// the batched forward): created on the first call that needs scratch on that device, or by zt_attn_reserve.
// It only ever grows, and an arena that has been outgrown is retired, not freed: a launch queued earlier, or a
// thread that read the old pointer a moment ago, may still be using it, and cudaFree would also stall the
// device.  Retired arenas are released when the process ends.  A steady-state caller -- same shapes step after
// step -- allocates on its first step (or in zt_attn_reserve) and never again.
// Growth is refused (nullptr, with the reason recorded) while `stream` is being captured into a CUDA graph:
// an allocation inside a capture would break it, and the caller can size the arena beforehand.
// Every call on a device shares the arena: calls that use it must not overlap on the GPU (see zt_attn.h).
static void *device_arena(size_t need, cudaStream_t stream, bool *refused_in_capture = nullptr,
                          size_t *held_now = nullptr) {
    static void *arena[64] = {};
    static size_t held[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (held_now) {  // a query: how large is the current device's arena
        *held_now = held[dev];
        return arena[dev];
    }
    if (need < kArenaBytes) need = kArenaBytes;
    if (held[dev] < need) {
        // (the legacy default stream cannot be captured, and asking about it would itself disturb a capture
        // running on another stream)
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (stream != nullptr && cudaStreamIsCapturing(stream, &cap) != cudaSuccess) cudaGetLastError();
        if (cap != cudaStreamCaptureStatusNone) {
            if (refused_in_capture) *refused_in_capture = true;
            return nullptr;
        }
        void *fresh = nullptr;
        if (cudaMalloc(&fresh, need) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        arena[dev] = fresh, held[dev] = need;  // the old arena, if any, stays allocated until exit
    }
    return arena[dev];
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The checks both reference launchers share, in the reference's order.
static int check_geometry(int T, int n_heads, int n_kv_heads, int dim) {
    if (T < 1)
        return refuse("T %d is not launchable. A zero or negative query count gives a grid with no "
                      "blocks, or one the driver cannot form.", T);
    if (!zt_attn_dim_ok(dim))
        return refuse("head_dim %d is refused. It must be even and in [%d, %d].", dim, kMinDim, kMaxDim);
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        return refuse("%d heads over %d kv heads is not a group.", n_heads, n_kv_heads);
    if (n_heads > 65535) return refuse("%d heads exceeds the 65535 gridDim.y limit.", n_heads);
    return 0;
}

static int need_device() {
    if (!device_info()) return refuse("no usable CUDA device (this library has no CPU path).");
    return 0;
}

static int forward_impl(const float *q, const float *k, const float *v, float *out, float *lse,
                        int batch, int T, int n_heads, int n_kv_heads, int dim, int q_offset,
                        int n_keys, cudaStream_t stream) {
    const float scale_log2 = kLog2e / sqrtf((float)dim);
    const long long q_bs = (long long)T * n_heads * dim;
    const long long kv_bs = (long long)n_keys * n_kv_heads * dim;
#ifndef ZT_NO_TC
    const int path = g_path.load();
    if ((path == 0 || path == 6 || path == 7 || path == 8) && n_kv_heads <= tcb::kPrepassMaxGroups &&
        tc_fwd16_supported(batch, T, dim, q_offset, n_keys, q, k, v, out)) {
        // The f16-split forward keeps its operand planes in the per-device arena (no entry point
        // of the forward takes a workspace); see device_arena for when that allocates.
        const size_t need = tc_fwd16_workspace_bytes(batch, T, n_heads, n_kv_heads, dim);
        bool in_capture = false;
        void *arena = device_arena(need, stream, &in_capture);
        if (in_capture)
            return refuse("this shape needs %zu bytes of the per-device arena, which would have to grow while the "
                          "stream is being captured: call zt_attn_reserve for the shape before the capture.", need);
        if (arena)
            return launch_fwd_tc16(q, k, v, out, lse, arena, batch, T, n_heads, n_kv_heads, dim, stream, nullptr, false,
                                   path == 6 ? 1 : (path == 7 ? 2 : 0));
    }
    if ((path == 0 || path == 2 || path == 6 || path == 7 || path == 8) &&
        tc_fwd_supported(batch, T, n_heads, n_kv_heads, dim, q_offset, n_keys, q, k, v, out)) {
        return launch_fwd_tc(q, k, v, out, lse, batch, T, n_heads, n_kv_heads, dim, stream);
    }
#endif
    SimtFwdParams p{};
    p.q = q, p.k = k, p.v = v, p.out = out, p.lse = lse;
    p.T = T, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads, p.dim = dim;
    p.q_offset = q_offset, p.n_keys = n_keys;
    p.q_batch_stride = q_bs, p.kv_batch_stride = kv_bs, p.lse_batch_stride = (long long)T * n_heads;
    p.scale_log2 = scale_log2;
    p.n_keys_dev = nullptr, p.bad_count = nullptr;
    return launch_fwd_simt(p, batch, stream);
}

static size_t backward_workspace(int batch, int T, int n_heads, int n_kv_heads, int dim) {
#ifndef ZT_NO_TC
    if ((dim == 32 || dim == 64 || dim == 96 || dim == 128) && T >= 128)
        return tc_bwd_workspace_bytes(batch, T, n_heads, n_kv_heads, dim);
    // head_dim 192 and 256: the planes of the fused form, then a row-scaled copy of Q's and the planes of P and dS
    if ((dim == 192 || dim == 256) && T >= 128) return tc_bwd_wide_workspace_bytes(batch, T, n_heads, n_kv_heads, dim);
#endif
    (void)batch, (void)n_heads, (void)n_kv_heads;
    return 0;
}

// The forward-for-training call (zt_attn_forward_batched_keep) leaves the f16 planes of q, k, v in the backward's
// workspace and hands the caller a token; a backward that is given the token back (zt_attn_backward_batched_kept)
// converts only dout.  The library keeps one record per (device, workspace) of which token is current, for which
// shape; a token is good for one backward, and any other call that writes the workspace retires it.  Nothing is
// ever inferred from pointer values of q, k, v: reuse happens only when the caller asks for it.
namespace {
struct KeptPlanes {
    const void *workspace = nullptr;
    int batch = 0, T = 0, n_heads = 0, n_kv_heads = 0, dim = 0;
    bool rope = false;  // the planes of q and k are rotated ones, for (pos, theta)
    int pos = 0;
    double theta = 0.0;
    unsigned long long token = 0;  // 0: no planes kept
};
constexpr int kKeptSlots = 8;
KeptPlanes g_kept[64][kKeptSlots];
unsigned long long g_next_token = 1;
std::mutex g_kept_mu;

// Forget whatever was kept in `workspace` (the caller is about to overwrite it).
void drop_kept_planes(const void *workspace) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return;
    std::lock_guard<std::mutex> lock(g_kept_mu);
    for (KeptPlanes &n : g_kept[dev])
        if (n.workspace == workspace) n = KeptPlanes{};
}
// Record that `workspace` now holds the planes of a forward of this shape; returns the token for them.
unsigned long long note_kept_planes(const void *workspace, int batch, int T, int n_heads, int n_kv_heads, int dim,
                                    bool rope = false, int pos = 0, double theta = 0.0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lock(g_kept_mu);
    KeptPlanes *slot = nullptr;
    for (KeptPlanes &n : g_kept[dev])
        if (n.workspace == workspace) slot = &n;
    if (!slot)
        for (KeptPlanes &n : g_kept[dev])
            if (n.token == 0) { slot = &n; break; }
    if (!slot) {  // every slot holds a live token: the oldest one goes
        slot = &g_kept[dev][0];
        for (KeptPlanes &n : g_kept[dev])
            if (n.token < slot->token) slot = &n;
    }
    *slot = KeptPlanes{workspace, batch, T, n_heads, n_kv_heads, dim, rope, pos, theta, g_next_token++};
    return slot->token;
}
// true (and the token is spent) when `token` is the current one of `workspace`, for exactly this shape.
bool take_kept_planes(const void *workspace, unsigned long long token, int batch, int T, int n_heads, int n_kv_heads,
                      int dim, bool rope = false, int pos = 0, double theta = 0.0) {
    int dev = 0;
    if (token == 0 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    std::lock_guard<std::mutex> lock(g_kept_mu);
    for (KeptPlanes &n : g_kept[dev]) {
        if (n.workspace != workspace || n.token != token) continue;
        const bool hit = n.batch == batch && n.T == T && n.n_heads == n_heads && n.n_kv_heads == n_kv_heads &&
                         n.dim == dim && n.rope == rope && (!rope || (n.pos == pos && n.theta == theta));
        n = KeptPlanes{};
        return hit;
    }
    return false;
}
}  // namespace

// delta = sum_j dout * out is formed here (into the caller's `delta`), then the gradients.  `out` may alias dq
// (the reference ABI's backward rebuilds the forward's output there): it is read before dq is written.
static int backward_impl(const float *q, const float *k, const float *v, const float *out, const float *lse,
                         float *delta, const float *dout, float *dq, float *dk, float *dv,
                         void *workspace, size_t workspace_bytes, int batch, int T, int n_heads,
                         int n_kv_heads, int dim, cudaStream_t stream, bool kept = false,
                         const PeerList *dq_peers = nullptr) {
#ifndef ZT_NO_TC
    if (g_path.load() != 1 && workspace &&
        workspace_bytes >= backward_workspace(batch, T, n_heads, n_kv_heads, dim) &&
        (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0 &&
        n_kv_heads <= tcb::kPrepassMaxGroups && tcb::tc_bwd_supported(batch, T, dim, q, k, v, dout, dq, dk, dv)) {
        // the tensor-core kernels also want each row's |dout| (their scale of dS): the same pass writes it
        float *rnorm = tcb::bwd_workspace(workspace, batch, T, n_heads, n_kv_heads, tc_tile_dim(dim)).rnorm;
        if (launch_delta(out, dout, delta, rnorm, (long long)batch * T * n_heads, dim, stream)) return 1;
        return launch_bwd_tc(q, k, v, dout, lse, delta, dq, dk, dv, workspace, batch, T, n_heads, n_kv_heads,
                             dim, stream, nullptr, nullptr, kept, dq_peers, g_path.load() == 8);
    }
    const size_t wide_need = backward_workspace(batch, T, n_heads, n_kv_heads, dim);
    if (g_path.load() != 1 && workspace && wide_need > 0 && workspace_bytes >= wide_need &&
        (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0 && n_kv_heads <= tcb::kPrepassMaxGroups &&
        !(dq_peers && dq_peers->n > 0) &&
        tcw::tc_bwd_wide_supported(batch, T, n_heads, n_kv_heads, dim, q, k, v, dout, dq, dk, dv)) {
        float *rnorm = tcw::wide_workspace(workspace, batch, T, n_heads, n_kv_heads, tc_tile_dim(dim)).base.rnorm;
        if (launch_delta(out, dout, delta, rnorm, (long long)batch * T * n_heads, dim, stream)) return 1;
        return launch_bwd_wide(q, k, v, dout, lse, delta, dq, dk, dv, workspace, batch, T, n_heads, n_kv_heads, dim,
                               stream, kept, g_path.load() == 8);
    }
#endif
    if (dq_peers && dq_peers->n > 0)
        return refuse("peer copies of dq are written by the tensor-core backward only, which does not take this shape.");
    (void)workspace, (void)workspace_bytes, (void)kept;
    if (launch_delta(out, dout, delta, nullptr, (long long)batch * T * n_heads, dim, stream)) return 1;
    SimtBwdParams p{};
    p.q = q, p.k = k, p.v = v, p.dout = dout, p.lse = lse, p.delta = delta;
    p.dq = dq, p.dk = dk, p.dv = dv;
    p.T = T, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads, p.dim = dim;
    p.q_batch_stride = (long long)T * n_heads * dim;
    p.kv_batch_stride = (long long)T * n_kv_heads * dim;
    p.lse_batch_stride = (long long)T * n_heads;
    p.scale = 1.0f / sqrtf((float)dim);
    p.scale_log2 = kLog2e / sqrtf((float)dim);
    return launch_bwd_simt(p, batch, stream);
}

// ---- decode scratch that nobody allocates ---------------------------------------------------
// Scratch for zt_attn_decode_static lives in the library image itself: a fixed array in device
// global memory that exists on every GPU that loads this library, from load until the process
// ends.  Host code cannot use the array's name as a pointer (on the host the name only stands
// for the symbol); the device address is asked for once per device, below.
constexpr size_t kStaticScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticScratchBytes];

// The array's address on the CURRENT device, looked up on the first call made with that device
// current and remembered.  Returns nullptr (with the reason refused) when the lookup fails.
static void *static_scratch_address() {
    static void *address[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        refuse("the current CUDA device could not be read.");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!address[dev]) {
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_static_decode_scratch);
        if (e != cudaSuccess || !ptr) {
            cudaGetLastError();
            refuse("the built-in decode scratch could not be located on device %d: %s", dev,
                   cudaGetErrorString(e));
            return nullptr;
        }
        address[dev] = ptr;
    }
    return address[dev];
}

}  // namespace zt

using namespace zt;

extern "C" {

int zt_attn_dim_ok(int dim) { return !(dim < kMinDim || dim > kMaxDim || (dim & 1) != 0); }

// The reference's formulas (src/cuda/attn_kernels.cu:103-104,375-376,697-706), kept so
// that the numbers a caller reads are the reference's numbers.
size_t zt_attn_forward_shmem(int dim, int tile, int group_q) {
    const size_t base = (size_t)dim + (size_t)tile + 2u * (size_t)tile * ((size_t)dim + 1u);
    return (base + (size_t)(group_q - 1) * (size_t)(dim + tile)) * sizeof(float);
}
size_t zt_attn_bwd_dq_shmem(int dim, int tile) {
    return (2u * (size_t)dim + 2u * (size_t)tile + 2u * (size_t)tile * ((size_t)dim + 1u)) * sizeof(float);
}
size_t zt_attn_bwd_dkdv_shmem(int dim) { return 2u * (size_t)dim * sizeof(float); }

const char *zt_attn_last_error(void) { return g_last_error; }
const char *zt_attn_last_path(void) { return g_last_path; }
void zt_attn_set_verbose(int on) { g_verbose.store(on ? 1 : 0); }
int zt_attn_set_path(int path) {
    return g_path.exchange((path == 1 || path == 2 || path == 6 || path == 7 || path == 8) ? path : 0);
}
unsigned long long zt_attn_launch_count(void) { return g_launches.load(); }

int zt_attn_tc_status(int *host_status) {
    if (!host_status) return refuse("a null pointer was passed.");
#ifndef ZT_NO_TC
    if (need_device()) return 1;
    if (tc_status_read(host_status)) {
        const cudaError_t e = cudaGetLastError();
        return refuse("reading the tensor-core status failed: %s", cudaGetErrorString(e));
    }
#else
    *host_status = 0;
#endif
    return 0;
}

int zt_attn_tc_saturated(unsigned int *host_count) {
    if (!host_count) return refuse("a null pointer was passed.");
#ifndef ZT_NO_TC
    if (need_device()) return 1;
    if (tc_saturated_read(host_count)) {
        const cudaError_t e = cudaGetLastError();
        return refuse("reading the saturation count failed: %s", cudaGetErrorString(e));
    }
#else
    *host_count = 0;
#endif
    return 0;
}

int zt_attn_reserve(int batch, int T, int n_heads, int n_kv_heads, int dim) {
    g_last_error[0] = 0;
    if (batch < 1 || batch > 65535) return refuse("batch %d is not launchable (1 .. 65535).", batch);
    if (check_geometry(T, n_heads, n_kv_heads, dim)) return 1;
    if (need_device()) return 1;
    size_t need = kArenaBytes;  // the decode-shaped forward's partial results
#ifndef ZT_NO_TC
    if (n_kv_heads <= tcb::kPrepassMaxGroups && T >= 128 &&
        (dim == 32 || dim == 64 || dim == 96 || dim == 128 || dim == 192 || dim == 256)) {
        const size_t f = tc_fwd16_workspace_bytes(batch, T, n_heads, n_kv_heads, dim);
        const size_t b = backward_workspace(batch, T, n_heads, n_kv_heads, dim);
        need = f > need ? f : need;
        need = b > need ? b : need;
    }
#endif
    bool in_capture = false;
    if (!device_arena(need, nullptr, &in_capture))
        return refuse("the per-device arena of %zu bytes could not be allocated.", need);
    return 0;
}

#ifdef ZT_DEFECTS
// Only in the harness build: selects the defect the kernels compute with (zt_common.cuh); 0 is the correct kernel.
int zt_attn_set_defect(int defect) {
    if (need_device()) return 1;
    if (cudaMemcpyToSymbol(g_defect, &defect, sizeof(int)) != cudaSuccess) {
        const cudaError_t e = cudaGetLastError();
        return refuse("setting the defect failed: %s", cudaGetErrorString(e));
    }
    return 0;
}
#endif

size_t zt_attn_arena_bytes(void) {
    size_t held = 0;
    device_arena(0, nullptr, nullptr, &held);
    return held;
}

void zt_attn_profile(int on) { g_profile.store(on ? 1 : 0); }

int zt_attn_profile_read(char *host_buf, size_t cap) {
    std::vector<ProfEntry> taken;
    {
        std::lock_guard<std::mutex> lock(g_prof_mu);
        taken.swap(g_prof);
    }
    struct Row { std::string name; int n; double ms; };
    std::vector<Row> rows;
    for (const ProfEntry &e : taken) {
        float ms = 0.f;
        if (e.name && cudaEventSynchronize(e.stop) == cudaSuccess &&
            cudaEventElapsedTime(&ms, e.start, e.stop) == cudaSuccess) {
            bool found = false;
            for (Row &r : rows)
                if (r.name == e.name) { r.n += 1, r.ms += ms, found = true; break; }
            if (!found) rows.push_back(Row{e.name, 1, (double)ms});
        } else {
            cudaGetLastError();
        }
        cudaEventDestroy(e.start);
        cudaEventDestroy(e.stop);
    }
    std::string text;
    char line[256];
    for (const Row &r : rows) {
        snprintf(line, sizeof(line), "%s %d %.6f\n", r.name.c_str(), r.n, r.ms);
        text += line;
    }
    if (host_buf && cap > 0) {
        const size_t n = text.size() < cap - 1 ? text.size() : cap - 1;
        memcpy(host_buf, text.data(), n);
        host_buf[n] = 0;
    }
    return (int)rows.size();
}

int zt_attn_forward(const float *q, const float *k, const float *v, float *out, int T, int n_heads,
                    int n_kv_heads, int dim, int group_q, int max_tile, int q_offset, int n_keys,
                    zt_stream_t stream) {
    g_last_error[0] = 0;
    if (check_geometry(T, n_heads, n_kv_heads, dim)) return 1;
    if (group_q < 1 || group_q > 64 || (size_t)dim * (size_t)group_q > 1024)
        return refuse("group_q %d at head_dim %d is not launchable.", group_q, dim);
    // `q_offset > n_keys - T`, not `q_offset + T > n_keys`: the sum can overflow int, the
    // difference cannot once T >= 1 and n_keys >= 1 (src/cuda/attn_kernels.cu:886-899).
    if (q_offset < 0 || n_keys < 1 || q_offset > n_keys - T)
        return refuse("q_offset %d, n_keys %d is not launchable.", q_offset, n_keys);
    if (max_tile < 1)
        return refuse("max_tile %d is not launchable. A tile of zero never advances the key loop.",
                      max_tile);
    if (!q || !k || !v || !out) return refuse("a null device pointer was passed.");
    if (need_device()) return 1;

    if (T == 1 && dim % 4 == 0 && aligned16(q) && aligned16(k) && aligned16(v)) {
        // A decode step: split the context over many blocks.  The one query row sits at
        // q_offset and sees keys 0 .. q_offset (q_offset <= n_keys - 1 was checked above).
        n_keys = q_offset + 1;
        const DecodePlan pl = decode_plan(1, n_keys, n_heads, n_kv_heads, dim);
        bool in_capture = false;
        void *arena = pl.total_bytes <= kArenaBytes ? device_arena(kArenaBytes, (cudaStream_t)stream, &in_capture) : nullptr;
        if (in_capture)
            return refuse("the per-device arena does not exist yet and the stream is being captured: call "
                          "zt_attn_reserve before the capture.");
        if (arena) {
            DecodeParams p{};
            p.q = q, p.k_cache = k, p.v_cache = v, p.n_keys = nullptr, p.n_keys_all = n_keys;
            p.out = out, p.lse = nullptr;
            p.batch = 1, p.n_ctx = n_keys, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads, p.dim = dim;
            p.cache_batch_stride = 0;
            p.scale_log2 = kLog2e / sqrtf((float)dim);
            return launch_decode(p, pl, arena, (cudaStream_t)stream);
        }
    }
    return forward_impl(q, k, v, out, nullptr, 1, T, n_heads, n_kv_heads, dim, q_offset, n_keys,
                        (cudaStream_t)stream);
}

int zt_attn_backward(const float *q, const float *k, const float *v, const float *dout, float *dq,
                     float *dk, float *dv, float *row_max, float *row_den, float *row_del, int T,
                     int n_heads, int n_kv_heads, int dim, int max_tile, zt_stream_t stream) {
    g_last_error[0] = 0;
    if (check_geometry(T, n_heads, n_kv_heads, dim)) return 1;
    if (max_tile < 1)
        return refuse("max_tile %d is not launchable. A tile of zero never advances the key loop.",
                      max_tile);
    if (!q || !k || !v || !dout || !dq || !dk || !dv || !row_max || !row_den || !row_del)
        return refuse("a null device pointer was passed.");
    if (need_device()) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    // the arena must hold the backward's planes (at least the forward's): grown, if at all, before any launch
    const size_t need = backward_workspace(1, T, n_heads, n_kv_heads, dim);
    bool in_capture = false;
    void *arena = need ? device_arena(need, s, &in_capture) : nullptr;
    if (in_capture)
        return refuse("this shape needs %zu bytes of the per-device arena, which would have to grow while the "
                      "stream is being captured: call zt_attn_reserve for the shape before the capture.", need);
    // The reference's backward sees neither the forward's output nor its log-sum-exp, so
    // both are rebuilt here: the forward runs into dq (same shape as out, assigned later)
    // with the log-sum-exp into row_max, then row_del = sum_j dout * out.
    if (forward_impl(q, k, v, dq, row_max, 1, T, n_heads, n_kv_heads, dim, 0, T, s)) return 1;
    const long long n = (long long)T * n_heads;
    if (ZT_LAUNCH("fill_kernel", s, fill_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(row_den, n, 1.0f)))
        return 1;
    return backward_impl(q, k, v, dq, row_max, row_del, dout, dq, dk, dv, arena, arena ? need : 0, 1, T, n_heads,
                         n_kv_heads, dim, s);
}

int zt_attn_forward_batched(const float *q, const float *k, const float *v, float *out, float *lse,
                            int batch, int T, int n_heads, int n_kv_heads, int dim,
                            zt_stream_t stream) {
    g_last_error[0] = 0;
    if (batch < 1 || batch > 65535) return refuse("batch %d is not launchable (1 .. 65535).", batch);
    if (check_geometry(T, n_heads, n_kv_heads, dim)) return 1;
    if (!q || !k || !v || !out) return refuse("a null device pointer was passed.");
    if (need_device()) return 1;
    return forward_impl(q, k, v, out, lse, batch, T, n_heads, n_kv_heads, dim, 0, T,
                        (cudaStream_t)stream);
}

static int check_peers(float *const *host_peers, int n_peers, PeerList *list) {
    list->n = 0;
    if (n_peers < 0 || n_peers > kMaxPeers) return refuse("%d peer copies is outside 0 .. %d.", n_peers, kMaxPeers);
    if (n_peers > 0 && !host_peers) return refuse("a null list of peer pointers was passed.");
    for (int i = 0; i < n_peers; ++i) {
        if (!host_peers[i] || (reinterpret_cast<uintptr_t>(host_peers[i]) & 15u) != 0)
            return refuse("peer pointer %d is null or not 16-byte aligned.", i);
        list->ptr[i] = host_peers[i];
    }
    list->n = n_peers;
    return 0;
}

static int forward_keep_impl(const float *q, const float *k, const float *v, float *out, float *lse,
                             void *workspace, size_t workspace_bytes, int batch, int T, int n_heads,
                             int n_kv_heads, int dim, zt_stream_t stream, unsigned long long *host_token,
                             const PeerList *out_peers) {
    g_last_error[0] = 0;
    if (host_token) *host_token = 0;
    if (batch < 1 || batch > 65535) return refuse("batch %d is not launchable (1 .. 65535).", batch);
    if (check_geometry(T, n_heads, n_kv_heads, dim)) return 1;
    if (!q || !k || !v || !out) return refuse("a null device pointer was passed.");
    if (need_device()) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    if (workspace) drop_kept_planes(workspace);
#ifndef ZT_NO_TC
    const size_t need = backward_workspace(batch, T, n_heads, n_kv_heads, dim);
    const int keep_path = g_path.load();
    if ((keep_path == 0 || keep_path == 6 || keep_path == 7 || keep_path == 8) && need > 0 && workspace && workspace_bytes >= need &&
        (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0 && n_kv_heads <= tcb::kPrepassMaxGroups &&
        tc_fwd16_supported(batch, T, dim, 0, T, q, k, v, out)) {
        if (launch_fwd_tc16(q, k, v, out, lse, workspace, batch, T, n_heads, n_kv_heads, dim, s, nullptr, true,
                            keep_path == 6 ? 1 : (keep_path == 7 ? 2 : 0), nullptr, out_peers))
            return 1;
        const unsigned long long token = note_kept_planes(workspace, batch, T, n_heads, n_kv_heads, dim);
        if (host_token) *host_token = token;
        return 0;
    }
#endif
    // shapes the f16-split kernels do not take: the ordinary forward, nothing kept
    (void)workspace, (void)workspace_bytes;
    if (out_peers && out_peers->n > 0)
        return refuse("peer copies of out are written by the forward that keeps its planes in a workspace only (a "
                      "tensor-core shape and a backward workspace are needed).");
    return forward_impl(q, k, v, out, lse, batch, T, n_heads, n_kv_heads, dim, 0, T, s);
}

int zt_attn_forward_batched_keep(const float *q, const float *k, const float *v, float *out, float *lse,
                                 void *workspace, size_t workspace_bytes, int batch, int T, int n_heads,
                                 int n_kv_heads, int dim, zt_stream_t stream, unsigned long long *host_token) {
    return forward_keep_impl(q, k, v, out, lse, workspace, workspace_bytes, batch, T, n_heads, n_kv_heads, dim, stream,
                             host_token, nullptr);
}

int zt_attn_forward_batched_keep_peers(const float *q, const float *k, const float *v, float *out, float *lse,
                                       void *workspace, size_t workspace_bytes, int batch, int T, int n_heads,
                                       int n_kv_heads, int dim, zt_stream_t stream, unsigned long long *host_token,
                                       float *const *host_out_peers, int n_peers) {
    g_last_error[0] = 0;
    PeerList peers{};
    if (check_peers(host_out_peers, n_peers, &peers)) return 1;
    return forward_keep_impl(q, k, v, out, lse, workspace, workspace_bytes, batch, T, n_heads, n_kv_heads, dim, stream,
                             host_token, &peers);
}

size_t zt_attn_backward_workspace_bytes(int batch, int T, int n_heads, int n_kv_heads, int dim) {
    if (batch < 1 || T < 1 || n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || !zt_attn_dim_ok(dim))
        return 0;
    return backward_workspace(batch, T, n_heads, n_kv_heads, dim);
}

static int backward_kept_impl(const float *q, const float *k, const float *v, const float *out,
                              const float *lse, const float *dout, float *dq, float *dk, float *dv,
                              float *delta, void *workspace, size_t workspace_bytes, int batch, int T,
                              int n_heads, int n_kv_heads, int dim, zt_stream_t stream,
                              unsigned long long token, const PeerList *dq_peers) {
    if (batch < 1 || batch > 65535) return refuse("batch %d is not launchable (1 .. 65535).", batch);
    if (check_geometry(T, n_heads, n_kv_heads, dim)) return 1;
    if (!q || !k || !v || !out || !lse || !dout || !dq || !dk || !dv || !delta)
        return refuse("a null device pointer was passed.");
    const size_t need = zt_attn_backward_workspace_bytes(batch, T, n_heads, n_kv_heads, dim);
    if (need > 0 && (!workspace || workspace_bytes < need))
        return refuse("the backward needs %zu bytes of workspace, %zu were given.", need, workspace_bytes);
    if (need > 0 && (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
        return refuse("the backward workspace must be 256-byte aligned.");
    if (need_device()) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    // spent or not, a token does not outlive a backward that rewrites the workspace
    const bool kept = take_kept_planes(workspace, token, batch, T, n_heads, n_kv_heads, dim);
    if (token != 0 && !kept)
        return refuse("token %llu is not the current one of this workspace for this shape: the planes it stood for "
                      "are gone (pass 0 to convert q, k, v again).", token);
    if (workspace) drop_kept_planes(workspace);
    return backward_impl(q, k, v, out, lse, delta, dout, dq, dk, dv, workspace, workspace_bytes, batch, T, n_heads,
                         n_kv_heads, dim, s, kept, dq_peers);
}

int zt_attn_backward_batched_kept(const float *q, const float *k, const float *v, const float *out,
                                  const float *lse, const float *dout, float *dq, float *dk, float *dv,
                                  float *delta, void *workspace, size_t workspace_bytes, int batch, int T,
                                  int n_heads, int n_kv_heads, int dim, zt_stream_t stream,
                                  unsigned long long token) {
    g_last_error[0] = 0;
    return backward_kept_impl(q, k, v, out, lse, dout, dq, dk, dv, delta, workspace, workspace_bytes, batch, T, n_heads,
                              n_kv_heads, dim, stream, token, nullptr);
}

int zt_attn_backward_batched_kept_peers(const float *q, const float *k, const float *v, const float *out,
                                        const float *lse, const float *dout, float *dq, float *dk, float *dv,
                                        float *delta, void *workspace, size_t workspace_bytes, int batch, int T,
                                        int n_heads, int n_kv_heads, int dim, zt_stream_t stream,
                                        unsigned long long token, float *const *host_dq_peers, int n_peers) {
    g_last_error[0] = 0;
    PeerList peers{};
    if (check_peers(host_dq_peers, n_peers, &peers)) return 1;
    return backward_kept_impl(q, k, v, out, lse, dout, dq, dk, dv, delta, workspace, workspace_bytes, batch, T, n_heads,
                              n_kv_heads, dim, stream, token, &peers);
}

int zt_attn_backward_batched(const float *q, const float *k, const float *v, const float *out,
                             const float *lse, const float *dout, float *dq, float *dk, float *dv,
                             float *delta, void *workspace, size_t workspace_bytes, int batch, int T,
                             int n_heads, int n_kv_heads, int dim, zt_stream_t stream) {
    return zt_attn_backward_batched_kept(q, k, v, out, lse, dout, dq, dk, dv, delta, workspace, workspace_bytes, batch,
                                         T, n_heads, n_kv_heads, dim, stream, 0ull);
}

// ---- attention with the rotary embedding of q and k fused in ------------------------------------------
namespace {
struct RopeWorkspace {
    float2 *table;         // [T][dim / 2] (cos, sin)
    float2 *table_t;       // the same, [dim / 2][T]
    float *q_rot, *k_rot;  // rotated copies, used only off the fused path
    void *inner;           // the tensor-core kernels' workspace (operand planes)
    size_t inner_bytes, total_bytes;
};
RopeWorkspace rope_workspace(void *base, int batch, int T, int n_heads, int n_kv_heads, int dim) {
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    RopeWorkspace w{};
    char *c = static_cast<char *>(base);
    size_t off = 0;
    w.table = reinterpret_cast<float2 *>(c + off), off += up((size_t)T * (dim / 2) * sizeof(float2));
    w.table_t = reinterpret_cast<float2 *>(c + off), off += up((size_t)T * (dim / 2) * sizeof(float2));
    w.q_rot = reinterpret_cast<float *>(c + off), off += up((size_t)batch * T * n_heads * dim * sizeof(float));
    w.k_rot = reinterpret_cast<float *>(c + off), off += up((size_t)batch * T * n_kv_heads * dim * sizeof(float));
    w.inner = c + off;
    w.inner_bytes = backward_workspace(batch, T, n_heads, n_kv_heads, dim);  // >= the forward's planes
    off += up(w.inner_bytes);
    w.total_bytes = off;
    return w;
}
int check_rope_call(const void *workspace, size_t workspace_bytes, size_t need, int pos, double theta) {
    if (pos < 0) return refuse("pos %d is negative: a row cannot sit before position 0.", pos);
    if (!(theta > 0.0)) return refuse("theta %g is not a positive rotary base.", theta);
    if (!workspace || workspace_bytes < need)
        return refuse("the rope calls need %zu bytes of workspace, %zu were given.", need, workspace_bytes);
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return refuse("the rope workspace must be 256-byte aligned.");
    return 0;
}
}  // namespace

size_t zt_attn_rope_workspace_bytes(int batch, int T, int n_heads, int n_kv_heads, int dim) {
    if (batch < 1 || T < 1 || n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || !zt_attn_dim_ok(dim))
        return 0;
    return rope_workspace(nullptr, batch, T, n_heads, n_kv_heads, dim).total_bytes;
}

// zt_attn_forward_rope_batched; with out_planes the tensor-core kernel also leaves out as f16 planes there and
// *planes_written says whether it did (false off the tensor-core path).
static int forward_rope_impl(const float *q, const float *k, const float *v, float *out, float *lse,
                             void *workspace, size_t workspace_bytes, int batch, int T, int n_heads,
                             int n_kv_heads, int dim, int pos, double theta, zt_stream_t stream,
                             unsigned long long *host_token, __half *out_planes, bool *planes_written) {
    g_last_error[0] = 0;
    if (planes_written) *planes_written = false;
    if (host_token) *host_token = 0;
    if (batch < 1 || batch > 65535) return refuse("batch %d is not launchable (1 .. 65535).", batch);
    if (check_geometry(T, n_heads, n_kv_heads, dim)) return 1;
    if (!q || !k || !v || !out) return refuse("a null device pointer was passed.");
    const RopeWorkspace w = rope_workspace(workspace, batch, T, n_heads, n_kv_heads, dim);
    if (check_rope_call(workspace, workspace_bytes, w.total_bytes, pos, theta)) return 1;
    if (need_device()) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    drop_kept_planes(w.inner);
    if (launch_rope_table(w.table, w.table_t, T, dim, pos, theta, s)) return 1;
#ifndef ZT_NO_TC
    if ((g_path.load() == 0 || g_path.load() == 8) && n_kv_heads <= tcb::kPrepassMaxGroups &&
        tc_fwd16_supported(batch, T, dim, 0, T, q, k, v, out) &&
        w.inner_bytes >= tc_fwd16_workspace_bytes(batch, T, n_heads, n_kv_heads, dim)) {
        // the planes (rotated q and k among them) go where the backward keeps its own: the rope backward that
        // follows with the same workspace, tensors, pos and theta converts only dout
        if (launch_fwd_tc16(q, k, v, out, lse, w.inner, batch, T, n_heads, n_kv_heads, dim, s, w.table, true, 0, out_planes)) return 1;
        const unsigned long long token = note_kept_planes(w.inner, batch, T, n_heads, n_kv_heads, dim, true, pos, theta);
        if (host_token) *host_token = token;
        if (planes_written) *planes_written = out_planes != nullptr;
        return 0;
    }
#endif
    // off the fused path: rotate into the workspace, then the ordinary forward
    if (launch_rope_apply(q, w.q_rot, w.table, batch, T, n_heads * dim, dim, false, s)) return 1;
    if (launch_rope_apply(k, w.k_rot, w.table, batch, T, n_kv_heads * dim, dim, false, s)) return 1;
    return forward_impl(w.q_rot, w.k_rot, v, out, lse, batch, T, n_heads, n_kv_heads, dim, 0, T, s);
}

int zt_attn_forward_rope_batched(const float *q, const float *k, const float *v, float *out, float *lse,
                                 void *workspace, size_t workspace_bytes, int batch, int T, int n_heads,
                                 int n_kv_heads, int dim, int pos, double theta, zt_stream_t stream,
                                 unsigned long long *host_token) {
    return forward_rope_impl(q, k, v, out, lse, workspace, workspace_bytes, batch, T, n_heads, n_kv_heads, dim, pos, theta,
                             stream, host_token, nullptr, nullptr);
}

int zt_attn_backward_rope_batched(const float *q, const float *k, const float *v, const float *out,
                                  const float *lse, const float *dout, float *dq, float *dk, float *dv,
                                  float *delta, void *workspace, size_t workspace_bytes, int batch, int T,
                                  int n_heads, int n_kv_heads, int dim, int pos, double theta,
                                  zt_stream_t stream, unsigned long long token) {
    g_last_error[0] = 0;
    if (batch < 1 || batch > 65535) return refuse("batch %d is not launchable (1 .. 65535).", batch);
    if (check_geometry(T, n_heads, n_kv_heads, dim)) return 1;
    if (!q || !k || !v || !out || !lse || !dout || !dq || !dk || !dv || !delta)
        return refuse("a null device pointer was passed.");
    const RopeWorkspace w = rope_workspace(workspace, batch, T, n_heads, n_kv_heads, dim);
    if (check_rope_call(workspace, workspace_bytes, w.total_bytes, pos, theta)) return 1;
    if (need_device()) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    const bool kept = take_kept_planes(w.inner, token, batch, T, n_heads, n_kv_heads, dim, true, pos, theta);
    if (token != 0 && !kept)
        return refuse("token %llu is not the current one of this workspace for this shape, pos and theta: the planes "
                      "it stood for are gone (pass 0 to convert q, k, v again).", token);
    drop_kept_planes(w.inner);
    if (launch_rope_table(w.table, w.table_t, T, dim, pos, theta, s)) return 1;
    bool fused = false, dq_in_kernel = false;
#ifndef ZT_NO_TC
    fused = g_path.load() != 1 && w.inner_bytes > 0 && n_kv_heads <= tcb::kPrepassMaxGroups &&
            tcb::tc_bwd_supported(batch, T, dim, q, k, v, dout, dq, dk, dv);
    // the dQ kernel's epilogue rotates whole 16- or 32-column pieces: not at head_dim 96, whose halves are 48 wide;
    // and the fused backward adds partial sums into dq, which can only be rotated once they are complete
    const bool two_kernels = g_path.load() == 8;
    dq_in_kernel = fused && dim != 96 && !tc_bwd_takes_fused(dim, two_kernels, nullptr);
    if (fused && launch_delta(out, dout, delta, tcb::bwd_workspace(w.inner, batch, T, n_heads, n_kv_heads, tc_tile_dim(dim)).rnorm,
                              (long long)batch * T * n_heads, dim, s))
        return 1;
    if (fused && launch_bwd_tc(q, k, v, dout, lse, delta, dq, dk, dv, w.inner, batch, T, n_heads, n_kv_heads, dim, s,
                               w.table, dq_in_kernel ? w.table_t : nullptr, kept, nullptr, two_kernels))
        return 1;
#endif
    if (!fused) {
        if (launch_rope_apply(q, w.q_rot, w.table, batch, T, n_heads * dim, dim, false, s)) return 1;
        if (launch_rope_apply(k, w.k_rot, w.table, batch, T, n_kv_heads * dim, dim, false, s)) return 1;
        // (head_dim 192 and 256 take the unfused tensor-core form, which wants the inner workspace)
        const bool wide = dim == 192 || dim == 256;
        if (backward_impl(w.q_rot, w.k_rot, v, out, lse, delta, dout, dq, dk, dv, wide ? w.inner : nullptr,
                          wide ? w.inner_bytes : 0, batch, T, n_heads, n_kv_heads, dim, s))
            return 1;
    }
    // the gradients of the unrotated q and k: R^T.  The tensor-core dQ kernel applies it as it writes dq; dk
    // (a quarter of dq's bytes here, flushed from its accumulator many times) takes a pass in place.
    if (!dq_in_kernel && launch_rope_apply(dq, dq, w.table, batch, T, n_heads * dim, dim, true, s)) return 1;
    return launch_rope_apply(dk, dk, w.table, batch, T, n_kv_heads * dim, dim, true, s);
}

// ---- the projection after attention: y = ctx . wo, and its gradients ------------------------------------------
namespace {
struct ProjWorkspace {
    uint32_t *amax_ctx, *amax_w, *amax_dy;  // [batch], [1], [batch]
    __half *ctx_planes, *w_planes, *dy_planes;
    size_t total_bytes, header_bytes;
};
ProjWorkspace proj_workspace(void *base, int batch, int T, int k, int n) {
    auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
    ProjWorkspace w{};
    char *c = static_cast<char *>(base);
    w.amax_ctx = reinterpret_cast<uint32_t *>(c), w.amax_w = w.amax_ctx + batch, w.amax_dy = w.amax_w + 1;
    w.header_bytes = up((size_t)(2 * batch + 1) * sizeof(uint32_t));
    size_t off = w.header_bytes;
    w.ctx_planes = reinterpret_cast<__half *>(c + off), off += up((size_t)2 * batch * T * k * sizeof(__half));
    w.w_planes = reinterpret_cast<__half *>(c + off), off += up((size_t)2 * k * n * sizeof(__half));
    w.dy_planes = reinterpret_cast<__half *>(c + off), off += up((size_t)2 * batch * T * n * sizeof(__half));
    w.total_bytes = off;
    return w;
}
int check_proj(const void *workspace, size_t workspace_bytes, int batch, int T, int k, int n) {
    if (batch < 1 || batch > 65535) return refuse("batch %d is not launchable (1 .. 65535).", batch);
    if (T < 1) return refuse("T %d is not launchable.", T);
    if (k < 64 || n < 64 || k % 64 != 0 || n % 64 != 0)
        return refuse("a projection of %d x %d is refused: both extents must be multiples of 64 (the tensor-core "
                      "tiles' column blocks); there is no CUDA-core form of this call.", k, n);
    const size_t need = proj_workspace(nullptr, batch, T, k, n).total_bytes;
    if (!workspace || workspace_bytes < need)
        return refuse("the projection needs %zu bytes of workspace, %zu were given.", need, workspace_bytes);
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return refuse("the projection workspace must be 256-byte aligned.");
    if (need_device()) return 1;
#ifdef ZT_NO_TC
    return refuse("this build has no tensor-core kernels.");
#else
    const DeviceInfo *d = device_info();
    if (!d || d->cc_major != 10 || get_encode_tiled() == nullptr) return refuse("the projection needs an sm_100 device.");
    return 0;
#endif
}
#ifndef ZT_NO_TC
// planes of x [batch][rows][width] with one scale per batch item
int proj_planes(const float *x, uint32_t *amax, __half *planes, int batch, int rows, int width, cudaStream_t s) {
    tcb::PrepassArgs pa{};
    pa.n = 1, pa.batch = batch, pa.T = rows;
    pa.t[0] = {x, amax, planes, width, width, width, width, nullptr};
    return tcb::launch_prepass(pa, s);
}
#endif
}  // namespace

size_t zt_proj_workspace_bytes(int batch, int T, int k, int n) {
    if (batch < 1 || T < 1 || k < 1 || n < 1) return 0;
    return proj_workspace(nullptr, batch, T, k, n).total_bytes;
}

#ifndef ZT_NO_TC
// amax_ctx[b] = max over the sequence's KV heads of max |v|: the scale the forward's epilogue gave out's planes
__global__ void seq_amax_kernel(const uint32_t *__restrict__ amax_v, uint32_t *__restrict__ amax_ctx, int n_kv_heads) {
    uint32_t top = 0;
    for (int g = 0; g < n_kv_heads; ++g) top = max(top, amax_v[blockIdx.x * n_kv_heads + g]);
    amax_ctx[blockIdx.x] = top;
}
#endif

// y = ctx . w.  ctx_planes_from: null (ctx is converted here), or the [batch, n_kv_heads] maxima of v that scaled the
// planes the attention kernel has already left in the workspace.
static int proj_forward_impl(const float *ctx, const float *w, float *y, void *workspace, int batch, int T, int k, int n,
                             cudaStream_t s, bool header_cleared, const uint32_t *ctx_planes_from, int n_kv_heads) {
#ifndef ZT_NO_TC
    const ProjWorkspace ws = proj_workspace(workspace, batch, T, k, n);
    const int pieces = (k + tcg::kPiece - 1) / tcg::kPiece;
    if ((!header_cleared && cudaMemsetAsync(ws.amax_ctx, 0, ws.header_bytes, s) != cudaSuccess) ||
        (pieces > 1 && cudaMemsetAsync(y, 0, (size_t)batch * T * n * sizeof(float), s) != cudaSuccess)) {
        cudaGetLastError();
        return refuse("could not clear the projection's buffers");
    }
    if (ctx_planes_from) {
        if (ZT_LAUNCH("seq_amax_kernel", s, (seq_amax_kernel<<<(unsigned)batch, 1, 0, s>>>(ctx_planes_from, ws.amax_ctx, n_kv_heads))))
            return 1;
    } else if (proj_planes(ctx, ws.amax_ctx, ws.ctx_planes, batch, T, k, s)) {
        return 1;
    }
    if (proj_planes(w, ws.amax_w, ws.w_planes, 1, k, n, s)) return 1;
    CUtensorMap amap, bmap;
    if (!tcg::make_plane_map(&amap, ws.ctx_planes, 2 * batch, T, k, 1, 128) ||   // rows x K, K-major
        !tcg::make_plane_map(&bmap, ws.w_planes, 2, k, n, 2, 64))                // K x N, N-major
        return refuse("the TMA tensor maps for the projection could not be encoded.");
    tcg::GemmParams p{};
    p.c = y, p.ldc = n, p.c_batch_stride = (long long)T * n, p.m_rows = T, p.n_cols = n, p.depth = k, p.pieces = pieces;
    p.batch = batch, p.amax_a = ws.amax_ctx, p.amax_b = ws.amax_w, p.a_shared = 0, p.b_shared = 1;
    g_last_path = "tcgen05";
    return tcg::launch_gemm<false, true>(amap, bmap, p, s);
#else
    return 1;
#endif
}

int zt_proj_forward(const float *ctx, const float *w, float *y, void *workspace, size_t workspace_bytes, int batch, int T,
                    int k, int n, zt_stream_t stream) {
    g_last_error[0] = 0;
    if (!ctx || !w || !y) return refuse("a null device pointer was passed.");
    if (check_proj(workspace, workspace_bytes, batch, T, k, n)) return 1;
    return proj_forward_impl(ctx, w, y, workspace, batch, T, k, n, (cudaStream_t)stream, false, nullptr, 0);
}

int zt_attn_block_forward(const float *q, const float *k, const float *v, const float *wo, float *ctx, float *lse, float *y,
                          void *rope_ws, size_t rope_ws_bytes, void *proj_workspace_, size_t proj_workspace_bytes,
                          int batch, int T, int n_heads, int n_kv_heads, int dim, int d_model, int pos, double theta,
                          zt_stream_t stream, unsigned long long *host_token) {
    g_last_error[0] = 0;
    if (host_token) *host_token = 0;
    if (!q || !k || !v || !wo || !ctx || !y) return refuse("a null device pointer was passed.");
    if (batch < 1 || batch > 65535) return refuse("batch %d is not launchable (1 .. 65535).", batch);
    if (check_geometry(T, n_heads, n_kv_heads, dim)) return 1;
    const int kdim = n_heads * dim;
    if (check_proj(proj_workspace_, proj_workspace_bytes, batch, T, kdim, d_model)) return 1;
    cudaStream_t s = (cudaStream_t)stream;
#ifndef ZT_NO_TC
    const ProjWorkspace pw = proj_workspace(proj_workspace_, batch, T, kdim, d_model);
    if (cudaMemsetAsync(pw.amax_ctx, 0, pw.header_bytes, s) != cudaSuccess) {
        cudaGetLastError();
        return refuse("could not clear the projection's buffers");
    }
    bool planes_written = false;
    if (forward_rope_impl(q, k, v, ctx, lse, rope_ws, rope_ws_bytes, batch, T, n_heads, n_kv_heads, dim, pos,
                          theta, stream, host_token, pw.ctx_planes, &planes_written))
        return 1;
    const uint32_t *from = nullptr;
    if (planes_written) {
        const RopeWorkspace rw = rope_workspace(rope_ws, batch, T, n_heads, n_kv_heads, dim);
        from = tcb::bwd_workspace(rw.inner, batch, T, n_heads, n_kv_heads, tc_tile_dim(dim)).amax_v;
    }
    return proj_forward_impl(ctx, wo, y, proj_workspace_, batch, T, kdim, d_model, s, true, from, n_kv_heads);
#else
    (void)s, (void)lse, (void)rope_ws, (void)rope_ws_bytes, (void)pos, (void)theta;
    return 1;
#endif
}

int zt_proj_backward(const float *ctx, const float *w, const float *dy, float *dctx, float *dw, void *workspace,
                     size_t workspace_bytes, int batch, int T, int k, int n, zt_stream_t stream) {
    g_last_error[0] = 0;
    if (!ctx || !w || !dy || !dctx || !dw) return refuse("a null device pointer was passed.");
    if (check_proj(workspace, workspace_bytes, batch, T, k, n)) return 1;
#ifndef ZT_NO_TC
    cudaStream_t s = (cudaStream_t)stream;
    const ProjWorkspace ws = proj_workspace(workspace, batch, T, k, n);
    const int pieces_in = (n + tcg::kPiece - 1) / tcg::kPiece;   // inputGrad contracts over n
    const int pieces_w = (T + tcg::kPiece - 1) / tcg::kPiece;    // weightGrad contracts over a sequence's rows
    if (cudaMemsetAsync(ws.amax_ctx, 0, ws.header_bytes, s) != cudaSuccess ||
        (pieces_in > 1 && cudaMemsetAsync(dctx, 0, (size_t)batch * T * k * sizeof(float), s) != cudaSuccess)) {
        cudaGetLastError();
        return refuse("could not clear the projection's buffers");
    }
    if (proj_planes(ctx, ws.amax_ctx, ws.ctx_planes, batch, T, k, s)) return 1;
    if (proj_planes(w, ws.amax_w, ws.w_planes, 1, k, n, s)) return 1;
    if (proj_planes(dy, ws.amax_dy, ws.dy_planes, batch, T, n, s)) return 1;
    CUtensorMap dy_k, w_k, ctx_m, dy_n;
    if (!tcg::make_plane_map(&dy_k, ws.dy_planes, 2 * batch, T, n, 1, 128) ||   // A: rows x N, K-major (contraction over n)
        !tcg::make_plane_map(&w_k, ws.w_planes, 2, k, n, 1, 128) ||             // B: w's rows are dctx's columns, K-major
        !tcg::make_plane_map(&ctx_m, ws.ctx_planes, 2 * batch, T, k, 2, 64) ||  // A: ctx^T, rows are the contraction
        !tcg::make_plane_map(&dy_n, ws.dy_planes, 2 * batch, T, n, 2, 64))      // B: rows x N, N-major
        return refuse("the TMA tensor maps for the projection could not be encoded.");
    g_last_path = "tcgen05";
    tcg::GemmParams p{};
    // inputGrad (src/autograd.zig:999-1022): dctx = dy . w^T, assigned
    p.c = dctx, p.ldc = k, p.c_batch_stride = (long long)T * k, p.m_rows = T, p.n_cols = k, p.depth = n, p.pieces = pieces_in;
    p.batch = batch, p.amax_a = ws.amax_dy, p.amax_b = ws.amax_w, p.a_shared = 0, p.b_shared = 1;
    if (tcg::launch_gemm<false, false>(dy_k, w_k, p, s)) return 1;
    // weightGrad (src/autograd.zig:958-972): dw += ctx^T . dy, every sequence and every piece of it added in
    tcg::GemmParams g{};
    g.c = dw, g.ldc = n, g.c_batch_stride = 0, g.m_rows = k, g.n_cols = n, g.depth = T, g.pieces = pieces_w;
    g.batch = batch, g.amax_a = ws.amax_ctx, g.amax_b = ws.amax_dy, g.a_shared = 0, g.b_shared = 0;
    return tcg::launch_gemm<true, true>(ctx_m, dy_n, g, s);
#else
    return 1;
#endif
}

size_t zt_attn_decode_workspace_bytes(int batch, int n_ctx, int n_heads, int n_kv_heads, int dim) {
    if (batch < 1 || n_ctx < 1 || n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 ||
        !zt_attn_dim_ok(dim))
        return 0;
    return decode_plan(batch, n_ctx, n_heads, n_kv_heads, dim).total_bytes;
}

int zt_attn_decode(const float *q, const float *k_cache, const float *v_cache, const int *n_keys,
                   float *out, float *lse, void *workspace, size_t workspace_bytes, int batch,
                   int n_ctx, int n_heads, int n_kv_heads, int dim, zt_stream_t stream) {
    g_last_error[0] = 0;
    if (batch < 1 || batch > 65535) return refuse("batch %d is not launchable (1 .. 65535).", batch);
    if (n_ctx < 1) return refuse("n_ctx %d is not a cache.", n_ctx);
    if (check_geometry(1, n_heads, n_kv_heads, dim)) return 1;
    if (!q || !k_cache || !v_cache || !n_keys || !out)
        return refuse("a null device pointer was passed.");
    const DecodePlan pl = decode_plan(batch, n_ctx, n_heads, n_kv_heads, dim);
    if (!workspace || workspace_bytes < pl.total_bytes)
        return refuse("decode needs %zu bytes of workspace, %zu were given.", pl.total_bytes,
                      workspace_bytes);
    if (!aligned16(workspace)) return refuse("the decode workspace must be 16-byte aligned.");
    if (need_device()) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    if (dim % 4 == 0 && aligned16(q) && aligned16(k_cache) && aligned16(v_cache)) {
        DecodeParams p{};
        p.q = q, p.k_cache = k_cache, p.v_cache = v_cache, p.n_keys = n_keys, p.n_keys_all = 0;
        p.out = out, p.lse = lse;
        p.batch = batch, p.n_ctx = n_ctx, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads, p.dim = dim;
        p.cache_batch_stride = (long long)n_ctx * n_kv_heads * dim;
        p.scale_log2 = kLog2e / sqrtf((float)dim);
        return launch_decode(p, pl, workspace, s);
    }
    // A width that is not a multiple of four floats (or unaligned buffers) cannot use
    // 128-bit loads: the general forward kernel runs one query row per sequence instead.
    if (cudaMemsetAsync(workspace, 0, kDecodeHeaderBytes, s) != cudaSuccess) {
        cudaGetLastError();
        return refuse("could not clear the decode workspace header");
    }
    SimtFwdParams p{};
    p.q = q, p.k = k_cache, p.v = v_cache, p.out = out, p.lse = lse;
    p.T = 1, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads, p.dim = dim;
    p.q_offset = 0, p.n_keys = n_ctx;
    p.q_batch_stride = (long long)n_heads * dim;
    p.kv_batch_stride = (long long)n_ctx * n_kv_heads * dim;
    p.lse_batch_stride = n_heads;
    p.scale_log2 = kLog2e / sqrtf((float)dim);
    p.n_keys_dev = n_keys, p.bad_count = reinterpret_cast<int *>(workspace);
    return launch_fwd_simt(p, batch, s);
}

size_t zt_attn_decode_static_capacity(void) { return kStaticScratchBytes; }

int zt_attn_decode_static(const float *q, const float *k_cache, const float *v_cache,
                          const int *n_keys, float *out, float *lse, int batch, int n_ctx,
                          int n_heads, int n_kv_heads, int dim, zt_stream_t stream) {
    g_last_error[0] = 0;
    if (batch < 1 || batch > 65535) return refuse("batch %d is not launchable (1 .. 65535).", batch);
    if (n_ctx < 1) return refuse("n_ctx %d is not a cache.", n_ctx);
    if (check_geometry(1, n_heads, n_kv_heads, dim)) return 1;
    if (!q || !k_cache || !v_cache || !n_keys || !out)
        return refuse("a null device pointer was passed.");
    if (dim % 4 != 0 || !aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache))
        return refuse("zt_attn_decode_static needs head_dim %% 4 == 0 and 16-byte aligned q and caches "
                      "(head_dim %d); use zt_attn_decode for other layouts.", dim);
    const DecodePlan pl = decode_plan(batch, n_ctx, n_heads, n_kv_heads, dim);
    if (pl.total_bytes > kStaticScratchBytes)
        return refuse("this decode shape needs %zu bytes of scratch and the built-in scratch holds %zu; "
                      "pass a workspace to zt_attn_decode instead.", pl.total_bytes, kStaticScratchBytes);
    if (need_device()) return 1;
    void *scratch = static_scratch_address();
    if (!scratch) return 1;
    DecodeParams p{};
    p.q = q, p.k_cache = k_cache, p.v_cache = v_cache, p.n_keys = n_keys, p.n_keys_all = 0;
    p.out = out, p.lse = lse;
    p.batch = batch, p.n_ctx = n_ctx, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads, p.dim = dim;
    p.cache_batch_stride = (long long)n_ctx * n_kv_heads * dim;
    p.scale_log2 = kLog2e / sqrtf((float)dim);
    // launch_decode clears the scratch's header (the bad-sequence counter) on `stream` first;
    // every other word of the scratch that the combine step reads is written by this call.
    return launch_decode(p, pl, scratch, (cudaStream_t)stream);
}

int zt_attn_decode_status(const void *workspace, int *host_bad_sequences) {
    if (!host_bad_sequences) return refuse("a null pointer was passed.");
    // a null workspace asks for the built-in scratch of zt_attn_decode_static on the current device
    if (!workspace) workspace = static_scratch_address();
    if (!workspace) return 1;
    if (cudaMemcpy(host_bad_sequences, workspace, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        const cudaError_t e = cudaGetLastError();
        return refuse("reading the decode status failed: %s", cudaGetErrorString(e));
    }
    return 0;
}

int zt_kv_append(float *k_cache, float *v_cache, int *n_keys, const float *k_new,
                 const float *v_new, int *full_count, int batch, int n_ctx, int n_kv_heads, int dim,
                 zt_stream_t stream) {
    g_last_error[0] = 0;
    if (batch < 1) return refuse("batch %d is not launchable.", batch);
    // kv_cache.Layer.init refuses a zero context or width (src/kv_cache.zig:66).
    if (n_ctx < 1 || n_kv_heads < 1 || dim < 1) return refuse("a cache of %d x %d x %d is degenerate.", n_ctx, n_kv_heads, dim);
    if (!k_cache || !v_cache || !n_keys || !k_new || !v_new) return refuse("a null device pointer was passed.");
    if (need_device()) return 1;
    g_last_path = "kv-append";
    cudaStream_t s = (cudaStream_t)stream;
    return ZT_LAUNCH("kv_append_kernel", s,
                     kv_append_kernel<<<(unsigned)batch, 256, 0, s>>>(k_cache, v_cache, n_keys, k_new, v_new,
                                                                      full_count, n_ctx, n_kv_heads * dim));
}

}  // extern "C"
