/*
 * zt_attn.h -- C ABI of libztattn, a Blackwell (sm_100a) implementation of
 * Z-TRANSFORMER's attention hot path.
 *
 * The first six functions are the reference library's own entry points, with the
 * reference's names, argument order, types and return conventions, so that the
 * reference's Zig holder (src/cuda/device.zig:58-105, `extern fn zt_attn_*`)
 * links against this library unchanged.  The rest are additive extensions for
 * the batched, log-sum-exp-saving, KV-cache-decode and sharded uses that the
 * reference's single-sequence ABI cannot express.
 *
 * Conventions (from src/cuda/attn_kernels.cu:21-54, kept):
 *   - every pointer is a DEVICE pointer unless its name starts with `host_`;
 *   - the caller owns all buffers; entry points taking a `workspace` argument
 *     never allocate.  The reference's two launching entry points and
 *     zt_attn_forward_batched take no workspace; their scratch (the 16-bit
 *     operand planes of q, k, v, dout: up to 4 bytes per element of those
 *     tensors, or 16 MiB for a decode-shaped call) lives in one per-device
 *     arena.  See "The per-device arena" below for when it allocates, how to
 *     make that never happen mid-run (zt_attn_reserve) and what calls that
 *     share it must not do;
 *   - return 0: the work was enqueued on `stream` (no synchronisation);
 *     return 1: refused, with the reason on stderr and in zt_attn_last_error();
 *     nothing was launched and no buffer was touched;
 *   - no entry point ever ends the process.
 *   - there is no CPU fallback anywhere: without a CUDA device every launching
 *     entry point returns 1.
 *
 * Layouts: q, out, dout, dq are [T, n_heads*dim] row-major f32 with head h in
 * columns h*dim .. (h+1)*dim-1; k, v, dk, dv are [T, n_kv_heads*dim]; query
 * head h reads KV head h / (n_heads / n_kv_heads) (src/attention.zig:29-35).
 * Batched forms hold `batch` such items back to back.
 */
#ifndef ZT_ATTN_H
#define ZT_ATTN_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t without pulling in the CUDA headers (it is `struct CUstream_st *`). */
typedef struct CUstream_st *zt_stream_t;

/* ------------------------------------------------------------------------- */
/* The reference's six entry points                                           */
/* ------------------------------------------------------------------------- */

/* Replaces src/cuda/attn_kernels.cu:648-659 (Zig: device.zig:58).
 * 1 iff dim is even and 32 <= dim <= 256.  Prints nothing. */
int zt_attn_dim_ok(int dim);

/* Replace src/cuda/attn_kernels.cu:697-706 (Zig: device.zig:65-67).  The
 * reference exports its kernels' shared-memory byte counts; the Zig side never
 * calls them.  They keep the reference's formulas so a caller comparing numbers
 * sees the same ones; this library's kernels size their own shared memory. */
size_t zt_attn_forward_shmem(int dim, int tile, int group_q);
size_t zt_attn_bwd_dq_shmem(int dim, int tile);
size_t zt_attn_bwd_dkdv_shmem(int dim);

/* Replaces src/cuda/attn_kernels.cu:833-938 (Zig: device.zig:69-86).
 * Fused causal GQA forward.  T query rows; n_keys rows of k and v exist;
 * q_offset is the absolute position of query row 0; key j is visible to query
 * row t iff j <= q_offset + t and j < n_keys.  Training shape: q_offset 0,
 * n_keys T.  Decode step: T 1, q_offset n_keys - 1.
 * group_q and max_tile are validated exactly as the reference validates them
 * and are otherwise advisory: tiling is this library's own business.
 * Refusals, in the reference's order: T < 1; dim not ok; heads not a group;
 * n_heads > 65535; group_q outside [1, 64] or dim*group_q > 1024;
 * q_offset < 0, n_keys < 1 or q_offset > n_keys - T; max_tile < 1.
 * A decode-shaped call (T == 1) splits the context over many blocks and keeps
 * its partial results in a per-device arena of 16 MiB that is allocated once,
 * on the first such call on that device. */
int zt_attn_forward(const float *q, const float *k, const float *v, float *out, int T, int n_heads,
                    int n_kv_heads, int dim, int group_q, int max_tile, int q_offset, int n_keys,
                    zt_stream_t stream);

/* Replaces src/cuda/attn_kernels.cu:952-1036 (Zig: device.zig:88-105).
 * Backward of the training-shaped forward.  dq, dk, dv are ASSIGNED (no
 * zeroing needed, nothing accumulated into).  row_max, row_den, row_del are
 * caller scratch of [T, n_heads] floats each; on return row_max holds each
 * row's log-sum-exp, row_den is 1 and row_del holds sum_j dout*out.  dq is used
 * as scratch for the recomputed forward output before it receives dq.
 * Refusals: T < 1; dim not ok; heads not a group; n_heads > 65535; max_tile < 1. */
int zt_attn_backward(const float *q, const float *k, const float *v, const float *dout, float *dq,
                     float *dk, float *dv, float *row_max, float *row_den, float *row_del, int T,
                     int n_heads, int n_kv_heads, int dim, int max_tile, zt_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Extensions                                                                 */
/* ------------------------------------------------------------------------- */

/* The per-device arena.  zt_attn_forward, zt_attn_backward and zt_attn_forward_batched have no
 * workspace argument (the reference's signatures have none, src/cuda/device.zig:69-105), so their
 * scratch comes from an arena this library keeps per device.  Rules:
 *  - it is allocated (cudaMalloc) by the first call on a device that needs it and grows when a
 *    later call needs more; it never shrinks, and an outgrown arena is kept until the process ends
 *    (work queued earlier may still be using it), so growth costs memory, never correctness;
 *  - zt_attn_reserve sizes it for a shape up front -- the place for it is where the reference's
 *    holder sizes its own eleven buffers (device.Attn.init, src/cuda/device.zig:221-299; that
 *    function already calls zt_attn_dim_ok).  After zt_attn_reserve(batch, T, ...) no call of
 *    that shape or a smaller one allocates.  (No counterpart in the reference, whose kernels need
 *    no scratch.)
 *  - while `stream` is being captured into a CUDA graph a call that would have to grow the arena
 *    is refused (return 1) instead of allocating inside the capture: reserve first;
 *  - every call on a device shares the arena: two calls that use it must not overlap on the GPU
 *    (different streams or host threads without an ordering between them) -- the second would
 *    overwrite the first one's operand planes.  Calls queued on one stream are safe.  The batched
 *    calls that take a caller workspace (_keep, backward_batched, _rope_, decode) do not touch it. */
int zt_attn_reserve(int batch, int T, int n_heads, int n_kv_heads, int dim);
/* Bytes the current device's arena holds now (0 before its first use). */
size_t zt_attn_arena_bytes(void);

/* The reason of the calling thread's most recent refusal ("" if none).  The
 * reference only prints to stderr (src/cuda/attn_kernels.cu:21-37); bindings
 * that cannot capture stderr read it here. */
const char *zt_attn_last_error(void);

/* 1 when stderr diagnostics are wanted (default), 0 to keep refusals silent
 * (the return code and zt_attn_last_error() still report them). */
void zt_attn_set_verbose(int on);

/* Which implementation the next launches use: 0 = automatic (the fastest tensor-core kernel the
 * shape allows, CUDA-core kernels elsewhere; the f16-split forward takes the same query rows of two
 * heads of a KV group per CTA when the group has an even number of query heads and that still gives
 * every SM a CTA, one head per CTA otherwise), 1 = CUDA-core kernels only, 2 = as 0 but the forward
 * uses the 3xTF32 kernel instead of the f16-split one, 6 = the f16-split forward with one head per
 * CTA, 7 = with two heads per CTA whatever the number of CTAs, 8 = as 0 but the backward takes its
 * earlier forms: up to head_dim 128 two kernels (dQ's, then dK/dV's) instead of the fused one --
 * slower by a quarter, and the only form whose dq is bit-reproducible run to run (the fused kernel
 * adds every key tile's share of dq in memory, in no fixed order: equal to rounding) -- and at 192
 * and 256 the scores kernel that loads every operand per tile.  Any other value selects 0.  For
 * tests, for bisecting a parity failure, and for a caller that needs run-to-run identical dq;
 * returns the previous value. */
int zt_attn_set_path(int path);

/* Batched training-shaped forward: `batch` independent sequences of T rows,
 * the batch loop around attention.forward (src/attention.zig:36-153).  Also
 * writes lse[batch, T, n_heads] = row max + ln(denominator) of the scaled
 * scores when lse is not NULL.  Same refusals as zt_attn_forward, plus batch < 1. */
int zt_attn_forward_batched(const float *q, const float *k, const float *v, float *out, float *lse,
                            int batch, int T, int n_heads, int n_kv_heads, int dim,
                            zt_stream_t stream);

/* Batched backward that consumes the forward's out and lse instead of
 * recomputing them (autograd.attentionBackward, src/autograd.zig:636-842, is the
 * arithmetic it must match).  delta is caller scratch [batch, T, n_heads].
 * dq, dk, dv are assigned.  workspace/workspace_bytes: see
 * zt_attn_backward_workspace_bytes; may be NULL/0 when that returns 0.
 * The workspace holds the 16-bit operand planes of q, k, v, dout;
 * at head_dim 192 and 256 it also holds the planes of P and dS of as many heads as fit in about 2 GiB
 * (at least one KV group's: 8 T^2 bytes a head), because the backward at those widths writes them to
 * memory between its launches; there dq, dk, dv are sums added in memory in no fixed order, equal run to
 * run to rounding only. */
int zt_attn_backward_batched(const float *q, const float *k, const float *v, const float *out,
                             const float *lse, const float *dout, float *dq, float *dk, float *dv,
                             float *delta, void *workspace, size_t workspace_bytes, int batch, int T,
                             int n_heads, int n_kv_heads, int dim, zt_stream_t stream);
size_t zt_attn_backward_workspace_bytes(int batch, int T, int n_heads, int n_kv_heads, int dim);

/* The forward of a training step: zt_attn_forward_batched, except that the 16-bit operand planes of
 * q, k, v it builds are written into the backward's workspace and kept there, and *host_token
 * (a host pointer, may be NULL) receives a token for them: non-zero when planes were kept, 0 when not
 * (a workspace that is NULL, short or misaligned, or a shape the tensor-core kernels do not take:
 * this is then the ordinary forward).  This call takes nothing from the per-device arena.
 * zt_attn_backward_batched_kept, given the same workspace, shape and that token, converts only dout
 * (a quarter less pre-pass traffic per step).  The token is the caller's statement that q, k, v have
 * not been written since the forward; the library never infers that from pointer values.  A token is
 * good for one backward; any other call that writes the workspace (another forward_keep, a plain
 * backward) retires it, and a retired or mismatched token is refused (return 1), never silently
 * honoured.  With token 0 the _kept call is zt_attn_backward_batched.  Tokens are checked on the
 * host when the call is made: when a CUDA graph is captured, capture the forward and its backward
 * together.  No reference counterpart (the reference's forward keeps nothing for its backward, which
 * recomputes the softmax statistics). */
int zt_attn_forward_batched_keep(const float *q, const float *k, const float *v, float *out, float *lse,
                                 void *workspace, size_t workspace_bytes, int batch, int T, int n_heads,
                                 int n_kv_heads, int dim, zt_stream_t stream, unsigned long long *host_token);
int zt_attn_backward_batched_kept(const float *q, const float *k, const float *v, const float *out,
                                  const float *lse, const float *dout, float *dq, float *dk, float *dv,
                                  float *delta, void *workspace, size_t workspace_bytes, int batch, int T,
                                  int n_heads, int n_kv_heads, int dim, zt_stream_t stream,
                                  unsigned long long token);

/* The training pair with the all-gather of out and dq done inside the kernels.  When independent sequences (or KV
 * groups) are sharded over the GPUs of a box and every GPU wants every shard's outputs, the gather that follows the
 * kernels moves as many bytes as the kernels write and, as an NCCL collective, competes with them for SMs.  These
 * two calls are zt_attn_forward_batched_keep and zt_attn_backward_batched_kept given, besides their own out / dq,
 * up to 7 PEER copies of it: device pointers into other GPUs' memory (mapped into this process: CUDA IPC, VMM
 * handles, torch symmetric memory), each pointing at the place this rank's shard has in that GPU's gathered tensor.
 * The kernel's epilogue stores every output row to all of them as it stores it locally -- plain stores over NVLink,
 * no loads from peer memory, no waits on a peer -- so when the kernel has finished (and the peers know it has: any
 * stream-ordered collective or barrier after it will do, e.g. the all-gather of dk and dv, which are small) the
 * gathered out and dq are complete everywhere.  host_*_peers is a host array of n_peers device pointers, 16-byte
 * aligned, each with room for the whole out / dq of this call.  Refusals: those of the plain calls; n_peers
 * outside 0..7; a null or misaligned peer pointer; a shape or workspace with which the plain call would leave the
 * tensor-core path (the CUDA-core kernels write no peer copies).  No reference counterpart (the reference is one
 * GPU). */
int zt_attn_forward_batched_keep_peers(const float *q, const float *k, const float *v, float *out, float *lse,
                                       void *workspace, size_t workspace_bytes, int batch, int T, int n_heads,
                                       int n_kv_heads, int dim, zt_stream_t stream, unsigned long long *host_token,
                                       float *const *host_out_peers, int n_peers);
int zt_attn_backward_batched_kept_peers(const float *q, const float *k, const float *v, const float *out,
                                        const float *lse, const float *dout, float *dq, float *dk, float *dv,
                                        float *delta, void *workspace, size_t workspace_bytes, int batch, int T,
                                        int n_heads, int n_kv_heads, int dim, zt_stream_t stream,
                                        unsigned long long token, float *const *host_dq_peers, int n_peers);

/* Attention with the rotary position embedding of its input side fused in: q and k are the
 * projections BEFORE rope.forward (src/rope.zig:21-55; the reference rotates them first,
 * src/model.zig:372-375 and src/decode.zig:244-246); row r sits at absolute position pos + r,
 * element i of a head pairs with element i + dim/2, angle = (pos + r) / theta^(2i/dim), cosine,
 * sine and the multiply-adds in f64.  On the tensor-core path the rotation happens while q and k are
 * converted into the kernels' operand planes, so the rotated tensors never exist in memory.
 *   forward:  out = attention(rope(q), rope(k), v), lse as zt_attn_forward_batched.
 *   backward: dq, dk are the gradients of the UNROTATED q and k (ropeBackward,
 *             src/autograd.zig:851-874, applied to the attention gradients), dv as usual; out and
 *             lse are the rope forward's.
 * Both take a caller workspace of zt_attn_rope_workspace_bytes(...) bytes (256-byte aligned; never
 * 0) and allocate nothing.  The forward keeps its operand planes (rotated q and k among them) in that
 * workspace and reports a token through *host_token (may be NULL) exactly as
 * zt_attn_forward_batched_keep does; the backward takes it back (`token`; 0 converts everything
 * again) under the same rules, pos and theta included.  Refusals: those of the batched calls, plus
 * pos < 0, theta <= 0, a missing, short or misaligned workspace, and a stale token. */
size_t zt_attn_rope_workspace_bytes(int batch, int T, int n_heads, int n_kv_heads, int dim);
int zt_attn_forward_rope_batched(const float *q, const float *k, const float *v, float *out, float *lse,
                                 void *workspace, size_t workspace_bytes, int batch, int T, int n_heads,
                                 int n_kv_heads, int dim, int pos, double theta, zt_stream_t stream,
                                 unsigned long long *host_token);
int zt_attn_backward_rope_batched(const float *q, const float *k, const float *v, const float *out,
                                  const float *lse, const float *dout, float *dq, float *dk, float *dv,
                                  float *delta, void *workspace, size_t workspace_bytes, int batch, int T,
                                  int n_heads, int n_kv_heads, int dim, int pos, double theta,
                                  zt_stream_t stream, unsigned long long token);

/* The projection on the output side of attention, y = ctx . wo (tensor.matmul(ctx, l.wo), src/model.zig:396;
 * src/tensor.zig:78-106), for `batch` sequences of T rows: ctx [batch, T, k], wo [k, n] row-major, y [batch, T, n].
 * On the tensor cores with the attention kernels' three-term f16 split (f32-class accuracy, f32 accumulation).
 * The reference reduces in f32 in ascending k, so two correct implementations differ by f32 rounding of a
 * k-term sum; tests gate max |got - ref| <= 1e-4 max |ref| (src/train.zig:706) rather than element-wise.
 *   zt_proj_forward   y is assigned.
 *   zt_proj_backward  the two gradients of that product (src/autograd.zig:553-557): dctx = dy . wo^T is assigned
 *                     (inputGrad, :999-1022); dwo += ctx^T . dy is ACCUMULATED into the caller's dwo, as
 *                     weightGrad accumulates into the layer's gradient (:958-972) -- zero it for a fresh one.
 * Both take a caller workspace of zt_proj_workspace_bytes(batch, T, k, n) bytes (256-byte aligned) and allocate
 * nothing.  Refusals: batch or T < 1; k or n not a multiple of 64 (there is no CUDA-core form of these calls);
 * a missing, short or misaligned workspace; a device that is not sm_100. */
size_t zt_proj_workspace_bytes(int batch, int T, int k, int n);
int zt_proj_forward(const float *ctx, const float *wo, float *y, void *workspace, size_t workspace_bytes, int batch,
                    int T, int k, int n, zt_stream_t stream);
int zt_proj_backward(const float *ctx, const float *wo, const float *dy, float *dctx, float *dwo, void *workspace,
                     size_t workspace_bytes, int batch, int T, int k, int n, zt_stream_t stream);

/* The forward of the attention part of a block in one call: zt_attn_forward_rope_batched followed by
 * zt_proj_forward on its output (src/model.zig:372-396), with the two fused where it pays: on the tensor-core path
 * the attention kernel's epilogue writes ctx a second time as the f16 operand planes of the projection, straight
 * into the projection's workspace, so the projection's own passes over ctx (one read for the maximum, one read and
 * one write for the planes) do not run -- an output row is a convex combination of rows of v, so its scale is
 * known from v's maxima before the row exists.  (Fusing the product itself into the attention kernel would have
 * every (query tile, head) CTA add a [128, d_model] partial product into y: n_heads / 2 times y's bytes in
 * atomic traffic, which costs more than the round trip it saves.)  ctx [batch, T, n_heads*dim] and lse are
 * written as by the rope forward (the backward needs them), y is [batch, T, d_model]; wo is [n_heads*dim, d_model].
 * Both workspaces are the caller's (zt_attn_rope_workspace_bytes, zt_proj_workspace_bytes with k = n_heads*dim,
 * n = d_model); *host_token as in zt_attn_forward_rope_batched.  Refusals: those of the two calls.
 * The backward of the block is zt_proj_backward followed by zt_attn_backward_rope_batched. */
int zt_attn_block_forward(const float *q, const float *k, const float *v, const float *wo, float *ctx, float *lse,
                          float *y, void *rope_workspace, size_t rope_workspace_bytes, void *proj_workspace,
                          size_t proj_workspace_bytes, int batch, int T, int n_heads, int n_kv_heads, int dim,
                          int d_model, int pos, double theta, zt_stream_t stream, unsigned long long *host_token);

/* KV-cache decode attention for a batch of sequences: decode.attnStep
 * (src/decode.zig:326-392) for every sequence at once, over device-resident
 * caches laid out as kv_cache.Layer lays them out (src/kv_cache.zig:60-95):
 * k_cache, v_cache are [batch, n_ctx, n_kv_heads*dim]; n_keys[b] in [1, n_ctx]
 * is how many rows of sequence b are filled, INCLUDING the new token's own row
 * (append before attend, src/decode.zig:259); q and out are
 * [batch, n_heads*dim]; lse (may be NULL) is [batch, n_heads].
 * The context is split over many blocks; partial results live in `workspace`
 * (zt_attn_decode_workspace_bytes) and are merged by log-sum-exp.
 * A sequence whose n_keys is outside [1, n_ctx] is not computed: its out row is
 * filled with NaN and (after the stream has been synchronised)
 * zt_attn_decode_status reports it. */
int zt_attn_decode(const float *q, const float *k_cache, const float *v_cache, const int *n_keys,
                   float *out, float *lse, void *workspace, size_t workspace_bytes, int batch,
                   int n_ctx, int n_heads, int n_kv_heads, int dim, zt_stream_t stream);
size_t zt_attn_decode_workspace_bytes(int batch, int n_ctx, int n_heads, int n_kv_heads, int dim);

/* zt_attn_decode for callers that have no workspace to give and must not allocate one.
 * (No counterpart in the reference: its decode arm has no split over the context and so needs
 * no scratch.)
 *
 * Who this is for: a caller that follows the reference's contract to the letter -- every buffer
 * is sized once, up front, and an entry point never allocates (src/cuda/attn_kernels.cu:39,50-54)
 * -- has nowhere to get zt_attn_decode's workspace from in the middle of a generation loop.
 * The same holds for a server that hands all of the device's memory to its own pool at start-up
 * (a later cudaMalloc fails or fragments the pool), and for a latency-bound decode loop, where
 * cudaMalloc/cudaFree stall because they synchronise the whole device.
 *
 * The scratch is a fixed 16 MiB array (zt_attn_decode_static_capacity()) compiled into the
 * library; every GPU that loads the library carries it until the process exits.  This entry
 * point calls no cudaMalloc, cudaFree or other allocating routine.  A shape whose split needs
 * more than the capacity (zt_attn_decode_workspace_bytes tells) is refused with return 1, as
 * are head widths that are not a multiple of 4 floats and q/cache pointers that are not
 * 16-byte aligned (zt_attn_decode accepts those).  Arguments, results, NaN rows for a bad
 * n_keys[b]: exactly zt_attn_decode's.
 *
 * Rules that come with a shared, permanent scratch:
 *  - the first call made with a given device current looks up the array's address on that
 *    device (and, where the CUDA runtime loads modules lazily, is what makes the array exist there):
 *    make that first call at start-up -- before any stream capture, and before a memory pool of the
 *    caller's takes the rest of the device;
 *  - all calls on a device use the same array, which still holds the previous call's partial
 *    results: two calls may not overlap on the GPU (different streams, or threads, without an
 *    ordering between them race on it).  Calls queued on one stream are safe. */
int zt_attn_decode_static(const float *q, const float *k_cache, const float *v_cache,
                          const int *n_keys, float *out, float *lse, int batch, int n_ctx,
                          int n_heads, int n_kv_heads, int dim, zt_stream_t stream);
size_t zt_attn_decode_static_capacity(void);

/* After synchronising: number of sequences the last zt_attn_decode that used
 * `workspace` skipped for a bad n_keys (the count is kept inside the workspace).
 * A NULL workspace reads the count of the last zt_attn_decode_static on the current device. */
int zt_attn_decode_status(const void *workspace, int *host_bad_sequences);

/* kv_cache.Layer.append for a batch of device-resident caches
 * (src/kv_cache.zig:88-95): copies one new row per sequence into row n_keys[b]
 * of its cache and increments n_keys[b].  A sequence that is full
 * (n_keys[b] >= n_ctx) is left untouched and counted in *full_count (device int,
 * may be NULL), the reference's Error.Full. */
int zt_kv_append(float *k_cache, float *v_cache, int *n_keys, const float *k_new,
                 const float *v_new, int *full_count, int batch, int n_ctx, int n_kv_heads, int dim,
                 zt_stream_t stream);

/* Number of kernels this library has launched in this process (all threads);
 * benchmarks report the difference over their timed region. */
unsigned long long zt_attn_launch_count(void);

/* After synchronising: 0 when no tensor-core kernel on the current device ever gave up on one
 * of its bounded internal waits, else the code of the wait that did (its outputs are then
 * invalid).  A correct run never sets it; tests assert 0. */
int zt_attn_tc_status(int *host_status);

/* After synchronising: how many thread blocks of the tensor-core backward met the bound on dS since
 * the last call of this function (which clears the count).  The backward hands dS to the tensor core
 * as 16-bit pieces, scaled so that its worst case stays inside their range; a value that reaches the
 * bound all the same (only an Inf or NaN arriving in dout or delta can) is clamped and counted here
 * instead of passing unnoticed.  A correct run reads 0; tests assert it. */
int zt_attn_tc_saturated(unsigned int *host_count);

/* Per-kernel device timing for benchmarks.  zt_attn_profile(1) makes every later launch
 * record a pair of CUDA events on its stream; zt_attn_profile_read waits for them, writes one
 * line per kernel name ("name launches total_ms\n") into host_buf, forgets them, and returns
 * the number of lines.  Off by default; when off, no event is ever created. */
void zt_attn_profile(int on);
int zt_attn_profile_read(char *host_buf, size_t cap);

/* Name of the kernel family the most recent launching call on this thread used
 * ("tcgen05", "simt", "decode-splitk", ...). */
const char *zt_attn_last_path(void);

#ifdef __cplusplus
}
#endif
#endif /* ZT_ATTN_H */
