/*
 * CPU oracle for Z-TRANSFORMER's attention hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the reference's CPU arithmetic for the three
 * functions the CUDA kernels of this repository replace.  It is the checker the
 * parity tests, the smoke test and the benchmark's CPU baseline use; nothing in
 * the shipped library links, loads or calls it.
 *
 * Followed, loop for loop (paths are within the reference project):
 *   src/attention.zig:60-153   forwardWith      -> zto_attention_forward
 *   src/autograd.zig:636-842   attentionBackward-> zto_attention_backward
 *   src/decode.zig:326-392     attnStep         -> zto_attn_step
 *   src/kv_cache.zig:60-135    Layer            -> zto_layer_*
 *   src/tensor.zig:78-106      matmul           -> zto_matmul
 *   src/autograd.zig:958-1022  weightGrad, inputGrad -> zto_weight_grad, zto_input_grad
 *   src/cuda/device.zig:162-182,489-501  bytesFor/toCInt/forwardBounds
 *                                               -> zto_bytes_for / zto_forward_bounds
 *
 * Arithmetic contract kept from the reference: f32 storage; every dot product,
 * score, exponential, denominator and probability-weighted sum is carried in
 * f64 and narrowed to f32 once, at the store.  The one exception is the
 * backward's dk/dv, which the reference accumulates IN f32 with one f64->f32
 * narrowing per term (autograd.zig:829-836); that order (head outer, query row,
 * then key ascending) is kept so the roundings land where the reference's do.
 *
 * Parity status: pinned.  The forward is pinned by the reference's own
 * known-answer tests (src/attention_test.zig), restated in
 * tests/test_oracle_kat.py.  The backward has no literal vectors anywhere in the
 * reference; it is pinned by outputs of the reference's own CUDA kernels
 * (src/cuda/attn_kernels.cu:402-634), which the reference graded against its Zig
 * CPU code at <= 8.4e-7 (outputs/bench/run-attn.log:36-46) and which, unlike the
 * Zig code (Zig 0.16 is needed), compile here: oracle/zt_ref.py builds them in
 * place into oracle/_ref/, tests/golden/make_ref_fixtures.py ran them on a B200
 * and tests/test_ref_cuda_fixtures.py holds this file to their dq, dk, dv (and
 * forward and decode outputs) under the reference's own gates.  Central
 * differences and an independent float64 autograd check it as well
 * (tests/test_oracle_backward.py).  The log-sum-exp the reference never emits
 * is defined here as row max + ln(denominator) in f64; it is pinned through the
 * backward, whose P = exp(S - lse) consumes it.
 *
 * The reference's Zig uses @exp/@sqrt on f64; glibc exp/sqrt in double are used
 * here.  A last-ulp difference in exp() disappears under the f32 store.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ZTO_OK 0
#define ZTO_INVALID_HEAD_CONFIG 1 /* attention.zig:71-73  error.InvalidHeadConfig */
#define ZTO_DIMENSION_MISMATCH 2  /* attention.zig:74-79  error.DimensionMismatch */
#define ZTO_OUT_OF_MEMORY 3
#define ZTO_FULL 4                /* kv_cache.zig Error.Full */
#define ZTO_SHAPE_TOO_LARGE 5     /* device.zig Error.ShapeTooLarge */
#define ZTO_DEGENERATE_SHAPE 6    /* device.zig Error.DegenerateShape */

/* One (head, query row) of the forward: attention.zig:113-149 with the key
 * bound generalised from `t + 1` to `n_vis`, which is also decode.zig:363-390.
 * `scores` is caller scratch of at least n_vis doubles. */
static void zto_row(const float *q_head, const float *k, const float *v, size_t kv_cols,
                    size_t kv_off, size_t dim, size_t n_vis, double scale, double *scores,
                    float *out_head, float *lse) {
    double row_max = -INFINITY;
    for (size_t s = 0; s < n_vis; ++s) {
        const float *k_head = k + s * kv_cols + kv_off;
        double dot = 0.0;
        for (size_t j = 0; j < dim; ++j) dot += (double)q_head[j] * (double)k_head[j];
        const double score = dot * scale;
        scores[s] = score;
        if (score > row_max) row_max = score;
    }
    double denom = 0.0;
    for (size_t s = 0; s < n_vis; ++s) {
        scores[s] = exp(scores[s] - row_max);
        denom += scores[s];
    }
    for (size_t s = 0; s < n_vis; ++s) scores[s] /= denom;
    for (size_t j = 0; j < dim; ++j) {
        double acc = 0.0;
        for (size_t s = 0; s < n_vis; ++s) acc += scores[s] * (double)v[s * kv_cols + kv_off + j];
        out_head[j] = (float)acc;
    }
    /* The reference's CPU path never emits a log-sum-exp; it is defined here by
     * restatement as row_max + ln(denom), both still in f64. */
    if (lse) *lse = (float)(row_max + log(denom));
}

/*
 * attention.forwardWith (src/attention.zig:60-153), null sink.
 * q is [q_rows, q_cols], k is [k_rows, k_cols], v is [v_rows, v_cols], out is
 * [q_rows, n_heads*dim]; lse (optional, may be NULL) is [q_rows, n_heads].
 * The shapes are passed separately so the reference's refusals can be restated.
 * threads > 1 spreads the (head) loop over OpenMP threads; every (head, row) is
 * computed by exactly one thread in the same order, so results do not depend on it.
 */
int zto_attention_forward(const float *q, size_t q_rows, size_t q_cols, const float *k,
                          size_t k_rows, size_t k_cols, const float *v, size_t v_rows,
                          size_t v_cols, size_t n_heads, size_t n_kv_heads, size_t dim,
                          float *out, float *lse, int threads) {
    if (n_kv_heads == 0 || dim == 0 || n_heads % n_kv_heads != 0) return ZTO_INVALID_HEAD_CONFIG;
    if (k_rows != v_rows || k_rows != q_rows || k_cols != n_kv_heads * dim || v_cols != k_cols ||
        q_cols != n_heads * dim)
        return ZTO_DIMENSION_MISMATCH;
    const size_t group = n_heads / n_kv_heads;
    const double scale = 1.0 / sqrt((double)dim);
    const size_t T = q_rows;
    if (T == 0) return ZTO_OK;
    int failed = 0;
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
    {
        double *scores = (double *)malloc(sizeof(double) * T);
        if (!scores) {
#pragma omp atomic write
            failed = 1;
        }
        /* (head, row-block) units so that more threads than heads still help;
         * rows are independent, so the split changes no value. */
        const size_t blk = 64;
        const size_t n_blk = (T + blk - 1) / blk;
        const long units = (long)(n_heads * n_blk);
#pragma omp for schedule(dynamic, 1)
        for (long u = 0; u < units; ++u) {
            if (!scores) continue;
            const size_t h = (size_t)u / n_blk;
            /* later row blocks are heavier; walk them first for balance */
            const size_t b = n_blk - 1 - (size_t)u % n_blk;
            const size_t kv = h / group;
            const size_t t_end = (b + 1) * blk < T ? (b + 1) * blk : T;
            for (size_t t = b * blk; t < t_end; ++t) {
                zto_row(q + t * q_cols + h * dim, k, v, k_cols, kv * dim, dim, t + 1, scale, scores,
                        out + t * q_cols + h * dim, lse ? lse + t * n_heads + h : NULL);
            }
        }
        free(scores);
    }
    return failed ? ZTO_OUT_OF_MEMORY : ZTO_OK;
}

/*
 * The C ABI's general forward (q_offset / n_keys form), stated on the CPU so the
 * decode use of zt_attn_forward has a checker: query row t sits at absolute
 * position q_offset + t and sees keys 0 .. min(n_keys, q_offset + t + 1) - 1
 * (src/cuda/attn_kernels.cu:276-283,310-321).  With q_offset = 0, n_keys = T it
 * is zto_attention_forward; with T = 1, q_offset = n_keys - 1 it is zto_attn_step.
 */
int zto_attention_forward_at(const float *q, const float *k, const float *v, float *out, float *lse,
                             size_t T, size_t n_heads, size_t n_kv_heads, size_t dim,
                             size_t q_offset, size_t n_keys, int threads) {
    if (n_kv_heads == 0 || dim == 0 || n_heads % n_kv_heads != 0) return ZTO_INVALID_HEAD_CONFIG;
    if (T < 1 || n_keys < 1 || q_offset + T > n_keys) return ZTO_DIMENSION_MISMATCH;
    const size_t group = n_heads / n_kv_heads;
    const size_t q_cols = n_heads * dim, kv_cols = n_kv_heads * dim;
    const double scale = 1.0 / sqrt((double)dim);
    int failed = 0;
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
    {
        double *scores = (double *)malloc(sizeof(double) * n_keys);
        if (!scores) {
#pragma omp atomic write
            failed = 1;
        }
        const long units = (long)(n_heads * T);
#pragma omp for schedule(dynamic, 1)
        for (long u = 0; u < units; ++u) {
            if (!scores) continue;
            const size_t h = (size_t)u / T, t = (size_t)u % T;
            size_t n_vis = q_offset + t + 1;
            if (n_vis > n_keys) n_vis = n_keys;
            zto_row(q + t * q_cols + h * dim, k, v, kv_cols, (h / group) * dim, dim, n_vis, scale,
                    scores, out + t * q_cols + h * dim, lse ? lse + t * n_heads + h : NULL);
        }
        free(scores);
    }
    return failed ? ZTO_OUT_OF_MEMORY : ZTO_OK;
}

/*
 * decode.attnStep (src/decode.zig:326-392): one query row over the filled prefix
 * of one layer's cache.  k_cache/v_cache are [n_ctx, cache_cols] row-major and
 * n_keys = layer.visible() rows of them are filled, the newest being this
 * token's own (append-before-attend, decode.zig:259).
 */
int zto_attn_step(const float *q, size_t q_cols, const float *k_cache, const float *v_cache,
                  size_t k_cols, size_t v_cols, size_t n_keys, size_t n_heads, size_t n_kv_heads,
                  size_t dim, float *out, float *lse, int threads) {
    if (n_kv_heads == 0 || dim == 0 || n_heads % n_kv_heads != 0) return ZTO_INVALID_HEAD_CONFIG;
    if (q_cols != n_heads * dim || k_cols != n_kv_heads * dim || v_cols != n_kv_heads * dim)
        return ZTO_DIMENSION_MISMATCH;
    if (n_keys < 1) return ZTO_DIMENSION_MISMATCH; /* decode.zig:350 */
    const size_t group = n_heads / n_kv_heads;
    const double scale = 1.0 / sqrt((double)dim);
    int failed = 0;
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
    {
        double *scores = (double *)malloc(sizeof(double) * n_keys);
        if (!scores) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(dynamic, 1)
        for (long h = 0; h < (long)n_heads; ++h) {
            if (!scores) continue;
            zto_row(q + (size_t)h * dim, k_cache, v_cache, k_cols, ((size_t)h / group) * dim, dim,
                    n_keys, scale, scores, out + (size_t)h * dim, lse ? lse + h : NULL);
        }
        free(scores);
    }
    return failed ? ZTO_OUT_OF_MEMORY : ZTO_OK;
}

/*
 * autograd.attentionBackward (src/autograd.zig:636-842): the body of its (head, row)
 * loop, for one query row t of head h.
 *
 * The reference unrolls four loops eight ways without ever adding one lane to
 * another (autograd.zig:622-635), so the scalar loops below run the same terms
 * into the same accumulator chains in the same order.
 *
 * dq is assigned (one f64 chain per element, `* scale` applied per term, one
 * narrowing).  dk and dv are f32 accumulators that receive one f32-narrowed term
 * per (head of the group, query row >= key).
 * probs, d_probs and p_ds are caller scratch of at least t + 1 doubles each.
 */
static void zto_backward_row(const float *q, const float *k, const float *v, const float *dout,
                             size_t q_cols, size_t k_cols, size_t dim, size_t h, size_t kv,
                             size_t t, double scale, double *probs, double *d_probs, double *p_ds,
                             float *dq, float *dk, float *dv) {
    const float *q_head = q + t * q_cols + h * dim;
    const float *dh = dout + t * q_cols + h * dim;
    /* softmax rebuild, autograd.zig:735-770 */
    double row_max = -INFINITY;
    for (size_t s = 0; s <= t; ++s) {
        const float *k_head = k + s * k_cols + kv * dim;
        double dot = 0.0;
        for (size_t j = 0; j < dim; ++j) dot += (double)q_head[j] * (double)k_head[j];
        probs[s] = dot * scale;
        if (probs[s] > row_max) row_max = probs[s];
    }
    double denom = 0.0;
    for (size_t s = 0; s <= t; ++s) {
        probs[s] = exp(probs[s] - row_max);
        denom += probs[s];
    }
    for (size_t s = 0; s <= t; ++s) probs[s] /= denom;
    /* d p and the Jacobian's dot, autograd.zig:774-797 */
    double dot_pp = 0.0;
    for (size_t s = 0; s <= t; ++s) {
        const float *v_head = v + s * k_cols + kv * dim;
        double acc = 0.0;
        for (size_t j = 0; j < dim; ++j) acc += (double)dh[j] * (double)v_head[j];
        d_probs[s] = acc;
        dot_pp += probs[s] * acc;
    }
    for (size_t s = 0; s <= t; ++s) p_ds[s] = probs[s] * (d_probs[s] - dot_pp);
    /* dq, autograd.zig:803-820 */
    for (size_t j = 0; j < dim; ++j) {
        double acc = 0.0;
        for (size_t s = 0; s <= t; ++s) acc += p_ds[s] * (double)k[s * k_cols + kv * dim + j] * scale;
        dq[t * q_cols + h * dim + j] = (float)acc;
    }
    /* dk, dv: f32 read-modify-write of an f32-narrowed term, autograd.zig:821-838 */
    for (size_t s = 0; s <= t; ++s) {
        float *dk_row = dk + s * k_cols + kv * dim;
        float *dv_row = dv + s * k_cols + kv * dim;
        const double p_ds_s = p_ds[s];
        const double probs_s = probs[s];
        for (size_t j = 0; j < dim; ++j) {
            dk_row[j] += (float)(p_ds_s * (double)q_head[j] * scale);
            dv_row[j] += (float)(probs_s * (double)dh[j]);
        }
    }
}

/* One KV head's group: heads outer, rows ascending (autograd.zig:723-725). */
static void zto_backward_group(const float *q, const float *k, const float *v, const float *dout,
                               size_t T, size_t q_cols, size_t k_cols, size_t dim, size_t group,
                               size_t kv, double scale, double *probs, double *d_probs,
                               double *p_ds, float *dq, float *dk, float *dv) {
    for (size_t h = kv * group; h < (kv + 1) * group; ++h)
        for (size_t t = 0; t < T; ++t)
            zto_backward_row(q, k, v, dout, q_cols, k_cols, dim, h, kv, t, scale, probs, d_probs,
                             p_ds, dq, dk, dv);
}

/*
 * autograd.attentionBackward, whole tensors, with the reference's refusals
 * (autograd.zig:659-685).  Heads of different KV groups touch disjoint dk/dv
 * columns, so the OpenMP split is over KV heads and keeps the reference's order
 * inside each; the result does not depend on the thread count.
 */
int zto_attention_backward(const float *q, size_t q_rows, size_t q_cols, const float *k,
                           size_t k_rows, size_t k_cols, const float *v, size_t v_rows,
                           size_t v_cols, const float *dout, size_t dout_rows, size_t dout_cols,
                           size_t n_heads, size_t n_kv_heads, size_t dim, float *dq, float *dk,
                           float *dv, int threads) {
    if (n_kv_heads == 0 || dim == 0 || n_heads % n_kv_heads != 0) return ZTO_INVALID_HEAD_CONFIG;
    if (k_rows != v_rows || k_rows != q_rows || k_cols != n_kv_heads * dim || v_cols != k_cols ||
        q_cols != n_heads * dim)
        return ZTO_DIMENSION_MISMATCH;
    if (dout_rows != q_rows || dout_cols != n_heads * dim) return ZTO_DIMENSION_MISMATCH;
    const size_t T = q_rows;
    const size_t group = n_heads / n_kv_heads;
    const double scale = 1.0 / sqrt((double)dim);
    /* Tensor.init zeroes (autograd.zig:700-704). */
    memset(dq, 0, sizeof(float) * T * q_cols);
    memset(dk, 0, sizeof(float) * T * k_cols);
    memset(dv, 0, sizeof(float) * T * k_cols);
    if (T == 0) return ZTO_OK;
    int failed = 0;
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
    {
        double *probs = (double *)malloc(sizeof(double) * T);
        double *d_probs = (double *)malloc(sizeof(double) * T);
        double *p_ds = (double *)malloc(sizeof(double) * T);
        const int ok = probs && d_probs && p_ds;
        if (!ok) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(dynamic, 1)
        for (long kv = 0; kv < (long)n_kv_heads; ++kv) {
            if (!ok) continue;
            zto_backward_group(q, k, v, dout, T, q_cols, k_cols, dim, group, (size_t)kv, scale,
                               probs, d_probs, p_ds, dq, dk, dv);
        }
        free(probs);
        free(d_probs);
        free(p_ds);
    }
    return failed ? ZTO_OUT_OF_MEMORY : ZTO_OK;
}

/*
 * One KV group of the backward only (all rows): the unit a CPU baseline times
 * when the whole tensor would take hours.  Writes dq columns of the group's
 * query heads and dk/dv columns of KV head `kv`; everything else is untouched.
 */
int zto_attention_backward_kv_group(const float *q, const float *k, const float *v,
                                    const float *dout, size_t T, size_t n_heads, size_t n_kv_heads,
                                    size_t dim, size_t kv, float *dq, float *dk, float *dv) {
    if (n_kv_heads == 0 || dim == 0 || n_heads % n_kv_heads != 0) return ZTO_INVALID_HEAD_CONFIG;
    if (kv >= n_kv_heads) return ZTO_DIMENSION_MISMATCH;
    const size_t group = n_heads / n_kv_heads;
    const size_t q_cols = n_heads * dim, k_cols = n_kv_heads * dim;
    const double scale = 1.0 / sqrt((double)dim);
    double *probs = (double *)malloc(sizeof(double) * (T ? T : 1));
    double *d_probs = (double *)malloc(sizeof(double) * (T ? T : 1));
    double *p_ds = (double *)malloc(sizeof(double) * (T ? T : 1));
    if (!probs || !d_probs || !p_ds) {
        free(probs);
        free(d_probs);
        free(p_ds);
        return ZTO_OUT_OF_MEMORY;
    }
    for (size_t s = 0; s < T; ++s)
        for (size_t j = 0; j < dim; ++j) {
            dk[s * k_cols + kv * dim + j] = 0.0f;
            dv[s * k_cols + kv * dim + j] = 0.0f;
        }
    zto_backward_group(q, k, v, dout, T, q_cols, k_cols, dim, group, kv, scale, probs, d_probs,
                       p_ds, dq, dk, dv);
    free(probs);
    free(d_probs);
    free(p_ds);
    return ZTO_OK;
}

/*
 * One (head, row range) of the forward: the unit a CPU baseline times when the
 * whole tensor would take hours.  Rows [t0, t1) of head h, training shape.
 */
int zto_attention_forward_rows(const float *q, const float *k, const float *v, float *out,
                               float *lse, size_t T, size_t n_heads, size_t n_kv_heads, size_t dim,
                               size_t h, size_t t0, size_t t1) {
    if (n_kv_heads == 0 || dim == 0 || n_heads % n_kv_heads != 0) return ZTO_INVALID_HEAD_CONFIG;
    if (h >= n_heads || t0 > t1 || t1 > T) return ZTO_DIMENSION_MISMATCH;
    const size_t group = n_heads / n_kv_heads;
    const size_t q_cols = n_heads * dim, k_cols = n_kv_heads * dim;
    const double scale = 1.0 / sqrt((double)dim);
    double *scores = (double *)malloc(sizeof(double) * (T ? T : 1));
    if (!scores) return ZTO_OUT_OF_MEMORY;
    for (size_t t = t0; t < t1; ++t)
        zto_row(q + t * q_cols + h * dim, k, v, k_cols, (h / group) * dim, dim, t + 1, scale, scores,
                out + t * q_cols + h * dim, lse ? lse + t * n_heads + h : NULL);
    free(scores);
    return ZTO_OK;
}

/*
 * A bounded sample of one forward+backward pass over a batch, for timing the CPU
 * path at sizes where the whole pass takes hours: of every head of every batch item,
 * only query rows t with t % row_stride == row_phase are computed (forward row,
 * then backward row).  The arithmetic of a computed row is exactly the reference's;
 * dk/dv therefore hold only the sampled rows' contributions.  (batch item, KV head)
 * units run on separate OpenMP threads; they touch disjoint outputs.
 * Returns through *flops the reference's own operation count for the rows computed:
 * 4 * dim * (t + 1) per forward row (2*H*D*T*(T+1) over a whole pass,
 * src/scale.zig:157-163) and 2.5 times that for the backward row.
 */
int zto_sampled_step(const float *q, const float *k, const float *v, const float *dout, float *out,
                     float *dq, float *dk, float *dv, size_t batch, size_t T, size_t n_heads,
                     size_t n_kv_heads, size_t dim, size_t row_stride, size_t row_phase,
                     int do_backward, int threads, double *flops) {
    if (n_kv_heads == 0 || dim == 0 || n_heads % n_kv_heads != 0) return ZTO_INVALID_HEAD_CONFIG;
    if (row_stride == 0 || row_phase >= row_stride) return ZTO_DIMENSION_MISMATCH;
    const size_t group = n_heads / n_kv_heads;
    const size_t q_cols = n_heads * dim, k_cols = n_kv_heads * dim;
    const double scale = 1.0 / sqrt((double)dim);
    int failed = 0;
    double total = 0.0;
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads) reduction(+ : total)
    {
        double *probs = (double *)malloc(sizeof(double) * (T ? T : 1));
        double *d_probs = (double *)malloc(sizeof(double) * (T ? T : 1));
        double *p_ds = (double *)malloc(sizeof(double) * (T ? T : 1));
        const int ok = probs && d_probs && p_ds;
        if (!ok) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(dynamic, 1)
        for (long u = 0; u < (long)(batch * n_kv_heads); ++u) {
            if (!ok) continue;
            const size_t b = (size_t)u / n_kv_heads, kv = (size_t)u % n_kv_heads;
            const float *qb = q + b * T * q_cols, *kb = k + b * T * k_cols, *vb = v + b * T * k_cols;
            const float *gb = dout + b * T * q_cols;
            float *ob = out + b * T * q_cols, *dqb = dq + b * T * q_cols;
            float *dkb = dk + b * T * k_cols, *dvb = dv + b * T * k_cols;
            for (size_t h = kv * group; h < (kv + 1) * group; ++h)
                for (size_t t = row_phase; t < T; t += row_stride) {
                    zto_row(qb + t * q_cols + h * dim, kb, vb, k_cols, kv * dim, dim, t + 1, scale,
                            probs, ob + t * q_cols + h * dim, NULL);
                    total += 4.0 * (double)dim * (double)(t + 1);
                    if (do_backward) {
                        zto_backward_row(qb, kb, vb, gb, q_cols, k_cols, dim, h, kv, t, scale, probs,
                                         d_probs, p_ds, dqb, dkb, dvb);
                        total += 10.0 * (double)dim * (double)(t + 1);
                    }
                }
        }
        free(probs);
        free(d_probs);
        free(p_ds);
    }
    *flops = total;
    return failed ? ZTO_OUT_OF_MEMORY : ZTO_OK;
}

/*
 * The backward of one KV group restricted to what a long-context check can afford:
 *   - dq of the query rows listed in `rows` (n_rows of them), every head of the group:
 *     dq_rows[(i * group + hh) * dim + j];
 *   - dk, dv of the LAST `window` keys (keys s >= T - window): dk_win[(s - s_lo) * dim + j].
 * A key's dk/dv receive terms only from query rows t >= s, so the window needs the rows
 * t >= s_lo of the group's heads and nothing else; each of those rows still needs its whole
 * softmax (keys 0..t), which is where the time goes.
 *
 * Arithmetic and order are exactly zto_backward_row's (autograd.zig:735-838): per row the
 * f64 score, max, exp, denominator, probability, d_probs and their dot; per key f32
 * accumulators that receive one f32-narrowed term per (head of the group -- outer --, query
 * row ascending).  Rows are independent, so the per-row statistics are computed in parallel
 * first; then every key of the window (independent of the other keys) replays its own
 * accumulation in the reference's order from those statistics.
 */
int zto_backward_window(const float *q, const float *k, const float *v, const float *dout, size_t T,
                        size_t n_heads, size_t n_kv_heads, size_t dim, size_t kv, const size_t *rows,
                        size_t n_rows, size_t window, float *dq_rows, float *dk_win, float *dv_win,
                        int threads) {
    if (n_kv_heads == 0 || dim == 0 || n_heads % n_kv_heads != 0) return ZTO_INVALID_HEAD_CONFIG;
    if (kv >= n_kv_heads || window > T) return ZTO_DIMENSION_MISMATCH;
    for (size_t i = 0; i < n_rows; ++i)
        if (rows[i] >= T) return ZTO_DIMENSION_MISMATCH;
    const size_t group = n_heads / n_kv_heads;
    const size_t q_cols = n_heads * dim, k_cols = n_kv_heads * dim;
    const double scale = 1.0 / sqrt((double)dim);
    const size_t s_lo = T - window;
    if (threads < 1) threads = 1;
    int failed = 0;
    /* per (head of the group, row t >= s_lo): row max, denominator, dot_pp */
    double *stats = (double *)malloc(sizeof(double) * 3 * (group * window > 0 ? group * window : 1));
    if (!stats) return ZTO_OUT_OF_MEMORY;
#pragma omp parallel num_threads(threads)
    {
        double *probs = (double *)malloc(sizeof(double) * (T ? T : 1));
        double *d_probs = (double *)malloc(sizeof(double) * (T ? T : 1));
        double *p_ds = (double *)malloc(sizeof(double) * (T ? T : 1));
        float *dk_dummy = (float *)malloc(sizeof(float) * (T ? T : 1) * k_cols);
        float *dq_dummy = (float *)malloc(sizeof(float) * q_cols);
        const int ok = probs && d_probs && p_ds && dk_dummy && dq_dummy;
        if (!ok) {
#pragma omp atomic write
            failed = 1;
        }
        /* dq of the listed rows: the reference's row body, its dk/dv side effects discarded */
#pragma omp for schedule(dynamic, 1)
        for (long u = 0; u < (long)(n_rows * group); ++u) {
            if (!ok) continue;
            const size_t i = (size_t)u / group, hh = (size_t)u % group, h = kv * group + hh, t = rows[i];
            /* zto_backward_row writes dq[t * q_cols + h * dim + j]: aim that at dq_dummy */
            zto_backward_row(q, k, v, dout, q_cols, k_cols, dim, h, kv, t, scale, probs, d_probs, p_ds,
                             dq_dummy - t * q_cols, dk_dummy, dk_dummy);
            memcpy(dq_rows + (i * group + hh) * dim, dq_dummy + h * dim, sizeof(float) * dim);
        }
        /* statistics of the rows that reach the window */
#pragma omp for schedule(dynamic, 4)
        for (long u = 0; u < (long)(group * window); ++u) {
            if (!ok) continue;
            const size_t hh = (size_t)u / window, t = s_lo + (size_t)u % window, h = kv * group + hh;
            const float *q_head = q + t * q_cols + h * dim;
            const float *dh = dout + t * q_cols + h * dim;
            double row_max = -INFINITY;
            for (size_t s = 0; s <= t; ++s) {
                const float *k_head = k + s * k_cols + kv * dim;
                double dot = 0.0;
                for (size_t j = 0; j < dim; ++j) dot += (double)q_head[j] * (double)k_head[j];
                probs[s] = dot * scale;
                if (probs[s] > row_max) row_max = probs[s];
            }
            double denom = 0.0;
            for (size_t s = 0; s <= t; ++s) {
                probs[s] = exp(probs[s] - row_max);
                denom += probs[s];
            }
            for (size_t s = 0; s <= t; ++s) probs[s] /= denom;
            double dot_pp = 0.0;
            for (size_t s = 0; s <= t; ++s) {
                const float *v_head = v + s * k_cols + kv * dim;
                double acc = 0.0;
                for (size_t j = 0; j < dim; ++j) acc += (double)dh[j] * (double)v_head[j];
                dot_pp += probs[s] * acc;
            }
            stats[3 * u] = row_max, stats[3 * u + 1] = denom, stats[3 * u + 2] = dot_pp;
        }
        /* every key of the window replays its accumulation: heads outer, rows ascending */
#pragma omp for schedule(dynamic, 4)
        for (long w = 0; w < (long)window; ++w) {
            if (!ok) continue;
            const size_t s = s_lo + (size_t)w;
            const float *k_head = k + s * k_cols + kv * dim;
            const float *v_head = v + s * k_cols + kv * dim;
            float *dk_row = dk_win + (size_t)w * dim, *dv_row = dv_win + (size_t)w * dim;
            for (size_t j = 0; j < dim; ++j) dk_row[j] = 0.0f, dv_row[j] = 0.0f;
            for (size_t hh = 0; hh < group; ++hh) {
                const size_t h = kv * group + hh;
                for (size_t t = s; t < T; ++t) {
                    const double *st = stats + 3 * (hh * window + (t - s_lo));
                    const float *q_head = q + t * q_cols + h * dim;
                    const float *dh = dout + t * q_cols + h * dim;
                    double dot = 0.0, acc = 0.0;
                    for (size_t j = 0; j < dim; ++j) dot += (double)q_head[j] * (double)k_head[j];
                    for (size_t j = 0; j < dim; ++j) acc += (double)dh[j] * (double)v_head[j];
                    const double probs_s = exp(dot * scale - st[0]) / st[1];
                    const double p_ds_s = probs_s * (acc - st[2]);
                    for (size_t j = 0; j < dim; ++j) {
                        dk_row[j] += (float)(p_ds_s * (double)q_head[j] * scale);
                        dv_row[j] += (float)(probs_s * (double)dh[j]);
                    }
                }
            }
        }
        free(probs);
        free(d_probs);
        free(p_ds);
        free(dk_dummy);
        free(dq_dummy);
    }
    free(stats);
    return failed ? ZTO_OUT_OF_MEMORY : ZTO_OK;
}

/* ---- the projection on the output side of attention -------------------------------------------- */

/*
 * tensor.matmul (src/tensor.zig:78-106): out[i, j] = sum_k a[i, k] * b[k, j], every element its own f32
 * accumulator over ascending k (the reference's eight lanes are never added to one another, so the scalar
 * loop below rounds where it does).  model.zig:396 calls it as matmul(ctx, l.wo).
 */
int zto_matmul(const float *a, size_t a_rows, size_t a_cols, const float *b, size_t b_rows, size_t b_cols,
               float *out, int threads) {
    if (a_cols != b_rows) return ZTO_DIMENSION_MISMATCH;
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long i = 0; i < (long)a_rows; ++i)
        for (size_t j = 0; j < b_cols; ++j) {
            float acc = 0.0f;
            for (size_t k = 0; k < a_cols; ++k) acc += a[(size_t)i * a_cols + k] * b[k * b_cols + j];
            out[(size_t)i * b_cols + j] = acc;
        }
    return ZTO_OK;
}

/*
 * inputGrad (src/autograd.zig:999-1022): out[t, i] += sum_j dout[t, j] * w[i, j], the sum in an f32
 * accumulator over ascending j, added to out once.
 */
int zto_input_grad(float *out, const float *dout, size_t rows, size_t dout_cols, const float *w, size_t w_rows,
                   size_t w_cols, int threads) {
    if (dout_cols != w_cols) return ZTO_DIMENSION_MISMATCH;
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long t = 0; t < (long)rows; ++t)
        for (size_t i = 0; i < w_rows; ++i) {
            float acc = 0.0f;
            for (size_t j = 0; j < w_cols; ++j) acc += dout[(size_t)t * dout_cols + j] * w[i * w_cols + j];
            out[(size_t)t * w_rows + i] += acc;
        }
    return ZTO_OK;
}

/*
 * weightGrad (src/autograd.zig:958-972): w[i, j] += input[t, i] * dout[t, j] for t ascending -- an f32
 * read-modify-write per term, into whatever w already holds.
 */
int zto_weight_grad(float *w, const float *input, size_t rows, size_t in_cols, const float *dout, size_t dout_cols,
                    int threads) {
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long i = 0; i < (long)in_cols; ++i)
        for (size_t t = 0; t < rows; ++t) {
            const float scale = input[t * in_cols + (size_t)i];
            for (size_t j = 0; j < dout_cols; ++j) w[(size_t)i * dout_cols + j] += scale * dout[t * dout_cols + j];
        }
    return ZTO_OK;
}

/* ---- kv_cache.Layer (src/kv_cache.zig:60-135), storage semantics only ------ */

typedef struct {
    float *k; /* [n_ctx, width] */
    float *v; /* [n_ctx, width] */
    size_t n_ctx, width, len;
} zto_layer;

int zto_layer_init(zto_layer *l, size_t n_ctx, size_t width) {
    if (n_ctx == 0 || width == 0) return ZTO_DIMENSION_MISMATCH; /* kv_cache.zig:66 */
    l->k = (float *)calloc(n_ctx * width, sizeof(float));
    l->v = (float *)calloc(n_ctx * width, sizeof(float));
    if (!l->k || !l->v) {
        free(l->k);
        free(l->v);
        l->k = l->v = NULL;
        return ZTO_OUT_OF_MEMORY;
    }
    l->n_ctx = n_ctx;
    l->width = width;
    l->len = 0;
    return ZTO_OK;
}

void zto_layer_deinit(zto_layer *l) {
    free(l->k);
    free(l->v);
    l->k = l->v = NULL;
    l->len = 0;
}

/* kv_cache.zig:88-95: width check first, then Full, and nothing is written on
 * either refusal. */
int zto_layer_append(zto_layer *l, const float *k_row, size_t k_len, const float *v_row,
                     size_t v_len) {
    if (k_len != l->width || v_len != l->width) return ZTO_DIMENSION_MISMATCH;
    if (l->len >= l->n_ctx) return ZTO_FULL;
    memcpy(l->k + l->len * l->width, k_row, sizeof(float) * l->width);
    memcpy(l->v + l->len * l->width, v_row, sizeof(float) * l->width);
    l->len += 1;
    return ZTO_OK;
}

size_t zto_layer_visible(const zto_layer *l) { return l->len; }
size_t zto_layer_bytes(const zto_layer *l) { return 2 * l->n_ctx * l->width * sizeof(float); }

/* ---- device.zig's pure host arithmetic ------------------------------------ */

/* bytesFor (src/cuda/device.zig:162-171). kind: 0 query_headed, 1 kv_headed, 2 per_row. */
int zto_bytes_for(int kind, uint64_t t, uint64_t n_heads, uint64_t n_kv_heads, uint64_t dim,
                  uint64_t *out_bytes) {
    if (t == 0 || dim == 0 || n_heads == 0 || n_kv_heads == 0) return ZTO_DEGENERATE_SHAPE;
    uint64_t cols;
    if (kind == 0) {
        if (__builtin_mul_overflow(n_heads, dim, &cols)) return ZTO_SHAPE_TOO_LARGE;
    } else if (kind == 1) {
        if (__builtin_mul_overflow(n_kv_heads, dim, &cols)) return ZTO_SHAPE_TOO_LARGE;
    } else {
        cols = n_heads;
    }
    uint64_t elems, bytes;
    if (__builtin_mul_overflow(t, cols, &elems)) return ZTO_SHAPE_TOO_LARGE;
    if (__builtin_mul_overflow(elems, (uint64_t)sizeof(float), &bytes)) return ZTO_SHAPE_TOO_LARGE;
    *out_bytes = bytes;
    return ZTO_OK;
}

/* forwardBounds (src/cuda/device.zig:489-501): 0 = addressable. */
int zto_forward_bounds(int c_t, int q_offset, int n_keys, int t) {
    if (n_keys < 1 || n_keys > c_t) return ZTO_SHAPE_TOO_LARGE;
    if (t < 1 || t > c_t) return ZTO_SHAPE_TOO_LARGE;
    if (q_offset < 0 || q_offset > c_t || t > c_t - q_offset) return ZTO_SHAPE_TOO_LARGE;
    if (q_offset + t > n_keys) return ZTO_SHAPE_TOO_LARGE;
    return ZTO_OK;
}

/* ---- seeded inputs --------------------------------------------------------- */

/* The reference's fixture generator (src/cuda/attn_twin.zig:283-289): a 32-bit
 * LCG, value = (x >> 8) / 2^24 - 0.5. */
void zto_fill_lcg(float *data, size_t n, uint32_t seed) {
    uint32_t x = seed;
    for (size_t i = 0; i < n; ++i) {
        x = x * 1664525u + 1013904223u;
        data[i] = (float)(x >> 8) / 16777216.0f - 0.5f;
    }
}

/* The decode test's index hash in [-1, 1) (src/decode_test.zig:35-42). The
 * reference multiplies a usize and truncates to u32, which equals the product
 * taken modulo 2^32. */
float zto_fill_hash(uint64_t i) {
    uint32_t x = (uint32_t)(i * 2654435761ull);
    x ^= x >> 15;
    x *= 2246822519u;
    x ^= x >> 13;
    return (float)(x >> 8) / 8388608.0f - 1.0f;
}

/* i.i.d. N(0,1) in f32 for the benchmark configurations: splitmix64 counter ->
 * two uniforms -> Box-Muller in f64 -> narrow. Element i of stream `stream`
 * depends only on (seed, stream, i), so any slice can be regenerated anywhere. */
static uint64_t zto_splitmix(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

void zto_fill_normal(float *data, size_t n, uint64_t seed, uint64_t stream, uint64_t first) {
    const uint64_t key = zto_splitmix(seed * 4u + stream);
#pragma omp parallel for schedule(static)
    for (long ii = 0; ii < (long)n; ++ii) {
        const uint64_t i = first + (uint64_t)ii;
        const uint64_t pair = i >> 1;
        const uint64_t a = zto_splitmix(key ^ (2 * pair));
        const uint64_t b = zto_splitmix(key ^ (2 * pair + 1));
        const double u1 = ((double)(a >> 11) + 1.0) * (1.0 / 9007199254740992.0); /* (0,1] */
        const double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);         /* [0,1) */
        const double r = sqrt(-2.0 * log(u1));
        const double th = 6.283185307179586476925286766559 * u2;
        data[ii] = (float)((i & 1) ? r * sin(th) : r * cos(th));
    }
}

/* ---- rotary position embedding -------------------------------------------------------------------
 * rope.forward (src/rope.zig:21-55): row r carries absolute position pos + r; every head block of
 * head_dim columns rotates on its own; element i pairs with element i + head_dim/2 of the same head
 * (the half-split layout, not interleaved pairs); frequency, angle and both multiply-adds in f64, one
 * narrowing at the store.  error.OddHeadDim for a zero or odd head_dim (:28), error.DimensionMismatch
 * when the row is not a whole number of head blocks (:29). */
#define ZTO_ODD_HEAD_DIM 7 /* rope.zig:28 error.OddHeadDim */

int zto_rope_forward(const float *x, size_t rows, size_t cols, size_t pos, double theta, size_t head_dim,
                     float *out) {
    if (head_dim == 0 || head_dim % 2 != 0) return ZTO_ODD_HEAD_DIM;
    if (cols % head_dim != 0) return ZTO_DIMENSION_MISMATCH;
    const size_t half = head_dim / 2;
    for (size_t r = 0; r < rows; ++r) {
        const float *src = x + r * cols;
        float *dst = out + r * cols;
        const double t = (double)(pos + r);
        for (size_t h = 0; h < cols / head_dim; ++h) {
            const size_t base = h * head_dim;
            for (size_t i = 0; i < half; ++i) {
                const double exponent = (double)(2 * i) / (double)head_dim;
                const double angle = t / pow(theta, exponent);
                const double c = cos(angle), s = sin(angle);
                const double lo = (double)src[base + i], hi = (double)src[base + i + half];
                dst[base + i] = (float)(lo * c - hi * s);
                dst[base + i + half] = (float)(hi * c + lo * s);
            }
        }
    }
    return ZTO_OK;
}

/* ropeBackward (src/autograd.zig:851-874): d x = R^T d y, the same two multiply-adds with the sine's
 * sign flipped, same pairing, same f64 angle. */
int zto_rope_backward(const float *dout, size_t rows, size_t cols, size_t pos, double theta, size_t head_dim,
                      float *din) {
    if (head_dim == 0 || head_dim % 2 != 0) return ZTO_ODD_HEAD_DIM;
    if (cols % head_dim != 0) return ZTO_DIMENSION_MISMATCH;
    const size_t half = head_dim / 2;
    for (size_t r = 0; r < rows; ++r) {
        const float *src = dout + r * cols;
        float *dst = din + r * cols;
        const double t = (double)(pos + r);
        for (size_t h = 0; h < cols / head_dim; ++h) {
            const size_t base = h * head_dim;
            for (size_t i = 0; i < half; ++i) {
                const double exponent = (double)(2 * i) / (double)head_dim;
                const double angle = t / pow(theta, exponent);
                const double c = cos(angle), s = sin(angle);
                const double lo = (double)src[base + i], hi = (double)src[base + i + half];
                dst[base + i] = (float)(lo * c + hi * s);
                dst[base + i + half] = (float)(hi * c - lo * s);
            }
        }
    }
    return ZTO_OK;
}
