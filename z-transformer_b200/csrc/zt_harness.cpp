// zt_attn_harness: grades libztattn against a directory written by the reference's twin program.
//
// The reference splits its GPU check in two (src/cuda/attn_twin.zig, src/cuda/attn.cu): the twin runs
// the CPU implementations and writes, per shape, the inputs and the reference answers as raw
// little-endian f32 blobs  <tag>.{q,k,v,y,dout,dq,dk,dv}.bin  plus  manifest.tsv  with one row per shape
//     tag  T  n_heads  n_kv_heads  head_dim  iters  cpu_us
// (attn_twin.zig:198-201,262-269; read back at attn.cu:170-224); the harness uploads them, launches the
// library and compares.  This program reads the same directory, so a maintainer can point it at the
// output of `zig build attn-twin` unchanged.  What it prints and gates, as attn.cu does:
//   * forward: max |out - y| per shape against 1e-4 (attn.cu:51), kernel time (minimum of three
//     timed batches, attn.cu:629-652) beside the manifest's CPU time;
//   * backward: max |.| of dq, dk, dv against 1e-5 (attn.cu:114);
//   * one launch of both entry points per shape at T = 8 on uninitialised memory: return codes and
//     a clean synchronise (attn.cu:851-909);
//   * negative controls (run-attn.sh:126-177): ZT_HARNESS_BROKEN=1..4 and ZT_HARNESS_BWD_BROKEN=1..4
//     each inject one defect and must make the run exit non-zero.  The library's kernels carry no
//     defect switches, so the defects are injected through its ABI, on the data or the call:
//       forward   1 key rows rotated by one position (every score meets the wrong key)
//                 2 grouped-query attention collapsed (every KV head replaced by KV head 0)
//                 3 K and V exchanged
//                 4 the 1/sqrt(head_dim) scale dropped (q pre-multiplied by sqrt(head_dim))
//       backward  1 dout rows rotated by one position
//                 2 grouped-query attention collapsed
//                 3 the softmax Jacobian dropped (delta = 0: the batched backward is handed out = 0);
//                   dv must then read exactly as in the correct run, dq and dk must not
//                 4 the scale dropped
//   * ZT_HARNESS_KERNEL_DEFECT=1|3|11|13 (only in zt_attn_harness_defects, which links the library built with
//     -DZT_DEFECTS) switches on a defect compiled INTO the kernels, as the reference's ATTN_BROKEN template variants
//     are (src/cuda/attn_kernels.cu:150-158,592-599,622-624): 1 the forward's causal mask dropped, 3 its
//     running-maximum correction skipped, 11 the backward's causal mask dropped, 13 its softmax Jacobian dropped.
//     Each must fail a gate; 13 must leave dv exactly right.
//   * ZT_HARNESS_DOUT_SCALE=<x> multiplies dout (and, the backward being linear in it, the reference
//     gradients) by x before the run and replaces the backward's absolute gate by a scale-relative one,
//     max |got - ref| <= 1e-4 max |ref| per tensor (attn_rel_tol, src/train.zig:706).  The absolute
//     gate is calibrated on a dout of order 0.5; a training step supplies one of order 1e-5
//     (attn.cu:103-113), where 1e-5 absolute would pass anything.
// `--list <dir>` parses the manifest and checks every blob's size without touching the GPU.
// Exit status: 0 all gates passed, 1 a gate failed or a file was unreadable, 2 usage.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/zt_attn.h"

namespace {

constexpr double kFwdTol = 1e-4;  // attn.cu:51
constexpr double kBwdTol = 1e-5;  // attn.cu:114
constexpr double kRelTol = 1e-4;  // src/train.zig:706 attn_rel_tol
constexpr int kTagCap = 40, kMaxShapes = 64;

struct Shape {
    char tag[kTagCap];
    int T, n_heads, n_kv_heads, head_dim, iters;
    double cpu_us;
    size_t qn() const { return (size_t)T * n_heads * head_dim; }
    size_t kn() const { return (size_t)T * n_kv_heads * head_dim; }
};

bool read_floats(const std::string &dir, const char *tag, const char *suffix, size_t expect, std::vector<float> *out) {
    const std::string path = dir + "/" + tag + suffix + ".bin";
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) {
        fprintf(stderr, "harness: FAIL cannot open %s\n", path.c_str());
        return false;
    }
    fseek(f, 0, SEEK_END);
    const long bytes = ftell(f);
    fseek(f, 0, SEEK_SET);
    if (bytes < 0 || (size_t)bytes != expect * sizeof(float)) {
        fprintf(stderr, "harness: FAIL %s holds %ld bytes, expected %zu\n", path.c_str(), bytes, expect * sizeof(float));
        fclose(f);
        return false;
    }
    if (out) {
        out->resize(expect);
        if (fread(out->data(), sizeof(float), expect, f) != expect) {
            fprintf(stderr, "harness: FAIL short read of %s\n", path.c_str());
            fclose(f);
            return false;
        }
    }
    fclose(f);
    return true;
}

int read_manifest(const std::string &dir, Shape *out) {
    const std::string path = dir + "/manifest.tsv";
    FILE *f = fopen(path.c_str(), "r");
    if (!f) {
        fprintf(stderr, "harness: FAIL cannot open %s. Write the directory first; this program compares, it does not "
                        "generate.\n", path.c_str());
        return -1;
    }
    int n = 0;
    while (n < kMaxShapes && fscanf(f, "%39s %d %d %d %d %d %lf", out[n].tag, &out[n].T, &out[n].n_heads,
                                    &out[n].n_kv_heads, &out[n].head_dim, &out[n].iters, &out[n].cpu_us) == 7)
        ++n;
    fclose(f);
    if (n == 0) {
        fprintf(stderr, "harness: FAIL manifest.tsv holds no readable rows\n");
        return -1;
    }
    for (int i = 0; i < n; ++i)
        if (out[i].T < 1 || out[i].n_heads < 1 || out[i].n_kv_heads < 1 || out[i].head_dim < 1) {
            fprintf(stderr, "harness: FAIL manifest row %s has a non-positive size\n", out[i].tag);
            return -1;
        }
    return n;
}

// NaN counts as the worst result there is (attn.cu:231-237).
double max_abs_diff(const std::vector<float> &got, const std::vector<float> &want, size_t *where) {
    double worst = 0.0;
    size_t at = 0;
    for (size_t i = 0; i < got.size(); ++i) {
        double d = fabs((double)got[i] - (double)want[i]);
        if (std::isnan(d)) d = INFINITY;
        if (d > worst) worst = d, at = i;
    }
    if (where) *where = at;
    return worst;
}

int env_variant(const char *name) {
    const char *e = getenv(name);
    if (!e || !*e) return 0;
    if (strlen(e) == 1 && e[0] >= '0' && e[0] <= '4') return e[0] - '0';
    fprintf(stderr, "harness: %s=%s is not a variant this program has. Variants are 0 (none) to 4.\n", name, e);
    exit(2);
}

void rotate_rows(std::vector<float> &x, int rows, size_t width) {  // row r := row (r + 1) % rows
    std::vector<float> first(x.begin(), x.begin() + width);
    memmove(x.data(), x.data() + width, (size_t)(rows - 1) * width * sizeof(float));
    memcpy(x.data() + (size_t)(rows - 1) * width, first.data(), width * sizeof(float));
}
void collapse_gqa(std::vector<float> &x, const Shape &s) {  // every KV head := KV head 0
    const size_t w = (size_t)s.n_kv_heads * s.head_dim;
    for (int t = 0; t < s.T; ++t)
        for (int h = 1; h < s.n_kv_heads; ++h)
            memcpy(&x[t * w + (size_t)h * s.head_dim], &x[t * w], s.head_dim * sizeof(float));
}

#define CUDA_OK(call)                                                                          \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            fprintf(stderr, "harness: FAIL %s: %s\n", #call, cudaGetErrorString(e_));          \
            return 1;                                                                          \
        }                                                                                      \
    } while (0)

struct DeviceBuf {
    float *p = nullptr;
    ~DeviceBuf() { if (p) cudaFree(p); }
    cudaError_t alloc(size_t n) { return cudaMalloc((void **)&p, (n ? n : 1) * sizeof(float)); }
    cudaError_t up(const std::vector<float> &h) { return cudaMemcpy(p, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice); }
    cudaError_t down(std::vector<float> *h, size_t n) { h->resize(n); return cudaMemcpy(h->data(), p, n * sizeof(float), cudaMemcpyDeviceToHost); }
};

int run(const std::string &dir) {
    Shape shapes[kMaxShapes];
    const int n = read_manifest(dir, shapes);
    if (n < 0) return 1;
    const int broken = env_variant("ZT_HARNESS_BROKEN"), bwd_broken = env_variant("ZT_HARNESS_BWD_BROKEN");
    if (broken) printf("harness: forward defect %d injected; the forward gate must fail\n", broken);
    if (bwd_broken) printf("harness: backward defect %d injected; the backward gate must fail\n", bwd_broken);
    int ok = 1;

    struct FwdRow { double max_abs, us; size_t where; const char *path; };
    struct BwdRow { double dq, dk, dv, us, rel; };
    double dout_scale = 1.0;
    if (const char *e = getenv("ZT_HARNESS_DOUT_SCALE")) {
        dout_scale = atof(e);
        if (!(dout_scale > 0.0)) {
            fprintf(stderr, "harness: ZT_HARNESS_DOUT_SCALE=%s is not a positive number\n", e);
            return 2;
        }
        printf("harness: dout and the reference gradients scaled by %g; the backward gate is %.0e of max |ref|\n", dout_scale, kRelTol);
    }
    if (const char *e = getenv("ZT_HARNESS_KERNEL_DEFECT")) {
        // a defect INSIDE the kernels: only a library built with -DZT_DEFECTS has the switch
        typedef int (*set_defect_fn)(int);
        set_defect_fn set_defect = reinterpret_cast<set_defect_fn>(dlsym(RTLD_DEFAULT, "zt_attn_set_defect"));
        const int defect = atoi(e);
        if (!set_defect) {
            fprintf(stderr, "harness: ZT_HARNESS_KERNEL_DEFECT needs the defects build of the library (zt_attn_harness_defects)\n");
            return 2;
        }
        if (!(defect == 0 || defect == 1 || defect == 3 || defect == 11 || defect == 13) || set_defect(defect) != 0) {
            fprintf(stderr, "harness: ZT_HARNESS_KERNEL_DEFECT=%s is not a defect the kernels have (0, 1, 3, 11, 13)\n", e);
            return 2;
        }
        if (defect) printf("harness: defect %d compiled into the kernels is switched on; a gate must fail\n", defect);
    }
    const bool relative_gate = dout_scale != 1.0;
    std::vector<FwdRow> frows(n);
    std::vector<BwdRow> brows(n);
    for (int i = 0; i < n; ++i) {
        const Shape &s = shapes[i];
        std::vector<float> q, k, v, y, dout, dq, dk, dv;
        if (!read_floats(dir, s.tag, ".q", s.qn(), &q) || !read_floats(dir, s.tag, ".k", s.kn(), &k) ||
            !read_floats(dir, s.tag, ".v", s.kn(), &v) || !read_floats(dir, s.tag, ".y", s.qn(), &y) ||
            !read_floats(dir, s.tag, ".dout", s.qn(), &dout) || !read_floats(dir, s.tag, ".dq", s.qn(), &dq) ||
            !read_floats(dir, s.tag, ".dk", s.kn(), &dk) || !read_floats(dir, s.tag, ".dv", s.kn(), &dv))
            return 1;
        const float root_d = sqrtf((float)s.head_dim);
        if (dout_scale != 1.0) {
            const float f = (float)dout_scale;
            for (float &x : dout) x *= f;
            for (float &x : dq) x *= f;
            for (float &x : dk) x *= f;
            for (float &x : dv) x *= f;
        }
        // ---- forward ------------------------------------------------------------------------------
        {
            std::vector<float> fq = q, fk = k, fv = v;
            if (broken == 1) rotate_rows(fk, s.T, (size_t)s.n_kv_heads * s.head_dim);
            if (broken == 2) collapse_gqa(fk, s), collapse_gqa(fv, s);
            if (broken == 3) fk.swap(fv);
            if (broken == 4) for (float &x : fq) x *= root_d;
            DeviceBuf dq_, dk_, dv_, do_;
            CUDA_OK(dq_.alloc(s.qn())); CUDA_OK(dk_.alloc(s.kn())); CUDA_OK(dv_.alloc(s.kn())); CUDA_OK(do_.alloc(s.qn()));
            CUDA_OK(dq_.up(fq)); CUDA_OK(dk_.up(fk)); CUDA_OK(dv_.up(fv));
            CUDA_OK(cudaMemset(do_.p, 0xff, s.qn() * sizeof(float)));  // NaN: the forward must not depend on out
            if (zt_attn_forward(dq_.p, dk_.p, dv_.p, do_.p, s.T, s.n_heads, s.n_kv_heads, s.head_dim, 1, 64, 0, s.T, nullptr)) {
                fprintf(stderr, "harness: FAIL zt_attn_forward refused %s\n", s.tag);
                return 1;
            }
            std::vector<float> got;
            CUDA_OK(do_.down(&got, s.qn()));
            frows[i].max_abs = max_abs_diff(got, y, &frows[i].where);
            frows[i].path = zt_attn_last_path();
            const int iters = s.iters < 1 ? 1 : (s.iters > 50 ? 50 : s.iters);
            cudaEvent_t e0, e1;
            CUDA_OK(cudaEventCreate(&e0)); CUDA_OK(cudaEventCreate(&e1));
            double best = 1e30;
            for (int rep = 0; rep < 3; ++rep) {
                CUDA_OK(cudaEventRecord(e0));
                for (int it = 0; it < iters; ++it)
                    zt_attn_forward(dq_.p, dk_.p, dv_.p, do_.p, s.T, s.n_heads, s.n_kv_heads, s.head_dim, 1, 64, 0, s.T, nullptr);
                CUDA_OK(cudaEventRecord(e1));
                CUDA_OK(cudaEventSynchronize(e1));
                float ms = 0.f;
                CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
                if (ms * 1e3 / iters < best) best = ms * 1e3 / iters;
            }
            frows[i].us = best;
            cudaEventDestroy(e0), cudaEventDestroy(e1);
            if (!(frows[i].max_abs <= kFwdTol)) ok = 0;
        }
        // ---- backward -----------------------------------------------------------------------------
        {
            std::vector<float> bq = q, bk = k, bv = v, bdo = dout;
            if (bwd_broken == 1) rotate_rows(bdo, s.T, (size_t)s.n_heads * s.head_dim);
            if (bwd_broken == 2) collapse_gqa(bk, s), collapse_gqa(bv, s);
            if (bwd_broken == 4) for (float &x : bq) x *= root_d;
            const size_t mn = (size_t)s.T * s.n_heads;
            DeviceBuf q_, k_, v_, do_, dq_, dk_, dv_, rm, rl, rd, out_;
            CUDA_OK(q_.alloc(s.qn())); CUDA_OK(k_.alloc(s.kn())); CUDA_OK(v_.alloc(s.kn())); CUDA_OK(do_.alloc(s.qn()));
            CUDA_OK(dq_.alloc(s.qn())); CUDA_OK(dk_.alloc(s.kn())); CUDA_OK(dv_.alloc(s.kn()));
            CUDA_OK(rm.alloc(mn)); CUDA_OK(rl.alloc(mn)); CUDA_OK(rd.alloc(mn));
            CUDA_OK(q_.up(bq)); CUDA_OK(k_.up(bk)); CUDA_OK(v_.up(bv)); CUDA_OK(do_.up(bdo));
            // dq, dk, dv are assigned, not accumulated into: start them from NaN
            CUDA_OK(cudaMemset(dq_.p, 0xff, s.qn() * sizeof(float)));
            CUDA_OK(cudaMemset(dk_.p, 0xff, s.kn() * sizeof(float)));
            CUDA_OK(cudaMemset(dv_.p, 0xff, s.kn() * sizeof(float)));
            void *ws = nullptr;
            size_t ws_bytes = 0;
            auto launch = [&]() -> int {
                if (bwd_broken != 3)
                    return zt_attn_backward(q_.p, k_.p, v_.p, do_.p, dq_.p, dk_.p, dv_.p, rm.p, rl.p, rd.p, s.T, s.n_heads,
                                            s.n_kv_heads, s.head_dim, 64, nullptr);
                // delta = sum dout * out with out = 0: the Jacobian term vanishes
                return zt_attn_backward_batched(q_.p, k_.p, v_.p, out_.p, rm.p, do_.p, dq_.p, dk_.p, dv_.p, rd.p, ws, ws_bytes, 1,
                                                s.T, s.n_heads, s.n_kv_heads, s.head_dim, nullptr);
            };
            if (bwd_broken == 3) {
                CUDA_OK(out_.alloc(s.qn()));
                // the log-sum-exp from a correct forward, then out := 0
                if (zt_attn_forward_batched(q_.p, k_.p, v_.p, out_.p, rm.p, 1, s.T, s.n_heads, s.n_kv_heads, s.head_dim, nullptr)) return 1;
                CUDA_OK(cudaMemset(out_.p, 0, s.qn() * sizeof(float)));
                ws_bytes = zt_attn_backward_workspace_bytes(1, s.T, s.n_heads, s.n_kv_heads, s.head_dim);
                if (ws_bytes) CUDA_OK(cudaMalloc(&ws, ws_bytes));
            }
            if (launch()) {
                fprintf(stderr, "harness: FAIL the backward refused %s\n", s.tag);
                return 1;
            }
            std::vector<float> g;
            CUDA_OK(dq_.down(&g, s.qn())); brows[i].dq = max_abs_diff(g, dq, nullptr);
            CUDA_OK(dk_.down(&g, s.kn())); brows[i].dk = max_abs_diff(g, dk, nullptr);
            CUDA_OK(dv_.down(&g, s.kn())); brows[i].dv = max_abs_diff(g, dv, nullptr);
            const int iters = s.iters < 1 ? 1 : (s.iters > 20 ? 20 : s.iters);
            cudaEvent_t e0, e1;
            CUDA_OK(cudaEventCreate(&e0)); CUDA_OK(cudaEventCreate(&e1));
            double best = 1e30;
            for (int rep = 0; rep < 3; ++rep) {
                CUDA_OK(cudaEventRecord(e0));
                for (int it = 0; it < iters; ++it) launch();
                CUDA_OK(cudaEventRecord(e1));
                CUDA_OK(cudaEventSynchronize(e1));
                float ms = 0.f;
                CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
                if (ms * 1e3 / iters < best) best = ms * 1e3 / iters;
            }
            brows[i].us = best;
            cudaEventDestroy(e0), cudaEventDestroy(e1);
            if (ws) cudaFree(ws);
            auto max_abs = [](const std::vector<float> &x) {
                double m = 0.0;
                for (float f : x) m = fmax(m, fabs((double)f));
                return m;
            };
            brows[i].rel = fmax(brows[i].dq / max_abs(dq), fmax(brows[i].dk / max_abs(dk), brows[i].dv / max_abs(dv)));
            if (relative_gate ? !(brows[i].rel <= kRelTol)
                              : !(brows[i].dq <= kBwdTol && brows[i].dk <= kBwdTol && brows[i].dv <= kBwdTol))
                ok = 0;
        }
    }

    printf("\nforward against attention.forward (gate %.0e):\n", kFwdTol);
    printf("  %-14s %6s %7s %5s  %-11s %6s  %11s %13s %9s  %s\n", "shape", "T", "heads", "dim", "max_abs", "used", "kernel_us",
           "cpu_us", "speedup", "path");
    for (int i = 0; i < n; ++i) {
        const Shape &s = shapes[i];
        char heads[16];
        snprintf(heads, sizeof heads, "%d/%d", s.n_heads, s.n_kv_heads);
        printf("  %-14s %6d %7s %5d  %.3e %5.1f%%  %11.2f %13.2f %8.0fx  %s%s\n", s.tag, s.T, heads, s.head_dim, frows[i].max_abs,
               100.0 * frows[i].max_abs / kFwdTol, frows[i].us, s.cpu_us, s.cpu_us / frows[i].us, frows[i].path,
               frows[i].max_abs <= kFwdTol ? "" : "   <-- FAIL");
    }
    if (relative_gate) printf("\nbackward against autograd.attentionBackward (gate %.0e of max |ref|):\n", kRelTol);
    else printf("\nbackward against autograd.attentionBackward (gate %.0e):\n", kBwdTol);
    printf("  %-14s %-11s %-11s %-11s %6s  %-11s %11s\n", "shape", "max_abs_dq", "max_abs_dk", "max_abs_dv", "used", "rel_to_max", "kernel_us");
    for (int i = 0; i < n; ++i) {
        const double worst = fmax(brows[i].dq, fmax(brows[i].dk, brows[i].dv));
        const bool pass = relative_gate ? brows[i].rel <= kRelTol : worst <= kBwdTol;
        printf("  %-14s %.3e   %.3e   %.3e %5.1f%%  %.3e   %11.2f%s\n", shapes[i].tag, brows[i].dq, brows[i].dk, brows[i].dv,
               relative_gate ? 100.0 * brows[i].rel / kRelTol : 100.0 * worst / kBwdTol, brows[i].rel, brows[i].us,
               pass ? "" : "   <-- FAIL");
    }

    // ---- one launch of both entry points per shape at T = 8, on uninitialised memory ----------------
    printf("\nlibrary entry points, one launch per manifest shape at T=8:\n");
    {
        const int Tp = 8;
        size_t qn = 0, kn = 0, mn = 0;
        for (int i = 0; i < n; ++i) {
            qn = std::max(qn, (size_t)Tp * shapes[i].n_heads * shapes[i].head_dim);
            kn = std::max(kn, (size_t)Tp * shapes[i].n_kv_heads * shapes[i].head_dim);
            mn = std::max(mn, (size_t)Tp * shapes[i].n_heads);
        }
        DeviceBuf pq, pk, pv, po, pdo, pdq, pdk, pdv, prm, prl, prd;
        CUDA_OK(pq.alloc(qn)); CUDA_OK(pk.alloc(kn)); CUDA_OK(pv.alloc(kn)); CUDA_OK(po.alloc(qn)); CUDA_OK(pdo.alloc(qn));
        CUDA_OK(pdq.alloc(qn)); CUDA_OK(pdk.alloc(kn)); CUDA_OK(pdv.alloc(kn));
        CUDA_OK(prm.alloc(mn)); CUDA_OK(prl.alloc(mn)); CUDA_OK(prd.alloc(mn));
        for (int i = 0; i < n; ++i) {
            const Shape &s = shapes[i];
            const int rf = zt_attn_forward(pq.p, pk.p, pv.p, po.p, Tp, s.n_heads, s.n_kv_heads, s.head_dim, 1, 64, 0, Tp, nullptr);
            const int rb = zt_attn_backward(pq.p, pk.p, pv.p, pdo.p, pdq.p, pdk.p, pdv.p, prm.p, prl.p, prd.p, Tp, s.n_heads,
                                            s.n_kv_heads, s.head_dim, 64, nullptr);
            CUDA_OK(cudaDeviceSynchronize());
            printf("  %-14s head_dim %-4d forward %d  backward %d%s\n", s.tag, s.head_dim, rf, rb,
                   (rf || rb) ? "   <-- REFUSED" : "");
            if (rf || rb) ok = 0;
        }
    }
    int tc_status = 0;
    if (zt_attn_tc_status(&tc_status) != 0 || tc_status != 0) {
        printf("harness: FAIL a tensor-core kernel gave up on a wait (status %d)\n", tc_status);
        ok = 0;
    }
    printf("\nharness: %s\n", ok ? "PASS" : "FAIL");
    return ok ? 0 : 1;
}

int list_only(const std::string &dir) {
    Shape shapes[kMaxShapes];
    const int n = read_manifest(dir, shapes);
    if (n < 0) return 1;
    static const char *q_like[] = {".q", ".y", ".dout", ".dq"}, *k_like[] = {".k", ".v", ".dk", ".dv"};
    for (int i = 0; i < n; ++i) {
        const Shape &s = shapes[i];
        for (const char *sfx : q_like)
            if (!read_floats(dir, s.tag, sfx, s.qn(), nullptr)) return 1;
        for (const char *sfx : k_like)
            if (!read_floats(dir, s.tag, sfx, s.kn(), nullptr)) return 1;
        printf("%s T=%d heads=%d/%d head_dim=%d iters=%d cpu_us=%.6f\n", s.tag, s.T, s.n_heads, s.n_kv_heads, s.head_dim,
               s.iters, s.cpu_us);
    }
    return 0;
}

}  // namespace

int main(int argc, char **argv) {
    if (argc == 3 && strcmp(argv[1], "--list") == 0) return list_only(argv[2]);
    if (argc != 2) {
        fprintf(stderr, "usage: %s <twin-dir>        grade the library against the directory\n"
                        "       %s --list <twin-dir> parse the manifest and check the blobs' sizes only\n", argv[0], argv[0]);
        return 2;
    }
    return run(argv[1]);
}
