// zt::device::Attn (zt_host.hpp) and a C shim over it.  Links against libztattn.so and the CUDA runtime.
#include "zt_host.hpp"

#include <cuda_runtime.h>

#include "../../../include/zt_attn.h"

namespace zt {
namespace device {

namespace {
Error alloc(uint64_t bytes, float **out) {  // device.zig:434-438
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess || p == nullptr) {
        cudaGetLastError();
        return Error::DeviceAllocFailed;
    }
    *out = static_cast<float *>(p);
    return Error::Ok;
}
}  // namespace

float *Attn::field(int i) const {
    float *const f[N_BUFFERS] = {q, k, v, out, dout, dq, dk, dv, row_max, row_den, row_del};
    return (i >= 0 && i < N_BUFFERS) ? f[i] : nullptr;
}

void Attn::deinitPartial(int taken) {
    float **const f[N_BUFFERS] = {&q, &k, &v, &out, &dout, &dq, &dk, &dv, &row_max, &row_den, &row_del};
    for (int i = 0; i < taken; ++i) {
        if (*f[i]) cudaFree(*f[i]);
        *f[i] = nullptr;
    }
}

void Attn::deinit() { deinitPartial(N_BUFFERS); }

Error Attn::init(uint64_t t_, uint64_t n_heads_, uint64_t n_kv_heads_, uint64_t dim_) {
    deinit();
    Error e;
    int ct, ch, ckv, cd;
    if ((e = toCInt(t_, &ct)) != Error::Ok) return e;
    if ((e = toCInt(n_heads_, &ch)) != Error::Ok) return e;
    if ((e = toCInt(n_kv_heads_, &ckv)) != Error::Ok) return e;
    if ((e = toCInt(dim_, &cd)) != Error::Ok) return e;
    // ask the C side before allocating anything (device.zig:227-241)
    if (zt_attn_dim_ok(cd) == 0) return Error::ConfigRefused;
    if (ch <= 0 || ckv <= 0 || ch % ckv != 0) return Error::ConfigRefused;
    if (n_heads_ > 65535) return Error::ConfigRefused;
    uint64_t qh, kvh, pr;
    if ((e = bytesFor(Kind::query_headed, t_, n_heads_, n_kv_heads_, dim_, &qh)) != Error::Ok) return e;
    if ((e = bytesFor(Kind::kv_headed, t_, n_heads_, n_kv_heads_, dim_, &kvh)) != Error::Ok) return e;
    if ((e = bytesFor(Kind::per_row, t_, n_heads_, n_kv_heads_, dim_, &pr)) != Error::Ok) return e;
    float **const f[N_BUFFERS] = {&q, &k, &v, &out, &dout, &dq, &dk, &dv, &row_max, &row_den, &row_del};
    const uint64_t size[N_BUFFERS] = {qh, kvh, kvh, qh, qh, qh, kvh, kvh, pr, pr, pr};
    for (int i = 0; i < N_BUFFERS; ++i) {
        if ((e = alloc(size[i], f[i])) != Error::Ok) {
            deinitPartial(i);
            return e;
        }
    }
    // The library's own scratch for this shape (the operand planes of its tensor-core kernels live in a per-device
    // arena, the reference's signatures having no workspace argument) is sized here, with the holder's buffers, so
    // that forward() and backward() never allocate: the one line a maintainer adds to device.Attn.init.
    if (zt_attn_reserve(1, ct, ch, ckv, cd) != 0) {
        deinitPartial(N_BUFFERS);
        return Error::DeviceAllocFailed;
    }
    t = t_, n_heads = n_heads_, n_kv_heads = n_kv_heads_, dim = dim_;
    c_t = ct, c_heads = ch, c_kv_heads = ckv, c_dim = cd;
    return Error::Ok;
}

uint64_t Attn::totalBytes() const {  // device.zig:355-360
    uint64_t qh = 0, kvh = 0, pr = 0;
    if (bytesFor(Kind::query_headed, t, n_heads, n_kv_heads, dim, &qh) != Error::Ok) qh = 0;
    if (bytesFor(Kind::kv_headed, t, n_heads, n_kv_heads, dim, &kvh) != Error::Ok) kvh = 0;
    if (bytesFor(Kind::per_row, t, n_heads, n_kv_heads, dim, &pr) != Error::Ok) pr = 0;
    return 4 * qh + 4 * kvh + 3 * pr;
}

Error Attn::forwardAt(int group_q, int max_tile, int q_offset, int n_keys, int t_rows) const {  // device.zig:387-398
    const Error e = forwardBounds(c_t, q_offset, n_keys, t_rows);
    if (e != Error::Ok) return e;
    const int rc = zt_attn_forward(q, k, v, out, t_rows, c_heads, c_kv_heads, c_dim, group_q, max_tile, q_offset, n_keys, nullptr);
    return rc != 0 ? Error::ConfigRefused : Error::Ok;
}

Error Attn::backward(int max_tile) const {  // device.zig:403-406
    const int rc = zt_attn_backward(q, k, v, dout, dq, dk, dv, row_max, row_den, row_del, c_t, c_heads, c_kv_heads, c_dim,
                                    max_tile, nullptr);
    return rc != 0 ? Error::ConfigRefused : Error::Ok;
}

uint64_t Attn::bufferBytes(const float *target) const {  // device.zig:440-458
    uint64_t qh = 0, kvh = 0, pr = 0;
    if (bytesFor(Kind::query_headed, t, n_heads, n_kv_heads, dim, &qh) != Error::Ok) return 0;
    if (bytesFor(Kind::kv_headed, t, n_heads, n_kv_heads, dim, &kvh) != Error::Ok) return 0;
    if (bytesFor(Kind::per_row, t, n_heads, n_kv_heads, dim, &pr) != Error::Ok) return 0;
    const uint64_t size[N_BUFFERS] = {qh, kvh, kvh, qh, qh, qh, kvh, kvh, pr, pr, pr};
    if (target == nullptr) return 0;
    for (int i = 0; i < N_BUFFERS; ++i)
        if (field(i) == target) return size[i];
    return 0;
}

// The reference maps a failed copy to DeviceAllocFailed (device.zig:418,429); kept.
Error Attn::upload(float *dst, const float *src, uint64_t n_floats) const {  // device.zig:412-419
    uint64_t n;
    if (!mul_usize(n_floats, sizeof(float), &n)) return Error::ShapeTooLarge;
    if (n > bufferBytes(dst)) return Error::ShapeTooLarge;
    if (cudaMemcpy(dst, src, n, cudaMemcpyHostToDevice) != cudaSuccess) return Error::DeviceAllocFailed;
    return Error::Ok;
}

Error Attn::download(float *dst, uint64_t n_floats, const float *src) const {  // device.zig:426-431
    uint64_t n;
    if (!mul_usize(n_floats, sizeof(float), &n)) return Error::ShapeTooLarge;
    if (n > bufferBytes(src)) return Error::ShapeTooLarge;
    if (cudaMemcpy(dst, src, n, cudaMemcpyDeviceToHost) != cudaSuccess) return Error::DeviceAllocFailed;
    return Error::Ok;
}

// ---- AttnPipeline ----------------------------------------------------------------------------------------
struct AttnPipeline::Slot {
    float *q = nullptr, *k = nullptr, *v = nullptr, *dout = nullptr, *out = nullptr, *lse = nullptr;
    float *dq = nullptr, *dk = nullptr, *dv = nullptr, *delta = nullptr;
    void *ws = nullptr;
    cudaEvent_t ready_f = nullptr, ready_b = nullptr, done_f = nullptr, done = nullptr, free_ = nullptr;
};

void AttnPipeline::deinit() {
    if (slot_) {
        for (int i = 0; i < slots_; ++i) {
            Slot &s = slot_[i];
            float *bufs[] = {s.q, s.k, s.v, s.dout, s.out, s.lse, s.dq, s.dk, s.dv, s.delta};
            for (float *b : bufs)
                if (b) cudaFree(b);
            if (s.ws) cudaFree(s.ws);
            cudaEvent_t evs[] = {s.ready_f, s.ready_b, s.done_f, s.done, s.free_};
            for (cudaEvent_t e : evs)
                if (e) cudaEventDestroy(e);
        }
        delete[] slot_;
        slot_ = nullptr;
    }
    void **streams[] = {&s_in_, &s_run_, &s_out_};
    for (void **st : streams) {
        if (*st) cudaStreamDestroy(static_cast<cudaStream_t>(*st));
        *st = nullptr;
    }
    slots_ = 0;
}

Error AttnPipeline::init(uint64_t t, uint64_t n_heads, uint64_t n_kv_heads, uint64_t dim, int slots) {
    deinit();
    Error e;
    if (slots < 1) return Error::DegenerateShape;
    if ((e = toCInt(t, &c_t)) != Error::Ok || (e = toCInt(n_heads, &c_heads)) != Error::Ok ||
        (e = toCInt(n_kv_heads, &c_kv_heads)) != Error::Ok || (e = toCInt(dim, &c_dim)) != Error::Ok)
        return e;
    if (zt_attn_dim_ok(c_dim) == 0) return Error::ConfigRefused;
    if (c_heads <= 0 || c_kv_heads <= 0 || c_heads % c_kv_heads != 0 || n_heads > 65535) return Error::ConfigRefused;
    if ((e = bytesFor(Kind::query_headed, t, n_heads, n_kv_heads, dim, &qh_)) != Error::Ok) return e;
    if ((e = bytesFor(Kind::kv_headed, t, n_heads, n_kv_heads, dim, &kvh_)) != Error::Ok) return e;
    if ((e = bytesFor(Kind::per_row, t, n_heads, n_kv_heads, dim, &pr_)) != Error::Ok) return e;
    ws_bytes_ = zt_attn_backward_workspace_bytes(1, c_t, c_heads, c_kv_heads, c_dim);
    slot_ = new Slot[slots];
    slots_ = slots;
    cudaStream_t st[3];
    for (int i = 0; i < 3; ++i)
        if (cudaStreamCreateWithFlags(&st[i], cudaStreamNonBlocking) != cudaSuccess) {
            for (int j = 0; j < i; ++j) cudaStreamDestroy(st[j]);
            deinit();
            return Error::DeviceAllocFailed;
        }
    s_in_ = st[0], s_run_ = st[1], s_out_ = st[2];
    for (int i = 0; i < slots; ++i) {
        Slot &s = slot_[i];
        float **bufs[] = {&s.q, &s.dout, &s.out, &s.dq, &s.k, &s.v, &s.dk, &s.dv, &s.lse, &s.delta};
        const uint64_t size[] = {qh_, qh_, qh_, qh_, kvh_, kvh_, kvh_, kvh_, pr_, pr_};
        for (int b = 0; b < 10; ++b)
            if (alloc(size[b], bufs[b]) != Error::Ok) {
                deinit();
                return Error::DeviceAllocFailed;
            }
        if (ws_bytes_ && cudaMalloc(&s.ws, ws_bytes_) != cudaSuccess) {
            deinit();
            return Error::DeviceAllocFailed;
        }
        cudaEvent_t *evs[] = {&s.ready_f, &s.ready_b, &s.done_f, &s.done, &s.free_};
        for (cudaEvent_t *ev : evs)
            if (cudaEventCreateWithFlags(ev, cudaEventDisableTiming) != cudaSuccess) {
                deinit();
                return Error::DeviceAllocFailed;
            }
    }
    return Error::Ok;
}

Error AttnPipeline::step(int batch, const float *q, const float *k, const float *v, const float *dout, float *out,
                         float *dq, float *dk, float *dv, float *lse) {
    if (!slot_ || batch < 1) return Error::DegenerateShape;
    cudaStream_t s_in = static_cast<cudaStream_t>(s_in_), s_run = static_cast<cudaStream_t>(s_run_),
                 s_out = static_cast<cudaStream_t>(s_out_);
    const uint64_t qf = qh_ / sizeof(float), kf = kvh_ / sizeof(float), pf = pr_ / sizeof(float);
    bool failed = false, refused = false;
    auto copy = [&](void *dst, const void *src, uint64_t bytes, cudaMemcpyKind kind, cudaStream_t st) {
        if (cudaMemcpyAsync(dst, src, bytes, kind, st) != cudaSuccess) failed = true;
    };
    for (int b = 0; b < batch && !failed && !refused; ++b) {
        Slot &s = slot_[b % slots_];
        const bool reused = b >= slots_;
        // The forward needs q, k, v only and its output can leave while the backward runs: dout goes up behind
        // them and out goes down ahead of the gradients.
        if (reused) cudaStreamWaitEvent(s_in, s.done, 0);  // the slot's inputs have been consumed
        copy(s.q, q + b * qf, qh_, cudaMemcpyHostToDevice, s_in);
        copy(s.k, k + b * kf, kvh_, cudaMemcpyHostToDevice, s_in);
        copy(s.v, v + b * kf, kvh_, cudaMemcpyHostToDevice, s_in);
        cudaEventRecord(s.ready_f, s_in);
        copy(s.dout, dout + b * qf, qh_, cudaMemcpyHostToDevice, s_in);
        cudaEventRecord(s.ready_b, s_in);

        cudaStreamWaitEvent(s_run, s.ready_f, 0);
        if (reused) cudaStreamWaitEvent(s_run, s.free_, 0);  // the slot's outputs have been read
        // q, k, v of the slot are not written between its forward and its backward, which is what the token says
        unsigned long long token = 0;
        if (zt_attn_forward_batched_keep(s.q, s.k, s.v, s.out, s.lse, s.ws, ws_bytes_, 1, c_t, c_heads, c_kv_heads, c_dim,
                                         reinterpret_cast<zt_stream_t>(s_run), &token))
            refused = true;
        cudaEventRecord(s.done_f, s_run);
        cudaStreamWaitEvent(s_run, s.ready_b, 0);
        if (!refused && zt_attn_backward_batched_kept(s.q, s.k, s.v, s.out, s.lse, s.dout, s.dq, s.dk, s.dv, s.delta,
                                                      s.ws, ws_bytes_, 1, c_t, c_heads, c_kv_heads, c_dim,
                                                      reinterpret_cast<zt_stream_t>(s_run), token))
            refused = true;
        cudaEventRecord(s.done, s_run);

        cudaStreamWaitEvent(s_out, s.done_f, 0);
        copy(out + b * qf, s.out, qh_, cudaMemcpyDeviceToHost, s_out);
        if (lse) copy(lse + b * pf, s.lse, pr_, cudaMemcpyDeviceToHost, s_out);
        cudaStreamWaitEvent(s_out, s.done, 0);
        copy(dq + b * qf, s.dq, qh_, cudaMemcpyDeviceToHost, s_out);
        copy(dk + b * kf, s.dk, kvh_, cudaMemcpyDeviceToHost, s_out);
        copy(dv + b * kf, s.dv, kvh_, cudaMemcpyDeviceToHost, s_out);
        cudaEventRecord(s.free_, s_out);
    }
    const bool sync_ok = cudaStreamSynchronize(s_in) == cudaSuccess && cudaStreamSynchronize(s_run) == cudaSuccess &&
                         cudaStreamSynchronize(s_out) == cudaSuccess;
    if (refused) return Error::ConfigRefused;
    if (failed || !sync_ok) {
        cudaGetLastError();
        return Error::DeviceTransferFailed;
    }
    return Error::Ok;
}

}  // namespace device
}  // namespace zt

// ---- C shim (for tests and other foreign-function callers); error codes are Error's values -------------
using zt::device::Attn;
using zt::device::Error;
using zt::device::Kind;

extern "C" {
int zth_bytes_for(int kind, uint64_t t, uint64_t n_heads, uint64_t n_kv_heads, uint64_t dim, uint64_t *bytes) {
    return (int)zt::device::bytesFor((Kind)kind, t, n_heads, n_kv_heads, dim, bytes);
}
int zth_to_c_int(uint64_t x, int *out) { return (int)zt::device::toCInt(x, out); }
int zth_forward_bounds(int c_t, int q_offset, int n_keys, int t) { return (int)zt::device::forwardBounds(c_t, q_offset, n_keys, t); }
int zth_attn_init(uint64_t t, uint64_t n_heads, uint64_t n_kv_heads, uint64_t dim, void **handle) {
    Attn *a = new Attn();
    const Error e = a->init(t, n_heads, n_kv_heads, dim);
    if (e != Error::Ok) {
        delete a;
        *handle = nullptr;
        return (int)e;
    }
    *handle = a;
    return 0;
}
void zth_attn_deinit(void *handle) { delete static_cast<Attn *>(handle); }
uint64_t zth_attn_total_bytes(const void *handle) { return static_cast<const Attn *>(handle)->totalBytes(); }
float *zth_attn_field(const void *handle, int i) { return static_cast<const Attn *>(handle)->field(i); }
int zth_attn_forward(const void *handle, int group_q, int max_tile) { return (int)static_cast<const Attn *>(handle)->forward(group_q, max_tile); }
int zth_attn_forward_at(const void *handle, int group_q, int max_tile, int q_offset, int n_keys, int t) {
    return (int)static_cast<const Attn *>(handle)->forwardAt(group_q, max_tile, q_offset, n_keys, t);
}
int zth_attn_backward(const void *handle, int max_tile) { return (int)static_cast<const Attn *>(handle)->backward(max_tile); }
int zth_attn_upload(const void *handle, float *dst, const float *src, uint64_t n) { return (int)static_cast<const Attn *>(handle)->upload(dst, src, n); }
int zth_attn_download(const void *handle, float *dst, uint64_t n, const float *src) { return (int)static_cast<const Attn *>(handle)->download(dst, n, src); }

int zth_pipeline_init(uint64_t t, uint64_t n_heads, uint64_t n_kv_heads, uint64_t dim, int slots, void **handle) {
    zt::device::AttnPipeline *p = new zt::device::AttnPipeline();
    const Error e = p->init(t, n_heads, n_kv_heads, dim, slots);
    if (e != Error::Ok) {
        delete p;
        *handle = nullptr;
        return (int)e;
    }
    *handle = p;
    return 0;
}
void zth_pipeline_deinit(void *handle) { delete static_cast<zt::device::AttnPipeline *>(handle); }
int zth_pipeline_step(void *handle, int batch, const float *q, const float *k, const float *v, const float *dout,
                      float *out, float *dq, float *dk, float *dv, float *lse) {
    return (int)static_cast<zt::device::AttnPipeline *>(handle)->step(batch, q, k, v, dout, out, dq, dk, dv, lse);
}
}
