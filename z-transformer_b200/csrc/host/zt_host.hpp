// C++ mirror of the reference's Zig holder, src/cuda/device.zig: the same names, argument meaning and
// error behaviour, over the same six C entry points (include/zt_attn.h).  Zig is not available where this
// library is built, so the host layer a Zig program would write against `device.Attn` is given here in the
// other compiled language the C ABI serves; `zt_host.cpp` adds a C shim so tests can drive it.
//
//   Error                     device.zig:119-125 (an enum; `Ok` stands for Zig's "no error")
//   Kind, bytesFor, toCInt    device.zig:127-182   pure, checked arithmetic, usable without a GPU
//   forwardBounds             device.zig:489-501
//   Attn                      device.zig:185-432   eleven device buffers of one (t, heads, kv heads, dim)
#pragma once

#include <cstddef>
#include <cstdint>
#include <limits>

namespace zt {
namespace device {

enum class Error { Ok = 0, DegenerateShape, ShapeTooLarge, ConfigRefused, DeviceAllocFailed, DeviceTransferFailed };

enum class Kind { query_headed = 0, kv_headed = 1, per_row = 2 };

// A checked product, as std.math.mul(usize, ...) is: false on overflow.
inline bool mul_usize(uint64_t a, uint64_t b, uint64_t *out) { return !__builtin_mul_overflow(a, b, out); }

// device.bytesFor (device.zig:162-171): DegenerateShape for a zero dimension, ShapeTooLarge on overflow.
inline Error bytesFor(Kind kind, uint64_t t, uint64_t n_heads, uint64_t n_kv_heads, uint64_t dim, uint64_t *bytes) {
    if (t == 0 || dim == 0 || n_heads == 0 || n_kv_heads == 0) return Error::DegenerateShape;
    uint64_t cols = n_heads, elems = 0;
    if (kind == Kind::query_headed && !mul_usize(n_heads, dim, &cols)) return Error::ShapeTooLarge;
    if (kind == Kind::kv_headed && !mul_usize(n_kv_heads, dim, &cols)) return Error::ShapeTooLarge;
    if (!mul_usize(t, cols, &elems)) return Error::ShapeTooLarge;
    if (!mul_usize(elems, sizeof(float), bytes)) return Error::ShapeTooLarge;
    return Error::Ok;
}

// device.toCInt (device.zig:179-182)
inline Error toCInt(uint64_t x, int *out) {
    if (x > (uint64_t)std::numeric_limits<int>::max()) return Error::ShapeTooLarge;
    *out = (int)x;
    return Error::Ok;
}

// device.forwardBounds (device.zig:489-501)
inline Error forwardBounds(int c_t, int q_offset, int n_keys, int t) {
    if (n_keys < 1 || n_keys > c_t) return Error::ShapeTooLarge;
    if (t < 1 || t > c_t) return Error::ShapeTooLarge;
    if (q_offset < 0 || q_offset > c_t || t > c_t - q_offset) return Error::ShapeTooLarge;
    if (q_offset + t > n_keys) return Error::ShapeTooLarge;
    return Error::Ok;
}

class Attn {
public:
    static constexpr int N_BUFFERS = 11;
    // device buffers, in the reference's field order (device.zig:186-196)
    float *q = nullptr, *k = nullptr, *v = nullptr, *out = nullptr, *dout = nullptr;
    float *dq = nullptr, *dk = nullptr, *dv = nullptr, *row_max = nullptr, *row_den = nullptr, *row_del = nullptr;
    uint64_t t = 0, n_heads = 0, n_kv_heads = 0, dim = 0;
    int c_t = 0, c_heads = 0, c_kv_heads = 0, c_dim = 0;

    Attn() = default;
    Attn(const Attn &) = delete;
    Attn &operator=(const Attn &) = delete;
    ~Attn() { deinit(); }

    // device.zig:208-297: every refusal comes before the first allocation; a failed allocation frees
    // the ones before it.
    Error init(uint64_t t, uint64_t n_heads, uint64_t n_kv_heads, uint64_t dim);
    void deinit();
    uint64_t totalBytes() const;
    Error forward(int group_q, int max_tile) const { return forwardAt(group_q, max_tile, 0, c_t, c_t); }
    Error forwardAt(int group_q, int max_tile, int q_offset, int n_keys, int t) const;
    Error backward(int max_tile) const;
    // `dst` / `src` must be one of this holder's buffers; more floats than it holds is ShapeTooLarge
    Error upload(float *dst, const float *src, uint64_t n_floats) const;
    Error download(float *dst, uint64_t n_floats, const float *src) const;
    float *field(int i) const;

private:
    uint64_t bufferBytes(const float *target) const;
    void deinitPartial(int taken);
};

// Forward + backward of a run of equally shaped sequences whose tensors live in (pinned) host memory, with the
// upload of sequence b+1, the kernels of b and the download of b-1 overlapped on three streams over `slots`
// sets of device buffers.  The reference's trainer drives device.Attn one sequence at a time, each step waiting
// for the one before (src/model.zig:481-514); over PCIe the copies take longer than the kernels.  Uses the
// batched entry points (batch 1): the forward keeps its operand planes for the backward and nothing is
// recomputed.  No reference counterpart.
class AttnPipeline {
public:
    AttnPipeline() = default;
    AttnPipeline(const AttnPipeline &) = delete;
    AttnPipeline &operator=(const AttnPipeline &) = delete;
    ~AttnPipeline() { deinit(); }

    Error init(uint64_t t, uint64_t n_heads, uint64_t n_kv_heads, uint64_t dim, int slots);
    void deinit();
    // q, dout, out, dq: host [batch][t][n_heads * dim]; k, v, dk, dv: host [batch][t][n_kv_heads * dim];
    // lse: host [batch][t][n_heads] or null.  Returns when every result is in host memory.
    Error step(int batch, const float *q, const float *k, const float *v, const float *dout, float *out, float *dq,
               float *dk, float *dv, float *lse);

private:
    struct Slot;
    Slot *slot_ = nullptr;
    int slots_ = 0;
    int c_t = 0, c_heads = 0, c_kv_heads = 0, c_dim = 0;
    uint64_t qh_ = 0, kvh_ = 0, pr_ = 0, ws_bytes_ = 0;
    void *s_in_ = nullptr, *s_run_ = nullptr, *s_out_ = nullptr;  // cudaStream_t
};

}  // namespace device
}  // namespace zt
