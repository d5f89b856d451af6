// Shared host/device helpers of libztattn: refusal reporting, launch accounting,
// per-device facts.  Nothing here computes attention.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace zt {

// ---- refusals --------------------------------------------------------------
// The reference prints a reason to stderr and returns 1
// (src/cuda/attn_kernels.cu:21-37).  The same, plus a per-thread copy of the text.
inline thread_local char g_last_error[768] = "";
inline thread_local const char *g_last_path = "none";
inline std::atomic<int> g_verbose{1};
inline std::atomic<int> g_path{0};
inline std::atomic<unsigned long long> g_launches{0};

inline int refuse(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    if (g_verbose.load(std::memory_order_relaxed)) fprintf(stderr, "zt_attn: %s\n", g_last_error);
    return 1;
}

// Checked after every launch, as the reference does between its two backward
// kernels (src/cuda/attn_kernels.cu:1025-1034): a failed launch is a refusal,
// never a dead process, and the error is cleared so a later call cannot inherit it.
inline int launch_failed(const char *what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return 0;
    }
    return refuse("%s failed: %s", what, cudaGetErrorString(e));
}

// ---- optional per-kernel timing ------------------------------------------------
// When switched on (zt_attn_profile), every launch is bracketed by two CUDA events on
// the launching stream; zt_attn_profile_read waits for them and reports, per kernel
// name, the launches and the summed device time.  Off by default: no events exist.
struct ProfEntry {
    const char *name;
    cudaEvent_t start, stop;
};
inline std::atomic<int> g_profile{0};
inline std::mutex g_prof_mu;
inline std::vector<ProfEntry> g_prof;

inline int prof_begin(cudaStream_t stream) {
    if (!g_profile.load(std::memory_order_relaxed)) return -1;
    ProfEntry e{nullptr, nullptr, nullptr};
    if (cudaEventCreate(&e.start) != cudaSuccess || cudaEventCreate(&e.stop) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    cudaEventRecord(e.start, stream);
    std::lock_guard<std::mutex> lock(g_prof_mu);
    g_prof.push_back(e);
    return (int)g_prof.size() - 1;
}

inline void prof_end(int idx, const char *name, cudaStream_t stream) {
    if (idx < 0) return;
    std::lock_guard<std::mutex> lock(g_prof_mu);
    if (idx >= (int)g_prof.size()) return;
    g_prof[idx].name = name;
    cudaEventRecord(g_prof[idx].stop, stream);
}

// Launch `...` (a <<<>>> statement), time it when profiling is on, and turn a failed
// launch into a refusal.  Evaluates to 0 on success, 1 on failure.
#define ZT_LAUNCH(name, stream, ...)                          \
    ([&]() -> int {                                           \
        const int zt_pi_ = ::zt::prof_begin(stream);          \
        __VA_ARGS__;                                          \
        ::zt::prof_end(zt_pi_, name, stream);                 \
        return ::zt::launch_failed(name " launch");           \
    }())

// ---- per-device facts, asked once per device --------------------------------
struct DeviceInfo {
    int known = 0;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    size_t smem_optin = 0;
};

inline const DeviceInfo *device_info() {
    static DeviceInfo table[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return nullptr;
    }
    DeviceInfo &d = table[dev];
    if (d.known) return &d;
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
    d.sm_count = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
        return nullptr;
    d.smem_optin = (size_t)v;
    cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
    d.known = 1;
    return &d;
}

// Opt a kernel into more than 48 KiB of dynamic shared memory; a refusal, not an exit
// (src/cuda/attn_kernels.cu:822-830).
inline int optin_smem(const void *fn, size_t bytes) {
    if (bytes <= 48u * 1024u) return 0;
    const cudaError_t e =
        cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) return 0;
    return refuse("the device would not grant %zu bytes of shared memory per block: %s", bytes,
                  cudaGetErrorString(e));
}

// ---- in-kernel negative controls (the harness build only) ---------------------------------------
// The reference compiles defects into its kernels as template variants and requires its parity gates
// to catch every one of them (src/cuda/attn_kernels.cu:150-158,592-599,622-624; src/cuda/run-attn.sh:126-177).
// The same here, for the defects that live INSIDE a kernel: built with -DZT_DEFECTS the kernels consult a
// device word that zt_attn_set_defect writes; every defect computes wrong numbers from valid addresses.
//   1  the causal mask is dropped in the forward (a query reads the keys after it in its diagonal tiles)
//   3  the forward's running-maximum correction is skipped (sum and accumulator are never rescaled)
//   11 the causal mask is dropped in the backward
//   13 the softmax Jacobian is dropped in the backward (dS = P dP)
// The shipped library is built without the macro: ZT_DEFECT(n) is then the constant false and no kernel
// carries a switch.
#ifdef ZT_DEFECTS
static __device__ int g_defect;
#define ZT_DEFECT(n) (g_defect == (n))
#else
#define ZT_DEFECT(n) false
#endif

// Copies of an output tensor in other GPUs' memory (peer device pointers, mapped into this process): a kernel that
// is given them stores every output element there as well as locally, so the all-gather of that output happens
// inside the kernel, element by element over NVLink, instead of as a collective after it.
constexpr int kMaxPeers = 7;
struct PeerList {
    float *ptr[kMaxPeers];
    int n;
};

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace zt
