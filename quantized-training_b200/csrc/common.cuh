// Shared host/device helpers for the sm_100a quantize + GEMM library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/qt_b200.h"

namespace qt {

// ---- host-side error reporting ---------------------------------------------------------------

// Per-thread message buffer behind qt_last_error().
char* last_error_buffer();
constexpr int kErrBufSize = 512;

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), kErrBufSize, fmt, ap);
    va_end(ap);
    return code;
}

#define QT_CUDA_CHECK(expr)                                                                    \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess)                                                                 \
            return ::qt::fail(QT_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                              __FILE__, __LINE__);                                             \
    } while (0)

#define QT_REQUIRE(cond, ...)                                  \
    do {                                                       \
        if (!(cond)) return ::qt::fail(QT_ERR_INVALID, __VA_ARGS__); \
    } while (0)

// Device status word: kernels that give up on a bounded wait store a non-zero code here.
// One word per device, reached through this accessor (address resolved per device).
int device_status_ptr(int** out);
// Host address of the pinned word that mirrors the current device's status (nullptr before first use).
volatile int* device_status_host_word();

inline int num_sms() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---- Philox4x32-10 --------------------------------------------------------------------------
// Counter-based generator (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
// The 128-bit counter is {lo32(c), hi32(c), lo32(offset), hi32(offset)} and the 64-bit key is the
// seed. The quantize kernels give element i 16 bits: counter c = i / 8, word (i % 8) / 2, half i % 2;
// the optimizer gives element i the low 16 bits of word (i % 4) of counter c = i / 4.

struct Philox4 {
    uint32_t x, y, z, w;
};

__host__ __device__ inline Philox4 philox4x32_10(uint64_t ctr, uint64_t offset, uint64_t seed) {
    uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32);
    uint32_t c2 = (uint32_t)offset, c3 = (uint32_t)(offset >> 32);
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        const uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return Philox4{c0, c1, c2, c3};
}

// The ten round keys of a seed, formed once on the host and handed to kernels inside their parameter
// block: a round then reads its keys as constant operands instead of carrying and advancing two registers.
struct PhiloxKeys {
    uint32_t k[20];
};

inline PhiloxKeys philox_keys(uint64_t seed) {
    PhiloxKeys out;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    for (int r = 0; r < 10; ++r) {
        out.k[2 * r] = k0;
        out.k[2 * r + 1] = k1;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return out;
}

// Same generator as philox4x32_10(ctr, offset, seed) with the round keys of `seed` precomputed.
__device__ __forceinline__ Philox4 philox4x32_10(uint64_t ctr, uint64_t offset, const PhiloxKeys& keys) {
    uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32);
    uint32_t c2 = (uint32_t)offset, c3 = (uint32_t)(offset >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ keys.k[2 * r];
        const uint32_t n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ keys.k[2 * r + 1];
        const uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    }
    return Philox4{c0, c1, c2, c3};
}

// ---- store guard (debug build) -----------------------------------------------------------------
// With -DQT_BOUNDS_CHECK every global store of the quantize kernels first checks its address against the
// output ranges the entry point declared for the launch. A store outside them is skipped and its site
// recorded in the device status word (0xB00 | site), which qt_device_status reports; nothing traps. The
// release build compiles the checks away. It covers what a memory checker would on the write side.
#ifdef QT_BOUNDS_CHECK
struct StoreGuard {
    const char* lo[8];
    const char* hi[8];
    int n;          // ranges in use; -1 = unchecked launch (peer destinations)
    int* status;
    void add(const void* p, int64_t bytes) {
        if (p != nullptr && bytes > 0 && n >= 0 && n < 8) { lo[n] = static_cast<const char*>(p); hi[n] = lo[n] + bytes; ++n; }
    }
    __device__ bool ok(const void* p, int bytes, int site) const {
        if (n < 0) return true;
        const char* c = static_cast<const char*>(p);
        for (int i = 0; i < n; ++i)
            if (c >= lo[i] && c + bytes <= hi[i]) return true;
        atomicCAS(status, 0, 0xB00 | site);
        return false;
    }
};
#define QT_GUARD_FIELD ::qt::StoreGuard guard;
#define QT_GUARD_OK(g, ptr, bytes, site) ((g).ok((ptr), (bytes), (site)))
#define QT_GUARD_INIT(g)                                          \
    do {                                                          \
        (g).n = 0;                                                \
        int* st_ = nullptr;                                       \
        if (int rc_ = ::qt::device_status_ptr(&st_)) return rc_;  \
        (g).status = st_;                                         \
    } while (0)
#define QT_GUARD_ADD(g, ptr, bytes) (g).add((ptr), (int64_t)(bytes))
#define QT_GUARD_OFF(g) ((g).n = -1)
#else
#define QT_GUARD_FIELD
#define QT_GUARD_OK(g, ptr, bytes, site) (true)
#define QT_GUARD_INIT(g) ((void)0)
#define QT_GUARD_ADD(g, ptr, bytes) ((void)0)
#define QT_GUARD_OFF(g) ((void)0)
#endif

// ---- device numerics ------------------------------------------------------------------------

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// Round an fp32 scale to the output scale dtype and store it.
__device__ __forceinline__ void store_scale(void* scale, int scale_dtype, int64_t idx, float v) {
    if (scale_dtype == QT_BF16)
        reinterpret_cast<__nv_bfloat16*>(scale)[idx] = __float2bfloat16_rn(v);
    else
        reinterpret_cast<float*>(scale)[idx] = v;
}

#define QT_STORE_SCALE(g, scale, scale_dtype, idx, v, site)                                                                 \
    do {                                                                                                                    \
        if (QT_GUARD_OK(g, static_cast<char*>(scale) + (int64_t)(idx) * ((scale_dtype) == QT_BF16 ? 2 : 4),                   \
                        (scale_dtype) == QT_BF16 ? 2 : 4, site))                                                            \
            ::qt::store_scale(scale, scale_dtype, idx, v);                                                                  \
    } while (0)

// One quantized byte from a pre-divided value v = x / scale.
//   int8: round-half-even (or floor(v + u) when stochastic), clamp [-128, 127]
//   e4m3/e5m2: round-to-nearest-even, saturating to the largest finite value
__device__ __forceinline__ uint32_t quantize_byte(float v, int q_dtype, bool stochastic, float u) {
    if (q_dtype == QT_I8) {
        float r = stochastic ? floorf(__fadd_rn(v, u)) : rintf(v);
        r = fminf(fmaxf(r, -128.0f), 127.0f);
        return (uint32_t)(__float2int_rn(r) & 0xFF);
    } else if (q_dtype == QT_E4M3) {
        return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    } else {
        return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2);
    }
}

__host__ __device__ inline float qmax_of(int q_dtype) {
    return q_dtype == QT_I8 ? 127.0f : (q_dtype == QT_E4M3 ? 448.0f : 57344.0f);
}

}  // namespace qt
