// BitNet b1.58 weight path: tensor-wise abs-mean scale, ternary quantize, 2-bit pack / unpack.
//
// Arithmetic follows the reference project (subclasses/bitnet.py):
//   scale = mean(|w|) in fp32                                   (get_bitnet_scale, :110-112)
//   q     = clip(round_half_even(w / max(scale, eps)), -1, 1)   (quantize_bitnet_weight, :115-118)
//   pack  = four 2-bit two's-complement values per byte, first value in the top bits (:185-195)
#include "common.cuh"

namespace qt {

namespace {

constexpr int kThreads = 256;
constexpr int kMaxPartials = 1024;

template <typename XT>
__device__ __forceinline__ float ldf(const XT* p, int64_t i);
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <>
__device__ __forceinline__ float ldf<float>(const float* p, int64_t i) { return p[i]; }

// Stage 1: each CTA sums |x| over a grid-strided slice (fp32 per thread, fp64 across the CTA).
template <typename XT>
__global__ void __launch_bounds__(kThreads) abs_sum_partial_kernel(const XT* __restrict__ x, int64_t n, double* __restrict__ partials) {
    __shared__ double s_red[kThreads / 32];
    float acc = 0.0f;
    const int64_t n8 = n / 8;
    if constexpr (sizeof(XT) == 2) {
        for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < n8; v += (int64_t)gridDim.x * kThreads) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + v * 8);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
            float part = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) part += fabsf(__uint_as_float(w[k] << 16)) + fabsf(__uint_as_float(w[k] & 0xFFFF0000u));
            acc += part;
        }
        for (int64_t i = n8 * 8 + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads)
            acc += fabsf(ldf<XT>(x, i));
    } else {
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads)
            acc += fabsf(ldf<XT>(x, i));
    }
    double d = (double)acc;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = d;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < kThreads / 32; ++w) t += s_red[w];
        partials[blockIdx.x] = t;
    }
}

// Stage 2: one warp folds the partials in a fixed order and writes the fp32 mean.
__global__ void abs_mean_final_kernel(const double* __restrict__ partials, int n_partials, int64_t n, float* __restrict__ out) {
    double t = 0.0;
    for (int i = threadIdx.x; i < n_partials; i += 32) t += partials[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
    if (threadIdx.x == 0) out[0] = (float)(t / (double)n);
}

template <typename XT>
__global__ void __launch_bounds__(kThreads) ternary_kernel(const XT* __restrict__ w, int64_t n, const float* __restrict__ scale,
                                                            float eps, int8_t* __restrict__ out, int pack) {
    const float d = fmaxf(scale[0], eps);
    const int64_t n4 = n / 4;
    for (int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x; q < n4; q += (int64_t)gridDim.x * kThreads) {
        int v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float r = rintf(__fdiv_rn(ldf<XT>(w, q * 4 + k), d));
            r = fminf(fmaxf(r, -1.0f), 1.0f);
            v[k] = (int)r;
        }
        if (pack) {
            out[q] = (int8_t)(((v[0] & 3) << 6) | ((v[1] & 3) << 4) | ((v[2] & 3) << 2) | (v[3] & 3));
        } else {
            const uint32_t word = (uint32_t)(v[0] & 0xFF) | ((uint32_t)(v[1] & 0xFF) << 8) | ((uint32_t)(v[2] & 0xFF) << 16) |
                                  ((uint32_t)(v[3] & 0xFF) << 24);
            *reinterpret_cast<uint32_t*>(out + q * 4) = word;
        }
    }
    if (!pack) {
        for (int64_t i = n4 * 4 + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads) {
            float r = rintf(__fdiv_rn(ldf<XT>(w, i), d));
            out[i] = (int8_t)fminf(fmaxf(r, -1.0f), 1.0f);
        }
    }
}

// The same quantization for bf16 weights without a division per element. clip(round_half_even(w / d), -1, 1)
// is sign(w) when fl(|w| / d) > 0.5 and 0 otherwise, and fl(|w| / d) > 0.5 exactly when |w| > d / 2: d / 2 is
// exact, the next float above it already divides to more than 0.5 + 2^-25 (which rounds up), and rounding is
// monotonic. A bf16 |w| exceeds the fp32 value d / 2 exactly when its 15 magnitude bits exceed the upper 16
// bits of d / 2, so one packed bf16 comparison per two weights decides everything. Requires d >= 2^-100.
// A thread takes 16 weights (two 16-byte loads) and writes 4 packed bytes, or 16 int8 values.
__global__ void __launch_bounds__(kThreads) ternary_bf16_kernel(const __nv_bfloat16* __restrict__ w, int64_t n, const float* __restrict__ scale,
                                                                 float eps, int8_t* __restrict__ out, int pack) {
    const float half_d = 0.5f * fmaxf(scale[0], eps);
    const uint32_t t16 = __float_as_uint(half_d) >> 16;
    const uint32_t thr = t16 | (t16 << 16);
    const __nv_bfloat162 thr2 = *reinterpret_cast<const __nv_bfloat162*>(&thr);
    const int64_t n16 = n / 16;
    for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < n16; v += (int64_t)gridDim.x * kThreads) {
        const uint4 a = reinterpret_cast<const uint4*>(w)[2 * v], b = reinterpret_cast<const uint4*>(w)[2 * v + 1];
        const uint32_t words[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t code[8];   // per word: 2-bit code (0, 1 = +1, 3 = -1) of the low half in bits 0-1, of the high half in bits 16-17
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t mag = words[k] & 0x7FFF7FFFu;
            const uint32_t nz = __hgt2_mask(*reinterpret_cast<const __nv_bfloat162*>(&mag), thr2);
            code[k] = nz & (((words[k] >> 14) & 0x00020002u) | 0x00010001u);
        }
        if (pack) {
            uint32_t bytes = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {   // byte j holds weights 4j .. 4j+3, the first in the top bits
                const uint32_t c0 = code[2 * j], c1 = code[2 * j + 1];
                const uint32_t byte = (((c0 << 6) | (c0 >> 12)) & 0xF0u) | (((c1 << 2) | (c1 >> 16)) & 0x0Fu);
                bytes |= byte << (8 * j);
            }
            reinterpret_cast<uint32_t*>(out)[v] = bytes;
        } else {
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // 2-bit two's complement -> int8: 0 -> 0x00, 1 -> 0x01, 3 -> 0xFF
                const uint32_t c0 = code[2 * j], c1 = code[2 * j + 1];
                const uint32_t e0 = c0 & 3u, e1 = (c0 >> 16) & 3u, e2 = c1 & 3u, e3 = (c1 >> 16) & 3u;
                o[j] = ((e0 ^ 2u) - 2u & 0xFFu) | (((e1 ^ 2u) - 2u & 0xFFu) << 8) | (((e2 ^ 2u) - 2u & 0xFFu) << 16) | (((e3 ^ 2u) - 2u & 0xFFu) << 24);
            }
            reinterpret_cast<uint4*>(out)[v] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

__global__ void __launch_bounds__(kThreads) unpack_i2_kernel(const int8_t* __restrict__ packed, int64_t n_packed, int8_t* __restrict__ out) {
    for (int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x; q < n_packed; q += (int64_t)gridDim.x * kThreads) {
        const int b = (int)packed[q];  // sign-extended
        // arithmetic shifts sign-extend each 2-bit field
        const int v0 = b >> 6;
        const int v1 = ((int)(int8_t)(b << 2)) >> 6;
        const int v2 = ((int)(int8_t)(b << 4)) >> 6;
        const int v3 = ((int)(int8_t)(b << 6)) >> 6;
        const uint32_t word = (uint32_t)(v0 & 0xFF) | ((uint32_t)(v1 & 0xFF) << 8) | ((uint32_t)(v2 & 0xFF) << 16) | ((uint32_t)(v3 & 0xFF) << 24);
        *reinterpret_cast<uint32_t*>(out + q * 4) = word;
    }
}

int grid_for(int64_t work_items) {
    const int64_t want = (work_items + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)num_sms() * 8;
    const int64_t g = want < cap ? want : cap;
    return (int)(g < 1 ? 1 : g);
}

}  // namespace

}  // namespace qt

using namespace qt;

extern "C" int qt_abs_mean(const void* x, int x_dtype, int64_t numel, float* out, void* workspace, int64_t workspace_bytes,
                           void* stream_) {
    QT_REQUIRE(x_dtype == QT_BF16 || x_dtype == QT_F32, "abs_mean: x_dtype must be QT_BF16 or QT_F32 (got %d)", x_dtype);
    QT_REQUIRE(numel > 0, "abs_mean: empty input");
    QT_REQUIRE(x && out && workspace, "abs_mean: null pointer");
    QT_REQUIRE(workspace_bytes >= (int64_t)(kMaxPartials * sizeof(double)), "abs_mean: workspace must hold %d bytes", (int)(kMaxPartials * sizeof(double)));
    QT_REQUIRE(aligned_to(x, 16) && aligned_to(workspace, 8), "abs_mean: x must be 16-byte and workspace 8-byte aligned");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    int grid = grid_for(numel / 8 + 1);
    if (grid > kMaxPartials) grid = kMaxPartials;
    double* partials = reinterpret_cast<double*>(workspace);
    if (x_dtype == QT_BF16) abs_sum_partial_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), numel, partials);
    else abs_sum_partial_kernel<float><<<grid, kThreads, 0, stream>>>(reinterpret_cast<const float*>(x), numel, partials);
    QT_CUDA_CHECK(cudaGetLastError());
    abs_mean_final_kernel<<<1, 32, 0, stream>>>(partials, grid, numel, out);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

extern "C" int qt_bitnet_quantize_weight(const void* w, int w_dtype, int64_t numel, const float* scale, float eps, void* out,
                                         int pack_2bit, void* stream_) {
    QT_REQUIRE(w_dtype == QT_BF16 || w_dtype == QT_F32, "bitnet_quantize_weight: w_dtype must be QT_BF16 or QT_F32 (got %d)", w_dtype);
    QT_REQUIRE(numel >= 0, "bitnet_quantize_weight: negative numel");
    if (numel == 0) return QT_OK;
    QT_REQUIRE(w && scale && out, "bitnet_quantize_weight: null pointer");
    QT_REQUIRE(!pack_2bit || numel % 4 == 0, "bitnet_quantize_weight: packing needs a multiple of 4 elements");
    QT_REQUIRE(aligned_to(out, 4), "bitnet_quantize_weight: output must be 4-byte aligned");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (w_dtype == QT_BF16 && aligned_to(w, 16) && aligned_to(out, 16) && numel >= 16 && eps >= 1e-30f) {
        // whole groups of 16 weights by the comparison kernel, the ragged tail (fewer than 16) by the dividing one
        const int64_t body = numel / 16 * 16;
        ternary_bf16_kernel<<<grid_for(body / 16), kThreads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(w), body, scale, eps,
                                                                        reinterpret_cast<int8_t*>(out), pack_2bit);
        QT_CUDA_CHECK(cudaGetLastError());
        if (body == numel) return QT_OK;
        const int64_t rest = numel - body;
        ternary_kernel<__nv_bfloat16><<<1, kThreads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(w) + body, rest, scale, eps,
                                                                  reinterpret_cast<int8_t*>(out) + (pack_2bit ? body / 4 : body), pack_2bit);
        QT_CUDA_CHECK(cudaGetLastError());
        return QT_OK;
    }
    const int grid = grid_for(numel / 4 + 1);
    if (w_dtype == QT_BF16) ternary_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(w), numel, scale, eps, reinterpret_cast<int8_t*>(out), pack_2bit);
    else ternary_kernel<float><<<grid, kThreads, 0, stream>>>(reinterpret_cast<const float*>(w), numel, scale, eps, reinterpret_cast<int8_t*>(out), pack_2bit);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

extern "C" int qt_unpack_i2(const void* packed, int64_t numel_packed, void* out, void* stream_) {
    QT_REQUIRE(numel_packed >= 0, "unpack_i2: negative numel");
    if (numel_packed == 0) return QT_OK;
    QT_REQUIRE(packed && out && aligned_to(out, 4), "unpack_i2: null or misaligned pointer");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    unpack_i2_kernel<<<grid_for(numel_packed), kThreads, 0, stream>>>(reinterpret_cast<const int8_t*>(packed), numel_packed, reinterpret_cast<int8_t*>(out));
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}
