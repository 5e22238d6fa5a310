// AdamW with bf16 optimizer states and a stochastically rounded bf16 weight write-back, one fused
// HBM pass per parameter tensor (14 bytes per bf16 parameter: read p, g, m, v; write p, m, v).
//
// Arithmetic follows `adamw` of the reference project (other_optim/bf16_sr.py:78-124), evaluated
// op by op in fp32 the way its eager form does:
//   m' = lerp(m, g, 1-beta1) ; v' = lerp(v, g*g, 1-beta2)          (lerp = one fused multiply-add)
//   denom = sqrt(v') / sqrt(bc2) + eps ; numer = m' / bc1
//   p' = (p - (lr*wd) * p) - (lr * numer) / denom
//   bf16 weights: bits(p') + 16 random bits, low 16 bits dropped     (bf16_sr.py:108-122)
// The bias corrections bc1, bc2 and sqrt(bc2) are computed by the caller (they are scalars).
#include "common.cuh"

namespace qt {

namespace {

constexpr int kThreads = 256;

struct AdamParams {
    void* p;
    const void* g;
    __nv_bfloat16* m;
    __nv_bfloat16* v;
    int64_t n;
    float lr_wd, lr, w1, w2, bc1, sqrt_bc2, eps;
    int stochastic;
    uint64_t seed, offset;
    PhiloxKeys keys;   // round keys of `seed`
    int vec;  // p and g are 16-byte, m and v 8-byte aligned: four elements move as one vector
};

template <typename T>
__device__ __forceinline__ float ld(const T* p, int64_t i);
template <>
__device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <>
__device__ __forceinline__ float ld<float>(const float* p, int64_t i) { return p[i]; }

__device__ __forceinline__ float lerp_fma(float a, float b, float w) {
    const float diff = __fsub_rn(b, a);
    return fabsf(w) < 0.5f ? __fmaf_rn(w, diff, a) : __fmaf_rn(-diff, __fsub_rn(1.0f, w), b);
}

// One element. Returns the fp32 updated weight; writes m, v through references.
__device__ __forceinline__ float adam_update(float p, float g, float& m, float& v, const AdamParams& a) {
    m = lerp_fma(m, g, a.w1);
    v = lerp_fma(v, __fmul_rn(g, g), a.w2);
    const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(v), a.sqrt_bc2), a.eps);
    const float numer = __fdiv_rn(m, a.bc1);
    const float decayed = __fsub_rn(p, __fmul_rn(a.lr_wd, p));
    return __fsub_rn(decayed, __fdiv_rn(__fmul_rn(a.lr, numer), denom));
}

__device__ __forceinline__ uint32_t sr_bf16_bits(float x, uint32_t rand16) {
    return (__float_as_uint(x) + (rand16 & 0xFFFFu)) >> 16;
}

// Elements [4q, 4q+4) of one tensor (fewer at the tail). The tensor's pointers and length are in `a`.
template <typename PT, typename GT>
__device__ __forceinline__ void adam_quad(const AdamParams& a, int64_t q) {
    PT* p = reinterpret_cast<PT*>(a.p);
    const GT* g = reinterpret_cast<const GT*>(a.g);
    {
        const int64_t i0 = q * 4;
        Philox4 r = {0, 0, 0, 0};
        if (a.stochastic) r = philox4x32_10((uint64_t)q, a.offset, a.keys);
        const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
        if (a.vec && i0 + 4 <= a.n) {
            float pv[4], gv[4], mv[4], vv[4];
            // 4 consecutive elements: 8-byte (bf16) or 16-byte (fp32) accesses (the host checked the
            // alignment of this tensor; views at odd offsets take the element path below)
            if constexpr (sizeof(PT) == 2) {
                const uint2 raw = *reinterpret_cast<const uint2*>(p + i0);
                pv[0] = __uint_as_float(raw.x << 16); pv[1] = __uint_as_float(raw.x & 0xFFFF0000u);
                pv[2] = __uint_as_float(raw.y << 16); pv[3] = __uint_as_float(raw.y & 0xFFFF0000u);
            } else {
                const float4 raw = *reinterpret_cast<const float4*>(p + i0);
                pv[0] = raw.x; pv[1] = raw.y; pv[2] = raw.z; pv[3] = raw.w;
            }
            if constexpr (sizeof(GT) == 2) {
                const uint2 raw = *reinterpret_cast<const uint2*>(g + i0);
                gv[0] = __uint_as_float(raw.x << 16); gv[1] = __uint_as_float(raw.x & 0xFFFF0000u);
                gv[2] = __uint_as_float(raw.y << 16); gv[3] = __uint_as_float(raw.y & 0xFFFF0000u);
            } else {
                const float4 raw = *reinterpret_cast<const float4*>(g + i0);
                gv[0] = raw.x; gv[1] = raw.y; gv[2] = raw.z; gv[3] = raw.w;
            }
            {
                const uint2 rm = *reinterpret_cast<const uint2*>(a.m + i0);
                const uint2 rv = *reinterpret_cast<const uint2*>(a.v + i0);
                mv[0] = __uint_as_float(rm.x << 16); mv[1] = __uint_as_float(rm.x & 0xFFFF0000u);
                mv[2] = __uint_as_float(rm.y << 16); mv[3] = __uint_as_float(rm.y & 0xFFFF0000u);
                vv[0] = __uint_as_float(rv.x << 16); vv[1] = __uint_as_float(rv.x & 0xFFFF0000u);
                vv[2] = __uint_as_float(rv.y << 16); vv[3] = __uint_as_float(rv.y & 0xFFFF0000u);
            }
            float np[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) np[k] = adam_update(pv[k], gv[k], mv[k], vv[k], a);
            uint2 om, ov;
            {
                const __nv_bfloat162 m01 = __floats2bfloat162_rn(mv[0], mv[1]), m23 = __floats2bfloat162_rn(mv[2], mv[3]);
                const __nv_bfloat162 v01 = __floats2bfloat162_rn(vv[0], vv[1]), v23 = __floats2bfloat162_rn(vv[2], vv[3]);
                om.x = *reinterpret_cast<const uint32_t*>(&m01); om.y = *reinterpret_cast<const uint32_t*>(&m23);
                ov.x = *reinterpret_cast<const uint32_t*>(&v01); ov.y = *reinterpret_cast<const uint32_t*>(&v23);
            }
            *reinterpret_cast<uint2*>(a.m + i0) = om;
            *reinterpret_cast<uint2*>(a.v + i0) = ov;
            if constexpr (sizeof(PT) == 2) {
                uint32_t b[4];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    b[k] = a.stochastic ? sr_bf16_bits(np[k], rw[k]) : (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(np[k]));
                *reinterpret_cast<uint2*>(p + i0) = make_uint2((b[0] & 0xFFFFu) | (b[1] << 16), (b[2] & 0xFFFFu) | (b[3] << 16));
            } else {
                *reinterpret_cast<float4*>(p + i0) = make_float4(np[0], np[1], np[2], np[3]);
            }
        } else {
            for (int k = 0; k < 4 && i0 + k < a.n; ++k) {
                const int64_t i = i0 + k;
                float m = __bfloat162float(a.m[i]), v = __bfloat162float(a.v[i]);
                const float np = adam_update(ld<PT>(p, i), ld<GT>(g, i), m, v, a);
                a.m[i] = __float2bfloat16_rn(m);
                a.v[i] = __float2bfloat16_rn(v);
                if constexpr (sizeof(PT) == 2) {
                    const uint32_t b = a.stochastic ? sr_bf16_bits(np, rw[k]) : (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(np));
                    p[i] = __ushort_as_bfloat16((unsigned short)(b & 0xFFFFu));
                } else {
                    p[i] = np;
                }
            }
        }
    }
}

template <typename PT, typename GT>
__global__ void __launch_bounds__(kThreads) adamw_kernel(const AdamParams a) {
    const int64_t n4 = (a.n + 3) / 4;
    for (int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x; q < n4; q += (int64_t)gridDim.x * kThreads)
        adam_quad<PT, GT>(a, q);
}

// ---- multi-tensor form: one launch updates many parameter tensors ---------------------------------
// A launch carries a table of up to kMaxTensors tensors; the grid is the total number of kChunk-element
// chunks of all of them, and a block finds its tensor by bisecting the running chunk count. Tensor t
// draws its random bits with Philox offset `offset + t`, i.e. exactly what a single-tensor call with
// that offset draws.

constexpr int kMaxTensors = 160;
constexpr int kChunk = 8192;   // elements per block: 8 quads per thread

struct MultiTable {
    void* p[kMaxTensors];
    const void* g[kMaxTensors];
    __nv_bfloat16* m[kMaxTensors];
    __nv_bfloat16* v[kMaxTensors];
    int64_t numel[kMaxTensors];
    uint32_t tensor_index[kMaxTensors];
    uint8_t vec[kMaxTensors];
    uint32_t chunk_begin[kMaxTensors + 1];   // first block of each tensor; [n] = grid size
    int n;
};

template <typename PT, typename GT>
__global__ void __launch_bounds__(kThreads) adamw_multi_kernel(const __grid_constant__ MultiTable tab, const AdamParams proto) {
    int lo = 0, hi = tab.n;   // the tensor t with chunk_begin[t] <= blockIdx.x < chunk_begin[t + 1]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tab.chunk_begin[mid] <= blockIdx.x) lo = mid; else hi = mid;
    }
    const int t = lo;
    AdamParams a = proto;
    a.p = tab.p[t]; a.g = tab.g[t]; a.m = tab.m[t]; a.v = tab.v[t]; a.n = tab.numel[t];
    a.offset = proto.offset + tab.tensor_index[t];
    a.vec = tab.vec[t];
    const int64_t q_begin = (int64_t)(blockIdx.x - tab.chunk_begin[t]) * (kChunk / 4);
    const int64_t n4 = (a.n + 3) / 4;
    const int64_t q_end = q_begin + kChunk / 4 < n4 ? q_begin + kChunk / 4 : n4;
    for (int64_t q = q_begin + threadIdx.x; q < q_end; q += kThreads) adam_quad<PT, GT>(a, q);
}

}  // namespace

}  // namespace qt

using namespace qt;

extern "C" int qt_adamw_bf16_sr(void* p, int p_dtype, const void* grad, int grad_dtype, void* exp_avg, void* exp_avg_sq,
                                int64_t numel, float lr, double beta1, double beta2, float weight_decay, float eps,
                                float bias_correction1, float sqrt_bias_correction2, int stochastic, uint64_t seed,
                                uint64_t offset, void* stream_) {
    QT_REQUIRE(p_dtype == QT_BF16 || p_dtype == QT_F32, "adamw: parameter dtype must be QT_BF16 or QT_F32 (got %d)", p_dtype);
    QT_REQUIRE(grad_dtype == QT_BF16 || grad_dtype == QT_F32, "adamw: gradient dtype must be QT_BF16 or QT_F32 (got %d)", grad_dtype);
    QT_REQUIRE(numel >= 0, "adamw: negative numel");
    QT_REQUIRE(!stochastic || p_dtype == QT_BF16, "adamw: stochastic rounding applies to bf16 parameters only");
    if (numel == 0) return QT_OK;
    QT_REQUIRE(p && grad && exp_avg && exp_avg_sq, "adamw: null pointer");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    AdamParams a;
    a.p = p; a.g = grad; a.m = reinterpret_cast<__nv_bfloat16*>(exp_avg); a.v = reinterpret_cast<__nv_bfloat16*>(exp_avg_sq);
    a.n = numel;
    a.lr = lr; a.lr_wd = lr * weight_decay;  // fp32 product, as `lr * weight_decay` on an fp32 lr tensor
    // lerp weights: the Python doubles (1 - beta) rounded to fp32, as ATen does for an fp32 tensor
    a.w1 = (float)(1.0 - beta1); a.w2 = (float)(1.0 - beta2);
    a.bc1 = bias_correction1; a.sqrt_bc2 = sqrt_bias_correction2; a.eps = eps;
    a.stochastic = stochastic; a.seed = seed; a.offset = offset; a.keys = philox_keys(seed);
    a.vec = aligned_to(p, 16) && aligned_to(grad, 16) && aligned_to(exp_avg, 8) && aligned_to(exp_avg_sq, 8);
    const int64_t want = ((numel + 3) / 4 + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)num_sms() * 16;
    const int grid = (int)(want < cap ? want : cap);
    if (p_dtype == QT_BF16 && grad_dtype == QT_BF16) adamw_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kThreads, 0, stream>>>(a);
    else if (p_dtype == QT_BF16) adamw_kernel<__nv_bfloat16, float><<<grid, kThreads, 0, stream>>>(a);
    else if (grad_dtype == QT_BF16) adamw_kernel<float, __nv_bfloat16><<<grid, kThreads, 0, stream>>>(a);
    else adamw_kernel<float, float><<<grid, kThreads, 0, stream>>>(a);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

extern "C" int qt_adamw_bf16_sr_multi(int n_tensors, void* const* p, const void* const* grad, void* const* exp_avg,
                                      void* const* exp_avg_sq, const int64_t* numel, int p_dtype, int grad_dtype, float lr,
                                      double beta1, double beta2, float weight_decay, float eps, float bias_correction1,
                                      float sqrt_bias_correction2, int stochastic, uint64_t seed, uint64_t offset,
                                      void* stream_) {
    QT_REQUIRE(n_tensors >= 0, "adamw_multi: negative tensor count");
    QT_REQUIRE(p_dtype == QT_BF16 || p_dtype == QT_F32, "adamw_multi: parameter dtype must be QT_BF16 or QT_F32 (got %d)", p_dtype);
    QT_REQUIRE(grad_dtype == QT_BF16 || grad_dtype == QT_F32, "adamw_multi: gradient dtype must be QT_BF16 or QT_F32 (got %d)", grad_dtype);
    QT_REQUIRE(!stochastic || p_dtype == QT_BF16, "adamw_multi: stochastic rounding applies to bf16 parameters only");
    if (n_tensors == 0) return QT_OK;
    QT_REQUIRE(p && grad && exp_avg && exp_avg_sq && numel, "adamw_multi: null table");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    AdamParams a = {};
    a.lr = lr; a.lr_wd = lr * weight_decay;
    a.w1 = (float)(1.0 - beta1); a.w2 = (float)(1.0 - beta2);
    a.bc1 = bias_correction1; a.sqrt_bc2 = sqrt_bias_correction2; a.eps = eps;
    a.stochastic = stochastic; a.seed = seed; a.offset = offset; a.keys = philox_keys(seed);

    MultiTable tab;
    tab.n = 0;
    tab.chunk_begin[0] = 0;
    auto flush = [&]() -> int {
        if (tab.n == 0) return QT_OK;
        const unsigned grid = tab.chunk_begin[tab.n];
        if (p_dtype == QT_BF16 && grad_dtype == QT_BF16) adamw_multi_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kThreads, 0, stream>>>(tab, a);
        else if (p_dtype == QT_BF16) adamw_multi_kernel<__nv_bfloat16, float><<<grid, kThreads, 0, stream>>>(tab, a);
        else if (grad_dtype == QT_BF16) adamw_multi_kernel<float, __nv_bfloat16><<<grid, kThreads, 0, stream>>>(tab, a);
        else adamw_multi_kernel<float, float><<<grid, kThreads, 0, stream>>>(tab, a);
        QT_CUDA_CHECK(cudaGetLastError());
        tab.n = 0;
        return QT_OK;
    };
    for (int t = 0; t < n_tensors; ++t) {
        QT_REQUIRE(numel[t] >= 0, "adamw_multi: negative numel for tensor %d", t);
        if (numel[t] == 0) continue;
        QT_REQUIRE(p[t] && grad[t] && exp_avg[t] && exp_avg_sq[t], "adamw_multi: null pointer for tensor %d", t);
        const int64_t chunks = (numel[t] + kChunk - 1) / kChunk;
        QT_REQUIRE(chunks < (1ll << 30), "adamw_multi: tensor %d is too large", t);
        // a launch holds at most kMaxTensors tensors and 2^31 - 1 blocks
        if (tab.n == kMaxTensors || (int64_t)tab.chunk_begin[tab.n] + chunks >= (1ll << 31)) {
            if (int rc = flush()) return rc;
        }
        const int slot = tab.n++;
        tab.p[slot] = p[t]; tab.g[slot] = grad[t];
        tab.m[slot] = reinterpret_cast<__nv_bfloat16*>(exp_avg[t]); tab.v[slot] = reinterpret_cast<__nv_bfloat16*>(exp_avg_sq[t]);
        tab.numel[slot] = numel[t]; tab.tensor_index[slot] = (uint32_t)t;
        tab.vec[slot] = aligned_to(p[t], 16) && aligned_to(grad[t], 16) && aligned_to(exp_avg[t], 8) && aligned_to(exp_avg_sq[t], 8);
        tab.chunk_begin[slot + 1] = tab.chunk_begin[slot] + (uint32_t)chunks;
    }
    return flush();
}
