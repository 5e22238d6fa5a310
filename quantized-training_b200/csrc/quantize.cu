// Absmax quantize kernels (HBM-bound): row-wise, row-wise + column absmax, column absmax,
// column-wise with transpose, tile-wise. bf16 / fp32 in; int8 or fp8 out plus one scale per
// row / column / tile.
//
// Arithmetic follows quantize_int8 of the reference project (subclasses/int8.py:12-26):
//   scale = absmax / qmax            (fp32, IEEE division)
//   v     = x / max(scale, eps)      (fp32, IEEE division -- never a reciprocal multiply)
//   q     = clamp(round_half_even(v)) or clamp(floor(v + u)), u ~ U[0,1)
//   the returned scale is the UNCLAMPED scale rounded to the scale dtype.
//
// Division: for bf16 inputs the quotient is produced by a correctly rounded reciprocal plus one
// fused residual correction (3 full-rate ops instead of the ~10 of div.rn). qt_selftest_division
// checks that sequence against div.rn over every (bf16 x, bf16 absmax) pair; fp32 inputs use
// div.rn directly.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace qt {

namespace {

constexpr int kThreads = 256;
constexpr float kRoundMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to integer (half-even)

// ---- 8-element vectors ----------------------------------------------------------------------

template <typename XT>
struct Vec8;

template <>
struct Vec8<__nv_bfloat16> {
    uint4 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void zero() { raw = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ void unpack(float (&f)[8]) const {
        f[0] = __uint_as_float(raw.x << 16); f[1] = __uint_as_float(raw.x & 0xFFFF0000u);
        f[2] = __uint_as_float(raw.y << 16); f[3] = __uint_as_float(raw.y & 0xFFFF0000u);
        f[4] = __uint_as_float(raw.z << 16); f[5] = __uint_as_float(raw.z & 0xFFFF0000u);
        f[6] = __uint_as_float(raw.w << 16); f[7] = __uint_as_float(raw.w & 0xFFFF0000u);
    }
};

template <>
struct Vec8<float> {
    float4 lo, hi;
    __device__ __forceinline__ void load(const float* p) {
        lo = *reinterpret_cast<const float4*>(p);
        hi = *reinterpret_cast<const float4*>(p + 4);
    }
    __device__ __forceinline__ void zero() { lo = make_float4(0, 0, 0, 0); hi = lo; }
    __device__ __forceinline__ void unpack(float (&f)[8]) const {
        f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w;
        f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
    }
};

template <typename XT>
__device__ __forceinline__ float to_float(XT v);
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }

// Load 8 elements starting at column `col` of a row; columns >= cols read as zero.
template <typename XT>
__device__ __forceinline__ void load_vec8(Vec8<XT>& v, const XT* row, int64_t col, int64_t cols, bool vec_ok) {
    if (col + 8 <= cols && vec_ok) {
        v.load(row + col);
    } else {
        float f[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = (col + k < cols) ? to_float<XT>(row[col + k]) : 0.0f;
        // re-pack through the float path (exact for bf16 and fp32 values)
        if constexpr (sizeof(XT) == 2) {
            v.raw.x = (__float_as_uint(f[0]) >> 16) | (__float_as_uint(f[1]) & 0xFFFF0000u);
            v.raw.y = (__float_as_uint(f[2]) >> 16) | (__float_as_uint(f[3]) & 0xFFFF0000u);
            v.raw.z = (__float_as_uint(f[4]) >> 16) | (__float_as_uint(f[5]) & 0xFFFF0000u);
            v.raw.w = (__float_as_uint(f[6]) >> 16) | (__float_as_uint(f[7]) & 0xFFFF0000u);
        } else {
            v.lo = make_float4(f[0], f[1], f[2], f[3]);
            v.hi = make_float4(f[4], f[5], f[6], f[7]);
        }
    }
}

// ---- division -------------------------------------------------------------------------------

__device__ __forceinline__ float recip_rn(float d) { return __frcp_rn(d); }
__device__ __forceinline__ float div_rn(float x, float d) { return __fdiv_rn(x, d); }

// Divider by a fixed positive d. EXACT selects div.rn; otherwise the reciprocal sequence, which
// needs 1/d to be finite and normal: callers guarantee d >= 1e-30 (eps >= 1e-30 is checked on the
// host, smaller eps takes the EXACT instantiation).
template <bool EXACT>
struct Divider {
    float d, r;
    __device__ __forceinline__ explicit Divider(float d_) : d(d_), r(EXACT ? 0.0f : recip_rn(d_)) {}
    __device__ __forceinline__ Divider(float d_, float r_) : d(d_), r(r_) {}
    __device__ __forceinline__ float operator()(float x) const {
        if constexpr (EXACT) {
            return div_rn(x, d);
        } else {
            const float q0 = __fmul_rn(x, r);
            const float e = __fmaf_rn(-q0, d, x);
            return __fmaf_rn(e, r, q0);
        }
    }
};

// The same division for two values at once on the packed fp32x2 instructions of sm_100 (one issue slot
// per pair): q0 = x * r, e = x - q0 * d, q = q0 + e * r, each lane rounded like the scalar sequence.
struct Divider2 {
    float2 r, nd;   // reciprocal and negated divisor per lane
    __device__ __forceinline__ explicit Divider2(float d) {
        const float rr = recip_rn(d);
        r = make_float2(rr, rr);
        nd = make_float2(-d, -d);
    }
    __device__ __forceinline__ Divider2(float d0, float r0, float d1, float r1) : r(make_float2(r0, r1)), nd(make_float2(-d0, -d1)) {}
    __device__ __forceinline__ float2 operator()(float2 x) const {
        const float2 q0 = __fmul2_rn(x, r);
        const float2 e = __ffma2_rn(q0, nd, x);
        return __ffma2_rn(e, r, q0);
    }
};

// absmax / qmax, correctly rounded, for qmax in {127, 448, 57344}: the reciprocal sequence with a constant
// reciprocal (qt_selftest_division checks it against div.rn for every bf16 absmax). Results that are not
// normal numbers (absmax below 2^-100) take div.rn.
__device__ __forceinline__ float scale_of(float amax, float qmax, float rq) {
    if (amax < 7.8886090522101181e-31f) return div_rn(amax, qmax);
    const float q0 = __fmul_rn(amax, rq);
    return __fmaf_rn(__fmaf_rn(-q0, qmax, amax), rq, q0);
}

// ---- rounding to a byte ---------------------------------------------------------------------

// int8 from a pre-divided value, round-half-even, clamp [-128, 127]. Clamping before rounding is
// equivalent because both bounds are integers.
__device__ __forceinline__ uint32_t int8_rne(float v) {
    v = fminf(fmaxf(v, -128.0f), 127.0f);
    return __float_as_uint(__fadd_rn(v, kRoundMagic)) & 0xFFu;
}

// int8 from floor(v + u), clamp [-128, 127]. Adding 1.5 * 2^23 with round-toward-minus-infinity
// leaves floor(w) in the low mantissa bits.
__device__ __forceinline__ uint32_t int8_sr(float v, float u) {
    float w = __fadd_rn(v, u);
    w = fminf(fmaxf(w, -128.0f), 127.5f);
    return __float_as_uint(__fadd_rd(w, kRoundMagic)) & 0xFFu;
}

// f[k] <- f[k] / d for 8 values. The reciprocal sequence returns +0 for -0; fp8 keeps the sign of
// zero, so zero inputs pass through unchanged there.
template <bool EXACT>
__device__ __forceinline__ void divide8(float (&f)[8], const Divider<EXACT>& div, bool keep_zero_sign) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float q = div(f[k]);
        f[k] = (keep_zero_sign && f[k] == 0.0f) ? f[k] : q;
    }
}

// Quantize 8 pre-divided values into 8 bytes (two 32-bit words).
__device__ __forceinline__ uint2 pack8(const float (&v)[8], int q_dtype, bool stochastic, const float (&u)[8]) {
    uint32_t b[8];
    if (q_dtype == QT_I8) {
        if (stochastic) {
#pragma unroll
            for (int k = 0; k < 8; ++k) b[k] = int8_sr(v[k], u[k]);
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) b[k] = int8_rne(v[k]);
        }
    } else {
        const __nv_fp8_interpretation_t kind = (q_dtype == QT_E4M3) ? __NV_E4M3 : __NV_E5M2;
#pragma unroll
        for (int k = 0; k < 8; k += 2) {
            const uint32_t two = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(v[k], v[k + 1]), __NV_SATFINITE, kind);
            b[k] = two & 0xFFu;
            b[k + 1] = (two >> 8) & 0xFFu;
        }
    }
    uint2 out;
    out.x = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
    out.y = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
    return out;
}

// Stochastic-rounding uniforms: element i takes 16 bits of the Philox stream -- counter i / 8,
// word (i % 8) / 2, low half for even i, high half for odd i -- as u = bits * 2^-16 in [0, 1).
__device__ __forceinline__ float u01_from_half(uint32_t word, int odd) { return (float)((word >> (16 * odd)) & 0xFFFFu) * (1.0f / 65536.0f); }

__device__ __forceinline__ float uniform1(int64_t idx, uint64_t seed, uint64_t offset) {
    const uint64_t i = (uint64_t)idx;
    const Philox4 a = philox4x32_10(i >> 3, offset, seed);
    const uint32_t sel = (uint32_t)(i >> 1) & 3u;
    const uint32_t w = sel == 0 ? a.x : (sel == 1 ? a.y : (sel == 2 ? a.z : a.w));
    return u01_from_half(w, (int)(i & 1));
}

// Uniforms for 4 consecutive elements starting at idx (one Philox call when they share a counter).
__device__ __forceinline__ void uniforms4(float (&u)[4], int64_t idx, uint64_t seed, uint64_t offset) {
    if ((idx & 7) <= 4) {
        const Philox4 a = philox4x32_10((uint64_t)idx >> 3, offset, seed);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t e = (uint32_t)(idx & 7) + j;
            const uint32_t sel = e >> 1;
            const uint32_t word = sel == 0 ? w[0] : (sel == 1 ? w[1] : (sel == 2 ? w[2] : w[3]));
            u[j] = u01_from_half(word, (int)(e & 1));
        }
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) u[j] = uniform1(idx + j, seed, offset);
    }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// Store 8 quantized bytes at q[idx .. idx+8) honouring the row end.
__device__ __forceinline__ void store_bytes8(uint8_t* q, int64_t idx, int64_t valid, uint2 bytes, bool vec_ok) {
    if (valid >= 8 && vec_ok) {
        *reinterpret_cast<uint2*>(q + idx) = bytes;
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (k < valid) q[idx + k] = (uint8_t)(((k < 4 ? bytes.x : bytes.y) >> (8 * (k & 3))) & 0xFFu);
    }
}

// ---- row-wise -------------------------------------------------------------------------------

constexpr int kMaxScatter = 16;   // destinations of the scatter form (GPUs of one NVLink domain)

struct RowwiseParams {
    QT_GUARD_FIELD
    const void* x;
    int64_t rows, cols, stride;
    uint8_t* q;
    void* scale;
    float* col_absmax;
    int q_dtype, scale_dtype;
    float eps;
    int stochastic;
    uint64_t seed, offset;
    PhiloxKeys keys;   // round keys of `seed`
    int vec_load, vec_store;
    // in-place weight update (UPD != 0): the row is not read from x but formed from the int8 weight
    // itself, its scale and one or two bf16 operand tensors
    const __nv_bfloat16* t1;
    const __nv_bfloat16* t2;
    float value;
    // scatter form (SCATTER): the quantized rows and scales of this shard are written at row offset
    // `dst_row0` into n_dst gathered buffers -- this GPU's own and its peers' (peer-to-peer stores) --
    // so the quantize and the all-gather of a row-sharded weight are one kernel
    uint8_t* q_dst[kMaxScatter];
    void* scale_dst[kMaxScatter];
    int n_dst;
    int64_t dst_row0;
    // producer forms (PRODUCER != 0): the row that gets quantized is first computed from x -- RMSNorm of
    // x with weight `w_norm`, or silu(x) * x2 -- and also written as bf16 to `y` (row pitch = cols); q may
    // be null, in which case only y (and rstd) are produced
    const __nv_bfloat16* w_norm;
    const __nv_bfloat16* x2;
    int64_t stride2;
    __nv_bfloat16* y;
    float* rstd;
    float norm_eps;
};

// ---- packed bf16 helpers -----------------------------------------------------------------------

__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t w) { return *reinterpret_cast<const __nv_bfloat162*>(&w); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 v) { return *reinterpret_cast<const uint32_t*>(&v); }

// Lane-wise maximum of two packed bf16 pairs.
__device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) { return as_u32(__hmax2(as_bf162(a), as_bf162(b))); }

// Four rounded floats (value + kRoundMagic) -> four int8 bytes: the low mantissa byte of each.
__device__ __forceinline__ uint32_t pack4_magic(float t0, float t1, float t2, float t3) {
    const uint32_t lo = __byte_perm(__float_as_uint(t0), __float_as_uint(t1), 0x0040);
    const uint32_t hi = __byte_perm(__float_as_uint(t2), __float_as_uint(t3), 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

// Four quotients -> four int8 bytes (first argument in the lowest byte): round-half-even to int32, then
// two saturating packs (cvt.pack.sat.s8.s32 d, a, b, c gives c[15:0] << 16 | sat8(a) << 8 | sat8(b)).
__device__ __forceinline__ uint32_t pack4_sat(float q0, float q1, float q2, float q3) {
    const int i0 = __float2int_rn(q0), i1 = __float2int_rn(q1), i2 = __float2int_rn(q2), i3 = __float2int_rn(q3);
    uint32_t hi, w;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(i3), "r"(i2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(i1), "r"(i0), "r"(hi));
    return w;
}

// max(|a|, |b|) of both bf16 halves in one instruction. The sign bits of the result are the XOR of the
// operands' signs (callers mask them off once, after the last fold), so no separate |x| is needed.
__device__ __forceinline__ uint32_t amax2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// The larger of the two (sign-cleared) bf16 halves as the bit pattern of an fp32 value. Bit patterns of
// non-negative floats order like unsigned integers.
__device__ __forceinline__ uint32_t fold_halves(uint32_t m) {
    const uint32_t lo = (m << 16) & 0x7FFF0000u, hi = m & 0x7FFF0000u;
    return lo > hi ? lo : hi;
}

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}

// Quantize the 8 bf16 values of `raw` (elements [8 ctr, 8 ctr + 8) of the output: `ctr` is the Philox
// counter of the stochastic form) with divider `div`, two elements per packed fp32x2 instruction.
// int8, round-half-even: add 1.5 * 2^23, the low mantissa byte is the result. No clamp: |x| <= absmax and
// d >= absmax/127 * (1 - 2^-24) bound the quotient by 127 + 2^-17, which rounds to 127.
// int8, stochastic: floor(fl(v + u)) with u = 16 Philox bits * 2^-16. The uniform is built without an
// integer-to-float conversion: OR-ing the 16 bits under the mantissa of 192.0 gives 192 + u exactly, and
// subtracting 192 is exact. fl(v + u) <= 128 - 2^-17 and >= -128, so again no clamp; adding 1.5 * 2^23
// rounding toward minus infinity leaves floor() in the low mantissa byte.
// fp8: cvt.rn.satfinite of the quotient; the reciprocal sequence returns +0 for x = -0, so the sign of
// the input is OR-ed back into the byte (a quotient never has the opposite sign of x).
template <bool SR>
__device__ __forceinline__ uint2 quantize_vec8(const uint4& raw, const Divider2& div, int q_dtype, uint64_t ctr,
                                               const PhiloxKeys& keys, uint64_t offset) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float2 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = div(unpack_bf16x2(w[k]));
    uint2 out;
    if (q_dtype == QT_I8) {
        const float2 magic2 = make_float2(kRoundMagic, kRoundMagic);
        if constexpr (SR) {
            const Philox4 a = philox4x32_10(ctr, offset, keys);
            const uint32_t rw[4] = {a.x, a.y, a.z, a.w};
            const float2 m192 = make_float2(-192.0f, -192.0f);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 big = make_float2(__uint_as_float(__byte_perm(rw[k], 0x43400000u, 0x7610)),
                                               __uint_as_float(__byte_perm(rw[k], 0x43400000u, 0x7632)));
                v[k] = __fadd2_rd(__fadd2_rn(v[k], __fadd2_rn(big, m192)), magic2);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = __fadd2_rn(v[k], magic2);
        }
        out.x = pack4_magic(v[0].x, v[0].y, v[1].x, v[1].y);
        out.y = pack4_magic(v[2].x, v[2].y, v[3].x, v[3].y);
    } else {
        uint32_t h[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            uint16_t two;
            if (q_dtype == QT_E4M3) asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(two) : "f"(v[k].y), "f"(v[k].x));
            else asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(two) : "f"(v[k].y), "f"(v[k].x));
            h[k] = two;
        }
        // sign bytes (0x00 / 0xFF) of the eight inputs in output order, then their top bits
        uint32_t s_lo, s_hi;   // selector nibbles with bit 3 set replicate the selected byte's top bit
        asm("prmt.b32 %0, %1, %2, 0xFDB9;" : "=r"(s_lo) : "r"(w[0]), "r"(w[1]));
        asm("prmt.b32 %0, %1, %2, 0xFDB9;" : "=r"(s_hi) : "r"(w[2]), "r"(w[3]));
        out.x = __byte_perm(h[0], h[1], 0x5410) | (s_lo & 0x80808080u);
        out.y = __byte_perm(h[2], h[3], 0x5410) | (s_hi & 0x80808080u);
    }
    return out;
}

// Eight updated bf16 weights, packed like eight loaded bf16 values. The arithmetic is the eager
// sequence on a bf16 weight, every step in fp32 and rounded to bf16 where eager materialises a tensor:
//   w = bf16(float(q) * s)                          de-quantize (int8 tensor * bf16 scale)
//   y = bf16(w + value * t1)            UPD == 1    add_(t1, alpha=value)
//   y = bf16(w + value * (t1 / t2))     UPD == 2    addcdiv_(t1, t2, value=value)
// with the multiply-add fused, as the compiled element-wise kernels of the framework do.
template <int UPD>
__device__ __forceinline__ uint4 updated_vec8(uint2 qb, float s, const uint4& a, const uint4& b, float value) {
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t out[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t qw = k < 2 ? qb.x : qb.y;
        const int q0 = (int)(int8_t)((qw >> (16 * (k & 1))) & 0xFFu);
        const int q1 = (int)(int8_t)((qw >> (16 * (k & 1) + 8)) & 0xFFu);
        const float w0 = __bfloat162float(__float2bfloat16_rn(__fmul_rn((float)q0, s)));
        const float w1 = __bfloat162float(__float2bfloat16_rn(__fmul_rn((float)q1, s)));
        float t0 = __uint_as_float(aw[k] << 16), t1 = __uint_as_float(aw[k] & 0xFFFF0000u);
        if constexpr (UPD == 2) {
            t0 = __fdiv_rn(t0, __uint_as_float(bw[k] << 16));
            t1 = __fdiv_rn(t1, __uint_as_float(bw[k] & 0xFFFF0000u));
        }
        out[k] = as_u32(__floats2bfloat162_rn(__fmaf_rn(value, t0, w0), __fmaf_rn(value, t1, w1)));
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

// End of the column-maxima variants: `colmax` holds each thread's running |x| maxima (packed bf16 pairs,
// sign bits undefined) of its VPT vectors. 1. The CTA's sub-rows, which cover the same columns, fold in
// shared memory. 2. The CTAs of the thread-block cluster fold through distributed shared memory; each CTA
// owns a slice of the columns and issues one atomic max per column for the whole cluster.
template <int TPR, int VPT>
__device__ __forceinline__ void fold_column_maxima(uint32_t (&colmax)[VPT][4], uint32_t* s_col, int sub, int t, const RowwiseParams& p) {
    const int64_t cols = p.cols;
    float* col_absmax = p.col_absmax;
    constexpr int RPC = kThreads / TPR;
    constexpr int PAIRS = TPR * VPT * 4;
    if constexpr (RPC > 1) {
#pragma unroll 1
        for (int turn = 0; turn < RPC; ++turn) {
            if (sub == turn) {
#pragma unroll
                for (int i = 0; i < VPT; ++i)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int pair = (i * TPR + t) * 4 + k;
                        s_col[pair] = max2(s_col[pair], colmax[i][k] & 0x7FFF7FFFu);
                    }
            }
            __syncthreads();
        }
    } else {
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int k = 0; k < 4; ++k) s_col[(i * TPR + t) * 4 + k] = colmax[i][k] & 0x7FFF7FFFu;
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const unsigned n_cta = cluster.num_blocks(), rank = cluster.block_rank();
    for (int pair = rank * kThreads + threadIdx.x; pair < PAIRS; pair += n_cta * kThreads) {
        uint32_t m = 0u;
        if (n_cta == 2) {
            // issue both reads together: the remote one is a trip across the cluster
            const uint32_t v0 = cluster.map_shared_rank(s_col, 0)[pair], v1 = cluster.map_shared_rank(s_col, 1)[pair];
            m = max2(v0, v1);
        } else {
            for (unsigned c = 0; c < n_cta; ++c) m = max2(m, cluster.map_shared_rank(s_col, c)[pair]);
        }
        const int64_t c0 = (int64_t)pair * 2;
        // fp32 bit patterns of non-negative values order like unsigned integers
        if (c0 < cols && (m & 0xFFFFu) && QT_GUARD_OK(p.guard, col_absmax + c0, 4, 27)) atomicMax(reinterpret_cast<unsigned int*>(col_absmax + c0), m << 16);
        if (c0 + 1 < cols && (m >> 16) && QT_GUARD_OK(p.guard, col_absmax + c0 + 1, 4, 27)) atomicMax(reinterpret_cast<unsigned int*>(col_absmax + c0 + 1), m & 0xFFFF0000u);
    }
    cluster.sync();  // nobody leaves while a peer may still read its shared memory
}

// Row-wise kernel for bf16 rows that fit in registers. TPR threads cooperate on one row, each
// holding VPT 16-byte vectors, so a row of up to TPR*VPT*8 columns is read from HBM exactly once.
// The next row's loads are issued before the current row is reduced and quantized (register double
// buffer), which keeps HBM requests in flight through the reduction and the stores. With COLABS
// each thread also keeps the running |x| maximum of its columns (packed bf16 pairs) over all rows
// the CTA visits; at the end the CTA folds its sub-rows in shared memory, a pair of CTAs (a 2-CTA
// cluster) folds through distributed shared memory, and one atomic max per column per pair goes out.
// With UPD != 0 the kernel re-quantizes an int8 weight in place: the "row" is the updated weight formed
// by updated_vec8 from q, scale and the operand tensors; q and scale are then overwritten (each row
// is complete in registers before its bytes are stored, and a prefetched row is a different row).
// CTAs per SM of the row kernel with up to 4 vectors per thread. Fewer CTAs leave the compiler more registers:
// the stochastic form measured 51.5 / 55.6 / 58.9 us per launch on [32768, 2048] with 2 / 3 / 4 CTAs per SM, the
// column-maxima form 43.5 / 41.7 / 45.7; round-to-nearest is indifferent (35.1 - 35.5).
#ifndef QT_SR_CTAS
#define QT_SR_CTAS 2
#endif
#ifndef QT_COLABS_CTAS
#define QT_COLABS_CTAS 3
#endif
#ifndef QT_RNE_CTAS
#define QT_RNE_CTAS 4
#endif
#ifndef QT_PRODUCER_CTAS
#define QT_PRODUCER_CTAS 3   // the RMSNorm / silu * up forms: silu * up + quantize on [32768, 5632] 248 us with 3, 314 us with 2
#endif

// Barrier among the TPR threads of row group `sub` (at most four groups of several warps per CTA). The
// barrier number is an immediate so that the CTA reserves five hardware barriers, not all sixteen.
template <int TPR>
__device__ __forceinline__ void row_barrier(int sub) {
    switch (sub) {
        case 0: asm volatile("bar.sync 1, %0;" ::"n"(TPR) : "memory"); break;
        case 1: asm volatile("bar.sync 2, %0;" ::"n"(TPR) : "memory"); break;
        case 2: asm volatile("bar.sync 3, %0;" ::"n"(TPR) : "memory"); break;
        default: asm volatile("bar.sync 4, %0;" ::"n"(TPR) : "memory"); break;
    }
}

template <int TPR, int VPT, bool COLABS, bool SR, int UPD = 0, bool SCATTER = false>
__global__ void __launch_bounds__(kThreads, (VPT <= 4 ? (UPD != 0 ? 3 : (SR ? QT_SR_CTAS : (COLABS ? QT_COLABS_CTAS : QT_RNE_CTAS))) : (VPT <= 8 ? 2 : 1)))
rowwise_kernel(const RowwiseParams p) {
    constexpr int RPC = kThreads / TPR;  // rows per CTA per iteration
    constexpr int WPR = TPR / 32;        // warps per row
    // the column-maxima variant spends its registers on the maxima instead of a second row buffer
    constexpr bool PREFETCH = VPT <= 8 && !COLABS;
    __shared__ uint32_t s_red[2][kThreads / 32];
    __shared__ uint32_t s_col[COLABS ? TPR * VPT * 4 : 1];  // packed bf16 pairs, one per two columns

    const int sub = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int warp = threadIdx.x >> 5;
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(p.x);
    const float qmax = qmax_of(p.q_dtype);
    const float rqmax = p.q_dtype == QT_I8 ? (1.0f / 127.0f) : (p.q_dtype == QT_E4M3 ? (1.0f / 448.0f) : (1.0f / 57344.0f));
    const int64_t step = (int64_t)gridDim.x * RPC;

    uint32_t colmax[COLABS ? VPT : 1][4];
    if constexpr (COLABS) {
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int k = 0; k < 4; ++k) colmax[i][k] = 0u;
        for (int i = threadIdx.x; i < TPR * VPT * 4; i += kThreads) s_col[i] = 0u;
        __syncthreads();
    }

    // the host only takes this kernel when cols is a multiple of 8 and q is 8-byte aligned, so every
    // vector is either wholly inside the row or wholly outside it
    auto load_row = [&](uint4 (&v)[VPT], int64_t row) {
        const bool valid = row < p.rows;
        if constexpr (UPD == 0) {
            const __nv_bfloat16* xrow = x + (valid ? row : 0) * p.stride;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int col = (i * TPR + t) * 8;
                v[i] = (valid && col < p.cols) ? *reinterpret_cast<const uint4*>(xrow + col) : make_uint4(0, 0, 0, 0);
            }
        } else {
            const int64_t r = valid ? row : 0;
            const float s = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.scale)[r]);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int col = (i * TPR + t) * 8;
                if (valid && col < p.cols) {
                    const int64_t at = r * p.cols + col;
                    const uint2 qb = *reinterpret_cast<const uint2*>(p.q + at);
                    const uint4 a = *reinterpret_cast<const uint4*>(p.t1 + at);
                    const uint4 b = UPD == 2 ? *reinterpret_cast<const uint4*>(p.t2 + at) : make_uint4(0, 0, 0, 0);
                    v[i] = updated_vec8<UPD>(qb, s, a, b, p.value);
                } else {
                    v[i] = make_uint4(0, 0, 0, 0);
                }
            }
        }
    };

    // One row held in `cur`: fold its absmax, derive the scale, quantize and store. `parity` alternates
    // between consecutive calls: rows spanning several warps exchange their partial maxima through one of
    // two shared-memory slots and meet at a barrier of their own (the row's TPR threads only), so one
    // barrier per row is enough and the CTA's other rows are not held up.
    auto process = [&](uint4 (&cur)[VPT], int64_t row, int parity) {
        const bool valid = row < p.rows;
        uint32_t m2 = 0u;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            m2 = amax2(m2, amax2(amax2(cur[i].x, cur[i].y), amax2(cur[i].z, cur[i].w)));
            if constexpr (COLABS) {
                colmax[i][0] = amax2(colmax[i][0], cur[i].x); colmax[i][1] = amax2(colmax[i][1], cur[i].y);
                colmax[i][2] = amax2(colmax[i][2], cur[i].z); colmax[i][3] = amax2(colmax[i][3], cur[i].w);
            }
        }
        uint32_t abits = __reduce_max_sync(0xFFFFFFFFu, fold_halves(m2));
        if constexpr (WPR > 1) {
            if ((threadIdx.x & 31) == 0) s_red[parity][warp] = abits;
            if constexpr (RPC == 1) __syncthreads();
            else row_barrier<TPR>(sub);
            abits = s_red[parity][sub * WPR];
#pragma unroll
            for (int w = 1; w < WPR; ++w) { const uint32_t o = s_red[parity][sub * WPR + w]; abits = o > abits ? o : abits; }
        }
        const float amax = __uint_as_float(abits);

        const float scale = scale_of(amax, qmax, rqmax);
        const Divider2 div(fmaxf(scale, p.eps));
        if constexpr (SCATTER) {
            if (valid && t == 0)
                for (int d = 0; d < p.n_dst; ++d) QT_STORE_SCALE(p.guard, p.scale_dst[d], p.scale_dtype, p.dst_row0 + row, scale, 1);
        } else {
            if (valid && t == 0) QT_STORE_SCALE(p.guard, p.scale, p.scale_dtype, row, scale, 2);
        }

        uint8_t* qrow = p.q + row * p.cols;
        const int64_t idx0 = SR ? row * p.cols : 0;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int col = (i * TPR + t) * 8;
            if (valid && col < p.cols) {
                const uint2 bytes = quantize_vec8<SR>(cur[i], div, p.q_dtype, (uint64_t)(idx0 + col) >> 3, p.keys, p.offset);
                if constexpr (SCATTER) {
                    const int64_t at = (p.dst_row0 + row) * p.cols + col;
                    for (int d = 0; d < p.n_dst; ++d)
                        if (QT_GUARD_OK(p.guard, p.q_dst[d] + at, 8, 3)) *reinterpret_cast<uint2*>(p.q_dst[d] + at) = bytes;
                } else {
                    if (QT_GUARD_OK(p.guard, qrow + col, 8, 4)) *reinterpret_cast<uint2*>(qrow + col) = bytes;
                }
            }
        }
    };

    int64_t base = (int64_t)blockIdx.x * RPC;
    if constexpr (PREFETCH) {
        // register double buffer, unrolled by two so the prefetched row is never copied: while one buffer
        // is reduced and quantized the loads of the row after it are in flight in the other
        uint4 a[VPT], b[VPT];
        if (base < p.rows) load_row(a, base + sub);
        while (base < p.rows) {
            if (base + step < p.rows) load_row(b, base + step + sub);
            process(a, base + sub, 0);
            base += step;
            if (base >= p.rows) break;
            if (base + step < p.rows) load_row(a, base + step + sub);
            process(b, base + sub, 1);
            base += step;
        }
    } else {
        uint4 a[VPT];
        int parity = 0;
        for (; base < p.rows; base += step) {
            load_row(a, base + sub);
            process(a, base + sub, parity);
            parity ^= 1;
        }
    }

    if constexpr (COLABS) fold_column_maxima<TPR, VPT>(colmax, s_col, sub, t, p);
}

// ---- producer arithmetic ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// bf16(a * b) per half: the product of two bf16 values is exact in fp32, so this is the single rounding
// of an eager bf16 multiply.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) { return as_u32(__hmul2(as_bf162(a), as_bf162(b))); }

// RMSNorm of one word (two bf16 values) the way an eager module evaluates it
// (transformers LlamaRMSNorm.forward): n = bf16(float(x) * rstd), y = bf16(weight * n).
__device__ __forceinline__ uint32_t rmsnorm_word(uint32_t x, uint32_t w, float2 rstd2) {
    const float2 n = __fmul2_rn(unpack_bf16x2(x), rstd2);
    return mul_bf16x2(w, pack_bf16x2_rn(n.x, n.y));
}

// silu(g) * u of one word: s = bf16(g / (1 + exp(-g))) in fp32 (fast exponential and division: the
// result is within a few fp32 ulp before the bf16 rounding), h = bf16(s * u).
__device__ __forceinline__ uint32_t silu_mul_word(uint32_t g, uint32_t u) {
    const float2 gf = unpack_bf16x2(g);
    const float2 den = __fadd2_rn(make_float2(__expf(-gf.x), __expf(-gf.y)), make_float2(1.0f, 1.0f));
    return mul_bf16x2(pack_bf16x2_rn(__fdividef(gf.x, den.x), __fdividef(gf.y, den.y)), u);
}

// The common case of the kernel above with everything that costs instructions removed: the row count is
// a multiple of the rows per CTA and below 2^30, so rows are counted in 32 bits and need no bounds check;
// which of a thread's vectors lie inside the row is decided once (those outside stay zero and are never
// loaded or stored); the load and store pointers advance by a fixed step instead of being recomputed.
// Same arithmetic, same results.
// TILE selects 1 x 128 tiles instead of whole rows (cols a multiple of 128): eight lanes own one tile, lane
// l of the group holding elements [8l, 8l + 8) and [64 + 8l, 64 + 8l + 8), so each of the two loads of a
// group covers 128 contiguous bytes, the tile's absmax is one 8-lane reduction, and the per-tile scalar
// work (scale, reciprocal, scale store) is shared by 16 elements per thread. Vectors 2j and 2j + 1 of a
// thread are the two halves of its j-th tile.
// PRODUCER selects what the row is: 0 = x itself; 1 = RMSNorm(x) * w_norm (also writes y and 1/rms per
// row); 2 = silu(x) * x2 (also writes y). The producer forms fold the activation quantize of the INT8
// linear layers into the kernel that produces the activation, so the activation is not read again.
template <int TPR, int VPT, bool COLABS, bool SR, bool TILE = false, int PRODUCER = 0>
__global__ void __launch_bounds__(kThreads, (PRODUCER != 0 ? (VPT <= 4 ? QT_PRODUCER_CTAS : 1) : (VPT <= 4 ? (SR ? QT_SR_CTAS : (COLABS ? QT_COLABS_CTAS : QT_RNE_CTAS)) : (VPT <= 8 ? 2 : 1))))
rowwise_full_kernel(const RowwiseParams p) {
    constexpr int RPC = kThreads / TPR;
    constexpr int WPR = TPR / 32;
    // the register double buffer: always for plain rows of up to 8 vectors per thread; with the column maxima
    // (which take VPT * 4 registers of their own) for up to 4; the producer forms spend theirs on operands
    constexpr bool PREFETCH = PRODUCER == 0 ? (COLABS ? VPT <= 4 : VPT <= 8) : (PRODUCER == 1 && !COLABS && VPT <= 4);
    static_assert(!TILE || (VPT % 2 == 0 && !COLABS && !SR), "tile form: vector pairs, no column maxima, round-to-nearest");
    static_assert(PRODUCER == 0 || (!TILE && !SR), "producer forms: whole rows, round-to-nearest");
    __shared__ uint32_t s_red[2][kThreads / 32];
    __shared__ float s_sum[2][kThreads / 32];
    __shared__ uint32_t s_col[COLABS ? TPR * VPT * 4 : 1];

    const int sub = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int warp = threadIdx.x >> 5;
    const float qmax = qmax_of(p.q_dtype);
    const float rqmax = p.q_dtype == QT_I8 ? (1.0f / 127.0f) : (p.q_dtype == QT_E4M3 ? (1.0f / 448.0f) : (1.0f / 57344.0f));
    const int rows = (int)p.rows;
    const int step = (int)gridDim.x * RPC;
    const int first = (int)blockIdx.x * RPC;
    int n_iter = first < rows ? (rows - first + step - 1) / step : 0;
    int row = first + sub;
    const int nvec = (int)(p.cols / 8);

    // position of vector i of this thread inside a row, in 8-element units, and whether it exists
    int vpos[VPT];
    bool ok[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if constexpr (TILE) vpos[i] = ((i >> 1) * (TPR / 8) + (t >> 3)) * 16 + (i & 1) * 8 + (t & 7);
        else vpos[i] = i * TPR + t;
        ok[i] = vpos[i] < nvec;
    }
    const uint32_t gmask = 0xFFu << (threadIdx.x & 24);   // the 8 lanes of this thread's tile (TILE)

    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.x) + (int64_t)row * p.stride);
    const int64_t src_step = (int64_t)step * (p.stride / 8);
    uint2* dst = reinterpret_cast<uint2*>(p.q + (int64_t)row * p.cols);
    const int64_t dst_step = (int64_t)step * nvec;
    uint64_t ctr = SR ? (uint64_t)row * (uint64_t)nvec : 0;   // Philox counter of the row's first vector

    uint32_t colmax[COLABS ? VPT : 1][4];
    if constexpr (COLABS) {
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int k = 0; k < 4; ++k) colmax[i][k] = 0u;
        for (int i = threadIdx.x; i < TPR * VPT * 4; i += kThreads) s_col[i] = 0u;
        __syncthreads();
    }

    // producer operands: the norm weight of this thread's columns stays in registers; the second input
    // and the bf16 output advance like the first
    uint4 wv[PRODUCER == 1 ? VPT : 1];
    const uint4* src2 = nullptr;
    int64_t src2_step = 0;
    uint4* ydst = nullptr;
    const bool quantizing = PRODUCER == 0 || p.q != nullptr;
    if constexpr (PRODUCER == 1) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) wv[i] = ok[i] ? reinterpret_cast<const uint4*>(p.w_norm)[vpos[i]] : make_uint4(0, 0, 0, 0);
    }
    if constexpr (PRODUCER == 2) {
        src2 = reinterpret_cast<const uint4*>(p.x2 + (int64_t)row * p.stride2);
        src2_step = (int64_t)step * (p.stride2 / 8);
    }
    if constexpr (PRODUCER != 0) ydst = reinterpret_cast<uint4*>(p.y + (int64_t)row * p.cols);

    uint4 u_buf[PRODUCER == 2 ? VPT : 1];   // second operand of the current row (silu-mul form)
    auto load_row = [&](uint4 (&v)[VPT]) {
#pragma unroll
        for (int i = 0; i < VPT; ++i)
            if (ok[i]) v[i] = src[vpos[i]];
        src += src_step;
        if constexpr (PRODUCER == 2) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) u_buf[i] = ok[i] ? src2[vpos[i]] : make_uint4(0, 0, 0, 0);
            src2 += src2_step;
        }
    };
    // Sum over the row of a per-thread partial (the TPR threads of the row), through the same slots and
    // barrier as the absmax fold.
    auto row_sum = [&](float v, int parity) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if constexpr (WPR > 1) {
            if ((threadIdx.x & 31) == 0) s_sum[parity][warp] = v;
            if constexpr (RPC == 1) __syncthreads();
            else row_barrier<TPR>(sub);
            v = s_sum[parity][sub * WPR];
#pragma unroll
            for (int w = 1; w < WPR; ++w) v += s_sum[parity][sub * WPR + w];
        }
        return v;
    };
    auto process = [&](uint4 (&cur)[VPT], int parity) {
        if constexpr (PRODUCER == 1) {
            // sum of squares in fp32 (two lanes of partial sums per thread), 1/rms, then the normed row
            // replaces x in `cur` and goes out as bf16
            float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const uint32_t w[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) { const float2 f = unpack_bf16x2(w[k]); acc = __ffma2_rn(f, f, acc); }
            }
            const float ss = row_sum(__fadd_rn(acc.x, acc.y), parity);
            const float rstd = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)p.cols), p.norm_eps));
            if (t == 0 && p.rstd && QT_GUARD_OK(p.guard, p.rstd + row, 4, 5)) p.rstd[row] = rstd;
            const float2 rstd2 = make_float2(rstd, rstd);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                cur[i] = make_uint4(rmsnorm_word(cur[i].x, wv[i].x, rstd2), rmsnorm_word(cur[i].y, wv[i].y, rstd2),
                                    rmsnorm_word(cur[i].z, wv[i].z, rstd2), rmsnorm_word(cur[i].w, wv[i].w, rstd2));
                if (ok[i] && QT_GUARD_OK(p.guard, ydst + vpos[i], 16, 6)) ydst[vpos[i]] = cur[i];
            }
            ydst += dst_step;
        }
        if constexpr (PRODUCER == 2) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const uint4 u = u_buf[i];
                cur[i] = make_uint4(silu_mul_word(cur[i].x, u.x), silu_mul_word(cur[i].y, u.y), silu_mul_word(cur[i].z, u.z),
                                    silu_mul_word(cur[i].w, u.w));
                if (ok[i] && QT_GUARD_OK(p.guard, ydst + vpos[i], 16, 6)) ydst[vpos[i]] = cur[i];
            }
            ydst += dst_step;
        }
        if (!quantizing) {
            row += step;
            return;
        }
        if constexpr (TILE) {
#pragma unroll
            for (int j = 0; j < VPT / 2; ++j) {
                const uint4 &lo = cur[2 * j], &hi = cur[2 * j + 1];
                const uint32_t m2 = amax2(amax2(amax2(lo.x, lo.y), amax2(lo.z, lo.w)), amax2(amax2(hi.x, hi.y), amax2(hi.z, hi.w)));
                // all 8 lanes of a tile take part (lanes of tiles beyond the row hold zeros)
                const float amax = __uint_as_float(__reduce_max_sync(gmask, fold_halves(m2)));
                const float scale = scale_of(amax, qmax, rqmax);
                const Divider2 div(fmaxf(scale, p.eps));
                // (the arithmetic runs unconditionally, on zeros where the tile lies beyond the row, so that only the
                // stores are predicated and the loop body has no branches)
                const uint2 qlo = quantize_vec8<false>(lo, div, p.q_dtype, 0, p.keys, 0);
                const uint2 qhi = quantize_vec8<false>(hi, div, p.q_dtype, 0, p.keys, 0);
                if (ok[2 * j] && (t & 7) == 0) QT_STORE_SCALE(p.guard, p.scale, p.scale_dtype, (int64_t)row * (nvec >> 4) + (vpos[2 * j] >> 4), scale, 7);
                if (ok[2 * j] && QT_GUARD_OK(p.guard, dst + vpos[2 * j], 8, 8)) dst[vpos[2 * j]] = qlo;
                if (ok[2 * j] && QT_GUARD_OK(p.guard, dst + vpos[2 * j + 1], 8, 8)) dst[vpos[2 * j + 1]] = qhi;
            }
        } else {
            uint32_t m2 = 0u;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                m2 = amax2(m2, amax2(amax2(cur[i].x, cur[i].y), amax2(cur[i].z, cur[i].w)));
                if constexpr (COLABS) {
                    colmax[i][0] = amax2(colmax[i][0], cur[i].x); colmax[i][1] = amax2(colmax[i][1], cur[i].y);
                    colmax[i][2] = amax2(colmax[i][2], cur[i].z); colmax[i][3] = amax2(colmax[i][3], cur[i].w);
                }
            }
            uint32_t abits = __reduce_max_sync(0xFFFFFFFFu, fold_halves(m2));
            if constexpr (WPR > 1) {
                if ((threadIdx.x & 31) == 0) s_red[parity][warp] = abits;
                if constexpr (RPC == 1) __syncthreads();
                else row_barrier<TPR>(sub);
                abits = s_red[parity][sub * WPR];
#pragma unroll
                for (int w = 1; w < WPR; ++w) { const uint32_t o = s_red[parity][sub * WPR + w]; abits = o > abits ? o : abits; }
            }
            const float scale = scale_of(__uint_as_float(abits), qmax, rqmax);
            const Divider2 div(fmaxf(scale, p.eps));
            if (t == 0) QT_STORE_SCALE(p.guard, p.scale, p.scale_dtype, row, scale, 9);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                // (computed unconditionally, on zeros where the vector lies beyond the row: only the store is predicated)
                const uint2 q = quantize_vec8<SR>(cur[i], div, p.q_dtype, ctr + vpos[i], p.keys, p.offset);
                if (ok[i] && QT_GUARD_OK(p.guard, dst + vpos[i], 8, 10)) dst[vpos[i]] = q;
            }
        }
        dst += dst_step;
        row += step;
        if constexpr (SR) ctr += (uint64_t)dst_step;
    };

    if constexpr (PREFETCH) {
        uint4 a[VPT], b[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) a[i] = b[i] = make_uint4(0, 0, 0, 0);
        if (n_iter > 0) load_row(a);
        while (n_iter > 0) {
            if (n_iter > 1) load_row(b);
            process(a, 0);
            if (--n_iter == 0) break;
            if (n_iter > 1) load_row(a);
            process(b, 1);
            --n_iter;
        }
    } else {
        uint4 a[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) a[i] = make_uint4(0, 0, 0, 0);
        for (int it = 0; it < n_iter; ++it) {
            load_row(a);
            process(a, it & 1);
        }
    }
    if constexpr (COLABS) fold_column_maxima<TPR, VPT>(colmax, s_col, sub, t, p);
}

// Any width, any alignment: one CTA per row, two passes (the second normally hits L2).
template <typename XT, bool COLABS>
__global__ void __launch_bounds__(kThreads) rowwise_generic_kernel(const RowwiseParams p) {
    __shared__ float s_red[kThreads / 32];
    __shared__ float s_amax;
    const XT* x = reinterpret_cast<const XT*>(p.x);
    const float qmax = qmax_of(p.q_dtype);
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const XT* xrow = x + row * p.stride;
        float amax = 0.0f;
        for (int64_t c = threadIdx.x; c < p.cols; c += kThreads) {
            const float a = fabsf(to_float<XT>(xrow[c]));
            amax = fmaxf(amax, a);
            if constexpr (COLABS) {
                if (QT_GUARD_OK(p.guard, p.col_absmax + c, 4, 11)) atomicMax(reinterpret_cast<unsigned int*>(p.col_absmax + c), __float_as_uint(a));
            }
        }
        amax = warp_max(amax);
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = s_red[0];
            for (int w = 1; w < kThreads / 32; ++w) m = fmaxf(m, s_red[w]);
            s_amax = m;
        }
        __syncthreads();
        const float scale = __fdiv_rn(s_amax, qmax);
        const float d = fmaxf(scale, p.eps);
        if (threadIdx.x == 0) QT_STORE_SCALE(p.guard, p.scale, p.scale_dtype, row, scale, 12);
        for (int64_t c = threadIdx.x; c < p.cols; c += kThreads) {
            const float v = __fdiv_rn(to_float<XT>(xrow[c]), d);
            const int64_t idx = row * p.cols + c;
            const float u = p.stochastic ? uniform1(idx, p.seed, p.offset) : 0.0f;
            if (QT_GUARD_OK(p.guard, p.q + idx, 1, 13)) p.q[idx] = (uint8_t)quantize_byte(v, p.q_dtype, p.stochastic != 0, u);
        }
        __syncthreads();
    }
}

// CTAs per cluster in the column-absmax variant. Pairs halve the column atomics at no cost; clusters
// of 4 or 8 constrain CTA placement enough to slow the streaming loop by a quarter (measured).
constexpr int kClusterSize = 2;

template <int TPR, int VPT, bool COLABS, bool SR, int UPD = 0, bool SCATTER = false>
int launch_rowwise_cfg(const RowwiseParams& p, cudaStream_t stream) {
    constexpr int RPC = kThreads / TPR;
    // the in-place weight update computes its row while loading it, so it hides latency with occupancy (3 CTAs:
    // 133 us against 163 us with 2 on [32768, 2048])
    constexpr int CTAS_PER_SM = (VPT <= 4 ? (UPD != 0 ? 3 : (SR ? QT_SR_CTAS : (COLABS ? QT_COLABS_CTAS : QT_RNE_CTAS))) : (VPT <= 8 ? 2 : 1));
    const int64_t want = (p.rows + RPC - 1) / RPC;
    const int64_t cap = (int64_t)num_sms() * CTAS_PER_SM;
    int64_t grid = want < cap ? want : cap;
    auto kfn = rowwise_kernel<TPR, VPT, COLABS, SR, UPD, SCATTER>;
    if constexpr (UPD == 0 && !SCATTER) {
        if (p.rows % RPC == 0 && p.rows < ((int64_t)1 << 30)) kfn = rowwise_full_kernel<TPR, VPT, COLABS, SR>;
    }
    if constexpr (COLABS) {
        constexpr int csize = kClusterSize;
        grid = (grid + csize - 1) / csize * csize;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = csize;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        QT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kfn, p));
    } else {
        kfn<<<(unsigned)grid, kThreads, 0, stream>>>(p);
        QT_CUDA_CHECK(cudaGetLastError());
    }
    return QT_OK;
}

template <bool COLABS, bool SR, int UPD = 0, bool SCATTER = false>
int launch_rowwise_bf16(const RowwiseParams& p, cudaStream_t stream) {
    const int64_t c = p.cols;
    if (c <= 256) return launch_rowwise_cfg<32, 1, COLABS, SR, UPD, SCATTER>(p, stream);
    if (c <= 512) return launch_rowwise_cfg<32, 2, COLABS, SR, UPD, SCATTER>(p, stream);
    if (c <= 1024) return launch_rowwise_cfg<32, 4, COLABS, SR, UPD, SCATTER>(p, stream);
    if (c <= 2048) return launch_rowwise_cfg<64, 4, COLABS, SR, UPD, SCATTER>(p, stream);
    if (c <= 4096) return launch_rowwise_cfg<128, 4, COLABS, SR, UPD, SCATTER>(p, stream);
    if (c <= 8192) return launch_rowwise_cfg<256, 4, COLABS, SR, UPD, SCATTER>(p, stream);
    if (c <= 16384) return launch_rowwise_cfg<256, 8, COLABS, SR, UPD, SCATTER>(p, stream);
    if constexpr (!COLABS) return launch_rowwise_cfg<256, 16, COLABS, SR, UPD, SCATTER>(p, stream);
    return fail(QT_ERR_UNSUPPORTED, "unreachable");
}

template <typename XT, bool COLABS>
int launch_rowwise_generic(const RowwiseParams& p, cudaStream_t stream) {
    const int64_t cap = (int64_t)num_sms() * 8;
    const int grid = (int)(p.rows < cap ? p.rows : cap);
    rowwise_generic_kernel<XT, COLABS><<<grid, kThreads, 0, stream>>>(p);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

// Fast path: bf16 rows, 16-byte aligned, a multiple of 8 columns, that fit the register-resident kernel, with a positive
// eps (the unclamped rounding relies on max(scale, eps) not being denormal). Everything else --
// fp32 input, odd alignment, very wide rows -- takes the generic two-pass kernel.
int launch_rowwise(const RowwiseParams& p, int x_dtype, bool colabs, cudaStream_t stream) {
    const bool fast = x_dtype == QT_BF16 && p.vec_load && p.vec_store && p.eps >= 1e-30f && p.cols <= (colabs ? 16384 : 32768);
    if (fast) {
        if (colabs) return p.stochastic ? launch_rowwise_bf16<true, true>(p, stream) : launch_rowwise_bf16<true, false>(p, stream);
        return p.stochastic ? launch_rowwise_bf16<false, true>(p, stream) : launch_rowwise_bf16<false, false>(p, stream);
    }
    if (x_dtype == QT_BF16)
        return colabs ? launch_rowwise_generic<__nv_bfloat16, true>(p, stream) : launch_rowwise_generic<__nv_bfloat16, false>(p, stream);
    return colabs ? launch_rowwise_generic<float, true>(p, stream) : launch_rowwise_generic<float, false>(p, stream);
}

// 1 x 128 tiles through the lean row kernel; -1 when the row count is not a multiple of the CTA's rows.
template <int TPR, int VPT>
int launch_tile_1x128(const RowwiseParams& p, cudaStream_t stream) {
    constexpr int RPC = kThreads / TPR;
    constexpr int CTAS_PER_SM = VPT <= 4 ? 4 : 2;
    if (p.rows % RPC != 0) return -1;
    const int64_t want = p.rows / RPC;
    const int64_t cap = (int64_t)num_sms() * CTAS_PER_SM;
    rowwise_full_kernel<TPR, VPT, false, false, true><<<(unsigned)(want < cap ? want : cap), kThreads, 0, stream>>>(p);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

// Producer forms through the lean row kernel (bf16, 16-byte aligned rows, cols a multiple of 8 and at most
// 16384, rows a multiple of the CTA's rows). With q null only the bf16 result is written.
template <int TPR, int VPT, int PRODUCER>
int launch_producer_cfg(const RowwiseParams& p, cudaStream_t stream) {
    constexpr int RPC = kThreads / TPR;
    constexpr int CTAS_PER_SM = VPT <= 4 ? QT_PRODUCER_CTAS : 1;
    if (p.rows % RPC != 0)
        return fail(QT_ERR_UNSUPPORTED, "fused producer: %lld rows are not a multiple of %d (rows per CTA at this width)", (long long)p.rows, RPC);
    const int64_t want = p.rows / RPC;
    const int64_t cap = (int64_t)num_sms() * CTAS_PER_SM;
    int64_t grid = want < cap ? want : cap;
    if (p.q) {
        grid = (grid + kClusterSize - 1) / kClusterSize * kClusterSize;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3(kThreads);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = kClusterSize;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        QT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, rowwise_full_kernel<TPR, VPT, true, false, false, PRODUCER>, p));
    } else {
        rowwise_full_kernel<TPR, VPT, false, false, false, PRODUCER><<<(unsigned)grid, kThreads, 0, stream>>>(p);
        QT_CUDA_CHECK(cudaGetLastError());
    }
    return QT_OK;
}

template <int PRODUCER>
int launch_producer(const RowwiseParams& p, cudaStream_t stream) {
    const int64_t c = p.cols;
    if (c <= 256) return launch_producer_cfg<32, 1, PRODUCER>(p, stream);
    if (c <= 512) return launch_producer_cfg<32, 2, PRODUCER>(p, stream);
    if (c <= 1024) return launch_producer_cfg<32, 4, PRODUCER>(p, stream);
    if (c <= 2048) return launch_producer_cfg<64, 4, PRODUCER>(p, stream);
    if (c <= 4096) return launch_producer_cfg<128, 4, PRODUCER>(p, stream);
    if (c <= 8192) return launch_producer_cfg<256, 4, PRODUCER>(p, stream);
    return launch_producer_cfg<256, 8, PRODUCER>(p, stream);
}

int producer_args(RowwiseParams& p, const void* x, int64_t rows, int64_t cols, int64_t stride, void* y, void* q, int q_dtype,
                  void* scale, int scale_dtype, float* col_absmax, float eps, cudaStream_t stream, const char* who) {
    QT_REQUIRE(rows >= 0 && cols >= 0 && stride >= cols, "%s: bad shape/stride", who);
    QT_REQUIRE(q_dtype == QT_I8 || q_dtype == QT_E4M3 || q_dtype == QT_E5M2, "%s: q_dtype must be QT_I8, QT_E4M3 or QT_E5M2 (got %d)", who, q_dtype);
    QT_REQUIRE(scale_dtype == QT_BF16 || scale_dtype == QT_F32, "%s: scale_dtype must be QT_BF16 or QT_F32 (got %d)", who, scale_dtype);
    if (q) QT_REQUIRE(scale && col_absmax, "%s: q given without scale / col_absmax", who);
    if (q && cols > 0) QT_CUDA_CHECK(cudaMemsetAsync(col_absmax, 0, sizeof(float) * cols, stream));
    if (rows == 0 || cols == 0) return QT_OK;
    QT_REQUIRE(x && y, "%s: null pointer", who);
    if (cols % 8 != 0 || cols > 16384 || rows >= ((int64_t)1 << 30) || !aligned_to(x, 16) || (stride * 2) % 16 != 0 || !aligned_to(y, 16) ||
        (q && !aligned_to(q, 8)) || eps < 1e-30f)
        return fail(QT_ERR_UNSUPPORTED, "%s: needs 16-byte aligned bf16 rows, cols a multiple of 8 and at most 16384, eps >= 1e-30", who);
    p.x = x; p.rows = rows; p.cols = cols; p.stride = stride;
    p.y = reinterpret_cast<__nv_bfloat16*>(y); p.q = reinterpret_cast<uint8_t*>(q); p.scale = scale; p.col_absmax = col_absmax;
    p.q_dtype = q_dtype; p.scale_dtype = scale_dtype; p.eps = eps; p.vec_load = 1; p.vec_store = 1;
    QT_GUARD_INIT(p.guard);
    QT_GUARD_ADD(p.guard, y, rows * cols * 2);
    QT_GUARD_ADD(p.guard, q, rows * cols);
    QT_GUARD_ADD(p.guard, scale, rows * (scale_dtype == QT_BF16 ? 2 : 4));
    QT_GUARD_ADD(p.guard, col_absmax, cols * 4);
    return QT_OK;
}

int check_quant_args(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t stride, const void* q,
                     int q_dtype, const void* scale, int scale_dtype) {
    QT_REQUIRE(x_dtype == QT_BF16 || x_dtype == QT_F32, "quantize: x_dtype must be QT_BF16 or QT_F32 (got %d)", x_dtype);
    QT_REQUIRE(q_dtype == QT_I8 || q_dtype == QT_E4M3 || q_dtype == QT_E5M2, "quantize: q_dtype must be QT_I8, QT_E4M3 or QT_E5M2 (got %d)", q_dtype);
    QT_REQUIRE(scale_dtype == QT_BF16 || scale_dtype == QT_F32, "quantize: scale_dtype must be QT_BF16 or QT_F32 (got %d)", scale_dtype);
    QT_REQUIRE(rows >= 0 && cols >= 0, "quantize: negative shape (%lld, %lld)", (long long)rows, (long long)cols);
    QT_REQUIRE(stride >= cols, "quantize: row stride %lld smaller than cols %lld", (long long)stride, (long long)cols);
    if (rows > 0 && cols > 0) QT_REQUIRE(x && q && scale, "quantize: null pointer");
    return QT_OK;
}

int quantize_rowwise_impl(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t stride, void* q,
                          int q_dtype, void* scale, int scale_dtype, float* col_absmax, bool want_colabs,
                          float eps, int stochastic, uint64_t seed, uint64_t offset, void* stream_) {
    if (int rc = check_quant_args(x, x_dtype, rows, cols, stride, q, q_dtype, scale, scale_dtype)) return rc;
    QT_REQUIRE(!stochastic || q_dtype == QT_I8, "quantize: stochastic rounding is defined for int8 output only");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (want_colabs) {
        QT_REQUIRE(col_absmax || cols == 0, "quantize: col_absmax is null");
        if (cols > 0) QT_CUDA_CHECK(cudaMemsetAsync(col_absmax, 0, sizeof(float) * cols, stream));
    }
    if (rows == 0 || cols == 0) return QT_OK;

    RowwiseParams p = {};
    p.x = x; p.rows = rows; p.cols = cols; p.stride = stride;
    p.q = reinterpret_cast<uint8_t*>(q); p.scale = scale; p.col_absmax = col_absmax;
    p.q_dtype = q_dtype; p.scale_dtype = scale_dtype; p.eps = eps; p.stochastic = stochastic;
    p.seed = seed; p.offset = offset; p.keys = philox_keys(seed);
    const size_t esz = x_dtype == QT_BF16 ? 2 : 4;
    p.vec_load = aligned_to(x, 16) && ((stride * esz) % 16 == 0);
    p.vec_store = aligned_to(q, 8) && (cols % 8 == 0);
    QT_GUARD_INIT(p.guard);
    QT_GUARD_ADD(p.guard, q, rows * cols);
    QT_GUARD_ADD(p.guard, scale, rows * (scale_dtype == QT_BF16 ? 2 : 4));
    if (want_colabs) QT_GUARD_ADD(p.guard, col_absmax, cols * 4);

    return launch_rowwise(p, x_dtype, want_colabs, stream);
}

// ---- column absmax --------------------------------------------------------------------------

// bf16 fast path: a CTA covers 256 columns (lane = 8 columns = 16 bytes, so a warp reads 512
// contiguous bytes of a row) x a slab of rows (warp w takes rows w, w+8, ...; four rows in flight
// per thread). Packed bf16 maxima; shared-memory fold over the 8 warps; one atomic per column per CTA.
__global__ void __launch_bounds__(kThreads) col_absmax_bf16_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows,
                                                                    int64_t cols, int64_t stride, float* __restrict__ out,
                                                                    int64_t rows_per_cta) {
    __shared__ uint32_t s_m[kThreads / 32][32 * 4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t col = (int64_t)blockIdx.x * 256 + lane * 8;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_cta;
    const int64_t r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
    uint32_t m[4] = {0u, 0u, 0u, 0u};
    if (col < cols) {
        const bool full = col + 8 <= cols;
        int64_t r = r0 + warp;
        for (; r + 24 < r1; r += 32) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (full) v[j] = *reinterpret_cast<const uint4*>(x + (r + 8 * j) * stride + col);
                else { Vec8<__nv_bfloat16> t; load_vec8<__nv_bfloat16>(t, x + (r + 8 * j) * stride, col, cols, false); v[j] = t.raw; }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                m[0] = amax2(m[0], v[j].x); m[1] = amax2(m[1], v[j].y);
                m[2] = amax2(m[2], v[j].z); m[3] = amax2(m[3], v[j].w);
            }
        }
        for (; r < r1; r += 8) {
            uint4 v;
            if (full) v = *reinterpret_cast<const uint4*>(x + r * stride + col);
            else { Vec8<__nv_bfloat16> t; load_vec8<__nv_bfloat16>(t, x + r * stride, col, cols, false); v = t.raw; }
            m[0] = amax2(m[0], v.x); m[1] = amax2(m[1], v.y);
            m[2] = amax2(m[2], v.z); m[3] = amax2(m[3], v.w);
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) s_m[warp][lane * 4 + k] = m[k] & 0x7FFF7FFFu;   // amax2 leaves the sign bits undefined
    __syncthreads();
    if (threadIdx.x < 128) {
        uint32_t f = 0u;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) f = max2(f, s_m[w][threadIdx.x]);
        const int64_t c0 = (int64_t)blockIdx.x * 256 + threadIdx.x * 2;
        if (c0 < cols) atomicMax(reinterpret_cast<unsigned int*>(out + c0), f << 16);
        if (c0 + 1 < cols) atomicMax(reinterpret_cast<unsigned int*>(out + c0 + 1), f & 0xFFFF0000u);
    }
}

// Generic path (fp32 input or unaligned rows): a strip of 256*8 columns x a slab of rows per CTA;
// threads hold 8 column maxima in registers, then one atomic max per column per CTA.
template <typename XT>
__global__ void __launch_bounds__(kThreads) col_absmax_kernel(const XT* __restrict__ x, int64_t rows, int64_t cols,
                                                               int64_t stride, float* __restrict__ out,
                                                               int64_t rows_per_cta, int vec_ok) {
    const int64_t col = ((int64_t)blockIdx.x * kThreads + threadIdx.x) * 8;
    if (col >= cols) return;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_cta;
    const int64_t r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
    float m[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) m[k] = 0.0f;
    int64_t r = r0;
    for (; r + 4 <= r1; r += 4) {
        Vec8<XT> v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) load_vec8<XT>(v[j], x + (r + j) * stride, col, cols, vec_ok != 0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float f[8];
            v[j].unpack(f);
#pragma unroll
            for (int k = 0; k < 8; ++k) m[k] = fmaxf(m[k], fabsf(f[k]));
        }
    }
    for (; r < r1; ++r) {
        Vec8<XT> v;
        float f[8];
        load_vec8<XT>(v, x + r * stride, col, cols, vec_ok != 0);
        v.unpack(f);
#pragma unroll
        for (int k = 0; k < 8; ++k) m[k] = fmaxf(m[k], fabsf(f[k]));
    }
#pragma unroll
    for (int k = 0; k < 8; ++k)
        if (col + k < cols) atomicMax(reinterpret_cast<unsigned int*>(out + col + k), __float_as_uint(m[k]));
}

// ---- column-wise quantize + transpose ---------------------------------------------------------

struct ColwiseParams {
    QT_GUARD_FIELD
    const void* x;
    int64_t rows, cols, stride;
    int64_t tiles_per_cta;  // consecutive 128-row tiles handled by one CTA
    const float* col_absmax;
    uint8_t* qt;
    void* scale;
    int q_dtype, scale_dtype;
    float eps;
    int stochastic;
    uint64_t seed, offset;
    int vec_load, vec_store;
};

// Tile = 128 rows x 64 columns of x. Thread (rq, cg) reads 4 consecutive rows x 8 columns,
// quantizes with the 8 column scales, packs the 4 row-consecutive bytes of each column into one
// word and parks it in shared memory; warps then stream each output row (128 bytes of the
// transposed tensor) to HBM. x is read once, qt written once.
constexpr int kTileR = 128, kTileC = 64;

template <typename XT, bool EXACT_DIV>
__global__ void __launch_bounds__(kThreads, 3) colwise_t_kernel(const ColwiseParams p) {
    // two tile buffers: tile i+1 is written while tile i is still being streamed out, one barrier per tile
    __shared__ uint32_t s_tile[2][kTileC][kTileR / 4 + 1];
    const XT* x = reinterpret_cast<const XT*>(p.x);
    const float qmax = qmax_of(p.q_dtype);
    const int cg = threadIdx.x & 7;   // column group (8 columns)
    const int rq = threadIdx.x >> 3;  // row quad (4 rows)
    const int64_t c0 = (int64_t)blockIdx.x * kTileC;
    const int64_t col = c0 + cg * 8;
    const bool rne_i8 = p.q_dtype == QT_I8 && !p.stochastic;

    // dividers for this thread's 8 columns (one correctly rounded reciprocal each, hoisted)
    float dsc[8], rcp[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float am = (col + k < p.cols) ? p.col_absmax[col + k] : 0.0f;
        const float sc = div_rn(am, qmax);
        dsc[k] = fmaxf(sc, p.eps);
        rcp[k] = EXACT_DIV ? 0.0f : recip_rn(dsc[k]);
        if (blockIdx.y == 0 && rq == 0 && col + k < p.cols) QT_STORE_SCALE(p.guard, p.scale, p.scale_dtype, col + k, sc, 14);
    }

    // A CTA walks `tiles_per_cta` consecutive row tiles of its column strip, so the 128-byte output
    // segments of one transposed row are written back to back, and the next tile's loads are in
    // flight while the current one is quantized (register double buffer).
    auto load_tile = [&](Vec8<XT> (&v)[4], int64_t rb) {
        const int64_t r0 = rb * kTileR + rq * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (r0 + j < p.rows && col < p.cols) load_vec8<XT>(v[j], x + (r0 + j) * p.stride, col, p.cols, p.vec_load != 0);
            else v[j].zero();
        }
    };
    const int64_t rb_begin = (int64_t)blockIdx.y * p.tiles_per_cta;
    int64_t rb_end = rb_begin + p.tiles_per_cta;
    const int64_t row_tiles = (p.rows + kTileR - 1) / kTileR;
    if (rb_end > row_tiles) rb_end = row_tiles;
    Vec8<XT> v[4], vn[4];
    if (rb_begin < rb_end) load_tile(v, rb_begin);
    for (int64_t rb = rb_begin; rb < rb_end; ++rb) {
        const int64_t r0 = rb * kTileR + rq * 4;
        uint32_t (*tile)[kTileR / 4 + 1] = s_tile[(rb - rb_begin) & 1];
        if (rb + 1 < rb_end) load_tile(vn, rb + 1);
        float f[4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j].unpack(f[j]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            Divider<EXACT_DIV> div(dsc[k], rcp[k]);
            float q[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) q[j] = div(f[j][k]);
            uint32_t word;
            if (rne_i8) {
                // saturating: col_absmax comes from the caller, not from this pass
                word = pack4_sat(q[0], q[1], q[2], q[3]);
            } else {
                word = 0;
                if (p.q_dtype == QT_I8) {
                    float u[4];
                    uniforms4(u, (col + k) * p.rows + r0, p.seed, p.offset);
#pragma unroll
                    for (int j = 0; j < 4; ++j) word |= int8_sr(q[j], u[j]) << (8 * j);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        word |= quantize_byte(f[j][k] == 0.0f ? f[j][k] : q[j], p.q_dtype, false, 0.0f) << (8 * j);
                }
            }
            tile[cg * 8 + k][rq] = word;
        }
        __syncthreads();
        // 8 warps x 8 output rows each; lane l carries bytes [4l, 4l+4) of the 128-byte row segment
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
        for (int i = 0; i < kTileC / 8; ++i) {
            const int cc = warp * (kTileC / 8) + i;
            const int64_t oc = c0 + cc;
            const int64_t orow0 = rb * kTileR + lane * 4;
            if (oc < p.cols && orow0 < p.rows) {
                const uint32_t word = tile[cc][lane];
                uint8_t* dst = p.qt + oc * p.rows + orow0;
                if (orow0 + 4 <= p.rows && p.vec_store) {
                    if (QT_GUARD_OK(p.guard, dst, 4, 15)) *reinterpret_cast<uint32_t*>(dst) = word;
                } else {
                    for (int j = 0; j < 4 && orow0 + j < p.rows; ++j)
                        if (QT_GUARD_OK(p.guard, dst + j, 1, 16)) dst[j] = (uint8_t)((word >> (8 * j)) & 0xFFu);
                }
            }
        }
        // no second barrier: the next tile goes to the other buffer, and the barrier of that iteration
        // orders these reads before the writes of the iteration after it
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = vn[j];
    }
}

// The common case of the same operation with everything that costs instructions removed: bf16 input,
// int8 round-half-even output, whole tiles only (rows % 128 == 0, cols % 64 == 0), 16-byte aligned rows.
// The generic kernel above issues 16 instructions per element and is bound by instruction issue
// (issue slots 67 % busy at 3.5 TB/s); here pointers advance instead of being recomputed, there are no
// bounds checks, the tile loop is unrolled by two so the prefetched registers are never copied, and the
// shared-memory tile is swizzled so that both its writes and its reads are free of bank conflicts.
__global__ void __launch_bounds__(kThreads, 3) colwise_t_fast_kernel(const ColwiseParams p) {
    __shared__ uint32_t s_tile[2][kTileC][kTileR / 4 + 1];
    const int cg = threadIdx.x & 7;   // column group (8 columns)
    const int rq = threadIdx.x >> 3;  // row quad (4 rows)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t c0 = (int64_t)blockIdx.x * kTileC;
    const int64_t col = c0 + cg * 8;

    float dsc[8], rcp[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float sc = div_rn(p.col_absmax[col + k], 127.0f);
        dsc[k] = fmaxf(sc, p.eps);
        rcp[k] = recip_rn(dsc[k]);
        if (blockIdx.y == 0 && rq == 0) QT_STORE_SCALE(p.guard, p.scale, p.scale_dtype, col + k, sc, 17);
    }

    const int64_t row_tiles = p.rows / kTileR;
    const int64_t rb_begin = (int64_t)blockIdx.y * p.tiles_per_cta;
    int64_t rb_end = rb_begin + p.tiles_per_cta;
    if (rb_end > row_tiles) rb_end = row_tiles;
    const int n_tiles = (int)(rb_end - rb_begin);
    if (n_tiles <= 0) return;

    // this thread's 4 rows x 8 columns of the current tile, as 16-byte vectors; `src` walks down the strip
    const int64_t pitch16 = p.stride / 8;                      // row pitch in 16-byte units
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.x) + (rb_begin * kTileR + rq * 4) * p.stride + col);
    const int64_t tile16 = (int64_t)kTileR * pitch16;
    // output: warp w streams rows w, w + 8, ... of the transposed tile, lane l the l-th 4-byte word
    uint8_t* dst = p.qt + (c0 + warp) * p.rows + rb_begin * kTileR + lane * 4;
    const int64_t dst_step = 8 * p.rows;
    // word position inside a tile row: columns 32..63 swap 4-word groups, which makes the 8 x 4 threads
    // of a warp hit 32 different banks when they park their words (row pitch 33 words)
    const int st_word = rq ^ ((cg >> 2) << 2);

    auto load_tile = [&](uint4 (&v)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = src[j * pitch16];
        src += tile16;
    };
    auto quantize_tile = [&](const uint4 (&v)[4], uint32_t (*tile)[kTileR / 4 + 1]) {
#pragma unroll
        for (int k2 = 0; k2 < 4; ++k2) {
            // columns 2*k2 and 2*k2 + 1 are the two halves of one loaded word: one packed division per row
            const Divider2 div(dsc[2 * k2], rcp[2 * k2], dsc[2 * k2 + 1], rcp[2 * k2 + 1]);
            float2 q[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t w = k2 == 0 ? v[j].x : (k2 == 1 ? v[j].y : (k2 == 2 ? v[j].z : v[j].w));
                q[j] = div(unpack_bf16x2(w));
            }
            // saturating: col_absmax is the caller's
            tile[cg * 8 + 2 * k2][st_word] = pack4_sat(q[0].x, q[1].x, q[2].x, q[3].x);
            tile[cg * 8 + 2 * k2 + 1][st_word] = pack4_sat(q[0].y, q[1].y, q[2].y, q[3].y);
        }
    };
    auto store_tile = [&](uint32_t (*tile)[kTileR / 4 + 1]) {
        uint8_t* d = dst;
#pragma unroll
        for (int i = 0; i < kTileC / 8; ++i) {
            const int cc = i * 8 + warp;
            if (QT_GUARD_OK(p.guard, d, 4, 18)) *reinterpret_cast<uint32_t*>(d) = tile[cc][lane ^ ((cc >> 5) << 2)];
            d += dst_step;
        }
        dst += kTileR;
    };

    uint4 a[4], b[4];
    load_tile(a);
    for (int t = 0; t < n_tiles; t += 2) {
        if (t + 1 < n_tiles) load_tile(b);
        quantize_tile(a, s_tile[0]);
        __syncthreads();   // one barrier per tile: the other buffer is written next, and that tile's
        store_tile(s_tile[0]);   // barrier orders these reads before this buffer is written again
        if (t + 1 < n_tiles) {
            if (t + 2 < n_tiles) load_tile(a);
            quantize_tile(b, s_tile[1]);
            __syncthreads();
            store_tile(s_tile[1]);
        }
    }
}

// Column-wise quantize WITHOUT the transpose: q[r][c] = round(x[r][c] / max(absmax[c] / qmax, eps)),
// one scale per column. This is the form a row-sharded weight takes for the grad-input GEMM (the
// reference quantizes the weight along its output dimension there, subclasses/mixed_precision.py:176-178
// through :102): every rank quantizes its own rows with column maxima agreed across the ranks, and the
// gathered rows are then bit-identical to quantizing the whole weight. Weights are small next to the
// activations, so this kernel is plain: one thread per 8 consecutive columns of a row, IEEE divisions.
template <typename XT>
__global__ void __launch_bounds__(kThreads) colwise_kernel(const ColwiseParams p) {
    const XT* x = reinterpret_cast<const XT*>(p.x);
    const float qmax = qmax_of(p.q_dtype);
    const int64_t nv = (p.cols + 7) / 8;
    const int64_t total = (p.rows > 0 ? p.rows : 1) * nv;
    for (int64_t idx = (int64_t)blockIdx.x * kThreads + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * kThreads) {
        const int64_t row = idx / nv, c0 = (idx - row * nv) * 8;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int64_t c = c0 + k;
            if (c >= p.cols) break;
            const float sc = div_rn(p.col_absmax[c], qmax);
            if (row == 0) QT_STORE_SCALE(p.guard, p.scale, p.scale_dtype, c, sc, 19);
            if (row < p.rows) {
                const float v = div_rn(to_float<XT>(x[row * p.stride + c]), fmaxf(sc, p.eps));
                const int64_t at = row * p.cols + c;
                const float u = p.stochastic ? uniform1(at, p.seed, p.offset) : 0.0f;
                if (QT_GUARD_OK(p.guard, p.qt + at, 1, 22)) p.qt[at] = (uint8_t)quantize_byte(v, p.q_dtype, p.stochastic != 0, u);
            }
        }
    }
}

// ---- tile-wise ------------------------------------------------------------------------------

struct TileParams {
    QT_GUARD_FIELD
    const void* x;
    int64_t rows, cols, stride;
    uint8_t* q;
    void* scale;
    int64_t scale_cols;
    int q_dtype, scale_dtype;
    float eps;
    int vec_load, vec_store;
};

// 1 x 128 tiles: 16 lanes own one tile (8 elements each). `tpr` threads (a power of two, 16..256)
// span a row chunk of tpr*8 columns, the CTA's other threads take further rows; a work item is
// 4 such row groups, so four 16-byte loads are in flight per thread and the next item's loads are
// issued before the current one is reduced and quantized.
template <typename XT, bool EXACT_DIV>
__global__ void __launch_bounds__(kThreads) tile_1x128_kernel(const TileParams p, int tpr_log2) {
    constexpr int ROWS = 4;
    const XT* x = reinterpret_cast<const XT*>(p.x);
    const float qmax = qmax_of(p.q_dtype);
    const int l16 = threadIdx.x & 15;
    const float zero_u[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int tpr = 1 << tpr_log2;
    const int rpp = kThreads >> tpr_log2;            // rows per pass
    const int sub = threadIdx.x >> tpr_log2, t = threadIdx.x & (tpr - 1);
    // an item is 4 x rpp rows by tpr x 8 columns (8192 elements): their count always fits 32 bits, and
    // 32-bit divisions keep the per-item index arithmetic cheap (64-bit ones are emulated)
    const uint32_t chunks = (uint32_t)((p.cols + tpr * 8 - 1) / (tpr * 8));
    const uint32_t row_blocks = (uint32_t)((p.rows + ROWS * rpp - 1) / (ROWS * rpp));
    const uint32_t items = row_blocks * chunks;

    auto load_item = [&](Vec8<XT> (&v)[ROWS], uint32_t item) {
        const uint32_t rblk = item / chunks, chunk = item - rblk * chunks;
        const int64_t col = ((int64_t)chunk * tpr + t) * 8;
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            const int64_t row = ((int64_t)rblk * ROWS + j) * rpp + sub;
            if (row < p.rows && col < p.cols) load_vec8<XT>(v[j], x + row * p.stride, col, p.cols, p.vec_load != 0);
            else v[j].zero();
        }
    };

    Vec8<XT> v[ROWS], vn[ROWS];
    uint32_t item = blockIdx.x;
    if (item < items) load_item(v, item);
    for (; item < items; item += gridDim.x) {
        if (item + gridDim.x < items) load_item(vn, item + gridDim.x);
        const uint32_t rblk = item / chunks, chunk = item - rblk * chunks;
        const int64_t col = ((int64_t)chunk * tpr + t) * 8;
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            const int64_t row = ((int64_t)rblk * ROWS + j) * rpp + sub;
            float f[8];
            v[j].unpack(f);
            float amax = 0.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(f[k]));
            // all 16 lanes of a tile take part (out-of-range lanes hold zeros)
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
            const float sc = div_rn(amax, qmax);
            const Divider<EXACT_DIV> div(fmaxf(sc, p.eps));
            if (row < p.rows && col < p.cols) {
                if (l16 == 0) QT_STORE_SCALE(p.guard, p.scale, p.scale_dtype, row * p.scale_cols + (col >> 7), sc, 23);
                uint2 bytes;
                if constexpr (sizeof(XT) == 2 && !EXACT_DIV) {
                    bytes = quantize_vec8<false>(v[j].raw, Divider2(div.d, div.r, div.d, div.r), p.q_dtype, 0, PhiloxKeys{}, 0);
                } else {
                    divide8(f, div, p.q_dtype != QT_I8);
                    bytes = pack8(f, p.q_dtype, false, zero_u);
                }
                if (QT_GUARD_OK(p.guard, p.q + row * p.cols + col, (int)((p.cols - col) < 8 ? (p.cols - col) : 8), 20))
                    store_bytes8(p.q, row * p.cols + col, p.cols - col, bytes, p.vec_store != 0);
            }
        }
#pragma unroll
        for (int j = 0; j < ROWS; ++j) v[j] = vn[j];
    }
}

// 128 x 128 tiles: one CTA per tile; thread (r16, c16) holds 8 vectors (rows r16 + 16 i).
template <typename XT, bool EXACT_DIV>
__global__ void __launch_bounds__(kThreads) tile_128x128_kernel(const TileParams p) {
    __shared__ float s_red[kThreads / 32];
    const XT* x = reinterpret_cast<const XT*>(p.x);
    const float qmax = qmax_of(p.q_dtype);
    const int64_t tile_c = blockIdx.x, tile_r = blockIdx.y;
    const int c16 = threadIdx.x & 15, r16 = threadIdx.x >> 4;
    const int64_t col = tile_c * 128 + c16 * 8;
    const float zero_u[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    Vec8<XT> v[8];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t row = tile_r * 128 + r16 + 16 * i;
        if (row < p.rows && col < p.cols) load_vec8<XT>(v[i], x + row * p.stride, col, p.cols, p.vec_load != 0);
        else v[i].zero();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float f[8];
        v[i].unpack(f);
#pragma unroll
        for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(f[k]));
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = s_red[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) amax = fmaxf(amax, s_red[w]);
    const float sc = __fdiv_rn(amax, qmax);
    const Divider<EXACT_DIV> div(fmaxf(sc, p.eps));
    if (threadIdx.x == 0) QT_STORE_SCALE(p.guard, p.scale, p.scale_dtype, tile_r * p.scale_cols + tile_c, sc, 24);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t row = tile_r * 128 + r16 + 16 * i;
        if (row < p.rows && col < p.cols) {
            uint2 bytes;
            if constexpr (sizeof(XT) == 2 && !EXACT_DIV) {
                bytes = quantize_vec8<false>(v[i].raw, Divider2(div.d, div.r, div.d, div.r), p.q_dtype, 0, PhiloxKeys{}, 0);
            } else {
                float f[8];
                v[i].unpack(f);
                divide8(f, div, p.q_dtype != QT_I8);
                bytes = pack8(f, p.q_dtype, false, zero_u);
            }
            if (QT_GUARD_OK(p.guard, p.q + row * p.cols + col, (int)((p.cols - col) < 8 ? (p.cols - col) : 8), 21))
                store_bytes8(p.q, row * p.cols + col, p.cols - col, bytes, p.vec_store != 0);
        }
    }
}

// 128 x 128 tiles, the same common case (bf16, rows and cols multiples of 128, aligned): a CTA walks
// tiles with a register double buffer; thread (r16, c16) holds 8 vectors of a tile (rows r16 + 16 i).
__global__ void __launch_bounds__(kThreads, 2) tile_128x128_fast_kernel(const TileParams p) {
    __shared__ uint32_t s_red[2][kThreads / 32];
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(p.x);
    const float qmax = qmax_of(p.q_dtype);
    const float rqmax = p.q_dtype == QT_I8 ? (1.0f / 127.0f) : (p.q_dtype == QT_E4M3 ? (1.0f / 448.0f) : (1.0f / 57344.0f));
    const int c16 = threadIdx.x & 15, r16 = threadIdx.x >> 4;
    const uint32_t tiles_c = (uint32_t)p.scale_cols;
    const uint32_t tiles = (uint32_t)(p.rows / 128) * tiles_c;
    const int64_t pitch16 = p.stride / 8;   // row pitch in 16-byte units

    auto load_tile = [&](uint4 (&v)[8], uint32_t tile) {
        const uint32_t tr = tile / tiles_c, tc = tile - tr * tiles_c;
        const uint4* src = reinterpret_cast<const uint4*>(x + ((int64_t)tr * 128 + r16) * p.stride + (int64_t)tc * 128 + c16 * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = src[(int64_t)i * 16 * pitch16];
    };
    auto process = [&](const uint4 (&v)[8], uint32_t tile, int parity) {
        const uint32_t tr = tile / tiles_c, tc = tile - tr * tiles_c;
        uint32_t m2 = 0u;
#pragma unroll
        for (int i = 0; i < 8; ++i) m2 = amax2(m2, amax2(amax2(v[i].x, v[i].y), amax2(v[i].z, v[i].w)));
        uint32_t abits = __reduce_max_sync(0xFFFFFFFFu, fold_halves(m2));
        if ((threadIdx.x & 31) == 0) s_red[parity][threadIdx.x >> 5] = abits;
        __syncthreads();   // one barrier per tile: the next tile uses the other slot
        abits = s_red[parity][0];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) { const uint32_t o = s_red[parity][w]; abits = o > abits ? o : abits; }
        const float sc = scale_of(__uint_as_float(abits), qmax, rqmax);
        const Divider2 div(fmaxf(sc, p.eps));
        if (threadIdx.x == 0) QT_STORE_SCALE(p.guard, p.scale, p.scale_dtype, (int64_t)tr * p.scale_cols + tc, sc, 25);
        uint8_t* dst = p.q + ((int64_t)tr * 128 + r16) * p.cols + (int64_t)tc * 128 + c16 * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (QT_GUARD_OK(p.guard, dst + (int64_t)i * 16 * p.cols, 8, 26))
                *reinterpret_cast<uint2*>(dst + (int64_t)i * 16 * p.cols) = quantize_vec8<false>(v[i], div, p.q_dtype, 0, PhiloxKeys{}, 0);
    };

    uint4 a[8], b[8];
    uint32_t tile = blockIdx.x;
    if (tile < tiles) load_tile(a, tile);
    while (tile < tiles) {
        if (tile + gridDim.x < tiles) load_tile(b, tile + gridDim.x);
        process(a, tile, 0);
        tile += gridDim.x;
        if (tile >= tiles) break;
        if (tile + gridDim.x < tiles) load_tile(a, tile + gridDim.x);
        process(b, tile, 1);
        tile += gridDim.x;
    }
}

// ---- exhaustive check of the reciprocal division ------------------------------------------------

// For every non-negative finite bf16 absmax a (blockIdx) and every finite bf16 x with |x| <= a,
// compare Divider<false> with div.rn for d = max(a / qmax, eps).
__global__ void division_selftest_kernel(int q_dtype, float eps, unsigned long long* mismatches) {
    const float qmax = qmax_of(q_dtype);
    unsigned long long bad = 0, bad_q = 0;
    for (uint32_t abits = blockIdx.x; abits < 0x7F80u; abits += gridDim.x) {
        const float a = bf16_bits_to_float(abits);
        const float d = fmaxf(__fdiv_rn(a, qmax), eps);
        const Divider<false> fast(d);
        const Divider2 fast2(d);
        // the scale itself: constant-reciprocal sequence against div.rn
        if (threadIdx.x == 0) {
            const float rq = q_dtype == QT_I8 ? (1.0f / 127.0f) : (q_dtype == QT_E4M3 ? (1.0f / 448.0f) : (1.0f / 57344.0f));
            bad += (__float_as_uint(scale_of(a, qmax, rq)) != __float_as_uint(__fdiv_rn(a, qmax)));
        }
        for (uint32_t xb = threadIdx.x; xb <= abits; xb += blockDim.x) {
            const float x = bf16_bits_to_float(xb);
            const float want = __fdiv_rn(x, d);
            // the fp8 paths pass zero inputs through (the reciprocal sequence loses the sign of -0)
            const bool keep = (q_dtype != QT_I8) && x == 0.0f;
            const float got = keep ? x : fast(x);
            bad += (__float_as_uint(want) != __float_as_uint(got));
            const float want_n = __fdiv_rn(-x, d), got_n = keep ? -x : fast(-x);
            bad += (__float_as_uint(want_n) != __float_as_uint(got_n));
            // the packed form used by the kernels: both lanes, both signs
            const float2 got2 = fast2(make_float2(x, -x));
            bad += (!keep && __float_as_uint(got2.x) != __float_as_uint(want)) + (!keep && __float_as_uint(got2.y) != __float_as_uint(want_n));
            bad_q += (quantize_byte(want, q_dtype, false, 0.f) != quantize_byte(got, q_dtype, false, 0.f));
            bad_q += (quantize_byte(want_n, q_dtype, false, 0.f) != quantize_byte(got_n, q_dtype, false, 0.f));
        }
    }
    if (bad) atomicAdd(mismatches, bad);
    if (bad_q) atomicAdd(mismatches + 1, bad_q);
}

}  // namespace

}  // namespace qt

// ---- C ABI ------------------------------------------------------------------------------------

using namespace qt;

extern "C" int qt_quantize_rowwise(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                                   void* q, int q_dtype, void* scale, int scale_dtype, float eps, int stochastic,
                                   uint64_t seed, uint64_t offset, void* stream) {
    return quantize_rowwise_impl(x, x_dtype, rows, cols, x_row_stride, q, q_dtype, scale, scale_dtype, nullptr, false,
                                 eps, stochastic, seed, offset, stream);
}

extern "C" int qt_quantize_rowwise_colabsmax(const void* x, int x_dtype, int64_t rows, int64_t cols,
                                             int64_t x_row_stride, void* q, int q_dtype, void* scale, int scale_dtype,
                                             float* col_absmax, float eps, int stochastic, uint64_t seed,
                                             uint64_t offset, void* stream) {
    return quantize_rowwise_impl(x, x_dtype, rows, cols, x_row_stride, q, q_dtype, scale, scale_dtype, col_absmax, true,
                                 eps, stochastic, seed, offset, stream);
}

extern "C" int qt_col_absmax(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                             float* col_absmax, void* stream_) {
    QT_REQUIRE(x_dtype == QT_BF16 || x_dtype == QT_F32, "col_absmax: x_dtype must be QT_BF16 or QT_F32 (got %d)", x_dtype);
    QT_REQUIRE(rows >= 0 && cols >= 0 && x_row_stride >= cols, "col_absmax: bad shape/stride");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (cols == 0) return QT_OK;
    QT_REQUIRE(col_absmax, "col_absmax: output is null");
    QT_CUDA_CHECK(cudaMemsetAsync(col_absmax, 0, sizeof(float) * cols, stream));
    if (rows == 0) return QT_OK;
    QT_REQUIRE(x, "col_absmax: x is null");
    const size_t esz = x_dtype == QT_BF16 ? 2 : 4;
    const int vec_ok = aligned_to(x, 16) && ((x_row_stride * esz) % 16 == 0);
    if (x_dtype == QT_BF16 && vec_ok) {
        const int64_t strips = (cols + 255) / 256;
        // enough row slabs to fill the machine about eight times over, at least 64 rows each
        int64_t slabs = ((int64_t)num_sms() * 8 + strips - 1) / strips;
        const int64_t max_slabs = (rows + 63) / 64;
        if (slabs > max_slabs) slabs = max_slabs;
        if (slabs < 1) slabs = 1;
        if (slabs > 65535) slabs = 65535;
        int64_t rows_per_cta = (rows + slabs - 1) / slabs;
        rows_per_cta = (rows_per_cta + 7) / 8 * 8;
        dim3 grid((unsigned)strips, (unsigned)((rows + rows_per_cta - 1) / rows_per_cta));
        col_absmax_bf16_kernel<<<grid, kThreads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), rows, cols, x_row_stride, col_absmax, rows_per_cta);
        QT_CUDA_CHECK(cudaGetLastError());
        return QT_OK;
    }
    const int64_t strips = (cols + kThreads * 8 - 1) / (kThreads * 8);
    int64_t slabs = ((int64_t)num_sms() * 8 + strips - 1) / strips;
    const int64_t max_slabs = (rows + 31) / 32;
    if (slabs > max_slabs) slabs = max_slabs;
    if (slabs < 1) slabs = 1;
    if (slabs > 65535) slabs = 65535;
    const int64_t rows_per_cta = (rows + slabs - 1) / slabs;
    dim3 grid((unsigned)strips, (unsigned)((rows + rows_per_cta - 1) / rows_per_cta));
    if (x_dtype == QT_BF16)
        col_absmax_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), rows, cols, x_row_stride, col_absmax, rows_per_cta, vec_ok);
    else
        col_absmax_kernel<float><<<grid, kThreads, 0, stream>>>(reinterpret_cast<const float*>(x), rows, cols, x_row_stride, col_absmax, rows_per_cta, vec_ok);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

extern "C" int qt_quantize_colwise_t(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                                     const float* col_absmax, void* qt_out, int q_dtype, void* scale, int scale_dtype,
                                     float eps, int stochastic, uint64_t seed, uint64_t offset, void* stream_) {
    if (int rc = check_quant_args(x, x_dtype, rows, cols, x_row_stride, qt_out, q_dtype, scale, scale_dtype)) return rc;
    QT_REQUIRE(!stochastic || q_dtype == QT_I8, "quantize: stochastic rounding is defined for int8 output only");
    if (cols == 0) return QT_OK;
    QT_REQUIRE(col_absmax, "quantize_colwise_t: col_absmax is null");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    ColwiseParams p;
    p.x = x; p.rows = rows; p.cols = cols; p.stride = x_row_stride; p.col_absmax = col_absmax;
    p.qt = reinterpret_cast<uint8_t*>(qt_out); p.scale = scale; p.q_dtype = q_dtype; p.scale_dtype = scale_dtype;
    p.eps = eps; p.stochastic = stochastic; p.seed = seed; p.offset = offset;
    const size_t esz = x_dtype == QT_BF16 ? 2 : 4;
    p.vec_load = aligned_to(x, 16) && ((x_row_stride * esz) % 16 == 0);
    p.vec_store = aligned_to(qt_out, 4) && (rows % 4 == 0);
    QT_GUARD_INIT(p.guard);
    QT_GUARD_ADD(p.guard, qt_out, rows * cols);
    QT_GUARD_ADD(p.guard, scale, cols * (scale_dtype == QT_BF16 ? 2 : 4));
    const int64_t col_tiles = (cols + kTileC - 1) / kTileC;
    int64_t row_tiles = (rows + kTileR - 1) / kTileR;
    if (row_tiles < 1) row_tiles = 1;  // rows == 0 still writes the (zero) scales
    // A CTA walks `per_cta` consecutive row tiles of one column strip. Three CTAs fit on an SM; pick
    // the walk length that wastes the least in the last, partly filled wave: cost = waves x (tiles per
    // CTA + the prologue that loads and inverts the column scales, about 0.7 of a tile).
    const int64_t slots = (int64_t)num_sms() * 3;
    int64_t per_cta = 1;
    double best = 1e300;
    for (int64_t cand = 1; cand <= 64 && cand <= row_tiles; ++cand) {
        const int64_t g = (row_tiles + cand - 1) / cand;
        if (g > 65535) continue;
        const int64_t waves = (col_tiles * g + slots - 1) / slots;
        const double cost = (double)waves * ((double)cand + 0.7);
        if (cost < best) { best = cost; per_cta = cand; }
    }
    int64_t groups = (row_tiles + per_cta - 1) / per_cta;
    while (groups > 65535) { per_cta *= 2; groups = (row_tiles + per_cta - 1) / per_cta; }
    p.tiles_per_cta = per_cta;
    dim3 grid((unsigned)col_tiles, (unsigned)groups);
    const bool fast = x_dtype == QT_BF16 && q_dtype == QT_I8 && !stochastic && eps >= 1e-30f && p.vec_load && p.vec_store &&
                      rows > 0 && rows % kTileR == 0 && cols % kTileC == 0;
    if (fast) colwise_t_fast_kernel<<<grid, kThreads, 0, stream>>>(p);
    else if (x_dtype == QT_BF16 && eps >= 1e-30f) colwise_t_kernel<__nv_bfloat16, false><<<grid, kThreads, 0, stream>>>(p);
    else if (x_dtype == QT_BF16) colwise_t_kernel<__nv_bfloat16, true><<<grid, kThreads, 0, stream>>>(p);
    else colwise_t_kernel<float, true><<<grid, kThreads, 0, stream>>>(p);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

extern "C" int qt_quantize_colwise(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                                   const float* col_absmax, void* q, int q_dtype, void* scale, int scale_dtype, float eps,
                                   int stochastic, uint64_t seed, uint64_t offset, void* stream_) {
    if (int rc = check_quant_args(x, x_dtype, rows, cols, x_row_stride, q, q_dtype, scale, scale_dtype)) return rc;
    QT_REQUIRE(!stochastic || q_dtype == QT_I8, "quantize: stochastic rounding is defined for int8 output only");
    if (cols == 0) return QT_OK;
    QT_REQUIRE(col_absmax && scale, "quantize_colwise: null pointer");
    ColwiseParams p = {};
    p.x = x; p.rows = rows; p.cols = cols; p.stride = x_row_stride; p.col_absmax = col_absmax;
    p.qt = reinterpret_cast<uint8_t*>(q); p.scale = scale; p.q_dtype = q_dtype; p.scale_dtype = scale_dtype;
    p.eps = eps; p.stochastic = stochastic; p.seed = seed; p.offset = offset;
    QT_GUARD_INIT(p.guard);
    QT_GUARD_ADD(p.guard, q, rows * cols);
    QT_GUARD_ADD(p.guard, scale, cols * (scale_dtype == QT_BF16 ? 2 : 4));
    const int64_t work = (rows > 0 ? rows : 1) * ((cols + 7) / 8);
    const int64_t want = (work + kThreads - 1) / kThreads, cap = (int64_t)num_sms() * 8;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (x_dtype == QT_BF16) colwise_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(p);
    else colwise_kernel<float><<<grid, kThreads, 0, stream>>>(p);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

extern "C" int qt_quantize_tile(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                                int tile_r, int tile_c, void* q, int q_dtype, void* scale, int scale_dtype, float eps,
                                void* stream_) {
    if (int rc = check_quant_args(x, x_dtype, rows, cols, x_row_stride, q, q_dtype, scale, scale_dtype)) return rc;
    if (!((tile_r == 1 || tile_r == 128) && tile_c == 128))
        return fail(QT_ERR_UNSUPPORTED, "quantize_tile: tile %dx%d not implemented (1x128 and 128x128 are)", tile_r, tile_c);
    if (rows == 0 || cols == 0) return QT_OK;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    TileParams p;
    p.x = x; p.rows = rows; p.cols = cols; p.stride = x_row_stride; p.q = reinterpret_cast<uint8_t*>(q);
    p.scale = scale; p.scale_cols = (cols + 127) / 128; p.q_dtype = q_dtype; p.scale_dtype = scale_dtype; p.eps = eps;
    const size_t esz = x_dtype == QT_BF16 ? 2 : 4;
    p.vec_load = aligned_to(x, 16) && ((x_row_stride * esz) % 16 == 0);
    p.vec_store = aligned_to(q, 8) && (cols % 8 == 0);
    QT_GUARD_INIT(p.guard);
    QT_GUARD_ADD(p.guard, q, rows * cols);
    QT_GUARD_ADD(p.guard, scale, ((rows + tile_r - 1) / tile_r) * p.scale_cols * (scale_dtype == QT_BF16 ? 2 : 4));
    const bool fast = x_dtype == QT_BF16 && eps >= 1e-30f && p.vec_load && p.vec_store && cols % 128 == 0;
    if (tile_r == 1 && fast && cols <= 16384 && rows < ((int64_t)1 << 30)) {
        RowwiseParams rp = {};
        rp.x = x; rp.rows = rows; rp.cols = cols; rp.stride = x_row_stride; rp.q = p.q; rp.scale = scale;
        rp.q_dtype = q_dtype; rp.scale_dtype = scale_dtype; rp.eps = eps;
        QT_GUARD_INIT(rp.guard);
        QT_GUARD_ADD(rp.guard, q, rows * cols);
        QT_GUARD_ADD(rp.guard, scale, rows * p.scale_cols * (scale_dtype == QT_BF16 ? 2 : 4));
        int rc = -1;
        if (cols <= 512) rc = launch_tile_1x128<32, 2>(rp, stream);
        else if (cols <= 1024) rc = launch_tile_1x128<32, 4>(rp, stream);
        else if (cols <= 2048) rc = launch_tile_1x128<64, 4>(rp, stream);
        else if (cols <= 4096) rc = launch_tile_1x128<128, 4>(rp, stream);
        else if (cols <= 8192) rc = launch_tile_1x128<256, 4>(rp, stream);
        else rc = launch_tile_1x128<256, 8>(rp, stream);
        if (rc >= 0) return rc;   // negative: the row count does not fit this kernel, fall through
    }
    if (tile_r == 128 && fast && rows % 128 == 0 && (rows / 128) * p.scale_cols < ((int64_t)1 << 31)) {
        const int64_t tiles = (rows / 128) * p.scale_cols;
        const int64_t cap = (int64_t)num_sms() * 2;
        tile_128x128_fast_kernel<<<(unsigned)(tiles < cap ? tiles : cap), kThreads, 0, stream>>>(p);
        QT_CUDA_CHECK(cudaGetLastError());
        return QT_OK;
    }
    if (tile_r == 1) {
        int tpr_log2 = 4;  // at least one 16-lane tile group per row
        while (tpr_log2 < 8 && ((int64_t)8 << tpr_log2) < cols) ++tpr_log2;
        const int tpr = 1 << tpr_log2, rpp = kThreads / tpr;
        const int64_t items = ((rows + 4 * rpp - 1) / (4 * rpp)) * ((cols + tpr * 8 - 1) / (tpr * 8));
        const int64_t cap = (int64_t)num_sms() * 6;
        const int grid = (int)(items < cap ? items : cap);
        if (x_dtype == QT_BF16 && eps >= 1e-30f) tile_1x128_kernel<__nv_bfloat16, false><<<grid, kThreads, 0, stream>>>(p, tpr_log2);
        else if (x_dtype == QT_BF16) tile_1x128_kernel<__nv_bfloat16, true><<<grid, kThreads, 0, stream>>>(p, tpr_log2);
        else tile_1x128_kernel<float, true><<<grid, kThreads, 0, stream>>>(p, tpr_log2);
    } else {
        const int64_t tr = (rows + 127) / 128;
        if (tr > 65535) return fail(QT_ERR_UNSUPPORTED, "quantize_tile: more than 65535 row tiles");
        dim3 grid((unsigned)p.scale_cols, (unsigned)tr);
        if (x_dtype == QT_BF16 && eps >= 1e-30f) tile_128x128_kernel<__nv_bfloat16, false><<<grid, kThreads, 0, stream>>>(p);
        else if (x_dtype == QT_BF16) tile_128x128_kernel<__nv_bfloat16, true><<<grid, kThreads, 0, stream>>>(p);
        else tile_128x128_kernel<float, true><<<grid, kThreads, 0, stream>>>(p);
    }
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

// ---- producer-fused activation quantize ---------------------------------------------------------------

extern "C" int qt_rmsnorm_quantize(const void* x, int64_t rows, int64_t cols, int64_t x_row_stride, const void* weight,
                                   float norm_eps, void* y, float* rstd, void* q, int q_dtype, void* scale, int scale_dtype,
                                   float* col_absmax, float eps, void* stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    RowwiseParams p = {};
    if (int rc = producer_args(p, x, rows, cols, x_row_stride, y, q, q_dtype, scale, scale_dtype, col_absmax, eps, stream, "rmsnorm_quantize")) return rc;
    if (rows == 0 || cols == 0) return QT_OK;
    QT_REQUIRE(weight, "rmsnorm_quantize: weight is null");
    if (!aligned_to(weight, 16)) return fail(QT_ERR_UNSUPPORTED, "rmsnorm_quantize: weight must be 16-byte aligned");
    p.w_norm = reinterpret_cast<const __nv_bfloat16*>(weight); p.norm_eps = norm_eps; p.rstd = rstd;
    QT_GUARD_ADD(p.guard, rstd, rows * 4);
    return launch_producer<1>(p, stream);
}

extern "C" int qt_silu_mul_quantize(const void* gate, const void* up, int64_t rows, int64_t cols, int64_t gate_row_stride,
                                    int64_t up_row_stride, void* y, void* q, int q_dtype, void* scale, int scale_dtype,
                                    float* col_absmax, float eps, void* stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    RowwiseParams p = {};
    if (int rc = producer_args(p, gate, rows, cols, gate_row_stride, y, q, q_dtype, scale, scale_dtype, col_absmax, eps, stream, "silu_mul_quantize")) return rc;
    if (rows == 0 || cols == 0) return QT_OK;
    QT_REQUIRE(up && up_row_stride >= cols, "silu_mul_quantize: bad second operand");
    if (!aligned_to(up, 16) || (up_row_stride * 2) % 16 != 0) return fail(QT_ERR_UNSUPPORTED, "silu_mul_quantize: the second operand's rows must be 16-byte aligned");
    p.x2 = reinterpret_cast<const __nv_bfloat16*>(up); p.stride2 = up_row_stride;
    return launch_producer<2>(p, stream);
}

// ---- row-wise quantize fused with the all-gather of a row-sharded weight ---------------------------

extern "C" int qt_quantize_rowwise_scatter(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                                          int n_dst, void* const* q_dst, void* const* scale_dst, int64_t dst_row0,
                                          int q_dtype, int scale_dtype, float eps, void* stream_) {
    QT_REQUIRE(n_dst >= 1 && n_dst <= kMaxScatter, "quantize_rowwise_scatter: 1..%d destinations (got %d)", kMaxScatter, n_dst);
    QT_REQUIRE(q_dst && scale_dst, "quantize_rowwise_scatter: null destination table");
    QT_REQUIRE(dst_row0 >= 0, "quantize_rowwise_scatter: negative row offset");
    for (int d = 0; d < n_dst; ++d) QT_REQUIRE(q_dst[d] && scale_dst[d], "quantize_rowwise_scatter: destination %d is null", d);
    if (int rc = check_quant_args(x, x_dtype, rows, cols, x_row_stride, q_dst[0], q_dtype, scale_dst[0], scale_dtype)) return rc;
    if (rows == 0 || cols == 0) return QT_OK;
    // the register-resident row kernel only: bf16 rows, 16-byte aligned, a multiple of 8 columns
    const bool vec_load = aligned_to(x, 16) && ((x_row_stride * 2) % 16 == 0);
    bool vec_store = cols % 8 == 0;
    for (int d = 0; d < n_dst; ++d) vec_store = vec_store && aligned_to(q_dst[d], 8);
    if (x_dtype != QT_BF16 || !vec_load || !vec_store || cols > 32768 || eps < 1e-30f)
        return fail(QT_ERR_UNSUPPORTED, "quantize_rowwise_scatter: needs bf16 rows, 16-byte aligned, cols a multiple of 8 and at most 32768");
    RowwiseParams p = {};
    p.x = x; p.rows = rows; p.cols = cols; p.stride = x_row_stride;
    p.q_dtype = q_dtype; p.scale_dtype = scale_dtype; p.eps = eps; p.vec_load = 1; p.vec_store = 1;
    p.n_dst = n_dst; p.dst_row0 = dst_row0;
    for (int d = 0; d < n_dst; ++d) { p.q_dst[d] = reinterpret_cast<uint8_t*>(q_dst[d]); p.scale_dst[d] = scale_dst[d]; }
    QT_GUARD_INIT(p.guard);
    QT_GUARD_OFF(p.guard);   // up to 16 gathered buffers, most of them in peers' memory: this launch is not range-checked
    return launch_rowwise_bf16<false, false, 0, true>(p, reinterpret_cast<cudaStream_t>(stream_));
}

extern "C" int qt_int8_weight_update(void* q, void* scale, int64_t rows, int64_t cols, int mode, const void* t1,
                                     const void* t2, float value, float eps, uint64_t seed, uint64_t offset,
                                     void* stream_) {
    QT_REQUIRE(mode == 0 || mode == 1, "int8_weight_update: mode must be 0 (add) or 1 (addcdiv), got %d", mode);
    QT_REQUIRE(rows >= 0 && cols >= 0, "int8_weight_update: negative shape (%lld, %lld)", (long long)rows, (long long)cols);
    if (rows == 0 || cols == 0) return QT_OK;
    QT_REQUIRE(q && scale && t1 && (mode == 0 || t2), "int8_weight_update: null pointer");
    if (cols % 8 != 0 || cols > 32768)
        return fail(QT_ERR_UNSUPPORTED, "int8_weight_update: cols must be a multiple of 8 and at most 32768 (got %lld)", (long long)cols);
    if (!aligned_to(q, 8) || !aligned_to(t1, 16) || (mode == 1 && !aligned_to(t2, 16)))
        return fail(QT_ERR_UNSUPPORTED, "int8_weight_update: q must be 8-byte and the operands 16-byte aligned");
    QT_REQUIRE(eps >= 1e-30f, "int8_weight_update: eps must be at least 1e-30");
    RowwiseParams p = {};
    p.rows = rows; p.cols = cols; p.stride = cols;
    p.q = reinterpret_cast<uint8_t*>(q); p.scale = scale;
    p.q_dtype = QT_I8; p.scale_dtype = QT_BF16; p.eps = eps; p.stochastic = 1;
    p.seed = seed; p.offset = offset; p.keys = philox_keys(seed); p.vec_load = 1; p.vec_store = 1;
    p.t1 = reinterpret_cast<const __nv_bfloat16*>(t1); p.t2 = reinterpret_cast<const __nv_bfloat16*>(t2); p.value = value;
    QT_GUARD_INIT(p.guard);
    QT_GUARD_ADD(p.guard, q, rows * cols);
    QT_GUARD_ADD(p.guard, scale, rows * 2);
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    return mode == 0 ? launch_rowwise_bf16<false, true, 1>(p, stream) : launch_rowwise_bf16<false, true, 2>(p, stream);
}

// ---- allocation-free column-wise quantize ---------------------------------------------------------

// Scratch for qt_quantize_colwise_t_noalloc: the per-column absmax that the two-call form keeps in
// a caller-allocated buffer. It lives in the library's own image (256 KB on every GPU that loads
// the library, until the process exits) so the entry point never has to ask anyone for memory.
constexpr int64_t kNoAllocMaxCols = 65536;
static __device__ __align__(256) float g_noalloc_col_absmax[kNoAllocMaxCols];

// In host code the array's name is only a handle; the device address has to be looked up, once
// per device, with that device current.
static float* g_noalloc_ptr[64] = {nullptr};

static int noalloc_scratch(float** out) {
    int dev = 0;
    QT_CUDA_CHECK(cudaGetDevice(&dev));
    QT_REQUIRE(dev >= 0 && dev < 64, "quantize_colwise_t_noalloc: device index %d out of range", dev);
    if (!g_noalloc_ptr[dev]) {
        float* ptr = nullptr;
        QT_CUDA_CHECK(cudaGetSymbolAddress((void**)&ptr, g_noalloc_col_absmax));
        g_noalloc_ptr[dev] = ptr;
    }
    *out = g_noalloc_ptr[dev];
    return QT_OK;
}

extern "C" int qt_quantize_colwise_t_noalloc(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                                             void* qt_out, int q_dtype, void* scale, int scale_dtype, float eps,
                                             int stochastic, uint64_t seed, uint64_t offset, void* stream) {
    if (int rc = check_quant_args(x, x_dtype, rows, cols, x_row_stride, qt_out, q_dtype, scale, scale_dtype)) return rc;
    if (cols > kNoAllocMaxCols)
        return fail(QT_ERR_UNSUPPORTED, "quantize_colwise_t_noalloc: %lld columns exceed the built-in scratch of %lld; use "
                    "qt_col_absmax + qt_quantize_colwise_t with your own buffer", (long long)cols, (long long)kNoAllocMaxCols);
    if (cols == 0) return QT_OK;
    float* scratch = nullptr;
    if (int rc = noalloc_scratch(&scratch)) return rc;
    // qt_col_absmax clears the columns it is about to use (the array still holds the last call's maxima)
    if (int rc = qt_col_absmax(x, x_dtype, rows, cols, x_row_stride, scratch, stream)) return rc;
    return qt_quantize_colwise_t(x, x_dtype, rows, cols, x_row_stride, scratch, qt_out, q_dtype, scale, scale_dtype, eps,
                                 stochastic, seed, offset, stream);
}

extern "C" int qt_selftest_division(int q_dtype, float eps, unsigned long long* mismatches_host) {
    QT_REQUIRE(mismatches_host, "selftest_division: null output");
    unsigned long long* d = nullptr;
    QT_CUDA_CHECK(cudaMalloc(&d, 2 * sizeof(unsigned long long)));
    QT_CUDA_CHECK(cudaMemset(d, 0, 2 * sizeof(unsigned long long)));
    division_selftest_kernel<<<num_sms() * 8, 256>>>(q_dtype, eps, d);
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(mismatches_host, d, 2 * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) return fail(QT_ERR_CUDA, "selftest_division: %s", cudaGetErrorString(e));
    return QT_OK;
}
