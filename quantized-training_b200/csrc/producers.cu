// Backward passes of the producer kernels (RMSNorm, silu * up) and rotary position embedding, forward
// and backward: the element-wise work around the INT8 linear layers of a decoder block, each as one
// HBM pass. The forward producers themselves (which also emit the quantized activation) live with the
// row-wise quantize kernel in quantize.cu.
//
// The reference project leaves these operations to the model code and torch.compile
// (llm_pretrain.py:134-139 compiles every decoder layer); it names the fusion of the activation
// quantize into its producer as the open optimisation (subclasses/int8.py:155-156).
#include "common.cuh"

namespace qt {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
__device__ __forceinline__ uint32_t word_of(const uint4& v, int k) { return k == 0 ? v.x : (k == 1 ? v.y : (k == 2 ? v.z : v.w)); }

template <int TPR>
__device__ __forceinline__ void row_barrier(int sub) {
    switch (sub) {
        case 0: asm volatile("bar.sync 1, %0;" ::"n"(TPR) : "memory"); break;
        case 1: asm volatile("bar.sync 2, %0;" ::"n"(TPR) : "memory"); break;
        case 2: asm volatile("bar.sync 3, %0;" ::"n"(TPR) : "memory"); break;
        default: asm volatile("bar.sync 4, %0;" ::"n"(TPR) : "memory"); break;
    }
}

// ---- RMSNorm backward ---------------------------------------------------------------------------------
//
// Forward (per row): n = x * rstd, y = weight * bf16(n), rstd = 1 / sqrt(mean(x^2) + eps).
// Backward, all in fp32 from the bf16 inputs:
//   g  = dy * weight
//   dx = rstd * (g - n * mean(g * n))
//   dweight[c] = sum over rows of dy * bf16(n)
// TPR threads hold one row (VPT 16-byte vectors each, like the row-wise quantize kernel); every thread
// also carries the running dweight sums of its own columns over all rows it visits and writes them, at the
// end, to its own row of `dw_partial` (one row per row group of the grid): a second kernel adds those rows
// in a fixed order, so the result does not depend on scheduling.

struct NormBwdParams {
    const __nv_bfloat16* dy;
    const __nv_bfloat16* x;
    const __nv_bfloat16* w;
    const float* rstd;
    __nv_bfloat16* dx;
    float* dw_partial;
    int64_t dy_stride, x_stride;
    int rows, cols;
};

template <int TPR, int VPT>
__global__ void __launch_bounds__(kThreads, VPT <= 4 ? 2 : 1) rmsnorm_bwd_kernel(const NormBwdParams p) {
    constexpr int RPC = kThreads / TPR;
    constexpr int WPR = TPR / 32;
    __shared__ float s_sum[2][kThreads / 32];
    const int sub = threadIdx.x / TPR, t = threadIdx.x % TPR, warp = threadIdx.x >> 5;
    const int step = (int)gridDim.x * RPC;
    const int first = (int)blockIdx.x * RPC;
    const int n_iter = first < p.rows ? (p.rows - first + step - 1) / step : 0;
    int row = first + sub;
    const int nvec = p.cols / 8;
    const float inv_cols = 1.0f / (float)p.cols;

    int vpos[VPT];
    bool ok[VPT];
    uint4 wv[VPT];
    float2 acc[VPT][4];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        vpos[i] = i * TPR + t;
        ok[i] = vpos[i] < nvec;
        wv[i] = ok[i] ? reinterpret_cast<const uint4*>(p.w)[vpos[i]] : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[i][k] = make_float2(0.0f, 0.0f);
    }
    const uint4* dy = reinterpret_cast<const uint4*>(p.dy + (int64_t)row * p.dy_stride);
    const uint4* x = reinterpret_cast<const uint4*>(p.x + (int64_t)row * p.x_stride);
    uint4* dx = reinterpret_cast<uint4*>(p.dx + (int64_t)row * p.cols);
    const int64_t dy_step = (int64_t)step * (p.dy_stride / 8), x_step = (int64_t)step * (p.x_stride / 8), dx_step = (int64_t)step * nvec;

    for (int it = 0; it < n_iter; ++it) {
        // rows beyond the end (the last iteration of a grid that does not divide the rows) read row 0 and store nothing
        const bool valid = row < p.rows;
        uint4 dv[VPT], xv[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            dv[i] = (ok[i] && valid) ? dy[vpos[i]] : make_uint4(0, 0, 0, 0);
            xv[i] = (ok[i] && valid) ? x[vpos[i]] : make_uint4(0, 0, 0, 0);
        }
        const float rstd = valid ? p.rstd[row] : 0.0f;
        const float2 rstd2 = make_float2(rstd, rstd);
        float2 c2 = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 d = unpack_bf16x2(word_of(dv[i], k));
                const float2 n = __fmul2_rn(unpack_bf16x2(word_of(xv[i], k)), rstd2);
                const float2 g = __fmul2_rn(d, unpack_bf16x2(word_of(wv[i], k)));
                c2 = __ffma2_rn(g, n, c2);
                acc[i][k] = __ffma2_rn(d, unpack_bf16x2(pack_bf16x2_rn(n.x, n.y)), acc[i][k]);
            }
        float c = __fadd_rn(c2.x, c2.y);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
        if constexpr (WPR > 1) {
            if ((threadIdx.x & 31) == 0) s_sum[it & 1][warp] = c;
            if constexpr (RPC == 1) __syncthreads();
            else row_barrier<TPR>(sub);
            c = s_sum[it & 1][sub * WPR];
#pragma unroll
            for (int w = 1; w < WPR; ++w) c += s_sum[it & 1][sub * WPR + w];
        }
        const float m = -c * inv_cols;
        const float2 m2 = make_float2(m, m);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 n = __fmul2_rn(unpack_bf16x2(word_of(xv[i], k)), rstd2);
                const float2 g = __fmul2_rn(unpack_bf16x2(word_of(dv[i], k)), unpack_bf16x2(word_of(wv[i], k)));
                const float2 r = __fmul2_rn(__ffma2_rn(n, m2, g), rstd2);
                o[k] = pack_bf16x2_rn(r.x, r.y);
            }
            if (ok[i] && valid) dx[vpos[i]] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        dy += dy_step; x += x_step; dx += dx_step; row += step;
    }
    // this row group's column sums: partial row (blockIdx.x * RPC + sub)
    float* out = p.dw_partial + (int64_t)(blockIdx.x * RPC + sub) * p.cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
        if (ok[i]) {
            float4* o4 = reinterpret_cast<float4*>(out + (int64_t)vpos[i] * 8);
            o4[0] = make_float4(acc[i][0].x, acc[i][0].y, acc[i][1].x, acc[i][1].y);
            o4[1] = make_float4(acc[i][2].x, acc[i][2].y, acc[i][3].x, acc[i][3].y);
        }
}

// out[c] = sum over r of partial[r][c], rows added in a fixed order: thread (cx, ry) adds rows ry, ry + 8,
// ... of column cx, the eight row groups are folded through shared memory in order.
__global__ void __launch_bounds__(kThreads) colsum_kernel(const float* __restrict__ partial, int n_rows, int cols, void* __restrict__ out,
                                                           int out_dtype) {
    __shared__ float s[8][33];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx;
    float a = 0.0f;
    if (c < cols)
        for (int r = ry; r < n_rows; r += 8) a += partial[(int64_t)r * cols + c];
    s[ry][cx] = a;
    __syncthreads();
    if (ry == 0 && c < cols) {
        float tsum = s[0][cx];
#pragma unroll
        for (int k = 1; k < 8; ++k) tsum += s[k][cx];
        if (out_dtype == QT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[c] = __float2bfloat16_rn(tsum);
        else reinterpret_cast<float*>(out)[c] = tsum;
    }
}

template <int TPR, int VPT>
int launch_norm_bwd(const NormBwdParams& p, int grid, cudaStream_t stream) {
    rmsnorm_bwd_kernel<TPR, VPT><<<grid, kThreads, 0, stream>>>(p);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

// (threads per row, CTAs per SM) of the configuration that serves `cols` columns
void norm_bwd_config(int64_t cols, int* tpr, int* ctas_per_sm) {
    if (cols <= 1024) { *tpr = 32; *ctas_per_sm = 2; }
    else if (cols <= 2048) { *tpr = 64; *ctas_per_sm = 2; }
    else if (cols <= 4096) { *tpr = 128; *ctas_per_sm = 2; }
    else if (cols <= 8192) { *tpr = 256; *ctas_per_sm = 2; }
    else { *tpr = 256; *ctas_per_sm = 1; }
}

int norm_bwd_grid(int64_t rows, int64_t cols) {
    int tpr, per_sm;
    norm_bwd_config(cols, &tpr, &per_sm);
    const int rpc = kThreads / tpr;
    const int64_t want = (rows + rpc - 1) / rpc;
    const int64_t cap = (int64_t)num_sms() * per_sm;
    return (int)(want < cap ? want : cap);
}

// ---- silu(gate) * up backward ---------------------------------------------------------------------------
//
// Forward: s = bf16(silu(gate)), h = bf16(s * up). Backward in fp32:
//   dup   = dh * s
//   dgate = dh * up * sigmoid(gate) * (1 + gate * (1 - sigmoid(gate)))
__global__ void __launch_bounds__(kThreads) silu_mul_bwd_kernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ gate,
                                                                 const __nv_bfloat16* __restrict__ up, __nv_bfloat16* __restrict__ dgate,
                                                                 __nv_bfloat16* __restrict__ dup, int rows, int cols, int64_t dh_stride,
                                                                 int64_t gate_stride, int64_t up_stride) {
    const int nvec = cols / 8;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4* d4 = reinterpret_cast<const uint4*>(dh + (int64_t)row * dh_stride);
        const uint4* g4 = reinterpret_cast<const uint4*>(gate + (int64_t)row * gate_stride);
        const uint4* u4 = reinterpret_cast<const uint4*>(up + (int64_t)row * up_stride);
        uint4* og = reinterpret_cast<uint4*>(dgate + (int64_t)row * cols);
        uint4* ou = reinterpret_cast<uint4*>(dup + (int64_t)row * cols);
        for (int v = threadIdx.x; v < nvec; v += kThreads) {
            const uint4 dv = d4[v], gv = g4[v], uv = u4[v];
            uint32_t rg[4], ru[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 d = unpack_bf16x2(word_of(dv, k)), g = unpack_bf16x2(word_of(gv, k)), u = unpack_bf16x2(word_of(uv, k));
                const float2 sig = make_float2(__fdividef(1.0f, 1.0f + __expf(-g.x)), __fdividef(1.0f, 1.0f + __expf(-g.y)));
                const float2 s = __fmul2_rn(g, sig);
                const float2 sb = unpack_bf16x2(pack_bf16x2_rn(s.x, s.y));
                const float2 du = __fmul2_rn(d, sb);
                // sigmoid * (1 + gate * (1 - sigmoid)) = sigmoid + s * (1 - sigmoid)
                const float2 one = make_float2(1.0f, 1.0f);
                const float2 ds = __ffma2_rn(s, __fadd2_rn(one, make_float2(-sig.x, -sig.y)), sig);
                const float2 dg = __fmul2_rn(__fmul2_rn(d, u), ds);
                rg[k] = pack_bf16x2_rn(dg.x, dg.y);
                ru[k] = pack_bf16x2_rn(du.x, du.y);
            }
            og[v] = make_uint4(rg[0], rg[1], rg[2], rg[3]);
            ou[v] = make_uint4(ru[0], ru[1], ru[2], ru[3]);
        }
    }
}

// ---- rotary position embedding ----------------------------------------------------------------------------
//
// x: [tokens, heads, dim] bf16 contiguous; cos, sin: [batch or 1, seq, dim] bf16; token = b * seq + s.
//   forward:  y1 = x1 * c1 - x2 * s1,  y2 = x2 * c2 + x1 * s2   (x1, x2 = the two halves of a head)
//   inverse:  y1 = x1 * c1 + x2 * s2,  y2 = x2 * c2 - x1 * s1   (the transpose: the backward pass)
// one rounding to bf16 per output. A thread handles 8 elements of the first half and the matching 8 of the
// second; the cos/sin rows are shared by the heads of a token and come from L2 after the first head.
__global__ void __launch_bounds__(kThreads) rope_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ cosp,
                                                         const __nv_bfloat16* __restrict__ sinp, __nv_bfloat16* __restrict__ y, int64_t tokens,
                                                         int heads, int dim, int seq, int64_t cos_batch_stride, int inverse) {
    const int hv = dim / 16;                       // 8-element vectors per half head
    const int64_t total = tokens * heads * hv;
    for (int64_t idx = (int64_t)blockIdx.x * kThreads + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * kThreads) {
        const int j = (int)(idx % hv);
        const int64_t head_row = idx / hv;          // token * heads + head
        const int64_t token = head_row / heads;
        const int64_t b = token / seq, s = token - b * seq;
        const int64_t xo = head_row * dim + j * 8;
        const int64_t co = b * cos_batch_stride + s * dim + j * 8;
        const uint4 x1 = *reinterpret_cast<const uint4*>(x + xo), x2 = *reinterpret_cast<const uint4*>(x + xo + dim / 2);
        const uint4 c1 = *reinterpret_cast<const uint4*>(cosp + co), c2 = *reinterpret_cast<const uint4*>(cosp + co + dim / 2);
        const uint4 s1 = *reinterpret_cast<const uint4*>(sinp + co), s2 = *reinterpret_cast<const uint4*>(sinp + co + dim / 2);
        uint32_t o1[4], o2[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 a = unpack_bf16x2(word_of(x1, k)), bb = unpack_bf16x2(word_of(x2, k));
            const float2 ca = unpack_bf16x2(word_of(c1, k)), cb = unpack_bf16x2(word_of(c2, k));
            const float2 sa = unpack_bf16x2(word_of(s1, k)), sb = unpack_bf16x2(word_of(s2, k));
            float2 r1, r2;
            if (!inverse) {
                r1 = __ffma2_rn(bb, make_float2(-sa.x, -sa.y), __fmul2_rn(a, ca));
                r2 = __ffma2_rn(a, sb, __fmul2_rn(bb, cb));
            } else {
                r1 = __ffma2_rn(bb, sb, __fmul2_rn(a, ca));
                r2 = __ffma2_rn(a, make_float2(-sa.x, -sa.y), __fmul2_rn(bb, cb));
            }
            o1[k] = pack_bf16x2_rn(r1.x, r1.y);
            o2[k] = pack_bf16x2_rn(r2.x, r2.y);
        }
        *reinterpret_cast<uint4*>(y + xo) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
        *reinterpret_cast<uint4*>(y + xo + dim / 2) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
    }
}

}  // namespace

}  // namespace qt

using namespace qt;

extern "C" int64_t qt_rmsnorm_backward_partial_rows(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0) return 0;
    int tpr, per_sm;
    norm_bwd_config(cols, &tpr, &per_sm);
    return (int64_t)norm_bwd_grid(rows, cols) * (kThreads / tpr);
}

extern "C" int qt_rmsnorm_backward(const void* dy, int64_t dy_row_stride, const void* x, int64_t x_row_stride, const void* weight,
                                   const float* rstd, int64_t rows, int64_t cols, void* dx, float* dw_partial,
                                   int64_t partial_rows, void* dweight, int dweight_dtype, void* stream_) {
    QT_REQUIRE(rows >= 0 && cols >= 0 && dy_row_stride >= cols && x_row_stride >= cols, "rmsnorm_backward: bad shape/stride");
    QT_REQUIRE(dweight_dtype == QT_BF16 || dweight_dtype == QT_F32, "rmsnorm_backward: dweight_dtype must be QT_BF16 or QT_F32 (got %d)", dweight_dtype);
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (cols == 0) return QT_OK;
    QT_REQUIRE(dweight, "rmsnorm_backward: dweight is null");
    if (rows == 0) {
        QT_CUDA_CHECK(cudaMemsetAsync(dweight, 0, (size_t)cols * (dweight_dtype == QT_BF16 ? 2 : 4), stream));
        return QT_OK;
    }
    QT_REQUIRE(dy && x && weight && rstd && dx && dw_partial, "rmsnorm_backward: null pointer");
    if (cols % 8 != 0 || cols > 16384 || rows >= ((int64_t)1 << 30) || !aligned_to(dy, 16) || !aligned_to(x, 16) || !aligned_to(weight, 16) ||
        !aligned_to(dx, 16) || !aligned_to(dw_partial, 16) || (dy_row_stride * 2) % 16 != 0 || (x_row_stride * 2) % 16 != 0)
        return fail(QT_ERR_UNSUPPORTED, "rmsnorm_backward: needs 16-byte aligned bf16 rows, cols a multiple of 8 and at most 16384");
    QT_REQUIRE(partial_rows >= qt_rmsnorm_backward_partial_rows(rows, cols), "rmsnorm_backward: dw_partial holds %lld rows, %lld needed",
               (long long)partial_rows, (long long)qt_rmsnorm_backward_partial_rows(rows, cols));
    NormBwdParams p;
    p.dy = reinterpret_cast<const __nv_bfloat16*>(dy); p.x = reinterpret_cast<const __nv_bfloat16*>(x);
    p.w = reinterpret_cast<const __nv_bfloat16*>(weight); p.rstd = rstd; p.dx = reinterpret_cast<__nv_bfloat16*>(dx);
    p.dw_partial = dw_partial; p.dy_stride = dy_row_stride; p.x_stride = x_row_stride; p.rows = (int)rows; p.cols = (int)cols;
    const int grid = norm_bwd_grid(rows, cols);
    int rc;
    if (cols <= 256) rc = launch_norm_bwd<32, 1>(p, grid, stream);
    else if (cols <= 512) rc = launch_norm_bwd<32, 2>(p, grid, stream);
    else if (cols <= 1024) rc = launch_norm_bwd<32, 4>(p, grid, stream);
    else if (cols <= 2048) rc = launch_norm_bwd<64, 4>(p, grid, stream);
    else if (cols <= 4096) rc = launch_norm_bwd<128, 4>(p, grid, stream);
    else if (cols <= 8192) rc = launch_norm_bwd<256, 4>(p, grid, stream);
    else rc = launch_norm_bwd<256, 8>(p, grid, stream);
    if (rc) return rc;
    const int n_partial = (int)qt_rmsnorm_backward_partial_rows(rows, cols);
    colsum_kernel<<<(unsigned)((cols + 31) / 32), kThreads, 0, stream>>>(dw_partial, n_partial, (int)cols, dweight, dweight_dtype);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

extern "C" int qt_silu_mul_backward(const void* dh, int64_t dh_row_stride, const void* gate, int64_t gate_row_stride, const void* up,
                                    int64_t up_row_stride, int64_t rows, int64_t cols, void* dgate, void* dup, void* stream_) {
    QT_REQUIRE(rows >= 0 && cols >= 0 && dh_row_stride >= cols && gate_row_stride >= cols && up_row_stride >= cols,
               "silu_mul_backward: bad shape/stride");
    if (rows == 0 || cols == 0) return QT_OK;
    QT_REQUIRE(dh && gate && up && dgate && dup, "silu_mul_backward: null pointer");
    if (cols % 8 != 0 || rows >= ((int64_t)1 << 31) || !aligned_to(dh, 16) || !aligned_to(gate, 16) || !aligned_to(up, 16) || !aligned_to(dgate, 16) ||
        !aligned_to(dup, 16) || (dh_row_stride * 2) % 16 != 0 || (gate_row_stride * 2) % 16 != 0 || (up_row_stride * 2) % 16 != 0)
        return fail(QT_ERR_UNSUPPORTED, "silu_mul_backward: needs 16-byte aligned bf16 rows and cols a multiple of 8");
    const int64_t cap = (int64_t)num_sms() * 8;
    silu_mul_bwd_kernel<<<(unsigned)(rows < cap ? rows : cap), kThreads, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
        reinterpret_cast<const __nv_bfloat16*>(dh), reinterpret_cast<const __nv_bfloat16*>(gate), reinterpret_cast<const __nv_bfloat16*>(up),
        reinterpret_cast<__nv_bfloat16*>(dgate), reinterpret_cast<__nv_bfloat16*>(dup), (int)rows, (int)cols, dh_row_stride, gate_row_stride,
        up_row_stride);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

extern "C" int qt_rope(const void* x, int64_t tokens, int heads, int head_dim, const void* cos, const void* sin, int64_t seq_len,
                       int64_t cos_batch_stride, int inverse, void* y, void* stream_) {
    QT_REQUIRE(tokens >= 0 && heads >= 0 && head_dim >= 0 && seq_len > 0, "rope: bad shape");
    if (tokens == 0 || heads == 0 || head_dim == 0) return QT_OK;
    QT_REQUIRE(x && cos && sin && y, "rope: null pointer");
    QT_REQUIRE(tokens % seq_len == 0, "rope: %lld tokens are not a whole number of sequences of %lld", (long long)tokens, (long long)seq_len);
    if (head_dim % 16 != 0 || !aligned_to(x, 16) || !aligned_to(y, 16) || !aligned_to(cos, 16) || !aligned_to(sin, 16) ||
        (cos_batch_stride * 2) % 16 != 0)
        return fail(QT_ERR_UNSUPPORTED, "rope: needs a head size that is a multiple of 16 and 16-byte aligned tensors");
    const int64_t total = tokens * heads * (head_dim / 16);
    const int64_t want = (total + kThreads - 1) / kThreads, cap = (int64_t)num_sms() * 16;
    rope_kernel<<<(unsigned)(want < cap ? want : cap), kThreads, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(cos), reinterpret_cast<const __nv_bfloat16*>(sin),
        reinterpret_cast<__nv_bfloat16*>(y), tokens, heads, head_dim, (int)seq_len, cos_batch_stride, inverse);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}
