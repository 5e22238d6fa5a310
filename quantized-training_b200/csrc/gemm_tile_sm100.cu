// Tile-scaled GEMM for sm_100a: per block of 128 reduction elements the int8 (or fp8) product is
// accumulated by tcgen05.mma into a fresh TMEM buffer, then "promoted" on the CUDA cores:
//     acc[m,n] += fp32(partial[m,n]) * scale_a[m / qm, kb] * scale_b[kb, n / qn]
// which is the loop of the reference's _tile_scaled_mm_kernel (kernels/gn_kernels/triton_mm.py:314-331).
//
// One persistent CTA per SM owns 128 x 256 tiles; 12 warps in three warpgroups: the first holds the TMA
// producer and the MMA issuer (its other two warps idle), the other two are the eight promotion / epilogue
// warps that keep the fp32 accumulator (128 values per thread: one row, 128 columns, i.e. one scale block of
// B) in registers. TMEM holds two 256-column partial buffers, so the tensor core works on the next K block
// while the current one is promoted. The promotion (one convert + one fused multiply-add per element per K
// block) is what bounds this kernel, not the tensor pipe: a TMEM load takes a couple of hundred cycles to
// return, so a warp needs a large chunk in flight while it promotes the previous one. The registers for that
// (128 accumulators + two 32-column chunks) come from the first warpgroup, which gives most of its share
// back (setmaxnreg). All waits are bounded.
#include "tcgen05.cuh"

namespace qt {

namespace {

using namespace tc;

constexpr int TBM = 128, TBN = 256, TBK = 128;
constexpr int T_UMMA_K = 32;
constexpr int T_STAGES = 4;
constexpr int T_A_BYTES = TBM * TBK, T_B_BYTES = TBN * TBK, T_STAGE_BYTES = T_A_BYTES + T_B_BYTES;
#ifndef QT_TILE_EPI_WARPS
#define QT_TILE_EPI_WARPS 8
#endif
// promotion warps: 8 (two per TMEM lane quarter, 128 columns each) or 16 (four, 64 columns each; measured 5-15 % slower:
// the chunks halve and the accumulators spill at 112 registers)
constexpr int T_EPI_WARPS = QT_TILE_EPI_WARPS;
constexpr int T_COL_PARTS = T_EPI_WARPS / 4;
constexpr int T_WARP_COLS = TBN / T_COL_PARTS;   // columns of the tile a promotion warp owns
constexpr int T_CHUNK = T_WARP_COLS / 4;         // a reduction block is promoted in four chunks
static_assert(T_EPI_WARPS == 8 || T_EPI_WARPS == 16, "promotion warps");
constexpr int T_FIRST_EPI_WARP = 4;              // warps 0..3: producer, MMA issuer and two idle warps (one warpgroup)
constexpr int T_THREADS = 32 * (T_FIRST_EPI_WARP + T_EPI_WARPS);
// registers per thread after the warpgroups rebalance: 128 x 56 + 256 x 224 = 64512, or 128 x 24 + 512 x 112 = 60416,
// of the SM's 65536. Slack is deliberate: with 32 / 120 (all 65536, every scheduler's 16384 exactly) the increase
// never completed and the kernel hung, and setmaxnreg has no timeout.
constexpr int T_REGS_SMALL = T_EPI_WARPS == 8 ? 56 : 24, T_REGS_LARGE = T_EPI_WARPS == 8 ? 224 : 112;
constexpr int T_BUFS = 2;                       // TMEM partial buffers of TBN columns
constexpr int T_TMEM_COLS = T_BUFS * TBN;       // 512
constexpr int T_SMEM_BAR_OFF = T_STAGES * T_STAGE_BYTES;
constexpr int T_NUM_BARRIERS = 2 * T_STAGES + 2 * T_BUFS;
constexpr int T_SMEM_TMEMPTR_OFF = T_SMEM_BAR_OFF + T_NUM_BARRIERS * 8;
constexpr int T_SMEM_ABORT_OFF = T_SMEM_TMEMPTR_OFF + 4;
constexpr int T_SMEM_TOTAL = T_SMEM_ABORT_OFF + 4 + 1024;

struct TileGemmParams {
    int64_t M, N, K;
    void* c;
    int64_t ldc;
    const void* scale_a;
    const void* scale_b;
    int64_t sa_s0, sa_s1, sb_s0, sb_s1;
    int qm, qn;
    int kq;   // 128-byte reduction blocks per scale block (qk / 128)
    int scale_dtype;
    int* status;
};

// NARROW: the scale blocks of B are narrower than a thread's columns (qn = 16, 32, 64 against 128); the common wide case
// keeps its own instantiation (the extra scale fetches cost registers the promotion loop has none to spare of).
template <int KIND, bool A_MN, bool B_MN, bool NARROW>
__global__ void __launch_bounds__(T_THREADS, 1)
tile_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const TileGemmParams p,
                 const uint32_t idesc) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    volatile uint32_t* s_tmem_ptr = reinterpret_cast<volatile uint32_t*>(smem + T_SMEM_TMEMPTR_OFF);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + T_SMEM_ABORT_OFF);
    const uint32_t bar_base = smem_base + T_SMEM_BAR_OFF;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (T_STAGES + s); };
    auto part_full_bar = [&](int b) { return bar_base + 8u * (2 * T_STAGES + b); };
    auto part_empty_bar = [&](int b) { return bar_base + 8u * (2 * T_STAGES + T_BUFS + b); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (int)((p.M + TBM - 1) / TBM), tiles_n = (int)((p.N + TBN - 1) / TBN);
    const int64_t num_tiles = (int64_t)tiles_m * tiles_n;
    const int num_kb = (int)(p.K / TBK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < T_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < T_BUFS; ++b) { mbar_init(part_full_bar(b), 1); mbar_init(part_empty_bar(b), T_EPI_WARPS); }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_base + T_SMEM_TMEMPTR_OFF), "r"(T_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *s_tmem_ptr;

    if (warp < T_FIRST_EPI_WARP) {
    // the first warpgroup hands registers back before its warps take their roles
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(T_REGS_SMALL));
    if (warp == 0) {
        // ===== TMA producer =====
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            const TileCoord tc_ = tile_coord(tile, tiles_m, tiles_n);
            const int m0 = tc_.m * TBM, n0 = tc_.n * TBN;
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(empty_bar(stage), phase ^ 1u, s_abort, p.status, 0x500 | stage);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t a_dst = smem_base + stage * T_STAGE_BYTES, b_dst = a_dst + T_A_BYTES;
                    const int k0 = kb * TBK;
                    mbar_expect_tx(full_bar(stage), T_STAGE_BYTES);
                    if constexpr (A_MN) tma_load_2d(a_dst, &tmap_a, full_bar(stage), m0, k0);
                    else tma_load_2d(a_dst, &tmap_a, full_bar(stage), k0, m0);
                    if constexpr (B_MN) {
                        tma_load_2d(b_dst, &tmap_b, full_bar(stage), n0, k0);
                        tma_load_2d(b_dst + TBK * 128, &tmap_b, full_bar(stage), n0 + 128, k0);
                    } else {
                        tma_load_2d(b_dst, &tmap_b, full_bar(stage), k0, n0);
                    }
                }
                __syncwarp();
                if (++stage == T_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        for (int s = 0; s < T_STAGES && ok; ++s) {
            ok = mbar_wait(empty_bar(stage), phase ^ 1u, s_abort, p.status, 0x580 | stage);
            if (++stage == T_STAGES) { stage = 0; phase ^= 1u; }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: every K block starts a fresh partial (accumulate = 0 on its first MMA) =====
        int stage = 0, buf = 0;
        uint32_t phase = 0, buf_phase = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(part_empty_bar(buf), buf_phase ^ 1u, s_abort, p.status, 0x600 | buf);
                if (!ok) break;
                ok = mbar_wait(full_bar(stage), phase, s_abort, p.status, 0x700 | stage);
                if (!ok) break;
                tcgen05_fence_after();
                if (lane == 0) {
                    const uint32_t a_addr = smem_base + stage * T_STAGE_BYTES, b_addr = a_addr + T_A_BYTES;
                    const uint32_t d_tmem = tmem_base + (uint32_t)(buf * TBN);
#pragma unroll
                    for (int k = 0; k < TBK / T_UMMA_K; ++k) {
                        const uint64_t a_desc = A_MN ? make_smem_desc(a_addr + k * T_UMMA_K * 128, TBK * 128, 1024)
                                                     : make_smem_desc(a_addr + k * T_UMMA_K, 16, 1024);
                        const uint64_t b_desc = B_MN ? make_smem_desc(b_addr + k * T_UMMA_K * 128, TBK * 128, 1024)
                                                     : make_smem_desc(b_addr + k * T_UMMA_K, 16, 1024);
                        tcgen05_mma<KIND>(d_tmem, a_desc, b_desc, idesc, k != 0 ? 1u : 0u);
                    }
                    tcgen05_commit(empty_bar(stage));
                    tcgen05_commit(part_full_bar(buf));
                }
                __syncwarp();
                if (++stage == T_STAGES) { stage = 0; phase ^= 1u; }
                if (++buf == T_BUFS) { buf = 0; buf_phase ^= 1u; }
            }
        }
    }
    } else {
        // ===== promotion + epilogue: thread = one row x 128 columns, fp32 accumulators in registers =====
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(T_REGS_LARGE));
        const int ew = warp & 3;
        const int half = (warp - T_FIRST_EPI_WARP) >> 2;
        constexpr int HN = T_WARP_COLS;
        constexpr int CW = T_CHUNK;
        int buf = 0;
        uint32_t buf_phase = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            const TileCoord tc_ = tile_coord(tile, tiles_m, tiles_n);
            const int64_t m0 = (int64_t)tc_.m * TBM, n0 = (int64_t)tc_.n * TBN;
            const int64_t row = m0 + ew * 32 + lane;
            const int64_t sa_row = (row < p.M ? row : p.M - 1) / p.qm;
            const int64_t sb_col = (n0 + half * HN < p.N ? n0 + half * HN : n0) / p.qn;
            float2 acc2[HN / 2];   // accumulators in pairs: the promotion uses packed fp32x2 instructions
#pragma unroll
            for (int j = 0; j < HN / 2; ++j) acc2[j] = make_float2(0.0f, 0.0f);
            // Scale blocks of B narrower than this thread's 128 columns (qn = 16, 32 or 64): one scale per
            // 16-column chunk, fetched per reduction block. Otherwise one scale serves the whole row segment.
            constexpr bool narrow = NARROW;
            // The scales of a reduction block are found by walking: element offsets of this thread's scale of A and
            // of B advance by one stride every kq-th block (no division or 64-bit multiply per block).
            int64_t sa_off = sa_row * p.sa_s0, sb_off = sb_col * p.sb_s1, sb_kb_off = 0;
            int until_next = p.kq;   // blocks left under the current scales
            auto chunk_scale = [&](int64_t kb_off, int c) {
                const int64_t col = n0 + half * HN + c * 16;
                return load_scale(p.scale_b, p.scale_dtype, kb_off + ((col < p.N ? col : n0) / p.qn) * p.sb_s1);
            };
            // The scales are requested one block ahead and kept as loaded (raw bits): decoding or multiplying them
            // where they are requested would make the warp wait there for the loads, once per block.
            const bool scale_is_bf16 = p.scale_dtype == QT_BF16;
            auto load_raw = [&](const void* base, int64_t off) -> uint32_t {
                return scale_is_bf16 ? (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(base) + off)
                                     : __ldg(reinterpret_cast<const uint32_t*>(base) + off);
            };
            auto decode = [&](uint32_t raw) { return __uint_as_float(scale_is_bf16 ? raw << 16 : raw); };
            uint32_t sa_raw = load_raw(p.scale_a, sa_off), sb_raw = narrow ? 0u : load_raw(p.scale_b, sb_off);
            // Chunks of a quarter of the warp's columns through two register buffers: the next TMEM load is in flight while the current
            // chunk is promoted, and the first chunk of the NEXT reduction block is requested before the last chunk
            // of this one is promoted, so a block does not start with a barrier wait and an exposed TMEM load.
            uint32_t ra[CW], rb[CW];
            auto partial_row = [&](int b) { return tmem_base + ((uint32_t)(ew * 32) << 16) + (uint32_t)(b * TBN + half * HN); };
            ok = mbar_wait(part_full_bar(buf), buf_phase, s_abort, p.status, 0x800 | buf);
            if (!ok) break;
            tcgen05_fence_after();
            tmem_ld_cols(partial_row(buf), ra);
            for (int kb = 0; kb < num_kb; ++kb) {
                const float s = decode(sa_raw) * (narrow ? 1.0f : decode(sb_raw));
                const int64_t sb_kb_cur = narrow ? sb_kb_off : 0;   // (narrow form: the current block's row of B scales)
                if (kb + 1 < num_kb) {
                    if (--until_next == 0) {
                        until_next = p.kq;
                        sa_off += p.sa_s1;
                        if constexpr (narrow) sb_kb_off += p.sb_s0;
                        else sb_off += p.sb_s0;
                        sa_raw = load_raw(p.scale_a, sa_off);
                        if constexpr (!narrow) sb_raw = load_raw(p.scale_b, sb_off);
                    }
                }
                const uint32_t t_row = partial_row(buf);
                // The int8 partial is converted by the integer-to-float instruction (not the fp32 pipe) and the
                // multiply-add is the packed fp32x2 form (half the issue slots); measured 1.37 -> 1.56 POPS at 8192^3
                // against a magic-number conversion that spent a second fp32 operation per element.
                auto promote = [&](const uint32_t (&r)[CW], int c) {
#pragma unroll
                    for (int h = 0; h < CW / 16; ++h) {
                        const float sc = narrow ? s * chunk_scale(sb_kb_cur, (CW / 16) * c + h) : s;
                        const float2 s2 = make_float2(sc, sc);
#pragma unroll
                        for (int j = 0; j < 16; j += 2) {
                            float2 x;
                            if constexpr (KIND == 0)
                                x = make_float2((float)(int32_t)r[h * 16 + j], (float)(int32_t)r[h * 16 + j + 1]);
                            else
                                x = make_float2(__uint_as_float(r[h * 16 + j]), __uint_as_float(r[h * 16 + j + 1]));
                            acc2[c * (CW / 2) + h * 8 + j / 2] = __ffma2_rn(x, s2, acc2[c * (CW / 2) + h * 8 + j / 2]);
                        }
                    }
                };
                tmem_ld_wait();
                tmem_ld_cols(t_row + CW, rb);
                promote(ra, 0);
                tmem_ld_wait();
                tmem_ld_cols(t_row + 2 * CW, ra);
                promote(rb, 1);
                tmem_ld_wait();
                tmem_ld_cols(t_row + 3 * CW, rb);
                promote(ra, 2);
                tmem_ld_wait();
                // every value of this partial is in registers (the wait above is warp-wide): the buffer goes back to
                // the tensor core
                tcgen05_fence_before();
                if (lane == 0) mbar_arrive(part_empty_bar(buf));
                if (++buf == T_BUFS) { buf = 0; buf_phase ^= 1u; }
                if (kb + 1 < num_kb) {
                    ok = mbar_wait(part_full_bar(buf), buf_phase, s_abort, p.status, 0x800 | buf);
                    if (!ok) break;
                    tcgen05_fence_after();
                    tmem_ld_cols(partial_row(buf), ra);
                }
                promote(rb, 3);
            }
            if (!ok) break;
            float acc[HN];
#pragma unroll
            for (int j = 0; j < HN / 2; ++j) { acc[2 * j] = acc2[j].x; acc[2 * j + 1] = acc2[j].y; }
            if (row < p.M) {
                const int64_t nh = n0 + half * HN;
                if (p.scale_dtype == QT_BF16) {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + row * p.ldc + nh;
                    if (nh + HN <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
                        for (int j = 0; j < HN; j += 8)
                            *reinterpret_cast<uint4*>(dst + j) =
                                make_uint4(pack_bf16x2(acc[j], acc[j + 1]), pack_bf16x2(acc[j + 2], acc[j + 3]),
                                           pack_bf16x2(acc[j + 4], acc[j + 5]), pack_bf16x2(acc[j + 6], acc[j + 7]));
                    } else {
#pragma unroll
                        for (int j = 0; j < HN; ++j)
                            if (nh + j < p.N) dst[j] = __float2bfloat16_rn(acc[j]);
                    }
                } else {
                    float* dst = reinterpret_cast<float*>(p.c) + row * p.ldc + nh;
#pragma unroll
                    for (int j = 0; j < HN; ++j)
                        if (nh + j < p.N) dst[j] = acc[j];
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(T_TMEM_COLS) : "memory");
    }
}

template <int KIND, bool A_MN, bool B_MN, bool NARROW>
int launch_tile(const CUtensorMap& ta, const CUtensorMap& tb, const TileGemmParams& p, uint32_t idesc, int grid, cudaStream_t stream) {
    auto kfn = tile_gemm_kernel<KIND, A_MN, B_MN, NARROW>;
    static bool attr_set[64] = {false};
    int dev = 0;
    QT_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        QT_CUDA_CHECK(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM_TOTAL));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    kfn<<<grid, T_THREADS, T_SMEM_TOTAL, stream>>>(ta, tb, p, idesc);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

template <int KIND>
int launch_tile_layout(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const TileGemmParams& p, uint32_t idesc,
                       int grid, cudaStream_t stream) {
    if (p.qn < T_WARP_COLS) {
        if (!a_mn && !b_mn) return launch_tile<KIND, false, false, true>(ta, tb, p, idesc, grid, stream);
        if (!a_mn && b_mn) return launch_tile<KIND, false, true, true>(ta, tb, p, idesc, grid, stream);
        if (a_mn && b_mn) return launch_tile<KIND, true, true, true>(ta, tb, p, idesc, grid, stream);
        return launch_tile<KIND, true, false, true>(ta, tb, p, idesc, grid, stream);
    }
    if (!a_mn && !b_mn) return launch_tile<KIND, false, false, false>(ta, tb, p, idesc, grid, stream);
    if (!a_mn && b_mn) return launch_tile<KIND, false, true, false>(ta, tb, p, idesc, grid, stream);
    if (a_mn && b_mn) return launch_tile<KIND, true, true, false>(ta, tb, p, idesc, grid, stream);
    return launch_tile<KIND, true, false, false>(ta, tb, p, idesc, grid, stream);
}

}  // namespace

}  // namespace qt

using namespace qt;
using namespace qt::tc;

extern "C" int qt_tile_scaled_mm(const void* a, int a_dtype, int64_t a_sm, int64_t a_sk, const void* b, int b_dtype,
                                 int64_t b_sk, int64_t b_sn, const void* scale_a, int64_t sa_s0, int64_t sa_s1,
                                 const void* scale_b, int64_t sb_s0, int64_t sb_s1, int qm, int qn, int qk, int scale_dtype,
                                 void* c, int64_t ldc, int64_t M, int64_t N, int64_t K, void* stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    QT_REQUIRE(M >= 0 && N >= 0 && K >= 0, "tile_scaled_mm: negative dimension");
    QT_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "tile_scaled_mm: dimension exceeds 2^31");
    QT_REQUIRE(((M + TBM - 1) / TBM) * ((N + TBN - 1) / TBN) < (1ll << 31), "tile_scaled_mm: too many output tiles for the 32-bit tile index");
    const bool is_i8 = a_dtype == QT_I8 && b_dtype == QT_I8;
    const bool is_f8 = (a_dtype == QT_E4M3 || a_dtype == QT_E5M2) && (b_dtype == QT_E4M3 || b_dtype == QT_E5M2);
    QT_REQUIRE(is_i8 || is_f8, "tile_scaled_mm: operands must both be int8 or both be fp8 (got %d, %d)", a_dtype, b_dtype);
    QT_REQUIRE(scale_dtype == QT_BF16 || scale_dtype == QT_F32, "tile_scaled_mm: scale_dtype must be QT_BF16 or QT_F32 (got %d)", scale_dtype);
    if (M == 0 || N == 0) return QT_OK;
    QT_REQUIRE(a && b && c && scale_a && scale_b, "tile_scaled_mm: null pointer");
    if (qk < TBK || qk % TBK != 0 || K % qk != 0 || K == 0)
        return fail(QT_ERR_UNSUPPORTED, "tile_scaled_mm: the reduction block must be a multiple of 128 and K a positive multiple of it (qk=%d, K=%lld)", qk, (long long)K);
    if (qm < 1 || !(qn == 16 || qn == 32 || qn == 64 || (qn >= 128 && qn % 128 == 0)))
        return fail(QT_ERR_UNSUPPORTED, "tile_scaled_mm: qm must be >= 1 and qn one of 16, 32, 64 or a multiple of 128 (qm=%d, qn=%d)", qm, qn);
    QT_REQUIRE((a_sk == 1) != (a_sm == 1) || M == 1, "tile_scaled_mm: exactly one stride of A must be 1");
    QT_REQUIRE((b_sk == 1) != (b_sn == 1) || N == 1, "tile_scaled_mm: exactly one stride of B must be 1");
    const bool a_mn = (a_sk != 1), b_mn = (b_sk != 1);
    const int64_t a_pitch = a_mn ? a_sk : a_sm, b_pitch = b_mn ? b_sk : b_sn;
    QT_REQUIRE(aligned_to(a, 16) && aligned_to(b, 16), "tile_scaled_mm: operand base pointers must be 16-byte aligned");
    QT_REQUIRE(a_pitch % 16 == 0 && b_pitch % 16 == 0, "tile_scaled_mm: the non-unit operand strides must be multiples of 16");
    QT_REQUIRE(ldc >= N, "tile_scaled_mm: ldc smaller than N");

    CUtensorMap ta, tb;
    if (a_mn) { if (int rc = make_tmap(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)a_pitch, 128, TBK)) return rc; }
    else      { if (int rc = make_tmap(&ta, a, (uint64_t)K, (uint64_t)M, (uint64_t)a_pitch, TBK, TBM)) return rc; }
    if (b_mn) { if (int rc = make_tmap(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)b_pitch, 128, TBK)) return rc; }
    else      { if (int rc = make_tmap(&tb, b, (uint64_t)K, (uint64_t)N, (uint64_t)b_pitch, TBK, TBN)) return rc; }

    TileGemmParams p = {};
    p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc; p.scale_a = scale_a; p.scale_b = scale_b;
    p.sa_s0 = sa_s0; p.sa_s1 = sa_s1; p.sb_s0 = sb_s0; p.sb_s1 = sb_s1; p.qm = qm; p.qn = qn; p.kq = qk / TBK; p.scale_dtype = scale_dtype;
    if (int rc = device_status_ptr(&p.status)) return rc;
    const int64_t tiles = ((M + TBM - 1) / TBM) * ((N + TBN - 1) / TBN);
    const int sms = num_sms();
    const int grid = (int)(tiles < sms ? tiles : sms);
    const uint32_t idesc = is_i8 ? make_idesc(2, 1, 1, a_mn, b_mn, TBM, TBN)
                                 : make_idesc(1, fp8_format(a_dtype), fp8_format(b_dtype), a_mn, b_mn, TBM, TBN);
    return is_i8 ? launch_tile_layout<0>(a_mn, b_mn, ta, tb, p, idesc, grid, stream)
                 : launch_tile_layout<1>(a_mn, b_mn, ta, tb, p, idesc, grid, stream);
}
