// tcgen05 GEMMs for sm_100a: int8 x int8 -> int32 (kind::i8) and fp8 x fp8 -> fp32 (kind::f8f6f4),
// with raw and row/column-scaled epilogues.
//
// Persistent kernel, one CTA per SM, 10 warps:
//   warp 0      TMA producer   global -> 128B-swizzled shared-memory stages (cp.async.bulk.tensor)
//   warp 1      MMA issuer     one elected lane issues tcgen05.mma; accumulators live in TMEM
//   warps 2..9  epilogue       two groups of four warps (one per TMEM lane quarter); group g drains
//                              accumulator g in chunks of 32 columns: tcgen05.ld TMEM -> registers -> scale ->
//                              swizzled staging box in shared memory -> TMA store (one box of 32 rows x 64
//                              bytes per chunk)
// Large problems run as CTA PAIRS (2-CTA clusters, tcgen05 cta_group::2): the pair owns a 256 x 256
// tile, each CTA stages its 128 rows of A and half of B, the leader CTA issues M=256 MMAs for both
// and each CTA drains its own 128 accumulator rows. Small problems (M <= 128 or K < 512) use one CTA
// per 128 x 256 tile. The accumulator is double-buffered in TMEM (2 x 256 columns), so while tile i+2
// is in the main loop tiles i and i+1 are in the two epilogue groups. Stages and accumulators are handed
// over through mbarriers; every wait is bounded and reports through the device status word instead of
// spinning forever.
//
// Operand layouts: both operands may be K-major or MN-major in global memory; MN-major tiles are
// fetched as [K][128 B of M or N] boxes and described to the tensor core as MN-major, so A@B.T,
// A@B and A.T@B run without any transpose pass. No TMA multicast is used anywhere: every CTA
// fetches its own tiles (the pair form only redirects the completion bytes to the leader's barrier).
#include <type_traits>

#include "tcgen05.cuh"

namespace qt {

namespace {

using namespace tc;

// ---- tile configuration ---------------------------------------------------------------------

constexpr int BM = 128;      // tile rows per CTA (one TMEM lane per row)
constexpr int BN = 256;      // tile cols (= UMMA N, one TMEM column per col)
constexpr int BK = 128;      // reduction elements per stage (8-bit => 128 bytes = one swizzle row)
constexpr int UMMA_K = 32;   // reduction elements per tcgen05.mma for 8-bit operands
// Epilogue shape. The three knobs below are compile-time so that alternatives can be built side by side; the
// defaults are what measured fastest on 16384 x 4096 x K (K = 128 .. 2048) and ties the rest at large K:
// sixteen warps (two per lane quarter) gained nothing over eight, 64-column chunks (128-byte boxes) were 5-15 %
// slower at K <= 2048, a second staging box per warp changed nothing (the wait for a box's read-out is short), and
// neither did letting every warp work on every tile (EPI_GROUPS 1: half the epilogue latency per tile).
#ifndef QT_EPI_WARPS
#define QT_EPI_WARPS 8
#endif
#ifndef QT_EPI_GROUPS
#define QT_EPI_GROUPS 2
#endif
#ifndef QT_EPI_CHUNK
#define QT_EPI_CHUNK 32
#endif
#ifndef QT_EPI_STAGE_BUFS
#define QT_EPI_STAGE_BUFS 1
#endif
constexpr int NUM_EPI_WARPS = QT_EPI_WARPS;            // two groups; group g drains accumulator g
constexpr int EPI_GROUPS = QT_EPI_GROUPS;              // 2: the groups take alternate tiles; 1: every warp works on every tile
constexpr int EPI_GROUP_WARPS = NUM_EPI_WARPS / EPI_GROUPS;   // four (one per TMEM lane quarter) or a multiple
constexpr int EPI_COL_SPLIT = EPI_GROUP_WARPS / 4;     // warps sharing a lane quarter split the tile's columns between them
constexpr int EPI_WARP_COLS = BN / EPI_COL_SPLIT;
constexpr int EPI_CHUNK = QT_EPI_CHUNK;                // accumulator columns an epilogue warp takes per step (one TMEM load)
constexpr int STORE_BOX_BYTES = EPI_CHUNK * 2;         // bytes per row of a staging box: one chunk of bf16 outputs, half a chunk of 4-byte ones
constexpr int STORE_BUFS = QT_EPI_STAGE_BUFS;          // staging boxes per epilogue warp, used in turn
constexpr int STORE_BOX_TOTAL = 32 * STORE_BOX_BYTES;  // one box: 32 rows, what one TMA store sends
constexpr int STORE_STAGE_BYTES = STORE_BUFS * STORE_BOX_TOTAL;
static_assert(NUM_EPI_WARPS == 8 || NUM_EPI_WARPS == 16, "epilogue warps");
static_assert(EPI_CHUNK == 32 || EPI_CHUNK == 64, "chunk width");
static_assert((EPI_WARP_COLS / EPI_CHUNK) % 2 == 0, "the staging boxes alternate by chunk parity");
constexpr int NUM_THREADS = 64 + 32 * NUM_EPI_WARPS;   // + TMA producer warp + MMA issuer warp
constexpr int TMEM_COLS = 512;                         // 2 accumulators x BN fp32/int32 columns
constexpr int MAX_STAGES = 6;

// CG = CTAs per MMA (tcgen05 cta_group). CG == 1: one CTA owns a 128 x 256 tile and stages all of
// B (4 stages of 48 KB). CG == 2: a pair of CTAs (a 2-CTA cluster) owns a 256 x 256 tile; each CTA
// stages its 128 rows of A and HALF of B (128 of the 256 columns), the leader issues one M=256
// MMA for both, and each CTA ends up with its own 128 rows of the accumulator in its own TMEM. Per
// CTA that is a third less shared-memory and L2->SM traffic for the same math (6 stages of 32 KB).
template <int CG>
struct Cfg {
    // KA = 128-byte K atoms per pipeline stage. The CTA pair stages 256 reduction bytes per
    // hand-over (8 MMAs per barrier round trip instead of 4): the single MMA-issuing thread spends
    // a fixed ~250 cycles per hand-over on the barrier wait and tcgen05.commit, which the tensor
    // pipe only hides when enough MMAs are queued behind it.
    static constexpr int KA = CG == 2 ? 2 : 1;
    static constexpr int BKS = BK * KA;                // reduction bytes per stage
    static constexpr int STAGES = CG == 2 ? 3 : 4;
    static constexpr int A_ATOM_BYTES = BM * BK;       // one [128 rows][128 B] (or [128 k][128 B]) atom
    static constexpr int A_STAGE_BYTES = A_ATOM_BYTES * KA;
    static constexpr int B_ROWS = BN / CG;             // columns of the tile staged by this CTA
    static constexpr int B_ATOM_BYTES = B_ROWS * BK;
    static constexpr int B_STAGE_BYTES = B_ATOM_BYTES * KA;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int SMEM_STORE_OFF = STAGES * STAGE_BYTES;         // output staging, one box per epilogue warp
    static constexpr int SMEM_COLSCALE_OFF = SMEM_STORE_OFF + NUM_EPI_WARPS * STORE_STAGE_BYTES;  // float [2 groups][BN]
    static constexpr int SMEM_BAR_OFF = SMEM_COLSCALE_OFF + 2 * BN * 4;                       // mbarriers
    static constexpr int NUM_BARRIERS = 2 * MAX_STAGES + 4;
    static constexpr int SMEM_TMEMPTR_OFF = SMEM_BAR_OFF + NUM_BARRIERS * 8;
    static constexpr int SMEM_ABORT_OFF = SMEM_TMEMPTR_OFF + 4;
    // no alignment slack: the dynamic shared memory is declared 1024-byte aligned (the kernel checks)
    static constexpr int SMEM_TOTAL = SMEM_ABORT_OFF + 4;
    static_assert(SMEM_TOTAL <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

enum Epilogue { EPI_RAW = 0, EPI_ROWCOL = 1, EPI_TILE = 2 };

struct GemmParams {
    int64_t M, N, K;
    void* c;
    int64_t ldc;
    const void* scale_a;
    const void* scale_b;
    int scale_b_is_scalar;
    int col_scale_first;   // epilogue (acc * col_scale) * row_scale instead of (acc * row_scale) * col_scale
    int group_m;           // row-tiles per rasterisation group (the A panel of a group stays in L2 while B streams past)
    int round_acc_first;   // the accumulator is rounded to bf16 before it is scaled (a bf16 matmul followed by a bf16 multiply)
    int scale_dtype;  // QT_BF16 | QT_F32 ; also the output dtype of scaled epilogues
    // tile-scaled only
    int64_t sa_s0, sa_s1, sb_s0, sb_s1;
    int qm, qn;
    int* status;
    // split-K: `splits` CTAs (or CTA pairs) share one output tile, each reducing `kb_per_split` stages
    // and writing raw partial accumulators to ws[split][M][N] (int32 / fp32 bits); a finishing kernel
    // sums them and applies the epilogue. splits == 1: no workspace, epilogue in this kernel.
    int splits;
    int kb_per_split;
    uint32_t* ws;
    // the output goes through shared memory and TMA stores (needs a 16-byte aligned base and pitch);
    // otherwise, and for split-K partials, every thread stores its own row directly
    int tma_store;
    int cs_vec;   // scale_b is 16-byte aligned: column scales load as vectors
};

// One lane's share of a tile's 256 column scales: columns n .. n+7, requested one tile ahead and kept
// raw until they are written to shared memory. bf16 scales that can be fetched as one vector stay
// packed in raw[0] (returns true); otherwise raw[0..1] hold eight fp32 values (zero beyond N).
__device__ __forceinline__ bool load_col_scales8(uint4 (&raw)[2], const GemmParams& p, int64_t n) {
    if (!p.scale_b_is_scalar && p.cs_vec && n + 8 <= p.N) {
        if (p.scale_dtype == QT_BF16) {
            raw[0] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.scale_b) + n));
            return true;
        }
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(p.scale_b) + n);
        raw[0] = __ldg(src);
        raw[1] = __ldg(src + 1);
        return false;
    }
    float cs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
        cs[j] = p.scale_b_is_scalar ? load_scale(p.scale_b, p.scale_dtype, 0)
                                    : ((n + j < p.N) ? load_scale(p.scale_b, p.scale_dtype, n + j) : 0.0f);
    raw[0] = make_uint4(__float_as_uint(cs[0]), __float_as_uint(cs[1]), __float_as_uint(cs[2]), __float_as_uint(cs[3]));
    raw[1] = make_uint4(__float_as_uint(cs[4]), __float_as_uint(cs[5]), __float_as_uint(cs[6]), __float_as_uint(cs[7]));
    return false;
}

// ---- the kernel -----------------------------------------------------------------------------

// KIND: 0 int8 (s32 accumulate), 1 fp8 (f32 accumulate). A_MN / B_MN: operand is MN-major in
// global memory. CG: CTAs per MMA (see Cfg). The fp8 element formats arrive in `idesc`.
template <int KIND, int EPI, bool A_MN, bool B_MN, int CG>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_c, const GemmParams p, const uint32_t idesc) {
    using C = Cfg<CG>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t smem_base = smem_u32(smem);
    if ((smem_base & 1023u) != 0u) {
        // the 128-byte swizzle of the TMA boxes and UMMA descriptors assumes this alignment
        if (threadIdx.x == 0) record_status(p.status, 0x900);
        return;
    }
    volatile uint32_t* s_tmem_ptr = reinterpret_cast<volatile uint32_t*>(smem + C::SMEM_TMEMPTR_OFF);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + C::SMEM_ABORT_OFF);

    const uint32_t bar_base = smem_base + C::SMEM_BAR_OFF;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
    auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + b); };
    auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + 2 + b); };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;  // 0 = leader of the pair
    const bool leader = cta_rank == 0;

    // tiles are BM*CG rows x BN columns, one per CTA (CG == 1) or per CTA pair (CG == 2)
    const int tiles_m = (int)((p.M + BM * CG - 1) / (BM * CG));
    const int tiles_n = (int)((p.N + BN - 1) / BN);
    const int num_kb = (int)((p.K + C::BKS - 1) / C::BKS);
    // a work item is (tile, K split); the host keeps their number below 2^30, so 32-bit indices do
    const uint32_t first_tile = blockIdx.x / CG;
    const uint32_t tile_step = gridDim.x / CG;
    const uint32_t num_work = (uint32_t)tiles_m * (uint32_t)tiles_n * (uint32_t)p.splits;
    struct WorkItem { int m, n, split; };
    auto locate = [&](uint32_t work) {
        uint32_t tile = work, split = 0;
        if (p.splits > 1) {
            tile = work / (uint32_t)p.splits;
            split = work - tile * (uint32_t)p.splits;
        }
        const TileCoord tc = tile_coord(tile, tiles_m, tiles_n, p.group_m);
        return WorkItem{tc.m, tc.n, (int)split};
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), EPI_GROUP_WARPS * CG);  // one arrival per warp of the group that drains it
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (CG == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_base + C::SMEM_TMEMPTR_OFF), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_base + C::SMEM_TMEMPTR_OFF), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if constexpr (CG == 2) cluster_sync_all();  // the peer's barriers exist before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *s_tmem_ptr;

    if (warp == 0) {
        // ===== TMA producer (every CTA fills its own stages) =====
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (uint32_t work = first_tile; work < num_work && ok; work += tile_step) {
            const WorkItem tc = locate(work);
            const int kb_begin = tc.split * p.kb_per_split;
            const int kb_end = (kb_begin + p.kb_per_split < num_kb) ? kb_begin + p.kb_per_split : num_kb;
            const int m0 = tc.m * (BM * CG) + (int)cta_rank * BM;
            const int n0 = tc.n * BN + (int)cta_rank * C::B_ROWS;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                ok = mbar_wait(empty_bar(stage), phase ^ 1u, s_abort, p.status, 0x100 | stage);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t a_dst = smem_base + stage * C::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + C::A_STAGE_BYTES;
                    const int k0 = kb * C::BKS;
                    if constexpr (CG == 2) {
                        // both CTAs' bytes are credited to the leader's barrier
                        const uint32_t bar = map_to_cta(full_bar(stage), 0);
                        if (leader) mbar_expect_tx(full_bar(stage), 2 * C::STAGE_BYTES);
#pragma unroll
                        for (int a = 0; a < C::KA; ++a) {
                            const int ka = k0 + a * BK;
                            if constexpr (A_MN) tma_load_2d_pair(a_dst + a * C::A_ATOM_BYTES, &tmap_a, bar, m0, ka);
                            else tma_load_2d_pair(a_dst + a * C::A_ATOM_BYTES, &tmap_a, bar, ka, m0);
                            if constexpr (B_MN) tma_load_2d_pair(b_dst + a * C::B_ATOM_BYTES, &tmap_b, bar, n0, ka);
                            else tma_load_2d_pair(b_dst + a * C::B_ATOM_BYTES, &tmap_b, bar, ka, n0);
                        }
                    } else {
                        mbar_expect_tx(full_bar(stage), C::STAGE_BYTES);
                        if constexpr (A_MN) tma_load_2d(a_dst, &tmap_a, full_bar(stage), m0, k0);
                        else tma_load_2d(a_dst, &tmap_a, full_bar(stage), k0, m0);
                        if constexpr (B_MN) {
                            tma_load_2d(b_dst, &tmap_b, full_bar(stage), n0, k0);
                            tma_load_2d(b_dst + BK * 128, &tmap_b, full_bar(stage), n0 + 128, k0);
                        } else {
                            tma_load_2d(b_dst, &tmap_b, full_bar(stage), k0, n0);
                        }
                    }
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        // Drain: wait until every stage this warp filled has been released, so no TMA write is
        // still in flight when the CTA exits.
        for (int s = 0; s < STAGES && ok; ++s) {
            ok = mbar_wait(empty_bar(stage), phase ^ 1u, s_abort, p.status, 0x180 | stage);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
    } else if (warp == 1) {
        // ===== MMA issuer (the leader CTA only when CG == 2) =====
        if (leader) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (uint32_t work = first_tile; work < num_work && ok; work += tile_step) {
                const int split = p.splits > 1 ? (int)(work % (uint32_t)p.splits) : 0;
                const int kb_begin = split * p.kb_per_split;
                const int kb_end = (kb_begin + p.kb_per_split < num_kb) ? kb_begin + p.kb_per_split : num_kb;
                ok = mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, s_abort, p.status, 0x200 | acc);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    ok = mbar_wait(full_bar(stage), phase, s_abort, p.status, 0x300 | stage);
                    if (!ok) break;
                    tcgen05_fence_after();
                    if (lane == 0) {
                        const uint32_t a_addr = smem_base + stage * C::STAGE_BYTES;
                        const uint32_t b_addr = a_addr + C::A_STAGE_BYTES;
#pragma unroll
                        for (int k = 0; k < C::BKS / UMMA_K; ++k) {
                            // K-major: atom (k / 4) of the stage, then 32 bytes inside the 128-byte
                            // swizzle row. MN-major: the stage is contiguous k-rows of 128 bytes.
                            constexpr int KPA = BK / UMMA_K;
                            const uint32_t a_off = A_MN ? k * UMMA_K * 128 : (k / KPA) * C::A_ATOM_BYTES + (k % KPA) * UMMA_K;
                            const uint32_t b_off = B_MN ? k * UMMA_K * 128 : (k / KPA) * C::B_ATOM_BYTES + (k % KPA) * UMMA_K;
                            const uint64_t a_desc = A_MN ? make_smem_desc(a_addr + a_off, C::BKS * 128, 1024) : make_smem_desc(a_addr + a_off, 16, 1024);
                            const uint64_t b_desc = B_MN ? make_smem_desc(b_addr + b_off, C::BKS * 128, 1024) : make_smem_desc(b_addr + b_off, 16, 1024);
                            if constexpr (CG == 2) tcgen05_mma_pair<KIND>(d_tmem, a_desc, b_desc, idesc, (kb > kb_begin || k != 0) ? 1u : 0u);
                            else tcgen05_mma<KIND>(d_tmem, a_desc, b_desc, idesc, (kb > kb_begin || k != 0) ? 1u : 0u);
                        }
                        // stage reusable (in both CTAs) once these MMAs retire
                        if constexpr (CG == 2) {
                            tcgen05_commit_pair(empty_bar(stage));
                            if (kb == kb_end - 1) tcgen05_commit_pair(tmem_full_bar(acc));
                        } else {
                            tcgen05_commit(empty_bar(stage));
                            if (kb == kb_end - 1) tcgen05_commit(tmem_full_bar(acc));
                        }
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ===== epilogue: two groups of warps; group g drains accumulator g, i.e. every second tile of this CTA, so
        // two tiles are in the epilogue at a time. Inside a group a warp owns the 32 accumulator rows of its TMEM lane
        // quarter and, when two warps share a quarter, one half of the tile's columns; it takes them in chunks of
        // EPI_CHUNK columns. The chunk code is a chain of short latencies (TMEM load, conversions, shared-memory
        // staging, proxy fence, TMA store) and is bound by instruction fetch and issue, so it is kept compact =====
        const int e = warp - 2;
        const int ew = warp & 3;                          // TMEM lane quarter this warp may read
        const int grp = e / EPI_GROUP_WARPS;
        int acc = EPI_GROUPS == 2 ? grp : 0;              // accumulator buffer = parity of the CTA's tile count
        const int half = (e >> 2) % EPI_COL_SPLIT;        // which part of the tile's columns
        const int esz = (EPI == EPI_RAW || p.scale_dtype == QT_F32) ? 4 : 2;
        const bool via_tma = p.tma_store == 1;
        const uint32_t stage_addr = smem_base + C::SMEM_STORE_OFF + (uint32_t)e * STORE_STAGE_BYTES;
        // this lane's row of the staging box; 16-byte piece q of the row sits at piece q ^ (row % 8) for 128-byte rows,
        // q ^ ((row / 2) % 4) for 64-byte rows (the swizzle the output tensor map declares): conflict-free vector stores
        const uint32_t stage_row = stage_addr + (uint32_t)lane * (uint32_t)STORE_BOX_BYTES;
        const uint32_t swz = STORE_BOX_BYTES == 128 ? (uint32_t)(lane & 7) : (uint32_t)((lane >> 1) & 3);
        constexpr int PIECES = STORE_BOX_BYTES / 16;
        uint32_t acc_phase = 0;
        bool ok = true;

        // Scales are requested one tile ahead and stay as loaded (raw bits) until the tile starts, so that nothing
        // waits for them where they are requested: this lane's row scale, and its 8 of the tile's 256 column
        // scales. Every warp of the group then writes all 256 column scales (as fp32) to the group's shared array:
        // the warps write identical values, so no barrier is needed between them, and a warp only gets here after
        // all of the group handed the previous accumulator back, which they do after their last read of the previous
        // tile's scales.
        const bool scale_is_bf16 = p.scale_dtype == QT_BF16;
        uint32_t next_rs_raw = 0;          // bf16: the 16 bits as loaded; fp32: the value's bits
        uint4 next_cs[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
        bool next_cs_packed = false;
        auto request_scales = [&](const WorkItem& w) {
            const int64_t r = (int64_t)w.m * (BM * CG) + (int64_t)cta_rank * BM + ew * 32 + lane;
            if (r >= p.M) next_rs_raw = 0u;
            else if (p.scale_a == nullptr) next_rs_raw = scale_is_bf16 ? 0x3F80u : 0x3F800000u;
            else if (scale_is_bf16) next_rs_raw = __ldg(reinterpret_cast<const unsigned short*>(p.scale_a) + r);
            else next_rs_raw = __ldg(reinterpret_cast<const uint32_t*>(p.scale_a) + r);
            next_cs_packed = load_col_scales8(next_cs, p, (int64_t)w.n * BN + lane * 8);
        };
        uint32_t work = first_tile + (EPI_GROUPS == 2 ? (uint32_t)grp * tile_step : 0u);
        const uint32_t work_step = (uint32_t)EPI_GROUPS * tile_step;
        WorkItem next_item = locate(work < num_work ? work : 0u);
        if constexpr (EPI == EPI_ROWCOL) {
            if (work < num_work) request_scales(next_item);
        }
        for (; work < num_work && ok; work += work_step) {
            const WorkItem tc = next_item;
            const int split = tc.split;
            const int64_t m0 = (int64_t)tc.m * (BM * CG) + (int64_t)cta_rank * BM;
            const int64_t n0 = (int64_t)tc.n * BN + half * EPI_WARP_COLS;   // first column of this warp's half
            const int64_t row0 = m0 + ew * 32;
            const int64_t row = row0 + lane;
            // split-K partials go out raw, one [M][N] plane per split
            uint32_t* ws_row = (p.splits > 1 && row < p.M) ? p.ws + ((int64_t)split * p.M + row) * p.N : nullptr;

            // the column scales of a tile sit in the shared array of its accumulator
            float* cs_grp = reinterpret_cast<float*>(smem + C::SMEM_COLSCALE_OFF) + acc * BN;
            const uint32_t cs_grp_addr = smem_base + C::SMEM_COLSCALE_OFF + (uint32_t)acc * BN * 4u;
            const uint32_t empty_bar_addr = CG == 2 ? map_to_cta(tmem_empty_bar(acc), 0) : tmem_empty_bar(acc);
            ok = mbar_wait(tmem_full_bar(acc), acc_phase, s_abort, p.status, 0x400 | acc);
            if (!ok) break;
            tcgen05_fence_after();
            const float row_scale = __uint_as_float(scale_is_bf16 ? next_rs_raw << 16 : next_rs_raw);
            if constexpr (EPI == EPI_ROWCOL) {
                if (p.splits == 1) {
                    uint4 lo = next_cs[0], hi = next_cs[1];
                    if (next_cs_packed) {
                        const uint4 w = next_cs[0];
                        lo = make_uint4(w.x << 16, w.x & 0xFFFF0000u, w.y << 16, w.y & 0xFFFF0000u);
                        hi = make_uint4(w.z << 16, w.z & 0xFFFF0000u, w.w << 16, w.w & 0xFFFF0000u);
                    }
                    st_shared_v4(cs_grp_addr + (uint32_t)lane * 32u, lo.x, lo.y, lo.z, lo.w);
                    st_shared_v4(cs_grp_addr + (uint32_t)lane * 32u + 16u, hi.x, hi.y, hi.z, hi.w);
                    __syncwarp();
                }
            }

            const uint32_t t_row = tmem_base + ((uint32_t)(ew * 32) << 16) + (uint32_t)(acc * BN + half * EPI_WARP_COLS);
            // hand the accumulator back to the MMA issuer (after this warp's last TMEM load has completed)
            auto release_acc = [&]() {
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (CG == 2) mbar_arrive_cluster_relaxed(empty_bar_addr);   // the pair's accumulator: both CTAs report to the leader
                    else mbar_arrive(empty_bar_addr);
                }
            };
            constexpr int CW = EPI_CHUNK;
            constexpr int CHUNKS = EPI_WARP_COLS / CW;
            uint32_t r[CW];
            auto tmem_ld_chunk = [&](uint32_t taddr) { tmem_ld_cols(taddr, r); };
            // The chunk loops below are real loops over compact bodies, one per output form, chosen once per tile:
            // the epilogue is bound by instruction fetch and issue, not by arithmetic. Every form issues the next
            // chunk's TMEM load as soon as r is free, so that it is in flight during the staging and the store.

            // r (accumulator values) -> scaled outputs: 16 bf16 pairs in w (BF16) or 32 fp32 values back in r.
            // cbase = the chunk's first column in the group's shared scale array.
            auto scale_chunk = [&](auto csf_tag, auto bf16_tag, uint32_t (&w)[CW / 2], int cbase) {
                constexpr bool CSF = decltype(csf_tag)::value;     // (acc * col_scale) * row_scale instead of (acc * row_scale) * col_scale
                constexpr bool BF16 = decltype(bf16_tag)::value;
                const float2 rs2 = make_float2(row_scale, row_scale);
#pragma unroll
                for (int g = 0; g < CW / 8; ++g) {
                    const float4 c0 = *reinterpret_cast<const float4*>(cs_grp + cbase + g * 8);      // broadcast reads
                    const float4 c1 = *reinterpret_cast<const float4*>(cs_grp + cbase + g * 8 + 4);
                    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        float a0 = (KIND == 0) ? (float)(int32_t)r[g * 8 + j] : __uint_as_float(r[g * 8 + j]);
                        float a1 = (KIND == 0) ? (float)(int32_t)r[g * 8 + j + 1] : __uint_as_float(r[g * 8 + j + 1]);
                        if constexpr (KIND == 2) {
                            if (p.round_acc_first) {
                                const uint32_t rb = pack_bf16x2(a0, a1);
                                a0 = __uint_as_float(rb << 16);
                                a1 = __uint_as_float(rb & 0xFFFF0000u);
                            }
                        }
                        // fp32 multiplication is not associative: the order is the caller's (a product computed in
                        // transposed form keeps the rounding of the untransposed one). Two columns per packed multiply.
                        const float2 cs2 = make_float2(cs[j], cs[j + 1]);
                        const float2 t = CSF ? __fmul2_rn(__fmul2_rn(make_float2(a0, a1), cs2), rs2)
                                             : __fmul2_rn(__fmul2_rn(make_float2(a0, a1), rs2), cs2);
                        if constexpr (BF16) {
                            w[g * 4 + j / 2] = pack_bf16x2(t.x, t.y);
                        } else {
                            r[g * 8 + j] = __float_as_uint(t.x);
                            r[g * 8 + j + 1] = __float_as_uint(t.y);
                        }
                    }
                }
            };
            // after the tile's last read of the shared column scales the accumulator can go back (its last TMEM load
            // completed before the chunk started); the arrive carries no memory ordering when it crosses to the peer
            // CTA, so it is made to wait for values computed from those reads
            auto release_after = [&](uint32_t a, uint32_t b, uint32_t c_, uint32_t d) {
                asm volatile("" ::"r"(a), "r"(b), "r"(c_), "r"(d) : "memory");
                release_acc();
            };

            tmem_ld_chunk(t_row);
            // while that load is in flight: find this group's next tile and request its scales
            if (work + work_step < num_work) {
                next_item = locate(work + work_step);
                if constexpr (EPI == EPI_ROWCOL) request_scales(next_item);
            }
            if (p.splits > 1) {
                // split-K partial: raw accumulators, this lane's row of the split's plane
#pragma unroll 1
                for (int c = 0; c < CHUNKS; ++c) {
                    const int64_t n = n0 + c * CW;
                    tmem_ld_wait();
                    if (c == CHUNKS - 1) release_acc();
                    if (ws_row != nullptr && n < p.N) {
                        uint32_t* dst = ws_row + n;
                        if (n + CW <= p.N && (p.N & 7) == 0) {
#pragma unroll
                            for (int j = 0; j < CW; j += 8)
                                st_global_v8(dst + j, r[j], r[j + 1], r[j + 2], r[j + 3], r[j + 4], r[j + 5], r[j + 6], r[j + 7]);
                        } else {
#pragma unroll
                            for (int j = 0; j < CW; ++j)
                                if (n + j < p.N) dst[j] = r[j];
                        }
                    }
                    if (c + 1 < CHUNKS) tmem_ld_chunk(t_row + (c + 1) * CW);
                }
            } else if (via_tma && esz == 2) {
                // bf16 output through the staging box: one chunk = one box of 32 rows
#pragma unroll 1
                for (int c = 0; c < CHUNKS; ++c) {
                    const int64_t n = n0 + c * CW;
                    uint32_t w[CW / 2];
                    tmem_ld_wait();
                    if (p.col_scale_first) scale_chunk(std::true_type{}, std::true_type{}, w, half * EPI_WARP_COLS + c * CW);
                    else scale_chunk(std::false_type{}, std::true_type{}, w, half * EPI_WARP_COLS + c * CW);
                    if (c + 1 < CHUNKS) tmem_ld_chunk(t_row + (c + 1) * CW);
                    else release_after(w[0], w[CW / 8 + 1], w[CW / 4 + 2], w[CW / 2 - 1]);
                    // the previous box's store was issued a whole chunk ago: its read of the staging buffer has
                    // overlapped this chunk's TMEM wait and arithmetic
                    const uint32_t buf = STORE_BUFS == 2 ? (uint32_t)(c & 1) * (uint32_t)STORE_BOX_TOTAL : 0u;   // (CHUNKS is even)
                    if (lane == 0) {
                        if constexpr (STORE_BUFS == 2) bulk_store_wait_read_but_one();
                        else bulk_store_wait_read();
                    }
                    __syncwarp();
#pragma unroll
                    for (int g = 0; g < PIECES; ++g)
                        st_shared_v4(stage_row + buf + (((uint32_t)g ^ swz) << 4), w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        // (a group is committed also when the box lies outside the output: the waits count groups)
                        if (row0 < p.M && n < p.N) tma_store_2d(&tmap_c, stage_addr + buf, (int)(n * 2), (int)row0);
                        bulk_store_commit();
                    }
                }
            } else {
                // 4-byte outputs (raw int32 / fp32, or scaled fp32): two boxes per chunk; and outputs
                // whose base or pitch is not 16-byte aligned: element stores
#pragma unroll 1
                for (int c = 0; c < CHUNKS; ++c) {
                    const int64_t n = n0 + c * CW;
                    uint32_t w[CW / 2];
                    tmem_ld_wait();
                    if constexpr (EPI == EPI_ROWCOL) {
                        if (esz == 2) {
                            if (p.col_scale_first) scale_chunk(std::true_type{}, std::true_type{}, w, half * EPI_WARP_COLS + c * CW);
                            else scale_chunk(std::false_type{}, std::true_type{}, w, half * EPI_WARP_COLS + c * CW);
                        } else {
                            if (p.col_scale_first) scale_chunk(std::true_type{}, std::false_type{}, w, half * EPI_WARP_COLS + c * CW);
                            else scale_chunk(std::false_type{}, std::false_type{}, w, half * EPI_WARP_COLS + c * CW);
                        }
                        if (c == CHUNKS - 1) {
                            if (esz == 2) release_after(w[0], w[CW / 8 + 1], w[CW / 4 + 2], w[CW / 2 - 1]);
                            else release_after(r[0], r[CW / 4 + 1], r[CW / 2 + 2], r[CW - 1]);
                        }
                    } else {
                        if (c == CHUNKS - 1) release_acc();
                    }
                    if (via_tma) {
#pragma unroll
                        for (int hb = 0; hb < 2; ++hb) {
                            const uint32_t buf = STORE_BUFS == 2 ? (uint32_t)hb * (uint32_t)STORE_BOX_TOTAL : 0u;
                            if (lane == 0) {
                                if constexpr (STORE_BUFS == 2) bulk_store_wait_read_but_one();   // the box used two stores ago has left shared memory
                                else bulk_store_wait_read();
                            }
                            __syncwarp();
#pragma unroll
                            for (int g = 0; g < PIECES; ++g)
                                st_shared_v4(stage_row + buf + (((uint32_t)g ^ swz) << 4), r[hb * (CW / 2) + 4 * g], r[hb * (CW / 2) + 4 * g + 1],
                                             r[hb * (CW / 2) + 4 * g + 2], r[hb * (CW / 2) + 4 * g + 3]);
                            fence_proxy_async_smem();
                            __syncwarp();
                            const int64_t nb = n + hb * (CW / 2);   // first column of the box
                            if (lane == 0) {
                                if (row0 < p.M && nb < p.N) tma_store_2d(&tmap_c, stage_addr + buf, (int)(nb * 4), (int)row0);
                                bulk_store_commit();
                            }
                        }
                    } else if (row < p.M) {
                        // (unrolled: the chunk registers must never be indexed dynamically)
#pragma unroll
                        for (int j = 0; j < CW; ++j) {
                            if (n + j < p.N) {
                                const int64_t at = row * p.ldc + n + j;
                                if (esz == 4) reinterpret_cast<uint32_t*>(p.c)[at] = r[j];
                                else reinterpret_cast<uint16_t*>(p.c)[at] = (uint16_t)((w[j >> 1] >> (16 * (j & 1))) & 0xFFFFu);
                            }
                        }
                    }
                    if (c + 1 < CHUNKS) tmem_ld_chunk(t_row + (c + 1) * CW);
                }
            }
            if constexpr (EPI_GROUPS == 2) {
                acc_phase ^= 1u;
            } else {
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
        // shared memory must outlive the last store's read of it; global visibility follows at grid end
        if (via_tma && lane == 0) bulk_store_wait_all();
    }

    tcgen05_fence_before();
    __syncthreads();
    // nobody leaves while the peer may still signal this CTA's barriers or read its shared memory
    if constexpr (CG == 2) cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        if constexpr (CG == 2)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// 0 = choose per problem, 1 / 2 = force that many CTAs per MMA (set through qt_set_gemm_cta_group)
int g_forced_cta_group = 0;
int g_forced_group_m = 0;   // test / tuning override of the rasterisation group height (0 = chosen per problem)
// SMs the persistent GEMM grids leave free for kernels that must run beside them (collectives)
int g_sm_margin = 0;

template <int KIND, int EPI, bool A_MN, bool B_MN, int CG>
int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, uint32_t idesc,
               int64_t tiles, cudaStream_t stream) {
    auto kfn = gemm_kernel<KIND, EPI, A_MN, B_MN, CG>;
    constexpr int SMEM = Cfg<CG>::SMEM_TOTAL;
    static bool attr_set[64] = {false};
    static int max_clusters[64] = {0};
    int dev = 0;
    QT_CUDA_CHECK(cudaGetDevice(&dev));
    const bool cacheable = dev >= 0 && dev < 64;
    if (!cacheable || !attr_set[dev]) {
        QT_CUDA_CHECK(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        if (cacheable) attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if constexpr (CG == 2) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n_clusters = cacheable ? max_clusters[dev] : 0;
        if (n_clusters == 0) {
            cfg.gridDim = dim3((unsigned)(num_sms() / 2 * 2));
            QT_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n_clusters, kfn, &cfg));
            if (n_clusters <= 0) return fail(QT_ERR_CUDA, "gemm: no 2-CTA cluster of this kernel fits on the device");
            if (cacheable) max_clusters[dev] = n_clusters;
        }
        int usable = n_clusters - (g_sm_margin + 1) / 2;
        if (usable < 1) usable = 1;
        const int64_t pairs = tiles < usable ? tiles : usable;
        cfg.gridDim = dim3((unsigned)(2 * pairs));
    } else {
        int sms = num_sms() - g_sm_margin;
        if (sms < 1) sms = 1;
        cfg.gridDim = dim3((unsigned)(tiles < sms ? tiles : sms));
    }
    QT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kfn, ta, tb, tc, p, idesc));
    return QT_OK;
}

template <int KIND, int EPI, int CG>
int launch_layout(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                  uint32_t idesc, int64_t tiles, cudaStream_t stream) {
    if (!a_mn && !b_mn) return launch_one<KIND, EPI, false, false, CG>(ta, tb, tc, p, idesc, tiles, stream);
    if (!a_mn && b_mn) return launch_one<KIND, EPI, false, true, CG>(ta, tb, tc, p, idesc, tiles, stream);
    if (a_mn && b_mn) return launch_one<KIND, EPI, true, true, CG>(ta, tb, tc, p, idesc, tiles, stream);
    return launch_one<KIND, EPI, true, false, CG>(ta, tb, tc, p, idesc, tiles, stream);
}

// Sums the split-K partial planes and applies the epilogue. Integer partials add exactly, so the
// result is bit-identical to the unsplit kernel; fp8 partials add in fp32 in split order.
template <int KIND, int EPI>
__global__ void __launch_bounds__(256) splitk_finish_kernel(const GemmParams p) {
    const int64_t total = p.M * p.N;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
        const int64_t row = i / p.N, col = i - row * p.N;
        float v;
        int32_t isum = 0;
        if constexpr (KIND == 0) {
            for (int s = 0; s < p.splits; ++s) isum += (int32_t)p.ws[(int64_t)s * total + i];
            v = (float)isum;
        } else {
            float fsum = 0.0f;
            for (int s = 0; s < p.splits; ++s) fsum = __fadd_rn(fsum, __uint_as_float(p.ws[(int64_t)s * total + i]));
            v = fsum;
        }
        if constexpr (EPI == EPI_RAW) {
            reinterpret_cast<uint32_t*>(p.c)[row * p.ldc + col] = (KIND == 0) ? (uint32_t)isum : __float_as_uint(v);
        } else {
            const float rs = p.scale_a ? load_scale(p.scale_a, p.scale_dtype, row) : 1.0f;
            if (KIND == 2 && p.round_acc_first) v = __bfloat162float(__float2bfloat16_rn(v));
            const float cs = load_scale(p.scale_b, p.scale_dtype, p.scale_b_is_scalar ? 0 : col);
            const float o = p.col_scale_first ? __fmul_rn(__fmul_rn(v, cs), rs) : __fmul_rn(__fmul_rn(v, rs), cs);
            if (p.scale_dtype == QT_BF16) reinterpret_cast<__nv_bfloat16*>(p.c)[row * p.ldc + col] = __float2bfloat16_rn(o);
            else reinterpret_cast<float*>(p.c)[row * p.ldc + col] = o;
        }
    }
}

template <int KIND, int EPI>
int launch_finish(const GemmParams& p, cudaStream_t stream) {
    const int64_t total = p.M * p.N;
    const int64_t want = (total + 255) / 256;
    const int64_t cap = (int64_t)num_sms() * 8;
    splitk_finish_kernel<KIND, EPI><<<(unsigned)(want < cap ? want : cap), 256, 0, stream>>>(p);
    QT_CUDA_CHECK(cudaGetLastError());
    return QT_OK;
}

// Split K when the output has too few tiles to occupy the machine (the grad-weight GEMMs: a small
// [K_out, N] result reduced over tens of thousands of tokens). Every split keeps at least 4 stages.
void choose_splits(int64_t M, int64_t N, int64_t K, int cg, int* splits, int* kb_per_split) {
    const int bks = cg == 2 ? Cfg<2>::BKS : Cfg<1>::BKS;
    const int64_t tiles = ((M + BM * cg - 1) / (BM * cg)) * ((N + BN - 1) / BN);
    const int num_kb = (int)((K + bks - 1) / bks);
    const int units = cg == 2 ? num_sms() / 2 : num_sms();
    *splits = 1;
    *kb_per_split = num_kb;
    if (tiles * 2 > units || num_kb < 8) return;
    int64_t s = units / tiles;
    if (s > num_kb / 4) s = num_kb / 4;
    if (s > 32) s = 32;
    if (s < 2) return;
    const int per = (int)((num_kb + s - 1) / s);
    *kb_per_split = per;
    *splits = (num_kb + per - 1) / per;
}

// CTA pairs pay off when there is more than one row block and the reduction is at least two stages long
// (512 bytes: int8 / fp8 K >= 512, bf16 K >= 256). With the current epilogue the pair form measured faster
// than the single-CTA form from that length up.
int pick_cta_group(int64_t M, int64_t K) {
    int cg = g_forced_cta_group;
    if (cg != 1 && cg != 2) cg = (M > BM && K >= 512) ? 2 : 1;
    return cg;
}

int gemm_dispatch(int epi, const void* a, int a_dtype, int64_t a_sm, int64_t a_sk, const void* b, int b_dtype, int64_t b_sk,
                  int64_t b_sn, GemmParams p, void* workspace, int64_t workspace_bytes, void* stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const bool is_bf16 = a_dtype == QT_BF16 && b_dtype == QT_BF16;
    if (is_bf16) {
        // 16-bit operands ride the same pipeline measured in bytes: a K-major tile is [rows][128 B of K] whatever
        // the element size, and one kind::f16 instruction consumes 32 reduction bytes like kind::i8. Only the
        // K-major layouts (A@B.T) are wired up; strides arrive in elements and turn into bytes here.
        QT_REQUIRE(a_sk == 1 && b_sk == 1, "gemm: bf16 operands must both be K-major (A [M,K] and B^T [N,K] with unit inner stride)");
        QT_REQUIRE(p.K < (1ll << 30), "gemm: dimension exceeds 2^30");
        p.K *= 2; a_sm *= 2; b_sn *= 2;
    }
    const int64_t M = p.M, N = p.N, K = p.K;
    QT_REQUIRE(M >= 0 && N >= 0 && K >= 0, "gemm: negative dimension");
    QT_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "gemm: dimension exceeds 2^31");
    const bool is_i8 = a_dtype == QT_I8 && b_dtype == QT_I8;
    const bool is_f8 = (a_dtype == QT_E4M3 || a_dtype == QT_E5M2) && (b_dtype == QT_E4M3 || b_dtype == QT_E5M2);
    QT_REQUIRE(is_i8 || is_f8 || is_bf16, "gemm: operands must both be int8, both fp8 or both bf16 (got %d, %d)", a_dtype, b_dtype);
    if (M == 0 || N == 0) return QT_OK;
    QT_REQUIRE(a && b && p.c, "gemm: null operand");
    QT_REQUIRE(K > 0, "gemm: K must be positive (zero-length reductions are handled by the caller)");
    QT_REQUIRE((a_sk == 1) != (a_sm == 1) || (M == 1 || K == 1), "gemm: exactly one stride of A must be 1 (got %lld, %lld)", (long long)a_sm, (long long)a_sk);
    QT_REQUIRE((b_sk == 1) != (b_sn == 1) || (N == 1 || K == 1), "gemm: exactly one stride of B must be 1 (got %lld, %lld)", (long long)b_sk, (long long)b_sn);
    const bool a_mn = (a_sk != 1);  // A stored [K][M]
    const bool b_mn = (b_sk != 1);  // B stored [K][N]
    const int64_t a_pitch = a_mn ? a_sk : a_sm;
    const int64_t b_pitch = b_mn ? b_sk : b_sn;
    QT_REQUIRE(aligned_to(a, 16) && aligned_to(b, 16), "gemm: operand base pointers must be 16-byte aligned");
    QT_REQUIRE(a_pitch % 16 == 0 && b_pitch % 16 == 0, "gemm: the non-unit operand strides must be multiples of 16 (got %lld, %lld)", (long long)a_pitch, (long long)b_pitch);
    QT_REQUIRE(a_pitch >= (a_mn ? M : K) && b_pitch >= (b_mn ? N : K), "gemm: operand stride smaller than the contiguous extent");
    QT_REQUIRE(p.ldc >= N, "gemm: ldc smaller than N");

    // A CTA pair per 256-row tile pays off once there are at least two row blocks of work per SM pair;
    // short problems keep the single-CTA form (more, smaller tiles).
    const int cg = pick_cta_group(M, K);
    const int b_rows = BN / cg;
    p.splits = 1;
    p.ws = nullptr;
    {
        const int bks = cg == 2 ? Cfg<2>::BKS : Cfg<1>::BKS;
        p.kb_per_split = (int)((K + bks - 1) / bks);
    }
    if (workspace != nullptr) {
        int splits = 1, per = 0;
        choose_splits(M, N, K, cg, &splits, &per);
        if (splits > 1 && workspace_bytes >= (int64_t)splits * M * N * 4 && aligned_to(workspace, 32)) {
            p.splits = splits;
            p.kb_per_split = per;
            p.ws = reinterpret_cast<uint32_t*>(workspace);
        }
    }

    // Rasterisation: a group of `group_m` row-tiles sweeps all column-tiles, so B is streamed from DRAM once per
    // group while the group's A panel sits in L2. Taller groups mean fewer passes over B (at 8192^3 with CTA
    // pairs: 16 instead of 8 halves them, 335 MB of DRAM traffic against 461 MB), but under the power cap the
    // GEMM's speed did not follow: 8 and 16 measured the same within run-to-run noise (2.83-2.92 POPS) and 32
    // was 6 % slower, so 8 stays the default and the height is a tuning knob.
    p.group_m = g_forced_group_m > 0 ? g_forced_group_m : GROUP_M;

    CUtensorMap ta, tb;
    if (a_mn) { if (int rc = make_tmap(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)a_pitch, 128, BK)) return rc; }
    else      { if (int rc = make_tmap(&ta, a, (uint64_t)K, (uint64_t)M, (uint64_t)a_pitch, BK, BM)) return rc; }
    if (b_mn) { if (int rc = make_tmap(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)b_pitch, 128, BK)) return rc; }
    else      { if (int rc = make_tmap(&tb, b, (uint64_t)K, (uint64_t)N, (uint64_t)b_pitch, BK, (uint32_t)b_rows)) return rc; }

    // the output as a byte tensor (rows of N * esz bytes): boxes of 32 rows x STORE_BOX_BYTES, clipped at the edges
    const int esz = (epi == EPI_RAW || p.scale_dtype == QT_F32) ? 4 : 2;
    p.tma_store = (p.splits == 1 && aligned_to(p.c, 16) && (p.ldc * esz) % 16 == 0) ? 1 : 0;
    p.cs_vec = (epi == EPI_ROWCOL && aligned_to(p.scale_b, 16)) ? 1 : 0;
    CUtensorMap tc = ta;  // a valid map even when unused
    if (p.tma_store) {
        if (int rc = make_tmap(&tc, p.c, (uint64_t)(N * esz), (uint64_t)M, (uint64_t)(p.ldc * esz), STORE_BOX_BYTES, 32,
                               STORE_BOX_BYTES == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B)) return rc;
    }

    if (int rc = device_status_ptr(&p.status)) return rc;

    const int64_t tiles = ((M + BM * cg - 1) / (BM * cg)) * ((N + BN - 1) / BN) * p.splits;  // work items
    QT_REQUIRE(tiles < (1ll << 30), "gemm: %lld work items exceed the kernel's 32-bit tile index", (long long)tiles);
    // kind::f16 operand formats: 0 = f16, 1 = bf16
    const uint32_t idesc = is_i8 ? make_idesc(2, 1, 1, a_mn, b_mn, BM * cg, BN)
                           : is_bf16 ? make_idesc(1, 1, 1, false, false, BM * cg, BN)
                                     : make_idesc(1, fp8_format(a_dtype), fp8_format(b_dtype), a_mn, b_mn, BM * cg, BN);
#define QT_DISPATCH(KIND, EPI)                                                                               \
    do {                                                                                                     \
        const int rc_ = cg == 2 ? launch_layout<KIND, EPI, 2>(a_mn, b_mn, ta, tb, tc, p, idesc, tiles, stream)   \
                                : launch_layout<KIND, EPI, 1>(a_mn, b_mn, ta, tb, tc, p, idesc, tiles, stream);  \
        if (rc_ != QT_OK || p.splits == 1) return rc_;                                                       \
        return launch_finish<KIND, EPI>(p, stream);                                                          \
    } while (0)
    if (is_i8) {
        if (epi == EPI_RAW) { QT_DISPATCH(0, EPI_RAW); }
        if (epi == EPI_ROWCOL) { QT_DISPATCH(0, EPI_ROWCOL); }
    } else if (is_bf16) {
        if (epi == EPI_ROWCOL) {
            const int rc_ = cg == 2 ? launch_one<2, EPI_ROWCOL, false, false, 2>(ta, tb, tc, p, idesc, tiles, stream)
                                    : launch_one<2, EPI_ROWCOL, false, false, 1>(ta, tb, tc, p, idesc, tiles, stream);
            if (rc_ != QT_OK || p.splits == 1) return rc_;
            return launch_finish<2, EPI_ROWCOL>(p, stream);
        }
    } else {
        if (epi == EPI_ROWCOL) { QT_DISPATCH(1, EPI_ROWCOL); }
    }
#undef QT_DISPATCH
    return fail(QT_ERR_UNSUPPORTED, "gemm: epilogue %d not implemented for this operand type", epi);
}

}  // namespace

}  // namespace qt

using namespace qt;

namespace qt {
namespace {
// One warp waits on an mbarrier that nothing ever arrives on, with a 50 ms limit: the wait gives up,
// sets the abort flag and records its code, and the kernel returns normally.
__global__ void wait_timeout_selftest_kernel(int* status) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    const uint32_t bar_addr = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(bar_addr, 1);
        abort_flag = 0;
    }
    __syncthreads();
    mbar_wait(bar_addr, 0u, &abort_flag, status, 0x7E57, 50000000ull);
}
}  // namespace
}  // namespace qt

extern "C" int qt_selftest_wait_timeout(int* observed_status, int leave_set) {
    QT_REQUIRE(observed_status, "selftest_wait_timeout: null output");
    int* status = nullptr;
    if (int rc = device_status_ptr(&status)) return rc;
    int before = 0;
    QT_CUDA_CHECK(cudaDeviceSynchronize());
    QT_CUDA_CHECK(cudaMemcpy(&before, status, sizeof(int), cudaMemcpyDeviceToHost));
    if (before != 0) return fail(QT_ERR_DEVICE, "selftest_wait_timeout: the device status word is already set (%#x)", before);
    wait_timeout_selftest_kernel<<<1, 32>>>(status);
    QT_CUDA_CHECK(cudaGetLastError());
    QT_CUDA_CHECK(cudaDeviceSynchronize());
    QT_CUDA_CHECK(cudaMemcpy(observed_status, status, sizeof(int), cudaMemcpyDeviceToHost));
    if (!leave_set) {   // the word is clean again for the real kernels
        QT_CUDA_CHECK(cudaMemset(status, 0, sizeof(int)));
        if (volatile int* h = device_status_host_word()) *h = 0;
    }
    return QT_OK;
}

extern "C" int qt_set_gemm_group_m(int group_m) {
    QT_REQUIRE(group_m >= 0 && group_m <= 1024, "set_gemm_group_m: 0 (automatic) or a number of row-tiles up to 1024 (got %d)", group_m);
    g_forced_group_m = group_m;
    return QT_OK;
}

extern "C" int qt_set_gemm_sm_margin(int sms) {
    QT_REQUIRE(sms >= 0 && sms < 128, "set_gemm_sm_margin: expected 0..127 (got %d)", sms);
    g_sm_margin = sms;
    return QT_OK;
}

extern "C" int qt_set_gemm_cta_group(int cta_group) {
    QT_REQUIRE(cta_group == 0 || cta_group == 1 || cta_group == 2, "set_gemm_cta_group: expected 0 (auto), 1 or 2");
    g_forced_cta_group = cta_group;
    return QT_OK;
}

extern "C" int64_t qt_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    int splits = 1, per = 0;
    choose_splits(M, N, K, pick_cta_group(M, K), &splits, &per);
    return splits > 1 ? (int64_t)splits * M * N * 4 : 0;
}

extern "C" int qt_int8_mm_ws(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, int32_t* c,
                             int64_t ldc, int64_t M, int64_t N, int64_t K, void* workspace, int64_t workspace_bytes, void* stream) {
    GemmParams p = {};
    p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc;
    return gemm_dispatch(EPI_RAW, a, QT_I8, a_sm, a_sk, b, QT_I8, b_sk, b_sn, p, workspace, workspace_bytes, stream);
}

extern "C" int qt_int8_mm(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, int32_t* c,
                          int64_t ldc, int64_t M, int64_t N, int64_t K, void* stream) {
    return qt_int8_mm_ws(a, a_sm, a_sk, b, b_sk, b_sn, c, ldc, M, N, K, nullptr, 0, stream);
}

extern "C" int qt_scaled_mm_ws(const void* a, int a_dtype, int64_t a_sm, int64_t a_sk, const void* b, int b_dtype, int64_t b_sk,
                               int64_t b_sn, const void* scale_a, const void* scale_b, int scale_b_is_scalar, int scale_dtype,
                               void* c, int64_t ldc, int64_t M, int64_t N, int64_t K, void* workspace, int64_t workspace_bytes,
                               void* stream) {
    QT_REQUIRE(scale_dtype == QT_BF16 || scale_dtype == QT_F32, "scaled_mm: scale_dtype must be QT_BF16 or QT_F32 (got %d)", scale_dtype);
    QT_REQUIRE((scale_a && scale_b) || M == 0 || N == 0, "scaled_mm: null scale pointer");
    GemmParams p = {};
    p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc;
    QT_REQUIRE(scale_b_is_scalar >= 0 && scale_b_is_scalar <= 3, "scaled_mm: scale_b_is_scalar holds flag bits 0 and 1 only (got %d)", scale_b_is_scalar);
    p.scale_a = scale_a; p.scale_b = scale_b; p.scale_b_is_scalar = scale_b_is_scalar & 1; p.col_scale_first = (scale_b_is_scalar >> 1) & 1;
    p.scale_dtype = scale_dtype;
    return gemm_dispatch(EPI_ROWCOL, a, a_dtype, a_sm, a_sk, b, b_dtype, b_sk, b_sn, p, workspace, workspace_bytes, stream);
}

extern "C" int qt_bf16_mm_colscale(const void* a, int64_t lda, const void* b, int64_t ldb, const void* col_scale, void* c, int64_t ldc,
                                   int64_t M, int64_t N, int64_t K, void* stream) {
    QT_REQUIRE(col_scale || M == 0 || N == 0, "bf16_mm_colscale: null scale pointer");
    QT_REQUIRE(lda >= K && ldb >= K, "bf16_mm_colscale: leading dimension smaller than K");
    if (K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0)
        return fail(QT_ERR_UNSUPPORTED, "bf16_mm_colscale: K and the leading dimensions must be multiples of 8 (16-byte rows)");
    GemmParams p = {};
    p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc;
    p.scale_a = nullptr; p.scale_b = col_scale; p.scale_b_is_scalar = 0; p.col_scale_first = 0; p.round_acc_first = 1;
    p.scale_dtype = QT_BF16;
    return gemm_dispatch(EPI_ROWCOL, a, QT_BF16, lda, 1, b, QT_BF16, 1, ldb, p, nullptr, 0, stream);
}

extern "C" int qt_scaled_mm(const void* a, int a_dtype, int64_t a_sm, int64_t a_sk, const void* b, int b_dtype, int64_t b_sk,
                            int64_t b_sn, const void* scale_a, const void* scale_b, int scale_b_is_scalar, int scale_dtype,
                            void* c, int64_t ldc, int64_t M, int64_t N, int64_t K, void* stream) {
    return qt_scaled_mm_ws(a, a_dtype, a_sm, a_sk, b, b_dtype, b_sk, b_sn, scale_a, scale_b, scale_b_is_scalar, scale_dtype, c,
                           ldc, M, N, K, nullptr, 0, stream);
}
