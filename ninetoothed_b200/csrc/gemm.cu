// matmul / addmm on tcgen05: the tiled dot-accumulate loop of the reference's
// matmul application (README.md:56-62, tests/test_matmul.py:41-45) and the addmm
// epilogue fused behind it (tests/test_addmm.py:35-38).
//
// Persistent CTAs, six warps each:
//   warp 0      TMA producer: A and B tiles -> 128-byte-swizzled shared-memory ring
//   warp 1      MMA issuer: one thread issues tcgen05.mma (fp32 accumulators in tensor
//               memory); also owns the TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one row per thread), round,
//               fuse beta*C + alpha*AB, store
// Two 256-column accumulator buffers fill the 512 TMEM columns, so the epilogue of
// tile i overlaps the main loop of tile i+1.
//
// Two shapes of the same kernel (template parameter CG = CTAs per MMA):
//   CG = 1  one CTA per 128 x 256 tile, 4 stages of 48 KB.
//   CG = 2  a cluster of two CTAs per 256 x 256 tile (tcgen05 cta_group::2): each CTA
//           loads its own 128 rows of A and its own 128 columns of B (half the B
//           traffic per SM, 6 stages of 32 KB), the even CTA issues one MMA that
//           spans both SMs, and each CTA drains its own 128 accumulator rows.  Loads
//           are plain (un-multicast) TMA; only barrier arrivals cross the pair.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <climits>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "host.h"
#include "ptx.cuh"

namespace nt {
namespace {

constexpr int BM = 128;   // accumulator rows per CTA
constexpr int MAX_BN = 256;  // tile columns: a template argument of the kernel, 256, 128 or 64
constexpr int BK = 64;    // 64 16-bit elements = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 16;  // default M-tiles per raster group (L2 reuse of A rows), in 128-row units
constexpr int TMEM_COLS = 512;
constexpr int MAX_STAGES = 8;
constexpr int MAX_PEERS = 7;   // other GPUs of one NVLink domain

template <int CG, int BN>
struct Shape {
    static constexpr int BN_CTA = BN / CG;                  // B columns this CTA loads
    static constexpr int B_STAGE_BYTES = BN_CTA * BK * 2;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    // as many stages as fit 192 KB (4 of 48 KB for a single CTA's 128 x 256 tile, 6 of 32 KB for a pair's CTA)
    static constexpr int STAGES = 192 * 1024 / STAGE_BYTES < MAX_STAGES ? 192 * 1024 / STAGE_BYTES : MAX_STAGES;
    static constexpr int TILE_M = BM * CG;
};

struct SharedControl {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

// Epilogue staging: each of the four epilogue warps owns 32 rows of 64 16-bit values; the 144-byte
// pitch keeps both the row-wise 16-byte writes and the transposed reads free of bank conflicts.
constexpr int STAGE_PITCH = 144;
constexpr int STAGE_OFFSET = (sizeof(SharedControl) + 15) / 16 * 16;
constexpr int STAGE_BYTES_TOTAL = 4 * 32 * STAGE_PITCH;

// (batched launches: control block, then eight 4 KB boxes for the bulk tensor stores)
template <int CG, int BN>
constexpr size_t smem_bytes_batched() {
    return 1024 + Shape<CG, BN>::STAGES * Shape<CG, BN>::STAGE_BYTES + 1024 + 4 * 2 * 32 * 128;
}

template <int CG, int BN>
constexpr size_t smem_bytes() {
    return 1024 /* alignment slack */ + Shape<CG, BN>::STAGES * Shape<CG, BN>::STAGE_BYTES + STAGE_OFFSET + STAGE_BYTES_TOTAL;
}

struct GemmParams {
    int m, n, k;
    int m_tiles, n_tiles, k_blocks;
    const void *c_in;  // addmm input (nullptr for matmul)
    void *out;         // destination 0
    // Further destinations with the same strides: buffers of peer GPUs (mapped into this process) that
    // receive a copy of every tile, which is how the all-gather of column slabs is fused into the epilogue.
    void *more_out[MAX_PEERS];
    int extra_dests;
    // out is a multicast address: every tile is stored once with multimem.st and the NVSwitch writes it into all
    // the ranks' buffers, this rank's included (no more_out then).
    int through_switch;
    int64_t c_stride0, c_stride1;
    int64_t out_stride0, out_stride1;
    float beta, alpha;
    uint32_t b_lbo, b_sbo;  // UMMA descriptor offsets of the B tile (bytes)
    unsigned int *status;
    // Split along K, for problems with too few tiles to occupy the device (split_workers > 0).  The k-blocks
    // of all tiles form one sequence of split_blocks entries, cut into split_workers equal runs, one per
    // worker.  A run is shorter than a tile's reduction, so it covers the end of one tile and possibly the
    // start of the next: its worker produces one or two partial accumulators, stored in split_partials in
    // the slot (worker, first/second, CTA of the pair).  A second kernel adds a tile's partials up in the
    // order of their k-ranges and applies the epilogue.
    int split_workers;
    int split_blocks;
    float *split_partials;
    // Raster: tiles are walked in groups of group_m tile-rows, row index fastest, so that the CTAs at work at any
    // moment cover a block of about group_m x (CTAs / group_m) tiles and share its A and B panels through L2.
    int group_m;
    // L2 eviction hints on the operand loads of unbatched launches (NINETOOTHED_B200_GEMM_L2_HINTS; a measurement
    // switch, default 0 = none: on the 8192^3 problem keeping the A panels of the raster group and letting B go
    // first raised DRAM reads from 1.4 to 2.4 GB, because the eight tiles of a column read a B panel at slightly
    // different times).
    int l2_hints;
    // Batched launches (BATCHED kernels only): `batches` independent problems that share A; B has a third
    // tensor-map dimension, the output of problem i starts out_batch_stride elements after that of i - 1.
    // Tiles are numbered batch-major.
    // a_batched: A has a batch dimension too (a batch of independent matmuls); otherwise one A serves them all.
    int batches;
    int a_batched;
    int64_t out_batch_stride;
    // Mixed tile widths (CTA pairs on 256-column tiles, unbatched, unsplit launches only; 0 = none).  When the
    // tiles make a whole number of waves plus a fraction, the last wave costs a whole tile's time with most pairs
    // idle.  In the first mixed_rows tile-rows, groups of three 256-column tiles are replaced by four tiles
    // of 192 columns each (the same 768 columns, one tile more per swap), which lets the host choose a
    // tile count that fills the waves with less work per pair: e.g. 128 tiles on 74 pairs (two waves, 512 columns
    // per pair) become 74 wide + 72 narrow ones (448 columns per pair).  Tiles are numbered: the tile-rows
    // without swaps in raster order, then the wide tiles of the mixed rows, then all the narrow ones, so that a
    // pair's stride through the numbers gives it the wide tiles first.
    int mixed_rows;
    int mixed_wide;    // 256-column tiles left in a mixed tile-row
    int mixed_narrow;  // 192-column tiles in a mixed tile-row (they follow the wide ones)
    int extra_tiles;   // tiles added by the swaps: mixed_rows * (mixed_wide + mixed_narrow - n_tiles)
};

constexpr int NARROW_BN = 192;

struct TilePlace {
    int m_tile, col0, width;
};

// One piece of work for a worker: k-blocks [kb0, kb1) of a tile.  slot < 0: the whole reduction, the
// accumulator goes straight to the output.  Otherwise a partial accumulator, stored in that slot.
struct Unit {
    int tile, kb0, kb1, slot;
};

// (the host only splits when split_workers * split_blocks fits 32 bits: 64-bit divisions are slow)
__device__ __forceinline__ int split_begin(const GemmParams &p, int worker) {
    return static_cast<int>(static_cast<uint32_t>(worker) * static_cast<uint32_t>(p.split_blocks) /
                            static_cast<uint32_t>(p.split_workers));
}

// The units of one worker, in the order all three warp roles walk them.
struct UnitWalk {
    int next_whole, whole_tiles, stride, g, g_end, slot;
    __device__ UnitWalk(const GemmParams &p, int worker, int workers)
        : next_whole(worker), whole_tiles(p.m_tiles * p.n_tiles * p.batches + p.extra_tiles), stride(workers), g(0),
          g_end(0), slot(0) {
        if (p.split_workers > 0) {
            whole_tiles = 0;
            g = split_begin(p, worker);
            g_end = split_begin(p, worker + 1);
        }
    }
    __device__ bool next(const GemmParams &p, Unit &u) {
        if (g < g_end) {
            const int t = g / p.k_blocks;
            u.tile = t;
            u.kb0 = g - t * p.k_blocks;
            u.kb1 = min(p.k_blocks, u.kb0 + (g_end - g));
            u.slot = slot++;
            g += u.kb1 - u.kb0;
            return true;
        }
        if (next_whole < whole_tiles) {
            u.tile = next_whole;
            u.kb0 = 0;
            u.kb1 = p.k_blocks;
            u.slot = -1;
            next_whole += stride;
            return true;
        }
        return false;
    }
};

// The worker whose run holds entry g of the split sequence.
__device__ __forceinline__ int split_owner(const GemmParams &p, int g) {
    int w = static_cast<int>(static_cast<uint32_t>(g) * static_cast<uint32_t>(p.split_workers) /
                             static_cast<uint32_t>(p.split_blocks));
    while (w + 1 < p.split_workers && split_begin(p, w + 1) <= g) ++w;
    while (w > 0 && split_begin(p, w) > g) --w;
    return w;
}

__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int group_m, int &m_tile,
                                            int &n_tile) {
    const bool serpentine = group_m < 0;
    group_m = serpentine ? -group_m : group_m;
    const int tiles_per_group = group_m * n_tiles;
    const int group = tile / tiles_per_group;
    const int first_m = group * group_m;
    const int group_rows = min(m_tiles - first_m, group_m);
    const int in_group = tile - group * tiles_per_group;
    m_tile = first_m + in_group % group_rows;
    n_tile = in_group / group_rows;
    // Odd groups walk the columns backwards, so that a group starts on the B panels the previous one ended on
    // (a negative group_m asks for that).
    if (serpentine && (group & 1)) n_tile = n_tiles - 1 - n_tile;
}

// Row, first column and width of a tile.  MIXED kernels follow the numbering described at GemmParams::mixed_rows.
template <bool MIXED, int BN>
__device__ __forceinline__ TilePlace tile_place(const GemmParams &p, int tile) {
    int m_tile, n_tile;
    if constexpr (MIXED) {
        if (p.mixed_rows != 0) {
            const int plain_rows = p.m_tiles - p.mixed_rows;
            const int plain = plain_rows * p.n_tiles;
            if (tile < plain) {
                tile_coords(tile, plain_rows, p.n_tiles, p.group_m, m_tile, n_tile);
                return {p.mixed_rows + m_tile, n_tile * BN, BN};
            }
            tile -= plain;
            const int wide = p.mixed_rows * p.mixed_wide;
            if (tile < wide) {
                m_tile = tile / p.mixed_wide;
                return {m_tile, (tile - m_tile * p.mixed_wide) * BN, BN};
            }
            tile -= wide;
            m_tile = tile / p.mixed_narrow;
            return {m_tile, p.mixed_wide * BN + (tile - m_tile * p.mixed_narrow) * NARROW_BN, NARROW_BN};
        }
    }
    tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_tile, n_tile);
    return {m_tile, n_tile * BN, BN};
}

template <bool BF16>
struct Half;
template <>
struct Half<false> {
    using T = __half;
    using T2 = __half2;
    __device__ static T from_float(float x) { return __float2half_rn(x); }
    __device__ static T2 from_floats(float a, float b) { return __floats2half2_rn(a, b); }
    // beta*c + alpha*ab, rounded to the storage type after each operation.
    __device__ static T2 axpby(T2 beta, T2 c, T2 alpha, T2 ab) {
        return __hadd2_rn(__hmul2_rn(beta, c), __hmul2_rn(alpha, ab));
    }
    __device__ static T axpby1(T beta, T c, T alpha, T ab) { return __hadd_rn(__hmul_rn(beta, c), __hmul_rn(alpha, ab)); }
    __device__ static T2 dup(float x) { return __float2half2_rn(x); }
};
template <>
struct Half<true> {
    using T = __nv_bfloat16;
    using T2 = __nv_bfloat162;
    __device__ static T from_float(float x) { return __float2bfloat16_rn(x); }
    __device__ static T2 from_floats(float a, float b) { return __floats2bfloat162_rn(a, b); }
    __device__ static T2 axpby(T2 beta, T2 c, T2 alpha, T2 ab) {
        return __hadd2_rn(__hmul2_rn(beta, c), __hmul2_rn(alpha, ab));
    }
    __device__ static T axpby1(T beta, T c, T alpha, T ab) { return __hadd_rn(__hmul_rn(beta, c), __hmul_rn(alpha, ab)); }
    __device__ static T2 dup(float x) { return __float2bfloat162_rn(x); }
};

// B_MN: rhs is [K, N] with unit stride along N (row-major); otherwise rhs is
// addressed as [N, K] with unit stride along K (a transposed view).
// FP8: operands are 8-bit e5m2 (128 of them per 128-byte swizzle row, 32 per MMA: the same bytes per
// stage and per instruction as the 16-bit types), the output is fp16 (tests/test_matmul.py:60-90).
template <int CG, int BN, bool BF16, bool B_MN, bool ADDMM, bool FP8 = false, bool BATCHED = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_out,
                const __grid_constant__ GemmParams p) {
    using S = Shape<CG, BN>;
    constexpr int STAGES = S::STAGES;
    constexpr int BK_ELEMS = FP8 ? 2 * BK : BK;  // elements along K in one stage (128 bytes)
    static_assert(!FP8 || (!BF16 && !B_MN && !ADDMM), "fp8 operands: K-major B, plain matmul, fp16 output");
    static_assert(!BATCHED || (!ADDMM && !FP8), "batched: plain matmul (the batch dimension is on a row-major B)");
    constexpr bool MIXED = CG == 2 && BN == 256 && !FP8 && !BATCHED;  // may get 192-column tiles among its 256s
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    SharedControl *ctl = reinterpret_cast<SharedControl *>(smem + STAGES * S::STAGE_BYTES);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
    const int lane = threadIdx.x & 31;
    const WaitCtx wait_ctx{&ctl->abort_flag, p.status, KID_GEMM};
    const uint32_t cta_rank = CG == 1 ? 0u : cluster_cta_rank();  // position in the pair
    const bool leader = cta_rank == 0;
    const int worker = blockIdx.x / CG;        // which persistent tile stream this CTA (pair) walks
    const int workers = gridDim.x / CG;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->tmem_full[b], 1);
            mbar_init(&ctl->tmem_empty[b], 128 * CG);
        }
        ctl->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if (warp == 1) {
        tmem_alloc<CG>(&ctl->tmem_base, TMEM_COLS);
        tmem_relinquish<CG>();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    if constexpr (CG == 2) cluster_sync();  // both CTAs' barriers and TMEM exist before anything crosses the pair
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, ctl->tmem_base, 0);  // warp-uniform for the tcgen05 operands

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            UnitWalk walk(p, worker, workers);
            Unit u;
            const bool hints = !BATCHED && p.l2_hints != 0;
            // 1: A evict_last, B evict_first; 2: both evict_last; 3: A evict_first, B evict_last
            const uint64_t keep = p.l2_hints == 3 ? l2_policy_evict_first() : l2_policy_evict_last();
            const uint64_t stream_through = p.l2_hints == 1 ? l2_policy_evict_first() : l2_policy_evict_last();
            while (walk.next(p, u)) {
                int m_tile, batch = 0, tile_in_batch = u.tile;
                if constexpr (BATCHED) {
                    batch = u.tile / (p.m_tiles * p.n_tiles);
                    tile_in_batch = u.tile - batch * (p.m_tiles * p.n_tiles);
                }
                const TilePlace place = tile_place<MIXED, BN>(p, tile_in_batch);
                m_tile = place.m_tile;
                const int m0 = m_tile * S::TILE_M + static_cast<int>(cta_rank) * BM;
                // Each CTA of a pair holds half of the tile's columns.  A narrow tile's half (96 columns) is loaded
                // as the same two 64-column boxes; the MMA reads the first 96 of them.
                const int n0 = place.col0 + static_cast<int>(cta_rank) * (place.width / CG);
                for (int kb = u.kb0; kb < u.kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phase = (it / STAGES) & 1;
                    mbar_wait(&ctl->empty[s], phase ^ 1, wait_ctx, 0x100 | s);
                    uint8_t *a_dst = smem + s * S::STAGE_BYTES;
                    uint8_t *b_dst = a_dst + A_STAGE_BYTES;
                    if constexpr (CG == 1) {
                        mbar_expect_tx(&ctl->full[s], S::STAGE_BYTES);
                        if constexpr (BATCHED)
                            tma_load_3d(a_dst, &map_a, &ctl->full[s], kb * BK_ELEMS, m0, p.a_batched ? batch : 0);
                        else if (hints)
                            tma_load_2d_hint(a_dst, &map_a, &ctl->full[s], kb * BK_ELEMS, m0, keep);
                        else
                            tma_load_2d(a_dst, &map_a, &ctl->full[s], kb * BK_ELEMS, m0);
                        if constexpr (B_MN) {
#pragma unroll
                            for (int j = 0; j < S::BN_CTA / 64; ++j) {
                                if constexpr (BATCHED)
                                    tma_load_3d(b_dst + j * (BK * 128), &map_b, &ctl->full[s], n0 + j * 64, kb * BK, batch);
                                else if (hints)
                                    tma_load_2d_hint(b_dst + j * (BK * 128), &map_b, &ctl->full[s], n0 + j * 64, kb * BK,
                                                     stream_through);
                                else
                                    tma_load_2d(b_dst + j * (BK * 128), &map_b, &ctl->full[s], n0 + j * 64, kb * BK);
                            }
                        } else if (hints) {
                            tma_load_2d_hint(b_dst, &map_b, &ctl->full[s], kb * BK_ELEMS, n0, stream_through);
                        } else {
                            tma_load_2d(b_dst, &map_b, &ctl->full[s], kb * BK_ELEMS, n0);
                        }
                    } else {
                        // Both CTAs' bytes are credited to the even CTA's barrier, which alone expects them.
                        if (leader) mbar_expect_tx(&ctl->full[s], S::STAGE_BYTES * CG);
                        if constexpr (BATCHED)
                            tma_load_3d_pair(a_dst, &map_a, &ctl->full[s], kb * BK_ELEMS, m0, p.a_batched ? batch : 0);
                        else if (hints)
                            tma_load_2d_pair_hint(a_dst, &map_a, &ctl->full[s], kb * BK_ELEMS, m0, keep);
                        else
                            tma_load_2d_pair(a_dst, &map_a, &ctl->full[s], kb * BK_ELEMS, m0);
                        if constexpr (B_MN) {
#pragma unroll
                            for (int j = 0; j < S::BN_CTA / 64; ++j) {
                                if constexpr (BATCHED)
                                    tma_load_3d_pair(b_dst + j * (BK * 128), &map_b, &ctl->full[s], n0 + j * 64, kb * BK,
                                                     batch);
                                else if (hints)
                                    tma_load_2d_pair_hint(b_dst + j * (BK * 128), &map_b, &ctl->full[s], n0 + j * 64, kb * BK,
                                                          stream_through);
                                else
                                    tma_load_2d_pair(b_dst + j * (BK * 128), &map_b, &ctl->full[s], n0 + j * 64, kb * BK);
                            }
                        } else if (hints) {
                            tma_load_2d_pair_hint(b_dst, &map_b, &ctl->full[s], kb * BK_ELEMS, n0, stream_through);
                        } else {
                            tma_load_2d_pair(b_dst, &map_b, &ctl->full[s], kb * BK_ELEMS, n0);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer -------------------------------
        // The whole warp walks the loop so that addresses and descriptors are warp-uniform values (the
        // MMA instruction takes its operands from uniform registers); one elected lane issues.
        if (leader) {
            // (format code 1 is bf16 for kind::f16 and e5m2 for kind::f8f6f4)
            constexpr uint32_t idesc_wide = umma_instr_desc(BM * CG, BN, BF16 || FP8, false, B_MN);
            constexpr uint32_t idesc_narrow = umma_instr_desc(BM * CG, NARROW_BN, BF16 || FP8, false, B_MN);
            // The tensor core queues little work ahead of the instruction it is running, so whatever this
            // warp does between two MMAs must fit in one MMA's time (~130 cycles) or the pipe idles.  The
            // probe of the NEXT stage's barrier therefore sits in the middle of this stage's MMAs, and the
            // blocking wait is only taken when that probe said "not yet".
            const bool issuer = elect_one();
            const uint32_t smem_base = smem_u32(smem);
            uint32_t s = 0, phase = 0;
            bool ready = false;
            uint32_t acc_it = 0;
            UnitWalk walk(p, worker, workers);
            Unit u;
            for (; walk.next(p, u); ++acc_it) {
                const uint32_t buf = acc_it & 1;
                const uint32_t acc_phase = (acc_it >> 1) & 1;
                mbar_wait(&ctl->tmem_empty[buf], acc_phase ^ 1, wait_ctx, 0x200 | buf);
                tcgen05_fence_after_sync();
                const uint32_t tmem_acc = tmem_base + buf * BN;
                const int kb0 = u.kb0, kb1 = u.kb1;
                uint32_t idesc = idesc_wide;
                if constexpr (MIXED) {
                    if (tile_place<MIXED, BN>(p, u.tile).width != BN) idesc = idesc_narrow;
                }
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!ready) mbar_wait(&ctl->full[s], phase, wait_ctx, 0x300 | s);
                    tcgen05_fence_after_sync();
                    const uint32_t a_addr = smem_base + s * S::STAGE_BYTES;
                    const uint32_t b_addr = a_addr + A_STAGE_BYTES;
                    const uint32_t s_next = s + 1 == STAGES ? 0 : s + 1;
                    const uint32_t phase_next = s_next == 0 ? phase ^ 1 : phase;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t desc_a = umma_smem_desc(a_addr + kk * (UMMA_K * 2), 16, 1024);
                        const uint64_t desc_b =
                            umma_smem_desc(b_addr + kk * (B_MN ? UMMA_K * 128 : UMMA_K * 2), p.b_lbo, p.b_sbo);
                        if (issuer) {
                            const uint32_t accumulate = (kb != kb0 || kk != 0) ? 1u : 0u;
                            if constexpr (FP8) umma_ss_f8<CG>(tmem_acc, desc_a, desc_b, idesc, accumulate);
                            else umma_ss<CG>(tmem_acc, desc_a, desc_b, idesc, accumulate);
                        }
                        if (kk == BK / UMMA_K / 2 - 1)
                            ready = __all_sync(0xffffffffu, mbar_test_wait(&ctl->full[s_next], phase_next));
                    }
                    // frees the stage (in both CTAs of a pair) once these MMAs have read it
                    if (issuer) {
                        if constexpr (CG == 1) umma_commit<1>(&ctl->empty[s]);
                        else umma_commit_pair_multicast(&ctl->empty[s], 0x3);
                    }
                    s = s_next;
                    phase = phase_next;
                }
                // accumulator complete (each CTA of a pair drains its own rows)
                if (issuer) {
                    if constexpr (CG == 1) umma_commit<1>(&ctl->tmem_full[buf]);
                    else umma_commit_pair_multicast(&ctl->tmem_full[buf], 0x3);
                }
                __syncwarp();
            }
        }
    } else {
        // -------------------------------- epilogue --------------------------------
        using H = Half<BF16>;
        using T = typename H::T;
        using T2 = typename H::T2;
        const int quadrant = warp & 3;            // TMEM lanes this warp may read
        const int row_in_tile = static_cast<int>(cta_rank) * BM + quadrant * 32 + lane;
        const T2 beta2 = H::dup(p.beta), alpha2 = H::dup(p.alpha);
        const T beta1 = H::from_float(p.beta), alpha1 = H::from_float(p.alpha);
        T *const out_base = static_cast<T *>(p.out);
        const T *c_in = static_cast<const T *>(p.c_in);
        const bool out_vec = p.out_stride1 == 1 && (p.out_stride0 % 8) == 0 &&
                             (reinterpret_cast<uintptr_t>(out_base) & 15) == 0;
        const bool c_vec = !ADDMM || (p.c_stride1 == 1 && (p.c_stride0 % 8) == 0 &&
                                      (reinterpret_cast<uintptr_t>(c_in) & 15) == 0);
        uint8_t *stage = reinterpret_cast<uint8_t *>(ctl) + STAGE_OFFSET + (warp - 2) * (32 * STAGE_PITCH);
        // Batched launches hand their tiles to TMA instead: 32 rows x 128 bytes per warp in the 128-byte swizzle
        // (1024-byte aligned, in place of the staging area), one bulk tensor store per 64-column step, two boxes
        // per warp so that a step does not wait for the previous step's box to be read out.
        uint8_t *const boxes = reinterpret_cast<uint8_t *>(ctl) + 1024 + (warp - 2) * (2 * 32 * 128);
        uint32_t box_it = 0;
        uint32_t acc_it = 0;
        UnitWalk walk(p, worker, workers);
        Unit u;
        // A partial accumulator is stored as float4s: element (row r of this CTA, columns 4q..4q+3) at
        // float4 index q * 128 + r, so that a warp's 32 rows make one 512-byte run.
        const int row_in_cta = quadrant * 32 + lane;
        constexpr int SLOT_FLOATS = BM * BN;
        for (; walk.next(p, u); ++acc_it) {
            int m_tile, batch = 0, tile_in_batch = u.tile;
            if constexpr (BATCHED) {
                batch = u.tile / (p.m_tiles * p.n_tiles);
                tile_in_batch = u.tile - batch * (p.m_tiles * p.n_tiles);
            }
            const TilePlace place = tile_place<MIXED, BN>(p, tile_in_batch);
            m_tile = place.m_tile;
            T *out = out_base + batch * p.out_batch_stride;  // (the host keeps the stride a multiple of 8 elements)
            const int64_t row = static_cast<int64_t>(m_tile) * S::TILE_M + row_in_tile;
            const int n0 = place.col0;
            const uint32_t buf = acc_it & 1;
            const uint32_t acc_phase = (acc_it >> 1) & 1;
            mbar_wait(&ctl->tmem_full[buf], acc_phase, wait_ctx, 0x400 | buf);
            tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quadrant * 32) << 16);
            if (u.slot >= 0) {
                // Partial tile: the accumulator goes to this unit's slot as it is; the second kernel does the rest.
                float4 *mine = reinterpret_cast<float4 *>(
                    p.split_partials + (static_cast<size_t>(worker * 2 + u.slot) * CG + cta_rank) * SLOT_FLOATS);
#pragma unroll 1
                for (int chunk = 0; chunk < BN / 32; ++chunk) {
                    uint32_t part[32];
                    tmem_ld_32x32(taddr + chunk * 32, part);
                    tmem_wait_ld();
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        mine[(chunk * 8 + q) * BM + row_in_cta] =
                            make_float4(__uint_as_float(part[4 * q]), __uint_as_float(part[4 * q + 1]),
                                        __uint_as_float(part[4 * q + 2]), __uint_as_float(part[4 * q + 3]));
                }
                tcgen05_fence_before_sync();
                if (CG == 1 || leader) mbar_arrive(&ctl->tmem_empty[buf]);
                else mbar_arrive_cluster(&ctl->tmem_empty[buf], 0);
                continue;
            }
#pragma unroll 1
            for (int step = 0; step < place.width / 64; ++step) {
                uint32_t acc[2][32];
                tmem_ld_32x32(taddr + step * 64, acc[0]);
                tmem_ld_32x32(taddr + step * 64 + 32, acc[1]);
                tmem_wait_ld();
                const int col0 = n0 + step * 64;
                if constexpr (BATCHED) {
                    // A batched launch has short reductions and lives in its epilogue.  Every thread rounds its row's
                    // 64 columns and writes them as eight swizzled 16-byte chunks; one lane then issues the store of
                    // the warp's 32 x 64 box, which clips rows and columns beyond the matrix by itself.
                    if (col0 >= p.n || row - lane >= p.m) continue;
                    uint8_t *box = boxes + (box_it++ & 1) * (32 * 128);
                    if (lane == 0) tma_store_wait_read<1>();  // the box of two steps ago has been read out of shared memory
                    __syncwarp();
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        uint4 packed;
                        T2 *h = reinterpret_cast<T2 *>(&packed);
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            h[j] = H::from_floats(__uint_as_float(acc[v >> 2][(v & 3) * 8 + 2 * j]),
                                                  __uint_as_float(acc[v >> 2][(v & 3) * 8 + 2 * j + 1]));
                        *reinterpret_cast<uint4 *>(box + lane * 128 + ((v ^ (lane & 7)) << 4)) = packed;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(&map_out, box, col0, static_cast<int>(row - lane), batch);
                        tma_store_commit();
                    }
                    continue;
                }
                if (out_vec && c_vec && col0 + 64 <= p.n && p.extra_dests == 0 && !p.through_switch) {
                    // Local output only: every thread stores its own row's 64 columns, 16 bytes at a time
                    // (full 32-byte sectors; measured a few percent faster than staging for HBM).
                    if (row < p.m) {
                        T *out_row = out + row * p.out_stride0 + col0;
                        const T *c_row = ADDMM ? c_in + row * p.c_stride0 + col0 : nullptr;
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            uint4 packed;
                            T2 *h = reinterpret_cast<T2 *>(&packed);
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                h[j] = H::from_floats(__uint_as_float(acc[v >> 2][(v & 3) * 8 + 2 * j]),
                                                      __uint_as_float(acc[v >> 2][(v & 3) * 8 + 2 * j + 1]));
                            if constexpr (ADDMM) {
                                const uint4 cv = *reinterpret_cast<const uint4 *>(c_row + v * 8);
                                const T2 *c2 = reinterpret_cast<const T2 *>(&cv);
#pragma unroll
                                for (int j = 0; j < 4; ++j) h[j] = H::axpby(beta2, c2[j], alpha2, h[j]);
                            }
                            *reinterpret_cast<uint4 *>(out_row + v * 8) = packed;
                        }
                    }
                } else if (out_vec && c_vec && col0 + 64 <= p.n) {
                    // Peer destinations (warp-uniform): every thread finishes its row's 64 columns, the warp
                    // transposes them through shared memory and stores 128-byte row segments, four rows per
                    // instruction, to every destination: NVLink wants long contiguous writes.
                    const T *c_row = ADDMM && row < p.m ? c_in + row * p.c_stride0 + col0 : nullptr;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        uint4 packed;
                        T2 *h = reinterpret_cast<T2 *>(&packed);
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            h[j] = H::from_floats(__uint_as_float(acc[v >> 2][(v & 3) * 8 + 2 * j]),
                                                  __uint_as_float(acc[v >> 2][(v & 3) * 8 + 2 * j + 1]));
                        if constexpr (ADDMM) {
                            if (c_row != nullptr) {
                                const uint4 cv = *reinterpret_cast<const uint4 *>(c_row + v * 8);
                                const T2 *c2 = reinterpret_cast<const T2 *>(&cv);
#pragma unroll
                                for (int j = 0; j < 4; ++j) h[j] = H::axpby(beta2, c2[j], alpha2, h[j]);
                            }
                        }
                        *reinterpret_cast<uint4 *>(stage + lane * STAGE_PITCH + v * 16) = packed;
                    }
                    __syncwarp();
                    const int64_t warp_row0 = row - lane;  // first of this warp's 32 rows
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = i * 4 + (lane >> 3), seg = lane & 7;
                        const uint4 val = *reinterpret_cast<const uint4 *>(stage + rr * STAGE_PITCH + seg * 16);
                        const int64_t grow = warp_row0 + rr;
                        if (grow < p.m) {
                            const int64_t off = grow * p.out_stride0 + col0 + seg * 8;
                            if (p.through_switch) {
                                multimem_st_16(out + off, val);
                            } else {
                                *reinterpret_cast<uint4 *>(out + off) = val;
                                for (int d = 0; d < p.extra_dests; ++d)
                                    *reinterpret_cast<uint4 *>(static_cast<T *>(p.more_out[d]) + off) = val;
                            }
                        }
                    }
                    __syncwarp();
                } else if (row < p.m && col0 < p.n) {
                    // Ragged edge or operands without 16-byte rows: element by element.
                    T *out_row = out + row * p.out_stride0;
                    const T *c_row = ADDMM ? c_in + row * p.c_stride0 : nullptr;
#pragma unroll
                    for (int j = 0; j < 64; ++j) {
                        const int col = col0 + j;
                        if (col < p.n) {
                            T value = H::from_float(__uint_as_float(acc[j >> 5][j & 31]));
                            if constexpr (ADDMM) value = H::axpby1(beta1, c_row[col * p.c_stride1], alpha1, value);
                            out_row[col * p.out_stride1] = value;
                            for (int d = 0; d < p.extra_dests; ++d)
                                static_cast<T *>(p.more_out[d])[row * p.out_stride0 + col * p.out_stride1] = value;
                        }
                    }
                }
            }
            tcgen05_fence_before_sync();
            // the accumulator buffer is released on the MMA issuer's (even CTA's) barrier
            if (CG == 1 || leader) mbar_arrive(&ctl->tmem_empty[buf]);
            else mbar_arrive_cluster(&ctl->tmem_empty[buf], 0);
        }
        if constexpr (BATCHED) {
            if (lane == 0) tma_store_wait<0>();  // this thread's bulk stores are complete before the CTA goes away
        }
    }

    __syncwarp();
    tcgen05_fence_before_sync();
    __syncthreads();
    if constexpr (CG == 2) cluster_sync();  // the partner may still be reading this CTA's tiles or signalling it
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc<CG>(tmem_base, TMEM_COLS);
    }
}

// Plain tiled kernel for operands no TMA descriptor can address (no unit-stride
// dimension, rows not 16-byte aligned, K == 0).  Same arithmetic: fp32
// accumulation over K, one rounding, then the storage-type epilogue.
template <bool BF16, bool ADDMM>
__global__ void __launch_bounds__(256)
    gemm_plain_kernel(const void *a_, const void *b_, const void *c_, void *out_, int m, int n, int k, int64_t as0,
                      int64_t as1, int64_t bs0, int64_t bs1, int64_t cs0, int64_t cs1, int64_t os0, int64_t os1,
                      float beta, float alpha) {
    using H = Half<BF16>;
    using T = typename H::T;
    const T *a = static_cast<const T *>(a_);
    const T *b = static_cast<const T *>(b_);
    const T *c = static_cast<const T *>(c_);
    T *out = static_cast<T *>(out_);
    __shared__ float sa[16][17];
    __shared__ float sb[16][17];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int64_t row = static_cast<int64_t>(blockIdx.y) * 16 + ty;
    const int64_t col = static_cast<int64_t>(blockIdx.x) * 16 + tx;
    float acc = 0.f;
    for (int k0 = 0; k0 < k; k0 += 16) {
        const int ka = k0 + tx, kb = k0 + ty;
        sa[ty][tx] = (row < m && ka < k) ? static_cast<float>(a[row * as0 + ka * as1]) : 0.f;
        sb[ty][tx] = (kb < k && col < n) ? static_cast<float>(b[kb * bs0 + col * bs1]) : 0.f;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) acc = fmaf(sa[ty][kk], sb[kk][tx], acc);
        __syncthreads();
    }
    if (row < m && col < n) {
        T value = H::from_float(acc);
        if constexpr (ADDMM)
            value = H::axpby1(H::from_float(beta), c[row * cs0 + col * cs1], H::from_float(alpha), value);
        out[row * os0 + col * os1] = value;
    }
}

// The same for 8-bit e5m2 operands (an e5m2 value is the high byte of the fp16 with the same value),
// fp16 output.
__global__ void __launch_bounds__(256)
    gemm_plain_fp8_kernel(const uint8_t *a, const uint8_t *b, __half *out, int m, int n, int k, int64_t as0, int64_t as1,
                          int64_t bs0, int64_t bs1, int64_t os0, int64_t os1) {
    __shared__ float sa[16][17];
    __shared__ float sb[16][17];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int64_t row = static_cast<int64_t>(blockIdx.y) * 16 + ty;
    const int64_t col = static_cast<int64_t>(blockIdx.x) * 16 + tx;
    const auto decode = [](uint8_t v) { return __half2float(__ushort_as_half(static_cast<unsigned short>(v) << 8)); };
    float acc = 0.f;
    for (int k0 = 0; k0 < k; k0 += 16) {
        const int ka = k0 + tx, kb = k0 + ty;
        sa[ty][tx] = (row < m && ka < k) ? decode(a[row * as0 + ka * as1]) : 0.f;
        sb[ty][tx] = (kb < k && col < n) ? decode(b[kb * bs0 + col * bs1]) : 0.f;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) acc = fmaf(sa[ty][kk], sb[kk][tx], acc);
        __syncthreads();
    }
    if (row < m && col < n) out[row * os0 + col * os1] = __float2half_rn(acc);
}

struct Operand2D {
    const void *data;
    int64_t rows, cols;
    int64_t stride0, stride1;
};

// Extra destinations of the epilogue (already offset to this rank's column slab).
struct PeerOutputs {
    int count;
    void *data[MAX_PEERS];
    bool through_switch = false;  // the output pointer is a multicast address (count is 0 then)
};

bool tma_addressable_k_major(const Operand2D &t) {
    // unit stride along cols, rows 16-byte aligned
    return t.stride1 == 1 && (t.stride0 % 8) == 0 && t.stride0 >= t.cols && aligned16(t.data);
}

template <bool BF16, bool ADDMM>
int launch_plain(cudaStream_t stream, const Operand2D &a, const Operand2D &b, const NineToothedTensor *c,
                 const NineToothedTensor &out, float beta, float alpha) {
    const int m = static_cast<int>(a.rows), n = static_cast<int>(b.cols), k = static_cast<int>(a.cols);
    dim3 grid((n + 15) / 16, (m + 15) / 16);
    if (grid.y > 65535) return fail(NINETOOTHED_B200_ERR_SHAPE, "matmul: M=%d too large for the plain kernel", m);
    gemm_plain_kernel<BF16, ADDMM><<<grid, 256, 0, stream>>>(
        a.data, b.data, c ? c->data : nullptr, out.data, m, n, k, a.stride0, a.stride1, b.stride0, b.stride1,
        c ? c->strides[0] : 0, c ? c->strides[1] : 0, out.strides[0], out.strides[1], beta, alpha);
    NT_CUDA_CHECK(cudaGetLastError());
    return 0;
}

// How many CTA pairs can be resident at once (pairs need two SMs of one cluster slot).
template <typename Kernel>
int max_active_pairs(Kernel kernel, const DeviceState &dev, size_t smem) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(dev.sm_count / 2 * 2));
    config.blockDim = dim3(NUM_THREADS);
    config.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess || clusters <= 0) {
        cudaGetLastError();
        return 0;
    }
    return clusters;
}

// Second kernel of a split launch: adds up the partial accumulators of every tile, in the order of
// their k-ranges (so the sum does not depend on timing), and applies the epilogue.  One block per
// (tile, CTA of the pair, 16 columns); thread (q, r) owns row r of the CTA's 128 and columns 4q..4q+3 of the
// 16, which is how the partials are laid out (a warp reads 512 contiguous bytes).  The kernel is all memory
// latency: a tile's partials are requested eight at a time before any is used, and nothing in a block waits
// for another thread.
constexpr int REDUCE_COLS = 16;
constexpr int REDUCE_THREADS = BM * REDUCE_COLS / 4;
constexpr int MAX_SPLIT_OWNERS = 16;  // partials per tile

template <bool BF16, bool ADDMM>
__global__ void __launch_bounds__(REDUCE_THREADS, 2)
    split_reduce_kernel(const __grid_constant__ GemmParams p, const int cg, const int bn) {
    using H = Half<BF16>;
    using T = typename H::T;
    using T2 = typename H::T2;
    const int CHUNKS = bn / REDUCE_COLS;
    const int SLOT_FLOATS = BM * bn;
    const int chunk = blockIdx.x % CHUNKS;
    const int cta = (blockIdx.x / CHUNKS) % cg;
    const int tile = blockIdx.x / (CHUNKS * cg);
    int m_tile, n_tile;
    tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_tile, n_tile);
    const int q = threadIdx.x / BM, r = threadIdx.x % BM;
    const int64_t row = static_cast<int64_t>(m_tile) * (BM * cg) + cta * BM + r;
    const int col = n_tile * bn + chunk * REDUCE_COLS + 4 * q;
    if (col >= p.n || row >= p.m) return;
    // which workers hold partials of this tile
    const int g_first = tile * p.k_blocks;
    const int first_owner = split_owner(p, g_first);
    const int owners = split_owner(p, g_first + p.k_blocks - 1) - first_owner + 1;
    // the tile is a worker's second unit exactly when its run began in an earlier tile: that can only be the
    // first owner, every later one starts inside this tile
    const int first_slot = split_begin(p, first_owner) < g_first ? 1 : 0;
    const size_t index = static_cast<size_t>(chunk * (REDUCE_COLS / 4) + q) * BM + r;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int batch = 0; batch < MAX_SPLIT_OWNERS; batch += 8) {
        if (batch >= owners) break;
        float4 part[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int o = batch + i;
            if (o < owners) {
                const int slot = o == 0 ? first_slot : 0;
                part[i] = __ldcg(reinterpret_cast<const float4 *>(
                                     p.split_partials +
                                     (static_cast<size_t>((first_owner + o) * 2 + slot) * cg + cta) * SLOT_FLOATS) +
                                 index);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (batch + i < owners) {
                if (batch + i == 0) sum = part[0];  // (not 0 + x: keeps a -0 result and the plain order of additions)
                else sum.x += part[i].x, sum.y += part[i].y, sum.z += part[i].z, sum.w += part[i].w;
            }
        }
    }
    const float acc[4] = {sum.x, sum.y, sum.z, sum.w};
    T *out = static_cast<T *>(p.out);
    const T *c_in = static_cast<const T *>(p.c_in);
    const bool out_vec = p.out_stride1 == 1 && (p.out_stride0 % 4) == 0 && (reinterpret_cast<uintptr_t>(out) & 7) == 0;
    const bool c_vec = !ADDMM || (p.c_stride1 == 1 && (p.c_stride0 % 4) == 0 && (reinterpret_cast<uintptr_t>(c_in) & 7) == 0);
    if (out_vec && c_vec && col + 4 <= p.n) {
        uint2 packed;
        T2 *h = reinterpret_cast<T2 *>(&packed);
        h[0] = H::from_floats(acc[0], acc[1]);
        h[1] = H::from_floats(acc[2], acc[3]);
        if constexpr (ADDMM) {
            const T2 beta2 = H::dup(p.beta), alpha2 = H::dup(p.alpha);
            const uint2 cv = *reinterpret_cast<const uint2 *>(c_in + row * p.c_stride0 + col);
            const T2 *c2 = reinterpret_cast<const T2 *>(&cv);
            h[0] = H::axpby(beta2, c2[0], alpha2, h[0]);
            h[1] = H::axpby(beta2, c2[1], alpha2, h[1]);
        }
        *reinterpret_cast<uint2 *>(out + row * p.out_stride0 + col) = packed;
    } else {
        const T beta1 = H::from_float(p.beta), alpha1 = H::from_float(p.alpha);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (col + j < p.n) {
                T value = H::from_float(acc[j]);
                if constexpr (ADDMM)
                    value = H::axpby1(beta1, c_in[row * p.c_stride0 + (col + j) * p.c_stride1], alpha1, value);
                out[row * p.out_stride0 + (col + j) * p.out_stride1] = value;
            }
        }
    }
}

// Scratch for split launches: the partial accumulators, two slots per CTA that can be resident, one
// array per (device, stream) so that launches on different streams do not share it.  Allocated at the
// first launch that wants it; a launch that cannot have one (a stream that is being captured into a
// graph and has none yet, more streams than MAX_SPLIT_STREAMS, no memory) runs without the split.
struct SplitScratch {
    int device;
    cudaStream_t stream;
    float *partials;
};
constexpr int MAX_SPLIT_STREAMS = 8;

// `allocate`: whether a missing array may be allocated now (a launch may; a launch whose stream handle is
// cudaStreamPerThread never gets one, because that handle names a different stream in every host thread and
// the threads would share the partials).
float *split_scratch(const DeviceState &dev, cudaStream_t stream, bool allocate = true) {
    static std::mutex mutex;
    static std::vector<SplitScratch> entries;
    if (stream == cudaStreamPerThread) return nullptr;
    std::lock_guard<std::mutex> lock(mutex);
    int on_device = 0;
    for (const SplitScratch &e : entries) {
        if (e.device != dev.device) continue;
        ++on_device;
        if (e.stream == stream) return e.partials;
    }
    if (!allocate || on_device >= MAX_SPLIT_STREAMS) return nullptr;
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess || capture != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return nullptr;
    }
    void *memory = nullptr;
    if (cudaMalloc(&memory, static_cast<size_t>(2) * dev.sm_count * BM * MAX_BN * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    entries.push_back(SplitScratch{dev.device, stream, static_cast<float *>(memory)});
    return static_cast<float *>(memory);
}

// NINETOOTHED_B200_GEMM_SPLIT_ALLOC=0: launches never allocate; only streams prepared with
// ninetoothed_b200_reserve_split_scratch split.
bool launches_may_allocate() {
    static const bool allowed = [] {
        const char *env = std::getenv("NINETOOTHED_B200_GEMM_SPLIT_ALLOC");
        return !(env && std::atoi(env) == 0);
    }();
    return allowed;
}

constexpr int SPLIT_FIXUP_BLOCKS = 40;  // the partials' round trip and the second launch cost about this many k-blocks

// How many workers a launch of `tiles` tiles with `k_blocks` K-blocks each is split over (see GemmParams), or 0
// when it is not split.  `workers` is the number of CTAs (or pairs) the device can hold at once.
int split_workers_for(int64_t tiles, int workers, int k_blocks, bool allowed) {
    // NINETOOTHED_B200_GEMM_SPLIT: 0 never splits; a value above 1 replaces SPLIT_FIXUP_BLOCKS.
    static const int mode = [] {
        const char *env = std::getenv("NINETOOTHED_B200_GEMM_SPLIT");
        return env ? std::atoi(env) : 1;
    }();
    constexpr int MIN_RUN = 4;  // k-blocks: shorter runs are all pipeline fill
    if (!allowed || mode == 0 || tiles >= workers || k_blocks < 4 * MIN_RUN) return 0;
    const int64_t blocks = tiles * k_blocks;
    if (blocks * workers >= (int64_t{1} << 32)) return 0;
    const int split_workers = static_cast<int>(
        std::min<int64_t>(std::min<int64_t>(workers, blocks / MIN_RUN), tiles * (MAX_SPLIT_OWNERS - 1)));
    // k-blocks of MMA time the split takes off the critical path
    const double saved_blocks = k_blocks * (1.0 - static_cast<double>(tiles) / split_workers);
    if (saved_blocks < (mode > 1 ? mode : SPLIT_FIXUP_BLOCKS)) return 0;
    return split_workers;
}

// Fills the split fields of the parameters; without scratch memory the launch is not split.
void plan_split(const DeviceState &dev, cudaStream_t stream, int workers, bool allowed, GemmParams &p) {
    const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles;
    p.split_workers = 0;
    p.split_blocks = 0;
    p.split_partials = nullptr;
    const int split_workers = split_workers_for(tiles, workers, p.k_blocks, allowed);
    if (split_workers == 0) return;
    float *partials = split_scratch(dev, stream, launches_may_allocate());
    if (partials == nullptr) return;
    p.split_blocks = static_cast<int>(tiles * p.k_blocks);
    p.split_workers = split_workers;
    p.split_partials = partials;
}

// Mixed tile widths for a launch of CTA pairs on 256-column tiles (see GemmParams::mixed_rows): which tile-rows
// trade 256-column tiles for 192-column ones so that the waves fill.  A pair walks the tile numbers with a stride
// of `workers`, wide tiles first, so the longest pair is pair 0: ceil(wide / workers) wide tiles and the rest of its
// ceil(tiles / workers) narrow.  Cycles per K-block: 560 for a wide tile (four N=256 MMAs plus the pipeline's slack),
// 445 for a narrow one (three quarters of the MMA time, the same operand bytes).
std::atomic<long long> mixed_width_launches{0};

struct MixedPlan {
    int rows = 0, swaps = 0;       // tile-rows with swaps, swaps in each (3 wide -> 4 narrow)
    int64_t cycles = 0;            // per K-block step of the longest pair, summed over its tiles
};
constexpr int WIDE_CYCLES = 560, NARROW_CYCLES = 445;

// The narrow tiles of a tile-row run after its wide ones, one or more waves later, and read the row's A panel
// again; beyond this many bytes of such panels the second read comes from HBM instead of L2 and the trade stops
// paying (measured: 8192 x 1024 x 8192 with 75 MB of them lost 3 %, shapes below 40 MB gained 3 to 8 %).
constexpr int64_t MIXED_PANEL_BYTES = int64_t{64} << 20;

MixedPlan plan_mixed(int64_t row_tiles, int64_t col_tiles, int workers, int64_t panel_bytes) {
    // NINETOOTHED_B200_GEMM_MIXED: 0 never mixes, "force" swaps wherever it can (for tests); read at every launch
    const char *env = std::getenv("NINETOOTHED_B200_GEMM_MIXED");
    MixedPlan best;
    const int64_t tiles = row_tiles * col_tiles;
    best.cycles = (tiles + workers - 1) / workers * WIDE_CYCLES;
    const int64_t max_swaps = col_tiles / 3;
    if ((env && env[0] == '0') || max_swaps == 0 || workers <= 0 || row_tiles > 0x7fff || col_tiles > 0x7fff) return best;
    const bool force = env && env[0] == 'f';
    const int64_t plain_cycles = best.cycles;
    for (int64_t swaps = 1; swaps <= max_swaps; ++swaps) {
        for (int64_t rows = 1; rows <= row_tiles; ++rows) {
            if (!force && rows * panel_bytes > MIXED_PANEL_BYTES) break;
            const int64_t wide = tiles - 3 * swaps * rows, all = tiles + swaps * rows;
            const int64_t wide_0 = (wide + workers - 1) / workers, all_0 = (all + workers - 1) / workers;
            const int64_t cycles = wide_0 * WIDE_CYCLES + (all_0 - wide_0) * NARROW_CYCLES;
            if (force ? (swaps == max_swaps && rows == row_tiles) : cycles < best.cycles) {
                best.rows = static_cast<int>(rows);
                best.swaps = static_cast<int>(swaps);
                best.cycles = cycles;
            }
        }
    }
    // not worth a different tile order for less than 3 %
    if (!force && best.cycles * 100 > plain_cycles * 97) {
        best = MixedPlan{};
        best.cycles = plain_cycles;
    }
    return best;
}

// A batch of problems that share A: problem i reads B at b.data + i * b_stride and writes out.data + i * out_stride
// (elements; both multiples of 8 so that every problem keeps the 16-byte alignment of the first).
struct Batch {
    int count;
    int64_t b_stride, out_stride;
    int64_t a_stride = 0;  // 0: every problem reads the same A
};

template <int CG, int BN, bool BF16, bool B_MN, bool ADDMM, bool FP8 = false, bool BATCHED = false>
int launch_tcgen05(cudaStream_t stream, const DeviceState &dev, int dtype, const Operand2D &a, const Operand2D &b,
                   const NineToothedTensor *c, const NineToothedTensor &out, float beta, float alpha, int pairs,
                   const PeerOutputs *peers, const Batch *batch = nullptr) {
    using S = Shape<CG, BN>;
    constexpr int ELEM = FP8 ? 1 : 2;              // bytes per operand element
    constexpr uint32_t BK_ELEMS = FP8 ? 2 * BK : BK;  // operand elements in a 128-byte swizzle row
    const int map_dtype = FP8 ? NINETOOTHED_UINT8 : dtype;  // (TMA moves e5m2 as bytes)
    const int64_t m = a.rows, k = a.cols, n = b.cols;
    CUtensorMap map_a, map_b;
    if constexpr (BATCHED) {
        // rows past M read zeros through the bounds of the second dimension instead of the next problem's rows
        const bool a_batched = batch->a_stride != 0;
        const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m),
                                  static_cast<uint64_t>(a_batched ? batch->count : 1)};
        const uint64_t strides[2] = {static_cast<uint64_t>(a.stride0) * ELEM,
                                     static_cast<uint64_t>(a_batched ? batch->a_stride : a.stride0 * m) * ELEM};
        const uint32_t box[3] = {BK_ELEMS, BM, 1};
        if (int rc = make_tensor_map(dev, &map_a, map_dtype, 3, a.data, dims, strides, box, true)) return rc;
    } else {
        const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m)};
        const uint64_t strides[1] = {static_cast<uint64_t>(a.stride0) * ELEM};
        const uint32_t box[2] = {BK_ELEMS, BM};
        if (int rc = make_tensor_map(dev, &map_a, map_dtype, 2, a.data, dims, strides, box, true)) return rc;
    }
    if (B_MN && BATCHED) {
        const uint64_t dims[3] = {static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(batch->count)};
        const uint64_t strides[2] = {static_cast<uint64_t>(b.stride0) * 2, static_cast<uint64_t>(batch->b_stride) * 2};
        const uint32_t box[3] = {64, BK, 1};
        if (int rc = make_tensor_map(dev, &map_b, dtype, 3, b.data, dims, strides, box, true)) return rc;
    } else if (B_MN) {
        const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(k)};
        const uint64_t strides[1] = {static_cast<uint64_t>(b.stride0) * 2};
        const uint32_t box[2] = {64, BK};
        if (int rc = make_tensor_map(dev, &map_b, dtype, 2, b.data, dims, strides, box, true)) return rc;
    } else {
        const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n)};
        const uint64_t strides[1] = {static_cast<uint64_t>(b.stride1) * ELEM};
        const uint32_t box[2] = {BK_ELEMS, static_cast<uint32_t>(S::BN_CTA)};
        if (int rc = make_tensor_map(dev, &map_b, map_dtype, 2, b.data, dims, strides, box, true)) return rc;
    }
    GemmParams p;
    p.m = static_cast<int>(m);
    p.n = static_cast<int>(n);
    p.k = static_cast<int>(k);
    p.m_tiles = static_cast<int>((m + S::TILE_M - 1) / S::TILE_M);
    p.n_tiles = static_cast<int>((n + BN - 1) / BN);
    p.k_blocks = static_cast<int>((k + BK_ELEMS - 1) / BK_ELEMS);
    p.c_in = c ? c->data : nullptr;
    p.c_stride0 = c ? c->strides[0] : 0;
    p.c_stride1 = c ? c->strides[1] : 0;
    p.out = out.data;
    p.extra_dests = peers ? peers->count : 0;
    p.through_switch = peers && peers->through_switch ? 1 : 0;
    for (int d = 0; d < p.extra_dests; ++d) p.more_out[d] = peers->data[d];
    p.out_stride0 = out.strides[0];
    p.out_stride1 = out.strides[1];
    p.beta = beta;
    p.alpha = alpha;
    // MN-major B: 64-column blocks are one TMA box (BK rows of 128 B) apart, 8-row
    // groups 1024 B apart.  K-major B: 8-row groups 1024 B apart, no leading offset.
    p.b_lbo = B_MN ? BK * 128 : 16;
    p.b_sbo = 1024;
    p.status = dev.status;
    // NINETOOTHED_B200_GEMM_GROUP_M: rows of 128 per raster group (a power of two between 2 and 128; default 16)
    static const int group_rows = [] {
        const char *env = std::getenv("NINETOOTHED_B200_GEMM_GROUP_M");
        const int value = env ? std::atoi(env) : GROUP_M;
        return (value >= 2 && value <= 128 && (value & (value - 1)) == 0) ? value : GROUP_M;
    }();
    p.group_m = std::max(1, group_rows / CG);
    // NINETOOTHED_B200_GEMM_SERPENTINE=0: every raster group walks the columns in the same direction
    static const bool serpentine = [] {
        const char *env = std::getenv("NINETOOTHED_B200_GEMM_SERPENTINE");
        return !(env && env[0] == '0');
    }();
    if (serpentine) p.group_m = -p.group_m;
    static const int l2_hints = [] {
        const char *env = std::getenv("NINETOOTHED_B200_GEMM_L2_HINTS");
        return env ? std::atoi(env) : 0;
    }();
    p.l2_hints = l2_hints;
    p.batches = BATCHED ? batch->count : 1;
    p.a_batched = BATCHED && batch->a_stride != 0 ? 1 : 0;
    p.out_batch_stride = BATCHED ? batch->out_stride : 0;

    auto kernel = gemm_kernel<CG, BN, BF16, B_MN, ADDMM, FP8, BATCHED>;
    constexpr size_t smem = BATCHED ? smem_bytes_batched<CG, BN>() : smem_bytes<CG, BN>();
    static_assert(smem <= 227 * 1024, "shared memory per CTA");
    static thread_local int configured_device = -1;  // per device: opt in to the large dynamic shared memory
    if (configured_device != dev.device) {
        NT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured_device = dev.device;
    }
    int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles * p.batches;
    cudaLaunchConfig_t config = {};
    config.blockDim = dim3(NUM_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    const int resident = CG == 1 ? dev.sm_count : pairs;
    plan_split(dev, stream, resident, !FP8 && !BATCHED && p.extra_dests == 0 && !p.through_switch, p);
    p.mixed_rows = p.mixed_wide = p.mixed_narrow = p.extra_tiles = 0;
    if constexpr (CG == 2 && BN == 256 && !FP8 && !BATCHED) {
        if (p.split_workers == 0 && tiles > resident) {
            const MixedPlan mixed = plan_mixed(p.m_tiles, p.n_tiles, resident, int64_t{S::TILE_M} * k * ELEM);
            if (mixed.rows > 0) {
                mixed_width_launches.fetch_add(1, std::memory_order_relaxed);
                p.mixed_rows = mixed.rows;
                p.mixed_wide = p.n_tiles - 3 * mixed.swaps;
                p.mixed_narrow = 4 * mixed.swaps;
                p.extra_tiles = mixed.rows * mixed.swaps;
                tiles += p.extra_tiles;
            }
        }
    }
    const int workers = p.split_workers > 0 ? p.split_workers : static_cast<int>(std::min<int64_t>(tiles, resident));
    if (CG == 1) {
        config.gridDim = dim3(static_cast<unsigned>(workers));
        config.numAttrs = 0;
    } else {
        config.gridDim = dim3(static_cast<unsigned>(2 * workers));
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        config.attrs = attr;
        config.numAttrs = 1;
    }
    CUtensorMap map_out = map_b;  // (only batched launches store through a tensor map)
    if constexpr (BATCHED) {
        const uint64_t dims[3] = {static_cast<uint64_t>(n), static_cast<uint64_t>(m), static_cast<uint64_t>(batch->count)};
        const uint64_t strides[2] = {static_cast<uint64_t>(out.strides[0]) * 2, static_cast<uint64_t>(batch->out_stride) * 2};
        const uint32_t box[3] = {64, 32, 1};
        if (int rc = make_tensor_map(dev, &map_out, dtype, 3, out.data, dims, strides, box, true)) return rc;
    }
    NT_CUDA_CHECK(cudaLaunchKernelEx(&config, kernel, map_a, map_b, map_out, p));
    if (p.split_workers > 0) {
        split_reduce_kernel<BF16, ADDMM><<<static_cast<unsigned>(tiles * CG * (BN / REDUCE_COLS)), REDUCE_THREADS, 0, stream>>>(p, CG, BN);
        NT_CUDA_CHECK(cudaGetLastError());
    }
    return 0;
}

// Picks the kernel shape: CTA pairs on 256 x 256 tiles, or single CTAs on 128 x 256, 128 x 128 or 128 x 64
// tiles.  The estimate is K-blocks on the longest worker x cycles per K-block.  A pair's K-block is four N=256 MMAs, 520 cycles, and
// its 63 B/clk per SM is within what L2 gives; a single CTA's K-block is bound by the bytes it pulls from L2
// (48, 32 or 24 KB) and by the issue cost of short MMAs, so a narrower tile costs fewer cycles per K-block
// although it does fewer flops in them, and it pays exactly when the wider tile leaves most SMs without a tile.
template <bool BF16, bool B_MN, bool ADDMM, bool FP8 = false>
int launch_shape(cudaStream_t stream, const DeviceState &dev, int dtype, const Operand2D &a, const Operand2D &b,
                 const NineToothedTensor *c, const NineToothedTensor &out, float beta, float alpha,
                 const PeerOutputs *peers) {
    static thread_local int configured_device = -1;
    static thread_local int pairs = 0;
    if (configured_device != dev.device) {
        NT_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<2, 256, BF16, B_MN, ADDMM, FP8>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem_bytes<2, 256>())));
        pairs = max_active_pairs(gemm_kernel<2, 256, BF16, B_MN, ADDMM, FP8>, dev, smem_bytes<2, 256>());
        configured_device = dev.device;
    }
    static const int forced = [] {
        const char *env = std::getenv("NINETOOTHED_B200_GEMM_CTA_GROUP");
        return env ? std::atoi(env) : 0;
    }();
    static const int forced_width = [] {
        const char *env = std::getenv("NINETOOTHED_B200_GEMM_TILE_N");
        return env ? std::atoi(env) : 0;
    }();
    const int64_t row_tiles = (a.rows + BM - 1) / BM;
    const int k_blocks = static_cast<int>((a.cols + (FP8 ? 2 * BK : BK) - 1) / (FP8 ? 2 * BK : BK));
    const bool may_split = !FP8 && (peers == nullptr || (peers->count == 0 && !peers->through_switch));
    // A split needs the stream's scratch array: the estimate must not count on a split that the launch would
    // then decline (no array and none to be had), so the array is looked for, once, when a candidate wants it.
    int scratch_state = -1;  // -1 not asked yet, 0 none, 1 there
    auto scratch_there = [&]() {
        if (scratch_state < 0) scratch_state = split_scratch(dev, stream, launches_may_allocate()) != nullptr ? 1 : 0;
        return scratch_state == 1;
    };
    // cycles of the longest worker: whole tiles in waves, or its run of K-blocks plus the fix-up when split
    auto estimate = [&](int64_t tiles, int workers, int cycles) -> int64_t {
        int split_workers = split_workers_for(tiles, workers, k_blocks, may_split);
        if (split_workers > 0 && !scratch_there()) split_workers = 0;
        if (split_workers > 0)
            return (tiles * k_blocks / split_workers + 1) * cycles + int64_t{SPLIT_FIXUP_BLOCKS + 20} * 520;
        return (tiles + workers - 1) / workers * k_blocks * cycles;
    };
    int64_t best = INT64_MAX;
    int cg = 1, width = 256;
    if (pairs > 0 && forced != 1) {
        const int64_t rows_256 = (a.rows + 255) / 256, cols_256 = (b.cols + 255) / 256;
        best = estimate(rows_256 * cols_256, pairs, WIDE_CYCLES);
        // unsplit launches with a ragged last wave trade some 256-column tiles for 192-column ones
        if (!FP8 && rows_256 * cols_256 > pairs)
            best = std::min(best, plan_mixed(rows_256, cols_256, pairs, 256 * a.cols * 2).cycles * k_blocks);
        cg = 2;
        // a pair on 256 x 128: each CTA pulls 24 KB per K-block for two N=128 MMA halves
        static const int pair_128_cycles = [] {
            const char *env = std::getenv("NINETOOTHED_B200_GEMM_PAIR_128_CYCLES");
            return env ? std::atoi(env) : 460;
        }();
        if (!FP8 && (forced_width == 0 || forced_width == 128)) {
            const int64_t cost = estimate(((a.rows + 255) / 256) * ((b.cols + 127) / 128), pairs, pair_128_cycles);
            if (cost < best || forced_width == 128) best = cost, width = 128;
        }
    }
    if (forced != 2 || pairs == 0) {
        const int widths[3] = {256, 128, 64};
        const int cycles[3] = {650, 550, 440};  // measured per K-block with most SMs busy
        for (int i = 0; i < (FP8 ? 1 : 3); ++i) {
            if (forced_width != 0 && forced_width != widths[i]) continue;
            const int64_t cost = estimate(row_tiles * ((b.cols + widths[i] - 1) / widths[i]), dev.sm_count, cycles[i]);
            if (cost < best) best = cost, cg = 1, width = widths[i];
        }
    }
    if constexpr (!FP8) {
        if (cg == 2 && width == 128)
            return launch_tcgen05<2, 128, BF16, B_MN, ADDMM, FP8>(stream, dev, dtype, a, b, c, out, beta, alpha, pairs, peers);
    }
    if (cg == 2)
        return launch_tcgen05<2, 256, BF16, B_MN, ADDMM, FP8>(stream, dev, dtype, a, b, c, out, beta, alpha, pairs, peers);
    if constexpr (!FP8) {
        if (width == 128)
            return launch_tcgen05<1, 128, BF16, B_MN, ADDMM, FP8>(stream, dev, dtype, a, b, c, out, beta, alpha, 0, peers);
        if (width == 64)
            return launch_tcgen05<1, 64, BF16, B_MN, ADDMM, FP8>(stream, dev, dtype, a, b, c, out, beta, alpha, 0, peers);
    }
    return launch_tcgen05<1, 256, BF16, B_MN, ADDMM, FP8>(stream, dev, dtype, a, b, c, out, beta, alpha, 0, peers);
}

template <bool BF16, bool ADDMM>
int dispatch(cudaStream_t stream, const DeviceState &dev, int dtype, const Operand2D &a, const Operand2D &b,
             const NineToothedTensor *c, const NineToothedTensor &out, float beta, float alpha,
             const PeerOutputs *peers) {
    const bool a_ok = tma_addressable_k_major(a) && a.cols > 0;
    if (a_ok && b.stride1 == 1 && (b.stride0 % 8) == 0 && b.stride0 >= b.cols && aligned16(b.data))
        return launch_shape<BF16, true, ADDMM>(stream, dev, dtype, a, b, c, out, beta, alpha, peers);
    if (a_ok && b.stride0 == 1 && (b.stride1 % 8) == 0 && b.stride1 >= b.rows && aligned16(b.data))
        return launch_shape<BF16, false, ADDMM>(stream, dev, dtype, a, b, c, out, beta, alpha, peers);
    if (peers && (peers->count > 0 || peers->through_switch))
        return fail(NINETOOTHED_B200_ERR_LAYOUT,
                    "addmm_allgather: operands must be addressable by TMA (unit-stride rows, 16-byte aligned)");
    note_plain_launch("%s %lld x %lld x %lld runs on the plain CUDA-core kernel: the tensor-core path needs a unit-stride "
                      "K in lhs, a unit-stride dimension in rhs, the other stride a multiple of 8 elements and 16-byte "
                      "aligned bases (lhs strides %lld, %lld; rhs strides %lld, %lld)",
                      ADDMM ? "addmm" : "matmul", (long long)a.rows, (long long)b.cols, (long long)a.cols,
                      (long long)a.stride0, (long long)a.stride1, (long long)b.stride0, (long long)b.stride1);
    return launch_plain<BF16, ADDMM>(stream, a, b, c, out, beta, alpha);
}

// 8-bit e5m2 operands, fp16 output.  The tensor-core path needs rhs as a transposed view (unit stride along
// K, the layout the reference's test passes: tests/test_matmul.py:78-80) and 16-byte addressable rows.
int run_fp8(cudaStream_t stream, const DeviceState &dev, const Operand2D &a, const Operand2D &b,
            const NineToothedTensor &out) {
    const bool a_ok = a.stride1 == 1 && (a.stride0 % 16) == 0 && a.stride0 >= a.cols && aligned16(a.data) && a.cols > 0;
    const bool b_ok = b.stride0 == 1 && (b.stride1 % 16) == 0 && b.stride1 >= b.rows && aligned16(b.data);
    if (a_ok && b_ok)
        return launch_shape<false, false, false, true>(stream, dev, NINETOOTHED_B200_FLOAT8_E5M2, a, b, nullptr, out, 0.f,
                                                       1.f, nullptr);
    const int m = static_cast<int>(a.rows), n = static_cast<int>(b.cols), k = static_cast<int>(a.cols);
    dim3 grid((n + 15) / 16, (m + 15) / 16);
    if (grid.y > 65535) return fail(NINETOOTHED_B200_ERR_SHAPE, "matmul: M=%d too large for the plain kernel", m);
    note_plain_launch("e5m2 matmul %d x %d x %d runs on the plain CUDA-core kernel: the tensor-core path needs rhs as a "
                      "transposed view (unit stride along K) and rows that are multiples of 16 bytes, 16-byte aligned "
                      "(lhs strides %lld, %lld; rhs strides %lld, %lld)",
                      m, n, k, (long long)a.stride0, (long long)a.stride1, (long long)b.stride0, (long long)b.stride1);
    gemm_plain_fp8_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t *>(a.data), static_cast<const uint8_t *>(b.data),
                                                    static_cast<__half *>(out.data), m, n, k, a.stride0, a.stride1,
                                                    b.stride0, b.stride1, out.strides[0], out.strides[1]);
    NT_CUDA_CHECK(cudaGetLastError());
    return 0;
}

int run(NineToothedStream stream, const NineToothedTensor &lhs, const NineToothedTensor &rhs,
        const NineToothedTensor *input, const NineToothedTensor &output, float beta, float alpha, int dtype,
        const char *what, const PeerOutputs *peers = nullptr) {
    clear_error();
    const NineToothedTensor *all[4] = {&lhs, &rhs, &output, input};
    for (int i = 0; i < (input ? 4 : 3); ++i)
        if (!all[i]->shape || !all[i]->strides) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "%s: null shape/strides", what);
    const bool fp8 = dtype == NINETOOTHED_B200_FLOAT8_E5M2;
    if (fp8 && (input || peers)) return fail(NINETOOTHED_B200_ERR_DTYPE, "%s: 8-bit operands are taken by matmul only", what);
    if (!fp8 && !is_16bit_float(dtype))
        return fail(NINETOOTHED_B200_ERR_DTYPE, "%s: dtype %d is not fp16/bf16 (or, for matmul, e5m2)", what, dtype);
    const int64_t m = lhs.shape[0], k = lhs.shape[1], n = rhs.shape[1];
    if (static_cast<int64_t>(rhs.shape[0]) != k || static_cast<int64_t>(output.shape[0]) != m ||
        static_cast<int64_t>(output.shape[1]) != n ||
        (input && (static_cast<int64_t>(input->shape[0]) != m || static_cast<int64_t>(input->shape[1]) != n)))
        return fail(NINETOOTHED_B200_ERR_SHAPE, "%s: shapes do not agree (lhs %lld x %lld, rhs %llu x %lld, out %llu x %llu)",
                    what, (long long)m, (long long)k, (unsigned long long)rhs.shape[0], (long long)n,
                    (unsigned long long)output.shape[0], (unsigned long long)output.shape[1]);
    if (m == 0 || n == 0) return 0;
    if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL)
        return fail(NINETOOTHED_B200_ERR_SHAPE, "%s: a dimension exceeds 32-bit indexing", what);
    if (!lhs.data || !rhs.data || !output.data || (input && !input->data))
        return fail(NINETOOTHED_B200_ERR_ARGUMENT, "%s: null data pointer", what);
    const DeviceState *dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    const Operand2D a{lhs.data, m, k, lhs.strides[0], lhs.strides[1]};
    const Operand2D b{rhs.data, k, n, rhs.strides[0], rhs.strides[1]};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (fp8) return run_fp8(s, *dev, a, b, output);
    if (dtype == NINETOOTHED_BFLOAT16)
        return input ? dispatch<true, true>(s, *dev, dtype, a, b, input, output, beta, alpha, peers)
                     : dispatch<true, false>(s, *dev, dtype, a, b, nullptr, output, beta, alpha, peers);
    return input ? dispatch<false, true>(s, *dev, dtype, a, b, input, output, beta, alpha, peers)
                 : dispatch<false, false>(s, *dev, dtype, a, b, nullptr, output, beta, alpha, peers);
}

}  // namespace

// The same on channels-last tensors is one GEMM over all pixels: y[N*HW, K] = x[N*HW, C] . w[K, C]^T.  It runs as
// a "batch" of one for the sake of the batched kernel's epilogue (bulk tensor stores): with 1 to 8 K-blocks per
// tile the kernel lives in its epilogue.
int conv1x1_channels_last_as_gemm(cudaStream_t stream, const DeviceState &dev, int dtype, const void *x, const void *w,
                                  void *y, int64_t pixels, int channels, int filters) {
    const Operand2D a{x, pixels, channels, channels, 1};
    const Operand2D b{w, channels, filters, 1, channels};  // [C, K] view of w[K, C]: unit stride along C
    uint64_t shape[2] = {static_cast<uint64_t>(pixels), static_cast<uint64_t>(filters)};
    int64_t strides[2] = {filters, 1};
    const NineToothedTensor out{y, shape, strides};
    const Batch batch{1, 0, pixels * filters};  // (one problem: the stride only has to be a valid one)
    const bool bf16 = dtype == NINETOOTHED_BFLOAT16;
    static thread_local int configured_device = -1;
    static thread_local int pairs = 0;
    if (configured_device != dev.device) {
        NT_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<2, 256, false, false, false, false, true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem_bytes_batched<2, 256>())));
        pairs = max_active_pairs(gemm_kernel<2, 256, false, false, false, false, true>, dev, smem_bytes_batched<2, 256>());
        configured_device = dev.device;
    }
    if (pairs > 0) {
        return bf16 ? launch_tcgen05<2, 256, true, false, false, false, true>(stream, dev, dtype, a, b, nullptr, out, 0.f, 1.f,
                                                                               pairs, nullptr, &batch)
                    : launch_tcgen05<2, 256, false, false, false, false, true>(stream, dev, dtype, a, b, nullptr, out, 0.f,
                                                                                1.f, pairs, nullptr, &batch);
    }
    return bf16 ? launch_tcgen05<1, 256, true, false, false, false, true>(stream, dev, dtype, a, b, nullptr, out, 0.f, 1.f, 0,
                                                                           nullptr, &batch)
                : launch_tcgen05<1, 256, false, false, false, false, true>(stream, dev, dtype, a, b, nullptr, out, 0.f, 1.f, 0,
                                                                            nullptr, &batch);
}

// A 1 x 1 convolution without padding on contiguous NCHW tensors is, per image, y[K, HW] = w[K, C] . x[C, HW]:
// a batch of row-major GEMMs that share A = w.  No layout pass, no workspace.
int conv1x1_as_gemm(cudaStream_t stream, const DeviceState &dev, int dtype, const void *x, const void *w, void *y,
                    int images, int channels, int pixels, int filters) {
    const Operand2D a{w, filters, channels, channels, 1};
    const Operand2D b{x, channels, pixels, pixels, 1};
    uint64_t shape[2] = {static_cast<uint64_t>(filters), static_cast<uint64_t>(pixels)};
    int64_t strides[2] = {pixels, 1};
    const NineToothedTensor out{y, shape, strides};
    const Batch batch{images, static_cast<int64_t>(channels) * pixels, static_cast<int64_t>(filters) * pixels};
    const bool bf16 = dtype == NINETOOTHED_BFLOAT16;
    static thread_local int configured_device = -1;
    static thread_local int pairs = 0;
    if (configured_device != dev.device) {
        NT_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<2, 256, false, true, false, false, true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem_bytes_batched<2, 256>())));
        pairs = max_active_pairs(gemm_kernel<2, 256, false, true, false, false, true>, dev, smem_bytes_batched<2, 256>());
        configured_device = dev.device;
    }
    // pairs (256 filters per tile) when there are more than 128 filters, else single CTAs (128 per tile)
    if (filters > BM && pairs > 0) {
        return bf16 ? launch_tcgen05<2, 256, true, true, false, false, true>(stream, dev, dtype, a, b, nullptr, out, 0.f, 1.f,
                                                                              pairs, nullptr, &batch)
                    : launch_tcgen05<2, 256, false, true, false, false, true>(stream, dev, dtype, a, b, nullptr, out, 0.f,
                                                                               1.f, pairs, nullptr, &batch);
    }
    return bf16 ? launch_tcgen05<1, 256, true, true, false, false, true>(stream, dev, dtype, a, b, nullptr, out, 0.f, 1.f, 0,
                                                                          nullptr, &batch)
                : launch_tcgen05<1, 256, false, true, false, false, true>(stream, dev, dtype, a, b, nullptr, out, 0.f, 1.f, 0,
                                                                           nullptr, &batch);
}

// A batch of independent matmuls, output[i] = lhs[i] . rhs[i].  Row-major operands that TMA can address in three
// dimensions run as ONE launch of the batched kernel (tiles numbered batch-major, 3-D tensor maps for both
// operands and for the output, whose bounds clip partial tiles); anything else runs one 2-D matmul per problem.
int run_bmm(NineToothedStream stream, const NineToothedTensor &lhs, const NineToothedTensor &rhs,
            const NineToothedTensor &output, int dtype) {
    clear_error();
    const NineToothedTensor *all[3] = {&lhs, &rhs, &output};
    for (auto *t : all)
        if (!t->shape || !t->strides) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "bmm: null shape/strides");
    if (!is_16bit_float(dtype)) return fail(NINETOOTHED_B200_ERR_DTYPE, "bmm: dtype %d is not fp16/bf16", dtype);
    const int64_t batches = lhs.shape[0], m = lhs.shape[1], k = lhs.shape[2], n = rhs.shape[2];
    if (static_cast<int64_t>(rhs.shape[0]) != batches || static_cast<int64_t>(rhs.shape[1]) != k ||
        static_cast<int64_t>(output.shape[0]) != batches || static_cast<int64_t>(output.shape[1]) != m ||
        static_cast<int64_t>(output.shape[2]) != n)
        return fail(NINETOOTHED_B200_ERR_SHAPE, "bmm: shapes do not agree (lhs [%lld, %lld, %lld], rhs [%llu, %llu, %lld], "
                    "out [%llu, %llu, %llu])", (long long)batches, (long long)m, (long long)k,
                    (unsigned long long)rhs.shape[0], (unsigned long long)rhs.shape[1], (long long)n,
                    (unsigned long long)output.shape[0], (unsigned long long)output.shape[1],
                    (unsigned long long)output.shape[2]);
    if (batches == 0 || m == 0 || n == 0) return 0;
    if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL || batches > 0x7fffffffLL ||
        batches * ((m + 127) / 128) * ((n + 255) / 256) > 0x7fffffffLL)
        return fail(NINETOOTHED_B200_ERR_SHAPE, "bmm: a dimension exceeds 32-bit indexing");
    if (!lhs.data || !rhs.data || !output.data) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "bmm: null data pointer");
    const DeviceState *dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    auto rows_ok = [](const NineToothedTensor &t, int64_t cols) {  // [batch][row][col]: unit-stride columns, 16-byte rows
        return t.strides[2] == 1 && t.strides[1] % 8 == 0 && t.strides[1] >= cols && t.strides[0] % 8 == 0 &&
               t.strides[0] > 0 && aligned16(t.data);
    };
    const bool one_launch = k > 0 && rows_ok(lhs, k) && rows_ok(rhs, n) && rows_ok(output, n);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (one_launch) {
        const Operand2D a{lhs.data, m, k, lhs.strides[1], 1};
        const Operand2D b{rhs.data, k, n, rhs.strides[1], 1};
        uint64_t shape[2] = {static_cast<uint64_t>(m), static_cast<uint64_t>(n)};
        int64_t strides[2] = {output.strides[1], 1};
        const NineToothedTensor out{output.data, shape, strides};
        Batch batch{static_cast<int>(batches), rhs.strides[0], output.strides[0]};
        batch.a_stride = batches > 1 ? lhs.strides[0] : 0;
        const bool bf16 = dtype == NINETOOTHED_BFLOAT16;
        static thread_local int configured_device = -1;
        static thread_local int pairs = 0;
        if (configured_device != dev->device) {
            NT_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<2, 256, false, true, false, false, true>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem_bytes_batched<2, 256>())));
            pairs = max_active_pairs(gemm_kernel<2, 256, false, true, false, false, true>, *dev, smem_bytes_batched<2, 256>());
            configured_device = dev->device;
        }
        // pairs (256 rows per tile) when a problem has more than 128 rows, else single CTAs (128 per tile)
        if (m > BM && pairs > 0)
            return bf16 ? launch_tcgen05<2, 256, true, true, false, false, true>(s, *dev, dtype, a, b, nullptr, out, 0.f, 1.f,
                                                                                  pairs, nullptr, &batch)
                        : launch_tcgen05<2, 256, false, true, false, false, true>(s, *dev, dtype, a, b, nullptr, out, 0.f,
                                                                                   1.f, pairs, nullptr, &batch);
        return bf16 ? launch_tcgen05<1, 256, true, true, false, false, true>(s, *dev, dtype, a, b, nullptr, out, 0.f, 1.f, 0,
                                                                              nullptr, &batch)
                    : launch_tcgen05<1, 256, false, true, false, false, true>(s, *dev, dtype, a, b, nullptr, out, 0.f, 1.f,
                                                                               0, nullptr, &batch);
    }
    for (int64_t i = 0; i < batches; ++i) {
        const int size = dtype_size(dtype);
        uint64_t a_shape[2] = {static_cast<uint64_t>(m), static_cast<uint64_t>(k)};
        uint64_t b_shape[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n)};
        uint64_t o_shape[2] = {static_cast<uint64_t>(m), static_cast<uint64_t>(n)};
        int64_t a_strides[2] = {lhs.strides[1], lhs.strides[2]};
        int64_t b_strides[2] = {rhs.strides[1], rhs.strides[2]};
        int64_t o_strides[2] = {output.strides[1], output.strides[2]};
        const NineToothedTensor a2{static_cast<char *>(lhs.data) + i * lhs.strides[0] * size, a_shape, a_strides};
        const NineToothedTensor b2{static_cast<char *>(rhs.data) + i * rhs.strides[0] * size, b_shape, b_strides};
        const NineToothedTensor o2{static_cast<char *>(output.data) + i * output.strides[0] * size, o_shape, o_strides};
        if (int rc = run(stream, a2, b2, nullptr, o2, 0.f, 1.f, dtype, "bmm")) return rc;
    }
    return 0;
}

}  // namespace nt

extern "C" NineToothedResult launch_bmm(NineToothedStream stream, NineToothedTensor lhs, NineToothedTensor rhs,
                                        NineToothedTensor output, int dtype) {
    return nt::run_bmm(stream, lhs, rhs, output, dtype);
}

extern "C" NineToothedResult launch_matmul(NineToothedStream stream, NineToothedTensor lhs, NineToothedTensor rhs,
                                           NineToothedTensor output, int dtype) {
    return nt::run(stream, lhs, rhs, nullptr, output, 0.f, 1.f, dtype, "matmul");
}

extern "C" NineToothedResult launch_addmm(NineToothedStream stream, NineToothedTensor input, NineToothedTensor mat1,
                                          NineToothedTensor mat2, NineToothedTensor beta, NineToothedTensor alpha,
                                          NineToothedTensor output, int dtype) {
    if (!beta.data || !alpha.data) return nt::fail(NINETOOTHED_B200_ERR_ARGUMENT, "addmm: null beta/alpha");
    return nt::run(stream, mat1, mat2, &input, output, static_cast<float>(nt::scalar_f64(beta)),
                   static_cast<float>(nt::scalar_f64(alpha)), dtype, "addmm");
}

extern "C" NineToothedResult launch_addmm_allgather(NineToothedStream stream, NineToothedTensor input,
                                                    NineToothedTensor mat1, NineToothedTensor mat2,
                                                    NineToothedTensor beta, NineToothedTensor alpha,
                                                    NineToothedTensor output, void *const *peer_outputs, int world,
                                                    int rank, int dtype) {
    using namespace nt;
    if (!beta.data || !alpha.data) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "addmm_allgather: null beta/alpha");
    if (world < 1 || world > MAX_PEERS + 1 || rank < 0 || rank >= world || (world > 1 && !peer_outputs))
        return fail(NINETOOTHED_B200_ERR_ARGUMENT, "addmm_allgather: world %d (1..%d), rank %d", world, MAX_PEERS + 1, rank);
    if (!output.shape || !output.strides || !mat2.shape)
        return fail(NINETOOTHED_B200_ERR_ARGUMENT, "addmm_allgather: null shape/strides");
    // `output` is this rank's slab view [M, N_local] inside its full [M, world * N_local] buffer; the peers'
    // buffers have the same layout, so the slab sits at the same byte offset in each of them.
    PeerOutputs peers;
    peers.count = 0;
    const ptrdiff_t offset = static_cast<const char *>(output.data) - static_cast<const char *>(peer_outputs ? peer_outputs[rank] : output.data);
    for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        if (!peer_outputs[r]) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "addmm_allgather: null buffer for rank %d", r);
        peers.data[peers.count++] = static_cast<char *>(peer_outputs[r]) + offset;
    }
    return run(stream, mat1, mat2, &input, output, static_cast<float>(scalar_f64(beta)),
               static_cast<float>(scalar_f64(alpha)), dtype, "addmm_allgather", &peers);
}

extern "C" NineToothedResult launch_addmm_allgather_multicast(NineToothedStream stream, NineToothedTensor input,
                                                              NineToothedTensor mat1, NineToothedTensor mat2,
                                                              NineToothedTensor beta, NineToothedTensor alpha,
                                                              NineToothedTensor output, void *multicast_output,
                                                              int dtype) {
    using namespace nt;
    if (!beta.data || !alpha.data) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "addmm_allgather_multicast: null beta/alpha");
    if (!multicast_output) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "addmm_allgather_multicast: null multicast address");
    if (!output.shape || !output.strides || !input.shape || !input.strides)
        return fail(NINETOOTHED_B200_ERR_ARGUMENT, "addmm_allgather_multicast: null shape/strides");
    // Every store is a whole 16-byte multimem.st of a 64-column step: no element-wise edge exists on this path.
    const bool whole_steps = output.shape[1] % 64 == 0 && output.strides[1] == 1 && output.strides[0] % 8 == 0 &&
                             aligned16(multicast_output) && input.strides[1] == 1 && input.strides[0] % 8 == 0 &&
                             aligned16(input.data);
    if (!whole_steps)
        return fail(NINETOOTHED_B200_ERR_LAYOUT,
                    "addmm_allgather_multicast: the slab must be a multiple of 64 columns wide, input and output with "
                    "unit-stride, 16-byte aligned rows (launch_addmm_allgather takes the rest)");
    PeerOutputs peers;
    peers.count = 0;
    peers.through_switch = true;
    NineToothedTensor through = output;  // same shape and strides; the stores go to the multicast mapping
    through.data = multicast_output;
    return run(stream, mat1, mat2, &input, through, static_cast<float>(scalar_f64(beta)),
               static_cast<float>(scalar_f64(alpha)), dtype, "addmm_allgather_multicast", &peers);
}

extern "C" long long ninetoothed_b200_plan_mixed_widths(long long tile_rows, long long tile_cols, int pairs,
                                                       long long row_panel_bytes, int *rows, int *swaps) {
    const nt::MixedPlan plan = nt::plan_mixed(tile_rows, tile_cols, pairs, row_panel_bytes);
    if (rows) *rows = plan.rows;
    if (swaps) *swaps = plan.swaps;
    return plan.cycles;
}

extern "C" long long ninetoothed_b200_mixed_width_launches(int reset) {
    return reset ? nt::mixed_width_launches.exchange(0) : nt::mixed_width_launches.load();
}

extern "C" NineToothedResult ninetoothed_b200_reserve_split_scratch(NineToothedStream stream) {
    nt::clear_error();
    const nt::DeviceState *dev = nullptr;
    if (int rc = nt::current_device_state(&dev)) return rc;
    if (static_cast<cudaStream_t>(stream) == cudaStreamPerThread)
        return nt::fail(NINETOOTHED_B200_ERR_ARGUMENT,
                        "reserve_split_scratch: cudaStreamPerThread names a different stream in every host thread; "
                        "pass a stream of your own");
    if (nt::split_scratch(*dev, static_cast<cudaStream_t>(stream), true) == nullptr)
        return nt::fail(NINETOOTHED_B200_ERR_ARGUMENT,
                        "reserve_split_scratch: no scratch for this stream (it is being captured, the device already "
                        "has %d such arrays, or cudaMalloc failed)", nt::MAX_SPLIT_STREAMS);
    return 0;
}
