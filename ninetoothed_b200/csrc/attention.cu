// Fused scaled-dot-product attention with online softmax on tcgen05: the kernel of
// the reference's attention application (tests/test_attention.py:45-70).
//
// One CTA owns TWO 128-row query tiles of one (batch, head) and walks the 80-row
// key/value tiles once for both, so every K/V tile fetched from L2 serves 256 query
// rows and the tensor core always has the other tile's work while one tile is in
// its softmax:
//   warp 0      TMA producer: Q0, Q1 once; K_j, V_j alternately through an eight-slot ring
//   warps 1, 2  MMA issuers of query tile 0 and 1 (each warp runs its loop uniformly, one
//               elected lane issues): S_t = Q'_t.K_j^T into tensor memory, and
//               O_t += P_t.V_j, P_t read from tensor memory, once tile t's softmax warps
//               have published P_t
//   warps 4..11 softmax of tile 0, warps 12..19 softmax of tile 1, two threads per query
//               row (40 key columns each): pre-scale Q by log2(e) in the storage type; per
//               K/V tile load the S row from tensor memory, mask, maximum (the two threads
//               of a row meet through shared memory to agree on it), p = exp2(s - m), row
//               sum, P rounded to the storage type and stored back into tensor memory (the
//               A operand of P.V); rescale O in tensor memory when the running maximum
//               moved; at the end O / l to global memory.  The two tiles' threads take
//               turns on the exp unit, the scarce unit of the kernel.
// Tensor memory (512 columns): S_t at 128 t (80 columns), P_t behind it (40 columns, two
// 16-bit values each), O_t at 256 + 128 t.  Shared memory (D = 128): Q 64 KB, K/V ring
// 8 x 20 KB.
//
// Why 80-row K/V tiles: with S, O and P all in tensor memory no shared memory is spent on
// P and none of its bandwidth on writing it, and the K/V ring can be eight tiles deep;
// 80 is the largest tile (a multiple of 16) for which S, P and O of both query tiles fit
// in the 512 columns.  (128-row tiles with P in shared memory measured the same speed.)
//
// Values follow the reference: fp32 S, statistics and O; P and Q' rounded to the
// storage type; l starts at 1 with m = -inf (so the first tile's alpha is 0).
// Two deliberate departures that do not change results beyond rounding noise:
// key/value tiles entirely above the causal diagonal are skipped (their p is 0 and
// alpha is 1), and O is only rescaled when the maximum grew by more than 2^8 (the
// stale maximum is used consistently for p, l and O, so O / l is unchanged).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstddef>
#include <cstdlib>

#include "host.h"
#include "ptx.cuh"

namespace nt {
namespace {

constexpr int BM = 128;            // rows of one query tile
constexpr int Q_TILES = 2;         // query tiles per CTA
constexpr int BN = 80;             // rows of one key/value tile
constexpr int KV_SLOTS = 8;        // ring of K/V tiles
constexpr int HALVES = 2;         // threads per query row in the softmax: each takes BN / 2 key columns
constexpr int NUM_THREADS = 128 + Q_TILES * HALVES * 128;  // warp group 0: producer, two MMA issuers, one idle warp
constexpr int Q_ATOM_BYTES = BM * 128;   // 128 rows x 64 16-bit elements, 128-byte swizzled
constexpr int KV_ATOM_BYTES = BN * 128;  // 80 rows x 64 16-bit elements
constexpr int TMEM_COLS = 512;
constexpr int P_COLS = BN / 2;     // P holds two 16-bit values per 32-bit column
constexpr int CAUSAL_CHUNK = 16;   // (batch, head) pairs whose query blocks are interleaved under the causal mask
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units
constexpr int HC = BN / HALVES;   // key columns per softmax thread
constexpr int HP = P_COLS / HALVES;  // packed P words per softmax thread
static_assert(BN % 16 == 0 && BN + P_COLS <= 128 && KV_ATOM_BYTES % 1024 == 0 && HC % 8 == 0 && HP % 4 == 0, "tile shape");

__host__ __device__ constexpr uint32_t s_col(int t) { return static_cast<uint32_t>(t * 128); }
__host__ __device__ constexpr uint32_t p_col(int t) { return static_cast<uint32_t>(t * 128 + BN); }
__host__ __device__ constexpr uint32_t o_col(int t) { return static_cast<uint32_t>(256 + t * 128); }

struct SharedControl {
    uint64_t q_full[Q_TILES], q_ready[Q_TILES];
    uint64_t kv_full[KV_SLOTS], kv_empty[KV_SLOTS];
    uint64_t s_full[Q_TILES], s_empty[Q_TILES], p_full[Q_TILES], pv_done[Q_TILES];
    uint32_t tmem_base;
    uint32_t abort_flag;
    float exchange[Q_TILES][HALVES][BM];  // row maxima (and at the end row sums) between the two threads of a row
};

template <int D>
struct Layout {
    static constexpr int ATOMS = D / 64;
    static constexpr int Q_TILE_BYTES = ATOMS * Q_ATOM_BYTES;  // a 128 x D tile of Q
    static constexpr int SLOT_BYTES = ATOMS * KV_ATOM_BYTES;   // an 80 x D tile of K or V
    static constexpr int Q_OFF = 0;
    static constexpr int KV_OFF = Q_OFF + Q_TILES * Q_TILE_BYTES;
    static constexpr int CTL_OFF = KV_OFF + KV_SLOTS * SLOT_BYTES;
    static constexpr size_t SMEM_BYTES = CTL_OFF + sizeof(SharedControl);
};

struct AttnParams {
    int batch, heads, s_q, s_kv;
    int causal;
    int has_scale;
    float scale;
    void *o;
    int64_t o_stride_b, o_stride_h, o_stride_s;
    unsigned int *status;
};

template <bool BF16>
struct Storage;
template <>
struct Storage<false> {
    using T = __half;
    using T2 = __half2;
    __device__ static T2 pack(float a, float b) { return __floats2half2_rn(a, b); }
    __device__ static T2 dup(float x) { return __float2half2_rn(x); }
    __device__ static T2 mul(T2 a, T2 b) { return __hmul2_rn(a, b); }
};
template <>
struct Storage<true> {
    using T = __nv_bfloat16;
    using T2 = __nv_bfloat162;
    __device__ static T2 pack(float a, float b) { return __floats2bfloat162_rn(a, b); }
    __device__ static T2 dup(float x) { return __float2bfloat162_rn(x); }
    __device__ static T2 mul(T2 a, T2 b) { return __hmul2_rn(a, b); }
};

// Named barriers 1 and 2 pass a token between the softmax threads of the two query tiles (512 threads:
// 256 that wait, 256 that only signal); barriers 3 and 4 let the two threads of a row meet.
// The exponentials are plain register arithmetic, which the assembler moves freely across a barrier
// instruction; both helpers therefore tie the barrier into the data flow with operands the assembler
// cannot see through.  token_wait returns a word read from shared memory after the barrier (the CTA's
// abort flag: zero, or a denormal when the kernel is already failing) for the caller to add to an input
// of the work that must follow; token_pass derives the barrier id from the sign of a non-negative result
// of the work that must precede it.
__device__ __forceinline__ float token_wait(int id, const uint32_t *zero_word) {
    uint32_t zero;
    asm volatile("bar.sync %1, 512;\n\tld.volatile.shared.u32 %0, [%2];"
                 : "=r"(zero)
                 : "r"(id), "r"(smem_u32(zero_word))
                 : "memory");
    return __uint_as_float(zero);
}
__device__ __forceinline__ void token_pass(int id, float non_negative) {
    asm volatile("bar.arrive %0, 512;" ::"r"(id + static_cast<int>(__float_as_uint(non_negative) >> 31)) : "memory");
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// N consecutive tensor-memory columns of this thread's lane into / out of r[0..N).
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t *r) {
    static_assert(N % 8 == 0, "columns come in groups of 8");
#pragma unroll
    for (int c = 0; c + 32 <= N; c += 32) tmem_ld_32x32(taddr + c, *reinterpret_cast<uint32_t(*)[32]>(r + c));
    if constexpr ((N % 32) >= 16)
        tmem_ld_32x16(taddr + (N / 32) * 32, *reinterpret_cast<uint32_t(*)[16]>(r + (N / 32) * 32));
    if constexpr ((N % 16) == 8)
        tmem_ld_32x8(taddr + (N / 16) * 16, *reinterpret_cast<uint32_t(*)[8]>(r + (N / 16) * 16));
}
template <int N>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t *r) {
    static_assert(N % 4 == 0, "columns come in groups of 4");
#pragma unroll
    for (int c = 0; c + 32 <= N; c += 32) tmem_st_32x32(taddr + c, *reinterpret_cast<const uint32_t(*)[32]>(r + c));
    if constexpr ((N % 32) >= 16)
        tmem_st_32x16(taddr + (N / 32) * 32, *reinterpret_cast<const uint32_t(*)[16]>(r + (N / 32) * 32));
    if constexpr ((N % 16) >= 8)
        tmem_st_32x8(taddr + (N / 16) * 16, *reinterpret_cast<const uint32_t(*)[8]>(r + (N / 16) * 16));
    if constexpr ((N % 8) == 4)
        tmem_st_32x4(taddr + (N / 8) * 8, *reinterpret_cast<const uint32_t(*)[4]>(r + (N / 8) * 8));
}

template <int D, bool BF16>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    using L = Layout<D>;
    using St = Storage<BF16>;
    using T = typename St::T;
    using T2 = typename St::T2;

    // Swizzled tiles need 1024-byte aligned bases; the whole budget is spoken for, so the
    // alignment is requested from the compiler instead of being padded for.
    extern __shared__ __align__(1024) uint8_t smem[];
    SharedControl *ctl = reinterpret_cast<SharedControl *>(smem + L::CTL_OFF);
    uint8_t *q_smem = smem + L::Q_OFF;
    uint8_t *kv_smem = smem + L::KV_OFF;

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
    const int lane = threadIdx.x & 31;
    const WaitCtx wait_ctx{&ctl->abort_flag, p.status, KID_ATTENTION};

    // Late query blocks carry the most key/value tiles under the causal mask: start them first.  Blocks are
    // dispatched in the order of their linear index.  Walking one (batch, head) pair's query blocks after another's
    // would start the last pairs' heaviest blocks when the device is about to run dry (16 units of work against an
    // average of 8.5 per block): the pairs are therefore taken in chunks of CAUSAL_CHUNK, and within a chunk the
    // query block is the slow index, so that every chunk - the last one included - ends on its lightest blocks.
    // A chunk's key/value tensors (16 x 2 MB at S = 4096, D = 128) stay in L2 while it runs.
    int q_block = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
    int head = blockIdx.y;
    int batch = blockIdx.z;
    if (p.causal) {
        const int q_blocks = gridDim.x, pairs = gridDim.y * gridDim.z;
        const int linear = blockIdx.x + q_blocks * (blockIdx.y + gridDim.y * blockIdx.z);
        const int chunk = linear / (CAUSAL_CHUNK * q_blocks);
        const int within = linear - chunk * (CAUSAL_CHUNK * q_blocks);
        const int chunk_pairs = min(CAUSAL_CHUNK, pairs - chunk * CAUSAL_CHUNK);
        const int q_rank = within / chunk_pairs;
        const int pair = chunk * CAUSAL_CHUNK + (within - q_rank * chunk_pairs);
        q_block = q_blocks - 1 - q_rank;
        head = pair % static_cast<int>(gridDim.y);
        batch = pair / static_cast<int>(gridDim.y);
    }
    const int m0 = q_block * (Q_TILES * BM);  // rows of tile t start at m0 + t * BM
    // key/value tiles each query tile visits (tile 1 sits 128 rows lower, so under the causal mask it sees more)
    const int all_tiles = (p.s_kv + BN - 1) / BN;
    int n_tiles[Q_TILES];
#pragma unroll
    for (int t = 0; t < Q_TILES; ++t)
        n_tiles[t] = p.causal ? min(all_tiles, (m0 + (t + 1) * BM + BN - 1) / BN) : all_tiles;
    const int n_max = n_tiles[Q_TILES - 1];

    if (threadIdx.x == 0) {
        if ((smem_u32(smem) & 1023u) != 0) atomicCAS(p.status, 0u, STATUS_WAIT_TIMEOUT | (KID_ATTENTION << 16) | 0xfff);
        for (int t = 0; t < Q_TILES; ++t) {
            mbar_init(&ctl->q_full[t], 1);
            mbar_init(&ctl->q_ready[t], 4 * HALVES);  // one arrival per softmax warp
            mbar_init(&ctl->s_full[t], 1);
            mbar_init(&ctl->s_empty[t], 4 * HALVES);
            mbar_init(&ctl->p_full[t], 4 * HALVES);
            mbar_init(&ctl->pv_done[t], 1);
        }
        for (int s = 0; s < KV_SLOTS; ++s) {
            mbar_init(&ctl->kv_full[s], 1);
            mbar_init(&ctl->kv_empty[s], Q_TILES);  // released by the issuer of each query tile
        }
        ctl->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
    }
    if (warp == 1) {
        tmem_alloc<1>(&ctl->tmem_base, TMEM_COLS);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, ctl->tmem_base, 0);  // warp-uniform for the tcgen05 operands
    // One arrival per warp: every lane has fenced its own writes, the warp converges, lane 0 signals.
    auto arrive_warp = [&](uint64_t *bar) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
    };

    // The register file is shared out per warp group: the four warps around the two
    // issuing roles need few registers and hand theirs to the softmax groups.
    // (640 threads at 96 registers each = 32 x 128 + 112 x 512 exactly: a larger sum would leave the last
    // group waiting for registers for ever.)
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 32;");
      if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < Q_TILES; ++t) {
                mbar_expect_tx(&ctl->q_full[t], L::Q_TILE_BYTES);
#pragma unroll
                for (int a = 0; a < L::ATOMS; ++a)
                    tma_load_4d(q_smem + t * L::Q_TILE_BYTES + a * Q_ATOM_BYTES, &map_q, &ctl->q_full[t], a * 64,
                                m0 + t * BM, head, batch);
            }
            // Ring order K_0, V_0, K_1, V_1, ...: item 2j is K_j, item 2j + 1 is V_j, item i sits in slot i % 8.
            for (int item = 0; item < 2 * n_max; ++item) {
                const int slot = item % KV_SLOTS;
                const uint32_t phase = (item / KV_SLOTS) & 1;
                const int j = item >> 1;
                mbar_wait(&ctl->kv_empty[slot], phase ^ 1, wait_ctx, 0x100 | slot);
                uint8_t *dst = kv_smem + slot * L::SLOT_BYTES;
                mbar_expect_tx(&ctl->kv_full[slot], L::SLOT_BYTES);
                const CUtensorMap *map = (item & 1) ? &map_v : &map_k;
#pragma unroll
                for (int a = 0; a < L::ATOMS; ++a)
                    tma_load_4d(dst + a * KV_ATOM_BYTES, map, &ctl->kv_full[slot], a * 64, j * BN, head, batch);
            }
        }
      } else if (warp <= Q_TILES) {
        // ------------------------------- MMA issuers ------------------------------
        // Warp 1 issues the MMAs of query tile 0, warp 2 those of tile 1 (different accumulators, shared
        // read-only operands), so that one warp's bookkeeping between batches overlaps the other's MMAs.
        // Each warp runs its loop uniformly, so that addresses and descriptors are warp-uniform values (the
        // MMA instruction takes its operands from uniform registers; a lone diverged thread pays a register
        // move for each), and one elected lane issues.  A warp executes one dependent instruction every few
        // cycles, and whatever it does per MMA beyond the MMA itself is time the tensor core may stand
        // idle: the loop is straight-line code, descriptors are a constant high word plus a low word that
        // one add derives from the ring slot, barrier addresses live in registers, and the two barriers of
        // the NEXT batch are probed (by one lane) between the MMAs of the current one, so that the blocking
        // wait is only taken when a probe said "not yet".  Per tile the order is
        //   S_t,0   [S_t,j  P.V_t,j-1] for j = 1 ...   P.V_t,n-1
        // S_t,j needs K_j and the softmax of tile t to have read S_t,j-1 (the start of its iteration);
        // P.V_t,j needs V_j and P_t,j (published at its end).
        const bool issuer = elect_one();
        constexpr uint32_t idesc_s = umma_instr_desc(BM, BN, BF16, false, false);  // Q' (K-major) . K^T (K-major)
        constexpr uint32_t idesc_o = umma_instr_desc(BM, D, BF16, false, true);    // P (tensor memory) . V (N-major)
        // shared-memory descriptor = constant high word (8-row groups 1024 B apart, version 1, 128-byte
        // swizzle) + low word (address / 16, leading-dimension offset / 16 << 16)
        constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
        auto desc = [](uint32_t lo) { return (static_cast<uint64_t>(DESC_HI) << 32) | lo; };
        const uint32_t q_lo = ((smem_u32(q_smem) & 0x3FFFFu) >> 4) | (1u << 16);
        const uint32_t k_lo = ((smem_u32(kv_smem) & 0x3FFFFu) >> 4) | (1u << 16);
        const uint32_t v_lo = ((smem_u32(kv_smem) & 0x3FFFFu) >> 4) | (static_cast<uint32_t>(KV_ATOM_BYTES >> 4) << 16);
        const uint32_t ctl_at = smem_u32(ctl);
        const uint32_t kv_full_at = ctl_at + offsetof(SharedControl, kv_full);
        const uint32_t kv_empty_at = ctl_at + offsetof(SharedControl, kv_empty);
        const uint32_t q_ready_at = ctl_at + offsetof(SharedControl, q_ready);
        const uint32_t s_full_at = ctl_at + offsetof(SharedControl, s_full);
        const uint32_t s_empty_at = ctl_at + offsetof(SharedControl, s_empty);
        const uint32_t p_full_at = ctl_at + offsetof(SharedControl, p_full);
        const uint32_t pv_done_at = ctl_at + offsetof(SharedControl, pv_done);
        const int t = warp - 1;           // the query tile this warp issues for
        const int n_mine = n_tiles[t];

        struct Gate {  // the two barriers a batch waits for: its K or V tile, and the softmax hand-off
            uint32_t tile_at, tile_parity, handoff_at, handoff_parity;
        };
        // K_j is ring item 2j, V_j item 2j + 1; item i sits in slot i % 8 in the slot's (i / 8)-th use
        auto gate_s = [&](int j) -> Gate {
            return {kv_full_at + 8u * ((2 * j) & 7), static_cast<uint32_t>(j >> 2) & 1u,
                    (j == 0 ? q_ready_at : s_empty_at) + 8u * t, j == 0 ? 0u : static_cast<uint32_t>(j - 1) & 1u};
        };
        auto gate_pv = [&](int j) -> Gate {
            return {kv_full_at + 8u * ((2 * j + 1) & 7), static_cast<uint32_t>(j >> 2) & 1u, p_full_at + 8u * t,
                    static_cast<uint32_t>(j) & 1u};
        };
        auto probe = [&](uint32_t bar, uint32_t parity) -> uint32_t {  // one lane looks, all lanes learn
            uint32_t ok = 0;
            if (lane == 0) ok = mbar_test_wait_at(bar, parity) ? 1u : 0u;
            return __shfl_sync(0xffffffffu, ok, 0);
        };
        // `seen`: bit 0 = the tile barrier, bit 1 = the hand-off barrier were already seen complete
        auto enter = [&](const Gate &g, uint32_t seen, uint32_t code) {
            if (!(seen & 1u)) mbar_wait_warp_at(g.tile_at, g.tile_parity, wait_ctx, code);
            if (!(seen & 2u)) mbar_wait_warp_at(g.handoff_at, g.handoff_parity, wait_ctx, code | 1u);
            tcgen05_fence_after_sync();
        };
        const uint32_t q_t = q_lo + t * (L::Q_TILE_BYTES >> 4);
        const uint32_t tmem_s = tmem_base + s_col(t), tmem_p = tmem_base + p_col(t), tmem_o = tmem_base + o_col(t);
        // S_t = Q'_t . K_j^T; returns what the probes of `next` saw
        auto batch_s = [&](int j, const Gate &next) -> uint32_t {
            const uint32_t slot = (2 * j) & 7;
            const uint32_t k_j = k_lo + slot * (L::SLOT_BYTES >> 4);
            uint32_t seen = 0;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t q_off = ((kk >> 2) * Q_ATOM_BYTES + (kk & 3) * 32) >> 4;
                const uint32_t k_off = ((kk >> 2) * KV_ATOM_BYTES + (kk & 3) * 32) >> 4;
                if (issuer) umma_ss<1>(tmem_s, desc(q_t + q_off), desc(k_j + k_off), idesc_s, kk != 0 ? 1u : 0u);
                if (kk == 1) seen |= probe(next.tile_at, next.tile_parity);
                if (kk == 2) seen |= probe(next.handoff_at, next.handoff_parity) << 1;
            }
            if (issuer) {
                umma_commit_at(s_full_at + 8u * t);
                umma_commit_at(kv_empty_at + 8u * slot);  // this tile is done with K_j
            }
            return seen;
        };
        // O_t (+)= P_t . V_j; the 16 key positions of step kk are P columns [8 kk, 8 kk + 8), and rows
        // [16 kk, 16 kk + 16) of the V tile (128 bytes each; 64-wide D blocks are one atom apart)
        auto batch_pv = [&](int j, const Gate &next) -> uint32_t {
            const uint32_t slot = (2 * j + 1) & 7;
            const uint32_t v_j = v_lo + slot * (L::SLOT_BYTES >> 4);
            uint32_t seen = 0;
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
                if (issuer) umma_ts<1>(tmem_o, tmem_p + kk * 8, desc(v_j + kk * (2048 >> 4)), idesc_o, (j | kk) != 0 ? 1u : 0u);
                if (kk == 1) seen |= probe(next.tile_at, next.tile_parity);
                if (kk == 2) seen |= probe(next.handoff_at, next.handoff_parity) << 1;
            }
            if (issuer) {
                umma_commit_at(pv_done_at + 8u * t);
                umma_commit_at(kv_empty_at + 8u * slot);  // this tile is done with V_j
            }
            return seen;
        };

        uint32_t seen = 0;  // what the previous batch learned about the next one in program order
        for (int j = 0; j <= n_mine; ++j) {
            if (j < n_mine) {
                enter(gate_s(j), seen, 0x200 | (t << 4));
                seen = batch_s(j, gate_pv(j - 1));
            } else {
                seen = 0;
            }
            if (j >= 1) {
                enter(gate_pv(j - 1), seen, 0x208 | (t << 4));
                seen = batch_pv(j - 1, gate_s(j + 1));
            } else {
                seen = 0;
            }
        }
        // Every ring slot is released by both tiles.  Under the causal mask tile 0 visits fewer key/value
        // tiles than tile 1: it lets the rest pass, each one only once it has landed (an early arrival
        // would be counted for the slot's previous use).
        for (int item = 2 * n_mine; item < 2 * n_max; ++item) {
            const uint32_t slot = item & 7;
            mbar_wait_warp_at(kv_full_at + 8u * slot, static_cast<uint32_t>(item >> 3) & 1u, wait_ctx, 0x240 | (t << 4));
            if (lane == 0) mbar_arrive(&ctl->kv_empty[slot]);
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 112;");
        // ---------------------- softmax / correction / epilogue ----------------------
        // Two threads per query row: warps 4..11 serve tile 0, warps 12..19 tile 1; within a tile the
        // first four warps take key columns [0, 40) of every S tile, the other four [40, 80).  A thread's
        // iteration is a chain of short dependent steps, so halving what each thread loads, reduces,
        // exponentiates and stores shortens the whole period.  The two threads of a row meet once per
        // tile to agree on the maximum; their row sums are only added at the end.
        const int sw = warp - 4;
        const int t = sw >> 3;             // which query tile this warp serves
        const int hf = (sw >> 2) & 1;      // which half of the key columns
        const int quadrant = warp & 3;     // TMEM lanes this warp may touch
        const int row_in_tile = quadrant * 32 + lane;
        const int tid = hf * 128 + row_in_tile;  // 0..255 within the tile's threads
        const uint32_t lane_off = static_cast<uint32_t>(quadrant * 32) << 16;
        const int row = m0 + t * BM + row_in_tile;
        const uint32_t tmem_s = tmem_base + s_col(t) + hf * HC + lane_off;
        const uint32_t tmem_p = tmem_base + p_col(t) + hf * HP + lane_off;
        const uint32_t tmem_o = tmem_base + o_col(t) + hf * (D / 2) + lane_off;  // this thread's half of the O row
        const int my_tiles = n_tiles[t];
        float *mine_slot = &ctl->exchange[t][hf][row_in_tile];
        const float *partner_slot = &ctl->exchange[t][1 - hf][row_in_tile];
        auto meet = [&]() { asm volatile("bar.sync %0, 256;" ::"r"(3 + t) : "memory"); };

        // Q' = Q * log2(e) (after Q * scale when a scale is given), each product rounded
        // to the storage type, in place in shared memory (element-wise, layout-agnostic).
        mbar_wait_warp(&ctl->q_full[t], 0, wait_ctx, 0x300 | t);
        {
            const T2 log2e = St::dup(1.44269504089f);
            const T2 scale2 = St::dup(p.scale);
            uint4 *q_vec = reinterpret_cast<uint4 *>(q_smem + t * L::Q_TILE_BYTES);
#pragma unroll 4
            for (int i = 0; i < L::Q_TILE_BYTES / 16 / 256; ++i) {
                uint4 v = q_vec[i * 256 + tid];
                T2 *h = reinterpret_cast<T2 *>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (p.has_scale) h[e] = St::mul(h[e], scale2);
                    h[e] = St::mul(h[e], log2e);
                }
                q_vec[i * 256 + tid] = v;
            }
        }
        fence_proxy_async_smem();
        arrive_warp(&ctl->q_ready[t]);

        // The exponentials of the two tiles take turns: both at once would share the exp unit and finish
        // together, and then both would sit in their hand-off phase with the unit idle.  Taking turns, one
        // tile's exponentials run at full rate under the other's loads, stores and barrier traffic.
        // Barrier 1 + t is tile t's turn; tile 1 hands the first turn to tile 0.  (The turn barrier also
        // keeps a thread from overwriting its exchange slot before its partner has read it.)
        if (t == 1) token_pass(1, 0.f);
        const int rounds = n_max;  // tile 0 keeps passing turns while tile 1 works on its extra key/value tiles

        float m_used = -INFINITY;        // the maximum baked into p, l and O so far
        float l = hf == 0 ? 1.0f : 0.0f;  // reference: l_i starts at 1, m_i at -inf (this thread's share of it)

        for (int j = 0; j < my_tiles; ++j) {
            mbar_wait_warp(&ctl->s_full[t], j & 1, wait_ctx, 0x310 | t);
            tcgen05_fence_after_sync();
            uint32_t sreg[HC];
            tmem_ld_cols<HC>(tmem_s, sreg);
            tmem_wait_ld();
            tcgen05_fence_before_sync();
            arrive_warp(&ctl->s_empty[t]);  // the S_t buffer may be overwritten by the next tile's scores

            const int col0 = j * BN + hf * HC;
            const bool ragged = col0 + HC > p.s_kv;
            const bool diagonal = p.causal && (col0 + HC - 1 > m0 + t * BM);
            if (ragged || diagonal) {
#pragma unroll
                for (int i = 0; i < HC; ++i) {
                    const int col = col0 + i;
                    const bool keep = col < p.s_kv && (!p.causal || col <= row);
                    if (!keep) sreg[i] = __float_as_uint(-INFINITY);
                }
            }
            // four independent chains: one running maximum would serialise the dependent ops
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < HC; i += 2)
                mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], __uint_as_float(sreg[i]), __uint_as_float(sreg[i + 1]));
            const float m_part = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            *mine_slot = m_part;
            meet();
            const float m_tile = fmaxf(m_part, *partner_slot);

            // Lazy rescale: keep the stale maximum while the true one is within 2^8 of it.
            const bool grow = m_tile > m_used + RESCALE_THRESHOLD;  // also true at j == 0 (m_used = -inf)
            const float m_next = grow ? m_tile : m_used;
            const float alpha = grow ? ex2(m_used - m_next) : 1.0f;  // 0 at j == 0
            m_used = m_next;

            // p = exp2(s - m) and the row sum in fp32, P rounded to the storage type, two values per
            // 32-bit word.  All of it stays in registers: nothing here touches P_t or O_t in tensor
            // memory, so it runs while the previous P.V of this tile may still be in flight.
            m_used += token_wait(1 + t, &ctl->abort_flag);  // (+ 0: the exponentials below now depend on the barrier)
            float ls[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t packed[HP];
#pragma unroll
            for (int i = 0; i < HC; i += 2) {
                const float p0 = ex2(__uint_as_float(sreg[i]) - m_used);
                const float p1 = ex2(__uint_as_float(sreg[i + 1]) - m_used);
                ls[(i >> 1) & 3] += p0 + p1;
                const T2 h = St::pack(p0, p1);
                packed[i >> 1] = *reinterpret_cast<const uint32_t *>(&h);
            }
            const float row_sum = (ls[0] + ls[1]) + (ls[2] + ls[3]);  // depends on every exponential
            if (t == 0 || j + 1 < rounds) token_pass(2 - t, row_sum);  // (tile 1's last turn is handed to nobody)
            l = l * alpha + row_sum;

            if (j > 0) {
                // O_t and P_t are stable once the previous P.V of this tile has completed.
                mbar_wait_warp(&ctl->pv_done[t], (j - 1) & 1, wait_ctx, 0x320 | t);
                tcgen05_fence_after_sync();
                if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
                    for (int c = 0; c < D / 2 / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld_32x32(tmem_o + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x32(tmem_o + c * 32, o);
                    }
                }
            }
            tmem_st_cols<HP>(tmem_p, packed);
            tmem_wait_st();
            tcgen05_fence_before_sync();
            arrive_warp(&ctl->p_full[t]);  // O_t rescaled, P_t published
        }

        if (t == 0) {
            for (int j = my_tiles; j < rounds; ++j) {
                token_pass(2, token_wait(1, &ctl->abort_flag));
            }
        }

        // ---- epilogue: O / l -> global; l is the sum of the two threads' shares ----
        meet();  // (the partner has read the last maximum)
        *mine_slot = l;
        meet();
        l += *partner_slot;
        if (my_tiles > 0) {
            mbar_wait_warp(&ctl->pv_done[t], (my_tiles - 1) & 1, wait_ctx, 0x330 | t);
            tcgen05_fence_after_sync();
        }
        const float inv_l = 1.0f / l;
        T *o_row = static_cast<T *>(p.o) + batch * p.o_stride_b + head * p.o_stride_h +
                   static_cast<int64_t>(row) * p.o_stride_s + hf * (D / 2);
        const bool vec_ok = (p.o_stride_s % 8) == 0 && (p.o_stride_h % 8) == 0 && (p.o_stride_b % 8) == 0 &&
                            (reinterpret_cast<uintptr_t>(p.o) & 15) == 0;
#pragma unroll
        for (int c = 0; c < D / 2 / 32; ++c) {
            uint32_t o[32];
            if (my_tiles > 0) {
                tmem_ld_32x32(tmem_o + c * 32, o);
                tmem_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = 0;
            }
            if (row < p.s_q) {
                if (vec_ok) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 out;
                        T2 *h = reinterpret_cast<T2 *>(&out);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            h[e] = St::pack(__uint_as_float(o[v * 8 + 2 * e]) * inv_l,
                                            __uint_as_float(o[v * 8 + 2 * e + 1]) * inv_l);
                        *reinterpret_cast<uint4 *>(o_row + c * 32 + v * 8) = out;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const T2 h = St::pack(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l);
                        o_row[c * 32 + i] = h.x;
                        o_row[c * 32 + i + 1] = h.y;
                    }
                }
            }
        }
    }

    __syncwarp();
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc<1>(tmem_base, TMEM_COLS);
    }
}

// Any head size up to 128, any strides, fp16 / bf16 / fp32: one thread per query
// row, keys visited one at a time with the same update rule.
template <typename T>
struct Scalar;
template <>
struct Scalar<__half> {
    __device__ static float load(const __half *p) { return __half2float(*p); }
    __device__ static __half round(float x) { return __float2half_rn(x); }
    __device__ static float mul_round(float a, float b) { return __half2float(__float2half_rn(a * b)); }
};
template <>
struct Scalar<__nv_bfloat16> {
    __device__ static float load(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
    __device__ static __nv_bfloat16 round(float x) { return __float2bfloat16_rn(x); }
    __device__ static float mul_round(float a, float b) { return __bfloat162float(__float2bfloat16_rn(a * b)); }
};
template <>
struct Scalar<float> {
    __device__ static float load(const float *p) { return *p; }
    __device__ static float round(float x) { return x; }
    __device__ static float mul_round(float a, float b) { return a * b; }
};

struct PlainParams {
    const void *q, *k, *v;
    void *o;
    int64_t qs[4], ks[4], vs[4], os[4];
    int batch, heads, s_q, s_kv, d;
    int causal, has_scale;
    float scale;
};

template <typename T>
__global__ void __launch_bounds__(128) attention_plain_kernel(const PlainParams p) {
    using Sc = Scalar<T>;
    const int row = blockIdx.x * 128 + threadIdx.x;
    const int head = blockIdx.y, batch = blockIdx.z;
    if (row >= p.s_q) return;
    const T *q = static_cast<const T *>(p.q) + batch * p.qs[0] + head * p.qs[1] + row * p.qs[2];
    const T *k = static_cast<const T *>(p.k) + batch * p.ks[0] + head * p.ks[1];
    const T *v = static_cast<const T *>(p.v) + batch * p.vs[0] + head * p.vs[1];
    T *o = static_cast<T *>(p.o) + batch * p.os[0] + head * p.os[1] + row * p.os[2];
    float ql[128], acc[128];
    const float scale_t = Sc::mul_round(p.scale, 1.0f);          // the scalars, in the storage type
    const float log2e_t = Sc::mul_round(1.44269504089f, 1.0f);
    for (int d = 0; d < p.d; ++d) {
        float x = Sc::load(q + d * p.qs[3]);
        if (p.has_scale) x = Sc::mul_round(x, scale_t);
        ql[d] = Sc::mul_round(x, log2e_t);
        acc[d] = 0.f;
    }
    float m = -INFINITY, l = 1.0f;
    const int last = p.causal ? min(p.s_kv, row + 1) : p.s_kv;
    for (int c = 0; c < last; ++c) {
        float s = 0.f;
        for (int d = 0; d < p.d; ++d) s = fmaf(ql[d], Sc::load(k + c * p.ks[2] + d * p.ks[3]), s);
        const float m_new = fmaxf(m, s);
        const float alpha = exp2f(m - m_new);
        const float pr = exp2f(s - m_new);
        const float pr_rounded = Sc::mul_round(pr, 1.0f);
        for (int d = 0; d < p.d; ++d) acc[d] = acc[d] * alpha + pr_rounded * Sc::load(v + c * p.vs[2] + d * p.vs[3]);
        l = l * alpha + pr;
        m = m_new;
    }
    for (int d = 0; d < p.d; ++d) o[d * p.os[3]] = Sc::round(acc[d] / l);
}

bool tma_ok(const NineToothedTensor &t) {
    return t.strides[3] == 1 && t.strides[2] % 8 == 0 && t.strides[1] % 8 == 0 && t.strides[0] % 8 == 0 &&
           aligned16(t.data) && t.strides[2] > 0 && t.strides[1] > 0 && t.strides[0] > 0;
}

int map_for(const DeviceState &dev, CUtensorMap *map, int dtype, const NineToothedTensor &t, uint32_t box_rows) {
    // dims innermost first: D, S, H, B.  Size-1 dimensions may carry any stride: give them a legal one.
    const uint64_t dims[4] = {t.shape[3], t.shape[2], t.shape[1], t.shape[0]};
    const uint64_t strides[3] = {static_cast<uint64_t>(t.strides[2]) * 2, static_cast<uint64_t>(t.strides[1]) * 2,
                                 static_cast<uint64_t>(t.strides[0]) * 2};
    const uint32_t box[4] = {64, box_rows, 1, 1};
    return make_tensor_map(dev, map, dtype, 4, t.data, dims, strides, box, true);
}

template <int D, bool BF16>
int launch_fast(cudaStream_t stream, const DeviceState &dev, int dtype, const NineToothedTensor &q,
                const NineToothedTensor &k, const NineToothedTensor &v, const NineToothedTensor &o, bool causal,
                bool has_scale, float scale) {
    CUtensorMap map_q, map_k, map_v;
    if (int rc = map_for(dev, &map_q, dtype, q, BM)) return rc;
    if (int rc = map_for(dev, &map_k, dtype, k, BN)) return rc;
    if (int rc = map_for(dev, &map_v, dtype, v, BN)) return rc;
    AttnParams p;
    p.batch = static_cast<int>(q.shape[0]);
    p.heads = static_cast<int>(q.shape[1]);
    p.s_q = static_cast<int>(q.shape[2]);
    p.s_kv = static_cast<int>(k.shape[2]);
    p.causal = causal ? 1 : 0;
    p.has_scale = has_scale ? 1 : 0;
    p.scale = scale;
    p.o = o.data;
    p.o_stride_b = o.strides[0];
    p.o_stride_h = o.strides[1];
    p.o_stride_s = o.strides[2];
    p.status = dev.status;
    auto kernel = attention_kernel<D, BF16>;
    constexpr size_t smem = Layout<D>::SMEM_BYTES;
    static thread_local int configured_device = -1;
    if (configured_device != dev.device) {
        NT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured_device = dev.device;
    }
    constexpr int rows_per_block = Q_TILES * BM;
    const dim3 grid(static_cast<unsigned>((p.s_q + rows_per_block - 1) / rows_per_block), p.heads, p.batch);
    kernel<<<grid, NUM_THREADS, smem, stream>>>(map_q, map_k, map_v, p);
    NT_CUDA_CHECK(cudaGetLastError());
    return 0;
}

template <typename T>
int launch_plain(cudaStream_t stream, const NineToothedTensor &q, const NineToothedTensor &k,
                 const NineToothedTensor &v, const NineToothedTensor &o, bool causal, bool has_scale, float scale) {
    PlainParams p;
    p.q = q.data;
    p.k = k.data;
    p.v = v.data;
    p.o = o.data;
    for (int i = 0; i < 4; ++i) {
        p.qs[i] = q.strides[i];
        p.ks[i] = k.strides[i];
        p.vs[i] = v.strides[i];
        p.os[i] = o.strides[i];
    }
    p.batch = static_cast<int>(q.shape[0]);
    p.heads = static_cast<int>(q.shape[1]);
    p.s_q = static_cast<int>(q.shape[2]);
    p.s_kv = static_cast<int>(k.shape[2]);
    p.d = static_cast<int>(q.shape[3]);
    p.causal = causal ? 1 : 0;
    p.has_scale = has_scale ? 1 : 0;
    p.scale = scale;
    dim3 grid((p.s_q + 127) / 128, p.heads, p.batch);
    attention_plain_kernel<T><<<grid, 128, 0, stream>>>(p);
    NT_CUDA_CHECK(cudaGetLastError());
    return 0;
}

int run(NineToothedStream stream, const NineToothedTensor &q, const NineToothedTensor &k, const NineToothedTensor &v,
        const NineToothedTensor &o, bool causal, bool has_scale, float scale, int dtype) {
    clear_error();
    const NineToothedTensor *all[4] = {&q, &k, &v, &o};
    for (auto *t : all)
        if (!t->data || !t->shape || !t->strides) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "attention: null tensor field");
    if (dtype != NINETOOTHED_FLOAT16 && dtype != NINETOOTHED_BFLOAT16 && dtype != NINETOOTHED_FLOAT32)
        return fail(NINETOOTHED_B200_ERR_DTYPE, "attention: dtype %d is not fp16/bf16/fp32", dtype);
    const uint64_t b = q.shape[0], h = q.shape[1], sq = q.shape[2], d = q.shape[3], skv = k.shape[2];
    for (auto *t : {&k, &v})
        if (t->shape[0] != b || t->shape[1] != h || t->shape[2] != skv || t->shape[3] != d)
            return fail(NINETOOTHED_B200_ERR_SHAPE, "attention: k/v must be [%llu, %llu, S_kv, %llu]",
                        (unsigned long long)b, (unsigned long long)h, (unsigned long long)d);
    if (o.shape[0] != b || o.shape[1] != h || o.shape[2] != sq || o.shape[3] != d)
        return fail(NINETOOTHED_B200_ERR_SHAPE, "attention: o must have the shape of q");
    if (d == 0 || d > 128) return fail(NINETOOTHED_B200_ERR_SHAPE, "attention: head size %llu not in [1, 128]", (unsigned long long)d);
    if (b == 0 || h == 0 || sq == 0) return 0;
    if (b > 65535 || h > 65535 || sq > 0x7fffff00ull || skv > 0x7fffff00ull)
        return fail(NINETOOTHED_B200_ERR_SHAPE, "attention: a dimension exceeds the launch limits");
    const DeviceState *dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool fast = is_16bit_float(dtype) && (d == 64 || d == 128) && skv > 0 && tma_ok(q) && tma_ok(k) && tma_ok(v) &&
                      o.strides[3] == 1;
    if (fast) {
        const bool bf16 = dtype == NINETOOTHED_BFLOAT16;
        if (d == 128)
            return bf16 ? launch_fast<128, true>(s, *dev, dtype, q, k, v, o, causal, has_scale, scale)
                        : launch_fast<128, false>(s, *dev, dtype, q, k, v, o, causal, has_scale, scale);
        return bf16 ? launch_fast<64, true>(s, *dev, dtype, q, k, v, o, causal, has_scale, scale)
                    : launch_fast<64, false>(s, *dev, dtype, q, k, v, o, causal, has_scale, scale);
    }
    note_plain_launch("attention [%llu, %llu, %llu, %llu] runs on the plain CUDA-core kernel (one thread per query row): "
                      "the tensor-core path needs a 16-bit dtype, a head size of 64 or 128, a unit-stride last dimension "
                      "and 16-byte aligned rows in q, k and v",
                      (unsigned long long)b, (unsigned long long)h, (unsigned long long)sq, (unsigned long long)d);
    if (dtype == NINETOOTHED_FLOAT16) return launch_plain<__half>(s, q, k, v, o, causal, has_scale, scale);
    if (dtype == NINETOOTHED_BFLOAT16) return launch_plain<__nv_bfloat16>(s, q, k, v, o, causal, has_scale, scale);
    return launch_plain<float>(s, q, k, v, o, causal, has_scale, scale);
}

}  // namespace
}  // namespace nt

extern "C" NineToothedResult launch_attention(NineToothedStream stream, NineToothedTensor q, NineToothedTensor k,
                                              NineToothedTensor v, NineToothedTensor is_causal, NineToothedTensor o,
                                              int dtype) {
    if (!is_causal.data) return nt::fail(NINETOOTHED_B200_ERR_ARGUMENT, "attention: null is_causal");
    return nt::run(stream, q, k, v, o, nt::scalar_i64(is_causal) != 0, false, 1.0f, dtype);
}

extern "C" NineToothedResult launch_attention_scaled(NineToothedStream stream, NineToothedTensor q,
                                                     NineToothedTensor k, NineToothedTensor v,
                                                     NineToothedTensor scale, NineToothedTensor is_causal,
                                                     NineToothedTensor o, int dtype) {
    if (!is_causal.data || !scale.data) return nt::fail(NINETOOTHED_B200_ERR_ARGUMENT, "attention: null scalar");
    return nt::run(stream, q, k, v, o, nt::scalar_i64(is_causal) != 0, true, static_cast<float>(nt::scalar_f64(scale)),
                   dtype);
}
