// Fused scaled-dot-product attention with online softmax on tcgen05: the kernel of
// the reference's attention application (tests/test_attention.py:45-70).
//
// One CTA owns TWO 128-row query tiles of one (batch, head) and walks the 128-row
// key/value tiles once for both, so every K/V tile fetched from L2 serves 256 query
// rows and the tensor core always has the other tile's work while one tile is in
// its softmax:
//   warp 0      TMA producer: Q0, Q1 once; K and V tiles through a three-slot ring, K one tile ahead
//   warp 1      MMA issuer, one thread: S_t = Q'_t.K_j^T into tensor memory, and
//               O_t += P_t.V_j once tile t's softmax warps have published P_t; the two
//               tiles advance independently (whichever MMA has its inputs ready goes next)
//   warps 4..7  softmax of tile 0, warps 8..11 softmax of tile 1, one thread per query
//               row: pre-scale Q by log2(e) in the storage type; per K/V tile load the
//               S row from tensor memory, mask, running max, p = exp2(s - m), row sum,
//               P rounded to the storage type into a swizzled shared-memory tile (the A
//               operand of P.V); rescale O in tensor memory when the running maximum
//               moved; at the end O / l to global memory
// Tensor memory: S0, S1, O0, O1 = 4 x 128 columns.  Shared memory (D = 128): Q 64 KB,
// P 64 KB, K/V ring 96 KB.
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
#include <cstdlib>

#include "host.h"
#include "ptx.cuh"

namespace nt {
namespace {

constexpr int BM = 128;            // rows of one query tile
constexpr int Q_TILES = 2;         // query tiles per CTA
constexpr int BN = 128;            // rows of one key/value tile
constexpr int MAX_KV_SLOTS = 6;    // ring of K/V tiles: three whole tiles (one CTA) or six half tiles (a CTA pair)
constexpr int NUM_THREADS = 128 + Q_TILES * 128;  // warp group 0: producer, MMA issuer, two idle warps
constexpr int ATOM_BYTES = 128 * 128;  // 128 rows x 64 16-bit elements, 128-byte swizzled
constexpr int TMEM_COLS = 512;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

struct SharedControl {
    uint64_t q_full[Q_TILES], q_ready[Q_TILES];
    uint64_t kv_full[MAX_KV_SLOTS], kv_empty[MAX_KV_SLOTS];
    uint64_t s_full[Q_TILES], s_empty[Q_TILES], p_full[Q_TILES], pv_done[Q_TILES];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

// CG = CTAs per MMA.  With CG = 2 (D = 128 only) two CTAs of a cluster work on 512 query rows:
// every K/V tile is loaded half by each CTA (K split by key rows, V by head columns), which is
// the operand split of a cta_group::2 MMA, so a CTA's ring holds six half tiles instead of
// three whole ones (the prefetch distance this kernel needs) and its L2 traffic halves.
template <int D, int CG>
struct Layout {
    static constexpr int ATOMS = D / 64;
    static constexpr int KV_SLOTS = 3 * CG;
    static constexpr int TILE_BYTES = ATOMS * ATOM_BYTES;  // a 128 x D tile of Q, K or V
    static constexpr int P_BYTES = 2 * ATOM_BYTES;         // 128 x 128
    static constexpr int Q_OFF = 0;
    static constexpr int P_OFF = Q_OFF + Q_TILES * TILE_BYTES;
    static constexpr int SLOT_BYTES = TILE_BYTES / CG;           // this CTA's share of a K or V tile
    static constexpr int K_ATOM_BYTES = ATOM_BYTES / CG;          // a K atom holds 128 / CG key rows
    static constexpr int KV_OFF = P_OFF + Q_TILES * P_BYTES;
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

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D, bool BF16, int CG>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    static_assert(CG == 1 || D == 128, "the CTA-pair split of V needs 64-column halves");
    using L = Layout<D, CG>;
    constexpr int KV_SLOTS = L::KV_SLOTS;
    using St = Storage<BF16>;
    using T = typename St::T;
    using T2 = typename St::T2;

    // Swizzled tiles need 1024-byte aligned bases; the whole budget is spoken for, so the
    // alignment is requested from the compiler instead of being padded for.
    extern __shared__ __align__(1024) uint8_t smem[];
    SharedControl *ctl = reinterpret_cast<SharedControl *>(smem + L::CTL_OFF);
    uint8_t *q_smem = smem + L::Q_OFF;
    uint8_t *p_smem = smem + L::P_OFF;
    uint8_t *kv_smem = smem + L::KV_OFF;

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
    const int lane = threadIdx.x & 31;
    const WaitCtx wait_ctx{&ctl->abort_flag, p.status, KID_ATTENTION};

    // Late query blocks carry the most key/value tiles under the causal mask: start them first.
    const uint32_t cta_rank = CG == 1 ? 0u : cluster_cta_rank();
    const bool leader = cta_rank == 0;
    const int q_block = static_cast<int>(gridDim.x / CG) - 1 - static_cast<int>(blockIdx.x / CG);
    const int head = blockIdx.y;
    const int batch = blockIdx.z;
    // rows of this CTA's tile t start at m0 + t * tile_stride: a pair interleaves its tiles
    // (pair tile t = rows of rank 0 then rank 1) so that paired tiles see almost the same keys
    constexpr int tile_stride = BM * CG;
    const int block0 = q_block * (Q_TILES * BM * CG);
    const int m0 = block0 + static_cast<int>(cta_rank) * BM;
    // key/value tiles each query tile visits (tile 1 sits 128 rows lower, so under the causal mask it sees one more)
    const int all_tiles = (p.s_kv + BN - 1) / BN;
    int n_tiles[Q_TILES];
#pragma unroll
    for (int t = 0; t < Q_TILES; ++t)  // counted for the lowest row of the (pair's) tile: both CTAs walk the same tiles
        n_tiles[t] = p.causal ? min(all_tiles, (block0 + t * tile_stride + tile_stride + BN - 1) / BN) : all_tiles;
    const int n_max = n_tiles[Q_TILES - 1];

    if (threadIdx.x == 0) {
        if ((smem_u32(smem) & 1023u) != 0) atomicCAS(p.status, 0u, STATUS_WAIT_TIMEOUT | (KID_ATTENTION << 16) | 0xfff);
        for (int t = 0; t < Q_TILES; ++t) {
            mbar_init(&ctl->q_full[t], 1);
            mbar_init(&ctl->q_ready[t], 4 * CG);  // one arrival per softmax warp
            mbar_init(&ctl->s_full[t], 1);
            mbar_init(&ctl->s_empty[t], 4 * CG);  // one arrival per softmax warp
            mbar_init(&ctl->p_full[t], 4 * CG);  // one arrival per softmax warp
            mbar_init(&ctl->pv_done[t], 1);
        }
        for (int s = 0; s < KV_SLOTS; ++s) {
            mbar_init(&ctl->kv_full[s], 1);
            mbar_init(&ctl->kv_empty[s], 1);
        }
        ctl->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
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
    // Arrivals that the MMA issuer polls for land on the even CTA's barrier.
    // One arrival per warp: every lane has fenced its own writes, the warp converges, lane 0 signals.
    auto arrive_at_issuer = [&](uint64_t *bar) {
        __syncwarp();
        if (lane == 0) {
            if (CG == 1 || leader) mbar_arrive(bar);
            else mbar_arrive_cluster(bar, 0);
        }
    };
    // columns: S0 [0,128)  S1 [128,256)  O0 [256,256+D)  O1 [384,384+D)

    // The register file is shared out per warp group: the four warps around the two
    // single-thread roles need few registers and hand theirs to the softmax groups, which
    // each hold a 128-column S row per thread.  (168 x 384 = 56 x 128 + 224 x 256.)
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
      if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < Q_TILES; ++t) {
                mbar_expect_tx(&ctl->q_full[t], L::TILE_BYTES);
#pragma unroll
                for (int a = 0; a < L::ATOMS; ++a)
                    tma_load_4d(q_smem + t * L::TILE_BYTES + a * ATOM_BYTES, &map_q, &ctl->q_full[t], a * 64,
                                m0 + t * tile_stride, head, batch);
            }
            // Ring order K_0, K_1, V_0, K_2, V_1, ..., K_{n-1}, V_{n-2}, V_{n-1}: K runs one tile ahead of
            // V, because S_{j+1} is issued as soon as S_j has been read while V_j is only needed after
            // the softmax; a K slot is also released early (after its two S MMAs), a V slot late.
            for (int item = 0; item < 2 * n_max; ++item) {
                const int slot = item % KV_SLOTS;
                const uint32_t phase = (item / KV_SLOTS) & 1;
                const bool is_v = item == 2 * n_max - 1 || (item >= 2 && (item & 1) == 0);
                const int j = is_v ? (item == 2 * n_max - 1 ? n_max - 1 : item / 2 - 1) : (item + 1) / 2;
                mbar_wait(&ctl->kv_empty[slot], phase ^ 1, wait_ctx, 0x100 | slot);
                uint8_t *dst = kv_smem + slot * L::SLOT_BYTES;
                if constexpr (CG == 1) {
                    mbar_expect_tx(&ctl->kv_full[slot], L::TILE_BYTES);
                    const CUtensorMap *map = is_v ? &map_v : &map_k;
#pragma unroll
                    for (int a = 0; a < L::ATOMS; ++a)
                        tma_load_4d(dst + a * ATOM_BYTES, map, &ctl->kv_full[slot], a * 64, j * BN, head, batch);
                } else {
                    // both halves are credited to the even CTA's barrier, which alone expects the bytes
                    if (leader) mbar_expect_tx(&ctl->kv_full[slot], L::TILE_BYTES);
                    if (is_v) {  // all 128 key rows, this CTA's 64 head columns
                        tma_load_4d_pair(dst, &map_v, &ctl->kv_full[slot], static_cast<int>(cta_rank) * 64, j * BN, head,
                                         batch);
                    } else {     // this CTA's 64 key rows, all head columns
#pragma unroll
                        for (int a = 0; a < L::ATOMS; ++a)
                            tma_load_4d_pair(dst + a * L::K_ATOM_BYTES, &map_k, &ctl->kv_full[slot], a * 64,
                                             j * BN + static_cast<int>(cta_rank) * 64, head, batch);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer -------------------------------
        // The whole warp runs the event loop, with every probe agreed on by a vote, so that its state,
        // addresses and descriptors are warp-uniform values (the MMA instruction takes its operands from
        // uniform registers; a lone diverged thread pays a register move for each); one elected lane issues.
        if (leader) {
            const bool issuer = elect_one();
            constexpr uint32_t idesc_s = umma_instr_desc(BM * CG, BN, BF16, false, false);  // Q' (K-major) . K^T (K-major)
            constexpr uint32_t idesc_o = umma_instr_desc(BM * CG, D, BF16, false, true);    // P (K-major) . V (N-major)

            // K/V tile `item` sits in ring slot item % 3; see the producer for the order of the items.
            auto k_item = [&](int j) { return j == 0 ? 0 : 2 * j - 1; };
            auto v_item = [&](int j) { return j == n_max - 1 ? 2 * n_max - 1 : 2 * j + 2; };
            // barriers the softmax threads of both CTAs arrive on
            auto arrived = [&](uint64_t *bar, uint32_t parity) {
                return __all_sync(0xffffffffu, CG == 1 ? mbar_test_wait(bar, parity) : mbar_test_wait_cluster(bar, parity)) != 0;
            };
            auto kv_ready = [&](int item) {
                return __all_sync(0xffffffffu, mbar_test_wait(&ctl->kv_full[item % KV_SLOTS], (item / KV_SLOTS) & 1)) != 0;
            };
            auto kv_addr = [&](int item) { return smem_u32(kv_smem + (item % KV_SLOTS) * L::SLOT_BYTES); };
            // completion signals reach both CTAs of a pair
            auto commit = [&](uint64_t *bar) {
                if (issuer) {
                    if constexpr (CG == 1) umma_commit<1>(bar);
                    else umma_commit_pair_multicast(bar, 0x3);
                }
            };
            auto release_kv = [&](int item) { commit(&ctl->kv_empty[item % KV_SLOTS]); };
            // S_t = Q'_t . K^T, K at k_addr
            auto issue_s = [&](int t, uint32_t k_addr) {
                const uint32_t q_addr = smem_u32(q_smem + t * L::TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t desc_q = umma_smem_desc(q_addr + (kk >> 2) * ATOM_BYTES + (kk & 3) * 32, 16, 1024);
                    const uint64_t desc_k = umma_smem_desc(k_addr + (kk >> 2) * L::K_ATOM_BYTES + (kk & 3) * 32, 16, 1024);
                    if (issuer) umma_ss<CG>(tmem_base + t * BN, desc_q, desc_k, idesc_s, kk != 0 ? 1u : 0u);
                }
                commit(&ctl->s_full[t]);
            };
            // O_t (+)= P_t . V, V at v_addr
            auto issue_pv = [&](int t, int j, uint32_t v_addr) {
                const uint32_t p_addr = smem_u32(p_smem + t * L::P_BYTES);
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint64_t desc_p = umma_smem_desc(p_addr + (kk >> 2) * ATOM_BYTES + (kk & 3) * 32, 16, 1024);
                    // V tile: rows are key positions (the MMA's K), 64-wide D blocks are ATOM_BYTES apart
                    const uint64_t desc_v = umma_smem_desc(v_addr + kk * (16 * 128), ATOM_BYTES, 1024);
                    if (issuer) umma_ss<CG>(tmem_base + 2 * BN + t * 128, desc_p, desc_v, idesc_o, (j | kk) != 0 ? 1u : 0u);
                }
                commit(&ctl->pv_done[t]);
            };

            // The two query tiles progress independently: whichever tile has an MMA whose inputs
            // are ready gets it issued next, so one tile's softmax never holds up the other's MMAs.
            //   S_t,j  needs K_j loaded and the softmax of tile t to have read S_t,j-1 (Q'_t for j = 0)
            //   PV_t,j needs V_j loaded and P_t,j published
            int s_next[Q_TILES] = {0, 0}, pv_next[Q_TILES] = {0, 0};
            uint64_t idle_since = 0;
            while (pv_next[0] < n_tiles[0] || pv_next[1] < n_tiles[1]) {
                bool progress = false;
#pragma unroll
                for (int t = 0; t < Q_TILES; ++t) {
                    const int o = 1 - t;  // the other tile
                    const int js = s_next[t];
                    if (js < n_tiles[t] && kv_ready(k_item(js)) &&
                        (js == 0 ? arrived(&ctl->q_ready[t], 0) : arrived(&ctl->s_empty[t], (js - 1) & 1))) {
                        tcgen05_fence_after_sync();
                        issue_s(t, kv_addr(k_item(js)));
                        s_next[t] = js + 1;
                        if (s_next[o] > js || js >= n_tiles[o]) release_kv(k_item(js));  // last reader of K_js
                        progress = true;
                    }
                    const int jp = pv_next[t];
                    if (jp < n_tiles[t] && jp < s_next[t] && kv_ready(v_item(jp)) &&
                        arrived(&ctl->p_full[t], jp & 1)) {
                        tcgen05_fence_after_sync();
                        issue_pv(t, jp, kv_addr(v_item(jp)));
                        pv_next[t] = jp + 1;
                        if (pv_next[o] > jp || jp >= n_tiles[o]) release_kv(v_item(jp));  // last reader of V_jp
                        progress = true;
                    }
                }
                if (progress) {
                    idle_since = 0;
                } else {
                    // bounded like every other wait: give up after the limit, record it, let the CTA drain
                    const uint64_t now = global_timer_ns();
                    if (idle_since == 0) idle_since = now;
                    const bool failed_before = ctl->abort_flag != 0;
                    const bool expired = now - idle_since > (failed_before ? WAIT_LIMIT_AFTER_FAILURE_NS : WAIT_LIMIT_NS);
                    if (__any_sync(0xffffffffu, expired)) {  // one verdict for the warp: the votes above need all lanes
                        if (!failed_before) {
                            ctl->abort_flag = 1;
                            atomicCAS(p.status, 0u, STATUS_WAIT_TIMEOUT | (KID_ATTENTION << 16) | 0x2ff);
                        }
                        break;
                    }
                }
            }
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        // ---------------------- softmax / correction / epilogue ----------------------
        const int t = (warp - 4) >> 2;     // which query tile this warp group serves
        const int quadrant = warp & 3;     // TMEM lanes this warp may touch
        const int row_in_tile = quadrant * 32 + lane;
        const int tid = row_in_tile;       // 0..127 within the group
        const uint32_t lane_off = static_cast<uint32_t>(quadrant * 32) << 16;
        const int row = m0 + t * tile_stride + row_in_tile;
        const uint32_t tmem_s = tmem_base + t * BN + lane_off;
        const uint32_t tmem_o = tmem_base + 2 * BN + t * 128 + lane_off;
        uint8_t *p_tile = p_smem + t * L::P_BYTES;
        const int my_tiles = n_tiles[t];

        // Q' = Q * log2(e) (after Q * scale when a scale is given), each product rounded
        // to the storage type, in place in shared memory (element-wise, layout-agnostic).
        mbar_wait(&ctl->q_full[t], 0, wait_ctx, 0x300 | t);
        {
            const T2 log2e = St::dup(1.44269504089f);
            const T2 scale2 = St::dup(p.scale);
            uint4 *q_vec = reinterpret_cast<uint4 *>(q_smem + t * L::TILE_BYTES);
#pragma unroll 4
            for (int i = 0; i < L::TILE_BYTES / 16 / 128; ++i) {
                uint4 v = q_vec[i * 128 + tid];
                T2 *h = reinterpret_cast<T2 *>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (p.has_scale) h[e] = St::mul(h[e], scale2);
                    h[e] = St::mul(h[e], log2e);
                }
                q_vec[i * 128 + tid] = v;
            }
        }
        fence_proxy_async_smem();
        arrive_at_issuer(&ctl->q_ready[t]);

        float m_used = -INFINITY;  // the maximum baked into p, l and O so far
        float l = 1.0f;            // reference: l_i starts at 1, m_i at -inf

        for (int j = 0; j < my_tiles; ++j) {
            mbar_wait(&ctl->s_full[t], j & 1, wait_ctx, 0x310 | t);
            tcgen05_fence_after_sync();
            uint32_t sreg[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32(tmem_s + c * 32, sreg[c]);
            tmem_wait_ld();
            tcgen05_fence_before_sync();
            arrive_at_issuer(&ctl->s_empty[t]);  // the S_t buffer may be overwritten by the next tile's scores

            const int col0 = j * BN;
            const bool ragged = col0 + BN > p.s_kv;
            const bool diagonal = p.causal && (col0 + BN - 1 > m0 + t * tile_stride);
            if (ragged || diagonal) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int col = col0 + c * 32 + i;
                        const bool keep = col < p.s_kv && (!p.causal || col <= row);
                        if (!keep) sreg[c][i] = __float_as_uint(-INFINITY);
                    }
            }
            // four independent chains: one running maximum would serialise 128 dependent ops
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(sreg[c][i]));
            const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));

            // Lazy rescale: keep the stale maximum while the true one is within 2^8 of it.
            const bool grow = m_tile > m_used + RESCALE_THRESHOLD;  // also true at j == 0 (m_used = -inf)
            const float m_next = grow ? m_tile : m_used;
            const float alpha = grow ? ex2(m_used - m_next) : 1.0f;  // 0 at j == 0
            m_used = m_next;

            // p = exp2(s - m) and the row sum in fp32, P rounded to the storage type.  All of it stays in
            // registers: nothing here touches the P tile or O, so it runs while the previous P.V of this
            // tile may still be in flight.
            float ls[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t packed[4][16];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0 = ex2(__uint_as_float(sreg[c][i]) - m_used);
                    const float p1 = ex2(__uint_as_float(sreg[c][i + 1]) - m_used);
                    ls[(i >> 1) & 3] += p0 + p1;
                    const T2 h = St::pack(p0, p1);
                    packed[c][i >> 1] = *reinterpret_cast<const uint32_t *>(&h);
                }
            }

            if (j > 0) {
                // O_t and the P_t buffer are stable once the previous P.V of this tile has completed.
                mbar_wait(&ctl->pv_done[t], (j - 1) & 1, wait_ctx, 0x320 | t);
                tcgen05_fence_after_sync();
                if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld_32x32(tmem_o + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x32(tmem_o + c * 32, o);
                    }
                    tmem_wait_st();
                }
            }

            // P into the 128-byte-swizzled K-major tile: 16-byte chunk c of row r lands at chunk
            // (c ^ (r & 7)) of the row's 128-byte line, 64-column halves one atom apart.
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const int chunk = c * 4 + v;  // 0..15 across the row
                    uint8_t *dst = p_tile + (chunk >> 3) * ATOM_BYTES + row_in_tile * 128 +
                                   (((chunk & 7) ^ (row_in_tile & 7)) << 4);
                    *reinterpret_cast<uint4 *>(dst) = make_uint4(packed[c][v * 4], packed[c][v * 4 + 1],
                                                                 packed[c][v * 4 + 2], packed[c][v * 4 + 3]);
                }
            }
            l = l * alpha + ((ls[0] + ls[1]) + (ls[2] + ls[3]));
            fence_proxy_async_smem();
            tcgen05_fence_before_sync();
            arrive_at_issuer(&ctl->p_full[t]);  // O_t rescaled, P_t published
        }

        // ---- epilogue: O / l -> global ----
        if (my_tiles > 0) {
            mbar_wait(&ctl->pv_done[t], (my_tiles - 1) & 1, wait_ctx, 0x330 | t);
            tcgen05_fence_after_sync();
        }
        const float inv_l = 1.0f / l;
        T *o_row = static_cast<T *>(p.o) + batch * p.o_stride_b + head * p.o_stride_h +
                   static_cast<int64_t>(row) * p.o_stride_s;
        const bool vec_ok = (p.o_stride_s % 8) == 0 && (p.o_stride_h % 8) == 0 && (p.o_stride_b % 8) == 0 &&
                            (reinterpret_cast<uintptr_t>(p.o) & 15) == 0;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
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
    if constexpr (CG == 2) cluster_sync();  // the partner may still be reading this CTA's tiles or signalling it
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc<CG>(tmem_base, TMEM_COLS);
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

template <int D, bool BF16, int CG>
int launch_fast(cudaStream_t stream, const DeviceState &dev, int dtype, const NineToothedTensor &q,
                const NineToothedTensor &k, const NineToothedTensor &v, const NineToothedTensor &o, bool causal,
                bool has_scale, float scale) {
    CUtensorMap map_q, map_k, map_v;
    if (int rc = map_for(dev, &map_q, dtype, q, BM)) return rc;
    if (int rc = map_for(dev, &map_k, dtype, k, BN / CG)) return rc;  // a pair's CTA loads half the key rows of a K tile
    if (int rc = map_for(dev, &map_v, dtype, v, BN)) return rc;       // ... and half the head columns of a V tile
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
    auto kernel = attention_kernel<D, BF16, CG>;
    constexpr size_t smem = Layout<D, CG>::SMEM_BYTES;
    static thread_local int configured_device = -1;
    if (configured_device != dev.device) {
        NT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured_device = dev.device;
    }
    constexpr int rows_per_block = Q_TILES * BM * CG;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(CG * ((p.s_q + rows_per_block - 1) / rows_per_block)), p.heads, p.batch);
    config.blockDim = dim3(NUM_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    if (CG == 2) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        config.attrs = attr;
        config.numAttrs = 1;
    }
    NT_CUDA_CHECK(cudaLaunchKernelEx(&config, kernel, map_q, map_k, map_v, p));
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
        if (d == 128) {
            // The CTA-pair variant halves each CTA's K/V traffic and doubles its prefetch depth, but the
            // extra cross-CTA hops on every S / P hand-off cost more than that buys at S = 4096
            // (measured 854 vs 1038 TFLOP/s), so it is opt-in: NINETOOTHED_B200_ATTENTION_CTA_GROUP=2.
            static const int forced = [] {
                const char *env = std::getenv("NINETOOTHED_B200_ATTENTION_CTA_GROUP");
                return env ? std::atoi(env) : 0;
            }();
            const bool pairs = forced == 2 && sq > 256;
            if (pairs)
                return bf16 ? launch_fast<128, true, 2>(s, *dev, dtype, q, k, v, o, causal, has_scale, scale)
                            : launch_fast<128, false, 2>(s, *dev, dtype, q, k, v, o, causal, has_scale, scale);
            return bf16 ? launch_fast<128, true, 1>(s, *dev, dtype, q, k, v, o, causal, has_scale, scale)
                        : launch_fast<128, false, 1>(s, *dev, dtype, q, k, v, o, causal, has_scale, scale);
        }
        return bf16 ? launch_fast<64, true, 1>(s, *dev, dtype, q, k, v, o, causal, has_scale, scale)
                    : launch_fast<64, false, 1>(s, *dev, dtype, q, k, v, o, causal, has_scale, scale);
    }
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
