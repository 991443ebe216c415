// conv2d as implicit GEMM on tcgen05 (NCHW, stride 1, dilation 1, zero padding):
// the reference's im2col arrangement under its matmul application
// (tests/test_conv2d.py:13-48, :106).  C[(n,p,q), k] = sum over (c,r,s) of
// x[n, c, p+r-pad_h, q+s-pad_w] * w[k, c, r, s], fp32 accumulate, one rounding.
//
// Two steps on the caller's stream, sharing a caller-provided workspace:
//   1. layout: x NCHW -> NHWC (channels padded to a multiple of 8) and
//      w [K,C,R,S] -> [R*S, K, C]; both make the reduction dimension (channels)
//      the unit-stride one, which is what TMA boxes and K-major MMA operands need.
//   2. the GEMM: an output tile is 2 images x 8 rows x 8 columns = 128 pixels by 256
//      output channels (128 or 64 when the filter count is no larger, so that a layer with
//      few filters does not spend MMA time and TMEM on channels it does not have; the
//      narrower stages also make the pipeline deeper).  For every filter tap (r,s) and 64-channel block, one 4-D
//      TMA box of the NHWC input shifted by (r-pad_h, s-pad_w) IS the im2col tile
//      (out-of-range rows/columns are zero-filled by TMA = the padding), and one 3-D
//      box of the re-laid-out filter is the B tile.  Same warp roles and
//      double-buffered TMEM accumulator as the matmul kernel; the epilogue writes
//      NCHW directly.  Large problems run on CTA pairs (tcgen05 cta_group::2): a pair's
//      tile is 4 images x 8 x 8 pixels by 256 channels, each CTA loads its own two
//      images and half of the filter rows, which takes a third off every CTA's
//      shared-memory traffic (the single-CTA tile asks more of L2 than it delivers).
// The reduction runs over (r,s,c) instead of the reference's (c,r,s): a different
// fp32 summation order, nothing else.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "host.h"
#include "ptx.cuh"

namespace nt {
namespace {

constexpr int TILE_N = 2, TILE_H = 8, TILE_W = 8;
constexpr int BM = TILE_N * TILE_H * TILE_W;  // 128 pixels
// BN, the output channels per tile, is a template argument: 64, 128 or 256, chosen by the filter count.
constexpr int BK = 64;                        // input channels per MMA block (128 bytes)
constexpr int UMMA_K = 16;
constexpr int MAX_STAGES = 8;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;

// CG = CTAs per tile: 1, or 2 for a cluster pair that shares the filter tile.
template <int CG, int BN>
struct Shape {
    static constexpr int BN_CTA = BN / CG;  // filter rows this CTA loads
    static constexpr int B_STAGE_BYTES = BN_CTA * BK * 2;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int STAGES = (192 * 1024 / STAGE_BYTES) < MAX_STAGES ? (192 * 1024 / STAGE_BYTES) : MAX_STAGES;
    static constexpr size_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + sizeof(uint64_t) * (2 * MAX_STAGES + 4) + 16;
};

struct SharedControl {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

static_assert(sizeof(SharedControl) == sizeof(uint64_t) * (2 * MAX_STAGES + 4) + 8, "control block size");

struct ConvParams {
    int n, c, h, w, k, r, s, p, q;
    int pad_h, pad_w;
    int tiles_n, tiles_p, tiles_q, tiles_k;
    int c_blocks;
    void *y;
    int64_t ys[4];
    unsigned int *status;
};

struct TileCoord {
    int n0, p0, q0, k0;
};

template <int CG, int BN>
__device__ __forceinline__ TileCoord tile_coord(int tile, const ConvParams &p) {
    TileCoord t;
    const int tk = tile % p.tiles_k;
    tile /= p.tiles_k;
    const int tq = tile % p.tiles_q;
    tile /= p.tiles_q;
    const int tp = tile % p.tiles_p;
    const int tn = tile / p.tiles_p;
    t.n0 = tn * TILE_N * CG;
    t.p0 = tp * TILE_H;
    t.q0 = tq * TILE_W;
    t.k0 = tk * BN;
    return t;
}

template <int CG, bool BF16, int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    conv2d_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                  const ConvParams p) {
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    using S = Shape<CG, BN>;
    constexpr int STAGES = S::STAGES;
    constexpr int STAGE_BYTES = S::STAGE_BYTES;
    SharedControl *ctl = reinterpret_cast<SharedControl *>(smem + STAGES * STAGE_BYTES);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
    const int lane = threadIdx.x & 31;
    const WaitCtx wait_ctx{&ctl->abort_flag, p.status, KID_CONV2D};
    const uint32_t cta_rank = CG == 1 ? 0u : cluster_cta_rank();  // position in the pair
    const bool leader = cta_rank == 0;
    const int worker = blockIdx.x / CG;   // which persistent tile stream this CTA (pair) walks
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
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w);
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

    const int num_tiles = p.tiles_n * p.tiles_p * p.tiles_q * p.tiles_k;
    const int taps = p.r * p.s;
    const int k_iters = taps * p.c_blocks;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = worker; tile < num_tiles; tile += workers) {
                const TileCoord t = tile_coord<CG, BN>(tile, p);
                const int n0 = t.n0 + static_cast<int>(cta_rank) * TILE_N;      // this CTA's two images
                const int k0 = t.k0 + static_cast<int>(cta_rank) * S::BN_CTA;   // ... and its filter rows
                for (int tap = 0; tap < taps; ++tap) {
                    const int fr = tap / p.s, fs = tap % p.s;
                    for (int cb = 0; cb < p.c_blocks; ++cb, ++it) {
                        const int s = it % STAGES;
                        const uint32_t phase = (it / STAGES) & 1;
                        mbar_wait(&ctl->empty[s], phase ^ 1, wait_ctx, 0x100 | s);
                        uint8_t *a_dst = smem + s * STAGE_BYTES;
                        uint8_t *b_dst = a_dst + A_STAGE_BYTES;
                        // im2col tile: input pixels (p0+fr-pad_h .., q0+fs-pad_w ..) of images n0, n0+1
                        if constexpr (CG == 1) {
                            mbar_expect_tx(&ctl->full[s], STAGE_BYTES);
                            tma_load_4d(a_dst, &map_x, &ctl->full[s], cb * BK, t.q0 + fs - p.pad_w,
                                        t.p0 + fr - p.pad_h, n0);
                            tma_load_3d(b_dst, &map_w, &ctl->full[s], cb * BK, k0, tap);
                        } else {
                            // Both CTAs' bytes are credited to the even CTA's barrier, which alone expects them.
                            if (leader) mbar_expect_tx(&ctl->full[s], STAGE_BYTES * CG);
                            tma_load_4d_pair(a_dst, &map_x, &ctl->full[s], cb * BK, t.q0 + fs - p.pad_w,
                                             t.p0 + fr - p.pad_h, n0);
                            tma_load_3d_pair(b_dst, &map_w, &ctl->full[s], cb * BK, k0, tap);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // The whole warp walks the loop so that addresses and descriptors are warp-uniform values (the MMA
        // instruction takes its operands from uniform registers); one elected lane issues.  The probe of the
        // next stage's barrier sits between this stage's MMAs, where the tensor core is busy anyway.
        if (leader) {
            constexpr uint32_t idesc = umma_instr_desc(BM * CG, BN, BF16, false, false);
            const bool issuer = elect_one();
            const uint32_t smem_base = smem_u32(smem);
            uint32_t s = 0, phase = 0, acc_it = 0;
            bool ready = false;
            for (int tile = worker; tile < num_tiles; tile += workers, ++acc_it) {
                const uint32_t buf = acc_it & 1;
                const uint32_t acc_phase = (acc_it >> 1) & 1;
                mbar_wait(&ctl->tmem_empty[buf], acc_phase ^ 1, wait_ctx, 0x200 | buf);
                tcgen05_fence_after_sync();
                const uint32_t tmem_acc = tmem_base + buf * BN;
                for (int kb = 0; kb < k_iters; ++kb) {
                    if (!ready) mbar_wait(&ctl->full[s], phase, wait_ctx, 0x300 | s);
                    tcgen05_fence_after_sync();
                    const uint32_t a_addr = smem_base + s * STAGE_BYTES;
                    const uint32_t b_addr = a_addr + A_STAGE_BYTES;
                    const uint32_t s_next = s + 1 == STAGES ? 0 : s + 1;
                    const uint32_t phase_next = s_next == 0 ? phase ^ 1 : phase;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t desc_a = umma_smem_desc(a_addr + kk * 32, 16, 1024);
                        const uint64_t desc_b = umma_smem_desc(b_addr + kk * 32, 16, 1024);
                        if (issuer) umma_ss<CG>(tmem_acc, desc_a, desc_b, idesc, (kb | kk) != 0 ? 1u : 0u);
                        if (kk == BK / UMMA_K / 2 - 1)
                            ready = __all_sync(0xffffffffu, mbar_test_wait(&ctl->full[s_next], phase_next));
                    }
                    if (issuer) {  // frees the stage (in both CTAs of a pair) once these MMAs have read it
                        if constexpr (CG == 1) umma_commit<1>(&ctl->empty[s]);
                        else umma_commit_pair_multicast(&ctl->empty[s], 0x3);
                    }
                    s = s_next;
                    phase = phase_next;
                }
                if (issuer) {  // accumulator complete (each CTA of a pair drains its own rows)
                    if constexpr (CG == 1) umma_commit<1>(&ctl->tmem_full[buf]);
                    else umma_commit_pair_multicast(&ctl->tmem_full[buf], 0x3);
                }
                __syncwarp();
            }
        }
    } else {
        const int quadrant = warp & 3;
        const int row_in_tile = quadrant * 32 + lane;  // = n_i * 64 + h_i * 8 + w_i, the TMA box order
        const int n_i = row_in_tile / (TILE_H * TILE_W);
        const int h_i = (row_in_tile / TILE_W) % TILE_H;
        const int w_i = row_in_tile % TILE_W;
        T *y = static_cast<T *>(p.y);
        uint32_t acc_it = 0;
        for (int tile = worker; tile < num_tiles; tile += workers, ++acc_it) {
            const TileCoord t = tile_coord<CG, BN>(tile, p);
            const int n = t.n0 + static_cast<int>(cta_rank) * TILE_N + n_i, op = t.p0 + h_i, oq = t.q0 + w_i;
            const bool pixel_valid = n < p.n && op < p.p && oq < p.q;
            T *y_pixel = y + n * p.ys[0] + op * p.ys[2] + oq * p.ys[3];
            // channels-last output: a pixel's channels are contiguous, 16 bytes at a time
            const bool channel_vectors = p.ys[1] == 1 && ((p.ys[0] | p.ys[2] | p.ys[3]) & 7) == 0 &&
                                         (reinterpret_cast<uintptr_t>(y) & 15) == 0;
            const uint32_t buf = acc_it & 1;
            const uint32_t acc_phase = (acc_it >> 1) & 1;
            mbar_wait(&ctl->tmem_full[buf], acc_phase, wait_ctx, 0x400 | buf);
            tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quadrant * 32) << 16);
#pragma unroll 1
            for (int chunk = 0; chunk < BN / 32; ++chunk) {
                uint32_t acc[32];
                tmem_ld_32x32(taddr + chunk * 32, acc);
                tmem_wait_ld();
                const int k_base = t.k0 + chunk * 32;
                if (pixel_valid && channel_vectors && k_base + 32 <= p.k) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 packed;
                        uint32_t *word = reinterpret_cast<uint32_t *>(&packed);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float lo = __uint_as_float(acc[v * 8 + 2 * j]), hi = __uint_as_float(acc[v * 8 + 2 * j + 1]);
                            if constexpr (BF16) {
                                const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                                word[j] = *reinterpret_cast<const uint32_t *>(&h);
                            } else {
                                const __half2 h = __floats2half2_rn(lo, hi);
                                word[j] = *reinterpret_cast<const uint32_t *>(&h);
                            }
                        }
                        *reinterpret_cast<uint4 *>(y_pixel + k_base + v * 8) = packed;
                    }
                } else if (pixel_valid && k_base < p.k) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (k_base + j < p.k) {
                            const float v = __uint_as_float(acc[j]);
                            T out;
                            if constexpr (BF16) out = __float2bfloat16_rn(v);
                            else out = __float2half_rn(v);
                            y_pixel[static_cast<int64_t>(k_base + j) * p.ys[1]] = out;
                        }
                    }
                }
            }
            tcgen05_fence_before_sync();
            if (CG == 1 || leader) mbar_arrive(&ctl->tmem_empty[buf]);
            else mbar_arrive_cluster(&ctl->tmem_empty[buf], 0);
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

// x[n][c][h][w] (any strides) -> xt[n][h][w][cp], channels >= C zero-filled.
// A 32(channel) x 32(pixel) tile goes through shared memory so that both the read
// (along w) and the write (along c) are coalesced.
template <typename T>
__global__ void __launch_bounds__(256)
    nchw_to_nhwc_kernel(const T *__restrict__ x, T *__restrict__ xt, int c, int hw, int w, int cp, int64_t xs_n,
                        int64_t xs_c, int64_t xs_h, int64_t xs_w) {
    __shared__ T tile[32][33];
    const int n = blockIdx.z;
    const int c0 = blockIdx.y * 32, px0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int i = ty; i < 32; i += 8) {
        const int ch = c0 + i, px = px0 + tx;
        T v = T(0.f);
        if (ch < c && px < hw) v = x[n * xs_n + ch * xs_c + (px / w) * xs_h + (px % w) * xs_w];
        tile[i][tx] = v;
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        const int px = px0 + i, ch = c0 + tx;
        if (px < hw && ch < cp) xt[(static_cast<int64_t>(n) * hw + px) * cp + ch] = tile[tx][i];
    }
}

// Fast layout kernel for the common case: (h, w) contiguous, 16-byte aligned rows.
// One CTA moves a 64-channel x 64-pixel tile: 16-byte loads along the pixels of each
// channel, a transpose through shared memory (row pitch 66 elements = 33 words, which
// spreads the transposed reads over the banks), 16-byte stores along the channels of
// each pixel (128 contiguous bytes per pixel across 8 threads).
template <typename T>
__device__ __forceinline__ void nchw_to_nhwc_vec_tile(const T *__restrict__ x, T *__restrict__ xt, int c, int hw, int cp,
                                                      int64_t xs_n, int64_t xs_c, int n) {
    constexpr int PITCH = 66;
    __shared__ __align__(16) T tile[64 * PITCH];
    const int c0 = blockIdx.y * 64, px0 = blockIdx.x * 64;
    const T *src = x + n * xs_n;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int idx = threadIdx.x + i * 256;
        const int cl = idx >> 3, v = idx & 7;  // channel row, 8-pixel vector
        const int ch = c0 + cl, px = px0 + v * 8;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (ch < c && px < hw) val = *reinterpret_cast<const uint4 *>(src + ch * xs_c + px);
        uint32_t *dst = reinterpret_cast<uint32_t *>(tile + cl * PITCH + v * 8);
        dst[0] = val.x;
        dst[1] = val.y;
        dst[2] = val.z;
        dst[3] = val.w;
    }
    __syncthreads();
    const unsigned short *raw = reinterpret_cast<const unsigned short *>(tile);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int idx = threadIdx.x + i * 256;
        const int pl = idx >> 3, cv = idx & 7;  // pixel, 8-channel vector
        const int px = px0 + pl, ch = c0 + cv * 8;
        if (px < hw && ch < cp) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t lo = raw[(cv * 8 + 2 * j) * PITCH + pl];
                const uint32_t hi = raw[(cv * 8 + 2 * j + 1) * PITCH + pl];
                w[j] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4 *>(xt + (static_cast<int64_t>(n) * hw + px) * cp + ch) =
                make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
    nchw_to_nhwc_vec_kernel(const T *__restrict__ x, T *__restrict__ xt, int c, int hw, int cp, int64_t xs_n,
                            int64_t xs_c) {
    nchw_to_nhwc_vec_tile(x, xt, c, hw, cp, xs_n, xs_c, static_cast<int>(blockIdx.z));
}

// w[k][c][r][s] (any strides) -> wt[r*s][k][cp], channels >= C zero-filled; `blocks` blocks of 256 threads share
// the elements, this one is number `block`.
template <typename T>
__device__ __forceinline__ void filter_relayout_part(const T *__restrict__ w, T *__restrict__ wt, int k, int c, int r, int s,
                                                     int cp, int64_t ws_k, int64_t ws_c, int64_t ws_r, int64_t ws_s,
                                                     int64_t block, int64_t blocks) {
    const int64_t total = static_cast<int64_t>(r) * s * k * cp;
    for (int64_t i = block * 256 + threadIdx.x; i < total; i += blocks * 256) {
        const int ch = static_cast<int>(i % cp);
        const int ko = static_cast<int>((i / cp) % k);
        const int tap = static_cast<int>(i / (static_cast<int64_t>(cp) * k));
        T v = T(0.f);
        if (ch < c) v = w[ko * ws_k + ch * ws_c + (tap / s) * ws_r + (tap % s) * ws_s];
        wt[i] = v;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
    filter_relayout_kernel(const T *__restrict__ w, T *__restrict__ wt, int k, int c, int r, int s, int cp,
                           int64_t ws_k, int64_t ws_c, int64_t ws_r, int64_t ws_s) {
    filter_relayout_part(w, wt, k, c, r, s, cp, ws_k, ws_c, ws_r, ws_s, blockIdx.x, gridDim.x);
}

// Both layout changes in one launch, so that the small filter pass runs beside the input pass instead of after
// it: the blocks of the first grid slice (z = 0, scheduled first) re-lay the filter, slice z = n + 1 moves image n.
template <typename T>
__global__ void __launch_bounds__(256)
    layout_fused_kernel(const T *__restrict__ x, T *__restrict__ xt, int c, int hw, int cp, int64_t xs_n, int64_t xs_c,
                        const T *__restrict__ w, T *__restrict__ wt, int k, int r, int s, int64_t ws_k, int64_t ws_c,
                        int64_t ws_r, int64_t ws_s) {
    if (blockIdx.z == 0) {
        filter_relayout_part(w, wt, k, c, r, s, cp, ws_k, ws_c, ws_r, ws_s,
                             static_cast<int64_t>(blockIdx.y) * gridDim.x + blockIdx.x,
                             static_cast<int64_t>(gridDim.x) * gridDim.y);
    } else {
        nchw_to_nhwc_vec_tile(x, xt, c, hw, cp, xs_n, xs_c, static_cast<int>(blockIdx.z) - 1);
    }
}

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

struct Workspace {
    int cp;
    size_t x_bytes, w_bytes, total;
};

Workspace workspace_layout(const NineToothedTensor &x, const NineToothedTensor &w) {
    Workspace ws;
    ws.cp = static_cast<int>(round_up(static_cast<int64_t>(x.shape[1]), 8));
    ws.x_bytes = static_cast<size_t>(round_up(static_cast<int64_t>(x.shape[0] * x.shape[2] * x.shape[3]) * ws.cp * 2, 256));
    ws.w_bytes = static_cast<size_t>(round_up(static_cast<int64_t>(w.shape[2] * w.shape[3] * w.shape[0]) * ws.cp * 2, 256));
    ws.total = ws.x_bytes + ws.w_bytes;
    return ws;
}

// A channels-last input (channels unit-stride, every other stride a multiple of 8 elements, 16-byte
// aligned) is what the im2col boxes want already: TMA reads it where it lies and the layout pass is
// skipped.  Channel counts that are not a multiple of 8 read zeros past C through the box's bounds.
bool input_read_in_place(const NineToothedTensor &x) {
    const int64_t c = static_cast<int64_t>(x.shape[1]);
    return x.strides[1] == 1 && x.strides[3] % 8 == 0 && x.strides[2] % 8 == 0 && x.strides[0] % 8 == 0 &&
           x.strides[3] >= c && x.strides[3] > 0 && x.strides[2] > 0 && x.strides[0] > 0 && aligned16(x.data);
}

// Likewise a channels-last filter (w[k][c][r][s] stored as [k][r][s][c], what torch gives a channels-last model):
// taps are then one stride apart and the re-layout pass is skipped.
bool filter_read_in_place(const NineToothedTensor &w) {
    const int64_t c = static_cast<int64_t>(w.shape[1]), r = static_cast<int64_t>(w.shape[2]),
                  s = static_cast<int64_t>(w.shape[3]);
    return w.strides[1] == 1 && w.strides[3] % 8 == 0 && w.strides[3] >= c && w.strides[0] % 8 == 0 && w.strides[0] > 0 &&
           (r == 1 || w.strides[2] == s * w.strides[3]) && aligned16(w.data);
}

// Which of the two unpadded 1 x 1 forms (a batch of GEMMs on contiguous NCHW tensors, one GEMM on dense
// channels-last tensors) a problem takes, if any: those touch no scratch at all.
enum class OneByOne { none, nchw, channels_last };
OneByOne one_by_one_form(const NineToothedTensor &input, const NineToothedTensor &filter, const NineToothedTensor &output,
                         int padding_h, int padding_w) {
    static const bool off = [] {
        const char *env = std::getenv("NINETOOTHED_B200_CONV2D_1X1_AS_GEMM");
        return env && std::atoi(env) == 0;
    }();
    const int64_t n = input.shape[0], c = input.shape[1], h = input.shape[2], wd = input.shape[3], hw = h * wd;
    const int64_t k = filter.shape[0];
    if (off || filter.shape[2] != 1 || filter.shape[3] != 1 || padding_h != 0 || padding_w != 0) return OneByOne::none;
    if (!(filter.strides[1] == 1 && filter.strides[0] == c) || c % 8 != 0) return OneByOne::none;
    if (!aligned16(input.data) || !aligned16(filter.data) || !aligned16(output.data)) return OneByOne::none;
    const bool x_nchw = input.strides[3] == 1 && input.strides[2] == wd && input.strides[1] == hw && input.strides[0] == c * hw;
    const bool y_nchw = output.strides[3] == 1 && output.strides[2] == wd && output.strides[1] == hw && output.strides[0] == k * hw;
    if (x_nchw && y_nchw && hw % 8 == 0) return OneByOne::nchw;
    const bool x_nhwc = input.strides[1] == 1 && input.strides[3] == c && input.strides[2] == wd * c && input.strides[0] == hw * c;
    const bool y_nhwc = output.strides[1] == 1 && output.strides[3] == k && output.strides[2] == wd * k && output.strides[0] == hw * k;
    if (x_nhwc && y_nhwc && k % 8 == 0 && n * hw <= 0x7fffffff) return OneByOne::channels_last;
    return OneByOne::none;
}

// Scratch bytes a launch really writes and reads: the re-laid-out input unless it is read in place, then
// the re-laid-out filter unless it is read in place (launch_conv2d_workspace_size is the sum of both, an
// upper bound that depends on the shapes alone).
size_t scratch_touched(const NineToothedTensor &input, const NineToothedTensor &filter, const NineToothedTensor &output,
                       int padding_h, int padding_w) {
    if (one_by_one_form(input, filter, output, padding_h, padding_w) != OneByOne::none) return 0;
    const Workspace ws = workspace_layout(input, filter);
    return (input_read_in_place(input) ? 0 : ws.x_bytes) + (filter_read_in_place(filter) ? 0 : ws.w_bytes);
}

// Cluster pairs of this kernel the device can hold at once (0: cluster launch unavailable).
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

// The filter as the tensor map sees it: [taps][filters][channels] with channels unit-stride.
struct FilterView {
    const void *data;
    int channels;                       // extent of the channel dimension (zeros are read beyond it)
    int64_t filter_stride, tap_stride;  // elements
};

// The GEMM itself for one channel-tile width: picks single CTAs or pairs, finishes the tiling, builds the
// filter's tensor map (its box depends on both) and launches.
template <bool BF16, int BN>
int launch_main(cudaStream_t stream, const DeviceState &dev, int dtype, ConvParams p, const CUtensorMap &map_x,
                const FilterView &filter) {
    // CTA pairs when there are enough pair tiles to occupy every pair the device can hold
    static thread_local int configured_device = -1;
    static thread_local int pairs = 0;
    if (configured_device != dev.device) {
        NT_CUDA_CHECK(cudaFuncSetAttribute(conv2d_kernel<1, BF16, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(Shape<1, BN>::SMEM_BYTES)));
        NT_CUDA_CHECK(cudaFuncSetAttribute(conv2d_kernel<2, BF16, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(Shape<2, BN>::SMEM_BYTES)));
        pairs = max_active_pairs(conv2d_kernel<2, BF16, BN>, dev, Shape<2, BN>::SMEM_BYTES);
        configured_device = dev.device;
    }
    static const int forced = [] {
        const char *env = std::getenv("NINETOOTHED_B200_CONV2D_CTA_GROUP");
        return env ? std::atoi(env) : 0;
    }();
    const int64_t pair_tiles = static_cast<int64_t>((p.n + 2 * TILE_N - 1) / (2 * TILE_N)) * ((p.p + TILE_H - 1) / TILE_H) *
                               ((p.q + TILE_W - 1) / TILE_W) * ((p.k + BN - 1) / BN);
    const bool use_pairs = forced == 2 ? pairs > 0 : forced == 1 ? false : (pairs > 0 && pair_tiles >= pairs);
    const int cg = use_pairs ? 2 : 1;
    p.tiles_n = (p.n + TILE_N * cg - 1) / (TILE_N * cg);
    p.tiles_p = (p.p + TILE_H - 1) / TILE_H;
    p.tiles_q = (p.q + TILE_W - 1) / TILE_W;
    p.tiles_k = (p.k + BN - 1) / BN;
    CUtensorMap map_w;
    {
        const uint64_t dims[3] = {static_cast<uint64_t>(filter.channels), static_cast<uint64_t>(p.k),
                                  static_cast<uint64_t>(p.r) * p.s};
        const uint64_t strides[2] = {static_cast<uint64_t>(filter.filter_stride) * 2,
                                     static_cast<uint64_t>(filter.tap_stride) * 2};
        const uint32_t box[3] = {BK, static_cast<uint32_t>(BN / cg), 1};  // a pair's CTA loads half the filter rows
        if (int rc = make_tensor_map(dev, &map_w, dtype, 3, filter.data, dims, strides, box, true)) return rc;
    }
    const int64_t tiles = static_cast<int64_t>(p.tiles_n) * p.tiles_p * p.tiles_q * p.tiles_k;
    if (use_pairs) {
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(static_cast<unsigned>(2 * std::min<int64_t>(tiles, pairs)));
        config.blockDim = dim3(NUM_THREADS);
        config.dynamicSmemBytes = Shape<2, BN>::SMEM_BYTES;
        config.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        config.attrs = attr;
        config.numAttrs = 1;
        NT_CUDA_CHECK(cudaLaunchKernelEx(&config, conv2d_kernel<2, BF16, BN>, map_x, map_w, p));
    } else {
        const int grid = static_cast<int>(tiles < dev.sm_count ? tiles : dev.sm_count);
        conv2d_kernel<1, BF16, BN><<<grid, NUM_THREADS, Shape<1, BN>::SMEM_BYTES, stream>>>(map_x, map_w, p);
        NT_CUDA_CHECK(cudaGetLastError());
    }
    return 0;
}

template <bool BF16>
int run_typed(cudaStream_t stream, const DeviceState &dev, int dtype, const NineToothedTensor &x,
              const NineToothedTensor &w, const NineToothedTensor &y, int pad_h, int pad_w, void *workspace) {
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const Workspace ws = workspace_layout(x, w);
    ConvParams p;
    p.n = static_cast<int>(x.shape[0]);
    p.c = static_cast<int>(x.shape[1]);
    p.h = static_cast<int>(x.shape[2]);
    p.w = static_cast<int>(x.shape[3]);
    p.k = static_cast<int>(w.shape[0]);
    p.r = static_cast<int>(w.shape[2]);
    p.s = static_cast<int>(w.shape[3]);
    p.p = p.h + 2 * pad_h - p.r + 1;
    p.q = p.w + 2 * pad_w - p.s + 1;
    p.pad_h = pad_h;
    p.pad_w = pad_w;
    p.c_blocks = (p.c + BK - 1) / BK;
    p.y = y.data;
    for (int i = 0; i < 4; ++i) p.ys[i] = y.strides[i];
    p.status = dev.status;

    const int hw = p.h * p.w;
    const bool x_in_place = input_read_in_place(x);
    const bool w_in_place = filter_read_in_place(w);
    T *xt = static_cast<T *>(workspace);
    T *wt = reinterpret_cast<T *>(static_cast<uint8_t *>(workspace) + (x_in_place ? 0 : ws.x_bytes));
    {
        const bool vectorizable = x.strides[3] == 1 && x.strides[2] == p.w && hw % 8 == 0 && x.strides[1] % 8 == 0 &&
                                  x.strides[0] % 8 == 0 && aligned16(x.data) && p.n <= 65535;
        bool filter_done = w_in_place;
        if (x_in_place) {
            // nothing to do for x
        } else if (vectorizable && p.n < 65535) {
            dim3 grid((hw + 63) / 64, (ws.cp + 63) / 64, p.n + 1);
            layout_fused_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T *>(x.data), xt, p.c, hw, ws.cp, x.strides[0],
                                                             x.strides[1], static_cast<const T *>(w.data), wt, p.k, p.r, p.s,
                                                             w.strides[0], w.strides[1], w.strides[2], w.strides[3]);
            filter_done = true;
        } else if (vectorizable) {
            dim3 grid((hw + 63) / 64, (ws.cp + 63) / 64, p.n);
            nchw_to_nhwc_vec_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T *>(x.data), xt, p.c, hw, ws.cp,
                                                                 x.strides[0], x.strides[1]);
        } else {
            dim3 grid((hw + 31) / 32, (ws.cp + 31) / 32, p.n);
            nchw_to_nhwc_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T *>(x.data), xt, p.c, hw, p.w, ws.cp,
                                                             x.strides[0], x.strides[1], x.strides[2], x.strides[3]);
        }
        NT_CUDA_CHECK(cudaGetLastError());
        if (!filter_done) {
            const int64_t total = static_cast<int64_t>(p.r) * p.s * p.k * ws.cp;
            const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 4096));
            filter_relayout_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<const T *>(w.data), wt, p.k, p.c, p.r, p.s,
                                                                  ws.cp, w.strides[0], w.strides[1], w.strides[2],
                                                                  w.strides[3]);
            NT_CUDA_CHECK(cudaGetLastError());
        }
    }
    CUtensorMap map_x;
    {
        const uint64_t dims[4] = {static_cast<uint64_t>(x_in_place ? p.c : ws.cp), static_cast<uint64_t>(p.w),
                                  static_cast<uint64_t>(p.h), static_cast<uint64_t>(p.n)};
        const uint64_t packed_strides[3] = {static_cast<uint64_t>(ws.cp) * 2, static_cast<uint64_t>(ws.cp) * 2 * p.w,
                                            static_cast<uint64_t>(ws.cp) * 2 * p.w * p.h};
        const uint64_t own_strides[3] = {static_cast<uint64_t>(x.strides[3]) * 2, static_cast<uint64_t>(x.strides[2]) * 2,
                                         static_cast<uint64_t>(x.strides[0]) * 2};
        const uint32_t box[4] = {BK, TILE_W, TILE_H, TILE_N};
        if (int rc = make_tensor_map(dev, &map_x, dtype, 4, x_in_place ? x.data : static_cast<void *>(xt), dims,
                                     x_in_place ? own_strides : packed_strides, box, true))
            return rc;
    }
    const FilterView filter = w_in_place ? FilterView{w.data, p.c, w.strides[0], w.strides[3]}
                                         : FilterView{wt, ws.cp, ws.cp, static_cast<int64_t>(ws.cp) * p.k};
    if (p.k <= 64) return launch_main<BF16, 64>(stream, dev, dtype, p, map_x, filter);
    if (p.k <= 128) return launch_main<BF16, 128>(stream, dev, dtype, p, map_x, filter);
    return launch_main<BF16, 256>(stream, dev, dtype, p, map_x, filter);
}

int check(const NineToothedTensor &x, const NineToothedTensor &w, int dtype) {
    if (!x.shape || !x.strides || !w.shape || !w.strides)
        return fail(NINETOOTHED_B200_ERR_ARGUMENT, "conv2d: null shape/strides");
    if (!is_16bit_float(dtype)) return fail(NINETOOTHED_B200_ERR_DTYPE, "conv2d: dtype %d is not fp16/bf16", dtype);
    if (x.shape[1] != w.shape[1])
        return fail(NINETOOTHED_B200_ERR_SHAPE, "conv2d: input has %llu channels, filter expects %llu",
                    (unsigned long long)x.shape[1], (unsigned long long)w.shape[1]);
    for (int i = 0; i < 4; ++i)
        if (x.shape[i] > 0x7fffffffull || w.shape[i] > 0x7fffffffull)
            return fail(NINETOOTHED_B200_ERR_SHAPE, "conv2d: a dimension exceeds 32-bit indexing");
    return 0;
}

}  // namespace
}  // namespace nt

extern "C" size_t launch_conv2d_workspace_size(NineToothedTensor input, NineToothedTensor filter, int dtype) {
    nt::clear_error();
    if (nt::check(input, filter, dtype) != 0) return 0;
    return nt::workspace_layout(input, filter).total;
}

namespace nt {
namespace {

// `exact`: the workspace only has to hold what this launch touches (scratch_touched) instead of the
// shape-only bound the public entry point documents.
int conv2d_checked(NineToothedStream stream, const NineToothedTensor &input, const NineToothedTensor &filter,
                   const NineToothedTensor &output, int padding_h, int padding_w, int dtype, void *workspace,
                   size_t workspace_size, bool exact) {
    clear_error();
    if (int rc = check(input, filter, dtype)) return rc;
    if (!output.shape || !output.strides) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "conv2d: null output shape/strides");
    if (padding_h < 0 || padding_w < 0) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "conv2d: negative padding");
    const int64_t n = input.shape[0], h = input.shape[2], wd = input.shape[3];
    const int64_t k = filter.shape[0], r = filter.shape[2], s = filter.shape[3];
    const int64_t p = h + 2 * padding_h - r + 1, q = wd + 2 * padding_w - s + 1;
    if (p < 0 || q < 0 || static_cast<int64_t>(output.shape[0]) != n || static_cast<int64_t>(output.shape[1]) != k ||
        static_cast<int64_t>(output.shape[2]) != p || static_cast<int64_t>(output.shape[3]) != q)
        return fail(NINETOOTHED_B200_ERR_SHAPE, "conv2d: output must be [%lld, %lld, %lld, %lld]", (long long)n,
                    (long long)k, (long long)p, (long long)q);
    if (n == 0 || k == 0 || p == 0 || q == 0) return 0;
    if (input.shape[1] == 0 || r == 0 || s == 0)
        return fail(NINETOOTHED_B200_ERR_SHAPE, "conv2d: empty reduction (C, R or S is 0)");
    if (r * s > 0xffff || padding_h > 0x7fff || padding_w > 0x7fff)
        return fail(NINETOOTHED_B200_ERR_SHAPE, "conv2d: filter or padding too large");
    if (!input.data || !filter.data || !output.data) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "conv2d: null data pointer");
    const size_t needed = exact ? scratch_touched(input, filter, output, padding_h, padding_w)
                                : workspace_layout(input, filter).total;
    if (workspace == nullptr || workspace_size < needed || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return fail(NINETOOTHED_B200_ERR_ARGUMENT,
                    "conv2d: workspace must be 256-byte aligned device memory of at least %zu bytes (got %zu at %p)",
                    needed, workspace_size, workspace);
    const DeviceState *dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // A 1 x 1 filter without padding needs no im2col and no layout pass: on contiguous NCHW tensors it is, per
    // image, y[K, HW] = w[K, C] . x[C, HW] (a batch of row-major GEMMs), on dense channels-last tensors one GEMM
    // over all pixels; the workspace stays unused.
    {
        const int64_t c = input.shape[1], hw = h * wd;
        const OneByOne form = one_by_one_form(input, filter, output, padding_h, padding_w);
        if (form == OneByOne::nchw)
            return conv1x1_as_gemm(st, *dev, dtype, input.data, filter.data, output.data, static_cast<int>(n),
                                   static_cast<int>(c), static_cast<int>(hw), static_cast<int>(k));
        if (form == OneByOne::channels_last)
            return conv1x1_channels_last_as_gemm(st, *dev, dtype, input.data, filter.data, output.data, n * hw,
                                                 static_cast<int>(c), static_cast<int>(k));
    }
    return dtype == NINETOOTHED_BFLOAT16
               ? run_typed<true>(st, *dev, dtype, input, filter, output, padding_h, padding_w, workspace)
               : run_typed<false>(st, *dev, dtype, input, filter, output, padding_h, padding_w, workspace);
}

}  // namespace
}  // namespace nt

extern "C" NineToothedResult launch_conv2d(NineToothedStream stream, NineToothedTensor input, NineToothedTensor filter,
                                           NineToothedTensor output, int padding_h, int padding_w, int dtype,
                                           void *workspace, size_t workspace_size) {
    return nt::conv2d_checked(stream, input, filter, output, padding_h, padding_w, dtype, workspace, workspace_size,
                              false);
}

// ---------------------------------------------------------------------------
// conv2d on the library's own scratch array, for callers that cannot allocate.
// ---------------------------------------------------------------------------

// The scratch itself: device memory that is part of the library image, one copy on
// every GPU that loads the library, alive until the process exits.  In host code
// this name is only a handle for the runtime's symbol lookup, never an address a
// kernel may be given; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_workspace[NINETOOTHED_B200_STATIC_WORKSPACE_BYTES];

namespace nt {
namespace {

std::mutex g_static_workspace_mutex;
std::unordered_map<int, void *> g_static_workspace_address;  // device ordinal -> device address

// Device address of the scratch array on the CURRENT device.  The first call on a
// device asks the runtime for it (which is why that call should precede any stream
// capture on the device); later calls read the remembered value.
int static_workspace(void **address) {
    int device = 0;
    NT_CUDA_CHECK(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(g_static_workspace_mutex);
    auto found = g_static_workspace_address.find(device);
    if (found == g_static_workspace_address.end()) {
        void *ptr = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_workspace);
        if (err != cudaSuccess || ptr == nullptr)
            return fail(err != cudaSuccess ? static_cast<int>(err) : NINETOOTHED_B200_ERR_DEVICE,
                        "conv2d (static workspace): cudaGetSymbolAddress failed on device %d: %s", device,
                        cudaGetErrorString(err));
        found = g_static_workspace_address.emplace(device, ptr).first;
    }
    *address = found->second;
    return 0;
}

}  // namespace
}  // namespace nt

// Same work as launch_conv2d, on the built-in scratch array: no allocation, no free.
// Calls on one device share the array (see the header for the rules).
extern "C" NineToothedResult launch_conv2d_static_workspace(NineToothedStream stream, NineToothedTensor input,
                                                            NineToothedTensor filter, NineToothedTensor output,
                                                            int padding_h, int padding_w, int dtype) {
    using namespace nt;
    clear_error();
    if (int rc = check(input, filter, dtype)) return rc;
    if (!output.shape || !output.strides) return fail(NINETOOTHED_B200_ERR_ARGUMENT, "conv2d: null output shape/strides");
    // What this launch will really write and read: nothing for the unpadded 1 x 1 forms, no input copy for a
    // channels-last input, no filter copy for a channels-last filter.
    const size_t needed = scratch_touched(input, filter, output, padding_h, padding_w);
    if (needed > static_cast<size_t>(NINETOOTHED_B200_STATIC_WORKSPACE_BYTES))
        return fail(NINETOOTHED_B200_ERR_ARGUMENT,
                    "conv2d (static workspace): this problem needs %zu bytes of scratch but the built-in array holds "
                    "%zu; call launch_conv2d with a workspace of your own instead",
                    needed, static_cast<size_t>(NINETOOTHED_B200_STATIC_WORKSPACE_BYTES));
    void *scratch = nullptr;
    if (int rc = static_workspace(&scratch)) return rc;
    return conv2d_checked(stream, input, filter, output, padding_h, padding_w, dtype, scratch,
                          static_cast<size_t>(NINETOOTHED_B200_STATIC_WORKSPACE_BYTES), true);
}
