// max_pool2d over non-overlapping windows of an NCHW tensor: the reference's
// max_pool2d arrangement and application (tests/test_max_pool2d.py:13-36).
// out[n,c,p,q] = max over the r x s window at (p r, q s); the window stride is the
// window itself; floor mode drops a ragged last window, ceil mode keeps it and
// positions outside the tensor count as -inf (the input's `other`, :59).
//
// The op moves every input element once and writes one output per window: it is
// bound by HBM, so the work is laid out for 16-byte accesses.  One thread produces
// 16 / sizeof(T) neighbouring outputs of two rows from s 16-byte loads per window row
// (consecutive threads read consecutive memory), reduces down the window rows with
// packed maxima and across each group of s columns in registers, and stores 16
// bytes.  Columns that do not fill such a group, windows wider than four and
// tensors whose rows are not 16-byte addressable go through a plain kernel, one
// thread per output.  max is exact, so both paths give the reference's bits.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>

#include "host.h"

namespace nt {
namespace {

struct PoolParams {
    const void *x;
    void *y;
    int n, c, h, w;      // input
    int p, q;            // output
    int r, s;            // window
    int64_t xs[4], ys[4];
};

template <typename T>
struct Num;
template <>
struct Num<__half> {
    static constexpr int kPerVec = 8;
    __device__ static float to_float(__half v) { return __half2float(v); }
    __device__ static __half from_float(float v) { return __float2half_rn(v); }
    __device__ static uint4 vmax(uint4 a, uint4 b) {
        const __half2 *x = reinterpret_cast<const __half2 *>(&a), *y = reinterpret_cast<const __half2 *>(&b);
        uint4 out;
        __half2 *o = reinterpret_cast<__half2 *>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __hmax2(x[i], y[i]);
        return out;
    }
    __device__ static __half smax(__half a, __half b) { return __hmax(a, b); }
};
template <>
struct Num<__nv_bfloat16> {
    static constexpr int kPerVec = 8;
    __device__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
    __device__ static uint4 vmax(uint4 a, uint4 b) {
        const __nv_bfloat162 *x = reinterpret_cast<const __nv_bfloat162 *>(&a),
                             *y = reinterpret_cast<const __nv_bfloat162 *>(&b);
        uint4 out;
        __nv_bfloat162 *o = reinterpret_cast<__nv_bfloat162 *>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __hmax2(x[i], y[i]);
        return out;
    }
    __device__ static __nv_bfloat16 smax(__nv_bfloat16 a, __nv_bfloat16 b) { return __hmax(a, b); }
};
template <>
struct Num<float> {
    static constexpr int kPerVec = 4;
    __device__ static float to_float(float v) { return v; }
    __device__ static float from_float(float v) { return v; }
    __device__ static uint4 vmax(uint4 a, uint4 b) {
        return make_uint4(__float_as_uint(fmaxf(__uint_as_float(a.x), __uint_as_float(b.x))),
                          __float_as_uint(fmaxf(__uint_as_float(a.y), __uint_as_float(b.y))),
                          __float_as_uint(fmaxf(__uint_as_float(a.z), __uint_as_float(b.z))),
                          __float_as_uint(fmaxf(__uint_as_float(a.w), __uint_as_float(b.w))));
    }
    __device__ static float smax(float a, float b) { return fmaxf(a, b); }
};

// Read-only 16-byte load that does allocate in L1: neighbouring threads' vectors are S x 16 bytes
// apart, so one warp instruction uses half of every 32-byte sector it touches and the next instruction
// the other half; with the sector kept in L1 the second half is a hit and L2 is asked once, not twice
// (measured 6.0 -> 6.6 TB/s on 2 x 2 windows).
__device__ __forceinline__ uint4 load_streaming(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// One thread: kPerVec outputs (n, c, p, q0 .. q0 + kPerVec) of ROWS neighbouring output rows, from S
// 16-byte loads per window row.  `groups` such chunks per output row; rows of x are 16-byte addressable.
// R is the window height when it is at most four (all of a thread's loads are then issued before anything
// is reduced), 0 for taller windows (a loop).  Index is the width of the item arithmetic: 32 bits whenever
// the item count allows (a 64-bit division costs more than the loads of a small window).
// store_mode: 0 element by element, 1 one 16-byte store per chunk (output rows 16-byte addressable),
// 2 (ROWS = 1, contiguous output, every output of a row covered by chunks) the warp packs its outputs,
// which are then one contiguous run of the output, into shared memory and stores the run with aligned
// 16-byte vectors: output rows of, say, 37 elements would otherwise be written two bytes at a time.
template <typename T, int R, int S, int ROWS, typename Index>
__global__ void __launch_bounds__(256)
    max_pool2d_vec_kernel(const PoolParams prm, int groups, int row_pairs, Index items, int store_mode) {
    constexpr int E = Num<T>::kPerVec;
    const Index own_item = static_cast<Index>(blockIdx.x) * blockDim.x + threadIdx.x;
    const bool live = own_item < items;
    if (!live && store_mode != 2) return;  // (the packing needs whole warps)
    const Index item = live ? own_item : items - 1;
    const int g = static_cast<int>(item % groups);
    Index rest = item / groups;
    const int p0 = static_cast<int>(rest % row_pairs) * ROWS;
    rest /= row_pairs;
    const int c = static_cast<int>(rest % prm.c);
    const int n = static_cast<int>(rest / prm.c);

    const T *x = static_cast<const T *>(prm.x) + n * prm.xs[0] + c * prm.xs[1] + static_cast<int64_t>(g) * (E * S);
    T *y = static_cast<T *>(prm.y) + n * prm.ys[0] + c * prm.ys[1] + static_cast<int64_t>(g) * E * prm.ys[3];
    // The last chunk of a row may be ragged: vectors past the row end count as -inf (W is a multiple of
    // the vector length here, so a vector is either inside the row or outside it), outputs past Q are
    // not stored.
    const int vectors = min(S, (prm.w - g * (E * S)) / E);
    const int outputs = min(E, prm.q - g * E);
    uint4 minus_inf;
    {
        T *fill = reinterpret_cast<T *>(&minus_inf);
#pragma unroll
        for (int o = 0; o < E; ++o) fill[o] = Num<T>::from_float(-INFINITY);
    }
    uint4 acc[ROWS][S];
    int rows[ROWS];
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
        const int h0 = (p0 + k) * prm.r;
        rows[k] = p0 + k < prm.p ? min(prm.r, prm.h - h0) : 0;  // ceil mode: the last window may hang over the edge
    }
    if constexpr (R > 0) {
        uint4 v[ROWS][R][S];
#pragma unroll
        for (int k = 0; k < ROWS; ++k)
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const uint4 *row = reinterpret_cast<const uint4 *>(x + ((p0 + k) * R + i) * prm.xs[2]);
#pragma unroll
                for (int j = 0; j < S; ++j) v[k][i][j] = i < rows[k] && j < vectors ? load_streaming(row + j) : minus_inf;
            }
#pragma unroll
        for (int k = 0; k < ROWS; ++k)
#pragma unroll
            for (int j = 0; j < S; ++j) {
                acc[k][j] = v[k][0][j];
#pragma unroll
                for (int i = 1; i < R; ++i) acc[k][j] = Num<T>::vmax(acc[k][j], v[k][i][j]);
            }
    } else {
#pragma unroll
        for (int k = 0; k < ROWS; ++k) {
            if (rows[k] > 0) {
                const uint4 *row = reinterpret_cast<const uint4 *>(x + (p0 + k) * prm.r * prm.xs[2]);
#pragma unroll
                for (int j = 0; j < S; ++j) acc[k][j] = j < vectors ? load_streaming(row + j) : minus_inf;
            }
        }
        for (int i = 1; i < prm.r; ++i) {
#pragma unroll
            for (int k = 0; k < ROWS; ++k) {
                if (i < rows[k]) {
                    const uint4 *row = reinterpret_cast<const uint4 *>(x + ((p0 + k) * prm.r + i) * prm.xs[2]);
#pragma unroll
                    for (int j = 0; j < S; ++j)
                        if (j < vectors) acc[k][j] = Num<T>::vmax(acc[k][j], load_streaming(row + j));
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
        if (rows[k] == 0) continue;
        // across each group of S neighbouring columns
        const T *flat = reinterpret_cast<const T *>(acc[k]);
        uint4 packed;
        T *out = reinterpret_cast<T *>(&packed);
#pragma unroll
        for (int o = 0; o < E; ++o) {
            T m = flat[o * S];
#pragma unroll
            for (int j = 1; j < S; ++j) m = Num<T>::smax(m, flat[o * S + j]);
            out[o] = m;
        }
        T *y_row = y + (p0 + k) * prm.ys[2];
        if constexpr (ROWS == 1) {
            if (store_mode == 2) {
                __shared__ __align__(16) T stage[8][32 * E + E];
                const int lane = threadIdx.x & 31;
                T *mine = stage[threadIdx.x >> 5];
                const int count = live ? outputs : 0;
                int before = count;  // inclusive prefix sum over the warp
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, before, d);
                    if (lane >= d) before += up;
                }
                const int total = __shfl_sync(0xffffffffu, before, 31);
                before -= count;
                // the run starts at lane 0's first output; keep its position within a 16-byte vector
                const uint64_t run_address = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(y_row), 0);
                T *run = reinterpret_cast<T *>(run_address);
                const int shift = static_cast<int>((run_address / sizeof(T)) % E);
#pragma unroll
                for (int o = 0; o < E; ++o)
                    if (o < count) mine[shift + before + o] = out[o];
                __syncwarp();
                const int head = min(total, (E - shift) % E);
                const int vectors_out = (total - head) / E;
                const int tail = head + vectors_out * E;
                if (lane < head) run[lane] = mine[shift + lane];
                for (int v = lane; v < vectors_out; v += 32)
                    *reinterpret_cast<uint4 *>(run + head + v * E) = *reinterpret_cast<const uint4 *>(mine + shift + head + v * E);
                if (lane < total - tail) run[tail + lane] = mine[shift + tail + lane];
                continue;
            }
        }
        if (store_mode == 1 && outputs == E) {
            *reinterpret_cast<uint4 *>(y_row) = packed;
        } else {
#pragma unroll
            for (int o = 0; o < E; ++o)
                if (o < outputs) y_row[o * prm.ys[3]] = out[o];
        }
    }
}

// Any strides, any window: one thread per output, columns [q_begin, Q).
template <typename T>
__global__ void __launch_bounds__(256) max_pool2d_plain_kernel(const PoolParams prm, int q_begin, int64_t items) {
    const int64_t item = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (item >= items) return;
    const int cols = prm.q - q_begin;
    const int q = q_begin + static_cast<int>(item % cols);
    int64_t rest = item / cols;
    const int p = static_cast<int>(rest % prm.p);
    rest /= prm.p;
    const int c = static_cast<int>(rest % prm.c);
    const int n = static_cast<int>(rest / prm.c);
    const T *x = static_cast<const T *>(prm.x) + n * prm.xs[0] + c * prm.xs[1];
    float m = -INFINITY;
    for (int i = 0; i < prm.r; ++i) {
        const int h = p * prm.r + i;
        if (h >= prm.h) break;
        for (int j = 0; j < prm.s; ++j) {
            const int w = q * prm.s + j;
            if (w >= prm.w) break;
            m = fmaxf(m, Num<T>::to_float(x[h * prm.xs[2] + w * prm.xs[3]]));
        }
    }
    static_cast<T *>(prm.y)[n * prm.ys[0] + c * prm.ys[1] + p * prm.ys[2] + q * prm.ys[3]] = Num<T>::from_float(m);
}

template <typename T>
int run(cudaStream_t stream, const PoolParams &prm) {
    constexpr int E = Num<T>::kPerVec;
    const int64_t rows_out = static_cast<int64_t>(prm.n) * prm.c * prm.p;
    const bool rows_addressable = prm.xs[3] == 1 && prm.xs[2] % E == 0 && prm.xs[1] % E == 0 && prm.xs[0] % E == 0 &&
                                  aligned16(prm.x);
    int groups = 0;
    if (rows_addressable && prm.s <= 4) {
        // whole chunks only, unless every vector lies inside or outside the row: then the ragged last chunk too
        groups = prm.w % E == 0 ? (prm.q + E - 1) / E : std::min(prm.q / E, prm.w / (E * prm.s));
    }
    if (groups > 0) {
        const bool rows_storable = prm.ys[3] == 1 && prm.ys[2] % E == 0 && prm.ys[1] % E == 0 && prm.ys[0] % E == 0 &&
                                   aligned16(prm.y);
        const bool contiguous_out = prm.ys[3] == 1 && prm.ys[2] == prm.q && prm.ys[1] == static_cast<int64_t>(prm.p) * prm.q &&
                                    prm.ys[0] == static_cast<int64_t>(prm.c) * prm.p * prm.q;
        const bool packed = !rows_storable && contiguous_out && groups * E >= prm.q;
        const int store_mode = rows_storable ? 1 : packed ? 2 : 0;
        const int ROWS = packed ? 1 : 2;  // output rows per thread
        const int row_pairs = (prm.p + ROWS - 1) / ROWS;
        const int64_t items = static_cast<int64_t>(prm.n) * prm.c * row_pairs * groups;
        const unsigned blocks = static_cast<unsigned>((items + 255) / 256);
#define NT_POOL_LAUNCH_RS(R_, S_)                                                                                       \
    if (packed && items < (1ll << 31))                                                                                  \
        max_pool2d_vec_kernel<T, R_, S_, 1, uint32_t><<<blocks, 256, 0, stream>>>(                                     \
            prm, groups, row_pairs, static_cast<uint32_t>(items), store_mode);                                          \
    else if (packed)                                                                                                    \
        max_pool2d_vec_kernel<T, R_, S_, 1, int64_t><<<blocks, 256, 0, stream>>>(prm, groups, row_pairs, items,        \
                                                                                 store_mode);                           \
    else if (items < (1ll << 31))                                                                                       \
        max_pool2d_vec_kernel<T, R_, S_, 2, uint32_t><<<blocks, 256, 0, stream>>>(                                     \
            prm, groups, row_pairs, static_cast<uint32_t>(items), store_mode);                                          \
    else                                                                                                                \
        max_pool2d_vec_kernel<T, R_, S_, 2, int64_t><<<blocks, 256, 0, stream>>>(prm, groups, row_pairs, items,        \
                                                                                 store_mode)
#define NT_POOL_LAUNCH(S_)                                   \
    switch (prm.r) {                                         \
        case 1: NT_POOL_LAUNCH_RS(1, S_); break;             \
        case 2: NT_POOL_LAUNCH_RS(2, S_); break;             \
        case 3: NT_POOL_LAUNCH_RS(3, S_); break;             \
        case 4: NT_POOL_LAUNCH_RS(4, S_); break;             \
        default: NT_POOL_LAUNCH_RS(0, S_); break;            \
    }
        switch (prm.s) {
            case 1: NT_POOL_LAUNCH(1); break;
            case 2: NT_POOL_LAUNCH(2); break;
            case 3: NT_POOL_LAUNCH(3); break;
            default: NT_POOL_LAUNCH(4); break;
        }
#undef NT_POOL_LAUNCH_RS
#undef NT_POOL_LAUNCH
        NT_CUDA_CHECK(cudaGetLastError());
    }
    const int q_begin = std::min(groups * E, prm.q);
    if (q_begin < prm.q) {
        const int64_t items = rows_out * (prm.q - q_begin);
        const unsigned blocks = static_cast<unsigned>((items + 255) / 256);
        max_pool2d_plain_kernel<T><<<blocks, 256, 0, stream>>>(prm, q_begin, items);
        NT_CUDA_CHECK(cudaGetLastError());
    }
    return 0;
}

}  // namespace
}  // namespace nt

extern "C" NineToothedResult launch_max_pool2d(NineToothedStream stream, NineToothedTensor input,
                                               NineToothedTensor output, int window_height, int window_width,
                                               int ceil_mode, int dtype) {
    using namespace nt;
    clear_error();
    if (!input.data || !input.shape || !input.strides || !output.data || !output.shape || !output.strides)
        return fail(NINETOOTHED_B200_ERR_ARGUMENT, "max_pool2d: null tensor field");
    if (dtype != NINETOOTHED_FLOAT16 && dtype != NINETOOTHED_BFLOAT16 && dtype != NINETOOTHED_FLOAT32)
        return fail(NINETOOTHED_B200_ERR_DTYPE, "max_pool2d: dtype %d is not fp16/bf16/fp32", dtype);
    if (window_height < 1 || window_width < 1)
        return fail(NINETOOTHED_B200_ERR_ARGUMENT, "max_pool2d: window %d x %d", window_height, window_width);
    PoolParams prm;
    prm.x = input.data;
    prm.y = output.data;
    for (int i = 0; i < 4; ++i) {
        if (input.shape[i] > 0x7fffffffull || output.shape[i] > 0x7fffffffull)
            return fail(NINETOOTHED_B200_ERR_SHAPE, "max_pool2d: a dimension exceeds 2^31 - 1");
        prm.xs[i] = input.strides[i];
        prm.ys[i] = output.strides[i];
    }
    prm.n = static_cast<int>(input.shape[0]);
    prm.c = static_cast<int>(input.shape[1]);
    prm.h = static_cast<int>(input.shape[2]);
    prm.w = static_cast<int>(input.shape[3]);
    prm.r = window_height;
    prm.s = window_width;
    if (prm.h < prm.r || prm.w < prm.s)
        return fail(NINETOOTHED_B200_ERR_SHAPE, "max_pool2d: the window %d x %d exceeds the input %d x %d", prm.r, prm.s,
                    prm.h, prm.w);
    // tests/test_max_pool2d.py:41-50: floor or ceil of (size - window) / window, plus one
    const auto tiles = [ceil_mode](int size, int window) {
        return (ceil_mode ? (size - window + window - 1) / window : (size - window) / window) + 1;
    };
    prm.p = tiles(prm.h, prm.r);
    prm.q = tiles(prm.w, prm.s);
    if (output.shape[0] != input.shape[0] || output.shape[1] != input.shape[1] ||
        output.shape[2] != static_cast<uint64_t>(prm.p) || output.shape[3] != static_cast<uint64_t>(prm.q))
        return fail(NINETOOTHED_B200_ERR_SHAPE, "max_pool2d: output must be [%d, %d, %d, %d] for this input, window and mode",
                    prm.n, prm.c, prm.p, prm.q);
    if (prm.n == 0 || prm.c == 0) return 0;
    const DeviceState *dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == NINETOOTHED_FLOAT16) return run<__half>(s, prm);
    if (dtype == NINETOOTHED_BFLOAT16) return run<__nv_bfloat16>(s, prm);
    return run<float>(s, prm);
}
