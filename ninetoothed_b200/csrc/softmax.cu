// Row softmax: one program per row, the whole row held in registers, fp32 math
// (the kernel of tests/test_softmax.py:10-27 in the reference project).
//
// Bandwidth-bound: every element is read once and written once.  The fast path
// moves 16-byte vectors (8 fp16 / 4 fp32), coalesced across the threads that
// share a row, reduces max and sum with warp shuffles plus one shared-memory hop
// per reduction, and evaluates one ex2 per element.  No tensor cores.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "host.h"

namespace nt {
namespace {

constexpr float kLog2e = 1.4426950408889634f;

template <typename T>
struct Elem;
template <>
struct Elem<__half> {
    static constexpr int kPerVec = 8;
    __device__ static void unpack(const uint4 &v, float (&f)[8]) {
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 p = __half22float2(h[i]);
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
    __device__ static uint4 pack(const float (&f)[8]) {
        uint4 v;
        __half2 *h = reinterpret_cast<__half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        return v;
    }
    __device__ static float load(const __half *p) { return __half2float(*p); }
    __device__ static void store(__half *p, float x) { *p = __float2half_rn(x); }
};
template <>
struct Elem<__nv_bfloat16> {
    static constexpr int kPerVec = 8;
    __device__ static void unpack(const uint4 &v, float (&f)[8]) {
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 p = __bfloat1622float2(h[i]);
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
    __device__ static uint4 pack(const float (&f)[8]) {
        uint4 v;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        return v;
    }
    __device__ static float load(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
    __device__ static void store(__nv_bfloat16 *p, float x) { *p = __float2bfloat16_rn(x); }
};
template <>
struct Elem<float> {
    static constexpr int kPerVec = 4;
    __device__ static void unpack(const uint4 &v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
    __device__ static uint4 pack(const float (&f)[4]) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
    __device__ static float load(const float *p) { return *p; }
    __device__ static void store(float *p, float x) { *p = x; }
};

__device__ __forceinline__ uint4 load_streaming(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void store_streaming(uint4 *p, const uint4 &v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool IS_MAX>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        float other = __shfl_xor_sync(0xffffffffu, v, offset);
        v = IS_MAX ? fmaxf(v, other) : v + other;
    }
    return v;
}

// Reduction over the ROW_THREADS threads (threadIdx.x) that share a row; rows of
// one CTA are indexed by threadIdx.y.  `scratch` holds ROWS * WARPS floats.
template <bool IS_MAX, int ROW_THREADS>
__device__ __forceinline__ float row_reduce(float v, float *scratch) {
    v = warp_reduce<IS_MAX>(v);
    if constexpr (ROW_THREADS > 32) {
        constexpr int WARPS = ROW_THREADS / 32;
        float *mine = scratch + threadIdx.y * WARPS;
        if ((threadIdx.x & 31) == 0) mine[threadIdx.x >> 5] = v;
        __syncthreads();
        v = mine[0];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) v = IS_MAX ? fmaxf(v, mine[w]) : v + mine[w];
    }
    return v;
}

// Fast path.  Requirements checked by the launcher: unit inner stride, cols a
// multiple of the vector width, 16-byte aligned rows, cols <= ROW_THREADS*VECS*E.
template <typename T, int ROW_THREADS, int VECS, int ROWS>
__global__ void __launch_bounds__(ROW_THREADS *ROWS)
    softmax_rows_kernel(const T *__restrict__ x, T *__restrict__ y, int rows, int cols, int64_t x_stride,
                        int64_t y_stride) {
    constexpr int E = Elem<T>::kPerVec;
    constexpr int WARPS = ROW_THREADS > 32 ? ROW_THREADS / 32 : 1;
    __shared__ float scratch_max[ROWS * WARPS];
    __shared__ float scratch_sum[ROWS * WARPS];

    const int64_t row_raw = static_cast<int64_t>(blockIdx.x) * ROWS + threadIdx.y;
    const bool row_valid = row_raw < rows;
    const int64_t row = row_valid ? row_raw : rows - 1;
    const int nvec = cols / E;
    const uint4 *xin = reinterpret_cast<const uint4 *>(x + row * x_stride);

    uint4 raw[VECS];
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
        const int v = threadIdx.x + i * ROW_THREADS;
        if (v < nvec) raw[i] = load_streaming(xin + v);
    }

    float vals[VECS][E];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
        const int v = threadIdx.x + i * ROW_THREADS;
        if (v < nvec) {
            Elem<T>::unpack(raw[i], vals[i]);
#pragma unroll
            for (int e = 0; e < E; ++e) m = fmaxf(m, vals[i][e]);
        }
    }
    m = row_reduce<true, ROW_THREADS>(m, scratch_max);

    // exp(x - m) = 2^(x*log2e - m*log2e): one FMA and one ex2 per element.
    const float neg_m_scaled = -m * kLog2e;
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
        const int v = threadIdx.x + i * ROW_THREADS;
        if (v < nvec) {
#pragma unroll
            for (int e = 0; e < E; ++e) {
                vals[i][e] = ex2(fmaf(vals[i][e], kLog2e, neg_m_scaled));
                sum += vals[i][e];
            }
        }
    }
    sum = row_reduce<false, ROW_THREADS>(sum, scratch_sum);
    const float inv = 1.0f / sum;

    if (row_valid) {
        uint4 *yout = reinterpret_cast<uint4 *>(y + row * y_stride);
#pragma unroll
        for (int i = 0; i < VECS; ++i) {
            const int v = threadIdx.x + i * ROW_THREADS;
            if (v < nvec) {
#pragma unroll
                for (int e = 0; e < E; ++e) vals[i][e] *= inv;
                store_streaming(yout + v, Elem<T>::pack(vals[i]));
            }
        }
    }
}

// Any shape, any strides: one CTA per row, three strided passes (the row stays
// in L2 between them).  Lanes past the row end do not exist here, which equals
// the reference's -inf padding (exp(-inf) = 0).
template <typename T>
__global__ void __launch_bounds__(256)
    softmax_rows_generic_kernel(const T *__restrict__ x, T *__restrict__ y, int cols, int64_t x_row_stride,
                                int64_t x_col_stride, int64_t y_row_stride, int64_t y_col_stride) {
    __shared__ float scratch_max[8];
    __shared__ float scratch_sum[8];
    const T *xin = x + static_cast<int64_t>(blockIdx.x) * x_row_stride;
    T *yout = y + static_cast<int64_t>(blockIdx.x) * y_row_stride;
    float m = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += 256) m = fmaxf(m, Elem<T>::load(xin + c * x_col_stride));
    m = row_reduce<true, 256>(m, scratch_max);
    const float neg_m_scaled = -m * kLog2e;
    float sum = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256)
        sum += ex2(fmaf(Elem<T>::load(xin + c * x_col_stride), kLog2e, neg_m_scaled));
    sum = row_reduce<false, 256>(sum, scratch_sum);
    const float inv = 1.0f / sum;
    for (int c = threadIdx.x; c < cols; c += 256)
        Elem<T>::store(yout + c * y_col_stride, ex2(fmaf(Elem<T>::load(xin + c * x_col_stride), kLog2e, neg_m_scaled)) * inv);
}

// Long rows, and rows that are not 16-byte addressable as a whole (a column count that is not a
// multiple of the vector length: every row then starts at another offset within a 16-byte vector): one
// CTA per row, the row staged once in shared memory.  The row's unaligned head and tail (fewer than a
// vector each) move element by element, everything between as 16-byte vectors, both from global memory
// and, shifted so that the same vectors are aligned there too, in shared memory.  Global traffic is one
// read and one write of the row, as in the register kernel; the exponential is computed twice (once for
// the sum, once for the result), which the exp unit can afford at HBM rate.
constexpr int SMEM_ROW_THREADS = 512;

template <typename T>
__global__ void __launch_bounds__(SMEM_ROW_THREADS)
    softmax_rows_smem_kernel(const T *__restrict__ x, T *__restrict__ y, int cols, int64_t x_stride, int64_t y_stride) {
    constexpr int E = Elem<T>::kPerVec;
    constexpr int WARPS = SMEM_ROW_THREADS / 32;
    extern __shared__ __align__(16) uint8_t row_bytes[];
    __shared__ float scratch_max[WARPS];
    __shared__ float scratch_sum[WARPS];
    const T *xin = x + static_cast<int64_t>(blockIdx.x) * x_stride;
    T *yout = y + static_cast<int64_t>(blockIdx.x) * y_stride;
    // elements before the first 16-byte boundary of the row, in global memory
    const int head = min(cols, static_cast<int>(((16u - (reinterpret_cast<uintptr_t>(xin) & 15u)) & 15u) / sizeof(T)));
    const int head_out = min(cols, static_cast<int>(((16u - (reinterpret_cast<uintptr_t>(yout) & 15u)) & 15u) / sizeof(T)));
    const int nvec = (cols - head) / E;
    const int tail_begin = head + nvec * E;
    // element i sits at staged[i]: shifted so that element `head` is 16-byte aligned in shared memory
    T *staged = reinterpret_cast<T *>(row_bytes) + (E - head % E) % E;
    const int tid = threadIdx.x;

    float m = -INFINITY;
    for (int i = tid; i < head; i += SMEM_ROW_THREADS) {
        const T v = xin[i];
        staged[i] = v;
        m = fmaxf(m, Elem<T>::load(&v));
    }
    for (int i = tail_begin + tid; i < cols; i += SMEM_ROW_THREADS) {
        const T v = xin[i];
        staged[i] = v;
        m = fmaxf(m, Elem<T>::load(&v));
    }
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(xin + head);
        uint4 *dst = reinterpret_cast<uint4 *>(staged + head);
        for (int v = tid; v < nvec; v += SMEM_ROW_THREADS) {
            const uint4 raw = load_streaming(src + v);
            dst[v] = raw;
            float f[E];
            Elem<T>::unpack(raw, f);
#pragma unroll
            for (int e = 0; e < E; ++e) m = fmaxf(m, f[e]);
        }
    }
    m = row_reduce<true, SMEM_ROW_THREADS>(m, scratch_max);  // (its barrier also publishes the staged row)

    const float neg_m_scaled = -m * kLog2e;
    float sum = 0.f;
    for (int i = tid; i < head; i += SMEM_ROW_THREADS) sum += ex2(fmaf(Elem<T>::load(staged + i), kLog2e, neg_m_scaled));
    for (int i = tail_begin + tid; i < cols; i += SMEM_ROW_THREADS)
        sum += ex2(fmaf(Elem<T>::load(staged + i), kLog2e, neg_m_scaled));
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(staged + head);
        for (int v = tid; v < nvec; v += SMEM_ROW_THREADS) {
            float f[E];
            Elem<T>::unpack(src[v], f);
#pragma unroll
            for (int e = 0; e < E; ++e) sum += ex2(fmaf(f[e], kLog2e, neg_m_scaled));
        }
    }
    sum = row_reduce<false, SMEM_ROW_THREADS>(sum, scratch_sum);
    const float inv = 1.0f / sum;

    if (head_out == head) {
        // the output row has the same position within a vector: the same split serves it
        for (int i = tid; i < head; i += SMEM_ROW_THREADS)
            Elem<T>::store(yout + i, ex2(fmaf(Elem<T>::load(staged + i), kLog2e, neg_m_scaled)) * inv);
        for (int i = tail_begin + tid; i < cols; i += SMEM_ROW_THREADS)
            Elem<T>::store(yout + i, ex2(fmaf(Elem<T>::load(staged + i), kLog2e, neg_m_scaled)) * inv);
        const uint4 *src = reinterpret_cast<const uint4 *>(staged + head);
        uint4 *dst = reinterpret_cast<uint4 *>(yout + head);
        for (int v = tid; v < nvec; v += SMEM_ROW_THREADS) {
            float f[E];
            Elem<T>::unpack(src[v], f);
#pragma unroll
            for (int e = 0; e < E; ++e) f[e] = ex2(fmaf(f[e], kLog2e, neg_m_scaled)) * inv;
            store_streaming(dst + v, Elem<T>::pack(f));
        }
    } else {
        for (int i = tid; i < cols; i += SMEM_ROW_THREADS)
            Elem<T>::store(yout + i, ex2(fmaf(Elem<T>::load(staged + i), kLog2e, neg_m_scaled)) * inv);
    }
}

template <typename T, int ROW_THREADS, int VECS>
void launch_rows(cudaStream_t stream, const T *x, T *y, int rows, int cols, int64_t xs, int64_t ys) {
    constexpr int ROWS = ROW_THREADS >= 128 ? 1 : 128 / ROW_THREADS;
    dim3 block(ROW_THREADS, ROWS);
    dim3 grid(static_cast<unsigned>((static_cast<int64_t>(rows) + ROWS - 1) / ROWS));
    softmax_rows_kernel<T, ROW_THREADS, VECS, ROWS><<<grid, block, 0, stream>>>(x, y, rows, cols, xs, ys);
}

// Picks threads-per-row and vectors-per-thread so that the row just fits.
// `prefer_vecs` (4 or 8) trades registers per thread against threads per row.
template <typename T>
bool launch_fast(cudaStream_t stream, const T *x, T *y, int rows, int cols, int64_t xs, int64_t ys,
                 int prefer_vecs) {
    constexpr int E = Elem<T>::kPerVec;
    const int nvec = cols / E;
#define NT_TRY(RT, V)                                             \
    if (nvec <= (RT) * (V)) {                                     \
        launch_rows<T, RT, V>(stream, x, y, rows, cols, xs, ys);  \
        return true;                                              \
    }
    NT_TRY(32, 1)
    NT_TRY(32, 2)
    NT_TRY(32, 4)
    NT_TRY(64, 4)
    NT_TRY(128, 4)
    if (prefer_vecs >= 8) {
        NT_TRY(128, 8)
        NT_TRY(256, 8)
    }
    NT_TRY(256, 4)
    NT_TRY(512, 4)
    NT_TRY(512, 8)
    NT_TRY(1024, 8)
#undef NT_TRY
    return false;
}

template <typename T>
int run(cudaStream_t stream, const NineToothedTensor &in, const NineToothedTensor &out) {
    const int64_t rows = static_cast<int64_t>(in.shape[0]);
    const int64_t cols = static_cast<int64_t>(in.shape[1]);
    if (rows == 0 || cols == 0) return 0;
    if (rows > 0x7fffffffLL || cols > 0x7fffffffLL)
        return fail(NINETOOTHED_B200_ERR_SHAPE, "softmax: %lld x %lld exceeds 32-bit indexing", (long long)rows,
                    (long long)cols);
    const T *x = static_cast<const T *>(in.data);
    T *y = static_cast<T *>(out.data);
    constexpr int E = Elem<T>::kPerVec;
    const bool vectorizable = in.strides[1] == 1 && out.strides[1] == 1 && cols % E == 0 &&
                              in.strides[0] % E == 0 && out.strides[0] % E == 0 && aligned16(x) && aligned16(y);
    static const int prefer_vecs = [] {
        const char *env = std::getenv("NINETOOTHED_B200_SOFTMAX_VECS");
        return env ? std::atoi(env) : 8;
    }();
    // long rows and rows that are not 16-byte addressable as a whole: staged in shared memory
    const size_t staged_bytes = (static_cast<size_t>(cols) + E) * sizeof(T);
    const bool unit_inner = in.strides[1] == 1 && out.strides[1] == 1;
    constexpr size_t kMaxStagedBytes = 200 * 1024;
    // (16-byte addressable rows stay on the register kernel unless at least two staged rows fit an SM)
    if (unit_inner && staged_bytes <= kMaxStagedBytes &&
        (!vectorizable || (cols > 16384 && staged_bytes <= 110 * 1024))) {
        static thread_local int configured_device = -1;
        int device = -1;
        NT_CUDA_CHECK(cudaGetDevice(&device));
        if (configured_device != device) {
            NT_CUDA_CHECK(cudaFuncSetAttribute(softmax_rows_smem_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(kMaxStagedBytes)));
            configured_device = device;
        }
        softmax_rows_smem_kernel<T><<<static_cast<unsigned>(rows), SMEM_ROW_THREADS, staged_bytes, stream>>>(
            x, y, static_cast<int>(cols), in.strides[0], out.strides[0]);
        NT_CUDA_CHECK(cudaGetLastError());
        return 0;
    }
    if (!(vectorizable && launch_fast<T>(stream, x, y, static_cast<int>(rows), static_cast<int>(cols),
                                         in.strides[0], out.strides[0], prefer_vecs))) {
        softmax_rows_generic_kernel<T><<<static_cast<unsigned>(rows), 256, 0, stream>>>(
            x, y, static_cast<int>(cols), in.strides[0], in.strides[1], out.strides[0], out.strides[1]);
    }
    NT_CUDA_CHECK(cudaGetLastError());
    return 0;
}

}  // namespace
}  // namespace nt

extern "C" NineToothedResult launch_softmax(NineToothedStream stream, NineToothedTensor input,
                                            NineToothedTensor output, int dtype) {
    using namespace nt;
    clear_error();
    if (!input.data || !output.data || !input.shape || !output.shape || !input.strides || !output.strides)
        return fail(NINETOOTHED_B200_ERR_ARGUMENT, "softmax: null tensor field");
    if (input.shape[0] != output.shape[0] || input.shape[1] != output.shape[1])
        return fail(NINETOOTHED_B200_ERR_SHAPE, "softmax: input is %llu x %llu but output is %llu x %llu",
                    (unsigned long long)input.shape[0], (unsigned long long)input.shape[1],
                    (unsigned long long)output.shape[0], (unsigned long long)output.shape[1]);
    const DeviceState *dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case NINETOOTHED_FLOAT16:
            return run<__half>(s, input, output);
        case NINETOOTHED_BFLOAT16:
            return run<__nv_bfloat16>(s, input, output);
        case NINETOOTHED_FLOAT32:
            return run<float>(s, input, output);
        default:
            return fail(NINETOOTHED_B200_ERR_DTYPE, "softmax: dtype %d is not fp16/bf16/fp32", dtype);
    }
}
