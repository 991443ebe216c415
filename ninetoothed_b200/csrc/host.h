// Host-side plumbing shared by the launchers: error text, argument checks,
// per-device state (status word, SM count, the driver's tensor-map encoder) kept
// in a map guarded by a shared mutex, and TMA descriptor construction.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/ninetoothed_b200.h"

namespace nt {

// Kernel ids recorded in the device status word next to a wait that gave up.
enum KernelId : uint32_t { KID_GEMM = 1, KID_ATTENTION = 2, KID_CONV2D = 3, KID_SELFTEST = 15 };

// printf-style: stores the text for ninetoothed_b200_last_error() and returns `code`.
int fail(int code, const char *fmt, ...);
void clear_error();

// A launch that left the tensor-core path for one of the plain CUDA-core kernels (orders of magnitude slower)
// says so: the text is kept for ninetoothed_b200_last_note() and a process-wide counter is bumped, so that a
// caller can notice the cliff without timing anything.  printf-style.
void note_plain_launch(const char *fmt, ...);

#define NT_CUDA_CHECK(expr)                                                                        \
    do {                                                                                           \
        cudaError_t nt_err_ = (expr);                                                              \
        if (nt_err_ != cudaSuccess) {                                                              \
            return ::nt::fail(static_cast<int>(nt_err_), "%s failed: %s", #expr,                   \
                              cudaGetErrorString(nt_err_));                                        \
        }                                                                                          \
    } while (0)

// What the launchers know about one device.  Created on first use of the device,
// with that device current; lives until the library is unloaded.
struct DeviceState {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0;
    int cc_minor = 0;
    size_t max_smem_optin = 0;
    unsigned int *status = nullptr;  // device address of the status word
    // cuTensorMapEncodeTiled, looked up through the runtime so that the library
    // has no link-time dependency on the driver and loads on a GPU-less host.
    CUresult (*encode_tiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                             const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
};

// Returns 0 and the state of the CURRENT device, or an error code (message set).
int current_device_state(const DeviceState **out);

struct DType {
    int tag;        // NineToothedDataType
    int size;       // bytes per element
};

inline bool is_16bit_float(int dtype) { return dtype == NINETOOTHED_FLOAT16 || dtype == NINETOOTHED_BFLOAT16; }
inline int dtype_size(int dtype) {
    switch (dtype) {
        case NINETOOTHED_FLOAT16:
        case NINETOOTHED_BFLOAT16:
            return 2;
        case NINETOOTHED_FLOAT32:
            return 4;
        default:
            return 0;
    }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Tiled tensor map over a row-major-ish view: dims[0] is the innermost
// (unit-stride) dimension.  strides_bytes[i] is the byte stride of dims[i+1].
// box[i] is the tile extent along dims[i].  128-byte swizzle, zero OOB fill.
int make_tensor_map(const DeviceState &dev, CUtensorMap *map, int dtype, int rank, const void *base,
                    const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box, bool swizzle128);

// gemm.cu: a 1 x 1, unpadded convolution on contiguous NCHW tensors as a batch of GEMMs that share the filter
// matrix (channels and pixels per image multiples of 8).
int conv1x1_as_gemm(cudaStream_t stream, const DeviceState &dev, int dtype, const void *x, const void *w, void *y,
                    int images, int channels, int pixels, int filters);

// ... and on dense channels-last tensors as one GEMM over all pixels (channels and filters multiples of 8).
int conv1x1_channels_last_as_gemm(cudaStream_t stream, const DeviceState &dev, int dtype, const void *x, const void *w,
                                  void *y, int64_t pixels, int channels, int filters);

// Host scalars of 0-dim tensors.
inline double scalar_f64(const NineToothedTensor &t) { return *static_cast<const double *>(t.data); }
inline int64_t scalar_i64(const NineToothedTensor &t) { return *static_cast<const int64_t *>(t.data); }

}  // namespace nt
