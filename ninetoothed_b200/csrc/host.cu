// Per-device state, error text and TMA descriptor construction.
#include "host.h"
#include "ptx.cuh"

#include <atomic>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <unordered_map>

namespace nt {

// One status word per device that loads this library (a __device__ variable is
// instantiated on every device).  Kernels receive its device address.
__device__ unsigned int g_device_status;

namespace {

thread_local std::string t_last_error;
thread_local std::string t_last_note;
std::atomic<long long> g_plain_launches{0};

// Lazily filled device table.  Readers take the shared lock; the first use of a
// device takes the unique lock and re-checks, the pattern the reference uses for
// its per-context kernel table (src/ninetoothed/templates/thread_safe_unordered_map.h:8-36).
std::shared_mutex g_devices_mutex;
std::unordered_map<int, DeviceState> g_devices;

int init_device_state(int device, DeviceState *state) {
    state->device = device;
    NT_CUDA_CHECK(cudaDeviceGetAttribute(&state->sm_count, cudaDevAttrMultiProcessorCount, device));
    NT_CUDA_CHECK(cudaDeviceGetAttribute(&state->cc_major, cudaDevAttrComputeCapabilityMajor, device));
    NT_CUDA_CHECK(cudaDeviceGetAttribute(&state->cc_minor, cudaDevAttrComputeCapabilityMinor, device));
    int smem = 0;
    NT_CUDA_CHECK(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
    state->max_smem_optin = static_cast<size_t>(smem);
    if (state->cc_major != 10) {
        return fail(NINETOOTHED_B200_ERR_DEVICE, "device %d is sm_%d%d; this library holds sm_100a code only", device,
                    state->cc_major, state->cc_minor);
    }
    void *status = nullptr;
    NT_CUDA_CHECK(cudaGetSymbolAddress(&status, g_device_status));
    state->status = static_cast<unsigned int *>(status);
    NT_CUDA_CHECK(cudaMemset(state->status, 0, sizeof(unsigned int)));

    void *fn = nullptr;
    cudaDriverEntryPointQueryResult query = cudaDriverEntryPointSymbolNotFound;
    NT_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query));
    if (query != cudaDriverEntryPointSuccess || fn == nullptr) {
        return fail(NINETOOTHED_B200_ERR_DEVICE, "the driver does not export cuTensorMapEncodeTiled");
    }
    state->encode_tiled = reinterpret_cast<decltype(state->encode_tiled)>(fn);
    return 0;
}

}  // namespace

int fail(int code, const char *fmt, ...) {
    char buffer[512];
    va_list args;
    va_start(args, fmt);
    vsnprintf(buffer, sizeof(buffer), fmt, args);
    va_end(args);
    t_last_error = buffer;
    return code;
}

void clear_error() { t_last_error.clear(); }

void note_plain_launch(const char *fmt, ...) {
    char buffer[512];
    va_list args;
    va_start(args, fmt);
    vsnprintf(buffer, sizeof(buffer), fmt, args);
    va_end(args);
    t_last_note = buffer;
    g_plain_launches.fetch_add(1, std::memory_order_relaxed);
}

int current_device_state(const DeviceState **out) {
    int device = 0;
    NT_CUDA_CHECK(cudaGetDevice(&device));
    {
        std::shared_lock<std::shared_mutex> lock(g_devices_mutex);
        auto it = g_devices.find(device);
        if (it != g_devices.end()) {
            *out = &it->second;
            return 0;
        }
    }
    std::unique_lock<std::shared_mutex> lock(g_devices_mutex);
    auto it = g_devices.find(device);
    if (it == g_devices.end()) {
        DeviceState state;
        int rc = init_device_state(device, &state);
        if (rc != 0) return rc;
        it = g_devices.emplace(device, state).first;
    }
    *out = &it->second;
    return 0;
}

int make_tensor_map(const DeviceState &dev, CUtensorMap *map, int dtype, int rank, const void *base,
                    const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box, bool swizzle128) {
    CUtensorMapDataType type;
    switch (dtype) {
        case NINETOOTHED_FLOAT16:
            type = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
            break;
        case NINETOOTHED_BFLOAT16:
            type = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
            break;
        case NINETOOTHED_FLOAT32:
            type = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
            break;
        case NINETOOTHED_UINT8:  // 8-bit floating point travels as bytes
            type = CU_TENSOR_MAP_DATA_TYPE_UINT8;
            break;
        default:
            return fail(NINETOOTHED_B200_ERR_DTYPE, "no tensor-map data type for dtype %d", dtype);
    }
    cuuint64_t gdims[5];
    cuuint64_t gstrides[4];
    cuuint32_t gbox[5];
    cuuint32_t elem_strides[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        elem_strides[i] = 1;
        if (i + 1 < rank) gstrides[i] = strides_bytes[i];
    }
    CUresult rc = dev.encode_tiled(map, type, static_cast<cuuint32_t>(rank), const_cast<void *>(base), gdims, gstrides,
                                   gbox, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        return fail(NINETOOTHED_B200_ERR_LAYOUT,
                    "cuTensorMapEncodeTiled rejected the operand (CUresult %d): rank %d base %p dims [%llu %llu %llu "
                    "%llu] box [%u %u %u %u]",
                    static_cast<int>(rc), rank, base, (unsigned long long)gdims[0],
                    (unsigned long long)(rank > 1 ? gdims[1] : 0), (unsigned long long)(rank > 2 ? gdims[2] : 0),
                    (unsigned long long)(rank > 3 ? gdims[3] : 0), gbox[0], rank > 1 ? gbox[1] : 0,
                    rank > 2 ? gbox[2] : 0, rank > 3 ? gbox[3] : 0);
    }
    return 0;
}

// A bounded wait that is made to run out: one warp waits on an mbarrier nobody arrives at, with the given
// limit; the wait gives up, records its code in the device status word and the kernel returns normally.
__global__ void selftest_wait_kernel(unsigned int *status, unsigned long long limit_ns) {
    __shared__ uint64_t barrier;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&barrier, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    const WaitCtx ctx{&abort_flag, status, KID_SELFTEST};
    if (threadIdx.x == 0) mbar_wait_limited(&barrier, 0, ctx, 0x5e1f, limit_ns);
    __syncthreads();
}

}  // namespace nt

extern "C" {

const char *ninetoothed_b200_last_error(void) { return nt::t_last_error.c_str(); }

NineToothedResult ninetoothed_b200_device_status(unsigned int *status, int clear) {
    if (status == nullptr) return nt::fail(NINETOOTHED_B200_ERR_ARGUMENT, "status pointer is null");
    const nt::DeviceState *dev = nullptr;
    int rc = nt::current_device_state(&dev);
    if (rc != 0) return rc;
    NT_CUDA_CHECK(cudaDeviceSynchronize());
    NT_CUDA_CHECK(cudaMemcpy(status, dev->status, sizeof(unsigned int), cudaMemcpyDeviceToHost));
    if (clear && *status != 0) NT_CUDA_CHECK(cudaMemset(dev->status, 0, sizeof(unsigned int)));
    if ((*status & nt::STATUS_WAIT_TIMEOUT) != 0)
        return nt::fail(NINETOOTHED_B200_ERR_TIMEOUT,
                        "a bounded device-side wait gave up: status 0x%08x (kernel id %u, wait code 0x%04x)", *status,
                        (*status >> 16) & 0xfffu, *status & 0xffffu);
    return 0;
}

const char *ninetoothed_b200_last_note(void) { return nt::t_last_note.c_str(); }

long long ninetoothed_b200_plain_launches(int reset) {
    return reset ? nt::g_plain_launches.exchange(0) : nt::g_plain_launches.load(std::memory_order_relaxed);
}

NineToothedResult ninetoothed_b200_selftest_wait_timeout(NineToothedStream stream, unsigned long long limit_ns) {
    nt::clear_error();
    if (limit_ns == 0 || limit_ns > 1000000000ull)
        return nt::fail(NINETOOTHED_B200_ERR_ARGUMENT, "selftest: the limit must be between 1 ns and 1 s");
    const nt::DeviceState *dev = nullptr;
    if (int rc = nt::current_device_state(&dev)) return rc;
    nt::selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(dev->status, limit_ns);
    NT_CUDA_CHECK(cudaGetLastError());
    return 0;
}

int ninetoothed_b200_version(void) { return 100; }

}  // extern "C"
