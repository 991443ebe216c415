// Placeholder until the implicit-GEMM conv2d kernel lands: rejects every call.
#include "host.h"

extern "C" NineToothedResult launch_conv2d(NineToothedStream, NineToothedTensor, NineToothedTensor, NineToothedTensor,
                                           int, int, int, void *, size_t) {
    return nt::fail(NINETOOTHED_B200_ERR_DEVICE, "conv2d: kernel not present in this build");
}
extern "C" size_t launch_conv2d_workspace_size(NineToothedTensor, NineToothedTensor, int) { return 0; }
