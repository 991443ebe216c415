// Placeholder until the tcgen05 attention kernel lands: rejects every call.
#include "host.h"

extern "C" NineToothedResult launch_attention(NineToothedStream, NineToothedTensor, NineToothedTensor,
                                              NineToothedTensor, NineToothedTensor, NineToothedTensor, int) {
    return nt::fail(NINETOOTHED_B200_ERR_DEVICE, "attention: kernel not present in this build");
}
extern "C" NineToothedResult launch_attention_scaled(NineToothedStream, NineToothedTensor, NineToothedTensor,
                                                     NineToothedTensor, NineToothedTensor, NineToothedTensor,
                                                     NineToothedTensor, int) {
    return nt::fail(NINETOOTHED_B200_ERR_DEVICE, "attention: kernel not present in this build");
}
