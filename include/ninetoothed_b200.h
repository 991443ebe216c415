/*
 * C ABI of the B200 (sm_100a) kernels that stand in for the kernels NineToothed
 * generates for matmul, addmm, row softmax, fused attention, conv2d and max_pool2d.
 *
 * The types and the calling convention are those of the header the reference
 * writes for its ahead-of-time ("cuda" caller) path, ninetoothed.h
 * (src/ninetoothed/aot.py:558-586 in the reference project):
 *   - tensors are passed BY VALUE as {data, shape, strides}; shape and strides are
 *     caller-owned arrays of element counts / element strides that are only read
 *     during the call (src/ninetoothed/aot.py:711-723);
 *   - a 0-dim tensor is a run-time scalar: `data` points to a HOST double (float
 *     scalars) or a HOST int64_t (integer / boolean scalars) and shape/strides
 *     are empty (src/ninetoothed/aot.py:725-733, 845-848);
 *   - the first parameter is the stream the kernel is enqueued on; the call
 *     returns without synchronising;
 *   - the result is 0 on success (src/ninetoothed/aot.py:859-860).  Non-zero is
 *     either a positive CUDA error code or one of the negative
 *     NINETOOTHED_B200_ERR_* codes below.  Nothing in this library calls exit().
 *   - trailing plain `int` parameters carry compile-time choices (data type,
 *     padding), the way the reference's build() appends them
 *     (src/ninetoothed/build.py:132-142, 162-170).
 *
 * Entry points are named launch_<kernel_name>, the name the reference gives the
 * launcher of a kernel (src/ninetoothed/aot.py:127-147); the kernel names are the
 * ones its AOT tests use (tests/test_aot.py:87, 147, 190, 259).
 */
#ifndef NINETOOTHED_B200_H
#define NINETOOTHED_B200_H

#include <stddef.h>
#include <stdint.h>

#define NINETOOTHED_TRUE 1
#define NINETOOTHED_FALSE 0
#define NINETOOTHED_NONE 0

/* Same order as the reference's enum (src/ninetoothed/aot.py:524-537). */
enum NineToothedDataType {
    NINETOOTHED_INT8,
    NINETOOTHED_INT16,
    NINETOOTHED_INT32,
    NINETOOTHED_INT64,
    NINETOOTHED_UINT8,
    NINETOOTHED_UINT16,
    NINETOOTHED_UINT32,
    NINETOOTHED_UINT64,
    NINETOOTHED_FLOAT16,
    NINETOOTHED_BFLOAT16,
    NINETOOTHED_FLOAT32,
    NINETOOTHED_FLOAT64
};

/*
 * Not in the reference's enum, which its ahead-of-time path is limited to: 8-bit e5m2 floating point,
 * which the reference's torch caller accepts for matmul (tests/test_matmul.py:60-90).
 */
#define NINETOOTHED_B200_FLOAT8_E5M2 100

typedef struct {
    void *data;
    uint64_t *shape;
    int64_t *strides;
} NineToothedTensor;

typedef void *NineToothedStream;

typedef int NineToothedResult;

/* Negative results: the call was rejected before anything was enqueued. */
#define NINETOOTHED_B200_ERR_DTYPE (-1)     /* data type not supported by this kernel        */
#define NINETOOTHED_B200_ERR_SHAPE (-2)     /* shapes of the arguments do not agree          */
#define NINETOOTHED_B200_ERR_LAYOUT (-3)    /* strides/alignment this kernel cannot address  */
#define NINETOOTHED_B200_ERR_ARGUMENT (-4)  /* null pointer, bad scalar, bad workspace size  */
#define NINETOOTHED_B200_ERR_DEVICE (-5)    /* not an sm_100 device, or driver entry missing */
#define NINETOOTHED_B200_ERR_TIMEOUT (-6)   /* a bounded device-side wait gave up            */

#ifdef __cplusplus
extern "C" {
#endif

/*
 * output[M,N] = lhs[M,K] . rhs[K,N], fp32 accumulate, one rounding at the store.
 * Replaces the kernel of README.md:40-67 / tests/test_matmul.py:14-45 and its
 * launcher launch_matmul (tests/test_aot.py:190).  dtype: FLOAT16, BFLOAT16, or
 * NINETOOTHED_B200_FLOAT8_E5M2 for e5m2 operands with an fp16 output
 * (tests/test_matmul.py:60-90; the tensor-core path wants rhs as a transposed view).
 * Any strides are accepted; operands that no TMA descriptor can address (no
 * unit-stride dimension, rows not 16-byte aligned) run on a slower plain kernel.
 *
 * Device memory: none, with one exception.  A problem with fewer output tiles
 * than the device has SMs and a long reduction (launch_matmul and launch_addmm
 * alike) is split along K; the partial accumulators live in a scratch array of
 * 2 x SM count x 128 KiB (38 MB on a B200), one per (device, stream handle), at
 * most 8 per device, kept until the process exits.  Rules:
 *   - the array comes from ninetoothed_b200_reserve_split_scratch(stream), or, if
 *     that was not called, from cudaMalloc inside the first split launch on the
 *     stream, which SYNCHRONISES THE DEVICE once; with
 *     NINETOOTHED_B200_GEMM_SPLIT_ALLOC=0 in the environment launches never allocate
 *     and only reserved streams split;
 *   - a launch that has no array and cannot get one (the stream is being captured
 *     into a graph, a ninth stream, no memory, or the handle is cudaStreamPerThread,
 *     which names a different stream in every host thread) runs unsplit: slower, and
 *     equal to the split result within rounding only (the fp32 partial sums are
 *     added in another order), so bit-for-bit reproducibility across streams needs
 *     either reserved scratch everywhere or NINETOOTHED_B200_GEMM_SPLIT=0;
 *   - the array is keyed by the stream HANDLE: launches that share a handle share it
 *     and are ordered by the stream; a graph captured on a stream and replayed on
 *     another still uses the capture stream's array, so do not run it concurrently
 *     with eager split launches on the capture stream.
 * NINETOOTHED_B200_GEMM_SPLIT=0 turns the split off altogether.
 */
NineToothedResult launch_matmul(NineToothedStream stream, NineToothedTensor lhs, NineToothedTensor rhs,
                                NineToothedTensor output, int dtype);

/*
 * A batch of matmuls on 3-D operands: output[b] = lhs[b] . rhs[b] with lhs [B,M,K], rhs [B,K,N],
 * output [B,M,N], fp32 accumulate, one rounding at the store (the matmul kernel under a leading
 * batch dimension: the operand shapes docs/source/build.rst:237-245 names for a batched matmul;
 * the reference's test-suite has no definition of it, examples/definitions.py holds the
 * arrangement).  dtype: FLOAT16 or BFLOAT16.  Row-major operands with 16-byte aligned rows and
 * batch strides run as one launch; any other strides as one matmul launch per problem.
 */
NineToothedResult launch_bmm(NineToothedStream stream, NineToothedTensor lhs, NineToothedTensor rhs,
                             NineToothedTensor output, int dtype);

/*
 * output = beta * input + alpha * round_to_dtype(mat1 . mat2); the epilogue is
 * evaluated in the storage data type with a rounding after every operation,
 * as the generated kernel does.  beta and alpha are 0-dim tensors (host double).
 * Replaces tests/test_addmm.py:13-38 and launch_addmm (tests/test_aot.py:87),
 * argument order (input, mat1, mat2, beta, alpha, output) as at
 * tests/test_addmm.py:52.
 */
NineToothedResult launch_addmm(NineToothedStream stream, NineToothedTensor input, NineToothedTensor mat1,
                               NineToothedTensor mat2, NineToothedTensor beta, NineToothedTensor alpha,
                               NineToothedTensor output, int dtype);

/*
 * addmm for one rank of an N-column split, with the all-gather of the column slabs
 * fused into the epilogue.  (No counterpart in the reference, which has no multi-GPU
 * path; this is the "N split across GPUs with column blocks all-gathered" step of the
 * benchmark configuration done as one kernel.)
 *
 * Every rank r of `world` GPUs holds a full [M, world * N_local] buffer whose memory
 * the other ranks can address (peer-mapped / symmetric memory); `peer_outputs[i]` is
 * rank i's buffer as seen from THIS process and `peer_outputs[rank]` is this rank's
 * own.  `output` is this rank's slab view of its own buffer, [M, N_local] starting at
 * column rank * N_local; `input` [M, N_local] and `mat2` [K, N_local] are the local
 * slabs, `mat1` [M, K] is replicated.  The kernel computes the slab like launch_addmm
 * and stores every tile to the same place in all `world` buffers with plain stores
 * over NVLink, overlapping the transfer with the remaining tiles.  The buffers are
 * complete on every rank once all ranks' kernels have finished; the caller orders
 * that with a barrier across the ranks.  Operands must be TMA-addressable.
 */
NineToothedResult launch_addmm_allgather(NineToothedStream stream, NineToothedTensor input, NineToothedTensor mat1,
                                         NineToothedTensor mat2, NineToothedTensor beta, NineToothedTensor alpha,
                                         NineToothedTensor output, void *const *peer_outputs, int world, int rank,
                                         int dtype);

/*
 * The same step with the copies made by the NVSwitch instead of by this GPU.  (No
 * counterpart in the reference.)  The ranks' full buffers are bound to one NVLink
 * multicast object (cuMulticastCreate / cuMulticastBindMem; a torch symmetric-memory
 * handle has done so when its `multicast_ptr` is non-zero) and `multicast_output` is
 * the address, in the multicast mapping, of the first element of this rank's slab:
 * multicast base + the byte offset of `output` in this rank's own buffer.  `output`
 * gives the slab's shape and strides; its memory is written like every other rank's,
 * by the switch.  Each tile leaves the GPU once (multimem.st), so the NVLink egress
 * and the store instructions are 1/world of launch_addmm_allgather's.  The slab
 * width must be a multiple of 64 columns, input and output rows unit-stride and
 * 16-byte aligned; other layouts get NINETOOTHED_B200_ERR_LAYOUT and belong to
 * launch_addmm_allgather.  Completion and ordering as for launch_addmm_allgather.
 */
NineToothedResult launch_addmm_allgather_multicast(NineToothedStream stream, NineToothedTensor input,
                                                   NineToothedTensor mat1, NineToothedTensor mat2,
                                                   NineToothedTensor beta, NineToothedTensor alpha,
                                                   NineToothedTensor output, void *multicast_output, int dtype);

/*
 * Row softmax over the last dimension of a 2-D tensor, fp32 math, one program
 * per row (tests/test_softmax.py:10-27).  dtype of input and output: FLOAT16,
 * BFLOAT16 or FLOAT32.
 */
NineToothedResult launch_softmax(NineToothedStream stream, NineToothedTensor input, NineToothedTensor output,
                                 int dtype);

/*
 * Fused attention with online softmax over [B,H,S,D] tensors, D <= 128
 * (tests/test_attention.py:14-70; launcher launch_attention, tests/test_aot.py:147).
 * is_causal is a 0-dim tensor (host int64_t).  No softmax scale is applied, like
 * the reference kernel; q is pre-multiplied by log2(e) in its own data type.
 */
NineToothedResult launch_attention(NineToothedStream stream, NineToothedTensor q, NineToothedTensor k,
                                   NineToothedTensor v, NineToothedTensor is_causal, NineToothedTensor o,
                                   int dtype);

/*
 * The same kernel with a run-time softmax scale (0-dim tensor, host double)
 * inserted before is_causal: q is multiplied by scale and then by log2(e), each
 * product rounded in the data type of q, which is what the reference's code
 * generator emits for `q * scale * 1.44269504089` (tests/test_attention.py:46
 * with one more 0-dim argument).
 */
NineToothedResult launch_attention_scaled(NineToothedStream stream, NineToothedTensor q, NineToothedTensor k,
                                          NineToothedTensor v, NineToothedTensor scale,
                                          NineToothedTensor is_causal, NineToothedTensor o, int dtype);

/*
 * conv2d as implicit GEMM, NCHW, stride 1, dilation 1, no bias, symmetric zero
 * padding (tests/test_conv2d.py:13-48 with the matmul application, :106;
 * launcher launch_conv2d, tests/test_aot.py:259).  `workspace` is device memory
 * of at least launch_conv2d_workspace_size(...) bytes, 256-byte aligned, owned
 * by the caller and free to reuse once the stream has passed this call.
 * Tensors may have any strides; a dense channels-last input is read in place.
 * A 1 x 1 filter without padding on dense NCHW or dense channels-last tensors
 * (channel counts and, for NCHW, pixels per image multiples of 8) needs no im2col:
 * it runs as a (batched) GEMM and leaves the workspace untouched, which the caller
 * must provide all the same.
 */
NineToothedResult launch_conv2d(NineToothedStream stream, NineToothedTensor input, NineToothedTensor filter,
                                NineToothedTensor output, int padding_h, int padding_w, int dtype,
                                void *workspace, size_t workspace_size);

size_t launch_conv2d_workspace_size(NineToothedTensor input, NineToothedTensor filter, int dtype);

/*
 * conv2d for callers that have no way to hand over scratch memory.  (This entry
 * point has no counterpart in the reference; it exists for this library's users.)
 *
 * launch_conv2d needs a workspace, and somebody has to allocate it.  Some callers
 * cannot: a C or C++ host that only holds the tensors and a stream it was given, a
 * plugin running inside another framework whose allocator owns all device memory, a
 * service that fixed its memory budget at start-up and must not grow it per request.
 * For them the library carries its own scratch: one array of
 * NINETOOTHED_B200_STATIC_WORKSPACE_BYTES bytes in device memory, part of the loaded
 * library image on every GPU that loads it, held until the process exits.  This call
 * runs the same kernels as launch_conv2d on that array.  It allocates nothing and
 * frees nothing, on the device or through any library.
 *
 * Limits and rules:
 *   - what the launch writes to scratch must not exceed
 *     NINETOOTHED_B200_STATIC_WORKSPACE_BYTES: the re-laid-out input unless the input is
 *     channels-last (read in place), plus the re-laid-out filter unless the filter is
 *     channels-last; nothing at all for an unpadded 1 x 1 filter on contiguous NCHW or
 *     dense channels-last tensors.  (launch_conv2d_workspace_size is the upper bound
 *     from the shapes alone.)  Larger problems are rejected with
 *     NINETOOTHED_B200_ERR_ARGUMENT and a message naming both sizes (use launch_conv2d
 *     with your own workspace for those);
 *   - the first call on each device looks up the array's device address (with that
 *     device current) and remembers it; make that first call before you start any
 *     stream capture on the device;
 *   - all calls on a device share the one array and it keeps whatever the previous
 *     call left in it; every call rewrites the part it reads, so nothing needs
 *     clearing, but two calls whose work overlaps on the GPU (different streams,
 *     or different host threads on different streams) race on it: keep them on one
 *     stream or order them yourself.
 */
#define NINETOOTHED_B200_STATIC_WORKSPACE_BYTES (32u * 1024u * 1024u)

NineToothedResult launch_conv2d_static_workspace(NineToothedStream stream, NineToothedTensor input,
                                                 NineToothedTensor filter, NineToothedTensor output,
                                                 int padding_h, int padding_w, int dtype);

/*
 * max_pool2d over non-overlapping windows (window stride = window) of an NCHW tensor:
 * output[n,c,p,q] = max of input[n, c, p*window_height .. , q*window_width ..]
 * (tests/test_max_pool2d.py:13-36).  With ceil_mode = 0 a ragged last window is
 * dropped (the arrangement tiles with floor_mode), with ceil_mode != 0 it is kept and
 * positions outside the tensor count as -inf; output must have the matching shape,
 * [N, C, (H - wh) / wh + 1, (W - ww) / ww + 1] with floor or ceil division (:41-50).
 * The window sizes are the kernel's constexpr arguments WINDOW_HEIGHT / WINDOW_WIDTH,
 * passed as trailing ints the way the reference's launchers take constexprs.  dtype:
 * FLOAT16, BFLOAT16 or FLOAT32; any strides.
 */
NineToothedResult launch_max_pool2d(NineToothedStream stream, NineToothedTensor input, NineToothedTensor output,
                                    int window_height, int window_width, int ceil_mode, int dtype);

/*
 * Text of the last error on the calling thread ("" if none).  The reference's
 * Python wrapper turns a non-zero result into _KernelLaunchError
 * (src/ninetoothed/aot.py:747-751); this gives that exception a message.
 */
const char *ninetoothed_b200_last_error(void);

/*
 * Device-side status word of the current device: 0, or a code recorded by a
 * kernel whose bounded wait gave up (the kernel then drains and returns; the
 * context stays usable): 0x10000000 | kernel id << 16 | wait code.  Synchronises
 * the device.  Writes 0 back when `clear`.  Returns 0 when the word is 0,
 * NINETOOTHED_B200_ERR_TIMEOUT (with *status filled and the text in
 * ninetoothed_b200_last_error) when it holds a give-up code, a CUDA error otherwise.
 * (No counterpart in the reference, whose kernels have no waits of their own.)
 */
NineToothedResult ninetoothed_b200_device_status(unsigned int *status, int clear);

/*
 * Self-test of that path, for health checks and the test-suite: launches one warp
 * that waits, for at most `limit_ns` nanoseconds (1 .. 1e9), on a barrier nobody
 * arrives at.  The wait runs out, the kernel records its code (kernel id 15, wait
 * code 0x5e1f) and returns normally; ninetoothed_b200_device_status then reports
 * NINETOOTHED_B200_ERR_TIMEOUT.  Nothing faults and nothing spins without a bound.
 * (No counterpart in the reference.)
 */
NineToothedResult ninetoothed_b200_selftest_wait_timeout(NineToothedStream stream, unsigned long long limit_ns);

/*
 * Prepares `stream` (a stream of your own, not cudaStreamPerThread) for launches
 * that split a long reduction (see launch_matmul): allocates the stream's scratch
 * array now, with the device that is current, so that no later launch allocates or
 * synchronises.  Idempotent.  (No counterpart in the reference.)
 */
NineToothedResult ninetoothed_b200_reserve_split_scratch(NineToothedStream stream);

/*
 * Operands that no TMA descriptor can address (odd strides, K not a multiple of 8,
 * a misaligned base), head sizes other than 64 and 128 and fp32 attention run on
 * plain CUDA-core kernels: same results, but orders of magnitude slower.  Every
 * such launch bumps a process-wide counter and leaves a sentence saying why on the
 * calling thread.  ninetoothed_b200_plain_launches returns the count (and zeroes it
 * when `reset`); ninetoothed_b200_last_note the sentence ("" if none yet).
 * (No counterpart in the reference.)
 */
long long ninetoothed_b200_plain_launches(int reset);
const char *ninetoothed_b200_last_note(void);

/*
 * matmul/addmm launches whose tiles would leave the last wave of CTA pairs mostly
 * idle run with some 256-column tiles traded for 192-column ones (same results bit
 * for bit, fewer idle pairs).  Returns how many launches did so in this process (and
 * zeroes the count when `reset`); NINETOOTHED_B200_GEMM_MIXED=0 in the environment
 * turns the trade off.  (No counterpart in the reference.)
 */
long long ninetoothed_b200_mixed_width_launches(int reset);

/*
 * The planner behind that trade, callable without a device (for tests and for
 * callers that want to know what a shape will get): a problem of tile_rows x
 * tile_cols tiles of 256 x 256 on `pairs` resident CTA pairs, whose tile-row of A
 * is row_panel_bytes long (256 * K * element size).  Writes how many tile-rows swap
 * 256-column tiles for 192-column ones and how many swaps (3 wide -> 4 narrow) each
 * makes (0, 0: the plain plan), and returns the modelled cycles per K-block step of
 * the longest pair.  (No counterpart in the reference.)
 */
long long ninetoothed_b200_plan_mixed_widths(long long tile_rows, long long tile_cols, int pairs,
                                             long long row_panel_bytes, int *rows, int *swaps);

/* Library version: major * 10000 + minor * 100 + patch. */
int ninetoothed_b200_version(void);

#ifdef __cplusplus
}
#endif

#endif /* NINETOOTHED_B200_H */
