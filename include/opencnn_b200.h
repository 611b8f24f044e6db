/*
 * opencnn_b200 - C ABI of the B200-native Winograd F(2x2,3x3) convolution operator.
 *
 * One shared library is built per output-staging variant, selected at build time exactly as in
 * the reference (Makefile:3,8): -DBASE, -DOPTSTS64 (default), -DOPTSTS64_CMP, -DOPTLDS64 give
 * libopencnn_b200_<VARIANT>.so.  All variants compute identical values.
 *
 * Tensor layouts (fp32, dense): input CHWN, filter CRSK, output KHWN, workspace [C][4][4][K]
 * (src/openCNN_winograd.cu:147-153,185; src/FX_m2.cu:58-59,84).  Constraints: N % 32 == 0,
 * K % 64 == 0, C % 8 == 0, 3x3 filter, stride 1, pad 1, m = 2 (src/config.hpp:19-21).  Unlike
 * the reference, violations are reported (cudaErrorInvalidValue) instead of computing garbage,
 * and rectangular images (in_h != in_w) are accepted.  The two legacy entry points keep
 * N % 32 == 0 and C % 8 == 0; every opencnn_* entry also takes a ragged last block of images
 * (N % 4 == 0 with OPENCNN_FP32, N % 8 == 0 with OPENCNN_TF32 / OPENCNN_BF16), any in_c >= 1 and,
 * with OPENCNN_FP32, filt_k % 4 == 0.
 *
 * Alignment: every device pointer must be 16-byte aligned; with OPENCNN_TF32 / OPENCNN_BF16 the
 * output must be 32-byte aligned (those kernels store 32 bytes per thread).  cudaMalloc gives
 * 256.  A pointer that is not is refused with cudaErrorInvalidValue before anything is launched.
 *
 * Return values are cudaError_t codes passed as int, so the header needs no CUDA include.
 * All pointers are device pointers unless a function says otherwise.  Calls are asynchronous
 * with respect to the host unless a function says otherwise.
 */
#ifndef OPENCNN_B200_H
#define OPENCNN_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque: a cudaStream_t. */
typedef void *opencnn_stream_t;

/* Arithmetic of the batched GEMM.  FP32 is the FFMA path that reproduces the reference bit for
 * bit; TF32 and BF16 run the GEMM on the tensor cores (operands rounded, fp32 accumulate). */
enum opencnn_precision { OPENCNN_FP32 = 0, OPENCNN_TF32 = 1, OPENCNN_BF16 = 2 };

/* Replaces convolutionForward_32x64x8 (src/convolutionForward_32x64x8.cu:264-284 and its
 * _baseline / ampere copies): filter transform into Ww, then the fused kernel, both enqueued on
 * the legacy default stream; returns the launch status without synchronising.  Same argument
 * list and meaning: k input, w filter, C output, Ww workspace of at least in_c*16*filt_k
 * floats, tiles_dim = ceil(in_w/2), tile_size = alpha = 4, m = 2; n (element count) is unused. */
int convolutionForward_32x64x8(float *k, int in_h, int in_w, float *w, int out_h, int out_w, int out_n,
                               int out_c, float *C, float *Ww, const unsigned int n, int tiles_dim,
                               int in_n, int tile_size, int in_c, int filt_k, int filt_c, int filt_h,
                               int filt_w, int alpha, int m);

/* Replaces convolutionForward (src/openCNN_winograd.cu:204-219), the dispatcher that the
 * reference's caller uses (src/openCNN_winograd.cu:429-440).  elems_dim is unused there too. */
int convolutionForward(float *k, int in_h, int in_w, float *w, int out_h, int out_w, int out_n, int out_c,
                       float *C, float *Ww, const unsigned int n, int tiles_dim, int in_n, int tile_size,
                       int elems_dim, int in_c, int filt_k, int filt_c, int filt_h, int filt_w, int alpha,
                       int m);

/* Same operator on a caller-chosen stream and arithmetic.  The reference has only the default
 * stream (src/convolutionForward_32x64x8.cu:274,281) and only fp32. */
int opencnn_convolutionForward_stream(const float *input, const float *filter, float *output,
                                      float *workspace, int in_n, int in_c, int in_h, int in_w, int filt_k,
                                      int precision, opencnn_stream_t stream);

/* The two halves of the operator on their own.  opencnn_filter_transform replaces the launch of
 * FX (src/convolutionForward_32x64x8.cu:274); opencnn_winograd_forward replaces the launch of
 * Winograd_kernel (:281) and expects the workspace that the former wrote.  Callers with fixed
 * weights can transform once and reuse the workspace. */
int opencnn_filter_transform(const float *filter, float *workspace, int in_c, int filt_k,
                             opencnn_stream_t stream);
/* The same for a given arithmetic: the TF32 / BF16 workspace holds the transformed filter rounded
 * to the tensor-core operand type (and is what opencnn_winograd_forward expects for that
 * precision). */
int opencnn_filter_transform_p(const float *filter, float *workspace, int in_c, int filt_k, int precision,
                               opencnn_stream_t stream);
int opencnn_winograd_forward(const float *input, const float *workspace, float *output, int in_n, int in_c,
                             int in_h, int in_w, int filt_k, int precision, opencnn_stream_t stream);

/* The tensor-core fused kernel with the kernel chosen by the caller instead of by the library's own
 * rule (precision must be OPENCNN_TF32 or OPENCNN_BF16; the workspace as written by
 * opencnn_filter_transform_p for that precision).  All of them compute the same operator; they
 * differ in how a tile is spread over SMs.  The reference has no counterpart (no tensor-core path). */
enum opencnn_tc_kernel {
  OPENCNN_TC_AUTO = 0,          /* what opencnn_winograd_forward would take */
  OPENCNN_TC_SINGLE_CTA = 1,    /* one CTA per tile of 128 filters x 32 images, all 16 Winograd positions */
  OPENCNN_TC_PAIR_LOCAL = 2,    /* CTA pair per 128 x 64 tile, positions split 8 / 8, each CTA transforms all 64 images */
  OPENCNN_TC_STACKED_BLOCKS = 3 /* filt_k <= 64 only: one CTA per 64 filters x 64 images, the two 32-image blocks in
                                   the two halves of the accumulator rows */
};
int opencnn_winograd_forward_kernel(const float *input, const float *workspace, float *output, int in_n,
                                    int in_c, int in_h, int in_w, int filt_k, int precision, int kernel,
                                    opencnn_stream_t stream);

/* Layout adapters for callers that hold cuDNN-style tensors.  They replace data_cpy
 * (src/openCNN_winograd.cu:147-153, launched :229-235), which scatters NCHW -> CHWN and
 * KCRS -> CRSK one element per thread, and the index arithmetic with which the reference compares
 * its KHWN output against an NCHW result (:185-186).  Dense fp32, src and dst must not overlap. */
int opencnn_nchw_to_chwn(const float *src, float *dst, int n, int c, int h, int w, opencnn_stream_t stream);
int opencnn_kcrs_to_crsk(const float *src, float *dst, int k, int c, opencnn_stream_t stream);
int opencnn_khwn_to_nkhw(const float *src, float *dst, int n, int k, int h, int w, opencnn_stream_t stream);

/* Bytes of workspace the operator needs: in_c*16*filt_k floats, as allocated by the reference's
 * caller (src/openCNN_winograd.cu:309-311). */
size_t opencnn_workspace_bytes(int in_c, int filt_k);

/* "BASE", "OPTSTS64", "OPTSTS64_CMP" or "OPTLDS64": the -D the library was built with
 * (src/convolutionForward_32x64x8.cu:18-27, src/config.hpp:28-34). */
const char *opencnn_variant_name(void);

/* Synchronises the current device and returns the device-side status word: 0 = ok, 1 = a
 * bounded wait inside a kernel ran out (results are invalid).  Resets the word to 0.  The
 * reference has no counterpart: its kernels contain no waits. */
int opencnn_last_device_status(void);

/* The whole operator for callers that must not allocate.  (No counterpart in the reference: there
 * the caller always cudaMallocs the workspace, src/openCNN_winograd.cu:309-311.)
 *
 * Some users of this library may not create device memory at the point where they convolve: a
 * serving loop whose device memory is handed out once by the application's own pool, a plugin
 * that is given its input and output tensors and nothing else, a process running under a fixed
 * memory budget where a late cudaMalloc can fail or stall the device.  For them the
 * transformed-filter workspace - the operator's only scratch memory - lives inside the library,
 * in a static device array of OPENCNN_NOALLOC_MAX_CK * 16 floats (4 MiB) that every GPU which
 * loads the library holds until the process exits.  The caller passes only input, filter and
 * output.  The call makes no CUDA allocation and frees nothing.
 *
 * Limits and rules:
 *  - in_c * filt_k must not exceed OPENCNN_NOALLOC_MAX_CK (65536, e.g. C = K = 256); larger
 *    problems are refused with cudaErrorInvalidValue and a message on stderr.  Use the entry
 *    points above with your own workspace for those.
 *  - The first call on each device looks up the array's device address (and does the library's
 *    usual one-time kernel set-up); later calls on that device do neither.
 *  - All calls on a device share the one array.  Nothing in it has to start at zero - every call
 *    first overwrites the part it then reads - but it does keep the previous call's contents, and
 *    two calls whose kernels overlap on the GPU (different streams, no ordering) race on it.
 *    Order them on one stream or with events. */
#define OPENCNN_NOALLOC_MAX_CK 65536
int opencnn_convolutionForward_noalloc(const float *input, const float *filter, float *output, int in_n,
                                       int in_c, int in_h, int in_w, int filt_k, opencnn_stream_t stream);

/* Host-buffer front end, the shape of the reference's main() around the operator
 * (src/openCNN_winograd.cu:300-316 allocation, :470-472 copy back): a plan owns device buffers
 * for one problem size; run copies input and filter host->device, runs the operator, copies the
 * output device->host and synchronises.  Host pointers; pinned memory makes the copies
 * asynchronous but is not required. */
int opencnn_host_plan_create(void **plan, int in_n, int in_c, int in_h, int in_w, int filt_k, int precision);
int opencnn_host_plan_run(void *plan, const float *input_host, const float *filter_host, float *output_host);
/* The same work enqueued on the plan's own stream without waiting, and the matching wait: plans
 * of different layers then overlap their uploads, kernels and downloads (pinned host memory
 * required for overlap).  The host buffers must stay valid until opencnn_host_plan_wait. */
int opencnn_host_plan_run_async(void *plan, const float *input_host, const float *filter_host,
                                float *output_host);
int opencnn_host_plan_wait(void *plan);
/* The three copies of opencnn_host_plan_run_async without the kernels between them, on the same
 * stream: what a step costs when the GPU work is free.  A measurement aid - the floor an
 * end-to-end time can be compared with; the output buffer receives whatever the plan's device
 * buffer holds.  The reference's main() has the same copies around its timed loop
 * (src/openCNN_winograd.cu:300-316, :470-472) and never times them. */
int opencnn_host_plan_copy_async(void *plan, const float *input_host, const float *filter_host,
                                 float *output_host);
int opencnn_host_plan_destroy(void *plan);

#ifdef __cplusplus
}
#endif
#endif /* OPENCNN_B200_H */
