// Measurement aid, not part of the operator: cuDNN's fp32 3x3 convolution through the legacy API,
// the yardstick the reference measures itself against (src/openCNN_winograd.cu:349-400 set-up,
// :449-464 timing; it pins algorithm 6, CUDNN_CONVOLUTION_FWD_ALGO_WINOGRAD, at :392).
// A stand-alone program (its own process, so that it uses the system cuDNN and never meets the
// copy another library may have loaded):
//
//     cudnn_probe N C H W K [calls]
//
// prints one JSON object: per algorithm that ran with true fp32 arithmetic (CUDNN_FMA_MATH: no
// TF32 down-conversion) the time of `calls` back-to-back cudnnConvolutionForward calls after one
// warm-up, the fastest of them, the cudnnFindConvolutionForwardAlgorithm ranking, and algorithm 6
// on its own (or why it does not run).  NCHW / KCRS fp32 tensors, cross-correlation, pad 1,
// stride 1, like the reference's descriptors.
#include <cuda_runtime.h>
#include <cudnn.h>

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#define CK(call)                                                                                  \
  do {                                                                                            \
    cudaError_t e_ = (call);                                                                      \
    if (e_ != cudaSuccess) {                                                                      \
      std::printf("{\"error\": \"%s: %s\"}\n", #call, cudaGetErrorString(e_));                  \
      return 1;                                                                                   \
    }                                                                                             \
  } while (0)
#define CD(call)                                                                                  \
  do {                                                                                            \
    cudnnStatus_t s_ = (call);                                                                    \
    if (s_ != CUDNN_STATUS_SUCCESS) {                                                             \
      std::printf("{\"error\": \"%s: %s\"}\n", #call, cudnnGetErrorString(s_));                 \
      return 1;                                                                                   \
    }                                                                                             \
  } while (0)

static const char *algo_name(int a) {
  static const char *names[] = {"IMPLICIT_GEMM", "IMPLICIT_PRECOMP_GEMM", "GEMM", "DIRECT", "FFT", "FFT_TILING",
                                "WINOGRAD", "WINOGRAD_NONFUSED"};
  return (a >= 0 && a < 8) ? names[a] : "?";
}

int main(int argc, char **argv) {
  if (argc < 6) {
    std::printf("{\"error\": \"usage: cudnn_probe N C H W K [calls]\"}\n");
    return 2;
  }
  const int N = std::atoi(argv[1]), C = std::atoi(argv[2]), H = std::atoi(argv[3]), W = std::atoi(argv[4]),
            K = std::atoi(argv[5]);
  const int calls = argc > 6 ? std::atoi(argv[6]) : 20;
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || K <= 0 || calls <= 0) {
    std::printf("{\"error\": \"bad sizes\"}\n");
    return 2;
  }
  cudnnHandle_t h;
  CD(cudnnCreate(&h));
  cudnnTensorDescriptor_t xd, yd;
  cudnnFilterDescriptor_t wd;
  cudnnConvolutionDescriptor_t cd;
  CD(cudnnCreateTensorDescriptor(&xd));
  CD(cudnnCreateTensorDescriptor(&yd));
  CD(cudnnCreateFilterDescriptor(&wd));
  CD(cudnnCreateConvolutionDescriptor(&cd));
  CD(cudnnSetTensor4dDescriptor(xd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, N, C, H, W));
  CD(cudnnSetFilter4dDescriptor(wd, CUDNN_DATA_FLOAT, CUDNN_TENSOR_NCHW, K, C, 3, 3));
  CD(cudnnSetConvolution2dDescriptor(cd, 1, 1, 1, 1, 1, 1, CUDNN_CROSS_CORRELATION, CUDNN_DATA_FLOAT));
  CD(cudnnSetConvolutionMathType(cd, CUDNN_FMA_MATH));
  int on, oc, oh, ow;
  CD(cudnnGetConvolution2dForwardOutputDim(cd, xd, wd, &on, &oc, &oh, &ow));
  CD(cudnnSetTensor4dDescriptor(yd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, on, oc, oh, ow));

  const size_t xb = (size_t)N * C * H * W * 4, wb = (size_t)K * C * 9 * 4, yb = (size_t)on * oc * oh * ow * 4;
  float *x = nullptr, *w = nullptr, *y = nullptr;
  CK(cudaMalloc(&x, xb));
  CK(cudaMalloc(&w, wb));
  CK(cudaMalloc(&y, yb));
  {  // seeded host fill, uploaded once: values in (-1, 1) and (-0.05, 0.05)
    std::vector<float> hx(xb / 4), hw(wb / 4);
    unsigned long long s = 0x9E3779B97F4A7C15ull;
    auto next = [&s]() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return (float)((s >> 11) * (1.0 / 9007199254740992.0)); };
    for (auto &v : hx) v = 2.f * next() - 1.f;
    for (auto &v : hw) v = 0.1f * next() - 0.05f;
    CK(cudaMemcpy(x, hx.data(), xb, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(w, hw.data(), wb, cudaMemcpyHostToDevice));
  }
  cudaEvent_t t0, t1;
  CK(cudaEventCreate(&t0));
  CK(cudaEventCreate(&t1));
  const float one = 1.f, zero = 0.f;

  // time one algorithm: workspace, 1 warm-up, `calls` back-to-back calls; < 0 and a reason if it does not run
  auto time_algo = [&](int algo, std::string &why, size_t &ws_bytes) -> double {
    ws_bytes = 0;
    cudnnStatus_t s = cudnnGetConvolutionForwardWorkspaceSize(h, xd, wd, cd, yd, (cudnnConvolutionFwdAlgo_t)algo, &ws_bytes);
    if (s != CUDNN_STATUS_SUCCESS) { why = cudnnGetErrorString(s); return -1.0; }
    void *ws = nullptr;
    if (ws_bytes && cudaMalloc(&ws, ws_bytes) != cudaSuccess) { why = "workspace allocation failed"; cudaGetLastError(); return -1.0; }
    s = cudnnConvolutionForward(h, &one, xd, x, wd, w, cd, (cudnnConvolutionFwdAlgo_t)algo, ws, ws_bytes, &zero, yd, y);
    if (s != CUDNN_STATUS_SUCCESS) { why = cudnnGetErrorString(s); if (ws) cudaFree(ws); return -1.0; }
    cudaEventRecord(t0, 0);
    for (int i = 0; i < calls; ++i)
      cudnnConvolutionForward(h, &one, xd, x, wd, w, cd, (cudnnConvolutionFwdAlgo_t)algo, ws, ws_bytes, &zero, yd, y);
    cudaEventRecord(t1, 0);
    float ms = -1.f;
    if (cudaEventSynchronize(t1) != cudaSuccess) { why = "execution failed"; if (ws) cudaFree(ws); return -1.0; }
    cudaEventElapsedTime(&ms, t0, t1);
    if (ws) cudaFree(ws);
    return (double)ms * 1e3 / calls;
  };

  std::printf("{\"cudnn_version\": %zu, \"shape\": [%d, %d, %d, %d, %d], \"calls\": %d, \"math\": \"CUDNN_FMA_MATH\", \"algos\": [",
              cudnnGetVersion(), N, C, H, W, K, calls);
  double best = -1.0;
  int best_algo = -1;
  bool first = true;
  for (int a = 0; a < 8; ++a) {
    std::string why;
    size_t wsb = 0;
    const double us = time_algo(a, why, wsb);
    std::printf("%s{\"algo\": %d, \"name\": \"%s\", ", first ? "" : ", ", a, algo_name(a));
    if (us >= 0) std::printf("\"us\": %.3f, \"workspace_bytes\": %zu}", us, wsb);
    else         std::printf("\"us\": null, \"why\": \"%s\"}", why.c_str());
    first = false;
    if (us >= 0 && (best < 0 || us < best)) { best = us; best_algo = a; }
  }
  std::printf("], ");
  // cudnnFind's own ranking under the same math type (the reference's alternative to pinning algo 6)
  cudnnConvolutionFwdAlgoPerf_t perf[16];
  int got = 0;
  cudnnStatus_t fs = cudnnFindConvolutionForwardAlgorithm(h, xd, wd, cd, yd, 16, &got, perf);
  std::printf("\"find\": [");
  if (fs == CUDNN_STATUS_SUCCESS) {
    bool f2 = true;
    for (int i = 0; i < got; ++i) {
      if (perf[i].status != CUDNN_STATUS_SUCCESS) continue;
      std::printf("%s{\"algo\": %d, \"name\": \"%s\", \"us\": %.3f, \"math\": %d}", f2 ? "" : ", ", (int)perf[i].algo,
                  algo_name((int)perf[i].algo), perf[i].time * 1e3, (int)perf[i].mathType);
      f2 = false;
    }
  }
  std::printf("], ");
  if (best_algo >= 0) std::printf("\"best_fp32\": {\"algo\": %d, \"name\": \"%s\", \"us\": %.3f}", best_algo, algo_name(best_algo), best);
  else                std::printf("\"best_fp32\": null");
  std::printf("}\n");
  cudaFree(x); cudaFree(w); cudaFree(y);
  cudnnDestroy(h);
  return 0;
}
