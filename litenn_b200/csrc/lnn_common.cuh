// Internal declarations shared by the translation units of liblitenn_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <map>
#include <vector>
#include "../../include/litenn_b200.h"

namespace lnn {

// Per-device state: one non-blocking stream, a size-keyed buffer pool, counters.
struct Device {
  bool inited = false;
  int ordinal = -1;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  cudaStream_t copy_stream = nullptr;            // host->device prefetches that overlap compute
  cudaEvent_t copy_event = nullptr;
  cudaStream_t readback_stream = nullptr;        // device->host reads that overlap the next batch's compute
  cudaEvent_t readback_event = nullptr;
  std::map<uint64_t, std::vector<void*>> pool;   // free buffers by exact byte size
  uint64_t allocated_bytes = 0;                  // live + pooled
  uint64_t pooled_bytes = 0;
  uint64_t launches = 0;
  int* status_dev = nullptr;                     // device status word (bounded waits)
  int* status_host = nullptr;                    // pinned mirror
  void* nccl_comm = nullptr;
  uint32_t smem_attr_done = 0;                   // kernels whose dynamic shared-memory limit was raised on this device
  bool profiling = false;
  struct ProfSpan { int slot; cudaEvent_t start, stop; };
  std::vector<ProfSpan> prof_spans;
};

// Brackets the launches made while it is alive with a pair of events (profiling only).
struct ProfScope {
  Device* d; int slot; cudaEvent_t start = nullptr;
  ProfScope(Device* dev, int s) : d(dev), slot(s) {
    if (d->profiling && cudaEventCreate(&start) == cudaSuccess) cudaEventRecord(start, d->stream);
  }
  ~ProfScope() {
    if (!start) return;
    cudaEvent_t stop;
    if (cudaEventCreate(&stop) != cudaSuccess) { cudaEventDestroy(start); return; }
    cudaEventRecord(stop, d->stream);
    d->prof_spans.push_back({slot, start, stop});
  }
};

Device* get_device(int dev);          // nullptr + error set when not initialised
int set_error(int code, const char* fmt, ...);
int alloc_bytes(Device* d, uint64_t bytes, void** out);
int free_bytes(Device* d, void* p, uint64_t bytes);

// RAII scratch buffer taken from the device pool; returned to the pool on scope exit.
// Stream order makes reuse safe: every consumer runs on the same in-order stream.
struct Scratch {
  Device* d; void* p = nullptr; uint64_t bytes = 0;
  explicit Scratch(Device* dev) : d(dev) {}
  int get(uint64_t nbytes) { bytes = nbytes; return alloc_bytes(d, nbytes, &p); }
  ~Scratch() { if (p) free_bytes(d, p, bytes); }
  template <class T> T* as() { return reinterpret_cast<T*>(p); }
};

// direct (FP32-pipe) convolution for layers with IC <= 4 (lnn_direct.cu)
bool conv_direct_applicable(const lnn_conv_geom* g);
int conv_direct_fwd(Device* d, const lnn_conv_geom* g, float* Y, const float* X, const float* W,
                    const float* bias, int act, float alpha, int accumulate, int pool, int packed = 0,
                    float* Ylo = nullptr, int ocp_out = 0);
// the same layers on the tensor cores, split-FP16 precision, 3x3 / unit stride (lnn_fewch.cu)
bool conv_fewch_applicable(const lnn_conv_geom* g);
int conv_fewch_fwd(Device* d, const lnn_conv_geom* g, float* Y, const float* X, const float* W,
                   const float* bias, int act, float alpha, int ep_mode, int ocp, const uint32_t* amax_x,
                   uint32_t* amax_out, float* Y_lo = nullptr, uint8_t* idx = nullptr);
// kernel gradient of the same layers (IC <= 4, 3x3): dW += ...
bool conv_direct_dw_applicable(const lnn_conv_geom* g);
int conv_direct_dw(Device* d, const lnn_conv_geom* g, float* dW, const float* dY, const float* X);
// the same gradient of a pooled block from the winners of its pooling windows (T, IDX: pooled size)
bool conv_dw_winners_applicable(const lnn_conv_geom* g);
int conv_dw_winners(Device* d, const lnn_conv_geom* g, float* dW, const float* T, const uint8_t* IDX, const float* X);

}  // namespace lnn

#define LNN_CUDA(call)                                                                   \
  do {                                                                                   \
    cudaError_t _e = (call);                                                             \
    if (_e != cudaSuccess)                                                               \
      return lnn::set_error(LNN_E_CUDA, "%s failed: %s (%s:%d)", #call,                  \
                            cudaGetErrorString(_e), __FILE__, __LINE__);                 \
  } while (0)

#define LNN_DEV(d, dev)                                                                  \
  lnn::Device* d = lnn::get_device(dev);                                                 \
  if (!d) return LNN_E_NOTINIT;                                                          \
  LNN_CUDA(cudaSetDevice(d->ordinal))

#define LNN_CHECK_LAUNCH(d)                                                              \
  do {                                                                                   \
    (d)->launches++;                                                                     \
    cudaError_t _e = cudaGetLastError();                                                 \
    if (_e != cudaSuccess)                                                               \
      return lnn::set_error(LNN_E_CUDA, "kernel launch failed: %s (%s:%d)",              \
                            cudaGetErrorString(_e), __FILE__, __LINE__);                 \
  } while (0)

#define LNN_REQUIRE(cond, ...)                                                           \
  do { if (!(cond)) return lnn::set_error(LNN_E_INVALID, __VA_ARGS__); } while (0)

static inline int64_t lnn_ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
