// Runtime of the C ABI: device table, stream, pooled allocator, copies, events.
// Counterpart of LiteNN's minicl layer (litenn/core/minicl/CLDevice.py, CLBuffer.py,
// devices.py): one in-order stream per device, a size-keyed buffer pool with
// evict-largest-and-retry on allocation failure, lazy nothing -- the host layer
// decides when to allocate.
#include "lnn_common.cuh"
#include <string.h>
#include <stdlib.h>

namespace lnn {

static Device g_devices[LNN_MAX_DEVICES];
static thread_local char g_err[1024] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

Device* get_device(int dev) {
  if (dev < 0 || dev >= LNN_MAX_DEVICES || !g_devices[dev].inited) {
    set_error(LNN_E_NOTINIT, "device %d is not initialised (call lnn_init first)", dev);
    return nullptr;
  }
  return &g_devices[dev];
}

// Host-side fault injection for tests (never touches the GPU): after LNN_FAIL_ALLOC_AFTER=n
// successful fresh cudaMalloc calls, the next LNN_FAIL_ALLOC_TIMES=k calls (default: all of
// them) report an allocation failure.
static long g_fail_alloc_after = -2;
static long g_fail_alloc_times = -1;
static long g_fresh_allocs = 0;
static long g_failed_allocs = 0;

static cudaError_t raw_malloc(void** p, uint64_t bytes) {
  if (g_fail_alloc_after == -2) {
    const char* e = getenv("LNN_FAIL_ALLOC_AFTER");
    g_fail_alloc_after = e ? atol(e) : -1;
    const char* t = getenv("LNN_FAIL_ALLOC_TIMES");
    g_fail_alloc_times = t ? atol(t) : -1;
  }
  if (g_fail_alloc_after >= 0 && g_fresh_allocs >= g_fail_alloc_after &&
      (g_fail_alloc_times < 0 || g_failed_allocs < g_fail_alloc_times)) {
    g_failed_allocs++;
    return cudaErrorMemoryAllocation;
  }
  g_fresh_allocs++;
  return cudaMalloc(p, bytes);
}

int alloc_bytes(Device* d, uint64_t bytes, void** out) {
  if (bytes == 0) return set_error(LNN_E_INVALID, "allocation of 0 bytes");
  auto it = d->pool.find(bytes);
  if (it != d->pool.end() && !it->second.empty()) {
    *out = it->second.back();
    it->second.pop_back();
    d->pooled_bytes -= bytes;
    return LNN_OK;
  }
  for (;;) {
    void* p = nullptr;
    cudaError_t e = raw_malloc(&p, bytes);
    if (e == cudaSuccess) {
      d->allocated_bytes += bytes;
      *out = p;
      return LNN_OK;
    }
    cudaGetLastError();  // clear the sticky-less allocation error
    if (e != cudaErrorMemoryAllocation)
      return set_error(LNN_E_CUDA, "cudaMalloc(%llu) failed: %s", (unsigned long long)bytes,
                       cudaGetErrorString(e));
    // evict the largest pooled buffer and retry (CLDevice.py:134-164)
    bool evicted = false;
    for (auto rit = d->pool.rbegin(); rit != d->pool.rend(); ++rit) {
      if (!rit->second.empty()) {
        void* victim = rit->second.back();
        rit->second.pop_back();
        cudaStreamSynchronize(d->stream);
        cudaFree(victim);
        d->pooled_bytes -= rit->first;
        d->allocated_bytes -= rit->first;
        evicted = true;
        break;
      }
    }
    if (!evicted)
      return set_error(LNN_E_NOMEM, "unable to allocate %llu MB on device %d",
                       (unsigned long long)(bytes >> 20), d->ordinal);
  }
}

int free_bytes(Device* d, void* p, uint64_t bytes) {
  d->pool[bytes].push_back(p);
  d->pooled_bytes += bytes;
  return LNN_OK;
}

}  // namespace lnn

using namespace lnn;

extern "C" {

int lnn_version(void) { return 100; }

const char* lnn_last_error(void) { return g_err; }

int lnn_device_count(int* count) {
  LNN_REQUIRE(count, "count is null");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    *count = 0;
    return set_error(LNN_E_CUDA, "cudaGetDeviceCount failed: %s", cudaGetErrorString(e));
  }
  *count = n < LNN_MAX_DEVICES ? n : LNN_MAX_DEVICES;
  return LNN_OK;
}

int lnn_device_info(int dev, char* name, int name_len, uint64_t* total_mem, int* sm_count,
                    int* cc_major, int* cc_minor) {
  cudaDeviceProp p;
  LNN_CUDA(cudaGetDeviceProperties(&p, dev));
  if (name && name_len > 0) {
    strncpy(name, p.name, name_len - 1);
    name[name_len - 1] = 0;
  }
  if (total_mem) *total_mem = p.totalGlobalMem;
  if (sm_count) *sm_count = p.multiProcessorCount;
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  return LNN_OK;
}

int lnn_init(int dev) {
  LNN_REQUIRE(dev >= 0 && dev < LNN_MAX_DEVICES, "device index %d out of range", dev);
  Device* d = &g_devices[dev];
  if (d->inited) return LNN_OK;
  cudaDeviceProp p;
  LNN_CUDA(cudaGetDeviceProperties(&p, dev));
  if (p.major != 10)
    return set_error(LNN_E_UNSUPPORTED,
                     "device %d is sm_%d%d; this library only contains sm_100a code", dev,
                     p.major, p.minor);
  LNN_CUDA(cudaSetDevice(dev));
  LNN_CUDA(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
  LNN_CUDA(cudaStreamCreateWithFlags(&d->copy_stream, cudaStreamNonBlocking));
  LNN_CUDA(cudaEventCreateWithFlags(&d->copy_event, cudaEventDisableTiming));
  LNN_CUDA(cudaStreamCreateWithFlags(&d->readback_stream, cudaStreamNonBlocking));
  LNN_CUDA(cudaEventCreateWithFlags(&d->readback_event, cudaEventDisableTiming));
  LNN_CUDA(cudaMalloc(&d->status_dev, sizeof(int) * 4));
  LNN_CUDA(cudaMemset(d->status_dev, 0, sizeof(int) * 4));
  LNN_CUDA(cudaMallocHost(&d->status_host, sizeof(int) * 4));
  d->ordinal = dev;
  d->sm_count = p.multiProcessorCount;
  d->allocated_bytes = d->pooled_bytes = 0;
  d->launches = 0;
  d->inited = true;
  return LNN_OK;
}

int lnn_pool_trim(int dev) {
  LNN_DEV(d, dev);
  LNN_CUDA(cudaStreamSynchronize(d->stream));
  for (auto& kv : d->pool) {
    for (void* p : kv.second) {
      cudaFree(p);
      d->pooled_bytes -= kv.first;
      d->allocated_bytes -= kv.first;
    }
    kv.second.clear();
  }
  d->pool.clear();
  return LNN_OK;
}

int lnn_nccl_destroy(int dev);

int lnn_shutdown(int dev) {
  LNN_DEV(d, dev);
  if (d->nccl_comm) lnn_nccl_destroy(dev);
  int rc = lnn_pool_trim(dev);
  if (rc) return rc;
  if (d->allocated_bytes != 0)
    return set_error(LNN_E_INVALID, "device %d still has %llu bytes in live buffers", dev,
                     (unsigned long long)d->allocated_bytes);
  cudaFree(d->status_dev);
  cudaFreeHost(d->status_host);
  cudaStreamDestroy(d->stream);
  cudaStreamDestroy(d->copy_stream);
  cudaEventDestroy(d->copy_event);
  cudaStreamDestroy(d->readback_stream);
  cudaEventDestroy(d->readback_event);
  *d = Device();
  return LNN_OK;
}

int lnn_alloc(int dev, uint64_t bytes, uint64_t* ptr) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(ptr, "ptr is null");
  void* p = nullptr;
  int rc = alloc_bytes(d, bytes, &p);
  *ptr = (uint64_t)(uintptr_t)p;
  return rc;
}

int lnn_free(int dev, uint64_t ptr, uint64_t bytes) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(ptr && bytes, "null buffer");
  return free_bytes(d, (void*)(uintptr_t)ptr, bytes);
}

int lnn_mem_stats(int dev, uint64_t* allocated_bytes, uint64_t* pooled_bytes) {
  LNN_DEV(d, dev);
  if (allocated_bytes) *allocated_bytes = d->allocated_bytes;
  if (pooled_bytes) *pooled_bytes = d->pooled_bytes;
  return LNN_OK;
}

int lnn_h2d(int dev, uint64_t dst, const void* src, uint64_t bytes) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dst && src, "null pointer");
  LNN_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, src, bytes, cudaMemcpyHostToDevice, d->stream));
  LNN_CUDA(cudaStreamSynchronize(d->stream));
  return LNN_OK;
}

// The device status word travels with every host synchronisation (its 16 bytes ride on the
// stream in front of the sync the caller pays anyway): a bounded wait that expired in a tile
// kernel makes the kernels after it return at once, so whatever the host is about to read is
// not a result.  Reporting clears the word, so that work can go on afterwards.
static int sync_and_report(lnn::Device* d) {
  LNN_CUDA(cudaMemcpyAsync(d->status_host, d->status_dev, sizeof(int) * 4, cudaMemcpyDeviceToHost, d->stream));
  LNN_CUDA(cudaStreamSynchronize(d->stream));
  if (d->status_host[0] != 0) {
    const int st[4] = {d->status_host[0], d->status_host[1], d->status_host[2], d->status_host[3]};
    LNN_CUDA(cudaMemsetAsync(d->status_dev, 0, sizeof(int) * 4, d->stream));
    LNN_CUDA(cudaStreamSynchronize(d->stream));
    return lnn::set_error(LNN_E_TIMEOUT,
                          "device status %d (role %d, tile %d, step %d): a bounded wait expired in a tile kernel; "
                          "results computed since then are invalid (the status has been cleared)",
                          st[0], st[1], st[2], st[3]);
  }
  return LNN_OK;
}

int lnn_d2h(int dev, void* dst, uint64_t src, uint64_t bytes) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dst && src, "null pointer");
  LNN_CUDA(cudaMemcpyAsync(dst, (const void*)(uintptr_t)src, bytes, cudaMemcpyDeviceToHost, d->stream));
  return sync_and_report(d);
}

int lnn_h2d_async(int dev, uint64_t dst, const void* src, uint64_t bytes) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dst && src, "null pointer");
  LNN_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, src, bytes, cudaMemcpyHostToDevice, d->stream));
  return LNN_OK;
}

int lnn_d2h_async(int dev, void* dst, uint64_t src, uint64_t bytes) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dst && src, "null pointer");
  LNN_CUDA(cudaMemcpyAsync(dst, (const void*)(uintptr_t)src, bytes, cudaMemcpyDeviceToHost, d->stream));
  return LNN_OK;
}

int lnn_h2d_prefetch(int dev, uint64_t dst, const void* src, uint64_t bytes, uint64_t after_event) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dst && src, "null pointer");
  if (after_event)
    LNN_CUDA(cudaStreamWaitEvent(d->copy_stream, (cudaEvent_t)(uintptr_t)after_event, 0));
  LNN_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, src, bytes, cudaMemcpyHostToDevice, d->copy_stream));
  return LNN_OK;
}

int lnn_wait_prefetch(int dev) {
  LNN_DEV(d, dev);
  LNN_CUDA(cudaEventRecord(d->copy_event, d->copy_stream));
  LNN_CUDA(cudaStreamWaitEvent(d->stream, d->copy_event, 0));
  return LNN_OK;
}

int lnn_d2h_readback(int dev, void* dst, uint64_t src, uint64_t bytes) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dst && src, "null pointer");
  // ordered after everything enqueued on the compute stream so far, but on its own stream: the
  // compute stream goes on with the next batch while the result travels to the host
  LNN_CUDA(cudaEventRecord(d->readback_event, d->stream));
  LNN_CUDA(cudaStreamWaitEvent(d->readback_stream, d->readback_event, 0));
  LNN_CUDA(cudaMemcpyAsync(dst, (const void*)(uintptr_t)src, bytes, cudaMemcpyDeviceToHost, d->readback_stream));
  return LNN_OK;
}

int lnn_wait_readback(int dev) {
  LNN_DEV(d, dev);
  LNN_CUDA(cudaStreamSynchronize(d->readback_stream));
  return LNN_OK;
}

int lnn_d2d(int dev, uint64_t dst, uint64_t src, uint64_t bytes) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dst && src, "null pointer");
  LNN_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, (const void*)(uintptr_t)src, bytes,
                           cudaMemcpyDeviceToDevice, d->stream));
  return LNN_OK;
}

int lnn_sync(int dev) {
  LNN_DEV(d, dev);
  return sync_and_report(d);
}

int lnn_debug_set_status(int dev, int code, int role, int tile, int step) {
  LNN_DEV(d, dev);
  const int st[4] = {code, role, tile, step};
  LNN_CUDA(cudaMemcpyAsync(d->status_dev, st, sizeof(st), cudaMemcpyHostToDevice, d->stream));
  LNN_CUDA(cudaStreamSynchronize(d->stream));
  return LNN_OK;
}

int lnn_host_alloc(uint64_t bytes, void** ptr) {
  LNN_REQUIRE(ptr && bytes, "bad arguments");
  LNN_CUDA(cudaMallocHost(ptr, bytes));
  return LNN_OK;
}

int lnn_host_free(void* ptr) {
  LNN_CUDA(cudaFreeHost(ptr));
  return LNN_OK;
}

int lnn_launch_count(int dev, uint64_t* count) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(count, "count is null");
  *count = d->launches;
  return LNN_OK;
}

int lnn_device_status(int dev, int* status) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(status, "status is null");
  LNN_CUDA(cudaMemcpyAsync(d->status_host, d->status_dev, sizeof(int) * 4, cudaMemcpyDeviceToHost, d->stream));
  LNN_CUDA(cudaMemsetAsync(d->status_dev, 0, sizeof(int) * 4, d->stream));
  LNN_CUDA(cudaStreamSynchronize(d->stream));
  *status = d->status_host[0];
  if (*status != 0)
    set_error(LNN_E_TIMEOUT, "device status %d (role %d, tile %d, step %d): a bounded wait expired",
              d->status_host[0], d->status_host[1], d->status_host[2], d->status_host[3]);
  return LNN_OK;
}

int lnn_event_create(int dev, uint64_t* ev) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(ev, "ev is null");
  cudaEvent_t e;
  LNN_CUDA(cudaEventCreate(&e));
  *ev = (uint64_t)(uintptr_t)e;
  return LNN_OK;
}

int lnn_event_record(int dev, uint64_t ev) {
  LNN_DEV(d, dev);
  LNN_CUDA(cudaEventRecord((cudaEvent_t)(uintptr_t)ev, d->stream));
  return LNN_OK;
}

int lnn_event_elapsed_ms(int dev, uint64_t ev_start, uint64_t ev_stop, float* ms) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(ms, "ms is null");
  LNN_CUDA(cudaEventSynchronize((cudaEvent_t)(uintptr_t)ev_stop));
  LNN_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)(uintptr_t)ev_start, (cudaEvent_t)(uintptr_t)ev_stop));
  return LNN_OK;
}

int lnn_profile_enable(int dev, int on) {
  LNN_DEV(d, dev);
  d->profiling = on != 0;
  return LNN_OK;
}

int lnn_profile_read(int dev, int slot, uint64_t* launches, float* total_ms) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(slot >= 0 && slot < LNN_PROF_SLOTS && launches && total_ms, "bad arguments");
  LNN_CUDA(cudaStreamSynchronize(d->stream));
  uint64_t n = 0;
  float total = 0.0f;
  std::vector<Device::ProfSpan> keep;
  for (auto& sp : d->prof_spans) {
    if (sp.slot != slot) { keep.push_back(sp); continue; }
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, sp.start, sp.stop) == cudaSuccess) { total += ms; ++n; }
    cudaEventDestroy(sp.start);
    cudaEventDestroy(sp.stop);
  }
  d->prof_spans.swap(keep);
  *launches = n;
  *total_ms = total;
  return LNN_OK;
}

int lnn_event_destroy(int dev, uint64_t ev) {
  LNN_DEV(d, dev);
  LNN_CUDA(cudaEventDestroy((cudaEvent_t)(uintptr_t)ev));
  return LNN_OK;
}

}  // extern "C"
