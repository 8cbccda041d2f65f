// Gradient all-reduce over NCCL (NVLink 5 / NVSwitch).  Replaces the reference's replica
// synchronisation, which reads every replica to the host, averages with numpy and writes
// it back (litenn/core/optimizer/Optimizer.py:149-153).  NCCL is opened with dlopen on
// first use so the library loads (and every non-collective entry works) without it.
#include "lnn_common.cuh"
#include <dlfcn.h>
#include <string.h>

namespace {

// Minimal slice of the NCCL ABI (stable across 2.x): opaque comm, 128-byte unique id.
typedef struct { char internal[128]; } nccl_uid;
typedef void* nccl_comm;
enum { kNcclFloat32 = 7, kNcclSum = 0, kNcclSuccess = 0 };

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(nccl_uid*) = nullptr;
  int (*CommInitRank)(nccl_comm*, int, nccl_uid, int) = nullptr;
  int (*CommInitAll)(nccl_comm*, int, const int*) = nullptr;
  int (*CommDestroy)(nccl_comm) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};

NcclApi g_nccl;

int load_nccl() {
  if (g_nccl.handle) return LNN_OK;
  const char* names[] = {getenv("LNN_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* n : names) {
    if (!n || !*n) continue;
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) return lnn::set_error(LNN_E_NCCL, "cannot dlopen libnccl.so.2: %s", dlerror());
#define LOAD(field, sym)                                                                   \
  *(void**)(&g_nccl.field) = dlsym(h, sym);                                                \
  if (!g_nccl.field) return lnn::set_error(LNN_E_NCCL, "libnccl lacks symbol %s", sym)
  LOAD(GetUniqueId, "ncclGetUniqueId");
  LOAD(CommInitRank, "ncclCommInitRank");
  LOAD(CommInitAll, "ncclCommInitAll");
  LOAD(CommDestroy, "ncclCommDestroy");
  LOAD(AllReduce, "ncclAllReduce");
  LOAD(GroupStart, "ncclGroupStart");
  LOAD(GroupEnd, "ncclGroupEnd");
  LOAD(GetErrorString, "ncclGetErrorString");
#undef LOAD
  g_nccl.handle = h;
  return LNN_OK;
}

#define LNN_NCCL(call)                                                                     \
  do {                                                                                     \
    int _r = (call);                                                                       \
    if (_r != kNcclSuccess)                                                                \
      return lnn::set_error(LNN_E_NCCL, "%s failed: %s", #call, g_nccl.GetErrorString(_r)); \
  } while (0)

}  // namespace

extern "C" {

int lnn_nccl_unique_id(void* id128) {
  LNN_REQUIRE(id128, "id128 is null");
  int rc = load_nccl();
  if (rc) return rc;
  nccl_uid id;
  LNN_NCCL(g_nccl.GetUniqueId(&id));
  memcpy(id128, &id, sizeof(id));
  return LNN_OK;
}

int lnn_nccl_init_rank(int dev, int nranks, int rank, const void* id128) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(id128 && nranks >= 1 && rank >= 0 && rank < nranks, "bad arguments");
  int rc = load_nccl();
  if (rc) return rc;
  LNN_REQUIRE(!d->nccl_comm, "device %d already has a communicator", dev);
  nccl_uid id;
  memcpy(&id, id128, sizeof(id));
  nccl_comm comm = nullptr;
  LNN_NCCL(g_nccl.CommInitRank(&comm, nranks, id, rank));
  d->nccl_comm = comm;
  return LNN_OK;
}

int lnn_nccl_init_all(const int* devs, int ndev) {
  LNN_REQUIRE(devs && ndev >= 1 && ndev <= LNN_MAX_DEVICES, "bad arguments");
  int rc = load_nccl();
  if (rc) return rc;
  nccl_comm comms[LNN_MAX_DEVICES];
  int ordinals[LNN_MAX_DEVICES];
  for (int i = 0; i < ndev; ++i) {
    lnn::Device* d = lnn::get_device(devs[i]);
    if (!d) return LNN_E_NOTINIT;
    LNN_REQUIRE(!d->nccl_comm, "device %d already has a communicator", devs[i]);
    ordinals[i] = d->ordinal;
  }
  LNN_NCCL(g_nccl.CommInitAll(comms, ndev, ordinals));
  for (int i = 0; i < ndev; ++i) lnn::get_device(devs[i])->nccl_comm = comms[i];
  return LNN_OK;
}

int lnn_nccl_allreduce_sum(int dev, uint64_t buf, int64_t count) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(buf && count > 0, "bad arguments");
  if (!d->nccl_comm) return lnn::set_error(LNN_E_NCCL, "device %d has no communicator", dev);
  void* p = (void*)(uintptr_t)buf;
  LNN_NCCL(g_nccl.AllReduce(p, p, (size_t)count, kNcclFloat32, kNcclSum, d->nccl_comm, d->stream));
  return LNN_OK;
}

int lnn_nccl_group_start(void) {
  int rc = load_nccl();
  if (rc) return rc;
  LNN_NCCL(g_nccl.GroupStart());
  return LNN_OK;
}

int lnn_nccl_group_end(void) {
  int rc = load_nccl();
  if (rc) return rc;
  LNN_NCCL(g_nccl.GroupEnd());
  return LNN_OK;
}

int lnn_nccl_destroy(int dev) {
  LNN_DEV(d, dev);
  if (!d->nccl_comm) return LNN_OK;
  if (g_nccl.CommDestroy) g_nccl.CommDestroy(d->nccl_comm);
  d->nccl_comm = nullptr;
  return LNN_OK;
}

}  // extern "C"
