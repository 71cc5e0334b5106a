// Minibatch data parallelism: one process per GPU, parameters replicated, one NCCL
// all-reduce (sum, fp32) of the packed sufficient statistics per update over
// NVLink/NVSwitch.  The reference has no multi-GPU layer; these entry points have no
// counterpart there.  NCCL is loaded with dlopen on first use so that single-GPU
// users need no NCCL at all.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>
#include <time.h>

#include "common.cuh"

using namespace b200;

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
} api;

ncclComm_t g_comm = nullptr;
int g_nranks = 1, g_rank = 0;

bool load_api() {
  if (api.handle) return true;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (api.handle) break;
  }
  if (!api.handle) {
    set_error("NCCL shared library not found (libnccl.so.2)");
    return false;
  }
#define LOAD(field, sym)                                            \
  *(void**)(&api.field) = dlsym(api.handle, sym);                   \
  if (!api.field) {                                                 \
    set_error("NCCL symbol missing: " sym);                         \
    return false;                                                   \
  }
  LOAD(GetUniqueId, "ncclGetUniqueId")
  LOAD(CommInitRank, "ncclCommInitRank")
  LOAD(AllReduce, "ncclAllReduce")
  LOAD(CommDestroy, "ncclCommDestroy")
  LOAD(CommAbort, "ncclCommAbort")
  LOAD(CommGetAsyncError, "ncclCommGetAsyncError")
  LOAD(GetErrorString, "ncclGetErrorString")
#undef LOAD
  return true;
}

int nccl_fail(ncclResult_t r) {
  set_error(api.GetErrorString ? api.GetErrorString(r) : "NCCL error");
  return ERROR_NCCL;
}

}  // namespace

extern "C" {

// Rank 0 calls this and hands the 128 bytes to the other ranks by any host channel.
int dp_unique_id(char* out128) {
  if (!load_api()) return ERROR_NCCL;
  ncclUniqueId id;
  ncclResult_t r = api.GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(r);
  memcpy(out128, &id, sizeof(id));
  return 0;
}

// Collective: every rank calls it with the same id.  The current CUDA device is the rank's GPU.
int dp_init(const char* id128, int nranks, int rank) {
  if (nranks == 1) {
    g_nranks = 1;
    g_rank = 0;
    return 0;
  }
  if (!load_api()) return ERROR_NCCL;
  if (g_comm) return set_error("dp_init called twice");
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  stream();  // create the library stream on this rank's device first
  ncclResult_t r = api.CommInitRank(&g_comm, nranks, id, rank);
  if (r != ncclSuccess) return nccl_fail(r);
  g_nranks = nranks;
  g_rank = rank;
  return 0;
}

int dp_world_size() { return g_nranks; }
int dp_rank() { return g_rank; }

// In-place sum over all ranks of the matrix's storage, enqueued on the library stream.
int dp_allreduce(cudamat* mat) {
  if (!mat->on_device) return ERROR_NOT_ON_DEVICE;
  if (g_nranks == 1) return 0;
  if (!g_comm) return set_error("dp_allreduce before dp_init");
  ncclResult_t r = api.AllReduce(mat->data_device, mat->data_device, (size_t)numel(mat), ncclFloat, ncclSum, g_comm,
                                 stream());
  if (r != ncclSuccess) return nccl_fail(r);
  return 0;
}

}  // extern "C"

namespace {

// The same all-reduce on a side stream, so that it runs beside the kernels that follow on the
// library stream: `begin` makes the side stream wait for what has been enqueued so far (the product
// that filled this buffer) and starts the all-reduce there; `end` makes the library stream wait for
// it.  The statistics of an update are reduced panel by panel this way while the next panel is
// still being multiplied.  slot = 0..7, one pending all-reduce each.
constexpr int kSlots = 8;
cudaStream_t g_side = nullptr;
cudaEvent_t g_ready[kSlots] = {nullptr}, g_done[kSlots] = {nullptr};

int ensure_side_stream() {
  if (g_side) return 0;
  if (cudaStreamCreateWithFlags(&g_side, cudaStreamNonBlocking) != cudaSuccess) return set_error("side stream creation failed");
  for (int i = 0; i < kSlots; i++)
    if (cudaEventCreateWithFlags(&g_ready[i], cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&g_done[i], cudaEventDisableTiming) != cudaSuccess)
      return set_error("event creation failed");
  return 0;
}

}  // namespace

extern "C" {

int dp_allreduce_begin(cudamat* mat, int slot) {
  if (!mat->on_device) return ERROR_NOT_ON_DEVICE;
  if (slot < 0 || slot >= kSlots) return ERROR_UNSUPPORTED;
  if (g_nranks == 1) return 0;
  if (!g_comm) return set_error("dp_allreduce_begin before dp_init");
  int err = ensure_side_stream();
  if (err) return err;
  if (cudaEventRecord(g_ready[slot], stream()) != cudaSuccess || cudaStreamWaitEvent(g_side, g_ready[slot], 0) != cudaSuccess)
    return set_error("dp_allreduce_begin: event hand-over failed");
  ncclResult_t r = api.AllReduce(mat->data_device, mat->data_device, (size_t)numel(mat), ncclFloat, ncclSum, g_comm, g_side);
  if (r != ncclSuccess) return nccl_fail(r);
  if (cudaEventRecord(g_done[slot], g_side) != cudaSuccess) return set_error("dp_allreduce_begin: cudaEventRecord failed");
  return 0;
}

int dp_allreduce_end(int slot) {
  if (slot < 0 || slot >= kSlots) return ERROR_UNSUPPORTED;
  if (g_nranks == 1 || !g_side) return 0;
  if (cudaStreamWaitEvent(stream(), g_done[slot], 0) != cudaSuccess) return set_error("dp_allreduce_end failed");
  return 0;
}

// Polls the communicator for an asynchronous error (a peer that died, a timeout).
int dp_check() {
  if (!g_comm) return 0;
  ncclResult_t st = ncclSuccess;
  ncclResult_t r = api.CommGetAsyncError(g_comm, &st);
  if (r != ncclSuccess) return nccl_fail(r);
  if (st != ncclSuccess && st != ncclInProgress) return nccl_fail(st);
  return 0;
}

// Host-side watchdog for the collectives: waits until everything enqueued on the library stream
// (all-reduces included) has completed, polling the communicator for asynchronous errors.  After
// timeout_ms without completion (a peer that never joined) the communicator is aborted, which
// ends its kernels, and ERROR_NCCL is returned; the stream is usable again afterwards.
int dp_wait(int timeout_ms) {
  timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  for (;;) {
    const cudaError_t q = cudaStreamQuery(stream());
    if (q == cudaSuccess) return 0;
    if (q != cudaErrorNotReady) return set_error(cudaGetErrorString(q));
    if (g_comm) {
      ncclResult_t st = ncclSuccess;
      if (api.CommGetAsyncError(g_comm, &st) == ncclSuccess && st != ncclSuccess && st != ncclInProgress) {
        api.CommAbort(g_comm);
        g_comm = nullptr;
        return nccl_fail(st);
      }
    }
    timespec t1;
    clock_gettime(CLOCK_MONOTONIC, &t1);
    const double ms = (t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6;
    if (ms > timeout_ms) {
      if (g_comm) {
        api.CommAbort(g_comm);
        g_comm = nullptr;
      }
      set_error("dp_wait: the collectives did not complete in time; the communicator was aborted");
      return ERROR_NCCL;
    }
    timespec nap = {0, 50000};
    nanosleep(&nap, nullptr);
  }
}

int dp_destroy() {
  if (g_comm) {
    cudaStreamSynchronize(stream());
    api.CommDestroy(g_comm);
    g_comm = nullptr;
  }
  g_nranks = 1;
  g_rank = 0;
  return 0;
}

int dp_abort() {
  if (g_comm) {
    api.CommAbort(g_comm);
    g_comm = nullptr;
  }
  g_nranks = 1;
  g_rank = 0;
  return 0;
}

}  // extern "C"
