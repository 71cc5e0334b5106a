// Device, stream and memory plumbing of the b200mat C ABI: the part of
// cudamat/cudamat.cu:25-435 that allocates, copies, slices and reshapes matrices.
// One process drives one GPU; every operation is enqueued on one library stream and
// the host only blocks where the reference API returns data to it.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace b200 {

static cudaStream_t g_stream = nullptr;
static bool g_own_stream = false;
static int g_sm_count = 0;
static int g_col0 = 0;
static int* g_status = nullptr;
static char g_err[512] = "";
static void* g_ws[8] = {nullptr};
static size_t g_ws_bytes[8] = {0};
static bool g_ws_fresh[8] = {false};   // allocated since it was last cleared (workspace_zeroed)
static std::mutex g_mu;

static int g_dependent_launch = -1;        // programmatic dependent launch of the hot kernels: -1 = read the environment
static uint32_t g_wait_limit = 1u << 24;   // iterations of a bounded device-side wait: ~1-2 s

// Creates the library stream and the device status word.  A failure (a device with no memory left,
// a context in an error state) is recorded and leaves the library uninitialised: stream() then
// returns null, status_word() null, and every entry point that launches reports CUDA_ERROR through
// check_launch() / its own checks instead of running on a garbage stream.
static void ensure_init() {
  if (g_stream) return;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_stream) return;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "library initialisation failed: %s", cudaGetErrorString(cudaGetLastError()));
    return;
  }
  int* status = nullptr;
  if (cudaMalloc(&status, sizeof(int)) != cudaSuccess || cudaMemset(status, 0, sizeof(int)) != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "library initialisation failed (status word): %s",
             cudaGetErrorString(cudaGetLastError()));
    if (status) cudaFree(status);
    return;
  }
  cudaStream_t s = nullptr;
  if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess || !s) {
    snprintf(g_err, sizeof(g_err), "library initialisation failed (stream): %s",
             cudaGetErrorString(cudaGetLastError()));
    cudaFree(status);
    return;
  }
  g_status = status;
  g_own_stream = true;
  g_stream = s;   // published last: a non-null stream means the library is usable
}

cudaStream_t stream() {
  ensure_init();
  return g_stream;
}
cudaStream_t stream_if_initialised() { return g_stream; }
static int g_sm_limit = 0;
int sm_count() {
  ensure_init();
  const int n = g_sm_count > 0 ? g_sm_count : 148;
  return (g_sm_limit > 0 && g_sm_limit < n) ? g_sm_limit : n;
}
int rng_col0() { return g_col0; }
int* status_word() {
  ensure_init();
  return g_status;
}
bool initialised() {
  ensure_init();
  return g_stream != nullptr;
}
uint32_t wait_limit() { return g_wait_limit; }
bool dependent_launch_enabled() {
  if (g_dependent_launch < 0) {
    const char* e = getenv("B200_DEPENDENT_LAUNCH");
    g_dependent_launch = (e && e[0] == '0') ? 0 : 1;
  }
  return g_dependent_launch != 0;
}

int set_error(const char* msg) {
  if (msg != g_err) snprintf(g_err, sizeof(g_err), "%s", msg);
  return CUDA_ERROR;
}

int check_launch_any_stream() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(cudaGetErrorString(e));
  return 0;
}
int check_launch() {
  if (!g_stream) return set_error(g_err[0] ? g_err : "the library is not initialised");
  return check_launch_any_stream();
}

void* workspace(int slot, size_t bytes) {
  ensure_init();
  if (slot < 0 || slot >= 8) return nullptr;
  if (g_ws_bytes[slot] >= bytes && g_ws[slot]) return g_ws[slot];
  if (g_ws[slot]) {
    cudaStreamSynchronize(g_stream);
    cudaFree(g_ws[slot]);
    g_ws[slot] = nullptr;
    g_ws_bytes[slot] = 0;
  }
  size_t want = bytes + bytes / 4 + 256;
  if (cudaMalloc(&g_ws[slot], want) != cudaSuccess) {
    cudaGetLastError();
    if (cudaMalloc(&g_ws[slot], bytes) != cudaSuccess) {
      set_error("workspace allocation failed");
      return nullptr;
    }
    want = bytes;
  }
  g_ws_bytes[slot] = want;
  g_ws_fresh[slot] = true;
  return g_ws[slot];
}

// The same, all zero when first handed out (and again after it had to grow): counters that their
// users leave at zero between calls.
void* workspace_zeroed(int slot, size_t bytes) {
  void* p = workspace(slot, bytes);
  if (p && g_ws_fresh[slot]) {
    if (cudaMemsetAsync(p, 0, g_ws_bytes[slot], g_stream) != cudaSuccess) {
      set_error("workspace clear failed");
      return nullptr;
    }
    g_ws_fresh[slot] = false;
  }
  return p;
}

}  // namespace b200

using namespace b200;

extern "C" {

// Text of the most recent failure.  Reading it clears it, so a later error of another kind (a raw
// CUDA error with no recorded text) is not reported under this one's words.
const char* get_last_cuda_error() {
  static char last[sizeof(g_err)];
  if (g_err[0]) {
    snprintf(last, sizeof(last), "%s", g_err);
    g_err[0] = 0;
    return last;
  }
  return cudaGetErrorString(cudaGetLastError());
}

// cudamat/cudamat.cu:31-44 created and destroyed the cuBLAS context; here the calls
// create the library stream and release cached scratch.
int cublas_init() {
  ensure_init();
  return g_stream ? 0 : CUDA_ERROR;
}

// Iterations a device-side wait (an mbarrier wait of the tensor-core product) may spin before
// the kernel gives up, records where in the status word (b200_read_status) and returns.  The
// default, 2^24, is one to two seconds; 0 restores it.  Failure-detection tests set a few
// thousand iterations (milliseconds) so that a wait that cannot complete ends quickly.
// SMs the library's kernels size their grids for (0 = all of the device).  The data-parallel step
// leaves a few SMs to the all-reduce that runs beside its statistics products: the persistent
// tensor-core kernel otherwise holds every SM until it ends.
int b200_sm_count() { return sm_count(); }
int b200_set_sm_limit(int sms) {
  g_sm_limit = sms > 0 ? sms : 0;
  return 0;
}

// Programmatic dependent launch of the hot kernels (a kernel is scheduled while its predecessor on
// the stream drains; it touches global memory only after the predecessor has completed): on by
// default, B200_DEPENDENT_LAUNCH=0 or this call with 0 turns it off.  No counterpart in the reference.
int b200_set_dependent_launch(int on) {
  g_dependent_launch = on ? 1 : 0;
  return 0;
}

int b200_set_wait_limit(unsigned int iterations) {
  g_wait_limit = iterations ? iterations : (1u << 24);
  return 0;
}

int cublas_shutdown() {
  if (!g_stream) return 0;
  cudaStreamSynchronize(g_stream);
  for (int i = 0; i < 8; i++) {
    if (g_ws[i]) cudaFree(g_ws[i]);
    g_ws[i] = nullptr;
    g_ws_bytes[i] = 0;
    g_ws_fresh[i] = false;
  }
  return 0;
}

// cudamat/cudamat.cu:46-53.  Must precede the first operation of the process.
int cuda_set_device(int deviceId) {
  if (g_stream) {
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != deviceId) return set_error("cuda_set_device after the library was initialised on another device");
    return 0;
  }
  if (cudaSetDevice(deviceId) != cudaSuccess) return set_error("cudaSetDevice failed");
  return 0;
}

int b200_device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// cudamat/cudamat.cu:103-105.
void cuda_sync_threads() { cudaStreamSynchronize(stream()); }

// Run the library on a caller's stream (0 restores the library's own).
int b200_set_stream(void* s) {
  ensure_init();
  static cudaStream_t own = nullptr;
  if (g_own_stream) own = g_stream;
  if (s) {
    g_stream = (cudaStream_t)s;
    g_own_stream = false;
  } else if (own) {
    g_stream = own;
    g_own_stream = true;
  }
  return 0;
}
void* b200_get_stream() { return (void*)stream(); }

// CUDA events on the library stream, for timing on the device.
void* b200_event_create() {
  cudaEvent_t ev = nullptr;
  if (cudaEventCreate(&ev) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return (void*)ev;
}
int b200_event_record(void* ev) {
  if (cudaEventRecord((cudaEvent_t)ev, stream()) != cudaSuccess) return set_error("cudaEventRecord failed");
  return 0;
}
// Milliseconds between two recorded events; blocks until `end` has happened.  < 0 on error.
float b200_event_elapsed_ms(void* start, void* end) {
  float ms = -1.0f;
  if (cudaEventSynchronize((cudaEvent_t)end) != cudaSuccess) return -1.0f;
  if (cudaEventElapsedTime(&ms, (cudaEvent_t)start, (cudaEvent_t)end) != cudaSuccess) return -1.0f;
  return ms;
}
void b200_event_destroy(void* ev) {
  if (ev) cudaEventDestroy((cudaEvent_t)ev);
}

// Reads and clears the device status word: non-zero means a kernel's bounded wait
// gave up (the value encodes where).  Blocks until the stream is idle.
int b200_read_status() {
  int v = 0;
  if (!initialised()) return ERROR_GENERIC;
  if (cudaStreamSynchronize(stream()) != cudaSuccess ||
      cudaMemcpy(&v, status_word(), sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
    set_error(cudaGetErrorString(cudaGetLastError()));
    return CUDA_ERROR;
  }
  if (v) cudaMemset(status_word(), 0, sizeof(int));
  return v;
}

// cudamat/cudamat.cu:55-83 loaded a multiplier table and seeded 12288 generators; the
// Philox stream needs only the key and a call counter.  `cudamatpath` is ignored.
int init_random(rnd_struct* rnd_state, int seed, char* cudamatpath) {
  (void)cudamatpath;
  rnd_state->seed = (unsigned long long)(unsigned int)seed;
  rnd_state->calls = 0;
  return 0;
}

// First global minibatch column held by this process (data-parallel shards draw the
// random numbers of their own columns of the global batch).
int set_rng_column_offset(int col0) {
  g_col0 = col0;
  return 0;
}

int get_leading_dimension(cudamat* mat) { return mat->is_trans ? mat->size[1] : mat->size[0]; }
int get_nonleading_dimension(cudamat* mat) { return mat->is_trans ? mat->size[0] : mat->size[1]; }
void set_transpose(cudamat* mat, int is_trans) { mat->is_trans = is_trans; }

// cudamat/cudamat.cu:109-123.
int allocate_device_memory(cudamat* mat) {
  const size_t bytes = (size_t)numel(mat) * sizeof(float);
  if (cudaMalloc((void**)&mat->data_device, bytes ? bytes : 4) != cudaSuccess) {
    cudaGetLastError();
    return set_error("cudaMalloc failed");
  }
  mat->on_device = 1;
  return 0;
}

// cudamat/cudamat.cu:153-165.  Blocks: the caller reads the host array next.
int copy_to_host(cudamat* mat) {
  if (!mat->on_device) return ERROR_NOT_ON_DEVICE;
  const size_t bytes = (size_t)numel(mat) * sizeof(float);
  if (cudaMemcpyAsync(mat->data_host, mat->data_device, bytes, cudaMemcpyDeviceToHost, stream()) != cudaSuccess)
    return set_error("copy_to_host failed");
  if (cudaStreamSynchronize(stream()) != cudaSuccess) return set_error(cudaGetErrorString(cudaGetLastError()));
  return 0;
}

// cudamat/cudamat.cu:167-186.
int copy_to_device(cudamat* mat) {
  if (!mat->on_device) {
    int err = allocate_device_memory(mat);
    if (err) return err;
  }
  const size_t bytes = (size_t)numel(mat) * sizeof(float);
  if (cudaMemcpyAsync(mat->data_device, mat->data_host, bytes, cudaMemcpyHostToDevice, stream()) != cudaSuccess)
    return set_error("copy_to_device failed");
  return 0;
}

// Copies `bytes` from any host pointer into the matrix's device buffer (used with
// pinned staging buffers so the transfer overlaps earlier kernels).
int copy_from_host_ptr(cudamat* mat, const float* src, size_t bytes) {
  if (!mat->on_device) return ERROR_NOT_ON_DEVICE;
  if (bytes > (size_t)numel(mat) * sizeof(float)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (cudaMemcpyAsync(mat->data_device, src, bytes, cudaMemcpyHostToDevice, stream()) != cudaSuccess)
    return set_error("copy_from_host_ptr failed");
  return 0;
}

// Host-to-device copy on a second stream, so the next minibatch travels while the
// current one is being processed.  b200_prefetch_wait makes the library stream wait for
// every copy started so far; b200_prefetch_fence makes later copies wait for the work
// already enqueued on the library stream (call it before overwriting a buffer in use).
static cudaStream_t g_copy_stream = nullptr;
static cudaEvent_t g_copy_done = nullptr, g_compute_done = nullptr;
static int ensure_copy_stream() {
  if (g_copy_stream) return 0;
  if (cudaStreamCreateWithFlags(&g_copy_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&g_copy_done, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&g_compute_done, cudaEventDisableTiming) != cudaSuccess)
    return set_error("copy stream creation failed");
  return 0;
}
int b200_prefetch(cudamat* mat, const float* src, size_t bytes) {
  if (!mat->on_device) return ERROR_NOT_ON_DEVICE;
  if (bytes > (size_t)numel(mat) * sizeof(float)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  int err = ensure_copy_stream();
  if (err) return err;
  if (cudaMemcpyAsync(mat->data_device, src, bytes, cudaMemcpyHostToDevice, g_copy_stream) != cudaSuccess)
    return set_error("b200_prefetch failed");
  return 0;
}
int b200_prefetch_wait() {
  int err = ensure_copy_stream();
  if (err) return err;
  if (cudaEventRecord(g_copy_done, g_copy_stream) != cudaSuccess ||
      cudaStreamWaitEvent(stream(), g_copy_done, 0) != cudaSuccess)
    return set_error("b200_prefetch_wait failed");
  return 0;
}
int b200_prefetch_fence() {
  int err = ensure_copy_stream();
  if (err) return err;
  if (cudaEventRecord(g_compute_done, stream()) != cudaSuccess ||
      cudaStreamWaitEvent(g_copy_stream, g_compute_done, 0) != cudaSuccess)
    return set_error("b200_prefetch_fence failed");
  return 0;
}

// Device-to-host read-back that does not stall the issuing thread: the copy is ordered after the
// work enqueued so far on the library stream and runs on a stream of its own (slot 0..7, one pending
// read-back each); b200_readback_wait blocks until the copy of that slot has landed.  `dst` is pinned
// host memory (b200_host_alloc); `src` must not be rewritten before the copy has run - read back a
// copy of a value that later work changes.  No counterpart in the reference.
static cudaStream_t g_rb_stream = nullptr;
static cudaEvent_t g_rb_ready[8] = {nullptr}, g_rb_done[8] = {nullptr};
int b200_readback_begin(cudamat* src, void* dst, size_t bytes, int slot) {
  if (!src->on_device) return ERROR_NOT_ON_DEVICE;
  if (slot < 0 || slot >= 8 || !dst) return ERROR_UNSUPPORTED;
  if (bytes > (size_t)numel(src) * sizeof(float)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (!initialised()) return CUDA_ERROR;
  if (!g_rb_stream && cudaStreamCreateWithFlags(&g_rb_stream, cudaStreamNonBlocking) != cudaSuccess)
    return set_error("read-back stream creation failed");
  if (!g_rb_ready[slot] && (cudaEventCreateWithFlags(&g_rb_ready[slot], cudaEventDisableTiming) != cudaSuccess ||
                            cudaEventCreateWithFlags(&g_rb_done[slot], cudaEventDisableTiming) != cudaSuccess))
    return set_error("read-back event creation failed");
  if (cudaEventRecord(g_rb_ready[slot], stream()) != cudaSuccess ||
      cudaStreamWaitEvent(g_rb_stream, g_rb_ready[slot], 0) != cudaSuccess ||
      cudaMemcpyAsync(dst, src->data_device, bytes, cudaMemcpyDeviceToHost, g_rb_stream) != cudaSuccess ||
      cudaEventRecord(g_rb_done[slot], g_rb_stream) != cudaSuccess)
    return set_error(cudaGetErrorString(cudaGetLastError()));
  return 0;
}
int b200_readback_wait(int slot) {
  if (slot < 0 || slot >= 8 || !g_rb_done[slot]) return ERROR_UNSUPPORTED;
  if (cudaEventSynchronize(g_rb_done[slot]) != cudaSuccess) return set_error(cudaGetErrorString(cudaGetLastError()));
  return 0;
}

void* b200_host_alloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMallocHost(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
void b200_host_free(void* p) {
  if (p) cudaFreeHost(p);
}

// cudamat/cudamat.cu:217-229.
int copy_on_device(cudamat* mat1, cudamat* mat2) {
  if (!same_shape(mat1, mat2)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (!mat1->on_device || !mat2->on_device) return ERROR_NOT_ON_DEVICE;
  if (cudaMemcpyAsync(mat2->data_device, mat1->data_device, (size_t)numel(mat1) * sizeof(float),
                      cudaMemcpyDeviceToDevice, stream()) != cudaSuccess)
    return set_error("copy_on_device failed");
  return 0;
}

// cudamat/cudamat.cu:298-310.
int free_device_memory(cudamat* mat) {
  if (mat->owns_data && mat->on_device) {
    cudaStreamSynchronize(stream());
    if (cudaFree(mat->data_device) != cudaSuccess) {
      cudaGetLastError();
      return set_error("cudaFree failed");
    }
    mat->on_device = 0;
    mat->data_device = nullptr;
  }
  return 0;
}

// cudamat/cudamat.cu:312-329.
int set_shape(cudamat* mat, unsigned int m, unsigned int n) {
  mat->size[0] = (int)m;
  mat->size[1] = (int)n;
  return 0;
}
int reshape(cudamat* mat, unsigned int m, unsigned int n) {
  if ((long)mat->size[0] * mat->size[1] != (long)m * n) return ERROR_INCOMPATIBLE_DIMENSIONS;
  mat->size[0] = (int)m;
  mat->size[1] = (int)n;
  return 0;
}

// cudamat/cudamat.cu:331-353: non-owning view of columns [first_col, last_col).
int get_slice(cudamat* source, cudamat* target, unsigned int first_col, unsigned int last_col) {
  if (source->is_trans) return ERROR_TRANSPOSED;
  if (!source->on_device) return ERROR_NOT_ON_DEVICE;
  if (last_col > (unsigned)source->size[1] || first_col >= last_col) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int num_rows = source->size[0];
  target->data_host = nullptr;
  target->data_device = source->data_device + (size_t)first_col * num_rows;
  target->on_device = 1;
  target->on_host = 0;
  target->size[0] = source->size[0];
  target->size[1] = (int)(last_col - first_col);
  target->is_trans = 0;
  target->owns_data = 0;
  return 0;
}

// cudamat/cudamat.cu:355-395: view of a range of a row or column vector.
int get_vector_slice(cudamat* source, cudamat* target, unsigned int first_ind, unsigned int last_ind) {
  if (source->size[0] > 1 && source->size[1] > 1) return ERROR_GENERIC;
  if (source->is_trans) return ERROR_TRANSPOSED;
  if (!source->on_device) return ERROR_NOT_ON_DEVICE;
  if (first_ind >= last_ind) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const unsigned int len = last_ind - first_ind;
  if (source->size[0] > 1) {
    if (last_ind > (unsigned)source->size[0]) return ERROR_INCOMPATIBLE_DIMENSIONS;
    target->size[0] = (int)len;
    target->size[1] = 1;
  } else {
    if (last_ind > (unsigned)source->size[1]) return ERROR_INCOMPATIBLE_DIMENSIONS;
    target->size[0] = 1;
    target->size[1] = (int)len;
  }
  target->data_host = nullptr;
  target->data_device = source->data_device + first_ind;
  target->on_device = 1;
  target->on_host = 0;
  target->is_trans = 0;
  target->owns_data = 0;
  return 0;
}

// cudamat/cudamat.cu:397-405.
void init_from_array(cudamat* mat, float* data, int m, int n) {
  mat->data_host = data;
  mat->data_device = nullptr;
  mat->size[0] = m;
  mat->size[1] = n;
  mat->on_device = 0;
  mat->on_host = 1;
  mat->is_trans = 0;
  mat->owns_data = 1;
}

void set_on_device(cudamat* mat) { mat->on_device = 1; }

// cudamat/cudamat.cu:425-435.  The memory is zero-filled, as eigenmat's empty() is
// (eigenmat/eigenmat.py:1339-1343).
int init_empty(cudamat* mat, int m, int n) {
  mat->data_host = nullptr;
  mat->size[0] = m;
  mat->size[1] = n;
  mat->on_device = 0;
  mat->on_host = 0;
  mat->is_trans = 0;
  mat->owns_data = 1;
  int err = allocate_device_memory(mat);
  if (err) return err;
  if (cudaMemsetAsync(mat->data_device, 0, (size_t)numel(mat) * sizeof(float), stream()) != cudaSuccess)
    return set_error("cudaMemsetAsync failed");
  return 0;
}

}  // extern "C"
