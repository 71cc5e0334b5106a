// Shared declarations of the b200mat library: the matrix handle, error codes, the
// library stream, launch helpers and the counter-based random stream.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Error codes of the reference C ABI (cudamat/cudamat.cuh:1-9) plus two new ones.
#define ERROR_INCOMPATIBLE_DIMENSIONS -1
#define CUBLAS_ERROR -2
#define CUDA_ERROR -3
#define VIEW_ERROR -4
#define ERROR_TRANSPOSED -5
#define ERROR_GENERIC -6
#define ERROR_TRANSPOSEDNESS -7
#define ERROR_NOT_ON_DEVICE -8
#define ERROR_UNSUPPORTED -9
#define ERROR_NCCL -10
#define ERROR_DEVICE_TIMEOUT -11

// Matrix handle, binary-compatible with cudamat/cudamat.cuh:21-29: float32,
// column-major, size[0] rows by size[1] columns, owned by the Python caller.
struct cudamat {
  float* data_host;
  float* data_device;
  int on_device;
  int on_host;
  int size[2];
  int is_trans;  // 0 or 1
  int owns_data;
};

// Random state.  Same size as the reference's two-pointer struct
// (cudamat/cudamat.cuh:31-34) so an unmodified wrapper can allocate it; it holds the
// Philox key and the number of sampling calls issued so far.
struct rnd_struct {
  unsigned long long seed;
  unsigned long long calls;
};

namespace b200 {

cudaStream_t stream();                 // the stream every operation of the library runs on
cudaStream_t stream_if_initialised();  // the same, or the default stream when the library was never initialised
int sm_count();                        // SMs of the current device
int check_launch();                    // cudaGetLastError -> 0 or CUDA_ERROR (message kept); CUDA_ERROR when the library failed to initialise
int check_launch_any_stream();         // the same for entry points that also run without the library stream
int set_error(const char* msg);        // records msg, returns CUDA_ERROR
int rng_col0();                        // first global column of this process's minibatch shard
void* workspace(int slot, size_t bytes);  // grow-only cached device scratch, slot 0..7
void* workspace_zeroed(int slot, size_t bytes);  // the same, cleared when first handed out or regrown (counters left at zero by their users)
int* status_word();                    // device int: non-zero after a bounded wait gave up
bool initialised();                    // the library stream and status word exist (tries to create them)
uint32_t wait_limit();                 // iterations a bounded device-side wait may spin (b200_set_wait_limit)

bool dependent_launch_enabled();       // b200_set_dependent_launch / B200_DEPENDENT_LAUNCH (default on)

// Programmatic dependent launch.  A kernel started with launch_dependent() may be scheduled while
// the kernel before it on the stream is still running (its blocks become resident, run their
// prologue and then block in grid_dependency_wait() until the predecessor has completed and its
// writes are visible).  RULE: every kernel launched this way calls grid_dependency_wait() on every
// thread before its first access to global memory; grid_dependents_launch() (optional, at the top)
// lets the successor be scheduled before this kernel's blocks exit.  Both are no-ops in a kernel
// that was launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline long numel(const cudamat* m) { return (long)m->size[0] * m->size[1]; }
inline bool same_shape(const cudamat* a, const cudamat* b) {
  return a->size[0] == b->size[0] && a->size[1] == b->size[1];
}

// ---------------------------------------------------------------- Philox4x32-10
// Element (row r, column c) of sampling call `call` under `seed` takes word (c & 3) of
// philox(ctr = {r, c >> 2, call_lo, call_hi}, key = {seed_lo, seed_hi}); c is the global
// column (local column + the shard's first column).  The layout depends on neither the
// launch shape nor the number of GPUs.
struct PhiloxKey {
  uint32_t k0, k1, c2, c3;  // key words and the call counter words
};

__host__ __device__ inline PhiloxKey make_philox_key(unsigned long long seed, unsigned long long call) {
  PhiloxKey k;
  k.k0 = (uint32_t)seed;
  k.k1 = (uint32_t)(seed >> 32);
  k.c2 = (uint32_t)call;
  k.c3 = (uint32_t)(call >> 32);
  return k;
}

#ifdef __CUDACC__
__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, const PhiloxKey& key) {
  uint32_t c2 = key.c2, c3 = key.c3, k0 = key.k0, k1 = key.k1;
#pragma unroll
  for (int r = 0; r < 10; r++) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// Word -> uniform in (0, 1], the reference mapping (cudamat/cudamat_kernels.cu:120).
__device__ __forceinline__ float word_to_uniform(uint32_t x) {
  return __fmul_rn(__fadd_rn(__uint2float_rn(x), 1.0f), 2.3283064365386963e-10f);
}

__device__ __forceinline__ uint32_t pick_word(const uint4& w, int i) {
  return i == 0 ? w.x : (i == 1 ? w.y : (i == 2 ? w.z : w.w));
}

// 1 / (1 + exp(-x)) to about 4e-7 relative (the reference's fast __expf of
// cudamat_kernels.cu:404 loses up to 5e-6 at large |x| and would miss the 1e-5 bound against
// libm).  exp(-x) = 2^y with y = -x * log2(e): the rounding of that product (exact residual
// by fma) and the part of log2(e) a float drops are folded back as 2^y * (1 + r * ln 2), so
// only the two special-function units' own errors remain (ex2.approx 2 ulp, rcp.approx
// 1 ulp).  Branch-free: libm's expf and the correctly rounded reciprocal, with their range
// checks and slow paths, made the tensor-core epilogue three times slower.  Saturates like
// the quotient: 2^y = inf gives 0, a flushed 2^y gives 1, NaN stays NaN.
__device__ __forceinline__ float sigmoid_accurate(float x) {
  const float kL = -1.4426950408889634f;        // -log2(e) rounded to float
  const float kLlo = -1.9259629911e-8f;         // -(log2(e) - float(log2(e)))
  const float y = x * kL;
  float r = fmaf(x, kL, -y);
  r = fmaf(x, kLlo, r);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(y));
  // r is finite and tiny whenever e is finite and non-zero; e = inf or 0 must stay so
  const float e2 = fmaf(e, r * 0.6931471805599453f, e);
  e = (fabsf(y) < 126.0f) ? e2 : e;
  float p;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(1.0f + e));
  return p;
}

// Split x = hi + lo with hi exactly representable in TF32 (low 13 mantissa bits zero)
// and lo = x - hi (exact in fp32).  The tensor core reads only the TF32 bits of lo.
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
  lo = (fabsf(hi) <= 3.4028234e38f) ? x - hi : 0.0f;  // inf/nan stay in hi alone
}

// bfloat16 (the upper 16 bits of a float), round to nearest even; inf and NaN keep their class.
__device__ __forceinline__ uint16_t float_to_bf16(float x) {
  const uint32_t u = __float_as_uint(x);
  if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)((u >> 16) | ((u & 0xffffu) ? 0x40u : 0u));
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ float bf16_to_float(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

// The bfloat16 companion ("aux matrix") of a rows x cols fp32 matrix x, for products that read
// the bfloat16 parts of x from memory instead of deriving them from x in the kernel: lda x cols
// floats of storage, lda = rows rounded up to a multiple of 8 (both planes of every column then
// start on 16 bytes, as TMA requires); column c holds two runs of lda bfloat16, the first
// `rows` of each in use,
//   plane 0: bf16(x - tf32(x))      plane 1: bf16(x)
// Element (r, c) of plane p is 16-bit word  c * 2 * lda + p * lda + r  of the aux storage.
__device__ __forceinline__ void split_aux(float x, uint16_t& lo16, uint16_t& b16) {
  float hi, lo;
  split_tf32(x, hi, lo);
  lo16 = float_to_bf16(lo);
  b16 = float_to_bf16(x);
}

// The same storage can hold the SCALED HALF-PRECISION form of x instead: with xs = x * 2^e,
//   plane 1: hi = fp16(xs)      plane 0: lo = fp16(xs - hi)
// hi + lo carries 22 significant bits of xs, and
//   a . b * 2^(ea + eb) ~= hi(a).hi(b) + hi(a).lo(b) + lo(a).hi(b)
// is three half-precision products (K = 16 per tcgen05.mma, exact in the fp32 accumulator), no
// TF32 term and no fp32 operand tile at all; what is left out (lo.lo and the rounding of lo) is
// below 2^-21 of |a||b| per term.  e is chosen so that the largest |xs| stays well inside the
// fp16 range (65504): a power of two, so the scaling is exact and the epilogue undoes it with
// alpha * 2^-(ea + eb).  Entries more than 2^14 below the largest lose relative (not absolute)
// precision in lo.
// A value that outgrows its exponent saturates at the largest fp16 instead of becoming infinite.
__device__ __forceinline__ void split_f16(float x, float scale, uint16_t& lo, uint16_t& hi) {
  const float xs = fminf(fmaxf(x * scale, -65504.0f), 65504.0f);
  const __half h = __float2half_rn(xs);
  const __half l = __float2half_rn(xs - __half2float(h));
  hi = __half_as_ushort(h);
  lo = __half_as_ushort(l);
}
__device__ __forceinline__ float f16_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

#endif

__host__ __device__ inline int aux_rows(int rows) { return (rows + 7) & ~7; }

}  // namespace b200
