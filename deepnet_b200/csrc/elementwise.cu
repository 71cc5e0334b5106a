// Elementwise, scalar, comparison and broadcast operations of the cudamat C ABI
// (cudamat/cudamat.cu:592-1146, 1318-1670, 1763-2102).  Each is one grid-stride kernel
// with 128-bit loads and stores where the operands are 16-byte aligned; the grid is a
// multiple of the SM count.  All are HBM-bound: bytes = 4 * (inputs + outputs) per element.
#include "common.cuh"

using namespace b200;

namespace {

constexpr int kThreads = 256;

inline int grid_for(long work_items) {
  long blocks = (work_items + kThreads - 1) / kThreads;
  long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// ---- unary -------------------------------------------------------------------
template <class F>
__global__ void __launch_bounds__(kThreads) k_map1(const float* a, float* t, long n, bool vec,
                                                   F f) {
  grid_dependents_launch();
  grid_dependency_wait();
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  if (vec) {
    const long n4 = n >> 2;
    for (long i = tid; i < n4; i += nth) {
      float4 x = reinterpret_cast<const float4*>(a)[i];
      x.x = f(x.x); x.y = f(x.y); x.z = f(x.z); x.w = f(x.w);
      reinterpret_cast<float4*>(t)[i] = x;
    }
    for (long i = (n4 << 2) + tid; i < n; i += nth) t[i] = f(a[i]);
  } else {
    for (long i = tid; i < n; i += nth) t[i] = f(a[i]);
  }
}

template <class F>
__global__ void __launch_bounds__(kThreads) k_map2(const float* a, const float* b, float* t, long n, bool vec, F f) {
  grid_dependents_launch();
  grid_dependency_wait();
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  if (vec) {
    const long n4 = n >> 2;
    for (long i = tid; i < n4; i += nth) {
      float4 x = reinterpret_cast<const float4*>(a)[i];
      const float4 y = reinterpret_cast<const float4*>(b)[i];
      x.x = f(x.x, y.x); x.y = f(x.y, y.y); x.z = f(x.z, y.z); x.w = f(x.w, y.w);
      reinterpret_cast<float4*>(t)[i] = x;
    }
    for (long i = (n4 << 2) + tid; i < n; i += nth) t[i] = f(a[i], b[i]);
  } else {
    for (long i = tid; i < n; i += nth) t[i] = f(a[i], b[i]);
  }
}

__global__ void __launch_bounds__(kThreads) k_fill(float* __restrict__ t, long n, bool vec, float v) {
  grid_dependents_launch();
  grid_dependency_wait();
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  if (vec) {
    const long n4 = n >> 2;
    const float4 x = make_float4(v, v, v, v);
    for (long i = tid; i < n4; i += nth) reinterpret_cast<float4*>(t)[i] = x;
    for (long i = (n4 << 2) + tid; i < n; i += nth) t[i] = v;
  } else {
    for (long i = tid; i < n; i += nth) t[i] = v;
  }
}

// Broadcast of a column vector (indexed by row) or a row vector (indexed by column).
// One thread handles 4 consecutive rows of one column when h % 4 == 0.
template <bool kByRow, class F>
__global__ void __launch_bounds__(kThreads) k_bcast(const float* m, const float* v, float* t, int h, int w, bool vec, F f) {
  grid_dependents_launch();
  grid_dependency_wait();
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  if (vec) {
    const int h4 = h >> 2;
    const long n4 = (long)h4 * w;
    for (long i = tid; i < n4; i += nth) {
      const int c = (int)(i / h4), r = (int)(i - (long)c * h4) << 2;
      float4 x = reinterpret_cast<const float4*>(m)[i];
      if (kByRow) {
        const float s = v[c];
        x.x = f(x.x, s); x.y = f(x.y, s); x.z = f(x.z, s); x.w = f(x.w, s);
      } else {
        const float4 s = *reinterpret_cast<const float4*>(v + r);
        x.x = f(x.x, s.x); x.y = f(x.y, s.y); x.z = f(x.z, s.z); x.w = f(x.w, s.w);
      }
      reinterpret_cast<float4*>(t)[i] = x;
    }
  } else {
    const long n = (long)h * w;
    for (long i = tid; i < n; i += nth) {
      const int c = (int)(i / h), r = (int)(i - (long)c * h);
      t[i] = f(m[i], kByRow ? v[c] : v[r]);
    }
  }
}

template <class F>
int map1(cudamat* mat, cudamat* target, F f) {
  if (!mat->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (mat->is_trans != target->is_trans) return ERROR_TRANSPOSEDNESS;
  if (!same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long n = numel(mat);
  if (n == 0) return 0;
  const bool vec = aligned16(mat->data_device) && aligned16(target->data_device);
  (void)launch_dependent(k_map1<F>, dim3(grid_for(vec ? (n + 3) / 4 : n)), dim3(kThreads), 0, stream(), mat->data_device,
                         target->data_device, n, vec, f);
  return check_launch();
}

template <class F>
int map2(cudamat* mat1, cudamat* mat2, cudamat* target, F f) {
  if (!mat1->on_device || !mat2->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (mat1->is_trans != mat2->is_trans) return ERROR_TRANSPOSEDNESS;
  if (!same_shape(mat1, mat2) || !same_shape(mat1, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long n = numel(mat1);
  if (n == 0) return 0;
  const bool vec = aligned16(mat1->data_device) && aligned16(mat2->data_device) && aligned16(target->data_device);
  (void)launch_dependent(k_map2<F>, dim3(grid_for(vec ? (n + 3) / 4 : n)), dim3(kThreads), 0, stream(), mat1->data_device,
                         mat2->data_device, target->data_device, n, vec, f);
  return check_launch();
}

template <bool kByRow, class F>
int bcast(cudamat* mat, cudamat* vec, cudamat* target, F f) {
  if (!mat->on_device || !vec->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (mat->is_trans) return ERROR_TRANSPOSED;
  const int h = mat->size[0], w = mat->size[1];
  if (kByRow) {
    if (w != vec->size[1] || vec->size[0] != 1 || !same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  } else {
    if (h != vec->size[0] || vec->size[1] != 1 || !same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  }
  if ((long)h * w == 0) return 0;
  const bool v4 = (h % 4 == 0) && aligned16(mat->data_device) && aligned16(target->data_device) &&
                  aligned16(vec->data_device);
  const long items = v4 ? (long)(h / 4) * w : (long)h * w;
  (void)launch_dependent(k_bcast<kByRow, F>, dim3(grid_for(items)), dim3(kThreads), 0, stream(), mat->data_device,
                         vec->data_device, target->data_device, h, w, v4, f);
  return check_launch();
}

// ---- functors ----------------------------------------------------------------
struct FSigmoid { __device__ float operator()(float x) const { return sigmoid_accurate(x); } };
struct FExp { __device__ float operator()(float x) const { return expf(x); } };
struct FTanh { __device__ float operator()(float x) const { return tanhf(x); } };
struct FAbs { __device__ float operator()(float x) const { return fabsf(x); } };
struct FSqrt { __device__ float operator()(float x) const { return sqrtf(x); } };
struct FRecip { __device__ float operator()(float x) const { return 1.0f / x; } };
struct FSign { __device__ float operator()(float x) const { return x < 0 ? -1.0f : (x > 0 ? 1.0f : 0.0f); } };
struct FLog { float tiny; __device__ float operator()(float x) const { return logf(x + tiny); } };
struct FLog1pExp {
  __device__ float operator()(float x) const { return x > 0 ? x + log1pf(expf(-x)) : log1pf(expf(x)); }
};
struct FPow { float p; __device__ float operator()(float x) const { return powf(x, p); } };
struct FMulS { float s; __device__ float operator()(float x) const { return x * s; } };
struct FDivS { float s; __device__ float operator()(float x) const { return x / s; } };
struct FAddS { float s; __device__ float operator()(float x) const { return x + s; } };
struct FLtS { float s; __device__ float operator()(float x) const { return x < s ? 1.0f : 0.0f; } };
struct FLeS { float s; __device__ float operator()(float x) const { return x <= s ? 1.0f : 0.0f; } };
struct FGtS { float s; __device__ float operator()(float x) const { return x > s ? 1.0f : 0.0f; } };
struct FGeS { float s; __device__ float operator()(float x) const { return x >= s ? 1.0f : 0.0f; } };
struct FUbS { float s; __device__ float operator()(float x) const { return x > s ? s : x; } };
struct FLbS { float s; __device__ float operator()(float x) const { return x < s ? s : x; } };

struct FAdd { __device__ float operator()(float a, float b) const { return a + b; } };
struct FSub { __device__ float operator()(float a, float b) const { return a - b; } };
struct FMul { __device__ float operator()(float a, float b) const { return a * b; } };
struct FDiv { __device__ float operator()(float a, float b) const { return a / b; } };
struct FLt { __device__ float operator()(float a, float b) const { return a < b ? 1.0f : 0.0f; } };
struct FLe { __device__ float operator()(float a, float b) const { return a <= b ? 1.0f : 0.0f; } };
struct FGt { __device__ float operator()(float a, float b) const { return a > b ? 1.0f : 0.0f; } };
struct FGe { __device__ float operator()(float a, float b) const { return a >= b ? 1.0f : 0.0f; } };
struct FUb { __device__ float operator()(float a, float b) const { return a > b ? b : a; } };
struct FLb { __device__ float operator()(float a, float b) const { return a < b ? b : a; } };
struct FAxpy { float s; __device__ float operator()(float a, float b) const { return a + b * s; } };
struct FAddMultSign {
  float s;
  __device__ float operator()(float a, float b) const { return a + (b == 0 ? 0.0f : (b > 0 ? s : -s)); }
};
struct FLogisticDeriv { __device__ float operator()(float a, float b) const { return a * b * (1.0f - b); } };
struct FCeBernoulli {
  float tiny;
  __device__ float operator()(float t, float p) const {
    return -t * logf(p + tiny) - (1.0f - t) * logf(1.0f - p + tiny);
  }
};
struct FCorrectPreds {
  float cutoff;
  __device__ float operator()(float t, float p) const { return t * (p >= cutoff) + (1.0f - t) * (p < cutoff); }
};

}  // namespace

extern "C" {

// cudamat/cudamat.cu:592-615, 617-639.
int add_col_vec(cudamat* mat, cudamat* vec, cudamat* target) { return bcast<false>(mat, vec, target, FAdd()); }
int add_col_mult(cudamat* mat, cudamat* vec, cudamat* target, float mult) {
  return bcast<false>(mat, vec, target, FAxpy{mult});
}
// cudamat/cudamat.cu:735-781.
int add_row_mult(cudamat* mat, cudamat* vec, cudamat* target, float mult) {
  return bcast<true>(mat, vec, target, FAxpy{mult});
}
int add_row_vec(cudamat* mat, cudamat* vec, cudamat* target) { return bcast<true>(mat, vec, target, FAdd()); }
// cudamat/cudamat.cu:783-876.
int mult_by_col_vec(cudamat* mat, cudamat* vec, cudamat* target) { return bcast<false>(mat, vec, target, FMul()); }
int mult_by_row_vec(cudamat* mat, cudamat* vec, cudamat* target) { return bcast<true>(mat, vec, target, FMul()); }
int div_by_col_vec(cudamat* mat, cudamat* vec, cudamat* target) { return bcast<false>(mat, vec, target, FDiv()); }
int div_by_row_vec(cudamat* mat, cudamat* vec, cudamat* target) { return bcast<true>(mat, vec, target, FDiv()); }

// cudamat/cudamat.cu:878-1146: comparisons and clamps write 0/1 (or the clamped value).
int less_than(cudamat* a, cudamat* b, cudamat* t) { return map2(a, b, t, FLt()); }
int less_than_eq(cudamat* a, cudamat* b, cudamat* t) { return map2(a, b, t, FLe()); }
int greater_than(cudamat* a, cudamat* b, cudamat* t) { return map2(a, b, t, FGt()); }
int greater_than_eq(cudamat* a, cudamat* b, cudamat* t) { return map2(a, b, t, FGe()); }
int upper_bound(cudamat* a, cudamat* b, cudamat* t) { return map2(a, b, t, FUb()); }
int lower_bound(cudamat* a, cudamat* b, cudamat* t) { return map2(a, b, t, FLb()); }
int less_than_scalar(cudamat* a, float v, cudamat* t) { return map1(a, t, FLtS{v}); }
int less_than_eq_scalar(cudamat* a, float v, cudamat* t) { return map1(a, t, FLeS{v}); }
int greater_than_scalar(cudamat* a, float v, cudamat* t) { return map1(a, t, FGtS{v}); }
int greater_than_eq_scalar(cudamat* a, float v, cudamat* t) { return map1(a, t, FGeS{v}); }
int upper_bound_scalar(cudamat* a, float v, cudamat* t) { return map1(a, t, FUbS{v}); }
int lower_bound_scalar(cudamat* a, float v, cudamat* t) { return map1(a, t, FLbS{v}); }

// cudamat/cudamat.cu:1318-1670.
int sign(cudamat* mat, cudamat* target) { return map1(mat, target, FSign()); }
int apply_sigmoid(cudamat* mat, cudamat* target) { return map1(mat, target, FSigmoid()); }
int apply_tanh(cudamat* mat, cudamat* target) { return map1(mat, target, FTanh()); }
int apply_abs(cudamat* mat, cudamat* target) { return map1(mat, target, FAbs()); }
int apply_log_1_plus_exp(cudamat* mat, cudamat* target) { return map1(mat, target, FLog1pExp()); }
int apply_log(cudamat* mat, cudamat* target, float tiny) { return map1(mat, target, FLog{tiny}); }
int apply_exp(cudamat* mat, cudamat* target) { return map1(mat, target, FExp()); }
int apply_sqrt(cudamat* mat, cudamat* target) { return map1(mat, target, FSqrt()); }
int apply_pow(cudamat* mat, float p, cudamat* target) { return map1(mat, target, FPow{p}); }
int reciprocal(cudamat* mat, cudamat* target) { return map1(mat, target, FRecip()); }
int compute_cross_entropy_bernoulli(cudamat* mat, cudamat* p, cudamat* target, float tiny) {
  return map2(mat, p, target, FCeBernoulli{tiny});
}
int correct_preds(cudamat* mat, cudamat* p, cudamat* target, float cutoff) {
  return map2(mat, p, target, FCorrectPreds{cutoff});
}
int apply_logistic_deriv(cudamat* mat1, cudamat* mat2, cudamat* target) {
  return map2(mat1, mat2, target, FLogisticDeriv());
}

// cudamat/cudamat.cu:1763-1894.
int add_mult(cudamat* mat1, cudamat* mat2, float alpha) { return map2(mat1, mat2, mat1, FAxpy{alpha}); }
int add_mult_sign(cudamat* mat1, cudamat* mat2, float mult) { return map2(mat1, mat2, mat1, FAddMultSign{mult}); }
int add_elementwise(cudamat* a, cudamat* b, cudamat* t) { return map2(a, b, t, FAdd()); }
int subtract_elementwise(cudamat* a, cudamat* b, cudamat* t) { return map2(a, b, t, FSub()); }
int divide_elementwise(cudamat* a, cudamat* b, cudamat* t) { return map2(a, b, t, FDiv()); }
int mult_elementwise(cudamat* a, cudamat* b, cudamat* t) { return map2(a, b, t, FMul()); }

// cudamat/cudamat.cu:2031-2102.
int assign_scalar(cudamat* mat, float alpha) {
  if (!mat->on_device) return ERROR_NOT_ON_DEVICE;
  const long n = numel(mat);
  if (n == 0) return 0;
  const bool vec = aligned16(mat->data_device);
  (void)launch_dependent(k_fill, dim3(grid_for(vec ? (n + 3) / 4 : n)), dim3(kThreads), 0, stream(), mat->data_device, n, vec, alpha);
  return check_launch();
}
int mult_by_scalar(cudamat* mat, float alpha, cudamat* target) { return map1(mat, target, FMulS{alpha}); }
int divide_by_scalar(cudamat* mat, float alpha, cudamat* target) { return map1(mat, target, FDivS{alpha}); }
int add_scalar(cudamat* mat, float alpha, cudamat* target) { return map1(mat, target, FAddS{alpha}); }

}  // extern "C"
