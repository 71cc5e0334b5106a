// Reductions of the C ABI: sums and maxima along an axis, arg-max one-hot sampling
// helpers, column softmax and the scalar reductions that return to the host
// (cudamat/cudamat.cu:1148-1258, 1733-1759, 2104-2118, 2192-2240; the axis sums replace
// the reference's GEMV with a ones vector, cudamat/cudamat.py:724-748,1546-1577).
// Warp-shuffle trees inside a block; HBM-bound: 4 bytes read per input element.
#include <mutex>

#include "common.cuh"

using namespace b200;

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <class T>
__device__ __forceinline__ T block_sum(T v, T* smem) {  // smem: 32 entries; result valid in every thread
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  T r = (lane < nw) ? smem[lane] : T(0);
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* smem) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  float r = (lane < nw) ? smem[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

// First-maximum arg-max: (value, index) pairs, ties to the smaller index, which equals
// the sequential `if (d[am] < d[r]) am = r` scan of eigenmat/eigenmat.cc:650-652.
__device__ __forceinline__ void argmax_combine(float& v, int& i, float v2, int i2) {
  if (v2 > v || (v2 == v && i2 < i)) {
    v = v2;
    i = i2;
  }
}
__device__ __forceinline__ void block_argmax(float& v, int& i, float* sv, int* si) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, i, o);
    argmax_combine(v, i, v2, i2);
  }
  __syncthreads();
  if (lane == 0) {
    sv[wid] = v;
    si[wid] = i;
  }
  __syncthreads();
  v = (lane < nw) ? sv[lane] : -INFINITY;
  i = (lane < nw) ? si[lane] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, i, o);
    argmax_combine(v, i, v2, i2);
  }
}

// ---- sum down each column (contiguous): one block per column -----------------
__global__ void __launch_bounds__(256) k_colsum(const float* __restrict__ m, float* __restrict__ t, int h, int w,
                                                float mult, float beta) {
  __shared__ float smem[32];
  for (int c = blockIdx.x; c < w; c += gridDim.x) {
    const float* col = m + (long)c * h;
    float s = 0;
    if ((h & 3) == 0 && (((uintptr_t)col) & 15) == 0) {
      const float4* col4 = reinterpret_cast<const float4*>(col);
      for (int r = threadIdx.x; r < (h >> 2); r += blockDim.x) {
        const float4 x = col4[r];
        s += (x.x + x.y) + (x.z + x.w);
      }
    } else {
      for (int r = threadIdx.x; r < h; r += blockDim.x) s += col[r];
    }
    s = block_sum(s, smem);
    if (threadIdx.x == 0) t[c] = (beta == 0 ? 0.0f : beta * t[c]) + mult * s;
  }
}

// ---- sum across columns for each row (strided) --------------------------------
// Block = 32 rows x 8 column lanes; blockIdx.y splits the columns.  With one split the
// block writes the result, otherwise a partial row into scratch[split][h].
constexpr int kRowLanes = 8;
__global__ void __launch_bounds__(32 * kRowLanes) k_rowsum(const float* __restrict__ m, float* __restrict__ out,
                                                           int h, int w, int cols_per_split, float mult, float beta,
                                                           bool final_pass) {
  __shared__ float smem[kRowLanes][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int r = blockIdx.x * 32 + tx;
  const int c0 = blockIdx.y * cols_per_split;
  const int c1 = min(w, c0 + cols_per_split);
  float s = 0;
  if (r < h) {
    int c = c0 + ty;
    // four independent loads in flight per thread
    for (; c + 3 * kRowLanes < c1; c += 4 * kRowLanes) {
      const float a0 = m[(long)c * h + r], a1 = m[(long)(c + kRowLanes) * h + r];
      const float a2 = m[(long)(c + 2 * kRowLanes) * h + r], a3 = m[(long)(c + 3 * kRowLanes) * h + r];
      s += (a0 + a1) + (a2 + a3);
    }
    for (; c < c1; c += kRowLanes) s += m[(long)c * h + r];
  }
  smem[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && r < h) {
    float tot = 0;
#pragma unroll
    for (int j = 0; j < kRowLanes; j++) tot += smem[j][tx];
    if (final_pass)
      out[r] = (beta == 0 ? 0.0f : beta * out[r]) + mult * tot;
    else
      out[(long)blockIdx.y * h + r] = tot;
  }
}
// Same sums with 128-bit loads: a thread owns 4 consecutive rows, a block 128 rows x 8 column
// lanes, and enough column splits are launched to keep every SM several blocks deep.
__global__ void __launch_bounds__(32 * kRowLanes) k_rowsum4(const float* __restrict__ m, float* __restrict__ out,
                                                            int h, int w, int cols_per_split, float mult, float beta,
                                                            bool final_pass) {
  __shared__ float4 smem[kRowLanes][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int r = (blockIdx.x * 32 + tx) * 4;
  const int c0 = blockIdx.y * cols_per_split;
  const int c1 = min(w, c0 + cols_per_split);
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (r < h) {
    const float* base = m + r;
    int c = c0 + ty;
    for (; c + 3 * kRowLanes < c1; c += 4 * kRowLanes) {
      const float4 a0 = *reinterpret_cast<const float4*>(base + (long)c * h);
      const float4 a1 = *reinterpret_cast<const float4*>(base + (long)(c + kRowLanes) * h);
      const float4 a2 = *reinterpret_cast<const float4*>(base + (long)(c + 2 * kRowLanes) * h);
      const float4 a3 = *reinterpret_cast<const float4*>(base + (long)(c + 3 * kRowLanes) * h);
      s.x += (a0.x + a1.x) + (a2.x + a3.x);
      s.y += (a0.y + a1.y) + (a2.y + a3.y);
      s.z += (a0.z + a1.z) + (a2.z + a3.z);
      s.w += (a0.w + a1.w) + (a2.w + a3.w);
    }
    for (; c < c1; c += kRowLanes) {
      const float4 a = *reinterpret_cast<const float4*>(base + (long)c * h);
      s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w;
    }
  }
  smem[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && r < h) {
    float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < kRowLanes; j++) {
      const float4 v = smem[j][tx];
      tot.x += v.x; tot.y += v.y; tot.z += v.z; tot.w += v.w;
    }
    if (final_pass) {
      float4 o = *reinterpret_cast<float4*>(out + r);
      o.x = (beta == 0 ? 0.0f : beta * o.x) + mult * tot.x;
      o.y = (beta == 0 ? 0.0f : beta * o.y) + mult * tot.y;
      o.z = (beta == 0 ? 0.0f : beta * o.z) + mult * tot.z;
      o.w = (beta == 0 ? 0.0f : beta * o.w) + mult * tot.w;
      *reinterpret_cast<float4*>(out + r) = o;
    } else {
      *reinterpret_cast<float4*>(out + (long)blockIdx.y * h + r) = tot;
    }
  }
}
__global__ void __launch_bounds__(256) k_rowsum_finish(const float* __restrict__ part, float* __restrict__ t, int h,
                                                       int splits, float mult, float beta) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= h) return;
  float tot = 0;
  for (int s = 0; s < splits; s++) tot += part[(long)s * h + r];
  t[r] = (beta == 0 ? 0.0f : beta * t[r]) + mult * tot;
}

// ---- column max / arg-max / one-hot -------------------------------------------
__global__ void __launch_bounds__(256) k_colmax(const float* __restrict__ m, float* __restrict__ t, int h, int w) {
  __shared__ float smem[32];
  for (int c = blockIdx.x; c < w; c += gridDim.x) {
    const float* col = m + (long)c * h;
    float v = -INFINITY;
    for (int r = threadIdx.x; r < h; r += blockDim.x) v = fmaxf(v, col[r]);
    v = block_max(v, smem);
    if (threadIdx.x == 0) t[c] = v;
  }
}
__global__ void __launch_bounds__(256) k_rowmax(const float* __restrict__ m, float* __restrict__ t, int h, int w) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= h) return;
  float v = m[r];
  for (int c = 1; c < w; c++) v = fmaxf(v, m[(long)c * h + r]);
  t[r] = v;
}

// mode 0: target = one-hot; 1: acc[argmax] += 1; 2: target[c] = argmax
__global__ void __launch_bounds__(256) k_col_argmax(const float* m, float* t, int h, int w,
                                                    int mode) {
  __shared__ float sv[32];
  __shared__ int si[32];
  for (int c = blockIdx.x; c < w; c += gridDim.x) {
    const float* col = m + (long)c * h;
    float v = -INFINITY;
    int i = 0x7fffffff;
    for (int r = threadIdx.x; r < h; r += blockDim.x) argmax_combine(v, i, col[r], r);
    block_argmax(v, i, sv, si);
    if (i == 0x7fffffff) i = 0;  // all-NaN column: the sequential scan keeps index 0
    if (mode == 0) {
      float* tc = t + (long)c * h;
      __syncthreads();  // every thread has read its part of the column (t may alias m)
      for (int r = threadIdx.x; r < h; r += blockDim.x) tc[r] = (r == i) ? 1.0f : 0.0f;
    } else if (threadIdx.x == 0) {
      if (mode == 1)
        t[(long)c * h + i] += 1.0f;
      else
        t[c] = (float)i;
    }
  }
}

// ---- column softmax -----------------------------------------------------------
__global__ void __launch_bounds__(256) k_softmax(const float* m, float* t, int h, int w) {
  __shared__ float smem[32];
  for (int c = blockIdx.x; c < w; c += gridDim.x) {
    const float* col = m + (long)c * h;
    float* tc = t + (long)c * h;
    float mx = -INFINITY;
    for (int r = threadIdx.x; r < h; r += blockDim.x) mx = fmaxf(mx, col[r]);
    mx = block_max(mx, smem);
    float s = 0;
    for (int r = threadIdx.x; r < h; r += blockDim.x) {
      const float e = expf(col[r] - mx);
      tc[r] = e;
      s += e;
    }
    s = block_sum(s, smem);
    for (int r = threadIdx.x; r < h; r += blockDim.x) tc[r] = tc[r] / s;
  }
}

// ---- scalar reductions --------------------------------------------------------
// mode 0: sum a; 1: sum a*a; 2: sum a*b; 3: sum (a-b)^2.  Stage 1 writes one double per
// block, stage 2 (one block) folds them.
__global__ void __launch_bounds__(256) k_scalar_partial(const float* __restrict__ a, const float* __restrict__ b,
                                                        long n, int mode, double* __restrict__ part) {
  __shared__ double smem[32];
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  double s = 0;
  long start = 0;
  if (((((uintptr_t)a) | (b ? (uintptr_t)b : 0)) & 15) == 0) {
    // 128-bit loads, four elements folded in fp32 before joining the fp64 running sum
    const long n4 = n >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    long i = tid;
    if (mode == 3) {
      // squared difference: two independent 128-bit load pairs in flight per thread
      for (; i + nth < n4; i += 2 * nth) {
        const float4 x0 = a4[i], y0 = b4[i], x1 = a4[i + nth], y1 = b4[i + nth];
        const float e0 = x0.x - y0.x, e1 = x0.y - y0.y, e2 = x0.z - y0.z, e3 = x0.w - y0.w;
        const float f0 = x1.x - y1.x, f1 = x1.y - y1.y, f2 = x1.z - y1.z, f3 = x1.w - y1.w;
        s += (double)((e0 * e0 + e1 * e1) + (e2 * e2 + e3 * e3)) + (double)((f0 * f0 + f1 * f1) + (f2 * f2 + f3 * f3));
      }
    }
    for (; i < n4; i += nth) {
      const float4 x = a4[i];
      float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
      if (mode >= 2) y = b4[i];
      if (mode == 3) {
        const float d0 = x.x - y.x, d1 = x.y - y.y, d2 = x.z - y.z, d3 = x.w - y.w;
        s += (double)(d0 * d0 + d1 * d1) + (double)(d2 * d2 + d3 * d3);
      } else if (mode == 0) {
        s += (double)(x.x + x.y) + (double)(x.z + x.w);
      } else if (mode == 1) {
        s += (double)(x.x * x.x + x.y * x.y) + (double)(x.z * x.z + x.w * x.w);
      } else {
        s += (double)(x.x * y.x + x.y * y.y) + (double)(x.z * y.z + x.w * y.w);
      }
    }
    start = n4 << 2;
  }
  for (long i = start + tid; i < n; i += nth) {
    const float x = a[i];
    if (mode == 3) {
      const float d = x - b[i];
      s += (double)d * d;
    } else {
      s += mode == 0 ? (double)x : (mode == 1 ? (double)x * x : (double)x * b[i]);
    }
  }
  s = block_sum(s, smem);
  if (threadIdx.x == 0) part[blockIdx.x] = s;
}
__global__ void __launch_bounds__(256) k_scalar_final(const double* __restrict__ part, int nparts,
                                                      double* __restrict__ out, float* acc) {
  __shared__ double smem[32];
  double s = 0;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += part[i];
  s = block_sum(s, smem);
  if (threadIdx.x == 0) {
    if (out) *out = s;
    if (acc) *acc += (float)s;
  }
}

int scalar_reduce(cudamat* a, cudamat* b, int mode, double* result) {
  if (!a->on_device || (b && !b->on_device)) return ERROR_NOT_ON_DEVICE;
  const long n = numel(a);
  int blocks = (int)((n + 255) / 256);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  double* part = (double*)workspace(1, (size_t)(blocks + 1) * sizeof(double));
  if (!part) return CUDA_ERROR;
  k_scalar_partial<<<blocks, 256, 0, stream()>>>(a->data_device, b ? b->data_device : nullptr, n, mode, part + 1);
  k_scalar_final<<<1, 256, 0, stream()>>>(part + 1, blocks, part, nullptr);
  int err = check_launch();
  if (err) return err;
  if (cudaMemcpyAsync(result, part, sizeof(double), cudaMemcpyDeviceToHost, stream()) != cudaSuccess)
    return set_error("scalar readback failed");
  if (cudaStreamSynchronize(stream()) != cudaSuccess) return set_error(cudaGetErrorString(cudaGetLastError()));
  return 0;
}

}  // namespace

namespace b200 {

// target (h or w entries) = beta*target + mult * sum along `axis` of the stored matrix.
int launch_axis_sum(const float* m, int h, int w, int axis, float* t, float mult, float beta) {
  if ((long)h * w == 0) return 0;
  if (axis == 0) {
    int blocks = w < sm_count() * 8 ? w : sm_count() * 8;
    k_colsum<<<blocks, 256, 0, stream()>>>(m, t, h, w, mult, beta);
    return check_launch();
  }
  const bool vec4 = (h % 4 == 0) && (((uintptr_t)m | (uintptr_t)t) & 15) == 0;
  const int rows_per_block = vec4 ? 128 : 32;
  const int bx = (h + rows_per_block - 1) / rows_per_block;
  // enough blocks for about two full waves of 8 resident blocks per SM
  int splits = (16 * sm_count() + bx - 1) / bx;
  const int max_splits = (w + 31) / 32;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  const int cps = (w + splits - 1) / splits;
  splits = (w + cps - 1) / cps;
  float* dst = t;
  if (splits > 1) {
    dst = (float*)workspace(0, (size_t)splits * h * sizeof(float));
    if (!dst) return CUDA_ERROR;
  }
  const bool final_pass = splits == 1;
  if (vec4)
    k_rowsum4<<<dim3(bx, splits), 32 * kRowLanes, 0, stream()>>>(m, dst, h, w, cps, final_pass ? mult : 1.0f,
                                                                final_pass ? beta : 0.0f, final_pass);
  else
    k_rowsum<<<dim3(bx, splits), 32 * kRowLanes, 0, stream()>>>(m, dst, h, w, cps, final_pass ? mult : 1.0f,
                                                               final_pass ? beta : 0.0f, final_pass);
  if (!final_pass) k_rowsum_finish<<<(h + 255) / 256, 256, 0, stream()>>>(dst, t, h, splits, mult, beta);
  return check_launch();
}

}  // namespace b200

extern "C" {

// eigenmat/eigenmat.cc:733-759 (cudamat builds the same from `dot` with a ones vector).
int add_sum_by_axis(cudamat* mat, cudamat* target, int axis, float mult) {
  if (!mat->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (axis != 0 && axis != 1) return ERROR_UNSUPPORTED;
  if (mat->is_trans) axis = 1 - axis;
  if (numel(target) != (axis == 0 ? mat->size[1] : mat->size[0])) return ERROR_INCOMPATIBLE_DIMENSIONS;
  return launch_axis_sum(mat->data_device, mat->size[0], mat->size[1], axis, target->data_device, mult, 1.0f);
}
int sum_by_axis(cudamat* mat, cudamat* target, int axis) {
  if (!mat->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (axis != 0 && axis != 1) return ERROR_UNSUPPORTED;
  if (mat->is_trans) axis = 1 - axis;
  if (numel(target) != (axis == 0 ? mat->size[1] : mat->size[0])) return ERROR_INCOMPATIBLE_DIMENSIONS;
  return launch_axis_sum(mat->data_device, mat->size[0], mat->size[1], axis, target->data_device, 1.0f, 0.0f);
}

// cudamat/cudamat.cu:1148-1176.
int max_by_axis(cudamat* mat, cudamat* target, int axis) {
  if (!mat->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (mat->is_trans) return ERROR_TRANSPOSED;
  const int h = mat->size[0], w = mat->size[1];
  if ((long)h * w == 0) return 0;
  if (axis == 0) {
    if (target->size[0] != 1 || target->size[1] != w) return ERROR_INCOMPATIBLE_DIMENSIONS;
    k_colmax<<<w < sm_count() * 8 ? w : sm_count() * 8, 256, 0, stream()>>>(mat->data_device, target->data_device, h, w);
  } else if (axis == 1) {
    if (target->size[1] != 1 || target->size[0] != h) return ERROR_INCOMPATIBLE_DIMENSIONS;
    k_rowmax<<<(h + 255) / 256, 256, 0, stream()>>>(mat->data_device, target->data_device, h, w);
  } else {
    return ERROR_UNSUPPORTED;
  }
  return check_launch();
}

// cudamat/cudamat.cu:1178-1201 with the meaning of eigenmat/eigenmat.cc:641-659.
int choose_max_and_accumulate(cudamat* mat, cudamat* acc) {
  if (!mat->on_device || !acc->on_device) return ERROR_NOT_ON_DEVICE;
  if (mat->is_trans) return ERROR_TRANSPOSED;
  if (!same_shape(mat, acc)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int h = mat->size[0], w = mat->size[1];
  if ((long)h * w == 0) return 0;
  k_col_argmax<<<w < sm_count() * 8 ? w : sm_count() * 8, 256, 0, stream()>>>(mat->data_device, acc->data_device, h, w, 1);
  return check_launch();
}

// cudamat/cudamat.cu:1203-1230; full one-hot per column as eigenmat/eigenmat.cc:661-671
// (the reference CUDA kernel clears only column 0, cudamat_kernels.cu:980).
int choose_max_by_axis(cudamat* mat, cudamat* target, int axis) {
  if (!mat->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (mat->is_trans) return ERROR_TRANSPOSED;
  if (axis != 0) return ERROR_UNSUPPORTED;
  if (!same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int h = mat->size[0], w = mat->size[1];
  if ((long)h * w == 0) return 0;
  k_col_argmax<<<w < sm_count() * 8 ? w : sm_count() * 8, 256, 0, stream()>>>(mat->data_device, target->data_device, h, w, 0);
  return check_launch();
}

// cudamat/cudamat.cu:1232-1258.
int argmax_by_axis(cudamat* mat, cudamat* target, int axis) {
  if (!mat->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (mat->is_trans) return ERROR_TRANSPOSED;
  if (axis != 0) return ERROR_UNSUPPORTED;
  const int h = mat->size[0], w = mat->size[1];
  if (target->size[0] != 1 || target->size[1] != w) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if ((long)h * w == 0) return 0;
  k_col_argmax<<<w < sm_count() * 8 ? w : sm_count() * 8, 256, 0, stream()>>>(mat->data_device, target->data_device, h, w, 2);
  return check_launch();
}

// cudamat/cudamat.cu:2192-2240.
int softmax(cudamat* mat, cudamat* target) {
  if (!mat->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (mat->is_trans) return ERROR_TRANSPOSED;
  if (!same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int h = mat->size[0], w = mat->size[1];
  if ((long)h * w == 0) return 0;
  k_softmax<<<w < sm_count() * 8 ? w : sm_count() * 8, 256, 0, stream()>>>(mat->data_device, target->data_device, h, w);
  return check_launch();
}
int softmax_overwrite(cudamat* mat) { return softmax(mat, mat); }
int apply_softmax(cudamat* mat, cudamat* target) { return softmax(mat, target); }

// cudamat/cudamat.cu:2104-2118.  Blocks: the value returns to the host.
float euclid_norm(cudamat* mat, int* err_code) {
  double r = 0;
  *err_code = scalar_reduce(mat, nullptr, 1, &r);
  return (float)sqrt(r);
}
// cudamat/cudamat.cu:1733-1759.
float vdot(cudamat* mat1, cudamat* mat2, int* err_code) {
  if (mat1->is_trans != mat2->is_trans) {
    *err_code = ERROR_TRANSPOSEDNESS;
    return 0;
  }
  if (!same_shape(mat1, mat2)) {
    *err_code = ERROR_INCOMPATIBLE_DIMENSIONS;
    return 0;
  }
  double r = 0;
  *err_code = scalar_reduce(mat1, mat2, 2, &r);
  return (float)r;
}
// acc[0] += sum((a - b)^2) without a host round trip: the squared reconstruction error of
// deepnet/logistic_layer.py:48-52 (subtract + euclid_norm()**2) kept on the device.
int add_sq_diff(cudamat* a, cudamat* b, cudamat* acc);   // defined with its single-launch kernel below

// Sum of all elements (cudamat/cudamat.py:719-721 computes it as a vdot with ones).
float sum_all(cudamat* mat, int* err_code) {
  double r = 0;
  *err_code = scalar_reduce(mat, nullptr, 0, &r);
  return (float)r;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Row sums without any allocation.
//
// Some hosts of this library must never reach cudaMalloc: a process that has handed the
// whole device to its own memory pool (a later cudaMalloc fails or eats into the pool's
// headroom), or a control loop that cannot tolerate the device-wide synchronisation an
// allocation may imply.  add_sum_by_axis above takes its scratch (the per-split partial row
// sums) from the library's grow-only workspace, which allocates on first use and whenever a
// larger matrix arrives.  The variant below keeps that scratch in a fixed array that is part
// of the loaded module instead: kNoAllocScratchFloats floats (128 KiB), resident on every GPU
// that loads the library until the process exits.
//
// Rules for callers:
//  * The first call on a device looks the array's device address up (once per device, with
//    that device current).  Make that first call during start-up, before any stream capture.
//  * The partial sums need splits x rows floats (splits is chosen from the SM count, at
//    most ceil(4 * SMs / ceil(rows / 32))).  A matrix that needs more than the array holds is
//    refused with ERROR_UNSUPPORTED and a message; nothing is launched.
//  * All calls share the one array and it keeps whatever the last call left in it.  Nothing
//    in it has to start at zero: every slot a call reads is written earlier in that same
//    call.  Two calls that overlap on the GPU (different streams or processes sharing the
//    module) race on it; issue them in order on one stream.
//  * Launches go to the library stream if the library was initialised, else to the default
//    stream; the call itself never creates streams or memory.
constexpr int kNoAllocScratchFloats = 32768;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];
constexpr int kMaxDevices = 64;
// Device address of the array and SM count per device ordinal, looked up once per device under a
// lock; the pointer is published last, so a thread that sees it also sees the SM count.
static float* g_noalloc_ptr[kMaxDevices] = {nullptr};
static int g_noalloc_sms[kMaxDevices] = {0};
static std::mutex g_noalloc_mu;

extern "C" int add_sum_by_axis_noalloc(cudamat* mat, cudamat* target, int axis, float mult) {
  if (!mat->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (axis != 0 && axis != 1) return ERROR_UNSUPPORTED;
  if (mat->is_trans) axis = 1 - axis;
  const int h = mat->size[0], w = mat->size[1];
  if (numel(target) != (axis == 0 ? w : h)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if ((long)h * w == 0) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return set_error("cudaGetDevice failed");
  if (dev < 0 || dev >= kMaxDevices)
    return set_error("add_sum_by_axis_noalloc: device ordinal beyond the 64 this entry point keeps addresses for");
  float* part = nullptr;
  int sms = 0;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
      // In host code the array's name is only a handle; the kernels need its device address.
      float* ptr = nullptr;
      if (cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch) != cudaSuccess || !ptr) {
        cudaGetLastError();
        return set_error("cudaGetSymbolAddress(g_noalloc_scratch) failed");
      }
      int n = 0;
      if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
        return set_error("cudaDeviceGetAttribute(multiprocessor count) failed");
      g_noalloc_sms[dev] = n;
      g_noalloc_ptr[dev] = ptr;
    }
    part = g_noalloc_ptr[dev];
    sms = g_noalloc_sms[dev];
  }
  cudaStream_t st = stream_if_initialised();
  if (axis == 0) {  // sums down the columns need no scratch
    const int blocks = w < sms * 8 ? w : sms * 8;
    k_colsum<<<blocks, 256, 0, st>>>(mat->data_device, target->data_device, h, w, mult, 1.0f);
    return check_launch_any_stream();
  }
  const int bx = (h + 31) / 32;
  int splits = (4 * sms + bx - 1) / bx;
  const int max_splits = (w + 63) / 64;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  const int cps = (w + splits - 1) / splits;
  splits = (w + cps - 1) / cps;
  if (splits == 1) {
    k_rowsum<<<dim3(bx, 1), 32 * kRowLanes, 0, st>>>(mat->data_device, target->data_device, h, w, cps, mult, 1.0f, true);
    return check_launch_any_stream();
  }
  if ((long)splits * h > kNoAllocScratchFloats) {
    set_error("add_sum_by_axis_noalloc: the partial sums of this matrix (splits x rows floats) exceed the "
              "32768-float static scratch; use add_sum_by_axis");
    return ERROR_UNSUPPORTED;
  }
  k_rowsum<<<dim3(bx, splits), 32 * kRowLanes, 0, st>>>(mat->data_device, part, h, w, cps, 1.0f, 0.0f, false);
  k_rowsum_finish<<<(h + 255) / 256, 256, 0, st>>>(part, target->data_device, h, splits, mult, 1.0f);
  return check_launch_any_stream();
}

// ---------------------------------------------------------------------------------------
// Single-launch reductions for the training step.  Both split their input over many blocks and
// let the block that finishes last fold the partial results, in a fixed order (the same bits
// every run): no second launch, which at the small configurations costs more than the sums.
namespace {

// A counter per reduction group, zero between calls (the last block resets it).
unsigned* ticket_counters(int n) {
  return (unsigned*)workspace_zeroed(3, (size_t)(n < 4096 ? 4096 : n) * sizeof(unsigned));
}

// out[r] = sum_c a[r, c] - sum_c b[r, c].  Block = 32 row lanes x 8 column lanes, kVec rows per
// lane (4 with 128-bit loads); blockIdx.y splits the columns.
template <int kVec>
__global__ void __launch_bounds__(32 * kRowLanes) k_rowsum_diff(const float* __restrict__ a, const float* __restrict__ b,
                                                                float* __restrict__ part, unsigned* counters,
                                                                float* __restrict__ out, int h, int w,
                                                                int cols_per_split) {
  __shared__ float smem[kRowLanes][32 * kVec + 1];
  __shared__ bool is_last;
  grid_dependents_launch();
  grid_dependency_wait();
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int r = (blockIdx.x * 32 + tx) * kVec;
  const int c0 = blockIdx.y * cols_per_split;
  const int c1 = min(w, c0 + cols_per_split);
  float s[kVec];
#pragma unroll
  for (int v = 0; v < kVec; v++) s[v] = 0.0f;
  if (r < h) {
    for (int c = c0 + ty; c < c1; c += kRowLanes) {
      const long o = (long)c * h + r;
      if (kVec == 4) {
        const float4 x = *reinterpret_cast<const float4*>(a + o), y = *reinterpret_cast<const float4*>(b + o);
        s[0] += x.x - y.x; s[1 % kVec] += x.y - y.y; s[2 % kVec] += x.z - y.z; s[3 % kVec] += x.w - y.w;
      } else {
        s[0] += a[o] - b[o];
      }
    }
  }
#pragma unroll
  for (int v = 0; v < kVec; v++) smem[ty][tx * kVec + v] = s[v];
  __syncthreads();
  const int splits = gridDim.y;
  // thread t < 32 * kVec owns row blockIdx.x * 32 * kVec + t of the block
  const int row = blockIdx.x * 32 * kVec + threadIdx.x;
  float tot = 0.0f;
  if (threadIdx.x < 32 * kVec) {
#pragma unroll
    for (int j = 0; j < kRowLanes; j++) tot += smem[j][threadIdx.x];
    if (row < h) {
      if (splits == 1) out[row] = tot;
      else part[(long)blockIdx.y * h + row] = tot;
    }
  }
  if (splits == 1) return;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&counters[blockIdx.x], 1u) == (unsigned)(splits - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (threadIdx.x < 32 * kVec && row < h) {
    float t = 0.0f;
    for (int sp = 0; sp < splits; sp++) t += __ldcg(part + (long)sp * h + row);
    out[row] = t;
  }
  if (threadIdx.x == 0) counters[blockIdx.x] = 0u;
}

// acc[0] += sum (a - b)^2: every block leaves a double, the last one folds them.
__global__ void __launch_bounds__(256) k_sq_diff_acc(const float* __restrict__ a, const float* __restrict__ b, long n,
                                                     double* __restrict__ part, unsigned* counter, float* acc) {
  __shared__ double smem[32];
  __shared__ bool is_last;
  grid_dependents_launch();
  grid_dependency_wait();
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  double s = 0;
  long start = 0;
  if ((((uintptr_t)a | (uintptr_t)b) & 15) == 0) {
    const long n4 = n >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    long i = tid;
    for (; i + nth < n4; i += 2 * nth) {   // two independent 128-bit load pairs in flight per thread
      const float4 x0 = a4[i], y0 = b4[i], x1 = a4[i + nth], y1 = b4[i + nth];
      const float e0 = x0.x - y0.x, e1 = x0.y - y0.y, e2 = x0.z - y0.z, e3 = x0.w - y0.w;
      const float f0 = x1.x - y1.x, f1 = x1.y - y1.y, f2 = x1.z - y1.z, f3 = x1.w - y1.w;
      s += (double)((e0 * e0 + e1 * e1) + (e2 * e2 + e3 * e3)) + (double)((f0 * f0 + f1 * f1) + (f2 * f2 + f3 * f3));
    }
    for (; i < n4; i += nth) {
      const float4 x = a4[i], y = b4[i];
      const float d0 = x.x - y.x, d1 = x.y - y.y, d2 = x.z - y.z, d3 = x.w - y.w;
      s += (double)(d0 * d0 + d1 * d1) + (double)(d2 * d2 + d3 * d3);
    }
    start = n4 << 2;
  }
  for (long i = start + tid; i < n; i += nth) {
    const float d = a[i] - b[i];
    s += (double)d * d;
  }
  s = block_sum(s, smem);
  if (gridDim.x == 1) {
    if (threadIdx.x == 0) *acc += (float)s;
    return;
  }
  if (threadIdx.x == 0) {
    part[blockIdx.x] = s;
    __threadfence();
    is_last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  double t = 0;
  for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) t += __ldcg(part + i);
  t = block_sum(t, smem);
  if (threadIdx.x == 0) {
    *acc += (float)t;
    *counter = 0u;
  }
}

}  // namespace

extern "C" {

// acc[0] += sum((a - b)^2) without a host round trip: the squared reconstruction error of
// deepnet/logistic_layer.py:48-52 (subtract + euclid_norm()**2) kept on the device; one launch.
int add_sq_diff(cudamat* a, cudamat* b, cudamat* acc) {
  if (!a->on_device || !b->on_device || !acc->on_device) return ERROR_NOT_ON_DEVICE;
  if (!same_shape(a, b)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (numel(acc) < 1) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long n = numel(a);
  if (n == 0) return 0;
  int blocks = (int)((n / 4 + 255) / 256);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  double* part = (double*)workspace(1, (size_t)(blocks + 1) * sizeof(double));
  unsigned* counter = ticket_counters(1);
  if (!part || !counter) return CUDA_ERROR;
  if (launch_dependent(k_sq_diff_acc, dim3(blocks), dim3(256), 0, stream(), a->data_device, b->data_device, n, part + 1, counter,
                       acc->data_device) != cudaSuccess)
    return set_error(cudaGetErrorString(cudaGetLastError()));
  return check_launch();
}

// target = row sums of a minus row sums of b, in one launch: the bias statistics of a layer,
// positive minus negative phase (deepnet/layer.py:202-213: sum(axis=1) then add_sums(axis=1, mult=-1)).
int row_sum_diff(cudamat* a, cudamat* b, cudamat* target) {
  if (!a->on_device || !b->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (a->is_trans || b->is_trans) return ERROR_TRANSPOSED;
  if (!same_shape(a, b) || numel(target) != a->size[0]) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int h = a->size[0], w = a->size[1];
  if ((long)h * w == 0) return 0;
  const bool vec4 = (h % 4 == 0) && (((uintptr_t)a->data_device | (uintptr_t)b->data_device) & 15) == 0;
  const int rows_per_block = vec4 ? 128 : 32;
  const int bx = (h + rows_per_block - 1) / rows_per_block;
  int splits = (8 * sm_count() + bx - 1) / bx;
  const int max_splits = (w + 31) / 32;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  const int cps = (w + splits - 1) / splits;
  splits = (w + cps - 1) / cps;
  float* part = nullptr;
  unsigned* counters = nullptr;
  if (splits > 1) {
    part = (float*)workspace(0, (size_t)splits * h * sizeof(float));
    counters = ticket_counters(bx + 1);
    if (!part || !counters) return CUDA_ERROR;
    counters += 1;   // slot 0 belongs to add_sq_diff
  }
  const cudaError_t e = launch_dependent(vec4 ? k_rowsum_diff<4> : k_rowsum_diff<1>, dim3(bx, splits), dim3(32 * kRowLanes), 0,
                                         stream(), a->data_device, b->data_device, part, counters, target->data_device, h, w, cps);
  if (e != cudaSuccess) return set_error(cudaGetErrorString(cudaGetLastError()));
  return check_launch();
}

}  // extern "C"
