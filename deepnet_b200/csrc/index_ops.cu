// Column gather and in-place column swap (cudamat/cudamat.cu:2120-2150, kernels
// cudamat_kernels.cu:720-758), the two index operations the device-resident data cache of
// deepnet/datahandler.py:364-375 shuffles with.  Indices are float32 values holding integers;
// negative ones count from the end; out-of-range ones yield NaN columns (select) or are skipped
// (swap).  One block per index, 128-bit copies when the column length allows.
#include "common.cuh"

using namespace b200;

namespace {

__device__ __forceinline__ int resolve(float f, int n) {
  int i = (int)f;
  if (i < 0) i += n;
  return (i < 0 || i >= n) ? -1 : i;
}

__global__ void __launch_bounds__(256) k_select_cols(const float* __restrict__ src, float* __restrict__ dst,
                                                     const float* __restrict__ idx, int nidx, int h, int src_cols,
                                                     bool vec) {
  for (int c = blockIdx.x; c < nidx; c += gridDim.x) {
    const int s = resolve(idx[c], src_cols);
    float* out = dst + (long)c * h;
    if (s < 0) {
      const float nan = __int_as_float(0x7fc00000);
      for (int r = threadIdx.x; r < h; r += blockDim.x) out[r] = nan;
      continue;
    }
    const float* in = src + (long)s * h;
    if (vec) {
      for (int r = threadIdx.x; r < (h >> 2); r += blockDim.x)
        reinterpret_cast<float4*>(out)[r] = reinterpret_cast<const float4*>(in)[r];
    } else {
      for (int r = threadIdx.x; r < h; r += blockDim.x) out[r] = in[r];
    }
  }
}

__global__ void __launch_bounds__(256) k_swap_cols(float* a, float* b, const float* __restrict__ idx1,
                                                   const float* __restrict__ idx2, int nidx, int h, int a_cols,
                                                   int b_cols, bool vec) {
  for (int c = blockIdx.x; c < nidx; c += gridDim.x) {
    const int i1 = resolve(idx1[c], a_cols), i2 = resolve(idx2[c], b_cols);
    if (i1 < 0 || i2 < 0) continue;
    float* pa = a + (long)i1 * h;
    float* pb = b + (long)i2 * h;
    if (pa == pb) continue;
    if (vec) {
      for (int r = threadIdx.x; r < (h >> 2); r += blockDim.x) {
        const float4 x = reinterpret_cast<float4*>(pa)[r];
        reinterpret_cast<float4*>(pa)[r] = reinterpret_cast<float4*>(pb)[r];
        reinterpret_cast<float4*>(pb)[r] = x;
      }
    } else {
      for (int r = threadIdx.x; r < h; r += blockDim.x) {
        const float x = pa[r];
        pa[r] = pb[r];
        pb[r] = x;
      }
    }
  }
}

}  // namespace

extern "C" {

// cudamat/cudamat.cu:2120-2136 (Python: select_columns): target[:, c] = source[:, indices[c]].
int selectRows(cudamat* source, cudamat* target, cudamat* indices) {
  if (!source->on_device || !target->on_device || !indices->on_device) return ERROR_NOT_ON_DEVICE;
  if (source->is_trans || target->is_trans) return ERROR_TRANSPOSED;
  const int n = (int)numel(indices), h = source->size[0];
  if (target->size[0] != h || target->size[1] != n) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (n == 0 || h == 0) return 0;
  const bool vec = (h % 4 == 0) && (((uintptr_t)source->data_device | (uintptr_t)target->data_device) & 15) == 0;
  const int blocks = n < sm_count() * 8 ? n : sm_count() * 8;
  k_select_cols<<<blocks, 256, 0, stream()>>>(source->data_device, target->data_device, indices->data_device, n, h,
                                              source->size[1], vec);
  return check_launch();
}

// cudamat/cudamat.cu:2138-2150 (Python: swap_columns): column indices1[c] of source and column
// indices2[c] of target change places.  With source == target and disjoint index sets this is
// the in-place shuffle of deepnet/datahandler.py:364-375.
int swapColumns(cudamat* source, cudamat* target, cudamat* indices1, cudamat* indices2) {
  if (!source->on_device || !target->on_device || !indices1->on_device || !indices2->on_device)
    return ERROR_NOT_ON_DEVICE;
  if (source->is_trans || target->is_trans) return ERROR_TRANSPOSED;
  const int n = (int)numel(indices1), h = source->size[0];
  if (numel(indices2) != n || target->size[0] != h) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (n == 0 || h == 0) return 0;
  const bool vec = (h % 4 == 0) && (((uintptr_t)source->data_device | (uintptr_t)target->data_device) & 15) == 0;
  const int blocks = n < sm_count() * 8 ? n : sm_count() * 8;
  k_swap_cols<<<blocks, 256, 0, stream()>>>(source->data_device, target->data_device, indices1->data_device,
                                            indices2->data_device, n, h, source->size[1], target->size[1], vec);
  return check_launch();
}

}  // extern "C"

// ---- transpose copy and column norm limit ------------------------------------------------
namespace {

// 32 x 32 tiles through shared memory (padded against bank conflicts): reads and writes coalesced.
__global__ void __launch_bounds__(256) k_transpose(const float* __restrict__ src, float* __restrict__ dst, int h, int w) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int tiles_r = (h + 31) / 32, tiles_c = (w + 31) / 32;
  for (long t = blockIdx.x; t < (long)tiles_r * tiles_c; t += gridDim.x) {
    const int r0 = (int)(t % tiles_r) * 32, c0 = (int)(t / tiles_r) * 32;
    __syncthreads();
#pragma unroll
    for (int j = ty; j < 32; j += 8)
      if (r0 + tx < h && c0 + j < w) tile[j][tx] = src[(long)(c0 + j) * h + r0 + tx];
    __syncthreads();
#pragma unroll
    for (int j = ty; j < 32; j += 8)
      if (c0 + tx < w && r0 + j < h) dst[(long)(r0 + j) * w + c0 + tx] = tile[tx][j];
  }
}

// One block per column: scale the column so that its Euclidean norm is at most `norm`.
__global__ void __launch_bounds__(256) k_normlimit_cols(const float* __restrict__ m, float* __restrict__ t, int h, int w,
                                                        float norm) {
  __shared__ float red[32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (int c = blockIdx.x; c < w; c += gridDim.x) {
    const float* col = m + (long)c * h;
    float* out = t + (long)c * h;
    float s = 0;
    for (int r = threadIdx.x; r < h; r += blockDim.x) s += col[r] * col[r];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();
    if (lane == 0) red[wid] = s;
    __syncthreads();
    s = lane < (int)(blockDim.x >> 5) ? red[lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float len = sqrtf(s);
    const float f = len < norm ? 1.0f : norm / len;
    for (int r = threadIdx.x; r < h; r += blockDim.x) out[r] = col[r] * f;
  }
}

}  // namespace

extern "C" {

// cudamat/cudamat.cu:271-296: target (w x h) = source' for an h x w source.
int copy_transpose(cudamat* source, cudamat* target) {
  if (!source->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (source->size[0] != target->size[1] || source->size[1] != target->size[0]) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int h = source->size[0], w = source->size[1];
  if ((long)h * w == 0) return 0;
  long tiles = (long)((h + 31) / 32) * ((w + 31) / 32);
  if (tiles > (long)sm_count() * 16) tiles = (long)sm_count() * 16;
  k_transpose<<<(int)tiles, 256, 0, stream()>>>(source->data_device, target->data_device, h, w);
  return check_launch();
}

// cudamat/cudamat.cu:1289-1314 (kNormLimitColumnwise, cudamat_kernels.cu:1068-1088): every column
// whose Euclidean norm exceeds `norm` is scaled back to it; only axis 0 exists in the reference.
// Called by the weight-norm branch of deepnet/parameter.py:101-102.
int normlimit_by_axis(cudamat* mat, cudamat* target, int axis, float norm) {
  if (!mat->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (mat->is_trans) return ERROR_TRANSPOSED;
  if (axis != 0) return ERROR_UNSUPPORTED;
  if (!same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int h = mat->size[0], w = mat->size[1];
  if ((long)h * w == 0) return 0;
  k_normlimit_cols<<<w < sm_count() * 8 ? w : sm_count() * 8, 256, 0, stream()>>>(mat->data_device, target->data_device,
                                                                                 h, w, norm);
  return check_launch();
}

}  // extern "C"
