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
