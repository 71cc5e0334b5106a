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

// ---- device-resident data feed -------------------------------------------------------------
// The data set stays on the device as one (dims x cases) matrix per modality, either fp32 or,
// for 0/1 data, one bit per value (32 rows per 32-bit word: a million 8192-dimensional binary
// cases take 1 GB instead of 33).  A minibatch is GATHERED: output column j is stored column
// perm(start + j), where perm is a keyed bijection of [0, cases) evaluated on the fly (a Feistel
// network on ceil(log2 cases) bits, walked until it lands inside the range), so an epoch's shuffle
// costs nothing and moves no data (the reference swaps columns in place after drawing the
// permutation on the host, deepnet/datahandler.py:364-375).  The same pass applies the
// mean / standard-deviation normalisation (datahandler.py:299-306) and writes, when asked, the
// 16-bit parts of the minibatch that the products read.
namespace {

__host__ __device__ inline uint32_t feed_mix(uint32_t r, uint32_t k) {
  uint32_t h = r * 0x9E3779B1u + k;
  h ^= h >> 15;
  h *= 0x85EBCA77u;
  h ^= h >> 13;
  h *= 0xC2B2AE3Du;
  h ^= h >> 16;
  return h;
}
constexpr int kFeedRounds = 6;
// Bijection of [0, n): alternating unbalanced Feistel rounds on `bits` bits (2^(bits-1) < n <= 2^bits,
// bits >= 2), repeated while the image falls outside [0, n) (fewer than two passes on average).
__host__ __device__ inline uint32_t feed_perm(uint32_t i, uint32_t n, uint32_t bits, uint32_t key_lo, uint32_t key_hi) {
  const uint32_t a = bits >> 1, b = bits - a;
  const uint32_t mask_a = (1u << a) - 1u, mask_b = (1u << b) - 1u;
  uint32_t x = i;
  do {
    uint32_t L = x >> a, R = x & mask_a;
    for (int round = 0; round < kFeedRounds; round++) {
      const uint32_t k = key_lo * 0x9E3779B9u + key_hi * 0x85EBCA6Bu + (uint32_t)round * 0xC2B2AE35u;
      if ((round & 1) == 0) L ^= feed_mix(R, k) & mask_b;
      else R ^= feed_mix(L, k) & mask_a;
    }
    x = (L << a) | R;
  } while (x >= n);
  return x;
}
inline uint32_t feed_bits(uint32_t n) {
  uint32_t bits = 2;
  while (bits < 32 && (1ull << bits) < n) bits++;
  return bits;
}

// One block per output column.  kPacked: the source holds one bit per value.
template <bool kPacked>
__global__ void __launch_bounds__(256) k_feed_gather(const float* __restrict__ src, int h, int src_ld, uint32_t n,
                                                     uint32_t bits, uint32_t key_lo, uint32_t key_hi, int shuffle,
                                                     uint32_t start, int count, const float* __restrict__ mean,
                                                     const float* __restrict__ stdv, float* __restrict__ out,
                                                     uint16_t* __restrict__ aux, int lda, int aux_mode, float aux_scale) {
  for (int j = blockIdx.x; j < count; j += gridDim.x) {
    const uint32_t pos = start + (uint32_t)j;
    const uint32_t c = shuffle ? feed_perm(pos, n, bits, key_lo, key_hi) : pos;
    const float* col = src + (size_t)c * src_ld;
    float* o = out + (size_t)j * h;
    uint16_t* a0 = aux ? aux + (size_t)j * 2 * lda : nullptr;
    for (int r = threadIdx.x; r < h; r += blockDim.x) {
      float x;
      if (kPacked) x = (float)((__float_as_uint(col[r >> 5]) >> (r & 31)) & 1u);
      else x = col[r];
      if (mean) x = __fdiv_rn(__fadd_rn(x, -mean[r]), stdv[r]);    // add_col_mult(mean, -1), then div_by_col(std)
      o[r] = x;
      if (aux_mode == 2) {
        uint16_t lo, hi;
        split_f16(x, aux_scale, lo, hi);
        a0[r] = lo;
        a0[lda + r] = hi;
      } else if (aux_mode == 1) {
        uint16_t lo, b16;
        split_aux(x, lo, b16);
        a0[r] = lo;
        a0[lda + r] = b16;
      }
    }
  }
}

}  // namespace

extern "C" {

// out (h x count) = columns perm(start .. start + count - 1) of the stored data set `src`
// (h x n fp32, or with packed != 0 ceil(h / 32) x n words of 32 rows each), normalised with
// mean / std (h x 1 each, or both null), plus the aux matrix of the minibatch (aux_mode 0 none,
// 1 bfloat16 parts, 2 scaled half-precision form with exponent aux_exp).  shuffle = 0 reads the
// columns in stored order.  No counterpart in the reference (its GPUCache slices and swaps).
int feed_gather(cudamat* src, int packed, int h, unsigned int key_lo, unsigned int key_hi, int shuffle, int start,
                cudamat* mean, cudamat* stdv, cudamat* out, cudamat* out_aux, int aux_mode, int aux_exp) {
  if (!src->on_device || !out->on_device || (out_aux && !out_aux->on_device)) return ERROR_NOT_ON_DEVICE;
  if ((mean && !mean->on_device) || (stdv && !stdv->on_device)) return ERROR_NOT_ON_DEVICE;
  if (src->is_trans || out->is_trans) return ERROR_TRANSPOSED;
  if ((mean == nullptr) != (stdv == nullptr)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int n = src->size[1], count = out->size[1];
  if (h <= 0 || out->size[0] != h || src->size[0] != (packed ? (h + 31) / 32 : h)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (start < 0 || count < 0 || (long)start + count > n) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (mean && (numel(mean) != h || numel(stdv) != h)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (aux_mode < 0 || aux_mode > 2 || (aux_mode != 0) != (out_aux != nullptr)) return ERROR_UNSUPPORTED;
  if (out_aux && (out_aux->size[0] != aux_rows(h) || out_aux->size[1] != count)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (count == 0) return 0;
  const int blocks = count < sm_count() * 8 ? count : sm_count() * 8;
  uint16_t* ap = out_aux ? reinterpret_cast<uint16_t*>(out_aux->data_device) : nullptr;
  const float scale = exp2f((float)aux_exp);
  const uint32_t bits = feed_bits((uint32_t)n);
  if (packed)
    k_feed_gather<true><<<blocks, 256, 0, stream()>>>(src->data_device, h, src->size[0], (uint32_t)n, bits, key_lo, key_hi,
                                                     shuffle, (uint32_t)start, count, mean ? mean->data_device : nullptr,
                                                     stdv ? stdv->data_device : nullptr, out->data_device, ap,
                                                     aux_rows(h), aux_mode, scale);
  else
    k_feed_gather<false><<<blocks, 256, 0, stream()>>>(src->data_device, h, src->size[0], (uint32_t)n, bits, key_lo, key_hi,
                                                      shuffle, (uint32_t)start, count, mean ? mean->data_device : nullptr,
                                                      stdv ? stdv->data_device : nullptr, out->data_device, ap,
                                                      aux_rows(h), aux_mode, scale);
  return check_launch();
}

// The stored column that position `pos` of an epoch keyed (key_lo, key_hi) reads, for n cases
// (what feed_gather evaluates on the device; host-side, for callers that need the order).
unsigned int feed_permutation_at(unsigned int pos, unsigned int n, unsigned int key_lo, unsigned int key_hi) {
  return feed_perm(pos, n, feed_bits(n), key_lo, key_hi);
}

}  // extern "C"
