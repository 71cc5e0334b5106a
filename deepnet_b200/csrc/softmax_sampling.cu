// Replicated-softmax visible layer on the device, two fused operations:
//   softmax_scaled      state = NN (x) softmax_col(pre): the six calls of
//                       deepnet/replicated_softmax_layer.py:12-21 (max, add_row_mult(-1), exp,
//                       sum, divide, mult_by_row) in one pass-structured kernel;
//   sample_multinomial  the per-document loop of replicated_softmax_layer.py:43-60
//                       (assign 0, add_col_vec, perturb_prob, choose_max, sum) as one kernel:
//                       NN[i] draws per document by the exponential race
//                       argmax_w p_w / (-log u_wd), counted per word.
// Random numbers: document i uses sampling call (calls + i); draw d of word w takes the
// uniform of element (w, d) of that call - exactly what the call-by-call path draws when it
// perturbs its (words x draws) scratch matrix, so both paths give the same counts.
#include "common.cuh"

using namespace b200;

namespace {

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256) k_softmax_scaled(const float* m, const float* __restrict__ scale, float* t,
                                                        int h, int w) {
  __shared__ float red[32];
  grid_dependents_launch();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int c = blockIdx.x; c < w; c += gridDim.x) {
    const float* col = m + (long)c * h;
    float* tc = t + (long)c * h;
    float mx = -INFINITY;
    for (int r = threadIdx.x; r < h; r += blockDim.x) mx = fmaxf(mx, col[r]);
    mx = warp_max_f(mx);
    __syncthreads();
    if (lane == 0) red[wid] = mx;
    __syncthreads();
    mx = warp_max_f(lane < nw ? red[lane] : -INFINITY);
    float s = 0;
    for (int r = threadIdx.x; r < h; r += blockDim.x) {
      const float e = expf(col[r] - mx);
      tc[r] = e;
      s += e;
    }
    s = warp_sum_f(s);
    __syncthreads();
    if (lane == 0) red[wid] = s;
    __syncthreads();
    s = warp_sum_f(lane < nw ? red[lane] : 0.0f);
    const float f = scale[c] / s;   // NN / sum, then one multiply per element (mult_by_row)
    for (int r = threadIdx.x; r < h; r += blockDim.x) tc[r] = tc[r] * f;
  }
}

// grid = (draw groups, documents); a block races 4 draws (the 4 words of one Philox block) of
// one document over all words.
__global__ void __launch_bounds__(256) k_sample_multinomial(const float* __restrict__ probs,
                                                            const float* __restrict__ nn, float* counts, int h, int w,
                                                            int max_draws, int col0, unsigned long long seed,
                                                            unsigned long long call0) {
  __shared__ float sv[4][8];
  __shared__ int si[4][8];
  grid_dependents_launch();
  grid_dependency_wait();
  for (int doc = blockIdx.y; doc < w; doc += gridDim.y) {
  int ndraws = (int)nn[doc];
  if (ndraws > max_draws) ndraws = max_draws;
  const float* p = probs + (long)doc * h;
  const PhiloxKey key = make_philox_key(seed, call0 + (unsigned long long)doc);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  // global draw columns of this document's scratch matrix: col0 + d, d = 0 .. ndraws-1
  const int first_blk = col0 >> 2, last_blk = (col0 + ndraws - 1) >> 2;
  for (int blk = first_blk + blockIdx.x; ndraws > 0 && blk <= last_blk; blk += gridDim.x) {
    float bv[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    int bi[4] = {0x7fffffff, 0x7fffffff, 0x7fffffff, 0x7fffffff};
    // The first words are raced in full; the best value any thread has then seen is a lower bound of
    // the winner's, and most of the remaining words cannot reach it: v = -p / log u > bound needs
    // -log u < p / bound, and -log u >= 1 - u, so a word with 1 - u >= (p / bound)(1 + 2e-6) is out
    // without its logarithm and division (the margin covers the rounding of either side; ties are
    // never skipped).  What is raced in full, and its outcome, are those of the plain loop.
    const int seed_rows = h < 2 * (int)blockDim.x ? h : 2 * (int)blockDim.x;
    for (int r = threadIdx.x; r < seed_rows; r += blockDim.x) {
      const uint4 wd = philox4x32_10((uint32_t)r, (uint32_t)blk, key);
      const float pr = p[r];
      const float u[4] = {word_to_uniform(wd.x), word_to_uniform(wd.y), word_to_uniform(wd.z), word_to_uniform(wd.w)};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float v = -pr / logf(u[j]);        // perturb_prob: cudamat_kernels.cu:227-238
        if (v > bv[j] || (v == bv[j] && r < bi[j])) {
          bv[j] = v;
          bi[j] = r;
        }
      }
    }
    float inv[4];                                 // (1 + 2e-6) / bound, or 0: no usable bound for this draw
    {
      float lb[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        lb[j] = bv[j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lb[j] = fmaxf(lb[j], __shfl_xor_sync(0xffffffffu, lb[j], o));
      }
      __syncthreads();                            // (sv is free: the previous block of draws has been read)
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < 4; j++) sv[j][wid] = lb[j];
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float m = sv[j][0];
        for (int k = 1; k < (int)(blockDim.x >> 5); k++) m = fmaxf(m, sv[j][k]);
        inv[j] = (m > 0.0f && m < INFINITY) ? 1.000002f / m : 0.0f;
      }
      __syncthreads();                            // sv is written again below
    }
    for (int r = seed_rows + threadIdx.x; r < h; r += blockDim.x) {
      const uint4 wd = philox4x32_10((uint32_t)r, (uint32_t)blk, key);
      const float pr = p[r];
      const float u[4] = {word_to_uniform(wd.x), word_to_uniform(wd.y), word_to_uniform(wd.z), word_to_uniform(wd.w)};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        if (inv[j] > 0.0f && 1.0f - u[j] >= pr * inv[j]) continue;   // cannot reach the bound (NaN compares false: raced)
        const float v = -pr / logf(u[j]);
        if (v > bv[j] || (v == bv[j] && r < bi[j])) {
          bv[j] = v;
          bi[j] = r;
          if (v > 0.0f && v < INFINITY) {            // a better bound of this thread's own
            const float c = 1.000002f / v;
            if (inv[j] == 0.0f || c < inv[j]) inv[j] = c;
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, bv[j], o);
        const int i2 = __shfl_xor_sync(0xffffffffu, bi[j], o);
        if (v2 > bv[j] || (v2 == bv[j] && i2 < bi[j])) {
          bv[j] = v2;
          bi[j] = i2;
        }
      }
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        sv[j][wid] = bv[j];
        si[j][wid] = bi[j];
      }
    }
    __syncthreads();
    if (threadIdx.x < 4) {
      const int j = threadIdx.x;
      const int d = (blk << 2) + j - col0;       // draw index of this word of the block
      if (d >= 0 && d < ndraws) {
        float v = sv[j][0];
        int i = si[j][0];
        for (int k = 1; k < (int)(blockDim.x >> 5); k++) {
          if (sv[j][k] > v || (sv[j][k] == v && si[j][k] < i)) {
            v = sv[j][k];
            i = si[j][k];
          }
        }
        if (i == 0x7fffffff) i = 0;              // all-NaN column: the sequential scan keeps word 0
        atomicAdd(&counts[(long)doc * h + i], 1.0f);   // choose_max one-hot summed over the draws
      }
    }
    __syncthreads();   // sv / si are reused by the next block of draws
  }
  }
}

// Column softmax and one categorical draw per column in one kernel: the label layer of a DBM
// (deepnet/softmax_layer.py:11-16: apply_softmax, then perturb_prob_for_softmax_sampling and
// choose_max(axis=0)).  state = softmax(pre) (optionally after adding a per-row bias), sample =
// one-hot of argmax_r state[r] / (-log u[r]) with u the uniforms of element (r, global column) of
// this sampling call, the first maximum winning: what the three calls give on the same stream.
__global__ void __launch_bounds__(128) k_softmax_sample(const float* pre, const float* __restrict__ bias, float* state,
                                                        float* sample, int h, int w, int col0, PhiloxKey key) {
  __shared__ float red[4];
  __shared__ int redi[4];
  grid_dependents_launch();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int c = blockIdx.x; c < w; c += gridDim.x) {
    const float* col = pre + (long)c * h;
    float* st = state + (long)c * h;
    float mx = -INFINITY;
    for (int r = threadIdx.x; r < h; r += blockDim.x) mx = fmaxf(mx, col[r] + (bias ? bias[r] : 0.0f));
    mx = warp_max_f(mx);
    __syncthreads();
    if (lane == 0) red[wid] = mx;
    __syncthreads();
    mx = warp_max_f(lane < nw ? red[lane] : -INFINITY);
    float s = 0;
    for (int r = threadIdx.x; r < h; r += blockDim.x) {
      const float e = expf(col[r] + (bias ? bias[r] : 0.0f) - mx);
      st[r] = e;
      s += e;
    }
    s = warp_sum_f(s);
    __syncthreads();
    if (lane == 0) red[wid] = s;
    __syncthreads();
    s = warp_sum_f(lane < nw ? red[lane] : 0.0f);
    const int gc = c + col0;                       // global column: which Philox block and word
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = threadIdx.x; r < h; r += blockDim.x) {
      const float pr = st[r] / s;                  // apply_softmax divides (cudamat_kernels.cu:868)
      st[r] = pr;
      if (sample) {
        const uint4 wd = philox4x32_10((uint32_t)r, (uint32_t)(gc >> 2), key);
        const float v = -pr / logf(word_to_uniform(pick_word(wd, gc & 3)));
        if (v > bv || (v == bv && r < bi)) {
          bv = v;
          bi = r;
        }
      }
    }
    if (!sample) continue;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float v2 = __shfl_xor_sync(0xffffffffu, bv, o);
      const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
      if (v2 > bv || (v2 == bv && i2 < bi)) {
        bv = v2;
        bi = i2;
      }
    }
    __syncthreads();
    if (lane == 0) {
      red[wid] = bv;
      redi[wid] = bi;
    }
    __syncthreads();
    bv = red[0];
    bi = redi[0];
    for (int q = 1; q < nw; q++)
      if (red[q] > bv || (red[q] == bv && redi[q] < bi)) {
        bv = red[q];
        bi = redi[q];
      }
    if (bi == 0x7fffffff) bi = 0;                  // all-NaN column: the sequential scan keeps row 0
    float* sm = sample + (long)c * h;
    for (int r = threadIdx.x; r < h; r += blockDim.x) sm[r] = r == bi ? 1.0f : 0.0f;
  }
}

// D independent Gumbel-max draws per column from the energies of a softmax, counted per row: the
// loop of deepnet/ais.py:16-30 (SampleEnergySoftmax: for each of D draws,
// perturb_energy_for_softmax_sampling then choose_max_and_accumulate) as one kernel.  Draw d of
// column c takes the uniform of element (row, global column) of sampling call (calls + d): what
// the call-by-call loop draws, so both give the same counts.  grid = (blocks of 4 columns, draw
// groups); a block races one draw of its 4 columns (the 4 words of a Philox block) over all rows.
__global__ void __launch_bounds__(256) k_sample_energy_softmax(const float* __restrict__ energy, float* counts, int h,
                                                               int w, int ndraws, int col0, unsigned long long seed,
                                                               unsigned long long call0) {
  __shared__ float sv[4][8];
  __shared__ int si[4][8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int first_blk = col0 >> 2, nblk = ((col0 + w - 1) >> 2) - first_blk + 1;
  for (int b = blockIdx.x; b < nblk; b += gridDim.x) {
    const int blk = first_blk + b;
    for (int d = blockIdx.y; d < ndraws; d += gridDim.y) {
      const PhiloxKey key = make_philox_key(seed, call0 + (unsigned long long)d);
      float bv[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      int bi[4] = {0x7fffffff, 0x7fffffff, 0x7fffffff, 0x7fffffff};
      for (int r = threadIdx.x; r < h; r += blockDim.x) {
        const uint4 wd = philox4x32_10((uint32_t)r, (uint32_t)blk, key);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int c = (blk << 2) + j - col0;
          if (c < 0 || c >= w) continue;
          const float v = energy[(long)c * h + r] - logf(-logf(word_to_uniform(pick_word(wd, j))));   // cudamat_kernels.cu:240-251
          if (v > bv[j] || (v == bv[j] && r < bi[j])) {
            bv[j] = v;
            bi[j] = r;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float v2 = __shfl_xor_sync(0xffffffffu, bv[j], o);
          const int i2 = __shfl_xor_sync(0xffffffffu, bi[j], o);
          if (v2 > bv[j] || (v2 == bv[j] && i2 < bi[j])) {
            bv[j] = v2;
            bi[j] = i2;
          }
        }
      }
      __syncthreads();
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          sv[j][wid] = bv[j];
          si[j][wid] = bi[j];
        }
      }
      __syncthreads();
      if (threadIdx.x < 4) {
        const int j = threadIdx.x, c = (blk << 2) + j - col0;
        if (c >= 0 && c < w) {
          float v = sv[j][0];
          int i = si[j][0];
          for (int q = 1; q < (int)(blockDim.x >> 5); q++)
            if (sv[j][q] > v || (sv[j][q] == v && si[j][q] < i)) {
              v = sv[j][q];
              i = si[j][q];
            }
          if (i == 0x7fffffff) i = 0;
          atomicAdd(&counts[(long)c * h + i], 1.0f);
        }
      }
      __syncthreads();
    }
  }
}

}  // namespace

extern "C" {

// target[:, j] = scale[j] * softmax(mat[:, j]); scale is 1 x cols (the document lengths NN).
int softmax_scaled(cudamat* mat, cudamat* scale, cudamat* target) {
  if (!mat->on_device || !scale->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (mat->is_trans || target->is_trans) return ERROR_TRANSPOSED;
  if (!same_shape(mat, target) || numel(scale) != mat->size[1]) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int h = mat->size[0], w = mat->size[1];
  if ((long)h * w == 0) return 0;
  (void)launch_dependent(k_softmax_scaled, dim3(w < sm_count() * 8 ? w : sm_count() * 8), dim3(256), 0, stream(), mat->data_device,
                         scale->data_device, target->data_device, h, w);
  return check_launch();
}

// target[:, i] = word counts of int(nn[i]) draws (at most max_draws) from the distribution
// proportional to probs[:, i].  Consumes one sampling call per document.
int sample_multinomial(rnd_struct* rnd_state, cudamat* probs, cudamat* nn, cudamat* target, int max_draws) {
  if (!probs->on_device || !nn->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (probs->is_trans || target->is_trans) return ERROR_TRANSPOSED;
  if (!same_shape(probs, target) || numel(nn) != probs->size[1]) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (max_draws < 1) return ERROR_UNSUPPORTED;
  const int h = probs->size[0], w = probs->size[1];
  if ((long)h * w == 0) return 0;
  if (cudaMemsetAsync(target->data_device, 0, (size_t)h * w * sizeof(float), stream()) != cudaSuccess)
    return set_error("cudaMemsetAsync failed");
  const unsigned long long call0 = rnd_state->calls;
  rnd_state->calls += (unsigned long long)w;
  int groups = (max_draws + 3) / 4 + 1;
  if (groups > 64) groups = 64;
  (void)launch_dependent(k_sample_multinomial, dim3(groups, w < 65535 ? w : 65535), dim3(256), 0, stream(), probs->data_device,
                         nn->data_device, target->data_device, h, w, max_draws, rng_col0(), rnd_state->seed, call0);
  return check_launch();
}

// state[:, j] = softmax(pre[:, j] (+ bias)); sample[:, j] = one categorical draw from it as a one-hot
// column (sample may be null: activation only, no sampling call consumed).  pre and state may be
// the same matrix.  One sampling call, the one perturb_prob_for_softmax_sampling would consume.
int softmax_sample(rnd_struct* rnd_state, cudamat* pre, cudamat* bias, cudamat* state, cudamat* sample) {
  if (!pre->on_device || !state->on_device || (sample && !sample->on_device) || (bias && !bias->on_device))
    return ERROR_NOT_ON_DEVICE;
  if (pre->is_trans || state->is_trans || (sample && sample->is_trans)) return ERROR_TRANSPOSED;
  if (!same_shape(pre, state) || (sample && !same_shape(pre, sample))) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (bias && numel(bias) != pre->size[0]) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int h = pre->size[0], w = pre->size[1];
  PhiloxKey key = make_philox_key(0, 0);
  if (sample) {
    if (!rnd_state) return ERROR_GENERIC;
    key = make_philox_key(rnd_state->seed, rnd_state->calls);
    rnd_state->calls += 1;
  }
  if ((long)h * w == 0) return 0;
  (void)launch_dependent(k_softmax_sample, dim3(w < sm_count() * 16 ? w : sm_count() * 16), dim3(128), 0, stream(),
                         pre->data_device, bias ? bias->data_device : nullptr, state->data_device,
                         sample ? sample->data_device : nullptr, h, w, rng_col0(), key);
  return check_launch();
}

// target[:, c] = counts over `ndraws` Gumbel-max draws from the softmax whose energies are
// energy[:, c] (deepnet/ais.py:16-30).  Consumes ndraws sampling calls.
int sample_energy_softmax(rnd_struct* rnd_state, cudamat* energy, cudamat* target, int ndraws) {
  if (!energy->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (energy->is_trans || target->is_trans) return ERROR_TRANSPOSED;
  if (!same_shape(energy, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (ndraws < 0) return ERROR_UNSUPPORTED;
  const int h = energy->size[0], w = energy->size[1];
  if ((long)h * w == 0) return 0;
  if (cudaMemsetAsync(target->data_device, 0, (size_t)h * w * sizeof(float), stream()) != cudaSuccess)
    return set_error("cudaMemsetAsync failed");
  const unsigned long long call0 = rnd_state->calls;
  rnd_state->calls += (unsigned long long)ndraws;
  if (ndraws == 0) return 0;
  const int col0 = rng_col0();
  const int nblk = ((col0 + w - 1) >> 2) - (col0 >> 2) + 1;
  int gy = ndraws < 64 ? ndraws : 64;
  int gx = nblk;
  if ((long)gx * gy > 65535L * 4) gx = (int)(65535L * 4 / gy);
  k_sample_energy_softmax<<<dim3(gx, gy), 256, 0, stream()>>>(energy->data_device, target->data_device, h, w, ndraws, col0,
                                                            rnd_state->seed, call0);
  return check_launch();
}

}  // extern "C"
