// Sampling operations of the C ABI (cudamat/cudamat.cu:437-590) on a counter-based
// Philox4x32-10 stream instead of the reference's table of 12288 multiply-with-carry
// generators: no state arrays, any number of threads, and the number drawn for a
// matrix element depends only on (seed, call number, row, global column).
// One thread produces the four columns {4j..4j+3} of one row from one Philox block;
// consecutive threads take consecutive rows, so every store is coalesced.
#include "common.cuh"

using namespace b200;

namespace {

enum RngOp { kUniform = 0, kNormal, kBernoulli, kBernoulliTanh, kGaussianAdd, kPerturbProb, kPerturbEnergy, kDropout };

template <int kOp>
__global__ void __launch_bounds__(256) k_rng(const float* src, float* dst, int h, int w, int col0, PhiloxKey key,
                                             float p0, float p1) {
  grid_dependents_launch();
  grid_dependency_wait();
  // global column blocks covered by this matrix: [col0 >> 2, (col0 + w - 1) >> 2]
  const int blk0 = col0 >> 2;
  const int nblk = ((col0 + w - 1) >> 2) - blk0 + 1;
  const long items = (long)h * nblk;
  for (long it = (long)blockIdx.x * blockDim.x + threadIdx.x; it < items; it += (long)gridDim.x * blockDim.x) {
    const int b = (int)(it / h), r = (int)(it - (long)b * h);
    const uint4 wd = philox4x32_10((uint32_t)r, (uint32_t)(blk0 + b), key);
    float z[4];
    if (kOp == kNormal || kOp == kGaussianAdd) {
      // Box-Muller on word pairs (0,1) and (2,3), as cudamat_kernels.cu:125-143 pairs its draws
      const float u0 = word_to_uniform(wd.x), u1 = word_to_uniform(wd.y);
      const float u2 = word_to_uniform(wd.z), u3 = word_to_uniform(wd.w);
      const float r0 = sqrtf(-2.0f * logf(u0)), r1 = sqrtf(-2.0f * logf(u2));
      const float a0 = 6.283185307179586f * u1, a1 = 6.283185307179586f * u3;
      z[0] = r0 * cosf(a0); z[1] = r0 * sinf(a0); z[2] = r1 * cosf(a1); z[3] = r1 * sinf(a1);
    } else {
      z[0] = word_to_uniform(wd.x); z[1] = word_to_uniform(wd.y);
      z[2] = word_to_uniform(wd.z); z[3] = word_to_uniform(wd.w);
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int c = ((blk0 + b) << 2) + j - col0;  // local column
      if (c < 0 || c >= w) continue;
      const long idx = (long)c * h + r;
      const float u = z[j];
      float out;
      if (kOp == kUniform || kOp == kNormal) out = u;
      else if (kOp == kBernoulli) out = u < src[idx] ? 1.0f : 0.0f;
      else if (kOp == kBernoulliTanh) out = u < (1.0f + src[idx]) * 0.5f ? 1.0f : -1.0f;
      else if (kOp == kGaussianAdd) out = src[idx] + p0 * u;
      else if (kOp == kPerturbProb) out = -src[idx] / logf(u);
      else if (kOp == kPerturbEnergy) out = src[idx] - logf(-logf(u));
      else out = u > p0 ? src[idx] : p1;  // dropout
      dst[idx] = out;
    }
  }
}

template <int kOp>
int launch(rnd_struct* rnd, cudamat* mat, cudamat* target, float p0 = 0, float p1 = 0) {
  if (!mat->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (!same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const PhiloxKey key = make_philox_key(rnd->seed, rnd->calls);
  rnd->calls += 1;
  // A transposed handle shares its parent's storage; numbers are assigned by stored position.
  const int h = mat->size[0], w = mat->size[1];
  if ((long)h * w == 0) return 0;
  const int col0 = rng_col0();
  const long items = (long)h * (((col0 + w - 1) >> 2) - (col0 >> 2) + 1);
  long blocks = (items + 255) / 256;
  if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
  (void)launch_dependent(k_rng<kOp>, dim3((unsigned)blocks), dim3(256), 0, stream(), mat->data_device, target->data_device, h, w,
                         col0, key, p0, p1);
  return check_launch();
}

}  // namespace

extern "C" {

// cudamat/cudamat.cu:437-467.
int fill_with_rand(rnd_struct* rnd_state, cudamat* mat) { return launch<kUniform>(rnd_state, mat, mat); }
int fill_with_randn(rnd_struct* rnd_state, cudamat* mat) { return launch<kNormal>(rnd_state, mat, mat); }
// cudamat/cudamat.cu:469-501: target = (u < mat) ? 1 : 0 (strict, u in (0, 1]).
int sample_bernoulli(rnd_struct* rnd_state, cudamat* mat, cudamat* target) {
  return launch<kBernoulli>(rnd_state, mat, target);
}
int sample_bernoulli_tanh(rnd_struct* rnd_state, cudamat* mat, cudamat* target) {
  return launch<kBernoulliTanh>(rnd_state, mat, target);
}
// cudamat/cudamat.cu:520-536.
int sample_gaussian(rnd_struct* rnd_state, cudamat* mat, cudamat* target, float mult) {
  return launch<kGaussianAdd>(rnd_state, mat, target, mult);
}
// cudamat/cudamat.cu:538-572.
int perturb_energy(rnd_struct* rnd_state, cudamat* mat, cudamat* target) {
  return launch<kPerturbEnergy>(rnd_state, mat, target);
}
int perturb_prob(rnd_struct* rnd_state, cudamat* mat, cudamat* target) {
  return launch<kPerturbProb>(rnd_state, mat, target);
}
// cudamat/cudamat.cu:574-590.
int dropout(rnd_struct* rnd_state, cudamat* mat, float dropprob, float val) {
  return launch<kDropout>(rnd_state, mat, mat, dropprob, val);
}

}  // extern "C"
