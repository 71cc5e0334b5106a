// The data-parallel exchange and the parameter update as ONE pass over peer memory.
//
// With NCCL the update of a data-parallel step is: all-reduce of the packed statistics (every rank
// ends up with all 268 MB of sums), then every rank applies the same update to its whole copy of W.
// Here rank r owns the columns [r H/G, (r+1) H/G) of W.  The statistics product itself delivers every
// column panel to its owner: its epilogue stores the tiles of panel q into slot r of rank q's receive
// buffer with plain stores over NVLink while the product runs (set_product_scatter in gemm_tc.cu; when
// H/G is not a whole number of 256-column tiles the owners fetch the panels with plain loads instead).
// Once every rank's statistics are in place, r adds the G partial statistics of its columns in rank
// order (all of them in its own memory), applies the momentum / decay update to its
// shard of W and of the update history, and stores the new shard (and its 16-bit planes) into EVERY
// rank's copy of W with plain stores.  Each rank moves (G-1)/G of the statistics in and (G-1)/G
// of W + planes out, in both directions of its links at once, instead of the all-reduce's two
// passes followed by a separate update; replicas are bit-identical by construction (every element
// is computed once, by its owner).  The bias statistics (V + H floats) are summed by every rank.
//
// Synchronisation: three integers per peer in a small flag array that every rank maps from every
// other (CUDA IPC): ready[g] = g's statistics of update n are complete, done[g] = g has stored its
// shard of update n everywhere, maxbits[g] = the largest |w| of g's new shard.  All waits are
// bounded (b200_set_wait_limit); on expiry the kernel records a status word and returns.
// No multimem, no TMA, no library kernel touches peer memory: plain ld / st in this file only.
// The reference has no multi-GPU layer; nothing here has a counterpart there.
#include <stdlib.h>
#include <string.h>

#include "gemm.cuh"

using namespace b200;

namespace {

constexpr int kMaxRanks = 8;
enum { kReady = 0, kDone = 8, kMaxBits = 16, kFlagInts = 32 };

struct PeerCtx {
  int nranks = 0, rank = 0;
  float* pack[kMaxRanks] = {nullptr};      // every rank's packed statistics [W | b_v | b_h]
  float* w[kMaxRanks] = {nullptr};         // every rank's copy of W
  uint16_t* aux[kMaxRanks] = {nullptr};    // ... and of W's 16-bit planes (or null)
  int* flags[kMaxRanks] = {nullptr};       // every rank's flag array
  float* recv[kMaxRanks] = {nullptr};      // every rank's receive buffer: G slots (one per sender) of one column panel each
  float* own_recv = nullptr;
  long recv_floats = 0;
  bool push = false;                       // the statistics product delivers the panels (else the owners fetch them)
  int* own_flags = nullptr;
  unsigned* ticket = nullptr;
  int epoch = 0;
  bool open[kMaxRanks][5] = {};
} g;

struct PeerPtrs {
  const float* stat[kMaxRanks];   // rank q's statistics of THIS rank's panel, indexed like W (element e of W at stat[q][e])
  float* pack[kMaxRanks];
  float* w[kMaxRanks];
  uint16_t* aux[kMaxRanks];
  int* flags[kMaxRanks];
};

__device__ __forceinline__ int ld_flag(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_flag(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Tells every rank that this rank's statistics of update `epoch` are complete (runs after them on the stream).
__global__ void k_peer_signal(PeerPtrs pp, int nranks, int rank, int epoch) {
  if (threadIdx.x < nranks) {
    __threadfence_system();
    st_flag(pp.flags[threadIdx.x] + kReady + rank, epoch);
  }
}

// Bounded wait until flags[base + g] >= epoch for every g.  One thread per rank; returns false on time-out.
__device__ bool wait_all(const int* flags, int base, int nranks, int epoch, uint32_t limit, int* status, int code) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < nranks) {
    bool seen = false;
    for (uint32_t i = 0; i < limit; i++) {
      if (ld_flag(flags + base + threadIdx.x) >= epoch) {
        seen = true;
        break;
      }
      __nanosleep(100);
    }
    if (!seen) {
      ok = 0;
      atomicCAS(status, 0, code);
    }
  }
  __syncthreads();
  return ok != 0;
}

__device__ __forceinline__ void update_elem(float& w, float& d, float suff, float ninv_batch, float momentum, float neps,
                                            float l2, float l1) {
  // the call sequence of deepnet/dbm.py:254 + parameter.py:89-106, products and sums rounded separately
  const float grad = __fmul_rn(suff, ninv_batch);
  d = __fmul_rn(d, momentum);
  if (l2 != 0.0f) d = __fadd_rn(d, __fmul_rn(w, l2));
  if (l1 != 0.0f) d = __fadd_rn(d, w == 0.0f ? 0.0f : (w > 0.0f ? l1 : -l1));
  d = __fadd_rn(d, grad);
  w = __fadd_rn(w, __fmul_rn(d, neps));
}

// aux_mode 0 none, 1 bfloat16 parts, 2 scaled half precision (scale = 2^(scale_state[0])).
__global__ void __launch_bounds__(256) k_peer_reduce_update(PeerPtrs pp, int nranks, int rank, int epoch, float* delta,
                                                            int rows, int lda, long first, long count, int aux_mode,
                                                            const float* scale_state, float ninv_batch, float momentum,
                                                            float neps, float l2, float l1, float* bias, float* dbias,
                                                            long bias_first, int nbias, float mom_b, float neps_b,
                                                            unsigned* ticket, uint32_t limit, int* status) {
  if (!wait_all(pp.flags[rank], kReady, nranks, epoch, limit, status, 21)) return;
  const float f16_scale = aux_mode == 2 ? exp2f(scale_state[0]) : 1.0f;
  float wmax = 0.0f;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  for (long i = tid; i < (count >> 2); i += nth) {           // rows % 4 == 0: four elements share a column
    const long e = first + (i << 2);
    float4 S = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < nranks; q++) {                        // rank order: the same sum whoever computes it
      const float4 s = *reinterpret_cast<const float4*>(pp.stat[q] + e);
      S.x += s.x; S.y += s.y; S.z += s.z; S.w += s.w;
    }
    float4 W = *reinterpret_cast<const float4*>(pp.w[rank] + e);
    float4 D = *reinterpret_cast<const float4*>(delta + e);
    update_elem(W.x, D.x, S.x, ninv_batch, momentum, neps, l2, l1);
    update_elem(W.y, D.y, S.y, ninv_batch, momentum, neps, l2, l1);
    update_elem(W.z, D.z, S.z, ninv_batch, momentum, neps, l2, l1);
    update_elem(W.w, D.w, S.w, ninv_batch, momentum, neps, l2, l1);
    *reinterpret_cast<float4*>(delta + e) = D;
    ushort4 L = make_ushort4(0, 0, 0, 0), Hh = L;
    const long c = e / rows, r = e - c * rows;
    if (aux_mode == 2) {
      wmax = fmaxf(fmaxf(wmax, fmaxf(fabsf(W.x), fabsf(W.y))), fmaxf(fabsf(W.z), fabsf(W.w)));
      split_f16(W.x, f16_scale, L.x, Hh.x); split_f16(W.y, f16_scale, L.y, Hh.y);
      split_f16(W.z, f16_scale, L.z, Hh.z); split_f16(W.w, f16_scale, L.w, Hh.w);
    } else if (aux_mode == 1) {
      split_aux(W.x, L.x, Hh.x); split_aux(W.y, L.y, Hh.y); split_aux(W.z, L.z, Hh.z); split_aux(W.w, L.w, Hh.w);
    }
    for (int q = 0; q < nranks; q++) {                        // the new shard goes into every replica
      *reinterpret_cast<float4*>(pp.w[q] + e) = W;
      if (aux_mode) {
        uint16_t* dst = pp.aux[q] + c * 2 * lda + r;
        *reinterpret_cast<ushort4*>(dst) = L;
        *reinterpret_cast<ushort4*>(dst + lda) = Hh;
      }
    }
  }
  // every rank sums the bias statistics of all ranks itself (V + H floats) and updates its own biases
  // (before `done`: a peer may overwrite its statistics as soon as it has seen every rank's `done`)
  for (long i = tid; i < nbias; i += nth) {
    float sb = 0.0f;
    for (int q = 0; q < nranks; q++) sb += pp.pack[q][bias_first + i];
    float w = bias[i], d = dbias[i];
    update_elem(w, d, sb, ninv_batch, mom_b, neps_b, 0.0f, 0.0f);
    bias[i] = w;
    dbias[i] = d;
  }
  if (aux_mode == 2) {
    const unsigned m = __reduce_max_sync(0xffffffffu, __float_as_uint(wmax));
    if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<unsigned*>(pp.flags[rank]) + kMaxBits + rank, m);
  }
  // the block that finishes last publishes this rank's shard: its maximum, then `done`
  __shared__ bool is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence_system();
  if (threadIdx.x < nranks) {
    const int q = threadIdx.x;
    if (aux_mode == 2 && q != rank)
      reinterpret_cast<volatile unsigned*>(pp.flags[q])[kMaxBits + rank] =
          reinterpret_cast<volatile unsigned*>(pp.flags[rank])[kMaxBits + rank];
    __threadfence_system();
    st_flag(pp.flags[q] + kDone + rank, epoch);
  }
  if (threadIdx.x == 0) *ticket = 0u;
}

// Waits until every rank has stored its shard, then settles the exponent of the scaled half-precision
// form from the largest |w| over ALL shards (same decision on every rank): see k_update_scale.
__global__ void k_peer_finish(PeerPtrs pp, int nranks, int rank, int epoch, float* scale_state, uint32_t limit, int* status) {
  if (!wait_all(pp.flags[rank], kDone, nranks, epoch, limit, status, 22)) return;
  if (threadIdx.x != 0 || !scale_state) return;
  unsigned mb = 0;
  volatile unsigned* f = reinterpret_cast<volatile unsigned*>(pp.flags[rank]);
  for (int q = 0; q < nranks; q++) {
    mb = max(mb, f[kMaxBits + q]);
    f[kMaxBits + q] = 0u;      // (the owners write their next maximum only after the next `ready` round)
  }
  const float m = __uint_as_float(mb);
  float redo = 0.0f;
  if (m > 0.0f && m < 3.0e38f) {
    const float want = fminf(fmaxf(floorf(log2f(8192.0f / m)), -100.0f), 100.0f);
    const float d = scale_state[0] - want;
    if (d < -1.0f || d > 2.0f) {
      scale_state[0] = want;
      redo = 1.0f;
    }
  }
  scale_state[1] = scale_state[0];
  scale_state[3] = redo;
  reinterpret_cast<unsigned*>(scale_state)[2] = 0u;
}

PeerPtrs ptrs(long first, long shard) {
  PeerPtrs pp;
  for (int q = 0; q < kMaxRanks; q++) {
    // delivered: slot q of the own receive buffer holds rank q's panel (shard floats); fetched: rank q's whole statistics
    pp.stat[q] = g.push ? (g.own_recv ? g.own_recv + (long)q * shard - first : nullptr) : g.pack[q];
    pp.pack[q] = g.pack[q];
    pp.w[q] = g.w[q];
    pp.aux[q] = g.aux[q];
    pp.flags[q] = g.flags[q];
  }
  return pp;
}

}  // namespace

extern "C" {

// Bytes of one exported handle.
int dp_peer_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }

// handle_out (dp_peer_handle_bytes() bytes) lets another process on this node map the matrix's storage
// (it must be a whole allocation of this library, not a view).
int dp_peer_export(cudamat* m, char* handle_out) {
  if (!m->on_device) return ERROR_NOT_ON_DEVICE;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, m->data_device) != cudaSuccess) return set_error(cudaGetErrorString(cudaGetLastError()));
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

// The library's flag array of this rank (created on first use), exported like a matrix.
int dp_peer_export_flags(char* handle_out) {
  if (!g.own_flags) {
    if (cudaMalloc(&g.own_flags, kFlagInts * sizeof(int)) != cudaSuccess || cudaMemset(g.own_flags, 0, kFlagInts * sizeof(int)) != cudaSuccess ||
        cudaMalloc(&g.ticket, sizeof(unsigned)) != cudaSuccess || cudaMemset(g.ticket, 0, sizeof(unsigned)) != cudaSuccess)
      return set_error("dp_peer: flag allocation failed");
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, g.own_flags) != cudaSuccess) return set_error(cudaGetErrorString(cudaGetLastError()));
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

// The receive buffer of this rank (created here: `floats` = elements of W; G slots of one column panel
// each, slot r written by rank r's statistics product), exported like a matrix.
int dp_peer_export_recv(long floats, char* handle_out) {
  if (floats <= 0) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (g.own_recv && g.recv_floats != floats) {
    cudaFree(g.own_recv);
    g.own_recv = nullptr;
  }
  if (!g.own_recv) {
    if (cudaMalloc(&g.own_recv, (size_t)floats * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      g.own_recv = nullptr;
      return set_error("dp_peer: receive buffer allocation failed");
    }
    g.recv_floats = floats;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, g.own_recv) != cudaSuccess) return set_error(cudaGetErrorString(cudaGetLastError()));
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

// handles: for every rank q (in rank order) five handles {pack, W, W_aux, flags, receive buffer} as
// exported by that rank (W_aux all zero when there is none).  Own entries are taken from the matrices
// passed here.  From here on the product whose result is the statistics area of `pack` (its first
// rows(W) x cols(W) floats) delivers its column panels to their owners.
int dp_peer_setup(int nranks, int rank, const char* handles, cudamat* pack, cudamat* w, cudamat* w_aux) {
  if (nranks < 2 || nranks > kMaxRanks || rank < 0 || rank >= nranks) return ERROR_UNSUPPORTED;
  if (!pack->on_device || !w->on_device || (w_aux && !w_aux->on_device) || !g.own_flags || !g.own_recv) return ERROR_NOT_ON_DEVICE;
  if (g.recv_floats != numel(w) || w->size[1] % nranks != 0) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const size_t hb = sizeof(cudaIpcMemHandle_t);
  g.nranks = nranks;
  g.rank = rank;
  for (int q = 0; q < nranks; q++) {
    if (q == rank) {
      g.pack[q] = pack->data_device;
      g.w[q] = w->data_device;
      g.aux[q] = w_aux ? reinterpret_cast<uint16_t*>(w_aux->data_device) : nullptr;
      g.flags[q] = g.own_flags;
      g.recv[q] = g.own_recv;
      continue;
    }
    void* p[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    for (int k = 0; k < 5; k++) {
      if (k == 2 && !w_aux) continue;
      cudaIpcMemHandle_t h;
      memcpy(&h, handles + ((size_t)q * 5 + k) * hb, hb);
      if (cudaIpcOpenMemHandle(&p[k], h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
        return set_error(cudaGetErrorString(cudaGetLastError()));
      g.open[q][k] = true;
    }
    g.pack[q] = (float*)p[0];
    g.w[q] = (float*)p[1];
    g.aux[q] = (uint16_t*)p[2];
    g.flags[q] = (int*)p[3];
    g.recv[q] = (float*)p[4];
  }
  // a second set-up in one process starts from clean flags (the peers write into them only after the
  // host barrier that precedes the first update, and the previous user closed behind a barrier)
  g.epoch = 0;
  if (cudaMemset(g.own_flags, 0, kFlagInts * sizeof(int)) != cudaSuccess || cudaMemset(g.ticket, 0, sizeof(unsigned)) != cudaSuccess)
    return set_error(cudaGetErrorString(cudaGetLastError()));
  // whole 256-column tiles per panel: the statistics product delivers them; otherwise the owners fetch
  const int cols = w->size[1] / nranks;
  const long shard = (long)w->size[0] * cols;
  const char* pv = getenv("B200_DP_PEER_PUSH");      // 0: the owners fetch (measurements)
  g.push = cols % 256 == 0 && (!pv || atoi(pv) != 0);
  if (g.push) {
    float* targets[kMaxRanks];
    for (int q = 0; q < nranks; q++) targets[q] = g.recv[q] + (long)rank * shard;   // this rank's slot at owner q
    return set_product_scatter(pack->data_device, targets, nranks, cols);
  }
  return set_product_scatter(nullptr, nullptr, 0, 0);
}

// One data-parallel update without NCCL: statistics -> parameters on every rank (see the top of this
// file).  pack = [W statistics | b_v | b_h] of THIS rank (already complete on the library stream);
// b / db: the packed biases and their history (V + H); w_scale: the 1 x 4 exponent state or null.
// Every rank must call it once per update, in the same order.
int dp_peer_update(cudamat* w, cudamat* delta, cudamat* w_aux, cudamat* w_scale, cudamat* pack, cudamat* b, cudamat* db,
                   float inv_batch, float mom_b, float eps_b, float mom_w, float eps_w, float l2, float l1) {
  if (g.nranks < 2) return set_error("dp_peer_update before dp_peer_setup");
  if (w->data_device != g.w[g.rank] || pack->data_device != g.pack[g.rank]) return set_error("dp_peer_update: not the matrices of dp_peer_setup");
  const int rows = w->size[0], cols = w->size[1];
  if (rows % 4 != 0 || cols % g.nranks != 0) return ERROR_UNSUPPORTED;
  if (!same_shape(w, delta) || numel(b) != numel(db) || numel(pack) != numel(w) + numel(b)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int mode = !w_aux ? 0 : (w_scale ? 2 : 1);
  const long shard = (long)rows * (cols / g.nranks), first = shard * g.rank;
  const int epoch = ++g.epoch;
  const PeerPtrs pp = ptrs(first, shard);
  // waits on other ranks get sixteen times the limit of a wait inside one kernel (about half a
  // minute by default): a rank may be late by a host hiccup, which an in-kernel wait never sees
  const unsigned long long lim64 = (unsigned long long)wait_limit() * 16ull;
  const uint32_t peer_limit = lim64 > 0xffffffffull ? 0xffffffffu : (uint32_t)lim64;
  cudaStream_t st = stream();
  k_peer_signal<<<1, 32, 0, st>>>(pp, g.nranks, g.rank, epoch);
  long blocks = (shard / 4 + 255) / 256;
  if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
  if (blocks < 1) blocks = 1;
  float* sp = w_scale ? w_scale->data_device : nullptr;
  k_peer_reduce_update<<<(int)blocks, 256, 0, st>>>(pp, g.nranks, g.rank, epoch, delta->data_device, rows, aux_rows(rows), first,
                                                   shard, mode, sp, -inv_batch, mom_w, -eps_w, l2, l1, b->data_device,
                                                   db->data_device, numel(w), (int)numel(b), mom_b, -eps_b, g.ticket,
                                                   peer_limit, status_word());
  k_peer_finish<<<1, 32, 0, st>>>(pp, g.nranks, g.rank, epoch, mode == 2 ? sp : nullptr, peer_limit, status_word());
  int err = check_launch();
  if (err || mode != 2) return err;
  // rewrites the planes of the whole local W only when the exponent had to change (device flag)
  return rewrite_f16_planes_if(w->data_device, reinterpret_cast<uint16_t*>(w_aux->data_device), rows, numel(w), sp, sp + 3);
}

// 0: not set up; 1: the owners fetch the statistics panels; 2: the statistics product delivers them.
int dp_peer_mode() { return g.nranks < 2 ? 0 : (g.push ? 2 : 1); }

int dp_peer_close() {
  set_product_scatter(nullptr, nullptr, 0, 0);
  g.push = false;
  for (int q = 0; q < g.nranks; q++) {
    if (q == g.rank) continue;
    void* p[5] = {g.pack[q], g.w[q], g.aux[q], g.flags[q], g.recv[q]};
    for (int k = 0; k < 5; k++)
      if (g.open[q][k] && p[k]) {
        cudaIpcCloseMemHandle(p[k]);
        g.open[q][k] = false;
      }
  }
  g.nranks = 0;
  return 0;
}

}  // extern "C"
