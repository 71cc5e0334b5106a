// Tensor-core matrix product for sm_100a: tcgen05.mma (kind::tf32 and kind::f16 on bfloat16,
// mixed in one accumulator) with the accumulator in tensor memory, fp32 operand tiles staged
// in swizzled shared memory by TMA (cp.async.bulk.tensor, one copy per CTA, never multicast),
// a fused epilogue read back with tcgen05.ld and stored by TMA.  It replaces the cublasSgemm
// behind `dot` (cudamat/cudamat.cu:1671-1696) and the separate bias / sigmoid / Bernoulli
// passes that follow it in deepnet/dbm.py:88-105 and deepnet/logistic_layer.py:11-15.
//
// fp32-grade accuracy comes from the caller's term list over PARTS of the fp32 operands
// (x as TF32, x - tf32(x) as TF32 or bfloat16, bfloat16(x)), all accumulating into ONE fp32
// accumulator.  The parts other than x reach shared memory in one of two ways: four converter
// warps derive them from the staged fp32 tile, in the layout TMA would have produced (nothing
// but x in device memory; costs shared-memory bandwidth next to the tensor core's own operand
// reads), or TMA loads the bfloat16 ones from an aux matrix kept beside x (what the big
// products of the training step use).  The MMA issuer consumes a stage once its loads have
// landed and the converters are done with it.  A term may be negated (instruction-descriptor
// bit), which folds positive-minus-negative statistics into one kernel.
//
// Kernel shape: persistent, one CTA per SM (or a pair of CTAs on a 256-row tile), 512 threads
// (registers move from the first two warpgroups to the epilogue's with setmaxnreg):
//   warp 0      : TMA producer                    -> ring of stages {A tile, B tile}
//   warp 1      : TMEM allocation + MMA issuer (one lane), tcgen05.commit frees stages
//   warps 4..7  : converters: fp32 tile -> the derived tiles of the stage
//   warps 8..15 : epilogue; two warps share each TMEM lane quarter (half the columns each).
//                 They fold every finished chunk of the product into fp32 registers (two TMEM
//                 accumulators ping-pong with the MMA issuer) and run the fused epilogue from
//                 those registers at the end of the tile.
// Every mbarrier wait is bounded; on expiry the kernel records a status word, drains
// and frees its tensor memory and returns.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include <time.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "gemm.cuh"

namespace b200 {

namespace {

constexpr int BM = 128;
constexpr int kMaxStages = 8;
constexpr int kStageBudget = 193 * 1024;      // shared memory available to the operand ring
constexpr int kOutStageBytes = 32 * 1024;      // epilogue staging for TMA stores (two column halves x two buffers)
constexpr int kOutCols = 4;                    // columns per staged batch (one Philox block)
constexpr int kOutArrays = 5;                  // out, its aux planes 0 and 1, sample, plane 1 of the sample's aux
constexpr int kMaxLoads = 6;                   // A and B as fp32, and up to two bfloat16 planes of each from their aux
constexpr int kMaxTiles = 8;                   // tiles of a stage: A and B as loaded + up to three derived parts each
constexpr int kMaxMma = 4;                     // terms issued from one stage
constexpr uint32_t kNoTile = 0xffffffffu;

// How tcgen05 reads one staged tile.
struct TcTile {
  uint32_t desc_hi;        // upper 32 bits of the shared-memory matrix descriptor
  uint32_t desc_lo;        // leading-byte-offset field (bits 16-29 of the low word)
  uint32_t adv;            // descriptor advance per MMA (K = 8 floats or 16 bfloat16), in 16-byte units
  uint32_t smem_off;       // byte offset of the tile inside a stage
};
// One operand tile of a k-block as TMA loads it: fp32, or one bfloat16 plane of an aux matrix.
// (The parameter block travels with every launch: small types keep it under 4 KB, above which a
// launch costs about twice as much on the host.)
struct TcLoad {
  uint8_t map;             // index into TcParams::maps
  uint8_t mn;              // 1: M/N is the contiguous direction in memory (loaded as boxes of 128 bytes x bk)
  uint8_t is_a;
  uint8_t box_rows;        // rows of M/N per box of an MN-major tile: 32 floats or 64 bfloat16
  uint32_t smem_off;
};
// The parts derived from a loaded tile (offsets inside the stage, kNoTile = not wanted).
struct TcConv {
  uint32_t src_off;
  uint32_t lo32_off, lo16_off, b16_off;
  int mn;
  int is_a;
};
struct TcMma {
  uint8_t a, b;            // tiles of the group
  uint8_t f16;             // 0: kind::tf32 (K = 8 per instruction), 1: kind::f16 on bfloat16 (K = 16)
  uint32_t idesc;          // tcgen05 instruction descriptor (carries the negate bit)
};
// A group = the terms over one pair of fp32 operands (and so one K range).  Each k-block stages
// every tile the terms read once (the fp32 tiles and aux planes by TMA, derived parts by the
// converters), and all the group's products are issued from that one stage.
struct TcGroup {
  int k_iters;             // ceil(k / bk)
  int nload, nconv, nmma;
  uint32_t stage_tx;       // bytes TMA delivers per k-block and CTA
  TcLoad load[kMaxLoads];
  TcConv conv[2];
  TcTile tile[kMaxTiles];
  TcMma mma[kMaxMma];
};

constexpr int kMaxGroups = 4;   // pairs of operand matrices in one product (a DBM layer update and the statistics have two)
constexpr int kMaxScatter = 8;
constexpr int kMaxMaps = 16;    // tensor maps: operand tiles as loaded, then the outputs an activation epilogue stores

struct TcParams {
  CUtensorMap maps[kMaxMaps];
  TcGroup group[kMaxGroups];
  int ngroups;
  int M, N, tiles_m, tiles_n;
  int bk;                  // floats of K per k-block: 32 or 16
  int num_stages;          // ring depth
  uint32_t stage_bytes;    // ring pitch
  int chunk_iters;         // k-blocks per TMEM accumulation chunk (128 products)
  int splits;              // > 1: split-K: work item = (tile, split); split s multiplies k-blocks [ki*s/splits, ki*(s+1)/splits)
                           //      of every group and stores its raw fp32 partial at epi.out + s * split_stride
  long split_stride;       // floats between two partials
  int direct;              // 1: no group derives anything: the copies of both CTAs complete on the leader's `ready`
                           //    barrier and the converter warps stay out of the way
  int store16;             // 1: the epilogue's only outputs are 16-bit planes (the draw's, or the result's two): every
                           //    thread stores them straight to global memory (64 bytes per warp and column); no
                           //    staging, barriers or TMA stores, whose latency otherwise keeps the epilogue warps
                           //    from draining the next tile's first chunk in time
  GemmEpilogue epi;
  // Column panels of a plain result delivered to other GPUs (scatter_cols > 0): columns
  // [q * scatter_cols, (q + 1) * scatter_cols) go to scatter[q] (columns ldo apart, as epi.out) with
  // plain stores, over NVLink when scatter[q] is peer memory: the reduce-scatter of the data-parallel
  // statistics happens while the product runs (dp_peer.cu).  A tile never straddles two panels.
  float* scatter[kMaxScatter];
  int scatter_cols;
  int out_map[kOutArrays];   // tensor maps (indices into maps) of the outputs stored by TMA; -1 = absent
  int* status;
  uint32_t spin_limit;       // iterations a wait may spin before the kernel gives up (b200_set_wait_limit)
#ifdef B200_GEMM_TIMING
  unsigned long long* dbg;   // per CTA: issuer total, wait-full, wait-tmem-empty; producer wait-empty; epilogue wait
#endif
};
#ifdef B200_GEMM_TIMING
#define TIMED_WAIT(acc_var, call) \
  [&]() { const long long t0 = clock64(); const bool r = (call); acc_var += clock64() - t0; return r; }()
#else
#define TIMED_WAIT(acc_var, call) (call)
#endif

// ---- PTX wrappers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the limit ran out or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t limit) {
  for (uint32_t i = 0; i < limit; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(40);
    if ((i & 1023) == 1023 && *abort_flag) return false;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar));
}

// Shared -> global tile store (clipped at the tensor's edges), tracked by bulk async-groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y),
               "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- two-CTA (cta_group::2) forms: the pair of CTAs of a cluster works on one 256-row tile.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Shared-window addresses carry the CTA's rank within the pair in bit 24; clearing it names the
// same location in the pair's leader (rank 0).
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;
// Loads into THIS CTA's shared memory, completes the transaction on the LEADER's mbarrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar & kPeerBitMask));
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One instruction multiplies a 256-row A (128 rows from each CTA's shared memory) by B (half of
// its N rows from each CTA) into both CTAs' tensor memory.
__device__ __forceinline__ void mma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
}
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
}
// Arrives (once all earlier MMAs of this thread are done) on the barrier at this offset in
// every CTA named by the mask.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(cta_mask)
               : "memory");
}
// Arrive on the barrier at this offset in the pair's leader.  Default semantics (release at
// CTA scope), as a consumer releasing a stage to its producer does: a cluster-scope release
// costs about 0.5 us per arrive here, more than a whole k-block.  What the leader's tensor core
// then reads from this CTA's shared memory was made visible to the async proxy by the proxy
// fence that precedes the arrive.
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, 0;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}" ::"r"(bar)
      : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Tile order: groups of 16 row tiles sweep the column tiles, so that one wave of
// CTAs shares a compact set of A and B panels in L2.
template <int GM>
__device__ __forceinline__ void tile_coords_g(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = GM * tiles_n;
  const int g = t / per_group;
  const int first = g * GM;
  const int gsize = min(GM, tiles_m - first);
  const int r = t - g * per_group;
  tm = first + r % gsize;
  tn = r / gsize;
}
// One wave of CTAs should cover about as many A rows as B rows: 16 row tiles of 128 (one CTA per
// tile) or 8 row tiles of 256 (paired CTAs) against about 9 column tiles of 256.
#define tile_coords(t, tiles_m, tiles_n, tm, tn) tile_coords_g<(kTwo ? 8 : 16)>(t, tiles_m, tiles_n, tm, tn)

// The tensor core adds into its fp32 accumulator with truncation, not round-to-nearest:
// a same-sign sum loses about 0.6 ulp per tcgen05.mma (-646 ulp measured at K = 8192,
// 5e-5 relative).  To keep fp32-grade results the accumulation is split into chunks of
// kChunkIters k-iterations (128 products): each chunk starts a fresh TMEM accumulator
// (two of them ping-pong) and the epilogue warps add the finished chunk into fp32
// registers with ordinary rounding while the next chunk is being multiplied.
constexpr int kEpiWarps = 8;
constexpr int kConvWarps = 4;
constexpr int kFirstConvWarp = 4, kFirstEpiWarp = kFirstConvWarp + kConvWarps;   // warps 2, 3 only hold their place
constexpr int kThreadsTc = 32 * (kFirstEpiWarp + kEpiWarps);
// Registers per thread: the kernel starts with 65536 / 512 = 128 everywhere; the two epilogue
// warpgroups (128 accumulator columns per thread) grow to kEpiRegs with what the other two give up.
constexpr int kEpiRegs = 176, kOtherRegs = 80;
static_assert(kFirstEpiWarp == 8 && kEpiWarps == 8 && kEpiRegs + kOtherRegs <= 256, "register split between warpgroups");

template <int BN>
struct TcConfig {
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kColsPerWarp = BN / 2;   // each lane quarter is shared by two epilogue warps
  static constexpr int kSmemBytes = kStageBudget + kOutStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// Epilogue variants, chosen on the host.  The common cases are compiled without run-time
// branches (they are instruction-bound otherwise):
//   kEpiPlain      out = alpha * acc (+ beta * out)                  (`dot`, statistics)
//   kEpiSig        out = logistic(alpha * acc + bias)
//   kEpiSigSample  kEpiSig plus sample = Bernoulli(out)
//   kEpiLin        out = alpha * acc + bias
//   kEpiGeneric    every option tested at run time
//   kEpiPartial    kEpiPlain for one split of a split-K product: raw partial sums to the workspace
//                  (the only variant that carries the work-item bookkeeping of split-K)
enum { kEpiPlain = 0, kEpiGeneric = 1, kEpiSig = 2, kEpiSigSample = 3, kEpiLin = 4, kEpiPartial = 5 };
__host__ __device__ constexpr bool epi_is_plain(int e) { return e == kEpiPlain || e == kEpiPartial; }

// Two packed bfloat16 (round to nearest even): `lo` goes to the lower address.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
// (volatile keeps these in program order among themselves and with the barrier operations; no
// memory clobber, so that the arithmetic between them can be scheduled freely)
__device__ __forceinline__ void sts128(uint32_t addr, float4 v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w));
}
__device__ __forceinline__ void sts128u(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w));
}
__device__ __forceinline__ float tf32_rest(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

// Derives the wanted parts of sixteen elements: four 16-byte chunks of the fp32 tile at s[0..3]
// (s[0], s[1] are eight consecutive elements, s[2], s[3] the next eight).  x - tf32(x) goes as
// fp32 to the same places of the lo32 tile (d32 - src apart), and as bfloat16 / bfloat16(x) to one
// 16-byte chunk per eight elements of the lo16 / b16 tiles.  All loads are issued first.
__device__ __forceinline__ void convert16(const uint32_t (&s)[4], bool lo32, uint32_t d32_minus_src, bool lo16,
                                          uint32_t d_lo16_0, uint32_t d_lo16_1, bool b16, uint32_t d_b16_0,
                                          uint32_t d_b16_1) {
  float4 x[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; i++) x[i] = lds128(s[i]);
  if (lo32 || lo16) {
#pragma unroll
    for (int i = 0; i < 4; i++)
      l[i] = make_float4(tf32_rest(x[i].x), tf32_rest(x[i].y), tf32_rest(x[i].z), tf32_rest(x[i].w));
  }
  if (lo32) {
#pragma unroll
    for (int i = 0; i < 4; i++) sts128(s[i] + d32_minus_src, l[i]);
  }
  if (lo16) {
    sts128u(d_lo16_0, make_uint4(pack_bf16(l[0].x, l[0].y), pack_bf16(l[0].z, l[0].w), pack_bf16(l[1].x, l[1].y),
                                 pack_bf16(l[1].z, l[1].w)));
    sts128u(d_lo16_1, make_uint4(pack_bf16(l[2].x, l[2].y), pack_bf16(l[2].z, l[2].w), pack_bf16(l[3].x, l[3].y),
                                 pack_bf16(l[3].z, l[3].w)));
  }
  if (b16) {
    sts128u(d_b16_0, make_uint4(pack_bf16(x[0].x, x[0].y), pack_bf16(x[0].z, x[0].w), pack_bf16(x[1].x, x[1].y),
                                pack_bf16(x[1].z, x[1].w)));
    sts128u(d_b16_1, make_uint4(pack_bf16(x[2].x, x[2].y), pack_bf16(x[2].z, x[2].w), pack_bf16(x[3].x, x[3].y),
                                pack_bf16(x[3].z, x[3].w)));
  }
}

// kTwo: two CTAs of a cluster share one 256 x BN tile (cta_group::2): each stages its own 128
// rows of A and half of B's rows, the leader issues the MMAs for both.
template <int BN, int kEpi, bool kTwo>
__global__ void __launch_bounds__(kThreadsTc, 1) k_gemm_tc(const __grid_constant__ TcParams p) {
  using Cfg = TcConfig<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t out_stage_base = smem_base + kStageBudget;
  const uint32_t bar_base = out_stage_base + kOutStageBytes;
  // barrier layout (8 bytes each): full[kMaxStages], empty[kMaxStages], ready[kMaxStages], tmem_full[2], tmem_empty[2]
  //   full  : this CTA's TMA copies of the stage have landed            (producer -> converters)
  //   ready : the derived tiles of the stage are written, in both CTAs   (converters -> issuer of the leader);
  //           when nothing is derived (p.direct) the copies of both CTAs complete on it themselves
  //   empty : the MMAs that read the stage are done                      (issuer -> producer, both CTAs)
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto ready_bar = [&](int s) { return bar_base + 8u * (2 * kMaxStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (3 * kMaxStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (3 * kMaxStages + 2 + a); };
  static_assert(8 * (3 * kMaxStages + 4) <= 256, "barrier area");
  const int num_stages = p.num_stages;
  const uint32_t stage_bytes = p.stage_bytes;
  const int bk = p.bk;
  const uint32_t spin_limit = p.spin_limit;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  grid_dependents_launch();   // the next kernel of the stream may be scheduled as SMs free up
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int splits = (kEpi == kEpiPartial) ? p.splits : 1;
  const int num_tiles = p.tiles_m * p.tiles_n * splits;     // work items: every role walks the same list
  const uint32_t rank = kTwo ? cluster_ctarank() : 0u;        // 0 = leader of the pair
  const int first_tile = kTwo ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tile_step = kTwo ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  constexpr int TILE_M = kTwo ? 2 * BM : BM;                  // rows of the tile a CTA (pair) owns
  constexpr int BN_LOCAL = kTwo ? BN / 2 : BN;                // B rows staged by this CTA

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kMaxStages; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(ready_bar(s), p.direct ? 1 : (kTwo ? 2 * kConvWarps : kConvWarps));
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), kTwo ? 2 * kEpiWarps : kEpiWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (kTwo) {
      tmem_alloc2(smem_u32(&tmem_base_slot), Cfg::kTmemCols);
      tmem_relinquish2();
    } else {
      tmem_alloc(smem_u32(&tmem_base_slot), Cfg::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (kTwo) cluster_sync();   // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  // Everything above (barriers, TMEM) touched no global memory and may have run while the previous
  // kernel of the stream was still finishing; operands, biases and outputs are touched only from here on.
  grid_dependency_wait();

  const int kChunkIters = p.chunk_iters;
  // k-blocks of group q that split s multiplies (all of them when the product is not split)
  auto split_range = [&](int q, int s, int& kb0, int& kb1) {
    const int ki = p.group[q].k_iters;
    kb0 = (int)(((unsigned)ki * (unsigned)s) / (unsigned)splits);          // (k-blocks x splits stays far below 2^32)
    kb1 = (int)(((unsigned)ki * (unsigned)(s + 1)) / (unsigned)splits);
  };
  auto item_k_iters = [&](int s) {
    int n = 0;
    for (int q = 0; q < p.ngroups; q++) {
      int kb0, kb1;
      split_range(q, s, kb0, kb1);
      n += kb1 - kb0;
    }
    return n;
  };

  // Every warpgroup (four warps) passes ONE setmaxnreg instruction, at the top of its branch.
  if (warp < kFirstConvWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // The whole warp runs the loop; copy u = 8 * load + box (up to six loads of up to 8 boxes: an
    // MN-major tile comes as boxes of 128 bytes x bk) is issued by lane u % 32, so a lane issues at
    // most two copies per k-block.  The refill of a freed stage is on the critical path of a ring
    // this shallow: every constant sits in registers.
    {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long t_empty = 0;
      const bool direct = p.direct != 0;
      for (int w = first_tile; w < num_tiles && ok; w += tile_step) {
        const int t = w / splits, sp = w - t * splits;
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * TILE_M + (int)rank * BM, n0 = tn * BN + (int)rank * BN_LOCAL;
        for (int q = 0; q < p.ngroups && ok; q++) {
          const TcGroup& gr = p.group[q];
          int kb_first, kb_last;
          split_range(q, sp, kb_first, kb_last);
          bool active[2];
          const CUtensorMap* map[2];
          int row0[2], mn[2];
          uint32_t dst_off[2];
#pragma unroll
          for (int c = 0; c < 2; c++) {
            const int u = lane + 32 * c, li = u >> 3, box = u & 7;
            active[c] = li < gr.nload;
            const TcLoad ld = gr.load[active[c] ? li : 0];
            const int nboxes = ld.mn ? (ld.is_a ? BM : BN_LOCAL) / ld.box_rows : 1;
            active[c] = active[c] && box < nboxes;
            map[c] = &p.maps[ld.map];
            row0[c] = (ld.is_a ? m0 : n0) + (ld.mn ? ld.box_rows * box : 0);
            dst_off[c] = ld.smem_off + (ld.mn ? (uint32_t)(box * bk * 128) : 0u);
            mn[c] = ld.mn;
          }
          for (int kb = kb_first; kb < kb_last; kb++) {
            if (!TIMED_WAIT(t_empty, mbar_wait(empty_bar(stage), phase ^ 1u, &abort_flag, spin_limit))) {
              ok = false;
              if (!abort_flag) atomicCAS(p.status, 0, 1);
              abort_flag = 1;
              break;
            }
            const int k0 = kb * bk;
            if (direct) {
              // nothing to derive: the leader's `ready` barrier collects the bytes of both CTAs
              const uint32_t bar = ready_bar(stage);
              if (lane == 0 && rank == 0) mbar_expect_tx(bar, kTwo ? 2 * gr.stage_tx : gr.stage_tx);
#pragma unroll
              for (int c = 0; c < 2; c++) {
                if (active[c]) {
                  const uint32_t dst = smem_base + stage * stage_bytes + dst_off[c];
                  const int x = mn[c] ? row0[c] : k0, y = mn[c] ? k0 : row0[c];
                  if (kTwo) tma_load_2d_pair(dst, map[c], x, y, bar);
                  else tma_load_2d(dst, map[c], x, y, bar);
                }
              }
            } else {
              const uint32_t bar = full_bar(stage);
              if (lane == 0) mbar_expect_tx(bar, gr.stage_tx);
              __syncwarp();   // the expectation is posted before any copy can complete
#pragma unroll
              for (int c = 0; c < 2; c++) {
                if (active[c]) {
                  const uint32_t dst = smem_base + stage * stage_bytes + dst_off[c];
                  const int x = mn[c] ? row0[c] : k0, y = mn[c] ? k0 : row0[c];
                  tma_load_2d(dst, map[c], x, y, bar);
                }
              }
            }
            if (++stage == num_stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
#ifdef B200_GEMM_TIMING
      if (p.dbg && lane == 0) p.dbg[blockIdx.x * 8 + 3] = (unsigned long long)t_empty;
#else
      (void)t_empty;
#endif
      if (!ok && lane == 0) {
        // let copies already issued land before the CTA leaves
        for (int s = 0; s < num_stages; s++) {
          for (uint32_t i = 0; i < 4096; i++) {
            const uint32_t bar = direct ? ready_bar(s) : full_bar(s);   // (a peer's copies report to the leader)
            if (mbar_try_wait(bar, 0) || mbar_try_wait(bar, 1)) break;
            __nanosleep(100);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (the pair's leader only)
    // The whole warp walks the loops and one elected lane issues: computed by a single diverged
    // lane, every operand of a tcgen05.mma has to be moved from that lane's registers to the
    // uniform registers the instruction reads, about 50 ns per MMA whatever its size, and the
    // issuing thread, not the tensor pipe, bounds the kernel.
    if (rank == 0) {
      const bool elected = elect_one();
      uint32_t chunk = 0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long t_full = 0, t_tempty = 0;
      const long long t_start = clock64();
      for (int w = first_tile; w < num_tiles && ok; w += tile_step) {
        const int sp = w % splits;
        const int total_k_iters = item_k_iters(sp);
        int in_tile = 0, in_chunk = 0;
        uint32_t fresh = 1;
        for (int q = 0; q < p.ngroups && ok; q++) {
          const TcGroup& gr = p.group[q];
          int kb_first, kb_last;
          split_range(q, sp, kb_first, kb_last);
          // The issuing thread must launch an MMA every ~70 ns to keep the tensor pipe busy, and what
          // it does between two k-blocks is not hidden behind the pipe: all per-product constants
          // live in registers, the k-loop only adds the stage address, and the common term lists
          // (count and which terms are bfloat16 known at compile time) run as straight-line code.
          auto run_group = [&](auto nm_c, auto mask_c, auto steps_c) {
            constexpr int kNm = decltype(nm_c)::value;       // -1: count and kinds read from the group
            constexpr int kMask = decltype(mask_c)::value;   // bit i: term i is a bfloat16 product
            constexpr int kSteps16 = decltype(steps_c)::value;   // 16-bit MMAs (K = 16) per term and k-block: bk / 16
            const int nm = kNm >= 0 ? kNm : gr.nmma;
            const int k_iters = kb_last - kb_first;
            uint32_t a_lo[kMaxMma], b_lo[kMaxMma], a_hi[kMaxMma], b_hi[kMaxMma], a_adv[kMaxMma], b_adv[kMaxMma],
                idesc[kMaxMma];
            bool f16[kMaxMma];
#pragma unroll
            for (int i = 0; i < kMaxMma; i++) {
              a_lo[i] = b_lo[i] = a_hi[i] = b_hi[i] = a_adv[i] = b_adv[i] = idesc[i] = 0;
              f16[i] = false;
              if (i < nm) {
                f16[i] = kNm >= 0 ? ((kMask >> i) & 1) != 0 : gr.mma[i].f16 != 0;
                const TcTile ta = gr.tile[gr.mma[i].a];
                const TcTile tb = gr.tile[gr.mma[i].b];
                a_lo[i] = ta.desc_lo + (ta.smem_off >> 4);
                b_lo[i] = tb.desc_lo + (tb.smem_off >> 4);
                a_hi[i] = ta.desc_hi;
                b_hi[i] = tb.desc_hi;
                a_adv[i] = ta.adv;
                b_adv[i] = tb.adv;
                idesc[i] = gr.mma[i].idesc;
              }
            }
            for (int kb = 0; kb < k_iters; kb++) {
              const int acc = chunk & 1;
              if (in_chunk == 0) {
                // a new chunk: its TMEM accumulator must have been drained by the epilogue warps
                if (!TIMED_WAIT(t_tempty, mbar_wait(tempty_bar(acc), ((chunk >> 1) & 1u) ^ 1u, &abort_flag, spin_limit))) {
                  ok = false;
                  if (!abort_flag) atomicCAS(p.status, 0, 2);
                  abort_flag = 1;
                  break;
                }
                tc_fence_after();
                fresh = 1;
              }
              // the stage is loaded and converted in both CTAs
              if (!TIMED_WAIT(t_full, mbar_wait(ready_bar(stage), phase, &abort_flag, spin_limit))) {
                ok = false;
                if (!abort_flag) atomicCAS(p.status, 0, 3);
                abort_flag = 1;
                break;
              }
              // No tcgen05 fence here: a fence per k-block would make the issuer wait for the MMAs in
              // flight.  The tiles were written through the async proxy (TMA) or made visible to it by
              // the converters' proxy fence, ordered by the mbarriers.
              const uint32_t d_tmem = tmem_base + acc * BN;
              const uint32_t sb = (smem_base + stage * stage_bytes) >> 4;   // stage address, 16-byte units
#pragma unroll
              for (int i = 0; i < kMaxMma; i++) {
                if (i < nm) {
                  const uint32_t al = a_lo[i] + sb, bl = b_lo[i] + sb;
                  if (f16[i]) {
                    // 16-bit operands: K = 16 per instruction, bk / 16 instructions per k-block
#pragma unroll
                    for (int j = 0; j < kSteps16; j++) {
                      const uint64_t a_desc = ((uint64_t)a_hi[i] << 32) | (uint64_t)(al + j * a_adv[i]);
                      const uint64_t b_desc = ((uint64_t)b_hi[i] << 32) | (uint64_t)(bl + j * b_adv[i]);
                      const uint32_t accumulate = (i == 0 && j == 0) ? (fresh ^ 1u) : 1u;
                      if (elected) {
                        if (kTwo) mma_f16_pair(d_tmem, a_desc, b_desc, idesc[i], accumulate);
                        else mma_f16(d_tmem, a_desc, b_desc, idesc[i], accumulate);
                      }
                    }
                  } else {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                      const uint64_t a_desc = ((uint64_t)a_hi[i] << 32) | (uint64_t)(al + j * a_adv[i]);
                      const uint64_t b_desc = ((uint64_t)b_hi[i] << 32) | (uint64_t)(bl + j * b_adv[i]);
                      const uint32_t accumulate = (i == 0 && j == 0) ? (fresh ^ 1u) : 1u;
                      if (elected) {
                        if (kTwo) mma_tf32_pair(d_tmem, a_desc, b_desc, idesc[i], accumulate);
                        else mma_tf32(d_tmem, a_desc, b_desc, idesc[i], accumulate);
                      }
                    }
                  }
                }
              }
              fresh = 0;
              // the stage is free (in both CTAs of a pair) once these MMAs have read it
              if (elected) {
                if (kTwo) mma_commit_pair(empty_bar(stage), 3);
                else mma_commit(empty_bar(stage));
              }
              if (++stage == num_stages) {
                stage = 0;
                phase ^= 1u;
              }
              in_tile++;
              if (++in_chunk == kChunkIters || in_tile == total_k_iters) {
                // chunk complete: hand it to the epilogue warps (of both CTAs)
                if (elected) {
                  if (kTwo) mma_commit_pair(tfull_bar(acc), 3);
                  else mma_commit(tfull_bar(acc));
                }
                chunk++;
                in_chunk = 0;
              }
            }
          };
          int mask = 0;
          for (int i = 0; i < gr.nmma; i++) mask |= (gr.mma[i].f16 != 0 ? 1 : 0) << i;
          using std::integral_constant;
          const int shape = gr.nmma * 16 + mask;
          using S2 = integral_constant<int, 2>;
          using S4 = integral_constant<int, 4>;
          if (bk == 64) {   // every term on 16-bit planes
            if (shape == 3 * 16 + 7) run_group(integral_constant<int, 3>{}, integral_constant<int, 7>{}, S4{});
            else if (shape == 2 * 16 + 3) run_group(integral_constant<int, 2>{}, integral_constant<int, 3>{}, S4{});
            else if (shape == 1 * 16 + 1) run_group(integral_constant<int, 1>{}, integral_constant<int, 1>{}, S4{});
            else run_group(integral_constant<int, -1>{}, integral_constant<int, 0>{}, S4{});
          }
          else if (shape == 3 * 16 + 7) run_group(integral_constant<int, 3>{}, integral_constant<int, 7>{}, S2{});        // three half-precision terms
          else if (shape == 2 * 16 + 3) run_group(integral_constant<int, 2>{}, integral_constant<int, 3>{}, S2{});   // two
          else if (shape == 3 * 16 + 3) run_group(integral_constant<int, 3>{}, integral_constant<int, 3>{}, S2{});   // lo16.b16, b16.lo16, x.x
          else if (shape == 2 * 16 + 1) run_group(integral_constant<int, 2>{}, integral_constant<int, 1>{}, S2{});   // lo16.b16, x.x
          else if (shape == 3 * 16) run_group(integral_constant<int, 3>{}, integral_constant<int, 0>{}, S2{});       // three TF32 terms
          else if (shape == 2 * 16) run_group(integral_constant<int, 2>{}, integral_constant<int, 0>{}, S2{});
          else if (shape == 1 * 16) run_group(integral_constant<int, 1>{}, integral_constant<int, 0>{}, S2{});
          else run_group(integral_constant<int, -1>{}, integral_constant<int, 0>{}, S2{});
        }
      }
#ifdef B200_GEMM_TIMING
      if (p.dbg && elected) {
        p.dbg[blockIdx.x * 8 + 0] = (unsigned long long)(clock64() - t_start);
        p.dbg[blockIdx.x * 8 + 1] = (unsigned long long)t_full;
        p.dbg[blockIdx.x * 8 + 2] = (unsigned long long)t_tempty;
      }
#else
      (void)t_full; (void)t_tempty; (void)t_start;
#endif
    }
  }   // warps 2, 3: nothing to do
  } else if (warp < kFirstEpiWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
    // ------------------------------------------------------------ converters
    // For every k-block: wait for this CTA's fp32 tiles, write the derived tiles next to them in
    // the layout TMA would have produced for a tensor of that element type, make them visible to
    // the tensor core (async proxy) and arrive on the leader's `ready` barrier.
    //   K-major fp32 tile : rows of 128 B (32 floats of K), 16-byte chunk c of row r at c ^ (r & 7)
    //   K-major bf16 tile : rows of 64 B, chunk c of row r at c ^ ((r >> 1) & 3)
    //   MN-major fp32 tile: boxes of bk rows (one k each) of 128 B = 32 floats of M/N, 32-byte
    //                       group g of row k at g ^ (k & 3)
    //   MN-major bf16 tile: boxes of bk rows of 128 B = 64 bfloat16 of M/N (two fp32 boxes side
    //                       by side), 16-byte chunk c of row k at c ^ (k & 7)
    // A tile has as many units as rows of M/N (a row of a K-major tile, one k-row of one box of an
    // MN-major tile), each of four 8-element pieces; thread ct takes units ct, ct + 64, ...
    const int ct = threadIdx.x - 32 * kFirstConvWarp;
    constexpr int kConvThreads = 32 * kConvWarps;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = !p.direct;   // nothing to derive anywhere: the copies report to the issuer themselves
    long long t_cfull = 0, t_conv = 0;
    for (int w = first_tile; w < num_tiles && ok; w += tile_step) {
      const int sp = w % splits;
      for (int q = 0; q < p.ngroups && ok; q++) {
        const TcGroup& gr = p.group[q];
        int kb_first, kb_last;
        split_range(q, sp, kb_first, kb_last);
        const int k_iters = kb_last - kb_first, nconv = gr.nconv;
        const TcConv c0 = gr.conv[0], c1 = gr.conv[1];
        for (int kb = 0; kb < k_iters; kb++) {
          if (!TIMED_WAIT(t_cfull, mbar_wait(full_bar(stage), phase, &abort_flag, spin_limit))) {
            ok = false;
            if (!abort_flag) atomicCAS(p.status, 0, 5);
            abort_flag = 1;
            break;
          }
          const uint32_t sbase = smem_base + stage * stage_bytes;
#ifdef B200_GEMM_TIMING
          const long long t_c0 = clock64();
#endif
#pragma unroll
          for (int ci = 0; ci < 2; ci++) {
            if (ci < nconv) {
              const TcConv cv = ci == 0 ? c0 : c1;
              const int units = cv.is_a ? BM : BN_LOCAL;
              const bool w32 = cv.lo32_off != kNoTile, w16 = cv.lo16_off != kNoTile, wb = cv.b16_off != kNoTile;
              const uint32_t src = sbase + cv.src_off, d32 = sbase + cv.lo32_off, d16 = sbase + cv.lo16_off,
                             db = sbase + cv.b16_off;
              const uint32_t d32_minus_src = d32 - src;
              for (int u = ct; u < units; u += kConvThreads) {
                if (!cv.mn) {
                  const uint32_t r = (uint32_t)u, sw = r & 7u, sw16 = (r >> 1) & 3u;
                  const uint32_t row32 = src + r * 128u, row16 = r * 64u;
#pragma unroll
                  for (uint32_t h = 0; h < 2; h++) {   // half a row: 16 elements of K
                    const uint32_t sa[4] = {row32 + (((4 * h) ^ sw) << 4), row32 + (((4 * h + 1) ^ sw) << 4),
                                            row32 + (((4 * h + 2) ^ sw) << 4), row32 + (((4 * h + 3) ^ sw) << 4)};
                    const uint32_t o0 = row16 + (((2 * h) ^ sw16) << 4), o1 = row16 + (((2 * h + 1) ^ sw16) << 4);
                    convert16(sa, w32, d32_minus_src, w16, d16 + o0, d16 + o1, wb, db + o0, db + o1);
                  }
                } else {
                  const uint32_t box = (uint32_t)u >> 5, k = (uint32_t)u & 31u;
                  const uint32_t row32 = src + box * (uint32_t)(bk * 128) + k * 128u;
                  const uint32_t row16 = (box >> 1) * (uint32_t)(bk * 128) + k * 128u;
#pragma unroll
                  for (uint32_t h = 0; h < 2; h++) {   // half a k-row of the box: 16 elements of M/N
                    const uint32_t g0 = row32 + (((2 * h) ^ (k & 3u)) << 5), g1 = row32 + (((2 * h + 1) ^ (k & 3u)) << 5);
                    const uint32_t sa[4] = {g0, g0 + 16u, g1, g1 + 16u};
                    const uint32_t c0 = (box & 1u) * 4u + 2 * h;
                    const uint32_t o0 = row16 + ((c0 ^ (k & 7u)) << 4), o1 = row16 + (((c0 + 1) ^ (k & 7u)) << 4);
                    convert16(sa, w32, d32_minus_src, w16, d16 + o0, d16 + o1, wb, db + o0, db + o1);
                  }
                }
              }
            }
          }
          fence_async_smem();   // the derived tiles are read through the async proxy
          __syncwarp();
          if (lane == 0) {
            if (kTwo) mbar_arrive_leader(ready_bar(stage));
            else mbar_arrive(ready_bar(stage));
          }
#ifdef B200_GEMM_TIMING
          t_conv += clock64() - t_c0;
#endif
          if (++stage == num_stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
#ifdef B200_GEMM_TIMING
    if (p.dbg && ct == 0) {
      p.dbg[blockIdx.x * 8 + 6] = (unsigned long long)t_cfull;
      p.dbg[blockIdx.x * 8 + 7] = (unsigned long long)t_conv;
    }
#else
    (void)t_cfull; (void)t_conv;
#endif
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpiRegs));
    // ------------------------------------------------------------ epilogue warps
    constexpr int COLS = Cfg::kColsPerWarp;
    const int ew = warp - kFirstEpiWarp;
    const int wq = warp & 3;          // TMEM lane quarter this warp may read
    const int col_base = (ew >> 2) * COLS;
    uint32_t chunk = 0;
    // A private copy: read through the parameter block, every field would have to be
    // reloaded after each store (the stores could alias it as far as the compiler knows).
    GemmEpilogue e = p.epi;
    // scaled half-precision operands: the accumulator carries 2^(exponent sum); a power of two, exact
    e.alpha *= exp2f(-((e.scale_exp ? *e.scale_exp : 0.0f) + (float)e.scale_exp_const));
    const float aux_scale = exp2f((float)e.aux_exp);
    const uint16_t aux_one = e.aux_f16 ? __half_as_ushort(__float2half_rn(aux_scale)) : (uint16_t)0x3f80;
    const int pM = p.M, pN = p.N;
    bool ok = true;
    long long t_tfull = 0, t_epi = 0;
    for (int w = first_tile; w < num_tiles && ok; w += tile_step) {
      const int t = w / splits, sp = w - t * splits;
      const int nchunks = (item_k_iters(sp) + kChunkIters - 1) / kChunkIters;
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      float accum[COLS];
#pragma unroll
      for (int j = 0; j < COLS; j++) accum[j] = 0.0f;
      for (int c = 0; c < nchunks; c++, chunk++) {
        const int acc = chunk & 1;
        if (!TIMED_WAIT(t_tfull, mbar_wait(tfull_bar(acc), (chunk >> 1) & 1u, &abort_flag, spin_limit))) {
          if (!abort_flag) atomicCAS(p.status, 0, 4);
          abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(acc * BN + col_base);
#pragma unroll
        for (int j = 0; j < COLS / 32; j++) {
          float v[32];
          tmem_ld32(taddr + 32 * j, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i++) accum[32 * j + i] += v[i];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (kTwo) mbar_arrive_leader(tempty_bar(acc));   // the leader's issuer waits for both CTAs
          else mbar_arrive(tempty_bar(acc));
        }
      }
      if (!ok) break;
#ifdef B200_GEMM_TIMING
      const long long t_e0 = clock64();
#endif
      const int m = tm * TILE_M + (int)rank * BM + wq * 32 + lane;
      const int nc = tn * BN + col_base;
      if (m < pM && nc < pN) {
        if (epi_is_plain(kEpi)) {
          float* out = e.out + (long)sp * p.split_stride + (long)nc * e.ldo + m;
          if (kEpi == kEpiPlain && p.scatter_cols > 0) {
            const int owner = nc / p.scatter_cols;
            out = p.scatter[owner] + (long)(nc - owner * p.scatter_cols) * e.ldo + m;
          }
          const float alpha = e.alpha, beta = e.beta;
          const long ldo = e.ldo;
          const int ncols = pN - nc < COLS ? pN - nc : COLS;
          // a real loop over batches of 16 columns (the accumulator registers shifted down after each):
          // a product of one tile runs this code once, straight from a cold instruction cache
#pragma unroll 1
          for (int go = 0; go < COLS / 16; go++) {
            float* const o16 = out + (long)(16 * go) * ldo;
            const int left = ncols - 16 * go;
            if (beta == 0.0f) {
#pragma unroll
              for (int j = 0; j < 16; j++)
                if (j < left) o16[j * ldo] = alpha * accum[j];
            } else {
#pragma unroll
              for (int j = 0; j < 16; j++)
                if (j < left) o16[j * ldo] = alpha * accum[j] + beta * o16[j * ldo];
            }
#pragma unroll
            for (int i = 0; i + 16 < COLS; i++) accum[i] = accum[i + 16];
          }
        }
      }
      if (!epi_is_plain(kEpi)) {
        // Activation epilogues leave through shared memory and TMA stores.  Per-thread global
        // stores (three arrays, 128 columns, 32 KB apart) cost 55 us per tile here against 7 us
        // for the arithmetic; a batch of four columns (one Philox block) is staged as
        // [array][column][128 rows], and one thread of each column-half group of four warps
        // sends it on with cp.async.bulk.tensor while the next batch is computed (two buffers).
        const bool spec = kEpi != kEpiGeneric;      // specialised variants: bias set; beta = 0; no col_scale
        const bool row_ok = m < pM;
        const int hf = ew >> 2;                     // column half = store group
        const bool leader = (ew & 3) == 0 && lane == 0;
        const int row = wq * 32 + lane;             // row of the CTA's 128
        const float alpha = e.alpha, beta = spec ? 0.0f : e.beta;
        const float bias = ((spec || e.bias) && row_ok) ? e.bias[m] : 0.0f;
        const bool logistic = spec ? (kEpi != kEpiLin) : (e.activation == 1);
        const bool draw = spec ? (kEpi == kEpiSigSample) : (e.sample != nullptr || e.sample_aux != nullptr);
        const bool has_out = e.out != nullptr;
        const bool has_aux = e.out_aux != nullptr;
        const bool has_smp = e.sample != nullptr;
        const bool has_smp_aux = draw && e.sample_aux != nullptr;
        const PhiloxKey key = e.key;
        const uint32_t cblk0 = (uint32_t)((nc + e.col0) >> 2);
        const long off = (long)nc * e.ldo + m, ldo = e.ldo;
        const int m_tile = tm * TILE_M + (int)rank * BM;     // first row of this CTA's part of the tile
        // one staged batch: [out f32][aux plane 0 bf16][aux plane 1 bf16][sample f32][sample bf16],
        // each kOutCols columns of BM rows
        constexpr uint32_t kF32 = kOutCols * BM * 4, kB16 = kOutCols * BM * 2;
        constexpr uint32_t kOffLo = kF32, kOffB = kF32 + kB16, kOffSmp = kF32 + 2 * kB16, kOffSmpB = 2 * kF32 + 2 * kB16;
        constexpr uint32_t kBufBytes = 2 * kF32 + 3 * kB16;
        static_assert(4 * kBufBytes <= kOutStageBytes, "epilogue staging");
        const uint32_t group_base = out_stage_base + (uint32_t)hf * 2u * kBufBytes;
        // The loop over the batches is a real loop (four batches unrolled per trip, the accumulator
        // registers shifted down by 16 after each): unrolled over all 128 columns the epilogue was
        // 200-400 KB of straight-line code that every tile fetched anew (the tile phase took 43 us
        // with the arithmetic and the stores removed); as a loop it stays in the instruction cache.
#pragma unroll 1
        for (int go = 0; go < COLS / 16; go++) {
#pragma unroll
        for (int gi = 0; gi < 4; gi++) {
          const int g4 = 4 * go + gi;
          const int c0 = nc + 4 * g4;               // first global column of the batch
          float x[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            float t = alpha * accum[4 * gi + j];
            if (!spec) {
              if (beta != 0.0f && row_ok && c0 + j < pN) t += beta * e.out[off + (long)(4 * g4 + j) * ldo];
              if (e.bias) t += e.col_scale ? (c0 + j < pN ? bias * e.col_scale[c0 + j] : 0.0f) : bias;
            } else {
              t += bias;
            }
            x[j] = logistic ? sigmoid_accurate(t) : t;
          }
          uint4 w = make_uint4(0, 0, 0, 0);
          if (draw) w = philox4x32_10((uint32_t)m, cblk0 + g4, key);
          if (p.store16) {
            uint16_t* const ob = reinterpret_cast<uint16_t*>(e.out_aux);
            uint16_t* const sb = reinterpret_cast<uint16_t*>(e.sample_aux);
            const long lda2 = 2L * e.ld_aux;
#pragma unroll
            for (int j = 0; j < 4; j++) {
              if (!row_ok || c0 + j >= pN) continue;
              const long word = (long)(c0 + j) * lda2 + m;
              if (has_aux) {
                uint16_t lo16, b16;
                if (e.aux_f16) {
                  split_f16(x[j], aux_scale, lo16, b16);
                } else {
                  lo16 = (uint16_t)pack_bf16(tf32_rest(x[j]), 0.0f);
                  b16 = (uint16_t)pack_bf16(x[j], 0.0f);
                }
                ob[word] = lo16;
                ob[word + e.ld_aux] = b16;
              }
              if (has_smp_aux) {
                const bool on = word_to_uniform(pick_word(w, j)) < x[j];
                sb[word + e.ld_aux] = (uint16_t)(on ? aux_one : 0);
              }
            }
            continue;
          }
          // buffer (g4 & 1) is free once the stores of batch g4 - 2 have read it (the leader waited)
          named_bar_sync(1 + hf, 128);
          const uint32_t buf = group_base + (uint32_t)(gi & 1) * kBufBytes;
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const uint32_t a32 = buf + (uint32_t)(j * BM + row) * 4u, a16 = buf + (uint32_t)(j * BM + row) * 2u;
            if (has_out) asm volatile("st.shared.f32 [%0], %1;" ::"r"(a32), "f"(x[j]) : "memory");
            if (has_aux) {
              uint16_t lo16, b16;
              if (e.aux_f16) {
                split_f16(x[j], aux_scale, lo16, b16);
              } else {
                lo16 = (uint16_t)pack_bf16(tf32_rest(x[j]), 0.0f);
                b16 = (uint16_t)pack_bf16(x[j], 0.0f);
              }
              asm volatile("st.shared.u16 [%0], %1;" ::"r"(a16 + kOffLo), "h"(lo16) : "memory");
              asm volatile("st.shared.u16 [%0], %1;" ::"r"(a16 + kOffB), "h"(b16) : "memory");
            }
            if (draw) {
              const bool on = word_to_uniform(pick_word(w, j)) < x[j];
              if (has_smp) asm volatile("st.shared.f32 [%0], %1;" ::"r"(a32 + kOffSmp), "f"(on ? 1.0f : 0.0f) : "memory");
              if (has_smp_aux)
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(a16 + kOffSmpB), "h"((uint16_t)(on ? aux_one : 0)) : "memory");
            }
          }
          fence_async_smem();                       // generic-proxy writes visible to the TMA engine
          named_bar_sync(1 + hf, 128);
          if (leader && c0 < pN && m_tile < pM) {
            if (has_out) tma_store_2d(&p.maps[p.out_map[0]], m_tile, c0, buf);
            if (has_aux) {
              tma_store_2d(&p.maps[p.out_map[1]], m_tile, c0, buf + kOffLo);
              tma_store_2d(&p.maps[p.out_map[2]], m_tile, c0, buf + kOffB);
            }
            if (has_smp) tma_store_2d(&p.maps[p.out_map[3]], m_tile, c0, buf + kOffSmp);
            if (has_smp_aux) tma_store_2d(&p.maps[p.out_map[4]], m_tile, c0, buf + kOffSmpB);
          }
          if (leader) {
            tma_store_commit();
            tma_store_wait_read<1>();               // the other buffer's stores have read it
          }
        }
#pragma unroll
        for (int i = 0; i + 16 < COLS; i++) accum[i] = accum[i + 16];
        }
        if (leader && !p.store16) tma_store_wait_all();   // results are in memory before the kernel can end
      }
#ifdef B200_GEMM_TIMING
      t_epi += clock64() - t_e0;
#endif
    }
    // tiles delivered to other GPUs: this thread's stores are performed system-wide before it leaves (once
    // per launch; a fence per tile held the epilogue, and with it the issuer, for 0.24 ms per product)
    if (kEpi == kEpiPlain && p.scatter_cols > 0) __threadfence_system();
#ifdef B200_GEMM_TIMING
    if (p.dbg && threadIdx.x == 32 * kFirstEpiWarp) {
      p.dbg[blockIdx.x * 8 + 4] = (unsigned long long)t_tfull;
      p.dbg[blockIdx.x * 8 + 5] = (unsigned long long)t_epi;
    }
#else
    (void)t_tfull; (void)t_epi;
#endif
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (kTwo) cluster_sync();   // neither CTA leaves (or frees tensor memory) while its peer may still use it
  if (warp == 1) {
    tc_fence_after();
    if (kTwo) tmem_dealloc2(tmem_base, Cfg::kTmemCols);
    else tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}


// ---- host side ------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
    else
      cudaGetLastError();
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t d0, d1, ld;
  uint32_t b0, b1;
  int swz;  // 0: 128B swizzle, 1: 128B swizzle with 32B atoms, 2: 64B swizzle, 3: none (output tiles)
  int bf16;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && ld == o.ld && b0 == o.b0 && b1 == o.b1 && swz == o.swz &&
           bf16 == o.bf16;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ k.d0;
    h = h * 1000003u ^ k.d1;
    h = h * 1000003u ^ k.ld;
    h = h * 1000003u ^ ((uint64_t)k.b0 << 32 | k.b1 << 3 | (uint32_t)k.swz << 1 | (uint32_t)k.bf16);
    return h;
  }
};

// 2-D map over fp32 or bfloat16 elements: inner (contiguous) extent d0, outer extent d1 with a
// stride of ld elements, box b0 x b1, zero fill outside the tensor.  swz 0: 128-byte swizzle of
// 16-byte chunks (K-major fp32 tiles, 32 floats of K per row; MN-major bfloat16 tiles, 64 per
// row); 2: 64-byte swizzle (K-major bfloat16, 32 per row); 1: 128-byte swizzle of 32-byte
// chunks, the only shared-memory layout tcgen05 accepts for MN-major 32-bit operands;
// 3: none (output tiles).  Encoded maps are cached.
bool make_map(CUtensorMap* out, const void* ptr, uint64_t d0, uint64_t d1, uint64_t ld, uint32_t b0, uint32_t b1,
              int swz, int bf16) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  const MapKey key{ptr, d0, d1, ld, b0, b1, swz, bf16};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {d0, d1};
  const cuuint64_t strides[1] = {ld * (bf16 ? 2 : 4)};
  const cuuint32_t box[2] = {b0, b1};
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  const CUresult r = fn(&m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)ptr,
                        dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swz == 1 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                 : (swz == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                                             : (swz == 3 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B)),
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

// TMA needs a 16-byte aligned base and column stride.
inline bool tma_ok(const GemmOperand& o) {
  return (o.ld % 4 == 0) && (((uintptr_t)(o.ptr + o.row0) & 15) == 0) &&
         (!o.aux || (o.lda % 8 == 0 && ((uintptr_t)o.aux & 15) == 0 && o.row0 % 8 == 0));
}

// Shared-memory matrix descriptor, upper 32 bits: stride byte offset (bits 32-45, in
// 16-byte units), descriptor version 1 for sm_100 (bits 46-47), layout type in bits 61-63.
//  K-major fp32, rows of 128 B (32 floats of K): 8-row groups 1024 B apart, 128B swizzle (type 2).
//  K-major bf16, rows of 64 B (32 bfloat16 of K): 8-row groups 512 B apart, 64B swizzle (type 4).
//  MN-major fp32: rows (one k each) of 128 B = 32 floats along M/N, 4-row groups 512 B apart,
//                 128B swizzle with 32-byte atoms (type 1).
//  MN-major bf16: rows (one k each) of 128 B = 64 bfloat16 along M/N, 8-row groups 1024 B apart,
//                 128B swizzle (type 2).
// The lower word carries the start address and the leading byte offset (for MN-major tiles the
// distance between two 128-byte wide column blocks = bk rows of 128 B).
constexpr uint32_t kDescHiK32 = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t kDescHiK16 = (512u >> 4) | (1u << 14) | (4u << 29);
constexpr uint32_t kDescHiMN = (512u >> 4) | (1u << 14) | (1u << 29);
constexpr uint32_t kDescHiMN16 = (1024u >> 4) | (1u << 14) | (2u << 29);

// The tcgen05 view of a staged tile of fp32 (as loaded, or the lo32 part) or of bfloat16 (a derived part).
TcTile tile_view(bool mn, bool bf16, int bk, uint32_t smem_off) {
  TcTile t;
  t.smem_off = smem_off;
  if (mn) {
    t.desc_hi = bf16 ? kDescHiMN16 : kDescHiMN;
    t.desc_lo = ((uint32_t)(bk * 128) >> 4) << 16;   // distance between column blocks = bk rows x 128 B
    t.adv = (bf16 ? 2048u : 1024u) >> 4;             // one MMA reads 16 (bfloat16) or 8 (fp32) rows of 128 B
  } else {
    t.desc_hi = (bf16 && bk == 32) ? kDescHiK16 : kDescHiK32;   // 64 16-bit elements of K are a 128-byte row too
    t.desc_lo = 1u << 16;                            // leading byte offset is unused for swizzled K-major tiles
    t.adv = 32u >> 4;                                // one MMA reads 32 bytes of K inside the swizzled row
  }
  return t;
}

inline bool same_operand(const GemmOperand& a, const GemmOperand& b) {
  return a.ptr == b.ptr && a.ld == b.ld && a.trans == b.trans && a.aux == b.aux && a.lda == b.lda && a.row0 == b.row0;
}

static_assert(sizeof(TcParams) <= 4096, "kernel parameter block");

// Host-side failure injection for the bounded waits: the next tensor-core product is told to
// expect this many more bytes per stage than its copies deliver, so the stage's barrier can
// never complete, the waiting role runs into the wait limit, records a status word and the
// kernel drains and returns.  Nothing traps, faults or spins without bound.
int g_inject_stage_bytes = 0;

template <int BN, int kEpi, bool kTwo>
int launch_tc(TcParams& p) {
  using Cfg = TcConfig<BN>;
  // The shared-memory attribute of a kernel and the number of resident CTA pairs belong to a
  // device, not to the process: kept per device ordinal for a host that drives several GPUs.
  constexpr int kMaxDev = 64;
  static bool attr_set[kMaxDev] = {false};
  static int pairs_of[kMaxDev] = {0};
  static std::mutex mu;
  auto kernel = k_gemm_tc<BN, kEpi, kTwo>;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return set_error("cudaGetDevice failed");
  int max_pairs = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!attr_set[dev]) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
        return set_error("cudaFuncSetAttribute(max dynamic shared memory) failed");
      if (kTwo) {
        // how many CTA pairs the device can keep resident at once (a pair needs two SMs of one TPC)
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(2 * (sm_count() / 2));
        q.blockDim = dim3(kThreadsTc);
        q.dynamicSmemBytes = Cfg::kSmemBytes;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        q.attrs = at;
        q.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &q) != cudaSuccess || n < 1) {
          cudaGetLastError();
          return set_error("cudaOccupancyMaxActiveClusters failed for the paired-CTA product");
        }
        pairs_of[dev] = n;
      }
      attr_set[dev] = true;
    }
    max_pairs = pairs_of[dev];
  }
  constexpr int TILE_M = kTwo ? 2 * BM : BM;
  p.tiles_m = (p.M + TILE_M - 1) / TILE_M;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n * p.splits;   // work items
  if (!kTwo) {
    const int grid = tiles < sm_count() ? tiles : sm_count();
    if (launch_dependent(kernel, dim3(grid), dim3(kThreadsTc), Cfg::kSmemBytes, stream(), p) != cudaSuccess)
      return set_error(cudaGetErrorString(cudaGetLastError()));
    return check_launch();
  }
  int pairs = tiles < max_pairs ? tiles : max_pairs;
  if (pairs > sm_count() / 2) pairs = sm_count() / 2;   // an SM limit in force (b200_set_sm_limit) leaves the rest free
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreadsTc);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream();
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = dependent_launch_enabled() ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return set_error(cudaGetErrorString(cudaGetLastError()));
  return check_launch();
}

// Split-K: the partial products of the splits are summed in split order (the same bits every run)
// and the epilogue runs once per element, on CUDA cores: one thread per row and block of four
// columns, which share one Philox block exactly as the tensor-core epilogue assigns them.
__global__ void __launch_bounds__(256) k_splitk_finish(const float* __restrict__ part, int splits, long stride, int M,
                                                       int N, const GemmEpilogue e) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int nblk = (N + 3) >> 2;
  const long items = (long)M * nblk;
  const bool draw = e.sample != nullptr || e.sample_aux != nullptr;
  for (long it = (long)blockIdx.x * blockDim.x + threadIdx.x; it < items; it += (long)gridDim.x * blockDim.x) {
    const int b = (int)(it / M), m = (int)(it - (long)b * M);
    uint4 w = make_uint4(0, 0, 0, 0);
    if (draw) w = philox4x32_10((uint32_t)m, (uint32_t)(b + (e.col0 >> 2)), e.key);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = 4 * b + j;
      if (n >= N) break;
      const float* src = part + (long)n * M + m;
      float acc = 0.0f;
      for (int sp = 0; sp < splits; sp++) acc += src[(long)sp * stride];
      epilogue_store(e, acc, m, n, word_to_uniform(pick_word(w, j)));
    }
  }
}

int g_split_mode = 0;   // 0: split when the tiles would leave most SMs idle; 1: never; n > 1: always n splits (tests)

}  // namespace

extern "C" int b200_set_split_k(int mode) {
  g_split_mode = mode < 0 ? 0 : mode;
  return 0;
}

namespace {
}  // namespace

bool gemm_tc_supported(const GemmProblem& g) {
  if (g.M <= 0 || g.N <= 0 || g.npass <= 0 || g.npass > kMaxPass) return false;
  for (int q = 0; q < g.npass; q++) {
    const GemmPass& ps = g.pass[q];
    if (!tma_ok(ps.a) || !tma_ok(ps.b) || ps.k <= 0) return false;
    if (part_is_16bit(ps.a.part) != part_is_16bit(ps.b.part) || part_is_f16(ps.a.part) != part_is_f16(ps.b.part)) return false;
    if (part_is_f16(ps.a.part) && (!ps.a.aux || !ps.b.aux)) return false;
  }
  const GemmEpilogue& e = g.epi;
  if ((e.sample || e.sample_aux) && (e.col0 & 3)) return false;
  // activation epilogues store whole column segments with TMA: 16-byte aligned columns (the
  // planes of an aux matrix are, its columns being a multiple of 8 floats)
  const bool plain = !e.bias && e.activation == 0 && !e.sample && !e.out_aux && !e.sample_aux && e.out;
  if (!plain) {
    if (e.ldo % 4 != 0 || e.ld_aux % 8 != 0) return false;
    if (((uintptr_t)e.out | (uintptr_t)e.sample | (uintptr_t)e.out_aux | (uintptr_t)e.sample_aux) & 15) return false;
  }
  return encode_fn() != nullptr;
}

#ifdef B200_HOST_TIMING
// Debug build only: where the host time of a product goes (printed when the process exits).
struct HostTimes {
  double setup = 0, launch = 0;
  long calls = 0;
  static double now() {
    timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return t.tv_sec * 1e6 + t.tv_nsec * 1e-3;
  }
  ~HostTimes() {
    if (calls) fprintf(stderr, "gemm_tc host time per call: set-up %.2f us, launch %.2f us (%ld calls)\n", setup / calls, launch / calls, calls);
  }
};
static HostTimes g_host_times;
#endif

// Scatter registration (dp_peer.cu): products whose result is `match` deliver column panels to `out`.
static const float* g_scatter_match = nullptr;
static float* g_scatter_out[kMaxScatter] = {nullptr};
static int g_scatter_n = 0, g_scatter_cols = 0;

int set_product_scatter(const float* match, float* const* out, int n, int cols) {
  if (n < 0 || n > kMaxScatter || (n > 0 && (!match || cols <= 0))) return ERROR_UNSUPPORTED;
  g_scatter_match = n > 0 ? match : nullptr;
  g_scatter_n = n;
  g_scatter_cols = n > 0 ? cols : 0;
  for (int i = 0; i < n; i++) g_scatter_out[i] = out[i];
  return 0;
}

bool product_is_scattered(const float* out) { return g_scatter_n > 0 && out != nullptr && out == g_scatter_match; }

int gemm_tc(const GemmProblem& g) {
#ifdef B200_HOST_TIMING
  const double t_begin = HostTimes::now();
#endif
  const bool scatter = g_scatter_n > 0 && g.epi.out != nullptr && g.epi.out == g_scatter_match;
  if (!gemm_tc_supported(g))
    return scatter ? set_error("a product whose result is scattered to peers must run on the tensor cores") : ERROR_UNSUPPORTED;
  const int BN = g.N > 128 ? 256 : (g.N > 64 ? 128 : 64);
  static int pair_mode = -1;   // B200_GEMM_2CTA=0 keeps one CTA per tile
  static int chunk_k = 0;
  if (pair_mode < 0) {
    const char* e = getenv("B200_GEMM_2CTA");
    pair_mode = e ? atoi(e) : 1;
    const char* c = getenv("B200_CHUNK_K");
    chunk_k = c ? atoi(c) : 0;
  }
  // pairs of CTAs (cta_group::2) on 256-row tiles when the product has at least two row tiles
  const bool two = pair_mode != 0 && BN == 256 && g.M > BM;
  const int BN_LOCAL = two ? BN / 2 : BN;      // rows of B staged per CTA
  // Elements of K per k-block: 32 (one 128-byte swizzle row of floats; 16 doubles the stage count but
  // measured slower: 64-byte rows, twice the MMA and TMA issues).  When every term reads 16-bit planes
  // from aux matrices (no fp32 tile, nothing derived) a k-block is 64 elements: again 128-byte rows,
  // four MMAs per term and k-block, half the barrier round trips and copies per flop.
  static int wide16 = -1;
  if (wide16 < 0) {
    const char* wv = getenv("B200_GEMM_BK64");
    wide16 = wv ? atoi(wv) : 1;
  }
  bool all16 = wide16 != 0;
  for (int q = 0; q < g.npass && all16; q++) {
    const GemmPass& ps = g.pass[q];
    all16 = part_is_16bit(ps.a.part) && part_is_16bit(ps.b.part) && ps.a.aux && ps.b.aux;
  }
  const int bk = all16 ? 64 : 32;
  TcParams p;
  p.M = g.M;
  p.N = g.N;
  p.bk = bk;
  p.epi = g.epi;
  p.status = status_word();
  if (!p.status) return set_error("the library is not initialised (no device status word)");
  p.spin_limit = wait_limit();
#ifdef B200_GEMM_TIMING
  p.dbg = (unsigned long long*)workspace(7, 8 * 512 * sizeof(unsigned long long));
#endif

  // ---- group consecutive terms over the same two fp32 matrices (at most kMaxMma of them)
  int ngroups = 0, nmaps = 0;
  bool map_overflow = false;   // more operand tiles than the parameter block has tensor maps for
  uint32_t stage_bytes = 0;
  const GemmPass* first_of[kMaxPass];
  for (int q = 0; q < g.npass; q++) {
    const GemmPass& ps = g.pass[q];
    if (ngroups > 0) {
      const GemmPass& f = *first_of[ngroups - 1];
      if (same_operand(f.a, ps.a) && same_operand(f.b, ps.b) && f.k == ps.k && p.group[ngroups - 1].nmma < kMaxMma) {
        p.group[ngroups - 1].nmma++;
        continue;
      }
    }
    if (ngroups == kMaxGroups) return ERROR_UNSUPPORTED;   // more operand pairs than one launch carries
    first_of[ngroups] = &ps;
    p.group[ngroups].nmma = 1;
    ngroups++;
  }
  int q0 = 0;
  for (int gi = 0; gi < ngroups; gi++) {
    TcGroup& tg = p.group[gi];
    const GemmPass& f = g.pass[q0];
    tg.k_iters = (f.k + bk - 1) / bk;
    // op(A) is M x k: trans -> stored k x M, k contiguous (K-major); else M contiguous.
    // op(B) is k x N: not trans -> stored k x N, k contiguous (K-major); trans -> N contiguous.
    const bool mn[2] = {f.a.trans == 0, f.b.trans != 0};
    const GemmOperand* src[2] = {&f.a, &f.b};
    const int rows[2] = {BM, BN_LOCAL}, extent[2] = {g.M, g.N};
    // which parts the group's terms read
    bool want[2][kNumParts] = {};
    for (int i = 0; i < tg.nmma; i++) {
      want[0][g.pass[q0 + i].a.part] = true;
      want[1][g.pass[q0 + i].b.part] = true;
    }
    uint32_t off = 0;
    int tile_of[2][kNumParts];
    int ntiles = 0;
    tg.nload = tg.nconv = 0;
    auto add_load = [&](int o, const void* ptr, uint64_t ld, bool bf16) {
      if (nmaps >= kMaxMaps - kOutArrays) {
        map_overflow = true;
        return false;
      }
      TcLoad& l = tg.load[tg.nload++];
      l.map = nmaps;
      l.mn = mn[o];
      l.is_a = o == 0;
      l.box_rows = bf16 ? 64 : 32;                     // 128 bytes of M/N per box row
      l.smem_off = off;
      // K-major: one box of bk elements of K x the tile's rows; MN-major: boxes of 128 bytes x bk
      const bool ok = mn[o] ? make_map(&p.maps[nmaps], ptr, (uint64_t)extent[o], (uint64_t)f.k, ld,
                                       (uint32_t)l.box_rows, (uint32_t)bk, bf16 ? 0 : 1, bf16)
                            : make_map(&p.maps[nmaps], ptr, (uint64_t)f.k, (uint64_t)extent[o], ld, (uint32_t)bk,
                                       (uint32_t)rows[o], (bf16 && bk == 32) ? 2 : 0, bf16);
      nmaps++;
      return ok;
    };
    uint32_t x_off[2] = {0, 0};
    for (int o = 0; o < 2; o++) {   // the fp32 tiles first: wanted as they are, or as the source of derived parts
      const bool from_aux = src[o]->aux != nullptr;
      if (!(want[o][kPartX] || want[o][kPartLo32] || (!from_aux && (want[o][kPartLo16] || want[o][kPartB16])))) continue;
      x_off[o] = off;
      if (!add_load(o, src[o]->ptr + src[o]->row0, (uint64_t)src[o]->ld, false))
        return map_overflow ? ERROR_UNSUPPORTED : set_error("cuTensorMapEncodeTiled failed for an operand");
      tile_of[o][kPartX] = ntiles;
      tg.tile[ntiles++] = tile_view(mn[o], false, bk, off);
      off += (uint32_t)rows[o] * bk * 4;
    }
    for (int o = 0; o < 2; o++) {   // bfloat16 parts read from the operand's aux matrix
      if (!src[o]->aux) continue;
      for (int part = kPartLo16; part < kNumParts; part++) {
        if (!want[o][part]) continue;
        const uint16_t* plane =
            reinterpret_cast<const uint16_t*>(src[o]->aux) + (part_plane(part) ? src[o]->lda : 0) + src[o]->row0;
        if (!add_load(o, plane, (uint64_t)(2 * src[o]->lda), true))
          return map_overflow ? ERROR_UNSUPPORTED : set_error("cuTensorMapEncodeTiled failed for an aux plane");
        tile_of[o][part] = ntiles;
        tg.tile[ntiles++] = tile_view(mn[o], true, bk, off);
        off += (uint32_t)rows[o] * bk * 2;
        want[o][part] = false;   // not the converters' job
      }
    }
    tg.stage_tx = off;
    for (int o = 0; o < 2; o++) {   // then the parts the converters derive
      if (!want[o][kPartLo32] && !want[o][kPartLo16] && !want[o][kPartB16]) continue;
      TcConv& cv = tg.conv[tg.nconv++];
      cv.src_off = x_off[o];
      cv.mn = mn[o];
      cv.is_a = o == 0;
      cv.lo32_off = cv.lo16_off = cv.b16_off = kNoTile;
      for (int part = kPartLo32; part <= kPartB16; part++) {
        if (!want[o][part]) continue;
        const bool bf16 = part != kPartLo32;
        (part == kPartLo32 ? cv.lo32_off : (part == kPartLo16 ? cv.lo16_off : cv.b16_off)) = off;
        tile_of[o][part] = ntiles;
        tg.tile[ntiles++] = tile_view(mn[o], bf16, bk, off);
        off += (uint32_t)rows[o] * bk * (bf16 ? 2 : 4);
      }
    }
    if (off > stage_bytes) stage_bytes = off;
    for (int i = 0; i < tg.nmma; i++) {
      const GemmPass& ps = g.pass[q0 + i];
      TcMma& m = tg.mma[i];
      m.a = tile_of[0][ps.a.part];
      m.b = tile_of[1][ps.b.part];
      m.f16 = part_is_16bit(ps.a.part);
      // instruction descriptor: D fp32 (bit 4), A and B format at bits 7 and 10 (TF32 = 2 for
      // kind::tf32; BF16 = 1, F16 = 0 for kind::f16), negate A (bit 13), A / B MN-major (bits
      // 15 / 16), N >> 3 at bit 17, M >> 4 at bit 24
      const uint32_t fmt = part_is_f16(ps.a.part) ? 0u : (m.f16 ? 1u : 2u);
      m.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((ps.negate ? 1u : 0u) << 13) | ((mn[0] ? 1u : 0u) << 15) |
                ((mn[1] ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((two ? 2 * BM : BM) >> 4) << 24);
    }
    q0 += tg.nmma;
  }
  if (g_inject_stage_bytes) {
    for (int gi = 0; gi < ngroups; gi++) p.group[gi].stage_tx += (uint32_t)g_inject_stage_bytes;
    g_inject_stage_bytes = 0;
  }
  p.ngroups = ngroups;
  p.direct = 1;
  for (int gi = 0; gi < ngroups; gi++)
    if (p.group[gi].nconv > 0) p.direct = 0;
  p.stage_bytes = stage_bytes;
  p.num_stages = (int)(kStageBudget / p.stage_bytes);
  if (p.num_stages > kMaxStages) p.num_stages = kMaxStages;
  if (p.num_stages < 1) return ERROR_UNSUPPORTED;
  // Products folded in tensor memory before they join the fp32 registers.  The error of a chunk
  // grows linearly with its length (the accumulator truncates at every MMA).  128 keeps linear
  // outputs (statistics, `dot`) within 2e-6 of the largest entry at K = 4096..8192.  Behind a
  // logistic epilogue (slope <= 1/4, small pre-activations) 2048 leaves the probabilities within
  // 3e-6 absolute at K = 8192 (measured on zero-mean, same-sign and trained-like weights: 0.7e-6
  // at 512, 1.3e-6 at 1024, 2.9e-6 at 2048, 6e-6 at 4096; the bar is 1e-5).  Long chunks cover
  // the tile epilogue: the issuer runs two chunks ahead of the epilogue warps, which are busy for
  // 40-50 us per tile while the products of a tile take about 100 us.
  const int ck = chunk_k >= 16 ? chunk_k : (g.epi.activation == 1 ? 2048 : 128);
  p.chunk_iters = ck / bk < 1 ? 1 : ck / bk;

  // Split-K: a product whose tiles would occupy less than half of the SMs and whose inner dimension
  // is long is cut along K into work items (tile, split); every item stores its raw partial and a
  // finishing kernel sums them and runs the epilogue.  (Configuration 1's down product, 1024 x 256
  // with K = 4096, is 4 paired tiles = 8 SMs otherwise.)
  p.splits = 1;
  p.split_stride = 0;
  {
    const int tile_m = two ? 2 * BM : BM;
    const int tiles = ((g.M + tile_m - 1) / tile_m) * ((g.N + BN - 1) / BN);
    const int ctas = two ? 2 * tiles : tiles;
    int min_ki = p.group[0].k_iters;
    for (int gi = 1; gi < ngroups; gi++) min_ki = p.group[gi].k_iters < min_ki ? p.group[gi].k_iters : min_ki;
    int want = 1;
    static int min_ki_to_split = -1;   // a split costs a second (finishing) launch: only long inner dimensions repay it
    if (min_ki_to_split < 0) {
      const char* mv = getenv("B200_SPLITK_MIN_KI");
      min_ki_to_split = mv ? atoi(mv) : 8;
    }
    if (g_split_mode == 0) {
      if (ctas * 2 <= sm_count() && min_ki >= min_ki_to_split) {
        want = sm_count() / ctas;
        if (want > min_ki / 4) want = min_ki / 4;
        if (want > 32) want = 32;
      }
    } else if (g_split_mode > 1) {
      want = g_split_mode < min_ki ? g_split_mode : min_ki;
    }
    if (scatter) want = 1;   // a partial is not a result: the panels go out whole
    if (want > 1) {
      float* ws = (float*)workspace(2, (size_t)want * g.M * g.N * sizeof(float));
      if (!ws) return CUDA_ERROR;
      p.splits = want;
      p.split_stride = (long)g.M * g.N;
      GemmEpilogue& pe = p.epi;       // the kernel stores raw partials; g.epi runs in the finishing kernel
      pe.alpha = 1.0f;
      pe.beta = 0.0f;
      pe.bias = pe.col_scale = nullptr;
      pe.activation = 0;
      pe.out = ws;
      pe.out_aux = pe.sample = pe.sample_aux = nullptr;
      pe.scale_exp = nullptr;
      pe.scale_exp_const = 0;
      pe.ldo = g.M;
    }
  }
  const GemmEpilogue& e = p.epi;
  int epi = kEpiGeneric;
  if (!e.bias && e.activation == 0 && !e.sample && !e.out_aux && !e.sample_aux && e.out) {
    epi = p.splits > 1 ? kEpiPartial : kEpiPlain;
  } else if (e.bias && !e.col_scale && e.beta == 0.0f && (e.out || e.sample || e.out_aux || e.sample_aux)) {
    if (e.activation == 1 && (e.sample || e.sample_aux)) epi = kEpiSigSample;
    else if (e.activation == 1 && !e.sample && !e.sample_aux) epi = kEpiSig;
    else if (e.activation == 0 && !e.sample && !e.sample_aux) epi = kEpiLin;
  }
  p.scatter_cols = 0;
  if (scatter) {
    // whole tiles per panel, the plain epilogue, no split (a partial is not a result), nothing added to old contents
    if (epi != kEpiPlain || p.splits != 1 || e.beta != 0.0f || g.N != g_scatter_n * g_scatter_cols || g_scatter_cols % BN != 0)
      return set_error("a product whose result is scattered to peers must be plain, unsplit, with whole tiles per panel");
    for (int i = 0; i < g_scatter_n; i++) p.scatter[i] = g_scatter_out[i];
    p.scatter_cols = g_scatter_cols;
  }
  static int store16_mode = -1;
  if (store16_mode < 0) {
    const char* sv = getenv("B200_EPI_STORE16");
    store16_mode = sv ? atoi(sv) : 1;
  }
  p.store16 = store16_mode != 0 && !epi_is_plain(epi) && !e.out && !e.sample && (e.out_aux || e.sample_aux);
  for (int i = 0; i < kOutArrays; i++) p.out_map[i] = -1;
  if (!epi_is_plain(epi)) {
    // outputs of the activation epilogues, stored as boxes of 128 rows x 4 columns: M x N floats
    // with columns ldo apart, or one bfloat16 plane of an aux matrix (columns 2 ld_aux bfloat16
    // apart, plane 1 starting ld_aux bfloat16 into the column)
    const uint16_t* oa = reinterpret_cast<const uint16_t*>(e.out_aux);
    const uint16_t* sa = reinterpret_cast<const uint16_t*>(e.sample_aux);
    const void* outs[kOutArrays] = {e.out, oa, oa ? oa + e.ld_aux : nullptr, e.sample, sa ? sa + e.ld_aux : nullptr};
    const int is16[kOutArrays] = {0, 1, 1, 0, 1};
    for (int i = 0; i < kOutArrays; i++) {
      if (!outs[i]) continue;
      if (!make_map(&p.maps[nmaps], outs[i], (uint64_t)g.M, (uint64_t)g.N, (uint64_t)(is16[i] ? 2 * e.ld_aux : e.ldo), BM,
                    kOutCols, 3, is16[i]))
        return set_error("cuTensorMapEncodeTiled failed for an output");
      p.out_map[i] = nmaps++;
    }
  }
#define B200_TC_CASE(BNV, TWO)                                        \
  switch (epi) {                                                      \
    case kEpiPlain: return launch_tc<BNV, kEpiPlain, TWO>(p);         \
    case kEpiPartial: return launch_tc<BNV, kEpiPartial, TWO>(p);     \
    case kEpiSig: return launch_tc<BNV, kEpiSig, TWO>(p);             \
    case kEpiSigSample: return launch_tc<BNV, kEpiSigSample, TWO>(p); \
    case kEpiLin: return launch_tc<BNV, kEpiLin, TWO>(p);             \
    default: return launch_tc<BNV, kEpiGeneric, TWO>(p);              \
  }
  auto launch = [&]() -> int {
    if (BN == 256 && two) { B200_TC_CASE(256, true) }
    if (BN == 256) { B200_TC_CASE(256, false) }
    if (BN == 128) { B200_TC_CASE(128, false) }
    B200_TC_CASE(64, false)
  };
#undef B200_TC_CASE
#ifdef B200_HOST_TIMING
  const double t_launch = HostTimes::now();
  const int err = launch();
  g_host_times.setup += t_launch - t_begin;
  g_host_times.launch += HostTimes::now() - t_launch;
  g_host_times.calls++;
#else
  const int err = launch();
#endif
  if (err || p.splits == 1) return err;
  const long items = (long)g.M * ((g.N + 3) / 4);
  long blocks = (items + 255) / 256;
  if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
  if (launch_dependent(k_splitk_finish, dim3((unsigned)blocks), dim3(256), 0, stream(), p.epi.out, p.splits, p.split_stride,
                       g.M, g.N, g.epi) != cudaSuccess)
    return set_error(cudaGetErrorString(cudaGetLastError()));
  return check_launch();
}

}  // namespace b200

// Test hook (see g_inject_stage_bytes): applies to the next tensor-core product only.
extern "C" int b200_test_inject_stage_bytes(int extra_bytes) {
  b200::g_inject_stage_bytes = extra_bytes > 0 ? extra_bytes : 0;
  return 0;
}

#ifdef B200_GEMM_TIMING
// Debug build only: copies the per-CTA cycle counters of the last launch (8 words per CTA).
extern "C" int b200_gemm_timing(unsigned long long* out, int nctas) {
  cudaStreamSynchronize(b200::stream());
  void* ws = b200::workspace(7, 8 * 512 * sizeof(unsigned long long));
  return cudaMemcpy(out, ws, (size_t)nctas * 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -3;
}
#endif
