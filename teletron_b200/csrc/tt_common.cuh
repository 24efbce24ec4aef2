// Shared device/host helpers for the sm_100a kernels of teletron_b200.
//
// Conventions used by every kernel in this directory:
//  * entry points are plain C symbols (`TT_API int tt_xxx(..., cudaStream_t)`) that
//    return 0 or a negative error code; the message is read with tt_last_error().
//  * every device-side wait on an mbarrier is bounded: when the budget (about two
//    seconds of SM clocks) runs out the kernel records a code in the caller's
//    status word, stops issuing work, releases its tensor memory and returns, so
//    a protocol bug can never leave the GPU spinning.
//  * TMA loads never carry a cluster-broadcast qualifier: each CTA fetches its own
//    tiles.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#define TT_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// ---------------------------------------------------------------------------
// host-side error reporting
// ---------------------------------------------------------------------------
void tt_set_error(const char* fmt, ...);
#define TT_CHECK(cond, ...)            \
  do {                                 \
    if (!(cond)) {                     \
      tt_set_error(__VA_ARGS__);       \
      return -1;                       \
    }                                  \
  } while (0)
#define TT_CUDA(expr)                                                         \
  do {                                                                        \
    cudaError_t _e = (expr);                                                  \
    if (_e != cudaSuccess) {                                                  \
      tt_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                   __FILE__, __LINE__);                                       \
      return -2;                                                              \
    }                                                                         \
  } while (0)
// every kernel launch is followed by one TT_LAUNCH_CHECK(): it also counts launches so that
// callers can report how many of this library's kernels ran (tt_launch_count()).
void tt_count_launch();
#define TT_LAUNCH_CHECK()          \
  do {                             \
    tt_count_launch();             \
    TT_CUDA(cudaGetLastError());   \
  } while (0)

// Builds a tiled TMA descriptor for a row-major bf16/fp32 tensor of up to 4 dims.
// dims[0] is the innermost (contiguous) extent; strides_bytes[i] is the stride of
// dims[i+1]. Returns 0 on success.
int tt_make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank,
                 const uint64_t* dims, const uint64_t* strides_bytes,
                 const uint32_t* box, int swizzle128);

// status codes written by kernels into the caller's status word
enum : unsigned {
  TT_ST_OK = 0,
  TT_ST_TIMEOUT_PRODUCER = 0x100,
  TT_ST_TIMEOUT_MMA = 0x200,
  TT_ST_TIMEOUT_EPILOGUE = 0x300,
  TT_ST_TIMEOUT_SOFTMAX = 0x400,
  TT_ST_TIMEOUT_PEER = 0x500,
  TT_ST_BAD_SMEM_ALIGN = 0x600,  // dynamic shared memory did not start on a 1024-byte boundary
};

// Ulysses all-to-all as a store pattern: where an element of a local tensor lands in peer memory.
//   mode 1 (seq -> head): source [B, S_l, H, D] on rank r  ->  peer h / Hl, [B, S_pad, Hl, D] at
//                         token r*S_l + s, head h % Hl
//   mode 2 (head -> seq): source [B, S_pad, Hl, D] on rank r ->  peer t / S_l, [B, S_l, H, D] at
//                         token t % S_l, head r*Hl + hl; `ld` (elements, 0 = H*D) is the destination's token stride,
//                         so that the destination may be a column block of a wider matrix
// mode 0 means "no scatter" (store locally).
// H need not divide by the group size: Hl = ceil(H / world), the last ranks own fewer (or no) heads and callers
// run only the heads that exist.
// Joint sequences (video tokens followed by replicated text tokens): the head-parallel buffers hold `dst_rows` rows per
// sample (0 = S_pad) of which only the first `n_rows` (0 = all) take part in the exchange; a kernel that scatters
// (mode 2) stores rows >= n_rows to its local output instead.
#define TT_MAX_PEERS 16
struct TTScatter {
  void* peer[TT_MAX_PEERS];
  int mode;
  int S_l, S_pad, Hl, H, D, rank, world;
  long long ld;
  int dst_rows, n_rows;
};

#ifdef __CUDACC__
namespace tt {

// Destination of element (batch b, token tok, head hd, d = 0) of the source tensor; bf16 elements.
__device__ __forceinline__ bf16* scatter_dst(const TTScatter& sc, int b, int tok, int hd) {
  if (sc.mode == 1) {
    const int p = hd / sc.Hl;
    const int rows = sc.dst_rows ? sc.dst_rows : sc.S_pad;
    const long long idx = ((long long)b * rows + sc.rank * sc.S_l + tok) * sc.Hl * sc.D + (long long)(hd - p * sc.Hl) * sc.D;
    return reinterpret_cast<bf16*>(sc.peer[p]) + idx;
  }
  const int p = tok / sc.S_l;
  const long long ld = sc.ld ? sc.ld : (long long)sc.H * sc.D;
  const long long idx = (long long)(b * sc.S_l + (tok - p * sc.S_l)) * ld + (long long)(sc.rank * sc.Hl + hd) * sc.D;
  return reinterpret_cast<bf16*>(sc.peer[p]) + idx;
}

// whether row `row` of a kernel that scatters its output (mode 2) goes to a peer (else: to the local output)
__device__ __forceinline__ bool scatter_row(const TTScatter& sc, int row, int rows_total) {
  return sc.mode == 2 && row < rows_total && (sc.n_rows == 0 || row < sc.n_rows);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Row staging for epilogues whose accumulator comes out of tensor memory one row per lane.  Written from the
// registers as they are, a warp's store instruction touches 32 rows with 16 bytes each: fine for the local L2,
// wasteful over NVLink, where every 16-byte piece travels as a packet of its own.  The warp instead parks its
// 32 x (CH x 16 B) block in its own shared-memory area (chunks XOR-swizzled by the row, so neither the writes nor
// the reads conflict) and writes it out with CH lanes per row: each row leaves as one contiguous piece of
// CH x 16 bytes.  Only the warp itself touches the area: __syncwarp() is the only synchronisation.
template <int CH>
__device__ __forceinline__ void stage_put(uint8_t* stage, int lane, int chunk, const uint4& v) {
  *reinterpret_cast<uint4*>(stage + lane * (CH * 16) + ((chunk ^ (lane & (CH - 1))) << 4)) = v;
}
// dst0 / dst1: this lane's row in up to two destinations (nullptr: skip that destination for the row)
template <int CH>
__device__ __forceinline__ void stage_flush(const uint8_t* stage, int lane, bf16* dst0, bf16* dst1) {
  constexpr int RPI = 32 / CH;  // rows per store instruction
  const int chunk = lane & (CH - 1);
  const unsigned long long a0 = reinterpret_cast<unsigned long long>(dst0);
  const unsigned long long a1 = reinterpret_cast<unsigned long long>(dst1);
  __syncwarp();
#pragma unroll 4
  for (int i = 0; i < 32 / RPI; ++i) {
    const int row = i * RPI + lane / CH;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + row * (CH * 16) + ((chunk ^ (row & (CH - 1))) << 4));
    const unsigned long long r0 = __shfl_sync(0xffffffffu, a0, row);
    const unsigned long long r1 = __shfl_sync(0xffffffffu, a1, row);
    if (r0) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(r0) + chunk * 8) = v;
    if (r1) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(r1) + chunk * 8) = v;
  }
  __syncwarp();
}
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Budget for any single wait, in SM clocks (about 2 s at 2 GHz).
#ifndef TT_WAIT_BUDGET_CLOCKS
#define TT_WAIT_BUDGET_CLOCKS (4000000000ll)
#endif

// Bounded wait. `abort_flag` lives in shared memory and is raised by whichever
// role times out first, so that the other roles leave their loops quickly.
// Returns false when the wait was abandoned.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          volatile uint32_t* abort_flag, unsigned* status,
                                          unsigned code) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > TT_WAIT_BUDGET_CLOCKS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0u, code);
        return false;
      }
    }
  }
  return true;
}

// The same wait for a whole (converged) warp: lane 0 polls and the outcome is broadcast.  Thirty-two lanes
// polling one mbarrier are served one after the other (about 200 clocks per wait even when the phase has
// already completed); the shuffle also orders the other lanes' later reads behind lane 0's acquire.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity,
                                               volatile uint32_t* abort_flag, unsigned* status,
                                               unsigned code) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag, status, code) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4, %5, %6}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// generic-proxy writes to shared memory -> visible to the async proxy (UMMA / TMA)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives on `bar` once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrives on the barrier at this shared-memory offset in every CTA of `mask` once all MMAs issued so far are done
__device__ __forceinline__ void tc_commit2(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}
template <uint32_t HI_A, uint32_t HI_B>
__device__ __forceinline__ void umma2_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 ad, bd;\n\t"
      "mov.b64 ad, {%1, %5};\n\t"
      "mov.b64 bd, {%2, %6};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], ad, bd, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "n"(HI_A), "n"(HI_B)
      : "memory");
}
// TMA load into this CTA's shared memory whose completion bytes are counted on a barrier given as a
// shared::cluster address (the leader's)
__device__ __forceinline__ void tma2_load_2d(void* dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0,
                                             int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem] on a CTA pair: each CTA's tensor memory supplies its 128 rows of A
template <uint32_t HI_B>
__device__ __forceinline__ void umma2_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\t"
      "mov.b64 bd, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], bd, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "n"(HI_B)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0,
                                             int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Shared-memory matrix descriptor for 128-byte swizzled tiles (the layout TMA
// writes with CU_TENSOR_MAP_SWIZZLE_128B; tile base aligned to 1024 bytes).
//  K-major operand  : rows of 64 bf16 (128 B); sbo = distance between 8-row groups.
//  MN-major operand : rows of 64 bf16 along M/N, one row per k; lbo = distance
//                     between successive 64-wide M/N groups, sbo = distance
//                     between successive groups of 8 k-rows.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // 128-byte swizzle
  return d;
}
// The same descriptor as two 32-bit words.  The high word (stride between 8-row groups, version,
// swizzle mode) is the same for every k-step of an operand and the low word moves by (bytes >> 4),
// so an MMA loop costs one integer add per operand instead of rebuilding 64-bit descriptors: the single
// issuing thread runs a dependent instruction chain, and rebuilding them was measured to cap the issue
// rate at one tcgen05.mma per 70-100 clocks.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
  return ((smem_addr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__host__ __device__ constexpr uint32_t umma_desc_hi(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
// D[tmem] (+)= A[smem] * B[smem]; descriptors given as (low word, shared high word)
template <uint32_t HI_A, uint32_t HI_B>
__device__ __forceinline__ void umma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 ad, bd;\n\t"
      "mov.b64 ad, {%1, %5};\n\t"
      "mov.b64 bd, {%2, %6};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ad, bd, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "n"(HI_A), "n"(HI_B)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
template <uint32_t HI_B>
__device__ __forceinline__ void umma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\t"
      "mov.b64 bd, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "n"(HI_B)
      : "memory");
}
// Instruction descriptor: bf16 x bf16 -> fp32, shape M x N (K = 16 per instruction).
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives row
// (lane quarter base + t), columns [col, col+32).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}
// 32 lanes x 16 columns (e.g. 32 packed bf16 per row: an A operand slice for tcgen05.mma)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- math
// 2^x on the special-function unit, no range fix-ups (inputs here are <= ~0 or masked to -1e30)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + fast_tanh(u));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  float t = tanhf(u);
  float du = k0 * (1.f + 3.f * k1 * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float silu_grad(float x) {
  float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  bf162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  bf162 v = *reinterpret_cast<bf162*>(&u);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace tt
#endif  // __CUDACC__
