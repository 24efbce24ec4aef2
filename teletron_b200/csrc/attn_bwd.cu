// K-ATTN backward for head_dim 128 on tcgen05 / TMEM, as two kernels without atomics
// (deterministic), plus the row-dot preprocess  delta[b,h,q] = sum_d dO * O:
//
//   attn_bwd_dkdv : one CTA owns 128 keys of one (batch, head) and walks the queries in tiles of 128.
//   attn_bwd_dq   : one CTA owns 128 queries and walks the keys in tiles of 128.
//
// Every product is a 128 x 128 x 16 tcgen05.mma: narrower instructions (N = 64) were measured at
// 46-55 clocks instead of 32, and full-width ones at their nominal 64.  P is recomputed from the saved
// log-sum-exp; the bf16 P^T / dS^T / dS operands are written over the fp32 scores in tensor memory and
// read from there (A operand in tensor memory), so they never touch shared memory.  Roles per CTA
// (320 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 elementwise (two per lane quarter,
// each owning 64 of a tile's 128 columns).  Every wait is bounded.
#include "tt_common.cuh"
#include <stdlib.h>

using namespace tt;

namespace {

constexpr int NTHREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2..9 elementwise (two per lane quarter)
constexpr int BIG = 128 * 128 * 2;     // 128 x 128 bf16 tile (two 64-wide halves of 16 KB)
constexpr int BIG_HALF = 128 * 128;    // 128 rows x 128 B
constexpr float LOG2E = 1.4426950408889634f;
constexpr uint32_t HI_K = umma_desc_hi(1024);  // both operand layouts here step 1024 bytes between 8-row groups

struct BwdParams {
  int Sq, Skv, H, B;
  float scale, scale_log2;
  const float* lse2;   // [B,H,Sq_pad]  log-sum-exp in log2 units, padding = 1e30
  const float* delta;  // [B,H,Sq_pad]  padding = 0
  int Sq_pad;
  bf16* out0;          // dK (dkdv) or dQ (dq)
  bf16* out1;          // dV (dkdv)
  long long ld0, bs0, ld1, bs1;
  const int* kv_lens;
  unsigned* status;
  TTScatter sc0;  // mode 2: out0 (dK or dQ) is stored into the owning peer's [B, S_l, H, D] buffer
  TTScatter sc1;  // likewise for out1 (dV)
};

// plain (untiled) bulk copy global -> shared, completion counted on an mbarrier
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ===================================================================== dK / dV
// One CTA owns 128 keys (tensor-memory lanes) and walks the queries in tiles of 128.
//   S^T(j)  = K Q_j^T               128 x 128 fp32;  P^T(j) (bf16) is written over it
//   dP^T(j) = V dO_j^T              128 x 128 fp32;  dS^T(j) (bf16) is written over it
//   dV += P^T(j) dO_j,  dK += dS^T(j) Q_j            A operands read from tensor memory
// S^T, dP^T, dV and dK fill the 512 columns of tensor memory.  The tensor pipe executes
//   ... dV(j) S^T(j+1) dK(j) dP^T(j+1) | dV(j+1) S^T(j+2) dK(j+1) dP^T(j+2) ...
// phase 1 (P^T from S^T) of tile j+1 runs under dK(j) and dP^T(j+1), phase 2 (dS^T) under dV(j+1), S^T(j+2).
constexpr int A_QST = 3;                         // Q stages (a Q tile lives from S^T(j) to dK(j))
constexpr int A_DST = 2;                         // dO stages, each with the tile's 128 lse and 128 delta values
constexpr int A_SM_K = 0;
constexpr int A_SM_V = A_SM_K + BIG;
constexpr int A_SM_Q = A_SM_V + BIG;
constexpr int A_SM_DO = A_SM_Q + A_QST * BIG;
constexpr int A_SM_LSE = A_SM_DO + A_DST * BIG;  // A_DST x (128 lse2 + 128 delta) floats
constexpr int A_SM_BAR = A_SM_LSE + A_DST * 256 * 4;
constexpr int A_SMEM = A_SM_BAR + 256;
constexpr int A_TM_ST = 0, A_TM_DPT = 128, A_TM_DV = 256, A_TM_DK = 384;

// column (32-bit) of k-step `ks` of a packed bf16 operand that the two elementwise warp groups wrote over
// the first 32 columns of their own 64-column halves of a 128-column fp32 tile
__device__ __forceinline__ uint32_t packed_kstep_col(int ks) { return (uint32_t)((ks >> 2) * 64 + (ks & 3) * 8); }

__global__ void __launch_bounds__(NTHREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A_SM_BAR);
  uint64_t* kv_full = bars;                 // 1
  uint64_t* q_full = bars + 1;              // A_QST
  uint64_t* q_empty = q_full + A_QST;       // A_QST
  uint64_t* do_full = q_empty + A_QST;      // A_DST
  uint64_t* do_empty = do_full + A_DST;     // A_DST
  uint64_t* s_full = do_empty + A_DST;      // 1
  uint64_t* dp_full = s_full + 1;           // 1
  uint64_t* p_full = dp_full + 1;           // 1 (8 arrivals): P^T is in place
  uint64_t* ds_full = p_full + 1;           // 1 (8 arrivals): dS^T is in place
  uint64_t* done_bar = ds_full + 1;         // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* lse_s = reinterpret_cast<float*>(smem + A_SM_LSE);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv0 = blockIdx.x * 128;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int n_it = (p.Sq + 127) / 128;

  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0u, TT_ST_BAD_SMEM_ALIGN);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < A_QST; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    for (int i = 0; i < A_DST; ++i) { mbar_init(&do_full[i], 1); mbar_init(&do_empty[i], 1); }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_full, 8);
    mbar_init(ds_full, 8);
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * BIG);
      for (int hf = 0; hf < 2; ++hf) {
        tma_load_3d(smem + A_SM_K + hf * BIG_HALF, &tmK, kv_full, h * 128 + hf * 64, kv0, b);
        tma_load_3d(smem + A_SM_V + hf * BIG_HALF, &tmV, kv_full, h * 128 + hf * 64, kv0, b);
      }
      for (int j = 0; j < n_it; ++j) {
        const int qs = j % A_QST, ds_ = j % A_DST;
        if (!mbar_wait(&q_empty[qs], ((j / A_QST) & 1) ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&q_full[qs], BIG);
        for (int hf = 0; hf < 2; ++hf)
          tma_load_3d(smem + A_SM_Q + qs * BIG + hf * BIG_HALF, &tmQ, &q_full[qs], h * 128 + hf * 64, j * 128, b);
        if (!mbar_wait(&do_empty[ds_], ((j / A_DST) & 1) ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_PRODUCER + 1)) break;
        mbar_expect_tx(&do_full[ds_], BIG + 1024);
        for (int hf = 0; hf < 2; ++hf)
          tma_load_3d(smem + A_SM_DO + ds_ * BIG + hf * BIG_HALF, &tmdO, &do_full[ds_], h * 128 + hf * 64, j * 128, b);
        const long long roff = ((long long)b * p.H + h) * p.Sq_pad + j * 128;
        bulk_load(lse_s + ds_ * 256, p.lse2 + roff, 512, &do_full[ds_]);
        bulk_load(lse_s + ds_ * 256 + 128, p.delta + roff, 512, &do_full[ds_]);
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the schedule with warp-uniform values and lane 0 issues the tcgen05 instructions.
    // What runs between two groups of MMAs decides whether the tensor pipe runs dry, and was tuned by
    // measurement: all lanes poll a barrier and vote (lane 0 polling alone, followed by a shuffle, was slower,
    // as was a single-thread loop); ring positions are counters; the wait on TMA data precedes the wait on the
    // elementwise warps, so that the MMAs that follow go out back to back.
    constexpr uint32_t idesc_s = umma_idesc(128, 128, 0, 0);
    constexpr uint32_t idesc_o = umma_idesc(128, 128, 0, 1);
    const bool leader = lane == 0;
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem_base, 0);
    const uint32_t k_lo = umma_desc_lo(smem_u32(smem + A_SM_K), 16);
    const uint32_t v_lo = umma_desc_lo(smem_u32(smem + A_SM_V), 16);
    const uint32_t q_base = smem_u32(smem + A_SM_Q);
    const uint32_t do_base = smem_u32(smem + A_SM_DO);
    auto wait_w = [&](uint64_t* bar, uint32_t parity, unsigned code) -> bool {
      const bool w = mbar_wait(bar, parity, abort_flag, p.status, code);
      return __all_sync(0xffffffffu, w);
    };
    auto mma_st = [&](uint32_t q_st) {
      const uint32_t qb = umma_desc_lo(q_base + q_st * BIG, 16);
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * BIG_HALF + (ks & 3) * 32) >> 4;
          umma_ss_lo<HI_K, HI_K>(tm + A_TM_ST, k_lo + off, qb + off, idesc_s, ks != 0);
        }
        tc_commit(s_full);
      }
    };
    auto mma_dpt = [&](uint32_t d_st) {
      const uint32_t dob = umma_desc_lo(do_base + d_st * BIG, 16);
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * BIG_HALF + (ks & 3) * 32) >> 4;
          umma_ss_lo<HI_K, HI_K>(tm + A_TM_DPT, v_lo + off, dob + off, idesc_s, ks != 0);
        }
        tc_commit(dp_full);
      }
    };
    // dV += P^T dO and dK += dS^T Q with the A operand read from tensor memory
    auto mma_dv = [&](uint32_t d_st, uint32_t acc0) {
      const uint32_t dob = umma_desc_lo(do_base + d_st * BIG, BIG_HALF);
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts_lo<HI_K>(tm + A_TM_DV, tm + A_TM_ST + packed_kstep_col(ks), dob + ks * (2048 >> 4), idesc_o,
                           ks != 0 ? 1u : acc0);
      }
    };
    auto mma_dk = [&](uint32_t q_st, uint32_t d_st, uint32_t acc0) {
      const uint32_t qb = umma_desc_lo(q_base + q_st * BIG, BIG_HALF);
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts_lo<HI_K>(tm + A_TM_DK, tm + A_TM_DPT + packed_kstep_col(ks), qb + ks * (2048 >> 4), idesc_o,
                           ks != 0 ? 1u : acc0);
        // the elementwise warps have read this tile's lse / delta by now, so its dO stage may be refilled too
        tc_commit(&q_empty[q_st]);
        tc_commit(&do_empty[d_st]);
      }
    };
    // ring positions: (stage, phase) of the tile that the next S^T / dP^T reads, stages of the tile that the
    // next dV / dK reads
    uint32_t qs = 0, qph = 0, ds = 0, dph = 0, qs_old = 0, ds_old = 0, eph = 0;
    bool ok = wait_w(kv_full, 0, TT_ST_TIMEOUT_MMA + 1);
    if (ok) ok = wait_w(&q_full[0], 0, TT_ST_TIMEOUT_MMA + 2);
    if (ok) ok = wait_w(&do_full[0], 0, TT_ST_TIMEOUT_MMA + 3);
    if (ok) {
      tc_fence_after();
      mma_st(0);
      mma_dpt(0);
      if (++qs == A_QST) { qs = 0; qph ^= 1; }
      if (++ds == A_DST) { ds = 0; dph ^= 1; }
    }
    for (int j = 0; j < n_it && ok; ++j) {
      const bool more = j + 1 < n_it;
      const uint32_t acc0 = j > 0 ? 1u : 0u;
      if (more) ok = wait_w(&q_full[qs], qph, TT_ST_TIMEOUT_MMA + 2);
      if (ok) ok = wait_w(p_full, eph, TT_ST_TIMEOUT_MMA + 4);
      if (!ok) break;
      tc_fence_after();
      mma_dv(ds_old, acc0);
      if (more) mma_st(qs);
      if (more) ok = wait_w(&do_full[ds], dph, TT_ST_TIMEOUT_MMA + 3);
      if (ok) ok = wait_w(ds_full, eph, TT_ST_TIMEOUT_MMA + 5);
      if (!ok) break;
      tc_fence_after();
      mma_dk(qs_old, ds_old, acc0);
      if (more) mma_dpt(ds);
      qs_old = qs;
      ds_old = ds;
      eph ^= 1;
      if (++qs == A_QST) { qs = 0; qph ^= 1; }
      if (++ds == A_DST) { ds = 0; dph ^= 1; }
    }
    if (ok && leader) tc_commit(done_bar);
  } else {
    // ------------------------------------------------------------ elementwise warps
    const int q = warp & 3;
    const int wg = (warp - 2) >> 2;  // which 64 of the tile's 128 query columns (and half of the output columns)
    const int r = q * 32 + lane;     // key row in the tile
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    bool ok = true;
    for (int j = 0; j < n_it; ++j) {
      const int ld = j % A_DST;
      const float* ls = lse_s + ld * 256 + wg * 64;
      const float* dl = ls + 128;
      if (!mbar_wait(&do_full[ld], (j / A_DST) & 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 4)) { ok = false; break; }
      if (!mbar_wait(s_full, j & 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 1)) { ok = false; break; }
      __syncwarp();
      tc_fence_after();
      float pr[64];
      // phase 1: P^T = 2^(S^T scale log2e - lse), bf16 copy over the first half of this group's S^T columns;
      // both 32-column loads are in flight before the first is used
      {
        const uint32_t s_addr = tmem_base + lane_addr + A_TM_ST + wg * 64;
        uint32_t s0[32], s1[32], pk[16];
        tmem_ld32(s_addr, s0);
        tmem_ld32(s_addr + 32, s1);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 a4 = *reinterpret_cast<const float4*>(ls + e);
          pr[e] = fast_exp2(fmaf(__uint_as_float(s0[e]), p.scale_log2, -a4.x));
          pr[e + 1] = fast_exp2(fmaf(__uint_as_float(s0[e + 1]), p.scale_log2, -a4.y));
          pr[e + 2] = fast_exp2(fmaf(__uint_as_float(s0[e + 2]), p.scale_log2, -a4.z));
          pr[e + 3] = fast_exp2(fmaf(__uint_as_float(s0[e + 3]), p.scale_log2, -a4.w));
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) pk[e] = pack_bf16(pr[2 * e], pr[2 * e + 1]);
        tmem_st16(s_addr, pk);
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 a4 = *reinterpret_cast<const float4*>(ls + 32 + e);
          pr[32 + e] = fast_exp2(fmaf(__uint_as_float(s1[e]), p.scale_log2, -a4.x));
          pr[32 + e + 1] = fast_exp2(fmaf(__uint_as_float(s1[e + 1]), p.scale_log2, -a4.y));
          pr[32 + e + 2] = fast_exp2(fmaf(__uint_as_float(s1[e + 2]), p.scale_log2, -a4.z));
          pr[32 + e + 3] = fast_exp2(fmaf(__uint_as_float(s1[e + 3]), p.scale_log2, -a4.w));
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) pk[e] = pack_bf16(pr[32 + 2 * e], pr[32 + 2 * e + 1]);
        tmem_st16(s_addr + 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      if (!mbar_wait(dp_full, j & 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 2)) { ok = false; break; }
      __syncwarp();
      tc_fence_after();
      // phase 2: dS^T = P^T o (dP^T - delta)
      {
        const uint32_t dp_addr = tmem_base + lane_addr + A_TM_DPT + wg * 64;
        uint32_t d0[32], d1[32], ds[16];
        tmem_ld32(dp_addr, d0);
        tmem_ld32(dp_addr + 32, d1);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(dl + e);
          ds[e / 2] = pack_bf16(pr[e] * (__uint_as_float(d0[e]) - d4.x), pr[e + 1] * (__uint_as_float(d0[e + 1]) - d4.y));
          ds[e / 2 + 1] = pack_bf16(pr[e + 2] * (__uint_as_float(d0[e + 2]) - d4.z),
                                    pr[e + 3] * (__uint_as_float(d0[e + 3]) - d4.w));
        }
        tmem_st16(dp_addr, ds);
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(dl + 32 + e);
          ds[e / 2] = pack_bf16(pr[32 + e] * (__uint_as_float(d1[e]) - d4.x),
                                pr[32 + e + 1] * (__uint_as_float(d1[e + 1]) - d4.y));
          ds[e / 2 + 1] = pack_bf16(pr[32 + e + 2] * (__uint_as_float(d1[e + 2]) - d4.z),
                                    pr[32 + e + 3] * (__uint_as_float(d1[e + 3]) - d4.w));
        }
        tmem_st16(dp_addr + 16, ds);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok) ok = mbar_wait(done_bar, 0, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 3);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int row = kv0 + r;
      int kv_len = p.Skv;
      if (p.kv_lens) kv_len = min(max(p.kv_lens[b], 1), p.Skv);
      const bool live = row < kv_len;
      // every operand tile has been consumed: the first Q stage stages the output rows, 4 KB per warp
      uint8_t* stage = smem + A_SM_Q + (warp - 2) * (32 * 128);
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {  // 0: dV, 1: dK
        bf16* dst = nullptr;
        if (which == 0)
          dst = scatter_row(p.sc1, row, p.Skv) ? scatter_dst(p.sc1, b, row, h)
                                                 : p.out1 + (long long)b * p.bs1 + (long long)row * p.ld1 + h * 128;
        else
          dst = scatter_row(p.sc0, row, p.Skv) ? scatter_dst(p.sc0, b, row, h)
                                                 : p.out0 + (long long)b * p.bs0 + (long long)row * p.ld0 + h * 128;
        dst = row < p.Skv ? dst + wg * 64 : nullptr;
        const float m2 = live ? (which == 0 ? 1.f : p.scale) : 0.f;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_base + lane_addr + A_TM_DV + which * 128 + (wg * 2 + c) * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(o[g * 8 + 0]) * m2, __uint_as_float(o[g * 8 + 1]) * m2);
            pk.y = pack_bf16(__uint_as_float(o[g * 8 + 2]) * m2, __uint_as_float(o[g * 8 + 3]) * m2);
            pk.z = pack_bf16(__uint_as_float(o[g * 8 + 4]) * m2, __uint_as_float(o[g * 8 + 5]) * m2);
            pk.w = pack_bf16(__uint_as_float(o[g * 8 + 6]) * m2, __uint_as_float(o[g * 8 + 7]) * m2);
            stage_put<8>(stage, lane, c * 4 + g, pk);
          }
        }
        stage_flush<8>(stage, lane, dst, nullptr);
      }
    }
  }
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ===================================================================== dQ
// One CTA owns 128 queries (tensor-memory lanes) and walks the keys in tiles of 128.
//   S(j)  = Q K_j^T            128 x 128, fp32, double-buffered in tensor memory
//   dP(j) = dO V_j^T           128 x 128, fp32, one buffer
//   dS(j) = P o (dP - delta)   bf16, written over dP(j) as the A operand of the next product
//   dQ   += dS(j) K_j          128 x 128 accumulator
// The tensor pipe executes S(0) dP(0) S(1) | dQ(0) dP(1) S(2) | dQ(1) dP(2) S(3) ... so that the exponentials
// of tile j+1 (phase 1) and the dS of tile j+1 (phase 2) run under the products of the neighbouring tiles.
constexpr int B_KST = 3;                            // K stages (a K tile lives from S(j) to dQ(j))
constexpr int B_VST = 2;                            // V stages
constexpr int B_SM_Q = 0;
constexpr int B_SM_DO = B_SM_Q + BIG;
constexpr int B_SM_K = B_SM_DO + BIG;
constexpr int B_SM_V = B_SM_K + B_KST * BIG;
constexpr int B_SM_BAR = B_SM_V + B_VST * BIG;
constexpr int B_SMEM = B_SM_BAR + 256;
constexpr int B_TM_S = 0, B_TM_DP = 256, B_TM_DQ = 384;

__global__ void __launch_bounds__(NTHREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + B_SM_BAR);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;             // B_KST
  uint64_t* k_empty = k_full + B_KST;      // B_KST
  uint64_t* v_full = k_empty + B_KST;      // B_VST
  uint64_t* v_empty = v_full + B_VST;      // B_VST
  uint64_t* s_full = v_empty + B_VST;      // 2
  uint64_t* dp_full = s_full + 2;          // 1
  uint64_t* ds_full = dp_full + 1;         // 1 (8 arrivals)
  uint64_t* done_bar = ds_full + 1;        // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 128;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  int kv_len = p.Skv;
  if (p.kv_lens) kv_len = min(max(p.kv_lens[b], 1), p.Skv);
  const int n_it = (kv_len + 127) / 128;

  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0u, TT_ST_BAD_SMEM_ALIGN);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < B_KST; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < B_VST; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(dp_full, 1);
    mbar_init(ds_full, 8);
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * BIG);
      for (int hf = 0; hf < 2; ++hf) {
        tma_load_3d(smem + B_SM_Q + hf * BIG_HALF, &tmQ, q_full, h * 128 + hf * 64, q0, b);
        tma_load_3d(smem + B_SM_DO + hf * BIG_HALF, &tmdO, q_full, h * 128 + hf * 64, q0, b);
      }
      for (int j = 0; j < n_it; ++j) {
        const int ks_ = j % B_KST, vs_ = j % B_VST;
        if (!mbar_wait(&k_empty[ks_], ((j / B_KST) & 1) ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&k_full[ks_], BIG);
        for (int hf = 0; hf < 2; ++hf)
          tma_load_3d(smem + B_SM_K + ks_ * BIG + hf * BIG_HALF, &tmK, &k_full[ks_], h * 128 + hf * 64, j * 128, b);
        if (!mbar_wait(&v_empty[vs_], ((j / B_VST) & 1) ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_PRODUCER + 1)) break;
        mbar_expect_tx(&v_full[vs_], BIG);
        for (int hf = 0; hf < 2; ++hf)
          tma_load_3d(smem + B_SM_V + vs_ * BIG + hf * BIG_HALF, &tmV, &v_full[vs_], h * 128 + hf * 64, j * 128, b);
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the schedule, lane 0 issues (see the note in attn_bwd_dkdv_kernel).
    constexpr uint32_t idesc_s = umma_idesc(128, 128, 0, 0);
    constexpr uint32_t idesc_o = umma_idesc(128, 128, 0, 1);
    const bool leader = lane == 0;
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem_base, 0);
    const uint32_t q_lo = umma_desc_lo(smem_u32(smem + B_SM_Q), 16);
    const uint32_t do_lo = umma_desc_lo(smem_u32(smem + B_SM_DO), 16);
    const uint32_t k_base = smem_u32(smem + B_SM_K);
    const uint32_t v_base = smem_u32(smem + B_SM_V);
    auto wait_w = [&](uint64_t* bar, uint32_t parity, unsigned code) -> bool {
      const bool w = mbar_wait(bar, parity, abort_flag, p.status, code);
      return __all_sync(0xffffffffu, w);
    };
    auto mma_s = [&](uint32_t k_st, uint32_t buf) {
      const uint32_t kb = umma_desc_lo(k_base + k_st * BIG, 16);
      const uint32_t d_s = tm + B_TM_S + buf * 128;
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * BIG_HALF + (ks & 3) * 32) >> 4;
          umma_ss_lo<HI_K, HI_K>(d_s, q_lo + off, kb + off, idesc_s, ks != 0);
        }
        tc_commit(&s_full[buf]);
      }
    };
    auto mma_dp = [&](uint32_t v_st) {
      const uint32_t vb = umma_desc_lo(v_base + v_st * BIG, 16);
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * BIG_HALF + (ks & 3) * 32) >> 4;
          umma_ss_lo<HI_K, HI_K>(tm + B_TM_DP, do_lo + off, vb + off, idesc_s, ks != 0);
        }
        tc_commit(dp_full);
        tc_commit(&v_empty[v_st]);
      }
    };
    auto mma_dq = [&](uint32_t k_st, uint32_t acc0) {
      const uint32_t kb = umma_desc_lo(k_base + k_st * BIG, BIG_HALF);
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts_lo<HI_K>(tm + B_TM_DQ, tm + B_TM_DP + packed_kstep_col(ks), kb + ks * (2048 >> 4), idesc_o,
                           ks != 0 ? 1u : acc0);
        tc_commit(&k_empty[k_st]);
      }
    };
    // ring positions: (stage, phase) of the K tile the next S reads and of the V tile the next dP reads;
    // stage of the K tile the next dQ reads
    uint32_t ks_ = 0, kph = 0, vs_ = 0, vph = 0, kq = 0, eph = 0, sbuf = 0;
    bool ok = wait_w(q_full, 0, TT_ST_TIMEOUT_MMA + 1);
    if (ok) ok = wait_w(&k_full[0], 0, TT_ST_TIMEOUT_MMA + 2);
    if (ok) ok = wait_w(&v_full[0], 0, TT_ST_TIMEOUT_MMA + 3);
    if (ok && n_it > 1) ok = wait_w(&k_full[1], 0, TT_ST_TIMEOUT_MMA + 2);
    if (ok) {
      tc_fence_after();
      mma_s(0, 0);
      mma_dp(0);
      ks_ = 1; vs_ = 1; sbuf = 1;
      if (n_it > 1) {
        mma_s(1, 1);
        ks_ = 2; sbuf = 0;
      }
    }
    // here: ks_/kph -> K(j+2), vs_/vph -> V(j+1), sbuf = (j+2) & 1, kq -> K(j)
    for (int j = 0; j < n_it && ok; ++j) {
      if (j + 1 < n_it) ok = wait_w(&v_full[vs_], vph, TT_ST_TIMEOUT_MMA + 3);
      if (ok && j + 2 < n_it) ok = wait_w(&k_full[ks_], kph, TT_ST_TIMEOUT_MMA + 2);
      if (ok) ok = wait_w(ds_full, eph, TT_ST_TIMEOUT_MMA + 4);
      if (!ok) break;
      tc_fence_after();
      mma_dq(kq, j > 0 ? 1u : 0u);
      if (j + 1 < n_it) mma_dp(vs_);
      if (j + 2 < n_it) mma_s(ks_, sbuf);
      if (++kq == B_KST) kq = 0;
      eph ^= 1;
      if (++vs_ == B_VST) { vs_ = 0; vph ^= 1; }
      sbuf ^= 1;
      if (++ks_ == B_KST) { ks_ = 0; kph ^= 1; }
    }
    if (ok && leader) tc_commit(done_bar);
  } else {
    const int q = warp & 3;
    const int wg = (warp - 2) >> 2;  // which 64 of the tile's 128 key columns
    const int r = q * 32 + lane;
    const int row = q0 + r;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    float lse2 = 1.0e30f, del = 0.f;
    if (row < p.Sq) {
      lse2 = p.lse2[((long long)b * p.H + h) * p.Sq_pad + row];
      del = p.delta[((long long)b * p.H + h) * p.Sq_pad + row];
    }
    bool ok = true;
    for (int j = 0; j < n_it; ++j) {
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 1)) { ok = false; break; }
      __syncwarp();
      tc_fence_after();
      const int valid = kv_len - j * 128 - wg * 64;  // live columns of this warp group's half
      float pr[64];
      // phase 1: P = 2^(S scale log2e - lse); both 32-column loads are in flight before the first is used
      {
        uint32_t s0[32], s1[32];
        const uint32_t s_addr = tmem_base + lane_addr + B_TM_S + (j & 1) * 128 + wg * 64;
        tmem_ld32(s_addr, s0);
        tmem_ld32(s_addr + 32, s1);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float pe = fast_exp2(fmaf(__uint_as_float(s0[e]), p.scale_log2, -lse2));
          pr[e] = (e < valid) ? pe : 0.f;
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float pe = fast_exp2(fmaf(__uint_as_float(s1[e]), p.scale_log2, -lse2));
          pr[32 + e] = (32 + e < valid) ? pe : 0.f;
        }
      }
      if (!mbar_wait(dp_full, j & 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 2)) { ok = false; break; }
      __syncwarp();
      tc_fence_after();
      // phase 2: dS = P o (dP - delta), packed bf16 over the first half of this warp group's dP columns
      {
        uint32_t d0[32], d1[32], ds[16];
        const uint32_t dp_addr = tmem_base + lane_addr + B_TM_DP + wg * 64;
        tmem_ld32(dp_addr, d0);
        tmem_ld32(dp_addr + 32, d1);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; ++e)
          ds[e] = pack_bf16(pr[2 * e] * (__uint_as_float(d0[2 * e]) - del),
                            pr[2 * e + 1] * (__uint_as_float(d0[2 * e + 1]) - del));
        tmem_st16(dp_addr, ds);
#pragma unroll
        for (int e = 0; e < 16; ++e)
          ds[e] = pack_bf16(pr[32 + 2 * e] * (__uint_as_float(d1[2 * e]) - del),
                            pr[32 + 2 * e + 1] * (__uint_as_float(d1[2 * e + 1]) - del));
        tmem_st16(dp_addr + 16, ds);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok) ok = mbar_wait(done_bar, 0, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 3);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      bf16* dst = scatter_row(p.sc0, row, p.Sq) ? scatter_dst(p.sc0, b, row, h)
                                                  : p.out0 + (long long)b * p.bs0 + (long long)row * p.ld0 + h * 128;
      dst = row < p.Sq ? dst + wg * 64 : nullptr;
      // every operand tile has been consumed: the first K stage stages the output rows, 4 KB per warp
      uint8_t* stage = smem + B_SM_K + (warp - 2) * (32 * 128);
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_base + lane_addr + B_TM_DQ + (wg * 2 + c) * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 pk;
          pk.x = pack_bf16(__uint_as_float(o[g * 8 + 0]) * p.scale, __uint_as_float(o[g * 8 + 1]) * p.scale);
          pk.y = pack_bf16(__uint_as_float(o[g * 8 + 2]) * p.scale, __uint_as_float(o[g * 8 + 3]) * p.scale);
          pk.z = pack_bf16(__uint_as_float(o[g * 8 + 4]) * p.scale, __uint_as_float(o[g * 8 + 5]) * p.scale);
          pk.w = pack_bf16(__uint_as_float(o[g * 8 + 6]) * p.scale, __uint_as_float(o[g * 8 + 7]) * p.scale);
          stage_put<8>(stage, lane, c * 4 + g, pk);
        }
      }
      stage_flush<8>(stage, lane, dst, nullptr);
    }
  }
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ===================================================================== preprocess
// delta[b,h,q] = sum_d dO*O and lse2 = lse * log2(e), both written to [B,H,Sq_pad] buffers whose
// padding rows hold 0 / 1e30 (so padded queries get probability 0).  Sixteen lanes per (b, q, h) row with 16-byte
// loads; a warp takes eight consecutive rows (2 KB of each tensor when the rows are dense) with all of its loads
// in flight before the first is used.
__global__ void __launch_bounds__(256)
attn_preprocess_kernel(const bf16* __restrict__ o, long long ldo, long long o_bs, const bf16* __restrict__ dout,
                       long long lddo, long long do_bs, const float* __restrict__ lse, float* __restrict__ lse2,
                       float* __restrict__ delta, int B, int H, int Sq, int Sq_pad) {
  // row counts stay below 2^31 (checked on the host), so the index arithmetic is 32-bit
  const unsigned gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int sub = lane >> 4, l16 = lane & 15;
  const unsigned total = (unsigned)B * (unsigned)Sq_pad * (unsigned)H;
  uint4 av[4], dv[4];
  unsigned bh[4], qv[4];
  int state[4];  // 0: beyond the end, 1: padding row, 2: live row
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const unsigned R = gw * 8 + it * 2 + sub;
    state[it] = 0;
    av[it] = make_uint4(0, 0, 0, 0);
    dv[it] = make_uint4(0, 0, 0, 0);
    bh[it] = qv[it] = 0;
    if (R < total) {
      const unsigned t = R / (unsigned)H;
      const unsigned hh = R - t * (unsigned)H;
      const unsigned bb = t / (unsigned)Sq_pad;
      const unsigned qi = t - bb * (unsigned)Sq_pad;
      bh[it] = bb * (unsigned)H + hh;
      qv[it] = qi;
      state[it] = qi < (unsigned)Sq ? 2 : 1;
      if (qi < (unsigned)Sq) {
        av[it] = *reinterpret_cast<const uint4*>(o + (long long)bb * o_bs + (long long)qi * ldo + hh * 128 + l16 * 8);
        dv[it] = *reinterpret_cast<const uint4*>(dout + (long long)bb * do_bs + (long long)qi * lddo + hh * 128 + l16 * 8);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const uint32_t* au = reinterpret_cast<const uint32_t*>(&av[it]);
    const uint32_t* du = reinterpret_cast<const uint32_t*>(&dv[it]);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16(au[j]), d = unpack_bf16(du[j]);
      s += a.x * d.x + a.y * d.y;
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (l16 == 0 && state[it] != 0) {
      const long long oi = (long long)bh[it] * Sq_pad + qv[it];
      if (state[it] == 1) {
        delta[oi] = 0.f;
        lse2[oi] = 1.0e30f;
      } else {
        delta[oi] = s;
        lse2[oi] = lse[(long long)bh[it] * Sq + qv[it]] * LOG2E;
      }
    }
  }
}

int make_map(CUtensorMap* tm, const void* ptr, long long ld, long long bs, int S, int H, int B, int rows) {
  uint64_t dims[3] = {(uint64_t)H * 128, (uint64_t)S, (uint64_t)B};
  uint64_t str[2] = {(uint64_t)ld * 2, (uint64_t)bs * 2};
  uint32_t box[3] = {64, (uint32_t)rows, 1};
  return tt_make_tmap(tm, ptr, 2, 3, dims, str, box, 1);
}

}  // namespace

// All tensors [B, S, H, 128] views (token stride ld*, batch stride *_bs, in elements).
// lse: fp32 [B,H,Sq] from the forward pass. scratch: fp32 [2, B, H, Sq_pad] with
// Sq_pad = Sq rounded up to 128 (tt_attn_bwd_scratch_floats gives the element count).
TT_API long long tt_attn_bwd_scratch_floats(int B, int H, int Sq) {
  return 2ll * B * H * ((Sq + 127) / 128 * 128);
}

static int attn_bwd_impl(const void* q, long long ldq, long long q_bs, const void* k, long long ldk,
                       long long k_bs, const void* v, long long ldv, long long v_bs, const void* o,
                       long long ldo, long long o_bs, const void* dout, long long lddo, long long do_bs,
                       const float* lse, float* scratch, void* dq, long long lddq, long long dq_bs,
                       void* dk, long long lddk, long long dk_bs, void* dv, long long lddv,
                       long long dv_bs, const int* kv_lens, int B, int H, int Sq, int Skv, int D,
                       float scale, unsigned* status, const TTScatter* scq, const TTScatter* sck,
                       const TTScatter* scv, cudaStream_t stream) {
  TT_CHECK(D == 128, "attn_bwd: head_dim must be 128 (got %d)", D);
  TT_CHECK(B > 0 && H > 0 && Sq > 0 && Skv > 0, "attn_bwd: empty problem");
  const long long lds[] = {ldq, ldk, ldv, ldo, lddo, lddq, lddk, lddv, q_bs, k_bs, v_bs, o_bs, do_bs, dq_bs, dk_bs, dv_bs};
  for (long long x : lds) TT_CHECK(x % 8 == 0, "attn_bwd: strides must be multiples of 8 elements");
  TT_CHECK((((uintptr_t)q | (uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv | (uintptr_t)o | (uintptr_t)dout) & 15) == 0,
           "attn_bwd: misaligned pointer");
  TT_CHECK(scq != nullptr || (dq && dk && dv), "attn_bwd: output pointers missing");
  TT_CHECK(((uintptr_t)scratch & 15) == 0, "attn_bwd: scratch misaligned");
  const int Sq_pad = (Sq + 127) / 128 * 128;
  float* lse2 = scratch;
  float* delta = scratch + (long long)B * H * Sq_pad;
  {
    TT_CHECK((long long)B * Sq_pad * H < (1ll << 31), "attn_bwd: too many (batch, token, head) rows");
    const long long warps = ((long long)B * Sq_pad * H + 7) / 8;  // eight rows per warp
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    attn_preprocess_kernel<<<(unsigned)blocks, threads, 0, stream>>>(
        (const bf16*)o, ldo, o_bs, (const bf16*)dout, lddo, do_bs, lse, lse2, delta, B, H, Sq, Sq_pad);
    TT_LAUNCH_CHECK();
  }
  BwdParams p;
  p.Sq = Sq; p.Skv = Skv; p.H = H; p.B = B; p.Sq_pad = Sq_pad;
  p.scale = scale; p.scale_log2 = scale * LOG2E;
  p.lse2 = lse2; p.delta = delta; p.kv_lens = kv_lens; p.status = status;
  memset(&p.sc0, 0, sizeof(p.sc0));
  memset(&p.sc1, 0, sizeof(p.sc1));
  static bool attr_done = false;
  if (!attr_done) {
    TT_CUDA(cudaFuncSetAttribute(attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A_SMEM));
    TT_CUDA(cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, B_SMEM));
    attr_done = true;
  }
  CUtensorMap tmQ, tmK, tmV, tmdO;  // boxes of 128 rows x 64 columns for both kernels
  if (make_map(&tmQ, q, ldq, q_bs, Sq, H, B, 128)) return -1;
  if (make_map(&tmdO, dout, lddo, do_bs, Sq, H, B, 128)) return -1;
  if (make_map(&tmK, k, ldk, k_bs, Skv, H, B, 128)) return -1;
  if (make_map(&tmV, v, ldv, v_bs, Skv, H, B, 128)) return -1;
  {
    p.out0 = (bf16*)dk; p.ld0 = lddk; p.bs0 = dk_bs;
    p.out1 = (bf16*)dv; p.ld1 = lddv; p.bs1 = dv_bs;
    if (sck) p.sc0 = *sck;
    if (scv) p.sc1 = *scv;
    dim3 grid((Skv + 127) / 128, H, B);
    attn_bwd_dkdv_kernel<<<grid, NTHREADS, A_SMEM, stream>>>(tmQ, tmK, tmV, tmdO, p);
    TT_LAUNCH_CHECK();
  }
  {
    p.out0 = (bf16*)dq; p.ld0 = lddq; p.bs0 = dq_bs;
    p.out1 = nullptr; p.ld1 = 0; p.bs1 = 0;
    memset(&p.sc0, 0, sizeof(p.sc0));
    memset(&p.sc1, 0, sizeof(p.sc1));
    if (scq) p.sc0 = *scq;
    dim3 grid((Sq + 127) / 128, H, B);
    attn_bwd_dq_kernel<<<grid, NTHREADS, B_SMEM, stream>>>(tmQ, tmK, tmV, tmdO, p);
    TT_LAUNCH_CHECK();
  }
  return 0;
}

TT_API int tt_attn_bwd(const void* q, long long ldq, long long q_bs, const void* k, long long ldk,
                       long long k_bs, const void* v, long long ldv, long long v_bs, const void* o,
                       long long ldo, long long o_bs, const void* dout, long long lddo, long long do_bs,
                       const float* lse, float* scratch, void* dq, long long lddq, long long dq_bs,
                       void* dk, long long lddk, long long dk_bs, void* dv, long long lddv,
                       long long dv_bs, const int* kv_lens, int B, int H, int Sq, int Skv, int D,
                       float scale, unsigned* status, cudaStream_t stream) {
  return attn_bwd_impl(q, ldq, q_bs, k, ldk, k_bs, v, ldv, v_bs, o, ldo, o_bs, dout, lddo, do_bs, lse, scratch,
                       dq, lddq, dq_bs, dk, lddk, dk_bs, dv, lddv, dv_bs, kv_lens, B, H, Sq, Skv, D, scale,
                       status, nullptr, nullptr, nullptr, stream);
}

// Backward over head-parallel tensors [B, S_total, Hl, D]; dQ, dK, dV of the first S_pad rows of every sample are
// stored with the Ulysses head -> seq pattern into every peer's [B, S_l, H_total, D] buffers (three peer tables) whose
// token stride is `dst_ld` elements (0 = H_total * D; larger when the three are column blocks of one
// [rows, 3 * H_total * D] matrix).  Rows S_pad .. S_total (the replicated text tokens of a joint sequence; none when
// S_total == S_pad) stay local: their dQ / dK / dV go to `dq_local` / `dk_local` / `dv_local` ([B, S_total, Hl, D],
// may be null when there are none).  `heads` <= Hl of this rank's head slots hold real heads; lse and scratch are
// sized for `heads` and S_total.
TT_API int tt_attn_bwd_scatter(const void* q, const void* k, const void* v, const void* o, const void* dout,
                               const float* lse, float* scratch, const long long* dq_peers,
                               const long long* dk_peers, const long long* dv_peers, long long dst_ld,
                               void* dq_local, void* dk_local, void* dv_local, const int* kv_lens, int B, int Hl,
                               int heads, int H_total, int S_pad, int S_total, int D, float scale, int world,
                               int rank, unsigned* status, cudaStream_t stream) {
  TT_CHECK(world >= 1 && world <= TT_MAX_PEERS && rank >= 0 && rank < world, "attn_bwd_scatter: bad world/rank");
  TT_CHECK(S_pad % world == 0 && S_total >= S_pad, "attn_bwd_scatter: padded sequence must divide by the group size");
  TT_CHECK(heads >= 1 && heads <= Hl && rank * Hl + heads <= H_total && H_total <= Hl * world,
           "attn_bwd_scatter: head slots do not match the head count");
  TT_CHECK(dst_ld == 0 || (dst_ld >= (long long)H_total * D && dst_ld % 8 == 0), "attn_bwd_scatter: bad destination stride");
  TT_CHECK(S_total == S_pad || (dq_local && dk_local && dv_local), "attn_bwd_scatter: rows that stay local need local outputs");
  TTScatter sc[3];
  const long long* tabs[3] = {dq_peers, dk_peers, dv_peers};
  for (int t = 0; t < 3; ++t) {
    memset(&sc[t], 0, sizeof(TTScatter));
    for (int i = 0; i < world; ++i) {
      sc[t].peer[i] = reinterpret_cast<void*>(tabs[t][i]);
      TT_CHECK(sc[t].peer[i] && ((uintptr_t)sc[t].peer[i] & 15) == 0, "attn_bwd_scatter: bad peer pointer");
    }
    sc[t].mode = 2; sc[t].S_l = S_pad / world; sc[t].S_pad = S_pad; sc[t].Hl = Hl; sc[t].H = H_total;
    sc[t].D = D; sc[t].rank = rank; sc[t].world = world; sc[t].ld = dst_ld; sc[t].n_rows = S_pad;
  }
  const long long ld = (long long)Hl * D, bs = (long long)S_total * Hl * D;
  // without local rows the local output pointers are never used; q is an aligned placeholder then
  void* lq = dq_local ? dq_local : const_cast<void*>(q);
  void* lk = dk_local ? dk_local : const_cast<void*>(q);
  void* lv = dv_local ? dv_local : const_cast<void*>(q);
  return attn_bwd_impl(q, ld, bs, k, ld, bs, v, ld, bs, o, ld, bs, dout, ld, bs, lse, scratch, lq, ld, bs, lk, ld, bs,
                       lv, ld, bs, kv_lens, B, heads, S_total, S_total, D, scale, status, &sc[0], &sc[1], &sc[2], stream);
}
