// K-ATTN backward for head_dim 128 on tcgen05 / TMEM, as two kernels without atomics
// (deterministic), plus the row-dot preprocess:
//
//   delta[b,h,q] = sum_d dO * O
//
//   attn_bwd_dkdv : one CTA owns 128 keys of one (batch, head) and walks the queries in
//                   tiles of 64.  Scores are produced transposed, S^T = K Q^T and
//                   dP^T = V dO^T (keys on tensor-memory lanes, thread <-> key row), so
//                   P^T and dS^T land in shared memory directly as K-major A operands of
//                   dV += P^T dO and dK += dS^T Q, whose B operands are the same Q / dO
//                   tiles read MN-major.  S^T / dP^T (2 x 64 columns each, double-buffered),
//                   dV and dK (128 columns each) fill the 512 columns of tensor memory.
//   attn_bwd_dq   : one CTA owns 128 queries and walks the keys in tiles of 64:
//                   S = Q K^T, dP = dO V^T, dS = P o (dP - delta), dQ += dS K.
//
// P is recomputed from the saved log-sum-exp.  Roles per CTA (192 threads): warp 0 TMA
// producer, warp 1 MMA issuer, warps 2..5 elementwise.  Every wait is bounded.
#include "tt_common.cuh"

using namespace tt;

namespace {

constexpr int NTHREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2..9 elementwise (two per lane quarter)
constexpr int BIG = 128 * 128 * 2;     // 128 x 128 bf16 tile (two 64-wide halves of 16 KB)
constexpr int BIG_HALF = 128 * 128;    // 128 rows x 128 B
constexpr int SMALL = 64 * 128 * 2;    // 64 x 128 bf16 tile (two halves of 8 KB)
constexpr int SMALL_HALF = 64 * 128;   // 64 rows x 128 B
constexpr int PT = 128 * 64 * 2;       // 128 x 64 bf16 tile (one 128-byte row per lane)
constexpr float LOG2E = 1.4426950408889634f;

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
constexpr int A_SM_K = 0;
constexpr int A_SM_V = A_SM_K + BIG;
constexpr int A_LST = 3;                        // load stages of (Q, dO, lse, delta): TMA latency stays hidden
constexpr int A_SM_Q = A_SM_V + BIG;            // A_LST stages of (Q, dO) 64-row tiles
constexpr int A_SM_P = A_SM_Q + A_LST * 2 * SMALL;  // 2 buffers of (P^T, dS^T)
constexpr int A_SM_LSE = A_SM_P + 2 * 2 * PT;   // A_LST x (64 lse + 64 delta) floats
constexpr int A_SM_BAR = A_SM_LSE + A_LST * 128 * 4;
constexpr int A_SMEM = A_SM_BAR + 128 + 1024;

__global__ void __launch_bounds__(NTHREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A_SM_BAR);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // 3
  uint64_t* qdo_empty = bars + 4;    // 3
  uint64_t* s_full = bars + 7;       // 2
  uint64_t* p_full = bars + 9;       // 2
  uint64_t* pds_free = bars + 11;    // 2
  uint64_t* done_bar = bars + 13;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* lse_s = reinterpret_cast<float*>(smem + A_SM_LSE);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv0 = blockIdx.x * 128;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int n_it = (p.Sq + 63) / 64;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < A_LST; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 8);
      mbar_init(&pds_free[i], 1);
    }
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
  // tensor-memory columns: S^T[2] 0,64 | dP^T[2] 128,192 | dV 256 | dK 384

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * BIG);
      for (int hf = 0; hf < 2; ++hf) {
        tma_load_3d(smem + A_SM_K + hf * BIG_HALF, &tmK, kv_full, h * 128 + hf * 64, kv0, b);
        tma_load_3d(smem + A_SM_V + hf * BIG_HALF, &tmV, kv_full, h * 128 + hf * 64, kv0, b);
      }
      for (int i = 0; i < n_it; ++i) {
        const int st = i % A_LST;
        if (!mbar_wait(&qdo_empty[st], ((i / A_LST) & 1) ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&qdo_full[st], 2 * SMALL + 512);
        uint8_t* dq_ = smem + A_SM_Q + st * 2 * SMALL;
        for (int hf = 0; hf < 2; ++hf) {
          tma_load_3d(dq_ + hf * SMALL_HALF, &tmQ, &qdo_full[st], h * 128 + hf * 64, i * 64, b);
          tma_load_3d(dq_ + SMALL + hf * SMALL_HALF, &tmdO, &qdo_full[st], h * 128 + hf * 64, i * 64, b);
        }
        const long long roff = ((long long)b * p.H + h) * p.Sq_pad + i * 64;
        bulk_load(lse_s + st * 128, p.lse2 + roff, 256, &qdo_full[st]);
        bulk_load(lse_s + st * 128 + 64, p.delta + roff, 256, &qdo_full[st]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(128, 64, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc(128, 128, 0, 1);
      const uint32_t k_base = smem_u32(smem + A_SM_K);
      const uint32_t v_base = smem_u32(smem + A_SM_V);
      const uint32_t q_base = smem_u32(smem + A_SM_Q);
      const uint32_t p_base = smem_u32(smem + A_SM_P);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 1);
      auto issue_sdp = [&](int i) -> bool {
        const int st = i & 1, ld = i % A_LST;
        if (!mbar_wait(&qdo_full[ld], (i / A_LST) & 1, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 2)) return false;
        tc_fence_after();
        const uint32_t qb = q_base + ld * 2 * SMALL;
        const uint32_t dob = qb + SMALL;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t offA = (ks >> 2) * BIG_HALF + (ks & 3) * 32;
          const uint32_t offB = (ks >> 2) * SMALL_HALF + (ks & 3) * 32;
          umma_ss(tmem_base + st * 64, umma_desc(k_base + offA, 16, 1024), umma_desc(qb + offB, 16, 1024),
                  idesc_s, ks != 0);
        }
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t offA = (ks >> 2) * BIG_HALF + (ks & 3) * 32;
          const uint32_t offB = (ks >> 2) * SMALL_HALF + (ks & 3) * 32;
          umma_ss(tmem_base + 128 + st * 64, umma_desc(v_base + offA, 16, 1024),
                  umma_desc(dob + offB, 16, 1024), idesc_s, ks != 0);
        }
        tc_commit(&s_full[st]);
        return true;
      };
      auto issue_dvdk = [&](int i) -> bool {
        const int st = i & 1, ld = i % A_LST;
        if (!mbar_wait(&p_full[st], (i >> 1) & 1, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 3)) return false;
        tc_fence_after();
        const uint32_t qb = q_base + ld * 2 * SMALL;
        const uint32_t dob = qb + SMALL;
        const uint32_t pb = p_base + st * 2 * PT;
        const uint32_t dsb = pb + PT;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem_base + 256, umma_desc(pb + ks * 32, 16, 1024),
                  umma_desc(dob + ks * 2048, SMALL_HALF, 1024), idesc_o, (i > 0 || ks != 0) ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem_base + 384, umma_desc(dsb + ks * 32, 16, 1024),
                  umma_desc(qb + ks * 2048, SMALL_HALF, 1024), idesc_o, (i > 0 || ks != 0) ? 1u : 0u);
        tc_commit(&pds_free[st]);
        tc_commit(&qdo_empty[ld]);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int i = 0; i < n_it && ok; ++i) {
        if (i + 1 < n_it) ok = issue_sdp(i + 1);
        if (ok) ok = issue_dvdk(i);
      }
      if (ok) tc_commit(done_bar);
    }
  } else {
    // ------------------------------------------------------------ elementwise warps
    const int q = warp & 3;
    const int wg = (warp - 2) >> 2;  // 0/1: which half of the 64 query columns (and of the output columns)
    const int r = q * 32 + lane;  // key row in the tile
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int sw = r & 7;
    bool ok = true;
    for (int i = 0; i < n_it; ++i) {
      const int st = i & 1, ld = i % A_LST;
      const float* ls = lse_s + ld * 128;
      const float* dl = ls + 64;
      if (!mbar_wait(&qdo_full[ld], (i / A_LST) & 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 4)) { ok = false; break; }
      if (!mbar_wait(&s_full[st], (i >> 1) & 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 1)) { ok = false; break; }
      if (!mbar_wait(&pds_free[st], ((i >> 1) & 1) ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 2)) { ok = false; break; }
      __syncwarp();
      tc_fence_after();
      uint8_t* prow = smem + A_SM_P + st * 2 * PT + r * 128;
      uint8_t* dsrow = prow + PT;
      {
        // this warp group's 32 of the 64 query columns
        uint32_t s[32], dp[32];
#ifdef TT_EXP_SKIP_TMEMLD
#pragma unroll
        for (int e = 0; e < 32; ++e) { s[e] = 0u; dp[e] = 0u; }
#else
        tmem_ld32(tmem_base + lane_addr + st * 64 + wg * 32, s);
        tmem_ld32(tmem_base + lane_addr + 128 + st * 64 + wg * 32, dp);
#endif
        float lv[32], dv_[32];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 a = *reinterpret_cast<const float4*>(ls + wg * 32 + e);
          const float4 d = *reinterpret_cast<const float4*>(dl + wg * 32 + e);
          lv[e] = a.x; lv[e + 1] = a.y; lv[e + 2] = a.z; lv[e + 3] = a.w;
          dv_[e] = d.x; dv_[e + 1] = d.y; dv_[e + 2] = d.z; dv_[e + 3] = d.w;
        }
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float pv[8], dv[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
#ifdef TT_EXP_SKIP_MATH
            pv[e] = __uint_as_float(s[g * 8 + e]);
            dv[e] = __uint_as_float(dp[g * 8 + e]);
#else
            pv[e] = fast_exp2(fmaf(__uint_as_float(s[g * 8 + e]), p.scale_log2, -lv[g * 8 + e]));
            dv[e] = pv[e] * (__uint_as_float(dp[g * 8 + e]) - dv_[g * 8 + e]);
#endif
          }
          uint4 a, d;
          a.x = pack_bf16(pv[0], pv[1]); a.y = pack_bf16(pv[2], pv[3]);
          a.z = pack_bf16(pv[4], pv[5]); a.w = pack_bf16(pv[6], pv[7]);
          d.x = pack_bf16(dv[0], dv[1]); d.y = pack_bf16(dv[2], dv[3]);
          d.z = pack_bf16(dv[4], dv[5]); d.w = pack_bf16(dv[6], dv[7]);
          const int chunk = wg * 4 + g;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ sw) << 4)) = a;
          *reinterpret_cast<uint4*>(dsrow + ((chunk ^ sw) << 4)) = d;
        }
      }
#ifndef TT_EXP_SKIP_FENCE
      fence_proxy_async_smem();
#endif
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[st]);
    }
    if (ok) ok = mbar_wait(done_bar, 0, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 3);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int row = kv0 + r;
      int kv_len = p.Skv;
      if (p.kv_lens) kv_len = min(max(p.kv_lens[b], 1), p.Skv);
      const bool live = row < kv_len;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {  // 0: dV, 1: dK
        bf16* dst;
        if (which == 0)
          dst = (p.sc1.mode == 2 && row < p.Skv) ? scatter_dst(p.sc1, b, row, h)
                                                 : p.out1 + (long long)b * p.bs1 + (long long)row * p.ld1 + h * 128;
        else
          dst = (p.sc0.mode == 2 && row < p.Skv) ? scatter_dst(p.sc0, b, row, h)
                                                 : p.out0 + (long long)b * p.bs0 + (long long)row * p.ld0 + h * 128;
        const float mul = which == 0 ? 1.f : p.scale;
#pragma unroll 1
        for (int c = wg * 2; c < wg * 2 + 2; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_base + lane_addr + 256 + which * 128 + c * 32, o);
          tmem_ld_wait();
          if (row < p.Skv) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 pk;
              const float m2 = live ? mul : 0.f;
              pk.x = pack_bf16(__uint_as_float(o[g * 8 + 0]) * m2, __uint_as_float(o[g * 8 + 1]) * m2);
              pk.y = pack_bf16(__uint_as_float(o[g * 8 + 2]) * m2, __uint_as_float(o[g * 8 + 3]) * m2);
              pk.z = pack_bf16(__uint_as_float(o[g * 8 + 4]) * m2, __uint_as_float(o[g * 8 + 5]) * m2);
              pk.w = pack_bf16(__uint_as_float(o[g * 8 + 6]) * m2, __uint_as_float(o[g * 8 + 7]) * m2);
              *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = pk;
            }
          }
          __syncwarp();
        }
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
constexpr int B_SM_Q = 0;
constexpr int B_SM_DO = B_SM_Q + BIG;
constexpr int B_LST = 4;                           // load stages of (K, V) 64-row tiles
constexpr int B_SM_KV = B_SM_DO + BIG;
constexpr int B_SM_DS = B_SM_KV + B_LST * 2 * SMALL;   // 2 buffers of dS (128 x 64)
constexpr int B_SM_BAR = B_SM_DS + 2 * PT;
constexpr int B_SMEM = B_SM_BAR + 256 + 1024;

__global__ void __launch_bounds__(NTHREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + B_SM_BAR);
  uint64_t* q_full = bars;           // 1
  uint64_t* kv_full = bars + 1;      // 4
  uint64_t* kv_empty = bars + 5;     // 4
  uint64_t* s_full = bars + 9;       // 2
  uint64_t* p_full = bars + 11;      // 2
  uint64_t* ds_free = bars + 13;     // 2
  uint64_t* done_bar = bars + 15;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 128;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  int kv_len = p.Skv;
  if (p.kv_lens) kv_len = min(max(p.kv_lens[b], 1), p.Skv);
  const int n_it = (kv_len + 63) / 64;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < B_LST; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 8);
      mbar_init(&ds_free[i], 1);
    }
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
  // tensor-memory columns: S[2] 0,64 | dP[2] 128,192 | dQ 256

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * BIG);
      for (int hf = 0; hf < 2; ++hf) {
        tma_load_3d(smem + B_SM_Q + hf * BIG_HALF, &tmQ, q_full, h * 128 + hf * 64, q0, b);
        tma_load_3d(smem + B_SM_DO + hf * BIG_HALF, &tmdO, q_full, h * 128 + hf * 64, q0, b);
      }
      for (int i = 0; i < n_it; ++i) {
        const int st = i % B_LST;
        if (!mbar_wait(&kv_empty[st], ((i / B_LST) & 1) ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&kv_full[st], 2 * SMALL);
        uint8_t* d_ = smem + B_SM_KV + st * 2 * SMALL;
        for (int hf = 0; hf < 2; ++hf) {
          tma_load_3d(d_ + hf * SMALL_HALF, &tmK, &kv_full[st], h * 128 + hf * 64, i * 64, b);
          tma_load_3d(d_ + SMALL + hf * SMALL_HALF, &tmV, &kv_full[st], h * 128 + hf * 64, i * 64, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(128, 64, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc(128, 128, 0, 1);
      const uint32_t q_base = smem_u32(smem + B_SM_Q);
      const uint32_t do_base = smem_u32(smem + B_SM_DO);
      const uint32_t kv_base = smem_u32(smem + B_SM_KV);
      const uint32_t ds_base = smem_u32(smem + B_SM_DS);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 1);
      auto issue_sdp = [&](int i) -> bool {
        const int st = i & 1, ld = i % B_LST;
        if (!mbar_wait(&kv_full[ld], (i / B_LST) & 1, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 2)) return false;
        tc_fence_after();
        const uint32_t kb = kv_base + ld * 2 * SMALL;
        const uint32_t vb = kb + SMALL;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t offA = (ks >> 2) * BIG_HALF + (ks & 3) * 32;
          const uint32_t offB = (ks >> 2) * SMALL_HALF + (ks & 3) * 32;
          umma_ss(tmem_base + st * 64, umma_desc(q_base + offA, 16, 1024), umma_desc(kb + offB, 16, 1024),
                  idesc_s, ks != 0);
        }
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t offA = (ks >> 2) * BIG_HALF + (ks & 3) * 32;
          const uint32_t offB = (ks >> 2) * SMALL_HALF + (ks & 3) * 32;
          umma_ss(tmem_base + 128 + st * 64, umma_desc(do_base + offA, 16, 1024),
                  umma_desc(vb + offB, 16, 1024), idesc_s, ks != 0);
        }
        tc_commit(&s_full[st]);
        return true;
      };
      auto issue_dq = [&](int i) -> bool {
        const int st = i & 1, ld = i % B_LST;
        if (!mbar_wait(&p_full[st], (i >> 1) & 1, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 3)) return false;
        tc_fence_after();
        const uint32_t kb = kv_base + ld * 2 * SMALL;
        const uint32_t dsb = ds_base + st * PT;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem_base + 256, umma_desc(dsb + ks * 32, 16, 1024),
                  umma_desc(kb + ks * 2048, SMALL_HALF, 1024), idesc_o, (i > 0 || ks != 0) ? 1u : 0u);
        tc_commit(&ds_free[st]);
        tc_commit(&kv_empty[ld]);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int i = 0; i < n_it && ok; ++i) {
        if (i + 1 < n_it) ok = issue_sdp(i + 1);
        if (ok) ok = issue_dq(i);
      }
      if (ok) tc_commit(done_bar);
    }
  } else {
    const int q = warp & 3;
    const int wg = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const int row = q0 + r;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int sw = r & 7;
    float lse2 = 1.0e30f, del = 0.f;
    if (row < p.Sq) {
      lse2 = p.lse2[((long long)b * p.H + h) * p.Sq_pad + row];
      del = p.delta[((long long)b * p.H + h) * p.Sq_pad + row];
    }
    bool ok = true;
    for (int i = 0; i < n_it; ++i) {
      const int st = i & 1;
      if (!mbar_wait(&s_full[st], (i >> 1) & 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 1)) { ok = false; break; }
      if (!mbar_wait(&ds_free[st], ((i >> 1) & 1) ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 2)) { ok = false; break; }
      __syncwarp();
      tc_fence_after();
      uint8_t* dsrow = smem + B_SM_DS + st * PT + r * 128;
      const int valid = kv_len - i * 64;
      {
        uint32_t s[32], dp[32];
        tmem_ld32(tmem_base + lane_addr + st * 64 + wg * 32, s);
        tmem_ld32(tmem_base + lane_addr + 128 + st * 64 + wg * 32, dp);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float dv[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = wg * 32 + g * 8 + e;
            float pe = fast_exp2(fmaf(__uint_as_float(s[g * 8 + e]), p.scale_log2, -lse2));
            if (col >= valid) pe = 0.f;
            dv[e] = pe * (__uint_as_float(dp[g * 8 + e]) - del);
          }
          uint4 d;
          d.x = pack_bf16(dv[0], dv[1]); d.y = pack_bf16(dv[2], dv[3]);
          d.z = pack_bf16(dv[4], dv[5]); d.w = pack_bf16(dv[6], dv[7]);
          const int chunk = wg * 4 + g;
          *reinterpret_cast<uint4*>(dsrow + ((chunk ^ sw) << 4)) = d;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[st]);
    }
    if (ok) ok = mbar_wait(done_bar, 0, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 3);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      bf16* dst = (p.sc0.mode == 2 && row < p.Sq) ? scatter_dst(p.sc0, b, row, h)
                                                  : p.out0 + (long long)b * p.bs0 + (long long)row * p.ld0 + h * 128;
#pragma unroll 1
      for (int c = wg * 2; c < wg * 2 + 2; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_base + lane_addr + 256 + c * 32, o);
        tmem_ld_wait();
        if (row < p.Sq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(o[g * 8 + 0]) * p.scale, __uint_as_float(o[g * 8 + 1]) * p.scale);
            pk.y = pack_bf16(__uint_as_float(o[g * 8 + 2]) * p.scale, __uint_as_float(o[g * 8 + 3]) * p.scale);
            pk.z = pack_bf16(__uint_as_float(o[g * 8 + 4]) * p.scale, __uint_as_float(o[g * 8 + 5]) * p.scale);
            pk.w = pack_bf16(__uint_as_float(o[g * 8 + 6]) * p.scale, __uint_as_float(o[g * 8 + 7]) * p.scale);
            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = pk;
          }
        }
        __syncwarp();
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

// ===================================================================== preprocess
// delta[b,h,q] = sum_d dO*O and lse2 = lse * log2(e), both written to [B,H,Sq_pad] buffers whose
// padding rows hold 0 / 1e30 (so padded queries get probability 0). One warp per (b, q, h).
__global__ void attn_preprocess_kernel(const bf16* __restrict__ o, long long ldo, long long o_bs,
                                       const bf16* __restrict__ dout, long long lddo, long long do_bs,
                                       const float* __restrict__ lse, float* __restrict__ lse2,
                                       float* __restrict__ delta, int B, int H, int Sq, int Sq_pad) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * Sq_pad * H;
  if (gw >= total) return;
  const int hh = (int)(gw % H);
  const long long t = gw / H;
  const int qi = (int)(t % Sq_pad);
  const int bb = (int)(t / Sq_pad);
  const long long oidx = ((long long)bb * H + hh) * Sq_pad + qi;
  if (qi >= Sq) {
    if (lane == 0) {
      delta[oidx] = 0.f;
      lse2[oidx] = 1.0e30f;
    }
    return;
  }
  const bf16* op = o + bb * o_bs + (long long)qi * ldo + hh * 128 + lane * 4;
  const bf16* dp = dout + bb * do_bs + (long long)qi * lddo + hh * 128 + lane * 4;
  uint2 a = *reinterpret_cast<const uint2*>(op);
  uint2 d = *reinterpret_cast<const uint2*>(dp);
  float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), d0 = unpack_bf16(d.x), d1 = unpack_bf16(d.y);
  float s = a0.x * d0.x + a0.y * d0.y + a1.x * d1.x + a1.y * d1.y;
  s = warp_sum(s);
  if (lane == 0) {
    delta[oidx] = s;
    lse2[oidx] = lse[((long long)bb * H + hh) * Sq + qi] * LOG2E;
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
// Sq_pad = Sq rounded up to 64 (tt_attn_bwd_scratch_floats gives the element count).
TT_API long long tt_attn_bwd_scratch_floats(int B, int H, int Sq) {
  return 2ll * B * H * ((Sq + 63) / 64 * 64);
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
  TT_CHECK((((uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv | (uintptr_t)o | (uintptr_t)dout) & 15) == 0,
           "attn_bwd: misaligned pointer");
  TT_CHECK(scq != nullptr || (dq && dk && dv), "attn_bwd: output pointers missing");
  TT_CHECK(((uintptr_t)scratch & 15) == 0, "attn_bwd: scratch misaligned");
  const int Sq_pad = (Sq + 63) / 64 * 64;
  float* lse2 = scratch;
  float* delta = scratch + (long long)B * H * Sq_pad;
  {
    const long long warps = (long long)B * Sq_pad * H;
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
  {
    CUtensorMap tmQ, tmK, tmV, tmdO;
    if (make_map(&tmQ, q, ldq, q_bs, Sq, H, B, 64)) return -1;
    if (make_map(&tmdO, dout, lddo, do_bs, Sq, H, B, 64)) return -1;
    if (make_map(&tmK, k, ldk, k_bs, Skv, H, B, 128)) return -1;
    if (make_map(&tmV, v, ldv, v_bs, Skv, H, B, 128)) return -1;
    p.out0 = (bf16*)dk; p.ld0 = lddk; p.bs0 = dk_bs;
    p.out1 = (bf16*)dv; p.ld1 = lddv; p.bs1 = dv_bs;
    if (sck) p.sc0 = *sck;
    if (scv) p.sc1 = *scv;
    dim3 grid((Skv + 127) / 128, H, B);
    attn_bwd_dkdv_kernel<<<grid, NTHREADS, A_SMEM, stream>>>(tmQ, tmK, tmV, tmdO, p);
    TT_LAUNCH_CHECK();
  }
  {
    CUtensorMap tmQ, tmK, tmV, tmdO;
    if (make_map(&tmQ, q, ldq, q_bs, Sq, H, B, 128)) return -1;
    if (make_map(&tmdO, dout, lddo, do_bs, Sq, H, B, 128)) return -1;
    if (make_map(&tmK, k, ldk, k_bs, Skv, H, B, 64)) return -1;
    if (make_map(&tmV, v, ldv, v_bs, Skv, H, B, 64)) return -1;
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

// Backward over head-parallel tensors [B, S_pad, Hl, D]; dQ, dK, dV are stored with the Ulysses
// head -> seq pattern into every peer's [B, S_l, H_total, D] buffers (three peer tables).
TT_API int tt_attn_bwd_scatter(const void* q, const void* k, const void* v, const void* o, const void* dout,
                               const float* lse, float* scratch, const long long* dq_peers,
                               const long long* dk_peers, const long long* dv_peers, const int* kv_lens,
                               int B, int Hl, int S_pad, int D, float scale, int world, int rank,
                               unsigned* status, cudaStream_t stream) {
  TT_CHECK(world >= 1 && world <= TT_MAX_PEERS && rank >= 0 && rank < world, "attn_bwd_scatter: bad world/rank");
  TT_CHECK(S_pad % world == 0, "attn_bwd_scatter: padded sequence must divide by the group size");
  TTScatter sc[3];
  const long long* tabs[3] = {dq_peers, dk_peers, dv_peers};
  for (int t = 0; t < 3; ++t) {
    memset(&sc[t], 0, sizeof(TTScatter));
    for (int i = 0; i < world; ++i) {
      sc[t].peer[i] = reinterpret_cast<void*>(tabs[t][i]);
      TT_CHECK(sc[t].peer[i] && ((uintptr_t)sc[t].peer[i] & 15) == 0, "attn_bwd_scatter: bad peer pointer");
    }
    sc[t].mode = 2; sc[t].S_l = S_pad / world; sc[t].S_pad = S_pad; sc[t].Hl = Hl; sc[t].H = Hl * world;
    sc[t].D = D; sc[t].rank = rank; sc[t].world = world;
  }
  const long long ld = (long long)Hl * D, bs = (long long)S_pad * Hl * D;
  // dq/dk/dv local pointers are unused in scatter mode; pass q as an aligned placeholder
  return attn_bwd_impl(q, ld, bs, k, ld, bs, v, ld, bs, o, ld, bs, dout, ld, bs, lse, scratch,
                       const_cast<void*>(q), ld, bs, const_cast<void*>(q), ld, bs, const_cast<void*>(q), ld, bs,
                       kv_lens, B, Hl, S_pad, S_pad, D, scale, status, &sc[0], &sc[1], &sc[2], stream);
}
