// Kernel-initiated communication over NVLink peer memory (one process per GPU; every rank maps
// every peer's symmetric buffers into its own address space).
//
//   peer_barrier      cross-GPU barrier: release-store an epoch into each peer's flag row, then
//                     acquire-spin (bounded) until every peer's epoch has arrived here.
//   rs_reduce         K-DP-RS-ADAMW, pass 1: pull this rank's shard of the gradient buffer from every
//                     peer (plain P2P loads), sum in fp32 in rank order (deterministic, identical
//                     on all ranks), write it to the local shard and emit sum-of-squares partials.
//   adamw_scatter     pass 2: AdamW on the owned shard (fp32 master, m, v) and P2P-store the new
//                     bf16 parameters into every peer's parameter buffer (the all-gather).
//   rs_adamw_scatter  both passes in one kernel when no global-norm clipping is needed.
//
// Together they replace the gradient all-reduce through a staging copy, apex FusedAdam and the
// parameter all-gather of the reference (teletron/core/distributed/param_and_grad_buffer.py:128-152,
// teletron/train/lr_scheduler.py:466-489).  Reductions are ordinary per-thread loads from
// peer pointers.  Spin waits are bounded and report through the status
// word instead of hanging.
#include "tt_common.cuh"

using namespace tt;

namespace {

constexpr int MAX_PEERS = 16;

struct PeerPtrs {
  void* p[MAX_PEERS];
};

__device__ __forceinline__ void st_release_sys(unsigned* addr, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* addr) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// flags: each rank owns unsigned[MAX_PEERS * slots]; row `slot` column r is written by rank r.
// One thread per peer. epoch must increase by one per use of a slot.
__global__ void peer_barrier_kernel(PeerPtrs flags, int world, int rank, int slot, unsigned epoch,
                                    long long budget_clocks, unsigned* status) {
  const int p = threadIdx.x;
  if (p >= world) return;
  __threadfence_system();
  unsigned* remote = reinterpret_cast<unsigned*>(flags.p[p]) + slot * MAX_PEERS + rank;
  st_release_sys(remote, epoch);
  const unsigned* mine = reinterpret_cast<const unsigned*>(flags.p[rank]) + slot * MAX_PEERS + p;
  const long long t0 = clock64();
  // epochs wrap: compare as a signed distance
  while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
    if (clock64() - t0 > budget_clocks) {
      if (status) atomicCAS(status, 0u, (unsigned)(TT_ST_TIMEOUT_PEER + p));
      return;
    }
    __nanosleep(200);
  }
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }

template <bool ADAM, bool REDUCE>
__global__ void __launch_bounds__(256)
dp_shard_kernel(PeerPtrs grads, PeerPtrs params16, int world, int rank, long long shard_start,
                long long shard_len, float* __restrict__ reduced, float* __restrict__ master,
                float* __restrict__ m, float* __restrict__ v, float grad_scale,
                const float* __restrict__ clip_coef, float lr, float beta1, float beta2, float eps,
                float wd, float bc1, float bc2, float* __restrict__ sumsq_partial) {
  __shared__ float red[8];
  const long long nv = shard_len >> 2;
  float ss = 0.f;
  const float gs = ADAM ? grad_scale * (clip_coef ? *clip_coef : 1.f) : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const long long off = shard_start + i * 4;
    float4 g;
    if (REDUCE) {
      g = ld4(reinterpret_cast<const float*>(grads.p[0]) + off);
      for (int r = 1; r < world; ++r) {
        const float4 t = ld4(reinterpret_cast<const float*>(grads.p[r]) + off);
        g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
      }
      ss += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
      if (reduced) reinterpret_cast<float4*>(reduced)[i] = g;
    } else {
      g = reinterpret_cast<const float4*>(reduced)[i];
    }
    if (ADAM) {
      float4 pp = reinterpret_cast<float4*>(master)[i];
      float4 mm = reinterpret_cast<float4*>(m)[i];
      float4 vv = reinterpret_cast<float4*>(v)[i];
      float P[4] = {pp.x, pp.y, pp.z, pp.w}, M[4] = {mm.x, mm.y, mm.z, mm.w};
      float V[4] = {vv.x, vv.y, vv.z, vv.w};
      const float G[4] = {g.x * gs, g.y * gs, g.z * gs, g.w * gs};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        M[j] = beta1 * M[j] + (1.f - beta1) * G[j];
        V[j] = beta2 * V[j] + (1.f - beta2) * G[j] * G[j];
        const float mh = M[j] / bc1, vh = V[j] / bc2;
        P[j] = P[j] - lr * (mh / (sqrtf(vh) + eps) + wd * P[j]);
      }
      reinterpret_cast<float4*>(master)[i] = make_float4(P[0], P[1], P[2], P[3]);
      reinterpret_cast<float4*>(m)[i] = make_float4(M[0], M[1], M[2], M[3]);
      reinterpret_cast<float4*>(v)[i] = make_float4(V[0], V[1], V[2], V[3]);
      uint2 o;
      o.x = pack_bf16(P[0], P[1]);
      o.y = pack_bf16(P[2], P[3]);
      for (int r = 0; r < world; ++r) {
        const int dst = (rank + r) % world;  // stagger destinations across ranks
        *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(params16.p[dst]) + off) = o;
      }
    }
  }
  if (REDUCE && sumsq_partial) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < 8; ++i) t += red[i];
      sumsq_partial[blockIdx.x] = t;
    }
  }
}

int fill_peers(PeerPtrs* out, const long long* ptrs, int world) {
  TT_CHECK(world >= 1 && world <= MAX_PEERS, "peer count %d out of range (max %d)", world, MAX_PEERS);
  for (int i = 0; i < MAX_PEERS; ++i) out->p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  for (int i = 0; i < world; ++i) TT_CHECK(out->p[i] != nullptr && ((uintptr_t)out->p[i] & 15) == 0, "peer pointer %d is null or misaligned", i);
  return 0;
}

}  // namespace

TT_API int tt_comm_max_peers() { return MAX_PEERS; }
TT_API int tt_comm_blocks() { return 148 * 4; }

// flag_ptrs: host array of `world` device addresses (each rank's flag buffer, >= MAX_PEERS*slots u32,
// zero-initialised once). timeout_ms bounds the wait.
TT_API int tt_peer_barrier(const long long* flag_ptrs, int world, int rank, int slot, unsigned epoch,
                           int timeout_ms, unsigned* status, cudaStream_t stream) {
  PeerPtrs f;
  if (fill_peers(&f, flag_ptrs, world)) return -1;
  TT_CHECK(rank >= 0 && rank < world && slot >= 0, "peer_barrier: bad rank/slot");
  const long long budget = (long long)(timeout_ms > 0 ? timeout_ms : 2000) * 2000000ll;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(f, world, rank, slot, epoch, budget, status);
  TT_LAUNCH_CHECK();
  return 0;
}

// mode 0: reduce only (writes `reduced`, sumsq partials); 1: AdamW from `reduced` + scatter;
// 2: reduce + AdamW + scatter in one pass (no clipping: clip_coef may still be given if known).
TT_API int tt_dp_shard_step(int mode, const long long* grad_ptrs, const long long* param_ptrs, int world,
                            int rank, long long shard_start, long long shard_len, float* reduced,
                            float* master, float* m, float* v, float grad_scale, const float* clip_coef,
                            float lr, float beta1, float beta2, float eps, float wd, int step,
                            float* sumsq_partial, cudaStream_t stream) {
  TT_CHECK(shard_len > 0 && shard_len % 4 == 0 && shard_start % 4 == 0, "dp_shard_step: shard must be 16-byte aligned");
  PeerPtrs g, p;
  if (mode != 1) {
    if (fill_peers(&g, grad_ptrs, world)) return -1;
  } else {
    for (int i = 0; i < MAX_PEERS; ++i) g.p[i] = nullptr;
  }
  if (mode != 0) {
    if (fill_peers(&p, param_ptrs, world)) return -1;
    TT_CHECK(master && m && v && step >= 1, "dp_shard_step: optimizer state missing");
  } else {
    for (int i = 0; i < MAX_PEERS; ++i) p.p[i] = nullptr;
  }
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  const int blocks = tt_comm_blocks();
  if (mode == 0)
    dp_shard_kernel<false, true><<<blocks, 256, 0, stream>>>(g, p, world, rank, shard_start, shard_len, reduced, master, m, v, grad_scale, clip_coef, lr, beta1, beta2, eps, wd, bc1, bc2, sumsq_partial);
  else if (mode == 1)
    dp_shard_kernel<true, false><<<blocks, 256, 0, stream>>>(g, p, world, rank, shard_start, shard_len, reduced, master, m, v, grad_scale, clip_coef, lr, beta1, beta2, eps, wd, bc1, bc2, sumsq_partial);
  else
    dp_shard_kernel<true, true><<<blocks, 256, 0, stream>>>(g, p, world, rank, shard_start, shard_len, reduced, master, m, v, grad_scale, clip_coef, lr, beta1, beta2, eps, wd, bc1, bc2, sumsq_partial);
  TT_LAUNCH_CHECK();
  return 0;
}
