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

// Geometry of one region of the flat parameter / gradient buffers cut into uniform buckets.  Rank r owns the r-th
// `share` of every bucket; its optimizer state is the concatenation of those shares ("owned-flat" order):
//   bucket b, element k of the share  ->  owned-flat  b * share + k
//                                     ->  global      region_start + b * bucket_elems + rank * share_b + k
// where share = bucket_elems / world and the last bucket may be shorter (share_last).
struct BucketGeom {
  long long region_start, bucket_elems, share, share_last;
  int n_buckets, world, rank;
};

template <bool ADAM, bool REDUCE>
__global__ void __launch_bounds__(256)
dp_bucket_kernel(PeerPtrs grads, PeerPtrs params16, BucketGeom geo, int b0, int b1,
                 float* __restrict__ reduced, float* __restrict__ master, float* __restrict__ m,
                 float* __restrict__ v, float grad_scale, const float* __restrict__ clip_coef,
                 const float* __restrict__ ss_slots, float clip_grad, float* __restrict__ norm_out, float lr,
                 float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                 float* __restrict__ sumsq_partial) {
  __shared__ float red[8];
  float ss = 0.f;
  float gs = 1.f;
  if (ADAM) {
    gs = grad_scale;
    if (clip_coef) {
      gs *= *clip_coef;
    } else if (ss_slots) {  // every rank sums the same values in the same order: identical coefficient everywhere
      float tot = 0.f;
      for (int r = 0; r < geo.world; ++r) tot += ss_slots[r];
      const float norm = sqrtf(tot) * grad_scale;
      if (clip_grad > 0.f) gs *= fminf(1.f, clip_grad / (norm + 1e-6f));
      if (norm_out && blockIdx.x == 0 && threadIdx.x == 0) *norm_out = norm;
    }
  }
  for (int b = b0; b < b1; ++b) {
    const long long share_b = (b == geo.n_buckets - 1) ? geo.share_last : geo.share;
    const long long flat0 = (long long)b * geo.share;
    const long long glob0 = geo.region_start + (long long)b * geo.bucket_elems + (long long)geo.rank * share_b;
    const long long nv = share_b >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
      const long long off = glob0 + i * 4;
      const long long fl = (flat0 >> 2) + i;
      float4 g;
      if (REDUCE) {
        g = ld4(reinterpret_cast<const float*>(grads.p[0]) + off);
        for (int r = 1; r < geo.world; ++r) {
          const float4 t = ld4(reinterpret_cast<const float*>(grads.p[r]) + off);
          g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
        }
        ss += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
        // the sum replaces this rank's own copy of its share (nobody else reads that part of this rank's buffer),
        // or goes to a separate owned-flat buffer when the caller gave one
        if (reduced) reinterpret_cast<float4*>(reduced)[fl] = g;
        else if (!ADAM) *reinterpret_cast<float4*>(reinterpret_cast<float*>(grads.p[geo.rank]) + off) = g;
      } else {
        g = reduced ? reinterpret_cast<const float4*>(reduced)[fl]
                    : ld4(reinterpret_cast<const float*>(grads.p[geo.rank]) + off);
      }
      if (ADAM) {
        float4 pp = reinterpret_cast<float4*>(master)[fl];
        float4 mm = reinterpret_cast<float4*>(m)[fl];
        float4 vv = reinterpret_cast<float4*>(v)[fl];
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
        reinterpret_cast<float4*>(master)[fl] = make_float4(P[0], P[1], P[2], P[3]);
        reinterpret_cast<float4*>(m)[fl] = make_float4(M[0], M[1], M[2], M[3]);
        reinterpret_cast<float4*>(v)[fl] = make_float4(V[0], V[1], V[2], V[3]);
        uint2 o;
        o.x = pack_bf16(P[0], P[1]);
        o.y = pack_bf16(P[2], P[3]);
        for (int r = 0; r < geo.world; ++r) {
          const int dst = (geo.rank + r) % geo.world;  // stagger destinations across ranks
          *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(params16.p[dst]) + off) = o;
        }
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

// Sum of `n` partial sums of squares in a fixed order (one CTA), stored into slot `rank` of every peer's
// slot array: after the barrier that follows, each rank holds every rank's share of the squared norm.
__global__ void __launch_bounds__(256)
dp_norm_exchange_kernel(const float* __restrict__ partials, int n, PeerPtrs slots, int world, int rank) {
  __shared__ float red[256];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) s += partials[i];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int w = 128; w > 0; w >>= 1) {
    if (threadIdx.x < w) red[threadIdx.x] += red[threadIdx.x + w];
    __syncthreads();
  }
  if (threadIdx.x < world) reinterpret_cast<float*>(slots.p[threadIdx.x])[rank] = red[0];
}

// dst[i] += float(src[i]) for up to FOLD_MAX small tensors in one launch (bf16 autograd gradients of biases,
// norm weights and modulation tables folded into the fp32 gradient buffer).
constexpr int FOLD_MAX = 48;
struct FoldTable {
  const bf16* src[FOLD_MAX];
  float* dst[FOLD_MAX];
  int n[FOLD_MAX];
};
__global__ void __launch_bounds__(256) multi_fold_kernel(FoldTable t) {
  const int k = blockIdx.y;
  const bf16* __restrict__ s = t.src[k];
  float* __restrict__ d = t.dst[k];
  const int n = t.n[k];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    d[i] += __bfloat162float(s[i]);
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

// One region of the flat buffers cut into `n_buckets` uniform buckets of `bucket_elems` elements (the last one
// `last_elems` long); works on buckets [b0, b1).
//   mode 0: pull-reduce each owned share from every peer + sum-of-squares partials; the sum goes to `reduced`
//           (owned-flat order) or, when `reduced` is null, over this rank's own copy of the share in its gradient buffer
//   mode 1: AdamW from `reduced` (or from that in-place sum) + bf16 parameter store into every peer
//   mode 2: both in one pass (no global-norm clipping)
// The clip coefficient is `*clip_coef` when given; otherwise, when `ss_slots` is given, the kernel sums that array's
// `world` entries (every rank's share of the squared norm, see tt_dp_norm_exchange), writes the norm to `norm_out`
// and clips to `clip_grad`.  `blocks` CTAs (0 = the default of tt_comm_blocks()); `sumsq_partial` takes one float
// per CTA.
TT_API int tt_dp_bucket_step(int mode, const long long* grad_ptrs, const long long* param_ptrs, int world, int rank,
                             long long region_start, long long bucket_elems, long long last_elems, int n_buckets,
                             int b0, int b1, float* reduced, float* master, float* m, float* v, float grad_scale,
                             const float* clip_coef, const float* ss_slots, float clip_grad, float* norm_out,
                             float lr, float beta1, float beta2, float eps, float wd, int step,
                             float* sumsq_partial, int blocks, cudaStream_t stream) {
  TT_CHECK(world >= 1 && n_buckets >= 1 && b0 >= 0 && b0 < b1 && b1 <= n_buckets, "dp_bucket_step: bad bucket range");
  TT_CHECK(bucket_elems > 0 && bucket_elems % (4ll * world) == 0 && last_elems > 0 && last_elems <= bucket_elems &&
               last_elems % (4ll * world) == 0 && region_start % 4 == 0,
           "dp_bucket_step: buckets must split into 16-byte aligned shares");
  PeerPtrs g, p;
  if (mode != 1 || reduced == nullptr) {
    if (fill_peers(&g, grad_ptrs, world)) return -1;
  } else {
    for (int i = 0; i < MAX_PEERS; ++i) g.p[i] = nullptr;
  }
  if (mode != 0) {
    if (fill_peers(&p, param_ptrs, world)) return -1;
    TT_CHECK(master && m && v && step >= 1, "dp_bucket_step: optimizer state missing");
  } else {
    for (int i = 0; i < MAX_PEERS; ++i) p.p[i] = nullptr;
  }
  BucketGeom geo{region_start, bucket_elems, bucket_elems / world, last_elems / world, n_buckets, world, rank};
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  if (blocks <= 0) blocks = tt_comm_blocks();
#define TT_DP_ARGS g, p, geo, b0, b1, reduced, master, m, v, grad_scale, clip_coef, ss_slots, clip_grad, norm_out, lr, beta1, beta2, eps, wd, bc1, bc2, sumsq_partial
  if (mode == 0)
    dp_bucket_kernel<false, true><<<blocks, 256, 0, stream>>>(TT_DP_ARGS);
  else if (mode == 1)
    dp_bucket_kernel<true, false><<<blocks, 256, 0, stream>>>(TT_DP_ARGS);
  else
    dp_bucket_kernel<true, true><<<blocks, 256, 0, stream>>>(TT_DP_ARGS);
#undef TT_DP_ARGS
  TT_LAUNCH_CHECK();
  return 0;
}

// Sums `n` partial sums of squares and stores the result into element `rank` of every peer's slot array
// (`slot_ptrs`: one fp32[>= world] array per rank in symmetric memory).
TT_API int tt_dp_norm_exchange(const float* partials, int n, const long long* slot_ptrs, int world, int rank,
                               cudaStream_t stream) {
  TT_CHECK(partials != nullptr && n > 0, "dp_norm_exchange: no partial sums");
  PeerPtrs s;
  if (fill_peers(&s, slot_ptrs, world)) return -1;
  TT_CHECK(rank >= 0 && rank < world, "dp_norm_exchange: bad rank");
  dp_norm_exchange_kernel<<<1, 256, 0, stream>>>(partials, n, s, world, rank);
  TT_LAUNCH_CHECK();
  return 0;
}

TT_API int tt_multi_fold_max() { return FOLD_MAX; }

// dst[k][i] += float(src[k][i]) for `count` tensors (bf16 sources, fp32 destinations, n[k] elements each).
TT_API int tt_multi_fold(const long long* src, const long long* dst, const int* n, int count, cudaStream_t stream) {
  TT_CHECK(count >= 1 && count <= FOLD_MAX, "multi_fold: between 1 and %d tensors per call", FOLD_MAX);
  FoldTable t;
  int mx = 0;
  for (int k = 0; k < count; ++k) {
    TT_CHECK(src[k] != 0 && dst[k] != 0 && n[k] > 0, "multi_fold: empty entry %d", k);
    t.src[k] = reinterpret_cast<const bf16*>(src[k]);
    t.dst[k] = reinterpret_cast<float*>(dst[k]);
    t.n[k] = n[k];
    mx = n[k] > mx ? n[k] : mx;
  }
  int bx = (mx + 255) / 256;
  if (bx > 64) bx = 64;
  multi_fold_kernel<<<dim3(bx, count), 256, 0, stream>>>(t);
  TT_LAUNCH_CHECK();
  return 0;
}
