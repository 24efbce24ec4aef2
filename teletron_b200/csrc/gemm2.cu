// K-GEMM on CTA pairs: the same contract as gemm.cu (C = epilogue(alpha * A * B^T), either operand K-major or
// MN-major) with tcgen05.mma.cta_group::2.  A cluster of two CTAs owns a 256 x 256 output tile: each CTA loads its
// own 128 rows of A and one 128-row half of the B tile, the leader CTA's MMA thread issues 256 x 256 x 16
// instructions that read A from each CTA's shared memory and the two B halves from both, and each CTA's tensor
// memory receives its 128 rows of the accumulator.
//
// Why: with one CTA per 128 x 256 tile a 64-deep stage needs 48 KB of operand reads and 48 KB of TMA writes per 512
// clocks of tensor work, 192 B/clock against the 128 B/clock of shared memory, which caps the one-CTA kernel at about
// two thirds of the tensor peak (measured: 0.67 at K = 8960).  Here a stage is 32 KB per CTA: 128 B/clock.
//
// Roles per CTA (320 threads): warp 0 TMA producer (both CTAs; completions of both land on the leader's barrier),
// warp 1 allocates tensor memory (both CTAs) and issues the MMAs (leader only), warps 2..9 epilogue.  Stage-free and
// accumulator-ready signals reach both CTAs through tcgen05.commit with a CTA mask; the epilogue warps of both CTAs
// arrive on the leader's accumulator-free barrier.  Every wait is bounded.
#include "gemm_epilogue.cuh"

using namespace tt;
using namespace tt_gemm;

namespace {

// all-gather -> GEMM in this one kernel (K-AG-GEMM): the A operand is the concatenation of one row segment per rank.
// Two extra warps per CTA copy it, 128-row block by block, from the ranks' buffers (plain loads over NVLink for the
// remote segments) into a local gathered matrix `G`, and publish one flag per block; the TMA producer of a tile waits
// for the flags of its rows and then loads A from `G`.  Tiles are visited starting with the local segment, blocks are
// copied in the same order, so the remote rows arrive while the local rows are multiplied and every remote element
// crosses NVLink exactly once.  Rows inside the rank's own segment are loaded straight from where they are (a second
// tensor map), without waiting for anything; their copy into `G`, which stays behind for the weight-gradient GEMM,
// is made last.
struct AgParams {
  const bf16* src[TP_MAX];  // rank s's segment [seg_rows, K] (its own included)
  bf16* G;                  // [world * seg_rows, K]
  unsigned* flags;          // one per 128-row block of G; a block is complete when its flag equals `epoch`
  unsigned epoch;
  int seg_rows, n_blocks, rot_tiles;  // rot_tiles: first 256-row tile that holds local rows
  int local_row0;                     // first row of this rank's own segment in G
};

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// bounded wait for a block flag; false (and the abort flag raised) when it runs out
__device__ __forceinline__ bool flag_wait(const unsigned* f, unsigned epoch, volatile uint32_t* abort_flag,
                                          unsigned* status, unsigned code) {
  const long long t0 = clock64();
  unsigned v;
  while (true) {
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (v == epoch) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > TT_WAIT_BUDGET_CLOCKS) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0u, code);
      return false;
    }
    __nanosleep(100);
  }
}

constexpr int BN2 = 256;
constexpr int STAGES2 = 6;
constexpr int ROUND2 = 3;  // stages consumed per wait / commit round of the MMA thread
constexpr int B_HALF_BYTES = 128 * BK * 2;
constexpr int STAGE2_BYTES = A_BYTES + B_HALF_BYTES;  // 32 KB per CTA and stage
constexpr int SMEM2_BYTES = STAGES2 * STAGE2_BYTES + 256 + 1024;

template <int A_MN, int B_MN, bool AG>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(AG ? 384 : 320, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
             const AgParams ag, const __grid_constant__ CUtensorMap tmL) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES2 * STAGE2_BYTES);  // used in the leader only
  uint64_t* empty = full + STAGES2;   // both CTAs (tcgen05.commit with mask 0b11)
  uint64_t* tfull = empty + STAGES2;  // both CTAs
  uint64_t* tempty = tfull + 2;       // leader only: 8 local + 8 remote epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + BN2 - 1) / BN2;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;
  // row tile of the i-th tile this cluster visits: with the gathered A operand the local segment comes first
  auto tile_m = [&](int tile) { return AG ? (tile / tiles_n + ag.rot_tiles) % tiles_m : tile / tiles_n; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 16);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anybody signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const int m0 = tile_m(tile) * 2 * BM + (int)cta * BM;
        const int n0 = (tile % tiles_n) * BN2 + (int)cta * 128;  // this CTA's half of the B tile
        // rows that lie entirely inside this rank's own segment are read where they are (tmL), at once; the others
        // come from the gathered matrix once some CTA's copier warps have put them there
        const int l0 = m0 - ag.local_row0;
        const bool a_local = AG && l0 >= 0 && l0 + BM <= ag.seg_rows;
        if (AG && !a_local && m0 < p.M) {
          if (!flag_wait(ag.flags + m0 / BM, ag.epoch, abort_flag, p.status, TT_ST_TIMEOUT_PRODUCER + 2)) break;
          fence_proxy_async_all();  // the copy was written with ordinary stores, the TMA engine reads it
        }
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES2;
          const uint32_t ph = (it / STAGES2) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE2_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (cta == 0) mbar_expect_tx(&full[s], 2 * STAGE2_BYTES);  // both CTAs' copies count on the leader's barrier
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma2_load_2d(sa + i * 8192, &tmA, bar, m0 + i * 64, k0);
          } else if (a_local) {
            tma2_load_2d(sa, &tmL, bar, k0, l0);
          } else {
            tma2_load_2d(sa, &tmA, bar, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < 2; ++i) tma2_load_2d(sb + i * 8192, &tmB, bar, n0 + i * 64, k0);
          } else {
            tma2_load_2d(sb, &tmB, bar, k0, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = umma_idesc(2 * BM, BN2, A_MN, B_MN);
      constexpr uint32_t HI = umma_desc_hi(1024);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++tcount) {
        const int a = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty[a], aph ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 1)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN2;
        // several stages per round: the waits and commits between groups of MMAs are what lets the tensor pipe run
        // dry, so they are taken for 4 * ROUND2 MMAs at a time
        for (int kb = 0; kb < num_kb; kb += ROUND2) {
          const int n_st = (kb + ROUND2 <= num_kb) ? ROUND2 : num_kb - kb;
          int st[ROUND2];
          for (int u = 0; u < n_st; ++u, ++it) {
            st[u] = it % STAGES2;
            const uint32_t ph = (it / STAGES2) & 1;
            if (!mbar_wait(&full[st[u]], ph, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 2)) ok = false;
          }
          if (!ok) break;
          tc_fence_after();
          for (int u = 0; u < n_st; ++u) {
            const uint32_t a_base = smem_u32(smem + st[u] * STAGE2_BYTES);
            const uint32_t a_lo = umma_desc_lo(a_base, A_MN ? 8192 : 16);
            const uint32_t b_lo = umma_desc_lo(a_base + A_BYTES, B_MN ? 8192 : 16);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma2_ss_lo<HI, HI>(d_tmem, a_lo + k * ((A_MN ? 2048 : 32) >> 4), b_lo + k * ((B_MN ? 2048 : 32) >> 4),
                                  idesc, ((kb + u) | k) != 0 ? 1u : 0u);
          }
          for (int u = 0; u < n_st; ++u) tc_commit2(&empty[st[u]], 3);
        }
        if (ok) tc_commit2(&tfull[a], 3);
      }
    }
  } else if (AG && warp >= 10) {
    // ------------------------------------------------------------ copier warps (all-gather of the A operand)
    const int t = threadIdx.x - 320;          // 0..63
    const int vec_per_row = p.K >> 3;         // 16-byte vectors per row
    // remote blocks first, in the order the tiles need them (the block after the local segment, onwards, wrapping);
    // the local segment's blocks, which gate nothing, fill the gathered matrix last
    const int first_remote = min((ag.local_row0 + ag.seg_rows) / BM, ag.n_blocks - 1);
    for (int j = blockIdx.x; j < ag.n_blocks; j += gridDim.x) {
      const int blk = (j + first_remote) % ag.n_blocks;
      const int r0 = blk * BM;
      const int nrows = min(BM, p.M - r0);
      const long long nvec = (long long)nrows * vec_per_row;
      for (long long v0 = t; v0 < nvec; v0 += 64 * 8) {
        uint4 buf[8];
        long long dsts[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const long long v = v0 + (long long)u * 64;
          dsts[u] = -1;
          if (v < nvec) {
            const int row = r0 + (int)(v / vec_per_row);
            const int col = (int)(v % vec_per_row) << 3;
            const int seg = row / ag.seg_rows;
            buf[u] = *reinterpret_cast<const uint4*>(ag.src[seg] + (long long)(row - seg * ag.seg_rows) * p.K + col);
            dsts[u] = (long long)row * p.K + col;
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (dsts[u] >= 0) *reinterpret_cast<uint4*>(ag.G + dsts[u]) = buf[u];
      }
      __threadfence();
      asm volatile("bar.sync 1, 64;" ::: "memory");   // both copier warps have written and fenced their part
      if (t == 0) {
        fence_proxy_async_all();
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ag.flags + blk), "r"(ag.epoch) : "memory");
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    const int eg = (warp - 2) >> 2;
    const uint32_t tempty_leader0 = map_to_cta(smem_u32(&tempty[0]), 0);
    int tcount = 0;
    for (int tile = cluster_id; tile < num_tiles; tile += num_clusters, ++tcount) {
      const int a = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      if (!mbar_wait(&tfull[a], aph, abort_flag, p.status, TT_ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const int m0 = tile_m(tile) * 2 * BM + (int)cta * BM;
      const int n0 = (tile % tiles_n) * BN2;
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      bf16* c_row = reinterpret_cast<bf16*>(p.C) + (long long)row * p.ldc;
      if (p.tp_mode == 2 && row_ok) {
        // GEMM -> reduce-scatter: this row of partial sums goes to the rank that owns it, into this rank's slot
        // of that rank's staging buffer [world, seg_rows, ldc]
        const int seg = row / p.seg_rows;
        c_row = p.peer_c[seg] + ((long long)p.rank * p.seg_rows + (row - seg * p.seg_rows)) * p.ldc;
      }
      if (p.epi == EPI_QKV_A2A)
        epilogue_tile_qkv<BN2>(p, tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN2), eg, row, row_ok, n0);
      else
        epilogue_tile<BN2>(p, tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN2), eg, row, row_ok, c_row, n0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader0 + a * 8);
    }
  }

  // ------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner may still be reading this CTA's shared memory through the pair's MMAs
  if (warp == 1) tmem_dealloc2(tmem_base, 512);
}

template <int A_MN, int B_MN, bool AG = false>
int launch2(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int sms, cudaStream_t stream,
            const AgParams* agp = nullptr, const CUtensorMap* tmLp = nullptr) {
  auto kern = gemm2_kernel<A_MN, B_MN, AG>;
  constexpr int NT2 = AG ? 384 : 320;
  AgParams ag;
  memset(&ag, 0, sizeof(ag));
  if (agp) ag = *agp;
  static bool attr_done = false;
  if (!attr_done) {
    TT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES));
    attr_done = true;
  }
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN2 - 1) / BN2);
  // persistent: as many CTA pairs as can be resident at once (GPCs with an odd SM count leave an SM unpaired)
  static int max_clusters = 0;
  if (max_clusters == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms, 1, 1);
    cfg.blockDim = dim3(NT2, 1, 1);
    cfg.dynamicSmemBytes = SMEM2_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    TT_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    max_clusters = n > 0 ? n : 1;
  }
  int clusters = max_clusters < sms / 2 ? max_clusters : sms / 2;
  if (tiles < clusters) clusters = tiles;
  kern<<<2 * clusters, NT2, SMEM2_BYTES, stream>>>(tmA, tmB, p, ag, tmLp ? *tmLp : tmA);
  TT_LAUNCH_CHECK();
  return 0;
}

}  // namespace

// Same arguments as tt_gemm_bf16 (without the CTA cap); shapes outside the pair kernel's domain return -3 so that
// the caller can fall back: N must be at least 256 and a multiple of 8, bf16 or fp32 output.
TT_API int tt_gemm2_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* C,
                         long long ldc, int c_fp32, int M, int N, int K, const void* bias, int epi,
                         const void* residual, long long ldr, const float* gate, long long gate_ld,
                         int rows_per_gate, void* aux_out, float alpha, unsigned* status, cudaStream_t stream) {
  if (N < 256 || M < 256) return -3;
  TT_CHECK(M > 0 && N > 0 && K > 0 && N % 8 == 0, "gemm2: bad shape %d x %d x %d", M, N, K);
  TT_CHECK(lda % 8 == 0 && ldb % 8 == 0, "gemm2: lda/ldb must be multiples of 8 elements");
  TT_CHECK(ldc % (c_fp32 ? 4 : 8) == 0 && ((uintptr_t)C & 15) == 0, "gemm2: C misaligned");
  TT_CHECK(epi >= 0 && epi <= EPI_LAST, "gemm2: unknown epilogue %d", epi);
  if (epi == EPI_GATE_RES) {
    TT_CHECK(residual && gate && rows_per_gate > 0, "gemm2: gate/residual epilogue needs both tensors");
    TT_CHECK(ldr % 8 == 0 && gate_ld % 4 == 0 && (((uintptr_t)residual | (uintptr_t)gate) & 15) == 0,
             "gemm2: residual/gate misaligned");
  }
  if (bias) TT_CHECK(((uintptr_t)bias & 15) == 0, "gemm2: bias is not 16-byte aligned");
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    if (a_mn) { dims[0] = (uint64_t)M; dims[1] = (uint64_t)K; box[0] = 64; box[1] = 64; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = 64; box[1] = BM; }
    str[0] = (uint64_t)lda * 2;
    if (tt_make_tmap(&tmA, A, 2, 2, dims, str, box, 1)) return -1;
    if (b_mn) { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; box[0] = 64; box[1] = 64; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; box[0] = 64; box[1] = 128; }
    str[0] = (uint64_t)ldb * 2;
    if (tt_make_tmap(&tmB, B, 2, 2, dims, str, box, 1)) return -1;
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.c_fp32 = c_fp32;
  p.bias = (const bf16*)bias; p.epi = epi;
  p.residual = (const bf16*)residual; p.ldr = ldr;
  p.gate = gate; p.gate_ld = gate_ld; p.rows_per_gate = rows_per_gate > 0 ? rows_per_gate : 1;
  p.aux_out = (bf16*)aux_out; p.alpha = alpha; p.status = status;
  p.world = 1;
  int dev = 0, sms = 0;
  TT_CUDA(cudaGetDevice(&dev));
  TT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (!a_mn && !b_mn) return launch2<0, 0>(tmA, tmB, p, sms, stream);
  if (!a_mn && b_mn) return launch2<0, 1>(tmA, tmB, p, sms, stream);
  if (a_mn && b_mn) return launch2<1, 1>(tmA, tmB, p, sms, stream);
  return launch2<1, 0>(tmA, tmB, p, sms, stream);
}

// K-QKV-A2A: [q | k | v] = x W^T + b for this rank's `M = B * S_l` tokens (W: [3C, K] K-major), with the Ulysses
// seq -> head exchange of v inside the epilogue.  `qk` ([M, 2C], row stride ldqk) receives the q and k blocks,
// `ssq` ([M, 2 * C / 128] fp32) the sum of squares of each 128-column half tile (tt_rmsrope_fwd_scatter turns them
// into the full-row statistics without re-reducing the row), and the v block is stored into the head owners'
// [B, S_pad, ceil(H / world), D] buffers (`v_peer_ptrs`, one device address per rank).  Returns -3 when the shape
// is outside the CTA-pair kernel's domain (the caller then runs the unfused sequence).
TT_API int tt_gemm_qkv_a2a(const void* x, long long ldx, const void* W, long long ldw, const void* bias, void* qk,
                           long long ldqk, float* ssq, const long long* v_peer_ptrs, int world, int rank, int M,
                           int C, int K, int S_l, int H, int D, unsigned* status, cudaStream_t stream) {
  if (M < 256) return -3;
  TT_CHECK(C > 0 && C % 256 == 0 && K > 0 && H * D == C && D % 8 == 0, "gemm_qkv_a2a: bad shape C=%d H=%d D=%d", C, H, D);
  TT_CHECK(world >= 1 && world <= TT_MAX_PEERS && rank >= 0 && rank < world, "gemm_qkv_a2a: bad world/rank");
  TT_CHECK(S_l > 0 && M % S_l == 0, "gemm_qkv_a2a: rows must be whole samples of S_l tokens");
  TT_CHECK(ldx % 8 == 0 && ldw % 8 == 0 && ldqk % 8 == 0 && ((uintptr_t)qk & 15) == 0 && ssq != nullptr,
           "gemm_qkv_a2a: misaligned operands");
  if (bias) TT_CHECK(((uintptr_t)bias & 15) == 0, "gemm_qkv_a2a: bias is not 16-byte aligned");
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = 64; box[1] = BM;
    str[0] = (uint64_t)ldx * 2;
    if (tt_make_tmap(&tmA, x, 2, 2, dims, str, box, 1)) return -1;
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)(3 * C); box[0] = 64; box[1] = 128;
    str[0] = (uint64_t)ldw * 2;
    if (tt_make_tmap(&tmB, W, 2, 2, dims, str, box, 1)) return -1;
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = 3 * C; p.K = K;
  p.C = qk; p.ldc = ldqk; p.c_fp32 = 0;
  p.bias = (const bf16*)bias; p.epi = EPI_QKV_A2A;
  p.rows_per_gate = 1; p.alpha = 1.f; p.status = status;
  p.world = 1;
  p.qkv_C = C; p.ssq = ssq;
  for (int i = 0; i < world; ++i) {
    p.sc.peer[i] = reinterpret_cast<void*>(v_peer_ptrs[i]);
    TT_CHECK(p.sc.peer[i] && ((uintptr_t)p.sc.peer[i] & 15) == 0, "gemm_qkv_a2a: bad peer pointer %d", i);
  }
  p.sc.mode = 1; p.sc.S_l = S_l; p.sc.S_pad = S_l * world; p.sc.Hl = (H + world - 1) / world; p.sc.H = H;
  p.sc.D = D; p.sc.rank = rank; p.sc.world = world;
  int dev = 0, sms = 0;
  TT_CUDA(cudaGetDevice(&dev));
  TT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  return launch2<0, 0>(tmA, tmB, p, sms, stream);
}

// K-AG-GEMM: C = epilogue([A_0; A_1; ...] B^T) where segment s of A ([seg_rows, K], row stride K) lives in rank s's
// buffer at device address a_ptrs[s] (peer memory; a_ptrs[rank] is this rank's own).  The kernel gathers the segments
// into `G` ([world * seg_rows, K], local, left filled for the caller) while it multiplies: see AgParams.  `flags`:
// uint32[ceil(world * seg_rows / 128)] that held no value equal to `epoch` before the call (zero-initialised once,
// then epoch = 1, 2, ... per call).  The caller has put a cross-rank barrier between the writes of the segments and
// this call.  Returns -3 for shapes outside the CTA-pair kernel's domain.
TT_API int tt_gemm2_bf16_ag(const long long* a_ptrs, const void* B, long long ldb, int b_mn, void* C, long long ldc,
                            void* G, unsigned* flags, unsigned epoch, int seg_rows, int world, int rank, int N, int K,
                            const void* bias, int epi, void* aux_out, unsigned* status, cudaStream_t stream) {
  const long long M = (long long)seg_rows * world;
  if (N < 256 || M < 256) return -3;
  TT_CHECK(world >= 1 && world <= TP_MAX && rank >= 0 && rank < world && seg_rows > 0, "gemm2_ag: bad world/rank");
  TT_CHECK(N % 8 == 0 && K % 8 == 0 && M < (1ll << 31), "gemm2_ag: bad shape");
  TT_CHECK(ldb % 8 == 0 && ldc % 8 == 0 && ((uintptr_t)C & 15) == 0 && ((uintptr_t)G & 15) == 0 && flags != nullptr,
           "gemm2_ag: misaligned operands");
  TT_CHECK(epi == EPI_NONE || epi == EPI_GELU || epi == EPI_SILU, "gemm2_ag: epilogue %d not supported", epi);
  if (bias) TT_CHECK(((uintptr_t)bias & 15) == 0, "gemm2_ag: bias is not 16-byte aligned");
  AgParams ag;
  memset(&ag, 0, sizeof(ag));
  for (int i = 0; i < world; ++i) {
    ag.src[i] = reinterpret_cast<const bf16*>(a_ptrs[i]);
    TT_CHECK(ag.src[i] && ((uintptr_t)ag.src[i] & 15) == 0, "gemm2_ag: bad segment pointer %d", i);
  }
  ag.G = (bf16*)G; ag.flags = flags; ag.epoch = epoch; ag.seg_rows = seg_rows;
  ag.n_blocks = (int)((M + BM - 1) / BM);
  ag.rot_tiles = (int)(((long long)rank * seg_rows) / (2 * BM));
  ag.local_row0 = rank * seg_rows;
  CUtensorMap tmA, tmB, tmL;
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = 64; box[1] = BM;
    str[0] = (uint64_t)K * 2;
    if (tt_make_tmap(&tmA, G, 2, 2, dims, str, box, 1)) return -1;
    dims[1] = (uint64_t)seg_rows;
    if (tt_make_tmap(&tmL, ag.src[rank], 2, 2, dims, str, box, 1)) return -1;
    if (b_mn) { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; box[0] = 64; box[1] = 64; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; box[0] = 64; box[1] = 128; }
    str[0] = (uint64_t)ldb * 2;
    if (tt_make_tmap(&tmB, B, 2, 2, dims, str, box, 1)) return -1;
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = (int)M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.c_fp32 = 0;
  p.bias = (const bf16*)bias; p.epi = epi;
  p.rows_per_gate = 1; p.aux_out = (bf16*)aux_out; p.alpha = 1.f; p.status = status;
  p.world = 1;
  int dev = 0, sms = 0;
  TT_CUDA(cudaGetDevice(&dev));
  TT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (b_mn) return launch2<0, 1, true>(tmA, tmB, p, sms, stream, &ag, &tmL);
  return launch2<0, 0, true>(tmA, tmB, p, sms, stream, &ag, &tmL);
}

// K-GEMM-RS on CTA pairs, first half: the partial product A B^T ([world * seg_rows, N]) is stored row by row into slot
// `rank` of the staging buffer [world, seg_rows, ldc] of the rank that owns the row (c_peers: one device address per
// rank, peer memory); after a cross-rank barrier tt_tp_reduce_rows sums the slots.  Returns -3 for shapes outside
// the pair kernel's domain (the one-CTA kernel, tt_gemm_bf16_rs, takes those).
TT_API int tt_gemm2_bf16_rs(const void* A, long long lda, const void* B, long long ldb, int b_mn,
                            const long long* c_peers, long long ldc, int seg_rows, int world, int rank, int N, int K,
                            unsigned* status, cudaStream_t stream) {
  const long long M = (long long)seg_rows * world;
  if (N < 256 || M < 256) return -3;
  TT_CHECK(world >= 1 && world <= TP_MAX && rank >= 0 && rank < world && seg_rows > 0, "gemm2_rs: bad world/rank");
  TT_CHECK(N % 8 == 0 && K % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0 && M < (1ll << 31), "gemm2_rs: bad shape");
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = 64; box[1] = BM;
    str[0] = (uint64_t)lda * 2;
    if (tt_make_tmap(&tmA, A, 2, 2, dims, str, box, 1)) return -1;
    if (b_mn) { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; box[0] = 64; box[1] = 64; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; box[0] = 64; box[1] = 128; }
    str[0] = (uint64_t)ldb * 2;
    if (tt_make_tmap(&tmB, B, 2, 2, dims, str, box, 1)) return -1;
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = (int)M; p.N = N; p.K = K;
  p.ldc = ldc; p.c_fp32 = 0; p.epi = EPI_NONE;
  p.rows_per_gate = 1; p.alpha = 1.f; p.status = status;
  p.tp_mode = 2; p.seg_rows = seg_rows; p.world = world; p.rank = rank;
  for (int s = 0; s < world; ++s) {
    TT_CHECK(c_peers[s] != 0 && (c_peers[s] & 15) == 0, "gemm2_rs: bad peer pointer %d", s);
    p.peer_c[s] = reinterpret_cast<bf16*>(c_peers[s]);
  }
  p.C = p.peer_c[rank];
  int dev = 0, sms = 0;
  TT_CUDA(cudaGetDevice(&dev));
  TT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  return b_mn ? launch2<0, 1>(tmA, tmB, p, sms, stream) : launch2<0, 0>(tmA, tmB, p, sms, stream);
}
