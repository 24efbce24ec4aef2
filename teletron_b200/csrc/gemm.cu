// K-GEMM: persistent, warp-specialised bf16 GEMM on the 5th-generation tensor cores.
//
//   C[M,N] = epilogue( alpha * A[M,K] * B[N,K]^T )        fp32 accumulation in tensor memory
//
// One CTA per SM walks output tiles of 128 x BN. Roles inside the CTA (320 threads):
//   warp 0      TMA producer: fills a ring of shared-memory stages (A 128x64, B BNx64)
//   warp 1      allocates tensor memory and issues tcgen05.mma (one thread)
//   warps 2..9  epilogue (two warps per tensor-memory lane quarter, half of the columns each): tcgen05.ld the accumulator, apply bias / GELU / gate+residual /
//               accumulate, store bf16 or fp32
// Two accumulator buffers in tensor memory let the epilogue of tile i overlap the
// main loop of tile i+1.
//
// Either operand may be "K-major" (reduction dim contiguous, e.g. activations [M,K] and
// nn.Linear weights [N,K]) or "MN-major" (output dim contiguous). That covers, without
// any transpose pass:
//   forward   Y  = X  W^T     A K-major,  B K-major
//   dgrad     dX = dY W       A K-major,  B MN-major   (W is [N,K] = [Kred, Nout])
//   wgrad     dW = dY^T X     A MN-major, B MN-major   (reduction over tokens)
// It replaces the cuBLAS calls behind nn.Linear in the reference
// (teletron/models/wan/wan_model.py:144-147,225-226).
#include "gemm_epilogue.cuh"

using namespace tt;
using namespace tt_gemm;

namespace {

template <int BN>
struct Cfg {
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = BN * 2 < 32 ? 32 : BN * 2;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + 1024;
};

template <int BN, int A_MN, int B_MN, int TP>
__global__ void __launch_bounds__(320, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ TmapSet tmAp, const GemmParams p) {
  using C_ = Cfg<BN>;
  constexpr int STAGES = C_::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * C_::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = p.seg_rows ? p.world * ((p.seg_rows + BM - 1) / BM) : (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    if (TP == 1) {
      for (int i = 0; i < p.world; ++i) tma_prefetch_desc(&tmAp.m[i]);
    } else {
      tma_prefetch_desc(&tmA);
    }
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C_::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const MTile mt = m_tile(p, tile / tiles_n);
        // all-gather variant: this tile's rows live in rank `seg`'s buffer (a plain TMA load from peer memory)
        const CUtensorMap* mapA = (TP == 1) ? &tmAp.m[mt.seg] : &tmA;
        const int m0 = (TP == 1) ? mt.seg_row0 : mt.row0;
        const int n0 = (tile % tiles_n) * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * C_::STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full[s], C_::STAGE_BYTES);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * 8192, mapA, &full[s], m0 + i * 64, k0);
          } else {
            tma_load_2d(sa, mapA, &full[s], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * 8192, &tmB, &full[s], n0 + i * 64, k0);
          } else {
            tma_load_2d(sb, &tmB, &full[s], k0, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, A_MN, B_MN);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const int a = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty[a], aph ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 1)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 2)) {
            ok = false;
            break;
          }
          tc_fence_after();
          // descriptors as (low word + constant): one integer add per operand and MMA
          const uint32_t a_base = smem_u32(smem + s * C_::STAGE_BYTES);
          const uint32_t a_lo = umma_desc_lo(a_base, A_MN ? 8192 : 16);
          const uint32_t b_lo = umma_desc_lo(a_base + A_BYTES, B_MN ? 8192 : 16);
          constexpr uint32_t HI = umma_desc_hi(1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_ss_lo<HI, HI>(d_tmem, a_lo + k * ((A_MN ? 2048 : 32) >> 4), b_lo + k * ((B_MN ? 2048 : 32) >> 4), idesc,
                               (kb | k) != 0 ? 1u : 0u);
          tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&tfull[a]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    const int eg = (warp - 2) >> 2;  // two warps share a quarter and split the tile's columns
    int tcount = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      const int a = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      if (!mbar_wait(&tfull[a], aph, abort_flag, p.status, TT_ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const MTile mt = m_tile(p, tile / tiles_n);
      const int n0 = (tile % tiles_n) * BN;
      const int row = mt.row0 + q * 32 + lane;
      const bool row_ok = q * 32 + lane < mt.valid;
      // reduce-scatter variant: the row goes to slot `rank` of the owner's staging buffer
      bf16* c_row = (TP == 2) ? p.peer_c[mt.seg] + ((long long)p.rank * p.seg_rows + mt.seg_row0 + q * 32 + lane) * p.ldc
                              : reinterpret_cast<bf16*>(p.C) + (long long)row * p.ldc;
      epilogue_tile<BN>(p, tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN), eg, row, row_ok, c_row, n0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[a]);
    }
  }

  // ------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    // let copies that are still in flight land before the CTA's shared memory goes away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C_::TMEM_COLS);
}

template <int BN, int A_MN, int B_MN, int TP = 0>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int sms,
           cudaStream_t stream, const TmapSet* tmAp = nullptr) {
  using C_ = Cfg<BN>;
  auto kern = gemm_kernel<BN, A_MN, B_MN, TP>;
  static TmapSet no_maps;
  if (!tmAp) tmAp = &no_maps;
  static bool attr_done = false;
  if (!attr_done) {
    TT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM_BYTES));
    attr_done = true;
  }
  const int tiles_m = p.seg_rows ? p.world * ((p.seg_rows + BM - 1) / BM) : (p.M + BM - 1) / BM;
  const int tiles = tiles_m * ((p.N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  kern<<<grid, 320, C_::SMEM_BYTES, stream>>>(tmA, tmB, *tmAp, p);
  TT_LAUNCH_CHECK();
  return 0;
}

template <int BN>
int dispatch_major(int a_mn, int b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB,
                   const GemmParams& p, int sms, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch<BN, 0, 0>(tmA, tmB, p, sms, stream);
  if (!a_mn && b_mn) return launch<BN, 0, 1>(tmA, tmB, p, sms, stream);
  if (a_mn && b_mn) return launch<BN, 1, 1>(tmA, tmB, p, sms, stream);
  return launch<BN, 1, 0>(tmA, tmB, p, sms, stream);
}

}  // namespace

// A: K-major -> memory [M, K] with row stride lda;  MN-major -> memory [K, M] with row stride lda.
// B: K-major -> memory [N, K] with row stride ldb;  MN-major -> memory [K, N] with row stride ldb.
// gate is fp32 [*, gate_ld]; row r uses gate row r / rows_per_gate.
TT_API int tt_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
                        void* C, long long ldc, int c_fp32, int M, int N, int K, const void* bias,
                        int epi, const void* residual, long long ldr, const float* gate,
                        long long gate_ld, int rows_per_gate, void* aux_out, float alpha,
                        unsigned* status, int max_ctas, cudaStream_t stream) {
  TT_CHECK(M > 0 && N > 0 && K > 0, "gemm: empty problem %d x %d x %d", M, N, K);
  TT_CHECK(N % 8 == 0, "gemm: N (%d) must be a multiple of 8", N);
  TT_CHECK(lda % 8 == 0 && ldb % 8 == 0, "gemm: lda/ldb must be multiples of 8 elements");
  TT_CHECK(ldc % (c_fp32 ? 4 : 8) == 0, "gemm: ldc (%lld) breaks 16-byte row alignment", ldc);
  TT_CHECK(((uintptr_t)C & 15) == 0, "gemm: C is not 16-byte aligned");
  TT_CHECK(epi >= 0 && epi <= EPI_LAST, "gemm: unknown epilogue %d", epi);
  if (epi == EPI_GATE_RES) {
    TT_CHECK(residual && gate && rows_per_gate > 0, "gemm: gate/residual epilogue needs both tensors");
    TT_CHECK(ldr % 8 == 0 && gate_ld % 4 == 0, "gemm: residual/gate leading dims misaligned");
    TT_CHECK((((uintptr_t)residual | (uintptr_t)gate) & 15) == 0, "gemm: residual/gate misaligned");
  }
  if (bias) TT_CHECK(((uintptr_t)bias & 15) == 0, "gemm: bias is not 16-byte aligned");
  const int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    if (a_mn) { dims[0] = (uint64_t)M; dims[1] = (uint64_t)K; box[0] = 64; box[1] = 64; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = 64; box[1] = BM; }
    str[0] = (uint64_t)lda * 2;
    if (tt_make_tmap(&tmA, A, 2, 2, dims, str, box, 1)) return -1;
    if (b_mn) { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; box[0] = 64; box[1] = 64; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; box[0] = 64; box[1] = (uint32_t)BN; }
    str[0] = (uint64_t)ldb * 2;
    if (tt_make_tmap(&tmB, B, 2, 2, dims, str, box, 1)) return -1;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.c_fp32 = c_fp32;
  p.bias = (const bf16*)bias; p.epi = epi;
  p.residual = (const bf16*)residual; p.ldr = ldr;
  p.gate = gate; p.gate_ld = gate_ld; p.rows_per_gate = rows_per_gate > 0 ? rows_per_gate : 1;
  p.aux_out = (bf16*)aux_out; p.alpha = alpha; p.status = status;
  p.tp_mode = 0; p.seg_rows = 0; p.world = 1; p.rank = 0;
  for (int i = 0; i < TP_MAX; ++i) p.peer_c[i] = nullptr;
  int dev = 0, sms = 0;
  TT_CUDA(cudaGetDevice(&dev));
  TT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (BN == 256) return dispatch_major<256>(a_mn, b_mn, tmA, tmB, p, sms, stream);
  if (BN == 128) return dispatch_major<128>(a_mn, b_mn, tmA, tmB, p, sms, stream);
  return dispatch_major<64>(a_mn, b_mn, tmA, tmB, p, sms, stream);
}

namespace {

__global__ void tp_reduce_rows_kernel(const bf16* __restrict__ staging, int world, long long rows, int N,
                                      long long ld, const bf16* __restrict__ bias, bf16* __restrict__ out,
                                      long long ldo) {
  const long long vec_per_row = N / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (bias) {
      const uint4 bv = *reinterpret_cast<const uint4*>(bias + c);
      const uint32_t* bu = reinterpret_cast<const uint32_t*>(&bv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(bu[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    for (int w = 0; w < world; ++w) {
      const uint4 v = *reinterpret_cast<const uint4*>(staging + ((long long)w * rows + r) * ld + c);
      const uint32_t* vu = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(vu[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]);
    o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]);
    o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + r * ldo + c) = o;
  }
}

int tp_common_checks(int seg_rows, int world, int N, int K, long long lda, long long ldb, long long ldc) {
  TT_CHECK(world >= 1 && world <= TP_MAX, "gemm_tp: group size %d outside [1, %d]", world, TP_MAX);
  TT_CHECK(seg_rows > 0 && N > 64 && K > 0, "gemm_tp: needs seg_rows > 0, N > 64, K > 0 (got %d, %d, %d)", seg_rows, N, K);
  TT_CHECK(N % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0, "gemm_tp: N and leading dims must be multiples of 8");
  return 0;
}

int make_b_map(CUtensorMap* tmB, const void* B, long long ldb, int b_mn, int N, int K, int BN) {
  uint64_t dims[2], str[1];
  uint32_t box[2];
  if (b_mn) { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; box[0] = 64; box[1] = 64; }
  else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; box[0] = 64; box[1] = (uint32_t)BN; }
  str[0] = (uint64_t)ldb * 2;
  return tt_make_tmap(tmB, B, 2, 2, dims, str, box, 1);
}

int make_a_map(CUtensorMap* tmA, const void* A, long long lda, int rows, int K) {
  uint64_t dims[2] = {(uint64_t)K, (uint64_t)rows}, str[1] = {(uint64_t)lda * 2};
  uint32_t box[2] = {64, BM};
  return tt_make_tmap(tmA, A, 2, 2, dims, str, box, 1);
}

void tp_base_params(GemmParams& p, int seg_rows, int world, int rank, int N, int K, unsigned* status) {
  memset(&p, 0, sizeof(p));
  p.M = seg_rows * world; p.N = N; p.K = K;
  p.rows_per_gate = 1; p.alpha = 1.f; p.status = status;
  p.seg_rows = seg_rows; p.world = world; p.rank = rank;
}

int num_sms(int* sms) {
  int dev = 0;
  TT_CUDA(cudaGetDevice(&dev));
  TT_CUDA(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
  return 0;
}

}  // namespace

// K-AG-GEMM.  C[world * seg_rows, N] = epilogue([A_0; A_1; ...] B^T) where A_s is rank s's [seg_rows, K] buffer
// (a_peers[s] = its device address, mapped into this process): the all-gather of a column-parallel linear
// happens inside the TMA loads of the GEMM, no gathered copy of the activations exists.  The caller orders the
// launch behind a barrier that says every rank has written its A.
TT_API int tt_gemm_bf16_ag(const long long* a_peers, long long lda, const void* B, long long ldb, int b_mn,
                           void* C, long long ldc, int seg_rows, int world, int N, int K, const void* bias,
                           int epi, void* aux_out, unsigned* status, cudaStream_t stream) {
  if (tp_common_checks(seg_rows, world, N, K, lda, ldb, ldc)) return -1;
  TT_CHECK(epi == EPI_NONE || epi == EPI_GELU || epi == EPI_SILU, "gemm_ag: epilogue %d not supported", epi);
  TT_CHECK(((uintptr_t)C & 15) == 0 && (!bias || ((uintptr_t)bias & 15) == 0), "gemm_ag: misaligned C / bias");
  const int BN = N > 128 ? 256 : 128;
  TmapSet maps;
  memset(&maps, 0, sizeof(maps));
  for (int s = 0; s < world; ++s) {
    TT_CHECK(a_peers[s] != 0 && (a_peers[s] & 15) == 0, "gemm_ag: bad peer pointer %d", s);
    if (make_a_map(&maps.m[s], reinterpret_cast<const void*>(a_peers[s]), lda, seg_rows, K)) return -1;
  }
  CUtensorMap tmB;
  if (make_b_map(&tmB, B, ldb, b_mn, N, K, BN)) return -1;
  GemmParams p;
  tp_base_params(p, seg_rows, world, 0, N, K, status);
  p.tp_mode = 1; p.C = C; p.ldc = ldc; p.bias = (const bf16*)bias; p.epi = epi; p.aux_out = (bf16*)aux_out;
  int sms = 0;
  if (num_sms(&sms)) return -2;
  if (BN == 256) return b_mn ? launch<256, 0, 1, 1>(maps.m[0], tmB, p, sms, stream, &maps)
                             : launch<256, 0, 0, 1>(maps.m[0], tmB, p, sms, stream, &maps);
  return b_mn ? launch<128, 0, 1, 1>(maps.m[0], tmB, p, sms, stream, &maps)
              : launch<128, 0, 0, 1>(maps.m[0], tmB, p, sms, stream, &maps);
}

// K-GEMM-RS, first half.  The partial product A[world * seg_rows, K] B^T is stored tile by tile into the staging
// buffers of the ranks that own the rows: c_peers[s] is rank s's buffer [world, seg_rows, ldc], this rank writes
// slot `rank`.  After a barrier each rank sums its slots with tt_tp_reduce_rows.
TT_API int tt_gemm_bf16_rs(const void* A, long long lda, const void* B, long long ldb, int b_mn,
                           const long long* c_peers, long long ldc, int seg_rows, int world, int rank, int N,
                           int K, unsigned* status, cudaStream_t stream) {
  if (tp_common_checks(seg_rows, world, N, K, lda, ldb, ldc)) return -1;
  TT_CHECK(rank >= 0 && rank < world, "gemm_rs: bad rank");
  const int BN = N > 128 ? 256 : 128;
  CUtensorMap tmA, tmB;
  if (make_a_map(&tmA, A, lda, seg_rows * world, K)) return -1;
  if (make_b_map(&tmB, B, ldb, b_mn, N, K, BN)) return -1;
  GemmParams p;
  tp_base_params(p, seg_rows, world, rank, N, K, status);
  p.tp_mode = 2; p.ldc = ldc;
  for (int s = 0; s < world; ++s) {
    TT_CHECK(c_peers[s] != 0 && (c_peers[s] & 15) == 0, "gemm_rs: bad peer pointer %d", s);
    p.peer_c[s] = reinterpret_cast<bf16*>(c_peers[s]);
  }
  p.C = p.peer_c[rank];
  int sms = 0;
  if (num_sms(&sms)) return -2;
  if (BN == 256) return b_mn ? launch<256, 0, 1, 2>(tmA, tmB, p, sms, stream) : launch<256, 0, 0, 2>(tmA, tmB, p, sms, stream);
  return b_mn ? launch<128, 0, 1, 2>(tmA, tmB, p, sms, stream) : launch<128, 0, 0, 2>(tmA, tmB, p, sms, stream);
}

// K-GEMM-RS, second half: out[r, :] = bias + sum_w staging[w, r, :]   (fp32 accumulation, bf16 in / out)
TT_API int tt_tp_reduce_rows(const void* staging, int world, long long rows, int N, long long ld, const void* bias,
                             void* out, long long ldo, cudaStream_t stream) {
  TT_CHECK(world >= 1 && rows > 0 && N > 0 && N % 8 == 0 && ld % 8 == 0 && ldo % 8 == 0, "tp_reduce_rows: bad shape");
  TT_CHECK((((uintptr_t)staging | (uintptr_t)out | (uintptr_t)bias) & 15) == 0, "tp_reduce_rows: misaligned pointer");
  const long long total = rows * (N / 8);
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  tp_reduce_rows_kernel<<<(unsigned)blocks, threads, 0, stream>>>((const bf16*)staging, world, rows, N, ld,
                                                                 (const bf16*)bias, (bf16*)out, ldo);
  TT_LAUNCH_CHECK();
  return 0;
}
