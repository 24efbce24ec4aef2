// K-ATTN forward: non-causal flash attention for head_dim 128 on tcgen05 / TMEM.
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles t = 0,1 and walks
// the keys in tiles of 128.  Roles (320 threads):
//   warp 0       TMA producer: Q once, then K_0, V_0, K_1, V_1, ... through a 5-slot ring
//   warp 1       tcgen05.mma issuer: S_t = Q_t K_j^T into tensor memory, O_t += P_t V_j
//   warps 2..5   softmax group for tile 0, warps 6..9 for tile 1; thread <-> query row
// Tensor memory: S_0, S_1, O_0, O_1, 128 fp32 columns each (all 512 columns).
// The bf16 probabilities P_t are written over the first 64 columns of S_t and read from there as the
// A operand of P*V: with P in shared memory the kernel was bound by shared-memory bandwidth (operand
// reads of 32 MMAs, 64 KB of bank-conflicted P stores and the TMA writes added up to the measured
// 4,700 clocks per key tile).  S_t(j+1) therefore follows P_t V_j on the tensor pipe, and the two tiles
// alternate: while one is in its softmax, the other's two products run.
// The softmax keeps a running maximum that is only raised when the tile maximum exceeds it
// by more than 8 (in log2 units), so O in tensor memory is rescaled rarely.
// V is consumed as an MN-major B operand straight from its [token, d] layout.
// Keys past kv_len (ragged last tile, or a per-batch key length for padded text) are
// masked to -inf.  Every barrier wait is bounded (see tt_common.cuh).
//
// Stands in for flash_attn / SDPA in the reference (teletron/models/wan/wan_model.py:43-74,
// teletron/core/context_parallel/context_parallel_mixin.py:107-114).
#include "tt_common.cuh"

using namespace tt;

namespace {

constexpr int TILE = 128;
constexpr int HALF_BYTES = 128 * 128;      // 128 rows x 64 bf16
constexpr int TILE_BYTES = 2 * HALF_BYTES;  // 128 x 128 bf16
constexpr int KV_SLOTS = 5;
constexpr int SM_Q = 0;
constexpr int SM_KV = SM_Q + 2 * TILE_BYTES;
constexpr int SM_BAR = SM_KV + KV_SLOTS * TILE_BYTES;
constexpr int SMEM_BYTES = SM_BAR + 256 + 1024;
constexpr int NTHREADS = 320;
constexpr float RESCALE_THRESHOLD = 8.0f;

struct AttnParams {
  int Sq, Skv, H, B;
  float scale_log2;
  bf16* O;
  long long ldo, o_batch_stride;
  float* lse;  // [B, H, Sq]
  const int* kv_lens;  // optional [B]
  unsigned* status;
  TTScatter sc;  // mode 2: also store O into the owning peer's [B, S_l, H, D] buffer (head -> seq)
};

__global__ void __launch_bounds__(NTHREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM_BAR);
  uint64_t* q_full = bars;                        // 1
  uint64_t* kv_full = bars + 1;                   // KV_SLOTS
  uint64_t* kv_empty = kv_full + KV_SLOTS;        // KV_SLOTS
  uint64_t* s_full = kv_empty + KV_SLOTS;         // 2
  uint64_t* p_full = s_full + 2;                  // 2 (4 arrivals)
  uint64_t* pv_done = p_full + 2;                 // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 2 * TILE;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  int kv_len = p.Skv;
  if (p.kv_lens) kv_len = min(max(p.kv_lens[b], 1), p.Skv);
  const int n_tiles = (kv_len + TILE - 1) / TILE;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < KV_SLOTS; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);
      mbar_init(&pv_done[t], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * TILE_BYTES);
      for (int t = 0; t < 2; ++t)
        for (int hf = 0; hf < 2; ++hf)
          tma_load_3d(smem + SM_Q + t * TILE_BYTES + hf * HALF_BYTES, &tmQ, q_full,
                      h * 128 + hf * 64, q0 + t * TILE, b);
      for (int i = 0; i < 2 * n_tiles; ++i) {
        const int slot = i % KV_SLOTS;
        const uint32_t ph = (i / KV_SLOTS) & 1;
        if (!mbar_wait(&kv_empty[slot], ph ^ 1, abort_flag, p.status, TT_ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&kv_full[slot], TILE_BYTES);
        const CUtensorMap* tm = (i & 1) ? &tmV : &tmK;
        uint8_t* dst = smem + SM_KV + slot * TILE_BYTES;
        for (int hf = 0; hf < 2; ++hf)
          tma_load_3d(dst + hf * HALF_BYTES, tm, &kv_full[slot], h * 128 + hf * 64, (i >> 1) * TILE, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(128, 128, 0, 1);
      constexpr uint32_t HI = umma_desc_hi(1024);
      const uint32_t q_base = smem_u32(smem + SM_Q);
      const uint32_t kv_base = smem_u32(smem + SM_KV);
      // descriptors as (low word + constant): one integer add per operand and MMA
      auto issue_s = [&](int t, uint32_t k_addr) {
        const uint32_t a_lo = umma_desc_lo(q_base + t * TILE_BYTES, 16);
        const uint32_t b_lo = umma_desc_lo(k_addr, 16);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
          umma_ss_lo<HI, HI>(tmem_base + t * 128, a_lo + off, b_lo + off, idesc_qk, ks != 0);
        }
        tc_commit(&s_full[t]);
      };
      // O_t += P_t V: P_t is the packed bf16 copy in the first 64 columns of S_t (8 columns per k-step)
      auto issue_pv = [&](int t, uint32_t v_addr, uint32_t acc) {
        const uint32_t b_lo = umma_desc_lo(v_addr, HALF_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts_lo<HI>(tmem_base + 256 + t * 128, tmem_base + t * 128 + ks * 8, b_lo + ks * (2048 >> 4), idesc_pv,
                         ks != 0 ? 1u : acc);
        tc_commit(&pv_done[t]);
      };
      // ring position (slot, phase) of the next tile to consume: K_0, V_0, K_1, V_1, ...
      uint32_t slot = 0, ph = 0;
      auto next_slot = [&]() { if (++slot == KV_SLOTS) { slot = 0; ph ^= 1; } };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 1);
      if (ok) ok = mbar_wait(&kv_full[0], 0, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 2);
      if (ok) {
        tc_fence_after();
        issue_s(0, kv_base);
        issue_s(1, kv_base);
        tc_commit(&kv_empty[0]);
        next_slot();
      }
      uint32_t eph = 0;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const bool more = j + 1 < n_tiles;
        // V_j and K_{j+1} were requested slots ago; waiting for them first keeps the waits on the softmax
        // groups the only ones between groups of MMAs
        const uint32_t v_slot = slot, v_ph = ph;
        next_slot();
        const uint32_t k_slot = slot, k_ph = ph;
        if (more) next_slot();
        if (!mbar_wait(&kv_full[v_slot], v_ph, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 5)) { ok = false; break; }
        if (more && !mbar_wait(&kv_full[k_slot], k_ph, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 3)) { ok = false; break; }
        const uint32_t acc = j > 0 ? 1u : 0u;
        for (int t = 0; t < 2; ++t) {
          if (!mbar_wait(&p_full[t], eph, abort_flag, p.status, TT_ST_TIMEOUT_MMA + 6)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, kv_base + v_slot * TILE_BYTES, acc);
          if (more) issue_s(t, kv_base + k_slot * TILE_BYTES);
        }
        if (!ok) break;
        tc_commit(&kv_empty[v_slot]);
        if (more) tc_commit(&kv_empty[k_slot]);
        eph ^= 1;
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax groups
    const int t = (warp - 2) >> 2;
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // row inside the tile
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + t * 128;
    const uint32_t o_addr = tmem_base + lane_addr + 256 + t * 128;
    float m_used = -1.0e30f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const uint32_t jph = j & 1;
      if (!mbar_wait(&s_full[t], jph, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 1)) { ok = false; break; }
      __syncwarp();
      tc_fence_after();
      uint32_t s[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, s[c]);
      tmem_ld_wait();
      const int valid = kv_len - j * TILE;  // >= 1
      if (valid < TILE) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i >= valid) s[c][i] = __float_as_uint(-1.0e30f);
      }
      // row maximum as eight independent chains (one dependent chain of 128 costs about 500 clocks)
      float mxa[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) mxa[a] = __uint_as_float(s[a >> 1][(a & 1) * 16]);
#pragma unroll
      for (int i = 1; i < 16; ++i)
#pragma unroll
        for (int a = 0; a < 8; ++a) mxa[a] = fmaxf(mxa[a], __uint_as_float(s[a >> 1][(a & 1) * 16 + i]));
      const float mx = fmaxf(fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])),
                             fmaxf(fmaxf(mxa[4], mxa[5]), fmaxf(mxa[6], mxa[7])));
      const float mx2 = mx * p.scale_log2;
      const bool need = mx2 > m_used + RESCALE_THRESHOLD;
      const float m_new = need ? mx2 : m_used;
      const float f = (need && j > 0) ? fast_exp2(m_used - mx2) : 1.f;
      // probabilities first (bf16, packed in registers): this is the long special-function phase
      // and it does not depend on the previous P*V, so it overlaps with it on the tensor pipe
      uint32_t pk[64];
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float e0 = fast_exp2(fmaf(__uint_as_float(s[c][i]), p.scale_log2, -m_new));
          const float e1 = fast_exp2(fmaf(__uint_as_float(s[c][i + 1]), p.scale_log2, -m_new));
          ls4[(i >> 1) & 3] += e0 + e1;
          pk[c * 16 + (i >> 1)] = pack_bf16(e0, e1);
        }
      }
      const float lsum = (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
      // S_t(j) was issued behind P_t V_{j-1}, so O_t is quiescent here and may be rescaled in place
      if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tmem_st32(o_addr + c * 32, o);
        }
      }
      l = l * f + lsum;
      m_used = m_new;
      // P_t over the first 64 columns of S_t: two bf16 per column, key order
      {
        uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[0]);
        uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[32]);
        tmem_st32(s_addr, lo);
        tmem_st32(s_addr + 32, hi);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    if (ok) ok = mbar_wait(&pv_done[t], (n_tiles - 1) & 1, abort_flag, p.status, TT_ST_TIMEOUT_SOFTMAX + 3);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int row = q0 + t * TILE + r;
      const float inv = 1.f / l;
      // the group's Q tile is no longer read (its last S and P*V have completed): it stages the output rows
      uint8_t* stage = smem + SM_Q + t * TILE_BYTES + q * (32 * 256);
      bf16* orow = row < p.Sq ? p.O + (long long)b * p.o_batch_stride + (long long)row * p.ldo + h * 128 : nullptr;
      bf16* prow = scatter_row(p.sc, row, p.Sq) ? scatter_dst(p.sc, b, row, h) : nullptr;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32(o_addr + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 pk;
          pk.x = pack_bf16(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
          pk.y = pack_bf16(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
          pk.z = pack_bf16(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
          pk.w = pack_bf16(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
          stage_put<16>(stage, lane, c * 4 + g, pk);
        }
      }
      stage_flush<16>(stage, lane, orow, prow);
      if (row < p.Sq && p.lse)
        p.lse[((long long)b * p.H + h) * p.Sq + row] = (m_used + log2f(l)) * 0.6931471805599453f;
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

int make_qkv_map(CUtensorMap* tm, const void* ptr, long long ld, long long batch_stride, int S, int H,
                 int B) {
  uint64_t dims[3] = {(uint64_t)H * 128, (uint64_t)S, (uint64_t)B};
  uint64_t str[2] = {(uint64_t)ld * 2, (uint64_t)batch_stride * 2};
  uint32_t box[3] = {64, 128, 1};
  return tt_make_tmap(tm, ptr, 2, 3, dims, str, box, 1);
}

}  // namespace

// q: [B, Sq, H, 128] with token stride ldq and batch stride q_bs (elements); k, v likewise
// with Skv tokens; o: [B, Sq, H*128] with token stride ldo; lse: fp32 [B, H, Sq] (may be null).
// kv_lens: optional int32 [B], keys at or beyond kv_lens[b] are masked.
static int attn_fwd_impl(const void* q, long long ldq, long long q_bs, const void* k, long long ldk,
                         long long k_bs, const void* v, long long ldv, long long v_bs, void* o,
                         long long ldo, long long o_bs, float* lse, const int* kv_lens, int B, int H,
                         int Sq, int Skv, int D, float scale, unsigned* status, const TTScatter& sc,
                         cudaStream_t stream) {
  TT_CHECK(D == 128, "attn_fwd: head_dim must be 128 (got %d)", D);
  TT_CHECK(B > 0 && H > 0 && Sq > 0 && Skv > 0, "attn_fwd: empty problem");
  TT_CHECK(ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 && ldo % 8 == 0, "attn_fwd: token strides must be multiples of 8");
  TT_CHECK(q_bs % 8 == 0 && k_bs % 8 == 0 && v_bs % 8 == 0 && o_bs % 8 == 0, "attn_fwd: batch strides must be multiples of 8");
  TT_CHECK(((uintptr_t)o & 15) == 0, "attn_fwd: output misaligned");
  CUtensorMap tmQ, tmK, tmV;
  if (make_qkv_map(&tmQ, q, ldq, q_bs, Sq, H, B)) return -1;
  if (make_qkv_map(&tmK, k, ldk, k_bs, Skv, H, B)) return -1;
  if (make_qkv_map(&tmV, v, ldv, v_bs, Skv, H, B)) return -1;
  AttnParams p;
  p.Sq = Sq; p.Skv = Skv; p.H = H; p.B = B;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.O = (bf16*)o; p.ldo = ldo; p.o_batch_stride = o_bs;
  p.lse = lse; p.kv_lens = kv_lens; p.status = status;
  p.sc = sc;
  static bool attr_done = false;
  if (!attr_done) {
    TT_CUDA(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    attr_done = true;
  }
  dim3 grid((Sq + 2 * TILE - 1) / (2 * TILE), H, B);
  attn_fwd_kernel<<<grid, NTHREADS, SMEM_BYTES, stream>>>(tmQ, tmK, tmV, p);
  TT_LAUNCH_CHECK();
  return 0;
}

TT_API int tt_attn_fwd(const void* q, long long ldq, long long q_bs, const void* k, long long ldk,
                       long long k_bs, const void* v, long long ldv, long long v_bs, void* o,
                       long long ldo, long long o_bs, float* lse, const int* kv_lens, int B, int H,
                       int Sq, int Skv, int D, float scale, unsigned* status, cudaStream_t stream) {
  TTScatter sc;
  memset(&sc, 0, sizeof(sc));
  return attn_fwd_impl(q, ldq, q_bs, k, ldk, k_bs, v, ldv, v_bs, o, ldo, o_bs, lse, kv_lens, B, H, Sq, Skv, D,
                       scale, status, sc, stream);
}

// Attention over head-parallel tensors [B, S_total, Hl, D] whose epilogue also stores the first S_pad rows of O of
// every sample with the Ulysses head -> seq pattern into every peer's [B, S_l, H_total, D] buffer (peer_ptrs), in
// addition to the local head-layout copy `o` that the backward pass needs (and that is the only copy of rows
// S_pad .. S_total, the replicated text tokens of a joint sequence).  `heads` <= Hl is how many of this rank's head
// slots hold real heads (H_total need not divide by the group size: the last ranks own fewer); lse is
// [B, heads, S_total].
TT_API int tt_attn_fwd_scatter(const void* q, long long ldq, long long q_bs, const void* k, long long ldk,
                               long long k_bs, const void* v, long long ldv, long long v_bs, void* o,
                               long long ldo, long long o_bs, float* lse, const int* kv_lens, int B, int Hl,
                               int heads, int H_total, int S_pad, int S_total, int D, float scale,
                               const long long* peer_ptrs, int world, int rank, unsigned* status,
                               cudaStream_t stream) {
  TT_CHECK(world >= 1 && world <= TT_MAX_PEERS && rank >= 0 && rank < world, "attn_fwd_scatter: bad world/rank");
  TT_CHECK(S_pad % world == 0 && S_total >= S_pad, "attn_fwd_scatter: padded sequence must divide by the group size");
  TT_CHECK(heads >= 1 && heads <= Hl && rank * Hl + heads <= H_total && H_total <= Hl * world,
           "attn_fwd_scatter: head slots %d x %d ranks do not match %d heads (%d on rank %d)", Hl, world, H_total,
           heads, rank);
  TTScatter sc;
  memset(&sc, 0, sizeof(sc));
  for (int i = 0; i < world; ++i) {
    sc.peer[i] = reinterpret_cast<void*>(peer_ptrs[i]);
    TT_CHECK(sc.peer[i] && ((uintptr_t)sc.peer[i] & 15) == 0, "attn_fwd_scatter: bad peer pointer %d", i);
  }
  sc.mode = 2; sc.S_l = S_pad / world; sc.S_pad = S_pad; sc.Hl = Hl; sc.H = H_total; sc.D = D;
  sc.rank = rank; sc.world = world; sc.n_rows = S_pad;
  return attn_fwd_impl(q, ldq, q_bs, k, ldk, k_bs, v, ldv, v_bs, o, ldo, o_bs, lse, kv_lens, B, heads, S_total,
                       S_total, D, scale, status, sc, stream);
}
