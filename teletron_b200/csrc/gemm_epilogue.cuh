// Definitions shared by the one-CTA (gemm.cu) and the CTA-pair (gemm2.cu) GEMM kernels: parameters, output tile
// addressing and the epilogue that turns one accumulator tile in tensor memory into bias / activation /
// gate+residual / accumulate results in global memory.
#pragma once
#include "tt_common.cuh"

namespace tt_gemm {
using namespace tt;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int TP_MAX = 8;  // ranks of a tensor-parallel group

// EPI_QKV_A2A: the fused q/k/v projection under Ulysses context parallelism (N = 3 * qkv_C).  The q and k column
// blocks are stored locally ([M, 2 * qkv_C]) together with the sum of squares of every 128-column half tile of each
// row (`ssq`, [M, 2 * qkv_C / 128] fp32: the row statistics of the full-row RMSNorm that follows); the v column block
// is stored straight into the head owner's [B, S_pad, Hl, D] buffer in peer memory (`sc`, the seq -> head exchange).
enum Epi : int { EPI_NONE = 0, EPI_GELU = 1, EPI_GATE_RES = 2, EPI_ACCUM = 3, EPI_SILU = 4, EPI_LAST = 4,
                 EPI_QKV_A2A = 7 };

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  int c_fp32;
  const bf16* bias;
  int epi;
  const bf16* residual;
  long long ldr;
  const float* gate;
  long long gate_ld;
  int rows_per_gate;
  bf16* aux_out;  // optional pre-activation copy (same ld as C)
  float alpha;
  unsigned* status;
  // tensor-parallel variants: the M dimension is `world` segments of `seg_rows` rows (one per rank) and
  // output tiles never straddle a segment.
  //   tp_mode 1 (all-gather -> GEMM): segment s of A is read from rank s's buffer through its own tensor map
  //   tp_mode 2 (GEMM -> reduce-scatter): the rows of segment s are stored into rank s's staging buffer
  //             [world, seg_rows, ldc] at slot `rank`; tt_tp_reduce_rows then sums the slots
  int tp_mode, seg_rows, world, rank;
  bf16* peer_c[TP_MAX];
  // EPI_QKV_A2A
  int qkv_C;
  float* ssq;
  TTScatter sc;
};

struct TmapSet {
  CUtensorMap m[TP_MAX];
};

// first global row, owning segment, first row inside the segment and number of live rows of m-tile `tm`
struct MTile {
  int row0, seg, seg_row0, valid;
};
__device__ __forceinline__ MTile m_tile(const GemmParams& p, int tm) {
  MTile t;
  if (p.seg_rows == 0) {
    t.row0 = tm * BM; t.seg = 0; t.seg_row0 = t.row0; t.valid = min(BM, p.M - t.row0);
  } else {
    const int tps = (p.seg_rows + BM - 1) / BM;
    t.seg = tm / tps;
    t.seg_row0 = (tm - t.seg * tps) * BM;
    t.row0 = t.seg * p.seg_rows + t.seg_row0;
    t.valid = min(BM, p.seg_rows - t.seg_row0);
  }
  return t;
}


// Epilogue of one 128-row accumulator tile for the warp that owns lane quarter `q` and column group `eg` (of 2):
// `acc` is the tensor-memory address of the tile's first column for this quarter, `row` the global output row of
// this lane, `c_row` where that row's output starts (column 0), `n0` the tile's first output column.
template <int BN>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t acc, int eg, int row, bool row_ok,
                                              bf16* c_row, int n0) {
  const float* gate_row = nullptr;
  if (p.epi == EPI_GATE_RES && row_ok)
    gate_row = p.gate + (long long)(row / p.rows_per_gate) * p.gate_ld;
#pragma unroll 1
  for (int c = eg * (BN / 64); c < (eg + 1) * (BN / 64); ++c) {
    uint32_t r[32];
    tmem_ld32(acc + (uint32_t)(c * 32), r);
    tmem_ld_wait();
    const int col0 = n0 + c * 32;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int col = col0 + g * 8;
      if (!row_ok || col >= p.N) break;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]) * p.alpha;
      if (p.bias) {
        uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
        const uint32_t* bu = reinterpret_cast<const uint32_t*>(&bv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16(bu[j]);
          v[2 * j] += f.x;
          v[2 * j + 1] += f.y;
        }
      }
      if (p.epi == EPI_GELU || p.epi == EPI_SILU) {
        if (p.aux_out) {
          uint4 o;
          o.x = pack_bf16(v[0], v[1]);
          o.y = pack_bf16(v[2], v[3]);
          o.z = pack_bf16(v[4], v[5]);
          o.w = pack_bf16(v[6], v[7]);
          *reinterpret_cast<uint4*>(p.aux_out + (long long)row * p.ldc + col) = o;
        }
        if (p.epi == EPI_GELU) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = silu(v[j]);
        }
      } else if (p.epi == EPI_GATE_RES) {
        if (p.aux_out) {  // keep the un-gated branch output: its gradient needs it
          uint4 o;
          o.x = pack_bf16(v[0], v[1]);
          o.y = pack_bf16(v[2], v[3]);
          o.z = pack_bf16(v[4], v[5]);
          o.w = pack_bf16(v[6], v[7]);
          *reinterpret_cast<uint4*>(p.aux_out + (long long)row * p.ldc + col) = o;
        }
        uint4 rv = *reinterpret_cast<const uint4*>(p.residual + (long long)row * p.ldr + col);
        const uint32_t* ru = reinterpret_cast<const uint32_t*>(&rv);
        float4 g0 = *reinterpret_cast<const float4*>(gate_row + col);
        float4 g1 = *reinterpret_cast<const float4*>(gate_row + col + 4);
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16(ru[j]);
          v[2 * j] = f.x + gg[2 * j] * v[2 * j];
          v[2 * j + 1] = f.y + gg[2 * j + 1] * v[2 * j + 1];
        }
      } else if (p.epi == EPI_ACCUM) {
        if (p.c_fp32) {
          const float* cp = reinterpret_cast<const float*>(p.C) + (long long)row * p.ldc + col;
          float4 c0 = *reinterpret_cast<const float4*>(cp);
          float4 c1 = *reinterpret_cast<const float4*>(cp + 4);
          v[0] += c0.x; v[1] += c0.y; v[2] += c0.z; v[3] += c0.w;
          v[4] += c1.x; v[5] += c1.y; v[6] += c1.z; v[7] += c1.w;
        } else {
          uint4 cv = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.C) +
                                                     (long long)row * p.ldc + col);
          const uint32_t* cu = reinterpret_cast<const uint32_t*>(&cv);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = unpack_bf16(cu[j]);
            v[2 * j] += f.x;
            v[2 * j + 1] += f.y;
          }
        }
      }
      if (p.c_fp32) {
        float* cp = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col;
        *reinterpret_cast<float4*>(cp) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(cp + 4) = make_float4(v[4], v[5], v[6], v[7]);
      } else {
        uint4 o;
        o.x = pack_bf16(v[0], v[1]);
        o.y = pack_bf16(v[2], v[3]);
        o.z = pack_bf16(v[4], v[5]);
        o.w = pack_bf16(v[6], v[7]);
        *reinterpret_cast<uint4*>(c_row + col) = o;
      }
    }
    __syncwarp();  // tcgen05.ld is warp-collective: reconverge before the next chunk
  }
}

// EPI_QKV_A2A epilogue of one 128-row x BN accumulator tile (BN = 256, tiles never straddle the q / k / v column
// blocks because qkv_C is a multiple of 256).  Same ownership as epilogue_tile: one output row per lane, column half
// `eg` per warp.
template <int BN>
__device__ __forceinline__ void epilogue_tile_qkv(const GemmParams& p, uint32_t acc, int eg, int row, bool row_ok,
                                                  int n0) {
  const int C = p.qkv_C;
  const int part = n0 / C;  // 0 = q, 1 = k, 2 = v
  const int b = row_ok ? row / p.sc.S_l : 0;
  const int tok = row_ok ? row - b * p.sc.S_l : 0;
  bf16* c_row = reinterpret_cast<bf16*>(p.C) + (long long)row * p.ldc;
  float ss = 0.f;
#pragma unroll 1
  for (int c = eg * (BN / 64); c < (eg + 1) * (BN / 64); ++c) {
    uint32_t r[32];
    tmem_ld32(acc + (uint32_t)(c * 32), r);
    tmem_ld_wait();
    const int col0 = n0 + c * 32;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int col = col0 + g * 8;
      if (!row_ok) break;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]) * p.alpha;
      if (p.bias) {
        uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
        const uint32_t* bu = reinterpret_cast<const uint32_t*>(&bv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16(bu[j]);
          v[2 * j] += f.x;
          v[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16(v[0], v[1]);
      o.y = pack_bf16(v[2], v[3]);
      o.z = pack_bf16(v[4], v[5]);
      o.w = pack_bf16(v[6], v[7]);
      if (part < 2) {
        // statistics of the values as stored (bf16), which is what the norm's backward recomputes from
        const uint32_t* ou = reinterpret_cast<const uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16(ou[j]);
          ss += f.x * f.x + f.y * f.y;
        }
        *reinterpret_cast<uint4*>(c_row + col) = o;
      } else {
        const int cin = col - 2 * C;
        const int hd = cin / p.sc.D;
        *reinterpret_cast<uint4*>(scatter_dst(p.sc, b, tok, hd) + (cin - hd * p.sc.D)) = o;
      }
    }
    __syncwarp();  // tcgen05.ld is warp-collective: reconverge before the next chunk
  }
  if (part < 2 && row_ok) {
    const int halves = C / 128;
    p.ssq[(long long)row * (2 * halves) + part * halves + (n0 - part * C) / 128 + eg] = ss;
  }
}

}  // namespace tt_gemm
