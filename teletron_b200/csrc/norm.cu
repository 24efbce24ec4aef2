// K-ADALN, K-RMSNORM (+K-ROPE3D): row-normalisation kernels, bf16 in/out, fp32 math.
//
// adaln:  y = LN(x) * m + a   with  m = (plus_one ? 1 + mul : mul), per-sample rows of
//         mul/add (timestep modulation) or one shared row (affine LayerNorm); mul/add
//         may be null (plain LayerNorm).  Saves mean and rstd per row.
//         Backward returns dx and, per CTA, fp32 partial column sums of dy*xhat and dy,
//         which tt_colsum_partials folds into [batch, C] gradients of mul / add.
// rmsrope: y = rope(x * rsqrt(mean(x^2) + eps) * w) over the whole row (Wan q/k norm) or
//         per head of D elements (HunyuanVideo), followed by the rotary embedding on
//         interleaved (even, odd) pairs with a per-token table of (cos, sin).  Either
//         stage can be switched off.  Backward is computed from the saved input and
//         rstd (never from y / w).
//
// Successors of teletron_op/fused_adaln/{adaln_forward,adaln_backward,scale_shift_backward}.cu
// and teletron_op/fused_rmsnorm/{rms_forward,rms_backward,weight_backward}.cu; unlike those,
// any C that is a multiple of 8 up to 6144 is accepted, modulation is per sample, launches
// go to the caller's stream and every argument is validated.
#include "tt_common.cuh"

using namespace tt;

namespace {

constexpr int NT = 256;  // threads per CTA; one row per CTA iteration

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float2 block_sum2(float2 v, float2* red) {
  v.x = warp_sum(v.x);
  v.y = warp_sum(v.y);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float2 t = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) {
    t.x += red[i].x;
    t.y += red[i].y;
  }
  return t;
}

__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = unpack_bf16(w[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16(v[0], v[1]);
  o.y = pack_bf16(v[2], v[3]);
  o.z = pack_bf16(v[4], v[5]);
  o.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}
__device__ __forceinline__ void loadf8(const float* p, float (&v)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// ------------------------------------------------------------------ AdaLN forward
template <int VPT>
__global__ void __launch_bounds__(NT)
adaln_fwd_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ y, long long ldy,
                 const float* __restrict__ mul, const float* __restrict__ add, long long mod_ld,
                 int plus_one, int rows, int C, int rows_per_batch, float eps,
                 float* __restrict__ mean_out, float* __restrict__ rstd_out) {
  __shared__ float red[NT / 32];
  const int nvec = C >> 3;
  const float invC = 1.f / (float)C;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float v[VPT][8];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vec = threadIdx.x + k * NT;
      if (vec < nvec) {
        load8(x + (long long)row * ldx + vec * 8, v[k]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[k][j];
      }
    }
    const float mean = block_sum(s, red) * invC;
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vec = threadIdx.x + k * NT;
      if (vec < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[k][j] - mean;
          s2 += d * d;
        }
      }
    }
    const float rstd = rsqrtf(block_sum(s2, red) * invC + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    const long long mrow = (long long)(row / rows_per_batch) * mod_ld;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vec = threadIdx.x + k * NT;
      if (vec < nvec) {
        float m[8], a[8], o[8];
        if (mul) {
          loadf8(mul + mrow + vec * 8, m);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) m[j] = plus_one ? 0.f : 1.f;
        }
        if (add) {
          loadf8(add + mrow + vec * 8, a);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float mm = plus_one ? 1.f + m[j] : m[j];
          o[j] = (v[k][j] - mean) * rstd * mm + a[j];
        }
        store8(y + (long long)row * ldy + vec * 8, o);
      }
    }
  }
}

// One row per warp (C = NV * 256, each lane holds NV 16-byte vectors): no block-wide barrier, eight rows per CTA in
// flight.  The row-per-CTA kernel above reached a quarter of the copy bandwidth at C = 1536 (four barriers per 3 KB).
template <int NV>
__global__ void __launch_bounds__(NT, NV <= 6 ? 3 : 2)
adaln_fwd_warp_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ y, long long ldy,
                      const float* __restrict__ mul, const float* __restrict__ add, long long mod_ld,
                      int plus_one, int rows, int rows_per_batch, float eps, float* __restrict__ mean_out,
                      float* __restrict__ rstd_out) {
  constexpr int C = NV * 256;
  // the modulation rows of the first batch this CTA meets stay in shared memory: read from global for every row
  // they are four times the bytes of the row itself
  __shared__ __align__(16) float mod_s[2][C];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float invC = 1.f / (float)C;
  const int first_row = blockIdx.x * (NT / 32);
  const int cached_b = first_row < rows ? first_row / rows_per_batch : -1;
  if (cached_b >= 0) {
    for (int i = threadIdx.x; i < C; i += NT) {
      const float mv = mul ? mul[(long long)cached_b * mod_ld + i] : (plus_one ? 0.f : 1.f);
      mod_s[0][i] = plus_one ? 1.f + mv : mv;
      mod_s[1][i] = add ? add[(long long)cached_b * mod_ld + i] : 0.f;
    }
  }
  __syncthreads();
  for (int row = first_row + warp; row < rows; row += gridDim.x * (NT / 32)) {
    float v[NV][8];
    float s = 0.f;
    const bf16* xr = x + (long long)row * ldx;
#pragma unroll
    for (int k = 0; k < NV; ++k) load8(xr + (lane + k * 32) * 8, v[k]);
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[k][j];
    const float mean = warp_sum(s) * invC;
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[k][j] - mean;
        s2 += d * d;
      }
    const float rstd = rsqrtf(warp_sum(s2) * invC + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    const int rb = row / rows_per_batch;
    const long long mrow = (long long)rb * mod_ld;
    bf16* yr = y + (long long)row * ldy;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c0 = (lane + k * 32) * 8;
      float m[8], a[8], o[8];
      if (rb == cached_b) {
        loadf8(&mod_s[0][c0], m);
        loadf8(&mod_s[1][c0], a);
      } else {
        if (mul) {
          loadf8(mul + mrow + c0, m);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) m[j] = plus_one ? 0.f : 1.f;
        }
        if (plus_one) {
#pragma unroll
          for (int j = 0; j < 8; ++j) m[j] += 1.f;
        }
        if (add) {
          loadf8(add + mrow + c0, a);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] = 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[k][j] - mean) * rstd * m[j] + a[j];
      store8(yr + c0, o);
    }
  }
}

// ------------------------------------------------------------------ AdaLN backward
// grid = (chunks, batch). CTA (chunk, b) owns rows [b*rpb + chunk*rpc, min(.. + rpc, (b+1)*rpb)).
template <int VPT>
__global__ void __launch_bounds__(NT)
adaln_bwd_kernel(const bf16* __restrict__ dy, long long lddy, const bf16* __restrict__ x,
                 long long ldx, const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                 const float* __restrict__ mul, long long mod_ld, int plus_one, bf16* __restrict__ dx,
                 long long lddx, const bf16* __restrict__ dx_add, long long ldadd,
                 float* __restrict__ partial, int C, int rows_per_batch, int rows_per_chunk) {
  __shared__ float2 red[NT / 32];
  const int nvec = C >> 3;
  const float invC = 1.f / (float)C;
  const int b = blockIdx.y;
  const int chunk = blockIdx.x;
  const int r0 = chunk * rows_per_chunk;
  const int r1 = min(r0 + rows_per_chunk, rows_per_batch);
  float m[VPT][8], acc_mul[VPT][8], acc_add[VPT][8];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int vec = threadIdx.x + k * NT;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc_mul[k][j] = 0.f;
      acc_add[k][j] = 0.f;
      m[k][j] = plus_one ? 0.f : 1.f;
    }
    if (vec < nvec && mul) loadf8(mul + (long long)b * mod_ld + vec * 8, m[k]);
    if (plus_one) {
#pragma unroll
      for (int j = 0; j < 8; ++j) m[k][j] += 1.f;
    }
  }
  for (int r = r0; r < r1; ++r) {
    const long long row = (long long)b * rows_per_batch + r;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float g[VPT][8], xh[VPT][8];
    float2 s = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vec = threadIdx.x + k * NT;
      if (vec < nvec) {
        float d[8], xv[8];
        load8(dy + row * lddy + vec * 8, d);
        load8(x + row * ldx + vec * 8, xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[k][j] = (xv[j] - mean) * rstd;
          acc_mul[k][j] += d[j] * xh[k][j];
          acc_add[k][j] += d[j];
          g[k][j] = d[j] * m[k][j];
          s.x += g[k][j];
          s.y += g[k][j] * xh[k][j];
        }
      }
    }
    s = block_sum2(s, red);
    const float c1 = s.x * invC, c2 = s.y * invC;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vec = threadIdx.x + k * NT;
      if (vec < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[k][j] - c1 - xh[k][j] * c2);
        if (dx_add) {  // fold the residual-branch gradient into the same pass
          float e[8];
          load8(dx_add + row * ldadd + vec * 8, e);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += e[j];
        }
        store8(dx + row * lddx + vec * 8, o);
      }
    }
  }
  if (partial) {
    float* pm = partial + ((long long)(b * gridDim.x + chunk) * 2) * C;
    float* pa = pm + C;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vec = threadIdx.x + k * NT;
      if (vec < nvec) {
        *reinterpret_cast<float4*>(pm + vec * 8) = make_float4(acc_mul[k][0], acc_mul[k][1], acc_mul[k][2], acc_mul[k][3]);
        *reinterpret_cast<float4*>(pm + vec * 8 + 4) = make_float4(acc_mul[k][4], acc_mul[k][5], acc_mul[k][6], acc_mul[k][7]);
        *reinterpret_cast<float4*>(pa + vec * 8) = make_float4(acc_add[k][0], acc_add[k][1], acc_add[k][2], acc_add[k][3]);
        *reinterpret_cast<float4*>(pa + vec * 8 + 4) = make_float4(acc_add[k][4], acc_add[k][5], acc_add[k][6], acc_add[k][7]);
      }
    }
  }
}

// out[g, c] (+)= sum_{i < n} partial[g*stride_g + i*stride_n + c]  (fixed order => deterministic)
// A CTA covers 32 columns; its 8 warps take every 8th partial row with four loads in flight each, then the 8 slice
// sums are added in a fixed order (one thread walking all n rows took 47 us for n = 592).
__global__ void __launch_bounds__(256)
colsum_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int groups, int n, int width,
                       long long stride_g, long long stride_n, int accumulate) {
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  const int g = blockIdx.y;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < width) {
    const float* p = partial + (long long)g * stride_g + c;
    int i = slice;
    for (; i + 24 < n; i += 32) {
      s0 += p[(long long)i * stride_n];
      s1 += p[(long long)(i + 8) * stride_n];
      s2 += p[(long long)(i + 16) * stride_n];
      s3 += p[(long long)(i + 24) * stride_n];
    }
    for (; i < n; i += 8) s0 += p[(long long)i * stride_n];
  }
  red[slice][lane] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (slice == 0 && c < width) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][lane];
    float* o = out + (long long)g * width + c;
    *o = accumulate ? *o + t : t;
  }
}

// ------------------------------------------------------------------ RMSNorm + RoPE
// norm_dim == C : statistics over the whole row; norm_dim == D : per head (16 threads own
// one head of 128). w may be null (no norm), freqs may be null (no rotary).
template <int VPT, bool BWD>
__global__ void __launch_bounds__(NT)
rmsrope_kernel(const bf16* __restrict__ in, long long ldi, const bf16* __restrict__ xsave,
               long long ldx, bf16* __restrict__ out, long long ldo, const float* __restrict__ w,
               const float2* __restrict__ freqs, int freq_rows, float* __restrict__ rstd_io,
               float* __restrict__ partial, int rows, int C, int D, int per_head, float eps,
               int rows_per_cta, const TTScatter sc, const float* __restrict__ ssq = nullptr, int ssq_n = 0,
               long long ssq_ld = 0) {
  __shared__ float red[NT / 32];
  const int nvec = C >> 3;
  const int vec_per_head = D >> 3;
  const int H = C / D;
  float accw[VPT][8];
  float wv[VPT][8];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int vec = threadIdx.x + k * NT;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      accw[k][j] = 0.f;
      wv[k][j] = 1.f;
    }
    if (w && vec < nvec) loadf8(w + (per_head ? (vec % vec_per_head) * 8 : vec * 8), wv[k]);
  }
  const int r0 = blockIdx.x * rows_per_cta;
  const int r1 = min(r0 + rows_per_cta, rows);
  for (int row = r0; row < r1; ++row) {
    float v[VPT][8];  // forward: x ; backward: dy then g
    float cs[VPT][8];
    const float2* frow = freqs ? freqs + (long long)(row % freq_rows) * (D >> 1) : nullptr;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vec = threadIdx.x + k * NT;
      if (vec < nvec) {
        load8(in + (long long)row * ldi + vec * 8, v[k]);
        if (frow) loadf8(reinterpret_cast<const float*>(frow + (vec % vec_per_head) * 4), cs[k]);
      }
    }
    if (!BWD) {
      float rs[VPT];
      if (w) {
        float ss[VPT];
        float tot = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          ss[k] = 0.f;
          if (threadIdx.x + k * NT < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) ss[k] += v[k][j] * v[k][j];
          }
          tot += ss[k];
        }
        if (per_head) {
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            float t = ss[k];
            for (int o = vec_per_head >> 1; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            rs[k] = rsqrtf(t / (float)D + eps);
            const int vec = threadIdx.x + k * NT;
            if (vec < nvec && (vec % vec_per_head) == 0 && rstd_io)
              rstd_io[(long long)row * H + vec / vec_per_head] = rs[k];
          }
        } else {
          float full;
          if (ssq) {  // row statistics from the GEMM that wrote this row; same value in every thread
            full = 0.f;
            for (int j = 0; j < ssq_n; ++j) full += ssq[(long long)row * ssq_ld + j];
          } else {
            full = block_sum(tot, red);
          }
          const float r = rsqrtf(full / (float)C + eps);
#pragma unroll
          for (int k = 0; k < VPT; ++k) rs[k] = r;
          if (threadIdx.x == 0 && rstd_io) rstd_io[row] = r;
        }
      } else {
#pragma unroll
        for (int k = 0; k < VPT; ++k) rs[k] = 1.f;
      }
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int vec = threadIdx.x + k * NT;
        if (vec < nvec) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[k][j] * rs[k] * wv[k][j];
          if (frow) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float c = cs[k][2 * j], s = cs[k][2 * j + 1];
              const float a = o[2 * j], b = o[2 * j + 1];
              o[2 * j] = a * c - b * s;
              o[2 * j + 1] = a * s + b * c;
            }
          }
          if (sc.mode == 0) {
            store8(out + (long long)row * ldo + vec * 8, o);
          } else {  // all-to-all fused into the store: write straight into the owning peer's buffer
            const int col = vec * 8;
            const int hd = col / D;
            store8(scatter_dst(sc, row / sc.S_l, row % sc.S_l, hd) + (col - hd * D), o);
          }
        }
      }
    } else {
      // backward: v = dy. un-rotate, then norm backward from saved x and rstd.
      float xh[VPT][8];
      float dot[VPT];
      float tot = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        dot[k] = 0.f;
        const int vec = threadIdx.x + k * NT;
        if (vec < nvec) {
          if (frow) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float c = cs[k][2 * j], s = cs[k][2 * j + 1];
              const float a = v[k][2 * j], b = v[k][2 * j + 1];
              v[k][2 * j] = a * c + b * s;
              v[k][2 * j + 1] = -a * s + b * c;
            }
          }
          if (w) {
            float xv[8];
            load8(xsave + (long long)row * ldx + vec * 8, xv);
            const float r = per_head ? rstd_io[(long long)row * H + vec / vec_per_head] : rstd_io[row];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              xh[k][j] = xv[j] * r;
              accw[k][j] += v[k][j] * xh[k][j];
              v[k][j] *= wv[k][j];
              dot[k] += v[k][j] * xh[k][j];
            }
          }
        }
        tot += dot[k];
      }
      if (w) {
        float full = 0.f;
        if (!per_head) full = block_sum(tot, red) / (float)C;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int vec = threadIdx.x + k * NT;
          float sdot;
          if (per_head) {
            float t = dot[k];
            for (int o = vec_per_head >> 1; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            sdot = t / (float)D;
          } else {
            sdot = full;
          }
          if (vec < nvec) {
            const float r = per_head ? rstd_io[(long long)row * H + vec / vec_per_head] : rstd_io[row];
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = r * (v[k][j] - xh[k][j] * sdot);
            store8(out + (long long)row * ldo + vec * 8, o);
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int vec = threadIdx.x + k * NT;
          if (vec < nvec) store8(out + (long long)row * ldo + vec * 8, v[k]);
        }
      }
    }
  }
  if (BWD && partial && w) {
    float* pw = partial + (long long)blockIdx.x * C;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vec = threadIdx.x + k * NT;
      if (vec < nvec) {
        *reinterpret_cast<float4*>(pw + vec * 8) = make_float4(accw[k][0], accw[k][1], accw[k][2], accw[k][3]);
        *reinterpret_cast<float4*>(pw + vec * 8 + 4) = make_float4(accw[k][4], accw[k][5], accw[k][6], accw[k][7]);
      }
    }
  }
}

int vpt_for(int C) { return (C / 8 + NT - 1) / NT; }
bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

#define TT_DISPATCH_VPT(vpt, ...)            \
  switch (vpt) {                             \
    case 1: { constexpr int VPT = 1; __VA_ARGS__; } break; \
    case 2: { constexpr int VPT = 2; __VA_ARGS__; } break; \
    case 3: { constexpr int VPT = 3; __VA_ARGS__; } break; \
    default: tt_set_error("row width too large (max 6144)"); return -1; \
  }

TT_API int tt_adaln_fwd(const void* x, long long ldx, void* y, long long ldy, const float* mul,
                        const float* add, long long mod_ld, int plus_one, int rows, int C,
                        int rows_per_batch, float eps, float* mean_out, float* rstd_out,
                        cudaStream_t stream) {
  TT_CHECK(rows > 0 && C > 0 && C % 8 == 0 && C <= 6144, "adaln_fwd: bad shape rows=%d C=%d", rows, C);
  TT_CHECK(ldx % 8 == 0 && ldy % 8 == 0 && mod_ld % 4 == 0, "adaln_fwd: leading dims misaligned");
  TT_CHECK(aligned16(x) && aligned16(y) && aligned16(mul) && aligned16(add), "adaln_fwd: misaligned pointer");
  TT_CHECK(rows_per_batch > 0, "adaln_fwd: rows_per_batch must be positive");
  if (C % 256 == 0 && C <= 3072) {  // one row per warp
    const int want = (rows + NT / 32 - 1) / (NT / 32);
    const int wgrid = want < 148 * 8 ? want : 148 * 8;
#define TT_ADALN_WARP(NVV)                                                                                   \
  adaln_fwd_warp_kernel<NVV><<<wgrid, NT, 0, stream>>>((const bf16*)x, ldx, (bf16*)y, ldy, mul, add, mod_ld, \
                                                       plus_one, rows, rows_per_batch, eps, mean_out, rstd_out)
    switch (C / 256) {
      case 1: TT_ADALN_WARP(1); break;
      case 2: TT_ADALN_WARP(2); break;
      case 3: TT_ADALN_WARP(3); break;
      case 4: TT_ADALN_WARP(4); break;
      case 5: TT_ADALN_WARP(5); break;
      case 6: TT_ADALN_WARP(6); break;
      case 7: TT_ADALN_WARP(7); break;
      case 8: TT_ADALN_WARP(8); break;
      case 9: TT_ADALN_WARP(9); break;
      case 10: TT_ADALN_WARP(10); break;
      case 11: TT_ADALN_WARP(11); break;
      default: TT_ADALN_WARP(12); break;
    }
#undef TT_ADALN_WARP
    TT_LAUNCH_CHECK();
    return 0;
  }
  const int grid = rows < 148 * 16 ? rows : 148 * 16;
  TT_DISPATCH_VPT(vpt_for(C), adaln_fwd_kernel<VPT><<<grid, NT, 0, stream>>>(
      (const bf16*)x, ldx, (bf16*)y, ldy, mul, add, mod_ld, plus_one, rows, C, rows_per_batch, eps,
      mean_out, rstd_out));
  TT_LAUNCH_CHECK();
  return 0;
}

// partial: fp32 [batch, chunks, 2, C] scratch (may be null when no mul/add gradient is wanted).
// dmul / dadd: fp32 [batch, C] (either may be null). accumulate: add into them.
TT_API int tt_adaln_bwd(const void* dy, long long lddy, const void* x, long long ldx,
                        const float* mean, const float* rstd, const float* mul, long long mod_ld,
                        int plus_one, void* dx, long long lddx, const void* dx_add, long long ldadd,
                        float* partial, int chunks, float* dmul, float* dadd, int accumulate,
                        int batch, int rows_per_batch, int C, cudaStream_t stream) {
  TT_CHECK(batch > 0 && rows_per_batch > 0 && C % 8 == 0 && C <= 6144, "adaln_bwd: bad shape");
  TT_CHECK(chunks > 0, "adaln_bwd: chunks must be positive");
  TT_CHECK(lddy % 8 == 0 && ldx % 8 == 0 && lddx % 8 == 0 && mod_ld % 4 == 0 && ldadd % 8 == 0,
           "adaln_bwd: leading dims misaligned");
  TT_CHECK(aligned16(dy) && aligned16(x) && aligned16(dx) && aligned16(mul) && aligned16(partial) &&
               aligned16(dx_add),
           "adaln_bwd: misaligned pointer");
  const int rpc = (rows_per_batch + chunks - 1) / chunks;
  dim3 grid(chunks, batch);
  TT_DISPATCH_VPT(vpt_for(C), adaln_bwd_kernel<VPT><<<grid, NT, 0, stream>>>(
      (const bf16*)dy, lddy, (const bf16*)x, ldx, mean, rstd, mul, mod_ld, plus_one, (bf16*)dx, lddx,
      (const bf16*)dx_add, ldadd, partial, C, rows_per_batch, rpc));
  TT_LAUNCH_CHECK();
  if (partial && (dmul || dadd)) {
    dim3 g2((C + 31) / 32, batch);
    const long long sg = (long long)chunks * 2 * C, sn = 2ll * C;
    if (dmul) {
      colsum_partials_kernel<<<g2, 256, 0, stream>>>(partial, dmul, batch, chunks, C, sg, sn, accumulate);
      TT_LAUNCH_CHECK();
    }
    if (dadd) {
      colsum_partials_kernel<<<g2, 256, 0, stream>>>(partial + C, dadd, batch, chunks, C, sg, sn, accumulate);
      TT_LAUNCH_CHECK();
    }
  }
  return 0;
}

TT_API int tt_colsum_partials(const float* partial, float* out, int groups, int n, int width,
                              int accumulate, cudaStream_t stream) {
  TT_CHECK(groups > 0 && n > 0 && width > 0, "colsum_partials: bad shape");
  dim3 grid((width + 31) / 32, groups);
  colsum_partials_kernel<<<grid, 256, 0, stream>>>(partial, out, groups, n, width, (long long)n * width, (long long)width, accumulate);
  TT_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------ RMSNorm + RoPE, one row per warp
// Full-row statistics only (Wan q / k norm), C = NV * 256: each lane holds NV 16-byte vectors of the row, the
// reductions are warp shuffles, eight rows per CTA are in flight.  The row-per-CTA kernel above reached a third of the
// copy bandwidth at C = 1536 (two block barriers per 3 KB row).  The weight row lives in shared memory.
template <int NV>
__global__ void __launch_bounds__(NT, 2)
rmsrope_fwd_warp_kernel(const bf16* __restrict__ in, long long ldi, bf16* __restrict__ out, long long ldo,
                        const float* __restrict__ w, const float2* __restrict__ freqs, int freq_rows,
                        float* __restrict__ rstd_io, int rows, int D, float eps, const TTScatter sc,
                        const float* __restrict__ ssq, int ssq_n, long long ssq_ld) {
  constexpr int C = NV * 256;
  __shared__ __align__(16) float w_s[C];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vec_per_head = D >> 3;
  for (int i = threadIdx.x; i < C; i += NT) w_s[i] = w ? w[i] : 1.f;
  __syncthreads();
  for (int row = blockIdx.x * (NT / 32) + warp; row < rows; row += gridDim.x * (NT / 32)) {
    float v[NV][8];
    const float2* frow = freqs ? freqs + (long long)(row % freq_rows) * (D >> 1) : nullptr;
    const bf16* xr = in + (long long)row * ldi;
#pragma unroll
    for (int k = 0; k < NV; ++k) load8(xr + (lane + k * 32) * 8, v[k]);
    float r = 1.f;
    if (w) {
      float tot = 0.f;
      if (ssq) {  // row statistics already produced (per 128-column piece) by the GEMM that wrote this row
        for (int j = 0; j < ssq_n; ++j) tot += ssq[(long long)row * ssq_ld + j];
      } else {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < NV; ++k)
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += v[k][j] * v[k][j];
        tot = warp_sum(ss);
      }
      r = rsqrtf(tot / (float)C + eps);
      if (lane == 0 && rstd_io) rstd_io[row] = r;
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vec = lane + k * 32;
      float o[8], wk[8];
      loadf8(&w_s[vec * 8], wk);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[k][j] * r * wk[j];
      if (frow) {
        float cs[8];
        loadf8(reinterpret_cast<const float*>(frow + (vec % vec_per_head) * 4), cs);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float c = cs[2 * j], sn = cs[2 * j + 1];
          const float a = o[2 * j], b = o[2 * j + 1];
          o[2 * j] = a * c - b * sn;
          o[2 * j + 1] = a * sn + b * c;
        }
      }
      if (sc.mode == 0) {
        store8(out + (long long)row * ldo + vec * 8, o);
      } else {  // all-to-all fused into the store: write straight into the owning peer's buffer
        const int col = vec * 8;
        const int hd = col / D;
        store8(scatter_dst(sc, row / sc.S_l, row % sc.S_l, hd) + (col - hd * D), o);
      }
    }
  }
}

// backward of the above.  Each warp keeps its weight-gradient sums in its own shared-memory slab (48 registers per
// lane otherwise); at the end the CTA's eight slabs are added in a fixed order into one partial row.
template <int NV>
__global__ void __launch_bounds__(NT, 2)
rmsrope_bwd_warp_kernel(const bf16* __restrict__ dy, long long lddy, const bf16* __restrict__ xsave, long long ldx,
                        bf16* __restrict__ dx, long long lddx, const float* __restrict__ w,
                        const float2* __restrict__ freqs, int freq_rows, const float* __restrict__ rstd_io,
                        float* __restrict__ partial, int rows, int D) {
  constexpr int C = NV * 256;
  extern __shared__ __align__(16) float dyn_s[];   // [1 + 8 warps][C]: weight row, then one slab per warp
  float* w_s = dyn_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* acc_s = dyn_s + (1 + warp) * C;
  const int vec_per_head = D >> 3;
  for (int i = threadIdx.x; i < C; i += NT) w_s[i] = w ? w[i] : 1.f;
  for (int i = threadIdx.x; i < (NT / 32) * C; i += NT) dyn_s[C + i] = 0.f;
  __syncthreads();
  for (int row = blockIdx.x * (NT / 32) + warp; row < rows; row += gridDim.x * (NT / 32)) {
    float v[NV][8], xh[NV][8];
    const float2* frow = freqs ? freqs + (long long)(row % freq_rows) * (D >> 1) : nullptr;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vec = lane + k * 32;
      load8(dy + (long long)row * lddy + vec * 8, v[k]);
      if (w) load8(xsave + (long long)row * ldx + vec * 8, xh[k]);
    }
    if (frow) {
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        float cs[8];
        loadf8(reinterpret_cast<const float*>(frow + ((lane + k * 32) % vec_per_head) * 4), cs);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float c = cs[2 * j], sn = cs[2 * j + 1];
          const float a = v[k][2 * j], b = v[k][2 * j + 1];
          v[k][2 * j] = a * c + b * sn;
          v[k][2 * j + 1] = -a * sn + b * c;
        }
      }
    }
    if (w) {
      const float r = rstd_io[row];
      float dot = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int c0 = (lane + k * 32) * 8;
        float wk[8], ak[8];
        loadf8(&w_s[c0], wk);
        loadf8(&acc_s[c0], ak);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[k][j] *= r;
          ak[j] += v[k][j] * xh[k][j];
          v[k][j] *= wk[j];
          dot += v[k][j] * xh[k][j];
        }
        *reinterpret_cast<float4*>(&acc_s[c0]) = make_float4(ak[0], ak[1], ak[2], ak[3]);
        *reinterpret_cast<float4*>(&acc_s[c0 + 4]) = make_float4(ak[4], ak[5], ak[6], ak[7]);
      }
      const float sdot = warp_sum(dot) / (float)C;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * (v[k][j] - xh[k][j] * sdot);
        store8(dx + (long long)row * lddx + (lane + k * 32) * 8, o);
      }
    } else {
#pragma unroll
      for (int k = 0; k < NV; ++k) store8(dx + (long long)row * lddx + (lane + k * 32) * 8, v[k]);
    }
  }
  if (partial && w) {
    __syncthreads();
    float* pw = partial + (long long)blockIdx.x * C;
    for (int c = threadIdx.x; c < C; c += NT) {
      float t = 0.f;
#pragma unroll
      for (int ww = 0; ww < NT / 32; ++ww) t += dyn_s[(1 + ww) * C + c];
      pw[c] = t;
    }
  }
}

// Forward: in = x. Saves rstd ([rows] or [rows, H]) when w != null.
static int rmsrope_fwd_impl(const void* x, long long ldx, void* y, long long ldy, const float* w,
                            const void* freqs, int freq_rows, float* rstd, int rows, int C, int D,
                            int per_head, float eps, const TTScatter& sc, cudaStream_t stream,
                            const float* ssq = nullptr, int ssq_n = 0, long long ssq_ld = 0) {
  TT_CHECK(ssq == nullptr || (!per_head && w != nullptr && ssq_n > 0 && ssq_ld >= ssq_n),
           "rmsrope_fwd: precomputed row statistics go with the full-row norm");
  TT_CHECK(rows > 0 && C % 8 == 0 && C <= 6144 && D > 0 && C % D == 0, "rmsrope_fwd: bad shape");
  TT_CHECK(!per_head || (D == 128 || D == 64), "rmsrope_fwd: per-head norm supports D = 64 or 128");
  TT_CHECK(freqs == nullptr || (D % 8 == 0 && freq_rows > 0), "rmsrope_fwd: bad rotary table");
  TT_CHECK(ldx % 8 == 0 && ldy % 8 == 0, "rmsrope_fwd: leading dims misaligned");
  TT_CHECK(aligned16(x) && aligned16(y) && aligned16(w) && aligned16(freqs), "rmsrope_fwd: misaligned pointer");
  if (!per_head && C % 256 == 0 && C <= 2048) {  // one row per warp
    const int want = (rows + NT / 32 - 1) / (NT / 32);
    const int wgrid = want < 148 * 8 ? want : 148 * 8;
#define TT_RMS_FWD_WARP(NVV)                                                                                        \
  rmsrope_fwd_warp_kernel<NVV><<<wgrid, NT, 0, stream>>>((const bf16*)x, ldx, (bf16*)y, ldy, w, (const float2*)freqs, \
                                                         freq_rows, rstd, rows, D, eps, sc, ssq, ssq_n, ssq_ld)
    switch (C / 256) {
      case 1: TT_RMS_FWD_WARP(1); break;
      case 2: TT_RMS_FWD_WARP(2); break;
      case 3: TT_RMS_FWD_WARP(3); break;
      case 4: TT_RMS_FWD_WARP(4); break;
      case 5: TT_RMS_FWD_WARP(5); break;
      case 6: TT_RMS_FWD_WARP(6); break;
      case 7: TT_RMS_FWD_WARP(7); break;
      default: TT_RMS_FWD_WARP(8); break;
    }
#undef TT_RMS_FWD_WARP
    TT_LAUNCH_CHECK();
    return 0;
  }
  const int rpc = rows > 148 * 32 ? (rows + 148 * 16 - 1) / (148 * 16) : 1;
  const int grid = (rows + rpc - 1) / rpc;
  TT_DISPATCH_VPT(vpt_for(C), rmsrope_kernel<VPT, false><<<grid, NT, 0, stream>>>(
      (const bf16*)x, ldx, nullptr, 0, (bf16*)y, ldy, w, (const float2*)freqs, freq_rows, rstd,
      nullptr, rows, C, D, per_head, eps, rpc, sc, ssq, ssq_n, ssq_ld));
  TT_LAUNCH_CHECK();
  return 0;
}

TT_API int tt_rmsrope_fwd(const void* x, long long ldx, void* y, long long ldy, const float* w,
                          const void* freqs, int freq_rows, float* rstd, int rows, int C, int D,
                          int per_head, float eps, cudaStream_t stream) {
  TTScatter sc;
  memset(&sc, 0, sizeof(sc));
  return rmsrope_fwd_impl(x, ldx, y, ldy, w, freqs, freq_rows, rstd, rows, C, D, per_head, eps, sc, stream);
}

// Same as tt_rmsrope_fwd, but the result is stored into peer memory with the Ulysses seq -> head
// pattern (TTScatter mode 1): x is this rank's [B*S_l, H*D] shard, the output lands in every
// peer's [B, S_pad, ceil(H / world), D] buffer. peer_ptrs: `world` device addresses of those buffers.
// ssq (optional): [rows, ssq_ld] fp32 whose first ssq_n entries per row add up to the row's sum of squares
// (written by tt_gemm_qkv_a2a), used instead of reducing the row again.  dst_rows (0 = S_pad): rows per sample of the
// peers' buffers when they hold more than the exchanged tokens (joint video + text sequences).
TT_API int tt_rmsrope_fwd_scatter(const void* x, long long ldx, const float* w, const void* freqs,
                                  int freq_rows, float* rstd, int rows, int C, int D, int per_head,
                                  float eps, const long long* peer_ptrs, int world, int rank, int S_l,
                                  int S_pad, const float* ssq, int ssq_n, long long ssq_ld, int dst_rows,
                                  cudaStream_t stream) {
  TT_CHECK(dst_rows == 0 || dst_rows >= S_pad, "rmsrope_fwd_scatter: destination holds fewer rows than the sequence");
  TT_CHECK(world >= 1 && world <= TT_MAX_PEERS && rank >= 0 && rank < world, "rmsrope_fwd_scatter: bad world/rank");
  const int H = C / D;
  TT_CHECK(S_l > 0 && S_pad == S_l * world && rows % S_l == 0, "rmsrope_fwd_scatter: bad sequence split");
  TTScatter sc;
  memset(&sc, 0, sizeof(sc));
  for (int i = 0; i < world; ++i) {
    sc.peer[i] = reinterpret_cast<void*>(peer_ptrs[i]);
    TT_CHECK(sc.peer[i] && ((uintptr_t)sc.peer[i] & 15) == 0, "rmsrope_fwd_scatter: bad peer pointer %d", i);
  }
  sc.mode = 1; sc.S_l = S_l; sc.S_pad = S_pad; sc.Hl = (H + world - 1) / world; sc.H = H; sc.D = D; sc.rank = rank;
  sc.world = world; sc.dst_rows = dst_rows;
  return rmsrope_fwd_impl(x, ldx, const_cast<void*>(x), ldx, w, freqs, freq_rows, rstd, rows, C, D, per_head, eps, sc,
                          stream, ssq, ssq_n, ssq_ld);
}

// Backward: dy -> dx, with x (saved forward input) and rstd. partial: fp32 [ctas, C] scratch for
// the weight gradient, ctas = tt_rmsrope_bwd_ctas(rows); fold it with tt_colsum_partials.
TT_API int tt_rmsrope_bwd_ctas(int rows) {
  const int rpc = (rows + 592 - 1) / 592;
  return (rows + rpc - 1) / rpc;
}
TT_API int tt_rmsrope_bwd(const void* dy, long long lddy, const void* x, long long ldx, void* dx,
                          long long lddx, const float* w, const void* freqs, int freq_rows,
                          float* rstd, float* partial, int rows, int C, int D, int per_head,
                          cudaStream_t stream) {
  TT_CHECK(rows > 0 && C % 8 == 0 && C <= 6144 && D > 0 && C % D == 0, "rmsrope_bwd: bad shape");
  TT_CHECK(!per_head || (D == 128 || D == 64), "rmsrope_bwd: per-head norm supports D = 64 or 128");
  TT_CHECK(lddy % 8 == 0 && ldx % 8 == 0 && lddx % 8 == 0, "rmsrope_bwd: leading dims misaligned");
  TT_CHECK(aligned16(dy) && aligned16(x) && aligned16(dx) && aligned16(w) && aligned16(freqs) &&
               aligned16(partial),
           "rmsrope_bwd: misaligned pointer");
  TT_CHECK(w == nullptr || (x != nullptr && rstd != nullptr), "rmsrope_bwd: norm backward needs x and rstd");
  const int rpc = (rows + 592 - 1) / 592;
  const int grid = (rows + rpc - 1) / rpc;  // = tt_rmsrope_bwd_ctas(rows): the number of partial rows the caller folds
  if (!per_head && C % 256 == 0 && C <= 2048) {  // one row per warp; every CTA writes its partial row (zeros if idle)
    const int dyn = 9 * C * 4;  // weight row + eight per-warp gradient slabs
#define TT_RMS_BWD_WARP(NVV)                                                                                            \
  do {                                                                                                                  \
    static bool attr_##NVV = false;                                                                                      \
    if (!attr_##NVV) {                                                                                                   \
      TT_CUDA(cudaFuncSetAttribute(rmsrope_bwd_warp_kernel<NVV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 9 * NVV * 256 * 4)); \
      attr_##NVV = true;                                                                                                 \
    }                                                                                                                   \
    rmsrope_bwd_warp_kernel<NVV><<<grid, NT, dyn, stream>>>((const bf16*)dy, lddy, (const bf16*)x, ldx, (bf16*)dx, lddx, \
                                                            w, (const float2*)freqs, freq_rows, rstd, partial, rows, D); \
  } while (0)
    switch (C / 256) {
      case 1: TT_RMS_BWD_WARP(1); break;
      case 2: TT_RMS_BWD_WARP(2); break;
      case 3: TT_RMS_BWD_WARP(3); break;
      case 4: TT_RMS_BWD_WARP(4); break;
      case 5: TT_RMS_BWD_WARP(5); break;
      case 6: TT_RMS_BWD_WARP(6); break;
      case 7: TT_RMS_BWD_WARP(7); break;
      default: TT_RMS_BWD_WARP(8); break;
    }
#undef TT_RMS_BWD_WARP
    TT_LAUNCH_CHECK();
    return 0;
  }
  TT_DISPATCH_VPT(vpt_for(C), rmsrope_kernel<VPT, true><<<grid, NT, 0, stream>>>(
      (const bf16*)dy, lddy, (const bf16*)x, ldx, (bf16*)dx, lddx, w, (const float2*)freqs, freq_rows,
      rstd, partial, rows, C, D, per_head, 0.f, rpc, TTScatter{}));
  TT_LAUNCH_CHECK();
  return 0;
}
