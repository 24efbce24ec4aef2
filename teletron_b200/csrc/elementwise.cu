// K-MISC: memory-bound kernels around the GEMMs. bf16 tensors, fp32 math, 16-byte accesses.
//
//   act_bwd          dpre = dact * f'(pre)                 f = GELU(tanh) or SiLU
//   gate_bwd         dy = gate[b,:] * dout ; partial column sums of dout*y (for dgate)
//   colsum           out[c] = sum_rows x[r,c]              (bias gradients), two-stage
//   adamw            fused AdamW over flat fp32 master / m / v buffers with bf16 write-back
//   sumsq            partial sums of squares of a flat fp32 buffer (gradient norm)
//   flow_mse         loss = w * mean((pred - (noise - x0))^2) and dpred in one pass
//   add_noise        x_t = (1 - sigma) x0 + sigma * noise
//
// Replace the unfused ATen chains and apex multi-tensor kernels the reference relies on
// (teletron/core/context_parallel/layers.py:24-53, teletron/train/lr_scheduler.py:16,
// teletron/models/flow_match.py:62-73).
#include "tt_common.cuh"

using namespace tt;

namespace {

__device__ __forceinline__ void ld8(const bf16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = unpack_bf16(w[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ void st8(bf16* p, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16(v[0], v[1]);
  o.y = pack_bf16(v[2], v[3]);
  o.z = pack_bf16(v[4], v[5]);
  o.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// ---------------------------------------------------------------- activation backward
__global__ void act_bwd_kernel(const bf16* __restrict__ dact, long long ldd, const bf16* __restrict__ pre,
                               long long ldp, bf16* __restrict__ dpre, long long ldo, int rows, int C,
                               int kind) {
  const int nvec = C >> 3;
  const long long total = (long long)rows * nvec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / nvec;
    const int c = (int)(idx % nvec) * 8;
    float d[8], x[8], o[8];
    ld8(dact + r * ldd + c, d);
    ld8(pre + r * ldp + c, x);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = d[j] * (kind == 0 ? gelu_tanh_grad(x[j]) : silu_grad(x[j]));
    st8(dpre + r * ldo + c, o);
  }
}

// ---------------------------------------------------------------- gate backward
// grid (chunks, batch), 256 threads; thread owns vectors tid + k*256 (C <= 6144).
template <int VPT>
__global__ void __launch_bounds__(256)
gate_bwd_kernel(const bf16* __restrict__ dout, long long ldd, const bf16* __restrict__ y, long long ldy,
                const float* __restrict__ gate, long long gate_ld, bf16* __restrict__ dy, long long lddy,
                float* __restrict__ partial, int C, int rows_per_batch, int rows_per_chunk) {
  const int nvec = C >> 3;
  const int b = blockIdx.y, chunk = blockIdx.x;
  const int r0 = chunk * rows_per_chunk;
  const int r1 = min(r0 + rows_per_chunk, rows_per_batch);
  float g[VPT][8], acc[VPT][8];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int vec = threadIdx.x + k * 256;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc[k][j] = 0.f;
      g[k][j] = 0.f;
    }
    if (vec < nvec) {
      float4 a = *reinterpret_cast<const float4*>(gate + (long long)b * gate_ld + vec * 8);
      float4 c = *reinterpret_cast<const float4*>(gate + (long long)b * gate_ld + vec * 8 + 4);
      g[k][0] = a.x; g[k][1] = a.y; g[k][2] = a.z; g[k][3] = a.w;
      g[k][4] = c.x; g[k][5] = c.y; g[k][6] = c.z; g[k][7] = c.w;
    }
  }
  for (int r = r0; r < r1; ++r) {
    const long long row = (long long)b * rows_per_batch + r;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vec = threadIdx.x + k * 256;
      if (vec < nvec) {
        float d[8], yy[8], o[8];
        ld8(dout + row * ldd + vec * 8, d);
        ld8(y + row * ldy + vec * 8, yy);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[k][j] += d[j] * yy[j];
          o[j] = d[j] * g[k][j];
        }
        st8(dy + row * lddy + vec * 8, o);
      }
    }
  }
  float* pp = partial + (long long)(b * gridDim.x + chunk) * C;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int vec = threadIdx.x + k * 256;
    if (vec < nvec) {
      *reinterpret_cast<float4*>(pp + vec * 8) = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
      *reinterpret_cast<float4*>(pp + vec * 8 + 4) = make_float4(acc[k][4], acc[k][5], acc[k][6], acc[k][7]);
    }
  }
}

// ---------------------------------------------------------------- column sums (bias grads)
// stage 1: grid (ceil(C/8/256), chunks): partial[chunk, c] = sum over the chunk's rows
__global__ void __launch_bounds__(256)
colsum_stage1_kernel(const bf16* __restrict__ x, long long ldx, float* __restrict__ partial, int rows,
                     int C, int rows_per_chunk) {
  const int vec = blockIdx.x * 256 + threadIdx.x;
  if (vec >= (C >> 3)) return;
  const int r0 = blockIdx.y * rows_per_chunk;
  const int r1 = min(r0 + rows_per_chunk, rows);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  int r = r0;
  for (; r + 3 < r1; r += 4) {  // four independent 16-byte loads in flight per thread
    float v0[8], v1[8], v2[8], v3[8];
    const bf16* px = x + (long long)r * ldx + vec * 8;
    ld8(px, v0);
    ld8(px + ldx, v1);
    ld8(px + 2 * ldx, v2);
    ld8(px + 3 * ldx, v3);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += (v0[j] + v1[j]) + (v2[j] + v3[j]);
  }
  for (; r < r1; ++r) {
    float v[8];
    ld8(x + (long long)r * ldx + vec * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += v[j];
  }
  float* pp = partial + (long long)blockIdx.y * C + vec * 8;
  *reinterpret_cast<float4*>(pp) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  *reinterpret_cast<float4*>(pp + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
}
// stage 2: a CTA covers 32 columns, its 8 warps take every 8th chunk; slice sums are added in a fixed order
__global__ void __launch_bounds__(256)
colsum_stage2_kernel(const float* __restrict__ partial, void* __restrict__ out, int n, int C, int out_fp32,
                     int accumulate) {
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s0 = 0.f, s1 = 0.f;
  if (c < C) {
    int i = slice;
    for (; i + 8 < n; i += 16) {
      s0 += partial[(long long)i * C + c];
      s1 += partial[(long long)(i + 8) * C + c];
    }
    for (; i < n; i += 8) s0 += partial[(long long)i * C + c];
  }
  red[slice][lane] = s0 + s1;
  __syncthreads();
  if (slice != 0 || c >= C) return;
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) s += red[k][lane];
  if (out_fp32) {
    float* o = reinterpret_cast<float*>(out) + c;
    *o = accumulate ? *o + s : s;
  } else {
    bf16* o = reinterpret_cast<bf16*>(out) + c;
    *o = __float2bfloat16(accumulate ? __bfloat162float(*o) + s : s);
  }
}

// ---------------------------------------------------------------- AdamW
// p32/m/v/g: flat fp32; p16: bf16 copy of the parameters that the model computes with.
// grad_scale multiplies the gradient first (clip coefficient x 1/accumulation);
// found_inf (optional) skips the whole update when non-zero.
__global__ void adamw_kernel(float* __restrict__ p32, bf16* __restrict__ p16, float* __restrict__ m,
                             float* __restrict__ v, const float* __restrict__ g, long long n, float lr,
                             float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ grad_scale_ptr, float grad_scale,
                             const int* __restrict__ found_inf) {
  if (found_inf && *found_inf) return;
  const float gs = grad_scale_ptr ? grad_scale * (*grad_scale_ptr) : grad_scale;
  const long long nv = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p32)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float P[4] = {pp.x, pp.y, pp.z, pp.w}, M[4] = {mm.x, mm.y, mm.z, mm.w};
    float V[4] = {vv.x, vv.y, vv.z, vv.w};
    const float G[4] = {gg.x * gs, gg.y * gs, gg.z * gs, gg.w * gs};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      M[j] = beta1 * M[j] + (1.f - beta1) * G[j];
      V[j] = beta2 * V[j] + (1.f - beta2) * G[j] * G[j];
      const float mh = M[j] / bc1, vh = V[j] / bc2;
      P[j] = P[j] - lr * (mh / (sqrtf(vh) + eps) + wd * P[j]);
    }
    reinterpret_cast<float4*>(p32)[i] = make_float4(P[0], P[1], P[2], P[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(M[0], M[1], M[2], M[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(V[0], V[1], V[2], V[3]);
    if (p16) {
      uint2 o;
      o.x = pack_bf16(P[0], P[1]);
      o.y = pack_bf16(P[2], P[3]);
      reinterpret_cast<uint2*>(p16)[i] = o;
    }
  }
}

// ---------------------------------------------------------------- sum of squares
__global__ void __launch_bounds__(256)
sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[8];
  float s = 0.f;
  const long long nv = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(x)[i];
    s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    partial[blockIdx.x] = t;
  }
}
// out[0] = sqrt(sum partial * 1) ; out[1] = clip coefficient min(1, max_norm / (norm + 1e-6))
__global__ void norm_finish_kernel(const float* __restrict__ partial, int n, float extra_sumsq_scale,
                                   float max_norm, float* __restrict__ out) {
  __shared__ float red[8];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    t *= extra_sumsq_scale;
    out[2] = t;  // raw sum of squares (for cross-rank reduction)
    const float nrm = sqrtf(t);
    out[0] = nrm;
    out[1] = (max_norm > 0.f) ? fminf(1.f, max_norm / (nrm + 1e-6f)) : 1.f;
  }
}

// ---------------------------------------------------------------- flow matching
__global__ void add_noise_kernel(const bf16* __restrict__ x0, const bf16* __restrict__ noise,
                                 bf16* __restrict__ xt, long long n_per_sample, int batch,
                                 const float* __restrict__ sigma) {
  const long long nv = n_per_sample >> 3;
  const long long total = nv * batch;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / nv);
    const float s = sigma[b];
    float a[8], z[8], o[8];
    ld8(x0 + i * 8, a);
    ld8(noise + i * 8, z);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = (1.f - s) * a[j] + s * z[j];
    st8(xt + i * 8, o);
  }
}
// loss partials and dpred = 2 * w[b] / N * (pred - (noise - x0)) * loss_scale
__global__ void __launch_bounds__(256)
flow_mse_kernel(const bf16* __restrict__ pred, const bf16* __restrict__ x0, const bf16* __restrict__ noise,
                bf16* __restrict__ dpred, long long n_per_sample, int batch, const float* __restrict__ weight,
                float grad_scale, float* __restrict__ partial) {
  __shared__ float red[8];
  const long long nv = n_per_sample >> 3;
  const long long total = nv * batch;
  const float invN = 1.f / (float)(n_per_sample * batch);
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / nv);
    const float w = weight ? weight[b] : 1.f;
    float p[8], a[8], z[8], o[8];
    ld8(pred + i * 8, p);
    ld8(x0 + i * 8, a);
    ld8(noise + i * 8, z);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float d = p[j] - (z[j] - a[j]);
      s += w * d * d;
      o[j] = 2.f * w * invN * grad_scale * d;
    }
    if (dpred) st8(dpred + i * 8, o);
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    partial[blockIdx.x] = t * invN;
  }
}
__global__ void sum_partials_kernel(const float* __restrict__ partial, int n, float* __restrict__ out) {
  __shared__ float red[8];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    *out = t;
  }
}

bool al16(const void* p) { return ((uintptr_t)p & 15) == 0; }
int grid_for(long long work_items, int threads) {
  long long g = (work_items + threads - 1) / threads;
  const long long cap = 148ll * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

TT_API int tt_act_bwd(const void* dact, long long ldd, const void* pre, long long ldp, void* dpre,
                      long long ldo, int rows, int C, int kind, cudaStream_t stream) {
  TT_CHECK(rows > 0 && C > 0 && C % 8 == 0, "act_bwd: bad shape");
  TT_CHECK(ldd % 8 == 0 && ldp % 8 == 0 && ldo % 8 == 0 && al16(dact) && al16(pre) && al16(dpre), "act_bwd: misaligned");
  TT_CHECK(kind == 0 || kind == 1, "act_bwd: kind must be 0 (gelu-tanh) or 1 (silu)");
  act_bwd_kernel<<<grid_for((long long)rows * (C / 8), 256), 256, 0, stream>>>(
      (const bf16*)dact, ldd, (const bf16*)pre, ldp, (bf16*)dpre, ldo, rows, C, kind);
  TT_LAUNCH_CHECK();
  return 0;
}

// partial: fp32 [batch, chunks, C] scratch; dgate fp32 [batch, C].
TT_API int tt_gate_bwd(const void* dout, long long ldd, const void* y, long long ldy, const float* gate,
                       long long gate_ld, void* dy, long long lddy, float* partial, int chunks,
                       float* dgate, int accumulate, int batch, int rows_per_batch, int C,
                       cudaStream_t stream);

TT_API int tt_colsum_partials(const float* partial, float* out, int groups, int n, int width,
                              int accumulate, cudaStream_t stream);

TT_API int tt_gate_bwd(const void* dout, long long ldd, const void* y, long long ldy, const float* gate,
                       long long gate_ld, void* dy, long long lddy, float* partial, int chunks,
                       float* dgate, int accumulate, int batch, int rows_per_batch, int C,
                       cudaStream_t stream) {
  TT_CHECK(batch > 0 && rows_per_batch > 0 && chunks > 0 && C % 8 == 0 && C <= 6144, "gate_bwd: bad shape");
  TT_CHECK(ldd % 8 == 0 && ldy % 8 == 0 && lddy % 8 == 0 && gate_ld % 4 == 0, "gate_bwd: leading dims misaligned");
  TT_CHECK(al16(dout) && al16(y) && al16(gate) && al16(dy) && al16(partial), "gate_bwd: misaligned pointer");
  const int rpc = (rows_per_batch + chunks - 1) / chunks;
  dim3 grid(chunks, batch);
  const int vpt = (C / 8 + 255) / 256;
  switch (vpt) {
    case 1: gate_bwd_kernel<1><<<grid, 256, 0, stream>>>((const bf16*)dout, ldd, (const bf16*)y, ldy, gate, gate_ld, (bf16*)dy, lddy, partial, C, rows_per_batch, rpc); break;
    case 2: gate_bwd_kernel<2><<<grid, 256, 0, stream>>>((const bf16*)dout, ldd, (const bf16*)y, ldy, gate, gate_ld, (bf16*)dy, lddy, partial, C, rows_per_batch, rpc); break;
    default: gate_bwd_kernel<3><<<grid, 256, 0, stream>>>((const bf16*)dout, ldd, (const bf16*)y, ldy, gate, gate_ld, (bf16*)dy, lddy, partial, C, rows_per_batch, rpc); break;
  }
  TT_LAUNCH_CHECK();
  if (dgate) return tt_colsum_partials(partial, dgate, batch, chunks, C, accumulate, stream);
  return 0;
}

// partial: fp32 [chunks, C] scratch. out: fp32 or bf16 [C].
TT_API int tt_colsum(const void* x, long long ldx, float* partial, int chunks, void* out, int out_fp32,
                     int accumulate, int rows, int C, cudaStream_t stream) {
  TT_CHECK(rows > 0 && C > 0 && C % 8 == 0 && chunks > 0, "colsum: bad shape");
  TT_CHECK(ldx % 8 == 0 && al16(x) && al16(partial), "colsum: misaligned");
  TT_CHECK(ldx >= C, "colsum: row stride %lld is smaller than the row width %d (rows would overlap)", ldx, C);
  const int rpc = (rows + chunks - 1) / chunks;
  dim3 g1((C / 8 + 255) / 256, chunks);
  colsum_stage1_kernel<<<g1, 256, 0, stream>>>((const bf16*)x, ldx, partial, rows, C, rpc);
  TT_LAUNCH_CHECK();
  colsum_stage2_kernel<<<(C + 31) / 32, 256, 0, stream>>>(partial, out, chunks, C, out_fp32, accumulate);
  TT_LAUNCH_CHECK();
  return 0;
}

TT_API int tt_adamw(float* p32, void* p16, float* m, float* v, const float* g, long long n, float lr,
                    float beta1, float beta2, float eps, float wd, int step, const float* grad_scale_ptr,
                    float grad_scale, const int* found_inf, cudaStream_t stream) {
  TT_CHECK(n > 0 && n % 4 == 0, "adamw: element count must be a positive multiple of 4");
  TT_CHECK(al16(p32) && al16(m) && al16(v) && al16(g) && (((uintptr_t)p16) & 7) == 0, "adamw: misaligned");
  TT_CHECK(step >= 1, "adamw: step counts from 1");
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = 1.f - powf(beta2, (float)step);
  adamw_kernel<<<grid_for(n / 4, 256), 256, 0, stream>>>(p32, (bf16*)p16, m, v, g, n, lr, beta1, beta2, eps,
                                                         wd, bc1, bc2, grad_scale_ptr, grad_scale, found_inf);
  TT_LAUNCH_CHECK();
  return 0;
}

// partial: fp32 scratch of tt_sumsq_blocks() entries. out: fp32[3] = {norm, clip_coef, sumsq}.
TT_API int tt_sumsq_blocks() { return 148 * 8; }
TT_API int tt_grad_norm(const float* x, long long n, float* partial, float max_norm, float* out,
                        cudaStream_t stream) {
  TT_CHECK(n > 0 && n % 4 == 0 && al16(x), "grad_norm: bad buffer");
  const int blocks = tt_sumsq_blocks();
  sumsq_kernel<<<blocks, 256, 0, stream>>>(x, n, partial);
  TT_LAUNCH_CHECK();
  norm_finish_kernel<<<1, 256, 0, stream>>>(partial, blocks, 1.f, max_norm, out);
  TT_LAUNCH_CHECK();
  return 0;
}

TT_API int tt_add_noise(const void* x0, const void* noise, void* xt, long long n_per_sample, int batch,
                        const float* sigma, cudaStream_t stream) {
  TT_CHECK(n_per_sample > 0 && n_per_sample % 8 == 0 && batch > 0, "add_noise: bad shape");
  TT_CHECK(al16(x0) && al16(noise) && al16(xt), "add_noise: misaligned");
  add_noise_kernel<<<grid_for(n_per_sample / 8 * batch, 256), 256, 0, stream>>>(
      (const bf16*)x0, (const bf16*)noise, (bf16*)xt, n_per_sample, batch, sigma);
  TT_LAUNCH_CHECK();
  return 0;
}

// partial: fp32 scratch of tt_sumsq_blocks() entries; loss: fp32 scalar.
TT_API int tt_flow_mse(const void* pred, const void* x0, const void* noise, void* dpred,
                       long long n_per_sample, int batch, const float* weight, float grad_scale,
                       float* partial, float* loss, cudaStream_t stream) {
  TT_CHECK(n_per_sample > 0 && n_per_sample % 8 == 0 && batch > 0, "flow_mse: bad shape");
  TT_CHECK(al16(pred) && al16(x0) && al16(noise) && al16(dpred), "flow_mse: misaligned");
  const int blocks = tt_sumsq_blocks();
  flow_mse_kernel<<<blocks, 256, 0, stream>>>((const bf16*)pred, (const bf16*)x0, (const bf16*)noise,
                                              (bf16*)dpred, n_per_sample, batch, weight, grad_scale, partial);
  TT_LAUNCH_CHECK();
  sum_partials_kernel<<<1, 256, 0, stream>>>(partial, blocks, loss);
  TT_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------- allocation-free column sums
// See tt_noalloc.h for who needs this and for the rules.  The partial sums of the two-stage
// reduction live in this fixed device array instead of caller scratch.
#include "tt_noalloc.h"
#include <mutex>

static __device__ __align__(256) float g_colsum_noalloc_scratch[TT_COLSUM_NOALLOC_CHUNKS * TT_COLSUM_NOALLOC_MAX_C];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device. In host code the array's name is
// only a handle; the address kernels may use comes from cudaGetSymbolAddress, looked up once
// per device while that device is current.
int noalloc_scratch(float** out) {
  int dev = -1;
  TT_CUDA(cudaGetDevice(&dev));
  TT_CHECK(dev >= 0 && dev < kMaxDevices, "colsum_noalloc: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    TT_CUDA(cudaGetSymbolAddress((void**)&p, g_colsum_noalloc_scratch));
    TT_CHECK(p != nullptr, "colsum_noalloc: scratch symbol has no device address");
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

TT_API int tt_colsum_noalloc(const void* x, long long ldx, void* out, int out_fp32, int accumulate,
                             int rows, int C, cudaStream_t stream) {
  TT_CHECK(rows > 0 && C > 0 && C % 8 == 0, "colsum_noalloc: bad shape rows=%d C=%d", rows, C);
  TT_CHECK(C <= TT_COLSUM_NOALLOC_MAX_C,
           "colsum_noalloc: C=%d exceeds the built-in scratch (max %d columns); use tt_colsum with "
           "caller-provided scratch instead",
           C, TT_COLSUM_NOALLOC_MAX_C);
  TT_CHECK(ldx % 8 == 0 && al16(x), "colsum_noalloc: input misaligned");
  TT_CHECK(ldx >= C, "colsum_noalloc: row stride %lld is smaller than the row width %d (rows would overlap)", ldx, C);
  TT_CHECK(out != nullptr, "colsum_noalloc: null output");
  float* partial = nullptr;
  if (noalloc_scratch(&partial)) return -2;
  const int chunks = rows < TT_COLSUM_NOALLOC_CHUNKS ? rows : TT_COLSUM_NOALLOC_CHUNKS;
  const int rpc = (rows + chunks - 1) / chunks;
  dim3 g1((C / 8 + 255) / 256, chunks);
  // stage 1 writes partial[chunk, 0..C) for every chunk < chunks: exactly what stage 2 reads,
  // so stale contents from an earlier call are never observed.
  colsum_stage1_kernel<<<g1, 256, 0, stream>>>((const bf16*)x, ldx, partial, rows, C, rpc);
  TT_LAUNCH_CHECK();
  colsum_stage2_kernel<<<(C + 31) / 32, 256, 0, stream>>>(partial, out, chunks, C, out_fp32, accumulate);
  TT_LAUNCH_CHECK();
  return 0;
}
