// Memory-bound kernels: RMSNorm, RoPE, SwiGLU, embedding, softmax cross-entropy, AdamW, reductions.
// All of them move 16 bytes per thread per access and keep intermediate math in fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"
#include "common/host.h"

namespace mdt {

static long long g_ew_launches = 0;
typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  bf162* h = reinterpret_cast<bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum; `red` is shared memory for 32 floats; every thread receives the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(t);
}

// ------------------------------------------------------------------------------------ RMSNorm
__global__ void rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                                   float* __restrict__ rstd, int rows, int cols, float eps) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * cols);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + (long long)row * cols);
  const int nv = cols / 8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8]; unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / cols + eps);
  if (threadIdx.x == 0 && rstd != nullptr) rstd[row] = r;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8], g[8]; unpack8(xr[i], f); unpack8(wr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * r * g[j];
    yr[i] = pack8(f);
  }
}

// dx = rstd * (dy*w - x * rstd^2 * mean(dy*w*x)) (+ dres, the gradient that reaches x past the norm through the
// residual connection);  dw partial sums per CTA (CTA loops over rows)
__global__ void rmsnorm_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ dy,
                                   const float* __restrict__ rstd, const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                   float* __restrict__ dw_partial, int rows, int cols) {
  __shared__ float red[32];
  const int nv = cols / 8;
  // each thread owns vectors i = threadIdx.x + k*blockDim.x, k < 8 (cols <= 8*8*blockDim.x)
  float acc[8][8];
#pragma unroll
  for (int k = 0; k < 8; ++k)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[k][j] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * cols);
    const uint4* dr = reinterpret_cast<const uint4*>(dy + (long long)row * cols);
    uint4* ox = reinterpret_cast<uint4*>(dx + (long long)row * cols);
    const uint4* rr = dres != nullptr ? reinterpret_cast<const uint4*>(dres + (long long)row * cols) : nullptr;
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float xf[8], df[8], wf[8]; unpack8(xr[i], xf); unpack8(dr[i], df); unpack8(wr[i], wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += df[j] * wf[j] * xf[j];
    }
    dot = block_sum(dot, red);
    const float c = dot * r * r / cols;
    int k = 0;
    for (int i = threadIdx.x; i < nv; i += blockDim.x, ++k) {
      float xf[8], df[8], wf[8], o[8]; unpack8(xr[i], xf); unpack8(dr[i], df); unpack8(wr[i], wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = r * (df[j] * wf[j] - xf[j] * c);
        if (k < 8) acc[k][j] += df[j] * xf[j] * r;
      }
      if (rr != nullptr) {
        float rf[8]; unpack8(rr[i], rf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += rf[j];
      }
      ox[i] = pack8(o);
    }
  }
  int k = 0;
  for (int i = threadIdx.x; i < nv && k < 8; i += blockDim.x, ++k) {
    float* dst = dw_partial + (long long)blockIdx.x * cols + i * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = acc[k][j];
  }
}

// dw[c] = sum over the partial rows (+ cast): finishes the weight gradient of rmsnorm_bwd_kernel in one launch
__global__ void rmsnorm_dw_finalize_kernel(const float* __restrict__ partial, int n_partial, int cols, bf16* __restrict__ dw_bf16,
                                           float* __restrict__ dw_f32) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int r = 0; r < n_partial; ++r) s += partial[(long long)r * cols + c];
  if (dw_bf16 != nullptr) dw_bf16[c] = __float2bfloat16(s);
  if (dw_f32 != nullptr) dw_f32[c] = s;
}

// ------------------------------------------------------------------------------------ RoPE
// x: [tokens, heads, d]; pairs (i, i + d/2) rotated by pos * theta^(-2i/d); inverse negates the angle
__global__ void rope_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, const int* __restrict__ pos, int tokens,
                            int heads, int d, float log2_theta, int inverse) {
  const int t = blockIdx.x;
  const int half = d / 2;
  const float p = (float)pos[t];
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    const float inv_freq = exp2f(-log2_theta * (2.0f * i / d));
    float s, c;
    sincosf(p * inv_freq, &s, &c);
    if (inverse) s = -s;
    const long long base = ((long long)t * heads + h) * d;
    const float a = __bfloat162float(x[base + i]), b = __bfloat162float(x[base + i + half]);
    y[base + i] = __float2bfloat16(a * c - b * s);
    y[base + i + half] = __float2bfloat16(b * c + a * s);
  }
}

// ------------------------------------------------------------------------------------ SwiGLU
__global__ void swiglu_fwd_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u, uint4* __restrict__ h, long long nv) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    float a[8], b[8]; unpack8(g[i], a); unpack8(u[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = a[j] / (1.f + __expf(-a[j])) * b[j];
    h[i] = pack8(a);
  }
}
__global__ void swiglu_bwd_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u, const uint4* __restrict__ dh,
                                  uint4* __restrict__ dg, uint4* __restrict__ du, long long nv,
                                  const int* __restrict__ rows_used, long long vecs_per_row) {
  // buffers sized for a capacity carry their row count in device memory: only that many rows are touched
  if (rows_used != nullptr) { const long long lim = (long long)rows_used[0] * vecs_per_row; nv = lim < nv ? lim : nv; }
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    float a[8], b[8], d[8], og[8], ou[8]; unpack8(g[i], a); unpack8(u[i], b); unpack8(dh[i], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-a[j]));
      const float silu = a[j] * sg;
      ou[j] = d[j] * silu;
      og[j] = d[j] * b[j] * sg * (1.f + a[j] * (1.f - sg));
    }
    dg[i] = pack8(og); du[i] = pack8(ou);
  }
}

// Copy of a capacity-sized row buffer that touches only the rows in use (count read from device memory).
__global__ void copy_rows_used_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long nv,
                                      const int* __restrict__ rows_used, long long vecs_per_row) {
  const long long lim = (long long)rows_used[0] * vecs_per_row;
  nv = lim < nv ? lim : nv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) dst[i] = src[i];
}

// ------------------------------------------------------------------------------------ embedding
__global__ void embedding_kernel(const bf16* __restrict__ table, const long long* __restrict__ ids, bf16* __restrict__ out, int cols) {
  const long long id = ids[blockIdx.x];
  const uint4* src = reinterpret_cast<const uint4*>(table + id * cols);
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)blockIdx.x * cols);
  for (int i = threadIdx.x; i < cols / 8; i += blockDim.x) dst[i] = src[i];
}
__global__ void embedding_bwd_kernel(const bf16* __restrict__ dout, const long long* __restrict__ ids, float* __restrict__ dtable, int cols) {
  const long long id = ids[blockIdx.x];
  const bf16* src = dout + (long long)blockIdx.x * cols;
  float* dst = dtable + id * cols;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) atomicAdd(dst + i, __bfloat162float(src[i]));
}

// ------------------------------------------------------------------------------------ cross entropy
// One CTA per row.  The row (vocab bf16 values) is staged in shared memory, so global memory is read
// once and written once.  Output: logits <- (softmax - onehot) * grad_scale / max(count,1), or 0 for
// ignored rows; loss_sum += lse - logit[label].  `count` must already hold the number of counted rows.
__global__ void cross_entropy_kernel(bf16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ loss_sum,
                                     const float* __restrict__ count, int vocab, long long ld, int ignore_index, float grad_scale) {
  extern __shared__ uint4 row_smem[];
  __shared__ float red[32];
  const int row = blockIdx.x;
  uint4* gr = reinterpret_cast<uint4*>(logits + (long long)row * ld);
  const int nv = vocab / 8;
  const long long label = labels[row];
  if (label == ignore_index) {
    for (int i = threadIdx.x; i < nv; i += blockDim.x) gr[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    uint4 u = gr[i]; row_smem[i] = u;
    float f[8]; unpack8(u, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[j]);
  }
  mx = block_max(mx, red);
  float se = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8]; unpack8(row_smem[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) se += __expf(f[j] - mx);
  }
  se = block_sum(se, red);
  const float lse = mx + logf(se);
  const float scale = grad_scale / fmaxf(*count, 1.f);
  const float inv = 1.f / se;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8]; unpack8(row_smem[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pz = __expf(f[j] - mx) * inv;
      if ((long long)i * 8 + j == label) {
        pz -= 1.f;
        atomicAdd(loss_sum, lse - f[j]);
      }
      f[j] = pz * scale;
    }
    gr[i] = pack8(f);
  }
}
__global__ void count_labels_kernel(const long long* __restrict__ labels, int rows, int ignore_index, float* __restrict__ count) {
  __shared__ float red[32];
  float c = 0.f;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += gridDim.x * blockDim.x) c += labels[i] != ignore_index ? 1.f : 0.f;
  c = block_sum(c, red);
  if (threadIdx.x == 0 && c != 0.f) atomicAdd(count, c);
}

// ------------------------------------------------------------------------------------ AdamW
template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

// bias corrections enter as reciprocals (ibc1 = 1 / (1 - beta1^t), ibc2 likewise) so that the update costs one
// square root and one division per element; both use the fast single-precision forms, whose error (a few ulp of
// fp32) is far below the bf16 resolution of the parameters and moments they are rounded to
__device__ __forceinline__ void adam_update(float& p, float g, float& m, float& v, float lr, float b1, float b2, float eps,
                                            float wd, float ibc1, float ibc2, float gscale) {
  const float gg = g * gscale;
  m = b1 * m + (1.f - b1) * gg;
  v = b2 * v + (1.f - b2) * gg * gg;
  const float denom = __fsqrt_rn(v * ibc2) + eps;
  p = p * (1.f - lr * wd) - __fdividef(lr * (m * ibc1), denom);
}
__device__ __forceinline__ bool aligned16(const void* a, const void* b, const void* c, const void* d) {
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
           reinterpret_cast<uintptr_t>(d)) & 15) == 0;
}

// One launch for all tensors (blockIdx.y = tensor).  All-bf16, 16-byte aligned tensors go eight elements per
// thread and iteration through 128-bit loads (four loads in flight per thread, 32 warps per SM); everything else,
// and the tail, element by element.
__global__ void __launch_bounds__(256, 4) adamw_kernel(const MdtAdamTensor* __restrict__ tensors, float lr, float b1, float b2,
                                                       float eps, float wd, float ibc1, float ibc2, float gscale) {
  const MdtAdamTensor t = tensors[blockIdx.y];
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  long long done = 0;
  if (!t.p_fp32 && !t.g_fp32 && !t.s_fp32 && aligned16(t.p, t.g, t.m, t.v)) {
    const long long nv = t.n / 8;
    uint4* __restrict__ pp = reinterpret_cast<uint4*>(t.p);
    const uint4* __restrict__ gp = reinterpret_cast<const uint4*>(t.g);
    uint4* __restrict__ mp = reinterpret_cast<uint4*>(t.m);
    uint4* __restrict__ vp = reinterpret_cast<uint4*>(t.v);
    for (long long i = tid; i < nv; i += nthreads) {
      uint4 P = pp[i], G = __ldcs(gp + i), M = mp[i], V = vp[i];
      bf162* ph = reinterpret_cast<bf162*>(&P); const bf162* gh = reinterpret_cast<const bf162*>(&G);
      bf162* mh = reinterpret_cast<bf162*>(&M); bf162* vh = reinterpret_cast<bf162*>(&V);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 p = __bfloat1622float2(ph[j]), g = __bfloat1622float2(gh[j]), m = __bfloat1622float2(mh[j]), v = __bfloat1622float2(vh[j]);
        adam_update(p.x, g.x, m.x, v.x, lr, b1, b2, eps, wd, ibc1, ibc2, gscale);
        adam_update(p.y, g.y, m.y, v.y, lr, b1, b2, eps, wd, ibc1, ibc2, gscale);
        ph[j] = __floats2bfloat162_rn(p.x, p.y); mh[j] = __floats2bfloat162_rn(m.x, m.y); vh[j] = __floats2bfloat162_rn(v.x, v.y);
      }
      pp[i] = P; mp[i] = M; vp[i] = V;
    }
    done = nv * 8;
  }
  for (long long i = done + tid; i < t.n; i += nthreads) {
    float p = t.p_fp32 ? ldf((const float*)t.p, i) : ldf((const bf16*)t.p, i);
    const float g = t.g_fp32 ? ldf((const float*)t.g, i) : ldf((const bf16*)t.g, i);
    float m = t.s_fp32 ? ldf((const float*)t.m, i) : ldf((const bf16*)t.m, i);
    float v = t.s_fp32 ? ldf((const float*)t.v, i) : ldf((const bf16*)t.v, i);
    adam_update(p, g, m, v, lr, b1, b2, eps, wd, ibc1, ibc2, gscale);
    if (t.p_fp32) stf((float*)t.p, i, p); else stf((bf16*)t.p, i, p);
    if (t.s_fp32) { stf((float*)t.m, i, m); stf((float*)t.v, i, v); }
    else { stf((bf16*)t.m, i, m); stf((bf16*)t.v, i, v); }
  }
}

__global__ void __launch_bounds__(256) sumsq_kernel(const void* __restrict__ x, long long n, int fp32, float* __restrict__ out) {
  __shared__ float red[32];
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  float s = 0.f;
  long long done = 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const uint4* __restrict__ xv = reinterpret_cast<const uint4*>(x);
    const int per = fp32 ? 4 : 8;
    const long long nv = n / per;
    for (long long i = tid; i < nv; i += nthreads) {
      const uint4 u = xv[i];
      if (fp32) {
        const float4 f = *reinterpret_cast<const float4*>(&u);
        s += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
      } else {
        const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); s += f.x * f.x + f.y * f.y; }
      }
    }
    done = nv * per;
  }
  for (long long i = done + tid; i < n; i += nthreads) {
    const float v = fp32 ? ((const float*)x)[i] : __bfloat162float(((const bf16*)x)[i]);
    s += v * v;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// y = a*y + b*x
__global__ void __launch_bounds__(256) axpby_kernel(void* __restrict__ y, const void* __restrict__ x, long long n, float a, float b,
                                                    int y_fp32, int x_fp32) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  long long done = 0;
  if (!y_fp32 && !x_fp32 && ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
    const long long nv = n / 8;
    uint4* __restrict__ yv = reinterpret_cast<uint4*>(y);
    const uint4* __restrict__ xv = reinterpret_cast<const uint4*>(x);
    for (long long i = tid; i < nv; i += nthreads) {
      const uint4 X = xv[i];
      uint4 Y = a == 0.f ? make_uint4(0, 0, 0, 0) : yv[i];
      bf162* yh = reinterpret_cast<bf162*>(&Y); const bf162* xh = reinterpret_cast<const bf162*>(&X);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 yf = __bfloat1622float2(yh[j]), xf = __bfloat1622float2(xh[j]);
        yh[j] = __floats2bfloat162_rn(a * yf.x + b * xf.x, a * yf.y + b * xf.y);
      }
      yv[i] = Y;
    }
    done = nv * 8;
  }
  for (long long i = done + tid; i < n; i += nthreads) {
    const float xv = x_fp32 ? ((const float*)x)[i] : __bfloat162float(((const bf16*)x)[i]);
    const float yv = a == 0.f ? 0.f : a * (y_fp32 ? ((float*)y)[i] : __bfloat162float(((bf16*)y)[i]));
    const float r = yv + b * xv;
    if (y_fp32) ((float*)y)[i] = r; else ((bf16*)y)[i] = __float2bfloat16(r);
  }
}

// cap: upper bound on the grid in CTAs; <= 0 means -cap CTAs per SM of the current device (default 16 per SM)
// dst_i (fp32) += src_i (bf16 or fp32) for up to MDT_MULTI_ADD_MAX tensors in one launch (pointers passed by value)
__global__ void multi_add_kernel(const MdtMultiAdd a) {
  const int t = blockIdx.y;
  if (t >= a.count) return;
  float* __restrict__ dst = a.dst[t];
  const long long n = a.n[t];
  if (a.src_fp32[t]) {
    const float* __restrict__ src = reinterpret_cast<const float*>(a.src[t]);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dst[i] += src[i];
  } else {
    const bf16* __restrict__ src = reinterpret_cast<const bf16*>(a.src[t]);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
      dst[i] += __bfloat162float(src[i]);
  }
}

static inline int grid_for(long long work_items, int block, int cap = -16) {
  if (cap <= 0) cap = sm_count_of_current_device() * -cap;
  long long g = (work_items + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}
#define MDT_CHECK_LAUNCH() do { ++g_ew_launches; cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return -100 - (int)e_; } while (0)

}  // namespace mdt

using namespace mdt;

extern "C" long long mdt_elementwise_launch_count() { return g_ew_launches; }

extern "C" int mdt_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps, cudaStream_t s) {
  if (cols % 8 != 0) return -1;
  if (rows == 0) return 0;
  rmsnorm_fwd_kernel<<<rows, 256, 0, s>>>((const bf16*)x, (const bf16*)w, (bf16*)y, rstd, rows, cols, eps);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres, void* dx,
                               float* dw_partial, int rows, int cols, int n_partial, cudaStream_t s) {
  if (cols % 8 != 0 || cols > 8 * 8 * 256) return -1;
  rmsnorm_bwd_kernel<<<n_partial, 256, 0, s>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (const bf16*)dres, (bf16*)dx, dw_partial,
                                              rows, cols);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_rmsnorm_dw_finalize(const float* dw_partial, int n_partial, int cols, void* dw_bf16, float* dw_f32, cudaStream_t s) {
  rmsnorm_dw_finalize_kernel<<<(cols + 255) / 256, 256, 0, s>>>(dw_partial, n_partial, cols, (bf16*)dw_bf16, dw_f32);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_rope(const void* x, void* y, const int* positions, int tokens, int heads, int head_dim, float theta,
                        int inverse, cudaStream_t s) {
  if (tokens == 0) return 0;
  rope_kernel<<<tokens, 256, 0, s>>>((const bf16*)x, (bf16*)y, positions, tokens, heads, head_dim, log2f(theta), inverse);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_swiglu_fwd(const void* g, const void* u, void* h, long long n, cudaStream_t s) {
  if (n % 8 != 0) return -1;
  if (n == 0) return 0;
  swiglu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const uint4*)g, (const uint4*)u, (uint4*)h, n / 8);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_copy_rows_used(const void* src, void* dst, long long n, const int* rows_used, long long cols, cudaStream_t s) {
  if (n % 8 != 0 || cols % 8 != 0 || rows_used == nullptr) return -1;
  if (n == 0) return 0;
  copy_rows_used_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const uint4*)src, (uint4*)dst, n / 8, rows_used, cols / 8);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_swiglu_bwd(const void* g, const void* u, const void* dh, void* dg, void* du, long long n,
                              const int* rows_used, long long cols, cudaStream_t s) {
  if (n % 8 != 0) return -1;
  if (n == 0) return 0;
  swiglu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const uint4*)g, (const uint4*)u, (const uint4*)dh, (uint4*)dg, (uint4*)du, n / 8, rows_used, cols / 8);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_embedding(const void* table, const long long* ids, void* out, int tokens, int cols, cudaStream_t s) {
  if (cols % 8 != 0) return -1;
  if (tokens == 0) return 0;
  embedding_kernel<<<tokens, 128, 0, s>>>((const bf16*)table, ids, (bf16*)out, cols);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_embedding_bwd(const void* dout, const long long* ids, float* dtable, int tokens, int cols, cudaStream_t s) {
  if (tokens == 0) return 0;
  embedding_bwd_kernel<<<tokens, 256, 0, s>>>((const bf16*)dout, ids, dtable, cols);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_cross_entropy(void* logits, const long long* labels, float* loss_sum, float* count, int rows, int vocab,
                                 long long ld, int ignore_index, float grad_scale, cudaStream_t s) {
  if (vocab % 8 != 0 || ld % 8 != 0) return -1;
  if (rows == 0) return 0;
  const int smem = vocab * 2;
  static int configured = 0;
  if (smem > 48 * 1024 && configured < smem) {
    if (cudaFuncSetAttribute(cross_entropy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    configured = smem;
  }
  count_labels_kernel<<<grid_for(rows, 256, 64), 256, 0, s>>>(labels, rows, ignore_index, count);
  MDT_CHECK_LAUNCH();
  cross_entropy_kernel<<<rows, 512, smem, s>>>((bf16*)logits, labels, loss_sum, count, vocab, ld, ignore_index, grad_scale);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_adamw(const MdtAdamTensor* tensors_device, int num_tensors, long long max_n, float lr, float beta1, float beta2,
                         float eps, float weight_decay, float bc1, float bc2, float grad_scale, cudaStream_t s) {
  if (num_tensors == 0) return 0;
  dim3 grid(grid_for((max_n + 7) / 8, 256, -16), num_tensors);
  adamw_kernel<<<grid, 256, 0, s>>>(tensors_device, lr, beta1, beta2, eps, weight_decay, 1.0f / bc1, 1.0f / bc2, grad_scale);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_multi_add(const MdtMultiAdd* a, cudaStream_t s) {
  if (a->count < 1) return 0;
  if (a->count > MDT_MULTI_ADD_MAX) return -1;
  long long max_n = 0;
  for (int i = 0; i < a->count; ++i) max_n = a->n[i] > max_n ? a->n[i] : max_n;
  if (max_n == 0) return 0;
  dim3 grid(grid_for(max_n, 256, -4), a->count);
  multi_add_kernel<<<grid, 256, 0, s>>>(*a);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_sumsq(const void* x, long long n, int fp32, float* out_accum, cudaStream_t s) {
  if (n == 0) return 0;
  sumsq_kernel<<<grid_for(n, 256 * 8, -4), 256, 0, s>>>(x, n, fp32, out_accum);
  MDT_CHECK_LAUNCH();
  return 0;
}
extern "C" int mdt_axpby(void* y, const void* x, long long n, float a, float b, int y_fp32, int x_fp32, cudaStream_t s) {
  if (n == 0) return 0;
  axpby_kernel<<<grid_for(n, 256 * 4), 256, 0, s>>>(y, x, n, a, b, y_fp32, x_fp32);
  MDT_CHECK_LAUNCH();
  return 0;
}
