// Router (linear + softmax + top-k + L1 normalise), the counting sort that places (token, choice)
// slots into block-padded expert groups, and the row gather / gate-weighted combine kernels.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>

#include "api.h"
#include "common/host.h"

namespace mdt {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;
static long long g_rt_launches = 0;
constexpr int MAX_E = 64;   // experts held in registers per lane in the router kernels
constexpr int MAX_K = 8;

__device__ __forceinline__ void unpack8r(const uint4& u, float (&f)[8]) {
  const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8r(const float (&f)[8]) {
  uint4 u;
  bf162* h = reinterpret_cast<bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// logits[e] = <x[t,:], w[e,:]> for one token per warp; every lane ends with all E logits.
// `w` may point to shared memory (see stage_router_weights).  Four 16-byte loads of x are in flight per lane.
template <int E_T>
__device__ __forceinline__ void token_logits(const bf16* __restrict__ x, const bf16* w, int hidden, int experts,
                                             int lane, float (&logit)[E_T]) {
#pragma unroll
  for (int e = 0; e < E_T; ++e) logit[e] = 0.f;
  const uint4* xr = reinterpret_cast<const uint4*>(x);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const int nv = hidden / 8;
  for (int i0 = lane; i0 < nv; i0 += 128) {
    uint4 xv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) xv[u] = (i0 + 32 * u < nv) ? xr[i0 + 32 * u] : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + 32 * u;
      if (i < nv) {
        float xf[8]; unpack8r(xv[u], xf);
#pragma unroll
        for (int e = 0; e < E_T; ++e) {
          if (e < experts) {
            float wf[8]; unpack8r(wr[(long long)e * nv + i], wf);
#pragma unroll
            for (int j = 0; j < 8; ++j) logit[e] += xf[j] * wf[j];
          }
        }
      }
    }
  }
#pragma unroll
  for (int e = 0; e < E_T; ++e) logit[e] = wsum(logit[e]);
}

// Copies the router matrix into shared memory once per CTA when the launch provided room for it.
__device__ __forceinline__ const bf16* stage_router_weights(const bf16* __restrict__ w, int experts, int hidden, int staged) {
  extern __shared__ uint4 router_w_smem[];
  if (!staged) return w;
  const int nv = experts * (hidden / 8);
  const uint4* src = reinterpret_cast<const uint4*>(w);
  for (int i = threadIdx.x; i < nv; i += blockDim.x * 8) {     // eight loads in flight per thread
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) { const int idx = i + u * blockDim.x; v[u] = idx < nv ? src[idx] : make_uint4(0, 0, 0, 0); }
#pragma unroll
    for (int u = 0; u < 8; ++u) { const int idx = i + u * blockDim.x; if (idx < nv) router_w_smem[idx] = v[u]; }
  }
  __syncthreads();
  return reinterpret_cast<const bf16*>(router_w_smem);
}

template <int E_T>
__device__ __forceinline__ void softmax_topk(const float (&logit)[E_T], int experts, int top_k, int normalize,
                                             float (&prob)[E_T], int (&sel)[MAX_K], float (&wsel)[MAX_K], float& denom) {
  float mx = -INFINITY;
#pragma unroll
  for (int e = 0; e < E_T; ++e) if (e < experts) mx = fmaxf(mx, logit[e]);
  float se = 0.f;
#pragma unroll
  for (int e = 0; e < E_T; ++e) { prob[e] = e < experts ? __expf(logit[e] - mx) : 0.f; se += prob[e]; }
  const float inv = 1.f / se;
#pragma unroll
  for (int e = 0; e < E_T; ++e) prob[e] *= inv;
  unsigned long long taken = 0ull;
  denom = 0.f;
  for (int c = 0; c < top_k; ++c) {
    int best = 0; float bv = -1.f;
#pragma unroll
    for (int e = 0; e < E_T; ++e)
      if (e < experts && !((taken >> e) & 1ull) && prob[e] > bv) { bv = prob[e]; best = e; }
    taken |= 1ull << best;
    sel[c] = best; wsel[c] = bv; denom += bv;
  }
  if (!normalize) denom = 1.f;
}

// `stats` (optional, fp32 [2 * experts], accumulated into): the per-expert histogram of the selected experts
// (stats[e] += number of (token, choice) slots routed to e) and the per-expert sums of the softmax scores
// (stats[experts + e] += sum_t scores[t, e]): the f_e and P_e of the load-balancing loss E * sum_e f_e P_e, and the
// tokens-per-expert counts, produced in the same pass that routes the tokens.
template <int E_T>
__global__ void router_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ scores,
                                  bf16* __restrict__ weights, int* __restrict__ idx, int tokens, int hidden, int experts,
                                  int top_k, int normalize, int w_staged, float* __restrict__ stats) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  __shared__ float s_stats[2 * MAX_E];
  if (stats != nullptr) {
    for (int i = threadIdx.x; i < 2 * experts; i += blockDim.x) s_stats[i] = 0.f;
  }
  const bf16* wp = stage_router_weights(w, experts, hidden, w_staged);   // (ends with a barrier when it stages)
  if (stats != nullptr && !w_staged) __syncthreads();
  float cnt[E_T], psum[E_T];
#pragma unroll
  for (int e = 0; e < E_T; ++e) { cnt[e] = 0.f; psum[e] = 0.f; }
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < tokens; t += gridDim.x * warps_per_block) {
    float logit[E_T], prob[E_T], wsel[MAX_K], denom;
    int sel[MAX_K];
    token_logits<E_T>(x + (long long)t * hidden, wp, hidden, experts, lane, logit);
    softmax_topk<E_T>(logit, experts, top_k, normalize, prob, sel, wsel, denom);
    if (lane == 0) {
#pragma unroll
      for (int e = 0; e < E_T; ++e) if (e < experts) scores[(long long)t * experts + e] = __float2bfloat16(prob[e]);
      for (int c = 0; c < top_k; ++c) {
        weights[(long long)t * top_k + c] = __float2bfloat16(wsel[c] / denom);
        idx[(long long)t * top_k + c] = sel[c];
      }
      if (stats != nullptr) {
#pragma unroll
        for (int e = 0; e < E_T; ++e) {
          // the rounded score, so that the sum equals what a reader of `scores` would add up
          if (e < experts) psum[e] += __bfloat162float(__float2bfloat16(prob[e]));
          for (int c = 0; c < top_k; ++c) cnt[e] += (sel[c] == e) ? 1.f : 0.f;
        }
      }
    }
  }
  if (stats != nullptr) {
    if (lane == 0) {
#pragma unroll
      for (int e = 0; e < E_T; ++e)
        if (e < experts) { atomicAdd(&s_stats[e], cnt[e]); atomicAdd(&s_stats[experts + e], psum[e]); }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * experts; i += blockDim.x) atomicAdd(stats + i, s_stats[i]);
  }
}

// Backward through normalise, top-k selection and softmax; writes dlogits (fp32 [tokens, experts]) and
// dx (+)= dlogits * W.  dW is produced by router_dw_kernel from dlogits.
template <int E_T>
__global__ void router_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const int* __restrict__ idx,
                                  const bf16* __restrict__ dweights, const bf16* __restrict__ dscores, bf16* __restrict__ dx,
                                  float* __restrict__ dlogits, int tokens, int hidden, int experts, int top_k, int normalize,
                                  int accumulate_dx, int w_staged) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const bf16* wp = stage_router_weights(w, experts, hidden, w_staged);
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < tokens; t += gridDim.x * warps_per_block) {
    float logit[E_T], prob[E_T], ds[E_T], wsel[MAX_K], denom;
    int sel[MAX_K];
    token_logits<E_T>(x + (long long)t * hidden, wp, hidden, experts, lane, logit);
    softmax_topk<E_T>(logit, experts, top_k, normalize, prob, sel, wsel, denom);
    // the forward's selection is authoritative (ties): take the saved indices
    for (int c = 0; c < top_k; ++c) sel[c] = idx[(long long)t * top_k + c];
    denom = 0.f;
    for (int c = 0; c < top_k; ++c) {
      float pv = 0.f;
#pragma unroll
      for (int e = 0; e < E_T; ++e) if (e == sel[c]) pv = prob[e];
      wsel[c] = pv; denom += pv;
    }
    if (!normalize) denom = 1.f;
#pragma unroll
    for (int e = 0; e < E_T; ++e) ds[e] = (dscores != nullptr && e < experts) ? __bfloat162float(dscores[(long long)t * experts + e]) : 0.f;
    float dot = 0.f;
    if (normalize)
      for (int c = 0; c < top_k; ++c) dot += __bfloat162float(dweights[(long long)t * top_k + c]) * wsel[c] / denom;
    for (int c = 0; c < top_k; ++c) {
      const float g = (__bfloat162float(dweights[(long long)t * top_k + c]) - dot) / denom;
#pragma unroll
      for (int e = 0; e < E_T; ++e) if (e == sel[c]) ds[e] += g;
    }
    float sdot = 0.f;
#pragma unroll
    for (int e = 0; e < E_T; ++e) sdot += prob[e] * ds[e];
    float dl[E_T];
#pragma unroll
    for (int e = 0; e < E_T; ++e) dl[e] = prob[e] * (ds[e] - sdot);
    if (lane == 0) {
#pragma unroll
      for (int e = 0; e < E_T; ++e) if (e < experts) dlogits[(long long)t * experts + e] = dl[e];
    }
    uint4* dxr = reinterpret_cast<uint4*>(dx + (long long)t * hidden);
    for (int i = lane; i < hidden / 8; i += 32) {
      float acc[8];
      if (accumulate_dx) unpack8r(dxr[i], acc);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < E_T; ++e) {
        if (e < experts) {
          float wf[8]; unpack8r(reinterpret_cast<const uint4*>(wp + (long long)e * hidden)[i], wf);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += dl[e] * wf[j];
        }
      }
      dxr[i] = pack8r(acc);
    }
  }
}

// dW[e, col] = sum_t dlogits[t, e] * x[t, col]; one thread per column, tokens split over blockIdx.y
template <int E_T>
__global__ void router_dw_kernel(const bf16* __restrict__ x, const float* __restrict__ dlogits, float* __restrict__ dw,
                                 int tokens, int hidden, int experts) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= hidden) return;
  float acc[E_T];
#pragma unroll
  for (int e = 0; e < E_T; ++e) acc[e] = 0.f;
  const int chunk = (tokens + gridDim.y - 1) / gridDim.y;
  const int t0 = blockIdx.y * chunk, t1 = min(tokens, t0 + chunk);
  for (int t = t0; t < t1; ++t) {
    const float xv = __bfloat162float(x[(long long)t * hidden + col]);
#pragma unroll
    for (int e = 0; e < E_T; ++e) if (e < experts) acc[e] += dlogits[(long long)t * experts + e] * xv;
  }
#pragma unroll
  for (int e = 0; e < E_T; ++e) if (e < experts) atomicAdd(dw + (long long)e * hidden + col, acc[e]);
}

// ---------------------------------------------------------------------------------- counting sort
constexpr int PLAN_CHUNK = 256;

__global__ void plan_hist_kernel(const int* __restrict__ ids, int n, int experts, int* __restrict__ block_counts) {
  __shared__ int hist[MAX_E];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int i = blockIdx.x * PLAN_CHUNK + threadIdx.x;
  if (i < n) {
    const int e = ids[i];
    if (e >= 0 && e < experts) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) block_counts[blockIdx.x * experts + e] = hist[e];
}

// single CTA: totals, padded group offsets, and per-(block, expert) first rows (in place in block_counts)
__global__ void plan_scan_kernel(int* __restrict__ block_counts, int num_blocks, int experts, int block,
                                 int* __restrict__ counts, int* __restrict__ padded_offsets) {
  __shared__ int total[MAX_E];
  __shared__ int start[MAX_E + 1];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int run = 0;
    for (int b = 0; b < num_blocks; ++b) {
      const int c = block_counts[b * experts + e];
      block_counts[b * experts + e] = run;
      run += c;
    }
    total[e] = run;
    counts[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = off;
      padded_offsets[e] = off;
      off += (total[e] + block - 1) / block * block;
    }
    start[experts] = off;
    padded_offsets[experts] = off;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < num_blocks * experts; i += blockDim.x) block_counts[i] += start[i % experts];
}

__global__ void plan_scatter_kernel(const int* __restrict__ ids, int n, int experts, const int* __restrict__ block_base,
                                    int capacity, int* __restrict__ dest_row, int* __restrict__ src_slot) {
  __shared__ int warp_cnt[PLAN_CHUNK / 32][MAX_E];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int i = blockIdx.x * PLAN_CHUNK + threadIdx.x;
  int my = (i < n) ? ids[i] : -1;
  if (my >= experts) my = -1;
  int rank_in_warp = 0;
  for (int e = 0; e < experts; ++e) {
    const unsigned m = __ballot_sync(0xffffffffu, my == e);
    if (lane == 0) warp_cnt[w][e] = __popc(m);
    if (my == e) rank_in_warp = __popc(m & ((1u << lane) - 1u));
  }
  __syncthreads();
  if (my >= 0) {
    int before = 0;
    for (int ww = 0; ww < w; ++ww) before += warp_cnt[ww][my];
    const int row = block_base[blockIdx.x * experts + my] + before + rank_in_warp;
    dest_row[i] = row;
    if (row < capacity) src_slot[row] = i;
  } else if (i < n) {
    dest_row[i] = 0;
  }
}

// ---------------------------------------------------------------------------------- gather / combine
// out[r, :] = scale * x[src_slot[r] / top_k, :]; padding rows (src_slot < 0) are written as zeros;
// rows at or beyond padded_offsets[E] are not touched.
__global__ void gather_rows_kernel(const bf16* __restrict__ x, const int* __restrict__ src_slot, const int* __restrict__ padded_offsets,
                                   int experts, const bf16* __restrict__ slot_scale, bf16* __restrict__ out, int cols, int top_k) {
  const int r = blockIdx.x;
  if (padded_offsets != nullptr && r >= padded_offsets[experts]) return;
  const int slot = src_slot[r];
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)r * cols);
  if (slot < 0) {
    for (int i = threadIdx.x; i < cols / 8; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)(slot / top_k) * cols);
  if (slot_scale == nullptr) {
    for (int i = threadIdx.x; i < cols / 8; i += blockDim.x) dst[i] = src[i];
  } else {
    const float s = __bfloat162float(slot_scale[slot]);
    for (int i = threadIdx.x; i < cols / 8; i += blockDim.x) {
      float f[8]; unpack8r(src[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= s;
      dst[i] = pack8r(f);
    }
  }
}

// out[t, :] = sum_c weights[t, c] * y[dest_row[t*k + c], :]
// (+ residual[t, :] when given)
__global__ void combine_rows_kernel(const bf16* __restrict__ y, const int* __restrict__ dest_row, const bf16* __restrict__ weights,
                                    const bf16* __restrict__ residual, bf16* __restrict__ out, int cols, int top_k) {
  const int t = blockIdx.x;
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)t * cols);
  for (int i = threadIdx.x; i < cols / 8; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (residual != nullptr) unpack8r(reinterpret_cast<const uint4*>(residual + (long long)t * cols)[i], acc);
    for (int c = 0; c < top_k; ++c) {
      const int row = dest_row[(long long)t * top_k + c];
      const float wv = weights != nullptr ? __bfloat162float(weights[(long long)t * top_k + c]) : 1.f;
      float f[8]; unpack8r(reinterpret_cast<const uint4*>(y + (long long)row * cols)[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += wv * f[j];
    }
    dst[i] = pack8r(acc);
  }
}

// dweights[t, c] = <y[dest_row[t*k + c], :], dout[t, :]>; one warp per (t, c)
__global__ void combine_wgrad_kernel(const bf16* __restrict__ y, const int* __restrict__ dest_row, const bf16* __restrict__ dout,
                                     bf16* __restrict__ dweights, int slots, int cols, int top_k) {
  const int lane = threadIdx.x & 31;
  const int s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (s >= slots) return;
  const int t = s / top_k;
  const uint4* a = reinterpret_cast<const uint4*>(y + (long long)dest_row[s] * cols);
  const uint4* b = reinterpret_cast<const uint4*>(dout + (long long)t * cols);
  float acc = 0.f;
  for (int i = lane; i < cols / 8; i += 32) {
    float fa[8], fb[8]; unpack8r(a[i], fa); unpack8r(b[i], fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += fa[j] * fb[j];
  }
  acc = wsum(acc);
  if (lane == 0) dweights[s] = __float2bfloat16(acc);
}

#define MDT_RT_CHECK() do { ++g_rt_launches; cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return -100 - (int)e_; } while (0)

}  // namespace mdt

using namespace mdt;

extern "C" long long mdt_router_launch_count() { return g_rt_launches; }

// One warp per token, four tokens per CTA in flight; enough CTAs to fill the GPU, each staging the router matrix once.
static int router_grid(int tokens) {
  const int g = (tokens + 3) / 4;
  const int cap = sm_count_of_current_device() * 3;
  return g < 1 ? 1 : (g > cap ? cap : g);
}
// The router matrix is staged in shared memory when it fits (E x H bf16 <= 96 KB); opt in above 48 KB once per kernel.
static int router_smem_ok(const void* kernel, size_t bytes) {
  if (bytes > 96 * 1024) return 0;
  if (bytes <= 48 * 1024) return 1;
  static std::map<const void*, int> done;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  auto it = done.find(kernel);
  if (it != done.end()) return it->second;
  const int ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) == cudaSuccess ? 1 : 0;
  done[kernel] = ok;
  return ok;
}

extern "C" int mdt_router_fwd(const void* x, const void* w, void* scores, void* weights, int* idx, int tokens, int hidden,
                              int experts, int top_k, int normalize, float* stats, cudaStream_t s) {
  if (hidden % 8 != 0 || experts > MAX_E || top_k > MAX_K || top_k > experts) return -1;
  if (tokens == 0) return 0;
  const int grid = router_grid(tokens);
  const size_t wbytes = (size_t)experts * hidden * 2;
#define RT_FWD(ET)                                                                                                             \
  {                                                                                                                            \
    const int staged = router_smem_ok((const void*)router_fwd_kernel<ET>, wbytes);                                             \
    router_fwd_kernel<ET><<<grid, 128, staged ? wbytes : 0, s>>>((const bf16*)x, (const bf16*)w, (bf16*)scores, (bf16*)weights, \
                                                                 idx, tokens, hidden, experts, top_k, normalize, staged, stats); \
  }
  if (experts <= 8) RT_FWD(8) else if (experts <= 16) RT_FWD(16) else RT_FWD(MAX_E)
#undef RT_FWD
  MDT_RT_CHECK();
  return 0;
}

extern "C" int mdt_router_bwd(const void* x, const void* w, const void* scores, const void* weights, const int* idx,
                              const void* dweights, const void* dscores, void* dx, float* dw, int tokens, int hidden, int experts,
                              int top_k, int normalize, int accumulate_dx, cudaStream_t s) {
  // `dw` must hold experts*hidden floats (accumulated into) followed by tokens*experts floats of scratch.
  if (hidden % 8 != 0 || experts > MAX_E || top_k > MAX_K) return -1;
  if (tokens == 0) return 0;
  float* dlogits = dw + (long long)experts * hidden;
  const int grid = router_grid(tokens);
  const size_t wbytes = (size_t)experts * hidden * 2;
  dim3 g2((hidden + 127) / 128, 16);
#define RT_BWD(ET)                                                                                                          \
  {                                                                                                                         \
    const int staged = router_smem_ok((const void*)router_bwd_kernel<ET>, wbytes);                                          \
    router_bwd_kernel<ET><<<grid, 128, staged ? wbytes : 0, s>>>((const bf16*)x, (const bf16*)w, idx, (const bf16*)dweights,  \
                                                                 (const bf16*)dscores, (bf16*)dx, dlogits, tokens, hidden,  \
                                                                 experts, top_k, normalize, accumulate_dx, staged);         \
  }                                                                                                                         \
  MDT_RT_CHECK();                                                                                                           \
  router_dw_kernel<ET><<<g2, 128, 0, s>>>((const bf16*)x, dlogits, dw, tokens, hidden, experts);                             \
  MDT_RT_CHECK();
  if (experts <= 8) { RT_BWD(8) } else if (experts <= 16) { RT_BWD(16) } else { RT_BWD(MAX_E) }
#undef RT_BWD
  return 0;
}

extern "C" int mdt_make_plan(const int* expert_ids, int num_slots, int num_experts, int block, int capacity, int* counts,
                             int* padded_offsets, int* dest_row, int* src_slot, int* scratch, cudaStream_t s) {
  if (num_experts > MAX_E || block < 1) return -1;
  const int nb = (num_slots + PLAN_CHUNK - 1) / PLAN_CHUNK;
  cudaMemsetAsync(src_slot, 0xFF, (size_t)capacity * sizeof(int), s);
  if (nb > 0) {
    plan_hist_kernel<<<nb, PLAN_CHUNK, 0, s>>>(expert_ids, num_slots, num_experts, scratch);
    MDT_RT_CHECK();
  }
  plan_scan_kernel<<<1, 256, 0, s>>>(scratch, nb, num_experts, block, counts, padded_offsets);
  MDT_RT_CHECK();
  if (nb > 0) {
    plan_scatter_kernel<<<nb, PLAN_CHUNK, 0, s>>>(expert_ids, num_slots, num_experts, scratch, capacity, dest_row, src_slot);
    MDT_RT_CHECK();
  }
  return 0;
}

extern "C" int mdt_gather_rows(const void* x, const int* src_slot, const int* padded_offsets, int num_experts, const void* slot_scale,
                               void* out, int capacity, int cols, int top_k, cudaStream_t s) {
  if (cols % 8 != 0) return -1;
  if (capacity == 0) return 0;
  gather_rows_kernel<<<capacity, 128, 0, s>>>((const bf16*)x, src_slot, padded_offsets, num_experts, (const bf16*)slot_scale, (bf16*)out, cols, top_k);
  MDT_RT_CHECK();
  return 0;
}
extern "C" int mdt_combine_rows(const void* y, const int* dest_row, const void* weights, const void* residual, void* out, int tokens, int cols,
                                int top_k, cudaStream_t s) {
  if (cols % 8 != 0) return -1;
  if (tokens == 0) return 0;
  combine_rows_kernel<<<tokens, 128, 0, s>>>((const bf16*)y, dest_row, (const bf16*)weights, (const bf16*)residual, (bf16*)out, cols, top_k);
  MDT_RT_CHECK();
  return 0;
}
extern "C" int mdt_combine_wgrad(const void* y, const int* dest_row, const void* dout, void* dweights, int tokens, int cols, int top_k,
                                 cudaStream_t s) {
  if (cols % 8 != 0) return -1;
  const int slots = tokens * top_k;
  if (slots == 0) return 0;
  combine_wgrad_kernel<<<(slots + 3) / 4, 128, 0, s>>>((const bf16*)y, dest_row, (const bf16*)dout, (bf16*)dweights, slots, cols, top_k);
  MDT_RT_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------- allocation-free plan builder
#include <atomic>

#include "noalloc.h"

namespace mdt {
constexpr int NOALLOC_MAX_BLOCKS = MDT_NOALLOC_MAX_SLOTS / PLAN_CHUNK;
constexpr int NOALLOC_MAX_DEVICES = 64;
// Scratch of mdt_make_plan_noalloc: per-(block, expert) counts, later first rows.  One copy per GPU.
static __device__ __align__(256) int g_plan_scratch[(NOALLOC_MAX_BLOCKS + 1) * MDT_NOALLOC_MAX_EXPERTS];
// Device address of g_plan_scratch on each device (the symbol itself is only a host-side handle).  Atomic: two
// host threads may make their first call on a device at the same time; both then look the address up and store
// the same value.
static std::atomic<int*> g_plan_scratch_addr[NOALLOC_MAX_DEVICES];
}  // namespace mdt

extern "C" const char* mdt_make_plan_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case MDT_NOALLOC_TOO_LARGE: return "problem larger than the built-in scratch (MDT_NOALLOC_MAX_SLOTS slots, MDT_NOALLOC_MAX_EXPERTS experts)";
    case MDT_NOALLOC_BAD_DEVICE: return "current device ordinal is beyond this library's per-device table";
    case MDT_NOALLOC_NO_SYMBOL: return "cudaGetSymbolAddress failed for the scratch array on the current device";
    case MDT_NOALLOC_BAD_ARGUMENT: return "invalid argument (block < 1, negative size or null pointer)";
    default: return code <= -100 ? "CUDA launch error (code = -100 - cudaError_t)" : "unknown code";
  }
}

extern "C" int mdt_make_plan_noalloc(const int* expert_ids, int num_slots, int num_experts, int block, int capacity,
                                     int* counts, int* padded_offsets, int* dest_row, int* src_slot, cudaStream_t s) {
  if (block < 1 || num_slots < 0 || num_experts < 1 || capacity < 0 || counts == nullptr || padded_offsets == nullptr ||
      (num_slots > 0 && (expert_ids == nullptr || dest_row == nullptr)) || (capacity > 0 && src_slot == nullptr))
    return MDT_NOALLOC_BAD_ARGUMENT;
  if (num_slots > MDT_NOALLOC_MAX_SLOTS || num_experts > MDT_NOALLOC_MAX_EXPERTS) return MDT_NOALLOC_TOO_LARGE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return MDT_NOALLOC_BAD_DEVICE;
  int* scratch = g_plan_scratch_addr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {   // set-up, once per device, with that device current
    int* addr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_plan_scratch) != cudaSuccess || addr == nullptr)
      return MDT_NOALLOC_NO_SYMBOL;
    g_plan_scratch_addr[dev].store(addr, std::memory_order_release);
    scratch = addr;
  }
  const int nb = (num_slots + PLAN_CHUNK - 1) / PLAN_CHUNK;
  if (capacity > 0) {
    const cudaError_t me = cudaMemsetAsync(src_slot, 0xFF, (size_t)capacity * sizeof(int), s);
    if (me != cudaSuccess) { cudaGetLastError(); return -100 - (int)me; }
  }
  if (nb > 0) {
    plan_hist_kernel<<<nb, PLAN_CHUNK, 0, s>>>(expert_ids, num_slots, num_experts, scratch);
    MDT_RT_CHECK();
  }
  plan_scan_kernel<<<1, 256, 0, s>>>(scratch, nb, num_experts, block, counts, padded_offsets);
  MDT_RT_CHECK();
  if (nb > 0) {
    plan_scatter_kernel<<<nb, PLAN_CHUNK, 0, s>>>(expert_ids, num_slots, num_experts, scratch, capacity, dest_row, src_slot);
    MDT_RT_CHECK();
  }
  return 0;
}
