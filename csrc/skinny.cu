// Products with a very narrow output, y[M, r] = alpha * x[M, K] * A^T with r <= 32 (LoRA down-projections:
// x A^T in the forward pass, dy B in the backward pass).
//
// A 128-row tensor-core tile would be 7/8 empty here and only M/128 CTAs would each walk the whole depth, so
// these run on the CUDA cores instead.  A CTA of 8 warps owns 4 rows of x; the warps split the depth in
// interleaved 256-element slabs, every lane holding 8 consecutive depth positions of the 4 rows and of all r
// rows of A in registers (no staging, every load independent), then the partial sums are reduced over lanes
// and warps.  M/4 CTAs are in flight and the op is bound by one pass over x and an L2-resident A.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace mdt {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

static long long g_skinny_launches = 0;

constexpr int SK_WARPS = 8;
constexpr int SK_ROWS = 4;                 // rows of x per CTA

__device__ __forceinline__ void sk_unpack(const uint4& u, float* f) {
  const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// TRANS = false: A is [r, K] (K contiguous).  TRANS = true: A is [K, r] (r contiguous).
// Vector loads of A need lda % 8 == 0, a 16-byte aligned base and (TRANS) r % 8 == 0; `a_vec` says so.
template <int R, bool TRANS>
__global__ void __launch_bounds__(SK_WARPS * 32) skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ A,
                                                               bf16* __restrict__ y, int M, int K, int r, long long ldx,
                                                               long long lda, float alpha, int a_vec) {
  __shared__ float red[SK_WARPS][SK_ROWS][R];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * SK_ROWS;
  float acc[SK_ROWS][R];
#pragma unroll
  for (int i = 0; i < SK_ROWS; ++i)
#pragma unroll
    for (int j = 0; j < R; ++j) acc[i][j] = 0.f;

  for (int k = warp * 256 + lane * 8; k < K; k += SK_WARPS * 256) {
    // all loads of an iteration are issued before any is used: the op is latency bound (two L2 round trips per
    // lane for K = 4096), so nothing may wait for one load at a time
    uint4 xv[SK_ROWS];
#pragma unroll
    for (int i = 0; i < SK_ROWS; ++i)
      xv[i] = (row0 + i < M) ? *reinterpret_cast<const uint4*>(x + (long long)(row0 + i) * ldx + k) : make_uint4(0, 0, 0, 0);
    if (!TRANS) {
#pragma unroll
      for (int j0 = 0; j0 < R; j0 += 16) {
        uint4 av[16];
        if (a_vec) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int jj = (j0 + j < r) ? j0 + j : r - 1;      // rows past r repeat the last one; their sums are dropped
            av[j] = *reinterpret_cast<const uint4*>(A + (long long)jj * lda + k);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int jj = (j0 + j < r) ? j0 + j : r - 1;
            bf16* dst = reinterpret_cast<bf16*>(&av[j]);
#pragma unroll
            for (int q = 0; q < 8; ++q) dst[q] = A[(long long)jj * lda + k + q];
          }
        }
        float xf[SK_ROWS][8];
#pragma unroll
        for (int i = 0; i < SK_ROWS; ++i) sk_unpack(xv[i], xf[i]);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float af[8];
          sk_unpack(av[j], af);
#pragma unroll
          for (int i = 0; i < SK_ROWS; ++i)
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[i][j0 + j] += xf[i][q] * af[q];
        }
      }
    } else {
      float xf[SK_ROWS][8];
#pragma unroll
      for (int i = 0; i < SK_ROWS; ++i) sk_unpack(xv[i], xf[i]);
#pragma unroll
      for (int jv0 = 0; jv0 < R / 8; jv0 += 2) {          // 16 outputs at a time: 8 depth rows x 2 vectors
        uint4 av[8][2];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const bf16* src = A + (long long)(k + q) * lda;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const int jv = jv0 + t;
            if (a_vec) {
              av[q][t] = (jv * 8 < r) ? *reinterpret_cast<const uint4*>(src + jv * 8) : make_uint4(0, 0, 0, 0);
            } else {
              bf16* dst = reinterpret_cast<bf16*>(&av[q][t]);
#pragma unroll
              for (int e = 0; e < 8; ++e) dst[e] = (jv * 8 + e < r) ? src[jv * 8 + e] : __float2bfloat16(0.f);
            }
          }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            float ar[8];
            sk_unpack(av[q][t], ar);
#pragma unroll
            for (int i = 0; i < SK_ROWS; ++i)
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[i][(jv0 + t) * 8 + e] += xf[i][q] * ar[e];
          }
      }
    }
  }
  // over lanes, then over warps
#pragma unroll
  for (int i = 0; i < SK_ROWS; ++i)
#pragma unroll
    for (int j = 0; j < R; ++j) {
      float v = acc[i][j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) red[warp][i][j] = v;
    }
  __syncthreads();
  for (int t = threadIdx.x; t < SK_ROWS * R; t += blockDim.x) {
    const int i = t / R, j = t % R;
    if (row0 + i < M && j < r) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) v += red[w][i][j];
      y[(long long)(row0 + i) * r + j] = __float2bfloat16(v * alpha);
    }
  }
}

}  // namespace mdt

extern "C" long long mdt_skinny_launch_count() { return mdt::g_skinny_launches; }

// y[M, r] = alpha * x[M, K] * op(A);  a_is_kr = 0: A is [r, K] row-major (lda = row stride), 1: A is [K, r].
// Requirements: bf16, r <= 32, K % 8 == 0, ldx % 8 == 0, x 16-byte aligned.
extern "C" int mdt_skinny_mm(const void* x, const void* A, void* y, int M, int K, int r, long long ldx, long long lda,
                             int a_is_kr, float alpha, cudaStream_t s) {
  using namespace mdt;
  if (r < 1 || r > 32 || K % 8 != 0 || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
  if (M == 0) return 0;
  int a_vec = (lda % 8 == 0) && (reinterpret_cast<uintptr_t>(A) & 15) == 0;
  if (a_is_kr && r % 8 != 0) a_vec = 0;
  const int grid = (M + SK_ROWS - 1) / SK_ROWS;
  const bf16 *xp = (const bf16*)x, *ap = (const bf16*)A;
  bf16* yp = (bf16*)y;
  if (r <= 16) {
    if (a_is_kr) skinny_kernel<16, true><<<grid, SK_WARPS * 32, 0, s>>>(xp, ap, yp, M, K, r, ldx, lda, alpha, a_vec);
    else skinny_kernel<16, false><<<grid, SK_WARPS * 32, 0, s>>>(xp, ap, yp, M, K, r, ldx, lda, alpha, a_vec);
  } else {
    if (a_is_kr) skinny_kernel<32, true><<<grid, SK_WARPS * 32, 0, s>>>(xp, ap, yp, M, K, r, ldx, lda, alpha, a_vec);
    else skinny_kernel<32, false><<<grid, SK_WARPS * 32, 0, s>>>(xp, ap, yp, M, K, r, ldx, lda, alpha, a_vec);
  }
  ++g_skinny_launches;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - (int)e;
}
