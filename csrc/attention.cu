// Causal grouped-query attention over packed variable-length sequences, head_dim 128, on tcgen05.
//
// Forward: one CTA per (sequence, 128-row query block, query head).  For every key/value block up to
// the diagonal: S = Q K^T (tcgen05.mma into TMEM), online softmax with one thread per query row
// (tcgen05.ld gives each thread its row), P written to shared memory in the 128-byte-swizzled operand
// layout, then P V through the tensor core again.  K/V tiles are double-buffered TMA loads.
//
// Backward: one CTA per (sequence, 128-row key block, query head), looping over the query blocks at or
// below the diagonal: S and dP = dO V^T recomputed into TMEM, P and dS formed per row, then
// dV += P^T dO, dK += dS^T Q (accumulated in TMEM over the loop) and dQ_i = dS K (added to an fp32
// buffer with atomics).  A [128 x 128] bf16 tile is always held as two [128 rows x 128 bytes] swizzled
// atoms; the same bytes serve as a K-major or an MN-major operand, only the descriptor changes, so
// the transposed products need no data movement.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdlib.h>

#include <mutex>

#include "api.h"
#include "common/host.h"
#include "common/ptx.cuh"

namespace mdt {

typedef __nv_bfloat16 bf16;
static long long g_att_launches = 0;
constexpr int AB = 128;            // rows per query / key block
constexpr int HD = 128;            // head dimension
constexpr int TILE_BYTES = AB * HD * 2;   // 32 KB
constexpr int ATOM_BYTES = AB * 128;      // 16 KB: [128 rows x 64 bf16]

struct AttnParams {
  CUtensorMap tmQ, tmK, tmV, tmdO;
  CUtensorMap tmK64, tmV64;                  // key / value maps with 64-row boxes (pipelined forward)
  const int* cu_seqlens;
  int num_seqs, heads_q, heads_kv;
  float scale_log2e, scale;
  bf16* o; float* lse;                       // forward outputs
  const float* delta; const float* lse_in;   // backward inputs
  float* dq; float* dk; float* dv;           // backward outputs (fp32, [T, heads_q, 128])
  int* status;
};

// descriptors over the canonical tile form (two swizzled atoms of [128 rows x 128 B])
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int kstep) {   // depth = the 128 columns
  return make_smem_desc(tile + (kstep >> 2) * ATOM_BYTES + (kstep & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int kstep) {  // depth = the 128 rows
  return make_smem_desc(tile + kstep * 2048, ATOM_BYTES, 1024);
}
// byte offset of 8 consecutive bf16 (columns c..c+7, c % 8 == 0) of row r inside a canonical tile
__device__ __forceinline__ uint32_t tile_offset(int r, int c) {
  return (c >> 6) * ATOM_BYTES + r * 128 + ((((c & 63) >> 3) ^ (r & 7)) << 4);
}
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int col0, int row0) {
  tma_load_2d(dst, map, bar, col0, row0);
  tma_load_2d(dst + ATOM_BYTES, map, bar, col0 + 64, row0);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// locate the block handled by this CTA: blockIdx.x enumerates 128-row blocks over all sequences
__device__ __forceinline__ bool find_block(const int* cu, int num_seqs, int flat, int& seq_start, int& seq_end, int& blk) {
  for (int s = 0; s < num_seqs; ++s) {
    const int a = cu[s], b = cu[s + 1];
    const int nb = (b - a + AB - 1) / AB;
    if (flat < nb) { seq_start = a; seq_end = b; blk = flat; return true; }
    flat -= nb;
  }
  return false;
}

// ------------------------------------------------------------------------------------------- forward
__global__ void __launch_bounds__(128, 1) attn_fwd_kernel(const __grid_constant__ AttnParams p) {
  int seq_start, seq_end, qb;
  if (!find_block(p.cu_seqlens, p.num_seqs, blockIdx.x, seq_start, seq_end, qb)) return;
  const int h = blockIdx.y, kvh = h / (p.heads_q / p.heads_kv);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE_BYTES;          // two stages
  uint8_t* sV = smem + 3 * TILE_BYTES;      // two stages
  uint8_t* sP = smem + 5 * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES);
  uint64_t* barQ = bars; uint64_t* barKV = bars + 1; uint64_t* barS = bars + 3; uint64_t* barO = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(barQ, 1); mbar_init(&barKV[0], 1); mbar_init(&barKV[1], 1); mbar_init(barS, 1); mbar_init(barO, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's lane quarter
  const int q0 = seq_start + qb * AB;
  const int n_kv = qb + 1;
  const uint32_t idesc = make_idesc_bf16(128, 128, 0, 0);
  const uint32_t idesc_pv = make_idesc_bf16(128, 128, 0, 1);
  if (tid == 0) {
    mbar_expect_tx(barQ, TILE_BYTES);
    load_tile(sQ, &p.tmQ, barQ, h * HD, q0);
    mbar_expect_tx(&barKV[0], 2 * TILE_BYTES);
    load_tile(sK, &p.tmK, &barKV[0], kvh * HD, seq_start);
    load_tile(sV, &p.tmV, &barKV[0], kvh * HD, seq_start);
  }
  float o[HD];
#pragma unroll
  for (int i = 0; i < HD; ++i) o[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int r = tid;                         // query row inside the block == TMEM lane
  bool ok = true;
  for (int j = 0; j < n_kv && ok; ++j) {
    const int st = j & 1;
    if (tid == 0) {
      if (j + 1 < n_kv) {
        mbar_expect_tx(&barKV[st ^ 1], 2 * TILE_BYTES);
        load_tile(sK + (st ^ 1) * TILE_BYTES, &p.tmK, &barKV[st ^ 1], kvh * HD, seq_start + (j + 1) * AB);
        load_tile(sV + (st ^ 1) * TILE_BYTES, &p.tmV, &barKV[st ^ 1], kvh * HD, seq_start + (j + 1) * AB);
      }
      bool w = (j > 0) || wait_parity(barQ, 0, abort_flag);
      w = w && wait_parity(&barKV[st], (j >> 1) & 1, abort_flag);
      if (w) {
        tc_fence_after();
        const uint32_t a = smem_u32(sQ), b = smem_u32(sK + st * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16(tmem, desc_kmajor(a, k), desc_kmajor(b, k), idesc, k > 0);
        umma_commit(barS);
      } else {
        *abort_flag = 1;
        if (p.status) atomicCAS(p.status, 0, ST_TIMEOUT_FULL);
      }
    }
    __syncwarp();
    if (!wait_parity(barS, j & 1, abort_flag)) { ok = false; break; }
    __syncwarp();
    tc_fence_after();
    // ---- online softmax on this thread's row (two passes over TMEM: row maximum, then exponentials)
    float mx = m;
    const bool diag = (j == qb);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t raw[32];
      tmem_ld_32x32(t_row + c * 32, raw);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (!(diag && (c * 32 + i) > r)) mx = fmaxf(mx, __uint_as_float(raw[i]) * p.scale_log2e);
      }
    }
    const float alpha = exp2f(m - mx);
    float rs = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t raw[32];
      tmem_ld_32x32(t_row + c * 32, raw);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        float e[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const bool masked = diag && (c * 32 + i + t) > r;
          e[t] = masked ? 0.f : exp2f(__uint_as_float(raw[i + t]) * p.scale_log2e - mx);
          rs += e[t];
        }
        uint4 u = make_uint4(pack2(e[0], e[1]), pack2(e[2], e[3]), pack2(e[4], e[5]), pack2(e[6], e[7]));
        *reinterpret_cast<uint4*>(sP + tile_offset(r, c * 32 + i)) = u;
      }
    }
    l = l * alpha + rs;
    m = mx;
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t a = smem_u32(sP), b = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
      for (int k = 0; k < 8; ++k) umma_bf16(tmem + 128, desc_kmajor(a, k), desc_mnmajor(b, k), idesc_pv, k > 0);
      umma_commit(barO);
    }
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] *= alpha;
    __syncwarp();
    if (!wait_parity(barO, j & 1, abort_flag)) { ok = false; break; }
    __syncwarp();
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t raw[32];
      tmem_ld_32x32(t_row + 128 + c * 32, raw);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(raw[i]);
    }
    tc_fence_before();
    __syncthreads();
  }
  if (!ok && tid == 0 && p.status) atomicCAS(p.status, 0, ST_TIMEOUT_TMEM_FULL);
  const int row = q0 + r;
  if (ok && row < seq_end) {
    const float inv = 1.f / l;
    bf16* dst = p.o + ((long long)row * p.heads_q + h) * HD;
#pragma unroll
    for (int i = 0; i < HD; i += 8) {
      uint4 u = make_uint4(pack2(o[i] * inv, o[i + 1] * inv), pack2(o[i + 2] * inv, o[i + 3] * inv),
                           pack2(o[i + 4] * inv, o[i + 5] * inv), pack2(o[i + 6] * inv, o[i + 7] * inv));
      *reinterpret_cast<uint4*>(dst + i) = u;
    }
    p.lse[(long long)row * p.heads_q + h] = (m + log2f(l)) * 0.6931471805599453f;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

// ------------------------------------------------------------------------------------------- forward, pipelined
// Warp-specialised forward: warps 0-3 do the softmax (one query row per thread), warp 4 loads (TMA) and issues the
// MMAs.  Keys / values come in blocks of 64 rows; S = Q K^T lives in two 64-column TMEM buffers, so the tensor core
// computes S of block j+1 while the softmax warps work on block j; O is accumulated in TMEM by the P V products
// themselves.  The running row maximum used for the exponentials is only raised when the true maximum has grown
// by more than 2^8 (the sum and O are rescaled then, rarely after the first blocks; the final division by the row
// sum makes the result independent of the reference point).  96 KB of shared memory and 256 TMEM columns per CTA:
// two CTAs share an SM, so that one's softmax also overlaps the other's products.
//   TMEM columns: [0,64) S buffer 0, [64,128) S buffer 1, [128,256) O
//   barriers: Q, K (one K tile, reloaded as soon as S of the previous block is done), V[2], S[2] (S ready),
//             Sfree[2] (softmax has read S), P (probabilities stored), O (P V done: O updated, P and V tile free)
constexpr int FB = 64;                        // key rows per block
constexpr int KV_TILE = FB * HD * 2;          // 16 KB: two atoms of [64 rows x 128 B]
constexpr int KV_ATOM = FB * 128;             // 8 KB
constexpr int P_TILE = AB * FB * 2;           // 16 KB: one atom of [128 rows x 128 B]
constexpr int FWD2_THREADS = 160;
constexpr int FWD2_SMEM = TILE_BYTES + KV_TILE + 2 * KV_TILE + P_TILE + 1024 + 128;
static_assert(2 * (FWD2_SMEM + 1024) <= 228 * 1024, "two CTAs of the pipelined forward must fit one SM");
constexpr float RESCALE_THRESHOLD = 8.0f;     // log2 units

__device__ __forceinline__ void load_kv_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int col0, int row0) {
  tma_load_2d(dst, map, bar, col0, row0);               // box {64 columns, 64 rows}
  tma_load_2d(dst + KV_ATOM, map, bar, col0 + 64, row0);
}

__global__ void __launch_bounds__(FWD2_THREADS, 2) attn_fwd_pipelined_kernel(const __grid_constant__ AttnParams p) {
  int seq_start, seq_end, qb;
  if (!find_block(p.cu_seqlens, p.num_seqs, blockIdx.x, seq_start, seq_end, qb)) return;
  const int h = blockIdx.y, kvh = h / (p.heads_q / p.heads_kv);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE_BYTES;
  uint8_t* sV = sK + KV_TILE;                 // two stages
  uint8_t* sP = sV + 2 * KV_TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_TILE);
  uint64_t* barQ = bars; uint64_t* barK = bars + 1; uint64_t* barV = bars + 2; uint64_t* barS = bars + 4;
  uint64_t* barSfree = bars + 6; uint64_t* barP = bars + 8; uint64_t* barO = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(barQ, 1); mbar_init(barK, 1); mbar_init(&barV[0], 1); mbar_init(&barV[1], 1);
    mbar_init(&barS[0], 1); mbar_init(&barS[1], 1); mbar_init(&barSfree[0], 4); mbar_init(&barSfree[1], 4);
    mbar_init(barP, 4); mbar_init(barO, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int q0 = seq_start + qb * AB;
  // key blocks up to the diagonal, and not past the end of the sequence
  const int len = seq_end - seq_start;
  int n_kv = 2 * qb + 2;
  const int n_seq = (len + FB - 1) / FB;
  if (n_kv > n_seq) n_kv = n_seq;
  auto fail = [&](int code) {
    *abort_flag = 1;
    if (p.status != nullptr) atomicCAS(p.status, 0, code);
  };

  if (warp == 4) {
    if (lane == 0) {
      // ---------------------------------------------------------------- loads and MMA issue
      const uint32_t idesc_s = make_idesc_bf16(128, FB, 0, 0);       // Q (K-major) x K^T (K-major)
      const uint32_t idesc_pv = make_idesc_bf16(128, HD, 0, 1);      // P (K-major) x V (MN-major)
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aP = smem_u32(sP);
      mbar_expect_tx(barQ, TILE_BYTES);
      load_tile(sQ, &p.tmQ, barQ, h * HD, q0);
      mbar_expect_tx(barK, KV_TILE);
      load_kv_tile(sK, &p.tmK64, barK, kvh * HD, seq_start);
      mbar_expect_tx(&barV[0], KV_TILE);
      load_kv_tile(sV, &p.tmV64, &barV[0], kvh * HD, seq_start);
      bool ok = wait_parity(barQ, 0, abort_flag) && wait_parity(barK, 0, abort_flag);
      if (!ok) fail(ST_TIMEOUT_FULL);
      auto issue_s = [&](int j) {     // S_j = Q K_j^T into S buffer j & 1
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tmem + (j & 1) * FB, desc_kmajor(aQ, k), make_smem_desc(aK + (k >> 2) * KV_ATOM + (k & 3) * 32, 16, 1024), idesc_s, k > 0);
        umma_commit(&barS[j & 1]);
      };
      if (ok) issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          // K tile free once S_j is done; S buffer (j+1)&1 free once the softmax of block j-1 has read it
          ok = wait_parity(&barS[j & 1], (j >> 1) & 1, abort_flag);
          if (!ok) { fail(ST_TIMEOUT_TMEM_FULL); break; }
          mbar_expect_tx(barK, KV_TILE);
          load_kv_tile(sK, &p.tmK64, barK, kvh * HD, seq_start + (j + 1) * FB);
          ok = wait_parity(barK, (j + 1) & 1, abort_flag);
          if (ok && j >= 1) ok = wait_parity(&barSfree[(j + 1) & 1], ((j - 1) >> 1) & 1, abort_flag);
          if (!ok) { fail(ST_TIMEOUT_FULL); break; }
          issue_s(j + 1);
        }
        // P_j stored (which also means P V of block j-1 is complete: the softmax warps waited for it)
        ok = wait_parity(barP, j & 1, abort_flag);
        if (!ok) { fail(ST_TIMEOUT_EMPTY); break; }
        if (j + 1 < n_kv) {
          mbar_expect_tx(&barV[(j + 1) & 1], KV_TILE);
          load_kv_tile(sV + ((j + 1) & 1) * KV_TILE, &p.tmV64, &barV[(j + 1) & 1], kvh * HD, seq_start + (j + 1) * FB);
        }
        ok = wait_parity(&barV[j & 1], (j >> 1) & 1, abort_flag);
        if (!ok) { fail(ST_TIMEOUT_FULL); break; }
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + (j & 1) * KV_TILE);
#pragma unroll
        for (int k = 0; k < FB / 16; ++k)
          umma_bf16(tmem + 128, make_smem_desc(aP + k * 32, 16, 1024), make_smem_desc(aV + k * 2048, KV_ATOM, 1024), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(barO);
      }
      if (!ok) {   // give copies in flight a bounded time to land before the CTA leaves
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 20000ull) {}
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: thread = query row
    const int r = tid;
    const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!wait_parity(&barS[j & 1], (j >> 1) & 1, abort_flag)) { ok = false; break; }
      __syncwarp();
      tc_fence_after();
      uint32_t s0[32], s1[32];
      tmem_ld_32x32(t_row + (j & 1) * FB, s0);
      tmem_ld_32x32(t_row + (j & 1) * FB + 32, s1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&barSfree[j & 1]);
      // causal mask: key column 64j + c is visible to query row 128qb + r iff it is not to the right of it
      const int visible = qb * AB + r - j * FB;         // columns c <= visible are kept
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float a = __uint_as_float(s0[c]) * p.scale_log2e, b = __uint_as_float(s1[c]) * p.scale_log2e;
        s0[c] = __float_as_uint(c <= visible ? a : -INFINITY);
        s1[c] = __float_as_uint(c + 32 <= visible ? b : -INFINITY);
        mx = fmaxf(mx, fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])));
      }
      // raise the reference point only when the maximum has outgrown it by more than the threshold
      float alpha = 1.f;
      const bool raise = mx > m_ref + RESCALE_THRESHOLD;    // (also true for the first visible block: m_ref = -inf)
      if (raise) { alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - mx); m_ref = mx; l *= alpha; }
      if (j > 0) {
        if (!wait_parity(barO, (j - 1) & 1, abort_flag)) { ok = false; break; }   // O of the blocks so far is complete, P free
        __syncwarp();
        if (__any_sync(0xffffffffu, raise)) {
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(t_row + 128 + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(t_row + 128 + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < 64; c += 8) {
        float e[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const float v = __uint_as_float(c < 32 ? s0[c + t] : s1[c - 32 + t]);
          e[t] = fast_exp2(v - m_ref);      // -inf -> 0; a row with nothing visible yet has m_ref = -inf: (-inf) - (-inf) = nan, guarded below
          if (m_ref == -INFINITY) e[t] = 0.f;
          rs += e[t];
        }
        *reinterpret_cast<uint4*>(sP + r * 128 + (((c >> 3) ^ (r & 7)) << 4)) =
            make_uint4(pack2(e[0], e[1]), pack2(e[2], e[3]), pack2(e[4], e[5]), pack2(e[6], e[7]));
      }
      l += rs;
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(barP);
    }
    if (ok && n_kv > 0 && !wait_parity(barO, (n_kv - 1) & 1, abort_flag)) ok = false;
    __syncwarp();
    ok = __all_sync(0xffffffffu, ok);
    if (!ok && lane == 0) fail(ST_TIMEOUT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      const int row = q0 + r;
      const bool valid = row < seq_end;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.o + ((long long)row * p.heads_q + h) * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_row + 128 + c * 32, o);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 u = make_uint4(pack2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv),
                                 pack2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
                                 pack2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv),
                                 pack2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv));
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = u;
          }
        }
        __syncwarp();
      }
      if (valid) p.lse[(long long)row * p.heads_q + h] = (m_ref + log2f(l)) * 0.6931471805599453f;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

// ------------------------------------------------------------------------------------------- backward
__global__ void attn_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout, float* __restrict__ delta, long long rows) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // (token, head) pair
  if (row >= rows) return;
  const uint2 a = reinterpret_cast<const uint2*>(o + row * HD)[lane];
  const uint2 b = reinterpret_cast<const uint2*>(dout + row * HD)[lane];
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) { float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]); s += x.x * y.x + x.y * y.y; }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[row] = s;
}

__global__ void __launch_bounds__(128, 1) attn_bwd_kernel(const __grid_constant__ AttnParams p) {
  int seq_start, seq_end, kb;
  if (!find_block(p.cu_seqlens, p.num_seqs, blockIdx.x, seq_start, seq_end, kb)) return;
  const int h = blockIdx.y, kvh = h / (p.heads_q / p.heads_kv);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem; uint8_t* sV = smem + TILE_BYTES; uint8_t* sQ = smem + 2 * TILE_BYTES;
  uint8_t* sdO = smem + 3 * TILE_BYTES; uint8_t* sP = smem + 4 * TILE_BYTES; uint8_t* sdS = smem + 5 * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES);
  uint64_t* barKV = bars; uint64_t* barQ = bars + 1; uint64_t* barS = bars + 2; uint64_t* barD = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(barKV, 1); mbar_init(barQ, 1); mbar_init(barS, 1); mbar_init(barD, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16);
  const int k0 = seq_start + kb * AB;
  const int nq = (seq_end - seq_start + AB - 1) / AB;
  const int r = tid;
  const uint32_t id_kk = make_idesc_bf16(128, 128, 0, 0);   // A K-major, B K-major
  const uint32_t id_mm = make_idesc_bf16(128, 128, 1, 1);   // A MN-major, B MN-major
  const uint32_t id_km = make_idesc_bf16(128, 128, 0, 1);   // A K-major, B MN-major
  if (tid == 0) {
    mbar_expect_tx(barKV, 2 * TILE_BYTES);
    load_tile(sK, &p.tmK, barKV, kvh * HD, k0);
    load_tile(sV, &p.tmV, barKV, kvh * HD, k0);
  }
  bool ok = true;
  int it = 0;
  for (int i = kb; i < nq && ok; ++i, ++it) {
    const int q0 = seq_start + i * AB;
    if (tid == 0) {
      mbar_expect_tx(barQ, 2 * TILE_BYTES);
      load_tile(sQ, &p.tmQ, barQ, h * HD, q0);
      load_tile(sdO, &p.tmdO, barQ, h * HD, q0);
      bool w = (it > 0) || wait_parity(barKV, 0, abort_flag);
      w = w && wait_parity(barQ, it & 1, abort_flag);
      if (w) {
        tc_fence_after();
        const uint32_t q = smem_u32(sQ), k = smem_u32(sK), d = smem_u32(sdO), v = smem_u32(sV);
#pragma unroll
        for (int s = 0; s < 8; ++s) umma_bf16(tmem, desc_kmajor(q, s), desc_kmajor(k, s), id_kk, s > 0);          // S = Q K^T
#pragma unroll
        for (int s = 0; s < 8; ++s) umma_bf16(tmem + 128, desc_kmajor(d, s), desc_kmajor(v, s), id_kk, s > 0);    // dP = dO V^T
        umma_commit(barS);
      } else {
        *abort_flag = 1;
        if (p.status) atomicCAS(p.status, 0, ST_TIMEOUT_FULL);
      }
    }
    __syncwarp();
    if (!wait_parity(barS, it & 1, abort_flag)) { ok = false; break; }
    __syncwarp();
    tc_fence_after();
    const int qrow = q0 + r;
    const bool qvalid = qrow < seq_end;
    const float lse2 = qvalid ? p.lse_in[(long long)qrow * p.heads_q + h] * 1.4426950408889634f : 0.f;
    const float dl = qvalid ? p.delta[(long long)qrow * p.heads_q + h] : 0.f;
    const bool diag = (i == kb);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t rs[32], rp[32];
      tmem_ld_32x32(t_row + c * 32, rs);
      tmem_ld_32x32(t_row + 128 + c * 32, rp);
      tmem_ld_wait();
#pragma unroll
      for (int x = 0; x < 32; x += 8) {
        float pv[8], ds[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const int col = c * 32 + x + t;
          float pr = fast_exp2(__uint_as_float(rs[x + t]) * p.scale_log2e - lse2);
          if (!qvalid || (diag && col > r) || (k0 + col >= seq_end)) pr = 0.f;
          pv[t] = pr;
          ds[t] = pr * (__uint_as_float(rp[x + t]) - dl) * p.scale;
        }
        const uint32_t off = tile_offset(r, c * 32 + x);
        *reinterpret_cast<uint4*>(sP + off) = make_uint4(pack2(pv[0], pv[1]), pack2(pv[2], pv[3]), pack2(pv[4], pv[5]), pack2(pv[6], pv[7]));
        *reinterpret_cast<uint4*>(sdS + off) = make_uint4(pack2(ds[0], ds[1]), pack2(ds[2], ds[3]), pack2(ds[4], ds[5]), pack2(ds[6], ds[7]));
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t q = smem_u32(sQ), k = smem_u32(sK), d = smem_u32(sdO), ps = smem_u32(sP), dss = smem_u32(sdS);
      const uint32_t acc = it > 0;
#pragma unroll
      for (int s = 0; s < 8; ++s) umma_bf16(tmem + 256, desc_mnmajor(ps, s), desc_mnmajor(d, s), id_mm, acc || s > 0);    // dV += P^T dO
#pragma unroll
      for (int s = 0; s < 8; ++s) umma_bf16(tmem + 384, desc_mnmajor(dss, s), desc_mnmajor(q, s), id_mm, acc || s > 0);   // dK += dS^T Q
#pragma unroll
      for (int s = 0; s < 8; ++s) umma_bf16(tmem, desc_kmajor(dss, s), desc_mnmajor(k, s), id_km, s > 0);                 // dQ_i = dS K
      umma_commit(barD);
    }
    __syncwarp();
    if (!wait_parity(barD, it & 1, abort_flag)) { ok = false; break; }
    __syncwarp();
    tc_fence_after();
    float* dqrow = p.dq + ((long long)qrow * p.heads_q + h) * HD;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t raw[32];
      tmem_ld_32x32(t_row + c * 32, raw);      // warp-aligned: every lane takes part, valid row or not
      tmem_ld_wait();
      if (qvalid) {
#pragma unroll
        for (int x = 0; x < 32; x += 4)
          red_add_v4_f32(dqrow + c * 32 + x, __uint_as_float(raw[x]), __uint_as_float(raw[x + 1]), __uint_as_float(raw[x + 2]),
                         __uint_as_float(raw[x + 3]));
      }
      __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
  }
  if (!ok && tid == 0 && p.status) atomicCAS(p.status, 0, ST_TIMEOUT_TMEM_FULL);
  const int krow = k0 + r;
  const bool kvalid = krow < seq_end;
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {   // warp-uniform: `ok` only changes together with the shared abort flag
    float* dv = p.dv + ((long long)krow * p.heads_q + h) * HD;
    float* dk = p.dk + ((long long)krow * p.heads_q + h) * HD;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t a[32], b[32];
      tmem_ld_32x32(t_row + 256 + c * 32, a);
      tmem_ld_32x32(t_row + 384 + c * 32, b);
      tmem_ld_wait();
      if (kvalid) {
#pragma unroll
        for (int x = 0; x < 32; x += 4) {
          *reinterpret_cast<float4*>(dv + c * 32 + x) = make_float4(__uint_as_float(a[x]), __uint_as_float(a[x + 1]), __uint_as_float(a[x + 2]), __uint_as_float(a[x + 3]));
          *reinterpret_cast<float4*>(dk + c * 32 + x) = make_float4(__uint_as_float(b[x]), __uint_as_float(b[x + 1]), __uint_as_float(b[x + 2]), __uint_as_float(b[x + 3]));
        }
      }
      __syncwarp();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// dq bf16 = dq fp32; dk/dv bf16 [T, heads_kv, 128] = sum over the query heads of each group
__global__ void attn_bwd_finalize_kernel(const float* __restrict__ dq32, const float* __restrict__ dk32, const float* __restrict__ dv32,
                                         bf16* __restrict__ dq, bf16* __restrict__ dk, bf16* __restrict__ dv, long long tokens,
                                         int heads_q, int heads_kv) {
  const int group = heads_q / heads_kv;
  const long long nq = tokens * heads_q * HD, nk = tokens * heads_kv * HD;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nq + 2 * nk; i += (long long)gridDim.x * blockDim.x) {
    if (i < nq) { dq[i] = __float2bfloat16(dq32[i]); continue; }
    const bool isv = i >= nq + nk;
    const long long e = i - nq - (isv ? nk : 0);
    const int d = (int)(e % HD);
    const long long th = e / HD;
    const int kvh = (int)(th % heads_kv);
    const long long t = th / heads_kv;
    const float* src = (isv ? dv32 : dk32) + ((t * heads_q + (long long)kvh * group) * HD) + d;
    float s = 0.f;
    for (int g = 0; g < group; ++g) s += src[(long long)g * HD];
    (isv ? dv : dk)[e] = __float2bfloat16(s);
  }
}

typedef CUresult (*EncodeTiledFnA)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFnA att_encode_fn() {
  static EncodeTiledFnA fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFnA>(ptr);
  });
  return fn;
}
// [tokens, heads*128] bf16, box 64 columns x `box_rows` rows
static int att_map(CUtensorMap* m, const void* ptr, long long tokens, int heads, int box_rows = AB) {
  EncodeTiledFnA fn = att_encode_fn();
  if (fn == nullptr) return -1;
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return -2;
  cuuint64_t dims[2] = {(cuuint64_t)heads * HD, (cuuint64_t)tokens};
  cuuint64_t strides[1] = {(cuuint64_t)heads * HD * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -3;
}
constexpr int ATT_SMEM = 6 * TILE_BYTES + 1024 + 128;

}  // namespace mdt

using namespace mdt;

extern "C" long long mdt_attention_launch_count() { return g_att_launches; }

extern "C" int mdt_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_seqlens,
                                 int num_seqs, int total_tokens, int max_seqlen, int heads_q, int heads_kv, int head_dim,
                                 float scale, cudaStream_t s) {
  if (head_dim != HD || heads_q % heads_kv != 0) return -1;
  if (total_tokens == 0) return 0;
  static thread_local bool bound = false;
  if (!bound) { cudaFree(nullptr); bound = true; }
  AttnParams p;
  memset(&p, 0, sizeof(p));
  // MDT_ATTN_FWD=serial selects the one-block-at-a-time kernel (for comparisons); default: the pipelined kernel
  static const bool serial = []() { const char* e = getenv("MDT_ATTN_FWD"); return e != nullptr && e[0] == 's'; }();
  int rc = att_map(&p.tmQ, q, total_tokens, heads_q) | att_map(&p.tmK, k, total_tokens, heads_kv) | att_map(&p.tmV, v, total_tokens, heads_kv);
  if (!serial) rc |= att_map(&p.tmK64, k, total_tokens, heads_kv, FB) | att_map(&p.tmV64, v, total_tokens, heads_kv, FB);
  if (rc) return rc;
  p.cu_seqlens = cu_seqlens; p.num_seqs = num_seqs; p.heads_q = heads_q; p.heads_kv = heads_kv;
  p.scale = scale; p.scale_log2e = scale * 1.4426950408889634f;
  p.o = (bf16*)o; p.lse = lse;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess) return -4;
    if (cudaFuncSetAttribute(attn_fwd_pipelined_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD2_SMEM) != cudaSuccess) return -4;
    if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess) return -4;
    configured = true;
  }
  dim3 grid((total_tokens + AB - 1) / AB + num_seqs, heads_q);
  if (serial) attn_fwd_kernel<<<grid, 128, ATT_SMEM, s>>>(p);
  else attn_fwd_pipelined_kernel<<<grid, FWD2_THREADS, FWD2_SMEM, s>>>(p);
  ++g_att_launches;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - (int)e;
}

extern "C" int mdt_attention_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                                 void* dq, void* dk, void* dv, float* scratch, const int* cu_seqlens, int num_seqs, int total_tokens,
                                 int max_seqlen, int heads_q, int heads_kv, int head_dim, float scale, cudaStream_t s) {
  // scratch: fp32, (1 + 3*128) * total_tokens * heads_q elements: delta | dq32 | dk32 | dv32
  if (head_dim != HD || heads_q % heads_kv != 0) return -1;
  if (total_tokens == 0) return 0;
  static thread_local bool bound = false;
  if (!bound) { cudaFree(nullptr); bound = true; }
  const long long th = (long long)total_tokens * heads_q;
  float* delta = scratch;
  float* dq32 = scratch + th;
  float* dk32 = dq32 + th * HD;
  float* dv32 = dk32 + th * HD;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  int rc = att_map(&p.tmQ, q, total_tokens, heads_q) | att_map(&p.tmK, k, total_tokens, heads_kv) |
           att_map(&p.tmV, v, total_tokens, heads_kv) | att_map(&p.tmdO, dout, total_tokens, heads_q);
  if (rc) return rc;
  p.cu_seqlens = cu_seqlens; p.num_seqs = num_seqs; p.heads_q = heads_q; p.heads_kv = heads_kv;
  p.scale = scale; p.scale_log2e = scale * 1.4426950408889634f;
  p.delta = delta; p.lse_in = lse; p.dq = dq32; p.dk = dk32; p.dv = dv32;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess) return -4;
    if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess) return -4;
    configured = true;
  }
  cudaMemsetAsync(dq32, 0, sizeof(float) * th * HD, s);
  attn_delta_kernel<<<(unsigned)((th + 3) / 4), 128, 0, s>>>((const bf16*)o, (const bf16*)dout, delta, th);
  ++g_att_launches;
  dim3 grid((total_tokens + AB - 1) / AB + num_seqs, heads_q);
  attn_bwd_kernel<<<grid, 128, ATT_SMEM, s>>>(p);
  ++g_att_launches;
  const long long total = th * HD + 2LL * total_tokens * heads_kv * HD;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count_of_current_device() * 16;
  if (blocks > cap) blocks = cap;
  attn_bwd_finalize_kernel<<<(unsigned)blocks, 256, 0, s>>>(dq32, dk32, dv32, (bf16*)dq, (bf16*)dk, (bf16*)dv, total_tokens, heads_q, heads_kv);
  ++g_att_launches;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - (int)e;
}
