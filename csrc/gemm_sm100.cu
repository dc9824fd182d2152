// Persistent warp-specialised bf16 GEMM family for sm_100a.
//
//   TMA (cp.async.bulk.tensor, 128-byte swizzle) -> shared memory ring -> tcgen05.mma (one issuing
//   thread, fp32 accumulators in TMEM, two accumulator buffers) -> tcgen05.ld epilogue.
//
// One kernel covers every matrix product of the training step:
//   mode 0  dense          C[M,N]        = A[M,K] * B[K,N]
//   mode 1  grouped rows   C[rows of g]  = A[rows of g] * B_g      (expert forward / dgrad; row groups
//                                                                   start on 128-row boundaries)
//   mode 2  grouped depth  C_g[M,N]      = sum over rows of g  A[row,:]^T B[row,:]   (weight gradients)
// Operands may be K-major or MN-major (the tensor core transposes from shared memory), so the same
// kernel serves x*W^T, dy*W and dy^T*x without materialising a transpose.
// Options: a second, short depth segment (LoRA: += (s*X*A) * B with its own tensor maps), a dual-B
// mode that computes gate and up projections in one 256-wide MMA and applies SwiGLU in the
// epilogue, alpha scaling and accumulation into C (gradient accumulation), fp32 or bf16 C.
//
// Role layout of a 192-thread CTA: warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM),
// warps 2-5 = epilogue (each owns one 32-lane quarter of TMEM).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <map>
#include <unordered_map>
#include <string.h>
#include <mutex>
#include <tuple>

#include "api.h"
#include "comm.h"
#include "common/ptx.cuh"

namespace mdt {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  CUtensorMap tmA, tmB, tmB2;        // main depth segment (tmB2: second B matrix of the dual mode)
  CUtensorMap tmA_l, tmB_l, tmB2_l;  // optional LoRA depth segment
  int M, N, K, K_l, G, mode;
  int a_mn, b_mn, a_mn_l, b_mn_l, dual;
  const int* offsets;
  void* C; void* C2; void* C3; const void* R;
  long long ldc, c_group_stride;
  int c_fp32, accumulate;
  float alpha;
  int store_gate_up;
  int* status;
  const unsigned* tile_ready; const int* tile_expected;
  const int* row_dest_rank; const int* row_dest_row; const long long* peer_out; const long long* peer_arrive; int num_peers;
  unsigned long long peer_wait_ns;   // limit of the waits for operands that other GPUs or streams deliver
  // B (and B2) may be part of a buffer that an all-gather is still filling: see MdtGemmDesc::b_ready
  MdtOperandReady rdy_b, rdy_b2, rdy_bl;
  long long b_rows, ldb, b_group_stride, bl_rows, ldb_l, bl_group_stride;
  // split of the last, partly filled wave of tiles along the depth (128-row kernel; see get_work)
  float* sk_ws; unsigned* sk_ctr;
};

// Bounded wait until the chunks of the gathered buffer that hold bytes [off, off + len) of an operand have landed.
__device__ __forceinline__ bool wait_operand_ready(const MdtOperandReady& r, long long off, long long len, unsigned long long limit_ns) {
  if (r.ready == nullptr || len <= 0) return true;
  const long long o0 = r.offset_bytes + off, o1 = o0 + len - 1;
  const int c0 = (int)(o0 / r.shard_bytes) * r.chunks_per_rank + (int)((o0 % r.shard_bytes) / r.chunk_bytes);
  const int c1 = (int)(o1 / r.shard_bytes) * r.chunks_per_rank + (int)((o1 % r.shard_bytes) / r.chunk_bytes);
  for (int c = c0; c <= c1; ++c)
    if (!wait_ge(r.ready + c, r.epoch, limit_ns)) return false;
  return true;
}
// The part of B that the tile (group g, columns from n0, `rows` output columns) reads: whole rows of a K-major B,
// the whole matrix of the group for an MN-major one.
__device__ __forceinline__ bool wait_b_tile(const GemmParams& p, int g, int n0, int rows) {
  if (p.rdy_bl.ready != nullptr && p.K_l > 0 &&
      !wait_operand_ready(p.rdy_bl, (long long)g * p.bl_group_stride * 2, p.bl_rows * p.ldb_l * 2, p.peer_wait_ns)) return false;   // whole matrix
  if (p.rdy_b.ready == nullptr && p.rdy_b2.ready == nullptr) return true;
  long long off, len;
  if (p.b_mn == 0) {
    const long long r = (long long)rows < p.b_rows - n0 ? rows : p.b_rows - n0;
    off = ((long long)g * p.b_group_stride + (long long)n0 * p.ldb) * 2;
    len = r * p.ldb * 2;
  } else {
    off = (long long)g * p.b_group_stride * 2;
    len = p.b_rows * p.ldb * 2;
  }
  return wait_operand_ready(p.rdy_b, off, len, p.peer_wait_ns) && wait_operand_ready(p.rdy_b2, off, len, p.peer_wait_ns);
}
// A GEMM that takes part in an exchange does nothing when the status word is already set (an earlier wait of the
// exchange ran out: its metadata describe no rows and nothing may be stored into a peer on the strength of them).
__device__ __forceinline__ bool gemm_dead(const GemmParams& p) {
  return p.status != nullptr && (p.tile_ready != nullptr || p.row_dest_rank != nullptr) && *reinterpret_cast<const volatile int*>(p.status) != 0;
}

struct Tile {
  int g, m0, n0, krow0, num_kb, num_kb_l;
};

// Maps a linear tile index to its coordinates; returns false past the last tile.  (Also callable on the host, where
// a unit test enumerates the tiles of random problems and checks that they cover every block exactly once.)
template <int BN_OUT>
__host__ __device__ __forceinline__ bool get_tile(const GemmParams& p, int t, Tile& o) {
  const int n_blocks = (p.N + BN_OUT - 1) / BN_OUT;
  o.num_kb_l = (p.K_l + BK - 1) / BK;
  if (p.mode == 2) {
    const int m_blocks = (p.M + BM - 1) / BM;
    const int per_group = m_blocks * n_blocks;
    if (t >= per_group * p.G) return false;
    o.g = t / per_group;
    int r = t - o.g * per_group;
    o.m0 = (r % m_blocks) * BM;
    o.n0 = (r / m_blocks) * BN_OUT;
    int k_begin = 0, k_end = p.K;
    if (p.offsets != nullptr) { k_begin = p.offsets[o.g]; k_end = p.offsets[o.g + 1]; }
    o.krow0 = k_begin;
    o.num_kb = (k_end - k_begin + BK - 1) / BK;
    return true;
  }
  int rows = p.M;
  if (p.mode == 1) rows = p.offsets[p.G];
  const int m_blocks = (rows + BM - 1) / BM;
  if (t >= m_blocks * n_blocks) return false;
  o.m0 = (t % m_blocks) * BM;
  o.n0 = (t / m_blocks) * BN_OUT;
  o.g = 0;
  if (p.mode == 1) {
    int g = 0;
    while (g + 1 < p.G && p.offsets[g + 1] <= o.m0) ++g;
    o.g = g;
  }
  o.krow0 = 0;
  o.num_kb = (p.K + BK - 1) / BK;
  return true;
}

// One unit of work of a CTA: a whole output tile, or a piece [kb0, kb1) of the depth of a tile that several CTAs share.
struct Work {
  Tile t;
  int kb0, kb1;        // k blocks of the tile this CTA computes (main segment first, then the LoRA segment)
  int split;           // -1: whole tile.  Otherwise the index of the shared tile (its slot in the fp32 workspace)
  int contributors;    // CTAs that share the tile
};

// Tiles are dealt to the CTAs round robin; when the last round would leave most SMs idle (fewer than 7/8 of them
// get a tile), the tiles of that round are not handed out whole: their k blocks, taken together, are cut into one
// contiguous piece per CTA (a piece spans at most two tiles).  Every CTA adds its piece's partial sums into an fp32
// workspace tile and counts itself in (per 32-row quarter of the tile, i.e. per epilogue warp); the warp that arrives
// last at a quarter reads the sums back and runs the normal epilogue for it.  Nobody waits for anybody.  With 160 tiles of depth 224 on 148 SMs that is 1 round + 18 k blocks per CTA instead of
// 2 rounds (measured 0.136 instead of 0.192 ms).  Products of less than one round are left alone.
// it = 0, 1, ... enumerates the CTA's work in order; returns false when there is no more.
template <int BN_OUT>
__host__ __device__ __forceinline__ bool get_work(const GemmParams& p, int cta, int num_ctas, int it, Work& w) {
  const int n_blocks = (p.N + BN_OUT - 1) / BN_OUT;
  int total_tiles;
  if (p.mode == 2) {
    total_tiles = ((p.M + BM - 1) / BM) * n_blocks * p.G;
  } else {
    const int rows = (p.mode == 1) ? p.offsets[p.G] : p.M;
    total_tiles = ((rows + BM - 1) / BM) * n_blocks;
  }
  const int kbt = (p.K + BK - 1) / BK + (p.K_l + BK - 1) / BK;        // k blocks per tile (modes 0 and 1)
  int whole = total_tiles;
  if (p.sk_ws != nullptr && p.mode != 2 && !p.dual && kbt >= 8) {
    const int rem = total_tiles % num_ctas;
    // (pieces shorter than 8 k blocks are not worth their partial-sum traffic)
    // and a product of less than one full round stays as it is: measured, 80 tiles of depth 64 cut into 148 pieces lose
    // more to the partial sums than they gain)
    if (rem != 0 && total_tiles > num_ctas && rem * 8 < num_ctas * 7 && (long long)rem * kbt >= 8ll * num_ctas) whole = total_tiles - rem;
  }
  const int n_whole = whole > cta ? (whole - cta + num_ctas - 1) / num_ctas : 0;
  w.split = -1; w.contributors = 1;
  if (it < n_whole) {
    if (!get_tile<BN_OUT>(p, cta + it * num_ctas, w.t)) return false;
    w.kb0 = 0;
    w.kb1 = w.t.num_kb + (w.t.num_kb > 0 || p.mode != 2 ? w.t.num_kb_l : 0);
    return true;
  }
  const int rem = total_tiles - whole;
  if (rem == 0) return false;
  const long long units = (long long)rem * kbt;
  const long long per = (units + num_ctas - 1) / num_ctas;
  const long long u0 = (long long)cta * per, u1 = (u0 + per < units) ? u0 + per : units;
  if (u0 >= u1) return false;
  const int t_first = (int)(u0 / kbt), t_last = (int)((u1 - 1) / kbt);
  const int tt = t_first + (it - n_whole);
  if (tt > t_last) return false;
  if (!get_tile<BN_OUT>(p, whole + tt, w.t)) return false;
  const long long lo = (long long)tt * kbt, hi = lo + kbt;
  w.kb0 = (int)((u0 > lo ? u0 : lo) - lo);
  w.kb1 = (int)((u1 < hi ? u1 : hi) - lo);
  w.contributors = (int)((hi - 1) / per) - (int)(lo / per) + 1;
  w.split = w.contributors > 1 ? tt : -1;
  return true;
}

__device__ __forceinline__ void store8(void* C, long long idx, const float (&v0)[8], int c_fp32, int accumulate, const void* R = nullptr) {
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = v0[i];
  if (R != nullptr) {   // residual connection: a bf16 matrix laid out like C
    const uint4 rv = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(R) + idx);
    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(r2[i]); v[2 * i] += f.x; v[2 * i + 1] += f.y; }
  }
  if (c_fp32) {
    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(C) + idx);
    float4 a = make_float4(v[0], v[1], v[2], v[3]), b = make_float4(v[4], v[5], v[6], v[7]);
    if (accumulate) {
      float4 oa = dst[0], ob = dst[1];
      a.x += oa.x; a.y += oa.y; a.z += oa.z; a.w += oa.w;
      b.x += ob.x; b.y += ob.y; b.z += ob.z; b.w += ob.w;
    }
    dst[0] = a; dst[1] = b;
  } else {
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(C) + idx);
    float w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = v[i];
    if (accumulate) {
      uint4 old = *dst;
      const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
      for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(o2[i]); w[2 * i] += f.x; w[2 * i + 1] += f.y; }
    }
    uint4 out;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = __floats2bfloat162_rn(w[2 * i], w[2 * i + 1]);
    *dst = out;
  }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_sm100_kernel(const __grid_constant__ GemmParams p) {
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: a power of two >= 32

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN_OUT = p.dual ? BN / 2 : BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 4); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto fail = [&](int code) {
    *abort_flag = 1;
    if (p.status != nullptr) atomicCAS(p.status, 0, code);
  };

  const bool dead = gemm_dead(p);
  if (dead) {
    // nothing to do; fall through to the common exit
  } else if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ TMA producer
    prefetch_tensormap(&p.tmA); prefetch_tensormap(&p.tmB);
    uint32_t it = 0;
    Work w;
    bool ok = true;
    for (int wi = 0; ok && (p.dual ? get_work<BN / 2>(p, blockIdx.x, gridDim.x, wi, w) : get_work<BN>(p, blockIdx.x, gridDim.x, wi, w)); ++wi) {
      const Tile& t = w.t;
      const int total_kb = w.kb1 - w.kb0;
      if (p.tile_ready != nullptr) {
        // rows of this tile are stored by peer GPUs: wait for them, then order the TMA reads after the acquire
        const int ti = t.m0 / BM;
        if (!wait_ge(p.tile_ready + ti, (unsigned)p.tile_expected[ti], p.peer_wait_ns)) { fail(ST_TIMEOUT_PEER); ok = false; break; }
        fence_proxy_async_all();
      }
      if (p.mode != 2 && total_kb > 0 && (p.rdy_b.ready != nullptr || p.rdy_b2.ready != nullptr || p.rdy_bl.ready != nullptr)) {
        // the weight operand is part of a buffer that an all-gather on another stream is still filling
        if (!wait_b_tile(p, t.g, t.n0, BN_OUT)) { fail(ST_TIMEOUT_PEER); ok = false; break; }
        fence_proxy_async_all();
      }
      for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!wait_parity(&empty_bar[s], ph ^ 1, abort_flag)) { fail(ST_TIMEOUT_EMPTY); ok = false; break; }
        uint8_t* sA = smem + s * STAGE_BYTES;
        uint8_t* sB = sA + A_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        const bool lora = kb >= t.num_kb;
        const int kk = (lora ? kb - t.num_kb : kb) * BK;
        const CUtensorMap* mA = lora ? &p.tmA_l : &p.tmA;
        const CUtensorMap* mB = lora ? &p.tmB_l : &p.tmB;
        const CUtensorMap* mB2 = lora ? &p.tmB2_l : &p.tmB2;
        const int a_mn = lora ? p.a_mn_l : p.a_mn, b_mn = lora ? p.b_mn_l : p.b_mn;
        const int krow = (lora ? 0 : t.krow0) + kk;
        const int zB = (p.mode == 2) ? 0 : t.g;
        if (a_mn == 0) {
          tma_load_2d(sA, mA, &full_bar[s], kk, t.m0);
        } else {
          tma_load_2d(sA, mA, &full_bar[s], t.m0, krow);
          tma_load_2d(sA + 8192, mA, &full_bar[s], t.m0 + 64, krow);
        }
        if (b_mn == 0) {
          if (p.dual) {
            tma_load_3d(sB, mB, &full_bar[s], kk, t.n0, zB);
            tma_load_3d(sB + B_BYTES / 2, mB2, &full_bar[s], kk, t.n0, zB);
          } else {
            tma_load_3d(sB, mB, &full_bar[s], kk, t.n0, zB);
          }
        } else {
          if (p.dual) {
#pragma unroll
            for (int c = 0; c < BN / 128; ++c) {
              tma_load_3d(sB + c * 8192, mB, &full_bar[s], t.n0 + 64 * c, krow, zB);
              tma_load_3d(sB + B_BYTES / 2 + c * 8192, mB2, &full_bar[s], t.n0 + 64 * c, krow, zB);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_3d(sB + c * 8192, mB, &full_bar[s], t.n0 + 64 * c, krow, zB);
          }
        }
      }
    }
    if (!ok) {  // give copies already in flight a bounded time to land before the CTA exits
      for (int s = 0; s < STAGES; ++s) {
        uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(&full_bar[s], 0) && !mbar_try_wait(&full_bar[s], 1) && global_timer_ns() - t0 < 1000000ull) {}
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    uint32_t it = 0, acc_it = 0;
    Work w;
    bool ok = true;
    for (int wi = 0; ok && (p.dual ? get_work<BN / 2>(p, blockIdx.x, gridDim.x, wi, w) : get_work<BN>(p, blockIdx.x, gridDim.x, wi, w)); ++wi) {
      const Tile& t = w.t;
      const int total_kb = w.kb1 - w.kb0;
      if (total_kb == 0) continue;
      const int buf = acc_it & 1;
      const uint32_t aph = (acc_it >> 1) & 1;
      if (!wait_parity(&tempty_bar[buf], aph ^ 1, abort_flag)) { fail(ST_TIMEOUT_TMEM_EMPTY); break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * BN;
      for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!wait_parity(&full_bar[s], ph, abort_flag)) { fail(ST_TIMEOUT_FULL); ok = false; break; }
        tc_fence_after();
        const bool lora = kb >= t.num_kb;
        const int a_mn = lora ? p.a_mn_l : p.a_mn, b_mn = lora ? p.b_mn_l : p.b_mn;
        const uint32_t idesc = make_idesc_bf16(BM, BN, a_mn, b_mn);
        const uint32_t sA = smem_u32(smem + s * STAGE_BYTES);
        const uint32_t sB = sA + A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t da = a_mn ? make_smem_desc(sA + k * 2048, 8192, 1024) : make_smem_desc(sA + k * 32, 16, 1024);
          const uint64_t db = b_mn ? make_smem_desc(sB + k * 2048, 8192, 1024) : make_smem_desc(sB + k * 32, 16, 1024);
          umma_bf16(d_tmem, da, db, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);   // frees the stage when these MMAs have read it
      }
      if (!ok) break;
      umma_commit(&tfull_bar[buf]);   // accumulator complete
      ++acc_it;
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    uint32_t acc_it = 0;
    Work w;
    for (int wi = 0; (p.dual ? get_work<BN / 2>(p, blockIdx.x, gridDim.x, wi, w) : get_work<BN>(p, blockIdx.x, gridDim.x, wi, w)); ++wi) {
      const Tile& t = w.t;
      const int total_kb = w.kb1 - w.kb0;
      const int row = t.m0 + q * 32 + lane;
      const int row_limit = (p.mode == 1) ? p.offsets[p.G] : p.M;
      const bool row_ok = row < row_limit;
      long long base = (p.mode == 2 ? (long long)t.g * p.c_group_stride : 0) + (long long)row * p.ldc;
      void* Cout = p.C;
      int dest = -1;
      bool store_ok = row_ok;
      if (p.row_dest_rank != nullptr) {          // result rows go straight into peers' buffers
        dest = row_ok ? p.row_dest_rank[row] : -1;
        const int drow = row_ok ? p.row_dest_row[row] : -1;
        if (dest >= p.num_peers || drow < 0) dest = -1;
        store_ok = dest >= 0;
        if (store_ok) { Cout = reinterpret_cast<void*>(p.peer_out[dest]); base = (long long)drow * p.ldc; }
      }
      if (total_kb == 0) {
        if (!p.accumulate && row_ok) {
          float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int c = 0; c < BN_OUT; c += 8)
            if (t.n0 + c < p.N) store8(p.C, base + t.n0 + c, z, p.c_fp32, 0);
        }
        continue;
      }
      const int buf = acc_it & 1;
      const uint32_t aph = (acc_it >> 1) & 1;
      if (!wait_parity(&tfull_bar[buf], aph, abort_flag)) { fail(ST_TIMEOUT_TMEM_FULL); break; }
      __syncwarp();   // lanes may leave the wait loop at different times; the TMEM loads below are warp-aligned
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
      if (p.dual) {
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr + c, rg);
          tmem_ld_32x32(taddr + BN / 2 + c, ru);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = t.n0 + c + v * 8;
              if (col < p.N) {
                float h[8], gg[8], uu[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  gg[i] = __uint_as_float(rg[v * 8 + i]);
                  uu[i] = __uint_as_float(ru[v * 8 + i]);
                  h[i] = gg[i] / (1.0f + __expf(-gg[i])) * uu[i];
                }
                store8(p.C, base + col, h, 0, 0);
                if (p.store_gate_up) { store8(p.C2, base + col, gg, 0, 0); store8(p.C3, base + col, uu, 0, 0); }
              }
            }
          }
          __syncwarp();   // the next TMEM load is warp-aligned
        }
      } else if (w.split >= 0) {
        // A piece of a shared tile: add the partial sums into the tile's fp32 workspace (column-major inside the tile,
        // so that the 32 rows of a warp are 128 contiguous bytes), release the accumulator, count this CTA in, and
        // if it is the last one of the tile's contributors, read the sums back and finish the tile.
        float* ws = p.sk_ws + (long long)w.split * (BM * BN) + (q * 32 + lane);
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) atomicAdd(ws + (c + i) * BM, __uint_as_float(r[i]));
          __syncwarp();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        ++acc_it;
        // Each 32-row quarter of the tile has its own counter, so a warp never has to meet the other warps of its CTA:
        // the warp that arrives last at its quarter finishes that quarter.
        __threadfence();
        __syncwarp();
        unsigned before = 0;
        if (lane == 0) before = atomicAdd(p.sk_ctr + w.split * 4 + q, 1u);
        before = __shfl_sync(0xffffffffu, before, 0);
        const bool last = before == (unsigned)w.contributors - 1u;
        if (!last) continue;
        __threadfence();
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          float acc[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) { acc[i] = __ldcg(ws + (c + i) * BM); __stcg(ws + (c + i) * BM, 0.f); }   // leave the workspace clean
          if (store_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = t.n0 + c + v * 8;
              if (col < p.N) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = acc[v * 8 + i] * p.alpha;
                store8(Cout, base + col, o, p.c_fp32, p.accumulate, p.R);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) p.sk_ctr[w.split * 4 + q] = 0;
        if (p.row_dest_rank != nullptr) {
          __threadfence_system();
          __syncwarp();
          for (int d = 0; d < p.num_peers; ++d) {
            const unsigned m = __ballot_sync(0xffffffffu, dest == d);
            if (lane == 0 && m != 0) red_add_release_sys(reinterpret_cast<unsigned*>(p.peer_arrive[d]), __popc(m));
          }
        }
        continue;
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
          if (store_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = t.n0 + c + v * 8;
              if (col < p.N) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[v * 8 + i]) * p.alpha;
                store8(Cout, base + col, o, p.c_fp32, p.accumulate, p.R);
              }
            }
          }
          __syncwarp();   // the next TMEM load is warp-aligned
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      ++acc_it;
      if (p.row_dest_rank != nullptr) {
        // publish this warp's rows: one count per (row, column tile) and destination
        __threadfence_system();
        __syncwarp();
        for (int d = 0; d < p.num_peers; ++d) {
          const unsigned m = __ballot_sync(0xffffffffu, dest == d);
          if (lane == 0 && m != 0) red_add_release_sys(reinterpret_cast<unsigned*>(p.peer_arrive[d]), __popc(m));
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2).  Two CTAs of a cluster share one 256 x 256 MMA tile: each CTA loads its own
// 128 rows of A and half of B's 256 columns (in the dual mode: the leader the gate matrix, its peer the up
// matrix), the leader's MMA thread reads both CTAs' shared memory, and each CTA's TMEM receives the accumulators
// of its own 128 rows.  Per CTA and 64-deep k block that is 32 KB of operands instead of 48 KB, which is what
// bounds the single-CTA kernel, and the ring holds 7 stages instead of 4.
//   full_bar[s]   (leader's is used): the leader's producer arrives and announces both CTAs' TMA bytes
//   empty_bar[s]  (one per CTA)     : arrives by the leader's commit, delivered to both CTAs
//   tfull_bar[b]  (one per CTA)     : same, when a tile's accumulators are complete
//   tempty_bar[b] (leader's is used): 8 arrivals, the 4 epilogue warps of each CTA
// Every load lands in the shared memory of the CTA that issued it.
// ---------------------------------------------------------------------------------------------
constexpr int PAIR_BN = 256;
constexpr int PAIR_STAGES = 7;
constexpr int PAIR_B_BYTES = 128 * BK * 2;
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;
static_assert(PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256 <= 227 * 1024, "pair kernel: stages + barriers exceed the shared memory of a CTA");

struct PairTile {
  int g, m0, n0, krow0, num_kb, num_kb_l, second_ok;
};

// Pair tiles cover 256 rows.  In the grouped-rows mode a pair never straddles two groups: a group with an odd
// number of 128-row blocks ends with a pair whose second half is idle (second_ok = 0).
template <int BN_OUT>
__host__ __device__ __forceinline__ bool get_pair_tile(const GemmParams& p, int t, PairTile& o) {
  const int n_blocks = (p.N + BN_OUT - 1) / BN_OUT;
  o.num_kb_l = (p.K_l + BK - 1) / BK;
  o.second_ok = 1;
  if (p.mode == 2) {
    const int m_pairs = (p.M + 2 * BM - 1) / (2 * BM);
    const int per_group = m_pairs * n_blocks;
    if (t >= per_group * p.G) return false;
    o.g = t / per_group;
    const int r = t - o.g * per_group;
    o.m0 = (r % m_pairs) * 2 * BM;
    o.n0 = (r / m_pairs) * BN_OUT;
    int k_begin = 0, k_end = p.K;
    if (p.offsets != nullptr) { k_begin = p.offsets[o.g]; k_end = p.offsets[o.g + 1]; }
    o.krow0 = k_begin;
    o.num_kb = (k_end - k_begin + BK - 1) / BK;
    return true;
  }
  o.krow0 = 0;
  o.num_kb = (p.K + BK - 1) / BK;
  if (p.mode == 0) {
    const int m_pairs = (p.M + 2 * BM - 1) / (2 * BM);
    if (t >= m_pairs * n_blocks) return false;
    o.g = 0;
    o.m0 = (t % m_pairs) * 2 * BM;
    o.n0 = (t / m_pairs) * BN_OUT;
    return true;
  }
  int total = 0;
  for (int g = 0; g < p.G; ++g) total += ((p.offsets[g + 1] - p.offsets[g]) / BM + 1) / 2;
  if (total == 0 || t >= total * n_blocks) return false;
  int mp = t % total;
  o.n0 = (t / total) * BN_OUT;
  for (int g = 0; g < p.G; ++g) {
    const int begin = p.offsets[g], end = p.offsets[g + 1];
    const int pairs = ((end - begin) / BM + 1) / 2;
    if (mp < pairs) {
      o.g = g;
      o.m0 = begin + mp * 2 * BM;
      o.second_ok = (o.m0 + BM < end) ? 1 : 0;
      return true;
    }
    mp -= pairs;
  }
  return false;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1) gemm_sm100_pair_kernel(const __grid_constant__ GemmParams p) {
  constexpr int STAGES = PAIR_STAGES;
  constexpr int BN = PAIR_BN;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared memory starts at the same offset in both CTAs, so the aligned tile addresses match too
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * PAIR_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();          // 0 = leader
  const int pair_id = (int)cluster_id_x(), num_pairs = (int)num_clusters_x();
  const int BN_OUT = p.dual ? BN / 2 : BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 8); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto fail = [&](int code) {
    *abort_flag = 1;
    if (p.status != nullptr) atomicCAS(p.status, 0, code);
  };

  const bool dead = gemm_dead(p);   // the same in both CTAs of the pair: the word never returns to zero while kernels run
  if (dead) {
    // nothing to do; fall through to the common exit
  } else if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ TMA producer (one per CTA)
    prefetch_tensormap(&p.tmA); prefetch_tensormap(&p.tmB);
    uint32_t it = 0;
    PairTile t;
    bool ok = true;
    for (int tile = pair_id; ok && (p.dual ? get_pair_tile<BN / 2>(p, tile, t) : get_pair_tile<BN>(p, tile, t)); tile += num_pairs) {
      const int total_kb = t.num_kb + (t.num_kb > 0 || p.mode != 2 ? t.num_kb_l : 0);
      const int my_m0 = t.m0 + (int)cta_rank * BM;
      const bool half_ok = cta_rank == 0 || t.second_ok;
      if (p.tile_ready != nullptr && half_ok && total_kb > 0) {
        const int ti = my_m0 / BM;
        if (!wait_ge(p.tile_ready + ti, (unsigned)p.tile_expected[ti], p.peer_wait_ns)) { fail(ST_TIMEOUT_PEER); ok = false; break; }
        fence_proxy_async_all();
      }
      if (p.mode != 2 && total_kb > 0 && (p.rdy_b.ready != nullptr || p.rdy_b2.ready != nullptr || p.rdy_bl.ready != nullptr)) {
        if (!wait_b_tile(p, t.g, t.n0, BN_OUT)) { fail(ST_TIMEOUT_PEER); ok = false; break; }
        fence_proxy_async_all();
      }
      for (int kb = 0; kb < total_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!wait_parity(&empty_bar[s], ph ^ 1, abort_flag)) { fail(ST_TIMEOUT_EMPTY); ok = false; break; }
        uint8_t* sA = smem + s * PAIR_STAGE_BYTES;
        uint8_t* sB = sA + A_BYTES;
        // Only the leader arrives, announcing both CTAs' bytes: a cluster-scope arrive from the peer would put a
        // memory barrier into every stage of its producer loop.  The peer's bytes may be counted before the
        // leader's announcement (the transaction count goes negative for a moment; the phase cannot complete
        // before the leader's arrival).
        const uint32_t bar = mapa_shared(smem_u32(&full_bar[s]), 0);
        if (cta_rank == 0) mbar_expect_tx(&full_bar[s], 2 * PAIR_STAGE_BYTES);
        const bool lora = kb >= t.num_kb;
        const int kk = (lora ? kb - t.num_kb : kb) * BK;
        const CUtensorMap* mA = lora ? &p.tmA_l : &p.tmA;
        const CUtensorMap* mB = lora ? &p.tmB_l : &p.tmB;
        const int a_mn = lora ? p.a_mn_l : p.a_mn, b_mn = lora ? p.b_mn_l : p.b_mn;
        const int krow = (lora ? 0 : t.krow0) + kk;
        if (a_mn == 0) {
          tma_load_2d_pair(sA, mA, bar, kk, my_m0);
        } else {
          tma_load_2d_pair(sA, mA, bar, my_m0, krow);
          tma_load_2d_pair(sA + 8192, mA, bar, my_m0 + 64, krow);
        }
        const int zB = (p.mode == 2) ? 0 : t.g;
        // this CTA's half of B: columns n0 + 128*rank, or in the dual mode the gate (leader) / up (peer) matrix
        if (p.dual && cta_rank == 1) mB = lora ? &p.tmB2_l : &p.tmB2;
        const int my_n0 = p.dual ? t.n0 : t.n0 + (int)cta_rank * 128;
        if (b_mn == 0) {
          tma_load_3d_pair(sB, mB, bar, kk, my_n0, zB);
        } else {
          tma_load_3d_pair(sB, mB, bar, my_n0, krow, zB);
          tma_load_3d_pair(sB + 8192, mB, bar, my_n0 + 64, krow, zB);
        }
      }
    }
    if (!ok) {  // give this CTA's copies already in flight a bounded time to land before it leaves
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {}
    }
  } else if (warp == 1 && lane == 0 && cta_rank == 0) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    uint32_t it = 0, acc_it = 0;
    PairTile t;
    bool ok = true;
    for (int tile = pair_id; ok && (p.dual ? get_pair_tile<BN / 2>(p, tile, t) : get_pair_tile<BN>(p, tile, t)); tile += num_pairs) {
      const int total_kb = t.num_kb + (t.num_kb > 0 || p.mode != 2 ? t.num_kb_l : 0);
      if (total_kb == 0) continue;
      const int buf = acc_it & 1;
      const uint32_t aph = (acc_it >> 1) & 1;
      if (!wait_parity(&tempty_bar[buf], aph ^ 1, abort_flag)) { fail(ST_TIMEOUT_TMEM_EMPTY); break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * BN;
      for (int kb = 0; kb < total_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!wait_parity(&full_bar[s], ph, abort_flag)) { fail(ST_TIMEOUT_FULL); ok = false; break; }
        tc_fence_after();
        const bool lora = kb >= t.num_kb;
        const int a_mn = lora ? p.a_mn_l : p.a_mn, b_mn = lora ? p.b_mn_l : p.b_mn;
        const uint32_t idesc = make_idesc_bf16(2 * BM, BN, a_mn, b_mn);
        const uint32_t sA = smem_u32(smem + s * PAIR_STAGE_BYTES);
        const uint32_t sB = sA + A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t da = a_mn ? make_smem_desc(sA + k * 2048, 8192, 1024) : make_smem_desc(sA + k * 32, 16, 1024);
          const uint64_t db = b_mn ? make_smem_desc(sB + k * 2048, 8192, 1024) : make_smem_desc(sB + k * 32, 16, 1024);
          umma_bf16_pair(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit_pair(&empty_bar[s], 3);   // frees the stage in both CTAs
      }
      if (!ok) break;
      umma_commit_pair(&tfull_bar[buf], 3);   // accumulators complete, in both CTAs
      ++acc_it;
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    uint32_t acc_it = 0;
    PairTile t;
    for (int tile = pair_id; (p.dual ? get_pair_tile<BN / 2>(p, tile, t) : get_pair_tile<BN>(p, tile, t)); tile += num_pairs) {
      const int total_kb = t.num_kb + (t.num_kb > 0 || p.mode != 2 ? t.num_kb_l : 0);
      const bool half_ok = cta_rank == 0 || t.second_ok;
      const int row = t.m0 + (int)cta_rank * BM + q * 32 + lane;
      const int row_limit = (p.mode == 1) ? p.offsets[p.G] : p.M;
      const bool row_ok = half_ok && row < row_limit;
      long long base = (p.mode == 2 ? (long long)t.g * p.c_group_stride : 0) + (long long)row * p.ldc;
      void* Cout = p.C;
      int dest = -1;
      bool store_ok = row_ok;
      if (p.row_dest_rank != nullptr) {          // result rows go straight into peers' buffers
        dest = row_ok ? p.row_dest_rank[row] : -1;
        const int drow = row_ok ? p.row_dest_row[row] : -1;
        if (dest >= p.num_peers || drow < 0) dest = -1;
        store_ok = dest >= 0;
        if (store_ok) { Cout = reinterpret_cast<void*>(p.peer_out[dest]); base = (long long)drow * p.ldc; }
      }
      if (total_kb == 0) {
        if (!p.accumulate && row_ok) {
          float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int c = 0; c < BN_OUT; c += 8)
            if (t.n0 + c < p.N) store8(p.C, base + t.n0 + c, z, p.c_fp32, 0);
        }
        continue;
      }
      const int buf = acc_it & 1;
      const uint32_t aph = (acc_it >> 1) & 1;
      if (!wait_parity(&tfull_bar[buf], aph, abort_flag)) { fail(ST_TIMEOUT_TMEM_FULL); break; }
      __syncwarp();   // lanes may leave the wait loop at different times; the TMEM loads below are warp-aligned
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
      if (p.dual) {
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr + c, rg);
          tmem_ld_32x32(taddr + BN / 2 + c, ru);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = t.n0 + c + v * 8;
              if (col < p.N) {
                float h[8], gg[8], uu[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  gg[i] = __uint_as_float(rg[v * 8 + i]);
                  uu[i] = __uint_as_float(ru[v * 8 + i]);
                  h[i] = gg[i] / (1.0f + __expf(-gg[i])) * uu[i];
                }
                store8(p.C, base + col, h, 0, 0);
                if (p.store_gate_up) { store8(p.C2, base + col, gg, 0, 0); store8(p.C3, base + col, uu, 0, 0); }
              }
            }
          }
          __syncwarp();   // the next TMEM load is warp-aligned
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
          if (store_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = t.n0 + c + v * 8;
              if (col < p.N) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[v * 8 + i]) * p.alpha;
                store8(Cout, base + col, o, p.c_fp32, p.accumulate, p.R);
              }
            }
          }
          __syncwarp();   // the next TMEM load is warp-aligned
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[buf]), 0));
      ++acc_it;
      if (p.row_dest_rank != nullptr) {
        // publish this warp's rows: one count per (row, column tile) and destination
        __threadfence_system();
        __syncwarp();
        for (int d = 0; d < p.num_peers; ++d) {
          const unsigned m = __ballot_sync(0xffffffffu, dest == d);
          if (lane == 0 && m != 0) red_add_release_sys(reinterpret_cast<unsigned*>(p.peer_arrive[d]), __popc(m));
        }
      }
    }
  }

  // Neither CTA may leave while its partner can still read its shared memory or arrive on its barriers.
  __syncwarp();
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}

// ---------------------------------------------------------------------------------------------
// Tall variant: one CTA computes a 256 x 256 tile as two 128-row MMAs that share the B operand.  Per 64-deep
// k block the CTA takes in 64 KB for 256 x 256 x 64 MACs, i.e. 32 KB per 128 x 256 x 64, against 48 KB in the
// 128 x 256 kernel, whose k blocks arrive more slowly than its MMAs retire them.  The two accumulators fill
// all 512 TMEM columns, so the epilogue of a tile does not overlap the next tile's MMAs (its loads do); eight
// epilogue warps (two per TMEM lane quarter, one per 128-row half) keep that phase short.
// Roles of the 320 threads: warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM), warps 2-9 = epilogue.
// ---------------------------------------------------------------------------------------------
// Coalesced bf16 store of one 32-row x 32-column block held as one row per lane: the warp transposes it through a
// 2 KB shared-memory stage (16-byte slots, XOR-swizzled so that both passes are conflict-free) and then writes
// 64 contiguous bytes per row, eight rows per instruction, instead of 16 bytes to each of 32 rows.
// row_ptr[i] / bit i of ok_mask describe row i*8 + lane/4, the row this lane stores in pass i.
__device__ __forceinline__ void store32_coalesced(uint8_t* stage, const float (&v)[32], int lane, const unsigned long long (&row_ptr)[4],
                                                  unsigned ok_mask, int col0, int N) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 out;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = __floats2bfloat162_rn(v[j * 8 + 2 * i], v[j * 8 + 2 * i + 1]);
    *reinterpret_cast<uint4*>(stage + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) = out;
  }
  __syncwarp();
  const int j = lane & 3;
  const int col = col0 + j * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = i * 8 + (lane >> 2);
    const uint4 val = *reinterpret_cast<const uint4*>(stage + row * 64 + ((j ^ ((row >> 1) & 3)) << 4));
    if (((ok_mask >> i) & 1u) && col < N)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(row_ptr[i]) + col) = val;
  }
  __syncwarp();
}

constexpr int TALL_THREADS = 320;
constexpr int TALL_STAGES = 3;
constexpr int TALL_BN = 256;
constexpr int TALL_STAGE_BYTES = 2 * A_BYTES + TALL_BN * BK * 2;
static_assert(TALL_STAGES * TALL_STAGE_BYTES + 1024 + 256 + 8 * 2048 <= 227 * 1024, "tall kernel: stages + barriers + store stage exceed the shared memory of a CTA");
static_assert(TALL_THREADS == 32 * (2 + 8), "tall kernel: producer, MMA issuer and eight epilogue warps");

__global__ void __launch_bounds__(TALL_THREADS, 1) gemm_sm100_tall_kernel(const __grid_constant__ GemmParams p) {
  constexpr int STAGES = TALL_STAGES;
  constexpr int BN = TALL_BN;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * TALL_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* store_stage = smem + STAGES * TALL_STAGE_BYTES + 256;   // 8 epilogue warps x 2 KB

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN_OUT = p.dual ? BN / 2 : BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto fail = [&](int code) {
    *abort_flag = 1;
    if (p.status != nullptr) atomicCAS(p.status, 0, code);
  };

  const bool dead = gemm_dead(p);
  if (dead) {
    // nothing to do; fall through to the common exit
  } else if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ TMA producer
    prefetch_tensormap(&p.tmA); prefetch_tensormap(&p.tmB);
    uint32_t it = 0;
    PairTile t;
    bool ok = true;
    for (int tile = blockIdx.x; ok && (p.dual ? get_pair_tile<BN / 2>(p, tile, t) : get_pair_tile<BN>(p, tile, t)); tile += gridDim.x) {
      const int total_kb = t.num_kb + (t.num_kb > 0 || p.mode != 2 ? t.num_kb_l : 0);
      if (p.tile_ready != nullptr && total_kb > 0) {
        for (int h = 0; h < (t.second_ok ? 2 : 1) && ok; ++h) {
          const int ti = t.m0 / BM + h;
          if (!wait_ge(p.tile_ready + ti, (unsigned)p.tile_expected[ti], p.peer_wait_ns)) { fail(ST_TIMEOUT_PEER); ok = false; }
        }
        if (!ok) break;
        fence_proxy_async_all();
      }
      if (p.mode != 2 && total_kb > 0 && (p.rdy_b.ready != nullptr || p.rdy_b2.ready != nullptr || p.rdy_bl.ready != nullptr)) {
        if (!wait_b_tile(p, t.g, t.n0, BN_OUT)) { fail(ST_TIMEOUT_PEER); ok = false; break; }
        fence_proxy_async_all();
      }
      for (int kb = 0; kb < total_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!wait_parity(&empty_bar[s], ph ^ 1, abort_flag)) { fail(ST_TIMEOUT_EMPTY); ok = false; break; }
        uint8_t* sA = smem + s * TALL_STAGE_BYTES;
        uint8_t* sB = sA + 2 * A_BYTES;
        mbar_expect_tx(&full_bar[s], TALL_STAGE_BYTES);
        const bool lora = kb >= t.num_kb;
        const int kk = (lora ? kb - t.num_kb : kb) * BK;
        const CUtensorMap* mA = lora ? &p.tmA_l : &p.tmA;
        const CUtensorMap* mB = lora ? &p.tmB_l : &p.tmB;
        const CUtensorMap* mB2 = lora ? &p.tmB2_l : &p.tmB2;
        const int a_mn = lora ? p.a_mn_l : p.a_mn, b_mn = lora ? p.b_mn_l : p.b_mn;
        const int krow = (lora ? 0 : t.krow0) + kk;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int m0 = t.m0 + h * BM;
          if (a_mn == 0) {
            tma_load_2d(sA + h * A_BYTES, mA, &full_bar[s], kk, m0);
          } else {
            tma_load_2d(sA + h * A_BYTES, mA, &full_bar[s], m0, krow);
            tma_load_2d(sA + h * A_BYTES + 8192, mA, &full_bar[s], m0 + 64, krow);
          }
        }
        const int zB = (p.mode == 2) ? 0 : t.g;
        if (b_mn == 0) {
          if (p.dual) {
            tma_load_3d(sB, mB, &full_bar[s], kk, t.n0, zB);
            tma_load_3d(sB + B_BYTES / 2, mB2, &full_bar[s], kk, t.n0, zB);
          } else {
            tma_load_3d(sB, mB, &full_bar[s], kk, t.n0, zB);
            tma_load_3d(sB + B_BYTES / 2, mB, &full_bar[s], kk, t.n0 + 128, zB);
          }
        } else {
          if (p.dual) {
#pragma unroll
            for (int c = 0; c < BN / 128; ++c) {
              tma_load_3d(sB + c * 8192, mB, &full_bar[s], t.n0 + 64 * c, krow, zB);
              tma_load_3d(sB + B_BYTES / 2 + c * 8192, mB2, &full_bar[s], t.n0 + 64 * c, krow, zB);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_3d(sB + c * 8192, mB, &full_bar[s], t.n0 + 64 * c, krow, zB);
          }
        }
      }
    }
    if (!ok) {  // give copies already in flight a bounded time to land before the CTA exits
      for (int s = 0; s < STAGES; ++s) {
        uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(&full_bar[s], 0) && !mbar_try_wait(&full_bar[s], 1) && global_timer_ns() - t0 < 1000000ull) {}
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    uint32_t it = 0, acc_it = 0;
    PairTile t;
    bool ok = true;
    for (int tile = blockIdx.x; ok && (p.dual ? get_pair_tile<BN / 2>(p, tile, t) : get_pair_tile<BN>(p, tile, t)); tile += gridDim.x) {
      const int total_kb = t.num_kb + (t.num_kb > 0 || p.mode != 2 ? t.num_kb_l : 0);
      if (total_kb == 0) continue;
      if (!wait_parity(tempty_bar, (acc_it & 1) ^ 1, abort_flag)) { fail(ST_TIMEOUT_TMEM_EMPTY); break; }
      tc_fence_after();
      for (int kb = 0; kb < total_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!wait_parity(&full_bar[s], ph, abort_flag)) { fail(ST_TIMEOUT_FULL); ok = false; break; }
        tc_fence_after();
        const bool lora = kb >= t.num_kb;
        const int a_mn = lora ? p.a_mn_l : p.a_mn, b_mn = lora ? p.b_mn_l : p.b_mn;
        const uint32_t idesc = make_idesc_bf16(BM, BN, a_mn, b_mn);
        const uint32_t sA = smem_u32(smem + s * TALL_STAGE_BYTES);
        const uint32_t sB = sA + 2 * A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t db = b_mn ? make_smem_desc(sB + k * 2048, 8192, 1024) : make_smem_desc(sB + k * 32, 16, 1024);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t a0 = sA + h * A_BYTES;
            const uint64_t da = a_mn ? make_smem_desc(a0 + k * 2048, 8192, 1024) : make_smem_desc(a0 + k * 32, 16, 1024);
            umma_bf16(tmem_base + h * BN, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(&empty_bar[s]);   // frees the stage when these MMAs have read it
      }
      if (!ok) break;
      umma_commit(tfull_bar);         // both accumulators complete
      ++acc_it;
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue: warp -> (lane quarter, row half)
    const int q = warp & 3;
    const int h = (warp - 2) >> 2;
    uint32_t acc_it = 0;
    PairTile t;
    for (int tile = blockIdx.x; (p.dual ? get_pair_tile<BN / 2>(p, tile, t) : get_pair_tile<BN>(p, tile, t)); tile += gridDim.x) {
      const int total_kb = t.num_kb + (t.num_kb > 0 || p.mode != 2 ? t.num_kb_l : 0);
      const bool half_ok = h == 0 || t.second_ok;
      const int row = t.m0 + h * BM + q * 32 + lane;
      const int row_limit = (p.mode == 1) ? p.offsets[p.G] : p.M;
      const bool row_ok = half_ok && row < row_limit;
      long long base = (p.mode == 2 ? (long long)t.g * p.c_group_stride : 0) + (long long)row * p.ldc;
      void* Cout = p.C;
      int dest = -1;
      bool store_ok = row_ok;
      if (p.row_dest_rank != nullptr) {          // result rows go straight into peers' buffers
        dest = row_ok ? p.row_dest_rank[row] : -1;
        const int drow = row_ok ? p.row_dest_row[row] : -1;
        if (dest >= p.num_peers || drow < 0) dest = -1;
        store_ok = dest >= 0;
        if (store_ok) { Cout = reinterpret_cast<void*>(p.peer_out[dest]); base = (long long)drow * p.ldc; }
      }
      if (total_kb == 0) {
        if (!p.accumulate && row_ok) {
          float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int c = 0; c < BN_OUT; c += 8)
            if (t.n0 + c < p.N) store8(p.C, base + t.n0 + c, z, p.c_fp32, 0);
        }
        continue;
      }
      if (!wait_parity(tfull_bar, acc_it & 1, abort_flag)) { fail(ST_TIMEOUT_TMEM_FULL); break; }
      __syncwarp();   // lanes may leave the wait loop at different times; the TMEM loads below are warp-aligned
      tc_fence_after();
      const uint32_t taddr = tmem_base + h * BN + ((uint32_t)(q * 32) << 16);
      // bf16 results without accumulation go out through the coalescing stage; the row this lane stores in pass i
      // is row i*8 + lane/4 of the warp's 32, whose address and validity come from the lane that owns it
      const bool fast = !p.c_fp32 && !p.accumulate && p.R == nullptr;
      uint8_t* stage = store_stage + (warp - 2) * 2048;
      unsigned long long rptr[4] = {0, 0, 0, 0};
      unsigned okm = 0;
      if (fast) {
        const unsigned long long mine = reinterpret_cast<unsigned long long>(reinterpret_cast<__nv_bfloat16*>(Cout) + base);
        const int okv = (p.dual ? row_ok : store_ok) ? 1 : 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int src = i * 8 + (lane >> 2);
          rptr[i] = __shfl_sync(0xffffffffu, mine, src);
          okm |= (unsigned)(__shfl_sync(0xffffffffu, okv, src) & 1) << i;
        }
      }
      if (p.dual) {
        const long long d2 = reinterpret_cast<const char*>(p.C2) - reinterpret_cast<const char*>(p.C);
        const long long d3 = reinterpret_cast<const char*>(p.C3) - reinterpret_cast<const char*>(p.C);
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr + c, rg);
          tmem_ld_32x32(taddr + BN / 2 + c, ru);
          tmem_ld_wait();
          if (fast) {
            float hh[32], gg[32], uu[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              gg[i] = __uint_as_float(rg[i]);
              uu[i] = __uint_as_float(ru[i]);
              hh[i] = gg[i] / (1.0f + __expf(-gg[i])) * uu[i];
            }
            store32_coalesced(stage, hh, lane, rptr, okm, t.n0 + c, p.N);
            if (p.store_gate_up) {
              unsigned long long r2[4], r3[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) { r2[i] = rptr[i] + d2; r3[i] = rptr[i] + d3; }
              store32_coalesced(stage, gg, lane, r2, okm, t.n0 + c, p.N);
              store32_coalesced(stage, uu, lane, r3, okm, t.n0 + c, p.N);
            }
          } else if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = t.n0 + c + v * 8;
              if (col < p.N) {
                float hh[8], gg[8], uu[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  gg[i] = __uint_as_float(rg[v * 8 + i]);
                  uu[i] = __uint_as_float(ru[v * 8 + i]);
                  hh[i] = gg[i] / (1.0f + __expf(-gg[i])) * uu[i];
                }
                store8(p.C, base + col, hh, 0, 0);
                if (p.store_gate_up) { store8(p.C2, base + col, gg, 0, 0); store8(p.C3, base + col, uu, 0, 0); }
              }
            }
          }
          __syncwarp();   // the next TMEM load is warp-aligned
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
          if (fast) {
            float o[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(r[i]) * p.alpha;
            store32_coalesced(stage, o, lane, rptr, okm, t.n0 + c, p.N);
          } else if (store_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = t.n0 + c + v * 8;
              if (col < p.N) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[v * 8 + i]) * p.alpha;
                store8(Cout, base + col, o, p.c_fp32, p.accumulate, p.R);
              }
            }
          }
          __syncwarp();   // the next TMEM load is warp-aligned
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar);
      ++acc_it;
      if (p.row_dest_rank != nullptr) {
        // publish this warp's rows: one count per (row, column tile) and destination
        __threadfence_system();
        __syncwarp();
        for (int d = 0; d < p.num_peers; ++d) {
          const unsigned m = __ballot_sync(0xffffffffu, dest == d);
          if (lane == 0 && m != 0) red_add_release_sys(reinterpret_cast<unsigned*>(p.peer_arrive[d]), __popc(m));
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// bf16 tensor [d2][d1][d0] (d0 contiguous), strides in elements; box = {b0, b1, 1}
// Encoded maps are cached per host thread: a training step re-uses the same (pointer, shape, box) combinations
// (weights, pooled gather buffers, allocator-recycled activations) thousands of times.
struct MapKey {
  uint64_t v[8];
  bool operator==(const MapKey& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i < 8; ++i) { h ^= k.v[i]; h *= 1099511628211ull; }
    return (size_t)h;
  }
};
static int make_map_uncached(CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2,
                             uint32_t b0, uint32_t b1, int rank);
static int make_map(CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2,
                    uint32_t b0, uint32_t b1, int rank) {
  static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey k{{(uint64_t)reinterpret_cast<uintptr_t>(ptr), d0, d1, d2, s1, s2, ((uint64_t)b0 << 32) | b1, (uint64_t)rank}};
  auto it = cache.find(k);
  if (it != cache.end()) { *m = it->second; return 0; }
  int rc = make_map_uncached(m, ptr, d0, d1, d2, s1, s2, b0, b1, rank);
  if (rc == 0) {
    if (cache.size() > 65536) cache.clear();
    cache.emplace(k, *m);
  }
  return rc;
}
static int make_map_uncached(CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2,
                             uint32_t b0, uint32_t b1, int rank) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1 * 2, s2 * 2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (strides[0] & 15) || (rank == 3 && (strides[1] & 15))) return -2;
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

static int g_num_sms = 0;
static long long g_launches = 0;

// Workspace of the split last wave: one fp32 tile per SM plus four counters per tile, zero between launches (the warp
// that finishes a shared tile clears what it read).  One workspace per stream, since launches on different streams may
// overlap on the GPU; created on the stream's first product that can use it.  MDT_GEMM_SPLIT=0 switches the split off.
struct SplitWorkspace { float* ws; unsigned* ctr; };
static std::mutex g_split_mutex;
static std::map<std::pair<int, cudaStream_t>, SplitWorkspace> g_split_ws;
static int g_split_enabled = -1;
static bool split_enabled() {
  if (g_split_enabled < 0) {
    const char* e = getenv("MDT_GEMM_SPLIT");
    g_split_enabled = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return g_split_enabled == 1;
}
static bool split_workspace(cudaStream_t stream, SplitWorkspace* out) {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(g_split_mutex);
  auto key = std::make_pair(dev, stream);
  auto it = g_split_ws.find(key);
  if (it == g_split_ws.end()) {
    if (g_split_ws.size() >= 64) return false;          // more streams than expected: those products run unsplit
    SplitWorkspace w{nullptr, nullptr};
    const size_t ws_bytes = (size_t)g_num_sms * BM * 256 * sizeof(float), ctr_bytes = (size_t)g_num_sms * 4 * sizeof(unsigned);
    if (cudaMalloc(&w.ws, ws_bytes) != cudaSuccess) { cudaGetLastError(); return false; }
    if (cudaMalloc(&w.ctr, ctr_bytes) != cudaSuccess) { cudaGetLastError(); cudaFree(w.ws); return false; }
    cudaMemset(w.ws, 0, ws_bytes);
    cudaMemset(w.ctr, 0, ctr_bytes);
    it = g_split_ws.emplace(key, w).first;
  }
  *out = it->second;
  return true;
}

template <int BN, int STAGES>
static cudaError_t launch(const GemmParams& p, int grid, cudaStream_t stream) {
  constexpr int smem = STAGES * (A_BYTES + BN * BK * 2) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_sm100_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  gemm_sm100_kernel<BN, STAGES><<<grid, GEMM_THREADS, smem, stream>>>(p);
  ++g_launches;
  return cudaGetLastError();
}

static cudaError_t launch_tall(const GemmParams& p, int grid, cudaStream_t stream) {
  constexpr int smem = TALL_STAGES * TALL_STAGE_BYTES + 1024 + 256 + 8 * 2048;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_sm100_tall_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  gemm_sm100_tall_kernel<<<grid, TALL_THREADS, smem, stream>>>(p);
  ++g_launches;
  return cudaGetLastError();
}

// Number of CTA pairs that can be resident at once (pairs never span GPCs, so this can be below SMs / 2); the
// persistent grid is sized to it because tiles are assigned to pairs statically.
static int g_max_pairs = 0;
static int g_pair_cap = 0;   // optional upper bound set through mdt_gemm_set_pair_cap (0 = none)

static cudaError_t launch_pair(const GemmParams& p, int pairs_wanted, cudaStream_t stream) {
  constexpr int smem = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_sm100_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(g_num_sms & ~1)); cfg.blockDim = dim3(GEMM_THREADS); cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_sm100_pair_kernel, &cfg) != cudaSuccess || n < 1) { cudaGetLastError(); n = g_num_sms / 2; }
    g_max_pairs = n < g_num_sms / 2 ? n : g_num_sms / 2;
    configured = true;
  }
  const int limit = (g_pair_cap > 0 && g_pair_cap < g_max_pairs) ? g_pair_cap : g_max_pairs;
  const int grid = 2 * (pairs_wanted < limit ? pairs_wanted : limit);
  gemm_sm100_pair_kernel<<<grid, GEMM_THREADS, smem, stream>>>(p);
  ++g_launches;
  return cudaGetLastError();
}

// Expected number of rows of the row-grouped products issued by this thread (0 = unknown); see mdt_gemm_rows_hint.
static thread_local long long t_rows_hint = 0;

// Which kernel takes the 256-wide tiles: 0 = the 128-row kernel always, 1 = the CTA-pair kernel where the shape
// fills 256-row tiles, 2 = the CTA-pair kernel always (tests), 3 = the tall kernel where the shape fills
// several waves of 256-row tiles (default), 4 = the tall kernel always (tests).  Initial value from MDT_GEMM_PAIR;
// mdt_gemm_set_pair_policy() changes it.
static int g_pair_policy = -1;
static int pair_policy() {
  if (g_pair_policy < 0) {
    const char* e = getenv("MDT_GEMM_PAIR");
    g_pair_policy = (e != nullptr && e[0] >= '0' && e[0] <= '4') ? e[0] - '0' : 3;
  }
  return g_pair_policy;
}

// Which kernel runs a product: 0 = 128-row tiles, 1 = CTA pair, 2 = tall 256 x 256 tiles.  Pure arithmetic on the
// descriptor (no CUDA call), so that it can be examined without a GPU.
static int choose_tiling(const MdtGemmDesc* d, int policy, long long thread_rows_hint, int num_sms) {
  const int G = d->G < 1 ? 1 : d->G;
  const int BN = (d->dual || d->N > 128) ? 256 : 128;
  const int bn_out = d->dual ? BN / 2 : BN;
  if (BN != 256) return 0;
  // The CTA-pair kernel needs 256-row pair tiles that are mostly full: dense and depth-grouped products with
  // M >= 256, and row-grouped products whose groups average at least four 128-row blocks.
  const long long rows_hint = (d->mode == 1) ? d->capacity_rows : d->M;
  const bool fills = rows_hint >= 2 * BM && (d->mode != 1 || rows_hint >= (long long)G * 4 * BM);
  if (policy == 2 || (policy == 1 && fills)) return 1;
  if (policy == 4) return 2;
  if (policy != 3) return 0;
  // The tall kernel retires k blocks faster (0.70 us per 256 x 256 x 64 against 0.47 us per 128 x 256 x 64, i.e.
  // 1.3x per flop) but exposes its epilogue (~5 us per tile, ~14 with the SwiGLU epilogue) and halves the number
  // of tiles, which changes how full the last wave is.  Where the row count is known (dense and depth-grouped
  // products, and row-grouped ones whose caller gave the expected rows of a capacity-sized buffer) the two are
  // compared by waves x time per tile; the typical win at one micro-batch's ~1300 expert rows is a product with
  // 4096 output columns whose 160 tiles would need a second, almost empty wave.  Without a row count only
  // products of >= 2048 rows and >= 3 waves of 128-row tiles take the tall kernel.
  long long r = rows_hint;
  const bool hinted = d->mode == 1 && thread_rows_hint > 0;
  if (hinted && thread_rows_hint < r) r = thread_rows_hint;
  long long grouped_depth = d->capacity_rows;          // mode 2 over row groups: the depth is the group's rows
  if (thread_rows_hint > 0 && thread_rows_hint < grouped_depth) grouped_depth = thread_rows_hint;
  const double blocks = (double)r / BM + (d->mode == 1 ? 0.5 * G : 0.0);
  const double nb = (double)((d->N + bn_out - 1) / bn_out) * (d->mode == 2 ? G : 1);
  const double depth = (d->mode == 2 && d->offsets != nullptr) ? (double)grouped_depth / G : (double)d->K;
  const double kb = ceil(depth / BK) + ceil((double)d->K_l / BK);
  bool tall;
  if (d->mode != 1 || hinted) {
    const double sms = num_sms;
    const double slow_epilogue = (!d->c_fp32 && !d->accumulate) ? 0.0 : 6.0;   // the uncoalesced epilogue costs more
    // rounds of 128-row tiles: whole rounds, except that a last round that fills less than 7/8 of the SMs is shared
    // by all of them along the depth (get_work), which costs about its share plus the partial-sum traffic
    double rounds = ceil(ceil(blocks) * nb / sms);
    if (split_enabled() && d->mode != 2 && !d->dual) {
      const double exact = ceil(blocks) * nb / sms, frac = exact - floor(exact);
      if (exact > 1.0 && frac > 0.0 && frac < 0.875 && kb >= 8.0) rounds = exact + 0.08;
    }
    const double t1 = rounds * (fmax(kb * 0.47, 2.0) + 1.0);
    const double t2 = ceil(ceil(blocks / 2 + (d->mode == 1 ? 0.25 * G : 0.0)) * nb / sms) * (kb * 0.70 + 5.0 + (d->dual ? 9.0 : 0.0) + slow_epilogue);
    tall = r >= 2 * BM && kb >= 32.0 && t2 < 0.9 * t1;
  } else {
    tall = r >= 16 * BM && ceil(blocks) * nb >= 3.0 * num_sms && kb >= 32.0;
  }
  return tall ? 2 : 0;
}

}  // namespace mdt

extern "C" long long mdt_gemm_launch_count() { return mdt::g_launches; }
extern "C" void mdt_gemm_rows_hint(long long rows) { mdt::t_rows_hint = rows; }
extern "C" int mdt_gemm_max_pairs() { return mdt::g_max_pairs; }
extern "C" int mdt_gemm_choose_tiling(const MdtGemmDesc* d, int policy, long long rows_hint, int num_sms) {
  return mdt::choose_tiling(d, policy, rows_hint, num_sms);
}
extern "C" void mdt_gemm_set_pair_cap(int pairs) { mdt::g_pair_cap = pairs; }
extern "C" int mdt_gemm_set_split(int on) {
  const int old = mdt::split_enabled() ? 1 : 0;
  if (on == 0 || on == 1) mdt::g_split_enabled = on;
  return old;
}
extern "C" int mdt_gemm_set_pair_policy(int policy) {
  const int old = mdt::pair_policy();
  if (policy >= 0 && policy <= 4) mdt::g_pair_policy = policy;
  return old;
}

extern "C" int mdt_gemm(const MdtGemmDesc* d, cudaStream_t stream) {
  using namespace mdt;
  // Tensor-map encoding is a driver call: make sure this host thread has the device's primary context
  // bound (a thread that has issued no runtime work yet, e.g. a fresh autograd worker, has none).
  static thread_local bool context_bound = false;
  if (!context_bound) { cudaFree(nullptr); context_bound = true; }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = d->M; p.N = d->N; p.K = d->K; p.K_l = d->K_l; p.G = d->G < 1 ? 1 : d->G; p.mode = d->mode;
  p.a_mn = d->a_mn; p.b_mn = d->b_mn; p.a_mn_l = d->a_mn_l; p.b_mn_l = d->b_mn_l; p.dual = d->dual;
  p.offsets = d->offsets; p.C = d->C; p.C2 = d->C2; p.C3 = d->C3; p.ldc = d->ldc; p.c_group_stride = d->c_group_stride;
  p.c_fp32 = d->c_fp32; p.accumulate = d->accumulate; p.alpha = d->alpha; p.store_gate_up = d->C2 != nullptr;
  p.status = d->status;
  p.tile_ready = d->tile_ready; p.tile_expected = d->tile_expected;
  p.row_dest_rank = d->row_dest_rank; p.row_dest_row = d->row_dest_row; p.peer_out = d->peer_out; p.peer_arrive = d->peer_arrive;
  p.num_peers = d->num_peers;
  p.peer_wait_ns = mdt_peer_wait_limit_ns();
  p.rdy_b = d->b_ready; p.rdy_b2 = d->b2_ready; p.rdy_bl = d->bl_ready;
  if (p.mode == 2) { p.rdy_b.ready = nullptr; p.rdy_b2.ready = nullptr; p.rdy_bl.ready = nullptr; }
  p.b_rows = d->b_rows; p.ldb = d->ldb; p.b_group_stride = d->b_group_stride;
  p.bl_rows = d->bl_rows; p.ldb_l = d->ldb_l; p.bl_group_stride = d->bl_group_stride;
  p.R = d->R;
  if (p.R != nullptr && (p.dual || p.mode == 2 || p.row_dest_rank != nullptr || (reinterpret_cast<uintptr_t>(p.R) & 15))) return -13;
  if (p.row_dest_rank != nullptr && (p.dual || p.c_fp32 || p.accumulate || p.mode == 2)) return -12;
  if (p.N % 8 != 0 || p.ldc % 8 != 0) return -10;
  if (p.dual && (p.b_mn != 0 || p.c_fp32 || p.accumulate)) return -11;
  const int BN = (p.dual || p.N > 128) ? 256 : 128;
  const int bn_out = p.dual ? BN / 2 : BN;
  const int tiling = choose_tiling(d, pair_policy(), t_rows_hint, g_num_sms);
  const bool pair = tiling == 1, tall = tiling == 2;
  const bool half_box = pair || tall;   // these kernels load B in 128-row boxes
  int rc = 0;
  // A: [a_rows, a_cols] row-major, a_cols contiguous.  K-major: rows = M, cols = K.  MN-major: rows = depth, cols = M.
  rc |= make_map(&p.tmA, d->A, d->a_cols, d->a_rows, 1, d->lda, 0, 64, d->a_mn ? 64 : BM, 2);
  // B: [G, b_rows, b_cols].  K-major: rows = N, cols = K.  MN-major: rows = depth, cols = N.
  const uint32_t b_box_rows = d->b_mn ? 64 : (half_box ? 128 : bn_out);
  rc |= make_map(&p.tmB, d->B, d->b_cols, d->b_rows, p.mode == 2 ? 1 : p.G, d->ldb, d->b_group_stride, 64, b_box_rows, 3);
  if (p.dual) rc |= make_map(&p.tmB2, d->B2, d->b_cols, d->b_rows, p.G, d->ldb, d->b_group_stride, 64, b_box_rows, 3);
  if (p.K_l > 0) {
    rc |= make_map(&p.tmA_l, d->A_l, d->al_cols, d->al_rows, 1, d->lda_l, 0, 64, d->a_mn_l ? 64 : BM, 2);
    const uint32_t bl_box_rows = d->b_mn_l ? 64 : (half_box ? 128 : bn_out);
    rc |= make_map(&p.tmB_l, d->B_l, d->bl_cols, d->bl_rows, p.G, d->ldb_l, d->bl_group_stride, 64, bl_box_rows, 3);
    if (p.dual) rc |= make_map(&p.tmB2_l, d->B2_l, d->bl_cols, d->bl_rows, p.G, d->ldb_l, d->bl_group_stride, 64, bl_box_rows, 3);
  }
  if (rc != 0) return rc;
  // upper bound on the number of tiles (the exact count may depend on device-side offsets)
  long long rows = (p.mode == 1) ? d->capacity_rows : p.M;
  long long tiles = ((rows + BM - 1) / BM) * ((p.N + bn_out - 1) / bn_out) * (p.mode == 2 ? p.G : 1);
  int grid = (int)(tiles < g_num_sms ? (tiles < 1 ? 1 : tiles) : g_num_sms);
  if (tall) {
    long long t256 = ((rows + 2 * BM - 1) / (2 * BM) + (p.mode == 1 ? p.G : 0)) * ((p.N + bn_out - 1) / bn_out) * (p.mode == 2 ? p.G : 1);
    const int g = (int)(t256 < 1 ? 1 : (t256 > g_num_sms ? g_num_sms : t256));
    cudaError_t e3 = launch_tall(p, g, stream);
    return e3 == cudaSuccess ? 0 : -100 - (int)e3;
  }
  if (pair) {
    long long pairs = ((rows + 2 * BM - 1) / (2 * BM) + (p.mode == 1 ? p.G : 0)) * ((p.N + bn_out - 1) / bn_out) * (p.mode == 2 ? p.G : 1);
    const int np = (int)(pairs < 1 ? 1 : (pairs > g_num_sms ? g_num_sms : pairs));
    cudaError_t e2 = launch_pair(p, np, stream);
    return e2 == cudaSuccess ? 0 : -100 - (int)e2;
  }
  if (split_enabled() && p.mode != 2 && !p.dual) {
    // the last, partly filled round of tiles may be cut along the depth and shared by all SMs (get_work)
    const long long kbt = (p.K + BK - 1) / BK + (p.K_l + BK - 1) / BK;
    SplitWorkspace w;
    if (kbt >= 8 && tiles > g_num_sms && split_workspace(stream, &w)) {
      p.sk_ws = w.ws; p.sk_ctr = w.ctr;
      grid = g_num_sms;
    }
  }
  cudaError_t e = (BN == 256) ? launch<256, 4>(p, grid, stream) : launch<128, 6>(p, grid, stream);
  return e == cudaSuccess ? 0 : -100 - (int)e;
}
