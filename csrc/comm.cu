// Expert-parallel token exchange and flat-buffer collectives over peer memory (NVLink / NVSwitch).
//
// Every rank of a group owns one symmetric workspace (same layout on every GPU, mapped into all peers'
// address spaces).  Kernels write straight into the peers' workspaces with plain vector stores, publish
// progress with system-scope release operations, and wait with system-scope acquire loads under a
// wall-clock limit; a wait that gives up sets a status word and the kernel returns.
//
// Dropless expert parallelism without host involvement:
//   ep_counts_send       my per-expert slot counts -> row `rank` of every peer's count matrix, then a flag
//   ep_counts_wait_meta  wait for all rows, derive every offset needed below (on the device)
//   ep_dispatch          copy each (token, choice) row into the buffer of the rank that owns its expert,
//                        at its final, expert-grouped, 128-row-padded position; count arrivals
//   ep_recv_prepare      zero the padding rows, wait until all expected rows have arrived
//   ep_combine_send      copy each expert-output row back to its source rank, in the source's sorted
//                        slot order; count arrivals
//   ep_wait_rows         wait at the source until all rows are back
// Sending and waiting are separate launches, so that a single GPU can run the kernels of several
// emulated ranks one after another (tests) and no kernel ever waits for a launch that follows it on
// the same stream.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.h"
#include "common/ptx.cuh"

namespace mdt {

static long long g_comm_launches = 0;
typedef __nv_bfloat16 bf16;

#ifndef MDT_PEER_WAIT_LIMIT_NS
#define MDT_PEER_WAIT_LIMIT_NS 10000000000ull   // 10 s: covers start-up skew between ranks
#endif

// ---------------------------------------------------------------------------------------- counts
__global__ void ep_counts_send_kernel(const int* __restrict__ counts, const long long* __restrict__ peer_base, MdtEpLayout L,
                                      int rank, int parity, unsigned epoch) {
  const int ws = L.ws, E = L.num_experts;
  for (int i = threadIdx.x; i < ws * E; i += blockDim.x) {
    const int peer = i / E, e = i - peer * E;
    int* dst = reinterpret_cast<int*>(peer_base[peer] + L.off_counts) + ((long long)parity * ws + rank) * E;
    dst[e] = counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < ws) {
    unsigned* flag = reinterpret_cast<unsigned*>(peer_base[threadIdx.x] + L.off_count_flags) + parity * ws + rank;
    st_release_sys(flag, epoch);
  }
}

// meta layout (ints): see MdtEpMeta offsets in comm.h
__global__ void ep_counts_wait_meta_kernel(long long my_base, MdtEpLayout L, int rank, int parity, unsigned epoch, int* __restrict__ meta,
                                           int* __restrict__ status) {
  const int ws = L.ws, E = L.num_experts, El = E / ws;
  __shared__ int ok_all;
  if (threadIdx.x == 0) ok_all = 1;
  __syncthreads();
  if (threadIdx.x < ws) {
    const unsigned* flag = reinterpret_cast<const unsigned*>(my_base + L.off_count_flags) + parity * ws + threadIdx.x;
    if (!wait_ge(flag, epoch, MDT_PEER_WAIT_LIMIT_NS)) { ok_all = 0; if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER); }
  }
  __syncthreads();
  if (!ok_all) return;
  const int* call = reinterpret_cast<const int*>(my_base + L.off_counts) + (long long)parity * ws * E;
  int* m_counts = meta + mdt_ep_meta_counts(ws, E);
  for (int i = threadIdx.x; i < ws * E; i += blockDim.x) m_counts[i] = call[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    int* recv_tot = meta + mdt_ep_meta_recv_tot(ws, E);
    int* recv_off = meta + mdt_ep_meta_recv_off(ws, E);
    int* dst_row = meta + mdt_ep_meta_dst_row(ws, E);
    int* send_start = meta + mdt_ep_meta_send_start(ws, E);
    int* seg_row = meta + mdt_ep_meta_seg_row(ws, E);
    int* seg_pos = meta + mdt_ep_meta_seg_pos(ws, E);
    int* scalars = meta + mdt_ep_meta_scalars(ws, E);
    // where my rows for expert e start inside the owner's buffer
    for (int d = 0; d < ws; ++d) {
      int base = 0;
      for (int le = 0; le < El; ++le) {
        const int e = d * El + le;
        int tot = 0, before_me = 0;
        for (int s = 0; s < ws; ++s) { const int c = m_counts[s * E + e]; if (s < rank) before_me += c; tot += c; }
        dst_row[e] = base + before_me;
        if (d == rank) { recv_tot[le] = tot; recv_off[le] = base; }
        base += (tot + 127) / 128 * 128;
      }
      if (d == rank) recv_off[El] = base;
    }
    int run = 0;
    for (int e = 0; e < E; ++e) { send_start[e] = run; run += m_counts[rank * E + e]; }
    send_start[E] = run;
    // segments of my receive buffer: (local expert, source) -> first row here, first position at the source
    int expected = 0;
    for (int le = 0; le < El; ++le) {
      const int e = rank * El + le;
      int row = recv_off[le];
      for (int s = 0; s < ws; ++s) {
        int pos = 0;
        for (int e2 = 0; e2 < e; ++e2) pos += m_counts[s * E + e2];
        seg_row[le * ws + s] = row;
        seg_pos[le * ws + s] = pos;
        row += m_counts[s * E + e];
        expected += m_counts[s * E + e];
      }
    }
    scalars[0] = expected;          // rows this rank receives
    scalars[1] = run;               // slots this rank sends (= rows it gets back)
    scalars[2] = recv_off[El];      // padded rows in use
    if (recv_off[El] > L.capacity_rows && status) atomicCAS(status, 0, ST_CAPACITY);
  }
}

// ---------------------------------------------------------------------------------------- dispatch
constexpr int EP_ROWS_PER_CTA = 16;   // two rows per warp
constexpr int EP_THREADS = 256;

// One warp copies a row; eight 16-byte loads per lane are in flight before the first store.
__device__ __forceinline__ void copy_row(const uint4* __restrict__ src, uint4* __restrict__ dst, int vecs, int lane, float scale, bool scaled) {
  for (int i = lane; i < vecs; i += 256) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) { const int idx = i + 32 * u; v[u] = idx < vecs ? src[idx] : make_uint4(0, 0, 0, 0); }
    if (scaled) {
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v[u]);
#pragma unroll
        for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(h[j]); h[j] = __floats2bfloat162_rn(f.x * scale, f.y * scale); }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) { const int idx = i + 32 * u; if (idx < vecs) dst[idx] = v[u]; }
  }
}

// x [T, cols]; sorted position p -> slot src_slot[p]; expert_of_slot [T*k]
__global__ void ep_dispatch_kernel(const bf16* __restrict__ x, const int* __restrict__ src_slot, const int* __restrict__ expert_of_slot,
                                   const bf16* __restrict__ slot_scale, const int* __restrict__ meta, const long long* __restrict__ peer_base,
                                   MdtEpLayout L, int top_k, int cols, int parity) {
  const int ws = L.ws, E = L.num_experts, El = E / ws;
  __shared__ unsigned sent[MDT_EP_MAX_RANKS];
  if (threadIdx.x < MDT_EP_MAX_RANKS) sent[threadIdx.x] = 0;
  __syncthreads();
  const int* dst_row = meta + mdt_ep_meta_dst_row(ws, E);
  const int* send_start = meta + mdt_ep_meta_send_start(ws, E);
  const int total = send_start[E];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int p0 = blockIdx.x * EP_ROWS_PER_CTA;
  // A warp copies all of its rows first and then makes them visible with one system-scope fence, instead of
  // waiting for the peers' acknowledgements once per row; lane j remembers where the j-th row went.
  int my_d = -1;
  long long my_row = 0;
  int n = 0;
  for (int p = p0 + warp; p < min(p0 + EP_ROWS_PER_CTA, total); p += nwarps) {
    const int slot = src_slot[p];
    const int e = expert_of_slot[slot];
    const int d = e / El;
    const long long row = dst_row[e] + (p - send_start[e]);
    if (row >= L.capacity_rows) continue;   // reported through the status word by the meta kernel
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)(slot / top_k) * cols);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(peer_base[d] + L.off_recv_x) + row * cols);
    const bool scaled = slot_scale != nullptr;
    copy_row(src, dst, cols / 8, lane, scaled ? __bfloat162float(slot_scale[slot]) : 1.f, scaled);
    if (lane == n) { my_d = d; my_row = row; }
    ++n;
  }
  // rows-arrived counters of the destinations' 128-row tiles (read by a GEMM that waits tile by tile)
  __threadfence_system();
  __syncwarp();
  if (lane < n) {
    unsigned* tctr = reinterpret_cast<unsigned*>(peer_base[my_d] + L.off_tile_ctr) + (long long)parity * (L.capacity_rows / 128) + my_row / 128;
    red_add_release_sys(tctr, 1u);
    atomicAdd(&sent[my_d], 1u);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < ws && sent[threadIdx.x] > 0) {
    unsigned* ctr = reinterpret_cast<unsigned*>(peer_base[threadIdx.x] + L.off_arrive_x) + parity;
    red_add_release_sys(ctr, sent[threadIdx.x]);
  }
}

// zero the padding rows of my receive buffer; block 0 additionally waits for all expected rows
__global__ void ep_recv_prepare_kernel(long long my_base, MdtEpLayout L, const int* __restrict__ meta, int cols, int parity,
                                       int wait_all, int* __restrict__ status) {
  const int ws = L.ws, E = L.num_experts, El = E / ws;
  const int* recv_tot = meta + mdt_ep_meta_recv_tot(ws, E);
  const int* recv_off = meta + mdt_ep_meta_recv_off(ws, E);
  bf16* buf = reinterpret_cast<bf16*>(my_base + L.off_recv_x);
  const int vecs = cols / 8;
  for (int le = 0; le < El; ++le) {
    const int first = recv_off[le] + recv_tot[le], last = min(recv_off[le + 1], L.capacity_rows);
    for (int r = first + blockIdx.x; r < last; r += gridDim.x) {
      uint4* dst = reinterpret_cast<uint4*>(buf + (long long)r * cols);
      for (int i = threadIdx.x; i < vecs; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    }
  }
  // the other parity's tile counters were consumed by the previous exchange and are written next by the
  // following one (which no peer starts before this rank has sent its results of the current one)
  {
    unsigned* other = reinterpret_cast<unsigned*>(my_base + L.off_tile_ctr) + (long long)(parity ^ 1) * (L.capacity_rows / 128);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < L.capacity_rows / 128; i += gridDim.x * blockDim.x) other[i] = 0;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned* ctr = reinterpret_cast<unsigned*>(my_base + L.off_arrive_x) + parity;
    const unsigned expected = (unsigned)meta[mdt_ep_meta_scalars(ws, E)];
    if (wait_all) {
      if (!wait_ge(ctr, expected, MDT_PEER_WAIT_LIMIT_NS)) { if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER); }
      *ctr = 0;   // this parity is next written two exchanges from now
    } else {
      // a consumer waits on the per-tile counters instead; the total counter of the other parity is
      // idle by the same argument as above
      reinterpret_cast<unsigned*>(my_base + L.off_arrive_x)[parity ^ 1] = 0;
    }
  }
}

// ---------------------------------------------------------------------------------------- combine
// y rows are in my receive layout; row of segment (le, s) number i returns to rank s at position seg_pos + i
__global__ void ep_combine_send_kernel(const bf16* __restrict__ y, const int* __restrict__ meta, const long long* __restrict__ peer_base,
                                       MdtEpLayout L, int rank, int cols, int parity) {
  const int ws = L.ws, E = L.num_experts, El = E / ws;
  __shared__ unsigned sent[MDT_EP_MAX_RANKS];
  __shared__ int seg_first[MDT_EP_MAX_SEGMENTS + 1];   // flat index of the first row of every segment
  if (threadIdx.x < MDT_EP_MAX_RANKS) sent[threadIdx.x] = 0;
  const int* m_counts = meta + mdt_ep_meta_counts(ws, E);
  const int* seg_row = meta + mdt_ep_meta_seg_row(ws, E);
  const int* seg_pos = meta + mdt_ep_meta_seg_pos(ws, E);
  const int nseg = El * ws;
  if (threadIdx.x == 0) {
    int run = 0;
    for (int g = 0; g < nseg; ++g) { seg_first[g] = run; run += m_counts[(g % ws) * E + rank * El + g / ws]; }
    seg_first[nseg] = run;
  }
  __syncthreads();
  const int total = seg_first[nseg];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int f0 = blockIdx.x * EP_ROWS_PER_CTA;
  for (int f = f0 + warp; f < min(f0 + EP_ROWS_PER_CTA, total); f += nwarps) {
    int g = 0;
    while (g + 1 < nseg && seg_first[g + 1] <= f) ++g;
    const int s = g % ws;
    const int i = f - seg_first[g];
    const uint4* src = reinterpret_cast<const uint4*>(y + (long long)(seg_row[g] + i) * cols);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(peer_base[s] + L.off_recv_y) + (long long)(seg_pos[g] + i) * cols);
    copy_row(src, dst, cols / 8, lane, 1.f, false);
    if (lane == 0) atomicAdd(&sent[s], 1u);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < ws && sent[threadIdx.x] > 0) {
    unsigned* ctr = reinterpret_cast<unsigned*>(peer_base[threadIdx.x] + L.off_arrive_y) + parity;
    red_add_release_sys(ctr, sent[threadIdx.x]);
  }
}

// For every row of my receive layout: the rank it returns to and its position there (-1 for padding), and for
// every 128-row tile the number of rows that must arrive before it may be read.
__global__ void ep_fused_meta_kernel(const int* __restrict__ meta, MdtEpLayout L, int rank, int* __restrict__ row_rank,
                                     int* __restrict__ row_pos, int* __restrict__ tile_expected) {
  const int ws = L.ws, E = L.num_experts, El = E / ws;
  const int* recv_tot = meta + mdt_ep_meta_recv_tot(ws, E);
  const int* recv_off = meta + mdt_ep_meta_recv_off(ws, E);
  const int* seg_row = meta + mdt_ep_meta_seg_row(ws, E);
  const int* seg_pos = meta + mdt_ep_meta_seg_pos(ws, E);
  const int used = min(recv_off[El], L.capacity_rows);
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < used; r += gridDim.x * blockDim.x) {
    int le = 0;
    while (le + 1 < El && recv_off[le + 1] <= r) ++le;
    int rk = -1, ps = -1;
    if (r - recv_off[le] < recv_tot[le]) {
      int s = 0;
      while (s + 1 < ws && seg_row[le * ws + s + 1] <= r) ++s;
      // (the last segment starting at or before r is never empty: empty ones share their start with the next)
      rk = s; ps = seg_pos[le * ws + s] + (r - seg_row[le * ws + s]);
    }
    row_rank[r] = rk; row_pos[r] = ps;
    if ((r & 127) == 0) {
      const int left = recv_tot[le] - (r - recv_off[le]);
      tile_expected[r >> 7] = left < 0 ? 0 : (left > 128 ? 128 : left);
    }
  }
}

__global__ void ep_wait_rows_kernel(long long my_base, MdtEpLayout L, const int* __restrict__ meta, int parity, int mult, int* __restrict__ status) {
  unsigned* ctr = reinterpret_cast<unsigned*>(my_base + L.off_arrive_y) + parity;
  const unsigned expected = (unsigned)meta[mdt_ep_meta_scalars(L.ws, L.num_experts) + 1] * (unsigned)mult;
  if (!wait_ge(ctr, expected, MDT_PEER_WAIT_LIMIT_NS)) { if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER); }
  *ctr = 0;
}

// ---------------------------------------------------------------------------------------- flat collectives
// all-gather by peer reads: out[r*n .. (r+1)*n) = shard of rank r.  16-byte vectors.
__global__ void ag_pull_kernel(uint4* __restrict__ out, const long long* __restrict__ peer_shard, int ws, long long vecs_per_rank) {
  const long long total = vecs_per_rank * ws;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vecs_per_rank);
    out[i] = reinterpret_cast<const uint4*>(peer_shard[r])[i - (long long)r * vecs_per_rank];
  }
}
// reduce-scatter by peer reads with fused scale / cast / accumulate:
//   out[i] (+)= scale * sum_r full_r[rank*n + i];  inputs fp32 or bf16, output bf16 or fp32
__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f(float* p, float v) { *p = v; }
__device__ __forceinline__ void from_f(bf16* p, float v) { *p = __float2bfloat16(v); }
template <typename TIn, typename TOut>
__global__ void rs_pull_kernel(TOut* __restrict__ out, const long long* __restrict__ peer_full, int ws, int rank, long long n,
                               float scale, int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int r = 0; r < ws; ++r) {
      const int rr = (r + rank) % ws;   // start with a different peer on every rank
      s += to_f(reinterpret_cast<const TIn*>(peer_full[rr])[(long long)rank * n + i]);
    }
    s *= scale;
    if (accumulate) s += to_f(out[i]);
    from_f(out + i, s);
  }
}
// cross-rank barrier on symmetric flags: arrive = write epoch into everyone's slot, then wait for all
__global__ void barrier_arrive_kernel(const long long* __restrict__ peer_flags, int ws, int rank, unsigned epoch) {
  __threadfence_system();
  if (threadIdx.x < ws) st_release_sys(reinterpret_cast<unsigned*>(peer_flags[threadIdx.x]) + rank, epoch);
}
__global__ void barrier_wait_kernel(const unsigned* __restrict__ my_flags, int ws, unsigned epoch, int* __restrict__ status,
                                    unsigned long long limit_ns) {
  if (threadIdx.x < ws && !wait_ge(my_flags + threadIdx.x, epoch, limit_ns)) { if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER); }
}

#define MDT_CM_CHECK() do { ++g_comm_launches; cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return -100 - (int)e_; } while (0)

}  // namespace mdt

using namespace mdt;

extern "C" long long mdt_comm_launch_count() { return g_comm_launches; }

extern "C" int mdt_ep_counts_send(const int* counts, const long long* peer_base, MdtEpLayout L, int rank, int parity, unsigned epoch, cudaStream_t s) {
  if (L.ws > MDT_EP_MAX_RANKS || L.num_experts % L.ws != 0 || L.num_experts / L.ws * L.ws > MDT_EP_MAX_SEGMENTS) return -1;
  ep_counts_send_kernel<<<1, 256, 0, s>>>(counts, peer_base, L, rank, parity, epoch);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_counts_wait_meta(long long my_base, MdtEpLayout L, int rank, int parity, unsigned epoch, int* meta, int* status, cudaStream_t s) {
  ep_counts_wait_meta_kernel<<<1, 256, 0, s>>>(my_base, L, rank, parity, epoch, meta, status);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_dispatch(const void* x, const int* src_slot, const int* expert_of_slot, const void* slot_scale, const int* meta,
                               const long long* peer_base, MdtEpLayout L, int num_slots, int top_k, int cols, int parity, cudaStream_t s) {
  if (cols % 8 != 0) return -1;
  if (num_slots == 0) return 0;
  const int grid = (num_slots + EP_ROWS_PER_CTA - 1) / EP_ROWS_PER_CTA;
  ep_dispatch_kernel<<<grid, EP_THREADS, 0, s>>>((const bf16*)x, src_slot, expert_of_slot, (const bf16*)slot_scale, meta, peer_base, L, top_k, cols, parity);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_recv_prepare(long long my_base, MdtEpLayout L, const int* meta, int cols, int parity, int wait_all, int* status, cudaStream_t s) {
  ep_recv_prepare_kernel<<<64, 256, 0, s>>>(my_base, L, meta, cols, parity, wait_all, status);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_combine_send(const void* y, const int* meta, const long long* peer_base, MdtEpLayout L, int rank, int max_rows, int cols,
                                   int parity, cudaStream_t s) {
  if (cols % 8 != 0) return -1;
  if (max_rows == 0) return 0;
  const int grid = (max_rows + EP_ROWS_PER_CTA - 1) / EP_ROWS_PER_CTA;
  ep_combine_send_kernel<<<grid, EP_THREADS, 0, s>>>((const bf16*)y, meta, peer_base, L, rank, cols, parity);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_fused_meta(const int* meta, MdtEpLayout L, int rank, int* row_rank, int* row_pos, int* tile_expected, cudaStream_t s) {
  ep_fused_meta_kernel<<<64, 256, 0, s>>>(meta, L, rank, row_rank, row_pos, tile_expected);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_wait_rows(long long my_base, MdtEpLayout L, const int* meta, int parity, int mult, int* status, cudaStream_t s) {
  ep_wait_rows_kernel<<<1, 1, 0, s>>>(my_base, L, meta, parity, mult < 1 ? 1 : mult, status);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ag_pull(void* out, const long long* peer_shard, int ws, long long bytes_per_rank, cudaStream_t s) {
  if (bytes_per_rank % 16 != 0) return -1;
  const long long vecs = bytes_per_rank / 16;
  long long blocks = (vecs * ws + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  ag_pull_kernel<<<(unsigned)blocks, 256, 0, s>>>((uint4*)out, peer_shard, ws, vecs);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_rs_pull(void* out, const long long* peer_full, int ws, int rank, long long n, int in_fp32, int out_fp32, float scale,
                           int accumulate, cudaStream_t s) {
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  if (in_fp32 && !out_fp32) rs_pull_kernel<float, bf16><<<(unsigned)blocks, 256, 0, s>>>((bf16*)out, peer_full, ws, rank, n, scale, accumulate);
  else if (in_fp32 && out_fp32) rs_pull_kernel<float, float><<<(unsigned)blocks, 256, 0, s>>>((float*)out, peer_full, ws, rank, n, scale, accumulate);
  else if (!in_fp32 && !out_fp32) rs_pull_kernel<bf16, bf16><<<(unsigned)blocks, 256, 0, s>>>((bf16*)out, peer_full, ws, rank, n, scale, accumulate);
  else rs_pull_kernel<bf16, float><<<(unsigned)blocks, 256, 0, s>>>((float*)out, peer_full, ws, rank, n, scale, accumulate);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_barrier_arrive(const long long* peer_flags, int ws, int rank, unsigned epoch, cudaStream_t s) {
  barrier_arrive_kernel<<<1, 32, 0, s>>>(peer_flags, ws, rank, epoch);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_barrier_wait(const void* my_flags, int ws, unsigned epoch, int* status, long long limit_ms, cudaStream_t s) {
  const unsigned long long limit_ns = limit_ms > 0 ? (unsigned long long)limit_ms * 1000000ull : MDT_PEER_WAIT_LIMIT_NS;
  barrier_wait_kernel<<<1, 32, 0, s>>>((const unsigned*)my_flags, ws, epoch, status, limit_ns);
  MDT_CM_CHECK();
  return 0;
}
