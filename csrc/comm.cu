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
#include "common/host.h"
#include "common/ptx.cuh"

namespace mdt {

static long long g_comm_launches = 0;
typedef __nv_bfloat16 bf16;

#ifndef MDT_PEER_WAIT_LIMIT_NS
#define MDT_PEER_WAIT_LIMIT_NS 10000000000ull   // 10 s: covers start-up skew between ranks
#endif
// Limit of every wait for a peer, in nanoseconds; mdt_set_peer_wait_limit_ms() changes it (tests use a fraction
// of a second to let a wait run out on purpose; a deployment may want less than the default too).
static unsigned long long g_peer_wait_ns = MDT_PEER_WAIT_LIMIT_NS;
static int sm_count() { return sm_count_of_current_device(); }
// A kernel of an exchange does nothing once the status word is set: after a wait that ran out the metadata of
// the exchange describe no rows, and nothing may be stored into a peer on the strength of them.
__device__ __forceinline__ bool status_set(const int* status) {
  return status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0;
}

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
// Everything below is derived by the threads of one CTA in four short parallel steps (per expert, per
// destination rank, per (local expert, source) segment, scalars).  If a peer's counts do not arrive within the
// limit, the status word is set and the metadata are written as all zeros: no rows to send, none expected, no
// tiles, so every later kernel of the exchange has nothing to do.
__global__ void ep_counts_wait_meta_kernel(long long my_base, MdtEpLayout L, int rank, int parity, unsigned epoch, int* __restrict__ meta,
                                           int* __restrict__ status, unsigned long long limit_ns) {
  const int ws = L.ws, E = L.num_experts, El = E / ws;
  __shared__ int ok_all;
  __shared__ int s_tot[MDT_EP_MAX_SEGMENTS], s_before[MDT_EP_MAX_SEGMENTS], s_recv_off[MDT_EP_MAX_SEGMENTS + 1];
  if (threadIdx.x == 0) ok_all = status_set(status) ? 0 : 1;
  __syncthreads();
  if (ok_all && threadIdx.x < ws) {
    const unsigned* flag = reinterpret_cast<const unsigned*>(my_base + L.off_count_flags) + parity * ws + threadIdx.x;
    if (!wait_ge(flag, epoch, limit_ns)) { ok_all = 0; if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER); }
  }
  __syncthreads();
  if (!ok_all) {
    for (int i = threadIdx.x; i < mdt_ep_meta_size(ws, E); i += blockDim.x) meta[i] = 0;
    return;
  }
  const int* call = reinterpret_cast<const int*>(my_base + L.off_counts) + (long long)parity * ws * E;
  int* m_counts = meta + mdt_ep_meta_counts(ws, E);
  for (int i = threadIdx.x; i < ws * E; i += blockDim.x) m_counts[i] = call[i];
  int* recv_tot = meta + mdt_ep_meta_recv_tot(ws, E);
  int* recv_off = meta + mdt_ep_meta_recv_off(ws, E);
  int* dst_row = meta + mdt_ep_meta_dst_row(ws, E);
  int* send_start = meta + mdt_ep_meta_send_start(ws, E);
  int* seg_row = meta + mdt_ep_meta_seg_row(ws, E);
  int* seg_pos = meta + mdt_ep_meta_seg_pos(ws, E);
  int* scalars = meta + mdt_ep_meta_scalars(ws, E);
  __syncthreads();
  // (1) per expert: rows it receives in total, and from ranks before me
  if (threadIdx.x < E) {
    const int e = threadIdx.x;
    int tot = 0, before = 0;
    for (int s = 0; s < ws; ++s) { const int c = m_counts[s * E + e]; if (s < rank) before += c; tot += c; }
    s_tot[e] = tot; s_before[e] = before;
  }
  __syncthreads();
  // (2) per destination rank: where my rows for each of its experts start inside its (128-row padded) buffer
  if (threadIdx.x < ws) {
    const int d = threadIdx.x;
    int base = 0;
    for (int le = 0; le < El; ++le) {
      const int e = d * El + le;
      dst_row[e] = base + s_before[e];
      if (d == rank) { recv_tot[le] = s_tot[e]; recv_off[le] = base; s_recv_off[le] = base; }
      base += (s_tot[e] + 127) / 128 * 128;
    }
    if (d == rank) { recv_off[El] = base; s_recv_off[El] = base; }
  }
  // first sorted position of every expert in my send order
  if (threadIdx.x == blockDim.x - 1) {
    int run = 0;
    for (int e = 0; e < E; ++e) { send_start[e] = run; run += m_counts[rank * E + e]; }
    send_start[E] = run;
    scalars[1] = run;               // slots this rank sends (= rows it gets back)
  }
  __syncthreads();
  // (3) segments of my receive buffer: (local expert, source) -> first row here, first position at the source
  if (threadIdx.x < El * ws) {
    const int le = threadIdx.x / ws, s = threadIdx.x - le * ws;
    const int e = rank * El + le;
    int row = s_recv_off[le];
    for (int s2 = 0; s2 < s; ++s2) row += m_counts[s2 * E + e];
    int pos = 0;
    for (int e2 = 0; e2 < e; ++e2) pos += m_counts[s * E + e2];
    seg_row[le * ws + s] = row;
    seg_pos[le * ws + s] = pos;
  }
  // (4) scalars
  if (threadIdx.x == 0) {
    int expected = 0;
    for (int le = 0; le < El; ++le) expected += s_tot[rank * El + le];
    scalars[0] = expected;          // rows this rank receives
    scalars[2] = s_recv_off[El];    // padded rows in use
    if (s_recv_off[El] > L.capacity_rows && status) atomicCAS(status, 0, ST_CAPACITY);
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
// Sorted positions are expert-major, i.e. destination-rank-major.  CTA b serves destination (rank + 1 + b % ws) % ws
// and walks that destination's rows in chunks of EP_ROWS_PER_CTA with stride gridDim.x / ws: at any moment a rank's
// stores are spread over all peers, and different ranks start with different peers.  (CTAs that walk the sorted
// order front to back make every rank store to rank 0 first, then rank 1, ...: one receiver's link carries all
// the traffic while the others idle.)
__global__ void ep_dispatch_kernel(const bf16* __restrict__ x, const int* __restrict__ src_slot, const int* __restrict__ expert_of_slot,
                                   const bf16* __restrict__ slot_scale, const int* __restrict__ meta, const long long* __restrict__ peer_base,
                                   MdtEpLayout L, int rank, int top_k, int cols, int parity, const int* __restrict__ status) {
  if (status_set(status)) return;
  const int ws = L.ws, E = L.num_experts, El = E / ws;
  const int* dst_row = meta + mdt_ep_meta_dst_row(ws, E);
  const int* send_start = meta + mdt_ep_meta_send_start(ws, E);
  const int d = (rank + 1 + (int)(blockIdx.x % ws)) % ws;
  const int chunk0 = blockIdx.x / ws, chunk_stride = gridDim.x / ws;
  const int first = send_start[d * El], last = send_start[(d + 1) * El];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const long long dbase = peer_base[d];
  unsigned* tile_ctr = reinterpret_cast<unsigned*>(dbase + L.off_tile_ctr) + (long long)parity * (L.capacity_rows / 128);
  __shared__ unsigned sent;
  if (threadIdx.x == 0) sent = 0;
  __syncthreads();
  unsigned mine = 0;
  for (int p0 = first + chunk0 * EP_ROWS_PER_CTA; p0 < last; p0 += chunk_stride * EP_ROWS_PER_CTA) {
    // A warp copies all of its rows of the chunk first and then makes them visible with one system-scope fence,
    // instead of waiting for the peer's acknowledgements once per row; lane j remembers where the j-th row went.
    long long my_row = -1;
    int n = 0;
    for (int p = p0 + warp; p < min(p0 + EP_ROWS_PER_CTA, last); p += nwarps) {
      const int slot = src_slot[p];
      const int e = expert_of_slot[slot];
      const long long row = (long long)dst_row[e] + (p - send_start[e]);
      // rows outside the receive buffer are dropped (the meta kernel has reported the overflow); an expert id
      // that does not belong to this destination means inconsistent inputs and is dropped as well
      if (row < 0 || row >= L.capacity_rows || e / El != d) continue;
      const uint4* src = reinterpret_cast<const uint4*>(x + (long long)(slot / top_k) * cols);
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dbase + L.off_recv_x) + row * cols);
      const bool scaled = slot_scale != nullptr;
      copy_row(src, dst, cols / 8, lane, scaled ? __bfloat162float(slot_scale[slot]) : 1.f, scaled);
      if (lane == n) my_row = row;
      ++n;
    }
    // rows-arrived counters of the destination's 128-row tiles (read by a GEMM that waits tile by tile)
    __threadfence_system();
    __syncwarp();
    if (lane < n && my_row >= 0) { red_add_release_sys(tile_ctr + my_row / 128, 1u); ++mine; }
  }
  if (mine) atomicAdd(&sent, mine);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0 && sent > 0) red_add_release_sys(reinterpret_cast<unsigned*>(dbase + L.off_arrive_x) + parity, sent);
}

// zero the padding rows of my receive buffer; block 0 additionally waits for all expected rows
__global__ void ep_recv_prepare_kernel(long long my_base, MdtEpLayout L, const int* __restrict__ meta, int cols, int parity,
                                       int wait_all, int* __restrict__ status, unsigned long long limit_ns) {
  if (status_set(status)) return;
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
      if (!wait_ge(ctr, expected, limit_ns)) { if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER); }
      *ctr = 0;   // this parity is next written two exchanges from now
    } else {
      // a consumer waits on the per-tile counters instead; the total counter of the other parity is
      // idle by the same argument as above
      reinterpret_cast<unsigned*>(my_base + L.off_arrive_x)[parity ^ 1] = 0;
    }
  }
}

// ---------------------------------------------------------------------------------------- combine
// y rows are in my receive layout; row of segment (le, s) number i returns to rank s at position seg_pos + i.
// CTA b serves source rank (rank + 1 + b % ws) % ws, as in the dispatch kernel.
__global__ void ep_combine_send_kernel(const bf16* __restrict__ y, const int* __restrict__ meta, const long long* __restrict__ peer_base,
                                       MdtEpLayout L, int rank, int cols, int parity, const int* __restrict__ status) {
  if (status_set(status)) return;
  const int ws = L.ws, E = L.num_experts, El = E / ws;
  const int* m_counts = meta + mdt_ep_meta_counts(ws, E);
  const int* seg_row = meta + mdt_ep_meta_seg_row(ws, E);
  const int* seg_pos = meta + mdt_ep_meta_seg_pos(ws, E);
  const int s = (rank + 1 + (int)(blockIdx.x % ws)) % ws;
  const int chunk0 = blockIdx.x / ws, chunk_stride = gridDim.x / ws;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const long long sbase = peer_base[s];
  __shared__ unsigned sent;
  if (threadIdx.x == 0) sent = 0;
  __syncthreads();
  unsigned mine = 0;
  for (int le = 0; le < El; ++le) {
    const int g = le * ws + s;
    const int cnt = m_counts[s * E + rank * El + le];
    const int row0 = seg_row[g], pos0 = seg_pos[g];
    for (int i0 = chunk0 * EP_ROWS_PER_CTA; i0 < cnt; i0 += chunk_stride * EP_ROWS_PER_CTA) {
      for (int i = i0 + warp; i < min(i0 + EP_ROWS_PER_CTA, cnt); i += nwarps) {
        const long long srow = (long long)row0 + i, drow = (long long)pos0 + i;
        if (srow < 0 || srow >= L.capacity_rows || drow < 0 || drow >= L.capacity_slots) continue;
        const uint4* src = reinterpret_cast<const uint4*>(y + srow * cols);
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(sbase + L.off_recv_y) + drow * cols);
        copy_row(src, dst, cols / 8, lane, 1.f, false);
        if (lane == 0) ++mine;
      }
    }
  }
  if (mine) atomicAdd(&sent, mine);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0 && sent > 0) red_add_release_sys(reinterpret_cast<unsigned*>(sbase + L.off_arrive_y) + parity, sent);
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

__global__ void ep_wait_rows_kernel(long long my_base, MdtEpLayout L, const int* __restrict__ meta, int parity, int mult, int* __restrict__ status,
                                    unsigned long long limit_ns) {
  if (status_set(status)) return;
  unsigned* ctr = reinterpret_cast<unsigned*>(my_base + L.off_arrive_y) + parity;
  const unsigned expected = (unsigned)meta[mdt_ep_meta_scalars(L.ws, L.num_experts) + 1] * (unsigned)mult;
  if (!wait_ge(ctr, expected, limit_ns)) { if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER); }
  *ctr = 0;
}

// ---------------------------------------------------------------------------------------- flat collectives
// all-gather by peer reads: out[r*n .. (r+1)*n) = shard of rank r.  16-byte vectors.
// The buffer is cut into chunks of `chunk_vecs` vectors (never across two shards); a CTA copies whole chunks, own
// shard first, then the peers' starting with rank + 1 (the first `prio_chunks` chunks of the buffer before all
// others: small parameters that the first kernels of a block read), and when `ready` is given publishes every
// finished chunk by storing `epoch` into ready[chunk] (release).  A consumer (the GEMM's TMA producer, or ag_wait_chunks) that
// knows which chunks hold its operand can start as soon as those have landed, while the rest is still in flight.
// Small CTAs (128 threads, no shared memory) so that they fit on an SM beside a CTA of the GEMM kernels, which a
// consumer of the progress flags relies on when it has filled the GPU before the gather has finished.
constexpr int AG_THREADS = 128;
__global__ void __launch_bounds__(AG_THREADS) ag_pull_kernel(uint4* __restrict__ out, const long long* __restrict__ peer_shard, int ws, int rank, long long vecs_per_rank,
                               long long chunk_vecs, int chunks_per_rank, unsigned* __restrict__ ready, unsigned epoch, int prio_chunks) {
  const int total_chunks = chunks_per_rank * ws;
  for (int c = blockIdx.x; c < prio_chunks + total_chunks; c += gridDim.x) {
    int idx = c;                                                // chunk index in buffer order
    if (c >= prio_chunks) {
      const int c2 = c - prio_chunks;
      idx = ((rank + c2 / chunks_per_rank) % ws) * chunks_per_rank + c2 % chunks_per_rank;   // shard order: mine, rank + 1, ...
      if (idx < prio_chunks) continue;                          // already fetched
    }
    const int r = idx / chunks_per_rank, cr = idx % chunks_per_rank;
    const long long v0 = (long long)cr * chunk_vecs;
    const long long v1 = v0 + chunk_vecs < vecs_per_rank ? v0 + chunk_vecs : vecs_per_rank;
    const uint4* src = reinterpret_cast<const uint4*>(peer_shard[r]);
    uint4* dst = out + (long long)r * vecs_per_rank;
    long long i = v0 + threadIdx.x;
    for (; i + 7ll * AG_THREADS < v1; i += 8ll * AG_THREADS) {   // eight 16-byte loads in flight per thread
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = src[i + (long long)u * AG_THREADS];
#pragma unroll
      for (int u = 0; u < 8; ++u) dst[i + (long long)u * AG_THREADS] = v[u];
    }
    for (; i < v1; i += AG_THREADS) dst[i] = src[i];
    if (ready != nullptr) {
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) st_release_sys(ready + (r * chunks_per_rank + cr), epoch);
      __syncthreads();
    }
  }
}
// one CTA: returns when ready[first .. last) have all reached `epoch` (for consumers that are not a GEMM)
__global__ void ag_wait_chunks_kernel(const unsigned* __restrict__ ready, int first, int last, unsigned epoch, int* __restrict__ status,
                                      unsigned long long limit_ns) {
  for (int c = first + threadIdx.x; c < last; c += blockDim.x)
    if (!wait_ge(ready + c, epoch, limit_ns)) { if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER); }
}

// reduce-scatter by peer reads with fused scale / cast / accumulate:
//   out[i] (+)= scale * sum_r full_r[rank*n + i];  inputs fp32 or bf16, output bf16 or fp32.  16-byte peer loads.
__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f(float* p, float v) { *p = v; }
__device__ __forceinline__ void from_f(bf16* p, float v) { *p = __float2bfloat16(v); }
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };
// `src_off`: first element of the range that is read from every peer's buffer (rank * n for a reduce-scatter, 0 for an
// all-reduce of n elements)
// V consecutive outputs as one 8-, 16- or 2 x 16-byte access (the caller has checked the alignment)
template <int V> __device__ __forceinline__ void load_out_vec(const bf16* p, float (&o)[V]) {
  if constexpr (V == 4) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    for (int j = 0; j < 2; ++j) { const float2 f = __bfloat1622float2(h[j]); o[2 * j] = f.x; o[2 * j + 1] = f.y; }
  } else {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); o[2 * j] = f.x; o[2 * j + 1] = f.y; }
  }
}
template <int V> __device__ __forceinline__ void load_out_vec(const float* p, float (&o)[V]) {
#pragma unroll
  for (int c = 0; c < V / 4; ++c) {
    const float4 v = reinterpret_cast<const float4*>(p)[c];
    o[4 * c] = v.x; o[4 * c + 1] = v.y; o[4 * c + 2] = v.z; o[4 * c + 3] = v.w;
  }
}
template <int V> __device__ __forceinline__ void store_out_vec(bf16* p, const float (&o)[V]) {
  if constexpr (V == 4) {
    uint2 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
    for (int j = 0; j < 2; ++j) h[j] = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]);
    *reinterpret_cast<uint2*>(p) = v;
  } else {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]);
    *reinterpret_cast<uint4*>(p) = v;
  }
}
template <int V> __device__ __forceinline__ void store_out_vec(float* p, const float (&o)[V]) {
#pragma unroll
  for (int c = 0; c < V / 4; ++c) reinterpret_cast<float4*>(p)[c] = make_float4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
}

template <typename TIn, typename TOut>
__device__ __forceinline__ void rs_pull_body(TOut* __restrict__ out, const long long* __restrict__ peer_full, int ws, int rank, long long n,
                                             float scale, int accumulate, long long tid, long long nthreads, long long src_off) {
  constexpr int V = Vec16<TIn>::N;
  constexpr int BATCH = 8;            // peers whose vectors are in flight together (the latency of a peer load is ~2 us)
  const long long nvec = n / V;
  const bool out_vec = (reinterpret_cast<unsigned long long>(out) % (V * sizeof(TOut))) == 0;
  for (long long i = tid; i < nvec; i += nthreads) {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    for (int r0 = 0; r0 < ws; r0 += BATCH) {
      uint4 v[BATCH];
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        if (r0 + u < ws) {
          const int rr = (r0 + u + rank) % ws;   // start with a different peer on every rank
          v[u] = reinterpret_cast<const uint4*>(reinterpret_cast<const TIn*>(peer_full[rr]) + src_off)[i];
        }
      }
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        if (r0 + u < ws) {
          const TIn* e = reinterpret_cast<const TIn*>(&v[u]);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += to_f(e[j]);
        }
      }
    }
    if (out_vec) {
      float o[V];
      if (accumulate) {
        load_out_vec<V>(out + i * V, o);
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] += acc[j] * scale;
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = acc[j] * scale;
      }
      store_out_vec<V>(out + i * V, o);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float sres = acc[j] * scale;
        if (accumulate) sres += to_f(out[i * V + j]);
        from_f(out + i * V + j, sres);
      }
    }
  }
  for (long long i = nvec * V + tid; i < n; i += nthreads) {   // tail (n not a multiple of the vector width)
    float sres = 0.f;
    for (int r = 0; r < ws; ++r) sres += to_f(reinterpret_cast<const TIn*>(peer_full[(r + rank) % ws])[src_off + i]);
    sres *= scale;
    if (accumulate) sres += to_f(out[i]);
    from_f(out + i, sres);
  }
}
template <typename TIn, typename TOut>
__global__ void rs_pull_kernel(TOut* __restrict__ out, const long long* __restrict__ peer_full, int ws, int rank, long long n,
                               float scale, int accumulate) {
  rs_pull_body<TIn, TOut>(out, peer_full, ws, rank, n, scale, accumulate, (long long)blockIdx.x * blockDim.x + threadIdx.x,
                          (long long)gridDim.x * blockDim.x, (long long)rank * n);
}
// Reduce-scatter of one parameter group in the middle of a backward pass, as one kernel on a side stream:
//   announce  my contribution (the group's full-size gradient buffer) is complete: store `epoch` into slot
//             [flag_index][rank] of every peer's flag table (release)
//   wait      until every peer has announced the same (bounded)
//   reduce    read my slice of every peer's buffer, scale, cast, write / accumulate the shard gradient
// The owners of the buffers must not overwrite them before all peers have read: see the caller's barrier.
// With `all_reduce` every rank reads the whole range [0, n) of every buffer instead of its own slice: the sum of the
// tensor-parallel ranks' partial expert outputs (the reference's dist.all_reduce, megablocks_utils/config_utils.py:168-184).
template <typename TIn, typename TOut>
__global__ void rs_block_kernel(TOut* __restrict__ out, const long long* __restrict__ peer_full, const long long* __restrict__ peer_flags,
                                long long my_flags, int flag_index, int ws, int rank, long long n, float scale, int accumulate,
                                unsigned epoch, int* __restrict__ status, unsigned long long limit_ns, int all_reduce) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = status_set(status) ? 0 : 1;
  __syncthreads();
  if (!ok) return;
  if (blockIdx.x == 0 && threadIdx.x < ws) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned*>(peer_flags[threadIdx.x]) + (long long)flag_index * ws + rank, epoch);
  }
  if (threadIdx.x < ws) {
    const unsigned* f = reinterpret_cast<const unsigned*>(my_flags) + (long long)flag_index * ws + threadIdx.x;
    if (!wait_ge(f, epoch, limit_ns)) { ok = 0; if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER); }
  }
  __syncthreads();
  if (!ok) return;
  rs_pull_body<TIn, TOut>(out, peer_full, ws, rank, n, scale, accumulate, (long long)blockIdx.x * blockDim.x + threadIdx.x,
                          (long long)gridDim.x * blockDim.x, all_reduce ? 0ll : (long long)rank * n);
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
extern "C" void mdt_set_peer_wait_limit_ms(long long ms) { g_peer_wait_ns = ms > 0 ? (unsigned long long)ms * 1000000ull : MDT_PEER_WAIT_LIMIT_NS; }
extern "C" unsigned long long mdt_peer_wait_limit_ns() { return g_peer_wait_ns; }

// CTAs of a row-moving kernel: a multiple of ws (CTA b serves peer b % ws), enough to give every SM a few
static int row_mover_grid(int ws, int max_rows_per_peer) {
  int per_peer = (max_rows_per_peer + EP_ROWS_PER_CTA - 1) / EP_ROWS_PER_CTA;
  const int cap = (sm_count() * 8 + ws - 1) / ws;
  if (per_peer > cap) per_peer = cap;
  if (per_peer < 1) per_peer = 1;
  return per_peer * ws;
}

extern "C" int mdt_ep_counts_send(const int* counts, const long long* peer_base, MdtEpLayout L, int rank, int parity, unsigned epoch, cudaStream_t s) {
  if (L.ws > MDT_EP_MAX_RANKS || L.num_experts % L.ws != 0 || L.num_experts > MDT_EP_MAX_SEGMENTS) return -1;
  ep_counts_send_kernel<<<1, 256, 0, s>>>(counts, peer_base, L, rank, parity, epoch);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_counts_wait_meta(long long my_base, MdtEpLayout L, int rank, int parity, unsigned epoch, int* meta, int* status, cudaStream_t s) {
  if (L.ws > MDT_EP_MAX_RANKS || L.num_experts % L.ws != 0 || L.num_experts > MDT_EP_MAX_SEGMENTS) return -1;
  ep_counts_wait_meta_kernel<<<1, 256, 0, s>>>(my_base, L, rank, parity, epoch, meta, status, g_peer_wait_ns);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_dispatch(const void* x, const int* src_slot, const int* expert_of_slot, const void* slot_scale, const int* meta,
                               const long long* peer_base, MdtEpLayout L, int rank, int num_slots, int top_k, int cols, int parity,
                               const int* status, cudaStream_t s) {
  if (cols % 8 != 0 || rank < 0 || rank >= L.ws) return -1;
  if (num_slots == 0) return 0;
  ep_dispatch_kernel<<<row_mover_grid(L.ws, num_slots), EP_THREADS, 0, s>>>((const bf16*)x, src_slot, expert_of_slot, (const bf16*)slot_scale, meta,
                                                                             peer_base, L, rank, top_k, cols, parity, status);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_recv_prepare(long long my_base, MdtEpLayout L, const int* meta, int cols, int parity, int wait_all, int* status, cudaStream_t s) {
  ep_recv_prepare_kernel<<<64, 256, 0, s>>>(my_base, L, meta, cols, parity, wait_all, status, g_peer_wait_ns);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_combine_send(const void* y, const int* meta, const long long* peer_base, MdtEpLayout L, int rank, int max_rows, int cols,
                                   int parity, const int* status, cudaStream_t s) {
  if (cols % 8 != 0 || rank < 0 || rank >= L.ws) return -1;
  if (max_rows == 0) return 0;
  ep_combine_send_kernel<<<row_mover_grid(L.ws, max_rows), EP_THREADS, 0, s>>>((const bf16*)y, meta, peer_base, L, rank, cols, parity, status);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_fused_meta(const int* meta, MdtEpLayout L, int rank, int* row_rank, int* row_pos, int* tile_expected, cudaStream_t s) {
  ep_fused_meta_kernel<<<64, 256, 0, s>>>(meta, L, rank, row_rank, row_pos, tile_expected);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ep_wait_rows(long long my_base, MdtEpLayout L, const int* meta, int parity, int mult, int* status, cudaStream_t s) {
  ep_wait_rows_kernel<<<1, 1, 0, s>>>(my_base, L, meta, parity, mult < 1 ? 1 : mult, status, g_peer_wait_ns);
  MDT_CM_CHECK();
  return 0;
}
// chunk size of the all-gather's progress flags for shards of `bytes_per_rank` bytes: about 512 KB, whole vectors
extern "C" long long mdt_ag_chunk_bytes(long long bytes_per_rank) {
  const long long target = 512ll << 10;
  long long chunks = (bytes_per_rank + target - 1) / target;
  if (chunks < 1) chunks = 1;
  long long vecs = (bytes_per_rank / 16 + chunks - 1) / chunks;
  if (vecs < 1) vecs = 1;
  return vecs * 16;
}
extern "C" int mdt_ag_chunks_per_rank(long long bytes_per_rank) {
  const long long cb = mdt_ag_chunk_bytes(bytes_per_rank);
  return (int)((bytes_per_rank + cb - 1) / cb);
}
extern "C" int mdt_ag_pull(void* out, const long long* peer_shard, int ws, int rank, long long bytes_per_rank, unsigned* ready, unsigned epoch,
                           int prio_chunks, int max_ctas, cudaStream_t s) {
  if (bytes_per_rank % 16 != 0 || rank < 0 || rank >= ws) return -1;
  const long long vecs = bytes_per_rank / 16;
  const long long chunk_vecs = mdt_ag_chunk_bytes(bytes_per_rank) / 16;
  const int cpr = mdt_ag_chunks_per_rank(bytes_per_rank);
  long long blocks = (long long)cpr * ws;
  long long cap = max_ctas > 0 ? max_ctas : sm_count() * 3;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (prio_chunks < 0) prio_chunks = 0;
  if (prio_chunks > cpr * ws) prio_chunks = cpr * ws;
  ag_pull_kernel<<<(unsigned)blocks, AG_THREADS, 0, s>>>((uint4*)out, peer_shard, ws, rank, vecs, chunk_vecs, cpr, ready, epoch, prio_chunks);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_ag_wait_chunks(const unsigned* ready, int first, int last, unsigned epoch, int* status, cudaStream_t s) {
  if (last <= first) return 0;
  ag_wait_chunks_kernel<<<1, 64, 0, s>>>(ready, first, last, epoch, status, g_peer_wait_ns);
  MDT_CM_CHECK();
  return 0;
}
constexpr int RS_THREADS = 128;
static long long rs_blocks(long long n, int cap_ctas) {
  long long blocks = (n / 4 + RS_THREADS - 1) / RS_THREADS;
  const long long cap = cap_ctas > 0 ? cap_ctas : sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return blocks;
}
extern "C" int mdt_rs_pull(void* out, const long long* peer_full, int ws, int rank, long long n, int in_fp32, int out_fp32, float scale,
                           int accumulate, cudaStream_t s) {
  const unsigned blocks = (unsigned)rs_blocks(n, 0);
  if (in_fp32 && !out_fp32) rs_pull_kernel<float, bf16><<<blocks, RS_THREADS, 0, s>>>((bf16*)out, peer_full, ws, rank, n, scale, accumulate);
  else if (in_fp32 && out_fp32) rs_pull_kernel<float, float><<<blocks, RS_THREADS, 0, s>>>((float*)out, peer_full, ws, rank, n, scale, accumulate);
  else if (!in_fp32 && !out_fp32) rs_pull_kernel<bf16, bf16><<<blocks, RS_THREADS, 0, s>>>((bf16*)out, peer_full, ws, rank, n, scale, accumulate);
  else rs_pull_kernel<bf16, float><<<blocks, RS_THREADS, 0, s>>>((float*)out, peer_full, ws, rank, n, scale, accumulate);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_rs_block(void* out, const long long* peer_full, const long long* peer_flags, long long my_flags, int flag_index, int ws, int rank,
                            long long n, int in_fp32, int out_fp32, float scale, int accumulate, unsigned epoch, int* status, int max_ctas,
                            int all_reduce, cudaStream_t s) {
  if (ws > 32 || rank < 0 || rank >= ws) return -1;
  const unsigned blocks = (unsigned)rs_blocks(n, max_ctas > 0 ? max_ctas : sm_count() * 2);
#define MDT_RS_BLOCK(TI, TO) rs_block_kernel<TI, TO><<<blocks, RS_THREADS, 0, s>>>((TO*)out, peer_full, peer_flags, my_flags, flag_index, ws, rank, n, scale, \
                                                                              accumulate, epoch, status, g_peer_wait_ns, all_reduce)
  if (in_fp32 && !out_fp32) MDT_RS_BLOCK(float, bf16);
  else if (in_fp32 && out_fp32) MDT_RS_BLOCK(float, float);
  else if (!in_fp32 && !out_fp32) MDT_RS_BLOCK(bf16, bf16);
  else MDT_RS_BLOCK(bf16, float);
#undef MDT_RS_BLOCK
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_barrier_arrive(const long long* peer_flags, int ws, int rank, unsigned epoch, cudaStream_t s) {
  barrier_arrive_kernel<<<1, 32, 0, s>>>(peer_flags, ws, rank, epoch);
  MDT_CM_CHECK();
  return 0;
}
extern "C" int mdt_barrier_wait(const void* my_flags, int ws, unsigned epoch, int* status, long long limit_ms, cudaStream_t s) {
  const unsigned long long limit_ns = limit_ms > 0 ? (unsigned long long)limit_ms * 1000000ull : g_peer_wait_ns;
  barrier_wait_kernel<<<1, 32, 0, s>>>((const unsigned*)my_flags, ws, epoch, status, limit_ns);
  MDT_CM_CHECK();
  return 0;
}
