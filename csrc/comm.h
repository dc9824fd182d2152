// Interface of the peer-memory communication kernels (comm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define MDT_EP_MAX_RANKS 16
#define MDT_EP_MAX_SEGMENTS 64

// Byte offsets of the regions of one rank's symmetric workspace (identical on every rank).
typedef struct MdtEpLayout {
  int ws, num_experts;
  int capacity_rows;        // rows of recv_x
  int capacity_slots;       // rows of recv_y
  long long off_counts;     // int   [2][ws][E]
  long long off_count_flags;// u32   [2][ws]
  long long off_arrive_x;   // u32   [2]
  long long off_arrive_y;   // u32   [2]
  long long off_recv_x;     // bf16  [capacity_rows][cols]
  long long off_recv_y;     // bf16  [capacity_slots][cols]
  long long off_tile_ctr;   // u32   [2][capacity_rows / 128]  rows arrived per 128-row tile of recv_x
} MdtEpLayout;

// Offsets (in ints) into the per-exchange metadata buffer written by mdt_ep_counts_wait_meta.
#ifdef __CUDACC__
#define MDT_HD __host__ __device__ inline
#else
#define MDT_HD static inline
#endif
MDT_HD int mdt_ep_meta_counts(int ws, int E) { return 0; }                                   // [ws][E] all ranks' counts
MDT_HD int mdt_ep_meta_recv_tot(int ws, int E) { return ws * E; }                            // [E/ws] rows per local expert
MDT_HD int mdt_ep_meta_recv_off(int ws, int E) { return ws * E + E / ws; }                   // [E/ws + 1] padded first rows
MDT_HD int mdt_ep_meta_dst_row(int ws, int E) { return ws * E + 2 * (E / ws) + 1; }          // [E] first row of my rows at the owner
MDT_HD int mdt_ep_meta_send_start(int ws, int E) { return mdt_ep_meta_dst_row(ws, E) + E; }  // [E + 1] first sorted position per expert
MDT_HD int mdt_ep_meta_seg_row(int ws, int E) { return mdt_ep_meta_send_start(ws, E) + E + 1; }   // [E/ws][ws] first row of a segment here
MDT_HD int mdt_ep_meta_seg_pos(int ws, int E) { return mdt_ep_meta_seg_row(ws, E) + E; }     // [E/ws][ws] first position at the source
MDT_HD int mdt_ep_meta_scalars(int ws, int E) { return mdt_ep_meta_seg_pos(ws, E) + E; }     // [0] rows expected, [1] slots sent, [2] padded rows
MDT_HD int mdt_ep_meta_size(int ws, int E) { return mdt_ep_meta_scalars(ws, E) + 4; }

#ifdef __cplusplus
extern "C" {
#endif
int mdt_ep_counts_send(const int* counts, const long long* peer_base, MdtEpLayout L, int rank, int parity, unsigned epoch, cudaStream_t s);
int mdt_ep_counts_wait_meta(long long my_base, MdtEpLayout L, int rank, int parity, unsigned epoch, int* meta, int* status, cudaStream_t s);
int mdt_ep_dispatch(const void* x, const int* src_slot, const int* expert_of_slot, const void* slot_scale, const int* meta,
                    const long long* peer_base, MdtEpLayout L, int num_slots, int top_k, int cols, int parity, cudaStream_t s);
int mdt_ep_recv_prepare(long long my_base, MdtEpLayout L, const int* meta, int cols, int parity, int wait_all, int* status, cudaStream_t s);
int mdt_ep_fused_meta(const int* meta, MdtEpLayout L, int rank, int* row_rank, int* row_pos, int* tile_expected, cudaStream_t s);
int mdt_ep_combine_send(const void* y, const int* meta, const long long* peer_base, MdtEpLayout L, int rank, int max_rows, int cols,
                        int parity, cudaStream_t s);
int mdt_ep_wait_rows(long long my_base, MdtEpLayout L, const int* meta, int parity, int mult, int* status, cudaStream_t s);
int mdt_ag_pull(void* out, const long long* peer_shard, int ws, long long bytes_per_rank, cudaStream_t s);
int mdt_rs_pull(void* out, const long long* peer_full, int ws, int rank, long long n, int in_fp32, int out_fp32, float scale,
                int accumulate, cudaStream_t s);
int mdt_barrier_arrive(const long long* peer_flags, int ws, int rank, unsigned epoch, cudaStream_t s);
int mdt_barrier_wait(const void* my_flags, int ws, unsigned epoch, int* status, long long limit_ms, cudaStream_t s);  // limit_ms <= 0: default
long long mdt_comm_launch_count(void);
#ifdef __cplusplus
}
#endif
