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
// `status` (device word, may be NULL): a kernel of an exchange returns at once when it is already non-zero.
int mdt_ep_dispatch(const void* x, const int* src_slot, const int* expert_of_slot, const void* slot_scale, const int* meta,
                    const long long* peer_base, MdtEpLayout L, int rank, int num_slots, int top_k, int cols, int parity,
                    const int* status, cudaStream_t s);
int mdt_ep_recv_prepare(long long my_base, MdtEpLayout L, const int* meta, int cols, int parity, int wait_all, int* status, cudaStream_t s);
int mdt_ep_fused_meta(const int* meta, MdtEpLayout L, int rank, int* row_rank, int* row_pos, int* tile_expected, cudaStream_t s);
int mdt_ep_combine_send(const void* y, const int* meta, const long long* peer_base, MdtEpLayout L, int rank, int max_rows, int cols,
                        int parity, const int* status, cudaStream_t s);
int mdt_ep_wait_rows(long long my_base, MdtEpLayout L, const int* meta, int parity, int mult, int* status, cudaStream_t s);
// All-gather by peer reads with optional progress flags: the buffer is cut into mdt_ag_chunks_per_rank() chunks per
// shard of mdt_ag_chunk_bytes() bytes; ready[r * chunks_per_rank + c] = epoch once chunk c of rank r's shard has landed.
long long mdt_ag_chunk_bytes(long long bytes_per_rank);
int mdt_ag_chunks_per_rank(long long bytes_per_rank);
// The first `prio_chunks` chunks of the buffer are fetched before all others.
int mdt_ag_pull(void* out, const long long* peer_shard, int ws, int rank, long long bytes_per_rank, unsigned* ready, unsigned epoch,
                int prio_chunks, int max_ctas, cudaStream_t s);
int mdt_ag_wait_chunks(const unsigned* ready, int first, int last, unsigned epoch, int* status, cudaStream_t s);
int mdt_rs_pull(void* out, const long long* peer_full, int ws, int rank, long long n, int in_fp32, int out_fp32, float scale,
                int accumulate, cudaStream_t s);
// announce + wait + reduce in one kernel (see rs_block_kernel); flag tables hold u32 [slots][ws].  all_reduce = 0: the
// result is this rank's slice [rank * n, (rank + 1) * n) of the sum; 1: the sum of the whole range [0, n) on every rank.
int mdt_rs_block(void* out, const long long* peer_full, const long long* peer_flags, long long my_flags, int flag_index, int ws, int rank,
                 long long n, int in_fp32, int out_fp32, float scale, int accumulate, unsigned epoch, int* status, int max_ctas,
                 int all_reduce, cudaStream_t s);
int mdt_barrier_arrive(const long long* peer_flags, int ws, int rank, unsigned epoch, cudaStream_t s);
int mdt_barrier_wait(const void* my_flags, int ws, unsigned epoch, int* status, long long limit_ms, cudaStream_t s);  // limit_ms <= 0: default
// limit of every wait for a peer (also the GEMM's waits for operands that other GPUs or streams deliver); ms <= 0 restores 10 s
void mdt_set_peer_wait_limit_ms(long long ms);
unsigned long long mdt_peer_wait_limit_ns(void);
long long mdt_comm_launch_count(void);
#ifdef __cplusplus
}
#endif
