// C launch interface of the sm_100a kernels.  Every function enqueues work on `stream` and returns
// 0 on success (negative: rejected arguments or a CUDA launch error).  Pointers are device pointers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- GEMM family (gemm_sm100.cu) -------------------------------------------------------------
// Readiness of an operand that lies inside a buffer which an all-gather (mdt_ag_pull with progress flags, csrc/comm.h)
// is still filling on another stream.  The buffer consists of shards of `shard_bytes`, each cut into
// `chunks_per_rank` chunks of `chunk_bytes`; ready[shard * chunks_per_rank + chunk] reaches `epoch` when that chunk
// has landed.  `offset_bytes` is the operand's offset inside the buffer.  ready == NULL: the operand is complete.
typedef struct MdtOperandReady {
  const unsigned* ready; unsigned epoch; int chunks_per_rank;
  long long offset_bytes, shard_bytes, chunk_bytes;
} MdtOperandReady;

typedef struct MdtGemmDesc {
  int mode;            // 0 dense, 1 grouped rows, 2 grouped depth (weight gradient)
  int M, N, K;         // mode 0/1: C is [M(or capacity), N], depth K.  mode 2: C_g is [M, N], depth = rows of g (K if offsets == NULL)
  int G;               // number of groups (1 for dense)
  const int* offsets;  // [G+1] device: first row of every group (multiples of 128); mode 0: NULL
  long long capacity_rows;  // mode 1: host-known upper bound of offsets[G]
  // A operand: bf16 [a_rows, a_cols], row stride lda.  a_mn = 0: rows are M, cols are depth.  a_mn = 1: rows are depth, cols are M.
  const void* A; long long a_rows, a_cols, lda; int a_mn;
  // B operand: bf16 [G, b_rows, b_cols].  b_mn = 0: rows are N, cols are depth.  b_mn = 1: rows are depth, cols are N.
  const void* B; const void* B2; long long b_rows, b_cols, ldb, b_group_stride; int b_mn;
  int dual;            // 1: B and B2 are gate / up matrices, the epilogue writes silu(A*B) * (A*B2)
  // optional second depth segment (LoRA): C += A_l * B_l with depth K_l
  int K_l;
  const void* A_l; long long al_rows, al_cols, lda_l; int a_mn_l;
  const void* B_l; const void* B2_l; long long bl_rows, bl_cols, ldb_l, bl_group_stride; int b_mn_l;
  // output
  void* C; void* C2; void* C3;   // dual mode: C = h, optional C2 = gate, C3 = up (all bf16)
  const void* R;                 // optional (mode 0/1, not dual): bf16 matrix laid out like C, added to the result (residual connection)
  long long ldc, c_group_stride;
  int c_fp32;          // C is fp32 instead of bf16
  int accumulate;      // C += alpha * (A*B) instead of C = alpha * (A*B)
  float alpha;
  int* status;         // optional device word: set to a non-zero code if a wait inside the kernel gave up
  // mode 1, optional: the A rows are being delivered by peer GPUs.  Before a CTA loads the 128-row tile t of A it
  // waits (bounded) until tile_ready[t] >= tile_expected[t] (counters incremented by the senders with release).
  const unsigned* tile_ready; const int* tile_expected;
  // mode 0/1, optional: instead of writing C, the epilogue stores row r of the result at row row_dest_row[r] of the
  // buffer peer_out[row_dest_rank[r]] (bf16, row stride ldc; rank < 0: row dropped) and then adds, per tile and
  // destination, the number of rows delivered to the counter peer_arrive[rank] (release, system scope).
  const int* row_dest_rank; const int* row_dest_row; const long long* peer_out; const long long* peer_arrive; int num_peers;
  // mode 0/1, optional: B (B2) is still being gathered from the peers' shards.  Before a CTA loads the part of B that
  // an output tile needs it waits (bounded) for the chunks that hold it, so the product starts on the weights that
  // have arrived (the local shard first) while the rest of the all-gather is in flight.
  MdtOperandReady b_ready, b2_ready;
  MdtOperandReady bl_ready;   // the same for B_l (the whole matrix of the tile's group is waited for)
} MdtGemmDesc;

int mdt_gemm(const MdtGemmDesc* desc, cudaStream_t stream);
long long mdt_gemm_launch_count(void);
long long mdt_skinny_launch_count(void);
// y[M, r] = alpha * x[M, K] * op(A), r <= 32: a_is_kr = 0 -> A is [r, K] (row stride lda), 1 -> A is [K, r]
int mdt_skinny_mm(const void* x, const void* A, void* y, int M, int K, int r, long long ldx, long long lda,
                  int a_is_kr, float alpha, cudaStream_t s);
// Kernel for 256-wide tiles: 0 the 128-row kernel, 1 / 2 the CTA-pair (cta_group::2) kernel where the shape fills
// 256-row tiles / always, 3 / 4 the tall single-CTA 256 x 256 kernel where it fills / always; returns the previous
// policy (policy < 0 only reads it).
int mdt_gemm_set_pair_policy(int policy);
// CTA pairs resident at once on this device (0 until the pair kernel has been launched)
int mdt_gemm_max_pairs(void);
// Expected total rows of the row-grouped (mode 1) products this host thread issues next, for buffers sized to a
// capacity; 0 = unknown.  Only guides the choice of tile shape.
void mdt_gemm_rows_hint(long long rows);
// The tiling mdt_gemm would pick for `d` under `policy` (see mdt_gemm_set_pair_policy) with that rows hint on a GPU with
// `num_sms` SMs: 0 = 128-row tiles, 1 = CTA pair, 2 = tall.  Reads only M, N, K, K_l, G, mode, dual, c_fp32, accumulate,
// capacity_rows and whether offsets is set; needs no GPU.
int mdt_gemm_choose_tiling(const MdtGemmDesc* d, int policy, long long rows_hint, int num_sms);
// Sharing of the last, partly filled round of 128-row tiles by all SMs along the depth (partial sums through an fp32
// workspace, finished by the last contributor): 1 on (default; MDT_GEMM_SPLIT=0 turns it off), 0 off; returns the
// previous setting (other values only read it).  Results of shared tiles depend on the order of fp32 additions.
int mdt_gemm_set_split(int on);
// upper bound on the pair kernel's grid, in pairs (0 = the resident maximum); for scaling measurements
void mdt_gemm_set_pair_cap(int pairs);

// ---- element-wise / normalisation / loss / optimizer (elementwise.cu) --------------------------
int mdt_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps, cudaStream_t s);
// dres (optional, bf16 [rows, cols]): added to dx (the gradient arriving over the residual connection)
int mdt_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres, void* dx, float* dw_partial,
                    int rows, int cols, int n_partial, cudaStream_t s);
// sums the n_partial rows of dw_partial into dw_bf16 and / or dw_f32 (either may be NULL)
int mdt_rmsnorm_dw_finalize(const float* dw_partial, int n_partial, int cols, void* dw_bf16, float* dw_f32, cudaStream_t s);
int mdt_rope(const void* x, void* y, const int* positions, int tokens, int heads, int head_dim, float theta,
             int inverse, cudaStream_t s);
// dst[0 : rows_used[0]] = src[0 : rows_used[0]] for row buffers of `cols` bf16 elements sized for a capacity (n elements)
int mdt_copy_rows_used(const void* src, void* dst, long long n, const int* rows_used, long long cols, cudaStream_t s);
// rows_used (optional, device): number of leading rows of `cols` elements that hold data; the rest is left untouched
int mdt_swiglu_bwd(const void* g, const void* u, const void* dh, void* dg, void* du, long long n,
                   const int* rows_used, long long cols, cudaStream_t s);
int mdt_swiglu_fwd(const void* g, const void* u, void* h, long long n, cudaStream_t s);
int mdt_embedding(const void* table, const long long* ids, void* out, int tokens, int cols, cudaStream_t s);
int mdt_embedding_bwd(const void* dout, const long long* ids, float* dtable, int tokens, int cols, cudaStream_t s);
// in place: logits (bf16, [rows, vocab]) become d(loss_sum)/dlogits * grad_scale; loss_sum/count accumulate
int mdt_cross_entropy(void* logits, const long long* labels, float* loss_sum, float* count, int rows, int vocab,
                      long long ld, int ignore_index, float grad_scale, cudaStream_t s);
typedef struct MdtAdamTensor { void* p; const void* g; void* m; void* v; long long n; int p_fp32, g_fp32, s_fp32; } MdtAdamTensor;
int mdt_adamw(const MdtAdamTensor* tensors_device, int num_tensors, long long max_n, float lr, float beta1, float beta2,
              float eps, float weight_decay, float bc1, float bc2, float grad_scale, cudaStream_t s);
int mdt_sumsq(const void* x, long long n, int fp32, float* out_accum, cudaStream_t s);
// dst_i (fp32) += src_i (bf16 or fp32), i < count <= MDT_MULTI_ADD_MAX, one launch
#define MDT_MULTI_ADD_MAX 16
typedef struct MdtMultiAdd { float* dst[MDT_MULTI_ADD_MAX]; const void* src[MDT_MULTI_ADD_MAX]; long long n[MDT_MULTI_ADD_MAX];
                             int src_fp32[MDT_MULTI_ADD_MAX]; int count; } MdtMultiAdd;
int mdt_multi_add(const MdtMultiAdd* a, cudaStream_t s);
int mdt_axpby(void* y, const void* x, long long n, float a, float b, int y_fp32, int x_fp32, cudaStream_t s);

// ---- router and permutation (router.cu) -----------------------------------------------------------
// stats (optional, fp32 [2 * experts], accumulated into): per-expert slot counts, then per-expert sums of the scores
int mdt_router_fwd(const void* x, const void* w, void* scores, void* weights, int* idx, int tokens, int hidden,
                   int experts, int top_k, int normalize, float* stats, cudaStream_t s);
int mdt_router_bwd(const void* x, const void* w, const void* scores, const void* weights, const int* idx,
                   const void* dweights, const void* dscores, void* dx, float* dw, int tokens, int hidden, int experts,
                   int top_k, int normalize, int accumulate_dx, cudaStream_t s);
// counting sort of slots by expert id with block-padded groups; all outputs on device
int mdt_make_plan(const int* expert_ids, int num_slots, int num_experts, int block, int capacity, int* counts,
                  int* padded_offsets, int* dest_row, int* src_slot, int* scratch, cudaStream_t s);
int mdt_gather_rows(const void* x, const int* src_slot, const int* padded_offsets, int num_experts, const void* slot_scale,
                    void* out, int capacity, int cols, int top_k, cudaStream_t s);
// residual (optional, bf16 [tokens, cols]): added to the combined rows
int mdt_combine_rows(const void* y, const int* dest_row, const void* weights, const void* residual, void* out, int tokens, int cols,
                     int top_k, cudaStream_t s);
int mdt_combine_wgrad(const void* y, const int* dest_row, const void* dout, void* dweights, int tokens, int cols, int top_k,
                      cudaStream_t s);

// ---- attention (attention.cu) -----------------------------------------------------------------------
int mdt_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_seqlens,
                      int num_seqs, int total_tokens, int max_seqlen, int heads_q, int heads_kv, int head_dim,
                      float scale, cudaStream_t s);
int mdt_attention_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                      void* dq, void* dk, void* dv, float* scratch, const int* cu_seqlens, int num_seqs, int total_tokens,
                      int max_seqlen, int heads_q, int heads_kv, int head_dim, float scale, cudaStream_t s);

long long mdt_launch_count(void);

#ifdef __cplusplus
}
#endif
