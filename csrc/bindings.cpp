// Python bindings: torch tensors in, C launch interface (api.h) out.  No math happens here.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <nvtx3/nvToolsExt.h>

#include <mutex>
#include <optional>
#include <vector>

#include "api.h"
#include "comm.h"

extern "C" long long mdt_elementwise_launch_count();
extern "C" long long mdt_router_launch_count();
extern "C" long long mdt_attention_launch_count();
extern "C" long long mdt_comm_launch_count();

using torch::Tensor;
typedef std::optional<Tensor> OptTensor;

// NVTX range around a phase of the C++-issued blocks (router / dispatch / experts / combine ...); on with MDT_NVTX=1
struct Phase {
  static bool enabled() { static const bool on = []() { const char* e = getenv("MDT_NVTX"); return e != nullptr && e[0] == '1'; }(); return on; }
  explicit Phase(const char* name) { if (enabled()) nvtxRangePushA(name); }
  ~Phase() { if (enabled()) nvtxRangePop(); }
  // ends the current range of a sequence and begins the next one (nullptr: only ends)
  static void next(const char* name, bool first = false) {
    if (!enabled()) return;
    if (!first) nvtxRangePop();
    if (name != nullptr) nvtxRangePushA(name);
  }
};

static cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
static void check(int rc, const char* what) { TORCH_CHECK(rc == 0, what, " failed with code ", rc); }
static const void* cptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }
static void* mptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }
#define CHECK_BF16(t) TORCH_CHECK((t).scalar_type() == at::kBFloat16 && (t).is_cuda(), #t " must be a CUDA bf16 tensor")

static void fill_operand(const Tensor& t, long long& rows, long long& cols, long long& ld) {
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, "operand must be 2-D with unit inner stride");
  rows = t.size(0); cols = t.size(1); ld = t.stride(0);
}
static void fill_operand3(const Tensor& t, long long& rows, long long& cols, long long& ld, long long& gs) {
  if (t.dim() == 2) { fill_operand(t, rows, cols, ld); gs = rows * ld; return; }
  TORCH_CHECK(t.dim() == 3 && t.stride(2) == 1, "B must be [G, rows, cols] with unit inner stride");
  rows = t.size(1); cols = t.size(2); ld = t.stride(1); gs = t.stride(0);
}

// ---- buffers that an all-gather with progress flags is filling (or has filled) -----------------------------------
// ag_pull_flagged() records (buffer range -> flags, epoch, chunk geometry) here; gemm() looks its B operands up and,
// on a hit, lets the kernel wait for the chunks it needs instead of the whole gather.  An entry keeps its flag tensor
// alive and stays until the same buffer is gathered again: flags of a finished gather all equal the epoch, so a
// product whose operand merely lies in memory that used to be such a buffer passes its waits at once.
namespace {
struct PendingGather { uintptr_t base; int64_t bytes; Tensor ready; unsigned epoch; int chunks_per_rank; int64_t shard_bytes, chunk_bytes; };
std::mutex g_pending_mutex;
std::vector<PendingGather> g_pending;
void lookup_ready(const void* ptr, MdtOperandReady* out) {
  out->ready = nullptr;
  if (ptr == nullptr) return;
  const uintptr_t a = reinterpret_cast<uintptr_t>(ptr);
  std::lock_guard<std::mutex> lock(g_pending_mutex);
  for (const auto& e : g_pending) {
    if (a >= e.base && a < e.base + (uintptr_t)e.bytes) {
      out->ready = (const unsigned*)e.ready.data_ptr();
      out->epoch = e.epoch; out->chunks_per_rank = e.chunks_per_rank;
      out->offset_bytes = (long long)(a - e.base); out->shard_bytes = e.shard_bytes; out->chunk_bytes = e.chunk_bytes;
      return;
    }
  }
}
}  // namespace
void gather_registry_clear() {
  std::lock_guard<std::mutex> lock(g_pending_mutex);
  g_pending.clear();
}

// C = alpha * op(A) op(B) (+ LoRA segment) with the options of MdtGemmDesc; see csrc/api.h
void gemm(int64_t mode, const Tensor& A, bool a_mn, const Tensor& B, bool b_mn, Tensor& C, int64_t M, int64_t N, int64_t K,
          int64_t G, const OptTensor& offsets, int64_t capacity_rows, const OptTensor& B2, const OptTensor& A_l,
          bool a_mn_l, const OptTensor& B_l, const OptTensor& B2_l, bool b_mn_l, int64_t K_l, const OptTensor& C2,
          const OptTensor& C3, bool accumulate, double alpha, const OptTensor& status, const OptTensor& tile_ready,
          const OptTensor& tile_expected, const OptTensor& row_dest_rank, const OptTensor& row_dest_row, const OptTensor& peer_out,
          const OptTensor& peer_arrive, const OptTensor& residual = std::nullopt) {
  CHECK_BF16(A); CHECK_BF16(B);
  c10::cuda::CUDAGuard guard(A.device());
  MdtGemmDesc d;
  memset(&d, 0, sizeof(d));
  d.mode = (int)mode; d.M = (int)M; d.N = (int)N; d.K = (int)K; d.G = (int)G;
  d.offsets = offsets.has_value() ? offsets->data_ptr<int>() : nullptr;
  d.capacity_rows = capacity_rows;
  d.A = A.data_ptr(); fill_operand(A, d.a_rows, d.a_cols, d.lda); d.a_mn = a_mn;
  d.B = B.data_ptr(); fill_operand3(B, d.b_rows, d.b_cols, d.ldb, d.b_group_stride); d.b_mn = b_mn;
  d.dual = B2.has_value();
  d.B2 = cptr(B2);
  d.K_l = (int)K_l;
  if (K_l > 0) {
    TORCH_CHECK(A_l.has_value() && B_l.has_value(), "LoRA segment needs A_l and B_l");
    d.A_l = A_l->data_ptr(); fill_operand(*A_l, d.al_rows, d.al_cols, d.lda_l); d.a_mn_l = a_mn_l;
    d.B_l = B_l->data_ptr(); fill_operand3(*B_l, d.bl_rows, d.bl_cols, d.ldb_l, d.bl_group_stride); d.b_mn_l = b_mn_l;
    d.B2_l = cptr(B2_l);
    TORCH_CHECK(!d.dual || B2_l.has_value(), "dual mode with LoRA needs B2_l");
  }
  TORCH_CHECK(C.is_cuda() && C.stride(-1) == 1, "C must be a CUDA tensor with unit inner stride");
  d.C = C.data_ptr(); d.C2 = mptr(C2); d.C3 = mptr(C3);
  d.ldc = C.stride(-2);
  d.c_group_stride = C.dim() == 3 ? C.stride(0) : 0;
  d.c_fp32 = C.scalar_type() == at::kFloat;
  TORCH_CHECK(d.c_fp32 || C.scalar_type() == at::kBFloat16, "C must be bf16 or fp32");
  d.accumulate = accumulate; d.alpha = (float)alpha;
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->dim() == 2 && residual->stride(1) == 1 && residual->stride(0) == d.ldc &&
                residual->size(0) >= M && residual->size(1) == N, "residual must be a bf16 matrix laid out like C");
    d.R = residual->data_ptr();
  }
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  if (tile_ready.has_value()) {
    d.tile_ready = (const unsigned*)tile_ready->data_ptr();
    d.tile_expected = tile_expected->data_ptr<int>();
  }
  if (row_dest_rank.has_value()) {
    d.row_dest_rank = row_dest_rank->data_ptr<int>(); d.row_dest_row = row_dest_row->data_ptr<int>();
    d.peer_out = (const long long*)peer_out->data_ptr<int64_t>(); d.peer_arrive = (const long long*)peer_arrive->data_ptr<int64_t>();
    d.num_peers = (int)peer_out->numel();
  }
  if (mode != 2) {
    lookup_ready(d.B, &d.b_ready);
    if (d.dual) lookup_ready(d.B2, &d.b2_ready);
    if (d.K_l > 0) lookup_ready(d.B_l, &d.bl_ready);
  }
  check(mdt_gemm(&d, cur_stream()), "mdt_gemm");
}

std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const Tensor& w, double eps) {
  CHECK_BF16(x); CHECK_BF16(w);
  c10::cuda::CUDAGuard guard(x.device());
  auto x2 = x.reshape({-1, x.size(-1)}).contiguous();
  auto y = torch::empty_like(x2);
  auto rstd = torch::empty({x2.size(0)}, x.options().dtype(at::kFloat));
  check(mdt_rmsnorm_fwd(x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), (int)x2.size(0), (int)x2.size(1), (float)eps, cur_stream()), "rmsnorm_fwd");
  return {y.view(x.sizes()), rstd};
}
// dres (optional): gradient that reaches x over the residual connection, added to dx in the same pass
std::vector<Tensor> rmsnorm_bwd(const Tensor& x, const Tensor& w, const Tensor& dy, const Tensor& rstd, const OptTensor& dres = std::nullopt) {
  c10::cuda::CUDAGuard guard(x.device());
  auto x2 = x.reshape({-1, x.size(-1)}).contiguous();
  auto dy2 = dy.reshape({-1, x.size(-1)}).contiguous();
  auto dx = torch::empty_like(x2);
  const int rows = (int)x2.size(0), cols = (int)x2.size(1);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int np = rows < sms ? (rows < 1 ? 1 : rows) : sms;
  auto dwp = torch::empty({np, cols}, x.options().dtype(at::kFloat));
  const void* dr = nullptr;
  Tensor drc;
  if (dres.has_value()) { drc = dres->reshape({-1, x.size(-1)}).contiguous(); TORCH_CHECK(drc.scalar_type() == at::kBFloat16); dr = drc.data_ptr(); }
  check(mdt_rmsnorm_bwd(x2.data_ptr(), w.data_ptr(), dy2.data_ptr(), rstd.data_ptr<float>(), dr, dx.data_ptr(), dwp.data_ptr<float>(), rows, cols, np, cur_stream()), "rmsnorm_bwd");
  return {dx.view(x.sizes()), dwp};
}
// weight gradient of RMSNorm from the per-CTA partial sums of rmsnorm_bwd, in w's dtype
Tensor rmsnorm_dw(const Tensor& dw_partial, const Tensor& like) {
  c10::cuda::CUDAGuard guard(dw_partial.device());
  auto out = torch::empty({dw_partial.size(1)}, like.options());
  const bool f32 = out.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || out.scalar_type() == at::kBFloat16);
  check(mdt_rmsnorm_dw_finalize(dw_partial.data_ptr<float>(), (int)dw_partial.size(0), (int)dw_partial.size(1), f32 ? nullptr : out.data_ptr(),
                                f32 ? out.data_ptr<float>() : nullptr, cur_stream()), "rmsnorm_dw_finalize");
  return out;
}
Tensor rope(const Tensor& x, const Tensor& positions, double theta, bool inverse) {
  CHECK_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 3 && positions.scalar_type() == at::kInt);
  auto xc = x.contiguous();
  auto y = torch::empty_like(xc);
  check(mdt_rope(xc.data_ptr(), y.data_ptr(), positions.data_ptr<int>(), (int)x.size(0), (int)x.size(1), (int)x.size(2), (float)theta, inverse, cur_stream()), "rope");
  return y;
}
Tensor swiglu_fwd(const Tensor& g, const Tensor& u) {
  c10::cuda::CUDAGuard guard(g.device());
  auto h = torch::empty_like(g);
  check(mdt_swiglu_fwd(g.data_ptr(), u.data_ptr(), h.data_ptr(), g.numel(), cur_stream()), "swiglu_fwd");
  return h;
}
// `offsets` (optional, int32 [G+1]): row-group offsets of block-padded buffers; rows past offsets[G] are not touched
std::vector<Tensor> swiglu_bwd(const Tensor& g, const Tensor& u, const Tensor& dh, const OptTensor& offsets) {
  c10::cuda::CUDAGuard guard(g.device());
  auto dg = torch::empty_like(g), du = torch::empty_like(u);
  const int* rows_used = nullptr;
  if (offsets.has_value() && offsets->defined()) {
    TORCH_CHECK(offsets->scalar_type() == at::kInt && offsets->is_contiguous() && g.dim() == 2);
    rows_used = offsets->data_ptr<int>() + (offsets->numel() - 1);
  }
  check(mdt_swiglu_bwd(g.data_ptr(), u.data_ptr(), dh.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(), rows_used,
                       g.size(-1), cur_stream()), "swiglu_bwd");
  return {dg, du};
}
// Copy of a block-padded row buffer sized for a capacity: only rows below offsets[G] are copied (the rest of the
// result is uninitialised and, like the source's, never read).
Tensor clone_used_rows(const Tensor& x, const Tensor& offsets) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.scalar_type() == at::kBFloat16 && offsets.scalar_type() == at::kInt);
  auto y = torch::empty_like(x);
  check(mdt_copy_rows_used(x.data_ptr(), y.data_ptr(), x.numel(), offsets.data_ptr<int>() + (offsets.numel() - 1), x.size(1),
                           cur_stream()), "copy_rows_used");
  return y;
}
Tensor embedding(const Tensor& table, const Tensor& ids) {
  CHECK_BF16(table);
  c10::cuda::CUDAGuard guard(table.device());
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_contiguous());
  auto out = torch::empty({ids.numel(), table.size(1)}, table.options());
  check(mdt_embedding(table.data_ptr(), ids.data_ptr<int64_t>() ? (const long long*)ids.data_ptr<int64_t>() : nullptr, out.data_ptr(), (int)ids.numel(), (int)table.size(1), cur_stream()), "embedding");
  return out;
}
void embedding_bwd(const Tensor& dout, const Tensor& ids, Tensor& dtable) {
  c10::cuda::CUDAGuard guard(dout.device());
  TORCH_CHECK(dtable.scalar_type() == at::kFloat && dout.is_contiguous());
  check(mdt_embedding_bwd(dout.data_ptr(), (const long long*)ids.data_ptr<int64_t>(), dtable.data_ptr<float>(), (int)ids.numel(), (int)dout.size(1), cur_stream()), "embedding_bwd");
}
// logits are overwritten with d(mean loss)/dlogits * grad_scale; returns [loss_sum, count]
Tensor cross_entropy(Tensor& logits, const Tensor& labels, int64_t ignore_index, double grad_scale) {
  CHECK_BF16(logits);
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && labels.scalar_type() == at::kLong && labels.is_contiguous());
  auto out = torch::zeros({2}, logits.options().dtype(at::kFloat));
  check(mdt_cross_entropy(logits.data_ptr(), (const long long*)labels.data_ptr<int64_t>(), out.data_ptr<float>(), out.data_ptr<float>() + 1,
                          (int)logits.size(0), (int)logits.size(1), logits.stride(0), (int)ignore_index, (float)grad_scale, cur_stream()), "cross_entropy");
  return out;
}
void adamw(std::vector<Tensor> ps, std::vector<Tensor> gs, std::vector<Tensor> ms, std::vector<Tensor> vs, double lr, double b1,
           double b2, double eps, double wd, int64_t step, double grad_scale) {
  if (ps.empty()) return;
  c10::cuda::CUDAGuard guard(ps[0].device());
  std::vector<MdtAdamTensor> host(ps.size());
  long long max_n = 0;
  for (size_t i = 0; i < ps.size(); ++i) {
    TORCH_CHECK(ps[i].is_contiguous() && gs[i].is_contiguous() && ms[i].is_contiguous() && vs[i].is_contiguous());
    host[i] = {ps[i].data_ptr(), gs[i].data_ptr(), ms[i].data_ptr(), vs[i].data_ptr(), ps[i].numel(),
               ps[i].scalar_type() == at::kFloat, gs[i].scalar_type() == at::kFloat, ms[i].scalar_type() == at::kFloat};
    max_n = std::max<long long>(max_n, ps[i].numel());
  }
  auto bytes = (int64_t)(host.size() * sizeof(MdtAdamTensor));
  auto staging = torch::empty({bytes}, torch::dtype(torch::kUInt8).pinned_memory(true));
  memcpy(staging.data_ptr(), host.data(), bytes);
  auto dev = staging.to(ps[0].device(), /*non_blocking=*/true);
  const float bc1 = 1.0f - (float)std::pow(b1, (double)step), bc2 = 1.0f - (float)std::pow(b2, (double)step);
  check(mdt_adamw((const MdtAdamTensor*)dev.data_ptr(), (int)host.size(), max_n, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, bc1, bc2, (float)grad_scale, cur_stream()), "adamw");
}
// dst[i] (fp32, contiguous) += src[i] (bf16 or fp32, same number of elements): the gradient accumulators of one unit
// in one launch per 16 tensors
void multi_add(std::vector<Tensor> dst, std::vector<Tensor> src) {
  TORCH_CHECK(dst.size() == src.size());
  if (dst.empty()) return;
  c10::cuda::CUDAGuard guard(dst[0].device());
  for (size_t base = 0; base < dst.size(); base += MDT_MULTI_ADD_MAX) {
    MdtMultiAdd a;
    memset(&a, 0, sizeof(a));
    const size_t n = std::min<size_t>(MDT_MULTI_ADD_MAX, dst.size() - base);
    std::vector<Tensor> keep;
    for (size_t i = 0; i < n; ++i) {
      const Tensor& d = dst[base + i];
      Tensor sx = src[base + i].contiguous();
      TORCH_CHECK(d.scalar_type() == at::kFloat && d.is_contiguous() && d.numel() == sx.numel(), "multi_add: fp32 contiguous destinations of matching size");
      TORCH_CHECK(sx.scalar_type() == at::kFloat || sx.scalar_type() == at::kBFloat16, "multi_add: bf16 or fp32 sources");
      a.dst[i] = d.data_ptr<float>(); a.src[i] = sx.data_ptr(); a.n[i] = d.numel(); a.src_fp32[i] = sx.scalar_type() == at::kFloat;
      keep.push_back(sx);
    }
    a.count = (int)n;
    check(mdt_multi_add(&a, cur_stream()), "multi_add");
  }
}
void sumsq(const Tensor& x, Tensor& out) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && out.scalar_type() == at::kFloat);
  check(mdt_sumsq(x.data_ptr(), x.numel(), x.scalar_type() == at::kFloat, out.data_ptr<float>(), cur_stream()), "sumsq");
}
void axpby(Tensor& y, const Tensor& x, double a, double b) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.numel() == y.numel());
  check(mdt_axpby(y.data_ptr(), x.data_ptr(), x.numel(), (float)a, (float)b, y.scalar_type() == at::kFloat, x.scalar_type() == at::kFloat, cur_stream()), "axpby");
}

// with_stats: a fourth result, fp32 [2 * E]: per-expert slot counts followed by per-expert sums of the scores
std::vector<Tensor> router_fwd(const Tensor& x, const Tensor& w, int64_t top_k, bool normalize, bool with_stats = false) {
  CHECK_BF16(x); CHECK_BF16(w);
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous());
  const int T = (int)x.size(0), H = (int)x.size(1), E = (int)w.size(0);
  auto scores = torch::empty({T, E}, x.options());
  auto weights = torch::empty({T, top_k}, x.options());
  auto idx = torch::empty({T, top_k}, x.options().dtype(at::kInt));
  Tensor stats;
  if (with_stats) stats = torch::zeros({2 * (int64_t)E}, x.options().dtype(at::kFloat));
  check(mdt_router_fwd(x.data_ptr(), w.data_ptr(), scores.data_ptr(), weights.data_ptr(), idx.data_ptr<int>(), T, H, E, (int)top_k, normalize,
                       with_stats ? stats.data_ptr<float>() : nullptr, cur_stream()), "router_fwd");
  if (with_stats) return {scores, weights, idx, stats};
  return {scores, weights, idx};
}
// dx_accum (optional, bf16 [T, H]): the input gradient is added to it instead of written to a new tensor
std::vector<Tensor> router_bwd(const Tensor& x, const Tensor& w, const Tensor& idx, const Tensor& dweights, const OptTensor& dscores,
                               bool normalize, const OptTensor& dx_accum = std::nullopt) {
  c10::cuda::CUDAGuard guard(x.device());
  const int T = (int)x.size(0), H = (int)x.size(1), E = (int)w.size(0), k = (int)idx.size(1);
  if (dx_accum.has_value()) TORCH_CHECK(dx_accum->is_contiguous() && dx_accum->scalar_type() == at::kBFloat16 && dx_accum->numel() == x.numel());
  auto dx = dx_accum.has_value() ? *dx_accum : torch::empty_like(x);
  auto buf = torch::zeros({(int64_t)E * H + (int64_t)T * E}, x.options().dtype(at::kFloat));
  auto dwc = dweights.contiguous();
  OptTensor dsc = dscores.has_value() ? OptTensor(dscores->contiguous()) : std::nullopt;
  check(mdt_router_bwd(x.data_ptr(), w.data_ptr(), nullptr, nullptr, idx.data_ptr<int>(), dwc.data_ptr(), cptr(dsc), dx.data_ptr(),
                       buf.data_ptr<float>(), T, H, E, k, normalize, dx_accum.has_value() ? 1 : 0, cur_stream()), "router_bwd");
  return {dx, buf.narrow(0, 0, (int64_t)E * H).view({E, H})};
}
// returns counts[E], padded_offsets[E+1], dest_row[n], src_slot[capacity]
std::vector<Tensor> make_plan(const Tensor& expert_ids, int64_t num_experts, int64_t block, int64_t capacity) {
  c10::cuda::CUDAGuard guard(expert_ids.device());
  TORCH_CHECK(expert_ids.scalar_type() == at::kInt && expert_ids.is_contiguous());
  const int n = (int)expert_ids.numel();
  auto opt = expert_ids.options();
  auto counts = torch::empty({num_experts}, opt), offs = torch::empty({num_experts + 1}, opt);
  auto dest = torch::empty({n}, opt), src = torch::empty({capacity}, opt);
  auto scratch = torch::empty({((n + 255) / 256 + 1) * num_experts}, opt);
  check(mdt_make_plan(expert_ids.data_ptr<int>(), n, (int)num_experts, (int)block, (int)capacity, counts.data_ptr<int>(), offs.data_ptr<int>(),
                      dest.data_ptr<int>(), src.data_ptr<int>(), scratch.data_ptr<int>(), cur_stream()), "make_plan");
  return {counts, offs, dest, src};
}
Tensor gather_rows(const Tensor& x, const Tensor& src_slot, const OptTensor& padded_offsets, int64_t num_experts, const OptTensor& slot_scale, int64_t top_k) {
  CHECK_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous());
  auto out = torch::empty({src_slot.numel(), x.size(1)}, x.options());
  check(mdt_gather_rows(x.data_ptr(), src_slot.data_ptr<int>(), padded_offsets.has_value() ? padded_offsets->data_ptr<int>() : nullptr, (int)num_experts,
                        cptr(slot_scale), out.data_ptr(), (int)src_slot.numel(), (int)x.size(1), (int)top_k, cur_stream()), "gather_rows");
  return out;
}
Tensor combine_rows(const Tensor& y, const Tensor& dest_row, const OptTensor& weights, int64_t top_k, const OptTensor& residual = std::nullopt) {
  CHECK_BF16(y);
  c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(y.is_contiguous());
  const int T = (int)(dest_row.numel() / top_k);
  auto out = torch::empty({T, y.size(1)}, y.options());
  if (residual.has_value())
    TORCH_CHECK(residual->is_contiguous() && residual->scalar_type() == at::kBFloat16 && residual->numel() == out.numel(), "residual must match the output");
  check(mdt_combine_rows(y.data_ptr(), dest_row.data_ptr<int>(), cptr(weights), cptr(residual), out.data_ptr(), T, (int)y.size(1), (int)top_k, cur_stream()), "combine_rows");
  return out;
}
Tensor combine_wgrad(const Tensor& y, const Tensor& dest_row, const Tensor& dout, int64_t top_k) {
  c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(y.is_contiguous() && dout.is_contiguous());
  const int T = (int)(dest_row.numel() / top_k);
  auto dw = torch::empty({T, top_k}, y.options());
  check(mdt_combine_wgrad(y.data_ptr(), dest_row.data_ptr<int>(), dout.data_ptr(), dw.data_ptr(), T, (int)y.size(1), (int)top_k, cur_stream()), "combine_wgrad");
  return dw;
}

// q [T, Hq, 128], k/v [T, Hkv, 128] -> (o [T, Hq, 128], lse [T, Hq])
std::vector<Tensor> attention_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& cu_seqlens, int64_t max_seqlen, double scale) {
  CHECK_BF16(q); CHECK_BF16(k); CHECK_BF16(v);
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && cu_seqlens.scalar_type() == at::kInt);
  const int T = (int)q.size(0), Hq = (int)q.size(1), Hkv = (int)k.size(1), D = (int)q.size(2);
  auto o = torch::empty_like(q);
  auto lse = torch::empty({T, Hq}, q.options().dtype(at::kFloat));
  check(mdt_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), cu_seqlens.data_ptr<int>(),
                          (int)cu_seqlens.numel() - 1, T, (int)max_seqlen, Hq, Hkv, D, (float)scale, cur_stream()), "attention_fwd");
  return {o, lse};
}
std::vector<Tensor> attention_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& dout, const Tensor& lse,
                                  const Tensor& cu_seqlens, int64_t max_seqlen, double scale) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(dout.is_contiguous() && o.is_contiguous());
  const int T = (int)q.size(0), Hq = (int)q.size(1), Hkv = (int)k.size(1), D = (int)q.size(2);
  auto dq = torch::empty_like(q), dk = torch::empty_like(k), dv = torch::empty_like(v);
  auto scratch = torch::empty({(int64_t)T * Hq * (1 + 3 * D)}, q.options().dtype(at::kFloat));
  check(mdt_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(), lse.data_ptr<float>(), dq.data_ptr(),
                          dk.data_ptr(), dv.data_ptr(), scratch.data_ptr<float>(), cu_seqlens.data_ptr<int>(), (int)cu_seqlens.numel() - 1, T,
                          (int)max_seqlen, Hq, Hkv, D, (float)scale, cur_stream()), "attention_bwd");
  return {dq, dk, dv};
}

// ---- peer-memory communication (comm.cu).  `layout` = [ws, E, capacity_rows, capacity_slots, off_counts,
// off_count_flags, off_arrive_x, off_arrive_y, off_recv_x, off_recv_y]; peer_base = int64 device tensor of
// the peers' workspace base addresses.
static MdtEpLayout to_layout(const std::vector<int64_t>& v) {
  TORCH_CHECK(v.size() == 11, "layout needs 11 entries");
  MdtEpLayout L;
  L.ws = (int)v[0]; L.num_experts = (int)v[1]; L.capacity_rows = (int)v[2]; L.capacity_slots = (int)v[3];
  L.off_counts = v[4]; L.off_count_flags = v[5]; L.off_arrive_x = v[6]; L.off_arrive_y = v[7]; L.off_recv_x = v[8]; L.off_recv_y = v[9]; L.off_tile_ctr = v[10];
  return L;
}
static const long long* ptrs(const Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kLong && t.is_cuda() && t.is_contiguous(), "pointer table must be a CUDA int64 tensor");
  return (const long long*)t.data_ptr<int64_t>();
}
void ep_counts_send(const Tensor& counts, const Tensor& peer_base, std::vector<int64_t> layout, int64_t rank, int64_t parity, int64_t epoch) {
  c10::cuda::CUDAGuard guard(counts.device());
  check(mdt_ep_counts_send(counts.data_ptr<int>(), ptrs(peer_base), to_layout(layout), (int)rank, (int)parity, (unsigned)epoch, cur_stream()), "ep_counts_send");
}
void ep_counts_wait_meta(int64_t my_base, std::vector<int64_t> layout, int64_t rank, int64_t parity, int64_t epoch, Tensor& meta, Tensor& status) {
  c10::cuda::CUDAGuard guard(meta.device());
  MdtEpLayout L = to_layout(layout);
  TORCH_CHECK(meta.scalar_type() == at::kInt && meta.numel() >= mdt_ep_meta_size(L.ws, L.num_experts));
  check(mdt_ep_counts_wait_meta(my_base, L, (int)rank, (int)parity, (unsigned)epoch, meta.data_ptr<int>(), status.data_ptr<int>(), cur_stream()), "ep_counts_wait_meta");
}
void ep_dispatch(const Tensor& x, const Tensor& src_slot, const Tensor& expert_of_slot, const OptTensor& slot_scale, const Tensor& meta,
                 const Tensor& peer_base, std::vector<int64_t> layout, int64_t rank, int64_t top_k, int64_t parity, const OptTensor& status) {
  CHECK_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && expert_of_slot.scalar_type() == at::kInt && expert_of_slot.is_contiguous());
  check(mdt_ep_dispatch(x.data_ptr(), src_slot.data_ptr<int>(), expert_of_slot.data_ptr<int>(), cptr(slot_scale), meta.data_ptr<int>(), ptrs(peer_base),
                        to_layout(layout), (int)rank, (int)expert_of_slot.numel(), (int)top_k, (int)x.size(1), (int)parity,
                        status.has_value() ? status->data_ptr<int>() : nullptr, cur_stream()), "ep_dispatch");
}
void ep_recv_prepare(int64_t my_base, std::vector<int64_t> layout, const Tensor& meta, int64_t cols, int64_t parity, Tensor& status, bool wait_all) {
  c10::cuda::CUDAGuard guard(meta.device());
  check(mdt_ep_recv_prepare(my_base, to_layout(layout), meta.data_ptr<int>(), (int)cols, (int)parity, wait_all, status.data_ptr<int>(), cur_stream()), "ep_recv_prepare");
}
void ep_combine_send(const Tensor& y, const Tensor& meta, const Tensor& peer_base, std::vector<int64_t> layout, int64_t rank, int64_t max_rows,
                     int64_t parity, const OptTensor& status) {
  CHECK_BF16(y);
  c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(y.is_contiguous());
  check(mdt_ep_combine_send(y.data_ptr(), meta.data_ptr<int>(), ptrs(peer_base), to_layout(layout), (int)rank, (int)max_rows, (int)y.size(1), (int)parity,
                            status.has_value() ? status->data_ptr<int>() : nullptr, cur_stream()), "ep_combine_send");
}
void ep_wait_rows(int64_t my_base, std::vector<int64_t> layout, const Tensor& meta, int64_t parity, Tensor& status, int64_t mult) {
  c10::cuda::CUDAGuard guard(meta.device());
  check(mdt_ep_wait_rows(my_base, to_layout(layout), meta.data_ptr<int>(), (int)parity, (int)mult, status.data_ptr<int>(), cur_stream()), "ep_wait_rows");
}
// row_rank / row_pos [capacity_rows] and tile_expected [capacity_rows / 128] of this rank's receive layout
std::vector<Tensor> ep_fused_meta(const Tensor& meta, std::vector<int64_t> layout, int64_t rank) {
  c10::cuda::CUDAGuard guard(meta.device());
  MdtEpLayout L = to_layout(layout);
  // the kernel writes every entry a consumer can read (rows / tiles below the padded row count in use)
  auto rr = torch::empty({L.capacity_rows}, meta.options());
  auto rp = torch::empty({L.capacity_rows}, meta.options());
  auto te = torch::empty({L.capacity_rows / 128}, meta.options());
  check(mdt_ep_fused_meta(meta.data_ptr<int>(), L, (int)rank, rr.data_ptr<int>(), rp.data_ptr<int>(), te.data_ptr<int>(), cur_stream()), "ep_fused_meta");
  return {rr, rp, te};
}
std::vector<int64_t> ep_meta_offsets(int64_t ws, int64_t E) {
  return {mdt_ep_meta_counts(ws, E), mdt_ep_meta_recv_tot(ws, E), mdt_ep_meta_recv_off(ws, E), mdt_ep_meta_dst_row(ws, E),
          mdt_ep_meta_send_start(ws, E), mdt_ep_meta_seg_row(ws, E), mdt_ep_meta_seg_pos(ws, E), mdt_ep_meta_scalars(ws, E), mdt_ep_meta_size(ws, E)};
}
void ag_pull(Tensor& out, const Tensor& peer_shard, int64_t ws, int64_t rank, int64_t bytes_per_rank, int64_t max_ctas) {
  c10::cuda::CUDAGuard guard(out.device());
  check(mdt_ag_pull(out.data_ptr(), ptrs(peer_shard), (int)ws, (int)rank, bytes_per_rank, nullptr, 0, 0, (int)max_ctas, cur_stream()), "ag_pull");
}
// Number of progress flags of a gathered buffer with shards of `bytes_per_rank` bytes, and the chunk size in bytes.
std::vector<int64_t> ag_chunks(int64_t ws, int64_t bytes_per_rank) {
  return {(int64_t)mdt_ag_chunks_per_rank(bytes_per_rank) * ws, (int64_t)mdt_ag_chunk_bytes(bytes_per_rank)};
}
// All-gather that publishes its progress in `ready` (int32 [ws * chunks per rank], values only ever grow; `epoch` must
// exceed every earlier epoch used with these flags) and registers the buffer, so that products whose weight operand
// lies inside it wait chunk by chunk.  Chunks [0, priority_chunks) of the buffer are fetched before all others.
void ag_pull_flagged(Tensor& out, const Tensor& peer_shard, int64_t ws, int64_t rank, int64_t bytes_per_rank, Tensor& ready, int64_t epoch,
                     int64_t priority_chunks, int64_t max_ctas) {
  c10::cuda::CUDAGuard guard(out.device());
  const int cpr = mdt_ag_chunks_per_rank(bytes_per_rank);
  TORCH_CHECK(ready.scalar_type() == at::kInt && ready.is_contiguous() && ready.numel() >= (int64_t)cpr * ws, "ready: int32 [ws * chunks per rank]");
  TORCH_CHECK(out.is_contiguous() && out.numel() * out.element_size() >= bytes_per_rank * ws);
  {
    std::lock_guard<std::mutex> lock(g_pending_mutex);
    const uintptr_t base = reinterpret_cast<uintptr_t>(out.data_ptr());
    PendingGather e{base, bytes_per_rank * ws, ready, (unsigned)epoch, cpr, bytes_per_rank, mdt_ag_chunk_bytes(bytes_per_rank)};
    bool found = false;
    for (auto& old : g_pending) {
      // a new gather into overlapping memory replaces what was known about it
      if (base < old.base + (uintptr_t)old.bytes && old.base < base + (uintptr_t)e.bytes) { if (!found) { old = e; found = true; } else { old.bytes = 0; } }
    }
    if (!found) g_pending.push_back(e);
  }
  check(mdt_ag_pull(out.data_ptr(), ptrs(peer_shard), (int)ws, (int)rank, bytes_per_rank, (unsigned*)ready.data_ptr(), (unsigned)epoch, (int)priority_chunks,
                    (int)max_ctas, cur_stream()), "ag_pull");
}
// the current stream waits (one small kernel) until chunks [first, last) of a flagged gather have landed
void ag_wait_chunks(const Tensor& ready, int64_t first, int64_t last, int64_t epoch, Tensor& status) {
  c10::cuda::CUDAGuard guard(ready.device());
  check(mdt_ag_wait_chunks((const unsigned*)ready.data_ptr(), (int)first, (int)last, (unsigned)epoch, status.data_ptr<int>(), cur_stream()), "ag_wait_chunks");
}
void rs_pull(Tensor& out, const Tensor& peer_full, int64_t ws, int64_t rank, bool in_fp32, double scale, bool accumulate) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_contiguous());
  check(mdt_rs_pull(out.data_ptr(), ptrs(peer_full), (int)ws, (int)rank, out.numel(), in_fp32, out.scalar_type() == at::kFloat, (float)scale, accumulate, cur_stream()), "rs_pull");
}
// announce + wait + reduce-scatter of one group in one kernel (csrc/comm.cu::rs_block_kernel)
void rs_block(Tensor& out, const Tensor& peer_full, const Tensor& peer_flags, int64_t my_flags, int64_t flag_index, int64_t ws, int64_t rank,
              bool in_fp32, double scale, bool accumulate, int64_t epoch, Tensor& status, int64_t max_ctas, bool all_reduce) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_contiguous());
  check(mdt_rs_block(out.data_ptr(), ptrs(peer_full), ptrs(peer_flags), my_flags, (int)flag_index, (int)ws, (int)rank, out.numel(), in_fp32,
                     out.scalar_type() == at::kFloat, (float)scale, accumulate, (unsigned)epoch, status.data_ptr<int>(), (int)max_ctas,
                     all_reduce ? 1 : 0, cur_stream()), "rs_block");
}
void barrier_arrive(const Tensor& peer_flags, int64_t ws, int64_t rank, int64_t epoch) {
  c10::cuda::CUDAGuard guard(peer_flags.device());
  check(mdt_barrier_arrive(ptrs(peer_flags), (int)ws, (int)rank, (unsigned)epoch, cur_stream()), "barrier_arrive");
}
void barrier_wait(int64_t my_flags, int64_t ws, int64_t epoch, Tensor& status, int64_t limit_ms) {
  c10::cuda::CUDAGuard guard(status.device());
  check(mdt_barrier_wait((const void*)my_flags, (int)ws, (unsigned)epoch, status.data_ptr<int>(), limit_ms, cur_stream()), "barrier_wait");
}

int64_t launch_count() {
  return mdt_gemm_launch_count() + mdt_skinny_launch_count() + mdt_elementwise_launch_count() + mdt_router_launch_count() + mdt_attention_launch_count() + mdt_comm_launch_count();
}


// =====================================================================================================
// Whole attention sub-block in one call each way (RMSNorm -> q/k/v (+LoRA) -> RoPE -> attention -> o (+LoRA)
// -> residual).  Same kernels as the per-op bindings; issuing them from C++ keeps the host ahead of the GPU.
// =====================================================================================================
// y[M, r] = alpha * x[M, K] * A^T (A [r, K]) or alpha * x * A (A [K, r], a_is_kr): CUDA-core kernel for r <= 32
bool skinny_ok(const Tensor& x, const Tensor& A, bool a_is_kr) {
  const int64_t K = x.size(1), r = a_is_kr ? A.size(1) : A.size(0);
  return x.scalar_type() == at::kBFloat16 && A.scalar_type() == at::kBFloat16 && x.dim() == 2 && A.dim() == 2 && r >= 1 && r <= 32 &&
         K % 8 == 0 && x.stride(1) == 1 && x.stride(0) % 8 == 0 && A.stride(1) == 1 &&
         (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0 && (a_is_kr ? A.size(0) : A.size(1)) == K;
}
Tensor skinny_mm(const Tensor& x, const Tensor& A, bool a_is_kr, double alpha) {
  TORCH_CHECK(skinny_ok(x, A, a_is_kr), "skinny_mm: unsupported operands");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t M = x.size(0), K = x.size(1), r = a_is_kr ? A.size(1) : A.size(0);
  auto y = torch::empty({M, r}, x.options());
  check(mdt_skinny_mm(x.data_ptr(), A.data_ptr(), y.data_ptr(), (int)M, (int)K, (int)r, x.stride(0), A.stride(0), a_is_kr ? 1 : 0,
                      (float)alpha, cur_stream()), "skinny_mm");
  return y;
}

namespace {

struct Lin { Tensor W; OptTensor A, B; double s; };   // y = x W^T + s (x A^T) B^T

void gemm_raw(int mode, const Tensor& A, bool a_mn, const Tensor& B, bool b_mn, Tensor& C, int64_t M, int64_t N, int64_t K,
              const OptTensor& A_l, const OptTensor& B_l, bool b_mn_l, int64_t K_l, bool accumulate, double alpha, const OptTensor& status,
              const OptTensor& residual = std::nullopt) {
  gemm(mode, A, a_mn, B, b_mn, C, M, N, K, 1, std::nullopt, 0, std::nullopt, A_l, false, B_l, std::nullopt, b_mn_l, K_l, std::nullopt,
       std::nullopt, accumulate, alpha, status, std::nullopt, std::nullopt, std::nullopt, std::nullopt, std::nullopt, std::nullopt, residual);
}
// y = x W^T (+ LoRA) (+ residual, added in the GEMM's epilogue); returns (y, t) with t = s x A^T
std::pair<Tensor, OptTensor> lin_fwd(const Tensor& x, const Lin& l, const OptTensor& status, const OptTensor& residual = std::nullopt) {
  const int64_t M = x.size(0), K = x.size(1), N = l.W.size(0);
  auto y = torch::empty({M, N}, x.options());
  if (!l.A.has_value()) {
    gemm_raw(0, x, false, l.W, false, y, M, N, K, std::nullopt, std::nullopt, false, 0, false, 1.0, status, residual);
    return {y, std::nullopt};
  }
  const int64_t r = l.A->size(0);
  Tensor t;
  if (skinny_ok(x, *l.A, false)) {
    t = skinny_mm(x, *l.A, false, l.s);
  } else {
    t = torch::empty({M, r}, x.options());
    gemm_raw(0, x, false, *l.A, false, t, M, r, K, std::nullopt, std::nullopt, false, 0, false, l.s, status);
  }
  gemm_raw(0, x, false, l.W, false, y, M, N, K, t, l.B, false, r, false, 1.0, status, residual);
  return {y, t};
}
// dx (+)= dy W (+ LoRA), and the requested parameter gradients
struct LinGrads { OptTensor dW, dA, dB; };
LinGrads lin_bwd(const Tensor& dy, const Tensor& xin, const Lin& l, const OptTensor& t, bool need_w, bool need_a, bool need_b,
                 Tensor& dx, bool accumulate, const OptTensor& status) {
  const int64_t M = dy.size(0), N = dy.size(1), K = l.W.size(1);
  LinGrads g;
  OptTensor dt;
  if (l.A.has_value()) {
    const int64_t r = l.A->size(0);
    if (skinny_ok(dy, *l.B, true)) {
      dt = skinny_mm(dy, *l.B, true, l.s);                                                                           // s dy B
    } else {
      dt = torch::empty({M, r}, dy.options());
      gemm_raw(0, dy, false, *l.B, true, *dt, M, r, N, std::nullopt, std::nullopt, false, 0, false, l.s, status);
    }
    gemm_raw(0, dy, false, l.W, true, dx, M, K, N, dt, l.A, true, r, accumulate, 1.0, status);                       // dy W + dt A
    if (need_a) { g.dA = torch::empty_like(*l.A); gemm_raw(2, *dt, true, xin, true, *g.dA, r, K, M, std::nullopt, std::nullopt, false, 0, false, 1.0, status); }
    if (need_b) { g.dB = torch::empty_like(*l.B); gemm_raw(2, dy, true, *t, true, *g.dB, N, r, M, std::nullopt, std::nullopt, false, 0, false, 1.0, status); }
  } else {
    gemm_raw(0, dy, false, l.W, true, dx, M, K, N, std::nullopt, std::nullopt, false, 0, accumulate, 1.0, status);
  }
  if (need_w) { g.dW = torch::empty_like(l.W); gemm_raw(2, dy, true, xin, true, *g.dW, N, K, M, std::nullopt, std::nullopt, false, 0, false, 1.0, status); }
  return g;
}
Lin make_lin(const std::vector<Tensor>& p, size_t& i, double s) {
  Lin l;
  l.W = p[i++];
  l.s = s;
  if (s >= 0.0) { l.A = p[i++]; l.B = p[i++]; }   // negative scaling = no adapter on this projection
  return l;
}

}  // namespace

// params: ln_w, then for q, k, v, o: W [, A, B].  scalings[j] < 0: projection j has no adapter.
// Returns {out, rstd, xn, qr, kr, v3, o, lse, tq, tk, tv, to} (adapter intermediates are empty tensors when absent).
std::vector<Tensor> attention_block_fwd(const Tensor& x, const std::vector<Tensor>& params, const std::vector<double>& scalings,
                                        const Tensor& positions, const Tensor& cu_seqlens, int64_t max_seqlen, double eps, double theta,
                                        int64_t Hq, int64_t Hkv, int64_t d, const Tensor& status_t) {
  c10::cuda::CUDAGuard guard(x.device());
  Phase ph("attention.forward");
  OptTensor status = status_t;
  const int64_t T = x.size(0);
  size_t i = 1;
  Lin lq = make_lin(params, i, scalings[0]), lk = make_lin(params, i, scalings[1]), lv = make_lin(params, i, scalings[2]),
      lo = make_lin(params, i, scalings[3]);
  auto nr = rmsnorm_fwd(x, params[0], eps);
  Tensor xn = nr[0], rstd = nr[1];
  // The k and v projections have 1024 output columns: for one micro-batch that is ~20 tiles walking the whole
  // depth, a latency-bound launch that fills a seventh of the GPU.  They run on two side streams beside the q
  // projection (80 tiles); the three kernels fit on the 148 SMs together.
  Tensor q, k, v, qr, kr;
  OptTensor tq, tk, tv;
  static const bool side_streams = []() { const char* e = getenv("MDT_QKV_STREAMS"); return !(e != nullptr && e[0] == '0'); }();
  if (side_streams) {
    auto main_stream = at::cuda::getCurrentCUDAStream();
    auto s1 = at::cuda::getStreamFromPool(false, x.device().index()), s2 = at::cuda::getStreamFromPool(false, x.device().index());
    at::cuda::CUDAEvent ready, done1, done2;
    ready.record(main_stream);
    auto keep = [&](const Tensor& t) { c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), main_stream); };
    {
      c10::cuda::CUDAStreamGuard g1(s1);
      ready.block(s1);
      std::tie(k, tk) = lin_fwd(xn, lk, status);
      kr = rope(k.view({T, Hkv, d}), positions, theta, false);
      keep(k); keep(kr); if (tk.has_value()) keep(*tk);
      done1.record(s1);
    }
    {
      c10::cuda::CUDAStreamGuard g2(s2);
      ready.block(s2);
      std::tie(v, tv) = lin_fwd(xn, lv, status);
      keep(v); if (tv.has_value()) keep(*tv);
      done2.record(s2);
    }
    std::tie(q, tq) = lin_fwd(xn, lq, status);
    qr = rope(q.view({T, Hq, d}), positions, theta, false);
    done1.block(main_stream);
    done2.block(main_stream);
  } else {
    std::tie(q, tq) = lin_fwd(xn, lq, status);
    std::tie(k, tk) = lin_fwd(xn, lk, status);
    std::tie(v, tv) = lin_fwd(xn, lv, status);
    qr = rope(q.view({T, Hq, d}), positions, theta, false);
    kr = rope(k.view({T, Hkv, d}), positions, theta, false);
  }
  Tensor v3 = v.view({T, Hkv, d});
  auto at = attention_fwd(qr, kr, v3, cu_seqlens, max_seqlen, 1.0 / std::sqrt((double)d));
  Tensor o = at[0], lse = at[1];
  auto [out, to] = lin_fwd(o.view({T, Hq * d}), lo, status, x.is_contiguous() ? OptTensor(x) : OptTensor(x.contiguous()));   // + x in the epilogue
  Tensor none = torch::empty({0}, x.options());
  return {out, rstd, xn, qr, kr, v3, o, lse, tq.value_or(none), tk.value_or(none), tv.value_or(none), to.value_or(none)};
}

// needs[j] for params[j]; returns {dx, grads of params in order (empty tensor where not needed)}
std::vector<Tensor> attention_block_bwd(const Tensor& dy, const std::vector<Tensor>& saved, const std::vector<Tensor>& params,
                                        const std::vector<double>& scalings, const std::vector<bool>& needs, const Tensor& positions,
                                        const Tensor& cu_seqlens, int64_t max_seqlen, double theta, int64_t Hq, int64_t Hkv, int64_t d,
                                        const Tensor& status_t) {
  c10::cuda::CUDAGuard guard(dy.device());
  Phase ph("attention.backward");
  OptTensor status = status_t;
  const Tensor &x = saved[0], &rstd = saved[1], &xn = saved[2], &qr = saved[3], &kr = saved[4], &v3 = saved[5], &o = saved[6], &lse = saved[7];
  auto opt = [](const Tensor& t) -> OptTensor { return t.numel() ? OptTensor(t) : std::nullopt; };
  OptTensor tq = opt(saved[8]), tk = opt(saved[9]), tv = opt(saved[10]), to = opt(saved[11]);
  const int64_t T = x.size(0), H = x.size(1);
  size_t i = 1;
  const size_t iq = i; Lin lq = make_lin(params, i, scalings[0]);
  const size_t ik = i; Lin lk = make_lin(params, i, scalings[1]);
  const size_t iv = i; Lin lv = make_lin(params, i, scalings[2]);
  const size_t io = i; Lin lo = make_lin(params, i, scalings[3]);
  Tensor none = torch::empty({0}, x.options());
  std::vector<Tensor> grads(params.size(), none);
  auto put = [&](size_t at, const Lin& l, const LinGrads& g) {
    if (g.dW.has_value()) grads[at] = *g.dW;
    if (l.A.has_value()) { if (g.dA.has_value()) grads[at + 1] = *g.dA; if (g.dB.has_value()) grads[at + 2] = *g.dB; }
  };
  auto nd = [&](size_t at, int k2) { return at + k2 < needs.size() ? (bool)needs[at + k2] : false; };
  Tensor dyc = dy.contiguous();
  Tensor o2 = o.view({T, Hq * d});
  Tensor d_o = torch::empty({T, Hq * d}, x.options());
  put(io, lo, lin_bwd(dyc, o2, lo, to, nd(io, 0), lo.A.has_value() && nd(io, 1), lo.A.has_value() && nd(io, 2), d_o, false, status));
  auto g3 = attention_bwd(qr, kr, v3, o, d_o.view({T, Hq, d}), lse, cu_seqlens, max_seqlen, 1.0 / std::sqrt((double)d));
  Tensor dq = rope(g3[0], positions, theta, true).view({T, Hq * d});
  Tensor dk = rope(g3[1], positions, theta, true).view({T, Hkv * d});
  Tensor dv = g3[2].view({T, Hkv * d});
  Tensor d_xn = torch::empty({T, H}, x.options());
  put(iq, lq, lin_bwd(dq, xn, lq, tq, nd(iq, 0), lq.A.has_value() && nd(iq, 1), lq.A.has_value() && nd(iq, 2), d_xn, false, status));
  put(ik, lk, lin_bwd(dk, xn, lk, tk, nd(ik, 0), lk.A.has_value() && nd(ik, 1), lk.A.has_value() && nd(ik, 2), d_xn, true, status));
  put(iv, lv, lin_bwd(dv, xn, lv, tv, nd(iv, 0), lv.A.has_value() && nd(iv, 1), lv.A.has_value() && nd(iv, 2), d_xn, true, status));
  auto rb = rmsnorm_bwd(x, params[0], d_xn, rstd, dyc);     // + dy: the residual connection's gradient
  Tensor dx = rb[0];
  if (needs[0]) grads[0] = rmsnorm_dw(rb[1], params[0]);
  std::vector<Tensor> out;
  out.reserve(1 + grads.size());
  out.push_back(dx);
  for (auto& g : grads) out.push_back(g);
  return out;
}

// =====================================================================================================
// Whole MoE sub-block (no expert adapters): RMSNorm -> router -> plan -> [peer exchange] -> grouped SwiGLU MLP
// -> [exchange back] -> gate-weighted combine -> residual.  `ep` carries the exchange state when the experts are
// expert-parallel: ints = {my_base, rank, count_epoch, count_parity, data_parity, num_col_tiles}, tensors =
// {peer_base, peer_out, peer_arrive(parity), tile_counters(parity), recv_x, recv_y, identity}.
// =====================================================================================================
namespace {
void ggemm(int mode, const Tensor& A, bool a_mn, const Tensor& B, bool b_mn, Tensor& C, int64_t M, int64_t N, int64_t K, int64_t G,
           const Tensor& offs, int64_t cap, const OptTensor& B2, const OptTensor& A_l, const OptTensor& B_l, bool b_mn_l, int64_t K_l,
           const OptTensor& C2, const OptTensor& C3, bool acc, double alpha, const OptTensor& status, const OptTensor& w0, const OptTensor& w1,
           const OptTensor& s0, const OptTensor& s1, const OptTensor& s2, const OptTensor& s3) {
  gemm(mode, A, a_mn, B, b_mn, C, M, N, K, G, offs, cap, B2, A_l, false, B_l, std::nullopt, b_mn_l, K_l, C2, C3, acc, alpha, status, w0, w1, s0, s1, s2, s3);
}
const OptTensor NONE = std::nullopt;
}  // namespace

// Tells the GEMM's tile-shape choice how many rows to expect in buffers that are sized for a capacity.
struct RowsHint {
  explicit RowsHint(int64_t rows) { mdt_gemm_rows_hint((long long)rows); }
  ~RowsHint() { mdt_gemm_rows_hint(0); }
};

// ckpt: 0 = plain call.  1 = graph-free first pass of a block that will be recomputed: everything the backward pass
// needs from the token exchange is returned as well (the `stash`: routing, counts, received rows, returned expert
// outputs).  2 = the recomputation, given that stash: only RMSNorm and the gate/up GEMM run again (for the SwiGLU
// inputs); there is no second dispatch, down projection or combine, and the returned block output is not computed
// (the backward pass does not read it).
// Returns {out, tokens_per_expert} (+ stash when ckpt == 1), or with grad_mode the state list that moe_block_bwd takes.
std::vector<Tensor> moe_block_fwd(const Tensor& x, const Tensor& ln_w, const Tensor& Wr, const Tensor& w1, const Tensor& w2, const Tensor& w3,
                                  double eps, int64_t top_k, int64_t E, bool grad_mode, const std::vector<int64_t>& layout,
                                  const std::vector<int64_t>& ep_ints, const std::vector<Tensor>& ep, const Tensor& status_t,
                                  int64_t ckpt, const std::vector<Tensor>& stash) {
  c10::cuda::CUDAGuard guard(x.device());
  OptTensor status = status_t;
  Tensor st = status_t;
  const int64_t T = x.size(0), H = x.size(1), El = w1.size(0), F = w1.size(1);
  if (ckpt == 2) {
    TORCH_CHECK(grad_mode && stash.size() == 14, "moe_block_fwd: recomputation needs the stash of the first pass");
    const Tensor &tpe = stash[0], &wts = stash[1], &idx = stash[2], &ys = stash[3], &p1 = stash[4], &p2 = stash[5], &p3 = stash[6],
                 &meta_c = stash[7], &rr = stash[8], &rp = stash[9], &te = stash[10], &xg = stash[11], &expert_sorted = stash[12],
                 &offs = stash[13];
    RowsHint rows_hint(meta_c.numel() > 0 ? T * top_k : 0);
    auto nr = rmsnorm_fwd(x, ln_w, eps);
    const int64_t R = xg.size(0);
    Tensor h = torch::empty({R, F}, x.options()), g = torch::empty({R, F}, x.options()), u = torch::empty({R, F}, x.options());
    ggemm(1, xg, false, w1, false, h, R, F, H, El, offs, R, w3, NONE, NONE, false, 0, g, u, false, 1.0, status, NONE, NONE, NONE, NONE, NONE, NONE);
    Tensor out = torch::empty({T, H}, x.options());
    return {out, tpe, nr[1], nr[0], wts, idx, ys, p1, p2, p3, meta_c, rr, rp, te, xg, g, u, h, expert_sorted, offs};
  }
  const bool is_ep = !ep.empty();
  const bool keep = grad_mode || ckpt == 1;      // tensors of the exchange outlive this call
  RowsHint rows_hint(is_ep ? T * top_k : 0);   // balanced routing: a rank receives about as many rows as it sends
  Tensor xn, rstd, wts, idx;
  {
    Phase ph("moe.router");
    auto nr = rmsnorm_fwd(x, ln_w, eps);
    xn = nr[0]; rstd = nr[1];
    auto rt = router_fwd(xn, Wr, top_k, true);
    wts = rt[1]; idx = rt[2];
  }
  Tensor none = torch::empty({0}, x.options());
  Tensor nonei = torch::empty({0}, idx.options());
  Tensor xg, offs, meta_c = nonei, rr = nonei, rp = nonei, te = nonei, expert_sorted = nonei, ys, out;
  int64_t cap;
  std::vector<Tensor> plan;
  OptTensor w0, w1o, s0, s1, s2, s3;
  const int64_t n_slots = idx.numel();
  Phase::next("moe.dispatch", true);
  if (!is_ep) {
    const int64_t c = std::max<int64_t>(128, ((n_slots + E * 127) / 128) * 128);
    plan = make_plan(idx.view({-1}), E, 128, c);
    xg = gather_rows(xn, plan[3], plan[1], E, NONE, top_k);
    offs = plan[1]; cap = c;
  } else {
    plan = make_plan(idx.view({-1}), E, 1, n_slots);
    const int64_t my_base = ep_ints[0], rank = ep_ints[1], epoch = ep_ints[2], cpar = ep_ints[3], dpar = ep_ints[4];
    MdtEpLayout L = to_layout(layout);
    meta_c = torch::empty({mdt_ep_meta_size(L.ws, L.num_experts)}, idx.options());
    ep_counts_send(plan[0], ep[0], layout, rank, cpar, epoch);
    ep_counts_wait_meta(my_base, layout, rank, cpar, epoch, meta_c, st);
    auto fm = ep_fused_meta(meta_c, layout, rank);
    rr = fm[0]; rp = fm[1]; te = fm[2];
    Tensor eos = idx.view({-1});
    if (keep) expert_sorted = eos.index_select(0, plan[3].to(at::kLong));
    ep_dispatch(xn, plan[3], eos, NONE, meta_c, ep[0], layout, rank, top_k, dpar, status);
    ep_recv_prepare(my_base, layout, meta_c, H, dpar, st, false);
    xg = ep[4];
    const int o2 = mdt_ep_meta_recv_off(L.ws, L.num_experts);
    offs = meta_c.narrow(0, o2, El + 1);
    cap = L.capacity_rows;
    w0 = ep[3]; w1o = te; s0 = rr; s1 = rp; s2 = ep[1]; s3 = ep[2];
  }
  Phase::next("moe.experts");
  const int64_t R = xg.size(0);
  Tensor h = torch::empty({R, F}, x.options());
  OptTensor g, u;
  if (grad_mode) { g = torch::empty({R, F}, x.options()); u = torch::empty({R, F}, x.options()); }
  ggemm(1, xg, false, w1, false, h, R, F, H, El, offs, cap, w3, NONE, NONE, false, 0, g, u, false, 1.0, status, w0, w1o, NONE, NONE, NONE, NONE);
  if (is_ep && keep) xg = clone_used_rows(xg, offs);   // the receive buffer is reused by the next exchange
  Tensor y = torch::empty({R, H}, x.options());
  ggemm(1, h, false, w2, true, y, R, H, F, El, offs, cap, NONE, NONE, NONE, false, 0, NONE, NONE, false, 1.0, status, NONE, NONE, s0, s1, s2, s3);
  Phase::next("moe.combine");
  if (!is_ep) {
    ys = y;
  } else {
    ep_wait_rows(ep_ints[0], layout, meta_c, ep_ints[4], st, ep_ints[5]);
    ys = ep[5].narrow(0, 0, n_slots);
    if (keep) ys = ys.clone();
  }
  out = combine_rows(ys, plan[2], wts, top_k, x.is_contiguous() ? OptTensor(x) : OptTensor(x.contiguous()));   // + x
  Phase::next(nullptr);
  if (ckpt == 1 && !grad_mode)
    return {out, plan[0], wts, idx, ys, plan[1], plan[2], plan[3], meta_c, rr, rp, te, xg, expert_sorted, offs};
  if (!grad_mode) return {out, plan[0]};
  return {out, plan[0], rstd, xn, wts, idx, ys, plan[1], plan[2], plan[3], meta_c, rr, rp, te, xg, *g, *u, h, expert_sorted, offs};
}

// state = the forward's return list; wg = {dw1, dw2, dw3} accumulation buffers ([El,F,H]) or empty when the experts are frozen.
// Returns {dx, d_ln, d_Wr}.
std::vector<Tensor> moe_block_bwd(const Tensor& dy, const std::vector<Tensor>& state, const Tensor& x, const Tensor& ln_w, const Tensor& Wr,
                                  const Tensor& w1, const Tensor& w2, const Tensor& w3, const std::vector<Tensor>& wg, double wscale,
                                  int64_t top_k, int64_t E, const std::vector<int64_t>& layout, const std::vector<int64_t>& ep_ints,
                                  const std::vector<Tensor>& ep, const Tensor& status_t, bool need_ln, bool need_router) {
  c10::cuda::CUDAGuard guard(dy.device());
  Phase ph("moe.backward");
  OptTensor status = status_t;
  Tensor st = status_t;
  const bool is_ep = !ep.empty();
  const Tensor &rstd = state[2], &xn = state[3], &wts = state[4], &idx = state[5], &ys = state[6], &p_offs = state[7], &dest_row = state[8],
               &src_slot = state[9], &meta_c = state[10], &rr = state[11], &rp = state[12], &te = state[13], &xg = state[14], &g = state[15],
               &u = state[16], &h = state[17], &expert_sorted = state[18], &offs = state[19];
  const int64_t H = x.size(1), El = w1.size(0), F = w1.size(1);
  RowsHint rows_hint(is_ep ? x.size(0) * top_k : 0);
  Tensor dyc = dy.contiguous();
  Tensor d_rows = gather_rows(dyc, src_slot, p_offs, E, wts.view({-1}), top_k);
  Tensor dwts = combine_wgrad(ys, dest_row, dyc, top_k);
  Tensor dyg;
  int64_t cap;
  OptTensor w0, w1o, s0, s1, s2, s3;
  const int64_t n_slots = dest_row.numel();
  if (!is_ep) {
    dyg = d_rows; cap = src_slot.numel();
  } else {
    const int64_t my_base = ep_ints[0], dpar = ep_ints[4];
    MdtEpLayout L = to_layout(layout);
    ep_dispatch(d_rows, ep[6].narrow(0, 0, n_slots), expert_sorted, NONE, meta_c, ep[0], layout, ep_ints[1], 1, dpar, status);
    ep_recv_prepare(my_base, layout, meta_c, H, dpar, st, false);
    dyg = ep[4]; cap = L.capacity_rows;
    w0 = ep[3]; w1o = te; s0 = rr; s1 = rp; s2 = ep[1]; s3 = ep[2];
  }
  const int64_t R = dyg.size(0);
  Tensor dh = torch::empty({R, F}, x.options());
  ggemm(1, dyg, false, w2, false, dh, R, F, H, El, offs, cap, NONE, NONE, NONE, false, 0, NONE, NONE, false, 1.0, status, w0, w1o, NONE, NONE, NONE, NONE);
  if (!wg.empty()) { Tensor c = wg[1]; ggemm(2, h, true, dyg, true, c, F, H, 0, El, offs, cap, NONE, NONE, NONE, false, 0, NONE, NONE, true, wscale, status, NONE, NONE, NONE, NONE, NONE, NONE); }
  auto gu = swiglu_bwd(g, u, dh, offs);
  Tensor dxg = torch::empty({R, H}, x.options());
  ggemm(1, gu[0], false, w1, true, dxg, R, H, F, El, offs, cap, NONE, gu[1], w3, true, F, NONE, NONE, false, 1.0, status, NONE, NONE, s0, s1, s2, s3);
  if (!wg.empty()) {
    Tensor c1 = wg[0], c3 = wg[2];
    ggemm(2, gu[0], true, xg, true, c1, F, H, 0, El, offs, cap, NONE, NONE, NONE, false, 0, NONE, NONE, true, wscale, status, NONE, NONE, NONE, NONE, NONE, NONE);
    ggemm(2, gu[1], true, xg, true, c3, F, H, 0, El, offs, cap, NONE, NONE, NONE, false, 0, NONE, NONE, true, wscale, status, NONE, NONE, NONE, NONE, NONE, NONE);
  }
  Tensor back;
  if (!is_ep) {
    back = dxg;
  } else {
    ep_wait_rows(ep_ints[0], layout, meta_c, ep_ints[4], st, ep_ints[5]);
    back = ep[5].narrow(0, 0, n_slots);
  }
  Tensor dxn = combine_rows(back, dest_row, NONE, top_k);
  auto rb = router_bwd(xn, Wr, idx, dwts, NONE, true, dxn);     // adds the router's input gradient to dxn
  auto nb = rmsnorm_bwd(x, ln_w, dxn, rstd, dyc);               // + dy: the residual connection's gradient
  Tensor dx = nb[0];
  Tensor none = torch::empty({0}, x.options());
  return {dx, need_ln ? rmsnorm_dw(nb[1], ln_w) : none, need_router ? rb[1].to(Wr.scalar_type()) : none};
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, py::arg("mode"), py::arg("A"), py::arg("a_mn"), py::arg("B"), py::arg("b_mn"), py::arg("C"), py::arg("M"), py::arg("N"), py::arg("K"),
        py::arg("G"), py::arg("offsets"), py::arg("capacity_rows"), py::arg("B2"), py::arg("A_l"), py::arg("a_mn_l"), py::arg("B_l"), py::arg("B2_l"),
        py::arg("b_mn_l"), py::arg("K_l"), py::arg("C2"), py::arg("C3"), py::arg("accumulate"), py::arg("alpha"), py::arg("status"), py::arg("tile_ready"),
        py::arg("tile_expected"), py::arg("row_dest_rank"), py::arg("row_dest_row"), py::arg("peer_out"), py::arg("peer_arrive"),
        py::arg("residual") = py::none());
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("x"), py::arg("w"), py::arg("dy"), py::arg("rstd"), py::arg("dres") = py::none());
  m.def("rmsnorm_dw", &rmsnorm_dw);
  m.def("rope", &rope);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd, py::arg("g"), py::arg("u"), py::arg("dh"), py::arg("offsets") = py::none());
  m.def("embedding", &embedding);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("cross_entropy", &cross_entropy);
  m.def("gemm_set_pair_policy", [](int64_t policy) { return (int64_t)mdt_gemm_set_pair_policy((int)policy); });
  m.def("gemm_set_pair_cap", [](int64_t n) { mdt_gemm_set_pair_cap((int)n); });
  m.def("gemm_set_split", [](int64_t on) { return (int64_t)mdt_gemm_set_split((int)on); });
  m.def("gemm_choose_tiling", [](int64_t mode, int64_t M, int64_t N, int64_t K, int64_t K_l, int64_t G, int64_t capacity_rows, bool dual,
                                 bool c_fp32, bool accumulate, bool has_offsets, int64_t policy, int64_t rows_hint, int64_t num_sms) {
    MdtGemmDesc d;
    memset(&d, 0, sizeof(d));
    static const int dummy_offsets = 0;
    d.mode = (int)mode; d.M = (int)M; d.N = (int)N; d.K = (int)K; d.K_l = (int)K_l; d.G = (int)G; d.capacity_rows = capacity_rows;
    d.dual = dual; d.c_fp32 = c_fp32; d.accumulate = accumulate; d.offsets = has_offsets ? &dummy_offsets : nullptr;
    return (int64_t)mdt_gemm_choose_tiling(&d, (int)policy, rows_hint, (int)num_sms);
  });
  m.def("gemm_rows_hint", [](int64_t rows) { mdt_gemm_rows_hint((long long)rows); });
  m.def("gemm_max_pairs", []() { return (int64_t)mdt_gemm_max_pairs(); });
  m.def("skinny_mm", &skinny_mm);
  m.def("adamw", &adamw);
  m.def("multi_add", &multi_add);
  m.def("sumsq", &sumsq);
  m.def("axpby", &axpby);
  m.def("router_fwd", &router_fwd, py::arg("x"), py::arg("w"), py::arg("top_k"), py::arg("normalize"), py::arg("with_stats") = false);
  m.def("router_bwd", &router_bwd, py::arg("x"), py::arg("w"), py::arg("idx"), py::arg("dweights"), py::arg("dscores"), py::arg("normalize"),
        py::arg("dx_accum") = py::none());
  m.def("make_plan", &make_plan);
  m.def("gather_rows", &gather_rows);
  m.def("combine_rows", &combine_rows, py::arg("y"), py::arg("dest_row"), py::arg("weights"), py::arg("top_k"), py::arg("residual") = py::none());
  m.def("combine_wgrad", &combine_wgrad);
  m.def("attention_fwd", &attention_fwd);
  m.def("attention_bwd", &attention_bwd);
  m.def("ep_counts_send", &ep_counts_send);
  m.def("ep_counts_wait_meta", &ep_counts_wait_meta);
  m.def("ep_dispatch", &ep_dispatch, py::arg("x"), py::arg("src_slot"), py::arg("expert_of_slot"), py::arg("slot_scale"), py::arg("meta"),
        py::arg("peer_base"), py::arg("layout"), py::arg("rank"), py::arg("top_k"), py::arg("parity"), py::arg("status") = py::none());
  m.def("ep_recv_prepare", &ep_recv_prepare);
  m.def("ep_combine_send", &ep_combine_send, py::arg("y"), py::arg("meta"), py::arg("peer_base"), py::arg("layout"), py::arg("rank"),
        py::arg("max_rows"), py::arg("parity"), py::arg("status") = py::none());
  m.def("ep_wait_rows", &ep_wait_rows);
  m.def("ep_fused_meta", &ep_fused_meta);
  m.def("ep_meta_offsets", &ep_meta_offsets);
  m.def("ag_pull", &ag_pull, py::arg("out"), py::arg("peer_shard"), py::arg("ws"), py::arg("rank"), py::arg("bytes_per_rank"), py::arg("max_ctas") = 0);
  m.def("ag_pull_flagged", &ag_pull_flagged, py::arg("out"), py::arg("peer_shard"), py::arg("ws"), py::arg("rank"), py::arg("bytes_per_rank"),
        py::arg("ready"), py::arg("epoch"), py::arg("priority_chunks") = 0, py::arg("max_ctas") = 0);
  m.def("ag_chunks", &ag_chunks);
  m.def("ag_wait_chunks", &ag_wait_chunks);
  m.def("gather_registry_clear", &gather_registry_clear);
  m.def("rs_block", &rs_block, py::arg("out"), py::arg("peer_full"), py::arg("peer_flags"), py::arg("my_flags"), py::arg("flag_index"), py::arg("ws"),
        py::arg("rank"), py::arg("in_fp32"), py::arg("scale"), py::arg("accumulate"), py::arg("epoch"), py::arg("status"), py::arg("max_ctas") = 0,
        py::arg("all_reduce") = false);
  m.def("set_peer_wait_limit_ms", [](int64_t ms) { mdt_set_peer_wait_limit_ms((long long)ms); });
  m.def("rs_pull", &rs_pull);
  m.def("barrier_arrive", &barrier_arrive);
  m.def("barrier_wait", &barrier_wait);
  m.def("attention_block_fwd", &attention_block_fwd);
  m.def("attention_block_bwd", &attention_block_bwd);
  m.def("moe_block_fwd", &moe_block_fwd);
  m.def("moe_block_bwd", &moe_block_bwd);
  m.def("launch_count", &launch_count);
}
