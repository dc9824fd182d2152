// Python bindings: torch tensors in, C launch interface (api.h) out.  No math happens here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

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

// C = alpha * op(A) op(B) (+ LoRA segment) with the options of MdtGemmDesc; see csrc/api.h
void gemm(int64_t mode, const Tensor& A, bool a_mn, const Tensor& B, bool b_mn, Tensor& C, int64_t M, int64_t N, int64_t K,
          int64_t G, const OptTensor& offsets, int64_t capacity_rows, const OptTensor& B2, const OptTensor& A_l,
          bool a_mn_l, const OptTensor& B_l, const OptTensor& B2_l, bool b_mn_l, int64_t K_l, const OptTensor& C2,
          const OptTensor& C3, bool accumulate, double alpha, const OptTensor& status, const OptTensor& tile_ready,
          const OptTensor& tile_expected, const OptTensor& row_dest_rank, const OptTensor& row_dest_row, const OptTensor& peer_out,
          const OptTensor& peer_arrive) {
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
std::vector<Tensor> rmsnorm_bwd(const Tensor& x, const Tensor& w, const Tensor& dy, const Tensor& rstd) {
  c10::cuda::CUDAGuard guard(x.device());
  auto x2 = x.reshape({-1, x.size(-1)}).contiguous();
  auto dy2 = dy.reshape({-1, x.size(-1)}).contiguous();
  auto dx = torch::empty_like(x2);
  const int rows = (int)x2.size(0), cols = (int)x2.size(1);
  const int np = rows < 148 ? (rows < 1 ? 1 : rows) : 148;
  auto dwp = torch::empty({np, cols}, x.options().dtype(at::kFloat));
  check(mdt_rmsnorm_bwd(x2.data_ptr(), w.data_ptr(), dy2.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(), dwp.data_ptr<float>(), rows, cols, np, cur_stream()), "rmsnorm_bwd");
  return {dx.view(x.sizes()), dwp};
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
std::vector<Tensor> swiglu_bwd(const Tensor& g, const Tensor& u, const Tensor& dh) {
  c10::cuda::CUDAGuard guard(g.device());
  auto dg = torch::empty_like(g), du = torch::empty_like(u);
  check(mdt_swiglu_bwd(g.data_ptr(), u.data_ptr(), dh.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(), cur_stream()), "swiglu_bwd");
  return {dg, du};
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

std::vector<Tensor> router_fwd(const Tensor& x, const Tensor& w, int64_t top_k, bool normalize) {
  CHECK_BF16(x); CHECK_BF16(w);
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous());
  const int T = (int)x.size(0), H = (int)x.size(1), E = (int)w.size(0);
  auto scores = torch::empty({T, E}, x.options());
  auto weights = torch::empty({T, top_k}, x.options());
  auto idx = torch::empty({T, top_k}, x.options().dtype(at::kInt));
  check(mdt_router_fwd(x.data_ptr(), w.data_ptr(), scores.data_ptr(), weights.data_ptr(), idx.data_ptr<int>(), T, H, E, (int)top_k, normalize, cur_stream()), "router_fwd");
  return {scores, weights, idx};
}
std::vector<Tensor> router_bwd(const Tensor& x, const Tensor& w, const Tensor& idx, const Tensor& dweights, const OptTensor& dscores,
                               bool normalize) {
  c10::cuda::CUDAGuard guard(x.device());
  const int T = (int)x.size(0), H = (int)x.size(1), E = (int)w.size(0), k = (int)idx.size(1);
  auto dx = torch::empty_like(x);
  auto buf = torch::zeros({(int64_t)E * H + (int64_t)T * E}, x.options().dtype(at::kFloat));
  auto dwc = dweights.contiguous();
  OptTensor dsc = dscores.has_value() ? OptTensor(dscores->contiguous()) : std::nullopt;
  check(mdt_router_bwd(x.data_ptr(), w.data_ptr(), nullptr, nullptr, idx.data_ptr<int>(), dwc.data_ptr(), cptr(dsc), dx.data_ptr(),
                       buf.data_ptr<float>(), T, H, E, k, normalize, 0, cur_stream()), "router_bwd");
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
Tensor combine_rows(const Tensor& y, const Tensor& dest_row, const OptTensor& weights, int64_t top_k) {
  CHECK_BF16(y);
  c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(y.is_contiguous());
  const int T = (int)(dest_row.numel() / top_k);
  auto out = torch::empty({T, y.size(1)}, y.options());
  check(mdt_combine_rows(y.data_ptr(), dest_row.data_ptr<int>(), cptr(weights), out.data_ptr(), T, (int)y.size(1), (int)top_k, cur_stream()), "combine_rows");
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
                 const Tensor& peer_base, std::vector<int64_t> layout, int64_t top_k, int64_t parity) {
  CHECK_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && expert_of_slot.scalar_type() == at::kInt && expert_of_slot.is_contiguous());
  check(mdt_ep_dispatch(x.data_ptr(), src_slot.data_ptr<int>(), expert_of_slot.data_ptr<int>(), cptr(slot_scale), meta.data_ptr<int>(), ptrs(peer_base),
                        to_layout(layout), (int)expert_of_slot.numel(), (int)top_k, (int)x.size(1), (int)parity, cur_stream()), "ep_dispatch");
}
void ep_recv_prepare(int64_t my_base, std::vector<int64_t> layout, const Tensor& meta, int64_t cols, int64_t parity, Tensor& status, bool wait_all) {
  c10::cuda::CUDAGuard guard(meta.device());
  check(mdt_ep_recv_prepare(my_base, to_layout(layout), meta.data_ptr<int>(), (int)cols, (int)parity, wait_all, status.data_ptr<int>(), cur_stream()), "ep_recv_prepare");
}
void ep_combine_send(const Tensor& y, const Tensor& meta, const Tensor& peer_base, std::vector<int64_t> layout, int64_t rank, int64_t max_rows, int64_t parity) {
  CHECK_BF16(y);
  c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(y.is_contiguous());
  check(mdt_ep_combine_send(y.data_ptr(), meta.data_ptr<int>(), ptrs(peer_base), to_layout(layout), (int)rank, (int)max_rows, (int)y.size(1), (int)parity, cur_stream()), "ep_combine_send");
}
void ep_wait_rows(int64_t my_base, std::vector<int64_t> layout, const Tensor& meta, int64_t parity, Tensor& status, int64_t mult) {
  c10::cuda::CUDAGuard guard(meta.device());
  check(mdt_ep_wait_rows(my_base, to_layout(layout), meta.data_ptr<int>(), (int)parity, (int)mult, status.data_ptr<int>(), cur_stream()), "ep_wait_rows");
}
// row_rank / row_pos [capacity_rows] and tile_expected [capacity_rows / 128] of this rank's receive layout
std::vector<Tensor> ep_fused_meta(const Tensor& meta, std::vector<int64_t> layout, int64_t rank) {
  c10::cuda::CUDAGuard guard(meta.device());
  MdtEpLayout L = to_layout(layout);
  auto rr = torch::full({L.capacity_rows}, -1, meta.options());
  auto rp = torch::full({L.capacity_rows}, -1, meta.options());
  auto te = torch::zeros({L.capacity_rows / 128}, meta.options());
  check(mdt_ep_fused_meta(meta.data_ptr<int>(), L, (int)rank, rr.data_ptr<int>(), rp.data_ptr<int>(), te.data_ptr<int>(), cur_stream()), "ep_fused_meta");
  return {rr, rp, te};
}
std::vector<int64_t> ep_meta_offsets(int64_t ws, int64_t E) {
  return {mdt_ep_meta_counts(ws, E), mdt_ep_meta_recv_tot(ws, E), mdt_ep_meta_recv_off(ws, E), mdt_ep_meta_dst_row(ws, E),
          mdt_ep_meta_send_start(ws, E), mdt_ep_meta_seg_row(ws, E), mdt_ep_meta_seg_pos(ws, E), mdt_ep_meta_scalars(ws, E), mdt_ep_meta_size(ws, E)};
}
void ag_pull(Tensor& out, const Tensor& peer_shard, int64_t ws, int64_t bytes_per_rank) {
  c10::cuda::CUDAGuard guard(out.device());
  check(mdt_ag_pull(out.data_ptr(), ptrs(peer_shard), (int)ws, bytes_per_rank, cur_stream()), "ag_pull");
}
void rs_pull(Tensor& out, const Tensor& peer_full, int64_t ws, int64_t rank, bool in_fp32, double scale, bool accumulate) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_contiguous());
  check(mdt_rs_pull(out.data_ptr(), ptrs(peer_full), (int)ws, (int)rank, out.numel(), in_fp32, out.scalar_type() == at::kFloat, (float)scale, accumulate, cur_stream()), "rs_pull");
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
  return mdt_gemm_launch_count() + mdt_elementwise_launch_count() + mdt_router_launch_count() + mdt_attention_launch_count() + mdt_comm_launch_count();
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope", &rope);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("embedding", &embedding);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("cross_entropy", &cross_entropy);
  m.def("adamw", &adamw);
  m.def("sumsq", &sumsq);
  m.def("axpby", &axpby);
  m.def("router_fwd", &router_fwd);
  m.def("router_bwd", &router_bwd);
  m.def("make_plan", &make_plan);
  m.def("gather_rows", &gather_rows);
  m.def("combine_rows", &combine_rows);
  m.def("combine_wgrad", &combine_wgrad);
  m.def("attention_fwd", &attention_fwd);
  m.def("attention_bwd", &attention_bwd);
  m.def("ep_counts_send", &ep_counts_send);
  m.def("ep_counts_wait_meta", &ep_counts_wait_meta);
  m.def("ep_dispatch", &ep_dispatch);
  m.def("ep_recv_prepare", &ep_recv_prepare);
  m.def("ep_combine_send", &ep_combine_send);
  m.def("ep_wait_rows", &ep_wait_rows);
  m.def("ep_fused_meta", &ep_fused_meta);
  m.def("ep_meta_offsets", &ep_meta_offsets);
  m.def("ag_pull", &ag_pull);
  m.def("rs_pull", &rs_pull);
  m.def("barrier_arrive", &barrier_arrive);
  m.def("barrier_wait", &barrier_wait);
  m.def("launch_count", &launch_count);
}
