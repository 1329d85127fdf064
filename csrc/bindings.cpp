// Python bindings: thin adapters from torch tensors to the C entry points. They run on the
// current CUDA stream of the tensor's device, never allocate on the hot path except where a
// result tensor is returned, and raise with the library's own error text.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>

#include "attention/attention.h"
#include "common/host.h"
#include "elementwise/elementwise.h"
#include "fused/cp_comm.h"
#include "fused/dp_zero.h"
#include "fused/ep_comm.h"
#include "fused/ep_var.h"
#include "fused/tp_comm.h"
#include "gemm/gemm.h"
#include "runtime/symm.h"

namespace {

void check(int rc, const char* what) {
  if (rc != 0) {
    TORCH_CHECK(false, what, " failed (", rc, "): ", pico_last_error());
  }
}

cudaStream_t stream_of(const at::Tensor& t) {
  return at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}

const void* cptr(const c10::optional<at::Tensor>& t) {
  return t.has_value() && t->defined() ? t->data_ptr() : nullptr;
}
void* mptr(const c10::optional<at::Tensor>& t) {
  return t.has_value() && t->defined() ? t->data_ptr() : nullptr;
}

// D = op(A) op(B) with explicit geometry so that views (row slices, transposes expressed
// through the *_mn_major flags, column slices through ld) need no copies.
void gemm(const at::Tensor& A, const at::Tensor& B, at::Tensor& D, int64_t M, int64_t N, int64_t K,
          int64_t lda, int64_t ldb, int64_t ldd, bool a_mn_major, bool b_mn_major, int64_t out_mode,
          int64_t max_ctas) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && D.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16,
              "gemm: bf16 operands required");
  TORCH_CHECK((out_mode == 0) == (D.scalar_type() == at::kBFloat16), "gemm: output dtype/mode mismatch");
  c10::cuda::CUDAGuard guard(A.device());
  check(pico_gemm_bf16(A.data_ptr(), B.data_ptr(), D.data_ptr(), (int)M, (int)N, (int)K, (int)lda,
                       (int)ldb, (int)ldd, a_mn_major, b_mn_major, (int)out_mode, (int)max_ctas,
                       stream_of(A)),
        "gemm");
}

void rmsnorm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& residual, const at::Tensor& w,
                 at::Tensor& y, const c10::optional<at::Tensor>& h_out,
                 const c10::optional<at::Tensor>& rstd, int64_t rows, int64_t H, double eps) {
  c10::cuda::CUDAGuard guard(x.device());
  check(pico_rmsnorm_fwd(x.data_ptr(), cptr(residual), w.data_ptr(), y.data_ptr(), mptr(h_out),
                         (float*)mptr(rstd), (int)rows, (int)H, (float)eps, stream_of(x)),
        "rmsnorm_fwd");
}

int64_t rmsnorm_bwd_num_partials() { return pico_rmsnorm_bwd_num_partials(); }

void rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& h, const at::Tensor& w, const at::Tensor& rstd,
                 const c10::optional<at::Tensor>& dres, at::Tensor& dh, at::Tensor& dw_partial,
                 const c10::optional<at::Tensor>& dw_f32, const c10::optional<at::Tensor>& dw_bf16,
                 bool accumulate, int64_t rows, int64_t H) {
  c10::cuda::CUDAGuard guard(dy.device());
  TORCH_CHECK(dw_partial.numel() >= pico_rmsnorm_bwd_num_partials() * H, "rmsnorm_bwd: scratch too small");
  check(pico_rmsnorm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), (const float*)rstd.data_ptr(),
                         cptr(dres), dh.data_ptr(), (float*)dw_partial.data_ptr(),
                         (float*)mptr(dw_f32), mptr(dw_bf16), accumulate, (int)rows, (int)H,
                         stream_of(dy)),
        "rmsnorm_bwd");
}

void rope_inplace(at::Tensor& x, int64_t row_stride, int64_t rows, int64_t seq, int64_t pos_offset,
                  int64_t nheads, int64_t d, const at::Tensor& cos, const at::Tensor& sin, int64_t sign) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat, "rope: fp32 tables");
  TORCH_CHECK(pos_offset + seq <= cos.size(0), "rope: position table too short");
  check(pico_rope_inplace(x.data_ptr(), row_stride, (int)rows, (int)seq, (int)pos_offset, (int)nheads,
                          (int)d, (const float*)cos.data_ptr(), (const float*)sin.data_ptr(),
                          (int)sign, stream_of(x)),
        "rope");
}

static const int* rows_dev_ptr(const c10::optional<at::Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->numel() >= 1, "row count: int32 CUDA tensor");
  return t->data_ptr<int>();
}
void swiglu_fwd(const at::Tensor& gu, int64_t ld_gu, at::Tensor& y, int64_t rows, int64_t I,
                const c10::optional<at::Tensor>& rows_dev) {
  c10::cuda::CUDAGuard guard(gu.device());
  check(pico_swiglu_fwd(gu.data_ptr(), ld_gu, y.data_ptr(), (int)rows, (int)I, rows_dev_ptr(rows_dev), stream_of(gu)),
        "swiglu_fwd");
}
void swiglu_bwd(const at::Tensor& dy, const at::Tensor& gu, int64_t ld_gu, at::Tensor& dgu,
                int64_t ld_dgu, int64_t rows, int64_t I, const c10::optional<at::Tensor>& rows_dev) {
  c10::cuda::CUDAGuard guard(gu.device());
  check(pico_swiglu_bwd(dy.data_ptr(), gu.data_ptr(), ld_gu, dgu.data_ptr(), ld_dgu, (int)rows, (int)I,
                        rows_dev_ptr(rows_dev), stream_of(gu)),
        "swiglu_bwd");
}

void ce_stats(const at::Tensor& logits, int64_t ldl, const at::Tensor& targets, at::Tensor& stats,
              int64_t rows, int64_t V, int64_t vocab_start) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(targets.scalar_type() == at::kLong && stats.scalar_type() == at::kFloat, "ce: dtypes");
  check(pico_ce_stats(logits.data_ptr(), ldl, (const int64_t*)targets.data_ptr(),
                      (float*)stats.data_ptr(), (int)rows, (int)V, (int)vocab_start, stream_of(logits)),
        "ce_stats");
}
void ce_loss_grad(const at::Tensor& logits, int64_t ldl, const at::Tensor& targets,
                  const at::Tensor& stats, const c10::optional<at::Tensor>& loss,
                  const c10::optional<at::Tensor>& dlogits, int64_t ldd, double grad_scale,
                  int64_t rows, int64_t V, int64_t vocab_start) {
  c10::cuda::CUDAGuard guard(logits.device());
  check(pico_ce_loss_grad(logits.data_ptr(), ldl, (const int64_t*)targets.data_ptr(),
                          (const float*)stats.data_ptr(), (float*)mptr(loss), mptr(dlogits), ldd,
                          (float)grad_scale, (int)rows, (int)V, (int)vocab_start, stream_of(logits)),
        "ce_loss_grad");
}

void adamw(const c10::optional<at::Tensor>& p, const c10::optional<at::Tensor>& master, at::Tensor& g,
           at::Tensor& m, at::Tensor& v, int64_t n, double lr, double beta1, double beta2, double eps,
           double wd, double bc1, double bc2, double grad_scale, bool zero_grad) {
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat &&
                  v.scalar_type() == at::kFloat, "adamw: fp32 grads and states");
  check(pico_adamw(mptr(p), (float*)mptr(master), (float*)g.data_ptr(), (float*)m.data_ptr(),
                   (float*)v.data_ptr(), n, (float)lr, (float)beta1, (float)beta2, (float)eps,
                   (float)wd, (float)bc1, (float)bc2, (float)grad_scale, zero_grad, stream_of(g)),
        "adamw");
}

void embedding_fwd(const at::Tensor& W, const at::Tensor& ids, at::Tensor& out, int64_t rows, int64_t H,
                   int64_t Vlocal, int64_t vocab_start) {
  c10::cuda::CUDAGuard guard(W.device());
  TORCH_CHECK(ids.scalar_type() == at::kLong, "embedding: int64 ids");
  check(pico_embedding_fwd(W.data_ptr(), (const int64_t*)ids.data_ptr(), out.data_ptr(), (int)rows,
                           (int)H, (int)Vlocal, (int)vocab_start, stream_of(W)),
        "embedding_fwd");
}
void embedding_bwd(const at::Tensor& dout, const at::Tensor& ids, at::Tensor& dW, int64_t rows, int64_t H,
                   int64_t Vlocal, int64_t vocab_start) {
  c10::cuda::CUDAGuard guard(dout.device());
  TORCH_CHECK(dW.scalar_type() == at::kFloat, "embedding_bwd: fp32 accumulator");
  check(pico_embedding_bwd(dout.data_ptr(), (const int64_t*)ids.data_ptr(), (float*)dW.data_ptr(),
                           (int)rows, (int)H, (int)Vlocal, (int)vocab_start, stream_of(dout)),
        "embedding_bwd");
}

void accumulate_bf16_into_f32(const at::Tensor& src, at::Tensor& dst, int64_t n) {
  c10::cuda::CUDAGuard guard(src.device());
  check(pico_accumulate_bf16_into_f32(src.data_ptr(), (float*)dst.data_ptr(), n, stream_of(src)),
        "accumulate");
}

void moe_route(const at::Tensor& logits, const c10::optional<at::Tensor>& bias, at::Tensor& probs, at::Tensor& idx,
               at::Tensor& w, at::Tensor& counts, int64_t k, bool renorm) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.scalar_type() == at::kBFloat16 && logits.stride(1) == 1, "moe_route: bf16 [T, E] logits");
  const int64_t T = logits.size(0), E = logits.size(1);
  TORCH_CHECK(probs.scalar_type() == at::kFloat && probs.is_contiguous() && probs.numel() == T * E &&
                  idx.scalar_type() == at::kInt && idx.is_contiguous() && idx.numel() == T * k &&
                  w.scalar_type() == at::kFloat && w.is_contiguous() && w.numel() == T * k &&
                  counts.scalar_type() == at::kInt && counts.numel() == E &&
                  (!bias.has_value() || !bias->defined() || (bias->scalar_type() == at::kFloat && bias->numel() == E)),
              "moe_route: output / bias tensors of the wrong type or size");
  check(pico_moe_route(logits.data_ptr(), logits.stride(0), (const float*)cptr(bias), (float*)probs.data_ptr(),
                       idx.data_ptr<int>(), (float*)w.data_ptr(), counts.data_ptr<int>(), (int)T, (int)E, (int)k,
                       renorm ? 1 : 0, stream_of(logits)),
        "moe_route");
}

void moe_route_bwd(const at::Tensor& probs, const at::Tensor& idx, const at::Tensor& w, const at::Tensor& dw,
                   const c10::optional<at::Tensor>& dprobs, at::Tensor& dlogits, int64_t k, bool renorm) {
  c10::cuda::CUDAGuard guard(probs.device());
  const int64_t T = probs.size(0), E = probs.size(1);
  TORCH_CHECK(probs.is_contiguous() && probs.scalar_type() == at::kFloat && dw.scalar_type() == at::kFloat &&
                  dw.is_contiguous() && dw.numel() == T * k && dlogits.scalar_type() == at::kFloat &&
                  dlogits.is_contiguous() && dlogits.numel() == T * E && idx.scalar_type() == at::kInt &&
                  w.scalar_type() == at::kFloat &&
                  (!dprobs.has_value() || !dprobs->defined() ||
                   (dprobs->scalar_type() == at::kFloat && dprobs->is_contiguous() && dprobs->numel() == T * E)),
              "moe_route_bwd: fp32 contiguous tensors of matching sizes");
  check(pico_moe_route_bwd((const float*)probs.data_ptr(), idx.data_ptr<int>(), (const float*)w.data_ptr(),
                           (const float*)dw.data_ptr(), (const float*)cptr(dprobs), (float*)dlogits.data_ptr(), (int)T,
                           (int)E, (int)k, renorm ? 1 : 0, stream_of(probs)),
        "moe_route_bwd");
}

void moe_slots(const at::Tensor& idx, int64_t E, int64_t C, at::Tensor& pos, const c10::optional<at::Tensor>& row_of_slot) {
  c10::cuda::CUDAGuard guard(idx.device());
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.is_contiguous() && pos.scalar_type() == at::kInt &&
                  pos.is_contiguous() && pos.numel() == idx.numel() &&
                  (!row_of_slot.has_value() || !row_of_slot->defined() ||
                   (row_of_slot->scalar_type() == at::kInt && row_of_slot->is_contiguous() && row_of_slot->numel() >= E * C)),
              "moe_slots: int32 contiguous tensors");
  check(pico_moe_slots(idx.data_ptr<int>(), (int)idx.numel(), (int)E, (int)C, pos.data_ptr<int>(),
                       row_of_slot.has_value() && row_of_slot->defined() ? row_of_slot->data_ptr<int>() : nullptr,
                       stream_of(idx)),
        "moe_slots");
}

void moe_combine(const at::Tensor& out, const at::Tensor& idx, const at::Tensor& pos, const at::Tensor& w, at::Tensor& y,
                 int64_t k, int64_t C) {
  c10::cuda::CUDAGuard guard(out.device());
  const int64_t T = y.size(0), d = y.size(1);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.size(-1) == d &&
                  y.scalar_type() == at::kBFloat16 && y.is_contiguous() && idx.scalar_type() == at::kInt &&
                  pos.scalar_type() == at::kInt && w.scalar_type() == at::kFloat && idx.numel() == T * k &&
                  pos.numel() == T * k && w.numel() == T * k && idx.is_contiguous() && pos.is_contiguous() &&
                  w.is_contiguous(),
              "moe_combine: tensors of the wrong type or size");
  check(pico_moe_combine(out.data_ptr(), idx.data_ptr<int>(), pos.data_ptr<int>(), (const float*)w.data_ptr(),
                         y.data_ptr(), (int)T, (int)k, (int)C, (int)d, stream_of(out)),
        "moe_combine");
}

void moe_combine_bwd(const at::Tensor& dy, const at::Tensor& out, const at::Tensor& row_of_slot, const at::Tensor& w,
                     at::Tensor& dout, at::Tensor& dw, int64_t k) {
  c10::cuda::CUDAGuard guard(out.device());
  const int64_t slots = out.numel() / out.size(-1), d = out.size(-1);
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && dy.size(-1) == d &&
                  out.scalar_type() == at::kBFloat16 && out.is_contiguous() && dout.scalar_type() == at::kBFloat16 &&
                  dout.is_contiguous() && dout.numel() == out.numel() && row_of_slot.scalar_type() == at::kInt &&
                  row_of_slot.is_contiguous() && row_of_slot.numel() >= slots && w.scalar_type() == at::kFloat &&
                  dw.scalar_type() == at::kFloat && w.is_contiguous() && dw.is_contiguous() && dw.numel() == w.numel(),
              "moe_combine_bwd: tensors of the wrong type or size");
  check(pico_moe_combine_bwd(dy.data_ptr(), out.data_ptr(), row_of_slot.data_ptr<int>(), (const float*)w.data_ptr(),
                             dout.data_ptr(), (float*)dw.data_ptr(), slots, (int)k, (int)d, stream_of(out)),
        "moe_combine_bwd");
}

void attn_merge(const at::Tensor& out_a, const at::Tensor& lse_a, const at::Tensor& out_b, const at::Tensor& lse_b,
                at::Tensor& out, at::Tensor& lse) {
  c10::cuda::CUDAGuard guard(out_b.device());
  TORCH_CHECK(out_a.dim() == 4 && out_a.sizes() == out_b.sizes() && out.sizes() == out_b.sizes() &&
                  out_a.is_contiguous() && out_b.is_contiguous() && out.is_contiguous() &&
                  out_b.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kFloat &&
                  (out_a.scalar_type() == at::kFloat || out_a.scalar_type() == at::kBFloat16),
              "attn_merge: contiguous [b, s, h, d] tensors (a: fp32 or bf16, b: bf16, result fp32)");
  TORCH_CHECK(lse_a.scalar_type() == at::kFloat && lse_b.scalar_type() == at::kFloat && lse.scalar_type() == at::kFloat &&
                  lse_a.is_contiguous() && lse_b.is_contiguous() && lse.is_contiguous() &&
                  lse_a.numel() == out.size(0) * out.size(1) * out.size(2) && lse_b.numel() == lse_a.numel() &&
                  lse.numel() == lse_a.numel(),
              "attn_merge: fp32 contiguous [b, h, s] log-sum-exp tensors");
  check(pico_attn_merge(out_a.data_ptr(), out_a.scalar_type() == at::kFloat ? 1 : 0, (const float*)lse_a.data_ptr(),
                        out_b.data_ptr(), (const float*)lse_b.data_ptr(), (float*)out.data_ptr(), (float*)lse.data_ptr(),
                        (int)out.size(0), (int)out.size(1), (int)out.size(2), (int)out.size(3), stream_of(out_b)),
        "attn_merge");
}

void scale_unless_one(at::Tensor& x, const at::Tensor& scale) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.is_contiguous() && scale.scalar_type() == at::kFloat &&
                  scale.is_cuda() && scale.numel() == 1, "scale_unless_one: contiguous bf16 tensor, fp32 device scalar");
  check(pico_scale_unless_one(x.data_ptr(), x.numel(), (const float*)scale.data_ptr(), stream_of(x)),
        "scale_unless_one");
}

void fill_u32(at::Tensor& dst, int64_t value, int64_t n_words) {
  c10::cuda::CUDAGuard guard(dst.device());
  check(pico_fill_u32(dst.data_ptr(), (uint32_t)value, n_words, stream_of(dst)), "fill");
}

// ---------------------------------------------------------------------------------------------
// symmetric memory + fused tensor-parallel communication
// ---------------------------------------------------------------------------------------------
PicoPeerTable table_of(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() <= PICO_MAX_PEERS, "at most ", PICO_MAX_PEERS, " peers");
  PicoPeerTable t;
  for (int i = 0; i < PICO_MAX_PEERS; ++i)
    t.ptr[i] = i < (int)ptrs.size() ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return t;
}

std::pair<int64_t, py::bytes> symm_alloc(int64_t nbytes) {
  void* p = nullptr;
  unsigned char h[64];
  check(pico_symm_alloc((size_t)nbytes, &p, h), "symm_alloc");
  return {reinterpret_cast<int64_t>(p), py::bytes(reinterpret_cast<const char*>(h), 64)};
}

int64_t symm_open(const std::string& handle) {
  TORCH_CHECK(handle.size() == 64, "IPC handle must be 64 bytes");
  void* p = nullptr;
  check(pico_symm_open(reinterpret_cast<const unsigned char*>(handle.data()), &p), "symm_open");
  return reinterpret_cast<int64_t>(p);
}

void symm_close(int64_t ptr) { pico_symm_close(reinterpret_cast<void*>(ptr)); }
void symm_free(int64_t ptr) { pico_symm_free(reinterpret_cast<void*>(ptr)); }

// A uint8 tensor over device memory owned elsewhere (no deleter).
at::Tensor tensor_from_ptr(int64_t ptr, int64_t nbytes, int64_t device_index) {
  auto opts = at::TensorOptions().dtype(at::kByte).device(at::kCUDA, (c10::DeviceIndex)device_index);
  return at::from_blob(reinterpret_cast<void*>(ptr), {nbytes}, opts);
}

void signal_peers(const std::vector<int64_t>& flag_ptrs, int64_t world, int64_t my_rank, int64_t slot,
                  int64_t epoch) {
  check(pico_signal_peers(table_of(flag_ptrs), (int)world, (int)my_rank, (int)slot, (uint32_t)epoch,
                          at::cuda::getCurrentCUDAStream().stream()),
        "signal_peers");
}

void wait_flags(int64_t local_flags, int64_t world, int64_t slot, int64_t epoch, int64_t timeout_ms) {
  check(pico_wait_flags(reinterpret_cast<const uint32_t*>(local_flags), (int)world, (int)slot,
                        (uint32_t)epoch, (uint32_t)timeout_ms, at::cuda::getCurrentCUDAStream().stream()),
        "wait_flags");
}

void epoch_base_add(int64_t local_flags, const std::vector<int64_t>& slots, const std::vector<int64_t>& deltas) {
  TORCH_CHECK(slots.size() == deltas.size() && slots.size() <= PICO_MAX_EPOCH_DELTAS, "epoch_base_add: at most ",
              PICO_MAX_EPOCH_DELTAS, " (slot, delta) pairs");
  PicoEpochDeltas d;
  memset(&d, 0, sizeof(d));
  d.n = (int)slots.size();
  for (size_t i = 0; i < slots.size(); ++i) {
    d.slot[i] = (int)slots[i];
    d.delta[i] = (uint32_t)deltas[i];
  }
  check(pico_epoch_base_add(reinterpret_cast<uint32_t*>(local_flags), &d, at::cuda::getCurrentCUDAStream().stream()),
        "epoch_base_add");
}

void push_rows(const at::Tensor& src, const std::vector<int64_t>& dst_ptrs,
               const std::vector<int64_t>& flag_ptrs, int64_t world, int64_t my_rank, int64_t rows,
               int64_t cols, int64_t slot, int64_t epoch, int64_t skip_self, int64_t piece_rows) {
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && src.scalar_type() == at::kBFloat16, "push_rows: contiguous bf16");
  check(pico_push_rows(src.data_ptr(), table_of(dst_ptrs), table_of(flag_ptrs), (int)world, (int)my_rank,
                       (int)rows, (int)cols, (int)piece_rows, (int)slot, (uint32_t)epoch, (int)skip_self,
                       stream_of(src)),
        "push_rows");
}

void slot_sum(const at::Tensor& staging, int64_t world, int64_t rows, int64_t cols,
              const c10::optional<at::Tensor>& addend, at::Tensor& out, int64_t local_flags, int64_t slot,
              int64_t epoch, int64_t timeout_ms) {
  c10::cuda::CUDAGuard guard(out.device());
  check(pico_slot_sum(staging.data_ptr(), (int)world, (int)rows, (int)cols, cptr(addend), out.data_ptr(),
                      reinterpret_cast<const uint32_t*>(local_flags), (int)slot, (uint32_t)epoch,
                      (uint32_t)timeout_ms, stream_of(out)),
        "slot_sum");
}

void slot_sum_from(const at::Tensor& staging, int64_t world, int64_t first_slot, int64_t rows, int64_t cols,
                   const c10::optional<at::Tensor>& addend, at::Tensor& out, int64_t local_flags, int64_t slot,
                   int64_t epoch, int64_t timeout_ms) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_contiguous() && (!addend.has_value() || addend->is_contiguous()), "slot_sum_from: contiguous");
  check(pico_slot_sum_from(staging.data_ptr(), (int)world, (int)first_slot, (int)rows, (int)cols, cptr(addend),
                           out.data_ptr(), reinterpret_cast<const uint32_t*>(local_flags), (int)slot,
                           (uint32_t)epoch, (uint32_t)timeout_ms, stream_of(out)),
        "slot_sum_from");
}

void scatter_rows(const at::Tensor& src, const std::vector<int64_t>& dst_ptrs,
                  const std::vector<int64_t>& flag_ptrs, int64_t world, int64_t my_rank, int64_t num_dst,
                  int64_t rows, int64_t cols, int64_t slot, int64_t epoch, int64_t piece_rows) {
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && src.scalar_type() == at::kBFloat16, "scatter_rows: contiguous bf16");
  TORCH_CHECK(src.numel() >= num_dst * rows * cols, "scatter_rows: source too small");
  check(pico_scatter_rows(src.data_ptr(), table_of(dst_ptrs), table_of(flag_ptrs), (int)world, (int)my_rank,
                          (int)num_dst, (int)rows, (int)cols, (int)piece_rows, (int)slot, (uint32_t)epoch,
                          stream_of(src)),
        "scatter_rows");
}

// Ulysses layout exchanges through peer memory; see fused/cp_comm.h. to_seq: src [b, s_local, world*cols]
// -> peers' [b, world*s_local, cols]; otherwise the inverse.
void a2a_push(const at::Tensor& src, const std::vector<int64_t>& dst_ptrs, const std::vector<int64_t>& flag_ptrs,
              int64_t world, int64_t my_rank, int64_t batch, int64_t s_local, int64_t cols, bool to_seq,
              int64_t slot, int64_t epoch) {
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && src.scalar_type() == at::kBFloat16, "a2a_push: contiguous bf16");
  TORCH_CHECK(src.numel() == batch * s_local * world * cols, "a2a_push: source size mismatch");
  if (to_seq)
    check(pico_a2a_heads_to_seq(src.data_ptr(), table_of(dst_ptrs), table_of(flag_ptrs), (int)world, (int)my_rank,
                                (int)batch, (int)s_local, (int)cols, (int)slot, (uint32_t)epoch, stream_of(src)),
          "a2a_heads_to_seq");
  else
    check(pico_a2a_seq_to_heads(src.data_ptr(), table_of(dst_ptrs), table_of(flag_ptrs), (int)world, (int)my_rank,
                                (int)batch, (int)s_local, (int)cols, (int)slot, (uint32_t)epoch, stream_of(src)),
          "a2a_seq_to_heads");
}

// Dropless expert-parallel exchange with device-side layout; see fused/ep_var.h.
void ep_var_layout(const at::Tensor& counts_table, int64_t ep, int64_t L, int64_t my_rank, int64_t max_rows,
                   at::Tensor& send_blocks, at::Tensor& return_blocks, at::Tensor& seg_start, at::Tensor& seg_len,
                   at::Tensor& tile_group) {
  c10::cuda::CUDAGuard guard(counts_table.device());
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&counts_table, &send_blocks, &return_blocks,
                                                                      &seg_start, &seg_len, &tile_group})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous(), "ep_var_layout: int32 CUDA tensors");
  TORCH_CHECK(counts_table.numel() >= ep * ep * L && send_blocks.numel() >= ep * L * 4 &&
                  return_blocks.numel() >= ep * L * 4 && seg_start.numel() >= L + 1 && seg_len.numel() >= L &&
                  tile_group.numel() >= max_rows / 128,
              "ep_var_layout: array too small");
  check(pico_ep_var_layout(counts_table.data_ptr<int>(), (int)ep, (int)L, (int)my_rank, (int)max_rows,
                           send_blocks.data_ptr<int>(), return_blocks.data_ptr<int>(), seg_start.data_ptr<int>(),
                           seg_len.data_ptr<int>(), tile_group.data_ptr<int>(), stream_of(counts_table)),
        "ep_var_layout");
}

void ep_var_exchange(const at::Tensor& src, const c10::optional<at::Tensor>& row_index, int64_t index_div,
                     const at::Tensor& blocks, int64_t num_blocks, const std::vector<int64_t>& dst_ptrs,
                     const std::vector<int64_t>& scale_ptrs, const std::vector<int64_t>& flag_ptrs, int64_t ep,
                     int64_t my_rank, int64_t d, bool quant, int64_t slot, int64_t epoch) {
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.scalar_type() == at::kBFloat16 && src.is_contiguous() && src.size(-1) == d,
              "ep_var_exchange: contiguous bf16 rows of width d");
  TORCH_CHECK(blocks.scalar_type() == at::kInt && blocks.is_contiguous() && blocks.numel() >= num_blocks * 4,
              "ep_var_exchange: int32 block table");
  const int32_t* idx = nullptr;
  if (row_index.has_value() && row_index->defined()) {
    TORCH_CHECK(row_index->scalar_type() == at::kInt && row_index->is_contiguous(), "ep_var_exchange: int32 row index");
    idx = row_index->data_ptr<int>();
  }
  check(pico_ep_var_exchange(src.data_ptr(), idx, (int)index_div, blocks.data_ptr<int>(), (int)num_blocks,
                             table_of(dst_ptrs), table_of(scale_ptrs), table_of(flag_ptrs), (int)ep, (int)my_rank,
                             (int)d, quant ? 1 : 0, (int)slot, (uint32_t)epoch, stream_of(src)),
        "ep_var_exchange");
}

void ep_var_dequant(const at::Tensor& payload, const at::Tensor& scales, at::Tensor& out, const at::Tensor& rows_in_use,
                    int64_t max_rows, int64_t d) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous() && rows_in_use.scalar_type() == at::kInt,
              "ep_var_dequant: bf16 output, int32 row count");
  check(pico_ep_var_dequant(payload.data_ptr(), (const float*)scales.data_ptr(), out.data_ptr(),
                            rows_in_use.data_ptr<int>(), (int)max_rows, (int)d, stream_of(out)),
        "ep_var_dequant");
}

void ep_var_copy_rows(const at::Tensor& src, at::Tensor& dst, const at::Tensor& rows_in_use, int64_t max_rows, int64_t d) {
  c10::cuda::CUDAGuard guard(dst.device());
  TORCH_CHECK(src.scalar_type() == at::kBFloat16 && dst.scalar_type() == at::kBFloat16 && src.is_contiguous() &&
                  dst.is_contiguous() && src.numel() >= max_rows * d && dst.numel() >= max_rows * d &&
                  rows_in_use.scalar_type() == at::kInt,
              "ep_var_copy_rows: contiguous bf16 [max_rows, d] buffers and an int32 row count");
  check(pico_ep_var_copy_rows(src.data_ptr(), dst.data_ptr(), rows_in_use.data_ptr<int>(), (int)max_rows, (int)d,
                              stream_of(dst)),
        "ep_var_copy_rows");
}

void ep_var_zero_padding(at::Tensor& buf, const at::Tensor& seg_start, const at::Tensor& seg_len, int64_t L, int64_t d) {
  c10::cuda::CUDAGuard guard(buf.device());
  TORCH_CHECK(buf.scalar_type() == at::kBFloat16 && buf.is_contiguous(), "ep_var_zero_padding: contiguous bf16");
  check(pico_ep_var_zero_padding(buf.data_ptr(), seg_start.data_ptr<int>(), seg_len.data_ptr<int>(), (int)L, (int)d,
                                 stream_of(buf)),
        "ep_var_zero_padding");
}

void ce_stats_push(const at::Tensor& logits, int64_t ldl, const at::Tensor& targets, int64_t rows, int64_t V,
                   int64_t vocab_start, const std::vector<int64_t>& dst_ptrs, const std::vector<int64_t>& flag_ptrs,
                   int64_t world, int64_t my_rank, int64_t slot, int64_t epoch) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(targets.scalar_type() == at::kLong && logits.scalar_type() == at::kBFloat16, "ce: dtypes");
  check(pico_ce_stats_push(logits.data_ptr(), ldl, (const int64_t*)targets.data_ptr(), (int)rows, (int)V,
                           (int)vocab_start, table_of(dst_ptrs), table_of(flag_ptrs), (int)world, (int)my_rank,
                           (int)slot, (uint32_t)epoch, stream_of(logits)),
        "ce_stats_push");
}

void ce_loss_grad_gathered(const at::Tensor& logits, int64_t ldl, const at::Tensor& targets,
                           const at::Tensor& gathered, const c10::optional<at::Tensor>& loss,
                           const c10::optional<at::Tensor>& dlogits, int64_t ldd, double grad_scale, int64_t rows,
                           int64_t V, int64_t vocab_start, int64_t local_flags, int64_t world, int64_t slot,
                           int64_t epoch, int64_t timeout_ms) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(gathered.scalar_type() == at::kFloat && gathered.numel() >= world * rows * 3,
              "ce_loss_grad_gathered: fp32 [world, rows, 3] table");
  check(pico_ce_loss_grad_gathered(logits.data_ptr(), ldl, (const int64_t*)targets.data_ptr(),
                                   (const float*)gathered.data_ptr(), (float*)mptr(loss), mptr(dlogits), ldd,
                                   (float)grad_scale, (int)rows, (int)V, (int)vocab_start,
                                   reinterpret_cast<const uint32_t*>(local_flags), (int)world, (int)slot,
                                   (uint32_t)epoch, (uint32_t)timeout_ms, stream_of(logits)),
        "ce_loss_grad_gathered");
}

void zero1_adamw(const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& param_ptrs, at::Tensor& m,
                 at::Tensor& v, const c10::optional<at::Tensor>& master, int64_t shard_start, int64_t shard_len,
                 int64_t world, int64_t my_rank, double lr, double beta1, double beta2, double eps, double wd,
                 double bc1, double bc2, double grad_scale, int64_t local_flags, int64_t ready_slot,
                 int64_t epoch, int64_t timeout_ms) {
  c10::cuda::CUDAGuard guard(m.device());
  TORCH_CHECK(m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat && m.numel() >= shard_len &&
                  v.numel() >= shard_len, "zero1_adamw: fp32 state of the shard's length");
  check(pico_zero1_adamw(table_of(grad_ptrs), table_of(param_ptrs), (float*)m.data_ptr(), (float*)v.data_ptr(),
                         (float*)mptr(master), shard_start, shard_len, (int)world, (int)my_rank, (float)lr,
                         (float)beta1, (float)beta2, (float)eps, (float)wd, (float)bc1, (float)bc2,
                         (float)grad_scale, reinterpret_cast<const uint32_t*>(local_flags), (int)ready_slot,
                         (uint32_t)epoch, (uint32_t)timeout_ms, stream_of(m)),
        "zero1_adamw");
}

void ep_dispatch(const at::Tensor& tokens, const at::Tensor& row_of_slot, int64_t top_k,
                 const std::vector<int64_t>& payload_ptrs, const std::vector<int64_t>& scale_ptrs,
                 const std::vector<int64_t>& flag_ptrs, int64_t ep, int64_t my_rank, int64_t L, int64_t C, int64_t d,
                 bool quant, int64_t slot, int64_t epoch) {
  c10::cuda::CUDAGuard guard(tokens.device());
  TORCH_CHECK(tokens.scalar_type() == at::kBFloat16 && tokens.is_contiguous() && tokens.size(-1) == d,
              "ep_dispatch: contiguous bf16 tokens [T, d]");
  TORCH_CHECK(row_of_slot.scalar_type() == at::kInt && row_of_slot.numel() == ep * L * C, "ep_dispatch: int32 row_of_slot[E*C]");
  check(pico_ep_dispatch(tokens.data_ptr(), (const int32_t*)row_of_slot.data_ptr(), (int)top_k, table_of(payload_ptrs),
                         table_of(scale_ptrs), table_of(flag_ptrs), (int)ep, (int)my_rank, (int)L, (int)C, (int)d,
                         quant, (int)slot, (uint32_t)epoch, stream_of(tokens)),
        "ep_dispatch");
}

void ep_dequant(const at::Tensor& payload, const at::Tensor& scales, at::Tensor& out, int64_t rows, int64_t d,
                int64_t local_flags, int64_t ep, int64_t slot, int64_t epoch, int64_t timeout_ms) {
  c10::cuda::CUDAGuard guard(out.device());
  check(pico_ep_dequant(payload.data_ptr(), (const float*)scales.data_ptr(), out.data_ptr(), rows, (int)d,
                        reinterpret_cast<const uint32_t*>(local_flags), (int)ep, (int)slot, (uint32_t)epoch,
                        (uint32_t)timeout_ms, stream_of(out)),
        "ep_dequant");
}

void ep_block_exchange(const at::Tensor& src, const std::vector<int64_t>& dst_ptrs,
                       const std::vector<int64_t>& flag_ptrs, int64_t ep, int64_t my_rank, int64_t L, int64_t C,
                       int64_t d, bool to_expert_major, int64_t slot, int64_t epoch) {
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.scalar_type() == at::kBFloat16 && src.is_contiguous() && src.numel() == ep * L * C * d,
              "ep_block_exchange: contiguous bf16 [E*C, d]");
  check(pico_ep_block_exchange(src.data_ptr(), table_of(dst_ptrs), table_of(flag_ptrs), (int)ep, (int)my_rank, (int)L,
                               (int)C, (int)d, to_expert_major, (int)slot, (uint32_t)epoch, stream_of(src)),
        "ep_block_exchange");
}

// GEMM with collective fusion; see PicoGemmComm in gemm/gemm.h.
void gemm_ex(const at::Tensor& A, const at::Tensor& B, const c10::optional<at::Tensor>& D, int64_t M,
             int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldd, bool a_mn_major, bool b_mn_major,
             int64_t out_mode, int64_t max_ctas, int64_t a_flags, int64_t a_slot, int64_t a_epoch,
             int64_t a_skip_block, const std::vector<int64_t>& d_ptrs, int64_t blk_rows, int64_t num_blocks,
             int64_t first_block, int64_t timeout_ms) {
  c10::cuda::CUDAGuard guard(A.device());
  PicoGemmComm c;
  memset(&c, 0, sizeof(c));
  c.a_flags = reinterpret_cast<const unsigned int*>(a_flags);
  c.a_slot = (int)a_slot;
  c.a_epoch = (unsigned int)a_epoch;
  c.a_skip_block = (int)a_skip_block;
  c.d_num_dest = (int)d_ptrs.size();
  TORCH_CHECK(d_ptrs.size() <= 8, "gemm_ex: at most 8 destinations");
  for (size_t i = 0; i < d_ptrs.size(); ++i) c.d_ptrs[i] = reinterpret_cast<void*>(d_ptrs[i]);
  c.blk_rows = (int)blk_rows;
  c.num_blocks = (int)num_blocks;
  c.first_block = (int)first_block;
  c.timeout_ms = (unsigned int)timeout_ms;
  void* dptr = D.has_value() && D->defined() ? D->data_ptr() : nullptr;
  TORCH_CHECK(dptr != nullptr || !d_ptrs.empty(), "gemm_ex: no output");
  check(pico_gemm_bf16_ex(A.data_ptr(), B.data_ptr(), dptr, (int)M, (int)N, (int)K, (int)lda, (int)ldb,
                          (int)ldd, a_mn_major, b_mn_major, (int)out_mode, (int)max_ctas, &c, stream_of(A)),
        "gemm_ex");
}

// Grouped GEMM over the local experts; see PicoGemmComm (tile_group / seg_start) in gemm/gemm.h.
// mode 0: row-grouped, `groups` = tile_group [ceil(M/128)] int32; mode 1: reduction-grouped,
// `groups` = seg_start [num_groups + 1] int32.
void gemm_grouped(const at::Tensor& A, const at::Tensor& B, at::Tensor& D, int64_t M, int64_t N, int64_t K,
                  int64_t lda, int64_t ldb, int64_t ldd, bool a_mn_major, bool b_mn_major, int64_t out_mode,
                  int64_t mode, const at::Tensor& groups, int64_t num_groups, int64_t b_group_rows) {
  c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && D.is_cuda() && groups.is_cuda(), "gemm_grouped: CUDA tensors required");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "gemm_grouped: bf16 operands");
  TORCH_CHECK((out_mode == 0) == (D.scalar_type() == at::kBFloat16), "gemm_grouped: output dtype/mode mismatch");
  TORCH_CHECK(groups.scalar_type() == at::kInt && groups.is_contiguous(), "gemm_grouped: int32 group array");
  PicoGemmComm c;
  memset(&c, 0, sizeof(c));
  c.num_groups = (int)num_groups;
  if (mode == 0) {
    TORCH_CHECK(groups.numel() >= (M + 127) / 128, "gemm_grouped: tile_group too short");
    c.tile_group = groups.data_ptr<int>();
    c.b_group_rows = (int)b_group_rows;
  } else {
    TORCH_CHECK(groups.numel() == num_groups + 1, "gemm_grouped: seg_start needs num_groups + 1 entries");
    c.seg_start = groups.data_ptr<int>();
  }
  check(pico_gemm_bf16_ex(A.data_ptr(), B.data_ptr(), D.data_ptr(), (int)M, (int)N, (int)K, (int)lda, (int)ldb,
                          (int)ldd, a_mn_major, b_mn_major, (int)out_mode, 0, &c, stream_of(A)),
        "gemm_grouped");
}

// ---------------------------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------------------------
PicoAttnParams attn_params(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o,
                           double sm_scale, bool causal, int64_t q_pos0, int64_t k_pos0) {
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4 && o.dim() == 4, "attention: [b, s, h, d] tensors");
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&q, &k, &v, &o}) {
    TORCH_CHECK(t->scalar_type() == at::kBFloat16 && t->is_cuda(), "attention: bf16 CUDA tensors");
    TORCH_CHECK(t->stride(3) == 1 && t->stride(2) == t->size(3), "attention: heads must be head_dim apart");
  }
  PicoAttnParams p;
  memset(&p, 0, sizeof(p));
  p.batch = (int)q.size(0);
  p.seq_q = (int)q.size(1);
  p.seq_k = (int)k.size(1);
  p.heads = (int)q.size(2);
  p.kv_heads = (int)k.size(2);
  p.head_dim = (int)q.size(3);
  p.q_batch_stride = q.stride(0); p.q_row_stride = q.stride(1);
  p.k_batch_stride = k.stride(0); p.k_row_stride = k.stride(1);
  p.v_batch_stride = v.stride(0); p.v_row_stride = v.stride(1);
  p.o_batch_stride = o.stride(0); p.o_row_stride = o.stride(1);
  p.sm_scale = (float)sm_scale;
  p.causal = causal;
  p.q_pos0 = (int)q_pos0;
  p.k_pos0 = (int)k_pos0;
  return p;
}

void attention_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& out,
                   at::Tensor& lse, double sm_scale, bool causal, int64_t q_pos0, int64_t k_pos0,
                   const c10::optional<at::Tensor>& trace) {
  c10::cuda::CUDAGuard guard(q.device());
  PicoAttnParams p = attn_params(q, k, v, out, sm_scale, causal, q_pos0, k_pos0);
  if (trace.has_value() && trace->defined()) {
    TORCH_CHECK(trace->scalar_type() == at::kLong && trace->numel() >= 1024, "trace: int64[1024]");
    p.trace = reinterpret_cast<unsigned long long*>(trace->data_ptr());
  }
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous(), "attention: fp32 contiguous lse");
  check(pico_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), (float*)lse.data_ptr(),
                           &p, stream_of(q)),
        "attention_fwd");
}

void attention_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& out,
                   const at::Tensor& dout, const at::Tensor& lse, at::Tensor& dq, at::Tensor& dk, at::Tensor& dv,
                   at::Tensor& delta, at::Tensor& dq_accum, double sm_scale, bool causal, int64_t q_pos0,
                   int64_t k_pos0) {
  c10::cuda::CUDAGuard guard(q.device());
  PicoAttnParams p = attn_params(q, k, v, out, sm_scale, causal, q_pos0, k_pos0);
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&dout, &dq, &dk, &dv}) {
    TORCH_CHECK(t->scalar_type() == at::kBFloat16 && t->dim() == 4 && t->stride(3) == 1 &&
                    t->stride(2) == t->size(3), "attention_bwd: [b, s, h, d] bf16 tensors with packed heads");
  }
  TORCH_CHECK(delta.scalar_type() == at::kFloat && dq_accum.scalar_type() == at::kFloat &&
                  dq_accum.is_contiguous() && delta.numel() >= lse.numel() && dq_accum.numel() >= q.numel(),
              "attention_bwd: fp32 scratch too small");
  check(pico_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                           (const float*)lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                           (float*)delta.data_ptr(), (float*)dq_accum.data_ptr(), &p, dout.stride(0),
                           dout.stride(1), dq.stride(0), dq.stride(1), dk.stride(0), dk.stride(1), dv.stride(0),
                           dv.stride(1), stream_of(q)),
        "attention_bwd");
}

// Returns the 8 status words after synchronising (word 0 != 0 means a kernel gave up a wait).
std::vector<int64_t> status_fetch() {
  int out[8] = {0};
  pico_status_fetch(out);
  return std::vector<int64_t>(out, out + 8);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rmsnorm_bwd_num_partials", &rmsnorm_bwd_num_partials);
  m.def("rope_inplace", &rope_inplace);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("ce_stats", &ce_stats);
  m.def("ce_loss_grad", &ce_loss_grad);
  m.def("adamw", &adamw);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("accumulate_bf16_into_f32", &accumulate_bf16_into_f32);
  m.def("fill_u32", &fill_u32);
  m.def("scale_unless_one", &scale_unless_one);
  m.def("attn_merge", &attn_merge);
  m.def("moe_route", &moe_route);
  m.def("moe_route_bwd", &moe_route_bwd);
  m.def("moe_slots", &moe_slots);
  m.def("moe_combine", &moe_combine);
  m.def("moe_combine_bwd", &moe_combine_bwd);
  m.def("status_fetch", &status_fetch);
  m.def("attention_fwd", &attention_fwd);
  m.def("attention_bwd", &attention_bwd);
  m.def("symm_alloc", &symm_alloc);
  m.def("symm_open", &symm_open);
  m.def("symm_close", &symm_close);
  m.def("symm_free", &symm_free);
  m.def("tensor_from_ptr", &tensor_from_ptr);
  m.def("signal_peers", &signal_peers);
  m.def("wait_flags", &wait_flags);
  m.def("epoch_base_add", &epoch_base_add);
  m.def("push_rows", &push_rows);
  m.def("slot_sum", &slot_sum);
  m.def("slot_sum_from", &slot_sum_from);
  m.def("scatter_rows", &scatter_rows);
  m.def("a2a_push", &a2a_push);
  m.def("ep_var_layout", &ep_var_layout);
  m.def("ep_var_exchange", &ep_var_exchange);
  m.def("ep_var_dequant", &ep_var_dequant);
  m.def("ep_var_copy_rows", &ep_var_copy_rows);
  m.def("ep_var_zero_padding", &ep_var_zero_padding);
  m.def("gemm_ex", &gemm_ex);
  m.def("gemm_grouped", &gemm_grouped);
  m.def("zero1_adamw", &zero1_adamw);
  m.def("ce_stats_push", &ce_stats_push);
  m.def("ce_loss_grad_gathered", &ce_loss_grad_gathered);
  m.def("ep_dispatch", &ep_dispatch);
  m.def("ep_dequant", &ep_dequant);
  m.def("ep_block_exchange", &ep_block_exchange);
}
