// Python bindings: torch tensors in, raw-pointer launchers (extern "C", defined in the .cu files)
// out.  All launches go to the current CUDA stream of the tensor's device.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdint>

extern "C" {
int apb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                  int a_mn_major, int b_mn_major, int out_fp32, uint32_t* status, int num_sms, cudaStream_t stream);
int apb_gemm_grouped_bf16(const void* A, const void* B, void* C, int G, int M, int N, int K, int a_mn_major, int b_mn_major,
                          int out_fp32, uint32_t* status, int num_sms, cudaStream_t stream);
void apb_gemm_set_pair_mode(int on);
int apb_gemm_get_pair_mode();
int apb_gemm_yield_request(int pairs, cudaStream_t stream);
int apb_gemm_yield_outstanding();
void apb_gemm_set_dynamic_tiles(int on);
int apb_gemm_get_dynamic_tiles();
void apb_gemm_set_pair_stages(int n);
int apb_gemm_get_pair_stages();
void apb_gemm_set_reserved_sms(int n);
int apb_gemm_get_reserved_sms();
int apb_gemm_fused_ctas(int fuse, int M, int N, int comm_ctas, int num_sms);
int apb_rms_norm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int D, float eps, int is_bf16,
                     cudaStream_t st);
int apb_rms_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw, float* dw_acc,
                     long long rows, int D, int is_bf16, int num_sms, cudaStream_t st);
int apb_cast(const void* src, void* dst, long long n, int src_bf16, int dst_bf16, int num_sms, cudaStream_t st);
int apb_rope(const void* x, const float* cs, const float* sn, void* y, long long B, int S, int H, int D, int conj, int is_bf16,
             int num_sms, cudaStream_t st);
int apb_swiglu_fwd(const void* a, const void* b, void* y, long long n, int is_bf16, int num_sms, cudaStream_t st);
int apb_swiglu_bwd(const void* dy, const void* a, const void* b, void* da, void* db, long long n, int is_bf16, int num_sms,
                   cudaStream_t st);
int apb_xent_fwd(const void* logits, const long long* labels, float* loss, float* lse, long long rows, int V, int is_bf16,
                 cudaStream_t st);
int apb_xent_bwd(const float* dloss, const void* logits, const long long* labels, const float* lse, void* dlogits,
                 long long rows, int V, int is_bf16, cudaStream_t st);
int apb_embedding_bwd(const void* dy, const long long* ids, float* out_f32, long long tokens, int D, int is_bf16,
                      cudaStream_t st);
int apb_embedding_fwd(const void* weight, const long long* ids, void* out, long long tokens, int D, long long num_rows,
                      int is_bf16, cudaStream_t st);
int apb_moe_slots_max_experts(int threads);
int apb_moe_slots(const long long* gate_idx, long long* slot, int num_blocks, int per_block, int E, int C, cudaStream_t st);
int apb_moe_scatter(const void* src, const long long* slot, const float* w, void* buf, long long T, int k, int d, int E, int C, int nb,
                    int is_bf16, cudaStream_t st);
int apb_moe_gather(const void* buf, const long long* slot, const float* w, void* out, long long T, int k, int d, int E, int C, int nb,
                   int is_bf16, cudaStream_t st);
int apb_moe_gate_grad(const void* buf, const long long* slot, const void* g, float* dw, long long T, int k, int d, int E, int C, int nb,
                      int is_bf16, cudaStream_t st);
int apb_symm_header_bytes();
int apb_symm_wait_probe(const uint32_t* flag, unsigned target, unsigned limit_ms, uint32_t* status, cudaStream_t st);
int apb_symm_collective(int mode, const unsigned long long* peer_ptrs, int rank, int n, unsigned epoch, const void* src,
                        void* dst, long long outer, long long inner_bytes, int elem_kind, float scale, long long stage_capacity,
                        uint32_t* status, int num_ctas, unsigned target0, unsigned target1, unsigned long long multicast_base, cudaStream_t st);
int apb_gemm_fused(int fuse, const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                   long long ldc, int a_mn_major, int b_mn_major, int out_fp32, const unsigned long long* peer_ptrs, int rank,
                   int n, unsigned epoch, int rows_per_shard, const void* shard_src, void* gbuf, long long shard_bytes,
                   uint32_t* landed, unsigned landed_target, int rows_per_rank, float scale, long long stage_capacity,
                   const unsigned* targets, int comm_ctas, uint32_t* status, int num_sms, cudaStream_t stream);
int apb_dma_flag_bytes();
int apb_dma_ring_max();
int apb_dma_barrier(const unsigned long long* flags, int rank, int n, unsigned epoch, uint32_t* status, cudaStream_t st);
int apb_dma_all_gather(void* dst, const unsigned long long* bases, long long offset, long long outer, long long inner_bytes,
                       int rank, int n, cudaStream_t st);
int apb_dma_rs_push(const void* src, const unsigned long long* bases, const unsigned long long* flags, long long stage_offset,
                    long long slot_bytes, long long chunk_bytes, int entry, int ring, unsigned seq, int rank, int n,
                    uint32_t* status, cudaStream_t st);
int apb_dma_rs_sum(const void* src, void* dst, const unsigned long long* bases, const unsigned long long* flags,
                   long long stage_offset, long long slot_bytes, long long chunk_bytes, int entry, unsigned seq, float scale,
                   int rank, int n, int num_ctas, uint32_t* status, cudaStream_t st);
int apb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int Sk, int H, int Hkv,
                      int D, int causal, float scale, uint32_t* status, cudaStream_t stream);
int apb_adamw(const void* tensors_dev, const void* chunks_dev, int num_chunks, float lr, float beta1, float beta2, float eps,
              float wd, float bc1, float bc2, float grad_scale, const float* hyper_dev, cudaStream_t st);
}

namespace {

int num_sms() { return at::cuda::getCurrentDeviceProperties()->multiProcessorCount; }
cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check(int err, const char* what) {
  TORCH_CHECK(err == 0, what, " failed with code ", err,
              err == 3 ? " (unsupported shape / alignment)" : err == 4 ? " (launch error)" : "");
}

bool is_bf16(const at::Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat, "expected bf16 or fp32, got ",
              t.scalar_type());
  return t.scalar_type() == at::kBFloat16;
}

// C[M,N] = opA * opB.  a: [M,K] (or [K,M] if a_mn_major); b: [N,K] (or [K,N] if b_mn_major).
void gemm(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool a_mn_major, bool b_mn_major, at::Tensor& status) {
  c10::cuda::CUDAGuard g(a.device());
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm: bf16 operands required");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && c.stride(1) == 1,
              "gemm: 2-d row-major operands required");
  const int M = c.size(0), N = c.size(1);
  const int K = a_mn_major ? a.size(0) : a.size(1);
  TORCH_CHECK((a_mn_major ? a.size(1) : a.size(0)) == M, "gemm: A shape mismatch");
  TORCH_CHECK((b_mn_major ? b.size(1) : b.size(0)) == N && (b_mn_major ? b.size(0) : b.size(1)) == K, "gemm: B shape mismatch");
  const bool out_fp32 = c.scalar_type() == at::kFloat;
  TORCH_CHECK(out_fp32 || c.scalar_type() == at::kBFloat16, "gemm: output must be bf16 or fp32");
  check(apb_gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, a.stride(0), b.stride(0), c.stride(0), a_mn_major,
                      b_mn_major, out_fp32, reinterpret_cast<uint32_t*>(status.data_ptr()), num_sms(), stream()),
        "apb_gemm_bf16");
}

// c[g] = opA[g] * opB[g]; a: [G,M,K] (or [G,K,M] if a_mn_major); b: [G,N,K] (or [G,K,N]); c: [G,M,N]; all contiguous.
void gemm_grouped(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool a_mn_major, bool b_mn_major, at::Tensor& status) {
  c10::cuda::CUDAGuard g(a.device());
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm_grouped: bf16 operands required");
  TORCH_CHECK(a.dim() == 3 && b.dim() == 3 && c.dim() == 3 && a.is_contiguous() && b.is_contiguous() && c.is_contiguous(),
              "gemm_grouped: contiguous 3-d operands required");
  const int G = c.size(0), M = c.size(1), N = c.size(2);
  const int K = a_mn_major ? a.size(1) : a.size(2);
  TORCH_CHECK(a.size(0) == G && b.size(0) == G && (a_mn_major ? a.size(2) : a.size(1)) == M, "gemm_grouped: A shape mismatch");
  TORCH_CHECK((b_mn_major ? b.size(2) : b.size(1)) == N && (b_mn_major ? b.size(1) : b.size(2)) == K, "gemm_grouped: B shape mismatch");
  const bool out_fp32 = c.scalar_type() == at::kFloat;
  TORCH_CHECK(out_fp32 || c.scalar_type() == at::kBFloat16, "gemm_grouped: output must be bf16 or fp32");
  check(apb_gemm_grouped_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), G, M, N, K, a_mn_major, b_mn_major, out_fp32,
                              reinterpret_cast<uint32_t*>(status.data_ptr()), num_sms(), stream()),
        "apb_gemm_grouped_bf16");
}

// q [B,S,H,D], k / v [B,Sk,Hkv,D] -> out [B,S,H,D] bf16, lse [B,H,S] fp32.  Returns false (nothing launched) for
// shapes the kernel does not cover.
bool attention_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& out, at::Tensor& lse, bool causal,
                   double scale, at::Tensor& status) {
  c10::cuda::CUDAGuard g(q.device());
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16 &&
                  out.scalar_type() == at::kBFloat16 && lse.scalar_type() == at::kFloat,
              "attention_fwd: bf16 q / k / v / out and fp32 lse required");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4 && q.is_contiguous() && k.is_contiguous() && v.is_contiguous() &&
                  out.is_contiguous() && lse.is_contiguous(),
              "attention_fwd: contiguous [B, S, H, D] tensors required");
  TORCH_CHECK(k.sizes() == v.sizes() && k.size(0) == q.size(0) && k.size(3) == q.size(3) && out.sizes() == q.sizes() &&
                  lse.numel() == q.size(0) * q.size(1) * q.size(2),
              "attention_fwd: shape mismatch");
  const int err = apb_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), q.size(0),
                                    q.size(1), k.size(1), q.size(2), k.size(2), q.size(3), causal, (float)scale,
                                    reinterpret_cast<uint32_t*>(status.data_ptr()), stream());
  if (err == 3) return false;
  check(err, "apb_attention_fwd");
  return true;
}

void rms_norm_fwd(const at::Tensor& x, const at::Tensor& w, at::Tensor& y, at::Tensor& rstd, double eps) {
  c10::cuda::CUDAGuard g(x.device());
  const int D = x.size(-1);
  check(apb_rms_norm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), x.numel() / D, D, (float)eps,
                         is_bf16(x), stream()),
        "apb_rms_norm_fwd");
}

void rms_norm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd, at::Tensor& dx,
                  at::Tensor& dw, at::Tensor& dw_acc) {
  c10::cuda::CUDAGuard g(x.device());
  const int D = x.size(-1);
  check(apb_rms_norm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(), dw.data_ptr(),
                         dw_acc.data_ptr<float>(), x.numel() / D, D, is_bf16(x), num_sms(), stream()),
        "apb_rms_norm_bwd");
}

void cast(const at::Tensor& src, at::Tensor& dst) {
  c10::cuda::CUDAGuard g(src.device());
  check(apb_cast(src.data_ptr(), dst.data_ptr(), src.numel(), is_bf16(src), is_bf16(dst), num_sms(), stream()), "apb_cast");
}

void rope(const at::Tensor& x, const at::Tensor& cs, const at::Tensor& sn, at::Tensor& y, bool conj) {
  c10::cuda::CUDAGuard g(x.device());
  check(apb_rope(x.data_ptr(), cs.data_ptr<float>(), sn.data_ptr<float>(), y.data_ptr(), x.size(0), x.size(1), x.size(2),
                 x.size(3), conj, is_bf16(x), num_sms(), stream()),
        "apb_rope");
}

void swiglu_fwd(const at::Tensor& a, const at::Tensor& b, at::Tensor& y) {
  c10::cuda::CUDAGuard g(a.device());
  check(apb_swiglu_fwd(a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), is_bf16(a), num_sms(), stream()), "apb_swiglu_fwd");
}

void swiglu_bwd(const at::Tensor& dy, const at::Tensor& a, const at::Tensor& b, at::Tensor& da, at::Tensor& db) {
  c10::cuda::CUDAGuard g(a.device());
  check(apb_swiglu_bwd(dy.data_ptr(), a.data_ptr(), b.data_ptr(), da.data_ptr(), db.data_ptr(), a.numel(), is_bf16(a), num_sms(),
                       stream()),
        "apb_swiglu_bwd");
}

void xent_fwd(const at::Tensor& logits, const at::Tensor& labels, at::Tensor& loss, at::Tensor& lse) {
  c10::cuda::CUDAGuard g(logits.device());
  const int V = logits.size(-1);
  check(apb_xent_fwd(logits.data_ptr(), (const long long*)labels.data_ptr<int64_t>(), loss.data_ptr<float>(),
                     lse.data_ptr<float>(), logits.numel() / V, V, is_bf16(logits), stream()),
        "apb_xent_fwd");
}

void xent_bwd(const at::Tensor& dloss, const at::Tensor& logits, const at::Tensor& labels, const at::Tensor& lse,
              at::Tensor& dlogits) {
  c10::cuda::CUDAGuard g(logits.device());
  const int V = logits.size(-1);
  check(apb_xent_bwd(dloss.data_ptr<float>(), logits.data_ptr(), (const long long*)labels.data_ptr<int64_t>(),
                     lse.data_ptr<float>(), dlogits.data_ptr(), logits.numel() / V, V, is_bf16(logits), stream()),
        "apb_xent_bwd");
}

void embedding_fwd(const at::Tensor& weight, const at::Tensor& ids, at::Tensor& out) {
  c10::cuda::CUDAGuard g(weight.device());
  TORCH_CHECK(weight.dim() == 2 && weight.is_contiguous() && ids.scalar_type() == at::kLong && ids.is_contiguous() && out.is_contiguous(),
              "embedding_fwd: contiguous [V, D] table, int64 ids");
  check(apb_embedding_fwd(weight.data_ptr(), reinterpret_cast<const long long*>(ids.data_ptr()), out.data_ptr(), ids.numel(),
                          (int)weight.size(1), weight.size(0), is_bf16(weight), stream()),
        "apb_embedding_fwd");
}

void embedding_bwd(const at::Tensor& dy, const at::Tensor& ids, at::Tensor& out_f32) {
  c10::cuda::CUDAGuard g(dy.device());
  check(apb_embedding_bwd(dy.data_ptr(), (const long long*)ids.data_ptr<int64_t>(), out_f32.data_ptr<float>(), ids.numel(),
                          dy.size(-1), is_bf16(dy), stream()),
        "apb_embedding_bwd");
}

// Mixture-of-experts dispatch (ops/moe_ops.py): gate_idx / slot [T, k] int64, w [T, k] fp32, buf [E, nb, C, d], src / out / g [T, d].
static void moe_check(const at::Tensor& x, const char* what) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), what, ": contiguous CUDA tensor expected");
}

int64_t moe_slots_max_experts(int64_t per_block) {
  int threads = per_block >= 1024 ? 1024 : (int)((per_block + 31) / 32) * 32;
  return apb_moe_slots_max_experts(threads);
}

void moe_slots(const at::Tensor& gate_idx, at::Tensor& slot, int64_t E, int64_t C, int64_t nb) {
  c10::cuda::CUDAGuard g(gate_idx.device());
  moe_check(gate_idx, "moe_slots");
  moe_check(slot, "moe_slots");
  TORCH_CHECK(gate_idx.scalar_type() == at::kLong && slot.scalar_type() == at::kLong && gate_idx.dim() == 2 &&
                  gate_idx.numel() == slot.numel() && nb > 0 && gate_idx.size(0) % nb == 0,
              "moe_slots: int64 [T, k] with T a multiple of the block count");
  const int64_t per_block = gate_idx.size(0) / nb * gate_idx.size(1);
  check(apb_moe_slots((const long long*)gate_idx.data_ptr<int64_t>(), (long long*)slot.data_ptr<int64_t>(), (int)nb, (int)per_block,
                      (int)E, (int)C, stream()),
        "apb_moe_slots");
}

void moe_scatter(const at::Tensor& src, const at::Tensor& slot, const at::Tensor& w, at::Tensor& buf, int64_t E, int64_t C, int64_t nb) {
  c10::cuda::CUDAGuard g(src.device());
  moe_check(src, "moe_scatter"); moe_check(slot, "moe_scatter"); moe_check(w, "moe_scatter"); moe_check(buf, "moe_scatter");
  TORCH_CHECK(src.dim() == 2 && slot.dim() == 2 && slot.scalar_type() == at::kLong && w.scalar_type() == at::kFloat &&
                  w.numel() == slot.numel() && slot.size(0) == src.size(0) && buf.scalar_type() == src.scalar_type() &&
                  buf.numel() == E * nb * C * src.size(1),
              "moe_scatter: src [T, d], slot [T, k] int64, w [T, k] fp32, buf [E, nb, C, d] of src's dtype");
  check(apb_moe_scatter(src.data_ptr(), (const long long*)slot.data_ptr<int64_t>(), w.data_ptr<float>(), buf.data_ptr(), src.size(0),
                        (int)slot.size(1), (int)src.size(1), (int)E, (int)C, (int)nb, is_bf16(src), stream()),
        "apb_moe_scatter");
}

void moe_gather(const at::Tensor& buf, const at::Tensor& slot, const at::Tensor& w, at::Tensor& out) {
  c10::cuda::CUDAGuard g(buf.device());
  moe_check(buf, "moe_gather"); moe_check(slot, "moe_gather"); moe_check(w, "moe_gather"); moe_check(out, "moe_gather");
  TORCH_CHECK(buf.dim() == 4 && slot.dim() == 2 && slot.scalar_type() == at::kLong && w.scalar_type() == at::kFloat &&
                  w.numel() == slot.numel() && out.dim() == 2 && out.size(0) == slot.size(0) && out.size(1) == buf.size(3) &&
                  out.scalar_type() == buf.scalar_type(),
              "moe_gather: buf [E, nb, C, d], slot [T, k] int64, w [T, k] fp32, out [T, d] of buf's dtype");
  check(apb_moe_gather(buf.data_ptr(), (const long long*)slot.data_ptr<int64_t>(), w.data_ptr<float>(), out.data_ptr(), slot.size(0),
                       (int)slot.size(1), (int)buf.size(3), (int)buf.size(0), (int)buf.size(2), (int)buf.size(1), is_bf16(buf), stream()),
        "apb_moe_gather");
}

void moe_gate_grad(const at::Tensor& buf, const at::Tensor& slot, const at::Tensor& g_, at::Tensor& dw) {
  c10::cuda::CUDAGuard g(buf.device());
  moe_check(buf, "moe_gate_grad"); moe_check(slot, "moe_gate_grad"); moe_check(g_, "moe_gate_grad"); moe_check(dw, "moe_gate_grad");
  TORCH_CHECK(buf.dim() == 4 && slot.dim() == 2 && slot.scalar_type() == at::kLong && g_.dim() == 2 && g_.size(0) == slot.size(0) &&
                  g_.size(1) == buf.size(3) && g_.scalar_type() == buf.scalar_type() && dw.scalar_type() == at::kFloat &&
                  dw.numel() == slot.numel(),
              "moe_gate_grad: buf [E, nb, C, d], slot [T, k] int64, g [T, d] of buf's dtype, dw [T, k] fp32");
  check(apb_moe_gate_grad(buf.data_ptr(), (const long long*)slot.data_ptr<int64_t>(), g_.data_ptr(), dw.data_ptr<float>(), slot.size(0),
                          (int)slot.size(1), (int)buf.size(3), (int)buf.size(0), (int)buf.size(2), (int)buf.size(1), is_bf16(buf), stream()),
        "apb_moe_gate_grad");
}

void adamw(const at::Tensor& table, const at::Tensor& chunks, int64_t num_chunks, double lr, double b1, double b2, double eps,
           double wd, double bc1, double bc2, double grad_scale, const c10::optional<at::Tensor>& hyper) {
  c10::cuda::CUDAGuard g(table.device());
  const float* hp = nullptr;
  if (hyper.has_value()) {
    TORCH_CHECK(hyper->scalar_type() == at::kFloat && hyper->numel() >= 3 && hyper->is_cuda(), "adamw: hyper = fp32 [3] on the device");
    hp = hyper->data_ptr<float>();
  }
  check(apb_adamw(table.data_ptr(), chunks.data_ptr(), (int)num_chunks, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd,
                  (float)bc1, (float)bc2, (float)grad_scale, hp, stream()),
        "apb_adamw");
}

int64_t symm_header_bytes() { return apb_symm_header_bytes(); }

// Bounded wait on a device flag (int32 tensor, element 0) that the caller may or may not ever raise.
void symm_wait_probe(const at::Tensor& flag, int64_t target, int64_t limit_ms, at::Tensor& status) {
  c10::cuda::CUDAGuard g(flag.device());
  TORCH_CHECK(flag.scalar_type() == at::kInt && flag.numel() >= 1, "symm_wait_probe: int32 flag tensor required");
  check(apb_symm_wait_probe(reinterpret_cast<const uint32_t*>(flag.data_ptr()), (unsigned)target, (unsigned)limit_ms,
                            reinterpret_cast<uint32_t*>(status.data_ptr()), stream()),
        "apb_symm_wait_probe");
}

// One collective on a symmetric workspace (see symm_comm.cu).  src/dst are ordinary device tensors.
void symm_collective(int64_t mode, const std::vector<int64_t>& peer_ptrs, int64_t rank, int64_t epoch, const at::Tensor& src,
                     at::Tensor& dst, int64_t outer, int64_t inner_bytes, int64_t elem_kind, double scale,
                     int64_t stage_capacity, at::Tensor& status, int64_t num_ctas, int64_t target0, int64_t target1,
                     int64_t multicast_base) {
  c10::cuda::CUDAGuard g(src.device());
  std::vector<unsigned long long> ptrs(peer_ptrs.begin(), peer_ptrs.end());
  check(apb_symm_collective((int)mode, ptrs.data(), (int)rank, (int)ptrs.size(), (unsigned)epoch, src.data_ptr(), dst.data_ptr(),
                            outer, inner_bytes, (int)elem_kind, (float)scale, stage_capacity,
                            reinterpret_cast<uint32_t*>(status.data_ptr()), (int)num_ctas, (unsigned)target0, (unsigned)target1,
                            (unsigned long long)multicast_base, stream()),
        "apb_symm_collective");
}

// GEMM fused with a collective (see gemm_fused.cu).  a/b follow the conventions of ``gemm``; for the
// gather modes the gathered operand passed here is the local full-size buffer ``gbuf``.
void gemm_fused(int64_t fuse, const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool a_mn_major, bool b_mn_major,
                const std::vector<int64_t>& peer_ptrs, int64_t rank, int64_t epoch, int64_t rows_per_shard,
                const at::Tensor& shard_src, const at::Tensor& landed, int64_t landed_target, int64_t rows_per_rank,
                double scale, int64_t stage_capacity, const std::vector<int64_t>& targets, int64_t comm_ctas,
                at::Tensor& status) {
  c10::cuda::CUDAGuard g(a.device());
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm_fused: bf16 operands required");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && c.is_contiguous(), "gemm_fused: layout");
  const int K = a_mn_major ? a.size(0) : a.size(1);
  const int M = a_mn_major ? a.size(1) : a.size(0);
  const int N = b_mn_major ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn_major ? b.size(0) : b.size(1)) == K, "gemm_fused: contraction mismatch");
  const bool out_fp32 = c.scalar_type() == at::kFloat;
  std::vector<unsigned long long> ptrs(peer_ptrs.begin(), peer_ptrs.end());
  unsigned tg[3] = {(unsigned)targets[0], (unsigned)targets[1], (unsigned)targets[2]};
  void* gbuf = fuse == 1 ? a.data_ptr() : b.data_ptr();
  check(apb_gemm_fused((int)fuse, a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                       c.dim() == 2 ? c.stride(0) : N, a_mn_major, b_mn_major, out_fp32, ptrs.data(), (int)rank, (int)ptrs.size(),
                       (unsigned)epoch, (int)rows_per_shard, shard_src.data_ptr(), gbuf,
                       (long long)shard_src.numel() * shard_src.element_size(),
                       reinterpret_cast<uint32_t*>(landed.data_ptr()), (unsigned)landed_target, (int)rows_per_rank, (float)scale,
                       stage_capacity, tg, (int)comm_ctas, reinterpret_cast<uint32_t*>(status.data_ptr()), num_sms(), stream()),
        "apb_gemm_fused");
}

// ------------------------------------------------------------------ copy-engine collectives (dma_comm.cu)
std::vector<unsigned long long> u64(const std::vector<int64_t>& v) { return std::vector<unsigned long long>(v.begin(), v.end()); }

void dma_barrier(const std::vector<int64_t>& flags, int64_t rank, int64_t epoch, at::Tensor& status) {
  c10::cuda::CUDAGuard g(status.device());
  auto f = u64(flags);
  check(apb_dma_barrier(f.data(), (int)rank, (int)f.size(), (unsigned)epoch, reinterpret_cast<uint32_t*>(status.data_ptr()), stream()),
        "apb_dma_barrier");
}

void dma_all_gather(at::Tensor& dst, const std::vector<int64_t>& bases, int64_t offset, int64_t outer, int64_t inner_bytes,
                    int64_t rank) {
  c10::cuda::CUDAGuard g(dst.device());
  auto b = u64(bases);
  TORCH_CHECK(dst.is_contiguous() && (int64_t)dst.nbytes() == outer * inner_bytes * (int64_t)b.size(), "dma_all_gather: output size");
  check(apb_dma_all_gather(dst.data_ptr(), b.data(), offset, outer, inner_bytes, (int)rank, (int)b.size(), stream()),
        "apb_dma_all_gather");
}

void dma_rs_push(const at::Tensor& src, const std::vector<int64_t>& bases, const std::vector<int64_t>& flags, int64_t stage_offset,
                 int64_t slot_bytes, int64_t entry, int64_t ring, int64_t seq, int64_t rank, at::Tensor& status) {
  c10::cuda::CUDAGuard g(src.device());
  auto b = u64(bases), f = u64(flags);
  TORCH_CHECK(src.is_contiguous() && src.nbytes() % b.size() == 0, "dma_rs_push: contiguous input of n equal chunks");
  check(apb_dma_rs_push(src.data_ptr(), b.data(), f.data(), stage_offset, slot_bytes, (long long)(src.nbytes() / b.size()), (int)entry,
                        (int)ring, (unsigned)seq, (int)rank, (int)b.size(), reinterpret_cast<uint32_t*>(status.data_ptr()), stream()),
        "apb_dma_rs_push");
}

void dma_rs_sum(const at::Tensor& src, at::Tensor& dst, const std::vector<int64_t>& bases, const std::vector<int64_t>& flags,
                int64_t stage_offset, int64_t slot_bytes, int64_t entry, int64_t seq, double scale, int64_t rank, int64_t num_ctas,
                at::Tensor& status) {
  c10::cuda::CUDAGuard g(src.device());
  auto b = u64(bases), f = u64(flags);
  TORCH_CHECK(src.scalar_type() == at::kFloat && dst.scalar_type() == at::kFloat && src.is_contiguous() && dst.is_contiguous(),
              "dma_rs_sum: contiguous fp32 tensors");
  TORCH_CHECK(dst.nbytes() * b.size() == src.nbytes(), "dma_rs_sum: output is one of n equal chunks");
  check(apb_dma_rs_sum(src.data_ptr(), dst.data_ptr(), b.data(), f.data(), stage_offset, slot_bytes, (long long)dst.nbytes(), (int)entry,
                       (unsigned)seq, (float)scale, (int)rank, (int)b.size(), (int)num_ctas,
                       reinterpret_cast<uint32_t*>(status.data_ptr()), stream()),
        "apb_dma_rs_sum");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("dma_flag_bytes", []() { return (int64_t)apb_dma_flag_bytes(); });
  m.def("dma_ring_max", []() { return (int64_t)apb_dma_ring_max(); });
  m.def("dma_barrier", &dma_barrier);
  m.def("dma_all_gather", &dma_all_gather);
  m.def("dma_rs_push", &dma_rs_push);
  m.def("dma_rs_sum", &dma_rs_sum);
  m.def("gemm", &gemm);
  m.def("gemm_grouped", &gemm_grouped);
  m.def("gemm_set_pair_mode", [](bool on) { apb_gemm_set_pair_mode(on ? 1 : 0); });
  m.def("gemm_yield_request", [](int64_t pairs) { check(apb_gemm_yield_request((int)pairs, stream()), "apb_gemm_yield_request"); });
  m.def("gemm_yield_outstanding", []() { return (int64_t)apb_gemm_yield_outstanding(); });
  m.def("gemm_set_dynamic_tiles", [](bool on) { apb_gemm_set_dynamic_tiles(on ? 1 : 0); });
  m.def("gemm_get_dynamic_tiles", []() { return apb_gemm_get_dynamic_tiles() != 0; });
  m.def("gemm_set_pair_stages", [](int64_t n) { apb_gemm_set_pair_stages((int)n); });
  m.def("gemm_get_pair_stages", []() { return (int64_t)apb_gemm_get_pair_stages(); });
  m.def("gemm_set_reserved_sms", [](int64_t n) { apb_gemm_set_reserved_sms((int)n); });
  m.def("gemm_get_reserved_sms", []() { return (int64_t)apb_gemm_get_reserved_sms(); });
  m.def("gemm_get_pair_mode", []() { return apb_gemm_get_pair_mode() != 0; });
  m.def("attention_fwd", &attention_fwd);
  m.def("rms_norm_fwd", &rms_norm_fwd);
  m.def("rms_norm_bwd", &rms_norm_bwd);
  m.def("cast", &cast);
  m.def("rope", &rope);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("xent_fwd", &xent_fwd);
  m.def("xent_bwd", &xent_bwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("adamw", &adamw);
  m.def("moe_slots_max_experts", &moe_slots_max_experts);
  m.def("moe_slots", &moe_slots);
  m.def("moe_scatter", &moe_scatter);
  m.def("moe_gather", &moe_gather);
  m.def("moe_gate_grad", &moe_gate_grad);
  m.def("symm_header_bytes", &symm_header_bytes);
  m.def("symm_wait_probe", &symm_wait_probe);
  m.def("symm_collective", &symm_collective);
  m.def("gemm_fused", &gemm_fused);
  m.def("gemm_fused_ctas", [](int64_t fuse, int64_t M, int64_t N, int64_t comm_ctas) {
    return (int64_t)apb_gemm_fused_ctas((int)fuse, (int)M, (int)N, (int)comm_ctas, num_sms());
  });
}
