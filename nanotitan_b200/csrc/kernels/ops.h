// Host entry points of the extension (one declaration per kernel family).
#pragma once
#include <ATen/ATen.h>

#include <string>
#include <tuple>
#include <vector>

#include "status.h"

namespace nt {

// ---- device status (bounded waits, checked indices)
StatusWord* device_status_word();
std::vector<int64_t> read_status(bool clear);
at::Tensor status_word_tensor();  // [code, kernel, detail, count]

int64_t bounded_wait_probe(double limit_ms);  // probe.cu: makes a bounded device wait run out, on purpose

// ---- symmetric heap (runtime/symmetric_heap.h behind integer handles; runtime/symmetric_heap_torch.cpp).
//   open: collective over the ranks of one machine that share `job`; alloc (collective) returns this rank's
//   piece as a byte tensor, every rank's address of the allocation, the multicast address (0: none) and the
//   allocation's id; free and close are collective too.
int64_t symm_heap_open(const std::string& job, int64_t rank, int64_t world, int64_t device, int64_t timeout_ms);
std::tuple<at::Tensor, std::vector<int64_t>, int64_t, int64_t> symm_heap_alloc(int64_t heap, int64_t bytes, bool multicast);
void symm_heap_free(int64_t heap, int64_t allocation);
void symm_heap_close(int64_t heap);

// ---- tcgen05 GEMM (gemm_tc.cu).
//   A: 2-D; a_mn=false -> [M, K] rows contiguous in K, a_mn=true -> [K, M] rows contiguous in M.
//   Bs: 1..3 tensors, 2-D or [G, ., .]; b_mn=false -> [N, K], b_mn=true -> [K, N].
//   b_split: 0 one source; 1 sources side by side along N; 2 sources stacked along K;
//            3 two sources whose columns pair up as (gate, value) for the SwiGLU epilogue.
//   Cs: 1..3 destinations ([M, N/len] each), or [G, M, N/len] in grouped-K mode.
//   mode: 0 dense, 1 rows segmented by `offsets` (B[g] per segment), 2 reduction segmented (C[g]).
//   epilogue: 0 store (+ residual `aux`, + old C when `accumulate`); 1 SwiGLU forward
//             (C = [rows, 2N] gate|value, aux_out = H [rows, N]); 2 SwiGLU backward (aux = gate|value
//             [rows, 2N], C = d(gate|value) [rows, 2N], the accumulator being dH).
void gemm_tc(const at::Tensor& A, bool a_mn, const std::vector<at::Tensor>& Bs, bool b_mn, int64_t b_split,
             const std::vector<at::Tensor>& Cs, int64_t mode, const c10::optional<at::Tensor>& offsets,
             int64_t epilogue, bool accumulate, const c10::optional<at::Tensor>& aux,
             const c10::optional<at::Tensor>& aux_out, int64_t force_bn);

// ---- CUDA-core GEMMs (gemm_simt.cu)
at::Tensor gemm_kernel(const at::Tensor& A, const at::Tensor& B, const std::string& implementation);
at::Tensor tiled_gemm_kernel(const at::Tensor& A, const at::Tensor& B);
at::Tensor naive_gemm_kernel(const at::Tensor& A, const at::Tensor& B);
at::Tensor simt_grouped_fwd(const at::Tensor& X, const at::Tensor& off, const at::Tensor& W);
at::Tensor simt_grouped_dx(const at::Tensor& W, const at::Tensor& off, const at::Tensor& dOut);
at::Tensor simt_grouped_dw(const at::Tensor& X, const at::Tensor& off, const at::Tensor& dOut);

// ---- grouped GEMM entry points with the reference's signatures (grouped.cu)
at::Tensor grouped_gemm_kernel(const at::Tensor& X, const at::Tensor& offset, const at::Tensor& W);
at::Tensor bwd_grouped_gemm_dX_kernel(const at::Tensor& W, const at::Tensor& offset, const at::Tensor& dOut);
at::Tensor bwd_grouped_gemm_dW_kernel(const at::Tensor& X, const at::Tensor& offset, const at::Tensor& dOut);

// ---- normalisation, loss, optimizer
std::vector<at::Tensor> layer_norm_fwd(const at::Tensor& x, const at::Tensor& gamma, const at::Tensor& beta, double eps);
// `dres` (optional, shaped like x): a gradient that reached x on a path around the normalisation
// (the residual connection); it is added to dx in the same pass.  `dgamma_out` / `dbeta_out`
// (optional, [d], fp32 or a 16-bit dtype): where to write the parameter gradients; without them
// two fp32 tensors are allocated.
std::vector<at::Tensor> layer_norm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& gamma,
                                       const at::Tensor& mean, const at::Tensor& rstd,
                                       const c10::optional<at::Tensor>& dres,
                                       const c10::optional<at::Tensor>& dgamma_out,
                                       const c10::optional<at::Tensor>& dbeta_out);
at::Tensor cross_entropy_fwd_bwd(at::Tensor logits, const at::Tensor& targets, int64_t V, double grad_scale, bool write_grad);
// `bc_dev` (optional, fp32 [2] on the device): {1 - beta1^t, 1 / sqrt(1 - beta2^t)} read by the kernel instead of being
// computed from `step` on the host, so that a captured launch stays valid as t advances.
at::Tensor adamw_step(at::Tensor param, const at::Tensor& grad, at::Tensor master, at::Tensor m, at::Tensor v, int64_t step,
                      double lr, double beta1, double beta2, double eps, double wd, double grad_scale, bool want_sq,
                      const c10::optional<at::Tensor>& bc_dev);

// ---- flash attention (flash_attn.cu): [B, S, H, Dh] tensors, Dh in {32, 64}
std::vector<at::Tensor> flash_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale);
std::vector<at::Tensor> flash_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                  const at::Tensor& out, const at::Tensor& lse, double scale, const std::vector<at::Tensor>& grads);

// ---- fused gradient-bucket all-reduce (+ AdamW) over NVLink peer / multicast memory (allreduce_adamw.cu)
void bucket_allreduce(at::Tensor grad_local, int64_t grad_mc, const at::Tensor& grad_peers, int64_t param_mc,
                      const at::Tensor& param_peers, const c10::optional<at::Tensor>& master, const c10::optional<at::Tensor>& m,
                      const c10::optional<at::Tensor>& v, at::Tensor flag_local, const at::Tensor& flag_peers, at::Tensor block_counter,
                      int64_t rank, int64_t world, int64_t slot, at::Tensor epoch_counters, int64_t step,
                      const c10::optional<at::Tensor>& bc_dev, double lr, double beta1, double beta2,
                      double eps, double wd, int64_t blocks, double wait_ms);

// ---- expert-parallel row exchange over NVLink peer memory (ep_exchange.cu)
void ep_allgather_counts(const at::Tensor& counts, const at::Tensor& cmat_peers, at::Tensor flag_local, const at::Tensor& flag_peers,
                         int64_t rank, int64_t world, at::Tensor epoch_counter, int64_t word_base, double wait_ms);
std::vector<at::Tensor> ep_dispatch(const at::Tensor& x, const at::Tensor& gates, const at::Tensor& idx, const at::Tensor& slot_of,
                                    const at::Tensor& counts, const at::Tensor& offsets, at::Tensor cmat_local,
                                    const at::Tensor& cmat_peers, const at::Tensor& dst_peers, int64_t capacity_rows, int64_t E_loc,
                                    at::Tensor block_counter, at::Tensor flag_local, const at::Tensor& flag_peers, int64_t rank,
                                    int64_t world, at::Tensor epoch_counter, double wait_ms, int64_t blocks);
void ep_push_rows(const at::Tensor& src, const at::Tensor& dst_peers, int64_t dst_capacity_rows, const at::Tensor& cmat, int64_t E_loc,
                  int64_t direction, bool entry_barrier, at::Tensor block_counter, at::Tensor flag_local, const at::Tensor& flag_peers,
                  int64_t rank, int64_t world, at::Tensor epoch_counter, int64_t word_base, double wait_ms, int64_t blocks);

// ---- MoE routing / dispatch
std::vector<at::Tensor> router_topk(const at::Tensor& x, const at::Tensor& w, int64_t k);
std::vector<at::Tensor> router_from_logits(const at::Tensor& logits, int64_t k);  // same outputs, logits formed elsewhere
std::vector<at::Tensor> router_bwd(const at::Tensor& gates, const at::Tensor& idx, const at::Tensor& probs,
                                   const c10::optional<at::Tensor>& dgates, const c10::optional<at::Tensor>& dprobs,
                                   const c10::optional<at::Tensor>& dprobs_mean, const at::Tensor& like);
std::vector<at::Tensor> assign_slots(const at::Tensor& idx, const at::Tensor& counts);
at::Tensor count_expert_kernel(const at::Tensor& topk, const at::Tensor& mask, int64_t E, int64_t k);
std::vector<at::Tensor> pack_fwd(const at::Tensor& x, const at::Tensor& gates, const at::Tensor& idx, const at::Tensor& slot_of);
at::Tensor combine_fwd(const at::Tensor& y, const at::Tensor& w, const at::Tensor& rows, const c10::optional<at::Tensor>& row_start,
                       int64_t tokens, const c10::optional<at::Tensor>& residual, bool out_f32);
std::vector<at::Tensor> combine_bwd(const at::Tensor& y, const at::Tensor& token, const at::Tensor& w, const at::Tensor& dout);
at::Tensor pack_bwd(const at::Tensor& dpacked, const at::Tensor& rows, const c10::optional<at::Tensor>& row_start, int64_t tokens);
std::vector<at::Tensor> pack_tokens_kernel(const at::Tensor& X, const at::Tensor& w, const at::Tensor& e, const at::Tensor& offset_cpy);
at::Tensor combine_tokens_kernel(const at::Tensor& Y, const at::Tensor& tokenId, const at::Tensor& w, int64_t T, int64_t d);
std::vector<at::Tensor> combine_kernel_backward(const at::Tensor& Y, const at::Tensor& tokenId, const at::Tensor& w, const at::Tensor& dOut, int64_t d);
std::vector<at::Tensor> pack_kernel_backward(const at::Tensor& dPackedX, const at::Tensor& dPackedW, const at::Tensor& tokenId,
                                             const at::Tensor& expert, const at::Tensor& topk);

// ---- copies and toys
void copy_scalar(const at::Tensor& src, at::Tensor dst, int64_t n);
void copy_vector(const at::Tensor& src, at::Tensor dst);
void copy_rows_prefix(const at::Tensor& src, at::Tensor dst, const at::Tensor& rows);
void peer_copy_scalar(const at::Tensor& src, at::Tensor dst);
at::Tensor random_op(const at::Tensor& t, int64_t x);

}  // namespace nt
