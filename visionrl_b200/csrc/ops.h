// Host entry points of the visionrl_b200 extension.
#pragma once

#include <cuda_runtime_api.h>
#include <torch/extension.h>

#include <vector>

namespace vrl {

// Operand checks shared by every host wrapper.  A wrapper hands raw pointers to its kernel, so EVERY
// tensor operand (not only the first) must live on the launch device; a CPU tensor or one on another
// GPU has to fail here as a Python error, never as an illegal address inside the kernel.
inline void check_operand(const torch::Tensor& t, const torch::Tensor& ref, const char* name,
                          c10::optional<c10::ScalarType> dtype = c10::nullopt, int64_t numel = -1) {
  TORCH_CHECK(t.defined(), name, ": undefined tensor");
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (got ", t.device(), ")");
  TORCH_CHECK(t.device() == ref.device(), name, " is on ", t.device(), " but the launch device is ",
              ref.device());
  if (dtype.has_value())
    TORCH_CHECK(t.scalar_type() == *dtype, name, " must have dtype ", *dtype, " (got ", t.scalar_type(), ")");
  if (numel >= 0) TORCH_CHECK(t.numel() == numel, name, " must have ", numel, " elements (got ", t.numel(), ")");
}
inline void check_operand(const c10::optional<torch::Tensor>& t, const torch::Tensor& ref, const char* name,
                          c10::optional<c10::ScalarType> dtype = c10::nullopt, int64_t numel = -1) {
  if (t.has_value()) check_operand(*t, ref, name, dtype, numel);
}
#define VRL_CHECK_OPERAND(t, ref, ...) ::vrl::check_operand((t), (ref), #t, ##__VA_ARGS__)

// status.cpp: the per-device block of kernel status words (one 16-byte read polls them all)
constexpr int kStatusWords = 4;
enum StatusIndex : int { kStatusGemm = 0, kStatusAttention = 1, kStatusInt4Gemm = 2 };
int* kernel_status_block(int device);
std::vector<int64_t> kernel_status_all();      // {gemm, attention, int4 gemm}; clears what it read

// elementwise.cu
int sde_blocks_per_sample(int64_t n);
void sde_step_launch(const float* v, const float* x, const float* a, const float* b,
                     const float* scale, const float* dt, const float* prev_in,
                     const float* noise, float* prev_out, float* mean_out, float* logp,
                     float* partial, int batch, int64_t n, bool deterministic, bool gaussian,
                     cudaStream_t stream);
std::vector<torch::Tensor> sde_step_fwd(torch::Tensor v, torch::Tensor x, torch::Tensor a,
                                        torch::Tensor b, torch::Tensor scale, torch::Tensor dt,
                                        c10::optional<torch::Tensor> prev_sample,
                                        c10::optional<torch::Tensor> noise, bool deterministic,
                                        bool gaussian);
void sde_rollout_step(torch::Tensor pred, bool has_cfg, double guidance, int64_t cfg_form,
                      torch::Tensor path, int64_t step, torch::Tensor a, torch::Tensor b,
                      torch::Tensor scale, torch::Tensor dt, c10::optional<torch::Tensor> noise,
                      int64_t seed, int64_t offset, torch::Tensor log_probs, bool deterministic,
                      bool gaussian);
std::vector<torch::Tensor> sde_step_bwd(torch::Tensor prev, torch::Tensor mean, torch::Tensor a,
                                        torch::Tensor b, torch::Tensor scale, torch::Tensor g_logp,
                                        c10::optional<torch::Tensor> g_mean, bool gaussian);
std::vector<torch::Tensor> token_loss_fwd(torch::Tensor lp, torch::Tensor old, torch::Tensor adv,
                                          c10::optional<torch::Tensor> mask,
                                          c10::optional<torch::Tensor> ref, double eps_clip,
                                          bool k3);
torch::Tensor per_sample_mse(torch::Tensor pred, torch::Tensor target);
torch::Tensor sum_squares(torch::Tensor g);
torch::Tensor colsum(torch::Tensor x);
void adamw_flat(torch::Tensor p, torch::Tensor g, torch::Tensor master, torch::Tensor m,
                torch::Tensor v, double lr, double b1, double b2, double eps, double wd,
                int64_t step, c10::optional<torch::Tensor> clip);

// norm.cu
std::vector<torch::Tensor> adaln_fwd(torch::Tensor x, torch::Tensor shift, torch::Tensor scale,
                                     double eps);
std::vector<torch::Tensor> adaln_bwd(torch::Tensor gy, torch::Tensor x, torch::Tensor scale,
                                     torch::Tensor mean, torch::Tensor rstd);
torch::Tensor gate_residual_fwd(torch::Tensor y, torch::Tensor gate, torch::Tensor residual);
std::vector<torch::Tensor> gate_residual_bwd(torch::Tensor g, torch::Tensor y, torch::Tensor gate);
std::vector<torch::Tensor> rmsnorm_fwd(torch::Tensor x, torch::Tensor w, double eps);
std::vector<torch::Tensor> rmsnorm_bwd(torch::Tensor gy, torch::Tensor x, torch::Tensor w,
                                       torch::Tensor rstd);
std::vector<torch::Tensor> qkv_prepare_fwd(torch::Tensor qkv, c10::optional<torch::Tensor> qw,
                                           c10::optional<torch::Tensor> kw,
                                           c10::optional<torch::Tensor> cos,
                                           c10::optional<torch::Tensor> sin, int64_t heads,
                                           double eps, c10::optional<torch::Tensor> dst_q,
                                           c10::optional<torch::Tensor> dst_k,
                                           c10::optional<torch::Tensor> dst_v, int64_t seq_offset);
torch::Tensor qkv_prepare_fwd_peers(torch::Tensor qkv, c10::optional<torch::Tensor> qw,
                                    c10::optional<torch::Tensor> kw, c10::optional<torch::Tensor> cos,
                                    c10::optional<torch::Tensor> sin, int64_t heads, double eps,
                                    torch::Tensor peers_q, torch::Tensor peers_k, torch::Tensor peers_v,
                                    int64_t world, int64_t seq_total, int64_t seq_offset);
std::vector<torch::Tensor> qkv_prepare_bwd(torch::Tensor gq, torch::Tensor gk, torch::Tensor gv,
                                           torch::Tensor qkv, c10::optional<torch::Tensor> qw,
                                           c10::optional<torch::Tensor> kw,
                                           c10::optional<torch::Tensor> cos,
                                           c10::optional<torch::Tensor> sin, torch::Tensor rstd,
                                           int64_t heads, int64_t seq_offset);

// collective.cu
torch::Tensor rs_sum_slice(torch::Tensor peers, torch::Tensor out, int64_t lo, int64_t n,
                           int64_t world, int64_t rank, bool is_bf16, double scale);
void adamw_slice_broadcast(torch::Tensor peers, torch::Tensor g, torch::Tensor master,
                           torch::Tensor m, torch::Tensor v, int64_t lo, int64_t n, int64_t world,
                           int64_t rank, double lr, double b1, double b2, double eps, double wd,
                           int64_t step, c10::optional<torch::Tensor> clip, bool is_bf16);
void p2p_broadcast_versioned(torch::Tensor src, torch::Tensor dst_peers, int64_t dst_offset_bytes,
                             torch::Tensor flag_peers, int64_t flag_slot, int64_t world,
                             int64_t rank, int64_t version, bool include_self);
torch::Tensor wait_flag(torch::Tensor flags, int64_t slot, int64_t expected, double timeout_s);
void flag_signal(torch::Tensor flag_peers, torch::Tensor flags, int64_t slot, int64_t world, int64_t value);
void flag_wait(torch::Tensor flags, int64_t slot0, int64_t count, int64_t expected, double timeout_s,
               torch::Tensor status);
void flag_barrier(torch::Tensor flag_peers, torch::Tensor flags, int64_t base, int64_t world, int64_t rank,
                  int64_t epoch, double timeout_s, torch::Tensor status);
void bucket_reduce_acc(torch::Tensor stage_peers, torch::Tensor table, torch::Tensor gshard, double scale,
                       int64_t world, int64_t rank, int64_t max_segment);
void p2p_broadcast_table(torch::Tensor src_flat, torch::Tensor dst_peers, torch::Tensor table,
                         int64_t world, int64_t rank, int64_t max_segment);
void p2p_gather_table(torch::Tensor shard_peers, torch::Tensor dst, torch::Tensor table, int64_t world,
                      int64_t rank, int64_t max_segment);
void p2p_gather_rows(torch::Tensor shard_peers, torch::Tensor full, int64_t shard_elems, int64_t world,
                     int64_t rank);
void ulysses_exchange_tm(torch::Tensor src, torch::Tensor dst_peers, int64_t batch, int64_t s_loc,
                         int64_t chunk_elems, int64_t world, int64_t rank, bool to_heads);
void ulysses_scatter(torch::Tensor src, torch::Tensor dst_peers, int64_t batch, int64_t heads,
                     int64_t s_loc, int64_t head_dim, int64_t world, int64_t rank, bool to_heads);

// ar_ops.cu
std::vector<torch::Tensor> token_logprob_fwd(torch::Tensor logits, torch::Tensor ids, double temperature);
torch::Tensor token_logprob_bwd(torch::Tensor logits, torch::Tensor ids, torch::Tensor lse,
                                torch::Tensor g, double temperature);
void lse_chunk_update(torch::Tensor chunk, torch::Tensor ids, torch::Tensor run_max,
                      torch::Tensor run_sum, torch::Tensor target, int64_t col0, double temperature);
torch::Tensor softmax_grad_chunk(torch::Tensor chunk, torch::Tensor ids, torch::Tensor lse,
                                 torch::Tensor g, int64_t col0, double temperature);
std::vector<torch::Tensor> sample_tokens(torch::Tensor cond, torch::Tensor uncond, torch::Tensor u,
                                         double cfg_weight, double temperature);
torch::Tensor decode_attention(torch::Tensor q, torch::Tensor k_cache, torch::Tensor v_cache,
                               torch::Tensor valid, int64_t length, double scale);
torch::Tensor decode_qkv_rope_append(torch::Tensor qkv, torch::Tensor cos, torch::Tensor sin, torch::Tensor pos,
                                     torch::Tensor k_cache, torch::Tensor v_cache, int64_t heads);
torch::Tensor swiglu_rows(torch::Tensor gate_up);
torch::Tensor add_rmsnorm_rows(torch::Tensor x, c10::optional<torch::Tensor> delta, torch::Tensor w, double eps);
torch::Tensor group_advantages(torch::Tensor rewards, torch::Tensor group_ids, double eps, double clip,
                               bool global_std);

// quant_moe.cu
torch::Tensor int4_gemv(torch::Tensor x, torch::Tensor qweight, torch::Tensor scales,
                        c10::optional<torch::Tensor> bias, int64_t group);
std::vector<torch::Tensor> moe_gate_topk(torch::Tensor logits, int64_t topk);
std::vector<torch::Tensor> moe_permute(torch::Tensor experts, int64_t num_experts, int64_t pad);
std::vector<torch::Tensor> moe_combine_bwd(torch::Tensor gy, torch::Tensor yp, torch::Tensor perm,
                                           torch::Tensor inv, torch::Tensor weights);
torch::Tensor moe_segment_colsum(torch::Tensor g, torch::Tensor offsets, int64_t num_experts);
void lora_apply_rows(torch::Tensor y, torch::Tensor x, torch::Tensor a, torch::Tensor b, double scale);
torch::Tensor moe_gather_rows(torch::Tensor x, torch::Tensor perm, int64_t topk);
torch::Tensor moe_combine(torch::Tensor yp, torch::Tensor inv, torch::Tensor weights);

// int4_gemm_sm100.cu
torch::Tensor int4_gemm(torch::Tensor x, torch::Tensor qweight, torch::Tensor scales,
                        c10::optional<torch::Tensor> bias, int64_t group);
int64_t int4_gemm_last_status();

// groupnorm.cu
torch::Tensor groupnorm_nhwc(torch::Tensor x, torch::Tensor weight, torch::Tensor bias, int64_t groups,
                             double eps, bool apply_silu);

// attention_sm100.cu
std::vector<torch::Tensor> flash_attn_fwd(torch::Tensor q, torch::Tensor k, torch::Tensor v, double scale,
                                          bool causal, int64_t variant);
std::vector<torch::Tensor> flash_attn_fwd_peers(torch::Tensor q, torch::Tensor k, torch::Tensor v, double scale,
                                                torch::Tensor out_peers, int64_t world, int64_t rank,
                                                int64_t heads_total);
int64_t flash_attn_last_status();

// attention_bwd_sm100.cu
std::vector<torch::Tensor> flash_attn_bwd(torch::Tensor dout, torch::Tensor q, torch::Tensor k, torch::Tensor v,
                                          torch::Tensor out, torch::Tensor lse, double scale, bool causal);
torch::Tensor flash_attn_bwd_timing(bool enable);

// mma_probe.cu
torch::Tensor mma_issue_probe(int64_t n, int64_t iters, int64_t group, bool commit_each, int64_t wait_each,
                              bool tmem_a);

// gemm_sm100.cu
torch::Tensor gemm_bf16(torch::Tensor a, torch::Tensor b, c10::optional<torch::Tensor> bias,
                        c10::optional<torch::Tensor> gate, c10::optional<torch::Tensor> residual,
                        int64_t act, int64_t rows_per_gate, bool a_mn_major, bool b_mn_major,
                        bool out_fp32);
std::vector<torch::Tensor> gemm_bf16_dual(torch::Tensor a, torch::Tensor b,
                                          c10::optional<torch::Tensor> bias, int64_t act);
std::vector<torch::Tensor> gemm_allgather(torch::Tensor x, torch::Tensor peer_ptrs, torch::Tensor full,
                                          torch::Tensor ready, c10::optional<torch::Tensor> bias, int64_t act,
                                          int64_t rank, int64_t world, c10::optional<torch::Tensor> gate,
                                          c10::optional<torch::Tensor> residual, int64_t rows_per_gate,
                                          bool dual);
void gemm_bf16_out(torch::Tensor a, torch::Tensor b, torch::Tensor out, bool a_mn_major, bool b_mn_major);
void gemm_bf16_acc(torch::Tensor a, torch::Tensor b, torch::Tensor acc, bool a_mn_major, bool b_mn_major);
int64_t gemm_last_status();

}  // namespace vrl
