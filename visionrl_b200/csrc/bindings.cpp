// Python bindings of the visionrl_b200 extension (module visionrl_b200._C).
#include <torch/extension.h>

#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

#include <cstdlib>

#include "head_lse.h"
#include "ops.h"

namespace {
// With VRL_SEGV_TRACE=1 a native backtrace is written to stderr before a SIGSEGV ends the
// process (debugging aid; off by default).
void segv_handler(int sig) {
  void* frames[64];
  const int n = backtrace(frames, 64);
  const char msg[] = "\n[visionrl_b200] SIGSEGV, native frames:\n";
  ssize_t ignored = write(STDERR_FILENO, msg, sizeof(msg) - 1);
  (void)ignored;
  backtrace_symbols_fd(frames, n, STDERR_FILENO);
  signal(sig, SIG_DFL);
  raise(sig);
}
}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "visionrl_b200 sm_100a kernels";
  if (const char* flag = std::getenv("VRL_SEGV_TRACE")) {
    if (flag[0] == '1') signal(SIGSEGV, segv_handler);
  }
  m.def("sde_step_fwd", &vrl::sde_step_fwd);
  m.def("sde_step_bwd", &vrl::sde_step_bwd);
  m.def("sde_rollout_step", &vrl::sde_rollout_step);
  m.def("token_loss_fwd", &vrl::token_loss_fwd);
  m.def("per_sample_mse", &vrl::per_sample_mse);
  m.def("sum_squares", &vrl::sum_squares);
  m.def("colsum", &vrl::colsum);
  m.def("adamw_flat", &vrl::adamw_flat);
  m.def("adaln_fwd", &vrl::adaln_fwd);
  m.def("adaln_bwd", &vrl::adaln_bwd);
  m.def("gate_residual_fwd", &vrl::gate_residual_fwd);
  m.def("gate_residual_bwd", &vrl::gate_residual_bwd);
  m.def("rmsnorm_fwd", &vrl::rmsnorm_fwd);
  m.def("rmsnorm_bwd", &vrl::rmsnorm_bwd);
  m.def("qkv_prepare_fwd", &vrl::qkv_prepare_fwd);
  m.def("qkv_prepare_bwd", &vrl::qkv_prepare_bwd);
  m.def("qkv_prepare_fwd_peers", &vrl::qkv_prepare_fwd_peers);
  m.def("rs_sum_slice", &vrl::rs_sum_slice);
  m.def("adamw_slice_broadcast", &vrl::adamw_slice_broadcast);
  m.def("p2p_broadcast_versioned", &vrl::p2p_broadcast_versioned);
  m.def("wait_flag", &vrl::wait_flag);
  m.def("ulysses_scatter", &vrl::ulysses_scatter);
  m.def("ulysses_exchange_tm", &vrl::ulysses_exchange_tm);
  m.def("flag_signal", &vrl::flag_signal);
  m.def("flag_wait", &vrl::flag_wait);
  m.def("flag_barrier", &vrl::flag_barrier);
  m.def("bucket_reduce_acc", &vrl::bucket_reduce_acc);
  m.def("p2p_gather_rows", &vrl::p2p_gather_rows);
  m.def("p2p_gather_table", &vrl::p2p_gather_table);
  m.def("p2p_broadcast_table", &vrl::p2p_broadcast_table);
  m.def("token_logprob_fwd", &vrl::token_logprob_fwd);
  m.def("token_logprob_bwd", &vrl::token_logprob_bwd);
  m.def("lse_chunk_update", &vrl::lse_chunk_update);
  m.def("softmax_grad_chunk", &vrl::softmax_grad_chunk);
  m.def("sample_tokens", &vrl::sample_tokens);
  m.def("decode_attention", &vrl::decode_attention);
  m.def("group_advantages", &vrl::group_advantages);
  m.def("decode_qkv_rope_append", &vrl::decode_qkv_rope_append);
  m.def("swiglu_rows", &vrl::swiglu_rows);
  m.def("add_rmsnorm_rows", &vrl::add_rmsnorm_rows);
  m.def("int4_gemv", &vrl::int4_gemv);
  m.def("moe_gate_topk", &vrl::moe_gate_topk);
  m.def("moe_permute", &vrl::moe_permute);
  m.def("moe_gather_rows", &vrl::moe_gather_rows);
  m.def("moe_combine", &vrl::moe_combine);
  m.def("moe_combine_bwd", &vrl::moe_combine_bwd);
  m.def("moe_segment_colsum", &vrl::moe_segment_colsum);
  m.def("lora_apply_rows", &vrl::lora_apply_rows);
  m.def("int4_gemm", &vrl::int4_gemm);
  m.def("int4_gemm_last_status", &vrl::int4_gemm_last_status);
  m.def("groupnorm_nhwc", &vrl::groupnorm_nhwc);
  m.def("flash_attn_fwd", &vrl::flash_attn_fwd, pybind11::arg("q"), pybind11::arg("k"), pybind11::arg("v"),
        pybind11::arg("scale"), pybind11::arg("causal") = false, pybind11::arg("variant") = 0);
  m.def("flash_attn_fwd_peers", &vrl::flash_attn_fwd_peers);
  m.def("flash_attn_last_status", &vrl::flash_attn_last_status);
  m.def("flash_attn_bwd", &vrl::flash_attn_bwd, pybind11::arg("dout"), pybind11::arg("q"), pybind11::arg("k"),
        pybind11::arg("v"), pybind11::arg("out"), pybind11::arg("lse"), pybind11::arg("scale"),
        pybind11::arg("causal") = false);
  m.def("flash_attn_bwd_timing", &vrl::flash_attn_bwd_timing);
  m.def("mma_issue_probe", &vrl::mma_issue_probe);
  m.def("gemm_bf16", &vrl::gemm_bf16);
  m.def("gemm_bf16_dual", &vrl::gemm_bf16_dual);
  m.def("gemm_allgather", &vrl::gemm_allgather);
  m.def("head_logprob_fwd", &vrl::head_logprob_fwd);
  m.def("head_softmax_grad", &vrl::head_softmax_grad);
  m.def("gemm_grouped", &vrl::gemm_grouped);
  m.def("gemm_grouped_wgrad", &vrl::gemm_grouped_wgrad);
  m.def("gemm_bf16_acc", &vrl::gemm_bf16_acc);
  m.def("gemm_bf16_out", &vrl::gemm_bf16_out);
  m.def("gemm_last_status", &vrl::gemm_last_status);
  m.def("kernel_status_all", &vrl::kernel_status_all);
}
