// Python bindings of the visionrl_b200 extension (module visionrl_b200._C).
#include <torch/extension.h>

#include "ops.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "visionrl_b200 sm_100a kernels";
  m.def("sde_step_fwd", &vrl::sde_step_fwd);
  m.def("sde_step_bwd", &vrl::sde_step_bwd);
  m.def("token_loss_fwd", &vrl::token_loss_fwd);
  m.def("per_sample_mse", &vrl::per_sample_mse);
  m.def("sum_squares", &vrl::sum_squares);
  m.def("adamw_flat", &vrl::adamw_flat);
  m.def("adaln_fwd", &vrl::adaln_fwd);
  m.def("adaln_bwd", &vrl::adaln_bwd);
  m.def("rmsnorm_fwd", &vrl::rmsnorm_fwd);
  m.def("rmsnorm_bwd", &vrl::rmsnorm_bwd);
  m.def("qkv_prepare_fwd", &vrl::qkv_prepare_fwd);
  m.def("qkv_prepare_bwd", &vrl::qkv_prepare_bwd);
  m.def("gemm_bf16", &vrl::gemm_bf16);
  m.def("gemm_last_status", &vrl::gemm_last_status);
}
