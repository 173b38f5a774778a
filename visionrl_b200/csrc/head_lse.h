// Entry points of gemm_sm100.cu beyond the plain product: the vocabulary head with the log-sum-exp
// folded into the epilogue, and grouped products.
#pragma once

#include <torch/extension.h>

#include <vector>

namespace vrl {

// {log_softmax((h W^T + bias) / T)[ids], row log-sum-exp}, both fp32 [rows]
std::vector<torch::Tensor> head_logprob_fwd(torch::Tensor h, torch::Tensor w, c10::optional<torch::Tensor> bias,
                                            torch::Tensor ids, double temperature);
// bf16 [rows, w.size(0)]: g / T * (onehot(ids - col0) - exp((h W^T + bias) / T - lse))
torch::Tensor head_softmax_grad(torch::Tensor h, torch::Tensor w, c10::optional<torch::Tensor> bias,
                                torch::Tensor ids, torch::Tensor lse, torch::Tensor g, int64_t col0,
                                double temperature);

// grouped products over expert-sorted rows (mixture of experts), see gemm_sm100.cu
std::vector<torch::Tensor> gemm_grouped(torch::Tensor a, torch::Tensor w, torch::Tensor tile_expert,
                                        c10::optional<torch::Tensor> bias, c10::optional<torch::Tensor> residual,
                                        int64_t act, bool w_row_major, bool dual);
torch::Tensor gemm_grouped_wgrad(torch::Tensor gy, torch::Tensor x, torch::Tensor offsets, int64_t experts);

}  // namespace vrl
