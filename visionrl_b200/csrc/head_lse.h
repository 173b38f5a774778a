// Vocabulary head with the log-sum-exp folded into the product's epilogue (gemm_sm100.cu).
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

}  // namespace vrl
