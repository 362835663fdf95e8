// AdamWPlan: device-resident launch plan of the fused multi-tensor AdamW kernel
// (kernels/adamw.cu): pointer tables of the parameters and their optimizer state, uploaded once,
// plus the table of gradient addresses, re-uploaded only when an address changed.
#pragma once

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cmath>
#include <vector>

#include "backend/tensor_checks.h"
#include "common/errors.h"
#include "kernels/optim_api.h"

namespace mccl {

#define MCCL_PLAN_CK(expr)                                                        \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess) {                                                      \
      cudaGetLastError();                                                         \
      throw DeviceError(std::string(#expr) + ": " + cudaGetErrorString(_e));      \
    }                                                                             \
  } while (0)

class AdamWPlan {
 public:
  AdamWPlan(std::vector<at::Tensor> params, std::vector<at::Tensor> exp_avg, std::vector<at::Tensor> exp_avg_sq)
      : params_(std::move(params)), m_(std::move(exp_avg)), v_(std::move(exp_avg_sq)) {
    MCCL_CHECK_TENSOR(!params_.empty() && params_.size() == m_.size() && params_.size() == v_.size(),
                      "AdamWPlan: list sizes differ");
    std::vector<int64_t> ptr_p, ptr_m, ptr_v, sizes;
    std::vector<int32_t> chunks;
    for (size_t i = 0; i < params_.size(); ++i) {
      for (const at::Tensor* t : {&params_[i], &m_[i], &v_[i]}) {
        MCCL_CHECK_TENSOR(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous(),
                          "AdamWPlan: float32 contiguous CUDA tensors only");
        MCCL_CHECK_TENSOR(t->numel() == params_[i].numel() && t->device() == params_[0].device(),
                          "AdamWPlan: shape/device mismatch");
      }
      ptr_p.push_back(reinterpret_cast<int64_t>(params_[i].data_ptr()));
      ptr_m.push_back(reinterpret_cast<int64_t>(m_[i].data_ptr()));
      ptr_v.push_back(reinterpret_cast<int64_t>(v_[i].data_ptr()));
      const int64_t n = params_[i].numel();
      sizes.push_back(n);
      for (int64_t c = 0; c * kern::kAdamWChunk < n; ++c) {
        chunks.push_back(static_cast<int32_t>(i));
        chunks.push_back(static_cast<int32_t>(c));
      }
    }
    auto dev = params_[0].device();
    auto up64 = [&](const std::vector<int64_t>& v) {
      return at::tensor(v, at::TensorOptions().dtype(at::kLong)).to(dev);
    };
    d_p_ = up64(ptr_p);
    d_m_ = up64(ptr_m);
    d_v_ = up64(ptr_v);
    d_sizes_ = up64(sizes);
    d_chunks_ = at::tensor(chunks, at::TensorOptions().dtype(at::kInt)).to(dev);
    num_chunks_ = static_cast<int>(chunks.size() / 2);
    grad_ptrs_.assign(params_.size(), 0);
    d_g_ = at::zeros({static_cast<int64_t>(params_.size())}, at::TensorOptions().dtype(at::kLong).device(dev));
  }

  // grads[i] may move between steps (zero_grad(set_to_none=True)); the pointer
  // table is re-uploaded only when an address changed.
  void step(const std::vector<at::Tensor>& grads, double lr, double beta1, double beta2, double eps,
            double weight_decay, int64_t step, double grad_scale) {
    bind_grads(grads);
    c10::cuda::CUDAGuard guard(params_[0].device());
    launch(at::cuda::getCurrentCUDAStream(), lr, beta1, beta2, eps, weight_decay, step, grad_scale);
  }

  // Points the plan at `grads` (uploads the pointer table only when an address changed).
  void bind_grads(const std::vector<at::Tensor>& grads) {
    MCCL_CHECK_TENSOR(grads.size() == params_.size(), "AdamWPlan.step: expected one gradient per parameter");
    bool changed = false;
    for (size_t i = 0; i < grads.size(); ++i) {
      const at::Tensor& g = grads[i];
      MCCL_CHECK_TENSOR(g.is_cuda() && g.scalar_type() == at::kFloat && g.is_contiguous() &&
                            g.numel() == params_[i].numel(),
                        "AdamWPlan.step: gradient " << i << " must be a float32 contiguous CUDA tensor of the parameter's size");
      int64_t a = reinterpret_cast<int64_t>(g.data_ptr());
      if (a != grad_ptrs_[i]) {
        grad_ptrs_[i] = a;
        changed = true;
      }
    }
    if (changed) {
      c10::cuda::CUDAGuard guard(params_[0].device());
      at::Tensor host = at::tensor(grad_ptrs_, at::TensorOptions().dtype(at::kLong));
      d_g_.copy_(host);
    }
  }

  void launch(cudaStream_t stream, double lr, double beta1, double beta2, double eps, double weight_decay,
              int64_t step, double grad_scale, int max_ctas = 0) {
    kern::AdamWTable tab;
    tab.params = reinterpret_cast<const uint64_t*>(d_p_.data_ptr<int64_t>());
    tab.grads = reinterpret_cast<const uint64_t*>(d_g_.data_ptr<int64_t>());
    tab.exp_avg = reinterpret_cast<const uint64_t*>(d_m_.data_ptr<int64_t>());
    tab.exp_avg_sq = reinterpret_cast<const uint64_t*>(d_v_.data_ptr<int64_t>());
    tab.sizes = d_sizes_.data_ptr<int64_t>();
    tab.chunks = reinterpret_cast<const int2*>(d_chunks_.data_ptr<int32_t>());
    tab.num_chunks = num_chunks_;
    kern::AdamWHyper h;
    h.lr = static_cast<float>(lr);
    h.beta1 = static_cast<float>(beta1);
    h.beta2 = static_cast<float>(beta2);
    h.eps = static_cast<float>(eps);
    h.weight_decay = static_cast<float>(weight_decay);
    const double bc1 = 1.0 - std::pow(beta1, static_cast<double>(step));
    const double bc2 = 1.0 - std::pow(beta2, static_cast<double>(step));
    h.step_size = static_cast<float>(lr / bc1);
    h.inv_sqrt_bias2 = static_cast<float>(1.0 / std::sqrt(bc2));
    h.grad_scale = static_cast<float>(grad_scale);
    MCCL_PLAN_CK(kern::launch_adamw_multi(tab, h, stream, max_ctas));
  }
  int num_chunks() const { return num_chunks_; }

 private:
  std::vector<at::Tensor> params_, m_, v_;
  std::vector<int64_t> grad_ptrs_;
  at::Tensor d_p_, d_g_, d_m_, d_v_, d_sizes_, d_chunks_;
  int num_chunks_ = 0;
};


}  // namespace mccl
