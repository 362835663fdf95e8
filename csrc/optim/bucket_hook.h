// Native DDP communication hook: per gradient bucket, ONE call enqueues the fused-average
// allreduce and, right behind it on the same communication stream, the AdamW update of the
// bucket's parameters.  Registered directly on DDP's C++ reducer, so no Python runs (and the GIL
// is never taken) between the moment autograd marks a bucket ready and the moment its kernels are
// queued; the optimizer work of early buckets overlaps the rest of backward and the serial
// "optimizer tail" after backward disappears.
//
// Python keeps ownership of the optimizer: it registers the parameters with their state tensors and
// param-group index once, pushes the groups' current hyper-parameters and the step number before
// every forward (so learning-rate schedulers keep working), and after backward asks which
// parameters were stepped here so that `optimizer.step()` only handles the rest and refreshes the
// step counters.  A bucket that spans several param groups is split into one launch plan per group.
//
// The reference has no optimizer integration; this belongs to the DDP overlap machinery
// (reference csrc/backend/ProcessGroupMCCL.cpp:1165-1378 is the allreduce entry it rides on).
#pragma once

#include <torch/csrc/distributed/c10d/comm.hpp>
#include <torch/csrc/distributed/c10d/reducer.hpp>

#include <map>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "backend/process_group.h"
#include "common/env.h"
#include "optim/adamw_plan.h"

namespace mccl {

struct BucketOptimizerState {
  struct Hyper {
    double lr = 1e-3, beta1 = 0.9, beta2 = 0.999, eps = 1e-8, weight_decay = 1e-2;
  };
  struct ParamEntry {
    at::Tensor p, m, v;
    int group = 0;
  };
  struct BucketPlan {
    std::vector<int64_t> signature;                      // addresses of the bucket's parameters
    std::vector<std::unique_ptr<AdamWPlan>> plans;       // one per param group present in the bucket
    std::vector<int> groups;
    std::vector<std::vector<size_t>> positions;          // indices into the bucket's parameter list
  };

  BucketOptimizerState(c10::intrusive_ptr<ProcessGroupMCCL> pg_, double scale_) : pg(std::move(pg_)), scale(scale_) {}

  void add_param(const at::Tensor& p, const at::Tensor& m, const at::Tensor& v, int group) {
    std::lock_guard<std::mutex> g(mu);
    params[reinterpret_cast<int64_t>(p.data_ptr())] = ParamEntry{p, m, v, group};
    buckets.clear();
  }
  void set_hyper(int group, double lr, double b1, double b2, double eps, double wd) {
    std::lock_guard<std::mutex> g(mu);
    if (static_cast<int>(hyper.size()) <= group) hyper.resize(group + 1);
    hyper[group] = Hyper{lr, b1, b2, eps, wd};
  }
  void set_step(int64_t s) {
    std::lock_guard<std::mutex> g(mu);
    step = s;
  }
  // (step used, addresses of the parameters updated since the last call)
  std::pair<int64_t, std::vector<int64_t>> take_stepped() {
    std::lock_guard<std::mutex> g(mu);
    std::pair<int64_t, std::vector<int64_t>> out{step, std::move(stepped)};
    stepped.clear();
    return out;
  }

  c10::intrusive_ptr<ProcessGroupMCCL> pg;
  double scale;
  std::mutex mu;
  std::unordered_map<int64_t, ParamEntry> params;
  std::vector<Hyper> hyper;
  int64_t step = 1;
  std::vector<int64_t> stepped;
  std::map<size_t, BucketPlan> buckets;
};

class BucketOptimizerHook : public c10d::CommHookInterface {
 public:
  explicit BucketOptimizerHook(std::shared_ptr<BucketOptimizerState> st) : st_(std::move(st)) {}

  c10::intrusive_ptr<c10::ivalue::Future> runHook(c10d::GradBucket& bucket) override {
    BucketOptimizerState& st = *st_;
    std::unique_lock<std::mutex> lk(st.mu);
    const std::vector<at::Tensor> params = bucket.getParameters();
    const std::vector<at::Tensor> grads = bucket.getGradients();
    std::vector<int64_t> sig;
    sig.reserve(params.size());
    for (const auto& p : params) sig.push_back(reinterpret_cast<int64_t>(p.data_ptr()));
    BucketOptimizerState::BucketPlan& bp = st.buckets[bucket.getIndex()];
    if (bp.signature != sig) {  // first use, or DDP rebuilt its buckets
      bp = BucketOptimizerState::BucketPlan();
      bp.signature = sig;
      std::map<int, std::vector<size_t>> by_group;
      for (size_t i = 0; i < params.size(); ++i) {
        auto it = st.params.find(sig[i]);
        MCCL_CHECK(it != st.params.end(), "a DDP bucket holds a parameter the optimizer was not given");
        by_group[it->second.group].push_back(i);
      }
      for (auto& kv : by_group) {
        std::vector<at::Tensor> ps, ms, vs;
        for (size_t i : kv.second) {
          const auto& e = st.params.at(sig[i]);
          ps.push_back(e.p);
          ms.push_back(e.m);
          vs.push_back(e.v);
        }
        bp.plans.push_back(std::make_unique<AdamWPlan>(ps, ms, vs));
        bp.groups.push_back(kv.first);
        bp.positions.push_back(kv.second);
      }
    }
    struct Launch {
      AdamWPlan* plan;
      BucketOptimizerState::Hyper h;
    };
    std::vector<Launch> launches;
    for (size_t k = 0; k < bp.plans.size(); ++k) {
      std::vector<at::Tensor> gs;
      for (size_t i : bp.positions[k]) gs.push_back(grads[i]);
      bp.plans[k]->bind_grads(gs);  // uploads the address table only when an address changed
      MCCL_CHECK(bp.groups[k] < static_cast<int>(st.hyper.size()), "hyper-parameters of param group " << bp.groups[k] << " were never set");
      launches.push_back({bp.plans[k].get(), st.hyper[bp.groups[k]]});
    }
    for (int64_t a : sig) st.stepped.push_back(a);
    const int64_t step = st.step;
    const float scale = static_cast<float>(st.scale);
    lk.unlock();
    std::vector<at::Tensor> v{bucket.getBufferRef()};
    // the last bucket of a backward pass has no backward kernels left to share the GPU with
    // (MCCL_LAST_BUCKET_ALONE=1 lets its allreduce use the larger, non-overlapped grid)
    static const bool last_alone = env_int("MCCL_LAST_BUCKET_ALONE", 0) != 0;
    const bool overlapped = !(last_alone && bucket.isLast());
    // A bucket's update runs beside the rest of backward: MCCL_OIB_ADAMW_CTAS caps its grid so that it
    // takes a share of the SMs and of HBM bandwidth instead of all of both (0 = no cap).  The last
    // bucket has nothing beside it and always runs uncapped.
    static const int capped = static_cast<int>(env_int("MCCL_OIB_ADAMW_CTAS", 0));
    const int max_ctas = bucket.isLast() ? 0 : capped;
    auto work = st.pg->allreduce_scaled_then(v, scale, [launches, step, max_ctas](cudaStream_t s) {
      for (const auto& l : launches)
        l.plan->launch(s, l.h.lr, l.h.beta1, l.h.beta2, l.h.eps, l.h.weight_decay, step, 1.0, max_ctas);
    }, overlapped);
    return work->getFuture();
  }

  at::Tensor parseHookResult(const c10::IValue& result) override {
    TORCH_INTERNAL_ASSERT(result.isTensorList() || result.isTensor(), "unexpected result of the bucket hook");
    return result.isTensor() ? result.toTensor() : result.toTensorVector()[0];
  }

 private:
  std::shared_ptr<BucketOptimizerState> st_;
};

}  // namespace mccl
