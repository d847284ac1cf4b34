// B200ModelBackend: the reference's IModelBackend implemented on librwkv7_b200.so.
//
// This file is compiled INSIDE the reference project (it includes the reference's own
// include/rwkv_server_backend.hpp, so GenerationState / DeviceLogits / DeviceBuffer are the
// reference's types, unchanged) and linked against librwkv7_b200.so.  The engine, sampler, state
// cache and HTTP layer of the reference keep working unmodified: construct this class where
// src/rwkv_fast_server.cpp:188-189 and src/rwkv_model_router.cpp:101-102 construct ModelBackend.
#pragma once

#include <string>
#include <vector>

#include "rwkv_server_backend.hpp"  // from the reference tree

struct rwkv7_b200_model;

namespace rwkv7_server {

class B200ModelBackend final : public IModelBackend {
 public:
  // Same arguments as ModelBackend (include/rwkv_server_backend.hpp:106-109); weight_format is one of
  // RWKV7_B200_FMT_* (0 = fp16 like the reference).
  explicit B200ModelBackend(std::string model_path, bool use_wkv32 = false, bool chunk_load = false, int weight_format = 0);
  ~B200ModelBackend() override;
  B200ModelBackend(const B200ModelBackend&) = delete;
  B200ModelBackend& operator=(const B200ModelBackend&) = delete;

  GenerationState create_state(int batch_size) const override;
  void forward_prefill(const std::vector<std::vector<int64_t>>& token_batches, GenerationState& state,
                       DeviceLogits& logits) const override;
  void forward_decode(const std::vector<int64_t>& token_batch, GenerationState& state, DeviceLogits& logits) const override;
  // Not part of IModelBackend: `steps` decode steps with the sampler's greedy case (top_p == 0,
  // src/utils/sampling.cu:507-512) applied on the device after each one; returns the ids [steps][B].  `penalties` is the
  // sampler state's device array fp32 [B][vocab] (src/rwkv_sampler.cpp:47-111 passes the same one to its kernel) or null.
  std::vector<int> decode_greedy(const std::vector<int64_t>& token_batch, int steps, GenerationState& state,
                                 DeviceLogits& logits, float* penalties, double alpha_presence, double alpha_frequency,
                                 double alpha_decay) const;
  void copy_state_slice(const GenerationState& src, int src_offset, GenerationState& dst, int dst_offset,
                        int count) const override;
  void copy_logits_slice(const DeviceLogits& src, int src_offset, DeviceLogits& dst, int dst_offset,
                         int count) const override;
  PrefillCapacity query_prefill_capacity(int prefill_chunk_size) const override;
  int vocab_size() const override;
  const std::string& model_path() const override { return model_path_; }
  const std::string& model_name() const override { return model_name_; }

 private:
  void run(const int64_t* tokens, int B, int T, GenerationState& state, DeviceLogits& logits) const;
  std::string model_path_, model_name_;
  bool use_wkv32_ = false;
  rwkv7_b200_model* model_ = nullptr;
  cudaStream_t stream_ = nullptr;
};

}  // namespace rwkv7_server
