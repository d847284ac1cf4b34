// See b200_model_backend.hpp.  Error behaviour mirrors the reference backend
// (src/rwkv7_fast_v4.cu:1053-1072,1373-1592): argument errors throw std::runtime_error with the
// same messages; CUDA errors also throw (the reference exits the process instead).
#include "b200_model_backend.hpp"

#include <stdexcept>
#include <unordered_map>

#include "rwkv7_b200.h"

namespace rwkv7_server {
namespace {

void check(int status) {
  if (status != RWKV7_B200_OK) throw std::runtime_error(rwkv7_b200_last_error());
}

std::string base_name(const std::string& path) {
  const size_t slash = path.find_last_of("/\\");
  std::string name = slash == std::string::npos ? path : path.substr(slash + 1);
  const size_t dot = name.find_last_of('.');
  return dot == std::string::npos ? name : name.substr(0, dot);
}

}  // namespace

B200ModelBackend::B200ModelBackend(std::string model_path, bool use_wkv32, bool chunk_load, int weight_format)
    : model_path_(std::move(model_path)), model_name_(base_name(model_path_)), use_wkv32_(use_wkv32) {
  // The checkpoint is read with the reference's own zip/pickle reader (src/pth_archive.cpp, src/pth_tensor.cpp).
  auto archive = llm_infer::PthArchive::open(model_path_, chunk_load);
  if (!archive.ok()) throw std::runtime_error(archive.status().message());
  auto records = llm_infer::parse_pth_tensor_records(archive.value());
  if (!records.ok()) throw std::runtime_error(records.status().message());
  const rwkv7_fast_v4::ModelDims dims = rwkv7_fast_v4::infer_model_dims(records.value());

  rwkv7_b200_config cfg{};
  cfg.layers = dims.layers; cfg.channels = dims.channels; cfg.ffn = dims.ffn; cfg.vocab = dims.vocab;
  cfg.weight_format = weight_format; cfg.wkv32 = use_wkv32 ? 1 : 0; cfg.device = -1; cfg.tp_size = 1;
  for (const auto& rec : records.value()) {  // LoRA ranks come from the tensor shapes (src/rwkv7_fast_v4.cu:1168-1171)
    if (rec.shape.size() != 2) continue;
    if (rec.name == "blocks.0.att.w1") cfg.rank_w = static_cast<int>(rec.shape[1]);
    if (rec.name == "blocks.0.att.a1") cfg.rank_a = static_cast<int>(rec.shape[1]);
    if (rec.name == "blocks.0.att.g1") cfg.rank_g = static_cast<int>(rec.shape[1]);
    if (rec.name == "blocks.1.att.v1") cfg.rank_v = static_cast<int>(rec.shape[1]);
  }
  if (cfg.rank_v == 0) cfg.rank_v = 8;  // single-layer model: the value residual is never used
  check(rwkv7_b200_model_create(&cfg, &model_));
  for (const auto& rec : records.value()) {
    if (rec.name == "blocks.0.att.v0" || rec.name == "blocks.0.att.v1" || rec.name == "blocks.0.att.v2") continue;
    auto data = llm_infer::load_bf16_tensor_select(archive.value(), rec, true, false, false);
    if (!data.ok()) throw std::runtime_error(data.status().message());
    const auto& bits = data.value().values_bf16;
    check(rwkv7_b200_model_set_tensor(model_, rec.name.c_str(), bits.data(), RWKV7_B200_DT_BF16,
                                      static_cast<long long>(bits.size()), 0));
  }
  check(rwkv7_b200_model_finalize(model_));
  if (cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking) != cudaSuccess) throw std::runtime_error("create backend stream");
}

B200ModelBackend::~B200ModelBackend() {
  if (stream_) cudaStreamDestroy(stream_);
  rwkv7_b200_model_destroy(model_);
}

GenerationState B200ModelBackend::create_state(int batch_size) const {
  size_t ns = 0, nw = 0, ne = 0;
  check(rwkv7_b200_state_sizes(model_, batch_size, &ns, &nw, &ne));
  GenerationState st;
  st.batch_size = batch_size;
  st.wkv32 = use_wkv32_;
  st.shift.resize(ns, "alloc backend shift state");
  if (use_wkv32_) st.wkv_state32.resize(nw, "alloc backend wkv32 state");
  else st.wkv_state.resize(nw, "alloc backend wkv state");
  st.elapsed.resize(ne, "alloc backend elapsed");
  void* wkv = use_wkv32_ ? static_cast<void*>(st.wkv_state32.p) : static_cast<void*>(st.wkv_state.p);
  check(rwkv7_b200_state_init(model_, batch_size, st.shift.p, wkv, st.elapsed.p, stream_));
  if (cudaStreamSynchronize(stream_) != cudaSuccess) throw std::runtime_error("sync backend state init");
  return st;
}

void B200ModelBackend::run(const int64_t* tokens, int B, int T, GenerationState& state, DeviceLogits& logits) const {
  if (state.batch_size != B) throw std::runtime_error("state batch size mismatch");
  if (state.wkv32 != use_wkv32_) throw std::runtime_error("state wkv precision mismatch");
  logits.rows = B;
  logits.vocab_size = vocab_size();
  logits.values.resize(static_cast<size_t>(B) * logits.vocab_size, "alloc backend logits f32");
  void* wkv = use_wkv32_ ? static_cast<void*>(state.wkv_state32.p) : static_cast<void*>(state.wkv_state.p);
  check(rwkv7_b200_forward(model_, tokens, B, T, state.shift.p, wkv, state.elapsed.p, logits.values.p, stream_));
  // synchronous on return, like the reference (src/rwkv7_fast_v4.cu:1343): callers use stream 0 next
  if (cudaStreamSynchronize(stream_) != cudaSuccess) throw std::runtime_error("sync backend stream");
  // a kernel that gave up on a bounded wait left this call's logits and state incomplete: report it like any other error
  int flags = 0;
  check(rwkv7_b200_timeout_flags(1, &flags));
  if (flags) throw std::runtime_error("rwkv7_b200: a bounded wait inside a kernel ran out (flags " + std::to_string(flags) + ")");
}

void B200ModelBackend::forward_prefill(const std::vector<std::vector<int64_t>>& token_batches, GenerationState& state,
                                       DeviceLogits& logits) const {
  const int B = static_cast<int>(token_batches.size());
  if (B <= 0) throw std::runtime_error("token_batches must not be empty");
  const int T = static_cast<int>(token_batches.front().size());
  if (T <= 0) throw std::runtime_error("token batch length must be positive");
  std::vector<int64_t> flat;
  flat.reserve(static_cast<size_t>(B) * T);
  for (const auto& row : token_batches) {
    if (static_cast<int>(row.size()) != T) throw std::runtime_error("all token batches must share the same length");
    flat.insert(flat.end(), row.begin(), row.end());
  }
  run(flat.data(), B, T, state, logits);
}

void B200ModelBackend::forward_decode(const std::vector<int64_t>& token_batch, GenerationState& state,
                                      DeviceLogits& logits) const {
  if (token_batch.empty()) throw std::runtime_error("token_batches must not be empty");
  run(token_batch.data(), static_cast<int>(token_batch.size()), 1, state, logits);
}

std::vector<int> B200ModelBackend::decode_greedy(const std::vector<int64_t>& token_batch, int steps, GenerationState& state,
                                                 DeviceLogits& logits, float* penalties, double alpha_presence,
                                                 double alpha_frequency, double alpha_decay) const {
  if (token_batch.empty()) throw std::runtime_error("token_batches must not be empty");
  const int B = static_cast<int>(token_batch.size());
  if (state.batch_size != B) throw std::runtime_error("state batch size mismatch");
  if (state.wkv32 != use_wkv32_) throw std::runtime_error("state wkv precision mismatch");
  if (steps <= 0) throw std::runtime_error("decode_greedy: steps must be positive");
  logits.rows = B;
  logits.vocab_size = vocab_size();
  logits.values.resize(static_cast<size_t>(B) * logits.vocab_size, "alloc backend logits f32");
  rwkv7_fast_v4::DeviceBuffer<int> ids_dev;
  ids_dev.resize(static_cast<size_t>(B) * steps, "alloc greedy token ids");
  std::vector<int> ids(static_cast<size_t>(B) * steps);
  void* wkv = use_wkv32_ ? static_cast<void*>(state.wkv_state32.p) : static_cast<void*>(state.wkv_state.p);
  // the host pointer makes the call copy the ids back and synchronise the stream
  check(rwkv7_b200_decode_greedy(model_, token_batch.data(), B, steps, state.shift.p, wkv, state.elapsed.p, logits.values.p,
                                 penalties, static_cast<float>(alpha_presence), static_cast<float>(alpha_frequency),
                                 static_cast<float>(alpha_decay), ids_dev.p, ids.data(), stream_));
  return ids;
}

void B200ModelBackend::copy_state_slice(const GenerationState& src, int src_offset, GenerationState& dst, int dst_offset,
                                        int count) const {
  if (src.wkv32 != dst.wkv32 || src.wkv32 != use_wkv32_) throw std::runtime_error("state slice wkv precision mismatch");
  const void* sw = use_wkv32_ ? static_cast<const void*>(src.wkv_state32.p) : static_cast<const void*>(src.wkv_state.p);
  void* dw = use_wkv32_ ? static_cast<void*>(dst.wkv_state32.p) : static_cast<void*>(dst.wkv_state.p);
  check(rwkv7_b200_copy_state_slice(model_, src.shift.p, sw, src.elapsed.p, src.batch_size, src_offset, dst.shift.p, dw,
                                    dst.elapsed.p, dst.batch_size, dst_offset, count, stream_));
  if (cudaStreamSynchronize(stream_) != cudaSuccess) throw std::runtime_error("sync backend state slice");
}

void B200ModelBackend::copy_logits_slice(const DeviceLogits& src, int src_offset, DeviceLogits& dst, int dst_offset,
                                         int count) const {
  if (src_offset < 0 || dst_offset < 0 || count <= 0) throw std::runtime_error("invalid backend logits slice range");
  if (src.rows <= 0 || src.vocab_size <= 0 || src.values.p == nullptr) throw std::runtime_error("logits slice requires non-empty source");
  if (dst.rows <= 0 || dst.vocab_size != src.vocab_size || dst.values.p == nullptr)
    throw std::runtime_error("logits slice destination shape mismatch");
  if (src_offset + count > src.rows || dst_offset + count > dst.rows) throw std::runtime_error("logits slice range exceeds row count");
  if (cudaMemcpy(dst.values.p + static_cast<size_t>(dst_offset) * dst.vocab_size,
                 src.values.p + static_cast<size_t>(src_offset) * src.vocab_size,
                 static_cast<size_t>(count) * src.vocab_size * sizeof(float), cudaMemcpyDeviceToDevice) != cudaSuccess)
    throw std::runtime_error("copy backend logits slice");
}

PrefillCapacity B200ModelBackend::query_prefill_capacity(int prefill_chunk_size) const {
  rwkv7_b200_capacity c{};
  check(rwkv7_b200_query_capacity(model_, prefill_chunk_size, &c));
  PrefillCapacity out;
  out.free_vram_bytes = c.free_vram_bytes; out.total_vram_bytes = c.total_vram_bytes;
  out.reserve_vram_bytes = c.reserve_vram_bytes; out.bytes_per_batch = c.bytes_per_batch; out.max_batch_size = c.max_batch_size;
  return out;
}

int B200ModelBackend::vocab_size() const { return rwkv7_b200_vocab_size(model_); }

}  // namespace rwkv7_server
