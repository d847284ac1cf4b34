// Host-side engine: see model.h.  The launch order follows the reference's
// run_backend_forward (src/rwkv7_fast_v4.cu:1158-1342) but with persistent workspaces, the
// embedding table on the device, fused row kernels and a captured CUDA graph per decode shape
// instead of per-call allocation, a host gather and ~14 separate launches per layer.
#include "model.h"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <limits>

namespace rk {

// ------------------------------------------------------------------ errors
namespace {
thread_local char g_error[512] = "";
thread_local long long g_launches = 0;
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_error; }
long long& launch_counter() { return g_launches; }

int cuda_status(cudaError_t err, const char* what) {
  if (err == cudaSuccess) return kOk;
  set_error("CUDA error in %s: %s", what, cudaGetErrorString(err));
  return kCuda;
}

// ------------------------------------------------------------------ buffers
int DevBuf::alloc(size_t n) {
  release();
  if (n == 0) return kOk;
  RK_CUDA(cudaMalloc(&p, n));
  bytes = n;
  return kOk;
}
void DevBuf::release() {
  if (p) cudaFree(p);
  p = nullptr;
  bytes = 0;
}

// ------------------------------------------------------------------ model
Model::Model(const rwkv7_b200_config& cfg) : cfg_(cfg) {
  H_ = cfg.channels / kHead;
  tp_size_ = cfg.tp_size > 1 ? cfg.tp_size : 1;
  tp_rank_ = tp_size_ > 1 ? cfg.tp_rank : 0;
  layers_.resize(static_cast<size_t>(cfg.layers));
}
Model::~Model() {
  drop_graphs();
  for (int i = 0; i < kSlots; ++i) {
    if (tokens_pinned_[i]) cudaFreeHost(tokens_pinned_[i]);
    if (tokens_copied_[i]) cudaEventDestroy(tokens_copied_[i]);
  }
  if (last_done_) cudaEventDestroy(last_done_);
  if (timeout_host_) cudaFreeHost(timeout_host_);
}

void Model::drop_graphs() {
  for (auto& kv : graphs_)
    if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
  graphs_.clear();
}

int Model::use_device() const {
  if (cfg_.device >= 0) RK_CUDA(cudaSetDevice(cfg_.device));
  return kOk;
}

int Model::upload(DevBuf& dst, const void* data, int dtype, long long count, int on_device, long long expect) {
  RK_REQUIRE(count == expect, kShape, "set_tensor: got %lld elements, expected %lld", count, expect);
  RK_REQUIRE(dtype == RWKV7_B200_DT_F16 || dtype == RWKV7_B200_DT_BF16, kBadArg, "set_tensor: unknown dtype %d", dtype);
  const size_t bytes = static_cast<size_t>(count) * 2;
  int s = dst.alloc(bytes);
  if (s != kOk) return s;
  const cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
  if (dtype == RWKV7_B200_DT_F16) {
    RK_CUDA(cudaMemcpy(dst.p, data, bytes, kind));
  } else {
    DevBuf tmp;
    s = tmp.alloc(bytes);
    if (s != kOk) return s;
    RK_CUDA(cudaMemcpy(tmp.p, data, bytes, kind));
    s = bf16_to_f16(nullptr, tmp.as<uint16_t>(), dst.as<half>(), count);
    if (s != kOk) return s;
    RK_CUDA(cudaDeviceSynchronize());
  }
  return kOk;
}

int Model::upload_matrix(Matrix& m, int N, int K, const void* data, int dtype, long long count, int on_device) {
  m.N = N;
  m.K = K;
  m.fmt = RWKV7_B200_FMT_F16;
  return upload(m.w, data, dtype, count, on_device, static_cast<long long>(N) * K);
}

// Copies the block [r0, r0+nr) x [c0, c0+nc) of a row-major [rows, cols] tensor (the caller always passes the whole
// tensor; a tensor-parallel rank keeps only its share).
int Model::upload_slice(DevBuf& dst, const void* data, int dtype, long long count, int on_device, int rows, int cols, int r0,
                        int nr, int c0, int nc) {
  if (nr == rows && nc == cols) return upload(dst, data, dtype, count, on_device, static_cast<long long>(rows) * cols);
  RK_REQUIRE(count == static_cast<long long>(rows) * cols, kShape, "set_tensor: got %lld elements, expected %lld", count,
             static_cast<long long>(rows) * cols);
  RK_REQUIRE(dtype == RWKV7_B200_DT_F16 || dtype == RWKV7_B200_DT_BF16, kBadArg, "set_tensor: unknown dtype %d", dtype);
  const size_t n = static_cast<size_t>(nr) * nc;
  int s = dst.alloc(n * 2);
  if (s != kOk) return s;
  DevBuf tmp;
  void* target = dst.p;
  if (dtype == RWKV7_B200_DT_BF16) {
    if ((s = tmp.alloc(n * 2)) != kOk) return s;
    target = tmp.p;
  }
  const char* src = static_cast<const char*>(data) + (static_cast<size_t>(r0) * cols + c0) * 2;
  RK_CUDA(cudaMemcpy2D(target, static_cast<size_t>(nc) * 2, src, static_cast<size_t>(cols) * 2, static_cast<size_t>(nc) * 2, nr,
                       on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
  if (dtype == RWKV7_B200_DT_BF16) {
    if ((s = bf16_to_f16(nullptr, tmp.as<uint16_t>(), dst.as<half>(), static_cast<long long>(n))) != kOk) return s;
    RK_CUDA(cudaDeviceSynchronize());
  }
  return kOk;
}

int Model::set_tensor(const char* name, const void* data, int dtype, long long count, int on_device) {
  RK_REQUIRE(name && data, kBadArg, "set_tensor: null argument");
  RK_REQUIRE(!finalized_, kBadArg, "set_tensor: model already finalised");
  int s = use_device();
  if (s != kOk) return s;
  const long long C = cfg_.channels, F = cfg_.ffn, V = cfg_.vocab;
  const std::string n(name);
  if (n == "emb_ln0") return upload(emb_ln0_, data, dtype, count, on_device, V * C);
  if (n == "emb.weight") {
    // kept in its source type: LN0 is evaluated from the checkpoint values, not from rounded halves
    RK_REQUIRE(count == V * C, kShape, "set_tensor: emb.weight has %lld elements, expected %lld", count, V * C);
    emb_dtype_ = dtype;
    s = emb_raw_.alloc(static_cast<size_t>(count) * 2);
    if (s != kOk) return s;
    RK_CUDA(cudaMemcpy(emb_raw_.p, data, static_cast<size_t>(count) * 2, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
    return kOk;
  }
  if (n == "ln_out.weight") return upload(ln_out_w_, data, dtype, count, on_device, C);
  if (n == "ln_out.bias") return upload(ln_out_b_, data, dtype, count, on_device, C);
  // tensor parallel: this rank keeps heads [rank*H/G, (rank+1)*H/G), the matching slice of ffn and of the vocabulary
  const int G = tp_size_, Cl = static_cast<int>(C) / G, Fl = static_cast<int>(F) / G, Vl = static_cast<int>(V) / G;
  const int c_lo = tp_rank_ * Cl, f_lo = tp_rank_ * Fl, v_lo = tp_rank_ * Vl;
  auto rows_of = [&](Matrix& m, int N, int K, int r0, int nr) {  // output-channel slice
    m.N = nr; m.K = K; m.fmt = RWKV7_B200_FMT_F16;
    return upload_slice(m.w, data, dtype, count, on_device, N, K, r0, nr, 0, K);
  };
  auto cols_of = [&](Matrix& m, int N, int K, int c0, int nc) {  // input-channel slice
    m.N = N; m.K = nc; m.fmt = RWKV7_B200_FMT_F16;
    return upload_slice(m.w, data, dtype, count, on_device, N, K, 0, N, c0, nc);
  };
  if (n == "head.weight") return rows_of(head_, static_cast<int>(V), static_cast<int>(C), v_lo, Vl);

  int layer = -1, off = 0;
  if (sscanf(name, "blocks.%d.%n", &layer, &off) < 1 || layer < 0 || layer >= cfg_.layers || off == 0) {
    set_error("set_tensor: unknown tensor name '%s'", name);
    return kBadArg;
  }
  const std::string key(name + off);
  LayerWeights& L = layers_[static_cast<size_t>(layer)];
  if (key == "ln0.weight" || key == "ln0.bias") {
    RK_REQUIRE(layer == 0 && count == C, kShape, "set_tensor: bad ln0 tensor");
    RK_REQUIRE(emb_dtype_ < 0 || emb_dtype_ == dtype, kBadArg, "set_tensor: ln0 and emb.weight must share a dtype");
    DevBuf& dst = key == "ln0.weight" ? ln0_w_raw_ : ln0_b_raw_;
    s = dst.alloc(static_cast<size_t>(count) * 2);
    if (s != kOk) return s;
    RK_CUDA(cudaMemcpy(dst.p, data, static_cast<size_t>(count) * 2, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
    if (emb_dtype_ < 0) emb_dtype_ = dtype;
    return kOk;
  }
  struct VecSlot { const char* key; DevBuf* buf; long long n; };
  const VecSlot vecs[] = {
      {"ln1.weight", &L.ln1_w, C}, {"ln1.bias", &L.ln1_b, C}, {"ln2.weight", &L.ln2_w, C}, {"ln2.bias", &L.ln2_b, C},
      {"att.x_r", &L.mix[0], C}, {"att.x_w", &L.mix[1], C}, {"att.x_k", &L.mix[2], C}, {"att.x_v", &L.mix[3], C},
      {"att.x_a", &L.mix[4], C}, {"att.x_g", &L.mix[5], C}, {"ffn.x_k", &L.ffn_x_k, C},
  };
  for (const VecSlot& v : vecs)
    if (key == v.key) return upload(*v.buf, data, dtype, count, on_device, v.n);
  const VecSlot per_head[] = {  // per-channel vectors applied after the projections: sliced with the heads
      {"att.w0", &L.w0, C}, {"att.a0", &L.a0, C}, {"att.v0", &L.v0, C}, {"att.k_k", &L.k_k, C}, {"att.k_a", &L.k_a, C},
      {"att.r_k", &L.r_k, C}, {"att.ln_x.weight", &L.lnx_w, C}, {"att.ln_x.bias", &L.lnx_b, C},
  };
  for (const VecSlot& v : per_head)
    if (key == v.key) return upload_slice(*v.buf, data, dtype, count, on_device, 1, static_cast<int>(C), 0, 1, c_lo, Cl);
  const int Ci = static_cast<int>(C), Fi = static_cast<int>(F);
  if (key == "att.receptance.weight") return rows_of(L.Wr, Ci, Ci, c_lo, Cl);
  if (key == "att.key.weight") return rows_of(L.Wk, Ci, Ci, c_lo, Cl);
  if (key == "att.value.weight") return rows_of(L.Wv, Ci, Ci, c_lo, Cl);
  if (key == "att.output.weight") return cols_of(L.Wo, Ci, Ci, c_lo, Cl);
  if (key == "ffn.key.weight") return rows_of(L.Wkey, Fi, Ci, f_lo, Fl);
  if (key == "ffn.value.weight") return cols_of(L.Wval, Ci, Fi, f_lo, Fl);
  struct LoraSlot { const char* key; int rank; bool up; };
  const LoraSlot loras[] = {
      {"att.w1", cfg_.rank_w, false}, {"att.w2", cfg_.rank_w, true}, {"att.a1", cfg_.rank_a, false}, {"att.a2", cfg_.rank_a, true},
      {"att.g1", cfg_.rank_g, false}, {"att.g2", cfg_.rank_g, true}, {"att.v1", cfg_.rank_v, false}, {"att.v2", cfg_.rank_v, true},
  };
  for (const LoraSlot& l : loras) {
    if (key != l.key) continue;
    // down-projections [C, R] are replicated; up-projections [R, C] keep this rank's output channels
    if (!l.up) return upload(lora_raw_[n], data, dtype, count, on_device, C * l.rank);
    return upload_slice(lora_raw_[n], data, dtype, count, on_device, l.rank, Ci, 0, l.rank, c_lo, Cl);
  }
  set_error("set_tensor: unknown tensor name '%s'", name);
  return kBadArg;
}

int Model::transpose_into(DevBuf& dst, const DevBuf& src, int rows, int cols) {
  RK_REQUIRE(src.p && src.bytes == static_cast<size_t>(rows) * cols * 2, kNotReady, "finalize: LoRA tensor missing");
  int s = dst.alloc(src.bytes);
  if (s != kOk) return s;
  return transpose_f16(nullptr, src.as<half>(), dst.as<half>(), rows, cols);
}

int Model::quantize(Matrix& m) {
  if (cfg_.weight_format == RWKV7_B200_FMT_F16) return kOk;
  RK_REQUIRE(m.w.p, kNotReady, "finalize: matrix missing");
  DevBuf q;
  int s;
  if (cfg_.weight_format == RWKV7_B200_FMT_W8A16) {
    if ((s = q.alloc(static_cast<size_t>(m.N) * m.K)) != kOk) return s;
    if ((s = m.scale.alloc(static_cast<size_t>(m.N) * 2)) != kOk) return s;
    if ((s = quant_pack_w8(nullptr, m.N, m.K, m.w.as<half>(), q.as<int8_t>(), m.scale.as<half>())) != kOk) return s;
  } else {
    RK_REQUIRE(m.K % 128 == 0, kShape, "finalize: W4A16 needs K %% 128 == 0 (K=%d)", m.K);
    const size_t groups = static_cast<size_t>(m.N) * (m.K / 128);
    if ((s = q.alloc(static_cast<size_t>(m.N) * m.K / 2)) != kOk) return s;
    if ((s = m.scale.alloc(groups * 2)) != kOk) return s;
    if ((s = m.zero.alloc(groups * 2)) != kOk) return s;
    if ((s = quant_pack_w4(nullptr, m.N, m.K, m.w.as<half>(), q.as<uint8_t>(), m.scale.as<half>(), m.zero.as<half>())) != kOk) return s;
  }
  RK_CUDA(cudaDeviceSynchronize());
  m.w = std::move(q);
  m.fmt = cfg_.weight_format;
  return kOk;
}

int Model::finalize() {
  RK_REQUIRE(!finalized_, kBadArg, "finalize: called twice");
  int s = use_device();
  if (s != kOk) return s;
  const int C = cfg_.channels, V = cfg_.vocab, Cl = C / tp_size_;
  if (!emb_ln0_.p) {
    RK_REQUIRE(emb_raw_.p && ln0_w_raw_.p && ln0_b_raw_.p, kNotReady, "finalize: need emb_ln0 or emb.weight + blocks.0.ln0.*");
    if ((s = emb_ln0_.alloc(static_cast<size_t>(V) * C * 2)) != kOk) return s;
    if ((s = emb_ln0(nullptr, V, C, emb_raw_.p, ln0_w_raw_.p, ln0_b_raw_.p, emb_dtype_ == RWKV7_B200_DT_BF16,
                     emb_ln0_.as<half>(), 1e-5f)) != kOk) return s;
    RK_CUDA(cudaDeviceSynchronize());
  }
  emb_raw_.release(); ln0_w_raw_.release(); ln0_b_raw_.release();
  RK_REQUIRE(ln_out_w_.p && ln_out_b_.p && head_.w.p, kNotReady, "finalize: ln_out / head missing");

  for (int li = 0; li < cfg_.layers; ++li) {
    LayerWeights& L = layers_[static_cast<size_t>(li)];
    const std::string pre = "blocks." + std::to_string(li) + ".att.";
    struct T { const char* key; DevBuf* dst; int rows, cols; };
    // checkpoint: x1 [C,R] (down), x2 [R,C] (up); device: down [R,C], up [C,R]
    const T ts[] = {
        {"w1", &L.w1t, C, cfg_.rank_w}, {"w2", &L.w2t, cfg_.rank_w, Cl}, {"a1", &L.a1t, C, cfg_.rank_a},
        {"a2", &L.a2t, cfg_.rank_a, Cl}, {"g1", &L.g1t, C, cfg_.rank_g}, {"g2", &L.g2t, cfg_.rank_g, Cl},
        {"v1", &L.v1t, C, cfg_.rank_v}, {"v2", &L.v2t, cfg_.rank_v, Cl},
    };
    for (const T& t : ts) {
      if (li == 0 && t.key[0] == 'v') continue;  // layer 0 has no value residual
      auto it = lora_raw_.find(pre + t.key);
      RK_REQUIRE(it != lora_raw_.end(), kNotReady, "finalize: %s%s missing", pre.c_str(), t.key);
      if ((s = transpose_into(*t.dst, it->second, t.rows, t.cols)) != kOk) return s;
    }
    const DevBuf* need[] = {&L.ln1_w, &L.ln1_b, &L.ln2_w, &L.ln2_b, &L.mix[0], &L.mix[1], &L.mix[2], &L.mix[3], &L.mix[4],
                            &L.mix[5], &L.w0, &L.a0, &L.k_k, &L.k_a, &L.r_k, &L.lnx_w, &L.lnx_b, &L.ffn_x_k,
                            &L.Wr.w, &L.Wk.w, &L.Wv.w, &L.Wo.w, &L.Wkey.w, &L.Wval.w};
    for (const DevBuf* b : need) RK_REQUIRE(b->p, kNotReady, "finalize: a tensor of layer %d is missing", li);
    RK_REQUIRE(li == 0 || L.v0.p, kNotReady, "finalize: att.v0 of layer %d missing", li);
    for (Matrix* m : {&L.Wr, &L.Wk, &L.Wv, &L.Wo, &L.Wkey, &L.Wval})
      if ((s = quantize(*m)) != kOk) return s;
  }
  RK_CUDA(cudaDeviceSynchronize());
  lora_raw_.clear();
  if ((s = quantize(head_)) != kOk) return s;
  // everything a forward call needs that is not a plain stream operation is set up here, outside any stream capture
  if ((s = timeout_word(&timeout_dev_)) != kOk) return s;
  RK_CUDA(cudaMallocHost(reinterpret_cast<void**>(&timeout_host_), sizeof(int)));
  *timeout_host_ = 0;
  RK_CUDA(cudaEventCreateWithFlags(&last_done_, cudaEventDisableTiming));
  for (int i = 0; i < kSlots; ++i) RK_CUDA(cudaEventCreateWithFlags(&tokens_copied_[i], cudaEventDisableTiming));
  finalized_ = true;
  return kOk;
}

int Model::enqueue_timeout_read(cudaStream_t stream) {
  RK_REQUIRE(timeout_dev_ && timeout_host_, kNotReady, "model not finalised");
  RK_CUDA(cudaMemcpyAsync(timeout_host_, timeout_dev_, sizeof(int), cudaMemcpyDeviceToHost, stream));
  return kOk;
}

int Model::timeout_result() {
  const int flags = *timeout_host_;
  if (!flags) return kOk;
  *timeout_host_ = 0;
  cudaMemset(timeout_dev_, 0, sizeof(int));
  return timeout_status(flags);
}

int Model::tp_init(const void* unique_id) {
  RK_REQUIRE(tp_size_ > 1, kBadArg, "tp_init: the model was created with tp_size <= 1");
  int s = use_device();
  if (s != kOk) return s;
  return tp_.init(unique_id, tp_rank_, tp_size_);
}

int Model::state_sizes(int B, size_t* shift_elems, size_t* wkv_elems, size_t* elapsed_elems) const {
  RK_REQUIRE(B > 0, kBadArg, "batch_size must be positive");
  if (shift_elems) *shift_elems = static_cast<size_t>(cfg_.layers) * 2 * B * cfg_.channels;
  if (wkv_elems) *wkv_elems = static_cast<size_t>(cfg_.layers) * B * (H_ / tp_size_) * kHead * kHead;
  if (elapsed_elems) *elapsed_elems = static_cast<size_t>(B);
  return kOk;
}

int Model::state_init(int B, void* shift, void* wkv, int* elapsed, cudaStream_t stream) const {
  size_t ns, nw, ne;
  int s = state_sizes(B, &ns, &nw, &ne);
  if (s != kOk) return s;
  RK_REQUIRE(shift && wkv && elapsed, kBadArg, "state_init: null state buffer");
  if ((s = use_device()) != kOk) return s;
  RK_CUDA(cudaMemsetAsync(shift, 0, ns * 2, stream));
  RK_CUDA(cudaMemsetAsync(wkv, 0, nw * (cfg_.wkv32 ? 4 : 2), stream));
  RK_CUDA(cudaMemsetAsync(elapsed, 0, ne * sizeof(int), stream));
  return kOk;
}

int Model::copy_state_slice(const void* src_shift, const void* src_wkv, const int* src_elapsed, int src_B, int src_off,
                            void* dst_shift, void* dst_wkv, int* dst_elapsed, int dst_B, int dst_off, int count,
                            cudaStream_t stream) const {
  RK_REQUIRE(src_off >= 0 && dst_off >= 0 && count > 0, kBadArg, "invalid backend state slice range");
  RK_REQUIRE(src_B > 0 && dst_B > 0, kBadArg, "state slice requires non-empty source and destination");
  RK_REQUIRE(src_off + count <= src_B && dst_off + count <= dst_B, kBadArg, "state slice range exceeds batch size");
  RK_REQUIRE(src_shift && src_wkv && src_elapsed && dst_shift && dst_wkv && dst_elapsed, kBadArg, "state slice: null buffer");
  int s = use_device();
  if (s != kOk) return s;
  const size_t C = static_cast<size_t>(cfg_.channels);
  const size_t lane = static_cast<size_t>(H_ / tp_size_) * kHead * kHead * (cfg_.wkv32 ? 4 : 2);
  // one strided copy per buffer: [layers*2] rows of count*C halves, [layers] rows of count*lane bytes
  RK_CUDA(cudaMemcpy2DAsync(static_cast<char*>(dst_shift) + static_cast<size_t>(dst_off) * C * 2, static_cast<size_t>(dst_B) * C * 2,
                            static_cast<const char*>(src_shift) + static_cast<size_t>(src_off) * C * 2, static_cast<size_t>(src_B) * C * 2,
                            static_cast<size_t>(count) * C * 2, static_cast<size_t>(cfg_.layers) * 2, cudaMemcpyDeviceToDevice, stream));
  RK_CUDA(cudaMemcpy2DAsync(static_cast<char*>(dst_wkv) + static_cast<size_t>(dst_off) * lane, static_cast<size_t>(dst_B) * lane,
                            static_cast<const char*>(src_wkv) + static_cast<size_t>(src_off) * lane, static_cast<size_t>(src_B) * lane,
                            static_cast<size_t>(count) * lane, static_cast<size_t>(cfg_.layers), cudaMemcpyDeviceToDevice, stream));
  RK_CUDA(cudaMemcpyAsync(dst_elapsed + dst_off, src_elapsed + src_off, static_cast<size_t>(count) * sizeof(int),
                          cudaMemcpyDeviceToDevice, stream));
  return kOk;
}

// Session records.  The reference's state cache keeps a paused sequence as three blobs -- shift [L][2][C] halves, wkv
// [L][H][64][64] halves or floats, elapsed [1] int -- copied with blocking cudaMemcpy calls out of / into a batch-1
// GenerationState that copy_state_slice filled first (src/rwkv_state_cache.cpp:132-223, blobs :268-333).  Here the blobs
// are gathered straight from / scattered straight into sequence `index` of a batch state by three strided asynchronous
// copies on the caller's stream (use pinned host memory for real overlap); same bytes, no staging state, no blocking.
int Model::state_export(const void* shift, const void* wkv, const int* elapsed, int B, int index, void* shift_blob, void* wkv_blob,
                        int* elapsed_blob, cudaStream_t stream) const {
  RK_REQUIRE(B > 0 && index >= 0 && index < B, kBadArg, "state slice range exceeds batch size");
  RK_REQUIRE(shift && wkv && elapsed && shift_blob && wkv_blob && elapsed_blob, kBadArg, "state_export: null buffer");
  int s = use_device();
  if (s != kOk) return s;
  const size_t C = static_cast<size_t>(cfg_.channels);
  const size_t lane = static_cast<size_t>(H_ / tp_size_) * kHead * kHead * (cfg_.wkv32 ? 4 : 2);
  RK_CUDA(cudaMemcpy2DAsync(shift_blob, C * 2, static_cast<const char*>(shift) + static_cast<size_t>(index) * C * 2, static_cast<size_t>(B) * C * 2,
                            C * 2, static_cast<size_t>(cfg_.layers) * 2, cudaMemcpyDeviceToHost, stream));
  RK_CUDA(cudaMemcpy2DAsync(wkv_blob, lane, static_cast<const char*>(wkv) + static_cast<size_t>(index) * lane, static_cast<size_t>(B) * lane, lane,
                            static_cast<size_t>(cfg_.layers), cudaMemcpyDeviceToHost, stream));
  RK_CUDA(cudaMemcpyAsync(elapsed_blob, elapsed + index, sizeof(int), cudaMemcpyDeviceToHost, stream));
  return kOk;
}

int Model::state_import(const void* shift_blob, const void* wkv_blob, const int* elapsed_blob, void* shift, void* wkv, int* elapsed, int B,
                        int index, cudaStream_t stream) const {
  RK_REQUIRE(B > 0 && index >= 0 && index < B, kBadArg, "state slice range exceeds batch size");
  RK_REQUIRE(shift && wkv && elapsed && shift_blob && wkv_blob && elapsed_blob, kBadArg, "state_import: null buffer");
  int s = use_device();
  if (s != kOk) return s;
  const size_t C = static_cast<size_t>(cfg_.channels);
  const size_t lane = static_cast<size_t>(H_ / tp_size_) * kHead * kHead * (cfg_.wkv32 ? 4 : 2);
  RK_CUDA(cudaMemcpy2DAsync(static_cast<char*>(shift) + static_cast<size_t>(index) * C * 2, static_cast<size_t>(B) * C * 2, shift_blob, C * 2, C * 2,
                            static_cast<size_t>(cfg_.layers) * 2, cudaMemcpyHostToDevice, stream));
  RK_CUDA(cudaMemcpy2DAsync(static_cast<char*>(wkv) + static_cast<size_t>(index) * lane, static_cast<size_t>(B) * lane, wkv_blob, lane, lane,
                            static_cast<size_t>(cfg_.layers), cudaMemcpyHostToDevice, stream));
  RK_CUDA(cudaMemcpyAsync(elapsed + index, elapsed_blob, sizeof(int), cudaMemcpyHostToDevice, stream));
  return kOk;
}

namespace {
size_t workspace_halves(const rwkv7_b200_config& c, size_t rows, size_t B) {
  const size_t C = c.channels;
  return rows * C * 27 + rows * static_cast<size_t>(c.ffn) + rows * 512 * 4 + B * C + 1024;
}
}  // namespace

int Model::query_capacity(int chunk, rwkv7_b200_capacity* out) const {
  RK_REQUIRE(chunk > 0, kBadArg, "prefill chunk size must be positive");
  RK_REQUIRE(out, kBadArg, "query_capacity: null output");
  int s = use_device();
  if (s != kOk) return s;
  RK_CUDA(cudaMemGetInfo(&out->free_vram_bytes, &out->total_vram_bytes));
  const size_t L = cfg_.layers, C = cfg_.channels;
  const size_t state = L * 2 * C * 2 + L * (H_ / tp_size_) * kHead * kHead * (cfg_.wkv32 ? 4 : 2) + sizeof(int);
  // per sequence: its state, its rows of the activation arena, its split-K partial sums and its logits
  const size_t arena = workspace_halves(cfg_, static_cast<size_t>(chunk), 1) * 2 + static_cast<size_t>(chunk) * 8;
  const size_t splitk = static_cast<size_t>(chunk) * C * sizeof(float) * 24;
  out->bytes_per_batch = state + arena + splitk + static_cast<size_t>(cfg_.vocab) * 4;
  // beside the reference's reserve: what the workspace may still have to grow by that does not scale with the batch
  // (the cap of the split-K scratch), less what it holds already
  size_t fixed = static_cast<size_t>(512) << 20;
  const size_t held = workspace_bytes();
  fixed = fixed > held ? fixed - held : 0;
  out->reserve_vram_bytes = std::max<size_t>(static_cast<size_t>(512) << 20, out->free_vram_bytes / 10) + fixed;
  const size_t usable = out->free_vram_bytes > out->reserve_vram_bytes ? out->free_vram_bytes - out->reserve_vram_bytes : 0;
  // the split-K scratch stops growing at its cap: do not count it beyond that
  size_t n = usable / out->bytes_per_batch;
  if (n * splitk > (static_cast<size_t>(512) << 20)) {
    const size_t per = out->bytes_per_batch - splitk;
    const size_t rest = usable > (static_cast<size_t>(512) << 20) ? usable - (static_cast<size_t>(512) << 20) : 0;
    n = std::max(rest / per, (static_cast<size_t>(512) << 20) / splitk);
  }
  out->max_batch_size = static_cast<int>(std::min<size_t>(n, std::numeric_limits<int>::max()));
  return kOk;
}

// Points ws_ at buffers for a forward of B sequences x T tokens.  The buffers only ever grow; growing waits for the
// device (earlier calls may still be using the old ones) and drops the captured decode graphs, which hold their
// addresses.  Must not be called while a stream is being captured.
int Model::prepare(int B, int T, cudaStream_t stream) {
  const size_t rows = static_cast<size_t>(B) * T, C = cfg_.channels, F = cfg_.ffn;
  const size_t arena_bytes = workspace_halves(cfg_, rows, B) * 2 + rows * 8 + 256;
  size_t scratch_bytes = 0, part_bytes = 0;
  if (rows >= 2) scratch_bytes = std::min<size_t>(static_cast<size_t>(512) << 20, rows * C * sizeof(float) * 24);
  if (tp_size_ > 1) part_bytes = std::max(rows * C, static_cast<size_t>(B) * cfg_.vocab * 2) * sizeof(float);
  const bool grow = arena_bytes > arena_.bytes || scratch_bytes > gemm_scratch_.bytes || part_bytes > part32_.bytes ||
                    rows > pinned_rows_;
  if (grow) {
    RK_CUDA(cudaDeviceSynchronize());
    drop_graphs();
    int s;
    if (arena_bytes > arena_.bytes && (s = arena_.alloc(arena_bytes)) != kOk) return s;
    if (scratch_bytes > gemm_scratch_.bytes && (s = gemm_scratch_.alloc(scratch_bytes)) != kOk) return s;
    if (part_bytes > part32_.bytes && (s = part32_.alloc(part_bytes)) != kOk) return s;
    if (rows > pinned_rows_) {
      for (int i = 0; i < kSlots; ++i) {
        if (tokens_pinned_[i]) cudaFreeHost(tokens_pinned_[i]);
        tokens_pinned_[i] = nullptr;
      }
      pinned_rows_ = 0;
      for (int i = 0; i < kSlots; ++i) RK_CUDA(cudaMallocHost(reinterpret_cast<void**>(&tokens_pinned_[i]), rows * sizeof(int64_t)));
      pinned_rows_ = rows;
    }
  }
  if (tp_size_ > 1) {  // room for this call's partial sums in the region the other ranks have mapped (a collective)
    const int s = tp_.ensure_peer(rows * C);
    if (s != kOk) return s;
  }
  Workspace& ws = ws_;
  ws.rows = static_cast<int>(rows);
  ws.B = B;
  half* p = arena_.as<half>();
  auto take = [&](size_t n) { half* q = p; p += (n + 7) & ~static_cast<size_t>(7); return q; };
  const size_t RC = rows * C;
  ws.xA = take(RC); ws.xB = take(RC);
  for (int i = 0; i < 6; ++i) ws.xm[i] = take(RC);
  ws.r = take(RC); ws.k = take(RC); ws.v = take(RC); ws.vfirst = take(RC); ws.vout = take(RC);
  ws.w12 = take(RC); ws.a12 = take(RC); ws.g = take(RC); ws.k2 = take(RC); ws.nkk = take(RC); ws.kka = take(RC);
  ws.y = take(RC); ws.y2 = take(RC); ws.att = take(RC); ws.mixed = take(RC); ws.ffn = take(RC);
  ws.hid = take(rows * F);
  for (int i = 0; i < 4; ++i) ws.l1[i] = take(rows * 512);
  ws.xf = take(static_cast<size_t>(B) * C);
  ws.n1 = take(RC); ws.n2 = take(RC);
  ws.tokens = reinterpret_cast<int64_t*>(take(rows * 4 + 8));
  ws.gemm_scratch = rows >= 2 ? gemm_scratch_.as<float>() : nullptr;
  ws.gemm_scratch_bytes = rows >= 2 ? gemm_scratch_.bytes : 0;
  ws.part32 = part32_.as<float>();
  // the buffers are shared by every call: work enqueued on another stream must be over before this call's begins
  if (have_last_ && last_stream_ != stream) RK_CUDA(cudaStreamWaitEvent(stream, last_done_, 0));
  return kOk;
}

// Row count from which quantised weights take the tensor-core route (the GEMM that expands packed tiles in shared
// memory); below it the GEMV kernels dequantise in registers, and their time grows with the row count.  Measured
// cross-over: 3 rows for W8A16, 2 rows for W4A16, whose dequantisation costs more per row.
static int quant_tc_rows(int fmt) {
  if (options().quant_tc_rows >= 2) return options().quant_tc_rows;
  if (options().gemv_mma >= 1) return 5;  // the 16-channel-tile kernel (gemv_mma.cu) costs the same for 1..4 rows
  return fmt == RWKV7_B200_FMT_W4A16 ? 2 : 3;
}

int Model::lin(cudaStream_t s, int M, const Matrix& W, const half* x, void* y, int epi) {
  LinearArgs a;
  a.M = M; a.K = W.K; a.N = W.N; a.x = x; a.w = W.w.p; a.fmt = W.fmt;
  a.scale = W.scale.as<half>(); a.zero = W.zero.as<half>(); a.epi = epi; a.y = y;
  a.w_dynamic = false;  // resident weights
  // 2..4 rows of a large matrix: tensor cores (the GEMV's time grows with the row count)
  a.prefer_tc = W.fmt == RWKV7_B200_FMT_F16 ? options().gemv_mma < 2 : M >= quant_tc_rows(W.fmt);
  if (cur_) { a.scratch = cur_->gemm_scratch; a.scratch_bytes = cur_->gemm_scratch_bytes; }
  return linear(s, a);
}

int Model::lin16(cudaStream_t s, int M, int K, int N, const half* x, const half* w, half* y, int in_act, int epi,
                 const EpiArgs& ea) {
  LinearArgs a;
  a.M = M; a.K = K; a.N = N; a.x = x; a.w = w; a.fmt = RWKV7_B200_FMT_F16; a.in_act = in_act; a.epi = epi; a.ea = ea; a.y = y;
  a.w_dynamic = false;
  if (cur_) { a.scratch = cur_->gemm_scratch; a.scratch_bytes = cur_->gemm_scratch_bytes; }
  return linear(s, a);
}

#define RK_TRY(expr)            \
  do {                          \
    int _s = (expr);            \
    if (_s != kOk) return _s;   \
  } while (0)

// Decode step for up to four sequences (fp16, W8A16 or W4A16 weights): five launches per layer.  The residual
// add + LayerNorm + token shift in front of the r/k/v (+LoRA down) projections, of ffn.key and of
// the lm-head run as the prologue of those GEMV kernels; the shift states are updated by the kernel
// that follows (the fused head kernel, the ffn.value GEMV).
int Model::enqueue_decode(Workspace& ws, int B, half* shift, void* wkv, int* elapsed, float* logits, cudaStream_t st) {
  const int C = cfg_.channels, L = cfg_.layers, rows = B;
  auto mat = [&](const Matrix& Wm, const half* x, void* y, int epi) {
    LinearArgs a;
    a.M = rows; a.K = Wm.K; a.N = Wm.N; a.x = x; a.w = Wm.w.p; a.fmt = Wm.fmt; a.epi = epi; a.y = y;
    a.scale = Wm.scale.as<half>(); a.zero = Wm.zero.as<half>();
    return a;
  };
  auto low = [&](const DevBuf& w, int R, const half* x, half* y) {
    LinearArgs a;
    a.M = rows; a.K = C; a.N = R; a.x = x; a.w = w.p; a.fmt = RWKV7_B200_FMT_F16; a.y = y;
    return a;
  };
  {
    RowOpArgs a;
    a.B = B; a.T = 1; a.C = C; a.tokens = ws.tokens; a.table = emb_ln0_.as<half>(); a.vocab = cfg_.vocab;
    a.x_out = ws.xA; a.ln_w = layers_[0].ln1_w.as<half>(); a.ln_b = layers_[0].ln1_b.as<half>();
    a.shift = shift; a.n_mix = 6;
    for (int i = 0; i < 6; ++i) { a.mix[i] = layers_[0].mix[i].as<half>(); a.mix_out[i] = ws.xm[i]; }
    RK_TRY(row_op(st, a));
  }
  for (int li = 0; li < L; ++li) {
    const LayerWeights& W = layers_[static_cast<size_t>(li)];
    half* shift0 = shift + static_cast<size_t>(li) * 2 * B * C;
    half* shift1 = shift0 + static_cast<size_t>(B) * C;
    half* v_lin = li == 0 ? ws.vfirst : ws.v;
    // time mix: inputs are xm[] for layer 0, otherwise computed in the prologue from xB + ffn
    const half* xin[6];
    for (int i = 0; i < 6; ++i) xin[i] = li == 0 ? ws.xm[i] : ws.xB;
    LinearArgs seg[7] = {mat(W.Wr, xin[0], ws.r, kEpiNone), mat(W.Wk, xin[2], ws.k, kEpiNone), mat(W.Wv, xin[3], v_lin, kEpiNone),
                         low(W.w1t, cfg_.rank_w, xin[1], ws.l1[0]), low(W.a1t, cfg_.rank_a, xin[4], ws.l1[1]),
                         low(W.g1t, cfg_.rank_g, xin[5], ws.l1[2]), low(W.v1t, cfg_.rank_v, xin[3], ws.l1[3])};
    if (li > 0) {
      const int mix_of[7] = {0, 2, 3, 1, 4, 5, 3};  // x_r, x_k, x_v, x_w, x_a, x_g, x_v
      for (int i = 0; i < 7; ++i) {
        seg[i].res = ws.ffn; seg[i].ln_w = W.ln1_w.as<half>(); seg[i].ln_b = W.ln1_b.as<half>();
        seg[i].shift = shift0; seg[i].mix = W.mix[mix_of[i]].as<half>();
      }
      seg[0].x_out = ws.xA; seg[0].n_out = ws.n1;
    }
    RK_TRY(linear_batch(st, seg, li == 0 ? 6 : 7));
    TmixDecodeArgs ta;
    ta.B = B; ta.C = C; ta.layer0 = li == 0; ta.wkv32 = cfg_.wkv32 != 0;
    ta.R[0] = cfg_.rank_w; ta.R[1] = cfg_.rank_a; ta.R[2] = cfg_.rank_g; ta.R[3] = cfg_.rank_v;
    for (int i = 0; i < 4; ++i) ta.l1[i] = ws.l1[i];
    ta.up[0] = W.w2t.as<half>(); ta.up[1] = W.a2t.as<half>(); ta.up[2] = W.g2t.as<half>(); ta.up[3] = W.v2t.as<half>();
    ta.r = ws.r; ta.k = ws.k; ta.v = v_lin; ta.v_first = ws.vfirst;
    ta.w0 = W.w0.as<half>(); ta.a0 = W.a0.as<half>(); ta.v0 = W.v0.as<half>(); ta.k_k = W.k_k.as<half>();
    ta.k_a = W.k_a.as<half>(); ta.r_k = W.r_k.as<half>(); ta.lnx_w = W.lnx_w.as<half>(); ta.lnx_b = W.lnx_b.as<half>();
    const size_t wkv_off = static_cast<size_t>(li) * B * H_ * kHead * kHead;
    ta.state = cfg_.wkv32 ? static_cast<void*>(static_cast<float*>(wkv) + wkv_off)
                          : static_cast<void*>(static_cast<half*>(wkv) + wkv_off);
    ta.elapsed = elapsed; ta.y2 = ws.y2;
    if (li > 0) { ta.shift_src = ws.n1; ta.shift_dst = shift0; }
    RK_TRY(tmix_decode(st, ta));
    LinearArgs wo = mat(W.Wo, ws.y2, ws.att, kEpiNone);
    RK_TRY(linear_batch(st, &wo, 1));
    // channel mix: x <- xA + att, LN2, token shift, ffn.key with relu^2
    LinearArgs key = mat(W.Wkey, ws.xA, ws.hid, kEpiRelu2);
    key.res = ws.att; key.ln_w = W.ln2_w.as<half>(); key.ln_b = W.ln2_b.as<half>(); key.shift = shift1;
    key.mix = W.ffn_x_k.as<half>(); key.x_out = ws.xB; key.n_out = ws.n2;
    RK_TRY(linear_batch(st, &key, 1));
    LinearArgs val = mat(W.Wval, ws.hid, ws.ffn, kEpiNone);
    val.copy_src = ws.n2; val.copy_dst = shift1; val.copy_n = B * C;
    RK_TRY(linear_batch(st, &val, 1));
  }
  RK_TRY(advance_i32(st, elapsed, 1, B));
  LinearArgs head = mat(head_, ws.xB, logits, kEpiF32);
  head.res = ws.ffn; head.ln_w = ln_out_w_.as<half>(); head.ln_b = ln_out_b_.as<half>();
  RK_TRY(linear_batch(st, &head, 1));
  return kOk;
}

int Model::enqueue(Workspace& ws, int B, int T, half* shift, void* wkv, int* elapsed, float* logits, cudaStream_t st) {
  const int C = cfg_.channels, L = cfg_.layers, rows = B * T;
  const int G = tp_size_, Cl = C / G, Hl = H_ / G;  // this rank's share of channels / heads
  const EpiArgs none;
  cur_ = &ws;
  {
    TmixDecodeArgs probe;
    probe.B = B; probe.C = C; probe.wkv32 = cfg_.wkv32 != 0;
    probe.R[0] = cfg_.rank_w; probe.R[1] = cfg_.rank_a; probe.R[2] = cfg_.rank_g; probe.R[3] = cfg_.rank_v;
    const bool rows_ok = cfg_.weight_format == RWKV7_B200_FMT_F16 ? C % 8 == 0 : (C % 128 == 0 && cfg_.ffn % 128 == 0);
    // Which one-token steps of up to four rows take the five-launch GEMV path (enqueue_decode); the others go through
    // the general path below, with the large matrices on the tensor cores.
    const bool quant_tc = cfg_.weight_format != RWKV7_B200_FMT_F16 && rows >= quant_tc_rows(cfg_.weight_format);
    // measured cross-over for fp16 weights: 2 rows from the 1.5B layer width up (1.5B: 1.51 vs 1.53 ms at 2 rows, 1.58 vs
    // 2.18 at 3), 4 rows for narrow models, whose steps are launch-bound (0.1B: 0.42 ms on the GEMV route vs 0.54 at 2 rows)
    // Dimensions the 16-channel-tile kernel takes (whole 128-byte boxes per weight row, channel counts in fours): with
    // it 2..4 rows cost what one row costs, so nothing up to four rows goes to the tensor-core GEMM.
    const bool mma_dims = C % 256 == 0 && cfg_.ffn % 256 == 0 && cfg_.vocab % 4 == 0 && cfg_.rank_w % 4 == 0 &&
                          cfg_.rank_a % 4 == 0 && cfg_.rank_g % 4 == 0 && cfg_.rank_v % 4 == 0;
    const bool mma_fp16 = mma_dims && options().gemv_mma >= 2 && rows >= 2 && cfg_.weight_format == RWKV7_B200_FMT_F16;
    const bool mma_quant = mma_dims && options().gemv_mma >= 1 && cfg_.weight_format != RWKV7_B200_FMT_F16;
    const int fp16_tc_rows = options().fp16_tc_rows >= 2 ? options().fp16_tc_rows : mma_fp16 ? 5 : (C < 1536 ? 4 : 2);
    const bool gemv_rows = rows == 1 || (cfg_.weight_format != RWKV7_B200_FMT_F16 && !quant_tc) ||
                           (cfg_.weight_format == RWKV7_B200_FMT_F16 && rows < fp16_tc_rows);
    // (the fused path stages a step's activations in shared memory: B rows of ffn inputs must fit)
    if (G == 1 && T == 1 && rows <= 4 && gemv_rows && tmix_decode_supported(probe) && C <= 4096 && rows_ok &&
        ((mma_fp16 || mma_quant) ? gemv_mma_fits(rows, std::max(C, cfg_.ffn))
                                 : (linear_batch_fused_fits(rows, cfg_.ffn) && linear_batch_fused_fits(rows, C))))
      return enqueue_decode(ws, B, shift, wkv, elapsed, logits, st);
  }
  {
    RowOpArgs a;
    a.B = B; a.T = T; a.C = C; a.tokens = ws.tokens; a.table = emb_ln0_.as<half>(); a.vocab = cfg_.vocab;
    a.x_out = ws.xA; a.ln_w = layers_[0].ln1_w.as<half>(); a.ln_b = layers_[0].ln1_b.as<half>();
    a.shift = shift; a.n_mix = 6;
    for (int i = 0; i < 6; ++i) { a.mix[i] = layers_[0].mix[i].as<half>(); a.mix_out[i] = ws.xm[i]; }
    RK_TRY(row_op(st, a));
  }
  for (int li = 0; li < L; ++li) {
    const LayerWeights& W = layers_[static_cast<size_t>(li)];
    half* shift0 = shift + static_cast<size_t>(li) * 2 * B * C;
    half* shift1 = shift0 + static_cast<size_t>(B) * C;
    half *xr = ws.xm[0], *xw = ws.xm[1], *xk = ws.xm[2], *xv = ws.xm[3], *xa = ws.xm[4], *xg = ws.xm[5];
    half* v_lin = li == 0 ? ws.vfirst : ws.v;
    const size_t wkv_off = static_cast<size_t>(li) * B * Hl * kHead * kHead;
    TmixDecodeArgs ta;
    ta.B = B; ta.C = C; ta.layer0 = li == 0; ta.wkv32 = cfg_.wkv32 != 0;
    ta.R[0] = cfg_.rank_w; ta.R[1] = cfg_.rank_a; ta.R[2] = cfg_.rank_g; ta.R[3] = cfg_.rank_v;
    if (G == 1 && T == 1 && rows <= 4 && tmix_decode_supported(ta)) {
      // decode: r/k/v projections and the LoRA down-projections as one launch, then the fused head kernel
      auto mat = [&](const Matrix& Wm, const half* x, half* y) {
        LinearArgs a;
        a.M = rows; a.K = Wm.K; a.N = Wm.N; a.x = x; a.w = Wm.w.p; a.fmt = Wm.fmt;
        a.scale = Wm.scale.as<half>(); a.zero = Wm.zero.as<half>(); a.y = y;
        return a;
      };
      auto low = [&](const DevBuf& w, int R, const half* x, half* y) {
        LinearArgs a;
        a.M = rows; a.K = C; a.N = R; a.x = x; a.w = w.p; a.fmt = RWKV7_B200_FMT_F16; a.y = y;
        return a;
      };
      LinearArgs seg[7] = {mat(W.Wr, xr, ws.r), mat(W.Wk, xk, ws.k), mat(W.Wv, xv, v_lin),
                           low(W.w1t, cfg_.rank_w, xw, ws.l1[0]), low(W.a1t, cfg_.rank_a, xa, ws.l1[1]),
                           low(W.g1t, cfg_.rank_g, xg, ws.l1[2]), low(W.v1t, cfg_.rank_v, xv, ws.l1[3])};
      if (rows >= 2 && (cfg_.weight_format == RWKV7_B200_FMT_F16 ? options().gemv_mma < 2 : rows >= quant_tc_rows(cfg_.weight_format))) {
        // 2..4 rows: the three C x C projections as one tensor-core launch, the small LoRA down-projections as one GEMV
        for (int i = 0; i < 3; ++i) {
          seg[i].prefer_tc = true; seg[i].w_dynamic = false;
          seg[i].scratch = ws.gemm_scratch; seg[i].scratch_bytes = ws.gemm_scratch_bytes;
        }
        RK_TRY(linear_group(st, seg, 3));
        RK_TRY(linear_batch(st, seg + 3, li == 0 ? 3 : 4));
      } else {
        RK_TRY(linear_batch(st, seg, li == 0 ? 6 : 7));
      }
      for (int i = 0; i < 4; ++i) ta.l1[i] = ws.l1[i];
      ta.up[0] = W.w2t.as<half>(); ta.up[1] = W.a2t.as<half>(); ta.up[2] = W.g2t.as<half>(); ta.up[3] = W.v2t.as<half>();
      ta.r = ws.r; ta.k = ws.k; ta.v = v_lin; ta.v_first = ws.vfirst;
      ta.w0 = W.w0.as<half>(); ta.a0 = W.a0.as<half>(); ta.v0 = W.v0.as<half>(); ta.k_k = W.k_k.as<half>();
      ta.k_a = W.k_a.as<half>(); ta.r_k = W.r_k.as<half>(); ta.lnx_w = W.lnx_w.as<half>(); ta.lnx_b = W.lnx_b.as<half>();
      ta.state = cfg_.wkv32 ? static_cast<void*>(static_cast<float*>(wkv) + wkv_off)
                            : static_cast<void*>(static_cast<half*>(wkv) + wkv_off);
      ta.elapsed = elapsed; ta.y2 = ws.y2;
      RK_TRY(tmix_decode(st, ta));
    } else {
      const bool big = rows > 4;  // the reference rounds tanh/sigmoid and the v LoRA output to half for larger row counts
      const half* v_use = ws.vfirst;
      bool gates_fused = false, core_done = false;
      if (big) {
        // many rows: two tensor-core launches -- r/k/v with the four LoRA down-projections (tanh / sigmoid as
        // their epilogues), then the four LoRA up-projections
        auto dense = [&](const Matrix& Wm, const half* x, void* y) {
          LinearArgs a;
          a.M = rows; a.K = Wm.K; a.N = Wm.N; a.x = x; a.w = Wm.w.p; a.fmt = Wm.fmt; a.y = y; a.w_dynamic = false;
          a.scale = Wm.scale.as<half>(); a.zero = Wm.zero.as<half>();
          a.scratch = ws.gemm_scratch; a.scratch_bytes = ws.gemm_scratch_bytes;
          return a;
        };
        auto low = [&](const DevBuf& w, int K, int N, const half* x, half* y, int epi) {
          LinearArgs a;
          a.M = rows; a.K = K; a.N = N; a.x = x; a.w = w.p; a.fmt = RWKV7_B200_FMT_F16; a.epi = epi; a.y = y; a.w_dynamic = false;
          a.scratch = ws.gemm_scratch; a.scratch_bytes = ws.gemm_scratch_bytes;
          return a;
        };
        LinearArgs grp[7];
        int ng = 0;
        grp[ng++] = dense(W.Wr, xr, ws.r); grp[ng++] = dense(W.Wk, xk, ws.k); grp[ng++] = dense(W.Wv, xv, v_lin);
        // A few sequences, one token each: the fused time-mix kernel (LoRA up + gates + WKV + GroupNorm, one CTA per
        // sequence and head) replaces five launches; it applies tanh / sigmoid itself, with the many-row rounding.
        TmixDecodeArgs tf;
        tf.B = B; tf.C = C; tf.layer0 = li == 0; tf.wkv32 = cfg_.wkv32 != 0; tf.round_act = true;
        tf.R[0] = cfg_.rank_w; tf.R[1] = cfg_.rank_a; tf.R[2] = cfg_.rank_g; tf.R[3] = cfg_.rank_v;
        // (every CTA re-reads its head's LoRA-up rows: worth it while those re-reads stay small -- measured faster at
        // 3.5 and 17 MB per layer, slower at 54 MB)
        const size_t up_reads = static_cast<size_t>(rows) * C * (cfg_.rank_w + cfg_.rank_a + cfg_.rank_g + cfg_.rank_v) * sizeof(half);
        const bool few = G == 1 && T == 1 && rows <= 16 && up_reads <= (static_cast<size_t>(20) << 20) && tmix_decode_supported(tf);
        grp[ng++] = low(W.w1t, C, cfg_.rank_w, xw, ws.l1[0], few ? kEpiNone : kEpiTanhH);
        grp[ng++] = low(W.a1t, C, cfg_.rank_a, xa, ws.l1[1], kEpiNone);
        grp[ng++] = low(W.g1t, C, cfg_.rank_g, xg, ws.l1[2], few ? kEpiNone : kEpiSigmoidH);
        if (li > 0) grp[ng++] = low(W.v1t, C, cfg_.rank_v, xv, ws.l1[3], kEpiNone);
        RK_TRY(linear_group(st, grp, ng));
        if (few) {
          for (int i = 0; i < 4; ++i) tf.l1[i] = ws.l1[i];
          tf.up[0] = W.w2t.as<half>(); tf.up[1] = W.a2t.as<half>(); tf.up[2] = W.g2t.as<half>(); tf.up[3] = W.v2t.as<half>();
          tf.r = ws.r; tf.k = ws.k; tf.v = v_lin; tf.v_first = ws.vfirst;
          tf.w0 = W.w0.as<half>(); tf.a0 = W.a0.as<half>(); tf.v0 = W.v0.as<half>(); tf.k_k = W.k_k.as<half>();
          tf.k_a = W.k_a.as<half>(); tf.r_k = W.r_k.as<half>(); tf.lnx_w = W.lnx_w.as<half>(); tf.lnx_b = W.lnx_b.as<half>();
          tf.state = cfg_.wkv32 ? static_cast<void*>(static_cast<float*>(wkv) + wkv_off)
                                : static_cast<void*>(static_cast<half*>(wkv) + wkv_off);
          tf.elapsed = elapsed; tf.y2 = ws.y2;
          RK_TRY(tmix_decode(st, tf));
          core_done = true;
        } else {
          ng = 0;
          grp[ng++] = low(W.w2t, cfg_.rank_w, Cl, ws.l1[0], ws.w12, kEpiNone);
          grp[ng++] = low(W.a2t, cfg_.rank_a, Cl, ws.l1[1], ws.a12, kEpiNone);
          grp[ng++] = low(W.g2t, cfg_.rank_g, Cl, ws.l1[2], ws.g, kEpiNone);
          if (li > 0) grp[ng++] = low(W.v2t, cfg_.rank_v, Cl, ws.l1[3], ws.y, kEpiNone);
          RK_TRY(linear_group(st, grp, ng));
          if (li > 0) {  // the value-residual gate runs in the kk / a gate launch below
            gates_fused = true;
            v_use = ws.vout;
          }
        }
      } else {
        RK_TRY(lin(st, rows, W.Wr, xr, ws.r, kEpiNone));
        RK_TRY(lin(st, rows, W.Wk, xk, ws.k, kEpiNone));
        RK_TRY(lin(st, rows, W.Wv, xv, v_lin, kEpiNone));
        RK_TRY(lin16(st, rows, C, cfg_.rank_w, xw, W.w1t.as<half>(), ws.l1[0], kActNone, kEpiNone, none));
        RK_TRY(lin16(st, rows, C, cfg_.rank_a, xa, W.a1t.as<half>(), ws.l1[1], kActNone, kEpiNone, none));
        RK_TRY(lin16(st, rows, C, cfg_.rank_g, xg, W.g1t.as<half>(), ws.l1[2], kActNone, kEpiNone, none));
        RK_TRY(lin16(st, rows, cfg_.rank_w, Cl, ws.l1[0], W.w2t.as<half>(), ws.w12, kActTanh, kEpiNone, none));
        RK_TRY(lin16(st, rows, cfg_.rank_a, Cl, ws.l1[1], W.a2t.as<half>(), ws.a12, kActNone, kEpiNone, none));
        RK_TRY(lin16(st, rows, cfg_.rank_g, Cl, ws.l1[2], W.g2t.as<half>(), ws.g, kActSigmoid, kEpiNone, none));
        if (li > 0) {
          RK_TRY(lin16(st, rows, C, cfg_.rank_v, xv, W.v1t.as<half>(), ws.l1[3], kActNone, kEpiNone, none));
          EpiArgs ea;
          ea.v = ws.v; ea.v_first = ws.vfirst; ea.v0 = W.v0.as<half>();
          RK_TRY(lin16(st, rows, cfg_.rank_v, Cl, ws.l1[3], W.v2t.as<half>(), ws.vout, kActNone, kEpiVres, ea));
          v_use = ws.vout;
        }
      }
      if (!core_done) {  // (otherwise everything up to y2 was done by the fused time-mix kernel)
        if (gates_fused) {
          RK_TRY(tmix_kk_a_vres_gate(st, rows, Cl, ws.k, W.k_k.as<half>(), W.a0.as<half>(), ws.a12, W.k_a.as<half>(), ws.k2, ws.nkk, ws.kka,
                                     ws.v, ws.vfirst, W.v0.as<half>(), ws.y, ws.vout));
        } else {
          RK_TRY(tmix_kk_a_gate(st, rows, Cl, ws.k, W.k_k.as<half>(), W.a0.as<half>(), ws.a12, W.k_a.as<half>(), ws.k2, ws.nkk, ws.kka));
        }
        if (cfg_.wkv32) {
          RK_TRY(wkv7_fp32(st, B, T, Cl, Hl, static_cast<float*>(wkv) + wkv_off, ws.r, ws.w12, W.w0.as<half>(), ws.k2, v_use,
                           ws.nkk, ws.kka, ws.y));
        } else {
          // the reference adds w0 in fp32 inside the kernel for T <= 16 and pre-rounds the sum otherwise
          RK_TRY(wkv7_fp16(st, B, T, Cl, Hl, static_cast<half*>(wkv) + wkv_off, ws.r, ws.w12, W.w0.as<half>(), T <= 16 ? 1 : 2,
                           ws.k2, v_use, ws.nkk, ws.kka, ws.y, elapsed, tp_rank_ * Cl));
        }
        RK_TRY(tmix_lnx_rkvres_xg(st, rows, Cl, ws.y, ws.r, ws.k2, v_use, W.r_k.as<half>(), W.lnx_w.as<half>(), W.lnx_b.as<half>(),
                                  ws.g, ws.y2));
      }
    }
    // Tensor parallel: att.output and ffn.value see only this rank's slice of their input, so they emit fp32
    // partial sums that are added across ranks (NCCL) and rounded to half once, like the single-GPU layer.
    if (G == 1) {
      RK_TRY(lin(st, rows, W.Wo, ws.y2, ws.att, kEpiNone));
    } else if (tp_.peer_ready()) {  // partial sums into the peer-mapped buffer, summed by one kernel over NVLink
      RK_TRY(lin(st, rows, W.Wo, ws.y2, tp_.peer_partial(0), kEpiRawF32));
      RK_TRY(tp_.all_reduce_peer(0, static_cast<size_t>(rows) * C, ws.part32, timeout_dev_, st));
    } else {
      RK_TRY(lin(st, rows, W.Wo, ws.y2, ws.part32, kEpiRawF32));
      RK_TRY(tp_.all_reduce_sum(ws.part32, static_cast<size_t>(rows) * C, st));
    }
    {
      RowOpArgs a;
      a.B = B; a.T = T; a.C = C; a.x = ws.xA; a.x_out = ws.xB;
      if (G == 1) a.residual = ws.att;
      else a.residual_f32 = ws.part32;
      a.ln_w = W.ln2_w.as<half>(); a.ln_b = W.ln2_b.as<half>(); a.shift = shift1; a.n_mix = 1;
      a.mix[0] = W.ffn_x_k.as<half>(); a.mix_out[0] = ws.mixed;
      RK_TRY(row_op(st, a));
    }
    RK_TRY(lin(st, rows, W.Wkey, ws.mixed, ws.hid, kEpiRelu2));
    RowOpArgs a;
    a.B = B; a.T = T; a.C = C; a.x = ws.xB;
    if (G == 1) {
      RK_TRY(lin(st, rows, W.Wval, ws.hid, ws.ffn, kEpiNone));
      a.residual = ws.ffn;
    } else if (tp_.peer_ready()) {  // (the two all-reduces of a layer alternate between the two partial buffers)
      RK_TRY(lin(st, rows, W.Wval, ws.hid, tp_.peer_partial(1), kEpiRawF32));
      RK_TRY(tp_.all_reduce_peer(1, static_cast<size_t>(rows) * C, ws.part32, timeout_dev_, st));
      a.residual_f32 = ws.part32;
    } else {
      RK_TRY(lin(st, rows, W.Wval, ws.hid, ws.part32, kEpiRawF32));
      RK_TRY(tp_.all_reduce_sum(ws.part32, static_cast<size_t>(rows) * C, st));
      a.residual_f32 = ws.part32;
    }
    if (li + 1 < L) {
      const LayerWeights& Nx = layers_[static_cast<size_t>(li) + 1];
      a.x_out = ws.xA; a.ln_w = Nx.ln1_w.as<half>(); a.ln_b = Nx.ln1_b.as<half>();
      a.shift = shift + static_cast<size_t>(li + 1) * 2 * B * C; a.n_mix = 6;
      for (int i = 0; i < 6; ++i) { a.mix[i] = Nx.mix[i].as<half>(); a.mix_out[i] = ws.xm[i]; }
    } else {
      a.ln_w = ln_out_w_.as<half>(); a.ln_b = ln_out_b_.as<half>(); a.n_out = ws.xf; a.last_only = true;
    }
    RK_TRY(row_op(st, a));
  }
  RK_TRY(advance_i32(st, elapsed, T, B));
  if (G == 1) {
    RK_TRY(lin(st, B, head_, ws.xf, logits, kEpiF32));
  } else {
    // every rank computes its slice of the vocabulary; gather [G][B][V/G] and interleave to [B][V]
    const int Vl = cfg_.vocab / G;
    float* loc = ws.part32;
    float* all = loc + static_cast<size_t>(B) * Vl;
    RK_TRY(lin(st, B, head_, ws.xf, loc, kEpiF32));
    RK_TRY(tp_.all_gather(loc, all, static_cast<size_t>(B) * Vl, st));
    RK_TRY(interleave_gathered(st, all, logits, G, B, Vl));
  }
  return kOk;
}

int Model::forward(const int64_t* tokens_host, int B, int T, void* shift, void* wkv, int* elapsed, float* logits,
                   cudaStream_t stream) {
  RK_REQUIRE(finalized_, kNotReady, "forward: model not finalised");
  RK_REQUIRE(B > 0, kBadArg, "token_batches must not be empty");
  RK_REQUIRE(T > 0, kBadArg, "token batch length must be positive");
  RK_REQUIRE(tokens_host && shift && wkv && elapsed && logits, kBadArg, "forward: null pointer");
  const long long rows = static_cast<long long>(B) * T;
  for (long long i = 0; i < rows; ++i)
    RK_REQUIRE(tokens_host[i] >= 0 && tokens_host[i] < cfg_.vocab, kBadArg, "token id out of range");
  int s = use_device();
  if (s != kOk) return s;
  std::lock_guard<std::mutex> lock(mu_);
  return step(tokens_host, B, T, shift, wkv, elapsed, logits, stream);
}

// One forward with mu_ held.  tokens_host == nullptr: the ids are in the workspace's device buffer already (written
// by the greedy pick of the previous step).
int Model::step(const int64_t* tokens_host, int B, int T, void* shift, void* wkv, int* elapsed, float* logits,
                cudaStream_t stream) {
  const long long rows = static_cast<long long>(B) * T;
  int s = kOk;
  if ((s = prepare(B, T, stream)) != kOk) return s;
  Workspace* ws = &ws_;
  if (tokens_host) {
    const int slot = slot_;
    slot_ = (slot + 1) % kSlots;
    RK_CUDA(cudaEventSynchronize(tokens_copied_[slot]));  // the copy that last read this slot is done
    std::memcpy(tokens_pinned_[slot], tokens_host, static_cast<size_t>(rows) * sizeof(int64_t));
    RK_CUDA(cudaMemcpyAsync(ws->tokens, tokens_pinned_[slot], static_cast<size_t>(rows) * sizeof(int64_t), cudaMemcpyHostToDevice, stream));
    RK_CUDA(cudaEventRecord(tokens_copied_[slot], stream));
  }
  s = run(*ws, B, T, shift, wkv, elapsed, logits, stream);
  if (s != kOk) return s;
  RK_CUDA(cudaEventRecord(last_done_, stream));
  last_stream_ = stream;
  have_last_ = true;
  return kOk;
}

int Model::run(Workspace& wsr, int B, int T, void* shift, void* wkv, int* elapsed, float* logits, cudaStream_t stream) {
  Workspace* ws = &wsr;
  int s = kOk;
  auto direct = [&]() {
    const long long before = launch_counter();
    const int r = enqueue(*ws, B, T, static_cast<half*>(shift), wkv, elapsed, logits, stream);
    launches_ += launch_counter() - before;
    return r;
  };
  if (stream == nullptr || !options().decode_graphs) return direct();
  // A call that repeats (same shape, same buffers: decode steps, the chunks of a long prompt) replays a captured graph
  // from its second occurrence on; the first one is enqueued directly (one-off shapes never pay for a capture, and
  // libraries that set themselves up on first use -- NCCL -- have done so before anything is captured).
  const GraphKey key{B, T, shift, wkv, elapsed, logits};
  auto it = graphs_.find(key);
  if (it == graphs_.end()) {
    if (graphs_.size() >= 16) {  // evict the least recently used
      auto victim = graphs_.begin();
      for (auto g = graphs_.begin(); g != graphs_.end(); ++g)
        if (g->second.last_use < victim->second.last_use) victim = g;
      if (victim->second.exec) cudaGraphExecDestroy(victim->second.exec);
      graphs_.erase(victim);
    }
    GraphEntry e;
    e.last_use = ++tick_;
    graphs_.emplace(key, e);
    return direct();
  }
  GraphEntry& e = it->second;
  e.last_use = ++tick_;
  if (e.failed) return direct();
  if (!e.exec) {
    cudaGraph_t graph = nullptr;
    RK_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    const long long before = launch_counter();
    s = enqueue(*ws, B, T, static_cast<half*>(shift), wkv, elapsed, logits, stream);
    e.launches = launch_counter() - before;
    const cudaError_t ce = cudaStreamEndCapture(stream, &graph);
    if (s != kOk) {
      if (graph) cudaGraphDestroy(graph);
      return s;
    }
    cudaError_t ie = ce;
    if (ce == cudaSuccess) {
      ie = cudaGraphInstantiate(&e.exec, graph, 0);
      cudaGraphDestroy(graph);
    }
    if (ie != cudaSuccess) {  // (a collective library that cannot be captured here, ...): nothing ran, enqueue directly
      cudaGetLastError();
      e.exec = nullptr;
      e.failed = true;
      return direct();
    }
  }
  RK_CUDA(cudaGraphLaunch(e.exec, stream));
  launches_ += e.launches;
  return kOk;
}

// A run of greedy decode steps without a host round trip: after every step one kernel picks each sequence's token
// and writes it where the next step's embedding gather reads it.  Replaces, for top_p == 0, the loop
// forward_decode -> sampler -> copy to the host -> next forward_decode of the reference's engine
// (src/rwkv_sampler.cpp:47-111, src/utils/sampling.cu:205-471,507-512).
int Model::decode_greedy(const int64_t* first_tokens_host, int B, int steps, void* shift, void* wkv, int* elapsed,
                         float* logits, float* penalties, float presence, float repetition, float decay, int* out_tokens,
                         cudaStream_t stream, const rwkv7_b200_sampling* sampling) {
  RK_REQUIRE(finalized_, kNotReady, "decode_greedy: model not finalised");
  RK_REQUIRE(B > 0, kBadArg, "token_batches must not be empty");
  RK_REQUIRE(steps > 0, kBadArg, "decode_greedy: steps must be positive");
  RK_REQUIRE(first_tokens_host && shift && wkv && elapsed && logits && out_tokens, kBadArg, "decode_greedy: null pointer");
  RK_REQUIRE(tp_size_ == 1, kBadArg, "decode_greedy: not available for a tensor-parallel model");
  for (int i = 0; i < B; ++i)
    RK_REQUIRE(first_tokens_host[i] >= 0 && first_tokens_host[i] < cfg_.vocab, kBadArg, "token id out of range");
  int s = use_device();
  if (s != kOk) return s;
  std::lock_guard<std::mutex> lock(mu_);
  if (sampling) {
    RK_REQUIRE(sampling->temperature >= 0.001f && sampling->temperature <= 1000.f, kBadArg, "decode_sample: temperature outside [0.001, 1000]");
    const size_t need = static_cast<size_t>(B) * cfg_.vocab * sizeof(float);
    if (need > probs_.bytes) {
      RK_CUDA(cudaDeviceSynchronize());
      if ((s = probs_.alloc(need)) != kOk) return s;
    }
  }
  for (int i = 0; i < steps; ++i) {
    s = step(i == 0 ? first_tokens_host : nullptr, B, 1, shift, wkv, elapsed, logits, stream);
    if (s != kOk) return s;
    Workspace* ws = &ws_;
    const long long before = launch_counter();
    int* out_i = out_tokens + static_cast<size_t>(i) * B;
    if (sampling)
      s = sample_tokens(stream, B, cfg_.vocab, logits, penalties, probs_.as<float>(), presence, repetition, decay, sampling->temperature,
                        sampling->top_k, sampling->top_p, sampling->seed, sampling->offset + static_cast<unsigned long long>(i), out_i, ws->tokens);
    else
      s = greedy_pick(stream, B, cfg_.vocab, logits, penalties, presence, repetition, decay, out_i, ws->tokens);
    launches_ += launch_counter() - before;
    if (s != kOk) return s;
    RK_CUDA(cudaEventRecord(last_done_, stream));  // the pick wrote the token buffer after the step's own record
  }
  return kOk;
}

}  // namespace rk
