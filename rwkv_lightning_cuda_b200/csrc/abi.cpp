// extern "C" surface of librwkv7_b200.so; declarations and reference citations are in
// include/rwkv7_b200.h.  Thin by design: argument checks, then the C++ engine or a launcher.
#include "../../include/rwkv7_b200.h"

#include <new>

#include "kernels.h"
#include "model.h"

namespace rk {
const char* last_error();
int gemm_tc_static_scratch(cudaStream_t stream, const LinearArgs& a);
int gemm_last_max_splits();
}

using rk::kBadArg;
using rk::kOk;

struct rwkv7_b200_model {
  rk::Model impl;
  explicit rwkv7_b200_model(const rwkv7_b200_config& c) : impl(c) {}
};

namespace {
inline cudaStream_t st(void* s) { return static_cast<cudaStream_t>(s); }
inline const half* h(const uint16_t* p) { return reinterpret_cast<const half*>(p); }
inline half* h(uint16_t* p) { return reinterpret_cast<half*>(p); }
}  // namespace

extern "C" {

const char* rwkv7_b200_last_error(void) { return rk::last_error(); }
int rwkv7_b200_abi_version(void) { return 1; }

int rwkv7_b200_model_create(const rwkv7_b200_config* cfg, rwkv7_b200_model** out) {
  RK_REQUIRE(cfg && out, kBadArg, "model_create: null argument");
  RK_REQUIRE(cfg->layers > 0 && cfg->channels > 0 && cfg->ffn > 0 && cfg->vocab > 0, rk::kShape, "model_create: dimensions must be positive");
  RK_REQUIRE(cfg->channels % 64 == 0, rk::kShape, "model_create: channels must be a multiple of the head size 64");
  RK_REQUIRE(cfg->ffn % 32 == 0 && cfg->channels % 32 == 0, rk::kShape, "model_create: channels and ffn must be multiples of 32");
  for (int r : {cfg->rank_w, cfg->rank_a, cfg->rank_v, cfg->rank_g})
    RK_REQUIRE(r > 0 && r <= 512 && r % 8 == 0, rk::kShape, "model_create: LoRA ranks must be multiples of 8 in (0, 512]");
  RK_REQUIRE(cfg->weight_format >= 0 && cfg->weight_format <= 2, kBadArg, "model_create: unknown weight format");
  RK_REQUIRE(cfg->weight_format != RWKV7_B200_FMT_W4A16 || (cfg->channels % 128 == 0 && cfg->ffn % 128 == 0), rk::kShape,
             "model_create: W4A16 needs channels and ffn to be multiples of 128");
  if (cfg->tp_size > 1) {
    const int G = cfg->tp_size;
    RK_REQUIRE(cfg->tp_rank >= 0 && cfg->tp_rank < G, kBadArg, "model_create: tp_rank %d outside [0, %d)", cfg->tp_rank, G);
    RK_REQUIRE(cfg->weight_format == RWKV7_B200_FMT_F16, kBadArg, "model_create: tensor parallelism supports fp16 weights only");
    RK_REQUIRE(cfg->channels % (64 * G) == 0, rk::kShape, "model_create: the head count %d does not divide over %d ranks",
               cfg->channels / 64, G);
    RK_REQUIRE(cfg->ffn % (32 * G) == 0 && cfg->vocab % (4 * G) == 0, rk::kShape,
               "model_create: ffn must be a multiple of 32*tp_size and vocab of 4*tp_size");
  }
  rwkv7_b200_model* m = new (std::nothrow) rwkv7_b200_model(*cfg);
  RK_REQUIRE(m, rk::kCuda, "model_create: out of host memory");
  *out = m;
  return kOk;
}

int rwkv7_b200_model_set_tensor(rwkv7_b200_model* m, const char* name, const void* data, int dtype, long long count,
                                int on_device) {
  RK_REQUIRE(m, kBadArg, "null model");
  return m->impl.set_tensor(name, data, dtype, count, on_device);
}
int rwkv7_b200_tp_unique_id(void* out128) { return rk::TpComm::make_unique_id(out128); }
int rwkv7_b200_model_tp_init(rwkv7_b200_model* m, const void* unique_id) {
  RK_REQUIRE(m, kBadArg, "null model");
  return m->impl.tp_init(unique_id);
}
int rwkv7_b200_model_finalize(rwkv7_b200_model* m) {
  RK_REQUIRE(m, kBadArg, "null model");
  return m->impl.finalize();
}
int rwkv7_b200_model_destroy(rwkv7_b200_model* m) {
  delete m;
  return kOk;
}
int rwkv7_b200_vocab_size(const rwkv7_b200_model* m) { return m ? m->impl.cfg().vocab : 0; }

int rwkv7_b200_state_sizes(const rwkv7_b200_model* m, int B, size_t* shift_elems, size_t* wkv_elems, size_t* elapsed_elems) {
  RK_REQUIRE(m, kBadArg, "null model");
  return m->impl.state_sizes(B, shift_elems, wkv_elems, elapsed_elems);
}
int rwkv7_b200_state_init(const rwkv7_b200_model* m, int B, void* shift, void* wkv, int* elapsed, void* stream) {
  RK_REQUIRE(m, kBadArg, "null model");
  return m->impl.state_init(B, shift, wkv, elapsed, st(stream));
}

int rwkv7_b200_forward(rwkv7_b200_model* m, const int64_t* tokens_host, int B, int T, void* shift, void* wkv, int* elapsed,
                       float* logits, void* stream) {
  RK_REQUIRE(m, kBadArg, "null model");
  return m->impl.forward(tokens_host, B, T, shift, wkv, elapsed, logits, st(stream));
}

int rwkv7_b200_forward_to_host(rwkv7_b200_model* m, const int64_t* tokens_host, int B, int T, void* shift, void* wkv,
                               int* elapsed, float* logits, float* logits_host, void* stream) {
  RK_REQUIRE(m && logits_host, kBadArg, "forward_to_host: null argument");
  int s = m->impl.forward(tokens_host, B, T, shift, wkv, elapsed, logits, st(stream));
  if (s != kOk) return s;
  RK_CUDA(cudaMemcpyAsync(logits_host, logits, static_cast<size_t>(B) * m->impl.cfg().vocab * sizeof(float),
                          cudaMemcpyDeviceToHost, st(stream)));
  if ((s = m->impl.enqueue_timeout_read(st(stream))) != kOk) return s;
  RK_CUDA(cudaStreamSynchronize(st(stream)));
  return m->impl.timeout_result();
}

int rwkv7_b200_decode_greedy(rwkv7_b200_model* m, const int64_t* first_tokens_host, int B, int steps, void* shift, void* wkv,
                             int* elapsed, float* logits, float* penalties, float presence_penalty, float repetition_penalty,
                             float penalty_decay, int* out_tokens, int* out_tokens_host, void* stream) {
  RK_REQUIRE(m, kBadArg, "null model");
  int s = m->impl.decode_greedy(first_tokens_host, B, steps, shift, wkv, elapsed, logits, penalties, presence_penalty,
                                repetition_penalty, penalty_decay, out_tokens, st(stream));
  if (s != kOk || !out_tokens_host) return s;
  RK_CUDA(cudaMemcpyAsync(out_tokens_host, out_tokens, static_cast<size_t>(B) * steps * sizeof(int), cudaMemcpyDeviceToHost,
                          st(stream)));
  if ((s = m->impl.enqueue_timeout_read(st(stream))) != kOk) return s;
  RK_CUDA(cudaStreamSynchronize(st(stream)));
  return m->impl.timeout_result();
}

int rwkv7_b200_decode_sample(rwkv7_b200_model* m, const int64_t* first_tokens_host, int B, int steps, void* shift, void* wkv,
                             int* elapsed, float* logits, float* penalties, float presence_penalty, float repetition_penalty,
                             float penalty_decay, const rwkv7_b200_sampling* sampling, int* out_tokens, int* out_tokens_host,
                             void* stream) {
  RK_REQUIRE(m && sampling, kBadArg, "decode_sample: null argument");
  int s = m->impl.decode_greedy(first_tokens_host, B, steps, shift, wkv, elapsed, logits, penalties, presence_penalty,
                                repetition_penalty, penalty_decay, out_tokens, st(stream), sampling);
  if (s != kOk || !out_tokens_host) return s;
  RK_CUDA(cudaMemcpyAsync(out_tokens_host, out_tokens, static_cast<size_t>(B) * steps * sizeof(int), cudaMemcpyDeviceToHost,
                          st(stream)));
  if ((s = m->impl.enqueue_timeout_read(st(stream))) != kOk) return s;
  RK_CUDA(cudaStreamSynchronize(st(stream)));
  return m->impl.timeout_result();
}

int rwkv7_b200_sample(void* stream, int B, int V, const float* logits, float* penalties, float* probs, float presence_penalty,
                      float repetition_penalty, float penalty_decay, const rwkv7_b200_sampling* sampling, int* out,
                      int64_t* next_tokens) {
  RK_REQUIRE(sampling, kBadArg, "sample: null sampling parameters");
  return rk::sample_tokens(st(stream), B, V, logits, penalties, probs, presence_penalty, repetition_penalty, penalty_decay,
                           sampling->temperature, sampling->top_k, sampling->top_p, sampling->seed, sampling->offset, out, next_tokens);
}

int rwkv7_b200_greedy_pick(void* stream, int B, int V, const float* logits, float* penalties, float presence_penalty,
                           float repetition_penalty, float penalty_decay, int* out, int64_t* next_tokens) {
  return rk::greedy_pick(st(stream), B, V, logits, penalties, presence_penalty, repetition_penalty, penalty_decay, out,
                         next_tokens);
}

int rwkv7_b200_copy_state_slice(const rwkv7_b200_model* m, const void* src_shift, const void* src_wkv, const int* src_elapsed,
                                int src_B, int src_offset, void* dst_shift, void* dst_wkv, int* dst_elapsed, int dst_B,
                                int dst_offset, int count, void* stream) {
  RK_REQUIRE(m, kBadArg, "null model");
  return m->impl.copy_state_slice(src_shift, src_wkv, src_elapsed, src_B, src_offset, dst_shift, dst_wkv, dst_elapsed, dst_B,
                                  dst_offset, count, st(stream));
}

int rwkv7_b200_state_blob_sizes(const rwkv7_b200_model* m, size_t* shift_bytes, size_t* wkv_bytes, size_t* elapsed_bytes) {
  RK_REQUIRE(m, kBadArg, "null model");
  size_t ns = 0, nw = 0, ne = 0;
  int s = m->impl.state_sizes(1, &ns, &nw, &ne);
  if (s != kOk) return s;
  if (shift_bytes) *shift_bytes = ns * 2;
  if (wkv_bytes) *wkv_bytes = nw * (m->impl.cfg().wkv32 ? 4 : 2);
  if (elapsed_bytes) *elapsed_bytes = ne * sizeof(int);
  return kOk;
}
int rwkv7_b200_state_export(const rwkv7_b200_model* m, const void* shift, const void* wkv, const int* elapsed, int B, int index,
                            void* shift_blob_host, void* wkv_blob_host, int* elapsed_blob_host, void* stream) {
  RK_REQUIRE(m, kBadArg, "null model");
  return m->impl.state_export(shift, wkv, elapsed, B, index, shift_blob_host, wkv_blob_host, elapsed_blob_host, st(stream));
}
int rwkv7_b200_state_import(const rwkv7_b200_model* m, const void* shift_blob_host, const void* wkv_blob_host,
                            const int* elapsed_blob_host, void* shift, void* wkv, int* elapsed, int B, int index, void* stream) {
  RK_REQUIRE(m, kBadArg, "null model");
  return m->impl.state_import(shift_blob_host, wkv_blob_host, elapsed_blob_host, shift, wkv, elapsed, B, index, st(stream));
}
int rwkv7_b200_state_convert_wkv(void* stream, const void* src, void* dst, long long elems, int src_is_fp32) {
  return rk::wkv_state_convert(st(stream), src, dst, elems, src_is_fp32);
}

int rwkv7_b200_query_capacity(const rwkv7_b200_model* m, int chunk, rwkv7_b200_capacity* out) {
  RK_REQUIRE(m, kBadArg, "null model");
  return m->impl.query_capacity(chunk, out);
}

long long rwkv7_b200_kernel_launches(const rwkv7_b200_model* m) { return m ? m->impl.launches() : 0; }

int rwkv7_b200_model_workspace_bytes(const rwkv7_b200_model* m, size_t* out) {
  RK_REQUIRE(m && out, kBadArg, "workspace_bytes: null argument");
  *out = m->impl.workspace_bytes();
  return kOk;
}

int rwkv7_b200_timeout_flags(int clear, int* flags) {
  RK_REQUIRE(flags, kBadArg, "timeout_flags: null output");
  return rk::timeout_read(flags, clear != 0);
}
int rwkv7_b200_debug_last_gemm_splits(void) { return rk::gemm_last_max_splits(); }
int rwkv7_b200_debug_timeout_detail(int* out15, int clear) { return rk::timeout_detail(out15, clear != 0); }
int rwkv7_b200_debug_wait_probe(void* stream, unsigned polls) { return rk::wait_probe(st(stream), polls); }
int rwkv7_b200_set_option(const char* name, int value) { return rk::set_option(name, value); }

// ---------------------------------------------------------------- op level

int rwkv7_b200_wkv_fp16_seq(void* stream, int B, int T, int C, int H, uint16_t* state, const uint16_t* r, const uint16_t* w,
                            const uint16_t* k, const uint16_t* v, const uint16_t* a, const uint16_t* b, uint16_t* y,
                            const int* elapsed) {
  return rk::wkv7_fp16(st(stream), B, T, C, H, h(state), h(r), h(w), nullptr, 0, h(k), h(v), h(a), h(b), h(y), elapsed);
}
int rwkv7_b200_wkv_fp16_seq_w0(void* stream, int B, int T, int C, int H, uint16_t* state, const uint16_t* r,
                               const uint16_t* w, const uint16_t* w0, const uint16_t* k, const uint16_t* v,
                               const uint16_t* a, const uint16_t* b, uint16_t* y, const int* elapsed) {
  return rk::wkv7_fp16(st(stream), B, T, C, H, h(state), h(r), h(w), h(w0), 1, h(k), h(v), h(a), h(b), h(y), elapsed);
}
int rwkv7_b200_wkv_fp32io16(void* stream, int B, int T, int C, int H, float* state, const uint16_t* r, const uint16_t* w,
                            const uint16_t* k, const uint16_t* v, const uint16_t* a, const uint16_t* b, uint16_t* y) {
  return rk::wkv7_fp32(st(stream), B, T, C, H, state, h(r), h(w), nullptr, h(k), h(v), h(a), h(b), h(y));
}

int rwkv7_b200_tmix_mix6(void* stream, int B, int T, int C, const uint16_t* x, uint16_t* shift, const uint16_t* const* mix,
                         uint16_t* const* out) {
  RK_REQUIRE(mix && out, kBadArg, "tmix_mix6: null pointer table");
  rk::RowOpArgs a;
  a.B = B; a.T = T; a.C = C; a.x = h(x); a.shift = h(shift); a.n_mix = 6; a.identity_norm = true;
  for (int i = 0; i < 6; ++i) { a.mix[i] = h(mix[i]); a.mix_out[i] = h(out[i]); }
  return rk::row_op(st(stream), a);
}
int rwkv7_b200_cmix_mix(void* stream, int B, int T, int C, const uint16_t* x, uint16_t* shift, const uint16_t* x_k,
                        uint16_t* out) {
  rk::RowOpArgs a;
  a.B = B; a.T = T; a.C = C; a.x = h(x); a.shift = h(shift); a.n_mix = 1; a.identity_norm = true;
  a.mix[0] = h(x_k); a.mix_out[0] = h(out);
  return rk::row_op(st(stream), a);
}
int rwkv7_b200_tmix_kk_a_gate(void* stream, int B, int T, int C, int H, const uint16_t* k, const uint16_t* k_k,
                              const uint16_t* a0, const uint16_t* a12, const uint16_t* k_a, uint16_t* new_k,
                              uint16_t* neg_kk, uint16_t* kka) {
  RK_REQUIRE(C == H * 64, rk::kShape, "kk_a_gate: C must equal 64*H");
  return rk::tmix_kk_a_gate(st(stream), B * T, C, h(k), h(k_k), h(a0), h(a12), h(k_a), h(new_k), h(neg_kk), h(kka));
}
int rwkv7_b200_tmix_lnx_rkvres_xg(void* stream, int B, int T, int C, int H, const uint16_t* x, const uint16_t* r,
                                  const uint16_t* k, const uint16_t* v, const uint16_t* r_k, const uint16_t* weight,
                                  const uint16_t* bias, const uint16_t* g, uint16_t* out) {
  RK_REQUIRE(C == H * 64, rk::kShape, "lnx_rkvres_xg: C must equal 64*H");
  return rk::tmix_lnx_rkvres_xg(st(stream), B * T, C, h(x), h(r), h(k), h(v), h(r_k), h(weight), h(bias), h(g), h(out));
}
int rwkv7_b200_tmix_vres_gate(void* stream, int B, int T, int C, const uint16_t* v, const uint16_t* v_first,
                              const uint16_t* v0, const uint16_t* v12, uint16_t* out) {
  return rk::tmix_vres_gate(st(stream), B * T, C, h(v), h(v_first), h(v0), h(v12), h(out));
}

int rwkv7_b200_layer_norm_f16(void* stream, int rows, int C, const uint16_t* x, const uint16_t* weight, const uint16_t* bias,
                              uint16_t* y, float eps) {
  rk::RowOpArgs a;
  a.B = rows; a.T = 1; a.C = C; a.x = h(x); a.ln_w = h(weight); a.ln_b = h(bias); a.n_out = h(y); a.eps = eps;
  RK_REQUIRE(y, kBadArg, "layer_norm: null output");
  return rk::row_op(st(stream), a);
}
int rwkv7_b200_add_layer_norm_f16(void* stream, int rows, int C, const uint16_t* x, const uint16_t* residual,
                                  const uint16_t* weight, const uint16_t* bias, uint16_t* x_out, uint16_t* y, float eps) {
  RK_REQUIRE(residual && y, kBadArg, "add_layer_norm: null pointer");
  rk::RowOpArgs a;
  a.B = rows; a.T = 1; a.C = C; a.x = h(x); a.residual = h(residual); a.x_out = h(x_out);
  a.ln_w = h(weight); a.ln_b = h(bias); a.n_out = h(y); a.eps = eps;
  return rk::row_op(st(stream), a);
}
int rwkv7_b200_add_last_layer_norm_f16(void* stream, int B, int T, int C, const uint16_t* x, const uint16_t* residual,
                                       const uint16_t* weight, const uint16_t* bias, uint16_t* y, float eps) {
  RK_REQUIRE(residual && y, kBadArg, "add_last_layer_norm: null pointer");
  rk::RowOpArgs a;
  a.B = B; a.T = T; a.C = C; a.x = h(x); a.residual = h(residual); a.ln_w = h(weight); a.ln_b = h(bias);
  a.n_out = h(y); a.last_only = true; a.eps = eps;
  return rk::row_op(st(stream), a);
}
int rwkv7_b200_add_layer_norm_cmix_mix_f16(void* stream, int B, int T, int C, const uint16_t* x, const uint16_t* residual,
                                           uint16_t* shift, const uint16_t* weight, const uint16_t* bias,
                                           const uint16_t* x_k, uint16_t* x_out, uint16_t* mixed, float eps) {
  RK_REQUIRE(residual, kBadArg, "add_layer_norm_cmix_mix: null pointer");
  rk::RowOpArgs a;
  a.B = B; a.T = T; a.C = C; a.x = h(x); a.residual = h(residual); a.x_out = h(x_out); a.ln_w = h(weight); a.ln_b = h(bias);
  a.shift = h(shift); a.n_mix = 1; a.mix[0] = h(x_k); a.mix_out[0] = h(mixed); a.eps = eps;
  return rk::row_op(st(stream), a);
}
int rwkv7_b200_add_layer_norm_tmix_mix6_f16(void* stream, int B, int T, int C, const uint16_t* x, const uint16_t* residual,
                                            uint16_t* shift, const uint16_t* weight, const uint16_t* bias,
                                            const uint16_t* const* mix, uint16_t* x_out, uint16_t* const* out, float eps) {
  RK_REQUIRE(residual && mix && out, kBadArg, "add_layer_norm_tmix_mix6: null pointer");
  rk::RowOpArgs a;
  a.B = B; a.T = T; a.C = C; a.x = h(x); a.residual = h(residual); a.x_out = h(x_out); a.ln_w = h(weight); a.ln_b = h(bias);
  a.shift = h(shift); a.n_mix = 6; a.eps = eps;
  for (int i = 0; i < 6; ++i) { a.mix[i] = h(mix[i]); a.mix_out[i] = h(out[i]); }
  return rk::row_op(st(stream), a);
}
int rwkv7_b200_emb_ln0(void* stream, int V, int C, const void* emb, const void* weight, const void* bias, int dtype,
                       uint16_t* out, float eps) {
  RK_REQUIRE(dtype == RWKV7_B200_DT_F16 || dtype == RWKV7_B200_DT_BF16, kBadArg, "emb_ln0: unknown dtype");
  return rk::emb_ln0(st(stream), V, C, emb, weight, bias, dtype == RWKV7_B200_DT_BF16, h(out), eps);
}
int rwkv7_b200_relu_square(void* stream, const uint16_t* x, uint16_t* out, long long elems) {
  return rk::relu_square(st(stream), h(x), h(out), elems);
}
int rwkv7_b200_advance_i32(void* stream, int* x, int amount, long long elems) {
  return rk::advance_i32(st(stream), x, amount, static_cast<int>(elems));
}

static int linear_common(void* stream, int M, int K, int N, const uint16_t* x, const void* w, int fmt, const uint16_t* scale,
                         const uint16_t* zero, int in_act, int epilogue, void* y) {
  RK_REQUIRE(epilogue == RWKV7_B200_EPI_NONE || epilogue == RWKV7_B200_EPI_RELU2 || epilogue == RWKV7_B200_EPI_F32, kBadArg,
             "linear: unknown epilogue %d", epilogue);
  RK_REQUIRE(in_act >= 0 && in_act <= 2, kBadArg, "linear: unknown input activation %d", in_act);
  rk::LinearArgs a;
  a.M = M; a.K = K; a.N = N; a.x = h(x); a.w = w; a.fmt = fmt; a.scale = h(scale); a.zero = h(zero);
  a.in_act = in_act; a.epi = epilogue; a.y = y;
  return rk::linear(st(stream), a);
}
int rwkv7_b200_linear_f16_orig(void* stream, int M, int K, int N, const uint16_t* x, const uint16_t* weight, int in_act,
                               int epilogue, void* y) {
  return linear_common(stream, M, K, N, x, weight, RWKV7_B200_FMT_F16, nullptr, nullptr, in_act, epilogue, y);
}
int rwkv7_b200_linear_f16_orig_static(void* stream, int M, int K, int N, const uint16_t* x, const uint16_t* weight,
                                      int epilogue, void* y) {
  RK_REQUIRE(epilogue == RWKV7_B200_EPI_NONE || epilogue == RWKV7_B200_EPI_RELU2 || epilogue == RWKV7_B200_EPI_F32, kBadArg,
             "linear: unknown epilogue %d", epilogue);
  RK_REQUIRE(M > 0 && K > 0 && N > 0 && x && weight && y, kBadArg, "linear (static scratch): bad argument");
  rk::LinearArgs a;
  a.M = M; a.K = K; a.N = N; a.x = h(x); a.w = weight; a.fmt = RWKV7_B200_FMT_F16; a.epi = epilogue; a.y = y;
  return rk::gemm_tc_static_scratch(st(stream), a);
}
int rwkv7_b200_linear_w8a16(void* stream, int M, int K, int N, const uint16_t* x, const int8_t* q, const uint16_t* scale,
                            int epilogue, void* y) {
  return linear_common(stream, M, K, N, x, q, RWKV7_B200_FMT_W8A16, scale, nullptr, 0, epilogue, y);
}
int rwkv7_b200_linear_w4a16(void* stream, int M, int K, int N, const uint16_t* x, const uint8_t* q, const uint16_t* scale,
                            const uint16_t* zero, int epilogue, void* y) {
  return linear_common(stream, M, K, N, x, q, RWKV7_B200_FMT_W4A16, scale, zero, 0, epilogue, y);
}
int rwkv7_b200_quant_pack_w8(void* stream, int N, int K, const uint16_t* W, int8_t* q, uint16_t* scale) {
  return rk::quant_pack_w8(st(stream), N, K, h(W), q, h(scale));
}
int rwkv7_b200_quant_unpack_w8(void* stream, int N, int K, const int8_t* q, const uint16_t* scale, uint16_t* W) {
  return rk::quant_unpack_w8(st(stream), N, K, q, h(scale), h(W));
}
int rwkv7_b200_quant_pack_w4(void* stream, int N, int K, const uint16_t* W, uint8_t* q, uint16_t* scale, uint16_t* zero) {
  return rk::quant_pack_w4(st(stream), N, K, h(W), q, h(scale), h(zero));
}
int rwkv7_b200_quant_unpack_w4(void* stream, int N, int K, const uint8_t* q, const uint16_t* scale, const uint16_t* zero,
                               uint16_t* W) {
  return rk::quant_unpack_w4(st(stream), N, K, q, h(scale), h(zero), h(W));
}

}  // extern "C"
