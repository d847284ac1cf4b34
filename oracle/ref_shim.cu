// C entry points around the UNMODIFIED reference sources (compiled from where they lie by
// oracle/Makefile target `ref`; nothing of the reference is copied into this repository).
// Test/benchmark infrastructure only: gives the parity tests and the benchmark's reference arm
// access to the reference's own kernels and to its real ModelBackend on the same GPU.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "rwkv7_fast_v4_kernels.cuh"
#include "rwkv_server_backend.hpp"

namespace {
thread_local std::string g_err;
inline const half* H(const uint16_t* p) { return reinterpret_cast<const half*>(p); }
inline half* H(uint16_t* p) { return reinterpret_cast<half*>(p); }
bool g_sync = true;  // op-level calls wait for their kernel unless a timing loop switches that off
int done(cudaStream_t s) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && g_sync) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    g_err = cudaGetErrorString(e);
    return 1;
  }
  return 0;
}
struct RefState {
  rwkv7_server::GenerationState st;
  rwkv7_server::DeviceLogits logits;
};
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }
// on = 0: the op-level calls below only enqueue (kernel-only timing with events around a run of them)
void ref_set_sync(int on) { g_sync = on != 0; }

int ref_wkv_fp16_seq(int B, int T, int C, int Hh, uint16_t* state, const uint16_t* r, const uint16_t* w, const uint16_t* k,
                     const uint16_t* v, const uint16_t* a, const uint16_t* b, uint16_t* y, const int* elapsed) {
  rwkv7_wkv_fp16_seq_launch(0, B, T, C, Hh, H(state), H(r), H(w), H(k), H(v), H(a), H(b), H(y), elapsed);
  return done(0);
}
int ref_wkv_fp16_seq_w0(int B, int T, int C, int Hh, uint16_t* state, const uint16_t* r, const uint16_t* w, const uint16_t* w0,
                        const uint16_t* k, const uint16_t* v, const uint16_t* a, const uint16_t* b, uint16_t* y,
                        const int* elapsed) {
  rwkv7_wkv_fp16_seq_w0_launch(0, B, T, C, Hh, H(state), H(r), H(w), H(w0), H(k), H(v), H(a), H(b), H(y), elapsed);
  return done(0);
}
int ref_wkv_fp32io16(int B, int T, int C, int Hh, float* state, const uint16_t* r, const uint16_t* w, const uint16_t* k,
                     const uint16_t* v, const uint16_t* a, const uint16_t* b, uint16_t* y) {
  rwkv7_wkv_fp32io16_launch(0, B, T, C, Hh, 0, state, H(r), H(w), H(k), H(v), H(a), H(b), H(y));
  return done(0);
}
int ref_add_vec(int C, const uint16_t* x, const uint16_t* vec, uint16_t* out, long long elems) {
  rwkv7_add_vec_launch(0, C, H(x), H(vec), H(out), elems);
  return done(0);
}
int ref_tmix_mix6(int B, int T, int C, const uint16_t* x, uint16_t* shift, const uint16_t* const* mix, uint16_t* const* out) {
  rwkv7_tmix_mix6_launch(0, B, T, C, H(x), H(shift), H(mix[0]), H(mix[1]), H(mix[2]), H(mix[3]), H(mix[4]), H(mix[5]),
                         H(out[0]), H(out[1]), H(out[2]), H(out[3]), H(out[4]), H(out[5]));
  return done(0);
}
int ref_cmix_mix(int B, int T, int C, const uint16_t* x, uint16_t* shift, const uint16_t* x_k, uint16_t* out) {
  rwkv7_cmix_mix_launch(0, B, T, C, H(x), H(shift), H(x_k), H(out));
  return done(0);
}
int ref_tmix_kk_a_gate(int B, int T, int C, int Hh, const uint16_t* k, const uint16_t* k_k, const uint16_t* a0,
                       const uint16_t* a12, const uint16_t* k_a, uint16_t* new_k, uint16_t* neg_kk, uint16_t* kka) {
  rwkv7_tmix_kk_a_gate_launch(0, B, T, C, Hh, H(k), H(k_k), H(a0), H(a12), H(k_a), H(new_k), H(neg_kk), H(kka));
  return done(0);
}
int ref_tmix_lnx_rkvres_xg(int B, int T, int C, int Hh, const uint16_t* x, const uint16_t* r, const uint16_t* k,
                           const uint16_t* v, const uint16_t* r_k, const uint16_t* w, const uint16_t* b, const uint16_t* g,
                           uint16_t* out) {
  rwkv7_tmix_lnx_rkvres_xg_launch(0, B, T, C, Hh, H(x), H(r), H(k), H(v), H(r_k), H(w), H(b), H(g), H(out));
  return done(0);
}
int ref_tmix_vres_gate(int B, int T, int C, const uint16_t* v, const uint16_t* v_first, const uint16_t* v0,
                       const uint16_t* v12, uint16_t* out) {
  rwkv7_tmix_vres_gate_launch(0, B, T, C, H(v), H(v_first), H(v0), H(v12), H(out));
  return done(0);
}
int ref_layer_norm(int rows, int C, const uint16_t* x, const uint16_t* w, const uint16_t* b, uint16_t* y, float eps) {
  rwkv7_v3a_layer_norm_f16_launch(0, rows, C, H(x), H(w), H(b), H(y), eps);
  return done(0);
}
int ref_add_layer_norm(int rows, int C, const uint16_t* x, const uint16_t* res, const uint16_t* w, const uint16_t* b,
                       uint16_t* x_out, uint16_t* y, float eps) {
  rwkv7_v3a_add_layer_norm_f16_launch(0, rows, C, H(x), H(res), H(w), H(b), H(x_out), H(y), eps);
  return done(0);
}
int ref_add_last_layer_norm(int B, int T, int C, const uint16_t* x, const uint16_t* res, const uint16_t* w,
                            const uint16_t* b, uint16_t* y, float eps) {
  rwkv7_v3a_add_last_layer_norm_f16_launch(0, B, T, C, H(x), H(res), H(w), H(b), H(y), eps);
  return done(0);
}
int ref_add_layer_norm_cmix_mix(int rows, int C, const uint16_t* x, const uint16_t* res, uint16_t* shift, const uint16_t* w,
                                const uint16_t* b, const uint16_t* x_k, uint16_t* x_out, uint16_t* mixed, float eps) {
  rwkv7_v3a_add_layer_norm_cmix_mix_f16_launch(0, rows, C, H(x), H(res), H(shift), H(w), H(b), H(x_k), H(x_out), H(mixed), eps);
  return done(0);
}
int ref_add_layer_norm_tmix_mix6(int rows, int C, const uint16_t* x, const uint16_t* res, uint16_t* shift, const uint16_t* w,
                                 const uint16_t* b, const uint16_t* const* mix, uint16_t* x_out, uint16_t* const* out,
                                 float eps) {
  rwkv7_v3a_add_layer_norm_tmix_mix6_f16_launch(0, rows, C, H(x), H(res), H(shift), H(w), H(b), H(mix[0]), H(mix[1]), H(mix[2]),
                                                H(mix[3]), H(mix[4]), H(mix[5]), H(x_out), H(out[0]), H(out[1]), H(out[2]),
                                                H(out[3]), H(out[4]), H(out[5]), eps);
  return done(0);
}
int ref_emb_ln0_bf16(int V, int C, const uint16_t* emb, const uint16_t* w, const uint16_t* b, uint16_t* out, float eps) {
  rwkv7_v4_emb_ln0_bf16_to_f16_launch(0, V, C, emb, w, b, out, eps);
  return done(0);
}
// exact = 1: the reference's own M<=2 GEMV kernel; 0: its cuBLAS path.
int ref_linear_orig(int M, int K, int N, const uint16_t* x, const uint16_t* w, uint16_t* y, int exact) {
  if (exact) rwkv7_v3a_linear_orig_rows_exact_f16_launch(0, M, K, N, H(x), H(w), 128, 2, false, H(y));
  else rwkv7_v3a_linear_f16_orig_launch(0, M, K, N, H(x), H(w), H(y));
  return done(0);
}
int ref_relu_square(const uint16_t* x, uint16_t* out, long long elems) {
  rwkv7_relu_square_launch(0, H(x), H(out), elems);
  return done(0);
}
int ref_cmix_sparse_down_relu_one(int C, int F, const uint16_t* preact, const uint16_t* value_fc, uint16_t* out) {
  rwkv7_cmix_sparse_down_relu_one_launch(0, C, F, H(preact), H(value_fc), H(out));
  return done(0);
}

// ---- the reference's real backend, fed from a bf16 .pth written by the caller
void* ref_backend_create(const char* path, int wkv32) {
  try {
    return new rwkv7_server::ModelBackend(path, wkv32 != 0, false);
  } catch (const std::exception& e) {
    g_err = e.what();
    return nullptr;
  }
}
void ref_backend_destroy(void* b) { delete static_cast<rwkv7_server::ModelBackend*>(b); }
void* ref_state_create(void* b, int B) {
  try {
    auto* s = new RefState();
    s->st = static_cast<rwkv7_server::ModelBackend*>(b)->create_state(B);
    return s;
  } catch (const std::exception& e) {
    g_err = e.what();
    return nullptr;
  }
}
void ref_state_destroy(void* s) { delete static_cast<RefState*>(s); }
// tokens [B][T] on the host.  logits_host may be NULL (then nothing is copied back).
int ref_forward(void* b, void* s, const int64_t* tokens, int B, int T, float* logits_host) {
  try {
    auto* be = static_cast<rwkv7_server::ModelBackend*>(b);
    auto* st = static_cast<RefState*>(s);
    if (T == 1) {
      std::vector<int64_t> tb(tokens, tokens + B);
      be->forward_decode(tb, st->st, st->logits);
    } else {
      std::vector<std::vector<int64_t>> tb(B);
      for (int i = 0; i < B; ++i) tb[i].assign(tokens + static_cast<size_t>(i) * T, tokens + static_cast<size_t>(i + 1) * T);
      be->forward_prefill(tb, st->st, st->logits);
    }
    if (logits_host) {
      cudaError_t e = cudaMemcpy(logits_host, st->logits.values.p, static_cast<size_t>(B) * be->vocab_size() * sizeof(float),
                                 cudaMemcpyDeviceToHost);
      if (e != cudaSuccess) {
        g_err = cudaGetErrorString(e);
        return 1;
      }
    }
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 2;
  }
}
// Copies the state buffers to the host (any pointer may be NULL).
int ref_state_read(void* s, uint16_t* shift, void* wkv, int* elapsed) {
  auto* st = static_cast<RefState*>(s);
  cudaError_t e = cudaSuccess;
  if (shift && e == cudaSuccess) e = cudaMemcpy(shift, st->st.shift.p, st->st.shift.n * 2, cudaMemcpyDeviceToHost);
  if (wkv && e == cudaSuccess) {
    if (st->st.wkv32) e = cudaMemcpy(wkv, st->st.wkv_state32.p, st->st.wkv_state32.n * 4, cudaMemcpyDeviceToHost);
    else e = cudaMemcpy(wkv, st->st.wkv_state.p, st->st.wkv_state.n * 2, cudaMemcpyDeviceToHost);
  }
  if (elapsed && e == cudaSuccess) e = cudaMemcpy(elapsed, st->st.elapsed.p, st->st.elapsed.n * 4, cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    g_err = cudaGetErrorString(e);
    return 1;
  }
  return 0;
}

}  // extern "C"
