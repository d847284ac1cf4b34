// Host-callable launchers of the sm_100a kernels (C++ linkage, used by the engine and by the
// C ABI's op-level exports).  All pointers are device pointers; every function enqueues work on
// `stream` and returns an rk::Status code without synchronising.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace rk {

// ---- status.cu : the device-side failure word and the library's run-time options
// Bits of the failure word: which kind of kernel gave up on a bounded wait.
enum TimeoutBit : int { kTimeoutGemv = 1, kTimeoutGemm = 2, kTimeoutTmix = 4, kTimeoutProbe = 8, kTimeoutPeer = 16 };
int timeout_word(int** device_ptr);           // address of the word on the current device (looked up once per device)
int* timeout_word_or_null();                  // the same for launchers: nullptr when the lookup fails
int timeout_detail(int* out15, bool clear);   // status.cu: the first expired GEMM wait of the current device
int timeout_read(int* flags, bool clear);     // blocking read (and reset) of the current device's word
int timeout_status(int flags);                // kOk, or kTimeout with the message set
int wait_probe(cudaStream_t stream, unsigned polls);  // a kernel whose bounded wait runs out by construction (tests)

// The few switches that exist for measurements and tests; rwkv7_b200_set_option() sets them by name.  Process-wide,
// read when a call is enqueued.
struct Options {
  int gemm_cta_pair = 0;     // 1: the tensor-core GEMM runs as CTA pairs (cta_group::2); measured equal, off by default
  int quant_tc_rows = 0;     // > 1: row count from which quantised weights take the tensor-core path (0: built-in)
  int fp16_tc_rows = 0;      // > 1: the same for fp16 weights
  int decode_graphs = 1;     // 0: decode steps are enqueued kernel by kernel instead of replaying a CUDA graph
  int wkv_chunked = 1;       // 0: fp32-state WKV over a chunk runs the per-token scan instead of the matrix form
  int tp_peer_ranks = 2;     // tensor parallelism: largest group whose all-reduce runs in the library's kernel over peer-mapped
                             // memory (larger groups use NCCL); read when a model first needs its peer region
  int gemv_mma_tall = 2;     // the mma.sync linear kernel walks the weights in tiles of 32 channels: 0 never, 1 one row of
                             // quantised weights, 2 one row of any format and up to three rows of fp16, 3 wherever they fit
  int gemv_mma = 3;          // 1..4 rows: 0 = scalar weight-streaming kernels only, 1 = the mma.sync kernel for quantised
                             // weights, 2 = also for 2..4 rows of fp16, 3 = also for one row of fp16 / W8A16 in large
                             // launches (8 MB and more, rows of 2 / 4 KiB and more), 4 = for every launch it accepts
};
Options& options();
int set_option(const char* name, int value);

// ---- wkv7.cu
int wkv7_fp16(cudaStream_t stream, int B, int T, int C, int H, half* state, const half* r, const half* w,
              const half* w0, int w_mode, const half* k, const half* v, const half* a, const half* b,
              half* y, const int* elapsed, int channel0 = 0);  // channel0: index of channel 0 in the whole model (a
                                                               // tensor-parallel rank's slice starts later): phase of the decay dither
int wkv7_fp32(cudaStream_t stream, int B, int T, int C, int H, float* state, const half* r, const half* w,
              const half* w0, const half* k, const half* v, const half* a, const half* b, half* y);
// wkv7_chunk.cu: the same recurrence over a chunk of tokens in matrix form on the tensor cores (wkv7_fp32 dispatches
// to it for chunks of 64 tokens and more)
bool wkv7_fp32_chunked_applies(int T);
int wkv7_fp32_chunked(cudaStream_t stream, int B, int T, int C, int H, float* state, const half* r, const half* w,
                      const half* w0, const half* k, const half* v, const half* a, const half* b, half* y);

// ---- rowops.cu : LayerNorm / residual / token-shift fusions, one CTA per activation row
struct RowOpArgs {
  int B = 0, T = 0, C = 0;
  float eps = 1e-5f;
  // source: either an embedding gather or x (+ residual)
  const int64_t* tokens = nullptr;  // [B*T] device, with `table`
  const half* table = nullptr;      // [V,C] embedding with LN0 folded in
  int vocab = 0;
  const half* x = nullptr;          // [B*T,C]
  const half* residual = nullptr;   // optional, added to x in fp32
  const float* residual_f32 = nullptr;  // instead of `residual`: fp32 values, rounded to half first (all-reduced partial sums)
  half* x_out = nullptr;            // optional: half(x + residual) or the gathered row
  // normalisation
  const half* ln_w = nullptr;
  const half* ln_b = nullptr;
  half* n_out = nullptr;            // optional: half(LN(.)) per row
  // token shift on the normalised rows
  half* shift = nullptr;            // [B,C] previous-token row, replaced by the last row
  int n_mix = 0;                    // 0, 1 (channel mix) or 6 (time mix)
  const half* mix[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  half* mix_out[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  // last_only: only row T-1 of each sequence is normalised, n_out is [B,C]
  bool identity_norm = false;        // token shift on the rows as given, no LayerNorm
  bool last_only = false;
  int* bad_token_flag = nullptr;    // set to 1 if a token id is outside [0, vocab)
};
int row_op(cudaStream_t stream, const RowOpArgs& args);

int tmix_kk_a_gate(cudaStream_t stream, int rows, int C, const half* k, const half* k_k, const half* a0,
                   const half* a12, const half* k_a, half* new_k, half* neg_kk, half* kka);
// tmix_kk_a_gate and tmix_vres_gate in one launch (the same warp handles a head's 64 channels for both)
int tmix_kk_a_vres_gate(cudaStream_t stream, int rows, int C, const half* k, const half* k_k, const half* a0, const half* a12,
                        const half* k_a, half* new_k, half* neg_kk, half* kka, const half* v, const half* v_first,
                        const half* v0, const half* v12, half* v_out);
int tmix_lnx_rkvres_xg(cudaStream_t stream, int rows, int C, const half* y, const half* r, const half* k,
                       const half* v, const half* r_k, const half* w, const half* b, const half* g, half* out);
int tmix_vres_gate(cudaStream_t stream, int rows, int C, const half* v, const half* v_first, const half* v0,
                   const half* v12, half* out);
int advance_i32(cudaStream_t stream, int* x, int amount, int n);
int wkv_state_convert(cudaStream_t stream, const void* src, void* dst, long long elems, int src_is_fp32);  // half <-> float

// Greedy token choice per sequence over fp32 logits [B, V] with optional penalties [B, V] (updated in place); the token
// goes to out[b] and, when next_tokens is given, to next_tokens[b] (the next decode step's input).  See greedy.cu.
int greedy_pick(cudaStream_t stream, int B, int V, const float* logits, float* penalties, float presence, float repetition,
                float decay, int* out, int64_t* next_tokens);
// Temperature / top-k / top-p sampling with penalties (sampler.cu): out[b] is drawn from the filtered distribution of
// row b with the counter-based random number of (seed, offset, b); probs is scratch, fp32 [B, V].
int sample_tokens(cudaStream_t stream, int B, int V, const float* logits, float* penalties, float* probs, float presence,
                  float repetition, float decay, float temperature, int top_k, float top_p, unsigned long long seed,
                  unsigned long long offset, int* out, int64_t* next_tokens);
// src [G][B][Vl] (one block per rank, as an all-gather leaves it) -> dst [B][G*Vl]
int interleave_gathered(cudaStream_t stream, const float* src, float* dst, int G, int B, int Vl);
int relu_square(cudaStream_t stream, const half* x, half* out, long long n);
int activate(cudaStream_t stream, const half* x, half* out, long long n, int act);  // half(tanh(x)) / half(sigmoid(x))
int bf16_to_f16(cudaStream_t stream, const uint16_t* src, half* dst, long long n);
int transpose_f16(cudaStream_t stream, const half* src, half* dst, int rows, int cols);
int emb_ln0(cudaStream_t stream, int V, int C, const void* emb, const void* w, const void* b, int src_is_bf16,
            half* out, float eps);

// ---- linear.cu : y = act(x) W^T with W [N,K] row-major ("orig" layout of the checkpoint)
struct LinearArgs {
  int M = 0, K = 0, N = 0;
  const half* x = nullptr;   // [M,K]
  int ldx = 0;               // row stride of x in elements (0 = K)
  const void* w = nullptr;   // fp16 [N,K] | int8 [N,K] | packed int4 [N,K/2]
  int fmt = 0;               // 0 fp16, 1 W8A16, 2 W4A16 (group 128)
  const half* scale = nullptr;  // W8: [N]; W4: [N,K/128]
  const half* zero = nullptr;   // W4: [N,K/128]
  int in_act = kActNone;
  int epi = kEpiNone;
  EpiArgs ea;
  void* y = nullptr;         // half [M,N], or float [M,N] for kEpiF32
  // optional scratch for the tensor-core path's split-K (rows > 4): fp32 partial sums [splits, M, N];
  // calls sharing it must not overlap on the GPU
  float* scratch = nullptr;
  size_t scratch_bytes = 0;
  // optional per-output-channel factor for the accumulator (tensor-core path)
  const half* out_scale = nullptr;
  // tensor-core path: true when w may have been written by the kernel launched just before this call on the same
  // stream (then its tiles are not requested until that kernel has completed); a model's resident weights set false
  bool w_dynamic = true;
  // 2..4 rows normally take the GEMV kernels (whose time grows with the row count); set this to send a large fp16
  // product of 2..4 rows to the tensor-core kernel instead, which streams the weights once whatever the row count
  bool prefer_tc = false;
  // optional fused prologue of the decode GEMV (M <= 4, fp16 weights, K == channels): see GemvSeg in gemv.h
  const half* res = nullptr;
  const half* ln_w = nullptr;
  const half* ln_b = nullptr;
  const half* shift = nullptr;
  const half* mix = nullptr;
  half* x_out = nullptr;
  half* n_out = nullptr;
  float eps = 1e-5f;
  const half* copy_src = nullptr;
  half* copy_dst = nullptr;
  int copy_n = 0;
};
int linear(cudaStream_t stream, const LinearArgs& args);
// Up to 8 independent problems sharing M <= 4 in a single launch.
int linear_batch(cudaStream_t stream, const LinearArgs* args, int n);
// Whether linear_batch can run M rows of K inputs with the fused prologue (bulk-copy kernel: activations in shared memory).
bool gemv_mma_fits(int M, int K);  // gemv_mma.cu: M rows of K activations leave room for a ring of weight boxes
bool linear_batch_fused_fits(int M, int K);
// Up to eight products with the same M > 4: one tensor-core launch when every product has fp16 weights and no
// input activation (split-K scratch is taken from args[0]); otherwise one linear() call per product.
int linear_group(cudaStream_t stream, const LinearArgs* args, int n);

// ---- tmix_decode.cu : fused one-token time-mix core (LoRA up + gates + WKV + GroupNorm/gate)
struct TmixDecodeArgs {
  int B = 0, C = 0;
  bool layer0 = false, wkv32 = false;
  // the many-row numerics of the reference (more than four rows): tanh / sigmoid of the LoRA inputs and the v LoRA
  // output are rounded to half, and the value-residual gate uses the stand-alone gate kernel's formula
  bool round_act = false;
  int R[4] = {0, 0, 0, 0};                                   // ranks of w, a, g, v
  const half* l1[4] = {nullptr, nullptr, nullptr, nullptr};  // [B,R] LoRA down outputs
  const half* up[4] = {nullptr, nullptr, nullptr, nullptr};  // [C,R] LoRA up matrices
  const half *r = nullptr, *k = nullptr, *v = nullptr, *v_first = nullptr;
  const half *w0 = nullptr, *a0 = nullptr, *v0 = nullptr, *k_k = nullptr, *k_a = nullptr, *r_k = nullptr;
  const half *lnx_w = nullptr, *lnx_b = nullptr;
  void* state = nullptr;  // this layer's [B,H,64,64] half or float
  const int* elapsed = nullptr;
  half* y2 = nullptr;
  const half* shift_src = nullptr;  // optional: [B,C] rows copied into shift_dst (the layer's time-mix shift state)
  half* shift_dst = nullptr;
};
bool tmix_decode_supported(const TmixDecodeArgs& args);
int tmix_decode(cudaStream_t stream, const TmixDecodeArgs& args);

// ---- quant.cu
int quant_pack_w8(cudaStream_t stream, int N, int K, const half* W, int8_t* q, half* scale);
int quant_unpack_w8(cudaStream_t stream, int N, int K, const int8_t* q, const half* scale, half* W);
int quant_pack_w4(cudaStream_t stream, int N, int K, const half* W, uint8_t* q, half* scale, half* zero);
int quant_unpack_w4(cudaStream_t stream, int N, int K, const uint8_t* q, const half* scale, const half* zero, half* W);

}  // namespace rk
