/*
 * rwkv7_b200 -- C ABI of the sm_100a RWKV-7 forward library (librwkv7_b200.so).
 *
 * This is the boundary a host program binds instead of the reference's C++ backend class
 * `rwkv7_server::ModelBackend` (include/rwkv_server_backend.hpp:104-147 of the reference) and,
 * for the op-level entry points, instead of the launchers declared in the reference's
 * cuda/rwkv7_fast_v4_kernels.cuh.  Every citation below is a path inside the reference project.
 *
 * Conventions
 *   - every function returns an int status (RWKV7_B200_OK == 0); on failure
 *     rwkv7_b200_last_error() returns a thread-local message.  Nothing exits or aborts.
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream.
 *   - pointers are device pointers unless the name ends in _host.
 *   - half tensors are IEEE binary16 passed as uint16_t bit patterns.
 *   - activations are row-major [B*T, C] (b major, then t); C = 64 * H.
 *   - functions only enqueue work; they synchronise only where stated.
 */
#ifndef RWKV7_B200_H
#define RWKV7_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RWKV7_B200_OK 0
#define RWKV7_B200_BAD_ARG 1
#define RWKV7_B200_SHAPE 2
#define RWKV7_B200_PRECISION 3   /* state precision does not match the model (fp16 vs fp32 WKV state) */
#define RWKV7_B200_CUDA 4
#define RWKV7_B200_NCCL 5
#define RWKV7_B200_TIMEOUT 6     /* a bounded wait inside a kernel ran out: see rwkv7_b200_timeout_flags */
#define RWKV7_B200_NOT_READY 7   /* model not finalised / tensor missing */

/* weight formats of the large matrices (att r/k/v/o, ffn key/value, head) */
#define RWKV7_B200_FMT_F16 0
#define RWKV7_B200_FMT_W8A16 1   /* int8, per output channel, symmetric, fp16 scale */
#define RWKV7_B200_FMT_W4A16 2   /* int4, group 128 along K, asymmetric, fp16 scale and zero */

/* element types accepted by rwkv7_b200_model_set_tensor */
#define RWKV7_B200_DT_F16 0
#define RWKV7_B200_DT_BF16 1

/* input activations / epilogues of rwkv7_b200_linear_* */
#define RWKV7_B200_ACT_NONE 0
#define RWKV7_B200_ACT_TANH 1
#define RWKV7_B200_ACT_SIGMOID 2
#define RWKV7_B200_EPI_NONE 0
#define RWKV7_B200_EPI_RELU2 1
#define RWKV7_B200_EPI_F32 3

const char* rwkv7_b200_last_error(void);
/* Compiled-in facts a binding can check at load time: head size (64) and ABI version. */
int rwkv7_b200_abi_version(void);

/* ------------------------------------------------------------------------------------------
 * Model-level entry points (replace rwkv7_server::ModelBackend)
 * ---------------------------------------------------------------------------------------- */

typedef struct rwkv7_b200_model rwkv7_b200_model;

typedef struct {
  int layers, channels, ffn, vocab;      /* heads = channels / 64 */
  int rank_w, rank_a, rank_v, rank_g;    /* LoRA ranks, multiples of 8, <= 512 */
  int weight_format;                     /* RWKV7_B200_FMT_* ; large matrices are quantised at finalize */
  int wkv32;                             /* 1: fp32 WKV state (the reference's --wkv32), 0: fp16 */
  int device;                            /* CUDA device ordinal; -1 = current device */
  int tp_rank, tp_size;                  /* head-sharded tensor parallelism; 0/1 = off */
} rwkv7_b200_config;

typedef struct {
  size_t free_vram_bytes, total_vram_bytes, reserve_vram_bytes, bytes_per_batch;
  int max_batch_size;
} rwkv7_b200_capacity;

/* Replaces ModelBackend::ModelBackend (src/rwkv7_fast_v4.cu:1364-1365): creates an empty model. */
int rwkv7_b200_model_create(const rwkv7_b200_config* cfg, rwkv7_b200_model** out);

/* Replaces the per-tensor upload of load_model_weights (src/rwkv7_fast_v4.cu:630-701).
 * `name` is the checkpoint tensor name (emb.weight, blocks.N.att.key.weight, ln_out.weight,
 * head.weight, ...; full list in src/rwkv7_fast_v4.cu:574-596).  `data` holds `count` elements of
 * `dtype`, on the host (on_device = 0) or on this model's device (1); it is copied and may be
 * freed on return.  bf16 is converted as half_rn(float(bf16)) like cuda/rwkv7_v3a_ops.cu:79-88.
 * The pseudo-tensor "emb_ln0" ([vocab, channels] fp16) may be given instead of emb.weight +
 * blocks.0.ln0.{weight,bias}. */
int rwkv7_b200_model_set_tensor(rwkv7_b200_model* m, const char* name, const void* data, int dtype,
                                long long count, int on_device);

/* Builds device layouts (LoRA transposes, emb+LN0 table as cuda/rwkv7_v3a_ops.cu:153-187,
 * quantisation) and frees staging copies.  Synchronises the device. */
int rwkv7_b200_model_finalize(rwkv7_b200_model* m);

/* Head-sharded tensor parallelism (no counterpart in the reference, which drives one GPU:
 * src/rwkv7_fast_v4.cu never selects a device).  One process or thread per GPU creates a model with
 * tp_size = G and its own tp_rank, feeds every rank the FULL tensors through set_tensor (each rank keeps
 * heads [rank*H/G, (rank+1)*H/G): rows of att.receptance/key/value, input columns of att.output, the
 * per-channel att vectors and LoRA up-projections of those heads, ffn.key rows / ffn.value columns
 * [rank*F/G, ...), head rows [rank*V/G, ...); LayerNorms, token-shift vectors, LoRA down-projections and
 * the embedding table are replicated).  Every rank then runs the same forward calls with the same tokens;
 * partial sums of att.output and ffn.value are added across ranks in fp32 (NCCL all-reduce, bound at run
 * time from libnccl.so.2) and rounded to half once; the logits are all-gathered, so every rank returns
 * the full [B, vocab].  The wkv state holds the rank's heads only (state_sizes reports the local size);
 * shift and elapsed are replicated.  fp16 weights only.
 *   rwkv7_b200_tp_unique_id: rank 0 fills 128 bytes and sends them to the other ranks (any host channel).
 *   rwkv7_b200_model_tp_init: collective over all ranks, before the first forward. */
int rwkv7_b200_tp_unique_id(void* out128);
int rwkv7_b200_model_tp_init(rwkv7_b200_model* m, const void* unique_id128);

int rwkv7_b200_model_destroy(rwkv7_b200_model* m);
int rwkv7_b200_vocab_size(const rwkv7_b200_model* m);   /* ModelBackend::vocab_size, src/rwkv7_fast_v4.cu:1582 */

/* Element counts of the three state buffers of a batch of B sequences, laid out exactly like
 * GenerationState (include/rwkv_server_backend.hpp:45-58, src/rwkv7_fast_v4.cu:1177-1185,1381-1390):
 *   shift   half  [layers][2][B][channels]
 *   wkv     half or float [layers][B][heads][64][64]   (element size 2, or 4 when wkv32)
 *   elapsed int32 [B] */
int rwkv7_b200_state_sizes(const rwkv7_b200_model* m, int B, size_t* shift_elems, size_t* wkv_elems,
                           size_t* elapsed_elems);
/* Zero-initialises caller-allocated state buffers (ModelBackend::create_state, :1373-1400). */
int rwkv7_b200_state_init(const rwkv7_b200_model* m, int B, void* shift, void* wkv, int* elapsed, void* stream);

/* Replaces run_backend_forward / forward_prefill / forward_decode (src/rwkv7_fast_v4.cu:1046-1345,
 * 1402-1419).  tokens_host is [B][T] row-major on the host (decode: T = 1); the state is updated
 * in place; logits receives fp32 [B][vocab] of the last token of every sequence.  Token ids are
 * validated on the host before anything is enqueued (BAD_ARG, state untouched).  Asynchronous:
 * the logits are valid once `stream` has completed; tokens_host may be reused on return.
 * Threading: calls may come from any thread.  A model owns ONE set of activation buffers (grown to the
 * largest B*T seen, never per shape), so calls on the same model are serialised on the host (a mutex around the
 * enqueue) and on the device (a call on another stream than the previous call's first waits for that call's
 * work).  Concurrent sequences belong in one batch, or in separate models.  A call that has to grow the
 * buffers synchronises the device first. */
int rwkv7_b200_forward(rwkv7_b200_model* m, const int64_t* tokens_host, int B, int T, void* shift, void* wkv,
                       int* elapsed, float* logits, void* stream);

/* Same call for a host program that keeps no device buffers for the result: additionally copies
 * the logits to logits_host (pinned memory recommended) and synchronises `stream`.  Because it synchronises,
 * it also reads the device's failure word: RWKV7_B200_TIMEOUT means a kernel gave up on a bounded wait and
 * the logits and the state of this call are not to be trusted (the word is reset, later calls run normally). */
int rwkv7_b200_forward_to_host(rwkv7_b200_model* m, const int64_t* tokens_host, int B, int T, void* shift,
                               void* wkv, int* elapsed, float* logits, float* logits_host, void* stream);

/* The step after the path, kept on the device: `steps` decode steps in a row, each followed by a greedy choice of
 * every sequence's next token, with no host round trip between them.  Replaces, for top_p == 0 (the sampler's greedy
 * case, src/utils/sampling.cu:507-512), the engine's loop forward_decode -> sampler -> copy to the host -> next
 * forward_decode (src/rwkv_sampler.cpp:47-111; kernel src/utils/sampling.cu:205-471).
 * first_tokens_host [B] feeds step 0.  penalties is NULL or a device array fp32 [B][vocab] that is subtracted from
 * the logits and updated after every choice as the reference's sampler does (:253, :460-469:
 * p = p * penalty_decay + (chosen ? (p == 0 ? presence_penalty : repetition_penalty) : 0)); +inf masks a token.
 * Among equal values the lowest token id wins (the reference draws among them at random).
 * out_tokens is a device array int32 [steps][B]; logits (fp32 [B][vocab], device) holds the last step's logits
 * afterwards.  out_tokens_host NULL: asynchronous like rwkv7_b200_forward; otherwise the tokens are also copied
 * there and `stream` is synchronised.  Not available for tensor-parallel models (BAD_ARG). */
int rwkv7_b200_decode_greedy(rwkv7_b200_model* m, const int64_t* first_tokens_host, int B, int steps, void* shift,
                             void* wkv, int* elapsed, float* logits, float* penalties, float presence_penalty,
                             float repetition_penalty, float penalty_decay, int* out_tokens, int* out_tokens_host,
                             void* stream);
/* The same loop with the sampler's general case -- temperature, top-k, top-p -- instead of the greedy choice
 * (src/utils/sampling.cu:205-471 with the argument rules of :492-512: top_k <= 0 or > vocab means no limit, top_p outside
 * [0, 1] means 1, top_p == 0 means greedy, temperature must lie in [0.001, 1000]).  Random numbers are Philox-4x32-10
 * words keyed by `seed` with the counter (offset + step, sequence): a run is reproducible from (seed, offset), where the
 * reference's cuRAND states are seeded from the clock (src/rwkv_sampler.cpp:14-19,39-42).  Step i uses offset + i; pass
 * offset + steps to the next call to continue the stream. */
typedef struct {
  float temperature;
  int top_k;
  float top_p;
  unsigned long long seed, offset;
} rwkv7_b200_sampling;
int rwkv7_b200_decode_sample(rwkv7_b200_model* m, const int64_t* first_tokens_host, int B, int steps, void* shift,
                             void* wkv, int* elapsed, float* logits, float* penalties, float presence_penalty,
                             float repetition_penalty, float penalty_decay, const rwkv7_b200_sampling* sampling,
                             int* out_tokens, int* out_tokens_host, void* stream);
/* One draw per row for a caller that runs its own loop (batch_sampling_repetition_temperature_topk_topp_raw,
 * src/utils/sampling.cu:474-541; penalties NULL: batch_sampling_temperature_topk_topp_raw).  probs is scratch, fp32
 * [B][V] on the device; out[b] and next_tokens[b] (int64, may be NULL) receive the token. */
int rwkv7_b200_sample(void* stream, int B, int V, const float* logits, float* penalties, float* probs,
                      float presence_penalty, float repetition_penalty, float penalty_decay,
                      const rwkv7_b200_sampling* sampling, int* out, int64_t* next_tokens);
/* The choice alone, for a caller that runs its own loop: out[b] = argmax_i (logits[b][i] - penalties[b][i]) with the
 * penalty update above; next_tokens (int64 [B], may be NULL) receives the same ids. */
int rwkv7_b200_greedy_pick(void* stream, int B, int V, const float* logits, float* penalties, float presence_penalty,
                           float repetition_penalty, float penalty_decay, int* out, int64_t* next_tokens);

/* Replaces ModelBackend::copy_state_slice (src/rwkv7_fast_v4.cu:1421-1504): copies `count`
 * sequences from a state of batch size src_B (starting at src_offset) into a state of batch size
 * dst_B (starting at dst_offset).  Enqueued on `stream`. */
int rwkv7_b200_copy_state_slice(const rwkv7_b200_model* m, const void* src_shift, const void* src_wkv,
                                const int* src_elapsed, int src_B, int src_offset, void* dst_shift,
                                void* dst_wkv, int* dst_elapsed, int dst_B, int dst_offset, int count,
                                void* stream);

/* Session records: one sequence's state as the three blobs the reference's state cache stores per session
 * (src/rwkv_state_cache.cpp:268-292: shift_blob = half [layers][2][channels], wkv_blob = half or float
 * [layers][heads][64][64], elapsed_blob = int32 [1]; same bytes, so records are interchangeable).  The reference
 * fills a batch-1 GenerationState with copy_state_slice and then copies buffer by buffer with blocking cudaMemcpy
 * (:132-223); these two calls gather / scatter sequence `index` of a batch state directly, as three asynchronous
 * strided copies on `stream` (pinned host memory makes them overlap with compute).  The blobs are valid / may be
 * reused once `stream` has completed. */
int rwkv7_b200_state_blob_sizes(const rwkv7_b200_model* m, size_t* shift_bytes, size_t* wkv_bytes,
                                size_t* elapsed_bytes);
int rwkv7_b200_state_export(const rwkv7_b200_model* m, const void* shift, const void* wkv, const int* elapsed, int B,
                            int index, void* shift_blob_host, void* wkv_blob_host, int* elapsed_blob_host, void* stream);
int rwkv7_b200_state_import(const rwkv7_b200_model* m, const void* shift_blob_host, const void* wkv_blob_host,
                            const int* elapsed_blob_host, void* shift, void* wkv, int* elapsed, int B, int index,
                            void* stream);
/* A WKV state (or blob on the device) from one precision to the other, for a session saved under one setting of the
 * reference's --wkv32 switch and resumed under the other (the reference refuses such a session,
 * src/rwkv_state_cache.cpp:180-187): half -> float is exact, float -> half rounds to nearest.  elems % 8 == 0. */
int rwkv7_b200_state_convert_wkv(void* stream, const void* src, void* dst, long long elems, int src_is_fp32);

/* Replaces ModelBackend::query_prefill_capacity (src/rwkv7_fast_v4.cu:1534-1580). */
int rwkv7_b200_query_capacity(const rwkv7_b200_model* m, int prefill_chunk_size, rwkv7_b200_capacity* out);

/* Number of kernels enqueued by forward calls since the model was created (for benchmarks). */
long long rwkv7_b200_kernel_launches(const rwkv7_b200_model* m);
/* Device bytes the model's activation workspace holds now (it replaces the reference's per-call arena +
 * 128 MiB workspace, src/rwkv7_fast_v4.cu:1087-1096; grow-only, sized by the largest call so far). */
int rwkv7_b200_model_workspace_bytes(const rwkv7_b200_model* m, size_t* out);

/* ------------------------------------------------------------------------------------------
 * Failure word and options (no counterpart in the reference, whose kernels have no bounded waits and
 * whose CUDA errors end the process, include/rwkv7_fast_v4_common.hpp:57-62)
 * ---------------------------------------------------------------------------------------- */

/* Every wait on a copy-completion barrier inside this library's kernels has a poll limit.  A kernel whose
 * limit runs out sets a bit in a per-device word and returns instead of hanging.  The calls that synchronise
 * (rwkv7_b200_forward_to_host, rwkv7_b200_decode_greedy with out_tokens_host) report it as
 * RWKV7_B200_TIMEOUT; callers of the asynchronous entry points read it here after synchronising their
 * stream.  *flags: 1 weight-streaming GEMV, 2 tensor-core GEMM, 4 time-mix core, 8 wait probe, 16 all-reduce through peer memory (a rank of the tensor-parallel group did not show up).
 * clear != 0 resets the word.  Blocking (a 4-byte device-to-host copy on the current device). */
int rwkv7_b200_timeout_flags(int clear, int* flags);
/* Diagnostic (no counterpart in the reference): the record the tensor-core GEMM leaves when one of its bounded waits
 * runs out for the first time since the record was cleared: {1, role (1 producer, 20/21/22 MMA thread waiting for an
 * accumulator / a stage / a dequantised tile, 3 dequantisation, 4 epilogue), CTA, work unit, K-block counter, stages,
 * units, product, M, N, K, format, row tile, K splits, 0}; all zero when nothing expired. */
int rwkv7_b200_debug_timeout_detail(int* out15, int clear);
/* Test aid: enqueues a one-thread kernel that polls a barrier nothing will ever complete `polls` times
 * (<= 2^20), then sets bit 8 of the failure word and returns.  No copy is in flight, nothing hangs. */
int rwkv7_b200_debug_wait_probe(void* stream, unsigned polls);
/* Test aid: the largest K split among the products of the calling thread's most recent tensor-core GEMM launch
 * (1: no fp32 partial sums were written; > 1: the split-K scratch was used).  Returns the count, not a status. */
int rwkv7_b200_debug_last_gemm_splits(void);
/* Process-wide switches for measurements and tests, read when a call is enqueued:
 *   "gemm_cta_pair" 0|1     tensor-core GEMM as CTA pairs (cta_group::2); default 0 (measured equal)
 *   "quant_tc_rows" n       row count from which quantised weights take the tensor-core path; 0 = built-in
 *   "fp16_tc_rows" n        the same for fp16 weights; 0 = built-in
 *   "decode_graphs" 0|1     decode steps replay a CUDA graph; default 1
 *   "wkv_chunked" 0|1       fp32-state WKV over 64 tokens or more runs in matrix form on the tensor cores; default 1
 *   "gemv_mma_tall" 0..3    the mma.sync linear kernel walks the weights in tiles of 32 instead of 16 channels: 0 never, 1 one
 *                           row of quantised weights, 2 one row of any format and up to three rows of fp16 (default), 3 wherever
 *                           shared memory allows
 *   "tp_peer_ranks" n       tensor-parallel groups of up to n ranks all-reduce in the library's own kernel over peer-mapped
 *                           memory, larger ones through NCCL; default 2 (set before the first forward call)
 *   "gemv_mma" 0..4         linear layers of 1..4 rows: 0 scalar weight-streaming kernels only, 1 the mma.sync kernel (weight
 *                           tiles by 2-D tensor copies, dequantised once for all rows) for W4A16 and for 2..4 rows of W8A16,
 *                           2 also for 2..4 rows of fp16, 3 also for one row of fp16 / W8A16 in large launches (8 MB and more, rows of 2 / 4 KiB and more)
 *                           (default), 4 for every launch the kernel accepts
 * BAD_ARG for an unknown name or a value out of range. */
int rwkv7_b200_set_option(const char* name, int value);

/* ------------------------------------------------------------------------------------------
 * Op-level entry points (replace launchers of cuda/rwkv7_fast_v4_kernels.cuh)
 * ---------------------------------------------------------------------------------------- */

/* rwkv7_wkv_fp16_seq_launch (cuda/rwkv7_wkv_fp16_v2.cu:676-742): w holds the decay pre-activation. */
int rwkv7_b200_wkv_fp16_seq(void* stream, int B, int T, int C, int H, uint16_t* state, const uint16_t* r,
                            const uint16_t* w, const uint16_t* k, const uint16_t* v, const uint16_t* a,
                            const uint16_t* b, uint16_t* y, const int* elapsed);
/* rwkv7_wkv_fp16_seq_w0_launch (cuda/rwkv7_wkv_fp16_v2.cu:744-830): w0 [C] added in fp32 inside. */
int rwkv7_b200_wkv_fp16_seq_w0(void* stream, int B, int T, int C, int H, uint16_t* state, const uint16_t* r,
                               const uint16_t* w, const uint16_t* w0, const uint16_t* k, const uint16_t* v,
                               const uint16_t* a, const uint16_t* b, uint16_t* y, const int* elapsed);
/* rwkv7_wkv_fp32io16_launch (cuda/rwkv7_wkv_fp32_v2.cu:237-294), mode 0. */
int rwkv7_b200_wkv_fp32io16(void* stream, int B, int T, int C, int H, float* state, const uint16_t* r,
                            const uint16_t* w, const uint16_t* k, const uint16_t* v, const uint16_t* a,
                            const uint16_t* b, uint16_t* y);

/* rwkv7_tmix_mix6_launch (cuda/rwkv7_fast_ops_fp16.cu:831-860); mix/out are arrays of 6 device pointers
 * in the order r, w, k, v, a, g; shift [B,C] is consumed and replaced by the last row. */
int rwkv7_b200_tmix_mix6(void* stream, int B, int T, int C, const uint16_t* x, uint16_t* shift,
                         const uint16_t* const* mix, uint16_t* const* out);
/* rwkv7_cmix_mix_launch (cuda/rwkv7_fast_ops_fp16.cu:924-940) */
int rwkv7_b200_cmix_mix(void* stream, int B, int T, int C, const uint16_t* x, uint16_t* shift,
                        const uint16_t* x_k, uint16_t* out);
/* rwkv7_tmix_kk_a_gate_launch (cuda/rwkv7_fast_ops_fp16.cu:862-884) */
int rwkv7_b200_tmix_kk_a_gate(void* stream, int B, int T, int C, int H, const uint16_t* k, const uint16_t* k_k,
                              const uint16_t* a0, const uint16_t* a12, const uint16_t* k_a, uint16_t* new_k,
                              uint16_t* neg_kk, uint16_t* kka);
/* rwkv7_tmix_lnx_rkvres_xg_launch (cuda/rwkv7_fast_ops_fp16.cu:886-906) */
int rwkv7_b200_tmix_lnx_rkvres_xg(void* stream, int B, int T, int C, int H, const uint16_t* x, const uint16_t* r,
                                  const uint16_t* k, const uint16_t* v, const uint16_t* r_k, const uint16_t* weight,
                                  const uint16_t* bias, const uint16_t* g, uint16_t* out);
/* rwkv7_tmix_vres_gate_launch (cuda/rwkv7_fast_ops_fp16.cu:908-922) */
int rwkv7_b200_tmix_vres_gate(void* stream, int B, int T, int C, const uint16_t* v, const uint16_t* v_first,
                              const uint16_t* v0, const uint16_t* v12, uint16_t* out);
/* rwkv7_v3a_layer_norm_f16_launch (cuda/rwkv7_v3a_ops.cu:2123-2140) */
int rwkv7_b200_layer_norm_f16(void* stream, int rows, int C, const uint16_t* x, const uint16_t* weight,
                              const uint16_t* bias, uint16_t* y, float eps);
/* rwkv7_v3a_add_layer_norm_f16_launch (cuda/rwkv7_v3a_ops.cu:2142-2160) */
int rwkv7_b200_add_layer_norm_f16(void* stream, int rows, int C, const uint16_t* x, const uint16_t* residual,
                                  const uint16_t* weight, const uint16_t* bias, uint16_t* x_out, uint16_t* y,
                                  float eps);
/* rwkv7_v3a_add_last_layer_norm_f16_launch (cuda/rwkv7_v3a_ops.cu:2162-2182) */
int rwkv7_b200_add_last_layer_norm_f16(void* stream, int B, int T, int C, const uint16_t* x,
                                       const uint16_t* residual, const uint16_t* weight, const uint16_t* bias,
                                       uint16_t* y, float eps);
/* rwkv7_v3a_add_layer_norm_cmix_mix_f16_launch (cuda/rwkv7_v3a_ops.cu:2184-2196), for any T */
int rwkv7_b200_add_layer_norm_cmix_mix_f16(void* stream, int B, int T, int C, const uint16_t* x,
                                           const uint16_t* residual, uint16_t* shift, const uint16_t* weight,
                                           const uint16_t* bias, const uint16_t* x_k, uint16_t* x_out,
                                           uint16_t* mixed, float eps);
/* rwkv7_v3a_add_layer_norm_tmix_mix6_f16_launch (cuda/rwkv7_v3a_ops.cu:2198-2215), for any B and T */
int rwkv7_b200_add_layer_norm_tmix_mix6_f16(void* stream, int B, int T, int C, const uint16_t* x,
                                            const uint16_t* residual, uint16_t* shift, const uint16_t* weight,
                                            const uint16_t* bias, const uint16_t* const* mix, uint16_t* x_out,
                                            uint16_t* const* out, float eps);
/* rwkv7_v4_emb_ln0_bf16_to_f16_launch (cuda/rwkv7_v3a_ops.cu:2101-2115); dtype RWKV7_B200_DT_* */
int rwkv7_b200_emb_ln0(void* stream, int V, int C, const void* emb, const void* weight, const void* bias,
                       int dtype, uint16_t* out, float eps);
/* rwkv7_relu_square_launch (cuda/rwkv7_fast_ops_fp16.cu:942-950) */
int rwkv7_b200_relu_square(void* stream, const uint16_t* x, uint16_t* out, long long elems);
/* rwkv7_v3a_advance_i32_launch (cuda/rwkv7_v3a_ops.cu:2117-2121) */
int rwkv7_b200_advance_i32(void* stream, int* x, int amount, long long elems);

/* rwkv7_v3a_linear_f16_orig_launch / linear_orig_rows_* / linear_t_act_* (cuda/rwkv7_v3a_ops.cu:2270-2302,
 * 2370-2507): y[M,N] = epi(act(x[M,K]) W^T), W [N,K] row-major fp16.  With RWKV7_B200_EPI_F32 y is
 * float [M,N] holding float(half(acc)) like the lm-head + rwkv7_v4_f16_to_f32_launch pair
 * (src/rwkv7_fast_v4.cu:1321-1342). */
int rwkv7_b200_linear_f16_orig(void* stream, int M, int K, int N, const uint16_t* x, const uint16_t* weight,
                               int in_act, int epilogue, void* y);
/* No counterpart in the reference.  The same layer as rwkv7_b200_linear_f16_orig for M > 4 rows, for host
 * programs that cannot allocate device memory around the call -- for instance a serving loop that runs under a
 * fixed memory budget and has closed its allocator once the model is resident, or a plugin host that forbids
 * cudaMalloc inside its callbacks.  The tensor-core kernel splits K over several CTAs and needs room for fp32 partial sums; this variant
 * keeps that room in a fixed 16 MiB device array inside the library image (held by every GPU that loads the
 * library until the process exits) and calls no cudaMalloc/cudaFree or allocating library routine.
 * Limits: M > 4, N % 4 == 0, M*N <= 2,097,152 (SHAPE otherwise).  The first call on a device looks the array's
 * device address up (cudaGetSymbolAddress) and makes the driver load the kernel and map the array; make one warm-up
 * call per device before the host closes its allocator or freezes its memory budget, and before any stream
 * capture.  All calls
 * share the array: nothing in it has to be cleared (every partial sum that is read is written by the same call), but
 * two calls whose kernels overlap on the GPU (different streams) race on it. */
int rwkv7_b200_linear_f16_orig_static(void* stream, int M, int K, int N, const uint16_t* x, const uint16_t* weight,
                                      int epilogue, void* y);
/* No counterpart in the reference (it has no quantised weights): the same layer on W8A16 / W4A16
 * weights in the formats written down in oracle/rwkv7_oracle.c and csrc/quant.cu. */
int rwkv7_b200_linear_w8a16(void* stream, int M, int K, int N, const uint16_t* x, const int8_t* q,
                            const uint16_t* scale, int epilogue, void* y);
int rwkv7_b200_linear_w4a16(void* stream, int M, int K, int N, const uint16_t* x, const uint8_t* q,
                            const uint16_t* scale, const uint16_t* zero, int epilogue, void* y);
int rwkv7_b200_quant_pack_w8(void* stream, int N, int K, const uint16_t* W, int8_t* q, uint16_t* scale);
int rwkv7_b200_quant_unpack_w8(void* stream, int N, int K, const int8_t* q, const uint16_t* scale, uint16_t* W);
int rwkv7_b200_quant_pack_w4(void* stream, int N, int K, const uint16_t* W, uint8_t* q, uint16_t* scale,
                             uint16_t* zero);
int rwkv7_b200_quant_unpack_w4(void* stream, int N, int K, const uint8_t* q, const uint16_t* scale,
                               const uint16_t* zero, uint16_t* W);

#ifdef __cplusplus
}
#endif
#endif /* RWKV7_B200_H */
