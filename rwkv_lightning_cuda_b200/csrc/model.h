// Host-side engine of the sm_100a RWKV-7 forward: weight storage, activation workspaces,
// the per-layer launch sequence and the CUDA-graph cache for decode steps.
#pragma once

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "../../include/rwkv7_b200.h"
#include "kernels.h"
#include "tp_comm.h"

namespace rk {

struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  DevBuf() = default;
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
  DevBuf(DevBuf&& o) noexcept : p(o.p), bytes(o.bytes) { o.p = nullptr; o.bytes = 0; }
  DevBuf& operator=(DevBuf&& o) noexcept {
    if (this != &o) { release(); p = o.p; bytes = o.bytes; o.p = nullptr; o.bytes = 0; }
    return *this;
  }
  ~DevBuf() { release(); }
  int alloc(size_t n);
  void release();
  template <typename T> T* as() const { return static_cast<T*>(p); }
};

// One large matrix in its device format.
struct Matrix {
  int N = 0, K = 0, fmt = RWKV7_B200_FMT_F16;
  DevBuf w, scale, zero;  // packed weights and their quantisation parameters (the only copy, whatever the row count)
};

struct LayerWeights {
  DevBuf ln1_w, ln1_b, ln2_w, ln2_b;
  DevBuf mix[6];  // x_r, x_w, x_k, x_v, x_a, x_g
  Matrix Wr, Wk, Wv, Wo, Wkey, Wval;
  DevBuf w0, a0, v0;
  DevBuf w1t, a1t, g1t, v1t;  // LoRA down, transposed to [R,C]
  DevBuf w2t, a2t, g2t, v2t;  // LoRA up, transposed to [C,R]
  DevBuf k_k, k_a, r_k, lnx_w, lnx_b, ffn_x_k;
};

// Activation buffers of one forward of `rows` = B*T rows: pointers into the model's arena (see Model::prepare).
struct Workspace {
  int rows = 0, B = 0;
  half *xA, *xB, *xm[6], *r, *k, *v, *vfirst, *vout, *w12, *a12, *g, *k2, *nkk, *kka, *y, *y2, *att, *mixed, *ffn;
  half *hid, *l1[4], *xf, *n1, *n2;
  int64_t* tokens;
  float* gemm_scratch = nullptr;  // split-K partial sums of the tensor-core GEMM (rows >= 2)
  size_t gemm_scratch_bytes = 0;
  float* part32 = nullptr;        // tensor parallel: fp32 partial sums [rows, C] / gathered logits
};

class Model {
 public:
  explicit Model(const rwkv7_b200_config& cfg);
  ~Model();

  int set_tensor(const char* name, const void* data, int dtype, long long count, int on_device);
  int finalize();
  int forward(const int64_t* tokens_host, int B, int T, void* shift, void* wkv, int* elapsed, float* logits,
              cudaStream_t stream);
  // sampling == nullptr: greedy choice
  int decode_greedy(const int64_t* first_tokens_host, int B, int steps, void* shift, void* wkv, int* elapsed, float* logits,
                    float* penalties, float presence, float repetition, float decay, int* out_tokens, cudaStream_t stream,
                    const rwkv7_b200_sampling* sampling = nullptr);
  int state_sizes(int B, size_t* shift_elems, size_t* wkv_elems, size_t* elapsed_elems) const;
  int state_init(int B, void* shift, void* wkv, int* elapsed, cudaStream_t stream) const;
  int copy_state_slice(const void* src_shift, const void* src_wkv, const int* src_elapsed, int src_B, int src_off,
                       void* dst_shift, void* dst_wkv, int* dst_elapsed, int dst_B, int dst_off, int count,
                       cudaStream_t stream) const;
  // One sequence's state <-> three contiguous host blobs (the reference's session record: shift, wkv, elapsed)
  int state_export(const void* shift, const void* wkv, const int* elapsed, int B, int index, void* shift_blob, void* wkv_blob,
                   int* elapsed_blob, cudaStream_t stream) const;
  int state_import(const void* shift_blob, const void* wkv_blob, const int* elapsed_blob, void* shift, void* wkv, int* elapsed, int B,
                   int index, cudaStream_t stream) const;
  int query_capacity(int chunk, rwkv7_b200_capacity* out) const;
  int tp_init(const void* unique_id);  // joins the tensor-parallel group (collective over all ranks)
  // Reads (and resets) the device's failure word through this model's pinned slot; `stream` must have been
  // given the copy by enqueue_timeout_read and be synchronised by the caller in between.
  int enqueue_timeout_read(cudaStream_t stream);
  int timeout_result();
  size_t workspace_bytes() const { return arena_.bytes + gemm_scratch_.bytes + part32_.bytes; }

  const rwkv7_b200_config& cfg() const { return cfg_; }
  long long launches() const { return launches_; }

 private:
  struct GraphKey {
    int B, T;
    const void *shift, *wkv, *elapsed, *logits;
    bool operator<(const GraphKey& o) const {
      return std::tie(B, T, shift, wkv, elapsed, logits) < std::tie(o.B, o.T, o.shift, o.wkv, o.elapsed, o.logits);
    }
  };
  struct GraphEntry {
    cudaGraphExec_t exec = nullptr;  // null until the call has been seen twice (the first one is enqueued directly)
    long long launches = 0;
    unsigned long long last_use = 0;
    bool failed = false;             // capture did not work for this call: always enqueue directly
  };

  int use_device() const;
  int upload(DevBuf& dst, const void* data, int dtype, long long count, int on_device, long long expect);
  int upload_matrix(Matrix& m, int N, int K, const void* data, int dtype, long long count, int on_device);
  int upload_slice(DevBuf& dst, const void* data, int dtype, long long count, int on_device, int rows, int cols, int r0, int nr,
                   int c0, int nc);
  int transpose_into(DevBuf& dst, const DevBuf& src, int rows, int cols);
  int quantize(Matrix& m);
  int prepare(int B, int T, cudaStream_t stream);
  void drop_graphs();
  int step(const int64_t* tokens_host, int B, int T, void* shift, void* wkv, int* elapsed, float* logits, cudaStream_t stream);
  int run(Workspace& ws, int B, int T, void* shift, void* wkv, int* elapsed, float* logits, cudaStream_t stream);
  int enqueue(Workspace& ws, int B, int T, half* shift, void* wkv, int* elapsed, float* logits, cudaStream_t s);
  int enqueue_decode(Workspace& ws, int B, half* shift, void* wkv, int* elapsed, float* logits, cudaStream_t s);
  int lin(cudaStream_t s, int M, const Matrix& W, const half* x, void* y, int epi);
  int lin16(cudaStream_t s, int M, int K, int N, const half* x, const half* w, half* y, int in_act, int epi,
            const EpiArgs& ea);

  rwkv7_b200_config cfg_;
  int H_ = 0;
  int tp_size_ = 1, tp_rank_ = 0;
  TpComm tp_;
  bool finalized_ = false;
  std::vector<LayerWeights> layers_;
  DevBuf emb_ln0_, ln_out_w_, ln_out_b_;
  Matrix head_;
  // staging until finalize
  DevBuf emb_raw_, ln0_w_raw_, ln0_b_raw_;
  int emb_dtype_ = -1;
  std::unordered_map<std::string, DevBuf> lora_raw_;  // checkpoint-orientation LoRA matrices

  // One set of activation buffers per model, grown to the largest call seen and never per shape: a server that
  // walks through many (batch, chunk) shapes holds the memory of the largest one only.  Calls are serialised on
  // the device as well as on the host: mu_ guards the enqueue, and a call on another stream than the previous one
  // first waits for that one's work (last_done_), because both would use these buffers.
  std::mutex mu_;
  DevBuf arena_, gemm_scratch_, part32_, probs_;  // probs_: the sampler's scratch, [B, vocab] fp32
  Workspace ws_;
  // ring of pinned host staging slots for the token ids; a slot is reused only after the copy that read it has
  // completed, so callers may overwrite their token array as soon as forward returns
  static constexpr int kSlots = 4;
  int64_t* tokens_pinned_[kSlots] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t tokens_copied_[kSlots] = {nullptr, nullptr, nullptr, nullptr};
  size_t pinned_rows_ = 0;
  int slot_ = 0;
  cudaEvent_t last_done_ = nullptr;
  cudaStream_t last_stream_ = nullptr;
  bool have_last_ = false;
  int* timeout_dev_ = nullptr;   // the device's failure word
  int* timeout_host_ = nullptr;  // pinned slot it is copied to
  std::map<GraphKey, GraphEntry> graphs_;
  unsigned long long tick_ = 0;
  long long launches_ = 0;
  Workspace* cur_ = nullptr;  // workspace of the forward being enqueued (guarded by mu_)
};

}  // namespace rk
