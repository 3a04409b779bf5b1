// One encoder replica on one GPU: weights, activation arena, stream, pinned staging and the
// per-call schedule.  It takes the place of the reference's `class bert`
// (utils/bert.cu:4-252), `global_handle` (utils/manager.cu:4-109) and the weight loader
// (utils/load_model.cc:15-98), with these differences by design:
//   * one stream, no per-layer host synchronisation (the reference synchronises once per layer
//     to rewind its bump arena, utils/bert.cu:232-234): buffers are fixed slots of one arena;
//   * persistent pinned staging instead of cudaMallocHost / cudaFreeHost per call
//     (utils/bert.cu:100,123); positions are t % S computed on the device;
//   * the arena is sized from max_batch * max_seq and grows on demand; it never takes "all free
//     memory" (utils/manager.cu:42-47);
//   * errors are recorded on the handle and reported, the process is never terminated
//     (the reference exits, utils/common.h:58-65).
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <tuple>
#include <vector>

#include "kernels.h"

namespace cb {

enum Precision : int { PREC_FP32 = 0, PREC_BF16 = 1, PREC_FP8 = 2 };
// how load_dense lays a weight out when an fp32 handle multiplies on the tensor cores: three bf16 planes
constexpr int PREC_FP32_SPLIT = 100;

enum KernelClass : int {
  KC_EMBED = 0, KC_GEMM_QKV, KC_ATTENTION, KC_GEMM_ATTN_OUT, KC_LAYERNORM, KC_GEMM_FFN1, KC_GEMM_FFN2,
  KC_POOLER, KC_OTHER, KC_COUNT
};

struct DenseWeight {      // one projection
  void* w = nullptr;      // fp32 [K, N] (fp32 mode); else fp16 [N, K] holding the bf16-rounded (x 4096) or e4m3 weights
  uint8_t* w_fp8 = nullptr;  // fp8 mode: e4m3 bytes [N, K], the weights the GEMM reads (null when they were widened at load)
  float* bias = nullptr;     // [N]
  float* colscale = nullptr; // fp8 mode: [N] de-quantisation scale per output column
  int K = 0, N = 0;
  CUtensorMap tmap;          // bf16 / fp8 modes
};

struct LayerWeights {
  DenseWeight qkv, attn_out, ffn1, ffn2;
  float *ln1_g = nullptr, *ln1_b = nullptr, *ln2_g = nullptr, *ln2_b = nullptr;
  // LayerNorms folded into the GEMMs around them (LnFold): gamma W and beta W + bias of the QKV GEMM (with the
  // previous layer's second LayerNorm) and of the FFN1 GEMM (with this layer's first)
  float *c_qkv = nullptr, *d_qkv = nullptr, *c_ffn1 = nullptr, *d_ffn1 = nullptr;
};

class Model {
 public:
  Model() = default;
  ~Model();
  // Returns false and fills error() on failure.  num_layers <= 0 means the model's own depth.
  bool init(bool large, int gpu, int max_batch, int max_seq, const std::string& dir, int precision, int num_layers);

  // Host arrays in (int32 [B, S]; mask may be null), pooler out (fp32 [B, H]) -- blocking.
  bool run_host(const int* ids, const int* seg, const int* mask, int B, int S, float* pooled_out,
                float* probs_out, int num_classes, bool want_hidden_f32 = false);
  // Same, but the results (pooler and fp32 final hidden states) stay on the device.
  bool run_host_keep(const int* ids, const int* seg, const int* mask, int B, int S) {
    return run_host(ids, seg, mask, B, S, nullptr, nullptr, 0, true);
  }
  void set_error(int code, const std::string& msg) { fail(code, msg); }
  // Device arrays in; asynchronous on stream(); results stay on the device.
  bool forward_device(const int* d_ids, const int* d_seg, const int* d_mask, int B, int S, bool want_hidden_f32,
                      bool want_probs);
  bool sync();
  // Enqueues the bounded-wait probe (kernels.h: wait_timeout_probe) on the handle's stream with this
  // handle's device error word, then synchronises: returns status() afterwards (4 after the time-out).
  int probe_wait_timeout(unsigned long long limit_ns);
  // CUDA graphs replayed / captured so far (a forward pass is captured the second time its exact
  // arguments are seen; CUDABERT_GRAPH=0 turns this off)
  long graph_replays() const { return graph_replays_; }
  long graph_captures() const { return graph_captures_; }

  float* pooled_dev() const { return pooled_; }
  // fp32 final hidden states [B, S, H] of the last call that asked for them (Cuda_Inference)
  float* hidden_f32_dev() const { return packed_ ? hidden_unpacked_ : xf_; }
  float* probs_dev() const { return probs_; }
  int hidden() const { return H_; }
  int layers() const { return L_; }
  int heads() const { return heads_; }
  int ffn() const { return F_; }
  int precision() const { return prec_; }
  int num_classes() const { return classes_; }
  cudaStream_t stream() const { return stream_; }
  int status() const { return status_; }
  const std::string& error() const { return error_; }
  void clear_error() { status_ = 0; error_.clear(); }

  long launches_last_forward() const { return launches_; }
  void set_profiling(bool on) { profiling_ = on; }
  void reset_profile();
  void get_profile(int kclass, double* ms, long* launches) const;

 private:
  bool fail(int code, const std::string& msg);
  bool check(cudaError_t e, const char* what);
  bool ensure_capacity(int B, int S, bool want_hidden_f32);
  bool load_weights(const std::string& dir);
  bool load_dense(const std::vector<std::string>& keys_kernel, const std::vector<std::string>& keys_bias,
                  int K, int N, DenseWeight* dst, int n_off, int n_total, int prec);
  bool finish_dense(DenseWeight* d, int prec);
  bool upload_vec(const std::vector<std::string>& keys, size_t n, float** dst);
  bool upload_table(const std::vector<std::string>& keys, size_t min_rows, float** dst, int* rows_out);
  const std::string* find_file(const std::vector<std::string>& keys) const;
  bool read_tensor(const std::vector<std::string>& keys, size_t expect, struct NpyArray* arr);
  void count(int kclass, int n);
  void prof_begin(int kclass);
  void prof_end(int kclass);
  bool collect_profile();
  bool dense(const DenseWeight& w, const void* A, const CUtensorMap* tmA, int lda, int M, void* out, int flags,
             const void* residual, int kclass, const LnFold* ln = nullptr, const float* bias = nullptr);

  // Enqueues the kernels of one forward pass on stream_ (directly, or into a stream capture).
  bool enqueue_forward(const int* d_ids, const int* d_seg, const int* d_mask, int B, int S, bool want_hidden_f32,
                       bool want_probs);
  void drop_graphs();

  // One captured forward pass per exact argument set.  The kernel arguments hold device addresses
  // of the activation arena, so every graph is dropped when the arena is reallocated.
  struct GraphKey {
    const int *ids, *seg, *mask;
    int B, S, flags;
    bool operator<(const GraphKey& o) const {
      return std::tie(ids, seg, mask, B, S, flags) < std::tie(o.ids, o.seg, o.mask, o.B, o.S, o.flags);
    }
  };
  struct GraphEntry {
    cudaGraphExec_t exec = nullptr;
    long launches = 0;
    int seen = 0;             // passes with this key so far; it is captured on pass GRAPH_CAPTURE_AT
    unsigned long long last_use = 0;
  };
  static constexpr int GRAPH_CAPTURE_AT = 3;     // a key seen once or twice is not worth a capture + instantiate
  static constexpr size_t GRAPH_CACHE_MAX = 64;  // beyond this the least recently used entry goes
  unsigned long long graph_tick_ = 0;
  std::map<GraphKey, GraphEntry> graphs_;
  bool graphs_enabled_ = true;
  bool nvtx_ = false;         // CUDABERT_NVTX=1: NVTX ranges around passes and launches
  bool fp8_widened_ = false;  // FP8 mode: weights expanded to fp16 at load (CUDABERT_FP8_OPERAND=widened)
  bool ln_fold_ = false;      // bf16 mode: LayerNorms folded into the GEMMs around them (CUDABERT_LN_FOLD=1)
  float* ln_stats1_ = nullptr;  // per row and 128-column slice: partial sum and sum of squares of the first ...
  float* ln_stats2_ = nullptr;  // ... and second LayerNorm's input of a layer
  bool f32_tensor_ = true;    // fp32 mode: dense layers on the tensor cores as sums of bf16 planes (CUDABERT_FP32_GEMM=cuda: CUDA cores)
  bool cls_last_ = true;  // pooler-only passes compute the last layer for the first token of every sequence only
  static constexpr int PDL_MAX_TOKENS = 4096;  // forward passes up to this many token slots use dependent launch
  long graph_replays_ = 0, graph_captures_ = 0;

  int dev_ = 0, num_sms_ = 148;
  bool large_ = false;
  int L_ = 0, H_ = 0, heads_ = 0, F_ = 0, prec_ = PREC_BF16, classes_ = 0, vocab_rows_ = 0;
  size_t esize_ = 2;
  cudaStream_t stream_ = nullptr;
  std::string dir_;
  std::vector<std::string> files_;

  // weights
  float *word_ = nullptr, *pos_ = nullptr, *type_ = nullptr;  // embedding tables stay fp32 in every mode
  float *emb_g_ = nullptr, *emb_b_ = nullptr;
  std::vector<LayerWeights> layer_;
  DenseWeight pooler_;
  float *cls_w_ = nullptr, *cls_b_ = nullptr;
  float* stage_f32_ = nullptr;  // device staging for load-time conversion
  size_t stage_elems_ = 0;
  struct Owned { void* p; size_t bytes; };
  std::vector<Owned> owned_;    // every cudaMalloc'ed weight buffer, in allocation order
  std::vector<void*> derived_;  // device buffers computed from the weights after loading (not part of the cache)
  bool prepare_ln_fold();       // the folded LayerNorms' vectors
  bool dev_alloc(void** p, size_t bytes);  // cudaMalloc + owned_

  // Weight cache (CUDABERT_WEIGHT_CACHE=<directory>): the device-ready weights of one (model directory,
  // mode) pair as one file, written after the first load and read back by later ones instead of
  // parsing, uploading and transposing some four hundred .npy files.  A cache file is used only if
  // its recorded signature (every .npy file's name, size and modification time, the mode and the
  // layout version) equals the directory's current one.
  std::string cache_dir_, cache_path_, cache_signature_;
  bool from_cache_ = false;             // this load fills the buffers from the cache file
  std::vector<size_t> cache_sizes_;     // from_cache_: size of every buffer, in allocation order
  bool cache_probe();                   // sets cache_path_ / cache_signature_; true if a valid file exists
  bool cache_fill();                    // file -> owned_ buffers
  void cache_write();                   // owned_ buffers -> file (failures are not errors)

  // activation arena
  size_t cap_tokens_ = 0;
  int cap_batch_ = 0;
  void* arena_ = nullptr;
  int *ids_ = nullptr, *kv_len_ = nullptr, *err_dev_ = nullptr;  // ids_: 3 * cap_tokens ints (ids | seg | mask)
  int* att_sched_ = nullptr;  // work order, mask flags (cap_batch each) and tile table (cap_tokens / 128) of the TMA-fed attention kernels
  // packed layout: padding tokens get no rows; row_start_[b] is the first row of sequence b and
  // row_start_[B] the live row count, all computed on the device (no host round trip)
  bool packed_ = true;
  int* row_start_ = nullptr;
  const int* m_dev_cur_ = nullptr;  // live row count of the forward being enqueued
  float* hidden_unpacked_ = nullptr;
  size_t hidden_unpacked_tokens_ = 0;
  // residual stream in fp32: xf_ (layer input / output), x1f_ (after the attention block),
  // y_ (dense outputs, added to the stream by the LayerNorm kernel).  xa_ / x1a_ are the copies that feed the GEMMs (fp16 in the bf16 and
  // fp8 modes; in fp32 mode they alias xf_ / x1f_).  ctx_, qkv_, z_ are in the GEMM element type.
  float *xf_ = nullptr, *x1f_ = nullptr;
  void* y_ = nullptr;  // dense outputs before the residual add: fp16 (bf16 / fp8 modes) or fp32 sums (fp32 mode)
  void *xa_ = nullptr, *x1a_ = nullptr, *ctx_ = nullptr, *qkv_ = nullptr, *z_ = nullptr;
  float *pooled_ = nullptr, *probs_ = nullptr;
  CUtensorMap tm_x_, tm_x1_, tm_ctx_, tm_z_, tm_qkv_;
  void* split_ = nullptr;          // fp32 mode on the tensor cores: the bf16 planes of the current GEMM's input, [tokens, 3 K]
  CUtensorMap tm_splitH_, tm_splitF_;  // ... viewed with K = H and K = F

  // pinned staging
  int* h_in_ = nullptr;
  size_t h_in_elems_ = 0;
  float* h_out_ = nullptr;
  size_t h_out_elems_ = 0;
  int* h_err_ = nullptr;

  // bookkeeping
  int status_ = 0;
  std::string error_;
  long launches_ = 0;
  bool profiling_ = false;
  std::vector<cudaEvent_t> ev_;
  std::vector<int> ev_class_;
  size_t ev_used_ = 0;
  double prof_ms_[KC_COUNT] = {};
  long prof_n_[KC_COUNT] = {};
};

}  // namespace cb
