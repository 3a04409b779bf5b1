// extern "C" surface of libcudaBERT.so; declarations and the reference citations for every
// entry point are in include/cudabert.h.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/cudabert.h"
#include "model.h"

using cb::Model;

namespace {

thread_local std::string g_init_error;

int precision_from_env() {
  const char* p = std::getenv("CUDABERT_PRECISION");
  if (!p || !*p) return cb::PREC_BF16;
  const std::string s(p);
  if (s == "fp32" || s == "0") return cb::PREC_FP32;
  if (s == "bf16" || s == "1") return cb::PREC_BF16;
  if (s == "fp8" || s == "2") return cb::PREC_FP8;
  return -1;
}

Model* as_model(void* h) { return static_cast<Model*>(h); }

// Non-CUDA errors (bad arguments, a device-side check) do not poison later calls.
void begin_call(Model* m) {
  if (m->status() != 0 && m->status() != 2) m->clear_error();
}

// The reference's seed input (cuda_bert/cuda_bert.cu:12-22, 94-103): an 11-token sequence whose
// first 10 entries are cycled up to seq_length - 1 and whose last entry closes the row.
std::vector<int> tile_seed(const int* seed, int seq_length, int batch) {
  std::vector<int> out(static_cast<size_t>(seq_length) * batch);
  for (int i = 0; i < seq_length - 1; ++i) out[i] = seed[i % 10];
  out[seq_length - 1] = seed[10];
  for (int b = 1; b < batch; ++b) std::memcpy(&out[static_cast<size_t>(b) * seq_length], &out[0], seq_length * sizeof(int));
  return out;
}

struct DevErr {  // scratch error word for the single-kernel entry points
  int* p = nullptr;
  bool ok() {
    if (!p && cudaMalloc(&p, sizeof(int)) != cudaSuccess) return false;
    return cudaMemset(p, 0, sizeof(int)) == cudaSuccess;
  }
};

}  // namespace

namespace cb {
void set_thread_error(const std::string& msg) { g_init_error = msg; }
}  // namespace cb

extern "C" {

void* cudabert_init_ex(bool large, int num_gpu, int max_batchsize, int max_seq_length, const char* dir, int precision,
                       int num_layers) {
  g_init_error.clear();
  if (precision < 0) precision = precision_from_env();
  if (precision < 0) {
    g_init_error = "CUDABERT_PRECISION must be fp32, bf16 or fp8";
    return nullptr;
  }
  if (max_batchsize < 0 || max_seq_length < 0) {
    g_init_error = "max_batchsize and max_seq_length must be >= 0";
    return nullptr;
  }
  Model* m = new Model();
  if (!m->init(large, num_gpu, max_batchsize, max_seq_length, dir ? dir : "", precision, num_layers)) {
    g_init_error = m->error();
    delete m;
    return nullptr;
  }
  return m;
}

void* init_model(bool large, int num_gpu, int max_batchsize, int max_seq_length, char* dir) {
  return cudabert_init_ex(large, num_gpu, max_batchsize, max_seq_length, dir, -1, 0);
}

void release_model(void* model) { delete as_model(model); }

Retval Cuda_Inference(void* model, int* words, int* token_types, int batchsize, int seq_length, int* masks) {
  Retval r = {nullptr, nullptr};
  Model* m = as_model(model);
  if (!m) return r;
  begin_call(m);
  // run_host with no host outputs: inputs are staged and copied, results stay on the device
  if (!m->run_host_keep(words, token_types, masks, batchsize, seq_length)) return r;
  r.tensor = m->hidden_f32_dev();
  r.pooled_output = m->pooled_dev();
  return r;
}

void Cuda_Bert(void* model, float* output, int* words, int* token_types, int batchsize, int seq_length,
               int* attention_mask) {
  Model* m = as_model(model);
  if (!m) return;
  begin_call(m);
  if (!output) {
    m->set_error(1, "output must not be null");
    return;
  }
  m->run_host(words, token_types, attention_mask, batchsize, seq_length, output, nullptr, 0);
}

void Cuda_Classify(void* model, float* output, int* words, int* token_types, int batchsize, int seq_length,
                   int num_classes, int* attention_mask) {
  Model* m = as_model(model);
  if (!m) return;
  begin_call(m);
  if (!output) {
    m->set_error(1, "output must not be null");
    return;
  }
  m->run_host(words, token_types, attention_mask, batchsize, seq_length, nullptr, output, num_classes);
}

void test(int batchsize, int seq_length, int nIter, bool large, int num_gpu) {
  if (batchsize < 1 || seq_length < 2 || nIter < 1) {
    std::printf("test: need batchsize >= 1, seq_length >= 2, nIter >= 1\n");
    return;
  }
  void* h = init_model(large, num_gpu, batchsize, seq_length, const_cast<char*>(""));
  if (!h) {
    std::printf("test: init_model failed: %s\n", g_init_error.c_str());
    return;
  }
  Model* m = as_model(h);
  const int word_seed[11] = {2040, 2001, 3958, 27227, 1029, 3958, 103, 2001, 1037, 13997, 11510};
  const int type_seed[11] = {0, 0, 0, 0, 0, 1, 1, 1, 1, 1, 1};
  const int mask_seed[11] = {1, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0};
  std::vector<int> ids = tile_seed(word_seed, seq_length, batchsize);
  std::vector<int> seg = tile_seed(type_seed, seq_length, batchsize);
  std::vector<int> msk = tile_seed(mask_seed, seq_length, batchsize);
  std::vector<float> out(static_cast<size_t>(batchsize) * m->hidden());
  std::printf(" Seq_length : %d\n Batchsize : %d\n%s\n", seq_length, batchsize,
              large ? "Using large Model" : "Using Base Model");
  for (int i = 0; i < 10; ++i) {
    if (!m->run_host(ids.data(), seg.data(), msk.data(), batchsize, seq_length, out.data(), nullptr, 0)) {
      std::printf("test: forward failed: %s\n", m->error().c_str());
      delete m;
      return;
    }
    if (i == 0) {
      const int step = std::max(batchsize / 10, 1);
      for (int b = 0; b < batchsize; b += step) {
        std::printf("unit_test row %d:", b);
        for (int j = 0; j < 10; ++j) std::printf(" %.6f", out[static_cast<size_t>(b) * m->hidden() + j]);
        std::printf("\n");
      }
    }
  }
  cudaEvent_t start, stop;
  cudaEventCreate(&start);
  cudaEventCreate(&stop);
  std::vector<float> latency(nIter);
  double total = 0;
  for (int i = 0; i < nIter; ++i) {
    cudaEventRecord(start, m->stream());
    m->run_host(ids.data(), seg.data(), msk.data(), batchsize, seq_length, out.data(), nullptr, 0);
    cudaEventRecord(stop, m->stream());
    cudaEventSynchronize(stop);
    float ms = 0;
    cudaEventElapsedTime(&ms, start, stop);
    latency[i] = ms;
    total += ms;
  }
  std::sort(latency.begin(), latency.end());
  std::printf(" 99 Latency : %fms\n", latency[std::min(nIter - 1, static_cast<int>(nIter * 0.99))]);
  std::printf(" Throughput: %f batches per second (%f sequences per second)\n", nIter * 1000.0 / total,
              nIter * 1000.0 / total * batchsize);
  std::printf("Time= %.2f(ms)\n\n", total / nIter);
  cudaEventDestroy(start);
  cudaEventDestroy(stop);
  delete m;
}

int cudabert_status(void* model) { return model ? as_model(model)->status() : (g_init_error.empty() ? 0 : 3); }

const char* cudabert_last_error(void* model) {
  if (!model) return g_init_error.c_str();
  return as_model(model)->error().c_str();
}

int cudabert_attention_kernel_for(int seq_length) { return cb::attention_kernel_for(seq_length); }

int cudabert_hidden_size(void* model) { return model ? as_model(model)->hidden() : 0; }
int cudabert_num_classes(void* model) { return model ? as_model(model)->num_classes() : 0; }

int cudabert_forward_dev(void* model, const int* ids_dev, const int* seg_dev, const int* mask_dev, int batchsize,
                         int seq_length) {
  Model* m = as_model(model);
  if (!m) return 1;
  begin_call(m);
  return m->forward_device(ids_dev, seg_dev, mask_dev, batchsize, seq_length, false, false) ? 0 : m->status();
}

int cudabert_classify_dev(void* model, const int* ids_dev, const int* seg_dev, const int* mask_dev, int batchsize,
                          int seq_length) {
  Model* m = as_model(model);
  if (!m) return 1;
  begin_call(m);
  return m->forward_device(ids_dev, seg_dev, mask_dev, batchsize, seq_length, false, true) ? 0 : m->status();
}

int cudabert_copy_to_host(void* dst_host, const void* src_dev, size_t bytes) {
  if (!dst_host || !src_dev) return 1;
  return cudaMemcpy(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 2;
}

float* cudabert_probs_dev(void* model) { return model ? as_model(model)->probs_dev() : nullptr; }

int cudabert_sync(void* model) {
  Model* m = as_model(model);
  if (!m) return 1;
  return m->sync() ? 0 : m->status();
}

int cudabert_test_wait_timeout(void* model, int limit_us) {
  Model* m = as_model(model);
  if (!m || limit_us <= 0) return 1;
  begin_call(m);
  return m->probe_wait_timeout(static_cast<unsigned long long>(limit_us) * 1000ull);
}

float* cudabert_pooled_dev(void* model) { return model ? as_model(model)->pooled_dev() : nullptr; }
void* cudabert_stream(void* model) { return model ? static_cast<void*>(as_model(model)->stream()) : nullptr; }
long cudabert_launch_count(void* model) { return model ? as_model(model)->launches_last_forward() : 0; }
long cudabert_graph_captures(void* model) { return model ? as_model(model)->graph_captures() : 0; }
long cudabert_graph_replays(void* model) { return model ? as_model(model)->graph_replays() : 0; }
void cudabert_profile_enable(void* model, int on) {
  if (model) as_model(model)->set_profiling(on != 0);
}
void cudabert_profile_reset(void* model) {
  if (model) as_model(model)->reset_profile();
}
int cudabert_profile_get(void* model, int kernel_class, double* total_ms, long* launches) {
  if (!model || !total_ms || !launches) return 1;
  as_model(model)->get_profile(kernel_class, total_ms, launches);
  return 0;
}

// ------------------------------------------------------------------ single kernels
int cudabert_k_gemm_tcgen05(const void* A_dev, long lda, const void* W_dev, int M, int N, int K, void* out_dev, int flags,
                         const float* bias_dev, const void* residual_dev, const float* colscale_dev, int* err_dev) {
  if (!A_dev || !W_dev || !out_dev || M <= 0 || N <= 0 || K <= 0 || lda < K) return 1;
  if (flags & cb::EPI_SPLIT3) return 1;  // operands of three planes: cudabert_k_gemm_f32_tensor builds them
  if (flags & (cb::EPI_LN_SUM | cb::EPI_LN_APPLY | cb::EPI_RES_LN)) return 1;  // folded LayerNorms need the model's buffers
  CUtensorMap tmA, tmW;
  if (!cb::make_tmap_16bit_kmajor(&tmA, A_dev, M, K, static_cast<uint64_t>(lda) * 2, 128)) return 2;
  if (flags & cb::EPI_W_FP8) {
    if (!cb::make_tmap_u8_kmajor(&tmW, W_dev, N, K)) return 2;
  } else if (!cb::make_tmap_16bit_kmajor(&tmW, W_dev, N, K, static_cast<uint64_t>(K) * 2, cb::gemm_w_box_rows(N))) {
    return 2;
  }
  static thread_local DevErr scratch;
  int* err = err_dev;
  if (!err) {
    if (!scratch.ok()) return 2;
    err = scratch.p;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cb::GemmEpilogue epi;
  epi.flags = flags;
  epi.bias = bias_dev;
  epi.residual = residual_dev;
  epi.colscale = colscale_dev;
  const int n = cb::gemm_tcgen05(&tmA, &tmW, M, N, K, out_dev, N, epi, err, sms, nullptr, nullptr);
  if (n < 0) return 3;
  if (cudaDeviceSynchronize() != cudaSuccess) return 4;
  int herr = 0;
  if (cudaMemcpy(&herr, err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return 4;
  return herr ? 5 : 0;
}

int cudabert_k_gemm_f32(const float* A_dev, int lda, const float* W_dev, int M, int N, int K, float* out_dev,
                        int flags, const float* bias_dev, const float* residual_dev) {
  cb::GemmEpilogue epi;
  epi.flags = flags;
  epi.bias = bias_dev;
  epi.residual = residual_dev;
  const int n = cb::gemm_f32(A_dev, lda, W_dev, M, N, K, out_dev, N, epi, nullptr, nullptr);
  if (n < 0) return 3;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : 4;
}

int cudabert_k_gemm_f32_tensor(const float* A_dev, int lda, const float* W_dev, int M, int N, int K, float* out_dev,
                               int flags, const float* bias_dev, const float* residual_dev) {
  if (!A_dev || !W_dev || !out_dev || M <= 0 || N <= 0 || K <= 0 || lda < K || (N % 128) || (K % 64) || (lda % 4))
    return 1;
  // the bf16 planes of both operands, then the tcgen05 GEMM over them
  __nv_bfloat16 *a3 = nullptr, *w3 = nullptr;
  int* err = nullptr;
  int rc = 0;
  if (cudaMalloc(&a3, static_cast<size_t>(M) * K * 6) != cudaSuccess ||
      cudaMalloc(&w3, static_cast<size_t>(N) * K * 6) != cudaSuccess || cudaMalloc(&err, sizeof(int)) != cudaSuccess)
    rc = 2;
  CUtensorMap tmA, tmW;
  if (!rc && (!cb::make_tmap_16bit_kmajor(&tmA, a3, M, 3ull * K, 6ull * K, 128) ||
              !cb::make_tmap_16bit_kmajor(&tmW, w3, N, 3ull * K, 6ull * K, cb::gemm_split_w_box_rows(N))))
    rc = 2;
  if (!rc) {
    cudaMemset(err, 0, sizeof(int));
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cb::GemmEpilogue epi;
    epi.flags = (flags & (cb::EPI_BIAS | cb::EPI_GELU | cb::EPI_RESIDUAL | cb::EPI_TANH)) | cb::EPI_OUT_F32 | cb::EPI_SPLIT3;
    epi.bias = bias_dev;
    epi.residual = residual_dev;
    if (cb::transpose_split_bf16x3(W_dev, w3, K, N, nullptr) < 0 ||
        cb::split_bf16x3(A_dev, lda, a3, M, K, nullptr, nullptr) < 0 ||
        cb::gemm_tcgen05(&tmA, &tmW, M, N, K, out_dev, N, epi, err, sms, nullptr, nullptr) < 0)
      rc = 3;
    if (cudaDeviceSynchronize() != cudaSuccess) rc = 4;
    int herr = 0;
    if (!rc && (cudaMemcpy(&herr, err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess || herr)) rc = 5;
  }
  cudaFree(a3);
  cudaFree(w3);
  cudaFree(err);
  return rc;
}

int cudabert_k_gemm_ln_folded(const void* A1_dev, const void* W1_dev, const float* b1_dev, const float* res_dev,
                              const float* gamma_dev, const float* beta_dev, const void* W2_dev, const float* b2_dev, int M,
                              int H, int K1, int N2, int gelu, float* sum_dev, void* out_dev) {
  if (!A1_dev || !W1_dev || !b1_dev || !res_dev || !gamma_dev || !beta_dev || !W2_dev || !b2_dev || !sum_dev || !out_dev)
    return 1;
  if (M <= 0 || H <= 0 || H % 256 != 0 || K1 % 64 != 0 || N2 % 128 != 0 || !cb::gemm_uses_pairs(H)) return 1;
  // scratch: s * gamma (fp16 [M, H]) | statistics (float2 [M, H / 128]) | gamma W2 [N2] | beta W2 + b2 [N2] | error word
  const size_t b_s16 = static_cast<size_t>(M) * H * 2, b_st = static_cast<size_t>(M) * (H / 128) * 8;
  char* scratch = nullptr;
  if (cudaMalloc(&scratch, b_s16 + b_st + 2 * static_cast<size_t>(N2) * 4 + 16) != cudaSuccess) return 2;
  __half* s16 = reinterpret_cast<__half*>(scratch);
  float* stats = reinterpret_cast<float*>(scratch + b_s16);
  float* c = reinterpret_cast<float*>(scratch + b_s16 + b_st);
  float* d = c + N2;
  int* err = reinterpret_cast<int*>(d + N2);
  cudaMemset(err, 0, sizeof(int));
  int rc = 0;
  CUtensorMap tmA1, tmW1, tmA2, tmW2;
  if (!cb::make_tmap_16bit_kmajor(&tmA1, A1_dev, M, K1, static_cast<uint64_t>(K1) * 2, 128) ||
      !cb::make_tmap_16bit_kmajor(&tmW1, W1_dev, H, K1, static_cast<uint64_t>(K1) * 2, cb::gemm_w_box_rows(H)) ||
      !cb::make_tmap_16bit_kmajor(&tmA2, s16, M, H, static_cast<uint64_t>(H) * 2, 128) ||
      !cb::make_tmap_16bit_kmajor(&tmW2, W2_dev, N2, H, static_cast<uint64_t>(H) * 2, cb::gemm_w_box_rows(N2)))
    rc = 2;
  if (!rc) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cb::GemmEpilogue p;  // the GEMM in front of the LayerNorm
    p.flags = cb::EPI_BIAS | cb::EPI_IN_F16 | cb::EPI_WSCALE | cb::EPI_OUT_F32 | cb::EPI_RESIDUAL | cb::EPI_LN_SUM;
    p.bias = b1_dev;
    p.residual = res_dev;
    p.ln.out16 = s16;
    p.ln.gamma = gamma_dev;
    p.ln.stats_out = stats;
    cb::GemmEpilogue q;  // the GEMM behind it
    q.flags = cb::EPI_BIAS | cb::EPI_IN_F16 | cb::EPI_WSCALE | cb::EPI_OUT_F16 | cb::EPI_LN_APPLY | (gelu ? cb::EPI_GELU : 0);
    q.bias = d;
    q.ln.stats_in = stats;
    q.ln.c = c;
    if (cb::ln_fold_vectors(static_cast<const __half*>(W2_dev), gamma_dev, beta_dev, b2_dev, c, d, N2, H, nullptr) < 0 ||
        cb::gemm_tcgen05(&tmA1, &tmW1, M, H, K1, sum_dev, H, p, err, sms, nullptr, nullptr) < 0 ||
        cb::gemm_tcgen05(&tmA2, &tmW2, M, N2, H, out_dev, N2, q, err, sms, nullptr, nullptr) < 0)
      rc = 3;
    if (cudaDeviceSynchronize() != cudaSuccess) rc = 4;
    int herr = 0;
    if (!rc && (cudaMemcpy(&herr, err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess || herr)) rc = 5;
  }
  cudaFree(scratch);
  return rc;
}

int cudabert_k_attention(int kernel, const void* qkv_dev, const int* mask_dev, void* ctx_dev, int B, int S, int heads) {
  if (!qkv_dev || !ctx_dev || B <= 0 || S <= 0 || heads <= 0) return 1;
  const int cls_only = (kernel & 16) ? 1 : 0;  // + 16: first query of every sequence only, ctx is [B, H]
  const bool packed = (kernel & 32) != 0;      // + 32: the sequences' valid rows lie back to back
  kernel &= 15;
  if (kernel > 3 || (cls_only && kernel == 0)) return 1;
  const size_t tiles = (static_cast<size_t>(B) * S + 127) / 128;
  int* kv = nullptr;  // kv_len [B] | error word | row_start [B + 1] | sched [2 B + tiles]
  if (cudaMalloc(&kv, (4 * static_cast<size_t>(B) + 2 + tiles) * sizeof(int)) != cudaSuccess) return 2;
  int* err = kv + B;
  int* rs = packed ? kv + B + 1 : nullptr;
  int* sched = (kernel == 2 || kernel == 3) ? kv + 2 * B + 2 : nullptr;
  cudaMemset(err, 0, sizeof(int));
  int rc = 0;
  if (cb::row_layout(mask_dev, kv, rs, sched, B, S, nullptr) < 0) rc = 3;
  if (!rc) {
    int n;
    if (kernel == 2 || kernel == 3) {  // tcgen05 kernel, persistent mma.sync kernel: both read K and V by TMA
      CUtensorMap tm;
      int dev = 0, sms = 148;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (!cb::make_tmap_qkv(&tm, qkv_dev, static_cast<uint64_t>(B) * S, heads * 64)) {
        cudaFree(kv);
        return 2;
      }
      if (kernel == 2)
        n = cb::attention_f16_tc(&tm, mask_dev, kv, rs, sched, static_cast<__half*>(ctx_dev), B, S, heads,
                                 sms, cls_only, err, nullptr);
      else
        n = cb::attention_f16_persist(&tm, mask_dev, kv, rs, sched, static_cast<__half*>(ctx_dev), B, S,
                                       heads, sms, cls_only, err, nullptr);
    } else if (kernel) {
      n = cb::attention_f16(static_cast<const __half*>(qkv_dev), mask_dev, kv, rs,
                             static_cast<__half*>(ctx_dev), B, S, heads, cls_only, nullptr);
    } else {
      n = cb::attention_f32(static_cast<const float*>(qkv_dev), mask_dev, kv, rs, static_cast<float*>(ctx_dev), B,
                            S, heads, nullptr);
    }
    if (n < 0) rc = 3;
  }
  if (cudaDeviceSynchronize() != cudaSuccess) rc = 4;
  int herr = 0;
  if (!rc && cudaMemcpy(&herr, err, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess && herr) rc = 5;
  cudaFree(kv);
  return rc;
}

int cudabert_k_embed_layernorm(int half, const int* ids_dev, const int* seg_dev, const float* word_dev,
                               const float* pos_dev, const float* type_dev, const float* gamma_dev,
                               const float* beta_dev, void* out_dev, float* out_f32_dev, int tokens, int S, int H,
                               int vocab) {
  static thread_local DevErr scratch;
  if (!scratch.ok()) return 2;
  int n;
  if (half)
    n = cb::embed_layernorm<__half>(ids_dev, seg_dev, word_dev, pos_dev, type_dev, gamma_dev, beta_dev,
                                           static_cast<__half*>(out_dev), out_f32_dev, tokens, S, H, vocab,
                                           scratch.p, nullptr, nullptr);
  else
    n = cb::embed_layernorm<float>(ids_dev, seg_dev, word_dev, pos_dev, type_dev, gamma_dev, beta_dev,
                                   static_cast<float*>(out_dev), out_f32_dev, tokens, S, H, vocab, scratch.p, nullptr,
                                   nullptr);
  if (n < 0) return 3;
  if (cudaDeviceSynchronize() != cudaSuccess) return 4;
  int herr = 0;
  cudaMemcpy(&herr, scratch.p, sizeof(int), cudaMemcpyDeviceToHost);
  return herr ? 5 : 0;
}

int cudabert_k_layernorm(int out_f16, int in_f16, const void* x_dev, const float* residual_dev,
                         const float* gamma_dev, const float* beta_dev, void* out_dev, float* out_f32_dev, int tokens,
                         int H) {
  int n;
  const __half* xh = static_cast<const __half*>(x_dev);
  const float* xf = static_cast<const float*>(x_dev);
  if (out_f16 && in_f16)
    n = cb::layernorm<__half, __half>(xh, residual_dev, gamma_dev, beta_dev,
                                             static_cast<__half*>(out_dev), out_f32_dev, tokens, H, nullptr, nullptr);
  else if (out_f16)
    n = cb::layernorm<float, __half>(xf, residual_dev, gamma_dev, beta_dev,
                                            static_cast<__half*>(out_dev), out_f32_dev, tokens, H, nullptr, nullptr);
  else if (in_f16)
    n = cb::layernorm<__half, float>(xh, residual_dev, gamma_dev, beta_dev, static_cast<float*>(out_dev), out_f32_dev,
                                     tokens, H, nullptr, nullptr);
  else
    n = cb::layernorm<float, float>(xf, residual_dev, gamma_dev, beta_dev, static_cast<float*>(out_dev), out_f32_dev,
                                    tokens, H, nullptr, nullptr);
  if (n < 0) return 3;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : 4;
}

}  // extern "C"
