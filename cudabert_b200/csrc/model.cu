#include "model.h"

#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <nvtx3/nvToolsExt.h>

#include "npy.h"

namespace cb {

namespace {
constexpr int MAX_CLASSES = 32;
constexpr int MAX_SEQ = 512;

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}  // namespace

bool Model::fail(int code, const std::string& msg) {
  if (status_ == 0) {
    status_ = code;
    error_ = msg;
  }
  if (std::getenv("CUDABERT_VERBOSE")) std::fprintf(stderr, "[cudaBERT] error %d: %s\n", code, msg.c_str());
  return false;
}

bool Model::check(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  return fail(2, std::string(what) + ": " + cudaGetErrorString(e));
}

Model::~Model() {
  cudaSetDevice(dev_);
  if (stream_) cudaStreamSynchronize(stream_);
  for (const Owned& o : owned_) cudaFree(o.p);
  for (void* p : derived_) cudaFree(p);
  if (arena_) cudaFree(arena_);
  if (stage_f32_) cudaFree(stage_f32_);
  if (hidden_unpacked_) cudaFree(hidden_unpacked_);
  if (err_dev_) cudaFree(err_dev_);
  if (h_in_) cudaFreeHost(h_in_);
  if (h_out_) cudaFreeHost(h_out_);
  if (h_err_) cudaFreeHost(h_err_);
  for (cudaEvent_t e : ev_) cudaEventDestroy(e);
  drop_graphs();
  if (stream_) cudaStreamDestroy(stream_);
}

void Model::drop_graphs() {
  for (auto& kv : graphs_)
    if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
  graphs_.clear();
}

bool Model::init(bool large, int gpu, int max_batch, int max_seq, const std::string& dir, int precision,
                 int num_layers) {
  if (precision < PREC_FP32 || precision > PREC_FP8) return fail(1, "precision must be 0 (fp32), 1 (bf16) or 2 (fp8)");
  int ndev = 0;
  if (!check(cudaGetDeviceCount(&ndev), "cudaGetDeviceCount")) return false;
  if (gpu < 0 || gpu >= ndev) return fail(1, "gpu id out of range");
  dev_ = gpu;
  if (!check(cudaSetDevice(gpu), "cudaSetDevice")) return false;
  cudaDeviceProp prop;
  if (!check(cudaGetDeviceProperties(&prop, gpu), "cudaGetDeviceProperties")) return false;
  if (prop.major != 10) return fail(2, "this library is built for sm_100a (B200) only");
  num_sms_ = prop.multiProcessorCount;
  large_ = large;
  // model dimensions are fixed by the `large` flag, as in utils/manager.cu:8-15
  if (large) { L_ = 24; H_ = 1024; heads_ = 16; F_ = 4096; }
  else       { L_ = 12; H_ = 768;  heads_ = 12; F_ = 3072; }
  if (num_layers > 0) L_ = std::min(L_, num_layers);
  prec_ = precision;
  {
    // CUDABERT_PACK=0 keeps the padded layout (hidden states are then computed for padding tokens too)
    const char* e = std::getenv("CUDABERT_PACK");
    packed_ = !(e && e[0] == '0');
    // CUDABERT_GRAPH=0: enqueue every forward pass kernel by kernel, never replay a captured graph
    const char* gr = std::getenv("CUDABERT_GRAPH");
    graphs_enabled_ = !(gr && gr[0] == '0');
    // CUDABERT_LAST_LAYER=full: compute the last layer for every token even when only the pooler
    // output is asked for
    const char* ll = std::getenv("CUDABERT_LAST_LAYER");
    cls_last_ = !(ll && ll[0] == 'f');
    // CUDABERT_FP8_OPERAND=widened: FP8 mode expands the quantised weights to fp16 once, at load, and
    // runs the 16-bit GEMM on them (same arithmetic, same results; twice the weight memory, and on
    // 1024 x 64 batches of BERT-large 25.2 against 28.9 ms per pass).  Default: the GEMM reads the E4M3 bytes.
    const char* f8 = std::getenv("CUDABERT_FP8_OPERAND");
    fp8_widened_ = f8 && f8[0] == 'w';
    // CUDABERT_FP32_GEMM=cuda: fp32 mode multiplies on the CUDA cores (gemm_f32) instead of splitting
    // both operands into three bf16 planes for the tensor cores
    const char* f32 = std::getenv("CUDABERT_FP32_GEMM");
    f32_tensor_ = !(f32 && f32[0] == 'c');
    // CUDABERT_LN_FOLD=1 (bf16 mode): the LayerNorms between the dense layers are not run as kernels;
    // the GEMM before one writes its input and row statistics, the GEMM after it normalises in its epilogue
    const char* lf = std::getenv("CUDABERT_LN_FOLD");
    ln_fold_ = lf && lf[0] == '1' && precision == PREC_BF16;
    const char* nv = std::getenv("CUDABERT_NVTX");
    nvtx_ = nv && nv[0] == '1';
  }
  esize_ = (precision == PREC_FP32) ? 4 : 2;
  if (!check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate")) return false;
  if (!check(cudaMalloc(&err_dev_, sizeof(int)), "cudaMalloc")) return false;
  if (!check(cudaMemset(err_dev_, 0, sizeof(int)), "cudaMemset")) return false;
  if (!check(cudaMallocHost(&h_err_, sizeof(int)), "cudaMallocHost")) return false;
  *h_err_ = 0;
  // default directories of the reference (utils/manager.cu:8-17)
  dir_ = dir.empty() ? (large ? "model_npy/large_uncased" : "model_npy/base_uncased") : dir;
  if (!load_weights(dir_)) return false;
  if (max_batch > 0 && max_seq > 0) {
    if (max_seq > MAX_SEQ) return fail(1, "max_seq_length exceeds the 512 positions of the position table");
    if (!ensure_capacity(max_batch, max_seq, false)) return false;
  }
  return true;
}

// ------------------------------------------------------------------ weight loading
const std::string* Model::find_file(const std::vector<std::string>& keys) const {
  // first file (sorted by name) whose NAME contains every key -- the reference matches the
  // same way on the full path in directory order (utils/load_model.cc:15-37)
  for (const std::string& f : files_) {
    bool all = true;
    for (const std::string& k : keys)
      if (f.find(k) == std::string::npos) { all = false; break; }
    if (all) return &f;
  }
  return nullptr;
}

bool Model::dev_alloc(void** p, size_t bytes) {
  if (from_cache_) {
    // the sizes were recorded when the cache was written; a difference means a stale or foreign file
    const size_t i = owned_.size();
    if (i >= cache_sizes_.size()) return fail(3, "weight cache " + cache_path_ + " does not match this model: delete it");
    if (bytes == 0) bytes = cache_sizes_[i];
    if (bytes != cache_sizes_[i]) return fail(3, "weight cache " + cache_path_ + " does not match this model: delete it");
  }
  if (!check(cudaMalloc(p, bytes), "cudaMalloc(weights)")) return false;
  owned_.push_back(Owned{*p, bytes});
  return true;
}

bool Model::read_tensor(const std::vector<std::string>& keys, size_t expect, NpyArray* arr) {
  if (from_cache_) return find_file(keys) != nullptr || fail(3, "weight cache: a tensor's file has disappeared");
  const std::string* f = find_file(keys);
  if (!f) {
    std::string k;
    for (const auto& s : keys) k += " " + s;
    return fail(3, "no weight file in " + dir_ + " matches keys:" + k);
  }
  std::string err;
  if (!load_npy_f32(dir_ + "/" + *f, arr, &err)) return fail(3, err);
  if (expect && arr->numel() != expect)
    return fail(3, *f + ": has " + std::to_string(arr->numel()) + " elements, expected " + std::to_string(expect));
  if (arr->numel() > stage_elems_) {
    if (stage_f32_) cudaFree(stage_f32_);
    stage_f32_ = nullptr;
    stage_elems_ = 0;
    if (!check(cudaMalloc(&stage_f32_, arr->numel() * sizeof(float)), "cudaMalloc(staging)")) return false;
    stage_elems_ = arr->numel();
  }
  if (!check(cudaMemcpyAsync(stage_f32_, arr->data.data(), arr->numel() * sizeof(float), cudaMemcpyHostToDevice,
                             stream_), "weight upload"))
    return false;
  return check(cudaStreamSynchronize(stream_), "weight upload");
}

bool Model::upload_vec(const std::vector<std::string>& keys, size_t n, float** dst) {
  NpyArray a;
  if (!read_tensor(keys, n, &a)) return false;
  if (!*dst && !dev_alloc(reinterpret_cast<void**>(dst), n * sizeof(float))) return false;
  if (from_cache_) return true;
  if (!check(cudaMemcpyAsync(*dst, stage_f32_, n * sizeof(float), cudaMemcpyDeviceToDevice, stream_), "copy"))
    return false;
  return check(cudaStreamSynchronize(stream_), "copy");
}

bool Model::upload_table(const std::vector<std::string>& keys, size_t min_rows, float** dst, int* rows_out) {
  NpyArray a;
  if (!read_tensor(keys, 0, &a)) return false;
  if (from_cache_) {  // the size comes from the cache's record; the shape was checked when it was written
    if (!dev_alloc(reinterpret_cast<void**>(dst), 0)) return false;
    if (rows_out) *rows_out = static_cast<int>(owned_.back().bytes / (sizeof(float) * H_));
    return true;
  }
  if (a.shape.size() != 2 || a.shape[1] != static_cast<size_t>(H_) || a.shape[0] < min_rows)
    return fail(3, "embedding table has the wrong shape");
  if (rows_out) *rows_out = static_cast<int>(a.shape[0]);
  const size_t n = a.numel();
  if (!dev_alloc(reinterpret_cast<void**>(dst), n * sizeof(float))) return false;
  if (!check(cudaMemcpyAsync(*dst, stage_f32_, n * 4, cudaMemcpyDeviceToDevice, stream_), "copy")) return false;
  return check(cudaStreamSynchronize(stream_), "table copy");
}

bool Model::load_dense(const std::vector<std::string>& keys_kernel, const std::vector<std::string>& keys_bias, int K,
                       int N, DenseWeight* d, int n_off, int n_total, int prec) {
  const size_t esize = (prec == PREC_FP32) ? 4 : (prec == PREC_FP32_SPLIT) ? 6 : 2;  // bytes per weight
  if (n_off == 0) {
    d->K = K;
    d->N = n_total;
    const size_t elems = static_cast<size_t>(K) * n_total;
    if ((prec != PREC_FP8 || fp8_widened_) && !dev_alloc(&d->w, elems * esize)) return false;
    if (!dev_alloc(reinterpret_cast<void**>(&d->bias), n_total * sizeof(float))) return false;
    if (prec == PREC_FP8) {
      // without widening the E4M3 bytes are the only copy of the weights; the GEMM reads them
      if (!fp8_widened_ && !dev_alloc(reinterpret_cast<void**>(&d->w_fp8), elems)) return false;
      if (!dev_alloc(reinterpret_cast<void**>(&d->colscale), n_total * sizeof(float))) return false;
    }
  }
  NpyArray a;
  if (!read_tensor(keys_kernel, static_cast<size_t>(K) * N, &a)) return false;
  if (from_cache_) return true;
  if (a.shape.size() != 2 || a.shape[0] != static_cast<size_t>(K) || a.shape[1] != static_cast<size_t>(N))
    return fail(3, "dense kernel is not stored [in, out]");
  if (prec == PREC_FP32) {
    // keep [K, N]; Q, K, V are packed side by side into [K, 3H]
    float* base = static_cast<float*>(d->w) + n_off;
    if (!check(cudaMemcpy2DAsync(base, static_cast<size_t>(n_total) * 4, stage_f32_, static_cast<size_t>(N) * 4,
                                 static_cast<size_t>(N) * 4, K, cudaMemcpyDeviceToDevice, stream_), "pack"))
      return false;
  } else if (prec == PREC_FP32_SPLIT) {
    if (transpose_split_bf16x3(stage_f32_, static_cast<__nv_bfloat16*>(d->w) + static_cast<size_t>(n_off) * 3 * K, K, N,
                               stream_) < 0)
      return fail(2, "transpose launch failed");
  } else if (prec == PREC_BF16) {
    if (transpose_round_bf16(stage_f32_, static_cast<__half*>(d->w) + static_cast<size_t>(n_off) * K, K, N,
                          stream_) < 0)
      return fail(2, "transpose launch failed");
  } else {
    float* scale_dev = d->colscale + n_off;  // first element of the segment doubles as the scalar slot
    const size_t w_off = static_cast<size_t>(n_off) * K;
    if (quantize_fp8_weight(stage_f32_, fp8_widened_ ? nullptr : d->w_fp8 + w_off,
                            fp8_widened_ ? static_cast<__half*>(d->w) + w_off : nullptr, scale_dev, K, N, stream_) < 0)
      return fail(2, "quantise launch failed");
    float scale = 0.f;
    if (!check(cudaMemcpyAsync(&scale, scale_dev, sizeof(float), cudaMemcpyDeviceToHost, stream_), "scale")) return false;
    if (!check(cudaStreamSynchronize(stream_), "scale")) return false;
    if (fill_f32(scale_dev, scale, N, stream_) < 0) return fail(2, "fill launch failed");
  }
  if (!check(cudaStreamSynchronize(stream_), "weight conversion")) return false;
  NpyArray b;
  if (!read_tensor(keys_bias, N, &b)) return false;
  if (!check(cudaMemcpyAsync(d->bias + n_off, stage_f32_, N * sizeof(float), cudaMemcpyDeviceToDevice, stream_),
             "bias"))
    return false;
  return check(cudaStreamSynchronize(stream_), "bias");
}

bool Model::finish_dense(DenseWeight* d, int prec) {
  if (prec == PREC_FP32) return true;
  if (prec == PREC_FP32_SPLIT) {
    if (d->N % 128 != 0 || d->K % 64 != 0) return fail(1, "the tensor-core fp32 GEMM needs widths in multiples of 128 and depths of 64");
    if (!make_tmap_16bit_kmajor(&d->tmap, d->w, d->N, 3 * static_cast<uint64_t>(d->K), static_cast<uint64_t>(d->K) * 6,
                                gemm_split_w_box_rows(d->N)))
      return fail(2, "cuTensorMapEncodeTiled failed for a weight matrix");
    return true;
  }
  if (prec == PREC_FP8 && !fp8_widened_) {
    if (d->N % 256 != 0) return fail(1, "FP8 mode needs dense widths that are multiples of 256");
    if (!make_tmap_u8_kmajor(&d->tmap, d->w_fp8, d->N, d->K))
      return fail(2, "cuTensorMapEncodeTiled failed for an FP8 weight matrix");
    return true;
  }
  if (!make_tmap_16bit_kmajor(&d->tmap, d->w, d->N, d->K, static_cast<uint64_t>(d->K) * 2, gemm_w_box_rows(d->N)))
    return fail(2, "cuTensorMapEncodeTiled failed for a weight matrix");
  return true;
}

bool Model::load_weights(const std::string& dir) {
  std::string err;
  if (!list_npy_files(dir, &files_, &err)) return fail(3, err);
  if (files_.empty()) return fail(3, "no .npy files in " + dir);
  from_cache_ = cache_probe();
  const size_t H = H_;
  // embeddings: key pairs as in ops/embedding.cuh:12-20
  if (!upload_table({"embeddings", "word"}, 2, &word_, &vocab_rows_)) return false;
  if (!upload_table({"embeddings", "position"}, MAX_SEQ, &pos_, nullptr)) return false;
  if (!upload_table({"embeddings", "token_type"}, 2, &type_, nullptr)) return false;
  if (!upload_vec({"embeddings_LayerNorm_gamma"}, H, &emb_g_)) return false;
  if (!upload_vec({"embeddings_LayerNorm_beta"}, H, &emb_b_)) return false;
  layer_.resize(L_);
  const int lprec = (prec_ == PREC_FP32 && f32_tensor_) ? PREC_FP32_SPLIT : prec_;  // layout of the layers' dense weights
  for (int i = 0; i < L_; ++i) {
    // per-layer keys "_<i>_" + suffix, as in utils/bert.cu:17-61
    const std::string p = "_" + std::to_string(i) + "_";
    LayerWeights& lw = layer_[i];
    const char* qkv_names[3] = {"query", "key", "value"};
    for (int j = 0; j < 3; ++j) {
      const std::string s = p + "attention_self_" + qkv_names[j];
      if (!load_dense({s + "_kernel"}, {s + "_bias"}, H_, H_, &lw.qkv, j * H_, 3 * H_, lprec)) return false;
    }
    if (!finish_dense(&lw.qkv, lprec)) return false;
    if (!load_dense({p + "attention_output_dense_kernel"}, {p + "attention_output_dense_bias"}, H_, H_, &lw.attn_out,
                    0, H_, lprec) || !finish_dense(&lw.attn_out, lprec))
      return false;
    if (!upload_vec({p + "attention_output_LayerNorm_gamma"}, H, &lw.ln1_g)) return false;
    if (!upload_vec({p + "attention_output_LayerNorm_beta"}, H, &lw.ln1_b)) return false;
    if (!load_dense({p + "intermediate_dense_kernel"}, {p + "intermediate_dense_bias"}, H_, F_, &lw.ffn1, 0, F_, lprec) ||
        !finish_dense(&lw.ffn1, lprec))
      return false;
    if (!load_dense({p + "output_dense_kernel"}, {p + "output_dense_bias"}, F_, H_, &lw.ffn2, 0, H_, lprec) ||
        !finish_dense(&lw.ffn2, lprec))
      return false;
    if (!upload_vec({p + "output_LayerNorm_gamma"}, H, &lw.ln2_g)) return false;
    if (!upload_vec({p + "output_LayerNorm_beta"}, H, &lw.ln2_b)) return false;
  }
  // the pooler is needed by the encoder although name.txt does not list it (utils/bert.cu:67-69)
  // (kept in fp32 in every mode: it is 2 H^2 FLOPs per sequence and reads the fp32 residual stream)
  if (!load_dense({"pooler_dense_kernel"}, {"pooler_dense_bias"}, H_, H_, &pooler_, 0, H_, PREC_FP32)) return false;
  // optional fine-tune head (apps/finetune.py:33-34)
  if (find_file({"classifier_kernel"}) && find_file({"classifier_bias"})) {
    NpyArray k;
    if (!read_tensor({"classifier_kernel"}, 0, &k)) return false;
    if (from_cache_) {
      if (owned_.size() < cache_sizes_.size()) {  // the cache holds a head: kernel [H, C], then bias [C]
        if (!dev_alloc(reinterpret_cast<void**>(&cls_w_), 0)) return false;
        classes_ = static_cast<int>(owned_.back().bytes / (sizeof(float) * H));
        if (!upload_vec({"classifier_bias"}, classes_, &cls_b_)) return false;
      }
    } else if (k.shape.size() == 2 && k.shape[0] == H && k.shape[1] >= 1 && k.shape[1] <= MAX_CLASSES) {
      classes_ = static_cast<int>(k.shape[1]);
      if (!dev_alloc(reinterpret_cast<void**>(&cls_w_), k.numel() * sizeof(float))) return false;
      if (!check(cudaMemcpy(cls_w_, stage_f32_, k.numel() * sizeof(float), cudaMemcpyDeviceToDevice), "copy"))
        return false;
      if (!upload_vec({"classifier_bias"}, classes_, &cls_b_)) return false;
    }
  }
  if (from_cache_) {
    if (!cache_fill()) return false;
  } else if (!cache_path_.empty()) {
    cache_write();
  }
  if (stage_f32_) {
    cudaFree(stage_f32_);
    stage_f32_ = nullptr;
    stage_elems_ = 0;
  }
  return prepare_ln_fold();
}

bool Model::prepare_ln_fold() {
  // needs the 256-wide tiles of the CTA-pair GEMM for the GEMMs that write the statistics (N = H)
  if (ln_fold_ && !(gemm_uses_pairs(H_) && H_ % 256 == 0 && L_ >= 2)) ln_fold_ = false;
  if (!ln_fold_) return true;
  auto vec = [&](float** p, int n) {
    if (!check(cudaMalloc(p, static_cast<size_t>(n) * sizeof(float)), "cudaMalloc(LayerNorm vectors)")) return false;
    derived_.push_back(*p);
    return true;
  };
  for (int l = 0; l < L_; ++l) {
    LayerWeights& lw = layer_[l];
    if (!vec(&lw.c_ffn1, F_) || !vec(&lw.d_ffn1, F_)) return false;
    if (ln_fold_vectors(static_cast<const __half*>(lw.ffn1.w), lw.ln1_g, lw.ln1_b, lw.ffn1.bias, lw.c_ffn1, lw.d_ffn1, F_,
                        H_, stream_) < 0)
      return fail(2, "launch failed");
    if (l == 0) continue;
    if (!vec(&lw.c_qkv, 3 * H_) || !vec(&lw.d_qkv, 3 * H_)) return false;
    if (ln_fold_vectors(static_cast<const __half*>(lw.qkv.w), layer_[l - 1].ln2_g, layer_[l - 1].ln2_b, lw.qkv.bias,
                        lw.c_qkv, lw.d_qkv, 3 * H_, H_, stream_) < 0)
      return fail(2, "launch failed");
  }
  return check(cudaStreamSynchronize(stream_), "LayerNorm vectors");
}

// ------------------------------------------------------------------ weight cache
namespace {
constexpr char CACHE_MAGIC[8] = {'C', 'B', 'W', 'C', 'A', 'C', 'H', '2'};

uint64_t fnv1a(const std::string& s) {
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
  return h;
}
}  // namespace

bool Model::cache_probe() {
  cache_path_.clear();
  cache_sizes_.clear();
  const char* e = std::getenv("CUDABERT_WEIGHT_CACHE");
  if (!e || !*e) return false;
  cache_dir_ = e;
  // what the device-ready weights depend on: every file of the directory and how this handle lays them out
  std::string sig = "layout 2|large " + std::to_string(large_) + "|prec " + std::to_string(prec_) + "|layers " +
                    std::to_string(L_) + "|fp8 widened " + std::to_string(fp8_widened_) + "|fp32 planes " + std::to_string(f32_tensor_) + "|scale " +
                    std::to_string(W_CONTAINER_SCALE) + "\n";
  for (const std::string& f : files_) {
    struct stat st;
    if (stat((dir_ + "/" + f).c_str(), &st) != 0) return false;
    sig += f + ":" + std::to_string(static_cast<long long>(st.st_size)) + ":" +
           std::to_string(static_cast<long long>(st.st_mtim.tv_sec)) + "." + std::to_string(st.st_mtim.tv_nsec) + "\n";
  }
  cache_signature_ = sig;
  char name[64];
  std::snprintf(name, sizeof(name), "/cudabert_%016llx.weights", static_cast<unsigned long long>(fnv1a(dir_ + "\n" + sig)));
  cache_path_ = cache_dir_ + name;
  std::FILE* fp = std::fopen(cache_path_.c_str(), "rb");
  if (!fp) return false;
  bool ok = false;
  char magic[8];
  uint64_t sig_len = 0, n = 0;
  if (std::fread(magic, 1, 8, fp) == 8 && std::memcmp(magic, CACHE_MAGIC, 8) == 0 &&
      std::fread(&sig_len, sizeof(sig_len), 1, fp) == 1 && sig_len == sig.size()) {
    std::string stored(sig_len, '\0');
    if (std::fread(&stored[0], 1, sig_len, fp) == sig_len && stored == sig &&
        std::fread(&n, sizeof(n), 1, fp) == 1 && n > 0 && n < (1u << 20)) {
      std::vector<uint64_t> sizes(n);
      if (std::fread(sizes.data(), sizeof(uint64_t), n, fp) == n) {
        cache_sizes_.assign(sizes.begin(), sizes.end());
        ok = true;
      }
    }
  }
  std::fclose(fp);
  if (!ok) cache_sizes_.clear();
  return ok;
}

bool Model::cache_fill() {
  if (owned_.size() != cache_sizes_.size())
    return fail(3, "weight cache " + cache_path_ + " does not match this model: delete it");
  std::FILE* fp = std::fopen(cache_path_.c_str(), "rb");
  if (!fp) return fail(3, "cannot reopen weight cache " + cache_path_);
  const long header = 8 + 8 + static_cast<long>(cache_signature_.size()) + 8 + 8 * static_cast<long>(cache_sizes_.size());
  bool ok = std::fseek(fp, header, SEEK_SET) == 0;
  size_t biggest = 0;
  for (const Owned& o : owned_) biggest = std::max(biggest, o.bytes);
  void* host = nullptr;
  if (ok && cudaMallocHost(&host, biggest) != cudaSuccess) { ok = false; host = nullptr; }
  for (size_t i = 0; ok && i < owned_.size(); ++i) {
    ok = std::fread(host, 1, owned_[i].bytes, fp) == owned_[i].bytes &&
         cudaMemcpyAsync(owned_[i].p, host, owned_[i].bytes, cudaMemcpyHostToDevice, stream_) == cudaSuccess &&
         cudaStreamSynchronize(stream_) == cudaSuccess;
  }
  if (host) cudaFreeHost(host);
  std::fclose(fp);
  return ok || fail(3, "weight cache " + cache_path_ + " is truncated or unreadable: delete it");
}

void Model::cache_write() {
  // written under a temporary name and renamed, so that a reader never sees half a file
  const std::string tmp = cache_path_ + ".tmp" + std::to_string(static_cast<long long>(getpid()));
  std::FILE* fp = std::fopen(tmp.c_str(), "wb");
  if (!fp) return;
  const uint64_t sig_len = cache_signature_.size(), n = owned_.size();
  bool ok = std::fwrite(CACHE_MAGIC, 1, 8, fp) == 8 && std::fwrite(&sig_len, sizeof(sig_len), 1, fp) == 1 &&
            std::fwrite(cache_signature_.data(), 1, sig_len, fp) == sig_len && std::fwrite(&n, sizeof(n), 1, fp) == 1;
  size_t biggest = 0;
  for (const Owned& o : owned_) {
    const uint64_t b = o.bytes;
    ok = ok && std::fwrite(&b, sizeof(b), 1, fp) == 1;
    biggest = std::max(biggest, o.bytes);
  }
  std::vector<char> host(biggest);
  for (size_t i = 0; ok && i < owned_.size(); ++i)
    ok = cudaMemcpy(host.data(), owned_[i].p, owned_[i].bytes, cudaMemcpyDeviceToHost) == cudaSuccess &&
         std::fwrite(host.data(), 1, owned_[i].bytes, fp) == owned_[i].bytes;
  ok = (std::fclose(fp) == 0) && ok;
  if (!ok || std::rename(tmp.c_str(), cache_path_.c_str()) != 0) std::remove(tmp.c_str());
}

// ------------------------------------------------------------------ arena
bool Model::ensure_capacity(int B, int S, bool want_hidden_f32) {
  const size_t T = static_cast<size_t>(B) * S;
  if (want_hidden_f32 && packed_ && hidden_unpacked_tokens_ < T) {
    if (!check(cudaStreamSynchronize(stream_), "sync")) return false;
    drop_graphs();
    if (hidden_unpacked_) cudaFree(hidden_unpacked_);
    hidden_unpacked_ = nullptr;
    hidden_unpacked_tokens_ = 0;
    const size_t tok = std::max(T, cap_tokens_);
    if (!check(cudaMalloc(&hidden_unpacked_, tok * H_ * sizeof(float)), "cudaMalloc(hidden states)")) return false;
    hidden_unpacked_tokens_ = tok;
  }
  if (T <= cap_tokens_ && B <= cap_batch_) return true;
  if (!check(cudaStreamSynchronize(stream_), "sync before arena growth")) return false;
  drop_graphs();  // they hold addresses inside the arena that is about to be replaced
  const size_t ct = std::max(T, cap_tokens_);
  const int cbatch = std::max(B, cap_batch_);
  if (arena_) cudaFree(arena_);
  arena_ = nullptr;
  cap_tokens_ = 0;
  cap_batch_ = 0;
  const bool lowp = prec_ != PREC_FP32;
  size_t off = 0;
  auto slot = [&](size_t bytes) { const size_t o = off; off = align_up(off + bytes, 1024); return o; };
  const size_t o_ints = slot(3 * ct * sizeof(int));
  const size_t o_kv = slot(static_cast<size_t>(cbatch) * sizeof(int));
  const size_t o_rs = slot((static_cast<size_t>(cbatch) + 1) * sizeof(int));
  const size_t o_sched = slot((2 * static_cast<size_t>(cbatch) + ct / 128 + 2) * sizeof(int));  // + tile table
  const size_t o_xf = slot(ct * H_ * sizeof(float));
  const size_t o_x1f = slot(ct * H_ * sizeof(float));
  const size_t o_y = slot(ct * H_ * (lowp ? 2 : 4));
  const size_t o_xa = lowp ? slot(ct * H_ * 2) : o_xf;
  const size_t o_x1a = lowp ? slot(ct * H_ * 2) : o_x1f;
  const size_t o_ctx = slot(ct * H_ * esize_);
  const size_t o_qkv = slot(ct * 3 * H_ * esize_);
  const size_t o_z = slot(ct * F_ * esize_);
  const size_t o_st1 = ln_fold_ ? slot(ct * (H_ / 128) * 2 * sizeof(float)) : 0;
  const size_t o_st2 = ln_fold_ ? slot(ct * (H_ / 128) * 2 * sizeof(float)) : 0;
  const bool planes = !lowp && f32_tensor_;
  const size_t o_split = planes ? slot(ct * F_ * 6) : 0;  // three bf16 planes of the widest GEMM input
  const size_t o_pool = slot(static_cast<size_t>(cbatch) * H_ * sizeof(float));
  const size_t o_probs = slot(static_cast<size_t>(cbatch) * MAX_CLASSES * sizeof(float));
  if (!check(cudaMalloc(&arena_, off), "cudaMalloc(activation arena)")) return false;
  char* base = static_cast<char*>(arena_);
  ids_ = reinterpret_cast<int*>(base + o_ints);
  kv_len_ = reinterpret_cast<int*>(base + o_kv);
  row_start_ = reinterpret_cast<int*>(base + o_rs);
  att_sched_ = reinterpret_cast<int*>(base + o_sched);
  xf_ = reinterpret_cast<float*>(base + o_xf);
  x1f_ = reinterpret_cast<float*>(base + o_x1f);
  y_ = base + o_y;
  xa_ = base + o_xa; x1a_ = base + o_x1a; ctx_ = base + o_ctx; qkv_ = base + o_qkv; z_ = base + o_z;
  pooled_ = reinterpret_cast<float*>(base + o_pool);
  probs_ = reinterpret_cast<float*>(base + o_probs);
  ln_stats1_ = ln_fold_ ? reinterpret_cast<float*>(base + o_st1) : nullptr;
  ln_stats2_ = ln_fold_ ? reinterpret_cast<float*>(base + o_st2) : nullptr;
  // zero once so that tile rows beyond the live token count never hold NaN patterns
  if (!check(cudaMemsetAsync(arena_, 0, off, stream_), "cudaMemset(arena)")) return false;
  if (lowp) {
    const uint64_t rows = ct;
    bool ok = make_tmap_16bit_kmajor(&tm_x_, xa_, rows, H_, static_cast<uint64_t>(H_) * 2, 128) &&
              make_tmap_16bit_kmajor(&tm_x1_, x1a_, rows, H_, static_cast<uint64_t>(H_) * 2, 128) &&
              make_tmap_16bit_kmajor(&tm_ctx_, ctx_, rows, H_, static_cast<uint64_t>(H_) * 2, 128) &&
              make_tmap_16bit_kmajor(&tm_z_, z_, rows, F_, static_cast<uint64_t>(F_) * 2, 128) &&
              make_tmap_qkv(&tm_qkv_, qkv_, rows, H_);
    if (!ok) return fail(2, "cuTensorMapEncodeTiled failed for an activation buffer");
  }
  if (planes) {
    split_ = base + o_split;
    const uint64_t rows = ct;
    if (!make_tmap_16bit_kmajor(&tm_splitH_, split_, rows, 3 * static_cast<uint64_t>(H_), static_cast<uint64_t>(H_) * 6, 128) ||
        !make_tmap_16bit_kmajor(&tm_splitF_, split_, rows, 3 * static_cast<uint64_t>(F_), static_cast<uint64_t>(F_) * 6, 128))
      return fail(2, "cuTensorMapEncodeTiled failed for an activation buffer");
  }
  if (h_in_) cudaFreeHost(h_in_);
  if (h_out_) cudaFreeHost(h_out_);
  h_in_ = nullptr; h_out_ = nullptr;
  if (!check(cudaMallocHost(&h_in_, 3 * ct * sizeof(int)), "cudaMallocHost")) return false;
  h_out_elems_ = static_cast<size_t>(cbatch) * (H_ + MAX_CLASSES);
  if (!check(cudaMallocHost(&h_out_, h_out_elems_ * sizeof(float)), "cudaMallocHost")) return false;
  cap_tokens_ = ct;
  cap_batch_ = cbatch;
  return true;
}

// ------------------------------------------------------------------ profiling
void Model::count(int kclass, int n) {
  if (n > 0) {
    launches_ += n;
    prof_n_[kclass] += profiling_ ? n : 0;
  }
}
namespace {
const char* const kKernelClassNames[KC_COUNT] = {"embed_layernorm", "gemm_qkv",  "attention",   "gemm_attn_out", "layernorm",
                                                 "gemm_ffn1",       "gemm_ffn2", "gemm_pooler", "other"};
}  // namespace

// CUDABERT_NVTX=1: an NVTX range around every forward pass and, for passes enqueued kernel by kernel
// (not graph replays), around each kernel's launch, named after its class.  The header-only NVTX
// does nothing unless a tool is attached.
void Model::prof_begin(int kclass) {
  if (nvtx_) nvtxRangePushA(kKernelClassNames[kclass]);
  if (!profiling_) return;
  if (ev_used_ + 2 > ev_.size()) {
    for (int i = 0; i < 64; ++i) {
      cudaEvent_t e;
      cudaEventCreate(&e);
      ev_.push_back(e);
    }
  }
  ev_class_.push_back(kclass);
  cudaEventRecord(ev_[ev_used_], stream_);
}
void Model::prof_end(int) {
  if (nvtx_) nvtxRangePop();
  if (!profiling_) return;
  cudaEventRecord(ev_[ev_used_ + 1], stream_);
  ev_used_ += 2;
}
bool Model::collect_profile() {
  for (size_t p = 0; p < ev_class_.size() && 2 * p + 1 < ev_.size(); ++p) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ev_[2 * p], ev_[2 * p + 1]) == cudaSuccess) prof_ms_[ev_class_[p]] += ms;
  }
  ev_used_ = 0;
  ev_class_.clear();
  return true;
}
void Model::reset_profile() {
  for (int i = 0; i < KC_COUNT; ++i) { prof_ms_[i] = 0; prof_n_[i] = 0; }
  ev_used_ = 0;
  ev_class_.clear();
}
void Model::get_profile(int kclass, double* ms, long* launches) const {
  if (kclass < 0 || kclass >= KC_COUNT) { *ms = 0; *launches = 0; return; }
  *ms = prof_ms_[kclass];
  *launches = prof_n_[kclass];
}

// ------------------------------------------------------------------ forward
bool Model::dense(const DenseWeight& w, const void* A, const CUtensorMap* tmA, int lda, int M, void* out, int flags,
                  const void* residual, int kclass, const LnFold* ln, const float* bias) {
  GemmEpilogue epi;
  epi.flags = flags;
  epi.bias = bias ? bias : w.bias;  // a folded LayerNorm's beta W + bias takes the bias's place
  epi.residual = residual;
  if (ln) epi.ln = *ln;
  int n;
  prof_begin(kclass);
  if (prec_ == PREC_FP32 && f32_tensor_) {
    // fp32 on the tensor cores: the input's three bf16 planes, then one GEMM over 6 K (kernels.h)
    n = split_bf16x3(static_cast<const float*>(A), lda, static_cast<__nv_bfloat16*>(split_), M, w.K, m_dev_cur_, stream_);
    if (n > 0) {
      epi.flags |= EPI_OUT_F32 | EPI_SPLIT3;
      const int g = gemm_tcgen05(w.K == H_ ? &tm_splitH_ : &tm_splitF_, &w.tmap, M, w.N, w.K, out, w.N, epi, err_dev_,
                                 num_sms_, m_dev_cur_, stream_);
      n = g < 0 ? g : n + g;
    }
  } else if (prec_ == PREC_FP32) {
    n = gemm_f32(static_cast<const float*>(A), lda, static_cast<const float*>(w.w), M, w.N, w.K,
                 static_cast<float*>(out), w.N, epi, m_dev_cur_, stream_);
  } else {
    // 16-bit modes: fp16 operands and output; the weights' container scale (bf16 mode) or their
    // FP8 de-quantisation scale comes out in the epilogue
    epi.flags |= EPI_IN_F16 | ((flags & EPI_OUT_F32) ? 0 : EPI_OUT_F16);
    if (prec_ == PREC_FP8) {
      epi.flags |= EPI_COLSCALE | (fp8_widened_ ? 0 : EPI_W_FP8);
      epi.colscale = w.colscale;
    } else {
      epi.flags |= EPI_WSCALE;
    }
    n = gemm_tcgen05(tmA, &w.tmap, M, w.N, w.K, out, w.N, epi, err_dev_, num_sms_, m_dev_cur_, stream_);
  }
  prof_end(kclass);
  if (n < 0) return fail(2, "GEMM launch rejected (code " + std::to_string(n) + ")");
  count(kclass, n);
  return true;
}

bool Model::forward_device(const int* d_ids, const int* d_seg, const int* d_mask, int B, int S, bool want_hidden_f32,
                           bool want_probs) {
  if (status_ != 0) return false;
  if (B < 1 || S < 1) return fail(1, "batch size and sequence length must be positive");
  if (S > MAX_SEQ) return fail(1, "sequence length exceeds the 512 positions of the position table");
  if (static_cast<long long>(B) * S > (1ll << 24)) return fail(1, "batch * seq too large");
  if (want_probs && classes_ == 0) return fail(1, "the model directory has no classifier_kernel/bias");
  if (!check(cudaSetDevice(dev_), "cudaSetDevice")) return false;
  if (!ensure_capacity(B, S, want_hidden_f32)) return false;
  struct NvtxScope {
    bool on;
    NvtxScope(bool enabled, int b, int s) : on(enabled) {
      if (on) nvtxRangePushA(("cudabert forward " + std::to_string(b) + " x " + std::to_string(s)).c_str());
    }
    ~NvtxScope() { if (on) nvtxRangePop(); }
  } nvtx_scope(nvtx_, B, S);
  if (!graphs_enabled_ || profiling_) return enqueue_forward(d_ids, d_seg, d_mask, B, S, want_hidden_f32, want_probs);

  // The first passes with a given argument set run kernel by kernel (the very first also does every
  // one-time set-up a launcher may need); pass number GRAPH_CAPTURE_AT is captured into a CUDA graph;
  // from then on the pass is one graph launch, which takes the per-kernel launch cost off the host
  // for small batches.  A caller whose shapes rarely repeat (the engine trims every batch to its own
  // longest line) thus pays for few captures, and a full cache drops only its least recently used
  // entry.
  const GraphKey key{d_ids, d_seg, d_mask, B, S, (want_hidden_f32 ? 1 : 0) | (want_probs ? 2 : 0)};
  auto it = graphs_.find(key);
  if (it == graphs_.end()) {
    if (graphs_.size() >= GRAPH_CACHE_MAX) {
      auto lru = graphs_.begin();
      for (auto g = graphs_.begin(); g != graphs_.end(); ++g)
        if (g->second.last_use < lru->second.last_use) lru = g;
      if (lru->second.exec) {
        // the graph may still be executing: it is the stream's most recent work at the earliest
        if (!check(cudaStreamSynchronize(stream_), "sync before dropping a graph")) return false;
        cudaGraphExecDestroy(lru->second.exec);
      }
      graphs_.erase(lru);
    }
    it = graphs_.emplace(key, GraphEntry()).first;
  }
  it->second.last_use = ++graph_tick_;
  if (!it->second.exec && ++it->second.seen < GRAPH_CAPTURE_AT)
    return enqueue_forward(d_ids, d_seg, d_mask, B, S, want_hidden_f32, want_probs);
  GraphEntry& entry = it->second;
  if (!entry.exec) {
    if (cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      cudaGetLastError();
      graphs_enabled_ = false;
      return enqueue_forward(d_ids, d_seg, d_mask, B, S, want_hidden_f32, want_probs);
    }
    const bool ok = enqueue_forward(d_ids, d_seg, d_mask, B, S, want_hidden_f32, want_probs);
    cudaGraph_t graph = nullptr;
    const cudaError_t e_end = cudaStreamEndCapture(stream_, &graph);
    if (!ok) {  // the same rejection a direct enqueue would have met; status_ says why
      if (graph) cudaGraphDestroy(graph);
      return false;
    }
    cudaGraphExec_t exec = nullptr;
    if (e_end != cudaSuccess || !graph || cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) {
      cudaGetLastError();
      if (graph) cudaGraphDestroy(graph);
      graphs_enabled_ = false;  // this driver does not take the capture: stay with direct launches
      return enqueue_forward(d_ids, d_seg, d_mask, B, S, want_hidden_f32, want_probs);
    }
    cudaGraphDestroy(graph);
    entry.exec = exec;
    entry.launches = launches_;
    ++graph_captures_;
  }
  launches_ = entry.launches;
  ++graph_replays_;
  return check(cudaGraphLaunch(entry.exec, stream_), "cudaGraphLaunch");
}

bool Model::enqueue_forward(const int* d_ids, const int* d_seg, const int* d_mask, int B, int S, bool want_hidden_f32,
                            bool want_probs) {
  const int T = B * S;
  launches_ = 0;
  int n;
  // programmatic dependent launch pays for short passes only (kernels.h: pdl_enabled)
  struct PdlScope {
    explicit PdlScope(bool on) { tl_pdl_allowed = on; }
    ~PdlScope() { tl_pdl_allowed = true; }
  } pdl_scope(T <= PDL_MAX_TOKENS);

#define CB_LAUNCH(kclass, call)                                         \
  do {                                                                  \
    prof_begin(kclass);                                                 \
    n = (call);                                                         \
    prof_end(kclass);                                                   \
    if (n < 0) return fail(2, "kernel launch rejected: " #call);        \
    count(kclass, n);                                                   \
  } while (0)

  m_dev_cur_ = packed_ ? row_start_ + B : nullptr;
  const int* rs = packed_ ? row_start_ : nullptr;          // first row of every sequence
  const int* live = packed_ ? row_start_ + B : nullptr;     // live row count (device)
  const bool lowp = prec_ != PREC_FP32;
  const int att_kernel = lowp ? attention_kernel_for(S) : ATT_KERNEL_MMA;
  int* sched = att_kernel != ATT_KERNEL_MMA ? att_sched_ : nullptr;  // work order and mask flags
  CB_LAUNCH(KC_OTHER, row_layout(d_mask, kv_len_, packed_ ? row_start_ : nullptr, sched, B, S, stream_));
  __half* xa = static_cast<__half*>(xa_);
  __half* x1a = static_cast<__half*>(x1a_);
  if (lowp) {
    CB_LAUNCH(KC_EMBED, embed_layernorm<__half>(d_ids, d_seg, word_, pos_, type_, emb_g_, emb_b_, xa, xf_, T, S,
                                                       H_, vocab_rows_, err_dev_, rs, stream_));
  } else {
    CB_LAUNCH(KC_EMBED, embed_layernorm<float>(d_ids, d_seg, word_, pos_, type_, emb_g_, emb_b_, xf_, nullptr, T, S, H_,
                                               vocab_rows_, err_dev_, rs, stream_));
  }
  bool compact_out = false;  // the final hidden states hold one row per sequence (rows [0, B))
  // Folded LayerNorms (LnFold): in layers 0 .. L-2 the first LayerNorm, in layers 0 .. L-3 the second one
  // are not run as kernels.  The last layer runs unfolded (it may work on the first tokens only and
  // ends in hidden states the pooler reads), so the layer before it ends in an ordinary LayerNorm.
  const bool fold = lowp && ln_fold_;
  for (int l = 0; l < L_; ++l) {
    const LayerWeights& w = layer_[l];
    const bool fold1 = fold && l <= L_ - 2, fold2 = fold && l <= L_ - 3;
    const bool in_folded = fold && l >= 1 && l - 1 <= L_ - 3;  // this layer's input is LN(sum) with sum in xf_, sum * gamma in xa_
    if (in_folded) {
      LnFold f;
      f.stats_in = ln_stats2_;
      f.c = w.c_qkv;
      if (!dense(w.qkv, xa_, &tm_x_, H_, T, qkv_, EPI_BIAS | EPI_LN_APPLY, nullptr, KC_GEMM_QKV, &f, w.d_qkv)) return false;
    } else if (!dense(w.qkv, xa_, &tm_x_, H_, T, qkv_, EPI_BIAS, nullptr, KC_GEMM_QKV)) {
      return false;
    }
    if (lowp) {
      // The pooler reads the first token of every sequence only.  When nothing else of the final
      // hidden states is wanted, the LAST layer therefore computes, after its K and V, only that
      // token: attention for the first query, then the rest of the layer on B rows written compactly
      // into rows [0, B) of the same buffers.  Every step is row-wise (or, in attention, per query),
      // so the pooler output has the same bits as after a full last layer.
      const int cls = (cls_last_ && !want_hidden_f32 && l == L_ - 1) ? 1 : 0;
      if (att_kernel == ATT_KERNEL_TC) {
        CB_LAUNCH(KC_ATTENTION, attention_f16_tc(&tm_qkv_, d_mask, kv_len_, rs, sched, static_cast<__half*>(ctx_), B,
                                                 S, heads_, num_sms_, cls, err_dev_, stream_));
      } else if (att_kernel == ATT_KERNEL_PERSIST) {
        CB_LAUNCH(KC_ATTENTION, attention_f16_persist(&tm_qkv_, d_mask, kv_len_, rs, sched,
                                                       static_cast<__half*>(ctx_), B, S, heads_, num_sms_, cls,
                                                       err_dev_, stream_));
      } else {
        CB_LAUNCH(KC_ATTENTION, attention_f16(static_cast<const __half*>(qkv_), d_mask, kv_len_, rs,
                                               static_cast<__half*>(ctx_), B, S, heads_, cls, stream_));
      }
      const int rows = cls ? B : T;               // rows the rest of the layer works on
      const int* rows_live = cls ? nullptr : live;  // ... all of them live in the compact case
      if (cls) m_dev_cur_ = nullptr;
      if (fold1) {
        // s1 = ctx.Wo + bo + x in fp32 -> x1f_, s1 * gamma1 in fp16 -> x1a_, row statistics -> ln_stats1_;
        // x is the materialised input (xf_) or LN(previous sum) recomputed from it
        LnFold f;
        f.out16 = x1a_;
        f.gamma = w.ln1_g;
        f.stats_out = ln_stats1_;
        int fl = EPI_BIAS | EPI_OUT_F32 | EPI_RESIDUAL | EPI_LN_SUM;
        if (in_folded) {
          fl |= EPI_RES_LN;
          f.res_stats = ln_stats2_;
          f.res_gamma = layer_[l - 1].ln2_g;
          f.res_beta = layer_[l - 1].ln2_b;
        }
        if (!dense(w.attn_out, ctx_, &tm_ctx_, H_, rows, x1f_, fl, xf_, KC_GEMM_ATTN_OUT, &f)) return false;
        // FFN1 normalises in its epilogue
        LnFold g;
        g.stats_in = ln_stats1_;
        g.c = w.c_ffn1;
        if (!dense(w.ffn1, x1a_, &tm_x1_, H_, rows, z_, EPI_BIAS | EPI_GELU | EPI_LN_APPLY, nullptr, KC_GEMM_FFN1, &g, w.d_ffn1))
          return false;
        // s2 = z.W2 + b2 + LN1(s1), the residual recomputed from s1 and its statistics
        LnFold h;
        h.res_stats = ln_stats1_;
        h.res_gamma = w.ln1_g;
        h.res_beta = w.ln1_b;
        if (fold2) {  // -> xf_ (fp32), s2 * gamma2 -> xa_, statistics -> ln_stats2_: the next layer's folded input
          h.out16 = xa_;
          h.gamma = w.ln2_g;
          h.stats_out = ln_stats2_;
          if (!dense(w.ffn2, z_, &tm_z_, F_, rows, xf_, EPI_BIAS | EPI_OUT_F32 | EPI_RESIDUAL | EPI_RES_LN | EPI_LN_SUM, x1f_,
                     KC_GEMM_FFN2, &h))
            return false;
        } else {      // the layer before the last: s2 in fp32 -> xf_, then an ordinary LayerNorm over it, in place
          if (!dense(w.ffn2, z_, &tm_z_, F_, rows, xf_, EPI_BIAS | EPI_OUT_F32 | EPI_RESIDUAL | EPI_RES_LN, x1f_, KC_GEMM_FFN2, &h))
            return false;
          CB_LAUNCH(KC_LAYERNORM, (layernorm<float, __half>(xf_, nullptr, w.ln2_g, w.ln2_b, xa, xf_, rows, H_, rows_live,
                                                            stream_)));
        }
        compact_out = false;
        continue;
      }
      // y = ctx.Wo + bo in fp16; x1 = LN(y + x) with the add in fp32 inside the LayerNorm kernel
      if (!dense(w.attn_out, ctx_, &tm_ctx_, H_, rows, y_, EPI_BIAS, nullptr, KC_GEMM_ATTN_OUT))
        return false;
      // compact case: the residual of output row b is the first row of sequence b
      CB_LAUNCH(KC_LAYERNORM, (layernorm<__half, __half>(static_cast<const __half*>(y_), xf_, w.ln1_g, w.ln1_b,
                                                                x1a, x1f_, rows, H_, rows_live, stream_,
                                                                cls ? rs : nullptr, (cls && !rs) ? S : 1)));
      if (!dense(w.ffn1, x1a_, &tm_x1_, H_, rows, z_, EPI_BIAS | EPI_GELU, nullptr, KC_GEMM_FFN1)) return false;
      if (!dense(w.ffn2, z_, &tm_z_, F_, rows, y_, EPI_BIAS, nullptr, KC_GEMM_FFN2)) return false;
      CB_LAUNCH(KC_LAYERNORM, (layernorm<__half, __half>(static_cast<const __half*>(y_), x1f_, w.ln2_g, w.ln2_b,
                                                                xa, xf_, rows, H_, rows_live, stream_)));
      compact_out = cls != 0;
    } else {
      CB_LAUNCH(KC_ATTENTION, attention_f32(static_cast<const float*>(qkv_), d_mask, kv_len_, rs,
                                            static_cast<float*>(ctx_), B, S, heads_, stream_));
      // fp32 mode: the GEMM epilogue adds the residual, y = ctx.Wo + bo + x
      if (!dense(w.attn_out, ctx_, nullptr, H_, T, y_, EPI_BIAS | EPI_RESIDUAL, xf_, KC_GEMM_ATTN_OUT)) return false;
      CB_LAUNCH(KC_LAYERNORM, (layernorm<float, float>(static_cast<const float*>(y_), nullptr, w.ln1_g, w.ln1_b, x1f_,
                                                       nullptr, T, H_, live, stream_)));
      if (!dense(w.ffn1, x1a_, nullptr, H_, T, z_, EPI_BIAS | EPI_GELU, nullptr, KC_GEMM_FFN1)) return false;
      if (!dense(w.ffn2, z_, nullptr, F_, T, y_, EPI_BIAS | EPI_RESIDUAL, x1f_, KC_GEMM_FFN2)) return false;
      CB_LAUNCH(KC_LAYERNORM, (layernorm<float, float>(static_cast<const float*>(y_), nullptr, w.ln2_g, w.ln2_b, xf_,
                                                       nullptr, T, H_, live, stream_)));
    }
  }
  // pooler: rows b*S of the fp32 final hidden states, tanh(dense) -> fp32 [B, H]
  // (utils/bert.cu:239-247); always the fp32 kernel, it is 2 H^2 FLOPs per sequence
  CB_LAUNCH(KC_POOLER, pooler_f32(xf_, compact_out ? 1 : S, compact_out ? nullptr : rs,
                                  static_cast<const float*>(pooler_.w), pooler_.bias, pooled_, B, H_, stream_));
  if (want_hidden_f32 && packed_)
    CB_LAUNCH(KC_OTHER, unpack_rows(xf_, row_start_, hidden_unpacked_, T, S, H_, stream_));
  if (want_probs)
    CB_LAUNCH(KC_OTHER, classify_softmax(pooled_, cls_w_, cls_b_, probs_, B, H_, classes_, stream_));
#undef CB_LAUNCH
  return true;
}

bool Model::sync() {
  if (!check(cudaSetDevice(dev_), "cudaSetDevice")) return false;
  if (!check(cudaMemcpyAsync(h_err_, err_dev_, sizeof(int), cudaMemcpyDeviceToHost, stream_), "error flag copy"))
    return false;
  if (!check(cudaStreamSynchronize(stream_), "stream synchronize")) return false;
  if (profiling_) collect_profile();
  if (*h_err_ != 0) {
    const int e = *h_err_;
    cudaMemsetAsync(err_dev_, 0, sizeof(int), stream_);
    if (e & 1)
      return fail(4, "a device-side wait in the GEMM pipeline timed out (site " + std::to_string(e >> 8) +
                         "); results of this call are invalid");
    return fail(4, "input ids or segment ids out of range (clamped); results of this call are suspect");
  }
  return true;
}

int Model::probe_wait_timeout(unsigned long long limit_ns) {
  if (!check(cudaSetDevice(dev_), "cudaSetDevice")) return status_;
  if (wait_timeout_probe(err_dev_, limit_ns, stream_) < 0) {
    fail(1, "wait probe: the limit must be between 1 ns and 2 s");
    return status_;
  }
  sync();
  return status_;
}

bool Model::run_host(const int* ids, const int* seg, const int* mask, int B, int S, float* pooled_out,
                     float* probs_out, int num_classes, bool want_hidden_f32) {
  if (status_ != 0) return false;
  if (!ids || !seg) return fail(1, "ids and segment ids must not be null");
  if (B < 1 || S < 1 || S > MAX_SEQ) return fail(1, "need batch >= 1 and 1 <= seq_length <= 512");
  if (probs_out && num_classes != classes_) return fail(1, "num_classes does not match classifier_kernel");
  if (!check(cudaSetDevice(dev_), "cudaSetDevice")) return false;
  if (!ensure_capacity(B, S, want_hidden_f32)) return false;
  const size_t T = static_cast<size_t>(B) * S;
  std::memcpy(h_in_, ids, T * sizeof(int));
  std::memcpy(h_in_ + T, seg, T * sizeof(int));
  if (mask) std::memcpy(h_in_ + 2 * T, mask, T * sizeof(int));
  if (!check(cudaMemcpyAsync(ids_, h_in_, (mask ? 3 : 2) * T * sizeof(int), cudaMemcpyHostToDevice, stream_),
             "input copy"))
    return false;
  if (!forward_device(ids_, ids_ + T, mask ? ids_ + 2 * T : nullptr, B, S, want_hidden_f32, probs_out != nullptr))
    return false;
  const size_t nh = static_cast<size_t>(B) * H_;
  if (pooled_out &&
      !check(cudaMemcpyAsync(h_out_, pooled_, nh * sizeof(float), cudaMemcpyDeviceToHost, stream_), "output copy"))
    return false;
  if (probs_out && !check(cudaMemcpyAsync(h_out_ + nh, probs_, static_cast<size_t>(B) * classes_ * sizeof(float),
                                          cudaMemcpyDeviceToHost, stream_), "output copy"))
    return false;
  if (!sync()) return false;
  if (pooled_out) std::memcpy(pooled_out, h_out_, nh * sizeof(float));
  if (probs_out) std::memcpy(probs_out, h_out_ + nh, static_cast<size_t>(B) * classes_ * sizeof(float));
  return true;
}

}  // namespace cb
