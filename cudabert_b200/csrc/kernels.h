// Host-side launchers of the hot-path kernels.  Every launcher enqueues on `stream`, never
// synchronises, never allocates, and returns the number of kernels it launched (>= 1) or a
// negative value when the arguments are rejected.
#pragma once
#include <cstdint>
#include <string>
#include <cstdlib>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace cb {

// Launch `kernel` so that it may start while the previous kernel of the stream is still draining
// (programmatic dependent launch).  Every kernel launched this way executes griddep_wait() before
// it reads or writes anything a predecessor produces or still reads; until then it only does work
// that is private to it (barrier set-up, TMEM allocation, descriptor prefetch).
// Whether launch_pdl asks for programmatic dependent launch.  Measured: it shortens a forward pass
// of a few thousand tokens (BERT-base, 8 x 128: 0.86 against 0.94 ms) and costs about 1 % on one of
// 25 600 tokens, so the forward pass switches it per call (`tl_pdl_allowed`); CUDABERT_PDL=0 turns it
// off everywhere, CUDABERT_PDL=1 on everywhere.
inline thread_local bool tl_pdl_allowed = true;
inline bool pdl_enabled() {
  static const int forced = [] {
    const char* e = std::getenv("CUDABERT_PDL");
    return !e || !*e ? -1 : (e[0] == '0' ? 0 : 1);
  }();
  return forced >= 0 ? forced == 1 : tl_pdl_allowed;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_plain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Epilogue selection, shared by the tcgen05 and the fp32 GEMM:
//   out = act( acc * colscale[n] + bias[n] + residual[m, n] )
enum EpiFlags : int {
  EPI_BIAS = 1,      // add bias[n] (fp32)
  EPI_GELU = 2,      // erf GELU (reference: ops/elementwise.cu:38-42)
  EPI_RESIDUAL = 4,  // add residual[m, n] (same element type and row stride as out)
  EPI_TANH = 8,      // tanh (pooler, reference: ops/elementwise.cu:57-61)
  EPI_OUT_F32 = 16,  // write fp32 instead of bf16 (tcgen05 GEMM only; the fp32 GEMM always does)
  EPI_COLSCALE = 32, // multiply the accumulator by colscale[n] (FP8 weight de-quantisation)
  EPI_OUT_F16 = 64,  // write fp16 instead of bf16 (tcgen05 GEMM only)
  EPI_WSCALE = 128,  // multiply the accumulator by 1 / W_CONTAINER_SCALE (weights held as scaled fp16, below)
  EPI_IN_F16 = 256,  // A and W are fp16 (tcgen05 GEMM only; bf16 otherwise)
  EPI_W_FP8 = 512,   // W is E4M3 bytes [N, K] (map from make_tmap_u8_kmajor), widened to fp16 inside the
                     // kernel; needs EPI_IN_F16 and N % 256 == 0
  EPI_SPLIT3 = 1024, // fp32 product on the tensor cores: A [M, 3 K] and W [N, 3 K] each hold three bf16 planes
                     // side by side (see split_bf16x3); the kernel sums the six leading cross terms over K
  EPI_LN_SUM = 2048,   // this GEMM's output is the input of a LayerNorm that is not run as a kernel (LnFold below)
  EPI_LN_APPLY = 4096, // this GEMM's A operand is such an input, times gamma: normalise in the epilogue
  EPI_RES_LN = 8192    // the residual is LayerNorm(residual) of such an input: recompute it
};

// LayerNorm folded into the GEMMs on either side of it.  With s the LayerNorm's input (a GEMM's
// accumulator + bias + residual) and mu_r, rstd_r its row statistics,
//   LN(s) W + b = rstd_r ((s * gamma) W - mu_r (gamma W)) + (beta W + b).
// The GEMM that produces s (EPI_LN_SUM; CTA-pair kernel, N % 256 == 0) writes s in fp32 (`out`, it is the
// residual stream), s * gamma in fp16 (`out16`, the next GEMM's A operand) and, per row and 128-column
// slice, the partial sum and sum of squares of s (`stats_out`, float2 [M][N / 128]).  The GEMM that consumes
// it (EPI_LN_APPLY) adds the partials of a row in slice order (deterministic), and applies the two row
// scalars with the vectors c = gamma W and d = beta W + b (d is passed as the bias).  Where the
// residual of a producing GEMM is itself LN(s') of an earlier such input (EPI_RES_LN), it is recomputed
// from s' (`residual`, fp32), its partials and its gamma, beta.
struct LnFold {
  const float* stats_in = nullptr;   // EPI_LN_APPLY: partials of the rows of A's LayerNorm input, [M][K / 128] float2
  const float* c = nullptr;          // EPI_LN_APPLY: gamma W, [N]
  void* out16 = nullptr;             // EPI_LN_SUM: fp16 [M][N], s * gamma
  const float* gamma = nullptr;      // EPI_LN_SUM: [N]
  float* stats_out = nullptr;        // EPI_LN_SUM: [M][N / 128] float2
  const float* res_stats = nullptr;  // EPI_RES_LN: partials of the residual's LayerNorm input, [M][N / 128] float2
  const float* res_gamma = nullptr;  // EPI_RES_LN: [N]
  const float* res_beta = nullptr;   // EPI_RES_LN: [N]
};
constexpr float LN_EPS_F = 1e-12f;

// fp32 on the 16-bit tensor-core path.  An fp32 number is the sum of three bf16 numbers, x = x0 + x1 +
// x2 with x0 = bf16(x), x1 = bf16(x - x0), x2 = bf16(x - x0 - x1) (the subtractions are exact; bf16 has
// fp32's exponent range, so nothing needs scaling); what is left is below 2^-24 |x|.  A product of two
// bf16 numbers is exact in the tensor core's fp32 accumulator, so
//   a . w = a2 w0 + a0 w2 + a1 w1 + a1 w0 + a0 w1 + a0 w0  (+ terms below 2^-24 |a| |w|, dropped)
// is a GEMM over 6 K with bf16 operands and fp32 accumulation, the small terms first.

// The encoder's dense weights are ROUNDED to bf16 (8 significand bits: the weight format of the bf16
// mode) and HELD as fp16 numbers, multiplied by this power of two so that even the smallest of them
// stay above fp16's subnormal range: every bf16 value of magnitude 2^-37 .. 15.9 is represented
// exactly.  Both MMA operands are then fp16, so the activations keep 11 significand bits instead
// of bf16's 8; the epilogue takes the factor out again (EPI_WSCALE).
constexpr float W_CONTAINER_SCALE = 4096.0f;

struct GemmEpilogue {
  int flags = 0;
  const float* bias = nullptr;
  const void* residual = nullptr;
  const float* colscale = nullptr;
  LnFold ln;
};

// ---- tcgen05 GEMM: out[M, N] = A[M, K] (K contiguous) x W[N, K]^T (K contiguous), both bf16, or both
// fp16 with EPI_IN_F16
// N must be a multiple of 128 and K of 64; M is arbitrary (tail rows are zero-filled by TMA
// and never stored).  `tmA` / `tmW` are tiled tensor maps made by make_tmap_16bit_kmajor with
// box rows 128 (A) and gemm_w_box_rows(N) (W).
// m_dev (device int, may be null): the live row count; the kernel then computes rows
// [0, min(M, *m_dev)) while the launch is sized for M.
int gemm_tcgen05(const CUtensorMap* tmA, const CUtensorMap* tmW, int M, int N, int K, void* out, int ldo,
                      const GemmEpilogue& epi, int* err_flag, int num_sms, const int* m_dev, cudaStream_t stream);
int gemm_block_n(int N);
// Launches one thread that runs the pipelines' bounded mbarrier wait on a barrier nobody arrives on,
// with a limit of `limit_ns` (<= the pipelines' own 2 s): after the limit it sets bit 0 of *err_flag
// (and the wait site in bits 8..) and the kernel ends.  For testing the host side of a time-out.
int wait_timeout_probe(int* err_flag, unsigned long long limit_ns, cudaStream_t stream);
// Box rows the W tensor map must be encoded with for the kernel variant that gemm_tcgen05
// will pick for this N (128 when CTA pairs each load half of a 256-row tile, else gemm_block_n).
int gemm_w_box_rows(int N);
bool gemm_uses_pairs(int N);  // the CTA-pair kernel (256 x 256 tiles) serves this width
// The same for the W operand of an EPI_SPLIT3 GEMM ([N, 3 K] bf16 planes): CTA pairs with 256 x 256
// tiles for N > 1024, single CTAs with 128 x 128 tiles otherwise.
int gemm_split_block_n(int N);
int gemm_split_w_box_rows(int N);
// Encode a 2-D tiled map over a row-major matrix of 16-bit elements [rows, cols] with
// `row_stride_bytes` between rows, box = 64 columns (128 bytes, 128-byte swizzle) x `box_rows` rows.
bool make_tmap_16bit_kmajor(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                           uint64_t row_stride_bytes, uint32_t box_rows);

// Map over a row-major matrix of bytes [rows, cols] (the E4M3 weights of the FP8 mode), box = 64 bytes x
// 128 rows, no swizzle.
bool make_tmap_u8_kmajor(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols);

// ---- fp32 CUDA-core GEMM: out[M, N] = A[M, K] (fp32, row stride lda) x W[K, N] (fp32, the
// on-disk [in, out] layout).  N % 4 == 0, K % 4 == 0.
int gemm_f32(const float* A, int lda, const float* W, int M, int N, int K, float* out, int ldo,
             const GemmEpilogue& epi, const int* m_dev, cudaStream_t stream);

// Pooler: out[b, :] = tanh(x[row(b)] . W[H, H] + bias[H]) in fp32; H % 64 == 0.  row(b) = b * rows_per_seq,
// or row_start[b] when row_start != null (packed layout).
int pooler_f32(const float* x, int rows_per_seq, const int* row_start, const float* W, const float* bias, float* out,
               int B, int H, cudaStream_t stream);

// ---- masked attention.  qkv is [rows, 3H] (Q | K | V column blocks, head h at columns h*64; fp16 for
// the 16-bit kernels, fp32 for attention_f32), ctx is [rows, H] (fp16 / fp32).  kv_len[b] > 0: keys >= kv_len[b] are all masked and are skipped; the
// int32 key mask [B, S] (may be null) is applied to the keys below kv_len.  kv_len[b] == 0: the row
// has no valid key, every key gets the same -10000 so the mask is ignored (softmax is shift
// invariant) and the row counts as S long.  Head size is 64.
// row_start == null: sequence b occupies rows [b*S, (b+1)*S) (padded layout).  row_start != null
// (B + 1 entries from row_layout): sequences are packed back to back, sequence b occupies rows
// [row_start[b], row_start[b+1]) and has no rows for its padding.
// cls_only != 0 (the three 16-bit kernels): only the first query of every sequence is computed and its
// result is written to row b of ctx ([B, H]) -- what the last encoder layer needs when only the
// pooler output is wanted; the arithmetic of that row is the same as in a full pass.
int attention_f16(const __half* qkv, const int* mask, const int* kv_len, const int* row_start,
                   __half* ctx, int B, int S, int heads, int cls_only, cudaStream_t stream);
int attention_f32(const float* qkv, const int* mask, const int* kv_len, const int* row_start, float* ctx, int B,
                  int S, int heads, cudaStream_t stream);
// tcgen05 variant of attention_f16 (attention_tc.cu): Q, K, V tiles arrive by TMA through `tm_qkv`,
// a map over the [rows, 3H] projection output made by make_tmap_qkv.  attention_kernel_for says which
// 16-bit kernel a forward pass of padded length S takes (CUDABERT_ATTENTION=tc|persist|mma forces one).
// Persistent variant of attention_f16 (one CTA per SM, TMA-fed K/V slots, query blocks drawn
// dynamically).  `sched` (2 B entries from row_layout, may be null) orders the items by descending
// length and says which rows need their mask read; S <= 256.
bool attention_persist_fits(int S);
int attention_f16_persist(const CUtensorMap* tm_qkv, const int* mask, const int* kv_len, const int* row_start,
                           const int* sched, __half* ctx, int B, int S, int heads, int num_sms, int cls_only,
                           int* err_flag, cudaStream_t stream);
enum AttentionKernel : int { ATT_KERNEL_MMA = 1, ATT_KERNEL_TC = 2, ATT_KERNEL_PERSIST = 3 };
int attention_kernel_for(int S);
bool make_tmap_qkv(CUtensorMap* out, const void* qkv, uint64_t rows, int H);
// `sched` (from row_layout, may be null): its mask flags say which rows need their mask read; with
// row_start as well it holds the tile table (sched[2 B + t] = sequence of packed row 128 t), and the
// kernel then cuts the packed rows into 128-row tiles across sequences where that pays (padded lengths
// that would leave a sequence's last tile under 85 % full), with the same bits as per-sequence tiles.
int attention_f16_tc(const CUtensorMap* tm_qkv, const int* mask, const int* kv_len, const int* row_start,
                     const int* sched, __half* ctx, int B, int S, int heads, int num_sms, int cls_only, int* err_flag,
                     cudaStream_t stream);
// kv_len[b] = 1 + index of the last non-zero mask entry of row b (0 if none); mask null => S.
// row_start (may be null): exclusive prefix sum of the sequence lengths (a length of 0 counts as S),
// B + 1 entries, the last one being the number of packed rows.  sched (may be null): 2 B entries (work
// order by descending length; mask flags), followed, when row_start is given, by ceil(B S / 128) entries
// of the tile table.
int row_layout(const int* mask, int* kv_len, int* row_start, int* sched, int B, int S, cudaStream_t stream);

// ---- row-wise kernels.  The residual stream is kept in fp32; TOut (float or __half) is
// the copy that feeds the next GEMM.  out_f32 (may be null) receives the same values in fp32.
// out[row(t)] = LayerNorm(word[ids[t]] + pos[t % S] + type[seg[t]]) for t < tokens = B*S; err bit 1
// set on a bad id.  row_start == null: row(t) = t.  Packed (row_start from row_layout): token
// (b, s) goes to row row_start[b] + s, tokens beyond a sequence's length are skipped.
template <typename TOut>
int embed_layernorm(const int* ids, const int* seg, const float* word, const float* pos, const float* type,
                    const float* gamma, const float* beta, TOut* out, float* out_f32, int tokens, int S, int H,
                    int vocab, int* err_flag, const int* row_start, cudaStream_t stream);
// out[t] = LayerNorm(x[t] + residual[t]) * gamma + beta; x is fp32 or fp16 (the tensor-core GEMM's
// dense output), residual (may be null) is the fp32 residual stream.  Rows t < min(tokens, *rows_dev)
// (rows_dev: device int, may be null) are processed.
template <typename TIn, typename TOut>
int layernorm(const TIn* x, const float* residual, const float* gamma, const float* beta, TOut* out, float* out_f32,
              int tokens, int H, const int* rows_dev, cudaStream_t stream, const int* res_rows = nullptr,
              int res_stride = 1);
// dst[B*S, H] (fp32) = packed src rows scattered back to the padded layout, zeros for padding.
int unpack_rows(const float* src, const int* row_start, float* dst, int tokens, int S, int H, cudaStream_t stream);
// probs[b, :] = softmax(pooled[b, :] . W[H, C] + bias[C]),  C <= 32
int classify_softmax(const float* pooled, const float* W, const float* bias, float* probs, int B, int H, int C,
                     cudaStream_t stream);

// ---- weight preparation (load time)
// dst[n, k] = bf16-rounded src[k, n] held as fp16 x W_CONTAINER_SCALE (on-disk [in, out] -> K-contiguous
// [out, in]); dst row offset lets Q, K, V be packed into one [3H, H] operand.
int transpose_round_bf16(const float* src, __half* dst, int K, int N, cudaStream_t stream);
// FP8 weights: q[n, k] = e4m3(src[k, n] / scale), written as bytes to dst_q (what the GEMM reads with
// EPI_W_FP8) and / or widened exactly to fp16 to dst_wide (either may be null); scale = maxabs / 448 is
// computed on the device and written to *scale_out.
int quantize_fp8_weight(const float* src, uint8_t* dst_q, __half* dst_wide, float* scale_out, int K, int N,
                        cudaStream_t stream);
int fill_f32(float* dst, float value, size_t n, cudaStream_t stream);
// LnFold's vectors for the GEMM with bf16-mode weights w ([N, K], fp16 container) that follows a LayerNorm
// with gamma, beta: c = gamma W, d = beta W + bias.
int ln_fold_vectors(const __half* w, const float* gamma, const float* beta, const float* bias, float* c, float* d, int N,
                    int K, cudaStream_t stream);
// The three bf16 planes of an fp32 weight matrix, K-contiguous: dst[n, p K + k] = plane p of src[k, n]
// (dst rows of 3 K elements; the row offset lets Q, K, V be packed into one operand).
int transpose_split_bf16x3(const float* src, __nv_bfloat16* dst, int K, int N, cudaStream_t stream);
// The three bf16 planes of fp32 activations: dst[m, p K + k] = plane p of src[m * lds + k] for the
// first `rows` rows (at most *rows_dev of them when rows_dev is given).
int split_bf16x3(const float* src, int lds, __nv_bfloat16* dst, int rows, int K, const int* rows_dev,
                 cudaStream_t stream);

// Message that cudabert_last_error(NULL) returns on the calling thread.
void set_thread_error(const std::string& msg);

}  // namespace cb
