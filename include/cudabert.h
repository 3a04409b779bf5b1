/* C ABI of libcudaBERT.so -- a B200 (sm_100a) BERT-encoder inference backend that is a drop-in
 * for the shared library of qsyao/cudaBERT.  The first five entry points have the reference's
 * names, argument order and meaning, so the reference's ctypes binding (cuda_bert/pybert.py:12-38)
 * and its unit_test program (cuda_bert/test/test.cpp) work against this library unchanged.
 *
 * All array arguments are caller-owned, C-contiguous host memory unless a name says "_dev".
 * No entry point terminates the process: failures are recorded on the handle
 * (cudabert_status / cudabert_last_error); init_model returns NULL on failure.
 * A handle is not re-entrant; distinct handles (one per GPU) may be used from distinct threads.
 */
#ifndef CUDABERT_H_
#define CUDABERT_H_

#include <stdbool.h>
#include <stddef.h>

#if defined(__GNUC__)
#define CUDABERT_API __attribute__((visibility("default")))
#else
#define CUDABERT_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Reference: `Retval` (cuda_bert/utils/common.h:174-177).  Both fields are DEVICE pointers
 * (fp32) owned by the handle and valid until its next call:
 *   tensor         final hidden states [batch, seq, hidden]
 *   pooled_output  pooler output       [batch, hidden]                                   */
typedef struct Retval {
  float* tensor;
  float* pooled_output;
} Retval;

/* Reference: init_model (cuda_bert/cuda_bert.cu:26-33; ctypes cuda_bert/pybert.py:14-16).
 * `large` picks the hard-coded dimensions (base 12/768/12/3072, large 24/1024/16/4096,
 * utils/manager.cu:8-15); `dir` is a directory of float32 .npy files (name.txt layout), "" means
 * "model_npy/base_uncased" or "model_npy/large_uncased"; max_batchsize == max_seq_length == 0
 * sizes the activation arena lazily at the first call.  The precision mode comes from the
 * environment variable CUDABERT_PRECISION = fp32 | bf16 (default) | fp8.  bf16: dense weights
 * rounded to bf16, activations between kernels in fp16, fp32 accumulation, fp32 residual stream.
 * fp8: the same with the dense weights quantised to E4M3 with one scale per tensor.           */
CUDABERT_API void* init_model(bool large, int num_gpu, int max_batchsize, int max_seq_length, char* dir);

/* Reference: release_model (cuda_bert/cuda_bert.cu:34-37). */
CUDABERT_API void release_model(void* model);

/* Reference: Cuda_Inference (cuda_bert/cuda_bert.cu:40-53).  Runs the forward pass on host
 * int32 arrays [batchsize, seq_length] (`masks` may be NULL = all valid) and returns device
 * pointers; the call returns after the work has been enqueued AND completed.              */
CUDABERT_API Retval Cuda_Inference(void* model, int* words, int* token_types, int batchsize, int seq_length, int* masks);

/* Reference: Cuda_Bert (cuda_bert/cuda_bert.cu:55-70).  Forward pass + copy of the pooler
 * output into `output` (host fp32 [batchsize, hidden]); blocking.  On failure `output` is
 * left untouched and the handle's status is set.                                           */
CUDABERT_API void Cuda_Bert(void* model, float* output, int* words, int* token_types, int batchsize, int seq_length,
               int* attention_mask);

/* Reference: test (cuda_bert/cuda_bert.cu:91-180, cuda_bert/cuda_bert.cuh:4-5).  Built-in
 * latency / throughput loop on the reference's 11-token seed input tiled to seq_length:
 * 10 warm-up calls, nIter timed calls, prints the p99 latency and batches per second.       */
CUDABERT_API void test(int batchsize, int seq_length, int nIter, bool large, int num_gpu);

/* Reference: Cuda_Classify, present but commented out (cuda_bert/cuda_bert.cu:72-89,
 * cuda_bert/pybert.py:40-42).  Pooler followed by Linear(hidden -> num_classes) + Softmax on
 * the device, with classifier_kernel.npy [hidden, num_classes] / classifier_bias.npy from the
 * model directory (the sample app's head, apps/finetune.py:16-44).  `output` is host fp32
 * [batchsize, num_classes].                                                                 */
CUDABERT_API void Cuda_Classify(void* model, float* output, int* words, int* token_types, int batchsize, int seq_length,
                   int num_classes, int* attention_mask);

/* ---- additions (no counterpart in the reference, which exits the process on any error) ---- */

/* init_model with an explicit precision (0 fp32, 1 bf16, 2 fp8-e4m3 weights; -1 = environment /
 * default) and an optional cap on the number of encoder layers (<= 0: all).                  */
CUDABERT_API void* cudabert_init_ex(bool large, int num_gpu, int max_batchsize, int max_seq_length, const char* dir,
                       int precision, int num_layers);
/* 0 = ok, 1 = bad argument, 2 = CUDA error (sticky), 3 = weight loading, 4 = device-side check. */
CUDABERT_API int cudabert_status(void* model);
/* Message of the first error since the last successful call; model == NULL: why the last
 * init_model on this thread failed.                                                          */
CUDABERT_API const char* cudabert_last_error(void* model);
CUDABERT_API int cudabert_hidden_size(void* model);
/* Which attention kernel a 16-bit forward pass of this padded sequence length runs (the lengths of the
 * sequences live on the device, so the choice depends on the padded length alone; environment
 * CUDABERT_ATTENTION=tc|persist|mma forces one): 1 = mma.sync, one CTA per sequence and head;
 * 2 = tcgen05 (with 128-row tiles that hold rows of several sequences unless the padded length fills
 * its last tile of 128 rows to 85 %; CUDABERT_ATTENTION_TILES=packed|sequence forces either, and the bits
 * do not depend on it);
 * 3 = mma.sync, persistent.                                                                          */
CUDABERT_API int cudabert_attention_kernel_for(int seq_length);
CUDABERT_API int cudabert_num_classes(void* model);

/* Forward pass on inputs that already live in device memory (int32 [batchsize, seq_length];
 * mask_dev may be NULL).  Enqueues on the handle's stream and returns; cudabert_sync waits.
 * Results: cudabert_pooled_dev (fp32 [batchsize, hidden]).  Returns 0 on success.            */
CUDABERT_API int cudabert_forward_dev(void* model, const int* ids_dev, const int* seg_dev, const int* mask_dev, int batchsize,
                         int seq_length);
/* Same with the classifier head appended (Cuda_Classify on device-resident inputs); results:
 * cudabert_probs_dev (fp32 [batchsize, num_classes]).                                          */
CUDABERT_API int cudabert_classify_dev(void* model, const int* ids_dev, const int* seg_dev, const int* mask_dev,
                                       int batchsize, int seq_length);
CUDABERT_API int cudabert_sync(void* model);
/* Test hook for the failure path of the device-side pipelines (no counterpart in the reference, whose
 * kernels have no waits).  Every mbarrier wait in the GEMM and attention kernels gives up after 2 s, sets
 * an error word and lets the kernel finish; the host then reports status 4.  This call runs that same wait,
 * in a one-thread kernel on the handle's stream, on a barrier nobody arrives on, with a limit of limit_us
 * microseconds (at most 2 000 000), waits for it and returns the handle's status: 4, with the wait site
 * in cudabert_last_error.  The handle stays usable; the next call clears the status.  Nothing faults or
 * hangs: the kernel returns by itself when the limit has passed.                                       */
CUDABERT_API int cudabert_test_wait_timeout(void* model, int limit_us);
CUDABERT_API float* cudabert_pooled_dev(void* model);
CUDABERT_API float* cudabert_probs_dev(void* model);
/* Blocking device-to-host copy, so that a ctypes caller can read what Retval points to. */
CUDABERT_API int cudabert_copy_to_host(void* dst_host, const void* src_dev, size_t bytes);
/* The handle's CUDA stream (a cudaStream_t), for event timing on the launching stream. */
CUDABERT_API void* cudabert_stream(void* model);

/* Kernels launched by the last forward pass of this handle. */
CUDABERT_API long cudabert_launch_count(void* model);
/* A forward pass is enqueued kernel by kernel the first time its exact arguments (input addresses,
 * batch, sequence length) are seen (and the second), captured into a CUDA graph the third time and replayed as one
 * graph launch from then on (environment CUDABERT_GRAPH=0: never).  These count the captures and the
 * replays of this handle so far. */
CUDABERT_API long cudabert_graph_captures(void* model);
CUDABERT_API long cudabert_graph_replays(void* model);
/* Per-kernel-class device timing with CUDA events on the handle's stream.  Classes: 0 embedding+LN,
 * 1 QKV GEMM, 2 attention, 3 attention-output GEMM, 4 LayerNorm, 5 FFN1 GEMM, 6 FFN2 GEMM,
 * 7 pooler GEMM, 8 other.  Enable, run forwards + sync, then read accumulated ms and launches. */
CUDABERT_API void cudabert_profile_enable(void* model, int on);
CUDABERT_API void cudabert_profile_reset(void* model);
CUDABERT_API int cudabert_profile_get(void* model, int kernel_class, double* total_ms, long* launches);

/* ---- length-bucketing batcher of the file-to-file engine (host only, no CUDA call) ----
 * Replaces the reference's Python reader-side batching: batch_container and queue_manager.put /
 * enqueue / force_enqueue (engine.py:12-130), optimize_batch (utils.py:3-13) and the valid
 * length of a line (utils.py:49-56).  boundaries[0..n): bucket q takes valid lengths in
 * (boundaries[q], boundaries[q+1]], the last bucket also everything longer. */
CUDABERT_API void* cudabert_batcher_create(const int* boundaries, int n_boundaries, int batch_size, int max_seq_length);
CUDABERT_API void cudabert_batcher_destroy(void* batcher);
/* Add one tokenised line (three int32 rows of n <= max_seq_length entries).  Returns its valid
 * length (1 + index of the last mask entry equal to 1; n if there is none), -1 on a bad argument. */
CUDABERT_API int cudabert_batcher_put(void* batcher, long long line_index, const int* ids, const int* seg, const int* mask,
                                      int n);
/* Turn every partly filled bucket into a ready batch; returns the number of ready batches. */
CUDABERT_API int cudabert_batcher_flush(void* batcher);
CUDABERT_API int cudabert_batcher_ready(void* batcher);
/* Lines put but not yet popped. */
CUDABERT_API long long cudabert_batcher_pending(void* batcher);
/* Shape of the batch the next pop returns (the ready batch with the smallest first line number):
 * 1 and rows / seq / first_line filled, 0 if no batch is ready. */
CUDABERT_API int cudabert_batcher_next(void* batcher, int* rows, int* seq, long long* first_line);
/* Pop that batch: line_index[rows], ids / seg / mask [rows, seq] right-trimmed to the batch's longest
 * line.  Returns rows, 0 if no batch is ready. */
CUDABERT_API int cudabert_batcher_pop(void* batcher, long long* line_index, int* ids, int* seg, int* mask);

/* ---- BERT tokenizer of the file-to-file engine's reader stage (host only, no CUDA call) ----
 * Replaces, for speed, the Python tokenisation of the reference's sample application: BertTokenizer =
 * BasicTokenizer + WordpieceTokenizer (apps/pytorch_pretrained_bert/tokenization.py:75-331) and the
 * packing of one or two texts into fixed-length features (apps/tokenlizer.py:45-134).  vocab_path: one
 * token per line (the line number is the id); it must hold [UNK], [CLS] and [SEP].  Returns NULL if the
 * file cannot be read or lacks them. */
CUDABERT_API void* cudabert_tokenizer_create(const char* vocab_path, int do_lower_case);
CUDABERT_API void cudabert_tokenizer_destroy(void* tokenizer);
CUDABERT_API int cudabert_tokenizer_vocab_size(void* tokenizer);
/* Word-piece ids of a UTF-8 text.  Returns their number (which may exceed capacity; at most capacity are
 * written), -1 on a bad argument. */
CUDABERT_API int cudabert_tokenizer_tokenize(void* tokenizer, const char* text_utf8, int* ids_out, int capacity);
/* [CLS] a [SEP] (b [SEP]) truncated and zero-padded to max_seq_length entries each of ids, mask (1 for
 * real tokens) and segment ids (1 for b and its [SEP]); text_b may be NULL or empty.  Returns the number
 * of real tokens, -1 on a bad argument. */
CUDABERT_API int cudabert_tokenizer_encode_pair(void* tokenizer, const char* text_a, const char* text_b, int max_seq_length,
                                                int* ids, int* mask, int* seg);

/* ---- reader stage of the file-to-file engine: file -> tokenizer threads -> batcher (host only) ----
 * Replaces the reference's reader process (engine.py:266-280 with apps/tokenlizer.py:136-147 as its
 * per-line function): `threads` threads read lines of `input_path` after its first skip_lines lines (a
 * header, lines a resumed run has written already), number them from first_index on, split them at
 * tabs into text_a and text_b, tokenise them with `tokenizer` (a cudabert_tokenizer, not owned) and put
 * them into length buckets (boundaries / batch_size as for cudabert_batcher_create).  NULL if the file
 * cannot be opened or an argument is bad. */
CUDABERT_API void* cudabert_reader_create(const char* input_path, void* tokenizer, int max_seq_length,
                                          const int* boundaries, int n_boundaries, int batch_size, int threads,
                                          long long skip_lines, long long first_index);
/* Stops the threads and frees the reader (the tokenizer stays). */
CUDABERT_API void cudabert_reader_destroy(void* reader);
/* Blocks until a batch is ready and takes it out of the buckets (1: its shape in rows / seq /
 * first_line; the batch waits inside the reader for cudabert_reader_pop), or until the file is
 * finished and every batch has been taken (0).  -1: a line was refused by the tokenizer or the buckets
 * (cudabert_reader_rejected says which); the stream ends there.  Lines end at "\n", "\r\n" or a lone
 * "\r", as in Python's text mode. */
CUDABERT_API int cudabert_reader_next(void* reader, int* rows, int* seq, long long* first_line);
/* Copies that batch out: line_index[rows], ids / seg / mask [rows, seq], raw_offsets[rows + 1] = where each
 * line's raw text (the line without NULs and trailing white space) starts in the text that
 * cudabert_reader_raw then copies out.  Returns rows. */
CUDABERT_API int cudabert_reader_pop(void* reader, long long* line_index, int* ids, int* seg, int* mask,
                                     long long* raw_offsets);
/* Raw text of the batch popped last, lines back to back (UTF-8, no terminator).  Returns its size in
 * bytes; copies at most capacity bytes. */
CUDABERT_API long long cudabert_reader_raw(void* reader, char* buf, long long capacity);
/* Turns the partly filled buckets into batches now (the writer asks for this when too many lines wait
 * for their predecessors).  Returns the number of ready batches. */
CUDABERT_API int cudabert_reader_flush(void* reader);
/* Lines tokenised so far. */
CUDABERT_API long long cudabert_reader_lines(void* reader);
/* Lines refused so far; *first_index (may be NULL) receives the number of the first one, -1 if none. */
CUDABERT_API long long cudabert_reader_rejected(void* reader, long long* first_index);

/* ---- single kernels on device buffers (stream 0, synchronous), for per-kernel parity tests ---- */

/* out[M,N] = epilogue(A[M,K] (row stride lda elements) x W[N,K]^T), A and W both bf16, or both fp16 with
 * flag 256; flags: 1 bias, 2 GELU, 4 residual, 8 tanh, 16 fp32 output, 32 per-column scale, 64 fp16 output
 * (bf16 otherwise), 128 accumulator x 1/4096 (the encoder holds its bf16-rounded weights as fp16 numbers
 * times 4096), 256 fp16 operands, 512 W given as E4M3 bytes (with 256 and 32; N % 256 == 0).  err_dev:
 * device int, set non-zero if a pipeline wait timed out.  N % 128 == 0, K % 64 == 0.  (Flag 1024, operands
 * of three bf16 planes, is refused here: cudabert_k_gemm_f32_tensor prepares such operands itself; so are
 * 2048, 4096 and 8192, the folded LayerNorms of CUDABERT_LN_FOLD=1, which exist inside a forward pass only.) */
CUDABERT_API int cudabert_k_gemm_tcgen05(const void* A_dev, long lda, const void* W_dev, int M, int N, int K, void* out_dev,
                         int flags, const float* bias_dev, const void* residual_dev, const float* colscale_dev,
                         int* err_dev);
/* out[M,N] = epilogue(A[M,K] fp32 (row stride lda) x W[K,N] fp32). */
CUDABERT_API int cudabert_k_gemm_f32(const float* A_dev, int lda, const float* W_dev, int M, int N, int K, float* out_dev,
                        int flags, const float* bias_dev, const float* residual_dev);
/* The same product on the tensor cores, as fp32 mode computes it by default: both operands are split
 * into three bf16 planes (x = x0 + x1 + x2, each the bf16 rounding of what the ones before leave) and
 * the tcgen05 GEMM sums the six leading cross terms with fp32 accumulation; what is dropped is below
 * 2^-24 of |a| |w|.  Same arguments as cudabert_k_gemm_f32; N % 128 == 0, K % 64 == 0, lda % 4 == 0. */
CUDABERT_API int cudabert_k_gemm_f32_tensor(const float* A_dev, int lda, const float* W_dev, int M, int N, int K,
                                            float* out_dev, int flags, const float* bias_dev, const float* residual_dev);
/* Two dense layers of bf16 mode with the LayerNorm between them folded into their epilogues, as a forward
 * pass runs them with CUDABERT_LN_FOLD=1:  sum = A1 W1 + b1 + res (fp32 [M, H], written to sum_dev);
 * out = act(LayerNorm(sum; gamma, beta) W2 + b2) in fp16 [M, N2], act = GELU if `gelu`.  A1 fp16 [M, K1]; W1
 * [H, K1] and W2 [N2, H] as the encoder holds its weights (bf16 values times 4096 in fp16); res fp32 [M, H].
 * H % 256 == 0, K1 % 64 == 0, N2 % 128 == 0. */
CUDABERT_API int cudabert_k_gemm_ln_folded(const void* A1_dev, const void* W1_dev, const float* b1_dev, const float* res_dev,
                                           const float* gamma_dev, const float* beta_dev, const void* W2_dev,
                                           const float* b2_dev, int M, int H, int K1, int N2, int gelu, float* sum_dev,
                                           void* out_dev);
/* ctx[T,H] = attention(qkv[T,3H]); mask_dev int32 [B,S] or NULL; kernel: 0 = fp32 kernel (fp32 in and
 * out), 1 = 16-bit mma.sync kernel (one CTA per sequence and head), 2 = 16-bit tcgen05 kernel, 3 = 16-bit
 * mma.sync kernel, persistent (S <= 256); the 16-bit kernels take fp16 Q, K, V and write fp16.  Adding 16
 * to a 16-bit kernel's number computes only the first query of every sequence and writes it to row b of
 * ctx_dev, then [B, H] (the last encoder layer of a pooler-only pass).  Adding 32 takes qkv_dev, and
 * writes ctx_dev, in the packed layout of a forward pass: the valid rows of the sequences back to back
 * (a sequence without a valid key counting as S rows), in buffers that still hold B * S rows; the
 * tcgen05 kernel then works on tiles of 128 consecutive rows whatever sequences they belong to. */
CUDABERT_API int cudabert_k_attention(int kernel, const void* qkv_dev, const int* mask_dev, void* ctx_dev, int B, int S, int heads);
/* No counterpart in the reference.  cudabert_k_attention for callers that must not allocate device
 * memory: code that runs where cudaMalloc is not allowed (inside another framework's memory pool
 * or allocator callback, in a process whose device memory is fully pre-partitioned, or in a
 * latency-critical loop that must not take the allocator's lock).  The per-row key counts, which
 * cudabert_k_attention keeps in a buffer it allocates and frees per call, live in a fixed array
 * inside the library image instead, so batch is limited to CUDABERT_NOALLOC_MAX_BATCH rows
 * (return code 6 and a message in cudabert_last_error(NULL) beyond that) and every GPU that loads
 * the library holds those 16 KiB until the process exits.  Inputs and outputs are the caller's, as
 * for cudabert_k_attention; no cudaMalloc / cudaFree or allocating library routine is called.
 * Only kernels 0 (fp32) and 1 (16-bit mma.sync), and 1 + 16 (first query only, output [B, H]), are
 * served: kernels 2 and 3 need scheduling and error scratch that the fixed array does not hold,
 * and any other number returns 1 before anything is launched.  Every non-zero return leaves its
 * reason in cudabert_last_error(NULL).
 * The first call on each device looks up the array's device address; make that first call before
 * starting any stream capture.  All calls share the one array: it is fully rewritten by each call
 * before use, and two calls of one process that overlap on the same GPU (for example from two
 * host threads) race on it -- serialise them.  Separate processes have separate copies.        */
#define CUDABERT_NOALLOC_MAX_BATCH 4096
CUDABERT_API int cudabert_k_attention_noalloc(int kernel, const void* qkv_dev, const int* mask_dev, void* ctx_dev,
                                              int B, int S, int heads);
/* out[T,H] = LayerNorm(word[ids] + pos[t % S] + type[seg]); tables fp32; out is fp16 (half != 0) or
 * fp32; out_f32_dev (may be NULL) receives the same values in fp32.  Returns 5 after clamping an
 * id outside [0, vocab) or a segment id outside {0, 1}.                                        */
CUDABERT_API int cudabert_k_embed_layernorm(int half, const int* ids_dev, const int* seg_dev, const float* word_dev,
                                            const float* pos_dev, const float* type_dev, const float* gamma_dev,
                                            const float* beta_dev, void* out_dev, float* out_f32_dev, int tokens,
                                            int S, int H, int vocab);
/* out[T,H] = LayerNorm(x[T,H] + residual[T,H]) * gamma + beta.  x is fp32, or fp16 when in_f16 != 0;
 * residual is fp32 or NULL; out is fp16 when out_f16 != 0, else fp32; out_f32_dev (may be NULL)
 * receives the same values in fp32.                                                          */
CUDABERT_API int cudabert_k_layernorm(int out_f16, int in_f16, const void* x_dev, const float* residual_dev,
                                      const float* gamma_dev, const float* beta_dev, void* out_dev,
                                      float* out_f32_dev, int tokens, int H);

#ifdef __cplusplus
}
#endif
#endif /* CUDABERT_H_ */
