// fp32 CUDA-core GEMM with the same fused epilogue as the tensor-core GEMM; it is the
// projection kernel of the fp32-accuracy mode (the mode that has to stay within 1e-3 max-abs
// of the reference's fp32 model).  out[M, N] = A[M, K] x W[K, N]; W keeps the on-disk
// [in, out] layout (convert_pytorch_model_to_npys.py:62-63), so no transpose is needed.
// Replaces the same reference calls as gemm_tcgen05.cu (ops/linear.cu:91-148, 241-319).
//
// 64 x 64 tile, k-step 16, 128 threads (8 x 4 outputs each), three shared-memory stages filled with
// cp.async two k-steps ahead.  The tile is small on purpose: the shapes of this mode are a few hundred
// to a few thousand rows against N = 768..4096, and 64 x 64 tiles give every SM several CTAs to
// overlap one CTA's load latency with another's arithmetic (the reduction is never split, so a row's
// result does not depend on the batch it is in).  Rows beyond M are loaded as zero and not stored.
#include "kernels.h"
#include "ptx.cuh"

namespace cb {
namespace {

constexpr int TM = 64, TN = 64, TK = 16, F32_STAGES = 3, F32_THREADS = 128;
constexpr int A_LD = TK + 4;  // padded row of the A tile: 80 bytes, keeps 16-byte alignment

__device__ __forceinline__ float gelu_erf_f32(float x) { return x * 0.5f * (1.0f + erff(x * 0.70710678118654752f)); }

__global__ void __launch_bounds__(F32_THREADS)
gemm_f32_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int M, int N, int K,
                float* __restrict__ out, int ldo, int flags, const float* __restrict__ bias,
                const float* __restrict__ residual, const float* __restrict__ colscale,
                const int* __restrict__ m_dev) {
  griddep_wait();
  griddep_launch();
  if (m_dev) M = min(M, __ldg(m_dev));
  const int m0 = blockIdx.y * TM;
  if (m0 >= M) return;
  __shared__ __align__(16) float As[F32_STAGES][TM][A_LD];
  __shared__ __align__(16) float Bs[F32_STAGES][TK][TN];
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * TN;
  const int ty = tid >> 4, tx = tid & 15;  // 8 x 16 threads; thread owns rows ty*8 + {0..7}, columns tx*4 + {0..3}

  // every thread moves two 16-byte pieces of A and two of B per k-step
  auto load_stage = [&](int stage, int ks) {
    const int k0 = ks * TK;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int c = tid + F32_THREADS * j;
      const int ar = c >> 2, ak = (c & 3) * 4;
      const bool a_ok = (m0 + ar) < M;
      cp_async16(smem_u32(&As[stage][ar][ak]), A + static_cast<size_t>(a_ok ? m0 + ar : 0) * lda + k0 + ak, a_ok);
      const int br = c >> 4, bn = (c & 15) * 4;
      const bool b_ok = (n0 + bn) < N;
      cp_async16(smem_u32(&Bs[stage][br][bn]), W + static_cast<size_t>(k0 + br) * N + (b_ok ? n0 + bn : 0), b_ok);
    }
  };

  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int ksteps = K / TK;
  load_stage(0, 0);
  cp_async_commit();
  if (ksteps > 1) load_stage(1, 1);
  cp_async_commit();
  for (int ks = 0; ks < ksteps; ++ks) {
    cp_async_wait<1>();  // the group of k-step ks has landed (one younger group may still be in flight)
    __syncthreads();     // ... for every thread's pieces, and everyone is done with the stage refilled below
    if (ks + 2 < ksteps) load_stage((ks + 2) % F32_STAGES, ks + 2);
    cp_async_commit();
    const int st = ks % F32_STAGES;
#pragma unroll
    for (int k4 = 0; k4 < TK; k4 += 4) {
      float4 a[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = *reinterpret_cast<const float4*>(&As[st][ty * 8 + i][k4]);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const float4 b = *reinterpret_cast<const float4*>(&Bs[st][k4 + kk][tx * 4]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float av = kk == 0 ? a[i].x : (kk == 1 ? a[i].y : (kk == 2 ? a[i].z : a[i].w));
          acc[i][0] = fmaf(av, b.x, acc[i][0]);
          acc[i][1] = fmaf(av, b.y, acc[i][1]);
          acc[i][2] = fmaf(av, b.z, acc[i][2]);
          acc[i][3] = fmaf(av, b.w, acc[i][3]);
        }
      }
    }
  }

  const int col = n0 + tx * 4;
  if (col >= N) return;
  float4 cs = make_float4(1.f, 1.f, 1.f, 1.f), bv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (flags & EPI_COLSCALE) cs = __ldg(reinterpret_cast<const float4*>(colscale + col));
  if (flags & EPI_BIAS) bv = __ldg(reinterpret_cast<const float4*>(bias + col));
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = m0 + ty * 8 + i;
    if (row >= M) continue;
    float v[4] = {acc[i][0], acc[i][1], acc[i][2], acc[i][3]};
    if (flags & EPI_COLSCALE) { v[0] *= cs.x; v[1] *= cs.y; v[2] *= cs.z; v[3] *= cs.w; }
    if (flags & EPI_BIAS) { v[0] += bv.x; v[1] += bv.y; v[2] += bv.z; v[3] += bv.w; }
    if (flags & EPI_RESIDUAL) {
      const float4 r = __ldg(reinterpret_cast<const float4*>(residual + static_cast<size_t>(row) * ldo + col));
      v[0] += r.x; v[1] += r.y; v[2] += r.z; v[3] += r.w;
    }
    if (flags & EPI_GELU) {
#pragma unroll
      for (int q = 0; q < 4; ++q) v[q] = gelu_erf_f32(v[q]);
    }
    if (flags & EPI_TANH) {
#pragma unroll
      for (int q = 0; q < 4; ++q) v[q] = tanhf(v[q]);
    }
    *reinterpret_cast<float4*>(out + static_cast<size_t>(row) * ldo + col) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

// Pooler: out[b, :] = tanh(x[first row of sequence b, 0..H) . W[H, H] + bias), fp32
// (reference: copy_pooler + op_Linear + op_Tanh, ops/elementwise.cu:6-32, 57-70, utils/bert.cu:239-247).
// It is a skinny product (B rows against an H x H matrix that has to be streamed once), so the work
// is cut for parallel weight streaming, not for arithmetic: a CTA owns PN = 64 output columns and
// PB = 8 sequences; its 256 threads are 4 slices of the reduction dimension x 64 columns, so that
// consecutive threads read consecutive weights of one row (coalesced), every weight is loaded
// once per CTA and used for 8 sequences, the 8 inputs of a k are a shared-memory broadcast, and the
// four partial sums meet in shared memory at the end.
constexpr int PN = 64, PB = 8, PSLICES = 4;

__global__ void __launch_bounds__(PN * PSLICES)
pooler_f32_kernel(const float* __restrict__ x, int rows_per_seq, const int* __restrict__ row_start,
                  const float* __restrict__ W, const float* __restrict__ bias, float* __restrict__ out, int B, int H) {
  extern __shared__ float pool_smem[];
  float* xs = pool_smem;                 // [H][PB]: the CTA's 8 input rows, k-major
  float* part = pool_smem + H * PB;      // [PSLICES][PB][PN] partial sums
  const int tid = threadIdx.x;
  const int c = tid % PN, slice = tid / PN;
  const int n0 = blockIdx.x * PN, b0 = blockIdx.y * PB;
  griddep_wait();
  griddep_launch();
  for (int i = tid; i < H * PB; i += PN * PSLICES) {
    const int r = i / H, k = i - r * H;  // consecutive threads read consecutive elements of a row
    const int bb = b0 + r;
    float v = 0.f;
    if (bb < B) {
      const size_t xrow = row_start ? static_cast<size_t>(row_start[bb]) : static_cast<size_t>(bb) * rows_per_seq;
      v = x[xrow * H + k];
    }
    xs[k * PB + r] = v;
  }
  __syncthreads();
  const int kper = H / PSLICES;
  const float* wp = W + static_cast<size_t>(slice) * kper * H + n0 + c;
  const float* xp = xs + slice * kper * PB;
  float acc[PB];
#pragma unroll
  for (int r = 0; r < PB; ++r) acc[r] = 0.f;
#pragma unroll 8
  for (int k = 0; k < kper; ++k) {
    const float w = __ldg(wp + static_cast<size_t>(k) * H);
    const float4 x0 = *reinterpret_cast<const float4*>(xp + k * PB);
    const float4 x1 = *reinterpret_cast<const float4*>(xp + k * PB + 4);
    acc[0] = fmaf(x0.x, w, acc[0]); acc[1] = fmaf(x0.y, w, acc[1]);
    acc[2] = fmaf(x0.z, w, acc[2]); acc[3] = fmaf(x0.w, w, acc[3]);
    acc[4] = fmaf(x1.x, w, acc[4]); acc[5] = fmaf(x1.y, w, acc[5]);
    acc[6] = fmaf(x1.z, w, acc[6]); acc[7] = fmaf(x1.w, w, acc[7]);
  }
#pragma unroll
  for (int r = 0; r < PB; ++r) part[(slice * PB + r) * PN + c] = acc[r];
  __syncthreads();
  for (int i = tid; i < PB * PN; i += PN * PSLICES) {
    const int r = i / PN, cc = i - r * PN;
    if (b0 + r >= B) continue;
    float v = bias[n0 + cc];
#pragma unroll
    for (int sl = 0; sl < PSLICES; ++sl) v += part[(sl * PB + r) * PN + cc];  // fixed order: deterministic
    out[static_cast<size_t>(b0 + r) * H + n0 + cc] = tanhf(v);
  }
}

}  // namespace

int pooler_f32(const float* x, int rows_per_seq, const int* row_start, const float* W, const float* bias, float* out,
               int B, int H, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || (H % PN) != 0 || (H % (4 * PSLICES)) != 0 || H > 1024) return -1;
  dim3 grid(H / PN, (B + PB - 1) / PB);
  if (grid.y > 65535) return -1;
  const size_t smem = (static_cast<size_t>(H) * PB + PSLICES * PB * PN) * sizeof(float);  // 40 KB at H = 1024
  return launch_pdl(pooler_f32_kernel, grid, dim3(PN * PSLICES), smem, stream, x, rows_per_seq, row_start, W, bias, out,
                    B, H) == cudaSuccess ? 1 : -3;
}

int gemm_f32(const float* A, int lda, const float* W, int M, int N, int K, float* out, int ldo,
             const GemmEpilogue& epi, const int* m_dev, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (N % 4) != 0 || (K % TK) != 0 || (lda % 4) != 0 || (ldo % 4) != 0) return -1;
  if ((epi.flags & EPI_BIAS) && !epi.bias) return -1;
  if ((epi.flags & EPI_RESIDUAL) && !epi.residual) return -1;
  if ((epi.flags & EPI_COLSCALE) && !epi.colscale) return -1;
  dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
  if (grid.y > 65535) return -1;
  // plain stream order: with dependent launch this kernel's forward pass took twice as long (BERT-base,
  // 8 x 128 tokens: 8.4 against 4.5 ms), its many small CTAs being scheduled ahead of their producers
  return launch_plain(gemm_f32_kernel, grid, dim3(F32_THREADS), 0, stream, A, lda, W, M, N, K, out, ldo, epi.flags,
                    epi.bias, static_cast<const float*>(epi.residual), epi.colscale, m_dev) == cudaSuccess ? 1 : -3;
}

}  // namespace cb
