// fp32 CUDA-core GEMM with the same fused epilogue as the tensor-core GEMM; it is the
// projection kernel of the fp32-accuracy mode (the mode that has to stay within 1e-3 max-abs
// of the reference's fp32 model).  out[M, N] = A[M, K] x W[K, N]; W keeps the on-disk
// [in, out] layout (convert_pytorch_model_to_npys.py:62-63), so no transpose is needed.
// Replaces the same reference calls as gemm_tcgen05.cu (ops/linear.cu:91-148, 241-319).
//
// 128x128 tile, k-step 8, 256 threads, 8x8 outputs per thread, register-prefetched next
// k-step.  Rows beyond M are loaded as zero and not stored.
#include "kernels.h"
#include "ptx.cuh"

namespace cb {
namespace {

constexpr int TM = 128, TN = 128, TK = 8;

__device__ __forceinline__ float gelu_erf_f32(float x) { return x * 0.5f * (1.0f + erff(x * 0.70710678118654752f)); }

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int M, int N, int K,
                float* __restrict__ out, int ldo, int flags, const float* __restrict__ bias,
                const float* __restrict__ residual, const float* __restrict__ colscale,
                const int* __restrict__ m_dev) {
  griddep_wait();
  griddep_launch();
  if (m_dev) M = min(M, __ldg(m_dev));
  if (static_cast<int>(blockIdx.y) * TM >= M) return;
  __shared__ float As[2][TK][TM + 4];
  __shared__ float Bs[2][TK][TN];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * TM;
  const int n0 = blockIdx.x * TN;
  const int a_row = tid >> 1, a_k = (tid & 1) * 4;
  const int b_k = tid >> 5, b_col = (tid & 31) * 4;
  const int ty = tid >> 4, tx = tid & 15;  // 16 x 16 threads; thread owns rows ty*4+{0..3}, 64+ty*4+{0..3}

  const bool a_ok = (m0 + a_row) < M;
  const bool b_ok = (n0 + b_col) < N;
  const float* a_ptr = A + static_cast<size_t>(m0 + a_row) * lda + a_k;
  const float* b_ptr = W + static_cast<size_t>(b_k) * N + n0 + b_col;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  float4 ra = a_ok ? __ldg(reinterpret_cast<const float4*>(a_ptr)) : make_float4(0, 0, 0, 0);
  float4 rb = b_ok ? __ldg(reinterpret_cast<const float4*>(b_ptr)) : make_float4(0, 0, 0, 0);
  int buf = 0;
  As[0][a_k][a_row] = ra.x; As[0][a_k + 1][a_row] = ra.y; As[0][a_k + 2][a_row] = ra.z; As[0][a_k + 3][a_row] = ra.w;
  *reinterpret_cast<float4*>(&Bs[0][b_k][b_col]) = rb;
  __syncthreads();

  const int ksteps = K / TK;
  for (int ks = 0; ks < ksteps; ++ks) {
    if (ks + 1 < ksteps) {
      ra = a_ok ? __ldg(reinterpret_cast<const float4*>(a_ptr + (ks + 1) * TK)) : make_float4(0, 0, 0, 0);
      rb = b_ok ? __ldg(reinterpret_cast<const float4*>(b_ptr + static_cast<size_t>(ks + 1) * TK * N))
                : make_float4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (ks + 1 < ksteps) {
      const int nb = buf ^ 1;
      As[nb][a_k][a_row] = ra.x; As[nb][a_k + 1][a_row] = ra.y; As[nb][a_k + 2][a_row] = ra.z; As[nb][a_k + 3][a_row] = ra.w;
      *reinterpret_cast<float4*>(&Bs[nb][b_k][b_col]) = rb;
      __syncthreads();
      buf = nb;
    }
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (row >= M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int col = n0 + h * 64 + tx * 4;
      if (col >= N) continue;
      float v[4] = {acc[i][h * 4], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]};
      if (flags & EPI_COLSCALE) {
        const float4 s = __ldg(reinterpret_cast<const float4*>(colscale + col));
        v[0] *= s.x; v[1] *= s.y; v[2] *= s.z; v[3] *= s.w;
      }
      if (flags & EPI_BIAS) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(bias + col));
        v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
      }
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
  return launch_pdl(gemm_f32_kernel, grid, dim3(256), 0, stream, A, lda, W, M, N, K, out, ldo, epi.flags, epi.bias,
                    static_cast<const float*>(epi.residual), epi.colscale, m_dev) == cudaSuccess ? 1 : -3;
}

}  // namespace cb
