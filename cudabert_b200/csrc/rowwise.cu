// Memory-bound row kernels: embedding gather + LayerNorm, LayerNorm, classifier head, and the
// load-time weight conversions.  One warp owns one row; 16-byte loads and stores; mean and
// variance by warp shuffles; variance as mean((x-u)^2) over values held in registers, the
// form the reference model uses (modeling.py:168-172; the CUDA reference reaches the same
// population variance by Welford, ops/layernorm.cu:52-134); eps 1e-12 inside the sqrt
// (ops/layernorm.cuh:43).
//
//   embed_layernorm  replaces DeviceApplyEmbeddings (ops/embedding.cu:3-20) + the LayerNorm
//                    that follows it (ops/embedding.cu:39-58): one pass instead of three.
//   layernorm        replaces cuApplyLayerNorm (ops/layernorm.cu:136-182), its in-place residual
//                    add included (`residual`, added in fp32; the fp32 mode passes none because
//                    its GEMM epilogue has added it already).
//   classify_softmax the sample app's fine-tune head (apps/finetune.py:16-24) on the device.
#include "kernels.h"
#include "ptx.cuh"

#include <atomic>
#include <cstdlib>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace cb {
namespace {

constexpr float LN_EPS = 1e-12f;
constexpr int ROWS_PER_BLOCK = 4;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// Each lane holds NV float4 vectors of its row: columns (i * 32 + lane) * 4 .. + 3, i < nvec.
// H <= 1024 -> at most 8 vectors per lane.
constexpr int MAXV = 8;

template <typename TOut>
__device__ __forceinline__ void store4(TOut* p, const float (&y)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&y)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(y[0], y[1], y[2], y[3]);
}
template <>
__device__ __forceinline__ void store4<__half>(__half* p, const float (&y)[4]) {
  uint2 t;
  t.x = pack_f16(y[0], y[1]);
  t.y = pack_f16(y[2], y[3]);
  *reinterpret_cast<uint2*>(p) = t;
}

template <typename TOut>
__device__ __forceinline__ void normalise_and_store(float (&x)[MAXV][4], int nvec, int lane, int H,
                                                    const float* __restrict__ gamma, const float* __restrict__ beta,
                                                    TOut* __restrict__ out_row, float* __restrict__ out_f32_row) {
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
    if (i < nvec) sum += (x[i][0] + x[i][1]) + (x[i][2] + x[i][3]);
  const float mean = warp_sum(sum) / static_cast<float>(H);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
    if (i < nvec)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float d = x[i][j] - mean;
        sq += d * d;
      }
  const float var = warp_sum(sq) / static_cast<float>(H);
  const float rstd = 1.0f / sqrtf(var + LN_EPS);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    if (i < nvec) {
      const int col = (i * 32 + lane) * 4;
      const float4 g = __ldg(reinterpret_cast<const float4*>(gamma + col));
      const float4 bt = __ldg(reinterpret_cast<const float4*>(beta + col));
      float y[4];
      y[0] = g.x * ((x[i][0] - mean) * rstd) + bt.x;
      y[1] = g.y * ((x[i][1] - mean) * rstd) + bt.y;
      y[2] = g.z * ((x[i][2] - mean) * rstd) + bt.z;
      y[3] = g.w * ((x[i][3] - mean) * rstd) + bt.w;
      store4<TOut>(out_row + col, y);
      if (out_f32_row) store4<float>(out_f32_row + col, y);
    }
  }
}

template <typename TOut>
__global__ void __launch_bounds__(ROWS_PER_BLOCK * 32)
embed_layernorm_kernel(const int* __restrict__ ids, const int* __restrict__ seg, const float* __restrict__ word,
                       const float* __restrict__ pos, const float* __restrict__ type, const float* __restrict__ gamma,
                       const float* __restrict__ beta, TOut* __restrict__ out, float* __restrict__ out_f32, int tokens,
                       int S, int H, int vocab, int* err, const int* __restrict__ row_start) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
  griddep_wait();
  griddep_launch();
  if (t >= tokens) return;
  // packed layout: token (b, s) goes to row row_start[b] + s; padding tokens have no row
  size_t orow = static_cast<size_t>(t);
  if (row_start) {
    const int b = t / S, sidx = t % S;
    const int first = row_start[b];
    if (sidx >= row_start[b + 1] - first) return;
    orow = static_cast<size_t>(first) + sidx;
  }
  int id = ids[t], sg = seg[t];
  if (id < 0 || id >= vocab || sg < 0 || sg > 1) {
    if (lane == 0) atomicOr(err, 2);  // bad token or segment id: clamp, report
    id = min(max(id, 0), vocab - 1);
    sg = min(max(sg, 0), 1);
  }
  const float* wr = word + static_cast<size_t>(id) * H;
  const float* pr = pos + static_cast<size_t>(t % S) * H;
  const float* tr = type + static_cast<size_t>(sg) * H;
  const int nvec = H / 128;
  float x[MAXV][4];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    if (i < nvec) {
      const int col = (i * 32 + lane) * 4;
      const float4 a = __ldg(reinterpret_cast<const float4*>(wr + col));
      const float4 b = __ldg(reinterpret_cast<const float4*>(pr + col));
      const float4 c = __ldg(reinterpret_cast<const float4*>(tr + col));
      x[i][0] = a.x + b.x + c.x; x[i][1] = a.y + b.y + c.y;
      x[i][2] = a.z + b.z + c.z; x[i][3] = a.w + b.w + c.w;
    }
  }
  normalise_and_store<TOut>(x, nvec, lane, H, gamma, beta, out + orow * H, out_f32 ? out_f32 + orow * H : nullptr);
}

template <typename TIn>
__device__ __forceinline__ void load4(const TIn* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<__half>(const __half* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

// out = LayerNorm(in + residual): `in` is the dense projection's output (fp32, or fp16 from the
// tensor-core GEMM), `residual` (may be null) the fp32 residual stream.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(ROWS_PER_BLOCK * 32)
layernorm_kernel(const TIn* __restrict__ in, const float* __restrict__ residual, const float* __restrict__ gamma,
                 const float* __restrict__ beta, TOut* __restrict__ out, float* __restrict__ out_f32, int tokens,
                 int H, const int* __restrict__ rows_dev, const int* __restrict__ res_rows, int res_stride) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
  griddep_wait();
  griddep_launch();
  if (t >= tokens || (rows_dev && t >= __ldg(rows_dev))) return;
  const TIn* row = in + static_cast<size_t>(t) * H;
  // the residual of output row t is row res_rows[t], or t * res_stride without a table (stride 1:
  // the same row; the compact last layer reads the first row of every sequence)
  const size_t res_row = res_rows ? static_cast<size_t>(__ldg(res_rows + t)) : static_cast<size_t>(t) * res_stride;
  const float* res = residual ? residual + res_row * H : nullptr;
  const int nvec = H / 128;
  float x[MAXV][4];
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
    if (i < nvec) {
      load4<TIn>(row + (i * 32 + lane) * 4, x[i]);
      if (res) {
        const float4 r = *reinterpret_cast<const float4*>(res + (i * 32 + lane) * 4);
        x[i][0] += r.x; x[i][1] += r.y; x[i][2] += r.z; x[i][3] += r.w;
      }
    }
  normalise_and_store<TOut>(x, nvec, lane, H, gamma, beta, out + static_cast<size_t>(t) * H,
                            out_f32 ? out_f32 + static_cast<size_t>(t) * H : nullptr);
}

// dst[b, s, :] = src[row_start[b] + s, :] for the rows a sequence has, 0 for its padding.
__global__ void unpack_rows_kernel(const float* __restrict__ src, const int* __restrict__ row_start,
                                   float* __restrict__ dst, int tokens, int S, int H) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
  griddep_wait();
  griddep_launch();
  if (t >= tokens) return;
  const int b = t / S, sidx = t % S;
  const int first = row_start[b];
  const bool live = sidx < row_start[b + 1] - first;
  const float4* s4 = reinterpret_cast<const float4*>(src + (static_cast<size_t>(first) + sidx) * H);
  float4* d4 = reinterpret_cast<float4*>(dst + static_cast<size_t>(t) * H);
  for (int i = lane; i < H / 4; i += 32) d4[i] = live ? s4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
}

__global__ void classify_softmax_kernel(const float* __restrict__ pooled, const float* __restrict__ W,
                                        const float* __restrict__ bias, float* __restrict__ probs, int B, int H,
                                        int C) {
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  griddep_wait();
  griddep_launch();
  if (b >= B) return;
  const float* x = pooled + static_cast<size_t>(b) * H;
  float logit = -INFINITY;  // lane c keeps class c
  for (int c = 0; c < C; ++c) {
    float s = 0.f;
    for (int k = lane; k < H; k += 32) s = fmaf(x[k], W[static_cast<size_t>(k) * C + c], s);
    s = warp_sum(s) + bias[c];
    if (lane == c) logit = s;
  }
  float mx = logit;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  const float e = (lane < C) ? expf(logit - mx) : 0.f;
  const float den = warp_sum(e);
  if (lane < C) probs[static_cast<size_t>(b) * C + lane] = e / den;
}

// dst[n, k] = the bf16 rounding of src[k, n], held as the fp16 number W_CONTAINER_SCALE times that
// value (exact, see kernels.h), through a 32x33 shared tile
__global__ void transpose_round_bf16_kernel(const float* __restrict__ src, __half* __restrict__ dst, int K, int N) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, n = n0 + threadIdx.x;
    tile[r][threadIdx.x] = (k < K && n < N) ? src[static_cast<size_t>(k) * N + n] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K)
      dst[static_cast<size_t>(n) * K + k] =
          __float2half_rn(__bfloat162float(__float2bfloat16_rn(tile[threadIdx.x][r])) * W_CONTAINER_SCALE);
  }
}

__device__ __forceinline__ void split3(float x, __nv_bfloat16& b0, __nv_bfloat16& b1, __nv_bfloat16& b2) {
  b0 = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(b0);  // exact
  b1 = __float2bfloat16_rn(r1);
  b2 = __float2bfloat16_rn(r1 - __bfloat162float(b1));
}

// dst[n, p K + k] = bf16 plane p of src[k, n], through a 32x33 shared tile
__global__ void transpose_split_bf16x3_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int K,
                                              int N) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, n = n0 + threadIdx.x;
    tile[r][threadIdx.x] = (k < K && n < N) ? src[static_cast<size_t>(k) * N + n] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) {
      __nv_bfloat16 b0, b1, b2;
      split3(tile[threadIdx.x][r], b0, b1, b2);
      __nv_bfloat16* row = dst + static_cast<size_t>(n) * 3 * K;
      row[k] = b0;
      row[K + k] = b1;
      row[2 * K + k] = b2;
    }
  }
}

// dst[m, p K + k] = bf16 plane p of src[m, k]; a thread takes four consecutive k (K % 4 == 0)
__global__ void __launch_bounds__(256)
split_bf16x3_kernel(const float* __restrict__ src, int lds, __nv_bfloat16* __restrict__ dst, int rows, int K,
                    const int* __restrict__ rows_dev) {
  griddep_wait();
  griddep_launch();
  if (rows_dev) rows = min(rows, __ldg(rows_dev));
  const int quads = K >> 2;
  const long long total = static_cast<long long>(rows) * quads;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / quads), k = static_cast<int>(i % quads) << 2;
    const float4 x = *reinterpret_cast<const float4*>(src + static_cast<size_t>(m) * lds + k);
    const float xs[4] = {x.x, x.y, x.z, x.w};
    __nv_bfloat16 p[3][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) split3(xs[j], p[0][j], p[1][j], p[2][j]);
    __nv_bfloat16* row = dst + static_cast<size_t>(m) * 3 * K + k;
#pragma unroll
    for (int q = 0; q < 3; ++q) *reinterpret_cast<uint2*>(row + q * K) = *reinterpret_cast<const uint2*>(p[q]);
  }
}

// The vectors of a LayerNorm folded into the GEMM that follows it (LnFold): c[n] = sum_k gamma[k] W[k, n],
// d[n] = sum_k beta[k] W[k, n] + bias[n], with W as the GEMM sees it (w[n, k] / W_CONTAINER_SCALE).  One warp per n.
__global__ void ln_fold_vectors_kernel(const __half* __restrict__ w, const float* __restrict__ gamma,
                                       const float* __restrict__ beta, const float* __restrict__ bias,
                                       float* __restrict__ c, float* __restrict__ d, int N, int K) {
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (n >= N) return;
  const __half* row = w + static_cast<size_t>(n) * K;
  float sc = 0.f, sd = 0.f;
  for (int k = lane; k < K; k += 32) {
    const float x = __half2float(row[k]);
    sc = fmaf(gamma[k], x, sc);
    sd = fmaf(beta[k], x, sd);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    sc += __shfl_xor_sync(0xffffffffu, sc, off);
    sd += __shfl_xor_sync(0xffffffffu, sd, off);
  }
  if (lane == 0) {
    c[n] = sc * (1.0f / W_CONTAINER_SCALE);
    d[n] = sd * (1.0f / W_CONTAINER_SCALE) + bias[n];
  }
}

__global__ void maxabs_kernel(const float* __restrict__ src, size_t n, unsigned int* __restrict__ out_bits) {
  float m = 0.f;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    m = fmaxf(m, fabsf(src[i]));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));  // non-negative floats order as uints
}

__global__ void finish_scale_kernel(float* scale_io) {
  const float m = *scale_io;
  *scale_io = (m > 0.f) ? m / 448.0f : 1.0f;
}

// dst_q (may be null): the E4M3 bytes; dst_wide (may be null): the same values widened exactly to fp16
__global__ void quantize_fp8_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst_q,
                                    __half* __restrict__ dst_wide, const float* __restrict__ scale, int K, int N) {
  __shared__ float tile[32][33];
  const float inv = 1.0f / *scale;
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, n = n0 + threadIdx.x;
    tile[r][threadIdx.x] = (k < K && n < N) ? src[static_cast<size_t>(k) * N + n] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) {
      const __nv_fp8_e4m3 q(tile[threadIdx.x][r] * inv);
      const size_t o = static_cast<size_t>(n) * K + k;
      if (dst_q) dst_q[o] = q.__x;
      if (dst_wide) dst_wide[o] = __float2half_rn(static_cast<float>(q));  // every E4M3 value is an fp16 value
    }
  }
}

__global__ void fill_f32_kernel(float* dst, float v, size_t n) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    dst[i] = v;
}

inline bool ln_shape_ok(int H) { return H > 0 && H % 128 == 0 && H <= 1024; }

}  // namespace

template <typename TOut>
int embed_layernorm(const int* ids, const int* seg, const float* word, const float* pos, const float* type,
                    const float* gamma, const float* beta, TOut* out, float* out_f32, int tokens, int S, int H,
                    int vocab, int* err_flag, const int* row_start, cudaStream_t stream) {
  if (tokens <= 0 || S <= 0 || !ln_shape_ok(H)) return -1;
  const int blocks = (tokens + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
  return launch_pdl(embed_layernorm_kernel<TOut>, dim3(blocks), dim3(ROWS_PER_BLOCK * 32), 0, stream, ids, seg, word, pos,
                    type, gamma, beta, out, out_f32, tokens, S, H, vocab, err_flag, row_start) == cudaSuccess ? 1 : -3;
}

// Persistent form of layernorm_kernel, the default: a fixed grid (two blocks of eight warps per SM)
// whose warps stride over the live rows, so rows that do not exist cost no blocks, and a warp issues
// the loads of its next row before it reduces and stores the current one, holding them raw
// (unconverted) so that nothing waits on them until the next turn.  Same arithmetic, same bits as
// layernorm_kernel; 31.8 against 34.1 us per launch on 14 000 rows x 1024.  The same grid without
// the look-ahead was slower than the block-per-four-rows kernel (45 us): it is the loads in
// flight across the reduce-and-store phase that pay, not the grid shape.
constexpr int LNP_THREADS = 256;
constexpr int LNP_BLOCKS_PER_SM = 2;

template <typename TIn> struct RawVec;
template <> struct RawVec<float> { typedef float4 type; };
template <> struct RawVec<__half> { typedef uint2 type; };
__device__ __forceinline__ void raw_to_float(const float4& t, float (&v)[4]) { v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
__device__ __forceinline__ void raw_to_float(const uint2& t, float (&v)[4]) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(LNP_THREADS, LNP_BLOCKS_PER_SM)
layernorm_persist_kernel(const TIn* __restrict__ in, const float* __restrict__ residual, const float* __restrict__ gamma,
                         const float* __restrict__ beta, TOut* __restrict__ out, float* __restrict__ out_f32,
                         int tokens, int H, const int* __restrict__ rows_dev, const int* __restrict__ res_rows,
                         int res_stride) {
  typedef typename RawVec<TIn>::type Raw;
  const int lane = threadIdx.x & 31;
  const int nwarps = gridDim.x * (LNP_THREADS / 32);
  int t = blockIdx.x * (LNP_THREADS / 32) + (threadIdx.x >> 5);
  griddep_wait();
  griddep_launch();
  const int rows = rows_dev ? min(tokens, __ldg(rows_dev)) : tokens;
  const int nvec = H / 128;
  Raw rin[MAXV];
  float4 rres[MAXV];
  auto issue = [&](int row_index) {
    const Raw* row = reinterpret_cast<const Raw*>(in + static_cast<size_t>(row_index) * H);
    const size_t res_row = res_rows ? static_cast<size_t>(__ldg(res_rows + row_index))
                                    : static_cast<size_t>(row_index) * res_stride;
    const float4* res = residual ? reinterpret_cast<const float4*>(residual + res_row * H) : nullptr;
#pragma unroll
    for (int i = 0; i < MAXV; ++i)
      if (i < nvec) {
        rin[i] = row[i * 32 + lane];
        rres[i] = res ? res[i * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
  };
  if (t < rows) issue(t);
  while (t < rows) {
    float x[MAXV][4];
#pragma unroll
    for (int i = 0; i < MAXV; ++i)
      if (i < nvec) {
        raw_to_float(rin[i], x[i]);
        x[i][0] += rres[i].x; x[i][1] += rres[i].y; x[i][2] += rres[i].z; x[i][3] += rres[i].w;
      }
    const int next = t + nwarps;
    if (next < rows) issue(next);
    normalise_and_store<TOut>(x, nvec, lane, H, gamma, beta, out + static_cast<size_t>(t) * H,
                              out_f32 ? out_f32 + static_cast<size_t>(t) * H : nullptr);
    t = next;
  }
}

// CUDABERT_LN=block selects layernorm_kernel (a block of four warps per four rows).
static bool layernorm_persistent() {
  static const bool on = [] {
    const char* e = std::getenv("CUDABERT_LN");
    return !(e && e[0] == 'b');
  }();
  return on;
}

static int sm_count() {
  static std::atomic<int> cached[64] = {};  // per device; racing threads store the same value
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && cached[dev].load(std::memory_order_relaxed) > 0) return cached[dev].load(std::memory_order_relaxed);
  int n = 148;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (dev >= 0 && dev < 64) cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

template <typename TIn, typename TOut>
int layernorm(const TIn* x, const float* residual, const float* gamma, const float* beta, TOut* out, float* out_f32,
              int tokens, int H, const int* rows_dev, cudaStream_t stream, const int* res_rows, int res_stride) {
  if (tokens <= 0 || !ln_shape_ok(H)) return -1;
  if (layernorm_persistent()) {
    const int warps_per_block = LNP_THREADS / 32;
    const int want = (tokens + warps_per_block - 1) / warps_per_block;
    const int cap = sm_count() * LNP_BLOCKS_PER_SM;
    return launch_pdl(layernorm_persist_kernel<TIn, TOut>, dim3(want < cap ? want : cap), dim3(LNP_THREADS), 0, stream, x,
                      residual, gamma, beta, out, out_f32, tokens, H, rows_dev, res_rows, res_stride) == cudaSuccess
               ? 1 : -3;
  }
  const int blocks = (tokens + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
  return launch_pdl(layernorm_kernel<TIn, TOut>, dim3(blocks), dim3(ROWS_PER_BLOCK * 32), 0, stream, x, residual, gamma,
                    beta, out, out_f32, tokens, H, rows_dev, res_rows, res_stride) == cudaSuccess ? 1 : -3;
}

template int embed_layernorm<float>(const int*, const int*, const float*, const float*, const float*, const float*,
                                    const float*, float*, float*, int, int, int, int, int*, const int*, cudaStream_t);
template int embed_layernorm<__half>(const int*, const int*, const float*, const float*, const float*,
                                            const float*, const float*, __half*, float*, int, int, int, int,
                                            int*, const int*, cudaStream_t);
template int layernorm<float, float>(const float*, const float*, const float*, const float*, float*, float*, int, int,
                                     const int*, cudaStream_t, const int*, int);
template int layernorm<float, __half>(const float*, const float*, const float*, const float*, __half*,
                                             float*, int, int, const int*, cudaStream_t, const int*, int);
template int layernorm<__half, float>(const __half*, const float*, const float*, const float*, float*, float*, int, int,
                                      const int*, cudaStream_t, const int*, int);
template int layernorm<__half, __half>(const __half*, const float*, const float*, const float*, __half*,
                                              float*, int, int, const int*, cudaStream_t, const int*, int);

int unpack_rows(const float* src, const int* row_start, float* dst, int tokens, int S, int H, cudaStream_t stream) {
  if (tokens <= 0 || S <= 0 || H % 4 != 0) return -1;
  const int blocks = (tokens + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
  return launch_pdl(unpack_rows_kernel, dim3(blocks), dim3(ROWS_PER_BLOCK * 32), 0, stream, src, row_start, dst, tokens,
                    S, H) == cudaSuccess ? 1 : -3;
}

int classify_softmax(const float* pooled, const float* W, const float* bias, float* probs, int B, int H, int C,
                     cudaStream_t stream) {
  if (B <= 0 || H <= 0 || C <= 0 || C > 32) return -1;
  return launch_pdl(classify_softmax_kernel, dim3((B + 3) / 4), dim3(128), 0, stream, pooled, W, bias, probs, B, H, C) ==
                 cudaSuccess ? 1 : -3;
}

int transpose_round_bf16(const float* src, __half* dst, int K, int N, cudaStream_t stream) {
  dim3 grid((N + 31) / 32, (K + 31) / 32), block(32, 8);
  transpose_round_bf16_kernel<<<grid, block, 0, stream>>>(src, dst, K, N);
  return cudaGetLastError() == cudaSuccess ? 1 : -3;
}

int quantize_fp8_weight(const float* src, uint8_t* dst_q, __half* dst_wide, float* scale_out, int K, int N,
                        cudaStream_t stream) {
  if (cudaMemsetAsync(scale_out, 0, sizeof(float), stream) != cudaSuccess) return -3;
  maxabs_kernel<<<296, 256, 0, stream>>>(src, static_cast<size_t>(K) * N, reinterpret_cast<unsigned int*>(scale_out));
  finish_scale_kernel<<<1, 1, 0, stream>>>(scale_out);
  dim3 grid((N + 31) / 32, (K + 31) / 32), block(32, 8);
  quantize_fp8_kernel<<<grid, block, 0, stream>>>(src, dst_q, dst_wide, scale_out, K, N);
  return cudaGetLastError() == cudaSuccess ? 3 : -3;
}

int transpose_split_bf16x3(const float* src, __nv_bfloat16* dst, int K, int N, cudaStream_t stream) {
  dim3 grid((N + 31) / 32, (K + 31) / 32), block(32, 8);
  transpose_split_bf16x3_kernel<<<grid, block, 0, stream>>>(src, dst, K, N);
  return cudaGetLastError() == cudaSuccess ? 1 : -3;
}

int split_bf16x3(const float* src, int lds, __nv_bfloat16* dst, int rows, int K, const int* rows_dev,
                 cudaStream_t stream) {
  if (rows <= 0 || K <= 0 || (K & 3) || (lds & 3)) return -1;
  const long long total = static_cast<long long>(rows) * (K >> 2);
  const long long want = (total + 255) / 256;
  const int grid = static_cast<int>(want < 148 * 8 ? want : 148 * 8);
  return launch_pdl(split_bf16x3_kernel, dim3(grid), dim3(256), 0, stream, src, lds, dst, rows, K, rows_dev) ==
                 cudaSuccess ? 1 : -3;
}

int ln_fold_vectors(const __half* w, const float* gamma, const float* beta, const float* bias, float* c, float* d, int N,
                    int K, cudaStream_t stream) {
  ln_fold_vectors_kernel<<<(N + 7) / 8, 256, 0, stream>>>(w, gamma, beta, bias, c, d, N, K);
  return cudaGetLastError() == cudaSuccess ? 1 : -3;
}

int fill_f32(float* dst, float value, size_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  fill_f32_kernel<<<296, 256, 0, stream>>>(dst, value, n);
  return cudaGetLastError() == cudaSuccess ? 1 : -3;
}

}  // namespace cb
