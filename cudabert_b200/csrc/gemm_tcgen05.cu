// Dense projection GEMM for sm_100a: out[M, N] = A[M, K] x W[N, K]^T with a fused epilogue.
//
// It replaces, in every mode (bf16 or FP8 weights with fp16 activations; fp32 with both operands as three
// bf16 planes, EPI_SPLIT3), the reference's cuBLAS SGEMM calls and the kernels around them: the bias pre-fill `MemoryCpyLinear` (ops/linear.cu:23-27), the GEMMs
// of `op_BatchedLinear::forward` (ops/linear.cu:241-319) and `op_Linear::forward`
// (ops/linear.cu:91-148), the GELU sweep (ops/elementwise.cu:38-51), the residual add that
// `cuApplyLayerNorm` does in place (ops/layernorm.cu:152-158) and the pooler's tanh
// (ops/elementwise.cu:57-70).
//
// Two variants share the epilogue.  `gemm_tcgen05_pair_kernel` (default when N is a multiple of
// 256) runs CTA pairs: a 256 x 256 tile per pair, `tcgen05.mma.cta_group::2`, each CTA loading its
// own 128 rows of A and its own half (128 rows) of the W tile, so an SM fills 32 KB of shared
// memory per k-block instead of 48 KB; the operand feed is what bounds the single-CTA variant.
// Loads are never shared between CTAs.  `gemm_tcgen05_kernel` is the single-CTA variant:
//
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0, one lane   TMA producer: per k-block one 128x64 tile of A and one BNx64 tile of W
//                      (128-byte swizzle) into a ring of shared-memory stages guarded by
//                      full/empty mbarriers.
//   warp 1, one lane   issues tcgen05.mma (128 x BN x 16, fp16 or bf16 in, fp32 accumulate in TMEM);
//                      tcgen05.commit releases a stage back to the producer and, after the
//                      last k-block, hands the accumulator to the epilogue.
//   warps 2-9          epilogue: tcgen05.ld of the accumulator (a warp can reach the TMEM lane
//                      quarter warp_id % 4 only, so two warps share a quarter and each takes
//                      half of the tile's columns: with one warp per SM sub-partition the
//                      epilogue issues from a single warp there and is latency-bound), bias /
//                      column scale / residual / GELU / tanh in registers, 16-byte stores.  Two
//                      accumulators (2 x BN TMEM columns) let the epilogue of tile i overlap the
//                      MMAs of tile i+1.
#include "kernels.h"
#include "ptx.cuh"

#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <mutex>

namespace cb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int EPI_WARPS = 8;                         // two per lane quarter, each takes half of the columns
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int GEMM_THREADS = 64 + EPI_THREADS;
constexpr int EPI_WARP_BYTES = 32 * 64;              // one 32-row x 64-byte piece per epilogue warp
constexpr int EPI_VEC_BYTES = 5 * 256 * 4;           // bias, column scale and three LayerNorm vectors of one tile
constexpr int EPI_STAGE_BYTES = EPI_WARPS * EPI_WARP_BYTES + EPI_VEC_BYTES;

template <int BN>
struct Cfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_STAGE_BYTES + BAR_BYTES + 1024;  // 1024: alignment slack
};

// erf-GELU x * 0.5 * (1 + erf(x / sqrt 2)) evaluated as 0.5 x (1 + tanh(x (c0 + c1 x^2 + c2 x^4))) with
// coefficients fitted to the erf form (max abs deviation 2.5e-5 over the reals, below one 16-bit
// rounding of the result everywhere) and the hardware tanh (relative error 2^-11), instead of ~45
// instructions per element for erff, which otherwise makes the FFN1 epilogue slower than its main loop.
// Two values at a time with the packed fp32 instructions of sm_100 (mul / fma .f32x2: one issue
// slot for two lanes of arithmetic; the epilogue of the GELU GEMM is bound by issue slots).  The
// clamp is applied to x^2 (<= 64), which keeps the polynomial positive, so that beyond |x| = 8 the
// tanh argument has the sign of x and a magnitude above 13: tanh is +-1 there.
__device__ __forceinline__ void gelu_erf2(float& a, float& b) {
  uint64_t x, x2, p, u, hx;
  asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(a), "f"(b));
  asm("mul.rn.f32x2 %0, %1, %1;" : "=l"(x2) : "l"(x));
  float qa, qb;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(qa), "=f"(qb) : "l"(x2));
  qa = fminf(qa, 64.0f);
  qb = fminf(qb, 64.0f);
  asm("mov.b64 %0, {%1, %2};" : "=l"(x2) : "f"(qa), "f"(qb));
  uint64_t c0, c1, c2, half;
  asm("mov.b64 %0, {%1, %1};" : "=l"(c2) : "f"(-0.000351516789798119f));
  asm("mov.b64 %0, {%1, %1};" : "=l"(c1) : "f"(0.03700564602858787f));
  asm("mov.b64 %0, {%1, %1};" : "=l"(c0) : "f"(0.7975078842834395f));
  asm("mov.b64 %0, {%1, %1};" : "=l"(half) : "f"(0.5f));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(p) : "l"(x2), "l"(c2), "l"(c1));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(p) : "l"(x2), "l"(p), "l"(c0));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(u) : "l"(x), "l"(p));
  float ua, ub, ta, tb;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(ua), "=f"(ub) : "l"(u));
  asm("tanh.approx.f32 %0, %1;" : "=f"(ta) : "f"(ua));
  asm("tanh.approx.f32 %0, %1;" : "=f"(tb) : "f"(ub));
  uint64_t t;
  asm("mov.b64 %0, {%1, %2};" : "=l"(t) : "f"(ta), "f"(tb));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(hx) : "l"(x), "l"(half));
  asm("fma.rn.f32x2 %0, %1, %2, %1;" : "=l"(x) : "l"(hx), "l"(t));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(x));
}

// Row statistics of a LayerNorm input from its per-slice partials (LnFold): mean and 1 / sqrt(var + eps)
__device__ __forceinline__ void ln_row_stats(const float* __restrict__ stats, int row, int slots, int n, float& mu,
                                             float& rstd) {
  const float2* p = reinterpret_cast<const float2*>(stats) + static_cast<size_t>(row) * slots;
  float sum = 0.f, sq = 0.f;
  for (int i = 0; i < slots; ++i) {
    const float2 t = __ldg(p + i);
    sum += t.x;
    sq += t.y;
  }
  const float inv_n = 1.0f / static_cast<float>(n);
  mu = sum * inv_n;
  const float var = fmaxf(sq * inv_n - mu * mu, 0.f);
  rstd = 1.0f / sqrtf(var + LN_EPS_F);
}

// Epilogue of the GEMM in front of a folded LayerNorm (EPI_LN_SUM): s = acc * scale + bias + residual.
// The accumulator leaves TMEM with a thread per row; everything that touches global memory happens after
// the transposition through the staging piece, where 4 lanes cover 64 contiguous bytes of a row: the fp32
// residual is read, s written in fp32 and s * gamma in fp16, all in full sectors, and a lane keeps the
// partial sum and sum of squares of the 4 rows it serves (rows i * 8 + lane / 4).  The residual of a
// 32-column chunk is in flight while the chunk before it is worked on; the first chunk's is requested
// before this warp waits for the accumulator (`tfull`).
template <int BN, int FLAGS>
__device__ __forceinline__ void epilogue_tile_sum(uint32_t t_acc, uint8_t* __restrict__ stage, const float* __restrict__ sbias,
                                                  const float* __restrict__ sscale, int warp, int half, int lane, int m0,
                                                  int n0, int M, int N, void* __restrict__ out, int ldo, int flags,
                                                  const void* __restrict__ residual, const LnFold& ln, uint64_t* tfull,
                                                  uint32_t tfull_phase, volatile int* abort_flag, int* err) {
  const int fl = (FLAGS >= 0) ? FLAGS : flags;
  const int quarter = warp & 3;
  const int row_base = m0 + quarter * 32;
  const uint32_t t_row = t_acc + (static_cast<uint32_t>(quarter * 32) << 16);
  const float* sv2 = sscale + 256;  // gamma of the LayerNorm this GEMM feeds
  const float* sv3 = sscale + 512;  // EPI_RES_LN: gamma and ...
  const float* sv4 = sscale + 768;  // ... beta of the residual's LayerNorm
  const int r2 = lane >> 2, p2 = lane & 3;
  uint8_t* my_row = stage + lane * 64;
  float* outf = static_cast<float*>(out);
  __half* outh = static_cast<__half*>(ln.out16);
  const float* resf = static_cast<const float*>(residual);
  const int c_begin = half * (BN / 64), c_end = c_begin + BN / 64;
  // the lane's 4 columns of pass h of a chunk, for its row i * 8 + r2
  auto cc_of = [&](int col, int h, int i) { return col + 16 * h + ((p2 ^ (((i * 8 + r2) >> 1) & 3)) << 2); };
  auto load_res = [&](int col, float4 (&q)[2][4]) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = row_base + i * 8 + r2;
        q[h][i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if ((fl & EPI_RESIDUAL) && row < M)
          q[h][i] = __ldg(reinterpret_cast<const float4*>(resf + static_cast<size_t>(row) * ldo + n0 + cc_of(col, h, i)));
      }
  };
  float4 q[2][4], qn[2][4];
  load_res(c_begin * 32, q);
  float rmu[4] = {0.f, 0.f, 0.f, 0.f}, rrs[4] = {1.f, 1.f, 1.f, 1.f}, ssum[4] = {0.f, 0.f, 0.f, 0.f},
        ssq[4] = {0.f, 0.f, 0.f, 0.f};
  if (fl & EPI_RES_LN) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (row_base + i * 8 + r2 < M) ln_row_stats(ln.res_stats, row_base + i * 8 + r2, N / 128, N, rmu[i], rrs[i]);
  }
  mbar_wait(tfull, tfull_phase, abort_flag, err, SITE_TMEM_FULL);
  tc_fence_after();
#pragma unroll
  for (int c = c_begin; c < c_end; ++c) {
    const int col = c * 32;
    if (c + 1 < c_end) load_res(col + 32, qn);
    uint32_t v[32];
    tmem_ld32(t_row + col, v);
    tmem_ld_wait();
    float f[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      f[j] = __uint_as_float(v[j]);
      if (fl & EPI_COLSCALE) f[j] *= sscale[col + j];
      if (fl & EPI_WSCALE) f[j] *= (1.0f / W_CONTAINER_SCALE);
      if (fl & EPI_BIAS) f[j] += sbias[col + j];
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<float4*>(my_row + ((j ^ ((lane >> 1) & 3)) << 4)) =
            make_float4(f[16 * h + 4 * j], f[16 * h + 4 * j + 1], f[16 * h + 4 * j + 2], f[16 * h + 4 * j + 3]);
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i * 8 + r2;
        const int row = row_base + r;
        float4 t = *reinterpret_cast<const float4*>(stage + r * 64 + (p2 << 4));
        const int cc = cc_of(col, h, i);
        if (row < M) {
          if (fl & EPI_RESIDUAL) {
            float4 x = q[h][i];
            if (fl & EPI_RES_LN) {
              x.x = (x.x - rmu[i]) * rrs[i] * sv3[cc] + sv4[cc];
              x.y = (x.y - rmu[i]) * rrs[i] * sv3[cc + 1] + sv4[cc + 1];
              x.z = (x.z - rmu[i]) * rrs[i] * sv3[cc + 2] + sv4[cc + 2];
              x.w = (x.w - rmu[i]) * rrs[i] * sv3[cc + 3] + sv4[cc + 3];
            }
            t.x += x.x; t.y += x.y; t.z += x.z; t.w += x.w;
          }
          ssum[i] += (t.x + t.y) + (t.z + t.w);
          ssq[i] += (t.x * t.x + t.y * t.y) + (t.z * t.z + t.w * t.w);
          const size_t o = static_cast<size_t>(row) * ldo + n0 + cc;
          *reinterpret_cast<float4*>(outf + o) = t;
          uint2 g;
          g.x = pack_f16(t.x * sv2[cc], t.y * sv2[cc + 1]);
          g.y = pack_f16(t.z * sv2[cc + 2], t.w * sv2[cc + 3]);
          *reinterpret_cast<uint2*>(outh + o) = g;
        }
      }
      __syncwarp();
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) q[h][i] = qn[h][i];
  }
  // a row's 4 lanes -> one partial per row and 128-column slice (BN = 256: one slice per warp of a row)
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    ssum[i] += __shfl_xor_sync(0xffffffffu, ssum[i], 1);
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 1);
    ssum[i] += __shfl_xor_sync(0xffffffffu, ssum[i], 2);
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 2);
    const int row = row_base + i * 8 + r2;
    if (p2 == 0 && row < M)
      reinterpret_cast<float2*>(ln.stats_out)[static_cast<size_t>(row) * (N / 128) + (n0 + half * (BN / 2)) / 128] =
          make_float2(ssum[i], ssq[i]);
  }
  tc_fence_before();
  __syncwarp();
}

// Epilogue of one accumulator (128 TMEM lanes x BN columns at `t_acc`), run by the eight epilogue
// warps; each owns the lane quarter warp % 4 and the column half `half`.  `m0` is the first output
// row of THIS CTA's 128 rows.
//
// FLAGS >= 0 fixes the epilogue at compile time (the combinations the model uses); FLAGS < 0 takes
// the run-time `flags`.  A thread reads one accumulator ROW from TMEM, but 32 threads storing to 32
// different rows touch 32 cache lines per instruction, so each warp transposes 32-column chunks
// through its own 2 KB of shared memory: phase 1, thread = row, writes 16-byte pieces at a swizzled
// position (conflict-free); phase 2, consecutive lanes cover consecutive bytes of a row, so global
// stores are full-sector, row-contiguous accesses.  Bias and column scale of the tile are staged
// in shared memory once per tile.  A residual (fp32 mode; the 16-bit modes add theirs in the LayerNorm
// kernel) is read by the row's own thread in phase 1.
template <int BN, int FLAGS>
__device__ __forceinline__ void epilogue_tile(uint32_t t_acc, uint8_t* __restrict__ stage, const float* __restrict__ sbias,
                                              const float* __restrict__ sscale, int warp, int half, int lane, int m0, int n0,
                                              int M, int N, int K, void* __restrict__ out, int ldo, int flags,
                                              const void* __restrict__ residual, const LnFold& ln, float mu, float rstd) {
  const int fl = (FLAGS >= 0) ? FLAGS : flags;
  tc_fence_after();
  const int quarter = warp & 3;
  const int row_base = m0 + quarter * 32;
  const int my_grow = row_base + lane;
  const uint32_t t_row = t_acc + (static_cast<uint32_t>(quarter * 32) << 16);
  const bool has_res = (fl & EPI_RESIDUAL) != 0 && my_grow < M;
  const float* sv2 = sscale + 256;  // gamma of the LayerNorm this GEMM feeds (EPI_LN_SUM) or gamma W (EPI_LN_APPLY)
  const float* sv3 = sscale + 512;  // EPI_RES_LN: gamma and ...
  const float* sv4 = sscale + 768;  // ... beta of the residual's LayerNorm
  const int r2 = lane >> 2, p2 = lane & 3;
  uint8_t* my_row = stage + lane * 64;
  // the residual's folded LayerNorm (without EPI_LN_SUM: the last GEMM before an ordinary LayerNorm)
  float rmu = 0.f, rrstd = 1.f;
  if ((fl & EPI_RES_LN) && has_res) ln_row_stats(ln.res_stats, my_grow, N / 128, N, rmu, rrstd);

  // acc * scale (normalised) + bias (+ residual) -> activation, for the 32 columns starting at n0 + col
  auto finish32 = [&](const uint32_t (&v)[32], float (&f)[32], int col) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      f[j] = __uint_as_float(v[j]);
      if (fl & EPI_COLSCALE) f[j] *= sscale[col + j];
      if (fl & EPI_WSCALE) f[j] *= (1.0f / W_CONTAINER_SCALE);  // fuses with the bias add into one FMA
      if (fl & EPI_LN_APPLY) f[j] = rstd * (f[j] - mu * sv2[col + j]);
      if (fl & EPI_BIAS) f[j] += sbias[col + j];
    }
    if (fl & EPI_RESIDUAL) {
      if (has_res) {
        if (fl & EPI_OUT_F32) {
          const float4* r = reinterpret_cast<const float4*>(static_cast<const float*>(residual) +
                                                            static_cast<size_t>(my_grow) * ldo + n0 + col);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 t = __ldg(r + j);
            if (fl & EPI_RES_LN) {
              t.x = (t.x - rmu) * rrstd * sv3[col + 4 * j] + sv4[col + 4 * j];
              t.y = (t.y - rmu) * rrstd * sv3[col + 4 * j + 1] + sv4[col + 4 * j + 1];
              t.z = (t.z - rmu) * rrstd * sv3[col + 4 * j + 2] + sv4[col + 4 * j + 2];
              t.w = (t.w - rmu) * rrstd * sv3[col + 4 * j + 3] + sv4[col + 4 * j + 3];
            }
            f[4 * j] += t.x; f[4 * j + 1] += t.y; f[4 * j + 2] += t.z; f[4 * j + 3] += t.w;
          }
        } else {
          const uint4* r = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(residual) +
                                                          static_cast<size_t>(my_grow) * ldo + n0 + col);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 t = __ldg(r + j);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[q]);
              f[8 * j + 2 * q] += __low2float(h);
              f[8 * j + 2 * q + 1] += __high2float(h);
            }
          }
        }
      }
    }
    if (fl & EPI_GELU) {
#pragma unroll
      for (int j = 0; j < 32; j += 2) gelu_erf2(f[j], f[j + 1]);
    }
    if (fl & EPI_TANH) {
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = tanhf(f[j]);
    }
  };

  // 32 fp32 columns of this warp's 32 rows -> dst[row][n0 + col ..]: two passes of 16 columns = 64 bytes
  // per row through the staging piece; phase 2: 4 lanes per row, 8 rows per instruction
  auto store_f32 = [&](const float (&f)[32], int col, float* dst) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<float4*>(my_row + ((j ^ ((lane >> 1) & 3)) << 4)) =
            make_float4(f[16 * h + 4 * j], f[16 * h + 4 * j + 1], f[16 * h + 4 * j + 2], f[16 * h + 4 * j + 3]);
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i * 8 + r2;
        const int row = row_base + r;
        const float4 t = *reinterpret_cast<const float4*>(stage + r * 64 + (p2 << 4));
        if (row < M)
          *reinterpret_cast<float4*>(dst + static_cast<size_t>(row) * ldo + n0 + col + 16 * h +
                                     ((p2 ^ ((r >> 1) & 3)) << 2)) = t;
      }
      __syncwarp();
    }
  };
  // 32 16-bit columns (bf16, or fp16 when `f16`) = 64 bytes per row, one pass
  auto store_16 = [&](const float (&f)[32], int col, uint16_t* dst, bool f16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 t;
      if (f16) {
        t.x = pack_f16(f[8 * j], f[8 * j + 1]);
        t.y = pack_f16(f[8 * j + 2], f[8 * j + 3]);
        t.z = pack_f16(f[8 * j + 4], f[8 * j + 5]);
        t.w = pack_f16(f[8 * j + 6], f[8 * j + 7]);
      } else {
        t.x = pack_bf16(f[8 * j], f[8 * j + 1]);
        t.y = pack_bf16(f[8 * j + 2], f[8 * j + 3]);
        t.z = pack_bf16(f[8 * j + 4], f[8 * j + 5]);
        t.w = pack_bf16(f[8 * j + 6], f[8 * j + 7]);
      }
      *reinterpret_cast<uint4*>(my_row + ((j ^ ((lane >> 1) & 3)) << 4)) = t;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i * 8 + r2;
      const int row = row_base + r;
      const uint4 t = *reinterpret_cast<const uint4*>(stage + r * 64 + (p2 << 4));
      if (row < M)
        *reinterpret_cast<uint4*>(dst + static_cast<size_t>(row) * ldo + n0 + col + ((p2 ^ ((r >> 1) & 3)) << 3)) = t;
    }
    __syncwarp();
  };

  // this warp's share of the tile: chunks of 32 columns in [half * BN / 2, (half + 1) * BN / 2)
  const int c_begin = half * (BN / 64), c_end = c_begin + BN / 64;
#pragma unroll
  for (int c = c_begin; c < c_end; ++c) {
    const int col = c * 32;
    uint32_t v[32];
    tmem_ld32(t_row + col, v);
    tmem_ld_wait();
    float f[32];
    finish32(v, f, col);
    if (fl & EPI_OUT_F32) {
      store_f32(f, col, static_cast<float*>(out));
    } else {
      store_16(f, col, static_cast<uint16_t*>(out), (fl & EPI_OUT_F16) != 0);
    }
  }
  tc_fence_before();
  __syncwarp();
}

// The epilogue warps (EPI_THREADS threads, named barrier 1) stage the per-column vectors of the tile's BN
// columns in shared memory: bias, column scale and, for folded LayerNorms, gamma (or gamma W) and the
// residual LayerNorm's gamma and beta.  The first barrier keeps a fast warp from overwriting values a
// slow warp still reads for the previous tile.
template <int BN, int FLAGS>
__device__ __forceinline__ void stage_tile_vectors(float* __restrict__ sbias, float* __restrict__ sscale, int flags,
                                                   const float* __restrict__ bias, const float* __restrict__ colscale,
                                                   const LnFold& ln, int n0) {
  const int fl = (FLAGS >= 0) ? FLAGS : flags;
  if (!(fl & (EPI_BIAS | EPI_COLSCALE | EPI_LN_SUM | EPI_LN_APPLY | EPI_RES_LN))) return;
  const int t = threadIdx.x - 64;  // 0..EPI_THREADS-1
  asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
  for (int i = t; i < BN; i += EPI_THREADS) {
    if (fl & EPI_BIAS) sbias[i] = __ldg(bias + n0 + i);
    if (fl & EPI_COLSCALE) sscale[i] = __ldg(colscale + n0 + i);
    if (fl & EPI_LN_SUM) sscale[256 + i] = __ldg(ln.gamma + n0 + i);
    if (fl & EPI_LN_APPLY) sscale[256 + i] = __ldg(ln.c + n0 + i);
    if (fl & EPI_RES_LN) {
      sscale[512 + i] = __ldg(ln.res_gamma + n0 + i);
      sscale[768 + i] = __ldg(ln.res_beta + n0 + i);
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
}

// The k-blocks a tile walks.  Plain: K / BK blocks at columns 0, BK, ... of both operands.  EPI_SPLIT3
// (operands of three bf16 planes of K columns each): six passes over K, one per cross term, the
// smallest terms first so that the fp32 accumulator keeps them: (A plane, W plane) = (2, 0), (0, 2),
// (1, 1), (1, 0), (0, 1), (0, 0).
struct KWalk {
  int per, kblocks, K;
  bool split;
  __device__ KWalk(int K_, bool split_) : per(K_ / BK), kblocks(split_ ? 6 * (K_ / BK) : K_ / BK), K(K_), split(split_) {}
  __device__ __forceinline__ int col(int kb, uint32_t planes) const {
    if (!split) return kb * BK;
    const int pass = kb / per;
    return static_cast<int>((planes >> (4 * pass)) & 15u) * K + (kb - pass * per) * BK;
  }
  __device__ __forceinline__ int a_col(int kb) const { return col(kb, 0x001102u); }
  __device__ __forceinline__ int w_col(int kb) const { return col(kb, 0x010120u); }
};

template <int BN, int FLAGS>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, int M, int N,
                    int K, void* __restrict__ out, int ldo, int flags, const float* __restrict__ bias,
                    const void* __restrict__ residual, const float* __restrict__ colscale, int* err,
                    const int* __restrict__ m_dev, const LnFold ln) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + C::STAGES * C::STAGE_BYTES;
  float* sbias = reinterpret_cast<float*>(epi_stage + EPI_WARPS * EPI_WARP_BYTES);
  float* sscale = sbias + 256;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + EPI_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + C::STAGES;
  uint64_t* tfull_bar = empty_bar + C::STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar + a, 1);
      mbar_init(tempty_bar + a, EPI_WARPS);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above is private to this CTA; from here on it touches the predecessor's output
  griddep_wait();
  griddep_launch();
  if (m_dev) M = min(M, __ldg(m_dev));

  const int tiles_n = N / BN;
  const int tiles_m = (M + BM - 1) / BM;
  const int num_tiles = tiles_m * tiles_n;
  const KWalk kw(K, (((FLAGS >= 0) ? FLAGS : flags) & EPI_SPLIT3) != 0);
  const int kblocks = kw.kblocks;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * BM;
        const int n0 = (tile % tiles_n) * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, err, SITE_EMPTY);
          uint8_t* sa = smem + stage * C::STAGE_BYTES;
          mbar_arrive_expect_tx(full_bar + stage, C::STAGE_BYTES);
          tma_load_2d(sa, &tmA, full_bar + stage, kw.a_col(kb), m0);
          tma_load_2d(sa + C::A_BYTES, &tmW, full_bar + stage, kw.w_col(kb), n0);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (((FLAGS >= 0) ? FLAGS : flags) & EPI_IN_F16) ? umma_idesc_f16(BM, BN) : umma_idesc_bf16(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        mbar_wait(tempty_bar + acc, acc_phase ^ 1, abort_flag, err, SITE_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait(full_bar + stage, phase, abort_flag, err, SITE_FULL);
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint64_t da = umma_desc_sw128(sa);
          const uint64_t db = umma_desc_sw128(sa + C::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advance 16 elements (32 bytes) along K inside the 128-byte swizzle row
            umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          }
          umma_commit(empty_bar + stage);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(tfull_bar + acc);
      }
    }
  } else {
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int n0 = (tile % tiles_n) * BN;
      const int m0 = (tile / tiles_n) * BM;
      stage_tile_vectors<BN, FLAGS>(sbias, sscale, flags, bias, colscale, ln, n0);
      if (((FLAGS >= 0) ? FLAGS : flags) & EPI_LN_SUM) {
        epilogue_tile_sum<BN, FLAGS>(tmem_base + acc * BN, epi_stage + (warp - 2) * EPI_WARP_BYTES, sbias, sscale, warp,
                                     (warp - 2) >> 2, lane, m0, n0, M, N, out, ldo, flags, residual, ln, tfull_bar + acc,
                                     acc_phase, abort_flag, err);
        if (lane == 0) mbar_arrive(tempty_bar + acc);
        continue;
      }
      float mu = 0.f, rstd = 1.f;  // a folded LayerNorm in front of this GEMM: the statistics of this thread's row
      if ((((FLAGS >= 0) ? FLAGS : flags) & EPI_LN_APPLY) && m0 + (warp & 3) * 32 + lane < M)
        ln_row_stats(ln.stats_in, m0 + (warp & 3) * 32 + lane, K / 128, K, mu, rstd);
      mbar_wait(tfull_bar + acc, acc_phase, abort_flag, err, SITE_TMEM_FULL);
      epilogue_tile<BN, FLAGS>(tmem_base + acc * BN, epi_stage + (warp - 2) * EPI_WARP_BYTES, sbias, sscale, warp,
                               (warp - 2) >> 2, lane, m0, n0, M, N, K, out, ldo, flags, residual, ln, mu, rstd);
      if (lane == 0) mbar_arrive(tempty_bar + acc);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: give copies that may still be in flight time to land before the
    // shared memory is released
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------------------------
// CTA-pair variant: cluster of 2, tile 256 (M) x BN (N) per pair, 6 stages of 32 KB per CTA.
//   both CTAs   warp 0 / one lane: TMA producer for the CTA's own A rows and W half; completion
//               bytes of both CTAs are counted on the LEADER's full barrier.
//   leader      warp 1 / one lane: tcgen05.mma.cta_group::2 for the pair; tcgen05.commit arrives
//               on the empty barrier (and, per tile, the accumulator-full barrier) of BOTH CTAs.
//   both CTAs   warps 2-9: epilogue of the CTA's own 128 accumulator rows; every epilogue warp
//               of the pair arrives on the leader's accumulator-empty barrier (count 16).
//
// W8 (FP8-weight mode): W lives in HBM as E4M3 bytes [N, K] and in no wider form.  The producer's TMA
// brings the CTA's 128 x 64 bytes of a k-block into a raw buffer beside the stage's A tile; four
// converter warps (10-13) widen them to fp16 (cvt.rn.f16x2.e4m3x2, exact) into one of five W operand
// tiles in the layout the MMA reads (128-byte rows, 16-byte chunk c of row r at position
// c ^ (r & 7)), fence them for the async proxy and arrive on the leader's "converted" barrier of that
// tile.  The weights cross HBM, L2 and the TMA at one byte per element; the tensor core sees fp16.
// Two rings (five stages of A + raw bytes, five converted tiles) instead of one of six: six stages of
// all three do not fit in shared memory.  Ring depths of 6 + 3 and 4 + 6 run at the same speed: what
// bounds this variant is shared-memory bandwidth (TMA writes, converter loads and stores, and the
// tensor core's operand reads come to 80 KB per k-block against 64 KB in the 16-bit kernel).
constexpr int CONV_WARPS = 4;
template <int BN, bool W8>
struct PairCfg {
  static constexpr int STAGES = W8 ? 5 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int RAW_BYTES = W8 ? (BN / 2) * BK : 0;  // E4M3 bytes of the CTA's W half per k-block
  // 16-bit kernel: a stage is A | W.  W8: a stage is A | raw bytes, and W operand tiles live in their own ring.
  static constexpr int STAGE_BYTES = A_BYTES + (W8 ? RAW_BYTES : B_BYTES);
  static constexpr int WBUFS = W8 ? 5 : 0;
  static constexpr int THREADS = GEMM_THREADS + (W8 ? CONV_WARPS * 32 : 0);
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + WBUFS * B_BYTES + EPI_STAGE_BYTES + BAR_BYTES + 1024;
};

template <int BN, int FLAGS, bool W8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<BN, W8>::THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, int M,
                         int N, int K, void* __restrict__ out, int ldo, int flags, const float* __restrict__ bias,
                         const void* __restrict__ residual, const float* __restrict__ colscale, int* err,
                         const int* __restrict__ m_dev, const LnFold ln) {
  using C = PairCfg<BN, W8>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* wbuf = smem + C::STAGES * C::STAGE_BYTES;  // W8: WBUFS converted W operand tiles
  uint8_t* epi_stage = wbuf + C::WBUFS * C::B_BYTES;
  float* sbias = reinterpret_cast<float*>(epi_stage + EPI_WARPS * EPI_WARP_BYTES);
  float* sscale = sbias + 256;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + EPI_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + C::STAGES;
  uint64_t* tfull_bar = empty_bar + C::STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* raw_full_bar = tempty_bar + 2;           // W8: this CTA's raw W bytes of a stage have landed
  uint64_t* wfull_bar = raw_full_bar + C::STAGES;    // W8 [3]: both CTAs' halves of a W operand tile are converted (leader's copy)
  uint64_t* wempty_bar = wfull_bar + 5;              // W8 [3]: the MMAs that read a W operand buffer have completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(wempty_bar + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar + s, 1);   // the leader's producer arrives; only the leader's copy is used
      mbar_init(empty_bar + s, 1);  // one commit arrival from the leader's MMA thread, in each CTA
      mbar_init(raw_full_bar + s, 1);
    }
    for (int b = 0; b < 5; ++b) {
      mbar_init(wfull_bar + b, 2 * CONV_WARPS);  // the converter warps of both CTAs
      mbar_init(wempty_bar + b, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar + a, 1);
      mbar_init(tempty_bar + a, 2 * EPI_WARPS);  // the epilogue warps of both CTAs; only the leader's copy is used
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, C::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above is private to this pair; from here on it touches the predecessor's output
  griddep_wait();
  griddep_launch();
  if (m_dev) M = min(M, __ldg(m_dev));

  const int tiles_n = N / BN;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int num_tiles = tiles_m * tiles_n;
  const KWalk kw(K, !W8 && (((FLAGS >= 0) ? FLAGS : flags) & EPI_SPLIT3) != 0);
  const int kblocks = kw.kblocks;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = pair_id; tile < num_tiles; tile += num_pairs) {
        const int m0 = (tile / tiles_n) * (2 * BM) + static_cast<int>(rank) * BM;
        const int n0 = (tile % tiles_n) * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, err, SITE_EMPTY);
          uint8_t* sa = smem + stage * C::STAGE_BYTES;
          if (leader) mbar_arrive_expect_tx(full_bar + stage, W8 ? 2 * C::A_BYTES : 2 * C::STAGE_BYTES);
          const uint32_t leader_full = mapa_u32(smem_u32(full_bar + stage), 0);
          tma_load_2d_pair(sa, &tmA, leader_full, kw.a_col(kb), m0);
          if (W8) {  // E4M3 bytes -> the stage's raw buffer; the converter warps take it from there
            mbar_arrive_expect_tx(raw_full_bar + stage, C::RAW_BYTES);
            tma_load_2d(sa + C::A_BYTES, &tmW, raw_full_bar + stage, kb * BK, n0);
          } else {
            tma_load_2d_pair(sa + C::A_BYTES, &tmW, leader_full, kw.w_col(kb), n0);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      const uint32_t idesc =
          (((FLAGS >= 0) ? FLAGS : flags) & EPI_IN_F16) ? umma_idesc_f16(2 * BM, BN) : umma_idesc_bf16(2 * BM, BN);
      int stage = 0, wb = 0;
      uint32_t phase = 0, wphase = 0;
      int it = 0;
      for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        mbar_wait(tempty_bar + acc, acc_phase ^ 1, abort_flag, err, SITE_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait(full_bar + stage, phase, abort_flag, err, SITE_FULL);
          if (W8) mbar_wait(wfull_bar + wb, wphase, abort_flag, err, SITE_FULL);
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint64_t da = umma_desc_sw128(sa);
          const uint64_t db = umma_desc_sw128(W8 ? smem_u32(wbuf + wb * C::B_BYTES) : sa + C::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) umma_f16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          umma_commit_pair(empty_bar + stage, 3);
          if (W8) {
            umma_commit_pair(wempty_bar + wb, 3);
            if (++wb == 5) { wb = 0; wphase ^= 1; }
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit_pair(tfull_bar + acc, 3);
      }
    }
  } else if (W8 && warp >= 2 + EPI_WARPS) {
    // converter warps: E4M3 bytes of the stage -> fp16 W operand tile.  Per pass a thread takes 16
    // consecutive bytes (a warp reads 512 contiguous bytes: rows r .. r + 7, four 16-element pieces
    // each) and writes the two 16-byte chunks they widen to at their swizzled places; the 32
    // stores of one instruction fall on all 32 banks four times over, the minimum for 512 bytes.
    const int t = threadIdx.x - (2 + EPI_WARPS) * 32;  // 0 .. 127
    const uint32_t leader_wfull0 = mapa_u32(smem_u32(wfull_bar), 0);
    int stage = 0, wb = 0;
    uint32_t phase = 0, wphase = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs) {
      for (int kb = 0; kb < kblocks; ++kb) {
        mbar_wait(raw_full_bar + stage, phase, abort_flag, err, SITE_FULL);       // the bytes have landed
        mbar_wait(wempty_bar + wb, wphase ^ 1, abort_flag, err, SITE_EMPTY);      // the buffer's last readers are done
        const uint8_t* src = smem + stage * C::STAGE_BYTES + C::A_BYTES;
        uint8_t* dst = wbuf + wb * C::B_BYTES;
#pragma unroll
        for (int i = 0; i < C::RAW_BYTES / (CONV_WARPS * 32 * 16); ++i) {
          const int idx = i * (CONV_WARPS * 32) + t;
          const int row = idx >> 2, q = idx & 3;
          const uint4 v = *reinterpret_cast<const uint4*>(src + idx * 16);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
          uint32_t h[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            h[2 * j] = e4m3x2_to_f16x2(static_cast<uint16_t>(w[j] & 0xffffu));
            h[2 * j + 1] = e4m3x2_to_f16x2(static_cast<uint16_t>(w[j] >> 16));
          }
          uint8_t* drow = dst + row * 128;
          *reinterpret_cast<uint4*>(drow + (((2 * q) ^ (row & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<uint4*>(drow + (((2 * q + 1) ^ (row & 7)) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
        }
        fence_proxy_async_smem();  // the tensor core reads the tile through the async proxy
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive(wfull_bar + wb);
          else mbar_arrive_remote(leader_wfull0 + wb * 8);
        }
        if (++wb == 5) { wb = 0; wphase ^= 1; }
        if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    int it = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int n0 = (tile % tiles_n) * BN;
      const int m0 = (tile / tiles_n) * (2 * BM) + static_cast<int>(rank) * BM;
      stage_tile_vectors<BN, FLAGS>(sbias, sscale, flags, bias, colscale, ln, n0);
      if (((FLAGS >= 0) ? FLAGS : flags) & EPI_LN_SUM) {
        epilogue_tile_sum<BN, FLAGS>(tmem_base + acc * BN, epi_stage + (warp - 2) * EPI_WARP_BYTES, sbias, sscale, warp,
                                     (warp - 2) >> 2, lane, m0, n0, M, N, out, ldo, flags, residual, ln, tfull_bar + acc,
                                     acc_phase, abort_flag, err);
        if (lane == 0) {
          if (leader) mbar_arrive(tempty_bar + acc);
          else mbar_arrive_remote(mapa_u32(smem_u32(tempty_bar + acc), 0));
        }
        continue;
      }
      float mu = 0.f, rstd = 1.f;  // a folded LayerNorm in front of this GEMM: the statistics of this thread's row
      if ((((FLAGS >= 0) ? FLAGS : flags) & EPI_LN_APPLY) && m0 + (warp & 3) * 32 + lane < M)
        ln_row_stats(ln.stats_in, m0 + (warp & 3) * 32 + lane, K / 128, K, mu, rstd);
      mbar_wait(tfull_bar + acc, acc_phase, abort_flag, err, SITE_TMEM_FULL);
      epilogue_tile<BN, FLAGS>(tmem_base + acc * BN, epi_stage + (warp - 2) * EPI_WARP_BYTES, sbias, sscale, warp,
                               (warp - 2) >> 2, lane, m0, n0, M, N, K, out, ldo, flags, residual, ln, mu, rstd);
      if (lane == 0) {
        if (leader) mbar_arrive(tempty_bar + acc);
        else mbar_arrive_remote(mapa_u32(smem_u32(tempty_bar + acc), 0));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  cluster_sync_all();  // neither CTA leaves while its peer may still signal its barriers or read its tiles
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

// One thread waits, with the pipeline's own bounded wait, on an mbarrier that nobody ever arrives
// on: the wait gives up after `limit_ns`, records the time-out in `err` exactly as a broken GEMM
// pipeline would, and the kernel returns.  Used to check the host's handling of that status.
__global__ void wait_timeout_probe_kernel(int* err, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
    mbar_wait(&bar, 0, &abort_flag, err, SITE_FULL, limit_ns);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Epilogue combinations compiled with the flags fixed (the ones the encoder uses; for CTA pairs
// also with the FP8 column scale); everything else runs the FLAGS = -1 instantiation.
constexpr int F_LIN = EPI_BIAS | EPI_OUT_F16 | EPI_IN_F16 | EPI_WSCALE;                  // QKV, attention-output, FFN2
constexpr int F_FFN1 = F_LIN | EPI_GELU;
constexpr int F_LIN8 = EPI_BIAS | EPI_OUT_F16 | EPI_IN_F16 | EPI_COLSCALE | EPI_W_FP8;   // the same in FP8-weight mode
constexpr int F_FFN18 = F_LIN8 | EPI_GELU;
constexpr int F_LIN8W = F_LIN8 & ~EPI_W_FP8;    // FP8-weight mode with the weights widened to fp16 at load
constexpr int F_FFN18W = F_FFN18 & ~EPI_W_FP8;
constexpr int F_LIN_LN = F_LIN | EPI_LN_APPLY;     // QKV after a folded LayerNorm
constexpr int F_FFN1_LN = F_FFN1 | EPI_LN_APPLY;   // FFN1 after a folded LayerNorm
// attention-output / FFN2 feeding a folded LayerNorm: fp32 sum out (+ fp16 operand, statistics), residual fp32 ...
constexpr int F_SUM = EPI_BIAS | EPI_IN_F16 | EPI_WSCALE | EPI_OUT_F32 | EPI_RESIDUAL | EPI_LN_SUM;
constexpr int F_SUM_RLN = F_SUM | EPI_RES_LN;      // ... or itself a folded LayerNorm's output
constexpr int F_S3 = EPI_BIAS | EPI_OUT_F32 | EPI_SPLIT3;   // fp32 mode on the tensor cores: QKV
constexpr int F_S3_RES = F_S3 | EPI_RESIDUAL;               // attention-output, FFN2 (+ fp32 residual)
constexpr int F_S3_FFN1 = F_S3 | EPI_GELU;

template <int BN, int FLAGS>
int launch_one(const CUtensorMap* tmA, const CUtensorMap* tmW, int M, int N, int K, void* out, int ldo,
               const GemmEpilogue& epi, int* err_flag, int num_sms, const int* m_dev, cudaStream_t stream) {
  using C = Cfg<BN>;
  static std::atomic<bool> attr_set[64] = {};  // per device; a repeated set by a racing thread is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, FLAGS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::SMEM_BYTES) != cudaSuccess)
      return -2;
    if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
  }
  const int tiles = ((M + BM - 1) / BM) * (N / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  return launch_pdl(gemm_tcgen05_kernel<BN, FLAGS>, dim3(grid), dim3(GEMM_THREADS), C::SMEM_BYTES, stream, *tmA, *tmW, M,
                    N, K, out, ldo, epi.flags, epi.bias, epi.residual, epi.colscale, err_flag, m_dev, epi.ln) == cudaSuccess
             ? 1 : -3;
}

template <int BN>
int launch(const CUtensorMap* tmA, const CUtensorMap* tmW, int M, int N, int K, void* out, int ldo,
           const GemmEpilogue& epi, int* err_flag, int num_sms, const int* m_dev, cudaStream_t stream) {
  switch (epi.flags) {
    case F_S3_RES:
      if (BN == 128) return launch_one<128, F_S3_RES>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, num_sms, m_dev, stream);
      break;
    default: break;
  }
  switch (epi.flags) {
    case F_LIN: return launch_one<BN, F_LIN>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, num_sms, m_dev, stream);
    case F_FFN1: return launch_one<BN, F_FFN1>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, num_sms, m_dev, stream);
    default: return launch_one<BN, -1>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, num_sms, m_dev, stream);
  }
}

// Number of CTA pairs that can be resident at once on this device (pairs need two SMs of one
// GPC); a persistent grid larger than that would run its last pairs after all the others.
template <int FLAGS, bool W8, int BN>
int max_resident_pairs(int dev) {
  static std::atomic<int> cached[64] = {};  // per device; racing threads compute the same value
  if (dev >= 0 && dev < 64 && cached[dev].load(std::memory_order_acquire) > 0) return cached[dev].load();
  using C = PairCfg<BN, W8>;
  if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<BN, FLAGS, W8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           C::SMEM_BYTES) != cudaSuccess)
    return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 148, 1, 1);
  cfg.blockDim = dim3(C::THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_pair_kernel<BN, FLAGS, W8>, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return -1;
  }
  if (dev >= 0 && dev < 64) cached[dev].store(n, std::memory_order_release);
  return n;
}

template <int FLAGS, bool W8 = false, int BN = 256>
int launch_pair_one(const CUtensorMap* tmA, const CUtensorMap* tmW, int M, int N, int K, void* out, int ldo,
                    const GemmEpilogue& epi, int* err_flag, const int* m_dev, cudaStream_t stream) {
  using C = PairCfg<BN, W8>;
  int dev = 0;
  cudaGetDevice(&dev);
  const int pairs = max_resident_pairs<FLAGS, W8, BN>(dev);
  if (pairs <= 0) return -2;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * (N / BN);
  const int grid = 2 * (tiles < pairs ? tiles : pairs);
  return launch_pdl(gemm_tcgen05_pair_kernel<BN, FLAGS, W8>, dim3(grid), dim3(C::THREADS), C::SMEM_BYTES, stream, *tmA,
                    *tmW, M, N, K, out, ldo, epi.flags, epi.bias, epi.residual, epi.colscale, err_flag, m_dev, epi.ln) ==
                 cudaSuccess ? 1 : -3;
}

int launch_pair(const CUtensorMap* tmA, const CUtensorMap* tmW, int M, int N, int K, void* out, int ldo,
                const GemmEpilogue& epi, int* err_flag, const int* m_dev, cudaStream_t stream) {
  switch (epi.flags) {
    case F_LIN: return launch_pair_one<F_LIN>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_FFN1: return launch_pair_one<F_FFN1>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_LIN8: return launch_pair_one<F_LIN8, true>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_FFN18: return launch_pair_one<F_FFN18, true>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_LIN8W: return launch_pair_one<F_LIN8W>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_FFN18W: return launch_pair_one<F_FFN18W>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_LIN_LN: return launch_pair_one<F_LIN_LN>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_FFN1_LN: return launch_pair_one<F_FFN1_LN>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_SUM: return launch_pair_one<F_SUM>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_SUM_RLN: return launch_pair_one<F_SUM_RLN>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_S3: return launch_pair_one<F_S3>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_S3_RES: return launch_pair_one<F_S3_RES>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    case F_S3_FFN1: return launch_pair_one<F_S3_FFN1>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    default:
      if (epi.flags & EPI_W_FP8) return launch_pair_one<-1, true>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
      return launch_pair_one<-1>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
  }
}

bool pair_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("CUDABERT_GEMM_PAIR");
    return !(e && e[0] == '0');
  }();
  return on;
}

}  // namespace

int wait_timeout_probe(int* err_flag, unsigned long long limit_ns, cudaStream_t stream) {
  if (!err_flag || limit_ns == 0 || limit_ns > WAIT_LIMIT_NS) return -1;
  wait_timeout_probe_kernel<<<1, 32, 0, stream>>>(err_flag, limit_ns);
  return cudaGetLastError() == cudaSuccess ? 1 : -3;
}

int gemm_block_n(int N) { return (N % 256 == 0) ? 256 : 128; }

// Tiles of the three-plane (fp32) GEMM.  Its k loop is six times as long, so with few rows the tiles of
// a narrow output are few and long: outputs of up to 1024 columns take single CTAs with 128 x 128
// tiles (four times as many, each half as long as a pair's), wider ones CTA pairs with 256 x 256.  The
// choice goes by N alone: what a row's result is must not depend on how many rows share its batch.
int gemm_split_block_n(int N) { return (N % 256 == 0 && N > 1024) ? 256 : 128; }
int gemm_split_w_box_rows(int N) { return 128; }  // half of a pair's 256-row tile, or all of a 128-row one

static bool small_tiles_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("CUDABERT_GEMM_SMALL_TILES");
    return e && e[0] == '1';
  }();
  return on;
}

bool gemm_uses_pairs(int N) { return pair_enabled() && (N % 256 == 0); }

// Rows of the W tensor map's box: a CTA of a pair loads half of the 256-row tile.
int gemm_w_box_rows(int N) { return gemm_uses_pairs(N) ? 128 : gemm_block_n(N); }

bool make_tmap_16bit_kmajor(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                           uint64_t row_stride_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) || box_rows == 0 || box_rows > 256)
    return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  // the copy moves 16-bit elements untouched (fp16 or bf16 alike); out-of-range elements read as zero bits
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool make_tmap_u8_kmajor(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (cols & 15)) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols};
  const cuuint32_t box[2] = {BK, 128};  // 64 bytes x the 128 rows one CTA of a pair converts per k-block
  const CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_NONE;
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int gemm_tcgen05(const CUtensorMap* tmA, const CUtensorMap* tmW, int M, int N, int K, void* out, int ldo,
                      const GemmEpilogue& epi, int* err_flag, int num_sms, const int* m_dev, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (N % 128) != 0 || (K % BK) != 0 || (ldo % 8) != 0) return -1;
  if ((epi.flags & EPI_BIAS) && !epi.bias) return -1;
  if ((epi.flags & EPI_RESIDUAL) && !epi.residual) return -1;
  if ((epi.flags & EPI_COLSCALE) && !epi.colscale) return -1;
  if ((epi.flags & EPI_SPLIT3) && (epi.flags & (EPI_IN_F16 | EPI_W_FP8))) return -1;  // the planes are bf16
  if (epi.flags & (EPI_LN_SUM | EPI_LN_APPLY | EPI_RES_LN)) {  // folded LayerNorm: see LnFold
    const LnFold& ln = epi.ln;
    if (epi.flags & EPI_SPLIT3) return -1;
    if ((epi.flags & EPI_LN_APPLY) && (!ln.stats_in || !ln.c || (K % 128) != 0)) return -1;  // one partial per 128 columns of A's LayerNorm input
    if (epi.flags & EPI_LN_SUM) {
      // one statistics slice per epilogue warp and row: 256-wide tiles, i.e. the CTA-pair kernel
      if (!ln.out16 || !ln.gamma || !ln.stats_out || !(epi.flags & EPI_OUT_F32) || (N % 256) != 0 || ldo != N) return -1;
      if (!gemm_uses_pairs(N) && gemm_block_n(N) != 256) return -1;
    }
    if ((epi.flags & EPI_RES_LN) &&
        (!ln.res_stats || !ln.res_gamma || !ln.res_beta || !(epi.flags & EPI_RESIDUAL) || !(epi.flags & EPI_OUT_F32)))
      return -1;
  }
  // Few rows: a CTA pair's 256 x 256 tiles are too few to occupy the SMs, and the k loop of one
  // tile is then the whole run time.  Single CTAs with 128 x 128 tiles have a k loop half as long
  // and four times as many tiles (BERT-base, 8 x 128 tokens: 0.80 against 0.88 ms per pass; one
  // sequence of 32 tokens: 0.71 against 0.78 ms).  It is opt-in (CUDABERT_GEMM_SMALL_TILES=1):
  // the two tile shapes do not round identically, so with it a sequence's result depends, in the
  // last bits, on how many other rows share its batch, and by default it never does.  The choice
  // compares (waves of tiles) x (tensor-pipe time of one tile's k loop) for the two shapes and takes
  // the small tiles only for a clear win.  The pair's W map has 128-row boxes, which is what the
  // 128 x 128 kernel loads too.
  if (epi.flags & EPI_W_FP8) {
    // E4M3 weight bytes: the CTA-pair kernel with converter warps is the one kernel that reads them
    if (N % 256 != 0 || !(epi.flags & EPI_IN_F16)) return -1;
    return launch_pair(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
  }
  if (epi.flags & EPI_SPLIT3) {  // tile shape by N alone (gemm_split_block_n)
    if (gemm_split_block_n(N) == 256) return launch_pair(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
    return launch<128>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, num_sms, m_dev, stream);
  }
  if (small_tiles_enabled() && gemm_uses_pairs(N) && gemm_w_box_rows(N) == 128 && !(epi.flags & EPI_LN_SUM)) {
    const long pairs = num_sms / 2 > 0 ? num_sms / 2 : 1;
    const long tiles_p = static_cast<long>((M + 2 * BM - 1) / (2 * BM)) * (N / 256);
    const long tiles_s = static_cast<long>((M + BM - 1) / BM) * (N / 128);
    const long cost_p = ((tiles_p + pairs - 1) / pairs) * 2;  // a 256 x 256 x 16 MMA takes twice a 128 x 128 x 16 one
    const long cost_s = (tiles_s + num_sms - 1) / num_sms;
    if (cost_s * 10 <= cost_p * 8)
      return launch<128>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, num_sms, m_dev, stream);
  }
  if (gemm_uses_pairs(N)) return launch_pair(tmA, tmW, M, N, K, out, ldo, epi, err_flag, m_dev, stream);
  if (gemm_block_n(N) == 256) return launch<256>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, num_sms, m_dev, stream);
  return launch<128>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, num_sms, m_dev, stream);
}

}  // namespace cb
