// Dense projection GEMM for sm_100a: out[M, N] = A[M, K] x W[N, K]^T with a fused epilogue.
//
// It replaces, for the bf16 / FP8-weight modes, the reference's cuBLAS SGEMM calls and the
// kernels around them: the bias pre-fill `MemoryCpyLinear` (ops/linear.cu:23-27), the GEMMs
// of `op_BatchedLinear::forward` (ops/linear.cu:241-319) and `op_Linear::forward`
// (ops/linear.cu:91-148), the GELU sweep (ops/elementwise.cu:38-51), the residual add that
// `cuApplyLayerNorm` does in place (ops/layernorm.cu:152-158) and the pooler's tanh
// (ops/elementwise.cu:57-70).
//
// Structure (one persistent CTA per SM, 192 threads, no clusters, no multicast):
//   warp 0, one lane   TMA producer: per k-block one 128x64 tile of A and one BNx64 tile of W
//                      (128-byte swizzle) into a ring of shared-memory stages guarded by
//                      full/empty mbarriers.
//   warp 1, one lane   issues tcgen05.mma (128 x BN x 16, bf16 in, fp32 accumulate in TMEM);
//                      tcgen05.commit releases a stage back to the producer and, after the
//                      last k-block, hands the accumulator to the epilogue.
//   warps 2-5          epilogue: tcgen05.ld of the accumulator (each warp owns the TMEM lane
//                      quarter warp_id % 4), bias / column scale / residual / GELU / tanh in
//                      registers, 16-byte stores.  Two accumulators (2 x BN TMEM columns) let
//                      the epilogue of tile i overlap the MMAs of tile i+1.
#include "kernels.h"
#include "ptx.cuh"

#include <cstdio>
#include <mutex>

namespace cb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

template <int BN>
struct Cfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // 1024: alignment slack
};

__device__ __forceinline__ float gelu_erf(float x) {
  return x * 0.5f * (1.0f + erff(x * 0.70710678118654752f));
}

// 32 consecutive output columns of one row: scale, bias, residual, activation, store.
template <bool OUT_F32>
__device__ __forceinline__ void epilogue_row32(const uint32_t (&v)[32], int flags, const float* __restrict__ bias,
                                               const float* __restrict__ colscale, const void* __restrict__ residual,
                                               void* __restrict__ out, size_t row_off, int col) {
  float f[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
  if (flags & EPI_COLSCALE) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 s = __ldg(reinterpret_cast<const float4*>(colscale + col + j));
      f[j] *= s.x; f[j + 1] *= s.y; f[j + 2] *= s.z; f[j + 3] *= s.w;
    }
  }
  if (flags & EPI_BIAS) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 b = __ldg(reinterpret_cast<const float4*>(bias + col + j));
      f[j] += b.x; f[j + 1] += b.y; f[j + 2] += b.z; f[j + 3] += b.w;
    }
  }
  if (flags & EPI_RESIDUAL) {
    if (OUT_F32) {
      const float4* r = reinterpret_cast<const float4*>(static_cast<const float*>(residual) + row_off + col);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 t = __ldg(r + j);
        f[4 * j] += t.x; f[4 * j + 1] += t.y; f[4 * j + 2] += t.z; f[4 * j + 3] += t.w;
      }
    } else {
      const uint4* r = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(residual) + row_off + col);
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
  if (flags & EPI_GELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = gelu_erf(f[j]);
  }
  if (flags & EPI_TANH) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = tanhf(f[j]);
  }
  if (OUT_F32) {
    float4* o = reinterpret_cast<float4*>(static_cast<float*>(out) + row_off + col);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
  } else {
    uint4* o = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out) + row_off + col);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 t;
      t.x = pack_bf16(f[8 * j], f[8 * j + 1]);
      t.y = pack_bf16(f[8 * j + 2], f[8 * j + 3]);
      t.z = pack_bf16(f[8 * j + 4], f[8 * j + 5]);
      t.w = pack_bf16(f[8 * j + 6], f[8 * j + 7]);
      o[j] = t;
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, int M, int N,
                    int K, void* __restrict__ out, int ldo, int flags, const float* __restrict__ bias,
                    const void* __restrict__ residual, const float* __restrict__ colscale, int* err) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
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
      mbar_init(tempty_bar + a, 4);  // one arrival per epilogue warp
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

  const int tiles_n = N / BN;
  const int tiles_m = (M + BM - 1) / BM;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = K / BK;

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
          tma_load_2d(sa, &tmA, full_bar + stage, kb * BK, m0);
          tma_load_2d(sa + C::A_BYTES, &tmW, full_bar + stage, kb * BK, n0);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
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
            umma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          }
          umma_commit(empty_bar + stage);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(tfull_bar + acc);
      }
    }
  } else {
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32) belong to this warp
    const int row_in_tile = quarter * 32 + lane;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int m0 = (tile / tiles_n) * BM;
      const int n0 = (tile % tiles_n) * BN;
      mbar_wait(tfull_bar + acc, acc_phase, abort_flag, err, SITE_TMEM_FULL);
      tc_fence_after();
      const int row = m0 + row_in_tile;
      const bool valid = row < M;
      const size_t row_off = static_cast<size_t>(row) * ldo;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(t_row + c * 32, v);
        tmem_ld_wait();
        if (valid) {
          if (flags & EPI_OUT_F32)
            epilogue_row32<true>(v, flags, bias, colscale, residual, out, row_off, n0 + c * 32);
          else
            epilogue_row32<false>(v, flags, bias, colscale, residual, out, row_off, n0 + c * 32);
        }
      }
      tc_fence_before();
      __syncwarp();
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

template <int BN>
int launch(const CUtensorMap* tmA, const CUtensorMap* tmW, int M, int N, int K, void* out, int ldo,
           const GemmEpilogue& epi, int* err_flag, int num_sms, cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) !=
        cudaSuccess)
      return -2;
    attr_set[dev] = true;
  }
  const int tiles = ((M + BM - 1) / BM) * (N / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_tcgen05_kernel<BN><<<grid, GEMM_THREADS, C::SMEM_BYTES, stream>>>(
      *tmA, *tmW, M, N, K, out, ldo, epi.flags, epi.bias, epi.residual, epi.colscale, err_flag);
  return cudaGetLastError() == cudaSuccess ? 1 : -3;
}

}  // namespace

int gemm_block_n(int N) { return (N % 256 == 0) ? 256 : 128; }

bool make_tmap_bf16_kmajor(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                           uint64_t row_stride_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) || box_rows == 0 || box_rows > 256)
    return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int gemm_bf16_tcgen05(const CUtensorMap* tmA, const CUtensorMap* tmW, int M, int N, int K, void* out, int ldo,
                      const GemmEpilogue& epi, int* err_flag, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (N % 128) != 0 || (K % BK) != 0 || (ldo % 8) != 0) return -1;
  if ((epi.flags & EPI_BIAS) && !epi.bias) return -1;
  if ((epi.flags & EPI_RESIDUAL) && !epi.residual) return -1;
  if ((epi.flags & EPI_COLSCALE) && !epi.colscale) return -1;
  if (gemm_block_n(N) == 256) return launch<256>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, num_sms, stream);
  return launch<128>(tmA, tmW, M, N, K, out, ldo, epi, err_flag, num_sms, stream);
}

}  // namespace cb
