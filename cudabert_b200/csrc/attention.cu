// Fused masked scaled-dot-product attention: QK^T, 1/8 scale, additive key mask, softmax and
// P.V in one kernel, never materialising the [B, S, heads, S] score tensor.  It replaces
// Query_Key::forward (ops/batch_matmul.cu:24-82), op_SoftMax::forward / cuApplySoftmax
// (ops/softmax.cu:86-143) and Prob_Value::forward (ops/batch_matmul.cu:85-140) of the
// reference, and reads Q, K, V straight from the packed projection output [T, 3H].
//
// The 16-bit kernels take Q, K and V in fp16 and round the probabilities to fp16 (both operands of
// QK^T and of P.V are activations, and fp16 keeps three more significand
// bits than bf16); accumulation and the softmax are fp32, the output is fp16, the
// A-operand format of the attention-output GEMM.
//
// Mask semantics (ops/softmax.cu:97-101, modeling.py:237-240): score/8 + (1-mask[key])*-10000.
// A masked key's probability is exactly 0 in fp32 whenever the row has at least one valid key,
// so key tiles at or beyond kv_len[b] (all padding) are skipped.  A row with no valid key
// gives every key the same -10000, which softmax ignores: the kernels then attend to all keys.
#include "kernels.h"
#include "ptx.cuh"
#include "../../include/cudabert.h"

#include <atomic>
#include <cmath>
#include <mutex>

namespace cb {
namespace {

constexpr int HD = 64;  // head size
constexpr float LOG2E = 1.4426950408889634f;
constexpr int ATT_MAX_WARPS = 8;

// Shared-memory rows are 128 bytes (64 fp16); the 16-byte chunk c of row r lives at position
// c ^ (r & 7), which makes ldmatrix (8 consecutive rows, one chunk column) conflict-free without
// padding.
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4));
}

// Where the 64-row tiles (8 KB: 128-byte rows, chunk c of row r at c ^ (r & 7)) of an item's K and V
// live in shared memory: back to back (per-item kernel), or anywhere in a ring of tiles
// (persistent kernel).
struct ContigTiles {
  const uint8_t *sK, *sV;
  __device__ __forceinline__ const uint8_t* k(int t) const { return sK + t * 8192; }
  __device__ __forceinline__ const uint8_t* v(int t) const { return sV + t * 8192; }
};
struct RingTiles {
  const uint8_t* ring;
  int nt, k0, v0;  // ring size in tiles; ring index (< nt) of the item's first K tile and first V tile
  __device__ __forceinline__ const uint8_t* at(int i) const { return ring + (i >= nt ? i - nt : i) * 8192; }
  __device__ __forceinline__ const uint8_t* k(int t) const { return at(k0 + t); }
  __device__ __forceinline__ const uint8_t* v(int t) const { return at(v0 + t); }
};

// One block of MB x 16 queries of one (sequence, head) against the sequence's keys and values
// resident in shared memory: QK^T -> scale + mask bias -> online softmax -> P.V over 64-key tiles,
// then a coalesced store of the (MB x 16) x 64 block.  Run by one warp.  With MB = 2 every K / V
// fragment a warp loads with ldmatrix feeds four MMAs instead of two and the warp has twice as
// many independent accumulator chains, at twice the registers (so half as many warps fit).
// `stage` is MB x 2 KB of shared memory that only this warp touches while it works on the block.
// The queries come either from global memory (`sQ` null: `base` points at the first Q element (fp16) of
// the sequence's first row, row stride `ld`; they pass through `stage`) or from shared memory
// (`sQ`: the block's own rows of a Q tile, which may be `stage` itself).  `out_base` points at the
// sequence's first output element (row stride `H`).  Bit t of `biased` says that key tile t needs
// the bias in `sBias`.
template <int MB, bool Q_IN_SMEM, typename Tiles>
__device__ __forceinline__ void attend_qblock(const Tiles tiles, const float* __restrict__ sBias, unsigned int biased,
                                              uint8_t* __restrict__ stage, const uint8_t* __restrict__ sQ,
                                              const __half* __restrict__ base, int ld,
                                              __half* __restrict__ out_base, int H, int q0, int nq,
                                              int ktiles, int lane) {
  const float scale = 0.125f * LOG2E;
  uint32_t qf[MB][4][4];
  if (Q_IN_SMEM) {
    // rows at or beyond nq hold other rows' (finite) values; their results are never stored
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        ldmatrix_x4(qf[mb][kk], smem_u32(sQ + swz(mb * 16 + (lane & 15), kk * 2 + (lane >> 4))));
  } else {
    // stage the Q block: lane l moves chunk l % 8 of rows l / 8 + 4 i
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4 * MB; ++i) {
      const int r = (lane >> 3) + 4 * i, c = lane & 7;
      uint4 t = make_uint4(0u, 0u, 0u, 0u);
      if (q0 + r < nq) t = __ldg(reinterpret_cast<const uint4*>(base + static_cast<size_t>(q0 + r) * ld + c * 8));
      *reinterpret_cast<uint4*>(stage + swz(r, c)) = t;
    }
    __syncwarp();
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        ldmatrix_x4(qf[mb][kk], smem_u32(stage + swz(mb * 16 + (lane & 15), kk * 2 + (lane >> 4))));
  }

  float o[MB][8][4];
  float m_run[MB][2], l_run[MB][2];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb) {
#pragma unroll
    for (int i = 0; i < 8; ++i) o[mb][i][0] = o[mb][i][1] = o[mb][i][2] = o[mb][i][3] = 0.f;
    m_run[mb][0] = m_run[mb][1] = -INFINITY;
    l_run[mb][0] = l_run[mb][1] = 0.f;
  }

  for (int t = 0; t < ktiles; ++t) {
    const int k0 = t << 6;
    const uint8_t* kt = tiles.k(t);
    const uint8_t* vt = tiles.v(t);
    // S = Q K^T for 64 keys: 8 n-tiles of 8 keys
    float s[MB][8][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < 8; ++i) s[mb][i][0] = s[mb][i][1] = s[mb][i][2] = s[mb][i][3] = 0.f;
    const int mid = lane >> 3;
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t kf[4];
        ldmatrix_x4(kf, smem_u32(kt + swz(nb * 16 + (mid >> 1) * 8 + (lane & 7), kk * 2 + (mid & 1))));
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          mma_f16_16816(s[mb][2 * nb], qf[mb][kk], kf[0], kf[1]);
          mma_f16_16816(s[mb][2 * nb + 1], qf[mb][kk], kf[2], kf[3]);
        }
      }
    }
    // running max of the scores in the log2 domain.  A tile whose keys are all valid keeps the
    // raw dot products (the scale is folded into the exponential's multiply-add below); any
    // other tile gets scale and mask bias applied here.
    const bool plain = ((biased >> t) & 1u) == 0u;
    const float e_scale = plain ? scale : 1.0f;  // p = 2^(s * e_scale - m)
    uint32_t pf[MB][4][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      float tmax[2] = {-INFINITY, -INFINITY};
      if (plain) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          tmax[0] = fmaxf(tmax[0], fmaxf(s[mb][i][0], s[mb][i][1]));
          tmax[1] = fmaxf(tmax[1], fmaxf(s[mb][i][2], s[mb][i][3]));
        }
        tmax[0] *= scale;  // scale > 0: max(scale * s) = scale * max(s)
        tmax[1] *= scale;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 bb = *reinterpret_cast<const float2*>(sBias + k0 + i * 8 + 2 * (lane & 3));
          s[mb][i][0] = fmaf(s[mb][i][0], scale, bb.x);
          s[mb][i][1] = fmaf(s[mb][i][1], scale, bb.y);
          s[mb][i][2] = fmaf(s[mb][i][2], scale, bb.x);
          s[mb][i][3] = fmaf(s[mb][i][3], scale, bb.y);
          tmax[0] = fmaxf(tmax[0], fmaxf(s[mb][i][0], s[mb][i][1]));
          tmax[1] = fmaxf(tmax[1], fmaxf(s[mb][i][2], s[mb][i][3]));
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
      }
      float alpha[2], m_new[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        m_new[r] = fmaxf(m_run[mb][r], tmax[r]);
        // tile 0 always holds key 0 with a finite bias, so m_new is finite from the first tile on
        alpha[r] = ex2_approx(m_run[mb][r] - m_new[r]);
        m_run[mb][r] = m_new[r];
        l_run[mb][r] *= alpha[r];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float p0 = ex2_approx(fmaf(s[mb][i][0], e_scale, -m_new[0]));
        const float p1 = ex2_approx(fmaf(s[mb][i][1], e_scale, -m_new[0]));
        const float p2 = ex2_approx(fmaf(s[mb][i][2], e_scale, -m_new[1]));
        const float p3 = ex2_approx(fmaf(s[mb][i][3], e_scale, -m_new[1]));
        l_run[mb][0] += p0 + p1;
        l_run[mb][1] += p2 + p3;
        pf[mb][i >> 1][(i & 1) * 2] = pack_f16(p0, p1);
        pf[mb][i >> 1][(i & 1) * 2 + 1] = pack_f16(p2, p3);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        o[mb][i][0] *= alpha[0]; o[mb][i][1] *= alpha[0];
        o[mb][i][2] *= alpha[1]; o[mb][i][3] *= alpha[1];
      }
    }
    // O += P V : 4 key steps of 16, 4 pairs of 8-wide d tiles
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int db = 0; db < 4; ++db) {
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, smem_u32(vt + swz(j * 16 + (mid & 1) * 8 + (lane & 7), db * 2 + (mid >> 1))));
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          mma_f16_16816(o[mb][2 * db], pf[mb][j], vf[0], vf[1]);
          mma_f16_16816(o[mb][2 * db + 1], pf[mb][j], vf[2], vf[3]);
        }
      }
    }
  }

  // stage the output block in the Q buffer, then store it with 16-byte row-contiguous pieces
  __syncwarp();
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int mb = 0; mb < MB; ++mb) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[mb][r] += __shfl_xor_sync(0xffffffffu, l_run[mb][r], 1);
      l_run[mb][r] += __shfl_xor_sync(0xffffffffu, l_run[mb][r], 2);
    }
    const float inv0 = 1.0f / l_run[mb][0], inv1 = 1.0f / l_run[mb][1];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // columns i*8 + 2*t4, +1 of rows g and g + 8: chunk i, byte offset 4 * t4 inside the chunk
      *reinterpret_cast<uint32_t*>(stage + swz(mb * 16 + g, i) + 4 * t4) =
          pack_f16(o[mb][i][0] * inv0, o[mb][i][1] * inv0);
      *reinterpret_cast<uint32_t*>(stage + swz(mb * 16 + g + 8, i) + 4 * t4) =
          pack_f16(o[mb][i][2] * inv1, o[mb][i][3] * inv1);
    }
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4 * MB; ++i) {
    const int r = (lane >> 3) + 4 * i, c = lane & 7;
    if (q0 + r < nq)
      *reinterpret_cast<uint4*>(out_base + static_cast<size_t>(q0 + r) * H + c * 8) =
          *reinterpret_cast<const uint4*>(stage + swz(r, c));
  }
}

// One CTA per (batch row, head).  All keys and values the row can attend to (kv_len[b], rounded
// up to 16) are loaded into shared memory once; then every warp takes 16-query blocks
// (warp, warp + nwarps, ...) and runs QK^T -> scale + mask bias -> online softmax -> P.V over 64-key
// tiles entirely out of shared memory, with no further block-wide synchronisation.
//   smem: K [R][64] | V [R][64] | per-warp Q / O staging [16][64] | bias [R]   (R = keys rounded to 64)
__global__ void __launch_bounds__(ATT_MAX_WARPS * 32, 2)
attention_f16_kernel(const __half* __restrict__ qkv, const int* __restrict__ mask,
                      const int* __restrict__ kv_len, const int* __restrict__ row_start,
                      __half* __restrict__ ctx, int S, int heads, int R, int cls_only) {
  extern __shared__ __align__(1024) uint8_t att_smem[];
  uint8_t* sK = att_smem;
  uint8_t* sV = sK + static_cast<size_t>(R) * 128;
  uint8_t* sQ = sV + static_cast<size_t>(R) * 128;
  const int nwarps = blockDim.x >> 5;
  float* sBias = reinterpret_cast<float*>(sQ + nwarps * 2048);
  __shared__ unsigned int s_biased;  // bit t: 64-key tile t holds a masked key or lies partly beyond klen

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int H = heads * HD, ld = 3 * H;
  griddep_wait();
  griddep_launch();
  int klen = kv_len[b];
  const bool use_mask = (klen > 0) && (mask != nullptr);
  if (klen <= 0) klen = S;
  // rows of this sequence: [first, first + nq).  Packed: only the klen rows that exist; else all S.
  const int first = row_start ? row_start[b] : b * S;
  // cls_only: only the sequence's first query is wanted, and its result goes to output row b
  const int nq = cls_only ? 1 : (row_start ? klen : S);
  const int ktiles = (klen + 63) >> 6;
  const int krows = ktiles << 6;  // rows of K / V the tiles touch; rows >= klen are zero-filled
  const __half* base = qkv + static_cast<size_t>(first) * ld + h * HD;

  for (int i = tid; i < krows * 8; i += blockDim.x) {
    const int r = i >> 3, c = i & 7;
    const bool ok = r < klen;
    const __half* src = base + static_cast<size_t>(ok ? r : 0) * ld + c * 8;
    cp_async16(smem_u32(sK + swz(r, c)), src + H, ok);
    cp_async16(smem_u32(sV + swz(r, c)), src + 2 * H, ok);
  }
  cp_async_commit();
  const int* mrow = mask ? mask + static_cast<size_t>(b) * S : nullptr;
  if (tid == 0) s_biased = 0u;
  __syncthreads();
  unsigned int bits = 0u;
  for (int key = tid; key < krows; key += blockDim.x) {
    float v = 0.f;
    if (key >= klen) v = -INFINITY;
    else if (use_mask && mrow[key] == 0) v = -10000.0f * LOG2E;
    sBias[key] = v;
    if (v != 0.f) bits |= 1u << (key >> 6);
  }
  if (bits) atomicOr(&s_biased, bits);
  cp_async_wait<0>();
  __syncthreads();
  const unsigned int biased = s_biased;

  uint8_t* myQ = sQ + warp * 2048;
  const int qblocks = (nq + 15) >> 4;
  __half* out_base = ctx + static_cast<size_t>(cls_only ? b : first) * H + h * HD;
  for (int qb = warp; qb < qblocks; qb += nwarps)
    attend_qblock<1, false>(ContigTiles{sK, sV}, sBias, biased, myQ, nullptr, base, ld, out_base, H, qb * 16, nq,
                            ktiles, lane);
}

// ---------------------------------------------------------------- persistent variant
// The same arithmetic as attention_f16_kernel (attend_qblock), scheduled differently.  With one
// CTA per (sequence, head) a short sequence leaves most of the CTA's warps without a query block
// while they still hold their registers, and every CTA first waits for its keys and values before
// any warp computes.  Here one persistent CTA per SM keeps 15 consumer warps busy and a producer
// warp several items ahead:
//   items      (sequence, head) pairs in descending order of sequence length (`sched`, made by
//              row_layout), dealt round-robin to the CTAs: every CTA gets the same mix of long and
//              short items, the long ones first, and nothing about the order has to be fetched
//              with an atomic, so the producer can look up a batch of 32 items' lengths and row
//              offsets in one go, one item per lane;
//   memory     a ring of 8 KB tiles (64 rows x 128 bytes, 128-byte swizzle = the layout swz()
//              describes) holds the K, V and Q rows of up to 8 items in flight; an item takes
//              exactly the tiles its length needs (3 for up to 64 rows, 12 for 193..256), so many
//              short items or two of the longest are resident at once;
//   producer   per item: waits (oldest item first) until enough tiles and an item record are
//              free, writes the per-key bias (reading the mask only for a sequence that has
//              masked keys below its last valid one), and issues the TMA box copies, which all
//              complete on the record's `full` mbarrier, so no consumer waits on a global load;
//   consumers  wait for `full`, then draw query blocks of the item from a shared-memory
//              counter until none is left, arrive on `empty` and move to the next record, so a
//              warp that finds no block in a short item is already working on the next one.  A
//              block's output is staged in the block's own Q rows, which nobody else reads.
// Rows of a K / V tile beyond the sequence's last key hold whatever follows in the buffer (finite
// activations of other rows, or zero fill beyond the tensor); their bias is -inf, so their
// probability is 0.
// Work unit of a consumer warp: PA_MB 16-query blocks.  Measured per layer on the benchmark workload
// (S = 200, lengths 16..200): 15 warps x 1 block 57 us, 7 warps x 2 blocks (254 registers) 59 us; the
// two tie within a few percent on every shape tried, so the kernel keeps the smaller unit, which
// wastes less on ragged lengths.
constexpr int PA_MB = 1;
constexpr int PA_QROWS = PA_MB * 16;
constexpr int PA_CONSUMERS = PA_MB == 1 ? 15 : 7;  // what the register file holds at 128 / 254 registers
constexpr int PA_THREADS = (PA_CONSUMERS + 1) * 32;
constexpr int PA_MAX_R = 256;   // longest sequence: two of them (12 tiles each) fit in the ring
constexpr int PA_RECORDS = 8;   // items in flight
constexpr int PA_TAIL_BYTES = 640;  // item records, mbarriers, abort flag
constexpr size_t PA_SMEM_LIMIT = 232448;
enum : int { SITE_PA_FULL = 21, SITE_PA_EMPTY = 22 };

struct PaItem {
  int first, nq, ktiles, qblocks, h, done;  // first: the sequence's first row in qkv
  unsigned int biased;
  int next_q;  // next query block to hand out
  int tile0;   // ring index of the item's first tile: K tiles, then V tiles, then Q tiles
  int out_row; // first output row of the item
  int pad[2];
};
static_assert(sizeof(PaItem) == 48, "record layout");

constexpr int pa_ring_tiles(int R) {
  return static_cast<int>((PA_SMEM_LIMIT - 1024 - PA_TAIL_BYTES - static_cast<size_t>(PA_RECORDS) * R * 4) / 8192);
}
constexpr size_t pa_smem_bytes(int R) {
  return static_cast<size_t>(pa_ring_tiles(R)) * 8192 + static_cast<size_t>(PA_RECORDS) * R * 4 + PA_TAIL_BYTES + 1024;
}
static_assert(pa_ring_tiles(PA_MAX_R) >= 24, "two items of the largest supported length must fit");

__global__ void __launch_bounds__(PA_THREADS, 1)
attention_f16_persist_kernel(const __grid_constant__ CUtensorMap tmQKV, const int* __restrict__ mask,
                              const int* __restrict__ kv_len, const int* __restrict__ row_start,
                              const int* __restrict__ sched, __half* __restrict__ ctx, int B, int S, int heads,
                              int R, int NT, int cls_only, int* __restrict__ err) {
  extern __shared__ uint8_t pa_smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pa_smem_raw) + 1023) & ~uintptr_t(1023));
  float* sBiasAll = reinterpret_cast<float*>(ring + static_cast<size_t>(NT) * 8192);
  uint8_t* tail = reinterpret_cast<uint8_t*>(sBiasAll + static_cast<size_t>(PA_RECORDS) * R);
  PaItem* items = reinterpret_cast<PaItem*>(tail);              // [PA_RECORDS], 48 bytes each
  uint64_t* full = reinterpret_cast<uint64_t*>(tail + 384);     // [PA_RECORDS]
  uint64_t* empty = full + PA_RECORDS;                          // [PA_RECORDS]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + PA_RECORDS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < PA_RECORDS; ++i) {
      mbar_init(full + i, 1);
      mbar_init(empty + i, PA_CONSUMERS);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQKV);
  }
  __syncthreads();
  griddep_wait();
  griddep_launch();
  const int H = heads * HD;
  const long long num_items = static_cast<long long>(B) * heads;

  if (warp == PA_CONSUMERS) {
    // All lanes keep the same bookkeeping (it is warp-uniform).  Records are used round-robin;
    // `oldest` is the record of the oldest item whose tiles have not been taken back yet.
    int rec = 0, oldest = 0, outstanding = 0;
    int head = 0, free_tiles = NT;
    unsigned int wait_parity = 0u;  // bit r: parity that completes the current use of empty[r]
    unsigned int rec_tiles_lo = 0u, rec_tiles_hi = 0u;  // 4 bits per record: tiles it holds (<= 12)
    auto get_tiles = [&](int r) { return static_cast<int>(((r < 4 ? rec_tiles_lo >> (8 * r) : rec_tiles_hi >> (8 * (r - 4)))) & 0xffu); };
    auto set_tiles = [&](int r, int n) {
      if (r < 4) rec_tiles_lo = (rec_tiles_lo & ~(0xffu << (8 * r))) | (static_cast<unsigned int>(n) << (8 * r));
      else rec_tiles_hi = (rec_tiles_hi & ~(0xffu << (8 * (r - 4)))) | (static_cast<unsigned int>(n) << (8 * (r - 4)));
    };
    // take back the oldest item's tiles once every consumer warp has left it
    auto reclaim_oldest = [&]() -> bool {
      if (!mbar_wait(empty + oldest, (wait_parity >> oldest) & 1u, abort_flag, err, SITE_PA_EMPTY)) return false;
      wait_parity ^= 1u << oldest;
      free_tiles += get_tiles(oldest);
      --outstanding;
      if (++oldest == PA_RECORDS) oldest = 0;
      return true;
    };
    bool running = true;
    for (long long it0 = 0; running; it0 += 32) {
      // this CTA's next 32 items, one per lane
      const long long idx = blockIdx.x + (it0 + lane) * static_cast<long long>(gridDim.x);
      const bool valid = idx < num_items;
      int my_h = 0, my_klen = 0, my_first = 0, my_nq = 0, my_b = 0, my_mask = 0;
      if (valid) {
        const int r = static_cast<int>(idx / heads);
        my_h = static_cast<int>(idx - static_cast<long long>(r) * heads);
        my_b = sched ? sched[r] : r;
        int klen = kv_len[my_b];
        // the mask row is read only if it exists, the row has a valid key, and (when known) it has holes
        my_mask = (klen > 0 && mask != nullptr && (!sched || sched[B + my_b] != 0)) ? 1 : 0;
        if (klen <= 0) klen = S;
        my_klen = klen;
        my_first = row_start ? row_start[my_b] : my_b * S;
        my_nq = cls_only ? 1 : (row_start ? klen : S);  // cls_only: the first query alone, result to row b
      }
      for (int j = 0; j < 32 && running; ++j) {
        const bool more = __shfl_sync(0xffffffffu, valid ? 1 : 0, j) != 0;
        const int h = __shfl_sync(0xffffffffu, my_h, j), b = __shfl_sync(0xffffffffu, my_b, j);
        const int klen = __shfl_sync(0xffffffffu, my_klen, j), first = __shfl_sync(0xffffffffu, my_first, j);
        const int nq = __shfl_sync(0xffffffffu, my_nq, j), read_mask = __shfl_sync(0xffffffffu, my_mask, j);
        const int ktiles = (klen + 63) >> 6, qtiles = (nq + 63) >> 6;
        const int need = more ? 2 * ktiles + qtiles : 0;
        while (running && outstanding > 0 && (outstanding == PA_RECORDS || free_tiles < need)) running = reclaim_oldest();
        if (!running) break;
        PaItem* pi = items + rec;
        if (!more) {  // no item left for this CTA: tell the consumers and stop
          if (lane == 0) {
            pi->done = 1;
            mbar_arrive(full + rec);
          }
          running = false;
          break;
        }
        const int krows = ktiles << 6;
        float* sBias = sBiasAll + static_cast<size_t>(rec) * R;
        const int* mrow = mask + static_cast<size_t>(b) * S;
        unsigned int bits = 0u;
        for (int key = lane; key < krows; key += 32) {
          float v = 0.f;
          if (key >= klen) v = -INFINITY;
          else if (read_mask && mrow[key] == 0) v = -10000.0f * LOG2E;
          sBias[key] = v;
          if (v != 0.f) bits |= 1u << (key >> 6);
        }
        bits = __reduce_or_sync(0xffffffffu, bits);
        __syncwarp();  // the bias written by all lanes is ordered before lane 0's arrive below
        if (lane == 0) {
          pi->first = first;
          pi->nq = nq;
          pi->ktiles = ktiles;
          pi->qblocks = (nq + PA_QROWS - 1) / PA_QROWS;
          pi->h = h;
          pi->done = 0;
          pi->biased = bits;
          pi->next_q = 0;
          pi->tile0 = head;
          pi->out_row = cls_only ? b : first;
          mbar_arrive_expect_tx(full + rec, static_cast<uint32_t>(need) * 8192u);
          int t_idx = head;
          auto next_tile = [&]() { uint8_t* p = ring + static_cast<size_t>(t_idx) * 8192; if (++t_idx == NT) t_idx = 0; return p; };
          for (int t = 0; t < ktiles; ++t) tma_load_2d(next_tile(), &tmQKV, full + rec, H + h * HD, first + t * 64);
          for (int t = 0; t < ktiles; ++t) tma_load_2d(next_tile(), &tmQKV, full + rec, 2 * H + h * HD, first + t * 64);
          for (int t = 0; t < qtiles; ++t) tma_load_2d(next_tile(), &tmQKV, full + rec, h * HD, first + t * 64);
        }
        head += need;
        if (head >= NT) head -= NT;
        free_tiles -= need;
        set_tiles(rec, need);
        ++outstanding;
        if (++rec == PA_RECORDS) rec = 0;
      }
    }
  } else {
    int rec = 0;
    uint32_t phase = 0;
    for (;;) {
      if (!mbar_wait(full + rec, phase, abort_flag, err, SITE_PA_FULL)) break;
      PaItem* pi = items + rec;
      if (pi->done) break;
      const int first = pi->first, nq = pi->nq, ktiles = pi->ktiles, qblocks = pi->qblocks, h = pi->h;
      const unsigned int biased = pi->biased;
      const int tile0 = pi->tile0, out_row = pi->out_row;
      RingTiles tiles;
      tiles.ring = ring;
      tiles.nt = NT;
      tiles.k0 = tile0;
      tiles.v0 = tile0 + ktiles >= NT ? tile0 + ktiles - NT : tile0 + ktiles;
      const int q_first = tiles.v0 + ktiles >= NT ? tiles.v0 + ktiles - NT : tiles.v0 + ktiles;
      const float* sBias = sBiasAll + static_cast<size_t>(rec) * R;
      __half* out_base = ctx + static_cast<size_t>(out_row) * H + h * HD;
      for (;;) {
        int qb = 0;
        if (lane == 0) qb = atomicAdd(&pi->next_q, 1);
        qb = __shfl_sync(0xffffffffu, qb, 0);
        if (qb >= qblocks) break;
        // the block's query rows inside the item's Q tiles (a tile holds 64 / PA_QROWS blocks)
        constexpr int PER_TILE = 64 / PA_QROWS;
        uint8_t* qrows = const_cast<uint8_t*>(tiles.at(q_first + qb / PER_TILE)) + (qb % PER_TILE) * (PA_QROWS * 128);
        attend_qblock<PA_MB, true>(tiles, sBias, biased, qrows, qrows, nullptr, 0, out_base, H, qb * PA_QROWS, nq,
                                   ktiles, lane);
      }
      __syncwarp();  // every lane has finished with the item's tiles
      if (lane == 0) mbar_arrive(empty + rec);
      if (++rec == PA_RECORDS) { rec = 0; phase ^= 1; }
    }
  }

  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: give copies that may still be in flight time to land before shared memory is released
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
}

// ---------------------------------------------------------------- fp32 path
constexpr int FQ = 32;  // queries per CTA: 8 warps x 4 queries
constexpr int FK = 32;  // keys per chunk: one per lane

__global__ void __launch_bounds__(256)
attention_f32_kernel(const float* __restrict__ qkv, const int* __restrict__ mask, const int* __restrict__ kv_len,
                     const int* __restrict__ row_start, float* __restrict__ ctx, int S, int heads) {
  __shared__ float sQ[FQ][HD];
  __shared__ float sK[FK][HD + 1];
  __shared__ float sV[FK][HD];
  __shared__ float sBias[FK];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q0 = blockIdx.x * FQ, h = blockIdx.y, b = blockIdx.z;
  const int H = heads * HD, ld = 3 * H;
  griddep_wait();
  griddep_launch();
  int klen = kv_len[b];
  const bool use_mask = (klen > 0) && (mask != nullptr);
  if (klen <= 0) klen = S;
  const int first = row_start ? row_start[b] : b * S;
  const int nq = row_start ? klen : S;
  if (q0 >= nq) return;
  const float* base = qkv + static_cast<size_t>(first) * ld + h * HD;
  const int* mrow = mask ? mask + static_cast<size_t>(b) * S : nullptr;

  for (int i = tid; i < FQ * HD; i += 256) {
    const int r = i / HD, c = i % HD;
    sQ[r][c] = (q0 + r < nq) ? base[static_cast<size_t>(q0 + r) * ld + c] : 0.f;
  }
  float m_run[4], l_run[4], o0[4], o1[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) { m_run[q] = -INFINITY; l_run[q] = 0.f; o0[q] = 0.f; o1[q] = 0.f; }

  for (int k0 = 0; k0 < klen; k0 += FK) {
    __syncthreads();
    for (int i = tid; i < FK * HD; i += 256) {
      const int r = i / HD, c = i % HD;
      const bool ok = (k0 + r) < klen;
      sK[r][c] = ok ? base[static_cast<size_t>(k0 + r) * ld + H + c] : 0.f;
      sV[r][c] = ok ? base[static_cast<size_t>(k0 + r) * ld + 2 * H + c] : 0.f;
    }
    if (tid < FK) {
      const int key = k0 + tid;
      float v = 0.f;
      if (key >= klen) v = -INFINITY;
      else if (use_mask && mrow[key] == 0) v = -10000.0f;
      sBias[tid] = v;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float* qr = sQ[warp * 4 + q];
      float s = 0.f;
#pragma unroll 16
      for (int d = 0; d < HD; ++d) s = fmaf(qr[d], sK[lane][d], s);
      s = s * 0.125f + sBias[lane];
      float mx = s;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_new = fmaxf(m_run[q], mx);
      const float alpha = expf(m_run[q] - m_new);
      const float p = expf(s - m_new);
      float ps = p;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
      l_run[q] = l_run[q] * alpha + ps;
      m_run[q] = m_new;
      float a0 = o0[q] * alpha, a1 = o1[q] * alpha;
#pragma unroll
      for (int j = 0; j < FK; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        a0 = fmaf(pj, sV[j][lane], a0);
        a1 = fmaf(pj, sV[j][lane + 32], a1);
      }
      o0[q] = a0;
      o1[q] = a1;
    }
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int row = q0 + warp * 4 + q;
    if (row < nq) {
      float* dst = ctx + (static_cast<size_t>(first) + row) * H + h * HD;
      dst[lane] = o0[q] / l_run[q];
      dst[lane + 32] = o1[q] / l_run[q];
    }
  }
}

// One block.  kv_len[b] = 1 + index of the last non-zero mask entry of row b (0 if none; S if
// mask is null).  With `row_start` (B + 1 entries) it also lays the sequences out back to back:
// row_start[b] = sum of the lengths of the rows before b, a row of length 0 (no valid key: it
// attends to everything) counting as S; row_start[B] is the number of packed rows.  With `sched`
// it also prepares the persistent attention kernel's work order: sched[r] = the sequence of rank r
// when sequences are sorted by descending length (counting sort; the order among equal lengths is
// arbitrary and only affects scheduling), and sched[B + b] = 1 if row b has a masked key below its
// last valid one (only then does attention have to read the mask).
// With both, sched[2 B + t] = the sequence that packed row 128 t belongs to, for every t with
// 128 t < row_start[B] (the tcgen05 attention kernel's tiles); `sched` then holds
// 2 B + ceil(B S / 128) entries.
__global__ void __launch_bounds__(1024)
row_layout_kernel(const int* __restrict__ mask, int* __restrict__ kv_len, int* __restrict__ row_start,
                  int* __restrict__ sched, int B, int S) {
  __shared__ int warp_tot[32];
  __shared__ int carry;
  __shared__ int hist[544];  // bin 512 - length; 17 bins per lane of warp 0
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  griddep_wait();
  griddep_launch();
  for (int b = warp; b < B; b += 32) {
    int last = 0, holes = 0;
    if (mask == nullptr) {
      last = S;
    } else {
      const int* row = mask + static_cast<size_t>(b) * S;
      for (int i = lane; i < S; i += 32)
        if (row[i] != 0) last = i + 1;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, off));
      if (sched) {
        for (int i = lane; i < last; i += 32)
          if (row[i] == 0) holes = 1;
        holes = __any_sync(0xffffffffu, holes);
      }
    }
    if (lane == 0) {
      kv_len[b] = last;
      if (sched) sched[B + b] = holes;
    }
  }
  if (sched) {
    for (int i = tid; i < 544; i += 1024) hist[i] = 0;
    __syncthreads();  // also orders the kv_len writes above before the reads below
    for (int b = tid; b < B; b += 1024) {
      int v = kv_len[b];
      if (v <= 0 || v > 512) v = min(S, 512);
      atomicAdd(&hist[512 - v], 1);
    }
    __syncthreads();
    if (warp == 0) {  // exclusive prefix sum over the 544 bins
      int local[17], sum = 0;
#pragma unroll
      for (int i = 0; i < 17; ++i) { local[i] = hist[lane * 17 + i]; sum += local[i]; }
      int incl = sum;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += n;
      }
      int run = incl - sum;
#pragma unroll
      for (int i = 0; i < 17; ++i) { hist[lane * 17 + i] = run; run += local[i]; }
    }
    __syncthreads();
    for (int b = tid; b < B; b += 1024) {
      int v = kv_len[b];
      if (v <= 0 || v > 512) v = min(S, 512);
      sched[atomicAdd(&hist[512 - v], 1)] = b;
    }
  }
  if (row_start == nullptr) return;
  if (tid == 0) carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < B; b0 += 1024) {
    const int b = b0 + tid;
    int v = 0;
    if (b < B) {
      v = kv_len[b];
      if (v <= 0) v = S;
    }
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += n;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = warp_tot[lane];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, w, off);
        if (lane >= off) w += n;
      }
      warp_tot[lane] = w;  // inclusive totals of the warps
    }
    __syncthreads();
    const int before = carry + (warp > 0 ? warp_tot[warp - 1] : 0) + incl - v;
    if (b < B) row_start[b] = before;
    __syncthreads();
    if (tid == 1023) carry = before + v;
    __syncthreads();
  }
  if (tid == 0) row_start[B] = carry;
  if (sched) {
    // tile table: the sequence that row 128 t of the packed layout belongs to
    __syncthreads();  // row_start, written above by other threads of this block, is read below
    for (int b = tid; b < B; b += 1024) {
      const int lo = row_start[b], hi = row_start[b + 1];
      for (int t = (lo + 127) / 128; t * 128 < hi; ++t) sched[2 * B + t] = b;
    }
  }
}

}  // namespace

int attention_f16(const __half* qkv, const int* mask, const int* kv_len, const int* row_start,
                   __half* ctx, int B, int S, int heads, int cls_only, cudaStream_t stream) {
  if (B <= 0 || S <= 0 || S > 512 || heads <= 0 || B > 65535) return -1;
  const int R = ((S + 63) / 64) * 64;
  const int qblocks = (S + 15) / 16;
  const int nwarps = qblocks < ATT_MAX_WARPS ? qblocks : ATT_MAX_WARPS;
  const size_t smem = static_cast<size_t>(R) * 256 + nwarps * 2048 + static_cast<size_t>(R) * 4;
  static std::atomic<bool> attr_set[64] = {};  // per device; a repeated set by a racing thread is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
    const size_t want = 512 * 256 + ATT_MAX_WARPS * 2048 + 512 * 4;  // the largest S
    if (cudaFuncSetAttribute(attention_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(want)) != cudaSuccess)
      return -2;
    if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
  }
  dim3 grid(heads, B);
  return launch_pdl(attention_f16_kernel, grid, dim3(nwarps * 32), smem, stream, qkv, mask, kv_len, row_start, ctx, S,
                    heads, R, cls_only) == cudaSuccess ? 1 : -3;
}

bool attention_persist_fits(int S) { return ((S + 63) / 64) * 64 <= PA_MAX_R; }

int attention_f16_persist(const CUtensorMap* tm_qkv, const int* mask, const int* kv_len, const int* row_start,
                           const int* sched, __half* ctx, int B, int S, int heads, int num_sms, int cls_only,
                           int* err_flag, cudaStream_t stream) {
  if (B <= 0 || S <= 0 || heads <= 0 || !attention_persist_fits(S)) return -1;
  const int R = ((S + 63) / 64) * 64;
  const int NT = pa_ring_tiles(R);
  static std::atomic<bool> attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(attention_f16_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(PA_SMEM_LIMIT)) != cudaSuccess)
      return -2;
    if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
  }
  const long long items = static_cast<long long>(B) * heads;
  const int grid = static_cast<int>(items < num_sms ? items : num_sms);
  return launch_pdl(attention_f16_persist_kernel, dim3(grid), dim3(PA_THREADS), pa_smem_bytes(R), stream, *tm_qkv, mask,
                    kv_len, row_start, sched, ctx, B, S, heads, R, NT, cls_only, err_flag) == cudaSuccess ? 1 : -3;
}

int attention_f32(const float* qkv, const int* mask, const int* kv_len, const int* row_start, float* ctx, int B,
                  int S, int heads, cudaStream_t stream) {
  if (B <= 0 || S <= 0 || heads <= 0 || B > 65535) return -1;
  dim3 grid((S + FQ - 1) / FQ, heads, B);
  return launch_pdl(attention_f32_kernel, grid, dim3(256), 0, stream, qkv, mask, kv_len, row_start, ctx, S, heads) ==
                 cudaSuccess ? 1 : -3;
}

int row_layout(const int* mask, int* kv_len, int* row_start, int* sched, int B, int S, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return -1;
  return launch_pdl(row_layout_kernel, dim3(1), dim3(1024), 0, stream, mask, kv_len, row_start, sched, B, S) == cudaSuccess
             ? 1 : -3;
}

}  // namespace cb

// ---------------------------------------------------------------- entry point without allocation
// Scratch of cudabert_k_attention_noalloc: the per-row key counts that cudabert_k_attention keeps
// in a buffer it allocates per call.  It lives in the library image, so every GPU that loads the
// library holds CUDABERT_NOALLOC_MAX_BATCH * 4 bytes (16 KiB) of it until the process exits.
static __device__ __align__(256) int g_noalloc_kv_len[CUDABERT_NOALLOC_MAX_BATCH];

extern "C" int cudabert_k_attention_noalloc(int kernel_code, const void* qkv_dev, const int* mask_dev, void* ctx_dev, int B,
                                            int S, int heads) {
  // Everything is validated before the first launch: a kernel number this entry point cannot serve
  // must not fall through to another kernel that would write a differently shaped output.
  if (!qkv_dev || !ctx_dev || B <= 0 || S <= 0 || heads <= 0) {
    cb::set_thread_error("cudabert_k_attention_noalloc: null buffer or non-positive size");
    return 1;
  }
  const int cls_only = (kernel_code & 16) ? 1 : 0;  // + 16: first query of every sequence only, ctx is [B, H]
  const int kernel = kernel_code & ~16;
  if (kernel != 0 && kernel != 1) {
    cb::set_thread_error("cudabert_k_attention_noalloc: only kernels 0 (fp32) and 1 (16-bit mma.sync, optionally + 16) "
                         "are served; kernels 2 and 3 need scheduling and error scratch beyond the built-in array");
    return 1;
  }
  if (cls_only && kernel == 0) {
    cb::set_thread_error("cudabert_k_attention_noalloc: + 16 (first query only) needs a 16-bit kernel");
    return 1;
  }
  if (kernel == 1 && S > 512) {
    cb::set_thread_error("cudabert_k_attention_noalloc: the 16-bit kernel holds sequences of up to 512 keys");
    return 1;
  }
  if (B > CUDABERT_NOALLOC_MAX_BATCH) {
    cb::set_thread_error("cudabert_k_attention_noalloc: batch exceeds CUDABERT_NOALLOC_MAX_BATCH (4096), the size "
                         "of the built-in scratch; use cudabert_k_attention or split the batch");
    return 6;
  }
  // In host code the array's name is only a handle for the runtime, not an address a kernel can
  // use; the device address is looked up once per device, with that device current.
  static std::mutex mu;
  static int* scratch_of_device[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cb::set_thread_error("cudabert_k_attention_noalloc: no current CUDA device");
    return 2;
  }
  int* kv = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!scratch_of_device[dev]) {
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_kv_len);
      if (e != cudaSuccess || !p) {
        cb::set_thread_error(std::string("cudabert_k_attention_noalloc: cudaGetSymbolAddress failed: ") +
                             cudaGetErrorString(e));
        return 2;
      }
      scratch_of_device[dev] = static_cast<int*>(p);
    }
    kv = scratch_of_device[dev];
  }
  // every entry [0, B) is rewritten before it is read, so nothing left by an earlier call matters
  int n = cb::row_layout(mask_dev, kv, nullptr, nullptr, B, S, nullptr);
  if (n >= 0)
    n = kernel ? cb::attention_f16(static_cast<const __half*>(qkv_dev), mask_dev, kv, nullptr,
                                    static_cast<__half*>(ctx_dev), B, S, heads, cls_only, nullptr)
               : cb::attention_f32(static_cast<const float*>(qkv_dev), mask_dev, kv, nullptr,
                                   static_cast<float*>(ctx_dev), B, S, heads, nullptr);
  if (n < 0) {
    cb::set_thread_error("cudabert_k_attention_noalloc: kernel launch rejected (code " + std::to_string(n) + ")");
    return 3;
  }
  const cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cb::set_thread_error(std::string("cudabert_k_attention_noalloc: ") + cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
