// Fused masked attention on the tcgen05 tensor cores (16-bit modes: fp16 Q, K, V in, fp16 context out).  Same contract as
// attention_f16 in attention.cu (which stays as the `mma.sync` variant): QK^T, 1/8 scale, additive
// key mask, softmax, P.V in one kernel, keys at or beyond kv_len[b] never touched.  Replaces
// Query_Key::forward (ops/batch_matmul.cu:24-82), cuApplySoftmax (ops/softmax.cu:86-143) and
// Prob_Value::forward (ops/batch_matmul.cu:85-140) of the reference.
//
// Persistent CTAs (two per SM) walk over work items: a tile of 128 query rows of one head, either of
// one sequence or, in the packed row layout, of whatever sequences 128 consecutive rows belong to (see
// Cursor).  Per item, for every step (a block of up to 64 keys of one sequence):
//   warp 4, one lane   TMA: Q tile (once per item), K block, V block -> shared memory (128-byte
//                      swizzle), two buffers each; a buffer is re-filled as soon as the MMAs that
//                      read it have completed (tcgen05.commit on its "empty" barrier).
//   warp 5, one lane   S = Q K^T   tcgen05.mma 128 x 64 x 16 (x4 over d = 64) into one of two S
//                      buffers in TMEM, issued one step AHEAD so that it runs while the softmax
//                      warps work; after they have written P: O (+)= P V, 128 x 64 x 16 (x4 over
//                      the 64 keys), V used as an MN-major operand straight from its [key][d]
//                      rows, O in TMEM columns [128, 192) or [192, 256), alternating between items.
//   warps 0-3          thread = query row = TMEM lane: scale, keys beyond the sequence cut by index
//                      (the mask row is read only for sequences with masked keys below their last
//                      valid one), row max (no shuffles: the whole row belongs to the thread),
//                      online-softmax correction of O in TMEM when a later key block raises the
//                      max, P = exp2(x - max) as fp16 into the swizzled A-operand tile in shared
//                      memory; O / sum -> fp16 -> coalesced stores one item late, while the next
//                      item's first step is in the tensor core.
// Every wait is bounded (ptx.cuh): a broken pipeline ends with an error flag, not a hang.
#include "kernels.h"
#include "ptx.cuh"

#include <atomic>
#include <cstdlib>

namespace cb {
namespace {

constexpr int HD = 64;
constexpr int TQ = 128;  // queries per item
constexpr int TK = 64;   // keys per block
constexpr float LOG2E = 1.4426950408889634f;
constexpr int ATC_THREADS = 192;
constexpr int Q_BYTES = TQ * 128;   // 128 query rows x 128 bytes (64 fp16)
constexpr int KV_BYTES = TK * 128;  // 64 key rows x 128 bytes
constexpr int P_BYTES = TQ * 128;   // 128 query rows x 64 keys (fp16)
// Q, K and V are double-buffered so that the loads and the QK^T of the next block (or item) run
// while the softmax warps work on the current one.
constexpr int SMEM_Q = 0, SMEM_K = 2 * Q_BYTES, SMEM_V = SMEM_K + 2 * KV_BYTES, SMEM_P = SMEM_V + 2 * KV_BYTES;
constexpr int SMEM_STAGE = SMEM_P + P_BYTES;
constexpr int STAGE_BYTES = TQ * 128;  // output staging: 128 rows x 64 fp16
constexpr int SMEM_BAR = SMEM_STAGE + STAGE_BYTES;
constexpr int ATC_SMEM = SMEM_BAR + 256 + 1024;  // + barriers + alignment slack: 97 KB, two CTAs per SM
// S buffers in columns [0, 64) and [64, 128); two O accumulators in [128, 192) and [192, 256), used by
// alternate items so that the output of one item is read while the next one accumulates
constexpr uint32_t TMEM_COLS = 256;
constexpr int ATC_PACKED_MAX_S = 80;  // padded lengths up to this prefer packed tiles to the persistent kernel
constexpr uint32_t S_COL = 0, O_COL = 128;

enum { SITE_ATT_Q = 10, SITE_ATT_K, SITE_ATT_V, SITE_ATT_S, SITE_ATT_P, SITE_ATT_O, SITE_ATT_E };

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory descriptor of an MN-major 16-bit operand stored as rows of 64 elements (128 bytes,
// 128-byte swizzle), one row per K index: 8-row groups are 1024 bytes apart (stride byte offset);
// the leading byte offset (distance between 64-element groups along MN) is unused for N = 64.
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3fff) | (64ull << 16) | (64ull << 32) | (1ull << 46) |
         (2ull << 61);
}
// Instruction descriptor: D fp32, A fp16 K-major, B fp16 MN-major, shape M x N (x 16).
__host__ __device__ constexpr uint32_t umma_idesc_f16_bmn(int m, int n) {
  return umma_idesc_f16(m, n) | (1u << 16);
}

// Position of one role (loader, MMA issuer, softmax warps) in this CTA's work: an item is a tile of
// 128 query rows of one head, a step is a block of up to 64 keys of ONE sequence.
//   per-sequence items (MULTI = false): (sequence, head, 128-query tile); the tile's rows all belong
//     to the sequence and its steps are that sequence's key blocks.  Used when the rows are not
//     packed and for the pass that wants only the first query of every sequence.
//   packed tiles (MULTI = true): (tile of 128 consecutive packed rows, head); the tile may hold rows
//     of several sequences, and its steps are the key blocks of every sequence it cuts, in order.  A
//     row takes part only in the steps of its own sequence (its probabilities are zero in the
//     others), so it sees exactly the blocks, in the order and with the contents, that it sees in a
//     per-sequence item: the results are the same bits, whatever the other rows of the batch are.
struct Cursor {
  int item, items_done, blocks_done;
  bool valid;
  // item
  int h, q_row, out_row, n_out, q_end, ji;  // head; first query row in the QKV buffer; first output row; rows to
                                            // store; (MULTI) end of the tile's rows; step index within the item
  // sequence of the current step
  int seq, ks, ke, nb, jb;  // its rows (= keys) [ks, ke) in the QKV buffer, its key blocks, the current one
  bool use_mask;            // some key below its last valid one is masked: the mask row has to be read
};

template <bool MULTI>
__global__ void __launch_bounds__(ATC_THREADS, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmQKV, const int* __restrict__ mask,
                    const int* __restrict__ kv_len, const int* __restrict__ row_start,
                    const int* __restrict__ sched, __half* __restrict__ ctx, int B, int S, int heads, int cls_only,
                    int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BAR);
  uint64_t *q_full = bars, *q_empty = bars + 2, *k_full = bars + 4, *k_empty = bars + 6, *v_full = bars + 8,
           *v_empty = bars + 10, *s_full = bars + 12, *p_full = bars + 14, *o_full = bars + 15;  // [2] each but the last two
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 14; ++i) mbar_init(bars + i, 1);
    mbar_init(p_full, 4);  // one arrival per softmax warp
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQKV);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  griddep_wait();
  griddep_launch();

  const int H = heads * HD;
  const int QT = (S + TQ - 1) / TQ;                                     // query tiles of a sequence
  const int R = MULTI ? row_start[B] : 0;                               // packed rows (written by row_layout)
  const int tiles = (R + TQ - 1) / TQ;                                  // (MULTI) tiles of 128 packed rows
  const int num_items = MULTI ? tiles * heads : B * heads * QT;

  // Every role walks the same steps and derives buffer indices and barrier parities from the same
  // counters (items_done, blocks_done).
  auto cursor_seek = [&](Cursor& c) {  // position on the first live item at or after c.item
    c.valid = false;
    c.ji = 0;
    c.jb = 0;
    if constexpr (MULTI) {
      // tiles run fastest: neighbouring CTAs work on neighbouring tiles of one head, which share the
      // keys and values of the sequence cut between them
      if (c.item >= num_items) return;
      const int t = c.item % tiles;
      c.h = c.item / tiles;
      c.q_row = c.out_row = t * TQ;
      c.n_out = R - t * TQ;
      c.q_end = min(t * TQ + TQ, R);
      c.seq = sched[2 * B + t];  // the sequence the tile's first row belongs to
      c.ks = row_start[c.seq];
      c.ke = row_start[c.seq + 1];
      c.nb = (c.ke - c.ks + TK - 1) / TK;
      c.use_mask = mask != nullptr && sched[B + c.seq] != 0;
      c.valid = true;
    } else {
      while (c.item < num_items) {
        const int q0 = (c.item % QT) * TQ, b = c.item / (QT * heads);
        int klen = kv_len[b];
        // with `sched` (from row_layout) the mask is read only for rows flagged as having holes
        c.use_mask = klen > 0 && mask != nullptr && (!sched || sched[B + b] != 0);
        if (klen <= 0) klen = S;  // no valid key: the row attends to everything
        const int nq = cls_only ? 1 : (row_start ? klen : S);
        if (q0 < nq) {
          c.h = (c.item / QT) % heads;
          c.seq = b;
          c.ks = row_start ? row_start[b] : b * S;
          c.ke = c.ks + klen;
          c.nb = (klen + TK - 1) / TK;
          c.q_row = c.ks + q0;
          c.out_row = cls_only ? b : c.q_row;  // first queries alone: one output row per sequence
          c.n_out = nq - q0;
          c.q_end = c.ke;
          c.valid = true;
          break;
        }
        c.item += gridDim.x;
      }
    }
  };
  auto cursor_last = [&](const Cursor& c) {  // the step under c is the last one of its item
    return c.jb == c.nb - 1 && (!MULTI || c.ke >= c.q_end);
  };
  auto cursor_next = [&](Cursor& c) {
    ++c.blocks_done;
    ++c.ji;
    if (++c.jb < c.nb) return;
    if (MULTI && c.ke < c.q_end) {  // the tile goes on into the next sequence
      ++c.seq;
      c.ks = c.ke;
      c.ke = row_start[c.seq + 1];
      c.nb = (c.ke - c.ks + TK - 1) / TK;
      c.use_mask = mask != nullptr && sched[B + c.seq] != 0;
      c.jb = 0;
      return;
    }
    ++c.items_done;
    c.item += gridDim.x;
    cursor_seek(c);
  };

  if (warp == 4) {
    if (lane == 0) {
      Cursor c{};
      c.item = static_cast<int>(blockIdx.x);
      for (cursor_seek(c); c.valid; cursor_next(c)) {
        if (c.ji == 0) {
          const int qb = c.items_done & 1;
          mbar_wait(q_empty + qb, ((c.items_done >> 1) & 1) ^ 1, abort_flag, err, SITE_ATT_E);
          mbar_arrive_expect_tx(q_full + qb, Q_BYTES);  // two 64-row boxes
          tma_load_2d(smem + SMEM_Q + qb * Q_BYTES, &tmQKV, q_full + qb, c.h * HD, c.q_row);
          tma_load_2d(smem + SMEM_Q + qb * Q_BYTES + Q_BYTES / 2, &tmQKV, q_full + qb, c.h * HD, c.q_row + 64);
        }
        const int kb = c.blocks_done & 1;
        const uint32_t par = ((c.blocks_done >> 1) & 1) ^ 1;
        mbar_wait(k_empty + kb, par, abort_flag, err, SITE_ATT_E);
        mbar_arrive_expect_tx(k_full + kb, KV_BYTES);
        tma_load_2d(smem + SMEM_K + kb * KV_BYTES, &tmQKV, k_full + kb, H + c.h * HD, c.ks + c.jb * TK);
        mbar_wait(v_empty + kb, par, abort_flag, err, SITE_ATT_E);
        mbar_arrive_expect_tx(v_full + kb, KV_BYTES);
        tma_load_2d(smem + SMEM_V + kb * KV_BYTES, &tmQKV, v_full + kb, 2 * H + c.h * HD, c.ks + c.jb * TK);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(TQ, TK);
      constexpr uint32_t idesc_o = umma_idesc_f16_bmn(TQ, HD);
      const uint32_t sq = smem_u32(smem + SMEM_Q), sk = smem_u32(smem + SMEM_K), sv = smem_u32(smem + SMEM_V),
                     sp = smem_u32(smem + SMEM_P);
      // S = Q K^T of the block under `c` into S buffer blocks_done & 1.  That buffer was last read by
      // the softmax of block blocks_done - 2, whose p_full this thread has already waited for.
      auto issue_s = [&](const Cursor& c) {
        const int qb = c.items_done & 1, kb = c.blocks_done & 1;
        if (c.ji == 0) mbar_wait(q_full + qb, (c.items_done >> 1) & 1, abort_flag, err, SITE_ATT_Q);
        mbar_wait(k_full + kb, (c.blocks_done >> 1) & 1, abort_flag, err, SITE_ATT_K);
        tc_fence_after();
        const uint64_t da = umma_desc_sw128(sq + qb * Q_BYTES), db = umma_desc_sw128(sk + kb * KV_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_f16(tmem_base + S_COL + kb * TK, da + 2 * k, db + 2 * k, idesc_s, k != 0);
        umma_commit(s_full + kb);
        umma_commit(k_empty + kb);
        if (cursor_last(c)) umma_commit(q_empty + qb);
      };
      // O (+)= P V over the block's 64 keys: A = P (K-major over the keys), B = V rows (MN-major)
      auto issue_pv = [&](const Cursor& c) {
        const int vb = c.blocks_done & 1;
        mbar_wait(v_full + vb, (c.blocks_done >> 1) & 1, abort_flag, err, SITE_ATT_V);
        mbar_wait(p_full, c.blocks_done & 1, abort_flag, err, SITE_ATT_P);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < TK / 16; ++k) {
          const uint64_t da = umma_desc_sw128(sp) + 2 * k;
          const uint64_t db = umma_desc_sw128_mn(sv + vb * KV_BYTES) + static_cast<uint64_t>(k) * (2048 >> 4);
          umma_f16(tmem_base + O_COL + (c.items_done & 1) * HD, da, db, idesc_o, (c.ji | k) != 0);
        }
        umma_commit(o_full);
        umma_commit(v_empty + vb);
      };
      Cursor cs{};
      cs.item = static_cast<int>(blockIdx.x);
      cursor_seek(cs);
      Cursor cp = cs;
      if (cs.valid) {
        issue_s(cs);
        cursor_next(cs);
      }
      while (cp.valid) {
        if (cs.valid) {  // the next block's QK^T runs while the softmax warps work on this one
          issue_s(cs);
          cursor_next(cs);
        }
        issue_pv(cp);
        cursor_next(cp);
      }
    }
  } else {
    // softmax warps 0-3: thread r owns query row r of the tile and TMEM lane r
    const int r = threadIdx.x;  // 0..127
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    uint8_t* my_p = smem + SMEM_P + r * 128;           // this row's 64 probabilities of the block
    uint8_t* stage = smem + SMEM_STAGE + warp * 4096;  // output staging: this warp's 32 rows x 128 B
    const float scale = 0.125f * LOG2E;
    uint32_t o_waits = 0;  // completions of o_full consumed so far
    float m_run = -INFINITY, l_run = 0.f;
    // The output of an item is written one step late: its last P.V runs while these warps already
    // work on the first key block of the next item (the two items accumulate in different TMEM
    // columns), and the finished accumulator is read, normalised and stored right after that block's
    // probabilities have been handed to the tensor core.  Per item this takes the P.V latency, the
    // TMEM read and the stores off the path the next MMA waits on.
    bool prev = false;  // an item's output is pending
    float prev_inv = 0.f;
    int prev_n = 0;
    __half* prev_out = nullptr;
    uint32_t prev_ocol = 0;
    auto finish_prev = [&]() {  // its last P.V has completed (o_full waited for): O / l -> fp16 -> staging -> stores
      uint8_t* my_row = stage + lane * 128;
      uint32_t ov[2][32];
      tmem_ld32(t_lane + prev_ocol, ov[0]);
      tmem_ld32(t_lane + prev_ocol + 32, ov[1]);
      tmem_ld_wait();
#pragma unroll
      for (int ch = 0; ch < HD / 32; ++ch) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 t;
          t.x = pack_f16(__uint_as_float(ov[ch][8 * q]) * prev_inv, __uint_as_float(ov[ch][8 * q + 1]) * prev_inv);
          t.y = pack_f16(__uint_as_float(ov[ch][8 * q + 2]) * prev_inv, __uint_as_float(ov[ch][8 * q + 3]) * prev_inv);
          t.z = pack_f16(__uint_as_float(ov[ch][8 * q + 4]) * prev_inv, __uint_as_float(ov[ch][8 * q + 5]) * prev_inv);
          t.w = pack_f16(__uint_as_float(ov[ch][8 * q + 6]) * prev_inv, __uint_as_float(ov[ch][8 * q + 7]) * prev_inv);
          *reinterpret_cast<uint4*>(my_row + (((ch * 4 + q) ^ (lane & 7)) << 4)) = t;
        }
      }
      tc_fence_before();  // the accumulator's next writer (an MMA two items on) comes after these reads
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = i * 4 + (lane >> 3), p2 = lane & 7;
        const int row = warp * 32 + rr;  // row of the tile
        const uint4 t = *reinterpret_cast<const uint4*>(stage + rr * 128 + (p2 << 4));
        if (row < prev_n)
          *reinterpret_cast<uint4*>(prev_out + static_cast<size_t>(row) * H + ((p2 ^ (rr & 7)) << 3)) = t;
      }
      __syncwarp();  // the staging rows are free for the next item
    };
    Cursor c{};
    c.item = static_cast<int>(blockIdx.x);
    for (cursor_seek(c); c.valid; cursor_next(c)) {
      const uint32_t t_s = t_lane + S_COL + (c.blocks_done & 1) * TK;
      const uint32_t t_o = t_lane + O_COL + (c.items_done & 1) * HD;
      // In a packed tile a row takes part only in the steps of its own sequence; elsewhere its
      // probabilities are zero and its running maximum and sum stay as they are.
      const bool member = !MULTI || (c.q_row + r >= c.ks && c.q_row + r < c.ke);
      const bool warp_in = !MULTI || __any_sync(0xffffffffu, member);
      // plain: every key of the block is valid.  Only the last block of a sequence can hold keys
      // beyond its length, and which ones follows from the length alone.  A sequence with masked keys
      // below its last valid one (rare) takes the mask row from global memory, every lane the same word.
      const int tail = c.ke - c.ks - c.jb * TK;  // keys of this block that exist (>= 64: all)
      const bool plain = !c.use_mask && tail >= TK;
      mbar_wait(s_full + (c.blocks_done & 1), (c.blocks_done >> 1) & 1, abort_flag, err, SITE_ATT_S);
      tc_fence_after();
      float alpha = 1.0f;
      uint4 pk[8];
      if (warp_in) {
      // the 64 scores of the row: one TMEM round trip, kept in registers for both steps
      uint32_t v[2][32];
      tmem_ld32(t_s, v[0]);
      tmem_ld32(t_s + 32, v[1]);
      tmem_ld_wait();
      // four independent chains for the maximum (and below for the sum): a single chain of 64
      // dependent operations would leave the two warps an SM sub-partition holds mostly stalled;
      // three-input maxima and packed pairs for the multiply-adds and the sums
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (plain) {
#pragma unroll
        for (int ch = 0; ch < 2; ++ch)
#pragma unroll
          for (int i = 0; i < 32; i += 8)
#pragma unroll
            for (int q = 0; q < 4; ++q)
              mx4[q] = max3(mx4[q], __uint_as_float(v[ch][i + 2 * q]), __uint_as_float(v[ch][i + 2 * q + 1]));
#pragma unroll
        for (int q = 0; q < 4; ++q) mx4[q] *= scale;  // the scale itself is folded into the exponential below
      } else if (c.use_mask) {
        const int* mk = mask + static_cast<size_t>(c.seq) * S + c.jb * TK;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float bias = -INFINITY;  // additive, log2 domain
            if (ch * 32 + i < tail) bias = __ldg(mk + ch * 32 + i) == 0 ? -10000.0f * LOG2E : 0.f;
            const float x = fmaf(__uint_as_float(v[ch][i]), scale, bias);
            v[ch][i] = __float_as_uint(x);
            mx4[i & 3] = fmaxf(mx4[i & 3], x);
          }
      } else {
        // last block of a sequence without masked keys: keys at or beyond `tail` do not exist
#pragma unroll
        for (int ch = 0; ch < 2; ++ch)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float x = (ch * 32 + i < tail) ? __uint_as_float(v[ch][i]) * scale : -INFINITY;
            v[ch][i] = __float_as_uint(x);
            mx4[i & 3] = fmaxf(mx4[i & 3], x);
          }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // Reference point of the exponentials.  It only has to keep exp2 in range, so it follows the
      // running maximum lazily: it moves (and O is rescaled in TMEM, a round trip) only when a block
      // exceeds it by more than 8 in the log2 domain; until then probabilities may reach 2^8, which
      // fp16 and the fp32 sums hold without loss.  The first block of a sequence sets it exactly.
      float m_new = m_run, l_new = l_run;
      if (c.jb == 0) {
        m_new = mx;  // finite: key 0 of block 0 is never masked with -inf
        l_new = 0.f;
      } else if (mx > m_run + 8.0f) {
        alpha = ex2_approx(m_run - mx);
        m_new = mx;
        l_new *= alpha;
      }
      // P = exp2(x - max) in registers first: nothing below depends on the previous P.V yet
      uint64_t l2[2] = {0ull, 0ull};  // two packed pairs of partial sums
      const float e_scale = plain ? scale : 1.0f;  // plain blocks still hold the raw dot products
      const uint64_t es2 = pack_f32x2(e_scale, e_scale), nm2 = pack_f32x2(-m_new, -m_new);
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a, b;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[ch][i]), __uint_as_float(v[ch][i + 1])), es2, nm2), a, b);
          p[i] = ex2_approx(a);
          p[i + 1] = ex2_approx(b);
          l2[(i >> 1) & 1] = add_f32x2(l2[(i >> 1) & 1], pack_f32x2(p[i], p[i + 1]));
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          pk[ch * 4 + q].x = pack_f16(p[8 * q], p[8 * q + 1]);
          pk[ch * 4 + q].y = pack_f16(p[8 * q + 2], p[8 * q + 3]);
          pk[ch * 4 + q].z = pack_f16(p[8 * q + 4], p[8 * q + 5]);
          pk[ch * 4 + q].w = pack_f16(p[8 * q + 6], p[8 * q + 7]);
        }
      }
      float l4[4];
      unpack_f32x2(l2[0], l4[0], l4[1]);
      unpack_f32x2(l2[1], l4[2], l4[3]);
      l_new += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      if (member) {
        m_run = m_new;
        l_run = l_new;
      } else {  // a row of another sequence: what was computed from its scores is dropped
        alpha = 1.0f;
#pragma unroll
        for (int q = 0; q < 8; ++q) pk[q] = make_uint4(0u, 0u, 0u, 0u);
      }
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) pk[q] = make_uint4(0u, 0u, 0u, 0u);
      }
      // The P tile (and, for a rescale, O) may be touched only after the P.V that last read it has
      // completed: the previous step's, or the last step's of the previous item.
      if (c.ji > 0 || prev) {
        mbar_wait(o_full, o_waits & 1, abort_flag, err, SITE_ATT_O);
        ++o_waits;
        tc_fence_after();
      }
      if (c.ji > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        uint32_t o[2][32];
        tmem_ld32(t_o, o[0]);
        tmem_ld32(t_o + 32, o[1]);
        tmem_ld_wait();
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[ch][i] = __float_as_uint(__uint_as_float(o[ch][i]) * alpha);
          tmem_st32(t_o + ch * 32, o[ch]);
        }
        tmem_st_wait();
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(my_p + ((q ^ (r & 7)) << 4)) = pk[q];
      fence_proxy_async_smem();  // the tensor core reads P through the async proxy
      tc_fence_before();
      __syncwarp();              // every lane's rows are written and fenced: one arrival for the warp
      if (lane == 0) mbar_arrive(p_full);
      if (c.ji == 0 && prev) {   // the previous item's accumulator is complete (waited for above)
        finish_prev();
        prev = false;
      }
      if (cursor_last(c)) {
        prev = true;
        prev_inv = 1.0f / l_run;
        prev_out = ctx + static_cast<size_t>(c.out_row) * H + c.h * HD;
        prev_n = c.n_out;
        prev_ocol = O_COL + (c.items_done & 1) * HD;
      }
    }
    if (prev) {
      mbar_wait(o_full, o_waits & 1, abort_flag, err, SITE_ATT_O);
      tc_fence_after();
      finish_prev();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

// Which 16-bit attention kernel a forward pass of padded length S uses.  The tcgen05 kernel works on
// 128-query tiles of 64-key blocks whatever the number of live rows in them.  With one sequence per
// tile it wins where the tiles are full and loses where a batch's rows are much shorter than the
// tile grid; with packed tiles (rows of several sequences in one tile, every tile walking the key
// blocks of each sequence it cuts) the tiles are full but a sequence cut by two tiles is walked
// twice, which pays for short sequences only.  Measured per layer, BERT-large (16 heads), in
// microseconds for tcgen05 packed tiles / tcgen05 one sequence per tile / persistent mma.sync:
//   1024 x 64 full rows 123 / 150 / 151;   1024 x 64 lengths 8..64: 133 / 167 / 142;
//   2048 x 32 lengths 4..32: 216 / 332 / 278;   800 x 80 lengths 8..80: 132 / 150 / 137;
//   512 x 96 lengths 8..96: 105 / 106 / 100;   512 x 96 full rows 154 / 129 / 157;
//   256 x 128 lengths 16..128: 77 / 72 / 77;   110 x 128 full rows 31 / 33 / 45;
//   128 x 200 lengths 16..200: 60 / 79 / 60;   110 x 192 full rows 60 / 65 / 75;
//   160 x 160 lengths 16..160: 59 / 74 / 54;   160 x 160 full rows 85 / 96 / 95;
//   55 x 256 full rows 44 / 48 / 68;   and, beyond the 256 positions the persistent kernel holds
//   (third figure: mma.sync with one CTA per item):   85 x 300 lengths 32..300: 80 / 87 / 98;
//   85 x 300 full rows 140 / 119 / 166;   64 x 400 lengths 32..400: 78 / 116 / 124;
//   64 x 400 full rows 155 / 165 / 275;   32 x 512 full rows 92 / 84 / 200;
//   32 x 512 lengths 64..512: 70 / 74 / 106.
// The lengths live on the device, so the choice uses S alone.  An S of at least 96 that fills its
// last 128-query tile to 85 % or more: tcgen05, one sequence per tile.  Otherwise: tcgen05 with
// packed tiles up to S = 80 and beyond S = 256, the persistent kernel in between.
// CUDABERT_ATTENTION=tc / persist / mma forces one kernel; CUDABERT_ATTENTION_TILES=packed / sequence
// forces the tcgen05 kernel's tiles (both give the same bits).
static bool tiles_fill_well(int S) {  // a sequence of S rows fills its last 128-query tile to 85 % or more
  const int tiles = (S + TQ - 1) / TQ;
  return S >= 96 && S * 100 >= tiles * TQ * 85;
}

int attention_kernel_for(int S) {
  static const int forced = []() -> int {
    const char* e = std::getenv("CUDABERT_ATTENTION");
    if (!e || !*e) return -1;
    if (e[0] == 't' || e[0] == '2') return ATT_KERNEL_TC;
    if (e[0] == 'p' || e[0] == '3') return ATT_KERNEL_PERSIST;
    if (e[0] == 'm' || e[0] == '0' || e[0] == '1') return ATT_KERNEL_MMA;
    return -1;
  }();
  int k = forced;
  if (k < 0) {
    k = (tiles_fill_well(S) || S <= ATC_PACKED_MAX_S || !attention_persist_fits(S)) ? ATT_KERNEL_TC : ATT_KERNEL_PERSIST;
  }
  if (k == ATT_KERNEL_PERSIST && !attention_persist_fits(S)) k = ATT_KERNEL_MMA;
  return k;
}

bool make_tmap_qkv(CUtensorMap* out, const void* qkv, uint64_t rows, int H) {
  return make_tmap_16bit_kmajor(out, qkv, rows, static_cast<uint64_t>(3) * H, static_cast<uint64_t>(3) * H * 2, TK);
}

int attention_f16_tc(const CUtensorMap* tm_qkv, const int* mask, const int* kv_len, const int* row_start,
                     const int* sched, __half* ctx, int B, int S, int heads, int num_sms, int cls_only, int* err_flag,
                     cudaStream_t stream) {
  if (B <= 0 || S <= 0 || S > 512 || heads <= 0) return -1;
  static std::atomic<bool> attr_set[64] = {};  // per device; a repeated set by a racing thread is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(attention_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_SMEM) !=
            cudaSuccess ||
        cudaFuncSetAttribute(attention_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_SMEM) !=
            cudaSuccess)
      return -2;
    if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
  }
  // Short sequences in packed rows (with the tile table of row_layout): tiles of 128 consecutive
  // rows, whatever sequences they belong to.  Otherwise one sequence per tile.
  static const int tiles_forced = []() {  // CUDABERT_ATTENTION_TILES=packed / sequence forces one (same bits)
    const char* e = std::getenv("CUDABERT_ATTENTION_TILES");
    return !e ? -1 : e[0] == 'p' ? 1 : e[0] == 's' ? 0 : -1;
  }();
  const bool want_multi = tiles_forced >= 0 ? tiles_forced == 1 : !tiles_fill_well(S);
  const bool multi = row_start != nullptr && sched != nullptr && !cls_only && want_multi;
  const long long tiles = multi ? (static_cast<long long>(B) * S + TQ - 1) / TQ
                                : static_cast<long long>(B) * ((S + TQ - 1) / TQ);
  const long long items = tiles * heads;
  const int grid = static_cast<int>(items < 2LL * num_sms ? items : 2LL * num_sms);
  const cudaError_t e =
      multi ? launch_pdl(attention_tc_kernel<true>, dim3(grid), dim3(ATC_THREADS), ATC_SMEM, stream, *tm_qkv, mask,
                         kv_len, row_start, sched, ctx, B, S, heads, cls_only, err_flag)
            : launch_pdl(attention_tc_kernel<false>, dim3(grid), dim3(ATC_THREADS), ATC_SMEM, stream, *tm_qkv, mask,
                         kv_len, row_start, sched, ctx, B, S, heads, cls_only, err_flag);
  return e == cudaSuccess ? 1 : -3;
}

}  // namespace cb
