// Fused attention forward for sm_100a: softmax(mod(Q K^T * scale) + mask) V in one pass.
//
// One CTA owns two 128-row query tiles ("stages") of one (batch, head) and walks the key/value
// tiles they need.  Sixteen warps, specialised by role:
//
//   warps 0-3   softmax for stage 0   (thread r owns query row r: TMEM lane r); a warp also
//   warps 4-7   softmax for stage 1    rescales its rows of O on the rare tiles where a row
//                                      maximum outgrows the lazy threshold
//   warps 8-11  epilogue for both stages (1/l normalisation, bf16 tile staged in shared memory,
//               TMA store)
//   warp 12     MMA issue (one lane): S = Q K^T (operands in shared memory) and
//               O += P V (P read from TMEM, V from shared memory, MN-major)
//   warp 13     TMA producer (one lane): Q once, then K(t), V(t) into a ring of slots
//
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+EV) O1 [256+EV,256+2EV).  P (bf16) is
// written over the first 64 columns of its S tile once the S row sits in registers (the
// differential variant puts a second, low-order bf16 term of P into the other 64 columns).  While the
// softmax warps of one stage work on tile t, the tensor core runs the other stage's MMAs.  Value
// heads of 64 or less leave columns [384,512) free; P then lives there (AttnCfg::SEP_P).
//
// Differential attention maps onto the same structure: both stages hold the same 128 query
// rows, stage 0 with (q, k) head h and stage 1 with head h + H, sharing each V tile; the
// epilogue combines the two accumulators and applies the per-head RMS normalisation.
//
// All waits are bounded (see ptx.cuh); on a timeout every role leaves through the common
// exit, TMEM is released and a status word is written.
#pragma once
#include <cuda.h>
#include <math_constants.h>

#include <type_traits>

#include "attn_params.h"
#include "ptx.cuh"

namespace flb {

template <int E_, int EV_, int SCORE_, int MASK_, int DIFF_, int STAGES_ = 2>
struct AttnCfg {
  static constexpr int E = E_, EV = EV_, SCORE = SCORE_, MASK = MASK_;
  static constexpr bool DIFF = DIFF_ != 0;  // differential attention: 1 = P as one bf16 term, 2 = as two, 3 = fp16
  // Query tiles per CTA.  Two: 512 threads, all of tensor memory, one CTA per SM, the stages share
  // every K/V tile.  One: 256 threads, half of tensor memory and of shared memory, two CTAs per
  // SM that run independently, so one CTA's set-up and epilogue hide behind the other's tiles
  // (short work items: sliding window, document mask, short sequences).
  static constexpr int STAGES = STAGES_;
  static_assert(STAGES == 2 || (STAGES == 1 && !DIFF_), "one or two query tiles per CTA");
  static constexpr int THREADS = STAGES == 2 ? 512 : 256;
  static constexpr int W_SOFTMAX_END = 4 * STAGES;                 // softmax warps [0, 4 * STAGES)
  static constexpr int W_EPI = STAGES == 2 ? 8 : 0;                // epilogue warps (one-stage: the softmax warps)
  static constexpr int W_MMA = STAGES == 2 ? 12 : 4;
  static constexpr int W_TMA = W_MMA + 1;
  // Differential attention subtracts two nearly equal softmax averages and then normalises the
  // result to unit RMS, which amplifies the rounding of P to bf16 to about the size of the
  // tolerance.  There P is written as two bf16 terms (hi + lo) and the PV product runs on both.
  // Without the normalisation one term is an order of magnitude inside the tolerance (mean-abs
  // 1.0e-4), and the second would cost 8 of 20 MMA steps per tile and the tile tried with the running
  // maximum: the kernel is built both ways.
  static constexpr bool SPLIT_P = DIFF_ == 2;
  // 3: P as one fp16 term against V converted to fp16 in shared memory (11 mantissa bits for 12 k-steps
  // a tile instead of 16 bits for 20)
  static constexpr bool PV_F16 = DIFF_ == 3;
  // ALiBi's bias grows along the keys, so a walk from the first key tile up would raise every
  // row maximum tile after tile and rescale the accumulator each time.  Walking the tiles from
  // the last one down meets the largest bias first; the result does not depend on the order.
  static constexpr bool REVERSE = SCORE_ == SCORE_ALIBI;
  // back-to-back product O = f(Q K^T * scale) V: no softmax; KT: K arrives as [E][S], keys contiguous
  // Resident pair bias: the CTA keeps one (head, query tile), loads that tile's pair-bias columns
  // once and walks a range of rows (MSA rows of Evoformer attention) that all add the same bias;
  // the two stages work on two rows at a time, each with its own Q, K and V.
  static constexpr bool ROWLOOP = SCORE_ == SCORE_BIAS_RES;
  static constexpr bool BIAS = SCORE_ == SCORE_BIAS || ROWLOOP;
  static_assert(!ROWLOOP || (STAGES_ == 2 && !DIFF_ && EV_ <= 64 && E_ == EV_), "resident bias: narrow heads, two stages");
  static constexpr bool B2B = SCORE_ == SCORE_B2B || SCORE_ == SCORE_B2BT;
  static constexpr bool KT = SCORE_ == SCORE_B2BT;
  static constexpr int KBOX = E >= 64 ? 64 : E;     // elements per swizzled row of a Q/K box
  static constexpr int VBOX = EV >= 64 ? 64 : EV;   // elements per swizzled row of a V box
  static constexpr int NKB = E / KBOX, NVB = EV / VBOX;
  static constexpr int QK_BOX_BYTES = 128 * KBOX * 2;
  static constexpr int V_BOX_BYTES = 128 * VBOX * 2;
  static constexpr int Q_BYTES = 128 * E * 2;                    // one stage
  static constexpr int K_HEAD_BYTES = 128 * E * 2;               // one head's K tile
  static constexpr int K_BYTES = K_HEAD_BYTES * (DIFF ? 2 : 1);  // diff: two heads side by side
  static constexpr int V_HEAD_BYTES = 128 * EV * 2;
  static constexpr int V_BYTES = V_HEAD_BYTES;
  static constexpr int SLOT_BYTES = K_BYTES > V_BYTES ? K_BYTES : V_BYTES;
  // Tensor-memory columns one CTA needs.  Two stages: all 512.  One stage: the score tile, the
  // accumulator and, for narrow heads, P: 256 columns (two CTAs per SM) up to value heads of 128,
  // 512 above (heads up to 256: one CTA per SM, which then also gets the whole shared memory).
  static constexpr bool WIDE = E_ > 128 || EV_ > 128;
  static_assert(!WIDE || STAGES_ == 1, "heads above 128 run one query tile per CTA");
  static constexpr int SMEM_BUDGET = (STAGES == 2 || WIDE) ? 224 * 1024 : 110 * 1024;
  static constexpr int NSTAGE_FIT = (SMEM_BUDGET - STAGES * Q_BYTES) / SLOT_BYTES;
  // Resident bias: everything between the Q tiles / output staging and the barriers is shared by
  // the K/V ring and the bias tiles; the launch decides the split (KernelParams::res_slots): the
  // bias takes 32 KB per key tile, the ring what is left, at least two slots and at most seven.
  static constexpr int NSTAGE = ROWLOOP ? 7 : (NSTAGE_FIT > 8 ? 8 : NSTAGE_FIT);
  static constexpr int AUX_BYTES = 2048;
  // output staging of its own (the Q tiles are reloaded for the next rows while a result is stored)
  static constexpr int OSTAGE_BYTES = ROWLOOP ? 2 * V_HEAD_BYTES : 0;
  static constexpr int SMEM_USED = ROWLOOP ? 232448 : 1024 + STAGES * Q_BYTES + NSTAGE * SLOT_BYTES + AUX_BYTES;
  // Shared memory also bounds how many CTAs share an SM, and with it their tensor-memory demand
  // (an allocation that does not fit would wait for a neighbour to leave): two-stage CTAs take
  // more than half of it (512 columns each), one-stage CTAs more than a third (256 columns each).
  static constexpr int SMEM_FLOOR = (STAGES == 2 || WIDE) ? 120 * 1024 : 80 * 1024;
  static constexpr int SMEM_BYTES = SMEM_USED < SMEM_FLOOR ? SMEM_FLOOR : SMEM_USED;
  static_assert(STAGES == 2 || WIDE || SMEM_BYTES <= 113 * 1024, "two one-stage CTAs must fit one SM");
  static constexpr uint32_t SWZ_K = KBOX == 64 ? kSwz128 : (KBOX == 32 ? kSwz64 : kSwz32);
  static constexpr uint32_t SWZ_V = VBOX == 64 ? kSwz128 : (VBOX == 32 ? kSwz64 : kSwz32);
  static constexpr int TMEM_COLS = (STAGES == 2 || WIDE) ? 512 : 256;
  static constexpr int COL_S0 = 0, COL_S1 = 128;
  static constexpr int COL_O0 = STAGES == 2 ? 256 : 128, COL_O1 = 256 + EV;
  // With value heads of 64 or less the accumulators leave 128 columns free: P gets columns of
  // its own instead of overwriting S.  The next QK product of a stage can then start as soon as
  // the softmax warps have read S, without waiting for P and the PV product: the softmax never
  // waits for the tensor core (narrow heads are bound by the exponentials, not by the MMAs).
  static constexpr bool SEP_P = !DIFF_ && EV_ <= 64;
  // softmax tries a tile with the running maximum first and looks for a new one only when the
  // tile's row sums say that it was too small (needs the whole P tile in registers at once, so
  // not where P has two terms; the document mask measured 3 % slower with it)
  static constexpr bool SPECULATE = MASK_ != MASK_DOCUMENT && !B2B && !SPLIT_P;
  static constexpr int COL_P0 = STAGES == 2 ? 384 : 128 + EV, COL_P1 = 448;
  static_assert(!SEP_P || COL_P0 + 64 <= TMEM_COLS, "P columns do not fit");
  static_assert(E % 16 == 0 && EV % 16 == 0, "head dims must be multiples of 16");
  static_assert(E <= 256 && EV <= 256, "head dims above 256 are not supported");
  static_assert(NSTAGE >= 2, "ring too small");
};

// barrier ids (also used in the status word)
enum : int {
  BAR_Q_FULL = 0,      // +s
  BAR_S_FULL = 2,      // +s   MMA -> softmax: S tile written
  BAR_P_FULL = 4,      // +s   softmax -> MMA: P tile written
  BAR_PV_DONE = 6,     // +s   MMA -> softmax / epilogue: O accumulated
  BAR_P_HALF = 8,      // +s   (free; the resident-bias kernel uses the pair as Q_EMPTY)
  BAR_SCALE_FULL = 10, // +s   softmax -> epilogue: final row sums published
  BAR_O_STAGED = 12,   // +s   epilogue threads -> storing thread: output tile written to shared memory
  BAR_KV_FULL = 14,    // +slot
  BAR_KV_EMPTY = 22,   // +slot
  BAR_S_FREE = 30,     // +s   softmax -> MMA: S tile read into registers (only with SEP_P)
  BAR_COUNT = 48,
  // resident-bias kernel: it does not use O_STAGED, and each stage has a K/V ring, a
  // producer and an MMA warp of its own (up to seven slots per stage)
  BAR_Q_EMPTY = BAR_P_HALF,    // +s   MMA -> producer: the row's last QK product has read Q
  BAR_O_FREE = BAR_O_STAGED,   // +s   epilogue -> MMA / softmax: the row's accumulator and row sums are read
  BAR_RING_FULL = 14,          // +8s+slot  (14..20 and 22..28)
  BAR_BIAS_FULL = 21,          //      producer -> softmax: the pair-bias tiles are in shared memory
  BAR_RING_EMPTY = 32,         // +8s+slot  (32..38 and 40..46)
  // fp16 P.V (differential attention): converter warps -> MMA, the V tile of a slot is fp16 now
  BAR_V_CONV = 32              // +slot
};

struct TileRange {
  int lo, hi;
};

FLB_DEV int prefix_of(const KernelParams& p, int n) {
  return p.prefix_len ? p.prefix_len[n] : p.prefix_scalar;
}

// kv tiles a 128-row query tile starting at r0 has to visit
template <int MASK>
FLB_DEV TileRange tile_range(const KernelParams& p, int n, int r0) {
  TileRange r{0, 0};
  if (r0 >= p.L) return r;
  const int nkv = (p.S + kTileN - 1) / kTileN;
  const int rlast = min(r0 + kTileM - 1, p.L - 1);
  if constexpr (MASK == MASK_NONE) {
    r.hi = nkv;
  } else if constexpr (MASK == MASK_CAUSAL) {
    r.hi = min(nkv, rlast / kTileN + 1);
  } else if constexpr (MASK == MASK_SLIDING) {
    r.hi = min(nkv, rlast / kTileN + 1);
    r.lo = max(0, r0 - p.window) / kTileN;
    if (r.lo > r.hi) r.lo = r.hi;
  } else if constexpr (MASK == MASK_PREFIX) {
    r.hi = min(nkv, max(prefix_of(p, n) - 1, rlast) / kTileN + 1);
  } else {
    const int nq = (p.L + kTileM - 1) / kTileM;
    const int32_t* e = p.map_range + (static_cast<int64_t>(n) * nq + r0 / kTileM) * 2;
    r.lo = e[0];
    r.hi = e[1];
  }
  return r;
}

// does kv tile t need element-wise masking for the query tile starting at r0?
template <int MASK>
FLB_DEV bool tile_partial(const KernelParams& p, int n, int r0, int t) {
  const int j0 = t * kTileN;
  bool partial = j0 + kTileN > p.S;  // ragged tail of the key axis
  if constexpr (MASK == MASK_CAUSAL) {
    partial |= j0 + kTileN - 1 > r0;
  } else if constexpr (MASK == MASK_SLIDING) {
    partial |= j0 + kTileN - 1 > r0;
    partial |= j0 < r0 + kTileM - 1 - p.window;
  } else if constexpr (MASK == MASK_PREFIX) {
    partial |= j0 + kTileN - 1 > max(prefix_of(p, n) - 1, r0);
  } else if constexpr (MASK == MASK_DOCUMENT) {
    const int nq = (p.L + kTileM - 1) / kTileM;
    const int nkv = (p.S + kTileN - 1) / kTileN;
    partial |= p.map_cls[(static_cast<int64_t>(n) * nq + r0 / kTileM) * nkv + t] != TILE_FULL;
  }
  return partial;
}

template <class C>
struct Smem {
  uint8_t* base;
  FLB_DEV uint8_t* q(int s) const { return base + s * C::Q_BYTES; }
  FLB_DEV uint8_t* ostage(int s) const { return base + C::STAGES * C::Q_BYTES + s * C::V_HEAD_BYTES; }
  FLB_DEV uint8_t* slot(int i) const {
    return base + C::STAGES * C::Q_BYTES + C::OSTAGE_BYTES + i * C::SLOT_BYTES;
  }
  // resident-bias kernel: slot i of stage s's ring (`slots` slots of one tile each per stage), and
  // the bias tiles behind the two rings
  FLB_DEV uint8_t* ring(int s, int i, int slots) const {
    return base + C::STAGES * C::Q_BYTES + C::OSTAGE_BYTES + (s * slots + i) * C::K_HEAD_BYTES;
  }
  FLB_DEV uint8_t* bias(int slots) const { return ring(2, 0, slots); }
  // behind the `nt` bias tiles, when the tensor cores add the key vector: 4 KB tiles of 128 rows of 16
  // bf16 (32-byte swizzle); tile 0 holds ones, then slots / 2 tiles per stage that travel with the K tiles
  FLB_DEV uint8_t* kvx(int slots, int nt, int i) const { return bias(slots) + nt * 32768 + i * 4096; }
  FLB_DEV uint8_t* aux() const { return base + (C::SMEM_USED - 1024 - C::AUX_BYTES); }
  FLB_DEV uint32_t bar(int id) const { return smem_u32(aux()) + id * 8; }
  FLB_DEV uint32_t* tmem_base() const { return reinterpret_cast<uint32_t*>(aux() + 384); }
  FLB_DEV WaitCtl* ctl() const { return reinterpret_cast<WaitCtl*>(aux() + 388); }
  FLB_DEV float* scale(int s) const { return reinterpret_cast<float*>(aux() + 512) + s * 128; }
  // pair exchange (differential attention with value heads of two kernel widths): a barrier the
  // partner CTA arrives at and the 128 row sums it stores here
  FLB_DEV uint32_t xbar() const { return smem_u32(aux()) + 408; }
  FLB_DEV float* xchg() const { return reinterpret_cast<float*>(aux() + 1536); }
};

#define FLB_WAIT_RET(sm, id, parity, ret)                         \
  do {                                                            \
    if (!mbar_wait((sm).bar(id), (parity), (sm).ctl())) {         \
      atomicCAS(&(sm).ctl()->fail_bar, -1, (id));                 \
      return ret;                                                 \
    }                                                             \
  } while (0)

#define FLB_WAIT(sm, id, parity)                                  \
  do {                                                            \
    if (!mbar_wait((sm).bar(id), (parity), (sm).ctl())) {         \
      atomicCAS(&(sm).ctl()->fail_bar, -1, (id));                 \
      return;                                                     \
    }                                                             \
  } while (0)

// ------------------------------------------------------------------------------------------
// TMA producer
// ------------------------------------------------------------------------------------------
template <class C>
FLB_DEV void load_role(const Smem<C>& sm, const CUtensorMap* tmQ, const CUtensorMap* tmK,
                       const CUtensorMap* tmV, const KernelParams& p, int n, int h, int vcol0,
                       const int (&r0)[2], const TileRange (&rg)[2], int lo, int hi) {
  // wait self-test: nothing is loaded, so the first wait of every other role runs into its limit
  if (p.withhold_loads) return;
  const int kvh = h / p.G;
#pragma unroll
  for (int s = 0; s < C::STAGES; ++s) {
    if (rg[s].hi > rg[s].lo) {
      const int qh = C::DIFF ? h + s * p.diff_heads : h;
      mbar_arrive_expect_tx(sm.bar(BAR_Q_FULL + s), C::Q_BYTES);
#pragma unroll
      for (int kb = 0; kb < C::NKB; ++kb)
        tma_load_4d(smem_u32(sm.q(s)) + kb * C::QK_BOX_BYTES, tmQ, sm.bar(BAR_Q_FULL + s),
                    kb * C::KBOX, r0[s], qh, n);
    }
  }
  int seq = 0;
#pragma unroll 1
  for (int u = 0; u < hi - lo; ++u) {
    const int t = C::REVERSE ? hi - 1 - u : lo + u;
    {  // K(t)
      const int slot = seq % C::NSTAGE;
      const uint32_t ph = (seq / C::NSTAGE) & 1;
      FLB_WAIT(sm, BAR_KV_EMPTY + slot, ph ^ 1);
      mbar_arrive_expect_tx(sm.bar(BAR_KV_FULL + slot), C::K_BYTES);
      const uint32_t dst = smem_u32(sm.slot(slot));
#pragma unroll
      if constexpr (C::KT) {
        // K^T tile: E feature rows of 128 keys, as two boxes of 64 keys (128-byte swizzled rows)
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
          tma_load_4d(dst + kb * (C::E * 128), tmK, sm.bar(BAR_KV_FULL + slot), t * kTileN + kb * 64, 0,
                      kvh, n);
      } else {
#pragma unroll
        for (int d = 0; d < (C::DIFF ? 2 : 1); ++d) {
          const int kh = C::DIFF ? kvh + d * p.diff_heads : kvh;
#pragma unroll
          for (int kb = 0; kb < C::NKB; ++kb)
            tma_load_4d(dst + d * C::K_HEAD_BYTES + kb * C::QK_BOX_BYTES, tmK,
                        sm.bar(BAR_KV_FULL + slot), kb * C::KBOX, t * kTileN, kh, n);
        }
      }
      ++seq;
    }
    {  // V(t)
      const int slot = seq % C::NSTAGE;
      const uint32_t ph = (seq / C::NSTAGE) & 1;
      FLB_WAIT(sm, BAR_KV_EMPTY + slot, ph ^ 1);
      mbar_arrive_expect_tx(sm.bar(BAR_KV_FULL + slot), C::V_BYTES);
      const uint32_t dst = smem_u32(sm.slot(slot));
#pragma unroll
      for (int vb = 0; vb < C::NVB; ++vb)
        tma_load_4d(dst + vb * C::V_BOX_BYTES, tmV, sm.bar(BAR_KV_FULL + slot), vcol0 + vb * C::VBOX,
                    t * kTileN, kvh, n);
      ++seq;
    }
  }
}

// Rows a resident-bias CTA walks: `count` rows from batch index n0 on, stage s taking the rows
// n0 + s, n0 + s + 2, ...; every row spans nt key tiles.
struct RowWalk {
  int n0, count, nt;
  FLB_DEV int items(int s) const { return (count + 1 - s) >> 1; }
};

// Producer of one stage of the resident-bias kernel: per row its Q tile and, tile by tile, K and V
// into the stage's ring.  The producer of stage 0 first brings in the pair-bias tiles.
template <class C>
FLB_DEV void load_role_rows(const Smem<C>& sm, const CUtensorMap* tmQ, const CUtensorMap* tmK,
                            const CUtensorMap* tmV, const CUtensorMap* tmB, const KernelParams& p,
                            int s, int b, int h, int r0, RowWalk rw) {
  if (p.withhold_loads) return;
  if (s == 0) {
    mbar_arrive_expect_tx(sm.bar(BAR_BIAS_FULL), rw.nt * 32768);
#pragma unroll 1
    for (int t = 0; t < rw.nt; ++t)
#pragma unroll
      for (int kb = 0; kb < 2; ++kb)
        tma_load_4d(smem_u32(sm.bias(p.res_slots)) + (t * 2 + kb) * 16384, tmB, sm.bar(BAR_BIAS_FULL),
                    t * kTileN + kb * 64, r0, h * p.pair_h, b * p.pair_b);
  }
  int slot = 0;
  uint32_t ph = 0;  // ring position of the next load and how often the ring has wrapped (parity)
  const int rows = rw.items(s);
#pragma unroll 1
  for (int r = 0; r < rows; ++r) {
    const int n = rw.n0 + 2 * r + s;
    // the Q tile is free once the previous row's last QK product has read it
    if (r > 0) FLB_WAIT(sm, BAR_Q_EMPTY + s, (r - 1) & 1);
    mbar_arrive_expect_tx(sm.bar(BAR_Q_FULL + s), C::Q_BYTES);
#pragma unroll
    for (int kb = 0; kb < C::NKB; ++kb)
      tma_load_4d(smem_u32(sm.q(s)) + kb * C::QK_BOX_BYTES, tmQ, sm.bar(BAR_Q_FULL + s), kb * C::KBOX, r0, h, n);
#pragma unroll 1
    for (int t = 0; t < rw.nt; ++t) {
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {  // K(t), then V(t)
        FLB_WAIT(sm, BAR_RING_EMPTY + 8 * s + slot, ph ^ 1);
        const uint32_t full = sm.bar(BAR_RING_FULL + 8 * s + slot);
        const bool with_x = kv == 0 && p.keyvec_rows != nullptr;   // the K tile's key-vector rows travel with it
        mbar_arrive_expect_tx(full, C::K_HEAD_BYTES + (with_x ? 4096 : 0));
        const uint32_t dst = smem_u32(sm.ring(s, slot, p.res_slots));
        if (kv == 0) {
#pragma unroll
          for (int kb = 0; kb < C::NKB; ++kb)
            tma_load_4d(dst + kb * C::QK_BOX_BYTES, tmK, full, kb * C::KBOX, t * kTileN, h, n);
          if (with_x)
            bulk_load_1d(smem_u32(sm.kvx(p.res_slots, rw.nt, 1 + s * (p.res_slots >> 1) + (slot >> 1))),
                         p.keyvec_rows + (static_cast<int64_t>(n) * p.keyvec_tiles + t) * 4096, 4096, full);
        } else {
#pragma unroll
          for (int vb = 0; vb < C::NVB; ++vb)
            tma_load_4d(dst + vb * C::V_BOX_BYTES, tmV, full, vb * C::VBOX, t * kTileN, h, n);
        }
        if (++slot == p.res_slots) {
          slot = 0;
          ph ^= 1;
        }
      }
    }
  }
}

// MMA issue for one stage of the resident-bias kernel (each stage has an issuing warp of its own, so
// neither waits for the other's softmax).  The stage's rows are strung together tile after tile; per
// position u: S = Q K(u)^T as soon as the softmax warps have read the previous scores, then
// O += P(u-1) V(u-1).  P has tensor-memory columns of its own (narrow heads).
template <class C>
FLB_DEV void mma_role_rows(const Smem<C>& sm, uint32_t tmem, const KernelParams& p, int s, RowWalk rw) {
  const uint32_t leader = elect_one() ? 1u : 0u;
  constexpr uint32_t idesc_qk = make_idesc_bf16(128, kTileN, 0, 0);
  constexpr uint32_t idesc_pv = make_idesc_bf16(128, C::EV, 0, 1);
  const uint32_t tS = tmem + (s ? C::COL_S1 : C::COL_S0), tO = tmem + (s ? C::COL_O1 : C::COL_O0);
  const uint32_t tP = tmem + (s ? C::COL_P1 : C::COL_P0);
  constexpr uint64_t kdesc0 = (static_cast<uint64_t>((8 * C::KBOX * 2) >> 4) << 32) |
                              (1ull << 16) | (1ull << 46) | (static_cast<uint64_t>(C::SWZ_K) << 61);
  constexpr uint64_t vdesc0 = (static_cast<uint64_t>((8 * C::VBOX * 2) >> 4) << 32) |
                              (static_cast<uint64_t>(C::V_BOX_BYTES >> 4) << 16) | (1ull << 46) |
                              (static_cast<uint64_t>(C::SWZ_V) << 61);
  constexpr uint32_t k_hi = static_cast<uint32_t>(kdesc0 >> 32), k_lo0 = static_cast<uint32_t>(kdesc0);
  constexpr uint32_t v_hi = static_cast<uint32_t>(vdesc0 >> 32), v_lo0 = static_cast<uint32_t>(vdesc0);
  const uint32_t q_lo = k_lo0 + ((smem_u32(sm.q(s)) & 0x3FFFFu) >> 4);
  const uint32_t ring0 = (smem_u32(sm.ring(s, 0, p.res_slots)) & 0x3FFFFu) >> 4;
  // K-major tiles of 32-byte swizzled rows (the key-vector k-step)
  constexpr uint64_t xdesc0 = (static_cast<uint64_t>(256 >> 4) << 32) | (1ull << 16) | (1ull << 46) |
                              (static_cast<uint64_t>(kSwz32) << 61);
  constexpr uint32_t x_hi = static_cast<uint32_t>(xdesc0 >> 32), x_lo0 = static_cast<uint32_t>(xdesc0);
  const uint32_t kvx0 = (smem_u32(sm.kvx(p.res_slots, rw.nt, 0)) & 0x3FFFFu) >> 4;
  const int total = rw.items(s) * rw.nt;
  // ring slots in load order K(0) V(0) K(1) V(1) ...: K(u) is load 2u, V(u-1) load 2u - 1
  int kslot = 0, vslot = p.res_slots > 1 ? p.res_slots - 1 : 0;  // load -1 precedes load 0
  uint32_t kph = 0, vph = 1;
  auto advance2 = [&](int& slot, uint32_t& ph) {
    slot += 2;
    if (slot >= p.res_slots) {
      slot -= p.res_slots;
      ph ^= 1;
    }
  };
  int qk_t = 0, qk_row = 0, pv_t = 0, pv_row = 0;
#pragma unroll 1
  for (int u = 0; u <= total; ++u) {
    if (u < total) {
      // S = Q K(u)^T
      FLB_WAIT(sm, BAR_RING_FULL + 8 * s + kslot, kph);
      if (qk_t == 0) FLB_WAIT(sm, BAR_Q_FULL + s, qk_row & 1);  // first tile of a row: its Q tile
      if (u > 0) FLB_WAIT(sm, BAR_S_FREE + s, (u - 1) & 1);     // the previous scores are in registers
      tc_fence_after();
      const uint32_t k_lo = k_lo0 + ring0 + kslot * (C::K_HEAD_BYTES >> 4);
      umma_ss_c<0>(leader, tS, q_lo, k_lo, k_hi, idesc_qk);
#pragma unroll
      for (int k = 1; k < C::E / 16; ++k) {
        const int kk = k * 16;
        const uint32_t off = ((kk / C::KBOX) * C::QK_BOX_BYTES + (kk % C::KBOX) * 2) >> 4;
        umma_ss_c<1>(leader, tS, q_lo + off, k_lo + off, k_hi, idesc_qk);
      }
      if (p.keyvec_rows != nullptr) {
        // one more k-step of 16: ones x [hi, lo, 0 ...] adds bias / scale of each key to its score column
        const uint32_t x_lo = x_lo0 + kvx0 + (1 + s * (p.res_slots >> 1) + (kslot >> 1)) * (4096 >> 4);
        umma_ss_c<1>(leader, tS, x_lo0 + kvx0, x_lo, x_hi, idesc_qk);
      }
      umma_commit_c(leader, sm.bar(BAR_S_FULL + s));
      umma_commit_c(leader, sm.bar(BAR_RING_EMPTY + 8 * s + kslot));
      if (++qk_t == rw.nt) {  // last tile of the row: its Q tile may be replaced
        qk_t = 0;
        ++qk_row;
        umma_commit_c(leader, sm.bar(BAR_Q_EMPTY + s));
      }
    }
    if (u > 0) {
      // O += P(u-1) V(u-1); the first product of a row overwrites the accumulator, which the
      // epilogue must have read for the previous row
      FLB_WAIT(sm, BAR_RING_FULL + 8 * s + vslot, vph);
      FLB_WAIT(sm, BAR_P_FULL + s, (u - 1) & 1);
      const bool fresh = pv_t == 0;
      if (fresh && pv_row > 0) FLB_WAIT(sm, BAR_O_FREE + s, (pv_row - 1) & 1);
      tc_fence_after();
      const uint32_t v_lo = v_lo0 + ring0 + vslot * (C::K_HEAD_BYTES >> 4);
      if (!fresh) umma_ts_c<1>(leader, tO, tP, v_lo, v_hi, idesc_pv);
      else umma_ts_c<0>(leader, tO, tP, v_lo, v_hi, idesc_pv);
#pragma unroll
      for (int k = 1; k < kTileN / 16; ++k)
        umma_ts_c<1>(leader, tO, tP + k * 8, v_lo + ((k * 16 * C::VBOX * 2) >> 4), v_hi, idesc_pv);
      umma_commit_c(leader, sm.bar(BAR_PV_DONE + s));
      umma_commit_c(leader, sm.bar(BAR_RING_EMPTY + 8 * s + vslot));
      if (++pv_t == rw.nt) {
        pv_t = 0;
        ++pv_row;
      }
    }
    advance2(kslot, kph);
    advance2(vslot, vph);
  }
}

// ------------------------------------------------------------------------------------------
// MMA issue (one warp, one issuing lane).  Order per step t:  PV0(t-1) QK0(t) PV1(t-1) QK1(t).  The tensor core
// executes in issue order, which keeps the two stages half a period apart: while one stage's
// MMAs run, the other stage's softmax warps work.  The issue loops are kept free of 64-bit
// arithmetic and predicates (see umma_*_c): a single thread then issues one 128x128x16 MMA
// per 64 clocks, the rate at which the tensor core retires them.
// ------------------------------------------------------------------------------------------
template <class C>
FLB_DEV void mma_role(const Smem<C>& sm, uint32_t tmem, const KernelParams& p,
                      const TileRange (&rg)[2], int lo, int hi) {
  const uint32_t leader = elect_one() ? 1u : 0u;  // the lane that issues; all lanes run the loop
  constexpr uint32_t idesc_qk = make_idesc_bf16(128, kTileN, 0, C::KT ? 1 : 0);
  constexpr uint32_t idesc_pv = C::PV_F16 ? make_idesc_f16(128, C::EV, 0, 1) : make_idesc_bf16(128, C::EV, 0, 1);
  const uint32_t tS[2] = {tmem + C::COL_S0, tmem + C::COL_S1};
  const uint32_t tO[2] = {tmem + C::COL_O0, tmem + C::COL_O1};
  [[maybe_unused]] const uint32_t tP[2] = {tmem + C::COL_P0, tmem + C::COL_P1};
  // descriptor templates with a zero start address; only the low word changes per operand
  constexpr uint64_t kdesc0 = (static_cast<uint64_t>((8 * C::KBOX * 2) >> 4) << 32) |
                              (1ull << 16) | (1ull << 46) | (static_cast<uint64_t>(C::SWZ_K) << 61);
  constexpr uint64_t vdesc0 = (static_cast<uint64_t>((8 * C::VBOX * 2) >> 4) << 32) |
                              (static_cast<uint64_t>(C::V_BOX_BYTES >> 4) << 16) | (1ull << 46) |
                              (static_cast<uint64_t>(C::SWZ_V) << 61);
  // K^T tile (keys contiguous): an MN-major operand like V; 8-row groups 1024 bytes apart, the two
  // 64-key boxes E * 128 bytes apart, 128-byte swizzle
  constexpr uint64_t ktdesc0 = (static_cast<uint64_t>(1024 >> 4) << 32) |
                               (static_cast<uint64_t>((C::E * 128) >> 4) << 16) | (1ull << 46) |
                               (static_cast<uint64_t>(kSwz128) << 61);
  [[maybe_unused]] constexpr uint32_t kt_hi = static_cast<uint32_t>(ktdesc0 >> 32),
                                      kt_lo0 = static_cast<uint32_t>(ktdesc0);
  constexpr uint32_t k_hi = static_cast<uint32_t>(kdesc0 >> 32), k_lo0 = static_cast<uint32_t>(kdesc0);
  constexpr uint32_t v_hi = static_cast<uint32_t>(vdesc0 >> 32), v_lo0 = static_cast<uint32_t>(vdesc0);
  // (matrix descriptors take the offset inside this CTA's shared memory: in a cluster launch the
  // shared-window address of every CTA but the first carries its rank in the high bits)
  const uint32_t q_lo[2] = {k_lo0 + ((smem_u32(sm.q(0)) & 0x3FFFFu) >> 4),
                            k_lo0 + ((smem_u32(sm.q(1)) & 0x3FFFFu) >> 4)};
  const uint32_t slot0 = (smem_u32(sm.slot(0)) & 0x3FFFFu) >> 4;
  bool q_ready[2] = {false, false};

  // position u of the walk holds tile lo + u (or hi - 1 - u when the walk is reversed); stage s
  // takes part in positions [first[s], first[s] + cnt[s])
  const int n_pos = hi - lo;
  const int cnt[2] = {rg[0].hi - rg[0].lo, rg[1].hi - rg[1].lo};
  const int first[2] = {C::REVERSE ? hi - rg[0].hi : rg[0].lo - lo,
                        C::REVERSE ? hi - rg[1].hi : rg[1].lo - lo};
#pragma unroll 1
  for (int u = 0; u <= n_pos; ++u) {
    const bool have_k = u < n_pos, have_v = u > 0;
    const int kseq = 2 * u, vseq = 2 * (u - 1) + 1;
    const int kslot = kseq % C::NSTAGE, vslot = have_v ? vseq % C::NSTAGE : 0;
    const uint32_t kph = (kseq / C::NSTAGE) & 1, vph = (vseq / C::NSTAGE) & 1;
    const uint32_t v_lo = v_lo0 + slot0 + vslot * (C::SLOT_BYTES >> 4);
    const uint32_t k_lo = k_lo0 + slot0 + kslot * (C::SLOT_BYTES >> 4);
    if (have_v) FLB_WAIT(sm, BAR_KV_FULL + vslot, vph);
    if constexpr (C::PV_F16) {
      if (have_v) FLB_WAIT(sm, BAR_V_CONV + vslot, vph);   // the V tile has been rewritten as fp16
    }
    if (have_k) FLB_WAIT(sm, BAR_KV_FULL + kslot, kph);
#pragma unroll
    for (int s = 0; s < C::STAGES; ++s) {
      // With P in columns of its own the scores of the next tile go first (they only wait for S to
      // be read), otherwise the PV product that frees the S tile.
#pragma unroll
      for (int ph = 0; ph < 2; ++ph) {
        if ((ph == 0) != C::SEP_P) {
          // O_s += P_s(t-1) V(t-1)
          if (have_v && u - 1 >= first[s] && u - 1 < first[s] + cnt[s]) {
            const int it = u - 1 - first[s];
            const uint32_t tA = C::SEP_P ? tP[s] : tS[s];  // where the softmax warps put P
            FLB_WAIT(sm, BAR_P_FULL + s, it & 1);
            tc_fence_after();
            if (it > 0) umma_ts_c<1>(leader, tO[s], tA, v_lo, v_hi, idesc_pv);
            else umma_ts_c<0>(leader, tO[s], tA, v_lo, v_hi, idesc_pv);
#pragma unroll
            for (int k = 1; k < kTileN / 32; ++k)
              umma_ts_c<1>(leader, tO[s], tA + k * 8, v_lo + ((k * 16 * C::VBOX * 2) >> 4), v_hi, idesc_pv);
            if constexpr (C::SPLIT_P) {
#pragma unroll
              for (int k = 0; k < kTileN / 32; ++k)
                umma_ts_c<1>(leader, tO[s], tA + 64 + k * 8, v_lo + ((k * 16 * C::VBOX * 2) >> 4), v_hi,
                             idesc_pv);
            }
#pragma unroll
            for (int k = kTileN / 32; k < kTileN / 16; ++k)
              umma_ts_c<1>(leader, tO[s], tA + k * 8, v_lo + ((k * 16 * C::VBOX * 2) >> 4), v_hi, idesc_pv);
            if constexpr (C::SPLIT_P) {
#pragma unroll
              for (int k = kTileN / 32; k < kTileN / 16; ++k)
                umma_ts_c<1>(leader, tO[s], tA + 64 + k * 8, v_lo + ((k * 16 * C::VBOX * 2) >> 4), v_hi,
                             idesc_pv);
            }
            umma_commit_c(leader, sm.bar(BAR_PV_DONE + s));
          }
        } else {
          // S_s = Q_s K(t)^T
          if (have_k && u >= first[s] && u < first[s] + cnt[s]) {
            if (!q_ready[s]) {
              FLB_WAIT(sm, BAR_Q_FULL + s, 0);
              q_ready[s] = true;
              tc_fence_after();
            }
            if constexpr (C::SEP_P) {
              // S may be overwritten once the softmax warps hold the previous tile in registers
              const int itq = u - first[s];
              if (itq > 0) {
                FLB_WAIT(sm, BAR_S_FREE + s, (itq - 1) & 1);
                tc_fence_after();
              }
            }
            if constexpr (C::KT) {
              const uint32_t kt_lo = k_lo - k_lo0 + kt_lo0;
              umma_ss2_c<0>(leader, tS[s], q_lo[s], k_hi, kt_lo, kt_hi, idesc_qk);
#pragma unroll
              for (int k = 1; k < C::E / 16; ++k) {
                const int kk = k * 16;
                const uint32_t off = ((kk / C::KBOX) * C::QK_BOX_BYTES + (kk % C::KBOX) * 2) >> 4;
                umma_ss2_c<1>(leader, tS[s], q_lo[s] + off, k_hi, kt_lo + ((kk * 128) >> 4), kt_hi, idesc_qk);
              }
            } else {
              const uint32_t ks_lo = k_lo + (C::DIFF ? s * (C::K_HEAD_BYTES >> 4) : 0);
              umma_ss_c<0>(leader, tS[s], q_lo[s], ks_lo, k_hi, idesc_qk);
#pragma unroll
              for (int k = 1; k < C::E / 16; ++k) {
                const int kk = k * 16;
                const uint32_t off = ((kk / C::KBOX) * C::QK_BOX_BYTES + (kk % C::KBOX) * 2) >> 4;
                umma_ss_c<1>(leader, tS[s], q_lo[s] + off, ks_lo + off, k_hi, idesc_qk);
              }
            }
            umma_commit_c(leader, sm.bar(BAR_S_FULL + s));
          }
        }
      }
    }
    // a slot goes back to the producer once every MMA that reads it has retired
    if (have_v) umma_commit_c(leader, sm.bar(BAR_KV_EMPTY + vslot));
    if (have_k) umma_commit_c(leader, sm.bar(BAR_KV_EMPTY + kslot));
  }
}

// ------------------------------------------------------------------------------------------
// softmax (one warpgroup per stage, one thread per query row)
// ------------------------------------------------------------------------------------------
FLB_DEV float u2f(uint32_t u) { return __uint_as_float(u); }
FLB_DEV uint32_t f2u(float f) { return __float_as_uint(f); }

// Largest log2-domain growth of a row maximum that is absorbed without rescaling O.
constexpr float kLazyRescaleLog2 = 8.0f;
// a tile tried with the running maximum stands when each of its row sums is at most this
constexpr float kSpeculateSumLimit = 1024.0f;
// largest (score / cap)^2 for which the softcap's tanh is taken from its odd polynomial
constexpr float kSoftcapPolyLimit = 0.09f;

// Register budgets after the roles split (setmaxnreg; 8 softmax warps, 4 epilogue warps, 4 warps
// around the MMA and TMA issuers: 256 * softmax + 128 * epilogue + 128 * issue <= 65536)
constexpr int kRegsSoftmax = 192, kRegsEpilogue = 64, kRegsIssue = 64;
// one query tile per CTA: 256 threads start with 128 registers each (two CTAs per SM); four
// softmax warps and the warpgroup around the two issuing warps: 128 * softmax + 128 * issue <= 32768
constexpr int kRegsSoftmax1 = 200, kRegsIssue1 = 56;

// Of every kPolyPeriod column pairs, kPolyCount go through exp2_poly2, the rest through ex2.approx.
// One pair in four measured best (a third or more is slower than none).  A P of two bf16 terms
// (differential attention with the RMS normalisation) keeps all pairs on ex2.approx.
constexpr int kPolyPeriod = 4, kPolyCount = 1;

template <class C>
FLB_DEV void softmax_role(const Smem<C>& sm, uint32_t tmem, const KernelParams& p, int s, int n,
                          int h, int r0, TileRange rg, [[maybe_unused]] int row_index = 0) {
  // resident-bias kernel: this call handles one row of the walk; its tiles continue the count of
  // the tiles of the stage's earlier rows (barrier phases run on that global count)
  const int it_base = C::ROWLOOP ? row_index * (rg.hi - rg.lo) : 0;
  const int row = threadIdx.x & 127;
  const int i = r0 + row;  // global query row
  const uint32_t lane_base = static_cast<uint32_t>((threadIdx.x >> 5) & 3) * 32u;
  const uint32_t tS = tmem + (s ? C::COL_S1 : C::COL_S0) + (lane_base << 16);
  const uint32_t tO = tmem + (s ? C::COL_O1 : C::COL_O0) + (lane_base << 16);
  // P overwrites the head of the S tile, or has columns of its own (see AttnCfg::SEP_P)
  const uint32_t tPs = C::SEP_P ? tmem + (s ? C::COL_P1 : C::COL_P0) + (lane_base << 16) : tS;
  float* sscale = sm.scale(s);
  constexpr float kLog2e = 1.4426950408889634f;
  // exp2 argument = v * kmul - m * mdom; for plain scores the softmax scale is folded in here
  const float kmul = C::SCORE == SCORE_NONE      ? p.scale_log2
                     : C::SCORE == SCORE_SOFTCAP ? p.softcap * kLog2e
                     : C::BIAS                   ? kLog2e
                                                 : 1.0f;
  // the running maximum m lives in the domain of the raw scores for plain attention, of
  // tanh(score / cap) for softcap and of the biased score (natural units) for additive biases
  // (log2 units after multiplying by mdom); ALiBi scores are in log2 units already
  const float mdom = C::SCORE == SCORE_NONE ? p.scale_log2
                     : C::SCORE == SCORE_SOFTCAP ? p.softcap * kLog2e
                     : C::BIAS ? kLog2e : 1.0f;

  float slope2 = 0.f;
  if constexpr (C::SCORE == SCORE_ALIBI) {
    const int qh = h + p.alibi_head0;  // the slope follows the query head
    slope2 = exp2f(static_cast<float>(qh + 1) * p.alibi_log2_slope_step) * kLog2e;
  }
  const __nv_bfloat16* brow[2] = {nullptr, nullptr};
  if constexpr (C::SCORE == SCORE_BIAS) {
    const int b = n / p.evo_inner, r = n % p.evo_inner;
    const int ic = min(i, p.L - 1);
#pragma unroll
    for (int q = 0; q < 2; ++q)
      if (p.bias[q])
        brow[q] = reinterpret_cast<const __nv_bfloat16*>(p.bias[q]) + b * p.bias_sb[q] +
                  r * p.bias_sr[q] + h * p.bias_sh[q] + ic * p.bias_sl[q];
  }
  if constexpr (C::ROWLOOP) {
    // the row's key vector (every query row adds the same values), if there is one
    const int b = n / p.evo_inner, r = n % p.evo_inner;
    if (p.bias[0])
      brow[0] = reinterpret_cast<const __nv_bfloat16*>(p.bias[0]) + b * p.bias_sb[0] + r * p.bias_sr[0] +
                h * p.bias_sh[0];
    if (row_index == 0) FLB_WAIT(sm, BAR_BIAS_FULL, 0);  // the pair-bias tiles, loaded once
  }
  int pl = 0;
  if constexpr (C::MASK == MASK_PREFIX) pl = prefix_of(p, n);
  int64_t my_doc = 0;
  const int64_t* docrow = nullptr;
  // ids that never decrease along the sequence: "same document" is the index interval
  // [doc_first, doc_last] around the row, found by the block-map builder
  [[maybe_unused]] bool doc_sorted = false;
  [[maybe_unused]] int doc_first = 0, doc_last = 0;
  if constexpr (C::MASK == MASK_DOCUMENT) {
    docrow = p.doc + n * p.doc_sn;
    const int ic = min(i, p.L - 1);
    my_doc = docrow[ic];
    doc_sorted = p.map_sorted[n] != 0;
    if (doc_sorted) {
      const int2* runs = reinterpret_cast<const int2*>(p.map_runs) + static_cast<int64_t>(n) * p.L;
      const int2 run = runs[ic];
      doc_first = run.x;
      doc_last = run.y;
    }
  }

  float m = -CUDART_INF_F;  // running maximum (in the domain of x below)
  float l = 0.f;            // running sum of exp2

#pragma unroll 1
  for (int it = 0; it < rg.hi - rg.lo; ++it) {
    const int t = C::REVERSE ? rg.hi - 1 - it : rg.lo + it;
    const int j0 = t * kTileN;
    const int git = it_base + it;  // tiles of this stage so far
    if constexpr (C::SCORE == SCORE_BIAS) {
      // pull this tile's bias rows (256 B each) into L1 while the scores are still being computed
#pragma unroll
      for (int q = 0; q < 2; ++q)
        if (brow[q]) {
          const char* a = reinterpret_cast<const char*>(brow[q] + min(j0, p.S - 1));
          const char* last = reinterpret_cast<const char*>(brow[q] + min(j0 + kTileN, p.S) - 1);
          prefetch_l1(a);
          prefetch_l1(a + 128 < last ? a + 128 : last);
          prefetch_l1(last);
        }
    }
    FLB_WAIT(sm, BAR_S_FULL + s, git & 1);
    tc_fence_after();
    uint32_t v[128];
    float m_new = m, m_use = 0.f, sc = 1.0f;
    // S from tensor memory into v, score modifier and mask applied.  `fold` leaves the ALiBi bias
    // out: the caller adds it inside the exponent FMA.
    auto fetch_scores = [&](auto fold) {
    tmem_ld128_sync(tS, v);

    // ---- score modifier: x = mod(s * scale) in log2 units (plain scores stay raw) ----
    if constexpr (C::SCORE == SCORE_ALIBI && decltype(fold)::value) {
      // nothing here
    } else if constexpr (C::SCORE == SCORE_ALIBI) {
      // log2 units, bias included: the row maximum below is then exact, so a row that sees a
      // single key gets P = 1 and its value row back unchanged
      const float base = slope2 * static_cast<float>(j0 - i);
#pragma unroll
      for (int c = 0; c < 128; ++c)
        v[c] = f2u(fmaf(u2f(v[c]), p.scale_log2, fmaf(slope2, static_cast<float>(c), base)));
    } else if constexpr (C::SCORE == SCORE_SOFTCAP) {
      const float inv = p.scale / p.softcap;
      // the cap and log2(e) join the exponent FMA below (kmul, mdom): tanh in, tanh out here.
      // A softcap is chosen well above the typical score, so y = score / cap is small and
      // tanh(y) = y (1 + y^2 (-1/3 + 2/15 y^2)) holds to 1.2e-5 for |y| <= 0.3: packed FMA-pipe
      // work instead of one more transcendental per score on the unit the exponentials already
      // saturate.  A warp whose tile holds a larger |y| (small caps) redoes it with tanh.approx.
      const float2 inv2 = make_float2(inv, inv), one2 = make_float2(1.f, 1.f);
      const float2 c3 = make_float2(-1.f / 3.f, -1.f / 3.f), c5 = make_float2(2.f / 15.f, 2.f / 15.f);
      float y2m = 0.f;
#pragma unroll
      for (int c = 0; c < 128; c += 2) {
        float2 y = __fmul2_rn(make_float2(u2f(v[c]), u2f(v[c + 1])), inv2);
        const float2 y2 = __fmul2_rn(y, y);
        y2m = max3(y2m, y2.x, y2.y);
        float2 a = __ffma2_rn(y2, c5, c3);
        a = __ffma2_rn(a, y2, one2);
        y = __fmul2_rn(y, a);
        v[c] = f2u(y.x);
        v[c + 1] = f2u(y.y);
      }
      if (!__all_sync(0xffffffffu, y2m <= kSoftcapPolyLimit)) {
        tmem_ld128_sync(tS, v);
#pragma unroll
        for (int c = 0; c < 128; ++c) v[c] = f2u(tanh_approx(u2f(v[c]) * inv));
      }
    } else if constexpr (C::ROWLOOP) {
      // s * scale + pair bias (this thread's row of the resident tile: 16 chunks of 8 columns, the
      // 128-byte rows of each 64-column box swizzled as the tensor map wrote them) + key vector
      const uint8_t* btile = sm.bias(p.res_slots) + t * 32768 + row * 128;
      const int sw = row & 7;
      const float2 mul2 = make_float2(p.scale, p.scale);
#pragma unroll
      for (int c8 = 0; c8 < 16; ++c8) {
        const uint4 w = *reinterpret_cast<const uint4*>(btile + (c8 >> 3) * 16384 + (((c8 & 7) ^ sw) << 4));
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = __ffma2_rn(make_float2(u2f(v[c8 * 8 + 2 * e]), u2f(v[c8 * 8 + 2 * e + 1])), mul2,
                                      make_float2(u2f(ww[e] << 16), u2f(ww[e] & 0xffff0000u)));
          v[c8 * 8 + 2 * e] = f2u(x.x);
          v[c8 * 8 + 2 * e + 1] = f2u(x.y);
        }
      }
      if (brow[0] && p.keyvec_rows == nullptr) {
        if (j0 + kTileN <= p.S && p.bias_vec[0]) {
          const uint4* src = reinterpret_cast<const uint4*>(brow[0] + j0);  // same address in every lane
#pragma unroll
          for (int c8 = 0; c8 < 16; ++c8) {
            const uint4 w = __ldg(src + c8);
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              v[c8 * 8 + 2 * e] = f2u(u2f(v[c8 * 8 + 2 * e]) + u2f(ww[e] << 16));
              v[c8 * 8 + 2 * e + 1] = f2u(u2f(v[c8 * 8 + 2 * e + 1]) + u2f(ww[e] & 0xffff0000u));
            }
          }
        } else {
#pragma unroll
          for (int c = 0; c < 128; ++c)
            v[c] = f2u(u2f(v[c]) + (j0 + c < p.S ? __bfloat162float(brow[0][j0 + c]) : 0.f));
        }
      }
    } else if constexpr (C::SCORE == SCORE_BIAS) {
      const bool ragged = j0 + kTileN > p.S;
      // s * scale + b0 + b1: the scale rides on the first bias as one FMA per score
      float mul = p.scale;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        if (brow[q]) {
          if (!ragged && p.bias_vec[q]) {
            const uint4* src = reinterpret_cast<const uint4*>(brow[q] + j0);
#pragma unroll
            for (int c8 = 0; c8 < 16; ++c8) {
              const uint4 w = __ldg(src + c8);
              const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                v[c8 * 8 + 2 * e] = f2u(fmaf(u2f(v[c8 * 8 + 2 * e]), mul, u2f(ww[e] << 16)));
                v[c8 * 8 + 2 * e + 1] =
                    f2u(fmaf(u2f(v[c8 * 8 + 2 * e + 1]), mul, u2f(ww[e] & 0xffff0000u)));
              }
            }
          } else {
#pragma unroll
            for (int c = 0; c < 128; ++c)
              v[c] = f2u(fmaf(u2f(v[c]), mul, j0 + c < p.S ? __bfloat162float(brow[q][j0 + c]) : 0.f));
          }
          mul = 1.0f;
        }
      }
      if (mul != 1.0f) {
#pragma unroll
        for (int c = 0; c < 128; ++c) v[c] = f2u(u2f(v[c]) * mul);
      }
    }

    // ---- mask (only tiles that straddle a mask edge) ----
    if (tile_partial<C::MASK>(p, n, r0, t)) {
      if (C::MASK == MASK_DOCUMENT && !doc_sorted) {
        // lane L fetches the ids of columns L, L+32, L+64, L+96 (coalesced); every column's id
        // then reaches all lanes by shuffle instead of 128 dependent global loads per thread
        const int lane = threadIdx.x & 31;
        uint32_t id_lo[4], id_hi[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int64_t d = docrow[min(j0 + 32 * g + lane, p.S - 1)];
          id_lo[g] = static_cast<uint32_t>(d);
          id_hi[g] = static_cast<uint32_t>(static_cast<uint64_t>(d) >> 32);
        }
        const uint32_t my_lo = static_cast<uint32_t>(my_doc);
        const uint32_t my_hi = static_cast<uint32_t>(static_cast<uint64_t>(my_doc) >> 32);
        const int jmax = p.causal ? min(i, p.S - 1) : p.S - 1;
#pragma unroll
        for (int c = 0; c < 128; ++c) {
          const uint32_t lo = __shfl_sync(0xffffffffu, id_lo[c >> 5], c & 31);
          const uint32_t hi = __shfl_sync(0xffffffffu, id_hi[c >> 5], c & 31);
          const bool keep = (lo == my_lo) & (hi == my_hi) & (j0 + c <= jmax);
          if (!keep) v[c] = f2u(-CUDART_INF_F);
        }
      } else {
        // keep columns clo <= c <= chi of this tile; first / last key a row may see:
        auto key_bounds = [&](int ii, int dfirst, int dlast, int& jlo, int& jhi) {
          jlo = 0;
          jhi = p.S - 1;
          if constexpr (C::MASK == MASK_CAUSAL) jhi = min(jhi, ii);
          if constexpr (C::MASK == MASK_SLIDING) {
            jhi = min(jhi, ii);
            jlo = ii - p.window;
          }
          if constexpr (C::MASK == MASK_PREFIX) jhi = min(jhi, max(pl - 1, ii));
          if constexpr (C::MASK == MASK_DOCUMENT) {
            jlo = dfirst;
            jhi = min(jhi, p.causal ? min(ii, dlast) : dlast);
          }
        };
        int jlo, jhi;
        key_bounds(i, doc_first, doc_last, jlo, jhi);
        const int clo = jlo - j0, chi = jhi - j0;
        // one bit per column of a 32-column group, then a bit test and a select per column: half
        // the cost of two integer compares and a select
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int lo_g = min(max(clo - 32 * g, 0), 32), hi_g = min(max(chi - 32 * g + 1, 0), 32);
          const uint32_t below_hi = hi_g >= 32 ? 0xffffffffu : ((1u << hi_g) - 1u);
          const uint32_t below_lo = lo_g >= 32 ? 0xffffffffu : ((1u << lo_g) - 1u);
          const uint32_t keep = below_hi & ~below_lo;
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (!((keep >> c) & 1u)) v[32 * g + c] = f2u(-CUDART_INF_F);
        }
      }
    }

    };  // fetch_scores

    // ---- the common case: the running maximum still fits ----
    // Every row has a finite maximum from earlier tiles: take exp2 against it right away and keep
    // the bf16 P tile in registers.  A row sum within the limit proves that no probability went
    // above it, which is all the lazy rescale asks for; then P is stored and the tile is done
    // without a pass over the scores for their maximum.  Otherwise (also for inf and NaN) nothing
    // was stored, S is intact in tensor memory and the exact path below takes the tile.
    bool done = false, retry = false;
    if constexpr (C::SPECULATE) {
      if (it > 0 && __all_sync(0xffffffffu, m != -CUDART_INF_F)) {
        fetch_scores(std::true_type{});
        const float mk = m * mdom;
        const float2 kmul2 = make_float2(kmul, kmul), nmk2 = make_float2(-mk, -mk);
        [[maybe_unused]] float2 slope22, base2, scale2;
        if constexpr (C::SCORE == SCORE_ALIBI) {
          const float base = slope2 * static_cast<float>(j0 - i) - mk;
          slope22 = make_float2(slope2, slope2);
          base2 = make_float2(base, base);
          scale2 = make_float2(p.scale_log2, p.scale_log2);
        }
        float2 suma = make_float2(0.f, 0.f), sumb = make_float2(0.f, 0.f);
        uint32_t pk[64];
#pragma unroll
        for (int idx = 0; idx < 128; idx += 2) {
          const float2 s2 = make_float2(u2f(v[idx]), u2f(v[idx + 1]));
          float2 x;
          if constexpr (C::SCORE == SCORE_ALIBI) {
            const float2 add = __ffma2_rn(
                slope22, make_float2(static_cast<float>(idx), static_cast<float>(idx + 1)), base2);
            x = __ffma2_rn(s2, scale2, add);
          } else {
            x = __ffma2_rn(s2, kmul2, nmk2);
          }
          float2 pr;
          if ((idx >> 1) % kPolyPeriod < kPolyCount) {
            pr = exp2_poly2(x);
          } else {
            pr.x = ex2(x.x);
            pr.y = ex2(x.y);
          }
          if (idx & 2) sumb = __fadd2_rn(sumb, pr); else suma = __fadd2_rn(suma, pr);
          pk[idx >> 1] = C::PV_F16 ? pack_f16_sat(pr.x, pr.y) : pack_bf16(pr.x, pr.y);
        }
        const float lt = (suma.x + suma.y) + (sumb.x + sumb.y);
        if (__all_sync(0xffffffffu, lt <= kSpeculateSumLimit)) {
          if constexpr (C::SEP_P) {
            // the scores are not needed again: the next tile's may come, and P of the previous tile
            // must have been consumed before it is overwritten
            tc_fence_before();
            mbar_arrive(sm.bar(BAR_S_FREE + s));
            FLB_WAIT(sm, BAR_PV_DONE + s, (git - 1) & 1);
          }
#pragma unroll
          for (int chunk = 0; chunk < 4; ++chunk) tmem_st16(tPs + chunk * 16, pk + chunk * 16);
          l += lt;
          done = true;
        } else {
          retry = true;
        }
      }
    }

    if (!done) {
    // Pass 0 fetches the scores and finds the row maximum.  Only when a row of this warp must
    // rescale its accumulator is there a pass 1: the score registers are given up for the rescale
    // and the scores fetched again.
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
    fetch_scores(std::false_type{});
    if (pass == 1) break;

    // ---- row maximum (four independent chains) ----
    float mxs[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float a = max3(u2f(v[32 * g]), u2f(v[32 * g + 1]), u2f(v[32 * g + 2]));
#pragma unroll
      for (int c = 3; c < 31; c += 2) a = max3(a, u2f(v[32 * g + c]), u2f(v[32 * g + c + 1]));
      mxs[g] = fmaxf(a, u2f(v[32 * g + 31]));
    }
    const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));

    if (m == -CUDART_INF_F) {
      m_new = mx;
    } else {
      m_new = fmaxf(m, mx);
      // absorb small growth, unless the tile was already tried with m and overflowed: then the
      // exact maximum spares the tiles that follow the same detour
      if (!retry && (m_new - m) * mdom <= kLazyRescaleLog2) m_new = m;
    }
    m_use = m_new == -CUDART_INF_F ? 0.f : m_new;
    // Factor the accumulator must be multiplied with.  The lazy threshold makes it 1 for almost
    // every tile; otherwise the warp waits for the tile's predecessor to be accumulated and
    // rescales its 32 rows of O itself.
    sc = (it == 0 || m == -CUDART_INF_F) ? 1.0f : ex2((m - m_use) * mdom);
    if (it == 0 || !__any_sync(0xffffffffu, sc != 1.0f)) break;
    FLB_WAIT(sm, BAR_PV_DONE + s, (git - 1) & 1);
    tc_fence_after();
#pragma unroll
    for (int c0 = 0; c0 < C::EV; c0 += 32) {
      uint32_t o[32];
      tmem_ld32_sync(tO + c0, o);
#pragma unroll
      for (int c = 0; c < 32; ++c) o[c] = f2u(u2f(o[c]) * sc);
      tmem_st32(tO + c0, o);
    }
    tmem_wait_st();
    }  // pass
    if constexpr (C::SEP_P) {
      // the scores sit in registers for good: the tensor core may write the next tile's over them
      tc_fence_before();
      mbar_arrive(sm.bar(BAR_S_FREE + s));
      // and P of the previous tile must have been consumed before it is overwritten below
      if (git > 0) FLB_WAIT(sm, BAR_PV_DONE + s, (git - 1) & 1);
    }
    l *= sc;
    m = m_new;

    // ---- probabilities, row sum, bf16 P back into TMEM ----
    const float mk = m_use * mdom;
    const float2 kmul2 = make_float2(kmul, kmul), nmk2 = make_float2(-mk, -mk);
    float2 suma = make_float2(0.f, 0.f), sumb = make_float2(0.f, 0.f);
#pragma unroll
    for (int chunk = 0; chunk < 4; ++chunk) {
      uint32_t pk[16];
      uint32_t pk_lo[C::SPLIT_P ? 16 : 1];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const int idx = chunk * 32 + c;
        const float2 x = __ffma2_rn(make_float2(u2f(v[idx]), u2f(v[idx + 1])), kmul2, nmk2);
        float2 pr;
        if (!C::SPLIT_P && (c >> 1) % kPolyPeriod < kPolyCount) {
          pr = exp2_poly2(x);
        } else {
          pr.x = ex2(x.x);
          pr.y = ex2(x.y);
        }
        if (c & 2) sumb = __fadd2_rn(sumb, pr); else suma = __fadd2_rn(suma, pr);
        const uint32_t hi = C::PV_F16 ? pack_f16_sat(pr.x, pr.y) : pack_bf16(pr.x, pr.y);
        pk[c >> 1] = hi;
        if constexpr (C::SPLIT_P) {
          // second bf16 term p - bf16(p): P = hi + lo carries 16 mantissa bits into the PV product
          const float2 rest =
              __fadd2_rn(pr, make_float2(-u2f(hi << 16), -u2f(hi & 0xffff0000u)));
          pk_lo[c >> 1] = pack_bf16(rest.x, rest.y);
        }
      }
      tmem_st16(tPs + chunk * 16, pk);   // stores overlap the next chunk's arithmetic
      if constexpr (C::SPLIT_P) tmem_st16(tPs + 64 + chunk * 16, pk_lo);
    }
    l += (suma.x + suma.y) + (sumb.x + sumb.y);
    }  // !done
    tmem_wait_st();
    tc_fence_before();
    mbar_arrive(sm.bar(BAR_P_FULL + s));
  }

  // Final row sum for the epilogue.  A row that saw no key (every score masked or -inf) still has
  // m = -inf; its sum may hold the tiny terms of clamped polynomial exponentials, so the running
  // maximum decides: such a row gets sum 0, which the epilogue turns into a row of zeros.
  const bool no_key = m == -CUDART_INF_F;
  if constexpr (C::ROWLOOP) {
    // the epilogue must have taken the previous row's sums before they are replaced
    if (row_index > 0) FLB_WAIT(sm, BAR_O_FREE + s, (row_index - 1) & 1);
  }
  sscale[row] = no_key ? 0.f : l;
  mbar_arrive(sm.bar(BAR_SCALE_FULL + s));
  if constexpr (!C::DIFF) {
    // log-sum-exp of the row: m and log2(l) are in log2 units of the modified scores
    if (p.lse != nullptr && i < p.L) {
      const float lse2 = (no_key || !(l > 0.f)) ? -CUDART_INF_F : fmaf(m, mdom, log2f(l));
      p.lse[n * p.lse_sn + h * p.lse_sh + i] = lse2 * 0.6931471805599453f;
    }
  }
}

// ------------------------------------------------------------------------------------------
// pointwise pass of the back-to-back product (takes the place of the softmax warps): bf16(f(S * scale))
// goes back to tensor memory as the A operand of the second product; no maximum, no sum, no rescale
// ------------------------------------------------------------------------------------------
template <class C>
FLB_DEV void pointwise_role(const Smem<C>& sm, uint32_t tmem, const KernelParams& p, int s, TileRange rg) {
  const int row = threadIdx.x & 127;
  const uint32_t lane_base = static_cast<uint32_t>((threadIdx.x >> 5) & 3) * 32u;
  const uint32_t tS = tmem + (s ? C::COL_S1 : C::COL_S0) + (lane_base << 16);
  const uint32_t tPs = C::SEP_P ? tmem + (s ? C::COL_P1 : C::COL_P0) + (lane_base << 16) : tS;
  const float2 sc2 = make_float2(p.scale, p.scale);
#pragma unroll 1
  for (int it = 0; it < rg.hi - rg.lo; ++it) {
    FLB_WAIT(sm, BAR_S_FULL + s, it & 1);
    tc_fence_after();
    uint32_t v[128];
    tmem_ld128_sync(tS, v);
    if constexpr (C::SEP_P) {
      tc_fence_before();
      mbar_arrive(sm.bar(BAR_S_FREE + s));
      if (it > 0) FLB_WAIT(sm, BAR_PV_DONE + s, (it - 1) & 1);
    }
    uint32_t pk[64];
    if (p.pointwise == PW_IDENTITY || p.pointwise == PW_RELU) {
      const float floor_ = p.pointwise == PW_RELU ? 0.f : -CUDART_INF_F;
#pragma unroll
      for (int c = 0; c < 128; c += 2) {
        const float2 x = __fmul2_rn(make_float2(u2f(v[c]), u2f(v[c + 1])), sc2);
        pk[c >> 1] = pack_bf16(fmaxf(x.x, floor_), fmaxf(x.y, floor_));
      }
    } else {
      // tanh(x), or sigmoid(x) = 0.5 tanh(x / 2) + 0.5
      const bool sig = p.pointwise == PW_SIGMOID;
      const float pre = sig ? 0.5f * p.scale : p.scale, mul = sig ? 0.5f : 1.0f, add = sig ? 0.5f : 0.0f;
#pragma unroll
      for (int c = 0; c < 128; c += 2) {
        const float a = fmaf(tanh_approx(u2f(v[c]) * pre), mul, add);
        const float b = fmaf(tanh_approx(u2f(v[c + 1]) * pre), mul, add);
        pk[c >> 1] = pack_bf16(a, b);
      }
    }
#pragma unroll
    for (int chunk = 0; chunk < 4; ++chunk) tmem_st16(tPs + chunk * 16, pk + chunk * 16);
    tmem_wait_st();
    tc_fence_before();
    mbar_arrive(sm.bar(BAR_P_FULL + s));
  }
  sm.scale(s)[row] = 1.0f;  // the epilogue's normalisation becomes a copy
  mbar_arrive(sm.bar(BAR_SCALE_FULL + s));
}

// ------------------------------------------------------------------------------------------
// fp16 P.V (differential attention with the RMS normalisation): the epilogue warps, idle until the last
// tile, rewrite every V tile in place as fp16 while the score products and the softmax of the tile run
// (a bf16 value is an fp16 value wherever the fp16 range holds it: V is first multiplied by the power of
// two that puts the tensor's largest magnitude at 2^13..2^14, which the RMS normalisation cancels).
// The tile is 128 rows of 128-byte swizzled boxes: element positions do not matter here, each thread
// converts 16-byte chunks where they lie.
// ------------------------------------------------------------------------------------------
template <class C>
FLB_DEV void convert_v_role(const Smem<C>& sm, const KernelParams& p, int lo, int hi) {
  static_assert(!C::PV_F16 || C::NSTAGE % 2 == 0, "V tiles must keep to the odd slots of the ring");
  const int tid = threadIdx.x & 127;
  const int n_pos = hi - lo;
  const float f = v_scale_from_absmax(*p.v_absmax);
#pragma unroll 1
  for (int t = 0; t < n_pos; ++t) {
    const int vseq = 2 * t + 1;
    const int vslot = vseq % C::NSTAGE;
    const uint32_t vph = (vseq / C::NSTAGE) & 1;
    FLB_WAIT(sm, BAR_KV_FULL + vslot, vph);
    uint4* tile = reinterpret_cast<uint4*>(sm.slot(vslot));
#pragma unroll 4
    for (int c = tid; c < C::V_BYTES / 16; c += 128) {
      uint4 w = tile[c];
      uint32_t* ww = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
      for (int e = 0; e < 4; ++e) ww[e] = pack_f16_sat(u2f(ww[e] << 16) * f, u2f(ww[e] & 0xffff0000u) * f);
      tile[c] = w;
    }
    fence_proxy_async_smem();
    mbar_arrive(sm.bar(BAR_V_CONV + vslot));
  }
}

// ------------------------------------------------------------------------------------------
// epilogue (one warpgroup serves both stages)
// ------------------------------------------------------------------------------------------
template <class C>
FLB_DEV void epilogue_role(const Smem<C>& sm, uint32_t tmem, const CUtensorMap* tmO,
                           const KernelParams& p, int n, int h, int vcol0, const int (&r0)[2],
                           const TileRange (&rg)[2], int lo, int hi) {
  const int row = threadIdx.x & 127;
  const uint32_t lane_base = static_cast<uint32_t>((threadIdx.x >> 5) & 3) * 32u;
  const uint32_t tO[2] = {tmem + C::COL_O0 + (lane_base << 16), tmem + C::COL_O1 + (lane_base << 16)};
  // The output tile goes to global memory as one TMA store per 64-column box: every thread puts
  // its row into shared memory (the stage's Q tile is dead by then) in the swizzled layout the
  // tensor map expects, and one thread issues the store once all 128 rows are in place.  Row-wise
  // 16-byte stores straight to global memory (32 sectors per warp instruction) kept the
  // load/store path busy for microseconds and held up the other stage's last tile.
  constexpr int ROWB = C::VBOX * 2;  // bytes per row of a box: 128, 64 or 32 = the swizzle span
  auto stage_row = [&](uint8_t* tile, int col, uint4 w) {
    const int box = col / C::VBOX, chunk = (col % C::VBOX) / 8;
    const int sw = ROWB == 128 ? (row & 7) : ROWB == 64 ? ((row >> 1) & 3) : ((row >> 2) & 1);
    *reinterpret_cast<uint4*>(tile + box * (128 * ROWB) + row * ROWB + ((chunk ^ sw) << 4)) = w;
  };
  auto store_tile = [&](uint8_t* tile, int s, int r_first) -> bool {
    fence_proxy_async_smem();  // generic-proxy writes above -> visible to the TMA engine
    mbar_arrive(sm.bar(BAR_O_STAGED + s));
    if (row == 0) {
      FLB_WAIT_RET(sm, BAR_O_STAGED + s, 0, false);
#pragma unroll
      for (int vb = 0; vb < C::NVB; ++vb)
        tma_store_4d(tmO, smem_u32(tile) + vb * (128 * ROWB), vcol0 + vb * C::VBOX, r_first, h, n);
      tma_store_commit();
    }
    return true;
  };
  if constexpr (!C::DIFF) {
#pragma unroll
    for (int s = 0; s < C::STAGES; ++s) {
      const int ns = rg[s].hi - rg[s].lo;
      if (ns <= 0) continue;
      FLB_WAIT(sm, BAR_SCALE_FULL + s, 0);
      const float l = sm.scale(s)[row];
      FLB_WAIT(sm, BAR_PV_DONE + s, (ns - 1) & 1);
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      uint8_t* tile = sm.q(s);  // E == EV here: the Q tile holds exactly one output tile
#pragma unroll
      for (int c0 = 0; c0 < C::EV; c0 += 32) {
        uint32_t o[32];
        tmem_ld32_sync(tO[s] + c0, o);
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          uint4 w;
          w.x = pack_bf16(u2f(o[c]) * inv, u2f(o[c + 1]) * inv);
          w.y = pack_bf16(u2f(o[c + 2]) * inv, u2f(o[c + 3]) * inv);
          w.z = pack_bf16(u2f(o[c + 4]) * inv, u2f(o[c + 5]) * inv);
          w.w = pack_bf16(u2f(o[c + 6]) * inv, u2f(o[c + 7]) * inv);
          stage_row(tile, c0 + c, w);
        }
      }
      if (!store_tile(tile, s, r0[s])) return;
    }
  } else {
    // out = O0 / l0 - lambda * O1 / l1, then x * rsqrt(mean(x^2) + eps) over the head's EV features
    const int ns = rg[0].hi - rg[0].lo;
    if (ns <= 0) return;
    float inv[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      FLB_WAIT(sm, BAR_SCALE_FULL + s, 0);
      const float l = sm.scale(s)[row];
      inv[s] = l > 0.f ? 1.0f / l : 0.f;
      FLB_WAIT(sm, BAR_PV_DONE + s, (ns - 1) & 1);
    }
    tc_fence_after();
    const float w1 = p.lambda * inv[1];
    float ss = 0.f;
    if (p.rms_norm) {
#pragma unroll
      for (int c0 = 0; c0 < C::EV; c0 += 16) {
        uint32_t a[16], b[16];
        tmem_ld16_sync(tO[0] + c0, a);
        tmem_ld16_sync(tO[1] + c0, b);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float d = u2f(a[c]) * inv[0] - u2f(b[c]) * w1;
          ss = fmaf(d, d, ss);
        }
      }
    }
    if (p.rms_norm && p.v_exchange) {
      // this CTA holds half of the row's columns: hand the partner this half's sum of squares (a
      // plain store into its shared memory, then an arrival on its barrier) and take its half
      const uint32_t partner = cluster_ctarank() ^ 1u;
      cluster_store_f32(cluster_map(smem_u32(sm.xchg() + row), partner), ss);
      cluster_mbar_arrive(cluster_map(sm.xbar(), partner));
      if (!mbar_wait_cluster(sm.xbar(), 0, sm.ctl())) {
        atomicCAS(&sm.ctl()->fail_bar, -1, static_cast<int>(BAR_COUNT));
        return;
      }
      ss += sm.xchg()[row];
    }
    float eps = p.rms_eps;
    if constexpr (C::PV_F16) {
      // the accumulators carry V's power-of-two factor f: eps * f^2 keeps x * rsqrt(mean(x^2) + eps) as it was
      const float f = v_scale_from_absmax(*p.v_absmax);
      eps *= f * f;
    }
    const float rs = p.rms_norm ? rsqrtf(ss * p.inv_ev + eps) : 1.0f;
    uint8_t* tile = sm.q(0);  // both Q tiles (2 * 128 * E * 2 bytes = one 128 x EV output tile)
    static_assert(2 * C::Q_BYTES >= 128 * C::EV * 2, "output tile does not fit the Q tiles");
#pragma unroll
    for (int c0 = 0; c0 < C::EV; c0 += 16) {
      uint32_t a[16], b[16];
      tmem_ld16_sync(tO[0] + c0, a);
      tmem_ld16_sync(tO[1] + c0, b);
      float d[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) d[c] = (u2f(a[c]) * inv[0] - u2f(b[c]) * w1) * rs;
#pragma unroll
      for (int c = 0; c < 16; c += 8) {
        uint4 w;
        w.x = pack_bf16(d[c], d[c + 1]);
        w.y = pack_bf16(d[c + 2], d[c + 3]);
        w.z = pack_bf16(d[c + 4], d[c + 5]);
        w.w = pack_bf16(d[c + 6], d[c + 7]);
        stage_row(tile, c0 + c, w);
      }
    }
    if (!store_tile(tile, 0, r0[0])) return;
  }
  // shared memory must stay intact until the stores have read it
  if (row == 0) tma_store_wait_read();
}

// Epilogue of the resident-bias kernel: one result tile per row and stage, staged in buffers of
// its own so that the next row's Q tile can load while the store reads.
template <class C>
FLB_DEV void epilogue_role_rows(const Smem<C>& sm, uint32_t tmem, const CUtensorMap* tmO,
                                const KernelParams& p, int h, int r0, RowWalk rw) {
  const int row = threadIdx.x & 127;
  const uint32_t lane_base = static_cast<uint32_t>((threadIdx.x >> 5) & 3) * 32u;
  const uint32_t tO[2] = {tmem + C::COL_O0 + (lane_base << 16), tmem + C::COL_O1 + (lane_base << 16)};
  constexpr int ROWB = C::VBOX * 2;
  const int sw = ROWB == 128 ? (row & 7) : ROWB == 64 ? ((row >> 1) & 3) : ((row >> 2) & 1);
  const int pairs = rw.items(0);
#pragma unroll 1
  for (int item = 0; item < pairs; ++item) {
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      if (item >= rw.items(s)) continue;
      FLB_WAIT(sm, BAR_SCALE_FULL + s, item & 1);
      const float l = sm.scale(s)[row];
      FLB_WAIT(sm, BAR_PV_DONE + s, ((item + 1) * rw.nt - 1) & 1);
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      // this stage's staging buffer is free once at most the other stage's store is still reading
      if (row == 0) tma_store_wait_read_pending<1>();
      named_bar_sync(3, 128);
      uint8_t* tile = sm.ostage(s);
#pragma unroll
      for (int c0 = 0; c0 < C::EV; c0 += 32) {
        uint32_t o[32];
        tmem_ld32_sync(tO[s] + c0, o);
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          uint4 w;
          w.x = pack_bf16(u2f(o[c]) * inv, u2f(o[c + 1]) * inv);
          w.y = pack_bf16(u2f(o[c + 2]) * inv, u2f(o[c + 3]) * inv);
          w.z = pack_bf16(u2f(o[c + 4]) * inv, u2f(o[c + 5]) * inv);
          w.w = pack_bf16(u2f(o[c + 6]) * inv, u2f(o[c + 7]) * inv);
          const int col = c0 + c, box = col / C::VBOX, chunk = (col % C::VBOX) / 8;
          *reinterpret_cast<uint4*>(tile + box * (128 * ROWB) + row * ROWB + ((chunk ^ sw) << 4)) = w;
        }
      }
      // accumulator and row sums are in registers: the next row may overwrite them
      tc_fence_before();
      mbar_arrive(sm.bar(BAR_O_FREE + s));
      fence_proxy_async_smem();
      named_bar_sync(3, 128);
      if (row == 0) {
#pragma unroll
        for (int vb = 0; vb < C::NVB; ++vb)
          tma_store_4d(tmO, smem_u32(tile) + vb * (128 * ROWB), vb * C::VBOX, r0, h, rw.n0 + 2 * item + s);
        tma_store_commit();
      }
    }
  }
  if (row == 0) tma_store_wait_read();
}

// ------------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------------
template <class C>
__global__ void __launch_bounds__(C::THREADS, C::STAGES == 2 ? 1 : 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                const __grid_constant__ CUtensorMap tmB, const __grid_constant__ KernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  Smem<C> sm{reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                        ~static_cast<uintptr_t>(1023))};
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Order of the work items over blockIdx.x (thread blocks start in that order): the (batch, head)
  // axis is cut into sections whose K/V fit in L2 together; inside a section the query blocks run
  // from the heaviest down, (batch, head) fastest, so the CTAs that run at the same time stream the
  // same K/V.
  const int bh_count = p.N * p.H;
  const int per_sec = p.sec_bh * p.nq_blocks;
  // (differential attention with wide value heads: neighbouring CTAs share a work item and take one
  // half of the value columns each)
  const int vhalves = C::DIFF ? p.v_halves : 1;
  const int item = static_cast<int>(blockIdx.x) / vhalves;
  const int vcol0 = C::DIFF ? (static_cast<int>(blockIdx.x) % vhalves) * C::EV : 0;
  const int sec = item / per_sec;
  const int bh0 = sec * p.sec_bh;
  const int width = min(p.sec_bh, bh_count - bh0);  // the last section may be narrower
  const int wi = item - sec * per_sec;
  const int qb = p.nq_blocks - 1 - wi / width;
  const int bh = bh0 + wi % width;
  const int n = bh / p.H, h = bh % p.H;
  int r0[2];
  if constexpr (C::DIFF || C::STAGES == 1) {
    r0[0] = r0[1] = qb * kTileM;
  } else {
    r0[0] = qb * 2 * kTileM;
    r0[1] = r0[0] + kTileM;
  }
  TileRange rg[2];
  rg[0] = tile_range<C::MASK>(p, n, r0[0]);
  rg[1] = C::STAGES == 2 ? tile_range<C::MASK>(p, n, r0[1]) : TileRange{0, 0};
  int lo = 0x7fffffff, hi = 0;
#pragma unroll
  for (int s = 0; s < C::STAGES; ++s)
    if (rg[s].hi > rg[s].lo) {
      lo = min(lo, rg[s].lo);
      hi = max(hi, rg[s].hi);
    }
  if (hi == 0) lo = 0;
  // Resident-bias kernel: blockIdx.x = ((batch element, head), query tile, chunk of rows), chunk
  // fastest; the "tile ranges" of the two stages string together the tiles of their rows.
  [[maybe_unused]] RowWalk rw{0, 0, 0};
  [[maybe_unused]] int rb_b = 0, rb_h = 0;
  if constexpr (C::ROWLOOP) {
    const int chunk = static_cast<int>(blockIdx.x) % p.res_chunks;
    const int rest = static_cast<int>(blockIdx.x) / p.res_chunks;
    const int qtile = rest % p.nq_blocks;
    const int bhh = rest / p.nq_blocks;
    rb_b = bhh / p.H;
    rb_h = bhh % p.H;
    const int ra = chunk * p.res_rows;
    rw.n0 = rb_b * p.evo_inner + ra;
    rw.count = max(0, min(p.evo_inner, ra + p.res_rows) - ra);
    rw.nt = (p.S + kTileN - 1) / kTileN;
    r0[0] = r0[1] = qtile * kTileM;
    rg[0] = TileRange{0, rw.items(0) * rw.nt};
    rg[1] = TileRange{0, rw.items(1) * rw.nt};
    lo = 0;
    hi = rg[0].hi;
    // A operand of the key-vector k-step: rows [1, 1, 0 x 6 | 1, 1, 0 x 6] (both 16-byte chunks alike,
    // so the 32-byte swizzle leaves the tile as written); the set-up barriers below publish it
    if (p.keyvec_rows != nullptr && threadIdx.x < 128) {
      uint4* r = reinterpret_cast<uint4*>(sm.kvx(p.res_slots, rw.nt, 0) + threadIdx.x * 32);
      r[0] = make_uint4(0x3F803F80u, 0, 0, 0);
      r[1] = make_uint4(0x3F803F80u, 0, 0, 0);
      fence_proxy_async_smem();
    }
  }

  // the warps that issue loads (the resident-bias kernel has one per stage, and one MMA warp per stage:
  // warps 12 / 13 serve stage 0, warps 14 / 15 stage 1)
  const bool is_producer = warp == C::W_TMA || (C::ROWLOOP && warp == C::W_TMA + 2);
  constexpr int kEarly = C::ROWLOOP ? 96 : 64;  // warp 0 and the producer warps meet on barrier 1
  // Set-up: the lanes of warp 0 initialise one mbarrier each while warp 1 allocates tensor memory
  // and the producer lane fetches the tensor maps.  The producer warp needs only the mbarriers: it
  // meets warp 0 on a barrier of their own and starts the first loads while the rest of the CTA
  // still waits for the tensor-memory allocation.
  if (warp == 0) {
    if (lane == 0) {
      sm.ctl()->abort = 0;
      sm.ctl()->fail_bar = -1;
      sm.ctl()->limit_us = p.wait_limit_us;
    }
    if (lane < 32) {
      const bool all_threads = (lane >= BAR_P_FULL && lane < BAR_PV_DONE) ||
                               (lane >= BAR_P_HALF && lane < BAR_KV_FULL) || lane >= BAR_S_FREE;
      // (resident-bias kernel: Q_EMPTY, which takes the place of P_HALF, is a single commit)
      const bool single = C::ROWLOOP && lane >= BAR_Q_EMPTY && lane < BAR_Q_EMPTY + 2;
      mbar_init(sm.bar(lane), all_threads && !single ? 128 : 1);  // 128 arriving threads, or one commit / TMA
      if (C::ROWLOOP && lane < 16) mbar_init(sm.bar(32 + lane), 1);  // ring slots handed back by commits
      if (C::PV_F16 && lane < 8) mbar_init(sm.bar(BAR_V_CONV + lane), 128);
    }
    if (C::DIFF && lane == 0) mbar_init(sm.xbar(), 128);
    fence_mbar_init();
    named_bar_sync(1, kEarly);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(sm.tmem_base()), C::TMEM_COLS);
    tmem_relinquish();
  }
  uint32_t tmem = 0;
  if (is_producer) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmO);
      if constexpr (C::ROWLOOP) tma_prefetch_desc(&tmB);
    }
    named_bar_sync(1, kEarly);
  } else {
    tc_fence_before();
    named_bar_sync(2, C::THREADS - (kEarly - 32));
    tc_fence_after();
    tmem = *sm.tmem_base();
  }
  // a CTA pair that will exchange row sums: neither may write into the other before its barrier
  // exists (the producer warp passed the barrier initialisation above, too)
  if (C::DIFF && p.v_exchange) cluster_sync_all();
  // A launch in which some CTA already gave up is not worth finishing: one thread of the MMA warp's
  // group that has nothing else to do looks at the status word and raises the abort flag, which
  // ends every role at its next long wait.  The look-up stays off the path to the first MMA.
  if (threadIdx.x == (C::W_MMA + 3) * 32 + 1 && p.status != nullptr &&
      *reinterpret_cast<volatile int*>(p.status) != 0)
    sm.ctl()->abort = 1;

  if (warp < C::W_SOFTMAX_END) {
    reg_inc<C::STAGES == 2 ? kRegsSoftmax : kRegsSoftmax1>();
    const int s = warp >> 2;
    if constexpr (C::ROWLOOP) {
      for (int ri = 0; ri < rw.items(s) && !sm.ctl()->abort; ++ri)
        softmax_role<C>(sm, tmem, p, s, rw.n0 + 2 * ri + s, rb_h, r0[s], TileRange{0, rw.nt}, ri);
    } else if (rg[s].hi > rg[s].lo) {
      if constexpr (C::B2B) pointwise_role<C>(sm, tmem, p, s, rg[s]);
      else softmax_role<C>(sm, tmem, p, s, n, h, r0[s], rg[s]);
    }
    // one query tile per CTA: its softmax warps also write the result
    if constexpr (C::STAGES == 1) epilogue_role<C>(sm, tmem, &tmO, p, n, h, vcol0, r0, rg, lo, hi);
  } else if (C::STAGES == 2 && warp < 12) {
    reg_dec<kRegsEpilogue>();
    if constexpr (C::PV_F16) convert_v_role<C>(sm, p, lo, hi);
    if constexpr (C::ROWLOOP) epilogue_role_rows<C>(sm, tmem, &tmO, p, rb_h, r0[0], rw);
    else epilogue_role<C>(sm, tmem, &tmO, p, n, h, vcol0, r0, rg, lo, hi);
  } else {
    reg_dec<C::STAGES == 2 ? kRegsIssue : kRegsIssue1>();
    if constexpr (C::ROWLOOP) {
      const int s = (warp - C::W_MMA) >> 1;  // warps 12, 13: stage 0; 14, 15: stage 1
      if (rw.items(s) > 0) {
        if (((warp - C::W_MMA) & 1) == 0) mma_role_rows<C>(sm, tmem, p, s, rw);
        else if (lane == 0) load_role_rows<C>(sm, &tmQ, &tmK, &tmV, &tmB, p, s, rb_b, rb_h, r0[0], rw);
      }
    } else if (hi > lo) {
      if (warp == C::W_MMA) mma_role<C>(sm, tmem, p, rg, lo, hi);
      if (warp == C::W_TMA && lane == 0) load_role<C>(sm, &tmQ, &tmK, &tmV, p, n, h, vcol0, r0, rg, lo, hi);
    }
    __syncwarp();
  }

  // common exit: every role arrives here, also after a timed-out wait
  tc_fence_before();
  __syncthreads();
  // a CTA pair leaves together: the partner may still be storing into this CTA's shared memory
  if (C::DIFF && p.v_exchange) cluster_sync_all();
  if (sm.ctl()->abort) {
    // give loads that are still in flight time to land before shared memory and TMEM go away
    for (int k = 0; k < 64; ++k) __nanosleep(20000);
    if (threadIdx.x == 0 && p.status) {
      const int word =
          (kStatusTimeout << 24) | ((sm.ctl()->fail_bar & 0xff) << 16) | (blockIdx.x & 0xffff);
      if (atomicCAS(p.status, 0, word) == 0 && p.status_host != nullptr) {
        *reinterpret_cast<volatile int*>(p.status_host) = word;
        __threadfence_system();
      }
    }
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(*sm.tmem_base(), C::TMEM_COLS);
}

}  // namespace flb
