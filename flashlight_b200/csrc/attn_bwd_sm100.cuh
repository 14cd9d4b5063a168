// Attention backward for sm_100a: dQ, dK, dV of softmax(Q K^T * scale [+ causal mask]) V from the
// forward's inputs, its output, its row-wise log-sum-exp and the output's gradient.
//
// Three kernels, none of which needs an atomic or a transpose in memory:
//
//   attn_bwd_delta_kernel   delta[i] = sum_d dO[i][d] * O[i][d]  (fp32, sixteen lanes per query row)
//
//   attn_bwd_dq_kernel      one CTA per (batch, query head, 128-row query tile); walks the key tiles:
//                             S = Q K^T, dP = dO V^T            (tcgen05 SS products into tensor memory)
//                             P = exp2(S * scale_log2 - lse2),  dS = P * (dP - delta)   (scale: epilogue)
//                             dQ += dS K                         (dS read from tensor memory)
//
//   attn_bwd_dkv_kernel     one CTA per (batch, kv head, 128-key tile); walks the query tiles of every
//                           query head of the group, with the roles of rows and columns swapped
//                           (tensor-memory lanes are keys):
//                             S^T = K Q^T, dP^T = V dO^T;  P^T, dS^T as above (lse2, delta per column)
//                             dV += P^T dO,  dK += dS^T Q
//                           Here lse2 and delta belong to the columns, and reading 128 of them per thread
//                           and step from shared memory cost as much as the exponentials.  The tensor
//                           cores subtract them instead: the delta kernel also writes, per query row,
//                           x = -lse / scale and y = -delta as two bf16 terms each (16-column rows
//                           [hi, lo, 0...]), and each score product takes one more k-step of 16 against a
//                           resident tile of ones: S^T + x_i = (s - lse / scale), dP^T + y_i = dP - delta.
//
// The score products are recomputed in both kernels (7 tile products per pair of tiles instead of 5);
// in exchange every accumulator stays in one CTA's tensor memory from start to finish.
// Tensor memory, one CTA per SM: dQ kernel S 2 x 128 (two buffers) + dP 128 + dQ D; dK/dV kernel
// S 128 + dP 128 + dV D + dK D (all 512 columns at D = 128).  320 threads: warps 0-7 pointwise pass and
// epilogue (two threads per tensor-memory lane, 64 of the tile's 128 columns each), warp 8 MMA issue,
// warp 9 TMA producer.  In the dQ kernel the products of the next key tile run under the pointwise
// pass of the current one: S(t+1) goes to the other score buffer as soon as its K tile has landed, the
// exponentials of a tile need only S, and dP(t+1) follows dQ(t) once the pass has released the dP
// columns (with two dP buffers and one score buffer instead, the kernel measured 12 % slower).
// All waits are bounded as in the forward kernel.
#pragma once
#include <cuda.h>
#include <math_constants.h>

#include "ptx.cuh"

namespace flb {

struct BwdParams {
  int N, Hq, Hkv, L, S, G;
  float scale, scale_log2;
  int causal;
  const float* lse;  // [N][Hq][L], natural log
  int64_t lse_sn, lse_sh;
  float* delta;      // [N][Hq][Lp], Lp = L rounded up to 128
  int Lp;
  int* status;
  int* status_host;
  uint32_t wait_limit_us;
  int withhold_loads;  // wait self-test: the producers load nothing, every role's first wait runs out
};

enum : int {
  BB_RES_FULL = 0,  // the CTA's resident tiles (Q, dO or K, V) have landed
  BB_SP_FULL = 1,   // MMA -> pointwise: score tile written (+buffer in the dQ kernel)
  BB_P_FULL = 6,    // pointwise -> MMA: P^T written back (dK/dV kernel, 256 arrivals)
  BB_DP_FULL = 3,   // MMA -> pointwise: dP written
  BB_DS_FULL = 4,   // pointwise -> MMA: P / dS written back (256 arrivals)
  BB_ACC_DONE = 5,  // MMA -> epilogue: accumulators final
  BB_RING_FULL = 8,    // +slot: the slot's first tile (dQ kernel: K), or both (dK/dV kernel)
  BB_RING_EMPTY = 12,  // +slot
  BB_RING2_FULL = 16,  // +slot: the slot's second tile (dQ kernel: V)
  BB_RING2_EMPTY = 20, // +slot
  BB_COUNT = 24
};
static_assert(BB_COUNT * 8 <= 256, "the barriers end where the tensor-memory base word begins");
constexpr int kBwdPointwiseThreads = 256;
// of every kBwdPolyPeriod column pairs, kBwdPolyCount take their exponentials from the FMA-pipe polynomial
// (none, one in four and one in two measured within 3 % of each other)
constexpr int kBwdPolyPeriod = 4, kBwdPolyCount = 1;
FLB_DEV float2 bwd_exp2_pair(float2 x, int pair) {
  if (pair % kBwdPolyPeriod < kBwdPolyCount) return exp2_poly2(x);
  return make_float2(ex2(x.x), ex2(x.y));
}
constexpr int kBwdThreads = kBwdPointwiseThreads + 64;

template <int D_>
struct BwdCfg {
  static constexpr int D = D_;
  static_assert(D == 64 || D == 128, "backward kernels are built for head dims 64 and 128");
  static constexpr int NB = D / 64;                 // 64-column boxes per tile
  static constexpr int BOX_BYTES = 128 * 64 * 2;    // 16 KB
  static constexpr int TILE_BYTES = 128 * D * 2;
  static constexpr int SLOT_BYTES = 2 * TILE_BYTES;  // a ring slot holds the step's two streamed tiles
  static constexpr int NSLOT = D == 128 ? 2 : 4;
  static constexpr int AUX_BYTES = 1024;
  static constexpr int AUG_TILE_BYTES = 128 * 16 * 2;  // 128 rows of 16 bf16, 32-byte swizzled
  static constexpr int AUG_BYTES = AUG_TILE_BYTES * (1 + 2 * NSLOT);   // ones, then (x, y) per ring slot
  static constexpr int SMEM_BYTES = 1024 + 2 * TILE_BYTES + NSLOT * SLOT_BYTES + AUX_BYTES + AUG_BYTES;
  static_assert(SMEM_BYTES > 120 * 1024, "one CTA per SM: each takes all of tensor memory");
};

template <class C>
struct BwdSmem {
  uint8_t* base;
  FLB_DEV uint8_t* res(int i) const { return base + i * C::TILE_BYTES; }  // resident tile 0 / 1
  FLB_DEV uint8_t* slot(int s, int i) const { return base + 2 * C::TILE_BYTES + s * C::SLOT_BYTES + i * C::TILE_BYTES; }
  FLB_DEV uint8_t* aux() const { return base + 2 * C::TILE_BYTES + C::NSLOT * C::SLOT_BYTES; }
  FLB_DEV uint8_t* ones() const { return aux() + C::AUX_BYTES; }
  FLB_DEV uint8_t* aug(int s, int i) const { return ones() + C::AUG_TILE_BYTES * (1 + 2 * s + i); }  // x: 0, y: 1
  FLB_DEV uint32_t bar(int id) const { return smem_u32(aux()) + id * 8; }
  FLB_DEV uint32_t* tmem_base() const { return reinterpret_cast<uint32_t*>(aux() + 256); }  // after BB_COUNT barriers
  FLB_DEV WaitCtl* ctl() const { return reinterpret_cast<WaitCtl*>(aux() + 260); }
};

#define FLB_BWAIT(sm, id, parity)                                 \
  do {                                                            \
    if (!mbar_wait((sm).bar(id), (parity), (sm).ctl())) {         \
      atomicCAS(&(sm).ctl()->fail_bar, -1, 64 + (id));            \
      return;                                                     \
    }                                                             \
  } while (0)

// descriptor low/high words for a 128-row tile of 64-column, 128-byte-swizzled boxes
//   K-major (rows are M or N, the features are the contraction axis)
//   MN-major (rows are the contraction axis, the features are N)
template <class C>
struct BwdDesc {
  static constexpr uint64_t kmaj = (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 16) | (1ull << 46) |
                                   (static_cast<uint64_t>(kSwz128) << 61);
  static constexpr uint64_t mnmaj = (static_cast<uint64_t>(1024 >> 4) << 32) |
                                    (static_cast<uint64_t>(C::BOX_BYTES >> 4) << 16) | (1ull << 46) |
                                    (static_cast<uint64_t>(kSwz128) << 61);
  static constexpr uint32_t k_hi = static_cast<uint32_t>(kmaj >> 32), k_lo = static_cast<uint32_t>(kmaj);
  static constexpr uint32_t mn_hi = static_cast<uint32_t>(mnmaj >> 32), mn_lo = static_cast<uint32_t>(mnmaj);
  FLB_DEV static uint32_t addr(const void* p) { return (smem_u32(p) & 0x3FFFFu) >> 4; }
};

// D[tmem 128 x 128] = A[128 x D] * B[128 x D]^T, both K-major tiles in shared memory
template <class C>
FLB_DEV void bwd_mma_scores(uint32_t leader, uint32_t d_tmem, const void* a_tile, const void* b_tile) {
  using Ds = BwdDesc<C>;
  constexpr uint32_t idesc = make_idesc_bf16(128, 128, 0, 0);
  const uint32_t a = Ds::k_lo + Ds::addr(a_tile), b = Ds::k_lo + Ds::addr(b_tile);
  umma_ss_c<0>(leader, d_tmem, a, b, Ds::k_hi, idesc);
#pragma unroll
  for (int k = 1; k < C::D / 16; ++k) {
    const int kk = k * 16;
    const uint32_t off = ((kk / 64) * C::BOX_BYTES + (kk % 64) * 2) >> 4;
    umma_ss_c<1>(leader, d_tmem, a + off, b + off, Ds::k_hi, idesc);
  }
}

// D[tmem 128 x 128] += A[128 x 16] * B[128 x 16]^T, both K-major tiles of 32-byte swizzled rows
template <class C>
FLB_DEV void bwd_mma_aug(uint32_t leader, uint32_t d_tmem, const void* a_tile, const void* b_tile) {
  constexpr uint64_t d32 = (static_cast<uint64_t>(256 >> 4) << 32) | (1ull << 16) | (1ull << 46) |
                           (static_cast<uint64_t>(kSwz32) << 61);
  constexpr uint32_t hi = static_cast<uint32_t>(d32 >> 32), lo = static_cast<uint32_t>(d32);
  constexpr uint32_t idesc = make_idesc_bf16(128, 128, 0, 0);
  umma_ss_c<1>(leader, d_tmem, lo + BwdDesc<C>::addr(a_tile), lo + BwdDesc<C>::addr(b_tile), hi, idesc);
}

// D[tmem 128 x D] (+)= A[tmem 128 x 128, bf16] * B[128 x D], B an MN-major tile in shared memory.  The A
// operand lies where the two pointwise threads of a lane wrote it: contraction indices 0-63 in columns
// 0-31 of the score buffer, 64-127 in columns 64-95 (each thread writes over columns it has read itself).
template <class C>
FLB_DEV void bwd_mma_acc(uint32_t leader, uint32_t d_tmem, uint32_t a_tmem, const void* b_tile, bool accumulate) {
  using Ds = BwdDesc<C>;
  constexpr uint32_t idesc = make_idesc_bf16(128, C::D, 0, 1);
  const uint32_t b = Ds::mn_lo + Ds::addr(b_tile);
  if (accumulate) umma_ts_c<1>(leader, d_tmem, a_tmem, b, Ds::mn_hi, idesc);
  else umma_ts_c<0>(leader, d_tmem, a_tmem, b, Ds::mn_hi, idesc);
#pragma unroll
  for (int k = 1; k < 8; ++k)
    umma_ts_c<1>(leader, d_tmem, a_tmem + (k / 4) * 64 + (k % 4) * 8, b + ((k * 16 * 128) >> 4), Ds::mn_hi, idesc);
}

template <class C>
FLB_DEV void bwd_load_tile(uint8_t* dst, const CUtensorMap* tm, uint32_t bar, int row0, int head, int n) {
#pragma unroll
  for (int b = 0; b < C::NB; ++b)
    tma_load_4d(smem_u32(dst) + b * C::BOX_BYTES, tm, bar, b * 64, row0, head, n);
}

// accumulator rows (fp32, `D` columns at `t_acc`) -> bf16 tile in shared memory in the layout of the
// output tensor map (128-byte swizzled boxes of 64 columns)
template <class C, int COLS>
FLB_DEV void bwd_stage_rows(uint32_t t_acc, uint8_t* tile, int row, int col_first, float mul) {
  const int sw = row & 7;
#pragma unroll
  for (int cc = 0; cc < COLS; cc += 32) {
    const int c0 = col_first + cc;
    uint32_t o[32];
    tmem_ld32_sync(t_acc + c0, o);
#pragma unroll
    for (int c = 0; c < 32; c += 8) {
      uint4 w;
      w.x = pack_bf16(__uint_as_float(o[c]) * mul, __uint_as_float(o[c + 1]) * mul);
      w.y = pack_bf16(__uint_as_float(o[c + 2]) * mul, __uint_as_float(o[c + 3]) * mul);
      w.z = pack_bf16(__uint_as_float(o[c + 4]) * mul, __uint_as_float(o[c + 5]) * mul);
      w.w = pack_bf16(__uint_as_float(o[c + 6]) * mul, __uint_as_float(o[c + 7]) * mul);
      const int col = c0 + c, box = col / 64, chunk = (col % 64) / 8;
      *reinterpret_cast<uint4*>(tile + box * C::BOX_BYTES + row * 128 + ((chunk ^ sw) << 4)) = w;
    }
  }
}

template <class C>
FLB_DEV void bwd_setup(const BwdSmem<C>& sm, const BwdParams& p, int warp, int lane) {
  if (warp == 0) {
    if (lane == 0) {
      sm.ctl()->abort = 0;
      sm.ctl()->fail_bar = -1;
      sm.ctl()->limit_us = p.wait_limit_us;
    }
    if (lane < BB_COUNT) mbar_init(sm.bar(lane), lane == BB_DS_FULL || lane == BB_P_FULL ? kBwdPointwiseThreads : 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(sm.tmem_base()), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 9 * 32 + 1 && p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0)
    sm.ctl()->abort = 1;
}

template <class C>
FLB_DEV void bwd_exit(const BwdSmem<C>& sm, const BwdParams& p, int warp) {
  tc_fence_before();
  __syncthreads();
  if (sm.ctl()->abort) {
    for (int k = 0; k < 64; ++k) __nanosleep(20000);
    if (threadIdx.x == 0 && p.status) {
      const int word = (1 << 24) | ((sm.ctl()->fail_bar & 0xff) << 16) | (blockIdx.x & 0xffff);
      if (atomicCAS(p.status, 0, word) == 0 && p.status_host != nullptr) {
        *reinterpret_cast<volatile int*>(p.status_host) = word;
        __threadfence_system();
      }
    }
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(*sm.tmem_base(), 512);
}

// ------------------------------------------------------------------------------------------
// delta[n][h][i] = sum_d dO * O   (rows beyond L of the padded array: 0)
// ------------------------------------------------------------------------------------------
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                      int64_t o_sn, int64_t o_sh, int64_t o_sl, int64_t do_sn, int64_t do_sh,
                                      int64_t do_sl, int E, int Hq, int L, int Lp, float* __restrict__ delta,
                                      const float* __restrict__ lse, int64_t lse_sn, int64_t lse_sh, float inv_scale,
                                      uint4* __restrict__ xrows, uint4* __restrict__ yrows) {
  // 16 lanes per (n, h, i) row, 8 features (one 16-byte load per tensor) per lane, four consecutive rows
  // per lane group with their eight loads in flight together; rows start on 16-byte boundaries (pointers
  // and strides are checked by the host; the padded row count is a multiple of 128)
  constexpr int kRows = 4;
  const int row0 = (blockIdx.x * 16 + (threadIdx.x >> 4)) * kRows;
  const int sub = threadIdx.x & 15;
  const int d = sub * 8;
  const int nh = row0 / Lp, h = nh % Hq, n = nh / Hq, i0 = row0 % Lp;   // the four rows share (n, h)
  const __nv_bfloat16* po = o + n * o_sn + h * o_sh + d;
  const __nv_bfloat16* pd = d_o + n * do_sn + h * do_sh + d;
  uint4 a[kRows], b[kRows];
  const bool vec = d + 8 <= E;
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    a[r] = b[r] = make_uint4(0, 0, 0, 0);
    if (vec && i0 + r < L) {
      a[r] = *reinterpret_cast<const uint4*>(po + (i0 + r) * o_sl);
      b[r] = *reinterpret_cast<const uint4*>(pd + (i0 + r) * do_sl);
    }
  }
  const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    const int i = i0 + r, row = row0 + r;
    float acc = 0.f;
    if (vec) {
      const uint32_t aw[4] = {a[r].x, a[r].y, a[r].z, a[r].w}, bw[4] = {b[r].x, b[r].y, b[r].z, b[r].w};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        // a bf16 is the upper half of an fp32
        acc = fmaf(__uint_as_float(aw[w] << 16), __uint_as_float(bw[w] << 16), acc);
        acc = fmaf(__uint_as_float(aw[w] & 0xffff0000u), __uint_as_float(bw[w] & 0xffff0000u), acc);
      }
    } else if (i < L && d < E) {
      for (int e = 0; d + e < E; ++e)
        acc = fmaf(__bfloat162float(po[i * o_sl + e]), __bfloat162float(pd[i * do_sl + e]), acc);
    }
#pragma unroll
    for (int s = 8; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    // the rows of the extra k-step of the dK/dV kernel: [hi, lo, 0 x 14] of -lse / scale and of -delta
    // (rows of the padding beyond L: zeros; their Q and dO rows are zero-filled, so they contribute nothing)
    if (sub == 0) {
      delta[row] = acc;
      yrows[2 * static_cast<int64_t>(row)] = make_uint4(i < L ? split_bf16_pair(-acc) : 0u, 0, 0, 0);
    } else if (sub == 1) {
      yrows[2 * static_cast<int64_t>(row) + 1] = zero;
    } else if (sub == 2) {
      const float x = i < L ? -lse[n * lse_sn + h * lse_sh + i] * inv_scale : 0.f;
      xrows[2 * static_cast<int64_t>(row)] = make_uint4(i < L ? split_bf16_pair(x) : 0u, 0, 0, 0);
    } else if (sub == 3) {
      xrows[2 * static_cast<int64_t>(row) + 1] = zero;
    }
  }
}

// ------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------
template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdQ, const __grid_constant__ BwdParams p) {
  using C = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  BwdSmem<C> sm{reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023))};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.L + 127) / 128;
  // consecutive CTAs take the query tiles of one (batch, head), latest (heaviest under the causal mask)
  // first: the CTAs in flight then share a few heads' K and V, which stay in L2
  const int qt = nq - 1 - static_cast<int>(blockIdx.x) % nq;
  const int nh = static_cast<int>(blockIdx.x) / nq;
  const int n = nh / p.Hq, h = nh % p.Hq, kvh = h / p.G;
  const int i0 = qt * 128;
  const int nk_all = (p.S + 127) / 128;
  const int nk = CAUSAL ? min(nk_all, min(i0 + 127, p.L - 1) / 128 + 1) : nk_all;
  bwd_setup<C>(sm, p, warp, lane);
  const uint32_t tmem = *sm.tmem_base();
  const uint32_t tS0 = tmem, tdP0 = tmem + 256, tdQ = tmem + 384;   // score buffer b at tS0 + 128 b

  auto pointwise = [&]() {
    // pointwise pass: thread (row, half) owns columns [64 half, 64 half + 64) of the row's scores
    const int row = threadIdx.x & 127, half = threadIdx.x >> 7;
    const int i = i0 + row;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const bool live = i < p.L;
    const float lse2 = live ? p.lse[n * p.lse_sn + h * p.lse_sh + i] * 1.4426950408889634f : CUDART_INF_F;
    const float delta = live ? p.delta[(static_cast<int64_t>(n) * p.Hq + h) * p.Lp + i] : 0.f;
    const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), nlse2 = make_float2(-lse2, -lse2);
    const float2 ndelta2 = make_float2(-delta, -delta);
    for (int t = 0; t < nk; ++t) {
      const uint32_t tSh = tS0 + (t & 1) * 128 + half * 64 + lane_off, tdP = tdP0 + half * 64 + lane_off;
      const int j0 = t * 128 + half * 64;
      const bool partial = CAUSAL && j0 + 63 > i0;
      float2 pr[32];
      FLB_BWAIT(sm, BB_SP_FULL + (t & 1), (t >> 1) & 1);
      tc_fence_after();
      {
        uint32_t sv[64];
        tmem_ld32_pair_sync(tSh, sv, tSh + 32, sv + 32);
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, nlse2);
          float2 e = bwd_exp2_pair(x, c >> 1);
          if (partial) {
            if (j0 + c > i) e.x = 0.f;
            if (j0 + c + 1 > i) e.y = 0.f;
          }
          pr[c >> 1] = e;
        }
      }
      FLB_BWAIT(sm, BB_DP_FULL, t & 1);
      tc_fence_after();
      {
        uint32_t dp[64];
        tmem_ld32_pair_sync(tdP, dp, tdP + 32, dp + 32);
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float2 d = __fadd2_rn(make_float2(__uint_as_float(dp[c0 + c]), __uint_as_float(dp[c0 + c + 1])), ndelta2);
            const float2 g = __fmul2_rn(pr[(c0 + c) >> 1], d);
            pk[c >> 1] = pack_bf16(g.x, g.y);
          }
          tmem_st16(tSh + (c0 >> 1), pk);  // dS (bf16) over the thread's own score columns
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(sm.bar(BB_DS_FULL));
    }
    // epilogue: dQ tile -> bf16 -> shared memory (the Q tile is dead) -> TMA store
    if (nk > 0) {
      FLB_BWAIT(sm, BB_ACC_DONE, 0);
      tc_fence_after();
      bwd_stage_rows<C, D / 2>(tdQ + lane_off, sm.res(0), row, half * (D / 2), p.scale);
    }
    fence_proxy_async_smem();
    named_bar_sync(1, kBwdPointwiseThreads);
    if (threadIdx.x == 0 && nk > 0) {
#pragma unroll
      for (int b = 0; b < C::NB; ++b)
        tma_store_4d(&tmdQ, smem_u32(sm.res(0)) + b * C::BOX_BYTES, b * 64, i0, h, n);
      tma_store_commit();
      tma_store_wait_read();
    }
  };
  auto issue = [&]() {
    const uint32_t leader = elect_one() ? 1u : 0u;
    if (nk > 0) {
      FLB_BWAIT(sm, BB_RES_FULL, 0);
      FLB_BWAIT(sm, BB_RING_FULL + 0, 0);
      tc_fence_after();
      bwd_mma_scores<C>(leader, tS0, sm.res(0), sm.slot(0, 0));                     // S(0) = Q K^T
      umma_commit_c(leader, sm.bar(BB_SP_FULL + 0));
      FLB_BWAIT(sm, BB_RING2_FULL + 0, 0);
      tc_fence_after();
      bwd_mma_scores<C>(leader, tdP0, sm.res(1), sm.slot(0, 1));                    // dP(0) = dO V^T
      umma_commit_c(leader, sm.bar(BB_RING2_EMPTY + 0));
      umma_commit_c(leader, sm.bar(BB_DP_FULL));
      for (int t = 0; t < nk; ++t) {
        const int slot = t % C::NSLOT;
        if (t + 1 < nk) {
          // the other score buffer held dS(t-1), which the dQ product issued before this point has read
          const int s1 = (t + 1) % C::NSLOT;
          FLB_BWAIT(sm, BB_RING_FULL + s1, ((t + 1) / C::NSLOT) & 1);
          tc_fence_after();
          bwd_mma_scores<C>(leader, tS0 + ((t + 1) & 1) * 128, sm.res(0), sm.slot(s1, 0));   // S(t+1)
          umma_commit_c(leader, sm.bar(BB_SP_FULL + ((t + 1) & 1)));
        }
        FLB_BWAIT(sm, BB_DS_FULL, t & 1);   // dS(t) written, the dP columns read
        tc_fence_after();
        bwd_mma_acc<C>(leader, tdQ, tS0 + (t & 1) * 128, sm.slot(slot, 0), t > 0);   // dQ += dS K
        umma_commit_c(leader, sm.bar(BB_RING_EMPTY + slot));
        if (t + 1 < nk) {
          const int s1 = (t + 1) % C::NSLOT;
          FLB_BWAIT(sm, BB_RING2_FULL + s1, ((t + 1) / C::NSLOT) & 1);
          tc_fence_after();
          bwd_mma_scores<C>(leader, tdP0, sm.res(1), sm.slot(s1, 1));                // dP(t+1)
          umma_commit_c(leader, sm.bar(BB_RING2_EMPTY + s1));
          umma_commit_c(leader, sm.bar(BB_DP_FULL));
        }
      }
      umma_commit_c(leader, sm.bar(BB_ACC_DONE));
    }
  };
  auto produce = [&]() {
    if (p.withhold_loads) return;
    if (nk > 0) {
      mbar_arrive_expect_tx(sm.bar(BB_RES_FULL), 2 * C::TILE_BYTES);
      bwd_load_tile<C>(sm.res(0), &tmQ, sm.bar(BB_RES_FULL), i0, h, n);
      bwd_load_tile<C>(sm.res(1), &tmdO, sm.bar(BB_RES_FULL), i0, h, n);
      for (int t = 0; t < nk; ++t) {
        const int slot = t % C::NSLOT;
        const uint32_t par = ((t / C::NSLOT) & 1) ^ 1;
        // a slot's V half is released by dP (early), its K half by dQ (late): K first for the first
        // tiles (their score product is what the CTA waits for), V first once the ring has wrapped
        if (t < C::NSLOT) {
          mbar_arrive_expect_tx(sm.bar(BB_RING_FULL + slot), C::TILE_BYTES);
          bwd_load_tile<C>(sm.slot(slot, 0), &tmK, sm.bar(BB_RING_FULL + slot), t * 128, kvh, n);
          mbar_arrive_expect_tx(sm.bar(BB_RING2_FULL + slot), C::TILE_BYTES);
          bwd_load_tile<C>(sm.slot(slot, 1), &tmV, sm.bar(BB_RING2_FULL + slot), t * 128, kvh, n);
        } else {
          FLB_BWAIT(sm, BB_RING2_EMPTY + slot, par);
          mbar_arrive_expect_tx(sm.bar(BB_RING2_FULL + slot), C::TILE_BYTES);
          bwd_load_tile<C>(sm.slot(slot, 1), &tmV, sm.bar(BB_RING2_FULL + slot), t * 128, kvh, n);
          FLB_BWAIT(sm, BB_RING_EMPTY + slot, par);
          mbar_arrive_expect_tx(sm.bar(BB_RING_FULL + slot), C::TILE_BYTES);
          bwd_load_tile<C>(sm.slot(slot, 0), &tmK, sm.bar(BB_RING_FULL + slot), t * 128, kvh, n);
        }
      }
    }
  };
  if (warp < 8) pointwise();
  else if (warp == 8) { issue(); __syncwarp(); }
  else if (warp == 9 && lane == 0) produce();
  bwd_exit<C>(sm, p, warp);
}

// ------------------------------------------------------------------------------------------
// dK, dV
// ------------------------------------------------------------------------------------------
template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                    const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                    const __grid_constant__ BwdParams p) {
  using C = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  BwdSmem<C> sm{reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023))};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.L + 127) / 128;
  // consecutive CTAs take the key tiles of one (batch, kv head), first (heaviest under the causal mask)
  // first: the CTAs in flight then stream the same few heads' Q and dO, which stay in L2
  const int nkt = (p.S + 127) / 128;
  const int kt = static_cast<int>(blockIdx.x) % nkt;
  const int nh = static_cast<int>(blockIdx.x) / nkt;
  const int n = nh / p.Hkv, kvh = nh % p.Hkv;
  const int j0 = kt * 128;
  const int q_lo = CAUSAL ? min(nq, j0 / 128) : 0;   // first query tile with a row i >= j0
  const int per_head = nq - q_lo;
  const int steps = per_head * p.G;                  // (query head of the group, query tile) pairs
  // the resident A operand of the extra k-step: rows [1, 1, 0 x 6 | 1, 1, 0 x 6] (both 16-byte chunks
  // alike, so the 32-byte swizzle leaves the tile as written); against a row [hi, lo, 0 x 14] it adds hi + lo
  if (threadIdx.x < 128) {
    uint4* r = reinterpret_cast<uint4*>(sm.ones() + threadIdx.x * 32);
    r[0] = make_uint4(0x3F803F80u, 0, 0, 0);
    r[1] = make_uint4(0x3F803F80u, 0, 0, 0);
    fence_proxy_async_smem();
  }
  bwd_setup<C>(sm, p, warp, lane);
  const uint32_t tmem = *sm.tmem_base();
  const uint32_t tS = tmem, tdP = tmem + 128, tdV = tmem + 256, tdK = tmem + 256 + D;

  // Per step the pointwise pass has two halves with a product hanging on each, so that the tensor pipe
  // works under both:  P^T written -> dV += P^T dO, then S^T of the next step;
  //                    dS^T written -> dK += dS^T Q, then dP^T of the next step.
  auto pointwise = [&]() {
    // thread (row, half) owns the key row's columns (queries) [64 half, 64 half + 64)
    const int row = threadIdx.x & 127, half = threadIdx.x >> 7;
    const int j = j0 + row;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tSh = tS + lane_off + half * 64, tdPh = tdP + lane_off + half * 64;
    const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
    for (int t = 0; t < steps; ++t) {
      FLB_BWAIT(sm, BB_SP_FULL, t & 1);
      tc_fence_after();
      const int i0 = (q_lo + t % per_head) * 128 + half * 64;   // first query of the thread's columns
      const bool partial = CAUSAL && j0 + 127 > i0;
      float2 pr[32];
      {
        uint32_t sv[64];
        tmem_ld32_pair_sync(tSh, sv, tSh + 32, sv + 32);
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          // the score columns arrive as s - lse / scale
          const float2 x = __fmul2_rn(make_float2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2);
          float2 e = bwd_exp2_pair(x, c >> 1);
          if (partial) {
            if (j > i0 + c) e.x = 0.f;   // key after the query
            if (j > i0 + c + 1) e.y = 0.f;
          }
          pr[c >> 1] = e;
        }
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) pk[c >> 1] = pack_bf16(pr[(c0 + c) >> 1].x, pr[(c0 + c) >> 1].y);
          tmem_st16(tSh + (c0 >> 1), pk);              // P^T (bf16) over the thread's own columns of S^T
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(sm.bar(BB_P_FULL));
      FLB_BWAIT(sm, BB_DP_FULL, t & 1);
      tc_fence_after();
      {
        uint32_t dp[64];
        tmem_ld32_pair_sync(tdPh, dp, tdPh + 32, dp + 32);
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            // the dP columns arrive as dP - delta
            const float2 g = __fmul2_rn(pr[(c0 + c) >> 1],
                                        make_float2(__uint_as_float(dp[c0 + c]), __uint_as_float(dp[c0 + c + 1])));
            pk[c >> 1] = pack_bf16(g.x, g.y);
          }
          tmem_st16(tdPh + (c0 >> 1), pk);             // dS^T over the thread's own columns of dP^T
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(sm.bar(BB_DS_FULL));
    }
    // epilogue: dV and dK tiles -> bf16 -> shared memory (the K and V tiles are dead) -> TMA stores
    if (steps > 0) {
      FLB_BWAIT(sm, BB_ACC_DONE, 0);
      tc_fence_after();
      if (half == 0) bwd_stage_rows<C, D>(tdV + lane_off, sm.res(1), row, 0, 1.0f);
      else bwd_stage_rows<C, D>(tdK + lane_off, sm.res(0), row, 0, p.scale);
    } else {
      // a key tile no query sees (causal with S > L): zeros
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int c = 0; c < C::TILE_BYTES / 128 / 16; ++c)
        reinterpret_cast<uint4*>(sm.res(half) + row * (C::TILE_BYTES / 128))[c] = z;
    }
    fence_proxy_async_smem();
    named_bar_sync(2, kBwdPointwiseThreads);
    if (threadIdx.x == 0) {
#pragma unroll
      for (int b = 0; b < C::NB; ++b) {
        tma_store_4d(&tmdK, smem_u32(sm.res(0)) + b * C::BOX_BYTES, b * 64, j0, kvh, n);
        tma_store_4d(&tmdV, smem_u32(sm.res(1)) + b * C::BOX_BYTES, b * 64, j0, kvh, n);
      }
      tma_store_commit();
      tma_store_wait_read();
    }
  };
  auto issue = [&]() {
    const uint32_t leader = elect_one() ? 1u : 0u;
    if (steps > 0) {
      FLB_BWAIT(sm, BB_RES_FULL, 0);
      FLB_BWAIT(sm, BB_RING_FULL + 0, 0);
      tc_fence_after();
      bwd_mma_scores<C>(leader, tS, sm.res(0), sm.slot(0, 0));          // S^T(0) = K Q^T
      bwd_mma_aug<C>(leader, tS, sm.ones(), sm.aug(0, 0));              //   - lse / scale per column
      umma_commit_c(leader, sm.bar(BB_SP_FULL));
      FLB_BWAIT(sm, BB_RING2_FULL + 0, 0);
      tc_fence_after();
      bwd_mma_scores<C>(leader, tdP, sm.res(1), sm.slot(0, 1));         // dP^T(0) = V dO^T
      bwd_mma_aug<C>(leader, tdP, sm.ones(), sm.aug(0, 1));             //   - delta per column
      umma_commit_c(leader, sm.bar(BB_DP_FULL));
      for (int t = 0; t < steps; ++t) {
        const int slot = t % C::NSLOT, s1 = (t + 1) % C::NSLOT;
        const uint32_t par1 = ((t + 1) / C::NSLOT) & 1;
        FLB_BWAIT(sm, BB_P_FULL, t & 1);
        tc_fence_after();
        bwd_mma_acc<C>(leader, tdV, tS, sm.slot(slot, 1), t > 0);       // dV += P^T dO
        umma_commit_c(leader, sm.bar(BB_RING2_EMPTY + slot));
        if (t + 1 < steps) {
          FLB_BWAIT(sm, BB_RING_FULL + s1, par1);
          tc_fence_after();
          bwd_mma_scores<C>(leader, tS, sm.res(0), sm.slot(s1, 0));     // S^T(t+1), after dV has read P^T(t)
          bwd_mma_aug<C>(leader, tS, sm.ones(), sm.aug(s1, 0));
          umma_commit_c(leader, sm.bar(BB_SP_FULL));
        }
        FLB_BWAIT(sm, BB_DS_FULL, t & 1);
        tc_fence_after();
        bwd_mma_acc<C>(leader, tdK, tdP, sm.slot(slot, 0), t > 0);      // dK += dS^T Q
        umma_commit_c(leader, sm.bar(BB_RING_EMPTY + slot));
        if (t + 1 < steps) {
          FLB_BWAIT(sm, BB_RING2_FULL + s1, par1);
          tc_fence_after();
          bwd_mma_scores<C>(leader, tdP, sm.res(1), sm.slot(s1, 1));    // dP^T(t+1), after dK has read dS^T(t)
          bwd_mma_aug<C>(leader, tdP, sm.ones(), sm.aug(s1, 1));
          umma_commit_c(leader, sm.bar(BB_DP_FULL));
        }
      }
      umma_commit_c(leader, sm.bar(BB_ACC_DONE));
    }
  };
  // a step's Q tile travels with its x rows, its dO tile with its y rows
  auto load_q = [&](int slot, int i0, int h) {
    mbar_arrive_expect_tx(sm.bar(BB_RING_FULL + slot), C::TILE_BYTES + C::AUG_TILE_BYTES);
    bwd_load_tile<C>(sm.slot(slot, 0), &tmQ, sm.bar(BB_RING_FULL + slot), i0, h, n);
    tma_load_4d(smem_u32(sm.aug(slot, 0)), &tmX, sm.bar(BB_RING_FULL + slot), 0, i0, h, n);
  };
  auto load_do = [&](int slot, int i0, int h) {
    mbar_arrive_expect_tx(sm.bar(BB_RING2_FULL + slot), C::TILE_BYTES + C::AUG_TILE_BYTES);
    bwd_load_tile<C>(sm.slot(slot, 1), &tmdO, sm.bar(BB_RING2_FULL + slot), i0, h, n);
    tma_load_4d(smem_u32(sm.aug(slot, 1)), &tmY, sm.bar(BB_RING2_FULL + slot), 0, i0, h, n);
  };
  auto produce = [&]() {
    if (p.withhold_loads) return;
    if (steps > 0) {
      mbar_arrive_expect_tx(sm.bar(BB_RES_FULL), 2 * C::TILE_BYTES);
      bwd_load_tile<C>(sm.res(0), &tmK, sm.bar(BB_RES_FULL), j0, kvh, n);
      bwd_load_tile<C>(sm.res(1), &tmV, sm.bar(BB_RES_FULL), j0, kvh, n);
      for (int t = 0; t < steps; ++t) {
        const int slot = t % C::NSLOT;
        const uint32_t par = ((t / C::NSLOT) & 1) ^ 1;
        const int h = kvh * p.G + t / per_head, i0 = (q_lo + t % per_head) * 128;
        // a slot's dO half is released by dV (early), its Q half by dK (late)
        if (t < C::NSLOT) {
          load_q(slot, i0, h);
          load_do(slot, i0, h);
        } else {
          FLB_BWAIT(sm, BB_RING2_EMPTY + slot, par);
          load_do(slot, i0, h);
          FLB_BWAIT(sm, BB_RING_EMPTY + slot, par);
          load_q(slot, i0, h);
        }
      }
    }
  };
  if (warp < 8) pointwise();
  else if (warp == 8) { issue(); __syncwarp(); }
  else if (warp == 9 && lane == 0) produce();
  bwd_exit<C>(sm, p, warp);
}

}  // namespace flb
