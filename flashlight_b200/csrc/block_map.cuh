// Block map for the document mask: for every (sequence n, 128-row query tile) the range of
// 128-key tiles that can hold a kept pair, and a class per tile (skip / partial / full).
//
// The classification works for arbitrary (unsorted) document ids: a tile pair is skipped when
// the id intervals [min,max] of its rows and of its keys are disjoint, and it is full when both
// sides carry one and the same id (and, with the causal flag, the tile lies on or below the
// diagonal band of full tiles).  Everything else is masked element-wise by the attention kernel.
#pragma once
#include "attn_params.h"
#include "ptx.cuh"

namespace flb {

__device__ __forceinline__ void warp_minmax(long long& lo, long long& hi) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
}

// grid (nq, N), 128 threads.  doc: [N][L] int64 with row stride doc_sn; L == S.
__global__ void __launch_bounds__(128)
doc_block_map_kernel(const long long* __restrict__ doc, long long doc_sn, int L, int causal,
                     int32_t* __restrict__ map_range, uint8_t* __restrict__ map_cls,
                     int32_t* __restrict__ map_sorted) {
  const int qt = blockIdx.x, n = blockIdx.y;
  const int nq = gridDim.x, nkv = (L + kTileN - 1) / kTileN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long* row = doc + static_cast<long long>(n) * doc_sn;
  __shared__ long long s_lo[4], s_hi[4];
  __shared__ int s_first, s_last;

  const int r0 = qt * kTileM;
  const int rlast = min(r0 + kTileM - 1, L - 1);
  long long qlo = LLONG_MAX, qhi = LLONG_MIN;
  if (r0 + (int)threadIdx.x <= rlast) qlo = qhi = row[r0 + threadIdx.x];
  warp_minmax(qlo, qhi);
  if (lane == 0) {
    s_lo[warp] = qlo;
    s_hi[warp] = qhi;
  }
  if (threadIdx.x == 0) {
    s_first = nkv;
    s_last = -1;
    if (qt == 0) map_sorted[n] = 1;  // doc_runs_kernel (next on the stream) clears it on a descent
  }
  __syncthreads();
  qlo = min(min(s_lo[0], s_lo[1]), min(s_lo[2], s_lo[3]));
  qhi = max(max(s_hi[0], s_hi[1]), max(s_hi[2], s_hi[3]));

  uint8_t* cls = map_cls + (static_cast<long long>(n) * nq + qt) * nkv;
  for (int t = warp; t < nkv; t += 4) {
    const int j0 = t * kTileN;
    long long klo = LLONG_MAX, khi = LLONG_MIN;
    for (int j = j0 + lane; j < min(j0 + kTileN, L); j += 32) {
      const long long d = row[j];
      klo = min(klo, d);
      khi = max(khi, d);
    }
    warp_minmax(klo, khi);
    if (lane == 0) {
      uint8_t c;
      if ((causal && j0 > rlast) || qhi < klo || khi < qlo) {
        c = TILE_SKIP;
      } else if (qlo == qhi && klo == khi && qlo == klo && j0 + kTileN <= L &&
                 (!causal || j0 + kTileN - 1 <= r0)) {
        c = TILE_FULL;
      } else {
        c = TILE_PARTIAL;
      }
      cls[t] = c;
      if (c != TILE_SKIP) {
        atomicMin(&s_first, t);
        atomicMax(&s_last, t);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t* e = map_range + (static_cast<long long>(n) * nq + qt) * 2;
    e[0] = s_last >= 0 ? s_first : 0;
    e[1] = s_last >= 0 ? s_last + 1 : 0;
  }
}

// Packed sequences carry ids that never decrease.  Then "same document" is an index interval per
// row, [first, last] of the run of equal ids around it, and the attention kernel masks a
// partial tile by comparing column indices instead of ids.  This kernel finds the runs by
// bisection (meaningful only for such a sequence) and clears map_sorted[n] if the ids of
// sequence n ever decrease; the attention kernel then compares ids.
// grid (ceil(L / 256), N), 256 threads; runs after doc_block_map_kernel on the same stream.
__global__ void __launch_bounds__(256)
doc_runs_kernel(const long long* __restrict__ doc, long long doc_sn, int L,
                int32_t* __restrict__ map_sorted, int32_t* __restrict__ map_runs) {
  const int n = blockIdx.y;
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= L) return;
  const long long* row = doc + static_cast<long long>(n) * doc_sn;
  const long long id = row[i];
  if (i + 1 < L && row[i + 1] < id) map_sorted[n] = 0;
  int a = 0, b = i;  // first index in [0, i] holding id
  while (a < b) {
    const int mid = (a + b) >> 1;
    if (row[mid] < id) a = mid + 1; else b = mid;
  }
  int c = i, d = L - 1;  // last index in [i, L - 1] holding id
  while (c < d) {
    const int mid = (c + d + 1) >> 1;
    if (row[mid] > id) d = mid - 1; else c = mid;
  }
  int32_t* e = map_runs + (static_cast<long long>(n) * L + i) * 2;
  e[0] = a;
  e[1] = c;
}

// Key-vector rows for the resident-bias kernel: out holds, per (row n, key tile t), the 4 KB shared-memory
// image of a tile of 128 rows of 16 bf16 with 32-byte swizzle (the 16-byte chunk index of row r is
// XORed with bit 2 of r), row j = [hi, lo, 0 ...] of bias[n][j] / scale; keys beyond S: zeros.
__global__ void keyvec_rows_kernel(const __nv_bfloat16* __restrict__ bias, int64_t sb, int64_t sr, int R, int S,
                                   int Sp, int64_t total, float inv_scale, uint4* __restrict__ out) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int j = static_cast<int>(idx % Sp);
  const int64_t n = idx / Sp;
  const int64_t b = n / R, r = n % R;
  const uint32_t word = j < S ? split_bf16_pair(__bfloat162float(bias[b * sb + r * sr + j]) * inv_scale) : 0u;
  const int swap = ((j & 127) >> 2) & 1;
  out[2 * idx + swap] = make_uint4(word, 0, 0, 0);
  out[2 * idx + (swap ^ 1)] = make_uint4(0, 0, 0, 0);
}

// max |v| over a [N][H][S][Ev] bf16 tensor (feature axis contiguous), as the bits of a non-negative float
// (their integer order is the order of the values; a NaN lands above infinity).  blockIdx.y = (n, h);
// sixteen lanes per row, one 16-byte load each (Ev <= 128), the blocks of a head stride over its rows.
__global__ void v_absmax_kernel(const __nv_bfloat16* __restrict__ v, int64_t sn, int64_t sh, int64_t ss, int H, int S,
                                int Ev, uint32_t* __restrict__ out) {
  const int n = blockIdx.y / H, h = blockIdx.y % H;
  const int c = threadIdx.x & 15;
  const unsigned short* base = reinterpret_cast<const unsigned short*>(v + n * sn + h * sh);
  uint32_t m = 0;
  if (c * 8 < Ev) {
    const int step = gridDim.x * 16;
    const bool vec = c * 8 + 8 <= Ev;
    for (int j = blockIdx.x * 16 + (threadIdx.x >> 4); j < S; j += 4 * step) {
      // four rows per trip, their loads in flight together
      uint4 w[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        w[r] = make_uint4(0, 0, 0, 0);
        const int jr = j + r * step;
        if (jr < S) {
          const unsigned short* row = base + static_cast<int64_t>(jr) * ss;
          if (vec) {
            w[r] = *reinterpret_cast<const uint4*>(row + c * 8);   // rows start on 16-byte boundaries
          } else {
            for (int e = c * 8; e < Ev; ++e) m = max(m, (static_cast<uint32_t>(row[e]) << 16) & 0x7fffffffu);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const uint32_t ww[4] = {w[r].x, w[r].y, w[r].z, w[r].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) m = max(m, max((ww[e] << 16) & 0x7fffffffu, ww[e] & 0x7fff0000u));
      }
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, s));
  if ((threadIdx.x & 31) == 0 && m != 0) atomicMax(out, m);
}

}  // namespace flb
