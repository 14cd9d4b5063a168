// C ABI of the library: validation, tensor-map encoding, kernel dispatch.
// Host logic only; the kernels live in attn_fwd_sm100.cuh / block_map.cuh.
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <mutex>

#include "../../include/flb200_attn.h"
#include "attn_launch.h"
#include "ptx.cuh"
#include "block_map.cuh"
#include "tmap.h"

namespace {
std::atomic<uint64_t> g_launches{0};
}

namespace flb {
void count_launches(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }
}  // namespace flb

namespace {

using namespace flb;


// Scratch for flb200_attn_fwd_noalloc: lives in the library image of every device that loads it.
// In host code `g_noalloc_scratch` is only a stand-in for the symbol; the device address comes
// from cudaGetSymbolAddress (see noalloc_scratch_ptr) and that is what kernels receive.
static __device__ __align__(256) unsigned char g_noalloc_scratch[FLB200_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
void* g_noalloc_ptr[kMaxDevices] = {};

// Device address of the static scratch on the current device; looked up once per device.
void* noalloc_scratch_ptr() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess) return nullptr;
    g_noalloc_ptr[dev] = ptr;
  }
  return g_noalloc_ptr[dev];
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool mult8(int64_t s) { return s % 8 == 0; }

struct MapLayout {
  int nq, nkv;
  // byte offsets of the sections inside the workspace, each 256-byte aligned
  size_t range_bytes, cls_bytes, sorted_off, runs_off, total;
};

MapLayout map_layout(const flb200_attn_params* p) {
  MapLayout m;
  m.nq = (p->L + kTileM - 1) / kTileM;
  m.nkv = (p->S + kTileN - 1) / kTileN;
  m.range_bytes = static_cast<size_t>(p->N) * m.nq * 2 * sizeof(int32_t);
  m.range_bytes = (m.range_bytes + 255) & ~static_cast<size_t>(255);
  m.cls_bytes = static_cast<size_t>(p->N) * m.nq * m.nkv;
  m.sorted_off = m.range_bytes + ((m.cls_bytes + 255) & ~static_cast<size_t>(255));
  const size_t sorted_bytes = (static_cast<size_t>(p->N) * sizeof(int32_t) + 255) & ~static_cast<size_t>(255);
  m.runs_off = m.sorted_off + sorted_bytes;
  const size_t runs_bytes = static_cast<size_t>(p->N) * p->L * 2 * sizeof(int32_t);
  m.total = m.runs_off + ((runs_bytes + 255) & ~static_cast<size_t>(255));
  return m;
}

// Head dims a kernel is built for.  Narrower heads run on the next wider kernel: the tensor maps
// carry the true widths, so the loads fill the missing feature columns with zeros (they add nothing
// to q.k, and the value columns beyond Ev are clipped by the output store).
bool kernel_built(int D, int score, int mask) {
  if (score == SCORE_BIAS_RES) return mask == MASK_NONE && (D == 32 || D == 64);
  if (score == SCORE_B2B || score == SCORE_B2BT)
    return mask == MASK_NONE && (D == 32 || D == 64 || D == 128 || D == 256);
  // heads above 128 (up to 256): plain and causal attention and the product chain, one stage per CTA
  if (D == 256) return score == SCORE_NONE && (mask == MASK_NONE || mask == MASK_CAUSAL);
  if (D == 32)
    return (score == SCORE_NONE && (mask == MASK_NONE || mask == MASK_CAUSAL)) ||
           (score == SCORE_BIAS && mask == MASK_NONE);
  if (D != 64 && D != 128) return false;
  switch (score) {
    case SCORE_NONE:
      return true;
    case SCORE_ALIBI:
    case SCORE_SOFTCAP:
      return mask == MASK_NONE || mask == MASK_CAUSAL;
    case SCORE_BIAS:
      return mask == MASK_NONE;
  }
  return false;
}

// Width of the kernel that serves (E, Ev): plain variants use one width for q/k and v; the
// differential kernels come as (q/k width, v width) = (32, 64), (64, 128) and (128, 128 per CTA of
// a pair), returned as the q/k width.  0 = no kernel.
int kernel_width(int E, int EV, int score, int mask, int diff) {
  if (diff) {
    if (score != SCORE_NONE || (mask != MASK_NONE && mask != MASK_CAUSAL)) return 0;
    if (E <= 32 && EV <= 64) return 32;
    if (E <= 64 && EV <= 128) return 64;
    // q/k heads up to 128 with value heads up to 256: two CTAs per work item, one half of the value
    // columns each (two accumulators of 256 columns and two score tiles exceed tensor memory)
    if (E <= 128 && EV <= 256) return 128;
    return 0;
  }
  const int need = E > EV ? E : EV;
  for (int D : {32, 64, 128, 256})
    if (D >= need && kernel_built(D, score, mask)) return D;
  return 0;
}

// kernel-internal score mode of a problem (the product chain has modes of its own)
int kernel_score(const flb200_attn_params* p) {
  if (p->product_chain) return p->k_keys_contiguous ? SCORE_B2BT : SCORE_B2B;
  return p->score_mod;
}

int validate(const flb200_attn_params* p) {
  if (!p) return FLB200_E_BAD_ARG;
  if (p->struct_size != sizeof(flb200_attn_params)) return FLB200_E_BAD_ARG;
  if (p->N <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->L <= 0 || p->S <= 0 || p->E <= 0 || p->Ev <= 0)
    return FLB200_E_BAD_ARG;
  if (!p->q || !p->k || !p->v || !p->o) return FLB200_E_BAD_ARG;
  if (p->score_mod < FLB200_SCORE_NONE || p->score_mod > FLB200_SCORE_BIAS) return FLB200_E_BAD_ARG;
  if (p->mask < FLB200_MASK_NONE || p->mask > FLB200_MASK_DOCUMENT) return FLB200_E_BAD_ARG;
  if (!(p->scale > 0.f) || !std::isfinite(p->scale)) return FLB200_E_BAD_ARG;
  if (p->Hq % p->Hkv != 0) return FLB200_E_BAD_ARG;
  if (p->lse) {
    if (p->diff) return FLB200_E_UNSUPPORTED;  // two softmaxes per output head: no single log-sum-exp
    if (reinterpret_cast<uintptr_t>(p->lse) & 3u) return FLB200_E_MISALIGNED;
    // rows of L floats that do not overlap
    if ((p->Hq > 1 && p->lse_stride[1] < p->L) || (p->N > 1 && p->lse_stride[0] < p->L))
      return FLB200_E_BAD_ARG;
    if (p->lse_stride[0] < 0 || p->lse_stride[1] < 0) return FLB200_E_BAD_ARG;
  }
  if (p->diff) {
    if (p->Hq != p->Hkv || p->Hq % 2 != 0) return FLB200_E_BAD_ARG;
    if (!std::isfinite(p->diff_lambda)) return FLB200_E_BAD_ARG;
    if (p->diff_rms_norm && !(p->diff_rms_eps >= 0.f)) return FLB200_E_BAD_ARG;
  }
  if (p->score_mod == FLB200_SCORE_ALIBI && (p->alibi_heads <= 0 || p->alibi_head0 < 0))
    return FLB200_E_BAD_ARG;
  if (p->score_mod == FLB200_SCORE_SOFTCAP && !(p->softcap > 0.f && std::isfinite(p->softcap)))
    return FLB200_E_BAD_ARG;
  if (p->score_mod == FLB200_SCORE_BIAS) {
    if (!p->bias[0] && !p->bias[1]) return FLB200_E_BAD_ARG;
    if (p->bias_inner <= 0 || p->N % p->bias_inner != 0) return FLB200_E_BAD_ARG;
  }
  if (p->mask == FLB200_MASK_SLIDING && p->window < 0) return FLB200_E_BAD_ARG;
  if (p->mask == FLB200_MASK_PREFIX && !p->prefix_len && p->prefix_scalar < 0)
    return FLB200_E_BAD_ARG;
  if (p->mask == FLB200_MASK_DOCUMENT) {
    if (!p->document_id) return FLB200_E_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(p->document_id) & 7u) return FLB200_E_MISALIGNED;
    // one row of L ids per sequence, or one shared row (stride 0)
    if (p->N > 1 && p->doc_stride_n != 0 && p->doc_stride_n < p->L) return FLB200_E_BAD_ARG;
    if (p->N > 65535) return FLB200_E_UNSUPPORTED;  // the map builder puts the batch on gridDim.y
  }
  // these masks are defined on square score matrices (sliding_window.py:27, prefix_lm.py:37-38,
  // document_mask.py:25-27 index keys and queries with the same ids)
  if ((p->mask == FLB200_MASK_SLIDING || p->mask == FLB200_MASK_PREFIX ||
       p->mask == FLB200_MASK_DOCUMENT) &&
      p->L != p->S)
    return FLB200_E_BAD_ARG;

  if (p->product_chain) {
    if (p->score_mod != FLB200_SCORE_NONE || p->mask != FLB200_MASK_NONE || p->diff || p->lse)
      return FLB200_E_BAD_ARG;
    if (p->pointwise < FLB200_PW_IDENTITY || p->pointwise > FLB200_PW_SIGMOID) return FLB200_E_BAD_ARG;
  } else if (p->k_keys_contiguous) {
    return FLB200_E_UNSUPPORTED;  // only the product chain reads K with the keys contiguous
  }
  if (!kernel_width(p->E, p->Ev, kernel_score(p), p->mask, p->diff)) return FLB200_E_UNSUPPORTED;
  if (p->L > (1 << 24) || p->S > (1 << 24)) return FLB200_E_UNSUPPORTED;
  {
    const int H = p->diff ? p->Hq / 2 : p->Hq;
    const int rows = p->diff ? kTileM : 2 * kTileM;
    const int64_t ctas = static_cast<int64_t>((p->L + rows - 1) / rows) * p->N * H * (p->diff ? 2 : 1);
    if (ctas > 0x7fffffffLL) return FLB200_E_UNSUPPORTED;
  }

  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->o))
    return FLB200_E_MISALIGNED;
  for (int i = 0; i < 3; ++i) {
    if (p->q_stride[i] < 0 || p->k_stride[i] < 0 || p->v_stride[i] < 0 || p->o_stride[i] < 0)
      return FLB200_E_BAD_ARG;
    if (!mult8(p->q_stride[i]) || !mult8(p->k_stride[i]) || !mult8(p->v_stride[i]) ||
        !mult8(p->o_stride[i]))
      return FLB200_E_MISALIGNED;
  }
  if (p->q_stride[2] < p->E || p->k_stride[2] < (p->k_keys_contiguous ? p->S : p->E) ||
      p->v_stride[2] < p->Ev || p->o_stride[2] < p->Ev)
    return FLB200_E_BAD_ARG;
  if (p->score_mod == FLB200_SCORE_BIAS) {
    for (int b = 0; b < 2; ++b) {
      if (!p->bias[b]) continue;
      if (reinterpret_cast<uintptr_t>(p->bias[b]) & 1u) return FLB200_E_MISALIGNED;
      for (int i = 0; i < 4; ++i)
        if (p->bias_stride[b][i] < 0) return FLB200_E_BAD_ARG;
    }
  }
  if (p->mask == FLB200_MASK_DOCUMENT) {
    if (!p->workspace || p->workspace_bytes < map_layout(p).total) return FLB200_E_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(p->workspace) & 255u) return FLB200_E_MISALIGNED;
  }
  return FLB200_OK;
}

// Query tiles per CTA (see AttnCfg::STAGES).  Two stages share every K/V tile: half the traffic from
// L2 to shared memory, which decides for heads of 128 on long rows of keys (no mask, causal, ALiBi,
// prefix-LM beyond about a thousand keys).  One stage per CTA, two CTAs per SM, lets one CTA's
// set-up, epilogue and waits hide behind the other's tiles; measured on the reference's grids it
// wins for every head width up to 64 (8-20 %), and at width 128 for short rows of keys, sliding
// windows, document masks, the softcap (whose tiles are long) and additive biases.
// FLB200_STAGES=1|2 overrides the choice for tuning.
int pick_stages(const flb200_attn_params* p) {
  if (p->E > 128 || p->Ev > 128) return p->diff ? 2 : 1;  // wide heads have one-stage kernels only
  if (p->diff || p->product_chain) return 2;
  if (const char* e = std::getenv("FLB200_STAGES")) {
    const int v = std::atoi(e);
    if (v == 1 || v == 2) return v;
  }
  if (p->E <= 64 && p->Ev <= 64) return 1;
  if (p->mask == FLB200_MASK_DOCUMENT || p->mask == FLB200_MASK_SLIDING ||
      p->score_mod == FLB200_SCORE_BIAS || p->score_mod == FLB200_SCORE_SOFTCAP)
    return 1;
  const long long ctas2 = static_cast<long long>((p->L + 2 * kTileM - 1) / (2 * kTileM)) * p->N * p->Hq;
  if (ctas2 < 2 * 148) return 1;  // too few two-stage CTAs to give every SM two waves
  if (p->mask == FLB200_MASK_NONE && p->score_mod == FLB200_SCORE_NONE) return p->S <= 512 ? 1 : 2;
  return p->S <= 1024 ? 1 : 2;
}

// Additive biases of the Evoformer kind: one "pair" bias that every row of a batch element shares
// (row stride 0) and at most one key vector per row (query stride 0).  Such a problem runs on the
// resident-bias kernel: a CTA keeps the pair-bias columns of its (head, query tile) in shared
// memory and walks a range of rows.  FLB200_BIAS_RESIDENT=0 turns the choice off for tuning.
// differential attention whose P.V product can run in fp16: RMS-normalised (the result does not depend on
// V's scale), one CTA per work item (value heads up to 128)
bool diff_pv_f16_eligible(const flb200_attn_params* p, int width) {
  if (!p->diff || !p->diff_rms_norm || width == 128 || p->Ev > 2 * width) return false;
  if (const char* e = std::getenv("FLB200_DIFF_PV_F16")) return std::atoi(e) != 0;
  return true;
}

struct ResidentPlan {
  bool use = false;
  int pair = -1, rowvec = -1;  // indices into p->bias
  int rows = 0, chunks = 0;    // rows per CTA, CTAs per (batch element, head, query tile)
  int slots = 0;               // K/V ring slots that fit beside the bias tiles
  // the key vector added by the tensor cores (one more k-step per score product): bytes of the rows the
  // pre-kernel writes into the caller's workspace (0: not eligible), and whether this call does it
  size_t keyvec_bytes = 0;
  bool keyvec = false;
};

ResidentPlan plan_resident(const flb200_attn_params* p, int width) {
  ResidentPlan r;
  if (p->score_mod != FLB200_SCORE_BIAS || p->diff || p->product_chain || width > 64) return r;
  if (const char* e = std::getenv("FLB200_BIAS_RESIDENT"))
    if (std::atoi(e) == 0) return r;
  const int R = p->bias_inner;
  if (R < 4) return r;
  for (int q = 0; q < 2; ++q) {
    if (!p->bias[q]) continue;
    const int64_t* st = p->bias_stride[q];  // {b, r, h, i}
    if (st[3] != 0 && st[1] == 0) {
      if (r.pair >= 0) return r;
      r.pair = q;
    } else if (st[3] == 0) {
      if (r.rowvec >= 0) return r;
      r.rowvec = q;
    } else {
      return r;  // a full bias per row: nothing to keep resident
    }
  }
  if (r.pair < 0) return r;
  const int64_t* st = p->bias_stride[r.pair];
  if (!aligned16(p->bias[r.pair]) || !mult8(st[0]) || !mult8(st[2]) || !mult8(st[3]) || st[3] < p->S) return r;
  // shared memory behind the Q tiles and the output staging: 32 KB per bias tile, the rest K/V slots
  // (two rows' tiles each), of which there must be at least two
  const int nt = (p->S + kTileN - 1) / kTileN;
  if (nt > 4) return r;
  const int tile_bytes = kTileM * width * 2;
  const int room = 232448 - 1024 - 2 * tile_bytes - 2 * tile_bytes - 2048 - nt * 32768;
  r.slots = std::min(7, room / (2 * tile_bytes));
  if (room < 0 || r.slots < 2) return r;
  const int H = p->Hq, B = p->N / R;
  const long long base = static_cast<long long>((p->L + kTileM - 1) / kTileM) * B * H;
  int chunks;
  if (base >= 148) chunks = static_cast<int>(std::max(1LL, std::min<long long>(R / 8, (4 * 148) / base)));
  else chunks = static_cast<int>(std::max(1LL, std::min<long long>(R / 2, 148 / base)));
  int rows = (R + chunks - 1) / chunks;
  rows += rows & 1;  // the two stages take the rows in pairs
  r.rows = rows;
  r.chunks = (R + rows - 1) / rows;
  r.use = true;
  // Key vector through the tensor cores: one vector per row (no head axis), and an even number of ring
  // slots per stage (K tiles in the even ones) beside the tile of ones and the slots / 2 tiles of rows per
  // stage that travel with the K tiles (4 KB each).  Even a ring of two slots (heads of 64 with two bias
  // tiles) measured 15 % faster with the vector on the tensor cores than three slots without.  It needs scratch memory from the caller; without it the
  // softmax threads add the vector as before.
  if (r.rowvec >= 0 && p->bias_stride[r.rowvec][2] == 0) {
    int even = std::min(6, r.slots) & ~1;
    while (even >= 2 && 2 * even * tile_bytes + 4096 * (1 + even) > room) even -= 2;
    // (a small problem, under about 6000 tile products, does not pay for the launch that lays the rows out)
    const long long work = static_cast<long long>(p->N) * p->Hq * ((p->L + kTileM - 1) / kTileM) * nt;
    bool on = even >= 2 && work >= 6144;
    if (const char* e = std::getenv("FLB200_KEYVEC_MMA")) on = on && std::atoi(e) != 0;
    if (on) {
      r.keyvec_bytes = static_cast<size_t>(p->N) * nt * 4096;
      if (p->workspace && p->workspace_bytes >= r.keyvec_bytes && aligned16(p->workspace)) {
        r.keyvec = true;
        r.slots = even;
      }
    }
  }
  return r;
}

int check_arch() {
  // cudaSetDevice binds the device's primary context to the calling thread: the tensor-map encoder is a
  // driver call and needs one even in a thread that has made no runtime call yet
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return FLB200_E_LAUNCH;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return FLB200_E_LAUNCH;
  return major == 10 ? FLB200_OK : FLB200_E_ARCH;
}

int build_block_map(const flb200_attn_params* p, cudaStream_t stream) {
  const MapLayout m = map_layout(p);
  auto* range = reinterpret_cast<int32_t*>(p->workspace);
  auto* cls = reinterpret_cast<uint8_t*>(p->workspace) + m.range_bytes;
  dim3 grid(m.nq, p->N);
  auto* sorted = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(p->workspace) + m.sorted_off);
  auto* runs = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(p->workspace) + m.runs_off);
  doc_block_map_kernel<<<grid, 128, 0, stream>>>(
      reinterpret_cast<const long long*>(p->document_id), p->doc_stride_n, p->L, p->causal, range,
      cls, sorted);
  dim3 grid2((p->L + 255) / 256, p->N);
  doc_runs_kernel<<<grid2, 256, 0, stream>>>(reinterpret_cast<const long long*>(p->document_id),
                                             p->doc_stride_n, p->L, sorted, runs);
  if (cudaGetLastError() != cudaSuccess) return FLB200_E_LAUNCH;
  g_launches.fetch_add(2, std::memory_order_relaxed);
  return FLB200_OK;
}

template <int E, int EV, int DIFF, int STAGES>
cudaError_t dispatch_mods(int score, int mask, const CUtensorMap& a, const CUtensorMap& b,
                          const CUtensorMap& c, const CUtensorMap& o, const KernelParams& kp,
                          int grid, int cluster, cudaStream_t st) {
#define FLB_CASE(SC, MK)          \
  if (score == SC && mask == MK)  \
    return launch_attn<E, EV, SC, MK, DIFF, STAGES>(a, b, c, o, a, kp, grid, cluster, st);
  if constexpr (DIFF != 0) {
    FLB_CASE(SCORE_NONE, MASK_NONE)
    FLB_CASE(SCORE_NONE, MASK_CAUSAL)
  } else if constexpr (E == 256) {
    FLB_CASE(SCORE_NONE, MASK_NONE)
    FLB_CASE(SCORE_NONE, MASK_CAUSAL)
    FLB_CASE(SCORE_B2B, MASK_NONE)
    FLB_CASE(SCORE_B2BT, MASK_NONE)
  } else if constexpr (E == 32) {
    FLB_CASE(SCORE_NONE, MASK_NONE)
    FLB_CASE(SCORE_NONE, MASK_CAUSAL)
    FLB_CASE(SCORE_BIAS, MASK_NONE)
    if constexpr (STAGES == 2) {
      FLB_CASE(SCORE_B2B, MASK_NONE)
      FLB_CASE(SCORE_B2BT, MASK_NONE)
    }
  } else {
    FLB_CASE(SCORE_NONE, MASK_NONE)
    FLB_CASE(SCORE_NONE, MASK_CAUSAL)
    FLB_CASE(SCORE_ALIBI, MASK_NONE)
    FLB_CASE(SCORE_ALIBI, MASK_CAUSAL)
    FLB_CASE(SCORE_SOFTCAP, MASK_NONE)
    FLB_CASE(SCORE_SOFTCAP, MASK_CAUSAL)
    FLB_CASE(SCORE_NONE, MASK_SLIDING)
    FLB_CASE(SCORE_NONE, MASK_PREFIX)
    FLB_CASE(SCORE_NONE, MASK_DOCUMENT)
    FLB_CASE(SCORE_BIAS, MASK_NONE)
    if constexpr (STAGES == 2) {
      FLB_CASE(SCORE_B2B, MASK_NONE)
      FLB_CASE(SCORE_B2BT, MASK_NONE)
    }
  }
#undef FLB_CASE
  return cudaErrorInvalidValue;
}

}  // namespace

extern "C" {

uint32_t flb200_abi_version(void) { return FLB200_ABI_VERSION; }

const char* flb200_strerror(int status) {
  switch (status) {
    case FLB200_OK: return "ok";
    case FLB200_E_BAD_ARG: return "bad argument (null pointer, non-positive size, bad enum or struct_size)";
    case FLB200_E_UNSUPPORTED: return "unsupported shape or variant combination (no kernel built, no fallback)";
    case FLB200_E_MISALIGNED: return "misaligned pointer or stride (16 bytes / 8 elements required)";
    case FLB200_E_WORKSPACE: return "workspace missing or too small";
    case FLB200_E_ARCH: return "device is not sm_100";
    case FLB200_E_LAUNCH: return "CUDA error while encoding descriptors or launching";
    case FLB200_E_TIMEOUT: return "a device-side wait expired";
    default: return "unknown status";
  }
}

int flb200_attn_validate(const flb200_attn_params* p) { return validate(p); }

size_t flb200_attn_workspace_bytes(const flb200_attn_params* p) {
  if (!p || p->struct_size != sizeof(flb200_attn_params)) return 0;
  if (p->N <= 0 || p->L <= 0 || p->S <= 0) return 0;
  if (p->score_mod == FLB200_SCORE_BIAS && p->mask == FLB200_MASK_NONE && validate(p) == FLB200_OK) {
    // optional scratch of the resident pair-bias kernel (the call also runs without it)
    const int width = kernel_width(p->E, p->Ev, kernel_score(p), p->mask, p->diff);
    return width ? plan_resident(p, width).keyvec_bytes : 0;
  }
  if (p->diff && p->mask != FLB200_MASK_DOCUMENT && validate(p) == FLB200_OK) {
    // optional scratch of the fp16 P.V path of differential attention (one word: max |v|)
    const int width = kernel_width(p->E, p->Ev, kernel_score(p), p->mask, p->diff);
    return width && diff_pv_f16_eligible(p, width) ? 256 : 0;
  }
  if (p->mask != FLB200_MASK_DOCUMENT) return 0;
  return map_layout(p).total;
}

int flb200_build_block_map(const flb200_attn_params* p, void* cuda_stream) {
  const int v = validate(p);
  if (v != FLB200_OK) return v;
  if (p->mask != FLB200_MASK_DOCUMENT) return FLB200_E_BAD_ARG;
  const int a = check_arch();
  if (a != FLB200_OK) return a;
  return build_block_map(p, static_cast<cudaStream_t>(cuda_stream));
}

namespace {
int attn_fwd_impl(const flb200_attn_params* p, void* cuda_stream, bool withhold_loads);
}

int flb200_attn_fwd(const flb200_attn_params* p, void* cuda_stream) {
  return attn_fwd_impl(p, cuda_stream, false);
}

int flb200_selftest_wait_timeout(const flb200_attn_params* p, void* cuda_stream) {
  if (!p || p->struct_size != sizeof(flb200_attn_params)) return FLB200_E_BAD_ARG;
  if (!p->status) return FLB200_E_BAD_ARG;
  flb200_attn_params q = *p;
  if (q.wait_limit_us == 0) q.wait_limit_us = 1000;
  return attn_fwd_impl(&q, cuda_stream, true);
}

namespace {
int attn_fwd_impl(const flb200_attn_params* p, void* cuda_stream, bool withhold_loads) {
  const int v = validate(p);
  if (v != FLB200_OK) return v;
  const int a = check_arch();
  if (a != FLB200_OK) return a;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

  KernelParams kp;
  std::memset(&kp, 0, sizeof(kp));
  const int H = p->diff ? p->Hq / 2 : p->Hq;
  kp.N = p->N;
  kp.H = H;
  kp.L = p->L;
  kp.S = p->S;
  kp.G = p->diff ? 1 : p->Hq / p->Hkv;
  kp.diff_heads = p->diff ? H : 0;
  kp.evo_inner = p->score_mod == FLB200_SCORE_BIAS ? p->bias_inner : 1;
  kp.o = p->o;
  kp.o_sn = p->o_stride[0];
  kp.o_sh = p->o_stride[1];
  kp.o_sl = p->o_stride[2];
  kp.scale = p->scale;
  kp.scale_log2 = p->scale * 1.4426950408889634f;
  kp.alibi_log2_slope_step = p->score_mod == FLB200_SCORE_ALIBI ? -8.0f / p->alibi_heads : 0.f;
  kp.alibi_head0 = p->alibi_head0;
  kp.softcap = p->softcap;
  kp.pointwise = p->pointwise;
  kp.lse = p->lse;
  kp.lse_sn = p->lse_stride[0];
  kp.lse_sh = p->lse_stride[1];
  for (int b = 0; b < 2; ++b) {
    kp.bias[b] = p->score_mod == FLB200_SCORE_BIAS ? p->bias[b] : nullptr;
    kp.bias_sb[b] = p->bias_stride[b][0];
    kp.bias_sr[b] = p->bias_stride[b][1];
    kp.bias_sh[b] = p->bias_stride[b][2];
    kp.bias_sl[b] = p->bias_stride[b][3];
    // rows that start on 16-byte boundaries are read with 128-bit loads, others element-wise
    kp.bias_vec[b] = aligned16(p->bias[b]) && mult8(p->bias_stride[b][0]) &&
                     mult8(p->bias_stride[b][1]) && mult8(p->bias_stride[b][2]) &&
                     mult8(p->bias_stride[b][3]);
  }
  kp.causal = p->causal;
  kp.window = p->window;
  kp.prefix_len = p->prefix_len;
  kp.prefix_scalar = p->prefix_scalar;
  kp.doc = reinterpret_cast<const int64_t*>(p->document_id);
  kp.doc_sn = p->doc_stride_n;
  kp.lambda = p->diff_lambda;
  kp.rms_norm = p->diff_rms_norm;
  kp.rms_eps = p->diff_rms_eps;
  kp.status = p->status;
  kp.status_host = p->status_host;
  kp.wait_limit_us = p->wait_limit_us ? p->wait_limit_us : kDefaultWaitLimitUs;
  kp.withhold_loads = withhold_loads ? 1 : 0;
  const int stages = pick_stages(p);
  const int rows_per_cta = (p->diff || stages == 1) ? kTileM : 2 * kTileM;
  kp.nq_blocks = (p->L + rows_per_cta - 1) / rows_per_cta;

  if (p->mask == FLB200_MASK_DOCUMENT) {
    const MapLayout m = map_layout(p);
    kp.map_range = reinterpret_cast<const int32_t*>(p->workspace);
    kp.map_cls = reinterpret_cast<const uint8_t*>(p->workspace) + m.range_bytes;
    kp.map_sorted = reinterpret_cast<const int32_t*>(reinterpret_cast<const uint8_t*>(p->workspace) + m.sorted_off);
    kp.map_runs = reinterpret_cast<const int32_t*>(reinterpret_cast<const uint8_t*>(p->workspace) + m.runs_off);
    if (!p->block_map_ready) {
      const int r = build_block_map(p, stream);
      if (r != FLB200_OK) return r;
    }
  }

  // tensor maps: innermost feature axis, then row, head, batch
  int kscore = kernel_score(p);
  const int width = kernel_width(p->E, p->Ev, kscore, p->mask, p->diff);  // q/k width
  const ResidentPlan res = plan_resident(p, width);
  if (res.use) kscore = SCORE_BIAS_RES;
  // value columns one CTA handles: twice the q/k width for the differential kernels, except the
  // widest, whose CTAs come in pairs that split value heads above 128
  const int vwidth = p->diff ? (width == 128 ? 128 : 2 * width) : width;
  kp.v_halves = (p->diff && width == 128 && p->Ev > 128) ? 2 : 1;
  kp.v_exchange = kp.v_halves == 2 && p->diff_rms_norm;
  kp.inv_ev = 1.0f / static_cast<float>(p->Ev);
  const uint32_t kbox = width >= 64 ? 64 : width;
  const uint32_t vbox = vwidth >= 64 ? 64 : vwidth;
  const int Hv = p->diff ? H : p->Hkv;
  CUtensorMap tmQ, tmK, tmV, tmO, tmB;
  if (res.use) {
    const int R = p->bias_inner, B = p->N / R;
    const int64_t* st = p->bias_stride[res.pair];
    kp.pair_h = st[2] != 0;
    kp.pair_b = st[0] != 0;
    kp.res_rows = res.rows;
    kp.res_chunks = res.chunks;
    kp.res_slots = res.slots;
    kp.nq_blocks = (p->L + kTileM - 1) / kTileM;
    // the key vector moves to slot 0 (strides b, r, h); slot 1 is unused by this kernel
    const int rv = res.rowvec;
    kp.bias[0] = rv >= 0 ? p->bias[rv] : nullptr;
    kp.bias_sb[0] = rv >= 0 ? p->bias_stride[rv][0] : 0;
    kp.bias_sr[0] = rv >= 0 ? p->bias_stride[rv][1] : 0;
    kp.bias_sh[0] = rv >= 0 ? p->bias_stride[rv][2] : 0;
    kp.bias_vec[0] = rv >= 0 && aligned16(p->bias[rv]) && mult8(p->bias_stride[rv][0]) &&
                     mult8(p->bias_stride[rv][1]) && mult8(p->bias_stride[rv][2]);
    kp.bias[1] = nullptr;
    if (res.keyvec) {
      const int nt = (p->S + kTileN - 1) / kTileN;
      const int64_t total = static_cast<int64_t>(p->N) * nt * kTileN;
      kp.keyvec_rows = static_cast<const uint8_t*>(p->workspace);
      kp.keyvec_tiles = nt;
      keyvec_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(p->bias[rv]), p->bias_stride[rv][0], p->bias_stride[rv][1], R, p->S,
          nt * kTileN, total, 1.0f / p->scale, reinterpret_cast<uint4*>(p->workspace));
      if (cudaGetLastError() != cudaSuccess) return FLB200_E_LAUNCH;
      flb::count_launches(1);
    }
    // pair bias as (key, query, head, batch element); broadcast axes get extent 1
    const uint64_t dh = kp.pair_h ? p->Hq : 1, db = kp.pair_b ? B : 1;
    const uint64_t sh = kp.pair_h ? st[2] : ((static_cast<uint64_t>(st[3]) * p->L + 7) & ~7ull);
    const uint64_t sb = kp.pair_b ? st[0] : sh * dh;
    if (make_tmap_bf16_4d(&tmB, p->bias[res.pair], p->S, p->L, dh, db, st[3], sh, sb, 64, kTileM))
      return FLB200_E_LAUNCH;
  }
  if (make_tmap_bf16_4d(&tmQ, p->q, p->E, p->L, p->Hq, p->N, p->q_stride[2], p->q_stride[1],
                        p->q_stride[0], kbox, kTileM) ||
      (p->k_keys_contiguous
           // K^T: keys innermost, one box = 64 keys x all feature rows
           ? make_tmap_bf16_4d(&tmK, p->k, p->S, p->E, p->Hkv, p->N, p->k_stride[2], p->k_stride[1],
                               p->k_stride[0], 64, width)
           : make_tmap_bf16_4d(&tmK, p->k, p->E, p->S, p->Hkv, p->N, p->k_stride[2], p->k_stride[1],
                               p->k_stride[0], kbox, kTileN)) ||
      make_tmap_bf16_4d(&tmV, p->v, p->Ev, p->S, Hv, p->N, p->v_stride[2], p->v_stride[1],
                        p->v_stride[0], vbox, kTileN) ||
      make_tmap_bf16_4d(&tmO, p->o, p->Ev, p->L, H, p->N, p->o_stride[2], p->o_stride[1],
                        p->o_stride[0], vbox, kTileM))
    return FLB200_E_LAUNCH;
  if (!res.use) tmB = tmQ;  // unused by every other kernel

  {
    // Sections pay when the K/V of all (batch, head) pairs exceed L2 and every query block reads
    // a long stretch of them (no mask, causal, prefix).  Sliding-window and document masks bound
    // what a block reads, so their working set fits without sections.
    const long long bh_count = static_cast<long long>(p->N) * H;
    kp.sec_bh = static_cast<int>(bh_count);
    const bool long_reach = p->mask == FLB200_MASK_NONE || p->mask == FLB200_MASK_CAUSAL ||
                            p->mask == FLB200_MASK_PREFIX;
    // K/V bytes one (batch, query head) streams, shared by the query heads of a GQA group
    const double kv_bytes = 2.0 * p->S * (p->E * (p->diff ? 2 : 1) + p->Ev) / kp.G;
    double budget = 64.0 * 1024 * 1024;  // about half of the 126 MB L2
    if (const char* e = std::getenv("FLB200_L2_SECTION_MB")) {  // tuning knob
      const double mb = std::atof(e);
      if (mb > 0) budget = mb * 1024 * 1024;
    }
    if (long_reach && kv_bytes * bh_count > budget) {
      long long sec = static_cast<long long>(budget / kv_bytes);
      sec -= sec % kp.G;
      if (sec < kp.G) sec = kp.G;
      if (sec < bh_count) kp.sec_bh = static_cast<int>(sec);
    }
  }
  const int grid = res.use ? kp.nq_blocks * (p->N / p->bias_inner) * H * res.chunks
                           : kp.nq_blocks * p->N * H * kp.v_halves;
  const int cluster = kp.v_exchange ? 2 : 1;
  cudaError_t e = cudaErrorInvalidValue;
  const int sc = kscore, mk = p->mask;
  if (p->diff) {
    // The RMS normalisation scales the small difference of two softmax averages up to unit size, and
    // the rounding of P with it: P then carries a second bf16 term.  FLB200_DIFF_SPLIT_P=0|1 forces
    // the choice (for measuring what the second term buys).
    bool split = p->diff_rms_norm != 0;
    if (const char* e2 = std::getenv("FLB200_DIFF_SPLIT_P")) split = std::atoi(e2) != 0;
#define FLB_DIFF(E, EV)                                                                                     \
  (split ? dispatch_mods<E, EV, 2, 2>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream)               \
         : dispatch_mods<E, EV, 1, 2>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream))
    // With the RMS normalisation and scratch from the caller, P.V runs in fp16 (one term of 11 mantissa bits
    // against V rewritten as fp16 in shared memory) instead of two bf16 terms: 12 k-steps a tile for 20.
    bool pv_f16 = diff_pv_f16_eligible(p, width) && split && p->workspace && p->workspace_bytes >= 16 &&
                  aligned16(p->workspace);
    if (pv_f16) {
      uint32_t* absmax = static_cast<uint32_t*>(p->workspace);
      if (cudaMemsetAsync(absmax, 0, sizeof(uint32_t), stream) != cudaSuccess) return FLB200_E_LAUNCH;
      // about eight waves of blocks over the heads' rows
      const int per_head = std::max(1, std::min((p->S + 63) / 64, (148 * 8 + p->N * H - 1) / (p->N * H)));
      v_absmax_kernel<<<dim3(per_head, p->N * H), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(p->v),
                                                                   p->v_stride[0], p->v_stride[1], p->v_stride[2], H,
                                                                   p->S, p->Ev, absmax);
      if (cudaGetLastError() != cudaSuccess) return FLB200_E_LAUNCH;
      flb::count_launches(1);
      kp.v_absmax = absmax;
    }
    if (pv_f16 && width == 64) e = dispatch_mods<64, 128, 3, 2>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream);
    else if (pv_f16) e = dispatch_mods<32, 64, 3, 2>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream);
    else if (width == 128) e = FLB_DIFF(128, 128);
    else if (width == 64) e = FLB_DIFF(64, 128);
    else e = FLB_DIFF(32, 64);
#undef FLB_DIFF
  } else if (res.use) {
    if (width == 64) e = launch_attn<64, 64, SCORE_BIAS_RES, MASK_NONE, 0, 2>(tmQ, tmK, tmV, tmO, tmB, kp, grid, 1, stream);
    else e = launch_attn<32, 32, SCORE_BIAS_RES, MASK_NONE, 0, 2>(tmQ, tmK, tmV, tmO, tmB, kp, grid, 1, stream);
  } else if (stages == 2) {
    if (width == 128) e = dispatch_mods<128, 128, 0, 2>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream);
    else if (width == 64) e = dispatch_mods<64, 64, 0, 2>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream);
    else e = dispatch_mods<32, 32, 0, 2>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream);
  } else {
    if (width == 256) e = dispatch_mods<256, 256, 0, 1>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream);
    else if (width == 128) e = dispatch_mods<128, 128, 0, 1>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream);
    else if (width == 64) e = dispatch_mods<64, 64, 0, 1>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream);
    else e = dispatch_mods<32, 32, 0, 1>(sc, mk, tmQ, tmK, tmV, tmO, kp, grid, cluster, stream);
  }
  if (e != cudaSuccess) return FLB200_E_LAUNCH;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FLB200_OK;
}
}  // namespace

int flb200_attn_fwd_noalloc(const flb200_attn_params* p, void* cuda_stream) {
  if (!p || p->struct_size != sizeof(flb200_attn_params)) return FLB200_E_BAD_ARG;
  flb200_attn_params q = *p;
  if (q.mask == FLB200_MASK_DOCUMENT) {
    if (q.N <= 0 || q.L <= 0 || q.S <= 0) return FLB200_E_BAD_ARG;
    if (map_layout(&q).total > FLB200_NOALLOC_SCRATCH_BYTES) return FLB200_E_WORKSPACE;
    // argument errors come before anything that needs the device; the workspace fields are
    // stand-ins until the array's address is known
    q.workspace = reinterpret_cast<void*>(static_cast<uintptr_t>(256));
    q.workspace_bytes = FLB200_NOALLOC_SCRATCH_BYTES;
    const int v = validate(&q);
    if (v != FLB200_OK) return v;
    const int a = check_arch();
    if (a != FLB200_OK) return a;
    void* scratch = noalloc_scratch_ptr();
    if (!scratch) return FLB200_E_LAUNCH;
    q.workspace = scratch;
    q.workspace_bytes = FLB200_NOALLOC_SCRATCH_BYTES;
    q.block_map_ready = 0;  // the array holds whatever the previous call left: always rebuild
  } else {
    // the workspace fields are ignored here: the optional-scratch paths (key vector and fp16 P.V through
    // the tensor cores) stay off, whatever the caller left in them
    q.workspace = nullptr;
    q.workspace_bytes = 0;
  }
  return flb200_attn_fwd(&q, cuda_stream);
}

int flb200_decode_status(int32_t status_word, int32_t* barrier, int32_t* block) {
  if (barrier) *barrier = (status_word >> 16) & 0xff;
  if (block) *block = status_word & 0xffff;
  if (status_word == 0) return FLB200_OK;
  return ((status_word >> 24) & 0xff) == kStatusTimeout ? FLB200_E_TIMEOUT : FLB200_E_LAUNCH;
}

uint64_t flb200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
