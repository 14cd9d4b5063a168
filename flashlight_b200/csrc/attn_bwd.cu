// C ABI of the backward pass: validation, tensor maps, the three launches.
#include <atomic>
#include <cmath>
#include <cstring>

#include "../../include/flb200_attn.h"
#include "attn_bwd_sm100.cuh"
#include "tmap.h"

namespace flb {
void count_launches(int n);  // capi.cu: the library's launch counter
}

namespace {

using namespace flb;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int validate_bwd(const flb200_attn_bwd_params* p) {
  if (!p || p->struct_size != sizeof(flb200_attn_bwd_params)) return FLB200_E_BAD_ARG;
  if (p->N <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->L <= 0 || p->S <= 0 || p->E <= 0) return FLB200_E_BAD_ARG;
  if (p->Hq % p->Hkv != 0) return FLB200_E_BAD_ARG;
  if (!p->q || !p->k || !p->v || !p->o || !p->dout || !p->lse || !p->dq || !p->dk || !p->dv) return FLB200_E_BAD_ARG;
  if (!(p->scale > 0.f) || !std::isfinite(p->scale)) return FLB200_E_BAD_ARG;
  if (p->E > 128) return FLB200_E_UNSUPPORTED;  // backward kernels: head dims up to 128, q/k and v alike
  if (p->L > (1 << 24) || p->S > (1 << 24)) return FLB200_E_UNSUPPORTED;
  // the per-row arrays of the workspace are indexed with 32-bit row numbers
  if (static_cast<int64_t>(p->N) * p->Hq * ((static_cast<int64_t>(p->L) + 127) / 128 * 128) > 0x7fffffffLL)
    return FLB200_E_UNSUPPORTED;
  const void* ptrs[] = {p->q, p->k, p->v, p->o, p->dout, p->dq, p->dk, p->dv};
  for (const void* x : ptrs)
    if (!aligned16(x)) return FLB200_E_MISALIGNED;
  if (reinterpret_cast<uintptr_t>(p->lse) & 3u) return FLB200_E_MISALIGNED;
  const int64_t* strides[] = {p->q_stride, p->k_stride, p->v_stride, p->o_stride, p->do_stride,
                              p->dq_stride, p->dk_stride, p->dv_stride};
  for (const int64_t* s : strides) {
    for (int i = 0; i < 3; ++i) {
      if (s[i] < 0) return FLB200_E_BAD_ARG;
      if (s[i] % 8 != 0) return FLB200_E_MISALIGNED;
    }
    if (s[2] < p->E) return FLB200_E_BAD_ARG;
  }
  if ((p->Hq > 1 && p->lse_stride[1] < p->L) || (p->N > 1 && p->lse_stride[0] < p->L)) return FLB200_E_BAD_ARG;
  const size_t need = flb200_attn_bwd_workspace_bytes(p);
  if (!p->workspace || p->workspace_bytes < need) return FLB200_E_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(p->workspace) & 255u) return FLB200_E_MISALIGNED;
  return FLB200_OK;
}

template <int D, bool CAUSAL>
cudaError_t launch_bwd(const flb200_attn_bwd_params* p, const BwdParams& bp, const CUtensorMap& tmQ,
                       const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmdO,
                       const CUtensorMap& tmdQ, const CUtensorMap& tmdK, const CUtensorMap& tmdV,
                       const CUtensorMap& tmX, const CUtensorMap& tmY, cudaStream_t stream) {
  using C = BwdCfg<D>;
  auto dq = attn_bwd_dq_kernel<D, CAUSAL>;
  auto dkv = attn_bwd_dkv_kernel<D, CAUSAL>;
  cudaError_t e = cudaFuncSetAttribute(dq, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(dkv, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  const int nq = (p->L + 127) / 128, nk = (p->S + 127) / 128;
  dkv<<<nk * p->N * p->Hkv, kBwdThreads, C::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmdO, tmdK, tmdV, tmX, tmY, bp);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dq<<<nq * p->N * p->Hq, kBwdThreads, C::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmdO, tmdQ, bp);
  return cudaGetLastError();
}

}  // namespace

extern "C" {

size_t flb200_attn_bwd_workspace_bytes(const flb200_attn_bwd_params* p) {
  if (!p || p->struct_size != sizeof(flb200_attn_bwd_params) || p->N <= 0 || p->Hq <= 0 || p->L <= 0) return 0;
  // per padded query row: delta (fp32), then the two 16-column bf16 rows of the dK/dV kernel's extra k-step
  const size_t lp = (static_cast<size_t>(p->L) + 127) / 128 * 128;
  return static_cast<size_t>(p->N) * p->Hq * lp * (sizeof(float) + 2 * 32);
}

namespace {
int attn_bwd_impl(const flb200_attn_bwd_params* p, void* cuda_stream, bool withhold_loads);
}

int flb200_attn_bwd(const flb200_attn_bwd_params* p, void* cuda_stream) {
  return attn_bwd_impl(p, cuda_stream, false);
}

int flb200_selftest_bwd_wait_timeout(const flb200_attn_bwd_params* p, void* cuda_stream) {
  if (!p || p->struct_size != sizeof(flb200_attn_bwd_params) || !p->status) return FLB200_E_BAD_ARG;
  flb200_attn_bwd_params q = *p;
  if (q.wait_limit_us == 0) q.wait_limit_us = 1000;
  return attn_bwd_impl(&q, cuda_stream, true);
}

}  // extern "C"

namespace {
int attn_bwd_impl(const flb200_attn_bwd_params* p, void* cuda_stream, bool withhold_loads) {
  const int v = validate_bwd(p);
  if (v != FLB200_OK) return v;
  // (cudaSetDevice binds the device's primary context to this thread: the tensor-map encoder is a
  // driver call, and a thread that has made no runtime call yet, such as an autograd worker, has no
  // current context)
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return FLB200_E_LAUNCH;
  if (major != 10) return FLB200_E_ARCH;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

  BwdParams bp;
  std::memset(&bp, 0, sizeof(bp));
  bp.N = p->N;
  bp.Hq = p->Hq;
  bp.Hkv = p->Hkv;
  bp.L = p->L;
  bp.S = p->S;
  bp.G = p->Hq / p->Hkv;
  bp.scale = p->scale;
  bp.scale_log2 = p->scale * 1.4426950408889634f;
  bp.causal = p->causal;
  bp.lse = p->lse;
  bp.lse_sn = p->lse_stride[0];
  bp.lse_sh = p->lse_stride[1];
  bp.delta = static_cast<float*>(p->workspace);
  bp.Lp = (p->L + 127) / 128 * 128;
  bp.status = p->status;
  bp.status_host = p->status_host;
  bp.wait_limit_us = p->wait_limit_us ? p->wait_limit_us : kDefaultWaitLimitUs;
  bp.withhold_loads = withhold_loads ? 1 : 0;

  // head dims below a built width run on it: the tensor maps zero-fill the missing feature columns
  const int width = p->E <= 64 ? 64 : 128;
  CUtensorMap tmQ, tmK, tmV, tmdO, tmdQ, tmdK, tmdV, tmX, tmY;
  auto map = [&](CUtensorMap* tm, const void* base, int rows, int heads, const int64_t* st) {
    return make_tmap_bf16_4d(tm, base, p->E, rows, heads, p->N, st[2], st[1], st[0], 64, 128);
  };
  if (map(&tmQ, p->q, p->L, p->Hq, p->q_stride) || map(&tmK, p->k, p->S, p->Hkv, p->k_stride) ||
      map(&tmV, p->v, p->S, p->Hkv, p->v_stride) || map(&tmdO, p->dout, p->L, p->Hq, p->do_stride) ||
      map(&tmdQ, p->dq, p->L, p->Hq, p->dq_stride) || map(&tmdK, p->dk, p->S, p->Hkv, p->dk_stride) ||
      map(&tmdV, p->dv, p->S, p->Hkv, p->dv_stride))
    return FLB200_E_LAUNCH;

  const int rows = p->N * p->Hq * bp.Lp;
  uint8_t* xrows = static_cast<uint8_t*>(p->workspace) + static_cast<size_t>(rows) * sizeof(float);
  uint8_t* yrows = xrows + static_cast<size_t>(rows) * 32;
  const uint64_t lp = static_cast<uint64_t>(bp.Lp);
  if (make_tmap_bf16_4d(&tmX, xrows, 16, lp, p->Hq, p->N, 16, lp * 16, lp * 16 * p->Hq, 16, 128) ||
      make_tmap_bf16_4d(&tmY, yrows, 16, lp, p->Hq, p->N, 16, lp * 16, lp * 16 * p->Hq, 16, 128))
    return FLB200_E_LAUNCH;
  attn_bwd_delta_kernel<<<rows / 64, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(p->o), static_cast<const __nv_bfloat16*>(p->dout), p->o_stride[0],
      p->o_stride[1], p->o_stride[2], p->do_stride[0], p->do_stride[1], p->do_stride[2], p->E, p->Hq, p->L, bp.Lp,
      bp.delta, p->lse, p->lse_stride[0], p->lse_stride[1], 1.0f / p->scale, reinterpret_cast<uint4*>(xrows),
      reinterpret_cast<uint4*>(yrows));
  if (cudaGetLastError() != cudaSuccess) return FLB200_E_LAUNCH;
  cudaError_t e;
  if (width == 64)
    e = p->causal ? launch_bwd<64, true>(p, bp, tmQ, tmK, tmV, tmdO, tmdQ, tmdK, tmdV, tmX, tmY, stream)
                  : launch_bwd<64, false>(p, bp, tmQ, tmK, tmV, tmdO, tmdQ, tmdK, tmdV, tmX, tmY, stream);
  else
    e = p->causal ? launch_bwd<128, true>(p, bp, tmQ, tmK, tmV, tmdO, tmdQ, tmdK, tmdV, tmX, tmY, stream)
                  : launch_bwd<128, false>(p, bp, tmQ, tmK, tmV, tmdO, tmdQ, tmdK, tmdV, tmX, tmY, stream);
  if (e != cudaSuccess) return FLB200_E_LAUNCH;
  flb::count_launches(3);
  return FLB200_OK;
}

}  // namespace
