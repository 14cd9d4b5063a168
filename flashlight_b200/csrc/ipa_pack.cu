// Operand assembly for invariant point attention: one kernel writes the augmented q / k / v rows that
// turn the operator into a pair-biased attention (see flb200_ipa_pack in the header).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/flb200_attn.h"
#include "ptx.cuh"

namespace flb {
void count_launches(int n);  // capi.cu: the library's launch counter
}

namespace {

using flb::split_bf16_pair;

struct IpaPack {
  int rows_q, rows_k, C, PQ, PV, E, Ev;  // PQ, PV: point coordinates per row (points x point_dim)
  const __nv_bfloat16 *qs, *ks, *vs, *qp, *kp, *vp;
  float a;
  __nv_bfloat16 *qa, *ka, *va;
};

// one thread per 8 output elements (one 16-byte store): chunks of the q' rows, then of the k' rows, then of v'
__global__ void ipa_pack_kernel(const IpaPack p) {
  const int cq = p.E / 8, cv = p.Ev / 8;
  const int64_t nq = static_cast<int64_t>(p.rows_q) * cq, nk = static_cast<int64_t>(p.rows_k) * cq;
  const int64_t nv = static_cast<int64_t>(p.rows_k) * cv;
  int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= nq + nk + nv) return;
  const unsigned short one = 0x3F80u;  // 1.0 as bf16
  unsigned short e[8];
  uint4* dst;
  if (idx < nq) {
    const int64_t r = idx / cq;
    const int c0 = static_cast<int>(idx % cq) * 8;
    const unsigned short* s = reinterpret_cast<const unsigned short*>(p.qs) + r * p.C;
    const unsigned short* pt = reinterpret_cast<const unsigned short*>(p.qp) + r * p.PQ;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = c0 + i;
      e[i] = c < p.C ? s[c]
             : c < p.C + p.PQ ? pt[c - p.C]                      // against hi(-2a k_p)
             : c < p.C + 2 * p.PQ ? pt[c - p.C - p.PQ]           // against lo(-2a k_p)
             : c < p.C + 2 * p.PQ + 2 ? one : 0;                 // against hi, lo of a |k_p|^2
    }
    dst = reinterpret_cast<uint4*>(p.qa + r * p.E + c0);
  } else if (idx < nq + nk) {
    idx -= nq;
    const int64_t r = idx / cq;
    const int c0 = static_cast<int>(idx % cq) * 8;
    const unsigned short* s = reinterpret_cast<const unsigned short*>(p.ks) + r * p.C;
    const __nv_bfloat16* pt = p.kp + r * p.PQ;
    const int cn = p.C + 2 * p.PQ;  // columns cn, cn + 1: the squared norm
    uint32_t wn = 0;
    if (c0 <= cn + 1 && c0 + 8 > cn) {
      float norm = 0.f;
      for (int i = 0; i < p.PQ; ++i) {
        const float x = __bfloat162float(pt[i]);
        norm = fmaf(x, x, norm);
      }
      wn = split_bf16_pair(p.a * norm);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = c0 + i;
      if (c < p.C) {
        e[i] = s[c];
      } else if (c < cn) {
        const bool lo = c >= p.C + p.PQ;
        const uint32_t w = split_bf16_pair(-2.0f * p.a * __bfloat162float(pt[c - p.C - (lo ? p.PQ : 0)]));
        e[i] = static_cast<unsigned short>(lo ? w >> 16 : w & 0xffffu);
      } else {
        e[i] = c == cn ? static_cast<unsigned short>(wn & 0xffffu) : c == cn + 1 ? static_cast<unsigned short>(wn >> 16) : 0;
      }
    }
    dst = reinterpret_cast<uint4*>(p.ka + r * p.E + c0);
  } else {
    idx -= nq + nk;
    const int64_t r = idx / cv;
    const int c0 = static_cast<int>(idx % cv) * 8;
    const unsigned short* s = reinterpret_cast<const unsigned short*>(p.vs) + r * p.C;
    const unsigned short* pt = reinterpret_cast<const unsigned short*>(p.vp) + r * p.PV;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = c0 + i;
      e[i] = c < p.C ? s[c] : c < p.C + p.PV ? pt[c - p.C] : 0;
    }
    dst = reinterpret_cast<uint4*>(p.va + r * p.Ev + c0);
  }
  *dst = make_uint4(e[0] | (static_cast<uint32_t>(e[1]) << 16), e[2] | (static_cast<uint32_t>(e[3]) << 16),
                    e[4] | (static_cast<uint32_t>(e[5]) << 16), e[6] | (static_cast<uint32_t>(e[7]) << 16));
}

}  // namespace

extern "C" int flb200_ipa_pack(const flb200_ipa_pack_params* p, void* cuda_stream) {
  if (!p || p->struct_size != sizeof(flb200_ipa_pack_params)) return FLB200_E_BAD_ARG;
  if (p->rows_q <= 0 || p->rows_k <= 0 || p->C < 0 || p->P_qk < 0 || p->P_v < 0 || p->point_dim <= 0)
    return FLB200_E_BAD_ARG;
  if (!p->q_scalar || !p->k_scalar || !p->v_scalar || !p->q_points || !p->k_points || !p->v_points || !p->q_aug ||
      !p->k_aug || !p->v_aug)
    return FLB200_E_BAD_ARG;
  const int PQ = p->P_qk * p->point_dim, PV = p->P_v * p->point_dim;
  if (p->E % 8 != 0 || p->Ev % 8 != 0 || p->E < p->C + 2 * PQ + 2 || p->Ev < p->C + PV) return FLB200_E_BAD_ARG;
  if (!(p->a == p->a)) return FLB200_E_BAD_ARG;
  const void* outs[] = {p->q_aug, p->k_aug, p->v_aug};
  for (const void* o : outs)
    if (reinterpret_cast<uintptr_t>(o) & 15u) return FLB200_E_MISALIGNED;  // 16-byte stores
  IpaPack k{p->rows_q, p->rows_k, p->C, PQ, PV, p->E, p->Ev,
            static_cast<const __nv_bfloat16*>(p->q_scalar), static_cast<const __nv_bfloat16*>(p->k_scalar),
            static_cast<const __nv_bfloat16*>(p->v_scalar), static_cast<const __nv_bfloat16*>(p->q_points),
            static_cast<const __nv_bfloat16*>(p->k_points), static_cast<const __nv_bfloat16*>(p->v_points), p->a,
            static_cast<__nv_bfloat16*>(p->q_aug), static_cast<__nv_bfloat16*>(p->k_aug),
            static_cast<__nv_bfloat16*>(p->v_aug)};
  const int64_t chunks = (static_cast<int64_t>(p->rows_q) + p->rows_k) * (p->E / 8) + static_cast<int64_t>(p->rows_k) * (p->Ev / 8);
  ipa_pack_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(k);
  if (cudaGetLastError() != cudaSuccess) return FLB200_E_LAUNCH;
  flb::count_launches(1);
  return FLB200_OK;
}
