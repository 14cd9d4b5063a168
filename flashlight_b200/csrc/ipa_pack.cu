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

// one thread per row; rows are short (tens of elements) and the whole job is a few megabytes
__global__ void ipa_pack_kernel(const IpaPack p) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const __nv_bfloat16 zero = __float2bfloat16_rn(0.f), one = __float2bfloat16_rn(1.f);
  if (r < p.rows_q) {
    __nv_bfloat16* o = p.qa + static_cast<int64_t>(r) * p.E;
    const __nv_bfloat16* s = p.qs + static_cast<int64_t>(r) * p.C;
    const __nv_bfloat16* pt = p.qp + static_cast<int64_t>(r) * p.PQ;
    int c = 0;
    for (int i = 0; i < p.C; ++i) o[c++] = s[i];
    for (int i = 0; i < p.PQ; ++i) o[c++] = pt[i];   // against hi(-2a k_p)
    for (int i = 0; i < p.PQ; ++i) o[c++] = pt[i];   // against lo(-2a k_p)
    o[c++] = one;                                     // against hi(a |k_p|^2)
    o[c++] = one;                                     // against lo(a |k_p|^2)
    while (c < p.E) o[c++] = zero;
  }
  if (r < p.rows_k) {
    __nv_bfloat16* o = p.ka + static_cast<int64_t>(r) * p.E;
    const __nv_bfloat16* s = p.ks + static_cast<int64_t>(r) * p.C;
    const __nv_bfloat16* pt = p.kp + static_cast<int64_t>(r) * p.PQ;
    int c = 0;
    for (int i = 0; i < p.C; ++i) o[c++] = s[i];
    float norm = 0.f;
    for (int i = 0; i < p.PQ; ++i) {
      const float x = __bfloat162float(pt[i]);
      norm = fmaf(x, x, norm);
      const uint32_t w = split_bf16_pair(-2.0f * p.a * x);
      o[c + i] = __ushort_as_bfloat16(static_cast<unsigned short>(w & 0xffffu));
      o[c + p.PQ + i] = __ushort_as_bfloat16(static_cast<unsigned short>(w >> 16));
    }
    c += 2 * p.PQ;
    const uint32_t w = split_bf16_pair(p.a * norm);
    o[c++] = __ushort_as_bfloat16(static_cast<unsigned short>(w & 0xffffu));
    o[c++] = __ushort_as_bfloat16(static_cast<unsigned short>(w >> 16));
    while (c < p.E) o[c++] = zero;

    __nv_bfloat16* ov = p.va + static_cast<int64_t>(r) * p.Ev;
    const __nv_bfloat16* sv = p.vs + static_cast<int64_t>(r) * p.C;
    const __nv_bfloat16* pv = p.vp + static_cast<int64_t>(r) * p.PV;
    int cv = 0;
    for (int i = 0; i < p.C; ++i) ov[cv++] = sv[i];
    for (int i = 0; i < p.PV; ++i) ov[cv++] = pv[i];
    while (cv < p.Ev) ov[cv++] = zero;
  }
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
  IpaPack k{p->rows_q, p->rows_k, p->C, PQ, PV, p->E, p->Ev,
            static_cast<const __nv_bfloat16*>(p->q_scalar), static_cast<const __nv_bfloat16*>(p->k_scalar),
            static_cast<const __nv_bfloat16*>(p->v_scalar), static_cast<const __nv_bfloat16*>(p->q_points),
            static_cast<const __nv_bfloat16*>(p->k_points), static_cast<const __nv_bfloat16*>(p->v_points), p->a,
            static_cast<__nv_bfloat16*>(p->q_aug), static_cast<__nv_bfloat16*>(p->k_aug),
            static_cast<__nv_bfloat16*>(p->v_aug)};
  const int rows = p->rows_q > p->rows_k ? p->rows_q : p->rows_k;
  ipa_pack_kernel<<<(rows + 127) / 128, 128, 0, static_cast<cudaStream_t>(cuda_stream)>>>(k);
  if (cudaGetLastError() != cudaSuccess) return FLB200_E_LAUNCH;
  flb::count_launches(1);
  return FLB200_OK;
}
