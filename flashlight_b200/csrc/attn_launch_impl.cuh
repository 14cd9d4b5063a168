// Definition of launch_attn<>; included by the attn_inst_*.cu files only.
#pragma once
#include "attn_fwd_sm100.cuh"
#include "attn_launch.h"

namespace flb {

template <int E, int EV, int SCORE, int MASK, bool DIFF, int STAGES>
cudaError_t launch_attn(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                        const CUtensorMap& tmO, const KernelParams& p, int grid, cudaStream_t stream) {
  using C = AttnCfg<E, EV, SCORE, MASK, DIFF, STAGES>;
  auto kernel = attn_fwd_kernel<C>;
  // per device and cheap, so it is simply repeated on every launch
  cudaError_t e =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  kernel<<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmO, p);
  return cudaGetLastError();
}

#define FLB_INSTANTIATE(E, EV, SCORE, MASK, DIFF, STAGES)                                    \
  template cudaError_t launch_attn<E, EV, SCORE, MASK, DIFF, STAGES>(                         \
      const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,         \
      const KernelParams&, int, cudaStream_t);

}  // namespace flb
