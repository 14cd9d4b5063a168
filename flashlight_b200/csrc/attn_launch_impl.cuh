// Definition of launch_attn<>; included by the attn_inst_*.cu files only.
#pragma once
#include "attn_fwd_sm100.cuh"
#include "attn_launch.h"

namespace flb {

template <int E, int EV, int SCORE, int MASK, int DIFF, int STAGES>
cudaError_t launch_attn(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                        const CUtensorMap& tmO, const CUtensorMap& tmB, const KernelParams& p, int grid,
                        int cluster,
                        cudaStream_t stream) {
  using C = AttnCfg<E, EV, SCORE, MASK, DIFF, STAGES>;
  auto kernel = attn_fwd_kernel<C>;
  // per device and cheap, so it is simply repeated on every launch
  cudaError_t e =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  if (cluster <= 1) {
    kernel<<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmO, tmB, p);
    return cudaGetLastError();
  }
  // neighbouring CTAs form a thread-block cluster (they exchange row sums through distributed
  // shared memory)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(C::THREADS);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = cluster;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, tmQ, tmK, tmV, tmO, tmB, p);
}

#define FLB_INSTANTIATE(E, EV, SCORE, MASK, DIFF, STAGES)                                    \
  template cudaError_t launch_attn<E, EV, SCORE, MASK, DIFF, STAGES>(                         \
      const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,         \
      const CUtensorMap&, const KernelParams&, int, int, cudaStream_t);

}  // namespace flb
