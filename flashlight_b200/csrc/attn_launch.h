// Declaration of the per-instantiation launchers.  Each attn_inst_*.cu file
// explicitly instantiates a group of them so the groups compile in parallel;
// capi.cu dispatches on (E, EV, score modifier, mask, diff, query tiles per CTA).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "attn_params.h"

namespace flb {

template <int E, int EV, int SCORE, int MASK, int DIFF, int STAGES>
cudaError_t launch_attn(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                        const CUtensorMap& tmO, const CUtensorMap& tmB, const KernelParams& p, int grid,
                        int cluster,
                        cudaStream_t stream);

}  // namespace flb
