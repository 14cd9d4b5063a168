// one query tile per CTA, head dim 128: plain and causal, with and without ALiBi / softcap
#include "attn_launch_impl.cuh"
namespace flb {
FLB_INSTANTIATE(128, 128, SCORE_NONE, MASK_NONE, false, 1)
FLB_INSTANTIATE(128, 128, SCORE_NONE, MASK_CAUSAL, false, 1)
FLB_INSTANTIATE(128, 128, SCORE_ALIBI, MASK_NONE, false, 1)
FLB_INSTANTIATE(128, 128, SCORE_ALIBI, MASK_CAUSAL, false, 1)
FLB_INSTANTIATE(128, 128, SCORE_SOFTCAP, MASK_NONE, false, 1)
FLB_INSTANTIATE(128, 128, SCORE_SOFTCAP, MASK_CAUSAL, false, 1)
}
