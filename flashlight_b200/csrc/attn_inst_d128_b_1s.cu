// one query tile per CTA, head dim 128: sliding window, prefix-LM, document mask, additive bias
#include "attn_launch_impl.cuh"
namespace flb {
FLB_INSTANTIATE(128, 128, SCORE_NONE, MASK_SLIDING, 0, 1)
FLB_INSTANTIATE(128, 128, SCORE_NONE, MASK_PREFIX, 0, 1)
FLB_INSTANTIATE(128, 128, SCORE_NONE, MASK_DOCUMENT, 0, 1)
FLB_INSTANTIATE(128, 128, SCORE_BIAS, MASK_NONE, 0, 1)
}
