// heads above 128 and up to 256: plain and causal attention and the product chain, one query tile per CTA
#include "attn_launch_impl.cuh"
namespace flb {
FLB_INSTANTIATE(256, 256, SCORE_NONE, MASK_NONE, 0, 1)
FLB_INSTANTIATE(256, 256, SCORE_NONE, MASK_CAUSAL, 0, 1)
FLB_INSTANTIATE(256, 256, SCORE_B2B, MASK_NONE, 0, 1)
FLB_INSTANTIATE(256, 256, SCORE_B2BT, MASK_NONE, 0, 1)
}
