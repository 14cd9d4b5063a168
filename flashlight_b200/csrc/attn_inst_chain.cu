// back-to-back product O = f(Q K^T * scale) V (no softmax), K as [S][E] rows or as [E][S]
#include "attn_launch_impl.cuh"
namespace flb {
FLB_INSTANTIATE(128, 128, SCORE_B2B, MASK_NONE, false, 2)
FLB_INSTANTIATE(128, 128, SCORE_B2BT, MASK_NONE, false, 2)
FLB_INSTANTIATE(64, 64, SCORE_B2B, MASK_NONE, false, 2)
FLB_INSTANTIATE(64, 64, SCORE_B2BT, MASK_NONE, false, 2)
FLB_INSTANTIATE(32, 32, SCORE_B2B, MASK_NONE, false, 2)
FLB_INSTANTIATE(32, 32, SCORE_B2BT, MASK_NONE, false, 2)
}
