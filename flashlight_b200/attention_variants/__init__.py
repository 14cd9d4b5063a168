"""The reference's `attention_variants` package, same names and signatures, backed by the
sm_100a kernels."""
from .vanilla import attention_pytorch, attention_pytorch_nogqa
from .causal import attention_pytorch_causal
from .alibi import AlibiScoreMod, alibi_bias, attention_pytorch_alibi, generate_alibi_bias_pytorch
from .softcap import attention_softcapped, generate_tanh_softcap
from .sliding_window import attention_pytorch_sliding_window, get_sliding_mask
from .document_mask import attention_pytorch_document_mask, create_document_id
from .prefix_lm import attention_pytorch_prefix_lm, get_prefix_lm_mask
from .diff_attn import diffattn
from .evoformer import attention_reference
from .ipa import invariant_point_attention

__all__ = [
    "attention_pytorch", "attention_pytorch_nogqa", "attention_pytorch_causal",
    "AlibiScoreMod", "alibi_bias", "attention_pytorch_alibi", "generate_alibi_bias_pytorch",
    "attention_softcapped", "generate_tanh_softcap",
    "attention_pytorch_sliding_window", "get_sliding_mask",
    "attention_pytorch_document_mask", "create_document_id",
    "attention_pytorch_prefix_lm", "get_prefix_lm_mask",
    "diffattn", "attention_reference", "invariant_point_attention",
]
