"""fmta_b200: B200-native fused multi-token (conv) attention.

Same operator API as the reference package (``ConvAttentionCUDA``,
``FlashConvAttentionCUDAFunction``, ``forward`` / ``dq_backward`` / ``dkdv_backward``,
``fwd_conv_attn_inference`` / ``forward_inference``, ``HeadConvAttentionFunction``,
``HeadConvAttention``, ``head_conv_attention``), backed by hand-written sm_100a CUDA behind a
C ABI (libfmta_b200.so).  Importing fails if the library has not been built.
"""
from ._lib import lib as _c_lib, LIB_PATH, check_device_status  # noqa: F401  (raises ImportError when missing)
from .conv_attn import (ConvAttentionCUDA, FlashConvAttentionCUDAFunction, forward, dq_backward,  # noqa: F401
                        dkdv_backward, backward, rowdot, ktilde_buffer)
from .inference import (forward_inference, fwd_conv_attn_inference, forward_inference_paged,  # noqa: F401
                        kv_append_paged)
from .head_conv import (HeadConvAttentionFunction, HeadConvAttention, head_conv_attention,  # noqa: F401
                        head_conv_attention_forward, head_conv_attention_bwd_dq_dw,
                        head_conv_attention_bwd_dkdv, conv_headmix_attention, conv_headmix_forward,
                        conv_headmix_bwd_dq_dw, conv_headmix_bwd_dkdv, conv_headmix_backward)
from . import sharding  # noqa: F401
from . import context_parallel  # noqa: F401
from .context_parallel import (ContextParallelConvAttentionFunction, context_parallel_conv_attention,  # noqa: F401
                               forward_window, backward_window, windows_for_rank)

__version__ = "0.1.0"
