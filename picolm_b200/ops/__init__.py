"""Python faces of the CUDA kernels.  Every function checks what it is given
(device, dtype, shape, contiguity), launches on the current CUDA stream and
raises `KernelError` if the kernel library refuses or fails.  There is no CPU
path: a tensor that is not on a CUDA device is an error.
"""
from ._lib import (PAGE_TOKENS, SM_COUNT, KernelError, check_status, count_launches, launch_count,  # noqa: F401
                   status_word, stream_scope, trace_report)
from .attention import (DECODE_CLUSTER_SPLITS, Rotation, attention, attention_decode,  # noqa: F401
                        attention_decode_rope, attention_decode_rope_supported, attention_mma_supported,
                        attention_prefill, attention_prefill_tc, attention_rows, attention_tc_supported, decode_splits)
from .chain import Chain, LazyRows  # noqa: F401
from .elementwise import (GATE_ACTIVATIONS, add_bias, add_rows, dyt_norm, embed, gather_rows, layernorm,  # noqa: F401
                          post_pre_norm, post_pre_norm_supported, qk_norm_rope_store, rmsnorm, rope_store, scaled_sum,
                          swiglu, token_gate, rope_rows, norm_pair_shift)
from .gemm import (PendingLinear, ScaledRows, gemm_simt, gemm_tc_skinny, gemm_tc_supported,  # noqa: F401
                   gemm_tc_wide, interleave_gate_up, linear, linear_residual_norm, linear_swiglu, pair_pays,
                   residual_norm_supported)
from .recurrent import (DECAY_SIGMOID, DECAY_STEP, GATE_AFTER_NORM, GATE_BEFORE_NORM, GATE_NONE, causal_conv,  # noqa: F401
                        delta_prep, delta_scan, diag_scan, gated_norm, head_linear, linear_scan, rglru_gates,
                        store_rows_paged, latent_store)
from .routed import (SortedPairs, moe_align, moe_combine, moe_down, moe_down_tc, moe_gate_up, moe_gate_up_tc,  # noqa: F401
                     moe_gather, moe_max_tiles, moe_tc_supported, route_topk, router_logits)
from .sampling import argmax, sample  # noqa: F401
