"""Python entry points of the hand-written kernels. Each function checks its
arguments, allocates its output with torch and launches on the current stream."""
from .basic import (embed, add_rmsnorm, residual_add, swiglu, short_conv, qk_norm_rope,
                    attention_plain, argmax, sample, upload, take_pending_tokens, keep_last_tokens,
                    stream_cast, gated_norm_add, mingru_scan, head_product, gated_act, attention_latent)
from .gemm import gemm, gemm_act, gemm_plain
from .recurrent import (embed_pairs, norm_pair, scaled_add2, pair_norm_mean, conv_state_update, sink_attn_prep, attention_plain_sink, attention_flash_sink,
                        hgrn2_scan, delta_prep, delta_scan, head_norm_gate, activation, attention_plain_masked, attention_flash_masked, gdelta_prep, gdelta_scan)
from .stream import add_scaled_norm, stream_add_rows, token_gate_mul, scaled_rms_add, weighted_sum2, xielu, head_gate_mul
from .attention import attention
from .gemm_bf16 import gemm_swiglu_bf16, tensor_core_ok

__all__ = ["embed", "add_rmsnorm", "residual_add", "swiglu", "short_conv", "qk_norm_rope",
           "attention_plain", "argmax", "sample", "upload", "take_pending_tokens", "keep_last_tokens", "gemm", "gemm_act", "gemm_plain", "attention", "gemm_swiglu_bf16", "tensor_core_ok",
           "embed_pairs", "norm_pair", "scaled_add2", "pair_norm_mean", "conv_state_update", "sink_attn_prep", "attention_plain_sink", "attention_flash_sink",
           "hgrn2_scan", "delta_prep", "delta_scan", "head_norm_gate", "activation",
           "attention_plain_masked", "attention_flash_masked", "gdelta_prep", "gdelta_scan", "add_scaled_norm", "stream_add_rows", "token_gate_mul", "scaled_rms_add",
           "weighted_sum2", "xielu", "head_gate_mul",
           "stream_cast", "gated_norm_add", "mingru_scan", "head_product", "gated_act", "attention_latent"]
