"""Python entry points of the hand-written CUDA kernels (sources in ../csrc)."""
from . import _lib
from ._lib import KernelError, Timeline, launches, mark, mark_tc_launched
from .attention import attention, attention_ext, check_head_geometry, check_row_widths, plan_splits, split_scratch_floats
from .elementwise import (ACT_GELU_TANH, ACT_SILU, activation_code, add_normed_copy, round_rows, row_inv_rms, GATE_SIGMOID, GATE_SILU, GATE_SILU_FIRST, add_into, add_normed, add_scaled, embed, embed_sinusoid, group_rmsnorm, qkv_rope_cache, random_fill, rmsnorm,
                          scale_inplace, select_tokens, swiglu, tanh_rows, head_encode, sigmoid_gate, tanh_cap)
from .experts import router_choice, routed_experts_rows, routed_experts_tiles, routed_tiles_ok, table_choice
from .streams import streams_fill, streams_step
from .gemm import (PendingNorm, check_tc_status, decode_gemm_tc, gemm_tc, gemm_tiled, gemv_rows, linear, product_adds_shares, set_gemm_tc_mode,
                   skinny_gemm)
from .mlstm import mlstm_gates, mlstm_read
from .latent import latent_expand, latent_heads, latent_query, latent_rows
from .scan import gated_scan, linear_scan, short_conv
from .sampling import sample
from .sigmoid import rownorm_qkv_store, sigmoid_attention

__all__ = ["ACT_GELU_TANH", "ACT_SILU", "activation_code", "add_normed_copy", "round_rows", "row_inv_rms", "router_choice", "mlstm_gates", "mlstm_read", "attention_ext", "check_row_widths", "head_encode", "sigmoid_gate", "tanh_cap", "routed_experts_rows", "routed_experts_tiles", "routed_tiles_ok", "table_choice", "streams_fill", "streams_step", "KernelError", "PendingNorm", "Timeline", "mark", "add_into", "attention", "check_head_geometry", "check_tc_status", "decode_gemm_tc", "embed", "launches", "mark_tc_launched", "gemm_tc", "gemm_tiled", "set_gemm_tc_mode", "gemv_rows",
           "GATE_SIGMOID", "GATE_SILU", "GATE_SILU_FIRST", "add_scaled", "gated_scan", "latent_expand", "latent_heads", "latent_query", "latent_rows", "short_conv",
           "add_normed", "embed_sinusoid", "group_rmsnorm", "linear_scan", "rownorm_qkv_store", "scale_inplace", "sigmoid_attention", "tanh_rows",
           "linear", "plan_splits", "product_adds_shares", "qkv_rope_cache", "random_fill", "rmsnorm", "select_tokens", "sample", "skinny_gemm", "split_scratch_floats", "swiglu"]
