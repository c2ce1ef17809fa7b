"""Choice of the attention kernel for a step.

float32: always the plain kernel (fixed reduction order per token).
bfloat16: the plain kernel as well, until a faster kernel covers the case.
"""
from __future__ import annotations

from . import kernels as K


def paged_attention(out, q, n_q_heads, n_kv_heads, head_dim, k_cache, v_cache, block_table, ctx, scale, window, rt):
    return K.paged_attention_generic(out, q, n_q_heads, n_kv_heads, head_dim, k_cache, v_cache, block_table,
                                     ctx.seq_of_token, ctx.positions, scale, window, rt.status)
