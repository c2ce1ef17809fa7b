"""The built-in part kinds: RMSNorm, rotary positions, grouped-query attention over
the paged cache, SwiGLU feed-forward, the pre-norm block, token embedding and
the linear output head.  Formulas follow the reference's Qwen3 forward pass
(src/graph/executor_forward.cu:252-820 attention, :826-1179 feed-forward,
:2701-3140 the whole step); each class cites the lines it restates.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch

from ..cache.manager import PagedKVSpec
from ..ops import kernels as K
from .base import (Block, Embedding, FeedForward, Head, LayerCache, Mixer, Norm, PositionEncoding, Runtime)
from .plan import PartSpec, TensorSpec
from .registry import part_class, register_part


def build_part(category: str, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
    """Construct one part from its spec; parts without tensors are shared between equal specs."""
    cls = part_class(category, spec.kind)
    if not spec.tensors:
        key = (category, spec.key())
        if key not in rt.shared:
            rt.shared[key] = cls(dict(spec.params), {}, rt)
        return rt.shared[key]
    return cls(dict(spec.params), tensors, rt)


def _cat_rows(tensors):
    """Stack weight matrices along the output dimension (widening to float32 if their types differ)."""
    dts = {t.dtype for t in tensors}
    if len(dts) > 1:
        tensors = [t.float() for t in tensors]
    return torch.cat(tensors, dim=0).contiguous()


# --------------------------------------------------------------------------- norm
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * (w + weight_offset), statistics in 32-bit
    (src/compute/layernorm.cu:50-82).  params: size, eps, weight_offset (default 0)."""

    @classmethod
    def tensor_specs(cls, params):
        return {"weight": TensorSpec((params["size"],), role="norm", init="one_plus_normal")}

    takes_split_sum = True

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.weight = tensors["weight"]
        self.eps = float(params["eps"])
        self.offset = float(params.get("weight_offset", 0.0))

    def add_norm(self, h, branch, rows=None):
        n = h.shape[0] if rows is None else rows.numel()
        out = self.rt.empty((n, h.shape[1]))
        return K.add_rmsnorm(h, branch, self.weight, out, self.eps, self.offset, rows=rows)

    def norm_rows(self, x: torch.Tensor) -> torch.Tensor:
        """Plain RMSNorm of the rows of a 2-D activation tensor."""
        return K.rmsnorm_rows(x, self.weight, torch.empty_like(x), self.eps, self.offset)


# ----------------------------------------------------------------------- position
class RotaryPosition(PositionEncoding):
    """Rotary encoding over pairs (i, i + rot/2) with angle pos * theta^(-2i/rot)
    (src/compute/rope.cu:84-101).  The cos/sin table is made in double precision
    on the host, once.  params: head_dim, theta, max_positions, rotary_dim (default head_dim)."""

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.head_dim = int(params["head_dim"])
        self.rot = int(params.get("rotary_dim") or self.head_dim)
        if self.rot % 2 or not 0 < self.rot <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rot} must be even and within head_dim {self.head_dim}")
        theta = float(params["theta"])
        n_pos = int(params["max_positions"])
        i = torch.arange(self.rot // 2, dtype=torch.float64)
        inv_freq = theta ** (-2.0 * i / self.rot)
        ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.cos = ang.cos().to(torch.float32).to(rt.device).contiguous()
        self.sin = ang.sin().to(torch.float32).to(rt.device).contiguous()

    def rotary_tables(self):
        return self.cos, self.sin, self.rot


# -------------------------------------------------------------------------- mixer
class GQAAttention(Mixer):
    """Grouped-query softmax attention over the paged cache.

    q,k,v = x Wq^T, x Wk^T, x Wv^T without bias (src/graph/executor_forward.cu:429-470);
    optional per-head RMSNorm on q and k with one [head_dim] weight each, before the
    position encoding (:536-546); keys and values go to the pages first, then every new
    token attends to its sequence's cached positions up to its own, within `window`
    if set; scale 1/sqrt(head_dim) (:566); out = attn Wo^T (:773-777).

    params: hidden_size, num_heads, num_kv_heads, head_dim, window (0 = all),
            qk_norm (bool), qk_norm_eps, position (PartSpec or None), scale (optional).
    """

    @classmethod
    def tensor_specs(cls, params):
        d, hq, hkv, dh = params["hidden_size"], params["num_heads"], params["num_kv_heads"], params["head_dim"]
        specs = {
            "q_proj": TensorSpec((hq * dh, d)),
            "k_proj": TensorSpec((hkv * dh, d)),
            "v_proj": TensorSpec((hkv * dh, d)),
            "o_proj": TensorSpec((d, hq * dh)),
        }
        if params.get("qk_norm"):
            specs["q_norm"] = TensorSpec((dh,), role="norm", init="one_plus_normal")
            specs["k_norm"] = TensorSpec((dh,), role="norm", init="one_plus_normal")
        return specs

    @classmethod
    def cache_spec(cls, params):
        return PagedKVSpec(int(params["num_kv_heads"]), int(params["head_dim"]), int(params.get("window") or 0))

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.hq, self.hkv, self.dh = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["head_dim"])
        if self.hq % self.hkv:
            raise ValueError(f"{self.hq} query heads are not a multiple of {self.hkv} kv heads")
        if self.dh % 16 or not 0 < self.dh <= 256:
            raise ValueError(f"head_dim {self.dh} must be a multiple of 16 in (0, 256]")
        self.window = int(params.get("window") or 0)
        self.scale = float(params.get("scale") or 1.0 / math.sqrt(self.dh))
        self.w_qkv = _cat_rows([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]])
        self.w_o = tensors["o_proj"]
        self.q_norm = tensors.get("q_norm") if params.get("qk_norm") else None
        self.k_norm = tensors.get("k_norm") if params.get("qk_norm") else None
        if self.q_norm is not None and self.q_norm.dtype != self.k_norm.dtype:
            self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()
        self.norm_eps = float(params.get("qk_norm_eps", 1e-6))
        # 32-bit copies of the two small weight vectors for the fused projection kernel
        self.q_norm_f32 = self.q_norm.float().contiguous() if self.q_norm is not None else None
        self.k_norm_f32 = self.k_norm.float().contiguous() if self.k_norm is not None else None
        pos = params.get("position")
        self.position = build_part("position", pos, {}, rt) if pos is not None else None
        tensors.clear()  # the separate q/k/v matrices are not kept

    def forward(self, x, ctx, cache: LayerCache):
        rt, T = self.rt, x.shape[0]
        tables = self.position.rotary_tables() if self.position is not None else None
        if tables is not None and cache.writes and not rt.is_float32 and tables[2] == self.dh:
            # long portions: projection, norm, rotation and cache write in one kernel
            q = rt.empty((T, self.hq * self.dh))
            if K.linear_qkv_rope(q, x, self.w_qkv, self.hq, self.hkv, self.dh, self.q_norm_f32, self.k_norm_f32,
                                 self.norm_eps, tables[0], tables[1], ctx.positions, ctx.seq_of_token, cache.block_table,
                                 cache.kv[0], cache.kv[1], rt.status):
                attn = rt.empty((T, self.hq * self.dh))
                self.attend(attn, q, ctx, cache)
                out = rt.empty((T, self.w_o.shape[0]))
                return K.linear(out, attn, self.w_o, may_defer=self.defer_out)
        qkv = rt.empty((T, (self.hq + 2 * self.hkv) * self.dh))
        K.linear(qkv, x, self.w_qkv)
        if tables is not None and cache.writes and not rt.is_float32 and tables[2] == self.dh and ctx.decode_only:
            # decode steps: the attention kernel normalises and rotates q and the new key itself and writes the new
            # key and value into their pages (no rotary kernel)
            from ..ops import attention as A
            attn = rt.empty((T, self.hq * self.dh))
            if A.decode_attention_fused(attn, qkv, self.hq, self.hkv, self.dh, cache.kv[0], cache.kv[1], cache.block_table,
                                        ctx.seq_of_token, ctx.positions, self.scale, self.window, self.q_norm_f32,
                                        self.k_norm_f32, self.norm_eps, tables[0], tables[1], rt.status):
                out = rt.empty((T, self.w_o.shape[0]))
                return K.linear(out, attn, self.w_o, may_defer=self.defer_out)
        k_cache = cache.kv[0] if cache.writes else None
        v_cache = cache.kv[1] if cache.writes else None
        if self.position is not None and tables is None:
            # An encoding the fused kernel does not know: let the part rewrite q and k, then norm-free write.
            q3 = qkv[:, :self.hq * self.dh].view(T, self.hq, self.dh)
            k3 = qkv[:, self.hq * self.dh:(self.hq + self.hkv) * self.dh].view(T, self.hkv, self.dh)
            if self.q_norm is not None:
                K.qk_norm_rope_kv_write(qkv, self.hq, self.hkv, self.dh, self.q_norm, self.k_norm, self.norm_eps,
                                        None, None, 0, ctx.positions, None, None, None, None, rt.status)
            self.position.apply(q3, k3, ctx)
            K.qk_norm_rope_kv_write(qkv, self.hq, self.hkv, self.dh, None, None, self.norm_eps, None, None, 0,
                                    ctx.positions, ctx.seq_of_token, cache.block_table, k_cache, v_cache, rt.status)
        else:
            cos, sin, rot = tables if tables is not None else (None, None, 0)
            K.qk_norm_rope_kv_write(qkv, self.hq, self.hkv, self.dh, self.q_norm, self.k_norm, self.norm_eps,
                                    cos, sin, rot, ctx.positions, ctx.seq_of_token, cache.block_table,
                                    k_cache, v_cache, rt.status)
        attn = rt.empty((T, self.hq * self.dh))
        self.attend(attn, qkv[:, :self.hq * self.dh], ctx, cache)
        out = rt.empty((T, self.w_o.shape[0]))
        return K.linear(out, attn, self.w_o, may_defer=self.defer_out)

    def attend(self, out, q, ctx, cache: LayerCache):
        """out[t] = softmax(scale * q[t] K^T) V over the cached positions token t may see."""
        from ..ops import attention as A
        A.paged_attention(out, q, self.hq, self.hkv, self.dh, cache.kv[0], cache.kv[1], cache.block_table, ctx,
                          self.scale, self.window, self.rt)


# ------------------------------------------------------------------- feed-forward
class SwiGLU(FeedForward):
    """down( silu(x Wg^T) * (x Wu^T) ), activation in 32-bit
    (src/graph/executor_forward.cu:933-951, 1124-1140; src/compute/activation.cu:67-87).
    params: hidden_size, intermediate_size."""

    @classmethod
    def tensor_specs(cls, params):
        d, f = params["hidden_size"], params["intermediate_size"]
        return {"gate_proj": TensorSpec((f, d)), "up_proj": TensorSpec((f, d)), "down_proj": TensorSpec((d, f))}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.f = int(params["intermediate_size"])
        gate, up = tensors["gate_proj"], tensors["up_proj"]
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        # Gate and up rows alternate in runs of 8 so that one kernel can produce the activation
        # from the fused product; a width that is no multiple of 8 keeps the two halves apart.
        self.interleaved = self.f % K.SWIGLU_INTERLEAVE == 0
        self.w_gu = K.interleave_gate_up(gate, up) if self.interleaved else _cat_rows([gate, up])
        self.w_down = tensors["down_proj"]
        tensors.clear()

    def forward(self, x, ctx):
        rt, T = self.rt, x.shape[0]
        act = rt.empty((T, self.f))
        if self.interleaved:
            K.linear_swiglu(act, x, self.w_gu)
        else:
            gu = rt.empty((T, 2 * self.f))
            K.linear(gu, x, self.w_gu)
            K.swiglu(act, gu)
        out = rt.empty((T, self.w_down.shape[0]))
        return K.linear(out, act, self.w_down, may_defer=self.defer_out)


# -------------------------------------------------------------------------- block
class PreNormBlock(Block):
    """h += mixer(norm1(h)); h += ffn(norm2(h))  (pre-norm, src/model/model.h:66).

    The second sum is handed on as `pending` and added by whoever normalises the stream
    next (the next block's first norm, or the final norm), in the same kernel."""

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, rt):
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm, rt)
        # the mixer's output goes to this block's second norm and nowhere else
        if ffn_norm.takes_split_sum:
            mixer.defer_out = True

    @property
    def takes_split_sum(self):
        return self.mixer_norm.takes_split_sum

    def forward(self, h, pending, ctx, cache):
        x = self.mixer_norm.add_norm(h, pending)
        a = self.mixer.forward(x, ctx, cache)
        x = self.ffn_norm.add_norm(h, a)
        self.feed_forward.defer_out = self.defer_pending
        f = self.feed_forward.forward(x, ctx)
        return h, f


# ---------------------------------------------------------------- embedding, head
class TokenEmbedding(Embedding):
    """h[t] = E[id[t]] * scale into the 32-bit stream (src/graph/executor_forward.cu:2786-2797).
    params: vocab_size, hidden_size, scale (default 1)."""

    @classmethod
    def tensor_specs(cls, params):
        return {"weight": TensorSpec((params["vocab_size"], params["hidden_size"]))}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.weight = tensors["weight"]
        self.scale = float(params.get("scale", 1.0))

    def forward(self, token_ids, ctx):
        out = self.rt.empty((token_ids.numel(), self.weight.shape[1]), torch.float32)
        return K.embedding(out, self.weight, token_ids, self.scale, self.rt.status)


class LinearHead(Head):
    """logits = x W^T in 32-bit (src/graph/executor_forward.cu:2953, 3075).
    params: vocab_size, hidden_size.  The weight may be the embedding's own tensor."""

    @classmethod
    def tensor_specs(cls, params):
        return {"weight": TensorSpec((params["vocab_size"], params["hidden_size"]))}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.weight = tensors["weight"]

    def forward(self, x):
        out = self.rt.empty((x.shape[0], self.weight.shape[0]), torch.float32)
        return K.linear(out, x, self.weight)


register_part("norm", "rmsnorm", RMSNorm)
register_part("position", "rotary", RotaryPosition)
register_part("mixer", "gqa_attention", GQAAttention)
register_part("feed_forward", "swiglu", SwiGLU)
register_part("block", "prenorm", PreNormBlock)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
