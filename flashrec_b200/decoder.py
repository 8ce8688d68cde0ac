"""Host-side call order of one Qwen3 decode step on the FP8 path — a mirror of
``Qwen3Attention / Qwen3MLP / Qwen3DecoderLayer / Qwen3ForCausalLM``
(models/qwen3.py:36-273); ``ForwardBatch`` (core.py:81-101) is re-exported from ``flashrec_b200.core``. Every
arithmetic step is one call into the sm_100a library; this file only sequences
them and owns the weights.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import List, Optional

import torch

from flashrec_b200._lib import call, ptr, stream_ptr
from flashrec_b200.attention import AttentionBackend, TokenToKVPool
from flashrec_b200.core import ForwardBatch
from flashrec_b200.kernel.qk_rope_kv import fp8_qkv_mm_norm_rope_store, fused_qk_norm_rope_store_fp8
from flashrec_b200.kernel.sglops import (fp8_scaled_mm_silu_mul, interleave_gate_up, per_token_quant_fp8,
                                         quant_known_amax_fp8)
from flashrec_b200.kernel.silu_fp8 import silu_and_mul_per_token_quant_fp8
from flashrec_b200.layers import Linear, RMSNorm, RotaryEmbedding


@dataclass
class Qwen3Config:
    hidden_size: int = 2048
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 6144
    num_hidden_layers: int = 28
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position_embeddings: int = 8192
    vocab_size: int = 151936 + 24576


class Qwen3Attention:
    def __init__(self, cfg: Qwen3Config, layer_id: int, attn: AttentionBackend, rotary: RotaryEmbedding, device=None):
        self.layer_id = layer_id
        self.head_dim = cfg.head_dim
        self.num_qo = cfg.num_attention_heads
        self.num_kv = cfg.num_key_value_heads
        self.qkv_proj = Linear(cfg.hidden_size, (self.num_qo + 2 * self.num_kv) * cfg.head_dim)
        self.o_proj = Linear(self.num_qo * cfg.head_dim, cfg.hidden_size)
        self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, device=device)
        self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, device=device)
        self.attn = attn
        self.rotary = rotary
        # run QK-norm + RoPE + the FP8 KV write inside the qkv GEMM's epilogue (same bits as the
        # reference's call order qkv_proj -> fused_qk_norm_rope_store_fp8, which stays as the other branch)
        self.fuse_rope_gemm = False
        self.fuse_rope_min_rows = 2048

    def forward(self, x, batch: ForwardBatch, *, q_fp8, a_scale, residual_inout=None) -> torch.Tensor:
        """``residual_inout``: the o_proj GEMM adds its output to this bf16 residual stream in place
        (and returns it) instead of returning the projection."""
        t = int(q_fp8.shape[0])
        pool = self.attn.kv_pool
        # (worth it from a few thousand rows on; below that the two separate kernels are faster)
        if self.fuse_rope_gemm and t >= self.fuse_rope_min_rows and self.head_dim == 128 and self.num_qo % 2 == 0 \
                and self.num_kv % 2 == 0 and self.qkv_proj.bias is None:
            # norm + RoPE + KV write in the qkv GEMM's epilogue: the qkv matrix is never materialised
            q = fp8_qkv_mm_norm_rope_store(
                q_fp8, self.qkv_proj._fp8_weight, a_scale, self.qkv_proj._fp8_scale, batch.positions,
                batch.out_cache_loc, self.q_norm.weight, self.k_norm.weight, self.q_norm.eps,
                self.rotary.cos_sin_cache, pool.k[self.layer_id], pool.v[self.layer_id], self.num_qo, self.num_kv)
            o = self.attn.forward(q, None, None, self.layer_id, batch, skip_store=True)
            if residual_inout is not None:
                o_fp8, o_scale = per_token_quant_fp8(o.reshape(t, -1))
                return self.o_proj.forward_fp8_add_(o_fp8, o_scale, residual_inout)
            return self.o_proj(o.reshape(t, -1))
        qkv = self.qkv_proj.forward_fp8(q_fp8, a_scale, (t, self.qkv_proj.in_features), torch.bfloat16)
        heads = qkv.view(t, self.num_qo + 2 * self.num_kv, self.head_dim)
        q = heads[:, : self.num_qo]
        k = heads[:, self.num_qo : self.num_qo + self.num_kv]
        v = heads[:, self.num_qo + self.num_kv :]
        fused_qk_norm_rope_store_fp8(
            q, k, v, batch.positions, batch.out_cache_loc, self.q_norm.weight, self.k_norm.weight,
            self.q_norm.eps, self.rotary.cos_sin_cache, pool.k[self.layer_id], pool.v[self.layer_id],
        )
        # the attention kernel reads the strided q view directly (no .contiguous() copy)
        o = self.attn.forward(q, k, v, self.layer_id, batch, skip_store=True)
        if residual_inout is not None:
            o_fp8, o_scale = per_token_quant_fp8(o.reshape(t, -1))
            return self.o_proj.forward_fp8_add_(o_fp8, o_scale, residual_inout)
        return self.o_proj(o.reshape(t, -1))


class Qwen3MLP:
    """``fuse_silu_gemm``: run SwiGLU inside the gate_up GEMM epilogue (weight rows
    interleaved once at load time); the result is bit-identical to the reference's
    call order gate_up GEMM -> silu_and_mul_per_token_quant_fp8, which is kept
    as the unfused branch."""

    def __init__(self, cfg: Qwen3Config, fuse_silu_gemm: bool = True):
        self.gate_up_proj = Linear(cfg.hidden_size, 2 * cfg.intermediate_size)
        self.down_proj = Linear(cfg.intermediate_size, cfg.hidden_size)
        self.fuse_silu_gemm = bool(fuse_silu_gemm) and cfg.intermediate_size % 128 == 0
        self._gu_w: Optional[torch.Tensor] = None
        self._gu_s: Optional[torch.Tensor] = None

    def prepare_fused(self, free_unfused: bool = False) -> None:
        """Build the interleaved gate_up weight from the loaded ``gate_up_proj``."""
        if not self.fuse_silu_gemm:
            return
        w_nk = self.gate_up_proj._fp8_weight.t()
        self._gu_w, self._gu_s = interleave_gate_up(w_nk, self.gate_up_proj._fp8_scale)
        if free_unfused:
            self.gate_up_proj._fp8_weight = None
            self.gate_up_proj._fp8_scale = None

    def forward(self, x, *, q_fp8, a_scale, residual_inout=None) -> torch.Tensor:
        """``residual_inout``: the down_proj GEMM adds its output to this bf16 residual stream in
        place (and returns it) instead of returning the projection."""
        rows = int(q_fp8.shape[0])
        if self.fuse_silu_gemm and self._gu_w is not None:
            y, amax = fp8_scaled_mm_silu_mul(q_fp8, self._gu_w, a_scale, self._gu_s)
            y_fp8, y_scale = quant_known_amax_fp8(y, amax)
        else:
            gu = self.gate_up_proj.forward_fp8(q_fp8, a_scale, (rows, self.gate_up_proj.in_features), torch.bfloat16)
            y_fp8, y_scale = silu_and_mul_per_token_quant_fp8(gu)
        if residual_inout is not None:
            return self.down_proj.forward_fp8_add_(y_fp8, y_scale, residual_inout)
        return self.down_proj.forward_fp8(y_fp8, y_scale, (rows, self.down_proj.in_features), torch.bfloat16)


class Qwen3DecoderLayer:
    def __init__(self, cfg: Qwen3Config, layer_id: int, attn: AttentionBackend, rotary: RotaryEmbedding, device=None):
        self.self_attn = Qwen3Attention(cfg, layer_id, attn, rotary, device=device)
        self.mlp = Qwen3MLP(cfg)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device=device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device=device)

    def forward_fused_residual(self, residual, batch: ForwardBatch):
        """The same layer with the residual adds folded into the o_proj and down_proj GEMM
        epilogues: ``residual`` (bf16 [T, hidden]) holds x + residual of the unfused flow on entry
        and on exit, is updated in place, and each norm reads it without an add. Bit-identical
        to ``forward`` (the GEMM output is rounded to bf16 before the bf16 add in both)."""
        q_fp8, a_scale = self.input_layernorm.quant_fp8(residual)
        self.self_attn.forward(None, batch, q_fp8=q_fp8, a_scale=a_scale, residual_inout=residual)
        q_fp8, a_scale = self.post_attention_layernorm.quant_fp8(residual)
        self.mlp.forward(None, q_fp8=q_fp8, a_scale=a_scale, residual_inout=residual)
        return residual

    def forward(self, x, residual, batch: ForwardBatch):
        """FP8 branch of Qwen3DecoderLayer.forward (models/qwen3.py:198-215)."""
        if residual is None:
            residual = x
            q_fp8, a_scale = self.input_layernorm.quant_fp8(x)
        else:
            q_fp8, a_scale, residual = self.input_layernorm.quant_fp8(x, residual)
        hidden = self.self_attn.forward(x, batch, q_fp8=q_fp8, a_scale=a_scale)
        q_fp8, a_scale, residual = self.post_attention_layernorm.quant_fp8(hidden, residual)
        hidden = self.mlp.forward(hidden, q_fp8=q_fp8, a_scale=a_scale)
        return hidden, residual


class Qwen3ForCausalLM:
    """Embedding -> layers -> final (add+)RMSNorm; returns the normalised hidden
    states, which the SID head consumes (models/qwen3.py:227-273)."""

    def __init__(self, cfg: Qwen3Config, attn: AttentionBackend, device, fuse_residual: bool = True,
                 fuse_rope_gemm: bool = True):
        self.cfg = cfg
        self.device = torch.device(device)
        # fold the residual adds into the o_proj / down_proj GEMM epilogues (same bits, one HBM
        # pass over the residual stream less per norm)
        self.fuse_residual = bool(fuse_residual)
        self.rotary = RotaryEmbedding(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_theta, device=device)
        self.layers: List[Qwen3DecoderLayer] = [
            Qwen3DecoderLayer(cfg, i, attn, self.rotary, device=device) for i in range(cfg.num_hidden_layers)
        ]
        for layer in self.layers:
            layer.self_attn.fuse_rope_gemm = bool(fuse_rope_gemm)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device=device)
        self.embed_tokens: Optional[torch.Tensor] = None  # bf16 [vocab, hidden]
        self.lm_head_weight: Optional[torch.Tensor] = None  # bf16 [vocab, hidden]; the embedding when tied
        self.attn = attn

    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        ids = input_ids.reshape(-1).to(torch.int64)
        out = torch.empty((ids.numel(), self.cfg.hidden_size), dtype=torch.bfloat16, device=ids.device)
        call("fr_embedding_bf16", ptr(self.embed_tokens), ptr(ids), ptr(out), ids.numel(), self.cfg.hidden_size,
             int(self.embed_tokens.shape[0]), stream_ptr(ids.device))
        return out

    def forward(self, batch: ForwardBatch) -> torch.Tensor:
        x = self.embed(batch.input_ids)
        if self.fuse_residual and self.layers:
            residual = x  # the embedding output is this wave's residual stream, updated in place
            for layer in self.layers:
                layer.forward_fused_residual(residual, batch)
            return self.norm(residual)
        residual = None
        for layer in self.layers:
            x, residual = layer.forward(x, residual, batch)
        if residual is None:
            return self.norm(x)
        x, _ = self.norm(x, residual)
        return x

    def last_token_hidden(self, hidden: torch.Tensor, batch: ForwardBatch) -> torch.Tensor:
        """Rows of ``hidden`` that feed the head: all of them for a decode batch, each request's
        last extend token for a prefill batch (ModelEngine.last_token_hidden, engine/engine.py:286-303).
        The offsets come from ``qo_indptr`` on the device when the batch has it (nothing is staged from
        the host), else from the host list ``extend_seq_lens`` as in the reference."""
        if not batch.is_prefill or not batch.extend_seq_lens:
            return hidden
        qo = getattr(batch, "qo_indptr", None)
        if qo is not None:
            idx = (qo[1:] - 1).to(torch.int64)
        else:
            offs = [o - 1 for o in itertools.accumulate(int(x) for x in batch.extend_seq_lens)]
            idx = torch.tensor(offs, dtype=torch.int64).to(hidden.device, non_blocking=True)
        out = torch.empty((idx.numel(), hidden.shape[1]), dtype=torch.bfloat16, device=hidden.device)
        call("fr_embedding_bf16", ptr(hidden), ptr(idx), ptr(out), idx.numel(), int(hidden.shape[1]),
             int(hidden.shape[0]), stream_ptr(hidden.device))
        return out

    # -- random initialisation used by the benchmark / tests --------------------
    def init_random(self, seed: int = 0, std: float = 0.02, embed: bool = True) -> None:
        """N(0, std) weights quantised per channel; norm weights = 1."""
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        cfg = self.cfg

        def rnd(n, k):
            return torch.randn((n, k), generator=g, device=self.device, dtype=torch.float32) * std

        for layer in self.layers:
            a = layer.self_attn
            a.qkv_proj.load(rnd(a.qkv_proj.out_features, cfg.hidden_size), quantize_fp8=True)
            a.o_proj.load(rnd(cfg.hidden_size, a.o_proj.in_features), quantize_fp8=True)
            layer.mlp.gate_up_proj.load(rnd(2 * cfg.intermediate_size, cfg.hidden_size), quantize_fp8=True)
            layer.mlp.down_proj.load(rnd(cfg.hidden_size, cfg.intermediate_size), quantize_fp8=True)
            layer.mlp.prepare_fused(free_unfused=True)
        if embed:
            self.embed_tokens = (
                torch.randn((cfg.vocab_size, cfg.hidden_size), generator=g, device=self.device, dtype=torch.float32)
                * std
            ).to(torch.bfloat16)
