"""Checkpoint loading for ``flashrec_b200.decoder.Qwen3ForCausalLM``: a mirror of the reference's
``models/weight.py`` (``merge_gate_up_weights`` :19-41, ``merge_qkv_weights`` :44-68, ``load_hf_config``
:71-87, ``load_weights`` :116-263) for the W8A8 model of this package.

A Hugging Face Qwen3 directory holds one ``model.safetensors`` (or shards listed by
``model.safetensors.index.json``) with ``q_proj / k_proj / v_proj`` and ``gate_proj / up_proj`` as separate
matrices; the engine runs them merged (``qkv_proj``, ``gate_up_proj``). Pre-quantised checkpoints carry e4m3
weights with a ``.weight_scale`` (or ``.weight_scale_inv``) tensor per matrix: those are concatenated, never
requantised (``layers/linear.py:96-106``). bf16 / fp16 / fp32 matrices are quantised per output channel at load
when ``quantize_fp8`` is set; without it they are refused, because this package has no bf16 linear layer.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Dict, Iterator, Optional, Tuple

import torch

from flashrec_b200.decoder import Qwen3Config, Qwen3ForCausalLM
from flashrec_b200.layers import as_channel_scale

_FP8 = torch.float8_e4m3fn


def merge_gate_up_weights(
    gate_w: torch.Tensor,
    up_w: torch.Tensor,
    gate_scale: Optional[torch.Tensor] = None,
    up_scale: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``[gate; up]`` along the output dimension; the per-channel scales follow their rows (no scale unless
    both matrices bring one)."""
    if tuple(gate_w.shape) != tuple(up_w.shape):
        raise ValueError(f"gate/up shape mismatch: {tuple(gate_w.shape)} vs {tuple(up_w.shape)}")
    weight = _cat_rows([gate_w, up_w])
    scale = None
    if gate_scale is not None and up_scale is not None:
        n = int(gate_w.shape[0])
        scale = torch.cat([as_channel_scale(gate_scale, n, gate_w.device), as_channel_scale(up_scale, n, up_w.device)])
    return weight, scale


def merge_qkv_weights(
    q_w: torch.Tensor,
    k_w: torch.Tensor,
    v_w: torch.Tensor,
    q_scale: Optional[torch.Tensor] = None,
    k_scale: Optional[torch.Tensor] = None,
    v_scale: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``[q; k; v]`` along the output dimension, scales likewise (only when all three are given)."""
    if q_w.shape[1] != k_w.shape[1] or q_w.shape[1] != v_w.shape[1]:
        raise ValueError(f"qkv in-dim mismatch: {tuple(q_w.shape)} / {tuple(k_w.shape)} / {tuple(v_w.shape)}")
    weight = _cat_rows([q_w, k_w, v_w])
    scale = None
    if q_scale is not None and k_scale is not None and v_scale is not None:
        scale = torch.cat([as_channel_scale(s, int(w.shape[0]), w.device)
                           for s, w in ((q_scale, q_w), (k_scale, k_w), (v_scale, v_w))])
    return weight, scale


def _cat_rows(parts) -> torch.Tensor:
    # torch.cat has no float8 kernel on every build: concatenate the bytes
    if parts[0].dtype == _FP8:
        return torch.cat([p.contiguous().view(torch.uint8) for p in parts], dim=0).view(_FP8)
    return torch.cat(parts, dim=0)


def load_hf_config(model_path: str) -> Qwen3Config:
    """``config.json`` of a Hugging Face Qwen3 directory as a ``Qwen3Config``."""
    cfg = json.loads((Path(model_path) / "config.json").read_text(encoding="utf-8"))
    return Qwen3Config(
        hidden_size=int(cfg["hidden_size"]),
        intermediate_size=int(cfg["intermediate_size"]),
        num_hidden_layers=int(cfg["num_hidden_layers"]),
        num_attention_heads=int(cfg["num_attention_heads"]),
        num_key_value_heads=int(cfg["num_key_value_heads"]),
        head_dim=int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]),
        vocab_size=int(cfg["vocab_size"]),
        rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-6)),
        rope_theta=float(cfg.get("rope_theta", 1000000)),
        max_position_embeddings=int(cfg.get("max_position_embeddings", 40960)),
    )


def iter_safetensors(model_path: str, key_filter: Optional[Callable[[str], bool]] = None) -> Iterator[Tuple[str, torch.Tensor]]:
    """``(key, tensor)`` of every shard; ``key_filter`` is applied before a tensor is read, so the pass over
    the scales does not read the matrices."""
    from safetensors import safe_open

    root = Path(model_path)
    index = root / "model.safetensors.index.json"
    if index.is_file():
        files = sorted(set(json.loads(index.read_text())["weight_map"].values()))
    else:
        files = ["model.safetensors"] if (root / "model.safetensors").is_file() else []
    for name in files:
        with safe_open(str(root / name), framework="pt", device="cpu") as f:
            for key in f.keys():
                if key_filter is None or key_filter(key):
                    yield key, f.get_tensor(key)


def _is_scale_key(key: str) -> bool:
    return key.endswith(".weight_scale") or key.endswith(".weight_scale_inv")


def load_weights(
    model: Qwen3ForCausalLM,
    model_path: str,
    device,
    compute_dtype: torch.dtype = torch.bfloat16,
    quantize_fp8: bool = False,
) -> None:
    """Fill ``model`` from the checkpoint directory: embedding, norms, the merged qkv and gate_up matrices,
    o_proj and down_proj (with their checkpoint scales when the matrices are e4m3), ``lm_head_weight`` (tied to
    the embedding when the checkpoint has none). Afterwards the gate_up weight is laid out for the SwiGLU
    epilogue (``Qwen3MLP.prepare_fused``). Keys that name nothing in the model are ignored, as the reference does."""
    device = torch.device(device)
    if compute_dtype != torch.bfloat16:
        raise NotImplementedError("flashrec_b200 runs bf16 activations only")
    scales: Dict[str, torch.Tensor] = {}
    for key, tensor in iter_safetensors(model_path, key_filter=_is_scale_key):
        if key.startswith("model.layers."):
            scales[key[len("model."):].rsplit(".", 1)[0]] = tensor.to(device=device)
    pending_qkv: Dict[int, Dict[str, torch.Tensor]] = {}
    pending_gu: Dict[int, Dict[str, torch.Tensor]] = {}
    lm_head = None

    def load_linear(lin, w: torch.Tensor, scale: Optional[torch.Tensor]) -> None:
        if w.dtype != _FP8 and w.dtype != compute_dtype:
            w = w.to(dtype=compute_dtype)
        lin.load(w, quantize_fp8=quantize_fp8 and w.dtype != _FP8, weight_scale=scale)

    def norm_weight(t: torch.Tensor) -> torch.Tensor:
        return t.to(device=device, dtype=compute_dtype).contiguous()

    for key, t in iter_safetensors(model_path, key_filter=lambda k: not _is_scale_key(k)):
        if key == "model.embed_tokens.weight":
            model.embed_tokens = t.to(device=device, dtype=compute_dtype).contiguous()
        elif key == "lm_head.weight":
            lm_head = t.to(device=device, dtype=compute_dtype).contiguous()
        elif key == "model.norm.weight":
            model.norm.weight = norm_weight(t)
        elif key.startswith("model.layers.") and key.endswith(".weight"):
            layer_s, _, tail = key[len("model.layers."):].partition(".")
            li = int(layer_s)
            if li >= len(model.layers):
                continue
            layer, name = model.layers[li], tail[: -len(".weight")]
            if name in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"):
                pending_qkv.setdefault(li, {})[name.rsplit(".", 1)[1]] = t.to(device=device)
            elif name in ("mlp.gate_proj", "mlp.up_proj"):
                pending_gu.setdefault(li, {})[name.rsplit(".", 1)[1]] = t.to(device=device)
            elif name == "self_attn.o_proj":
                load_linear(layer.self_attn.o_proj, t.to(device=device), scales.get(f"layers.{li}.{name}"))
            elif name == "mlp.down_proj":
                load_linear(layer.mlp.down_proj, t.to(device=device), scales.get(f"layers.{li}.{name}"))
            elif name == "input_layernorm":
                layer.input_layernorm.weight = norm_weight(t)
            elif name == "post_attention_layernorm":
                layer.post_attention_layernorm.weight = norm_weight(t)
            elif name == "self_attn.q_norm":
                layer.self_attn.q_norm.weight = norm_weight(t)
            elif name == "self_attn.k_norm":
                layer.self_attn.k_norm.weight = norm_weight(t)

    for li, parts in pending_qkv.items():
        if any(p not in parts for p in ("q_proj", "k_proj", "v_proj")):
            continue  # incomplete: the layer keeps what it had, as the reference (which logs a warning)
        pre = f"layers.{li}.self_attn."
        w, s = merge_qkv_weights(parts["q_proj"], parts["k_proj"], parts["v_proj"], scales.get(pre + "q_proj"),
                                 scales.get(pre + "k_proj"), scales.get(pre + "v_proj"))
        load_linear(model.layers[li].self_attn.qkv_proj, w, s)
    for li, parts in pending_gu.items():
        if "gate_proj" not in parts or "up_proj" not in parts:
            continue
        pre = f"layers.{li}.mlp."
        w, s = merge_gate_up_weights(parts["gate_proj"], parts["up_proj"], scales.get(pre + "gate_proj"),
                                     scales.get(pre + "up_proj"))
        mlp = model.layers[li].mlp
        load_linear(mlp.gate_up_proj, w, s)
        mlp.prepare_fused(free_unfused=False)
    model.lm_head_weight = lm_head if lm_head is not None else model.embed_tokens
