"""Model glue for the layer-sliding runtime: which modules form a layer unit, what each decoder
layer is called with, and the size bookkeeping the engine needs.

Counterpart of the reference's utils/model_compat.py for the dense decoder-only families the
benchmark configs name (Llama-style models through `get_decoder()`, and GPT-2).  Attention,
rotary embeddings and the layers themselves are the Hugging Face modules, as in the reference.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional

import torch
import torch.nn as nn


class GPT2Embedding(nn.Module):
    """Token + learned position embedding as one layer unit.  (The reference's embedding unit
    calls only the token embedding, transformer_layer.py:570-582, so its GPT path drops the
    positions; here they are part of the unit and are trained with it.)"""

    def __init__(self, wte: nn.Embedding, wpe: nn.Embedding, drop: Optional[nn.Module] = None):
        super().__init__()
        self.wte, self.wpe, self.drop = wte, wpe, drop

    def forward(self, input_ids, position_ids=None):
        if position_ids is None:
            position_ids = torch.arange(input_ids.shape[1], device=input_ids.device).unsqueeze(0)
        h = self.wte(input_ids) + self.wpe(position_ids)
        return self.drop(h) if self.drop is not None else h


@dataclass
class TextModelParts:
    """The pieces the engine streams: embedding unit, decoder layers, final norm, output head."""
    model: Any
    config: Any
    kind: str                      # "gpt2" or "decoder"
    embed: nn.Module
    layers: nn.ModuleList
    norm: nn.Module
    lm_head: nn.Module
    rotary_emb: Optional[nn.Module]
    tied_param: Optional[nn.Parameter]


def split_parts(model) -> TextModelParts:
    cfg = model.config
    if getattr(cfg, "is_encoder_decoder", False):
        raise ValueError("Only decoder-only text training is supported")
    if getattr(cfg, "model_type", "") == "gpt2":
        tr = model.transformer
        drop = tr.drop if getattr(tr.drop, "p", 0.0) > 0 else None
        embed = GPT2Embedding(tr.wte, tr.wpe, drop)
        parts = TextModelParts(model, cfg, "gpt2", embed, tr.h, tr.ln_f, model.lm_head, None, None)
        in_w = tr.wte.weight
    else:
        dec = model.get_decoder()
        if not hasattr(dec, "layers") or not hasattr(dec, "norm"):
            raise ValueError("The text decoder must expose layers and norm")  # utils/model_compat.py:88-89
        parts = TextModelParts(model, cfg, "decoder", model.get_input_embeddings(), dec.layers, dec.norm,
                               model.get_output_embeddings(), getattr(dec, "rotary_emb", None), None)
        in_w = model.get_input_embeddings().weight
    if parts.lm_head.weight is in_w:
        parts.tied_param = in_w
    return parts


def validate_model(model) -> TextModelParts:
    """Every parameter must belong to exactly one streamed unit (utils/model_compat.py:80-96)."""
    parts = split_parts(model)
    managed = {id(p) for mod in (parts.embed, *parts.layers, parts.norm, parts.lm_head) for p in mod.parameters()}
    extra = [n for n, p in model.named_parameters() if id(p) not in managed]
    if extra:
        raise ValueError(f"Parameters outside the text layer layout: {extra}")
    return parts


def parameter_sizes(model):
    """Largest unit size and total unique parameter count (utils/model_compat.py:99-107).  The
    output unit's size includes a tied weight, which it reads but does not own."""
    parts = split_parts(model)
    sizes = [sum(p.numel() for p in m.parameters()) for m in (parts.embed, *parts.layers)]
    sizes.append(sum(p.numel() for p in parts.norm.parameters()) + sum(p.numel() for p in parts.lm_head.parameters()))
    return max(sizes), sum(p.numel() for p in model.parameters())


def prepare_layer_inputs(parts: TextModelParts, hidden_states, attention_mask=None, position_ids=None) -> List[dict]:
    """Per-layer keyword arguments (utils/model_compat.py:124-164, the dense branch).  With no
    padding mask the layers get attention_mask=None and SDPA runs its causal fast path."""
    seq = hidden_states.shape[1]
    cache_position = torch.arange(seq, device=hidden_states.device)
    if position_ids is None:
        position_ids = cache_position.unsqueeze(0)
    mask = None
    if attention_mask is not None and not bool(attention_mask.all()):
        from transformers.masking_utils import create_causal_mask
        mask = create_causal_mask(config=parts.config, inputs_embeds=hidden_states, attention_mask=attention_mask,
                                  cache_position=cache_position, past_key_values=None, position_ids=position_ids)
    if parts.kind == "gpt2":
        return [dict(attention_mask=mask, use_cache=False) for _ in parts.layers]
    positions = parts.rotary_emb(hidden_states, position_ids) if parts.rotary_emb is not None else None
    return [dict(attention_mask=mask, position_ids=position_ids, position_embeddings=positions, use_cache=False)
            for _ in parts.layers]


def call_decoder_layer(layer, hidden_states, layer_kwargs):
    out = layer(hidden_states, **layer_kwargs)
    return out[0] if isinstance(out, tuple) else out


# ---- synthetic models of the benchmark configs (random init, no checkpoints needed) -------------
MODEL_SPECS = {
    "gpt2-small": dict(family="gpt2", n_layer=12, n_embd=768, n_head=12, vocab_size=50257, n_positions=1024),
    "gpt2-tiny": dict(family="gpt2", n_layer=2, n_embd=64, n_head=4, vocab_size=211, n_positions=64),
    "llama3.1-8b": dict(family="llama", num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                        num_key_value_heads=8, intermediate_size=14336, vocab_size=128256, rope_theta=500000.0,
                        max_position_embeddings=8192),
    "llama3.1-70b": dict(family="llama", num_hidden_layers=80, hidden_size=8192, num_attention_heads=64,
                         num_key_value_heads=8, intermediate_size=28672, vocab_size=128256, rope_theta=500000.0,
                         max_position_embeddings=8192),
    "llama-tiny": dict(family="llama", num_hidden_layers=3, hidden_size=64, num_attention_heads=4,
                       num_key_value_heads=2, intermediate_size=160, vocab_size=199, rope_theta=500000.0,
                       max_position_embeddings=128),
}


def build_random_model(name: str, device, dtype=torch.bfloat16, seed: int = 0, attn_implementation: str = "sdpa",
                       num_layers: Optional[int] = None, meta: bool = False):
    """Random-init model of a named architecture, created directly on `device` in `dtype`.
    meta=True builds only the module skeleton (parameters on the meta device); the engine then
    creates every unit's weights in place, so a model larger than one GPU never exists whole."""
    spec = dict(MODEL_SPECS[name])
    family = spec.pop("family")
    if num_layers is not None:
        spec["n_layer" if family == "gpt2" else "num_hidden_layers"] = num_layers
    torch.manual_seed(seed)
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device("meta" if meta else device):
            if family == "gpt2":
                from transformers import GPT2Config, GPT2LMHeadModel
                # "gelu_pytorch_tanh" is GPT-2's tanh-approximated GELU (HF's default "gelu_new") as one
                # fused kernel instead of eight elementwise ones
                cfg = GPT2Config(resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0, attn_implementation=attn_implementation,
                                 use_cache=False, activation_function="gelu_pytorch_tanh", **spec)
                model = GPT2LMHeadModel(cfg)
            else:
                from transformers import LlamaConfig, LlamaForCausalLM
                cfg = LlamaConfig(rms_norm_eps=1e-5, tie_word_embeddings=False, attention_dropout=0.0,
                                  attn_implementation=attn_implementation, use_cache=False, **spec)
                model = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(old)
    if meta and family != "gpt2":
        dec = model.get_decoder()
        if getattr(dec, "rotary_emb", None) is not None:   # its frequency table is a buffer, not a parameter
            dec.rotary_emb = type(dec.rotary_emb)(config=cfg, device=device)
    return model
