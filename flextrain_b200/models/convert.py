"""Weight-name converters between this package's models and the Hugging Face
``transformers`` layouts of the same architectures (``LlamaForCausalLM``,
``GPT2LMHeadModel``), for ``engine.import_state_dict`` / ``export_state_dict``.

The reference has no model and therefore no converters; its users move weights
with Megatron's own tools.  Differences bridged here: q / k / v and gate / up
projections are stored fused in this package (one GEMM each); GPT-2's ``Conv1D``
keeps weights ``[in, out]`` where ``linear`` here keeps ``[out, in]``.  Rotary
embeddings need no permutation: both sides pair element ``i`` with ``i + D/2``.
"""
from __future__ import annotations

from typing import Dict

import torch

from .gpt import GPTConfig
from .llama import LlamaConfig


# ------------------------------------------------------------------- Llama
def llama_config_from_hf(hf) -> LlamaConfig:
    """``hf``: a ``transformers.LlamaConfig`` (or anything with its attributes)."""
    return LlamaConfig(num_layers=hf.num_hidden_layers, hidden=hf.hidden_size,
                       num_heads=hf.num_attention_heads,
                       num_kv_heads=getattr(hf, "num_key_value_heads", None) or hf.num_attention_heads,
                       ffn=hf.intermediate_size, vocab=hf.vocab_size, eps=hf.rms_norm_eps,
                       rope_theta=float(getattr(hf, "rope_theta", None)
                                        or (getattr(hf, "rope_parameters", None) or {}).get("rope_theta", 10000.0)),
                       seq_len=hf.max_position_embeddings, name="hf-llama")


def llama_from_hf(sd: Dict[str, torch.Tensor], cfg: LlamaConfig) -> Dict[str, torch.Tensor]:
    out = {"embed": sd["model.embed_tokens.weight"], "final_norm": sd["model.norm.weight"],
           # checkpoints with a tied head carry no lm_head tensor
           "lm_head": sd.get("lm_head.weight", sd["model.embed_tokens.weight"])}
    for i in range(cfg.num_layers):
        hf, me = f"model.layers.{i}.", f"blocks.{i}."
        out[me + "attn_norm"] = sd[hf + "input_layernorm.weight"]
        out[me + "wqkv"] = torch.cat([sd[hf + f"self_attn.{n}_proj.weight"] for n in "qkv"], dim=0)
        out[me + "wo"] = sd[hf + "self_attn.o_proj.weight"]
        out[me + "ffn_norm"] = sd[hf + "post_attention_layernorm.weight"]
        out[me + "w_gate_up"] = torch.cat([sd[hf + "mlp.gate_proj.weight"], sd[hf + "mlp.up_proj.weight"]], dim=0)
        out[me + "w_down"] = sd[hf + "mlp.down_proj.weight"]
    return out


def llama_to_hf(sd: Dict[str, torch.Tensor], cfg: LlamaConfig) -> Dict[str, torch.Tensor]:
    q, kv = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    out = {"model.embed_tokens.weight": sd["embed"], "model.norm.weight": sd["final_norm"],
           "lm_head.weight": sd["lm_head"]}
    for i in range(cfg.num_layers):
        hf, me = f"model.layers.{i}.", f"blocks.{i}."
        out[hf + "input_layernorm.weight"] = sd[me + "attn_norm"]
        wq, wk, wv = sd[me + "wqkv"].split([q, kv, kv], dim=0)
        out[hf + "self_attn.q_proj.weight"], out[hf + "self_attn.k_proj.weight"] = wq, wk
        out[hf + "self_attn.v_proj.weight"] = wv
        out[hf + "self_attn.o_proj.weight"] = sd[me + "wo"]
        out[hf + "post_attention_layernorm.weight"] = sd[me + "ffn_norm"]
        gate, up = sd[me + "w_gate_up"].split(cfg.ffn, dim=0)
        out[hf + "mlp.gate_proj.weight"], out[hf + "mlp.up_proj.weight"] = gate, up
        out[hf + "mlp.down_proj.weight"] = sd[me + "w_down"]
    return out


# -------------------------------------------------------------------- GPT-2
def gpt2_config_from_hf(hf) -> GPTConfig:
    """``hf``: a ``transformers.GPT2Config``.  Its ``gelu_new`` activation is the
    tanh GELU used here; any other activation is refused."""
    act = getattr(hf, "activation_function", "gelu_new")
    if act not in ("gelu_new", "gelu_pytorch_tanh"):
        raise ValueError(f"activation '{act}' is not the tanh GELU of models.gpt")
    return GPTConfig(num_layers=hf.n_layer, hidden=hf.n_embd, num_heads=hf.n_head,
                     ffn=hf.n_inner or 4 * hf.n_embd, vocab=hf.vocab_size, seq_len=hf.n_positions,
                     eps=hf.layer_norm_epsilon, tie_embeddings=True, dropout=float(hf.resid_pdrop),
                     name="hf-gpt2")


_GPT2_PAIRS = (("ln_1.weight", "ln1_w", False), ("ln_1.bias", "ln1_b", False),
               ("attn.c_attn.weight", "wqkv", True), ("attn.c_attn.bias", "bqkv", False),
               ("attn.c_proj.weight", "wo", True), ("attn.c_proj.bias", "bo", False),
               ("ln_2.weight", "ln2_w", False), ("ln_2.bias", "ln2_b", False),
               ("mlp.c_fc.weight", "w_fc", True), ("mlp.c_fc.bias", "b_fc", False),
               ("mlp.c_proj.weight", "w_proj", True), ("mlp.c_proj.bias", "b_proj", False))


def gpt2_from_hf(sd: Dict[str, torch.Tensor], cfg: GPTConfig) -> Dict[str, torch.Tensor]:
    pre = "transformer." if "transformer.wte.weight" in sd else ""
    out = {"wte": sd[pre + "wte.weight"], "wpe": sd[pre + "wpe.weight"],
           "lnf_w": sd[pre + "ln_f.weight"], "lnf_b": sd[pre + "ln_f.bias"]}
    if not cfg.tie_embeddings:
        out["lm_head"] = sd.get("lm_head.weight", sd[pre + "wte.weight"])
    for i in range(cfg.num_layers):
        for hf_name, mine, transpose in _GPT2_PAIRS:
            t = sd[f"{pre}h.{i}.{hf_name}"]
            out[f"blocks.{i}.{mine}"] = t.t().contiguous() if transpose else t
    return out


def gpt2_to_hf(sd: Dict[str, torch.Tensor], cfg: GPTConfig) -> Dict[str, torch.Tensor]:
    out = {"transformer.wte.weight": sd["wte"], "transformer.wpe.weight": sd["wpe"],
           "transformer.ln_f.weight": sd["lnf_w"], "transformer.ln_f.bias": sd["lnf_b"],
           "lm_head.weight": sd["wte"] if cfg.tie_embeddings else sd["lm_head"]}
    for i in range(cfg.num_layers):
        for hf_name, mine, transpose in _GPT2_PAIRS:
            t = sd[f"blocks.{i}.{mine}"]
            out[f"transformer.h.{i}.{hf_name}"] = t.t().contiguous() if transpose else t
    return out
