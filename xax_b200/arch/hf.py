"""Loading HuggingFace-format checkpoints into the LLM of this path (xax/arch/llm.py:978-1416).

The reference downloads a repository and maps its safetensors into the module tree; here the
"repository" is a local directory holding ``config.json`` and ``*.safetensors`` (there is no network
path).  Names, fall-backs and placement follow the reference: ``embed_tokens`` / ``wte``,
``layers.{i}.self_attn.{q,k,v,o}_proj``, ``layers.{i}.mlp.{gate,up,down}_proj``, ``input_layernorm`` /
``post_attention_layernorm``, ``norm`` / ``ln_f``, each with or without the ``model.`` prefix; a
checkpoint without ``lm_head.weight`` ties the head to the embedding.  Under tensor parallelism every
rank keeps its slice per get_model_parallel_sharding_spec.  Weights are stored as bf16; the FP8 layers
quantise them to e4m3 once, on first use.
"""

from __future__ import annotations

import json
import os

import torch

from ..nn.fp8 import Fp8Linear
from .attention import Embedding, Linear, RMSNorm, RotaryEmbedding, SelfAttentionBlock, SwiGLU, TransformerBlock
from .llm import LLM, LLMConfig, tie_embedding_and_head, tp_shard_dim

BF16 = torch.bfloat16

# field -> accepted names in a HuggingFace config.json (xax/arch/llm.py:1027-1085)
_ALIASES = {
    "hidden_size": ("hidden_size", "n_embd"),
    "num_attention_heads": ("num_attention_heads", "n_head"),
    "num_key_value_heads": ("num_key_value_heads", "num_kv_heads", "n_kv_head"),
    "num_hidden_layers": ("num_hidden_layers", "n_layer"),
    "vocab_size": ("vocab_size", "n_vocab"),
    "intermediate_size": ("intermediate_size", "n_inner", "ffn_hidden_size"),
    "rope_theta": ("rope_theta", "rotary_emb_base"),
    "rms_norm_eps": ("rms_norm_eps", "layer_norm_epsilon"),
    "attention_bias": ("attention_bias",),
    "mlp_bias": ("mlp_bias",),
    "head_dim": ("head_dim",),
    "sliding_window": ("sliding_window", "sliding_window_size"),
    "layer_types": ("layer_types", "sliding_attention_map"),
    "model_type": ("model_type",),
}


def _field(cfg: dict, name: str):
    for alias in _ALIASES[name]:
        if cfg.get(alias) is not None:
            return cfg[alias]
    return None


def _parse_rope_scaling(cfg: dict) -> tuple[float, int | None, float, float]:
    """xax/arch/llm.py:1088-1115: YaRN parameters, identity unless rope_type == "yarn"."""
    rs = cfg.get("rope_scaling")
    if not isinstance(rs, dict) or rs.get("rope_type") != "yarn":
        return 1.0, None, 1.0, 32.0
    factor = float(rs["factor"]) if rs.get("factor") is not None else 1.0
    orig = int(rs["original_max_position_embeddings"]) if rs.get("original_max_position_embeddings") is not None else None
    slow = float(rs["beta_slow"]) if rs.get("beta_slow") is not None else 1.0
    fast = float(rs["beta_fast"]) if rs.get("beta_fast") is not None else 32.0
    return factor, orig, slow, fast


def hf_config_to_llm_config(cfg: dict) -> LLMConfig:
    """xax/arch/llm.py:1118-1188, defaults included (kv heads = q heads // 2, MLP width = 4 x hidden,
    theta 10000, eps 1e-6, QK-norm for the qwen3 family)."""
    for required in ("hidden_size", "num_attention_heads", "num_hidden_layers", "vocab_size"):
        if _field(cfg, required) is None:
            raise ValueError(f"HuggingFace config missing required field: {required}")
    embed_dim = int(_field(cfg, "hidden_size"))
    q_heads = int(_field(cfg, "num_attention_heads"))
    kv_heads = int(_field(cfg, "num_key_value_heads") or max(1, q_heads // 2))
    head_dim = int(_field(cfg, "head_dim") or (embed_dim // q_heads))
    mlp_hidden_dim = int(_field(cfg, "intermediate_size") or (embed_dim * 4))
    factor, orig, slow, fast = _parse_rope_scaling(cfg)
    layer_types = _field(cfg, "layer_types")
    layer_attention_types = tuple(layer_types) if layer_types else None
    return LLMConfig(
        vocab_size=int(_field(cfg, "vocab_size")), embed_dim=embed_dim, q_heads=q_heads, kv_heads=kv_heads,
        head_dim=head_dim, num_layers=int(_field(cfg, "num_hidden_layers")),
        rope_theta=float(_field(cfg, "rope_theta") or 10_000.0), dropout_rate=0.0,
        mlp_mult=max(1, mlp_hidden_dim // embed_dim), mlp_hidden_dim=mlp_hidden_dim,
        rms_eps=float(_field(cfg, "rms_norm_eps") or 1e-6),
        attention_bias=bool(_field(cfg, "attention_bias")) if _field(cfg, "attention_bias") is not None else False,
        mlp_bias=bool(_field(cfg, "mlp_bias")) if _field(cfg, "mlp_bias") is not None else False,
        rope_factor=factor, rope_original_max_position_embeddings=orig, rope_beta_slow=slow, rope_beta_fast=fast,
        sliding_window_size=_field(cfg, "sliding_window"), layer_attention_types=layer_attention_types,
        use_attention_sinks=layer_attention_types is not None,
        use_qk_norm=_field(cfg, "model_type") in ("qwen3", "qwen3_moe"))


def load_hf_config(path: str) -> dict:
    """config.json of a local checkpoint directory."""
    cfg_path = os.path.join(path, "config.json")
    if not os.path.isfile(cfg_path):
        raise FileNotFoundError(f"{cfg_path} not found: checkpoints are read from a local directory (no download)")
    with open(cfg_path) as f:
        return json.load(f)


def _fetch_state_dict(path: str) -> tuple[dict, dict]:
    """(config dict, {tensor name: CPU tensor}) of every *.safetensors file in the directory."""
    from safetensors.torch import load_file

    cfg = load_hf_config(path)
    state: dict[str, torch.Tensor] = {}
    files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no *.safetensors file in {path}")
    for f in files:
        state.update(load_file(os.path.join(path, f)))
    return cfg, state


def _get_weight(state: dict, *names: str) -> torch.Tensor:
    for n in names:
        if n in state:
            return state[n]
    raise KeyError(f"none of {names} found in the checkpoint")


def _get_bias(state: dict, *names: str):
    for n in names:
        if n in state:
            return state[n]
    return None


def load_hf_weights_into_llm(model: LLM, repo_id: str | dict, revision: str | None = None, dtype=None) -> LLM:
    """xax/arch/llm.py:1191-1416.  ``repo_id`` is a local checkpoint directory (or an already loaded
    ``{name: tensor}`` dict); ``model`` supplies the structure (layer types, FP8 or not, tensor-parallel
    rank and size) and is not modified: a new LLM holding the checkpoint's weights is returned."""
    if dtype not in (None, BF16):
        raise ValueError("weights of this path are stored as bf16")
    if revision is not None:
        raise ValueError("revisions belong to the hub; a local directory has one state")
    if isinstance(repo_id, dict):
        cfg, state = None, repo_id
    else:
        cfg, state = _fetch_state_dict(repo_id)
    if cfg is not None and _field(cfg, "hidden_size") not in (None, model.config.embed_dim):
        raise ValueError(f"HF hidden_size {_field(cfg, 'hidden_size')} != model.embed_dim {model.config.embed_dim}")
    dev = model.embed.weight.device
    rank, size = model.tp_rank, model.tp_size

    def place(arr: torch.Tensor, weight_name: str) -> torch.Tensor:
        dim = tp_shard_dim(weight_name, arr.dim())
        if size > 1 and dim is not None:
            n = arr.shape[dim] // size
            arr = arr.narrow(dim, rank * n, n)
        return arr.to(device=dev, dtype=BF16).contiguous()

    def map_linear(layer, w: torch.Tensor, b, weight_name: str):
        full = list(layer.weight.shape)
        dim = tp_shard_dim(weight_name, 2)
        if size > 1 and dim is not None:
            full[dim] *= size
        w_mapped = w if list(w.shape) == full else w.t()
        if list(w_mapped.shape) != full:
            raise ValueError(f"{weight_name}: checkpoint shape {tuple(w.shape)} does not fit {tuple(full)}")
        w_dev = place(w_mapped, weight_name)
        b_dev = None
        if b is not None and not (dim == 1 and rank > 0):  # a row-parallel bias is added once, by rank 0
            b_dev = place(b, weight_name + ".bias")
        if isinstance(layer, Fp8Linear):
            return Fp8Linear(w_dev.shape[1], w_dev.shape[0], weight=w_dev, bias=b_dev, use_bias=b_dev is not None,
                             use_fp8=layer.use_fp8)
        return Linear(w_dev.shape[1], w_dev.shape[0], use_bias=b_dev is not None, weight=w_dev, bias=b_dev)

    def both(prefix: str, name: str) -> tuple[str, str]:
        return f"{prefix}.{name}", f"model.{prefix}.{name}"

    embed_w = _get_weight(state, "embed_tokens.weight", "model.embed_tokens.weight", "wte.weight")
    embed = Embedding(embed_w.shape[0], embed_w.shape[1], weight=embed_w.to(device=dev, dtype=BF16).contiguous())
    blocks = []
    for idx, old in enumerate(model.blocks):
        a, f = old.self_attn, old.feed_forward
        sa, mlp, blk = f"layers.{idx}.self_attn", f"layers.{idx}.mlp", f"layers.{idx}"
        # QK-norm (Qwen3 style): taken when the checkpoint has the weights (:1331-1342), replicated
        qn_w, kn_w = state.get(f"model.{sa}.q_norm.weight"), state.get(f"model.{sa}.k_norm.weight")
        qn = a.q_norm if qn_w is None else RMSNorm(qn_w.to(device=dev, dtype=BF16).contiguous(), model.config.rms_eps)
        kn = a.k_norm if kn_w is None else RMSNorm(kn_w.to(device=dev, dtype=BF16).contiguous(), model.config.rms_eps)

        def proj(layer, prefix, name, tp_name):
            return map_linear(layer, _get_weight(state, *both(prefix, f"{name}.weight")),
                              _get_bias(state, *both(prefix, f"{name}.bias")), tp_name)

        attn = SelfAttentionBlock(
            proj(a.q_proj, sa, "q_proj", "q_proj"), proj(a.k_proj, sa, "k_proj", "k_proj"),
            proj(a.v_proj, sa, "v_proj", "v_proj"), proj(a.output_proj, sa, "o_proj", "o_proj"),
            a.rotary_emb,
            qn, kn, a.sinks, local_window_size=a.local_window_size, num_heads=a.num_heads, num_kv_heads=a.num_kv_heads, head_dim=a.head_dim, causal=a.causal, use_fp8=a.use_fp8)
        ff = SwiGLU(proj(f.gate, mlp, "gate_proj", "gate_proj"), proj(f.up, mlp, "up_proj", "up_proj"),
                    proj(f.down, mlp, "down_proj", "down_proj"))
        pre = _get_weight(state, *both(blk, "input_layernorm.weight"))
        post = _get_weight(state, *both(blk, "post_attention_layernorm.weight"))
        blocks.append(TransformerBlock(attn, ff, RMSNorm(pre.to(device=dev, dtype=BF16).contiguous(), old.attn_norm.eps),
                                       RMSNorm(post.to(device=dev, dtype=BF16).contiguous(), old.mlp_norm.eps),
                                       num_heads=a.num_heads, head_dim=a.head_dim, causal=a.causal, use_fp8=False))
    final = _get_bias(state, "norm.weight", "model.norm.weight", "ln_f.weight")
    norm = model.norm if final is None else RMSNorm(final.to(device=dev, dtype=BF16).contiguous(), model.norm.eps)
    head_keys = [k for k in state if "lm_head.weight" in k]
    if head_keys:
        hw = state[head_keys[0]].to(device=dev, dtype=BF16).contiguous()
        head = Linear(hw.shape[1], hw.shape[0], use_bias=False, weight=hw)
        out = LLM(embed, blocks, norm, head, model.config)
    else:
        out = LLM(embed, blocks, norm, Linear(embed_w.shape[1], embed_w.shape[0], use_bias=False, weight=embed.weight),
                  model.config)
        out = tie_embedding_and_head(out)
    out.tp_rank, out.tp_size = rank, size
    return out


def build_pretrained_llm(repo: str, dtype=None, *, use_cross_attention: bool = False, extra_tokens: int | None = None,
                         tied_extra_embed: bool = False, key=None, use_fp8: bool = True, device=None, tp_rank: int = 0,
                         tp_size: int = 1) -> LLM:
    """xax/arch/llm.py:658-710 for a local checkpoint directory.  ``use_fp8`` (an extension, as in
    LLM.build) makes the projections Fp8Linear layers; the reference reaches the same by swapping
    them into the module tree."""
    if extra_tokens is not None or tied_extra_embed:
        raise ValueError("extra tokens are outside the path this library covers")
    if use_cross_attention and key is None:
        raise ValueError("key is required if use_cross_attention is True or extra_tokens is not None.")  # :691-693
    config = hf_config_to_llm_config(load_hf_config(repo))
    shape = LLM.build(config, key=0 if key is None else key, use_fp8=use_fp8, init_std=0.0, device=device,
                      tp_rank=tp_rank, tp_size=tp_size)
    llm = load_hf_weights_into_llm(shape, repo, dtype=dtype)
    if use_cross_attention:  # :706-708: the cross-attention weights are freshly initialised
        from .llm import CrossAttentionLLM

        return CrossAttentionLLM.from_llm(llm, key=key)
    return llm
