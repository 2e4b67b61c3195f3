"""The ``--model_choice "<hf id>--<TAG>-<TAG>..."`` mini-language.

Behaviour follows the reference's ``get_modified_config`` (optimus/config_utils.py:3-196):

* DeepSeek-V3: ``L`` layers, ``DL`` first_k_dense_replace, ``H`` hidden, ``I`` dense ffn,
  ``MI`` expert ffn, ``A`` heads (and kv heads), ``N`` routed experts, ``K`` top-k,
  ``SE`` shared experts.
* OLMoE: ``L`` layers; multiplicative scales ``SA`` heads, ``SH`` hidden, ``SE`` experts,
  ``SC`` top-k, ``SI`` expert ffn; ``SM`` = SA+SH, ``S`` = SA+SH+SE+SI; flags ``NAL`` (no
  aux loss) and ``SKIPQKNORM``.  ``output_router_logits`` becomes ``not NAL``.
* OLMo: ``L`` layers, ``S`` (parsed, unused as in the reference), ``TWE``, ``RMS``;
  max positions forced to 4096.
* Llama: ``L``, ``H``, ``I``; head_dim re-derived; max positions forced to 4096.

Implemented as a table of per-family tag handlers instead of per-family if-chains; it also
offers ``build_config`` which constructs the family's config offline (the reference calls
``AutoConfig.from_pretrained`` for OLMo/Llama, which needs the HF hub).
"""
from __future__ import annotations

import re
from typing import Callable, Dict, Tuple

OLMOE_IDS = ("allenai/OLMoE-1B-7B-0924",)
OLMO_IDS = ("allenai/OLMo-1B-hf", "allenai/OLMo-7B-hf")
LLAMA_IDS = ("meta-llama/Llama-3.1-8B", "meta-llama/Llama-3.2-1B")
DSV3_IDS = ("deepseek-ai/DeepSeek-V3",)
SUPPORTED_MODEL_IDS = OLMOE_IDS + OLMO_IDS + LLAMA_IDS + DSV3_IDS

_TOKEN = re.compile(r"([A-Z]+)([0-9.]*)")


def split_model_choice(model_choice: str) -> Tuple[str, str | None]:
    parts = model_choice.split("--")
    if len(parts) == 2:
        return parts[0], parts[1]
    return model_choice, None


def model_family(model_choice: str) -> str:
    hf_id, _ = split_model_choice(model_choice)
    if hf_id in OLMOE_IDS:
        return "olmoe"
    if hf_id in OLMO_IDS:
        return "olmo"
    if hf_id in LLAMA_IDS:
        return "llama"
    if hf_id in DSV3_IDS:
        return "deepseek_v3"
    raise ValueError(f"{hf_id} is not supported for parallel model training")


def _parse_tokens(tag_string, valid=None) -> Dict[str, object]:
    """``"SM1.5-L4-NAL"`` -> ``{"SM": "1.5", "L": "4", "NAL": True}``."""
    out: Dict[str, object] = {}
    if not tag_string:
        return out
    for tok in tag_string.split("-"):
        if not tok:
            continue
        m = _TOKEN.match(tok)
        if m is None:
            raise ValueError(f"cannot parse model tag {tok!r}")
        key, val = m.groups()
        if valid is not None:
            assert key in valid, f"{key} should be among {list(valid)}"
        out[key] = val if val != "" else True
    return out


def _apply_dsv3(cfg, tags):
    setters = {
        "L": "num_hidden_layers", "DL": "first_k_dense_replace", "H": "hidden_size",
        "I": "intermediate_size", "MI": "moe_intermediate_size", "N": "n_routed_experts",
        "K": "num_experts_per_tok", "SE": "n_shared_experts",
    }
    req = _parse_tokens(tags)
    for key, attr in setters.items():
        if key in req:
            setattr(cfg, attr, int(req[key]))
    if "A" in req:
        cfg.num_attention_heads = int(req["A"])
    cfg.num_key_value_heads = cfg.num_attention_heads


def _apply_olmoe(cfg, tags):
    valid = ("L", "SA", "SH", "SE", "SC", "SI", "NAL", "SKIPQKNORM", "SM", "S")
    req = _parse_tokens(tags, valid)
    if "S" in req:
        assert not any(k in req for k in ("SA", "SH", "SE", "SI")), \
            "If S is provided, then SA,SH, SI and SE should not be provided"
    if "SM" in req:
        assert not any(k in req for k in ("SA", "SH")), "If SM is provided, then SA and SH should not be provided"
    scale = {"SA": 1.0, "SH": 1.0, "SE": 1.0, "SC": 1.0, "SI": 1.0}
    expands = {"S": ("SA", "SH", "SE", "SI"), "SM": ("SA", "SH")}
    for key, val in req.items():
        if key in expands:
            for k in expands[key]:
                scale[k] = float(val)
        elif key in scale:
            scale[key] = float(val)
    if "L" in req:
        cfg.num_hidden_layers = int(float(req["L"]))
    cfg.num_attention_heads = int(scale["SA"] * cfg.num_attention_heads)
    cfg.num_key_value_heads = int(scale["SA"] * cfg.num_key_value_heads)
    cfg.hidden_size = int(scale["SH"] * cfg.hidden_size)
    cfg.num_experts = int(scale["SE"] * cfg.num_experts)
    cfg.num_experts_per_tok = int(scale["SC"] * cfg.num_experts_per_tok)
    cfg.intermediate_size = int(scale["SI"] * cfg.intermediate_size)
    cfg.output_router_logits = not bool(req.get("NAL", False))
    cfg.skip_qk_norm = bool(req.get("SKIPQKNORM", False))


def _apply_olmo(cfg, tags):
    cfg.max_position_embeddings = 4096
    cfg.tie_word_embeddings = False
    req = _parse_tokens(tags)
    if "L" in req:
        cfg.num_hidden_layers = int(req["L"])
    if "TWE" in req:
        cfg.tie_word_embeddings = True
    if "RMS" in req:
        cfg.use_rms_norm = True


def _apply_llama(cfg, tags):
    cfg.max_position_embeddings = 4096
    cfg.tie_word_embeddings = False
    req = _parse_tokens(tags)
    for key, attr in (("L", "num_hidden_layers"), ("H", "hidden_size"), ("I", "intermediate_size")):
        if key in req:
            setattr(cfg, attr, int(req[key]))
    cfg.head_dim = cfg.hidden_size // cfg.num_attention_heads


_APPLY: Dict[str, Callable] = {"deepseek_v3": _apply_dsv3, "olmoe": _apply_olmoe, "olmo": _apply_olmo,
                               "llama": _apply_llama}


def get_modified_config(model_choice: str, config):
    """Apply the tags of ``model_choice`` to ``config`` in place and return it."""
    hf_id, tags = split_model_choice(model_choice)
    config.use_cache = False
    if hf_id in SUPPORTED_MODEL_IDS:
        _APPLY[model_family(model_choice)](config, tags)
    return config


# Architecture constants of the released checkpoints, so that no hub access is needed.
_BASE_ARCH = {
    "allenai/OLMo-1B-hf": dict(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=16),
    "allenai/OLMo-7B-hf": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32),
    "meta-llama/Llama-3.1-8B": dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                                    num_attention_heads=32, num_key_value_heads=8),
    "meta-llama/Llama-3.2-1B": dict(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                                    num_attention_heads=32, num_key_value_heads=8, head_dim=64),
}


def build_config(model_choice: str, **parallel_kwargs):
    """Construct the parallel config for ``model_choice`` without the HF hub."""
    hf_id, _ = split_model_choice(model_choice)
    fam = model_family(model_choice)
    if fam == "olmoe":
        from .models.olmoe.configuration_olmoe import OlmoeParallelConfig as C
        base = {}
    elif fam == "olmo":
        from .models.olmo.configuration_olmo import OlmoParallelConfig as C
        base = _BASE_ARCH[hf_id]
    elif fam == "llama":
        from .models.llama.configuration_llama import LlamaParallelConfig as C
        base = _BASE_ARCH[hf_id]
    else:
        from .models.deepseek_v3.configuration_deepseek_v3 import DeepseekV3ParallelConfig as C
        base = {}
    import inspect
    accepted = set(inspect.signature(C.__init__).parameters)
    kwargs = {k: v for k, v in parallel_kwargs.items() if k in accepted}
    cfg = C(**base, **kwargs)
    cfg = get_modified_config(model_choice, cfg)
    cfg.check_compatibility()
    return cfg


def cached_model_key(model_choice: str, pp: int, ep: int, tp: int, vpp: int, merged_mlp: bool = False) -> str:
    """Directory name of a sharded model (reference dist_train.py:320-330): ``/`` becomes
    ``__`` and the ``NAL``/``SKIPQKNORM`` tags, which do not change the weights, are dropped."""
    key = model_choice.replace("/", "__")
    for tag in ("NAL", "SKIPQKNORM"):
        if tag in key:
            key = key.replace("--" + tag, "").replace("-" + tag, "")
    key = f"{key}_pp{pp}-ep{ep}-tp{tp}-vpp{vpp}"
    return key + ("_mmlp" if merged_mlp else "")
