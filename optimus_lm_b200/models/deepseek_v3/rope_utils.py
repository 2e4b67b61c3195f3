"""DeepSeek-V3 rotary helpers under the reference's module name
(optimus/models/deepseek_v3/rope_utils.py:5-96); the implementations live in
``models/common/modeling_rope_utils.py``."""
from ..common.modeling_rope_utils import (_compute_yarn_parameters, apply_rotary_pos_emb_interleave,  # noqa: F401
                                          rotate_half, yarn_get_mscale)
