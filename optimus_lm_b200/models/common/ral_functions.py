"""Router auxiliary-loss functions (reference optimus/models/common/ral_functions.py:6-35 and
optimus/models/olmoe/modeling_olmoe.py:29-85): the *global* variant concatenates the router
logits of all layers and takes one mean; the *layer-level* variant averages per-layer losses."""
from ...ops.functional import (layer_level_load_balancing_loss_reference as layer_level_load_balancing_loss_func,
                               load_balancing_loss_reference as _global_loss)


def load_balancing_loss_func(gate_logits, num_experts=None, top_k=2, attention_mask=None):
    if gate_logits is None or not isinstance(gate_logits, tuple):
        return 0
    assert attention_mask is None, "padding masks are not used in pretraining"
    return _global_loss(gate_logits, num_experts, top_k)


global_load_balancing_loss_func = load_balancing_loss_func
