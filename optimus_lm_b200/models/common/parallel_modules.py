"""Vocabulary-parallel embedding and hidden-split LM head for tensor parallelism (reference
optimus/models/common/parallel_modules.py:9-89)."""
import torch
from torch import nn

from ...ops import functional as OF
from .comms_ptfunctions import forward_allreduce_backward_identity, forward_inner_split_backward_allgather


class ParallelEmbedding(nn.Module):
    """Each TP rank stores ``ceil(V/TP)`` rows; out-of-range ids read row 0 and are zeroed, the
    partial outputs are summed over the TP group."""

    def __init__(self, vocab_size, embedding_size, padding_idx=None, tensor_parallelism=1, tp_ind=0, group=None):
        super().__init__()
        self.vocab_size, self.embedding_size, self.padding_idx = vocab_size, embedding_size, padding_idx
        self.tensor_parallelism, self.tp_ind, self.group = tensor_parallelism, tp_ind, group
        self.vocab_size_per_rank = (vocab_size + tensor_parallelism - 1) // tensor_parallelism
        self.vocab_size_padded = tensor_parallelism * self.vocab_size_per_rank
        self.start_embedding_id = tp_ind * self.vocab_size_per_rank
        self.end_embedding_id = (tp_ind + 1) * self.vocab_size_per_rank
        self.weight = nn.Parameter(torch.empty((self.vocab_size_per_rank, embedding_size)))
        self.local_padding_idx = None
        if padding_idx is not None and self.start_embedding_id <= padding_idx < self.end_embedding_id:
            self.local_padding_idx = padding_idx - self.start_embedding_id

    def forward(self, input):
        from ...ops import functional as OF
        if self.tensor_parallelism == 1:
            return OF.embedding(input, self.weight, self.local_padding_idx)
        # rows of other ranks' vocabulary ranges come back as zeros; the all-reduce assembles the lookup
        out = OF.embedding(input, self.weight, self.local_padding_idx, v_start=self.start_embedding_id, masked=True)
        return forward_allreduce_backward_identity.apply(out, self.group)

    @torch.no_grad()
    def set_parameters_from_full_module(self, module):
        lo, hi = self.start_embedding_id, min(self.end_embedding_id, self.vocab_size)
        self.weight[:hi - lo].copy_(module.weight[lo:hi])
        self.weight[hi - lo:].zero_()

    def reset_parameters(self):
        nn.init.normal_(self.weight, mean=0, std=1)


class ParallelLMHead(nn.Module):
    """Splits the *hidden* dimension: every rank multiplies its hidden slice by
    ``weight [V, H/TP]`` and the full-vocabulary partial logits are all-reduced."""

    def __init__(self, hidden_size, vocab_size, bias=False, tensor_parallelism=1, tp_ind=0, group=None):
        super().__init__()
        assert not bias, "ParallelLMHead does not support bias currently."
        self.hidden_size, self.vocab_size = hidden_size, vocab_size
        self.tensor_parallelism, self.tp_ind, self.group = tensor_parallelism, tp_ind, group
        self.hidden_size_per_rank = hidden_size // tensor_parallelism
        self.weight = nn.Parameter(torch.empty((vocab_size, self.hidden_size_per_rank)))
        self.bias = None

    def forward(self, hidden_states):
        if self.tensor_parallelism > 1:
            hidden_states = forward_inner_split_backward_allgather.apply(hidden_states, self.tp_ind,
                                                                         self.tensor_parallelism, self.group)
        logits = OF.linear(hidden_states, self.weight)
        if self.tensor_parallelism > 1:
            logits = forward_allreduce_backward_identity.apply(logits, self.group)
        return logits

    @torch.no_grad()
    def set_parameters_from_full_module(self, module):
        w = self.hidden_size_per_rank
        self.weight.copy_(module.weight[:, self.tp_ind * w:(self.tp_ind + 1) * w])

    def reset_parameters(self):
        nn.init.normal_(self.weight, mean=0, std=1)


class VocabParallelLMHead(nn.Module):
    """LM head split along the *vocabulary*: every rank multiplies the full hidden state by its ``weight [V/TP, H]``
    and keeps its slice of the logits.  Used with ``ops.functional.vocab_parallel_cross_entropy`` the
    ``[tokens, vocabulary]`` logits never cross the links - only per-row softmax statistics are all-reduced - whereas
    ``ParallelLMHead`` (the reference's layout, optimus/models/common/parallel_modules.py:58-89) all-reduces the
    full logits.  The gradient of the hidden state is summed over the group in the backward."""

    def __init__(self, hidden_size, vocab_size, bias=False, tensor_parallelism=1, tp_ind=0, group=None):
        super().__init__()
        assert not bias, "VocabParallelLMHead does not support bias."
        assert vocab_size % tensor_parallelism == 0
        self.hidden_size, self.vocab_size = hidden_size, vocab_size
        self.tensor_parallelism, self.tp_ind, self.group = tensor_parallelism, tp_ind, group
        self.vocab_size_per_rank = vocab_size // tensor_parallelism
        self.vocab_start = tp_ind * self.vocab_size_per_rank
        self.weight = nn.Parameter(torch.empty((self.vocab_size_per_rank, hidden_size)))
        self.bias = None

    def forward(self, hidden_states):
        if self.tensor_parallelism > 1:
            from .comms_ptfunctions import forward_identity_backward_allreduce
            hidden_states = forward_identity_backward_allreduce.apply(hidden_states, self.group)
        return OF.linear(hidden_states, self.weight)

    def loss(self, hidden_states, labels, inplace_backward=False):
        """Shifted mean cross entropy of this head's logits against global ``labels [B, S]``."""
        return OF.vocab_parallel_cross_entropy(self.forward(hidden_states), labels, self.vocab_start, self.vocab_size,
                                               self.group if self.tensor_parallelism > 1 else None, inplace_backward)

    @torch.no_grad()
    def set_parameters_from_full_module(self, module):
        self.weight.copy_(module.weight[self.vocab_start:self.vocab_start + self.vocab_size_per_rank])

    def reset_parameters(self):
        nn.init.normal_(self.weight, mean=0, std=1)
