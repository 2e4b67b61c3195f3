"""Entry points with the names and argument lists of the reference's MoE custom-op extension.

The reference's FastMoE block calls a SYCL extension ``pcl_xpu_customops`` (csrc/ops/sparse_moe_block.sycl:
539-547) for its non-GEMM steps and keeps an ``IndexAddOpFunction`` in optimus/custom_ops.py:4-16.  Code
written against that interface can import this module instead:

    import optimus_lm_b200.custom_ops as pcl_xpu_customops

Data layout of that interface (R = routed rows on this rank, TH = ceil(T / 8) "threads" of 8 tokens):

* ``partial_token_counts [E_loc, TH]``: hits of each local expert inside each block of 8 tokens;
* ``expert_counts_ep [T]`` / ``cum_expert_counts_ep [T + 1]``: local-expert hits per token and their
  exclusive prefix - the token-major *slots*;
* rows are ordered by (expert, token block, token, k); ``input_indices [R]`` maps row -> token,
  ``output_indices [R]`` maps slot -> row, ``selected_experts_indices [R]`` maps slot -> k.

This framework's own MoE path does not go through these functions: it builds a padded,
tile-aligned index on the device in one pass (``ops.functional.MoEIndex``) and folds the routing
weight into the expert activation.  On CUDA tensors (int32 indices, contiguous bf16 or fp32 data) every
function runs its kernel of ``csrc/customops.cu``; elsewhere the vectorised tensor programs below, which are also
the kernels' test oracle.
"""
from __future__ import annotations

import torch

TOKENS_PER_THREAD = 8


def _native(*tensors):
    """The compiled extension when every tensor is a contiguous CUDA tensor the kernels take, else ``None``."""
    for t in tensors:
        if not (torch.is_tensor(t) and t.is_cuda and t.is_contiguous()):
            return None
        if t.dtype not in (torch.int32, torch.float32, torch.bfloat16):
            return None
    from .ops._ext import extension, kernels_disabled
    if kernels_disabled():
        return None
    C = extension()
    return C if hasattr(C, "co_index_gather") else None


def _local_mask(selected_experts, e_start, e_end):
    return (selected_experts >= e_start) & (selected_experts < e_end)


def compute_partial_token_counts(selected_experts, partial_token_counts, expert_counts_ep, expert_start_idx,
                                 expert_end_idx):
    """K1: fills ``partial_token_counts [E_loc, TH]`` and ``expert_counts_ep [T]``; returns the former."""
    C = _native(selected_experts, partial_token_counts, expert_counts_ep)
    if C is not None and selected_experts.dtype == torch.int32:
        return C.co_compute_partial_token_counts(selected_experts, partial_token_counts, expert_counts_ep,
                                                 expert_start_idx, expert_end_idx)
    T, K = selected_experts.shape
    E_loc = expert_end_idx - expert_start_idx
    TH = partial_token_counts.shape[1]
    local = _local_mask(selected_experts, expert_start_idx, expert_end_idx)
    expert_counts_ep.copy_(local.sum(dim=1).to(expert_counts_ep.dtype))
    tok = torch.arange(T, device=selected_experts.device).unsqueeze(1).expand(T, K)
    key = (selected_experts - expert_start_idx).long() * TH + tok // TOKENS_PER_THREAD
    counts = torch.bincount(key[local], minlength=E_loc * TH)[: E_loc * TH]
    partial_token_counts.copy_(counts.view(E_loc, TH).to(partial_token_counts.dtype))
    return partial_token_counts


def compute_input_and_output_indices(selected_experts, partial_cum_token_counts, input_increment_buffer,
                                     cum_expert_counts_ep, selected_experts_indices, input_indices, output_indices,
                                     expert_start_idx, expert_end_idx):
    """K3: deterministic bucket placement.  ``partial_cum_token_counts [E_loc * TH + 1]`` is the exclusive
    prefix of the flattened K1 counts; ``input_increment_buffer`` is scratch of the reference's kernel and
    is left untouched (the CUDA kernel uses it for its per-bucket counters)."""
    C = _native(selected_experts, partial_cum_token_counts, input_increment_buffer, cum_expert_counts_ep,
                selected_experts_indices, input_indices, output_indices)
    if C is not None and all(t.dtype == torch.int32 for t in (selected_experts, partial_cum_token_counts,
                                                               input_increment_buffer, cum_expert_counts_ep,
                                                               selected_experts_indices, input_indices, output_indices)):
        C.co_compute_input_and_output_indices(selected_experts, partial_cum_token_counts, input_increment_buffer,
                                              cum_expert_counts_ep, selected_experts_indices, input_indices,
                                              output_indices, expert_start_idx, expert_end_idx)
        return
    T, K = selected_experts.shape
    E_loc = expert_end_idx - expert_start_idx
    TH = (partial_cum_token_counts.numel() - 1) // E_loc
    dev = selected_experts.device
    local = _local_mask(selected_experts, expert_start_idx, expert_end_idx)
    tok = torch.arange(T, device=dev).unsqueeze(1).expand(T, K)[local]
    kk = torch.arange(K, device=dev).unsqueeze(0).expand(T, K)[local]
    e = (selected_experts[local] - expert_start_idx).long()
    # pairs are enumerated token-major (t, k); a stable sort by (expert, token block) keeps that order inside a bucket
    bucket = e * TH + tok // TOKENS_PER_THREAD
    order = torch.sort(bucket, stable=True).indices
    sorted_bucket = bucket[order]
    first = partial_cum_token_counts.long()[sorted_bucket]
    start_of_bucket = torch.searchsorted(sorted_bucket, sorted_bucket, right=False)
    rows = first + (torch.arange(order.numel(), device=dev) - start_of_bucket)
    row_of_pair = torch.empty_like(rows)
    row_of_pair[order] = rows
    # slot of a pair: token-major position among the local hits
    slot = torch.arange(tok.numel(), device=dev)
    input_indices[row_of_pair] = tok.to(input_indices.dtype)
    output_indices[slot] = row_of_pair.to(output_indices.dtype)
    selected_experts_indices[slot] = kk.to(selected_experts_indices.dtype)


def index_gather(inp, indices, out):
    """K4f: ``out[o, :] = inp[indices[o], :]``."""
    C = _native(inp, indices, out)
    if C is not None and indices.dtype == torch.int32 and inp.dtype == out.dtype != torch.int32:
        return C.co_index_gather(inp, indices, out)
    torch.index_select(inp, 0, indices.long(), out=out)
    return out


def _slot_tokens(cum_expert_counts_ep):
    counts = (cum_expert_counts_ep[1:] - cum_expert_counts_ep[:-1]).long()
    return torch.repeat_interleave(torch.arange(counts.numel(), device=counts.device), counts)


def shuffle_sub_matrix_reduce(ggemm_input_grad, cum_expert_counts_ep, output_indices, hidden_states_grad):
    """K4b: ``dX[t] = sum over the slots of t of dY[output_indices[slot]]`` (fp32 accumulation)."""
    C = _native(ggemm_input_grad, cum_expert_counts_ep, output_indices, hidden_states_grad)
    if C is not None and cum_expert_counts_ep.dtype == output_indices.dtype == torch.int32 \
            and ggemm_input_grad.dtype == hidden_states_grad.dtype != torch.int32:
        return C.co_shuffle_sub_matrix_reduce(ggemm_input_grad, cum_expert_counts_ep, output_indices, hidden_states_grad)
    tok = _slot_tokens(cum_expert_counts_ep)
    acc = torch.zeros(hidden_states_grad.shape, dtype=torch.float32, device=hidden_states_grad.device)
    acc.index_add_(0, tok, ggemm_input_grad[output_indices.long()].float())
    hidden_states_grad.copy_(acc.to(hidden_states_grad.dtype))
    return hidden_states_grad


def reduce_ggemm_output(ggemm_output, routing_weights, cum_expert_counts_ep, selected_experts_indices, output_indices,
                        final_hidden_states, accumulate=False):
    """K6f: ``out[t] (+)= sum over slots of w[t, k_slot] * Y[output_indices[slot]]`` (fp32 accumulation)."""
    C = _native(ggemm_output, routing_weights, cum_expert_counts_ep, selected_experts_indices, output_indices,
                final_hidden_states)
    if C is not None and cum_expert_counts_ep.dtype == selected_experts_indices.dtype == output_indices.dtype == torch.int32 \
            and ggemm_output.dtype == routing_weights.dtype == final_hidden_states.dtype != torch.int32:
        return C.co_reduce_ggemm_output(ggemm_output, routing_weights, cum_expert_counts_ep, selected_experts_indices,
                                        output_indices, final_hidden_states, bool(accumulate))
    tok = _slot_tokens(cum_expert_counts_ep)
    w = routing_weights[tok, selected_experts_indices.long()].float().unsqueeze(1)
    acc = final_hidden_states.float() if accumulate else torch.zeros(final_hidden_states.shape, dtype=torch.float32,
                                                                      device=final_hidden_states.device)
    acc = acc.index_add(0, tok, w * ggemm_output[output_indices.long()].float())
    final_hidden_states.copy_(acc.to(final_hidden_states.dtype))
    return final_hidden_states


def reduce_ggemm_output_backward(final_hidden_states_grad, ggemm_output, routing_weights, cum_expert_counts_ep,
                                 selected_experts_indices, input_indices, output_indices, ggemm_output_grad,
                                 routing_weights_grad):
    """K6b: ``dY[row] = w[t, k] * dOut[t]`` and ``dw[t, k] = <Y[row], dOut[t]>`` for every slot (t, k) -> row;
    entries of ``dw`` whose expert is not local stay as they were."""
    C = _native(final_hidden_states_grad, ggemm_output, routing_weights, cum_expert_counts_ep, selected_experts_indices,
                output_indices, ggemm_output_grad, routing_weights_grad)
    dts = {t.dtype for t in (final_hidden_states_grad, ggemm_output, routing_weights, ggemm_output_grad,
                             routing_weights_grad)}
    if C is not None and len(dts) == 1 and torch.int32 not in dts \
            and cum_expert_counts_ep.dtype == selected_experts_indices.dtype == output_indices.dtype == torch.int32:
        C.co_reduce_ggemm_output_backward(final_hidden_states_grad, ggemm_output, routing_weights, cum_expert_counts_ep,
                                          selected_experts_indices, input_indices, output_indices, ggemm_output_grad,
                                          routing_weights_grad)
        return
    tok = _slot_tokens(cum_expert_counts_ep)
    rows = output_indices.long()
    k = selected_experts_indices.long()
    g = final_hidden_states_grad[tok].float()
    ggemm_output_grad[rows] = (routing_weights[tok, k].float().unsqueeze(1) * g).to(ggemm_output_grad.dtype)
    routing_weights_grad[tok, k] = (ggemm_output[rows].float() * g).sum(dim=1).to(routing_weights_grad.dtype)


def index_add_op(expert_output, final_output, indices):
    """K7: ``final_output[indices[c], :] += expert_output[c, :]``."""
    C = _native(expert_output, final_output, indices)
    if C is not None and indices.dtype == torch.int32 and expert_output.dtype == final_output.dtype != torch.int32 \
            and expert_output.shape[1] % 2 == 0:
        return C.co_index_add_op(expert_output, final_output, indices)
    final_output.index_add_(0, indices.long(), expert_output.to(final_output.dtype))
    return final_output


def index_gather_op(grad_output, expert_output_grad, indices):
    """Backward of ``index_add_op`` with respect to ``expert_output`` (the reference calls an op of this name that
    its extension never defined, optimus/custom_ops.py:15)."""
    return index_gather(grad_output, indices, expert_output_grad)


class IndexAddOpFunction(torch.autograd.Function):
    """``final_output.index_add_(0, indices, expert_output)`` as an autograd function (reference
    optimus/custom_ops.py:4-16)."""

    @staticmethod
    def forward(ctx, expert_output, final_output, indices):
        ctx.save_for_backward(indices)
        index_add_op(expert_output, final_output, indices)
        ctx.mark_dirty(final_output)
        return final_output

    @staticmethod
    def backward(ctx, grad_output):
        (indices,) = ctx.saved_tensors
        grad_expert = torch.empty((indices.numel(), grad_output.shape[1]), dtype=grad_output.dtype,
                                  device=grad_output.device)
        index_gather_op(grad_output.contiguous(), grad_expert, indices)
        return grad_expert, grad_output, None


def RMSNormOp(hidden_states, weight, output, eps):
    """RMSNorm entry point (reference optimus/models/common/norm_modules.py:33): fused kernel on CUDA bf16."""
    from .ops import functional as OF

    output.copy_(OF.rms_norm(hidden_states, weight, eps))
    return output
