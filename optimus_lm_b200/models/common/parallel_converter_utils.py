"""Weight slicing helpers for tensor parallelism (reference
optimus/models/common/parallel_converter_utils.py:3-101 and custom_linear_modules.py:8-131):
a column-parallel layer keeps a block of output rows, a row-parallel layer a block of input
columns (its bias, if any, is divided by the TP size so that the all-reduce restores it)."""
import torch


def column_slice(weight, tp_ind, tensor_parallelism):
    rows = weight.shape[0] // tensor_parallelism
    return weight[tp_ind * rows:(tp_ind + 1) * rows]


def row_slice(weight, tp_ind, tensor_parallelism):
    cols = weight.shape[1] // tensor_parallelism
    return weight[:, tp_ind * cols:(tp_ind + 1) * cols]


@torch.no_grad()
def populate_ColumnLinear_from_Linear(src, dst, tp_ind, tensor_parallelism=1):
    dst.weight.copy_(column_slice(src.weight, tp_ind, tensor_parallelism))
    if getattr(dst, "bias", None) is not None and getattr(src, "bias", None) is not None:
        dst.bias.copy_(column_slice(src.bias, tp_ind, tensor_parallelism))


@torch.no_grad()
def populate_RowLinear_from_Linear(src, dst, tp_ind, tensor_parallelism=1):
    dst.weight.copy_(row_slice(src.weight, tp_ind, tensor_parallelism))
    if getattr(dst, "bias", None) is not None and getattr(src, "bias", None) is not None:
        dst.bias.copy_(src.bias / tensor_parallelism)


@torch.no_grad()
def populate_Linear_from_Linear(src, dst, *_, **__):
    dst.load_state_dict(src.state_dict())
