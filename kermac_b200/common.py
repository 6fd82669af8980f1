"""Host helpers of the kermac API that the distance operators and kermac's linalg
module import: layout classification, batch-size merging, stream wrapper, timer.

Behaviour follows src/kermac/common.py of the reference (enums :5-16, stream wrapper
:18-24, CudaTimer :26-42, ceil_div :44-45, merge_batch_size :47-70, TensorStats
:72-144); the code is written for this package.
"""
from __future__ import annotations

from enum import Enum, auto
from typing import Optional, Tuple, Union

import torch

__all__ = [
    "Majorness", "Alignment", "FillMode", "PyTorchStreamWrapper", "CudaTimer",
    "ceil_div", "merge_batch_size", "TensorStats", "tensor_stats",
]


class Majorness(Enum):
    COL_MAJOR = auto()
    ROW_MAJOR = auto()


class Alignment(Enum):
    """Whether an operand may be read in 16-byte (4 float) units."""
    ALIGN_1 = auto()
    ALIGN_4 = auto()


class FillMode(Enum):
    UPPER = auto()
    LOWER = auto()


class PyTorchStreamWrapper:
    """Adapts a torch stream to the ``__cuda_stream__`` protocol (version 0)."""

    def __init__(self, pt_stream):
        self.pt_stream = pt_stream

    def __cuda_stream__(self):
        return (0, self.pt_stream.cuda_stream)


class CudaTimer:
    """CUDA-event stopwatch on torch's current stream: ``start()`` then ``stop()`` -> ms."""

    def __init__(self):
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is not available")
        self.start_event = torch.cuda.Event(enable_timing=True)
        self.end_event = torch.cuda.Event(enable_timing=True)

    def start(self):
        self.start_event.record()

    def stop(self):
        self.end_event.record()
        self.end_event.synchronize()
        return self.start_event.elapsed_time(self.end_event)


def ceil_div(x, d):
    return int(-(-x // d))


def merge_batch_size(name: str, L: int, a: Union[None, float, torch.Tensor], expected_dims: int,
                     can_be_none: bool = False) -> int:
    """Folds the batch extent of one argument into the running batch size ``L``.

    An argument has either ``expected_dims`` dimensions (no batch) or one more
    (leading batch); batch extents must be 1 or agree (reference rule,
    src/kermac/common.py:47-70).
    """
    if a is None:
        if not can_be_none:
            raise ValueError(f'{name} is none, but can_be_none is False')
        return L
    if isinstance(a, float):
        if expected_dims != 0:
            raise ValueError(f'{name} is a float but expected_dims is {expected_dims}')
        return L
    if isinstance(a, torch.Tensor):
        if a.dim() == expected_dims:
            return L
        if a.dim() == expected_dims + 1:
            this_L = a.size(0)
            if this_L != 1 and L != 1 and this_L != L:
                raise ValueError(
                    f'{name} batch size of {this_L} does not match with another non-one batch size, {L}')
            return max(L, this_L)
        raise ValueError(
            f'{name} does have the right number of dimensions, expected_dims is {expected_dims} '
            f'or {expected_dims + 1}, got {a.dim()}')
    raise TypeError(f'{name} must be None, a float or a torch.Tensor')


class TensorStats:
    """Shape, majorness, pitch, batch stride and 16-byte alignment of a 2-D/3-D fp32 tensor.

    ROW_MAJOR: last stride 1 and row pitch >= columns.  COL_MAJOR: row stride 1 and
    column pitch >= rows.  Anything else is rejected (src/kermac/common.py:96-102).
    ``batch_stride`` is 0 for 2-D tensors and for a batch of one, which is what makes
    such operands broadcast over the batch.
    """

    ALIGN_BYTES = 16
    ALIGN_ELEMS = 4

    def __init__(self, tensor: torch.Tensor):
        if tensor.dim() not in (2, 3):
            raise ValueError("Input tensor must be 2 or 3-dimensional")
        if tensor.dtype != torch.float32:
            raise TypeError("Input tensor must have dtype torch.float32")
        sizes, strides = tuple(tensor.size()), tuple(tensor.stride())
        batched = tensor.dim() == 3
        self._num_batches = sizes[0] if batched else 1
        self._batch_stride = strides[0] if (batched and self._num_batches != 1) else 0
        rows, cols = sizes[-2], sizes[-1]
        s_row, s_col = strides[-2], strides[-1]
        self._shape = (self._num_batches, rows, cols)
        self._stride_row, self._stride_col = s_row, s_col
        if s_col == 1 and s_row >= cols:
            self._majorness = Majorness.ROW_MAJOR
        elif s_row == 1 and s_col >= rows:
            self._majorness = Majorness.COL_MAJOR
        else:
            raise ValueError(f"Tensor has non-standard memory layout: strides={strides}, shape={sizes}")
        self._leading_dimension_stride = max(s_row, s_col)
        ptr_ok = tensor.data_ptr() % self.ALIGN_BYTES == 0
        ld_ok = self._leading_dimension_stride % self.ALIGN_ELEMS == 0
        if self._majorness is Majorness.COL_MAJOR and ptr_ok and ld_ok:
            self._alignment = Alignment.ALIGN_4
        else:
            self._alignment = Alignment.ALIGN_1

    @property
    def shape(self) -> Tuple[int, int, int]:
        return self._shape

    @property
    def majorness(self) -> Majorness:
        return self._majorness

    @property
    def alignment(self) -> Alignment:
        return self._alignment

    @property
    def num_batches(self) -> int:
        return self._num_batches

    @property
    def batch_stride(self) -> int:
        return self._batch_stride

    @property
    def leading_dimension_stride(self) -> int:
        return self._leading_dimension_stride

    @property
    def matrix_strides(self) -> Tuple[int, int]:
        """(row stride, column stride) in elements; what the C-ABI takes."""
        return (self._stride_row, self._stride_col)


def tensor_stats(tensor: torch.Tensor) -> TensorStats:
    return TensorStats(tensor)
