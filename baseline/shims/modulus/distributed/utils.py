"""Uneven ceil-splitting of an axis over ranks, and the tensor split that goes with it."""

import torch


def compute_split_shapes(size, num_chunks):
    if num_chunks == 1:
        return [size]
    chunk = (size + num_chunks - 1) // num_chunks
    last = max(0, size - chunk * (num_chunks - 1))
    if last == 0:
        chunk = size // num_chunks
        last = size - chunk * (num_chunks - 1)
    return [chunk] * (num_chunks - 1) + [last]


def get_memory_format(tensor):
    return torch.channels_last if tensor.dim() == 4 and tensor.is_contiguous(memory_format=torch.channels_last) else torch.contiguous_format


def split_tensor_along_dim(tensor, dim, num_chunks):
    assert tensor.dim() > dim
    assert tensor.shape[dim] >= num_chunks
    return list(torch.split(tensor, compute_split_shapes(tensor.shape[dim], num_chunks), dim=dim))
