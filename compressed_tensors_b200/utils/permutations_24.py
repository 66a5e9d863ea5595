"""Marlin-24 weight and scale permutations (utils/permutations_24.py:32-65 of the reference) as index tables.
The CUDA packing kernels compute the same permutation from its closed form; these tables serve host code and
tests."""
import torch

__all__ = ["get_permutations_24"]


def get_permutations_24(num_bits: int):
    """(perm [1024], scale_perm [64], scale_perm_single [64]) for 4- or 8-bit Marlin-24 packing."""
    if num_bits not in (4, 8):
        raise ValueError("num_bits must be 4 or 8, got {}".format(num_bits))
    flat = []
    for i in range(32):
        col = i // 4
        base = [16 * row + (col // 2) * 256 + 8 * (col % 2) + 4 * block
                for block in (0, 1) for row in (2 * (i % 4), 2 * (i % 4) + 1, 2 * (i % 4 + 4), 2 * (i % 4 + 4) + 1)]
        for j in range(4):
            flat.extend(p + j for p in base)
    interleave = [0, 2, 4, 6, 1, 3, 5, 7] if num_bits == 4 else [0, 2, 1, 3]
    perm = torch.tensor(flat).reshape(-1, len(interleave))[:, interleave].reshape(-1)
    scale_perm = [8 * i + j for i in range(8) for j in (0, 4, 1, 5, 2, 6, 3, 7)]
    scale_perm_single = list(range(64))
    return perm, scale_perm, scale_perm_single
