"""Hadamard matrix construction (transform/utils/hadamard.py of the reference).  These are host-side objects
kept for inspection and serialisation; the rotation of the weights themselves runs in the CUDA kernels, which
only need the +-1 diagonal."""
import math
from typing import Optional

import torch

__all__ = ["random_hadamard_matrix", "deterministic_hadamard_matrix", "is_pow2", "random_hadamard_signs", "SYLVESTER_RANDOM_SIZES",
           "is_sylvester_random_size"]

# sizes up to 256 for which the reference's stored base matrix is the Sylvester matrix, so that
# random_hadamard_matrix(n) == diag(Q) @ H_n; other sizes need the reference's data file
SYLVESTER_RANDOM_SIZES = (1, 2, 4, 8, 16, 64, 128, 256)


def is_sylvester_random_size(size: int) -> bool:
    """True where random_hadamard_matrix(size) is diag(Q) @ Sylvester: the stored Sylvester sizes, and every larger
    power of two, which the reference builds as butterfly(size / 256) (x) stored H_256 (hadamard.py:102-163)."""
    return size in SYLVESTER_RANDOM_SIZES or (size >= 512 and size & (size - 1) == 0)


def is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1) == 0)


def deterministic_hadamard_matrix(size: int, dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cpu")) -> torch.Tensor:
    """Sylvester's construction, H[i][j] = (-1)^popcount(i & j) (hadamard.py:33-62)."""
    if size <= 0:
        raise ValueError("Cannot construct deterministic hadamard of size <= 0")
    if size != 2 ** int(math.log2(size)):
        raise ValueError("Cannot construct deterministic hadamard of size != 2^n")
    i = torch.arange(size, device=device)
    bits = i[:, None] & i[None, :]
    parity = torch.zeros_like(bits)
    while bool(bits.any()):
        parity ^= bits & 1
        bits = bits >> 1
    return (1 - 2 * parity).to(dtype)


def random_hadamard_signs(size: int, gen: Optional[torch.Generator] = None, dtype: torch.dtype = torch.float64) -> torch.Tensor:
    """The +-1 diagonal Q of random_hadamard_matrix, drawn exactly as the reference draws it
    (hadamard.py:85-87: torch.randint(0, 2, (size,), generator=gen, dtype=dtype) * 2 - 1 on the CPU)."""
    q = torch.randint(low=0, high=2, size=(size,), generator=gen, dtype=dtype)
    return q * 2 - 1


def random_hadamard_matrix(size: int, dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cpu"),
                           gen: Optional[torch.Generator] = None) -> torch.Tensor:
    """diag(Q) @ H_size with Q a seeded +-1 vector (hadamard.py:65-89)."""
    if not is_sylvester_random_size(size):
        raise NotImplementedError(f"random Hadamard matrices are built for sizes {SYLVESTER_RANDOM_SIZES} and powers of two from 512; size {size} needs "
                                  "the reference's table of stored base matrices")
    q = random_hadamard_signs(size, gen, dtype).to(device)
    return q[:, None] * deterministic_hadamard_matrix(size, dtype, device)
