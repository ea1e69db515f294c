"""Grid type and key-width helpers of the particle sort (host side).

Mirrors the names of the reference's shared module
(project_aether/src/custom_kernels/triton/radix_sort_reference.py:28-65) that
are part of the sort's public surface: `CellGrid`, `SHUFFLE_BITS`, `num_passes`.
The digit width is this implementation's own (8 bits, not the reference's 7);
it does not show in any result because every stable sort of the same keys
gives the same permutation.
"""

import math
from typing import NamedTuple, Tuple

SHUFFLE_BITS = 7
RADIX_BITS = 8
RADIX = 1 << RADIX_BITS
MAX_KEY_BITS = 32
MAX_PARTICLES = (1 << 30) - 1


class CellGrid(NamedTuple):
    """Uniform Cartesian grid of DSMC collision cells.

    Attributes:
      lo: lower corner (x, y, z).
      hi: upper corner (x, y, z).
      cells: number of cells (nx, ny, nz).
    """
    lo: Tuple[float, float, float]
    hi: Tuple[float, float, float]
    cells: Tuple[int, int, int]

    @property
    def num_cells(self) -> int:
        return self.cells[0] * self.cells[1] * self.cells[2]


def key_bits(num_cells: int, shuffle_bits: int = SHUFFLE_BITS) -> int:
    """Bits of the sort key: cell bits plus shuffle bits."""
    return max(1, (num_cells - 1).bit_length()) + shuffle_bits


def num_passes(num_cells: int, shuffle_bits: int = SHUFFLE_BITS) -> int:
    """Digit passes needed for keys of (cell bits + shuffle bits).

    Same contract as the reference's `num_passes`
    (radix_sort_reference.py:60-65) with two documented differences: digits are
    8 bits wide and keys are unsigned, so 32-bit keys are accepted (the
    reference raises above 31 bits).

    Raises:
      ValueError: if the keys need more than 32 bits.
    """
    bits = key_bits(num_cells, shuffle_bits)
    if bits > MAX_KEY_BITS:
        raise ValueError(f'Sort keys need {bits} bits; at most {MAX_KEY_BITS} fit.')
    return math.ceil(bits / RADIX_BITS)
