"""Small helpers for cache code (``keys_values/kvcache/utils.py:19-78``)."""
from typing import List, Tuple

import torch


def smallest_covering_ranges(slots: List[int], max_num_ranges: int) -> List[Tuple[int, int]]:
    """Cover the sorted set ``slots`` by at most ``max_num_ranges`` half-open
    ranges of minimal total length: start from one range per run of consecutive
    slots and close the smallest gaps until few enough remain."""
    if not slots:
        return []
    s = sorted(set(slots))
    ranges = []
    start = prev = s[0]
    for x in s[1:]:
        if x != prev + 1:
            ranges.append((start, prev + 1))
            start = x
        prev = x
    ranges.append((start, prev + 1))
    while len(ranges) > max_num_ranges:
        gaps = [(ranges[i + 1][0] - ranges[i][1], i) for i in range(len(ranges) - 1)]
        _, i = min(gaps)
        ranges[i : i + 2] = [(ranges[i][0], ranges[i + 1][1])]
    return ranges


def storage_id(x: torch.Tensor) -> int:
    """Identifier of the memory that backs ``x`` (equal for views of one tensor)."""
    return x.untyped_storage().data_ptr()
