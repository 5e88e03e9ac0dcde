"""Length-bucketed, rank-aware, resumable batch sampling
(``keys_values/data/iterators.py:39-316``).

Sequences are sorted by length and cut into global batches of ``micro_batch_size ·
num_devices`` neighbours, so that the rows of a micro-batch (and the micro-batches of the
ranks in one step) have similar lengths; the order of the global batches is shuffled per
epoch (or longest first). Every rank takes its slice of each global batch. The position
is part of ``state_dict`` so that training can resume mid-epoch."""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Sequence

import torch


class SimilarSequenceLengthIterator:
    def __init__(self, sequence_lengths: Sequence[int], micro_batch_size: int, num_devices: int = 1, rank: int = 0, shuffle: bool = True,
                 longest_first: bool = False, seed: int = 0, drop_last: bool = True, shortest_first: bool = False):
        if not (0 <= rank < num_devices):
            raise ValueError(f"rank = {rank} must be in [0, {num_devices})")
        self.lengths = list(sequence_lengths)
        self.micro_batch_size, self.num_devices, self.rank = micro_batch_size, num_devices, rank
        self.shuffle, self.longest_first, self.seed, self.drop_last = shuffle, longest_first, seed, drop_last
        self.shortest_first = shortest_first  # the first batch of every epoch holds the shortest sequences, the others are shuffled
        self.epoch = 0
        self.pos = 0
        self._batches: List[List[int]] = []
        self._build()

    def _build(self) -> None:
        gbs = self.micro_batch_size * self.num_devices
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        # random tie-breaking among equal lengths, then stable sort by length
        perm = torch.randperm(len(self.lengths), generator=g).tolist() if self.shuffle else list(range(len(self.lengths)))
        order = sorted(perm, key=lambda i: self.lengths[i], reverse=True)
        batches = [order[i : i + gbs] for i in range(0, len(order), gbs)]
        if batches and len(batches[-1]) < gbs:
            if self.drop_last:
                batches.pop()
            else:
                batches[-1] = batches[-1] + order[: gbs - len(batches[-1])]
        if self.shuffle and not self.longest_first:
            idx = torch.randperm(len(batches), generator=g).tolist()
            if self.shortest_first and batches:
                idx = [len(batches) - 1] + [i for i in idx if i != len(batches) - 1]
            batches = [batches[i] for i in idx]
        self._batches = batches

    def __len__(self) -> int:
        return len(self._batches)

    def __iter__(self) -> Iterator[List[int]]:
        return self

    def __next__(self) -> List[int]:
        if self.pos >= len(self._batches):
            self.epoch += 1
            self.pos = 0
            self._build()
            raise StopIteration
        gb = self._batches[self.pos]
        self.pos += 1
        lo = self.rank * self.micro_batch_size
        return gb[lo : lo + self.micro_batch_size]

    def state_dict(self) -> Dict[str, Any]:
        return {"epoch": self.epoch, "pos": self.pos, "seed": self.seed, "rank": self.rank, "num_devices": self.num_devices}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        if state.get("num_devices", self.num_devices) != self.num_devices or state.get("rank", self.rank) != self.rank:
            raise ValueError("sampler state was saved for a different rank layout")
        self.epoch, self.seed = state["epoch"], state["seed"]
        self._build()
        self.pos = state["pos"]


class SimilarSequenceLengthSampler(torch.utils.data.Sampler):
    """Batch sampler around :class:`SimilarSequenceLengthIterator`."""

    def __init__(self, *args, **kwargs):
        self.iterator = SimilarSequenceLengthIterator(*args, **kwargs)

    def __iter__(self):
        if not self.iterator.shuffle:
            # an evaluation pass that stopped early (a limit on the number of batches) must not make the next pass
            # start in the middle: batch k of every pass is the same batch. Training samplers (shuffled) keep their
            # position, which is what resuming in the middle of an epoch needs.
            self.iterator.pos = 0
        return iter(self.iterator)

    def __len__(self) -> int:
        return len(self.iterator)

    def state_dict(self):
        return self.iterator.state_dict()

    def load_state_dict(self, state):
        self.iterator.load_state_dict(state)
