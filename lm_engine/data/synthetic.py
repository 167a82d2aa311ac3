"""Synthetic pretraining data: uniform random token ids of the pretraining sample shape ``[micro_batch, seq + 1]``.

Used by the benchmark configs (no dataset files are needed) and by the CPU plumbing tests. Every data parallel
rank draws from its own generator stream, seeded from ``(seed, dp_rank)``; the stream position is restorable from
the number of consumed samples so that a resumed run sees the data an uninterrupted run would have seen.
"""

from __future__ import annotations

import torch


class SyntheticTokenLoader:
    def __init__(self, vocab_size: int, sequence_length: int, micro_batch_size: int, seed: int, dp_rank: int = 0,
                 dp_world_size: int = 1, pin_memory: bool = False, num_samples: int | None = None) -> None:
        self.vocab_size = vocab_size
        self.sequence_length = sequence_length
        self.micro_batch_size = micro_batch_size
        self.seed = seed
        self.dp_rank = dp_rank
        self.dp_world_size = dp_world_size
        self.pin_memory = pin_memory and torch.cuda.is_available()
        self.num_samples = num_samples
        self.batches_served = 0

    def _sample(self, sample_index: int) -> torch.Tensor:
        gen = torch.Generator().manual_seed((self.seed * 1000003 + sample_index) % (2**63 - 1))
        return torch.randint(0, self.vocab_size, (self.sequence_length + 1,), generator=gen, dtype=torch.long)

    def _batch(self, index: int) -> torch.Tensor:
        # Samples are numbered globally and every sample has its own generator stream, so the union of what all
        # ranks read in one step does not depend on the number of ranks: rank r reads samples
        # [(index * world + r) * micro_batch, ... + micro_batch).
        first = (index * self.dp_world_size + self.dp_rank) * self.micro_batch_size
        tokens = torch.stack([self._sample(first + i) for i in range(self.micro_batch_size)])
        return tokens.pin_memory() if self.pin_memory else tokens

    def __iter__(self):
        return self

    def __next__(self) -> dict:
        if self.num_samples is not None and self.batches_served * self.micro_batch_size * self.dp_world_size >= self.num_samples:
            raise StopIteration
        batch = {"text": self._batch(self.batches_served)}
        self.batches_served += 1
        return batch

    def state_dict(self) -> dict:
        return {"batches_served": self.batches_served}

    def load_state_dict(self, state: dict) -> None:
        self.batches_served = state["batches_served"]

    def set_consumed_samples(self, consumed_samples: int) -> None:
        self.batches_served = consumed_samples // (self.micro_batch_size * self.dp_world_size)
