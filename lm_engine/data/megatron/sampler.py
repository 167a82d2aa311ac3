"""Batch sampler with Megatron-LM's data order (parity: lm_engine/data/megatron/sampler.py:1-47).

Sample numbers run ``consumed_samples, consumed_samples + 1, ...``; every ``micro_batch_size * num_replicas`` of them
form one global micro-batch of which replica ``rank`` takes the ``rank``-th contiguous slice. Resuming is a matter of
passing the number of samples already consumed.
"""

from __future__ import annotations


class MegatronBatchSampler:
    def __init__(self, total_samples: int, consumed_samples: int, micro_batch_size: int, num_replicas: int, rank: int,
                 drop_last: bool = True) -> None:
        assert total_samples > 0, f"no sample to consume: {total_samples}"
        assert consumed_samples < total_samples, f"no samples left to consume: {consumed_samples}, {total_samples}"
        assert micro_batch_size > 0
        assert 0 <= rank < num_replicas
        self.total_samples = total_samples
        self.consumed_samples = consumed_samples
        self.micro_batch_size = micro_batch_size
        self.num_replicas = num_replicas
        self.rank = rank
        self.drop_last = drop_last
        self.micro_batch_times_num_replicas = micro_batch_size * num_replicas

    def __len__(self) -> int:
        return self.total_samples

    def __iter__(self):
        stride = self.micro_batch_times_num_replicas
        mine = slice(self.rank * self.micro_batch_size, (self.rank + 1) * self.micro_batch_size)
        start = self.consumed_samples
        while start + stride <= self.total_samples:
            yield list(range(start, start + stride))[mine]
            start += stride
        if start < self.total_samples and not self.drop_last:
            yield list(range(start, self.total_samples))[mine]
