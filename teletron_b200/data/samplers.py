"""Batch samplers that are resumable by the number of consumed samples and sliced per data-parallel
rank — behaviour of teletron/train/dataloader.py:123-263.

``PretrainingSampler``: sequential; skips ``consumed_samples``; each global step takes
``micro_batch_size * dp_size`` consecutive indices and hands rank r its contiguous slice.
``PretrainingRandomSampler``: per-epoch permutation seeded by the epoch, resumable in the
middle of an epoch; with ``data_sharding`` each rank permutes inside its own bucket.
"""
from __future__ import annotations

import torch


class PretrainingSampler:
    def __init__(self, total_samples, consumed_samples, micro_batch_size, data_parallel_rank,
                 data_parallel_size, drop_last=True):
        assert total_samples > 0 and consumed_samples < total_samples
        assert micro_batch_size > 0 and 0 <= data_parallel_rank < data_parallel_size
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size, self.drop_last = micro_batch_size, drop_last
        self.dp_rank, self.dp_size = data_parallel_rank, data_parallel_size
        self.step = micro_batch_size * data_parallel_size

    def __len__(self):
        return self.total_samples

    def _slice(self, batch):
        s = self.dp_rank * self.micro_batch_size
        return batch[s:s + self.micro_batch_size]

    def __iter__(self):
        batch = []
        for idx in range(self.consumed_samples, self.total_samples):
            batch.append(idx)
            if len(batch) == self.step:
                yield self._slice(batch)
                batch = []
        if batch and not self.drop_last:
            yield self._slice(batch)


class PretrainingRandomSampler:
    def __init__(self, total_samples, consumed_samples, micro_batch_size, data_parallel_rank,
                 data_parallel_size, data_sharding=True, seed=1234):
        assert total_samples > 0 and micro_batch_size > 0
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size, self.dp_rank, self.dp_size = micro_batch_size, data_parallel_rank, data_parallel_size
        self.data_sharding, self.seed = data_sharding, seed
        self.step = micro_batch_size * data_parallel_size
        self.last_batch_size = total_samples % self.step

    def __len__(self):
        return self.total_samples

    def __iter__(self):
        active = self.total_samples - self.last_batch_size
        epoch = self.consumed_samples // active
        in_epoch = self.consumed_samples % active
        assert in_epoch % self.step == 0
        g = torch.Generator().manual_seed(self.seed + epoch)
        if self.data_sharding:
            bucket = (self.total_samples // self.step) * self.micro_batch_size
            offset = in_epoch // self.dp_size
            start = self.dp_rank * bucket
            order = [start + x for x in torch.randperm(bucket, generator=g).tolist()][offset:]
        else:
            full = (self.total_samples // self.micro_batch_size) * self.micro_batch_size
            order = torch.randperm(full, generator=g).tolist()[in_epoch:][self.dp_rank::self.dp_size]
        batch = []
        for idx in order:
            batch.append(idx)
            if len(batch) == self.micro_batch_size:
                self.consumed_samples += self.step
                yield batch
                batch = []


class RandomSeedDataset(torch.utils.data.Dataset):
    """Reseeds torch / numpy / random per item from (seed, epoch, index) (dataloader.py:172-191)."""

    def __init__(self, dataset, seed=1234):
        self.dataset, self.base_seed, self.curr_seed = dataset, seed, seed

    def __len__(self):
        return len(self.dataset)

    def set_epoch(self, epoch):
        self.curr_seed = self.base_seed + epoch

    def __getitem__(self, idx):
        import random

        import numpy as np

        s = idx + self.curr_seed
        torch.manual_seed(s)
        random.seed(s)
        np.random.seed(s % (2 ** 32))
        return self.dataset[idx]


def build_data_loader(dataset, consumed_samples, micro_batch_size, dp_rank, dp_size, dataloader_type="single",
                      num_workers=0, seed=1234, pin_memory=True, collate_fn=None):
    if dataset is None:
        return None
    if dataloader_type == "single":
        sampler = PretrainingSampler(len(dataset), consumed_samples, micro_batch_size, dp_rank, dp_size)
    elif dataloader_type == "cyclic":
        sampler = PretrainingRandomSampler(len(dataset), consumed_samples, micro_batch_size, dp_rank, dp_size,
                                           seed=seed)
    else:
        raise ValueError(f"unsupported dataloader type {dataloader_type}")
    return torch.utils.data.DataLoader(dataset, batch_sampler=sampler, num_workers=num_workers,
                                       pin_memory=pin_memory and torch.cuda.is_available(),
                                       persistent_workers=num_workers > 0, collate_fn=collate_fn)
