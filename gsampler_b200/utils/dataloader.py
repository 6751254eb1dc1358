"""Seed loader with the behaviour of python/gs/utils/dataloader.py:4-44 in gSampler:
optional shuffle at the start of each iteration, then fixed-size slices."""
import torch


class SeedGenerator(object):
    def __init__(self, data: torch.Tensor, batch_size: int, shuffle: bool = False,
                 drop_last: bool = False):
        self.data = data
        self.batch_size = batch_size
        self.shuffle = shuffle
        self.drop_last = drop_last

    def __iter__(self):
        if self.shuffle:
            perm = torch.randperm(self.data.shape[0], device=self.data.device)
            self.data = self.data[perm]
        self.step = 0
        n = self.data.shape[0]
        self.last_step = n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size
        return self

    def __next__(self):
        if self.step >= self.last_step:
            raise StopIteration
        ret = self.data[self.step * self.batch_size:(self.step + 1) * self.batch_size].clone()
        self.step += 1
        return ret

    def __len__(self):
        return (self.data.shape[0] + self.batch_size - 1) // self.batch_size
