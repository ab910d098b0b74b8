"""Token batches for the DeepSeek-V3 example: resumable synthetic data.

``SyntheticBatches`` draws batch ``i`` of rank ``r`` from a generator seeded with
``seed + 1_000_000 * i + r``, so a run resumed at step ``i`` sees the same stream.
Role parity: ``examples/deepseek_v3/data.py:21-55`` of the reference (its streaming C4 loader needs
network access and a tokenizer and is not reproduced here).
"""
from __future__ import annotations

import torch


class SyntheticBatches:
    def __init__(self, vocab_size: int, batch_size: int, seq_len: int, seed: int = 0, rank: int = 0,
                 pin_memory: bool = False):
        self.vocab_size, self.batch_size, self.seq_len = vocab_size, batch_size, seq_len
        self.seed, self.rank, self.step = seed, rank, 0
        self.pin_memory = pin_memory

    def state_dict(self):
        return {"step": self.step}

    def load_state_dict(self, sd):
        self.step = int(sd["step"])

    def __iter__(self):
        return self

    def __next__(self):
        g = torch.Generator().manual_seed(self.seed + 1_000_000 * self.step + self.rank)
        self.step += 1
        t = torch.randint(0, self.vocab_size, (self.batch_size, self.seq_len + 1), generator=g)
        return t.pin_memory() if self.pin_memory else t
