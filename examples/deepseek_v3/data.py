"""Token batches for the DeepSeek-V3 example: resumable synthetic data.

``SyntheticBatches`` draws batch ``i`` of rank ``r`` from a generator seeded with
``seed + 1_000_000 * i + r``, so a run resumed at step ``i`` sees the same stream.
``PackedDocumentBatches`` packs tokenised documents from local files into rows the way the reference's
streaming C4 loader does (``examples/deepseek_v3/data.py:67-133``): every document becomes
``[BOS] tokens [EOS]``, documents are concatenated and cut into rows of ``seq_len`` tokens, a document that
crosses a row boundary continues in the next row, labels are the next token inside the document and
``positions`` restart with every document (and every ``seq_len`` tokens of a long one).  The documents come
from ``.npy`` / ``.pt`` files of token ids on disk (one 1-D array per document, or one 2-D/ragged list per
file), split across ranks file by file; the reference streams English C4 from the Hugging Face Hub through a
tokenizer, which needs network access.
Role parity: ``examples/deepseek_v3/data.py:21-55`` (synthetic) and ``:67-133`` (packed documents).
"""
from __future__ import annotations

import copy
import glob
import os

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


def _documents_of(path: str):
    if path.endswith(".npy"):
        import numpy as np

        arr = np.load(path, allow_pickle=True)
        docs = [arr] if arr.ndim == 1 and arr.dtype != object else list(arr)
    else:
        obj = torch.load(path, weights_only=False)
        docs = obj if isinstance(obj, (list, tuple)) else ([obj] if obj.dim() == 1 else list(obj))
    for d in docs:
        yield [int(t) for t in (d.tolist() if hasattr(d, "tolist") else d)]


class PackedDocumentBatches:
    """Rows of packed documents from token files: yields dicts with ``input``, ``labels``, ``positions``
    (each ``[batch, seq_len]``). Resumable: the state is (file index, document index, leftover tokens)."""

    def __init__(self, pattern: str, batch_size: int, seq_len: int, rank: int = 0, world_size: int = 1,
                 bos_id: int = 0, eos_id: int = 1, loop: bool = True):
        files = sorted(glob.glob(pattern) if any(c in pattern for c in "*?[") else
                       ([pattern] if os.path.isfile(pattern) else glob.glob(os.path.join(pattern, "*"))))
        self.files = files[rank::world_size]
        if not self.files:
            raise FileNotFoundError(f"no token files for rank {rank} of {world_size} under {pattern!r}")
        self.batch_size, self.seq_len, self.bos_id, self.eos_id, self.loop = batch_size, seq_len, bos_id, eos_id, loop
        self.file_index, self.doc_index = 0, 0
        self.buffer = ([], [], [])      # tokens packed but not yet batched: inputs, labels, positions
        self._docs = None

    def _next_document(self):
        while True:
            if self._docs is None:
                if self.file_index >= len(self.files):
                    if not self.loop:
                        raise StopIteration
                    self.file_index = 0
                docs = _documents_of(self.files[self.file_index])
                for _ in range(self.doc_index):     # resume inside a file
                    next(docs, None)
                self._docs = docs
            doc = next(self._docs, None)
            if doc is not None:
                self.doc_index += 1
                return doc
            self._docs, self.doc_index = None, 0
            self.file_index += 1

    def __iter__(self):
        return self

    def __next__(self):
        needed = self.batch_size * self.seq_len
        while len(self.buffer[0]) < needed:
            ids = [self.bos_id, *self._next_document(), self.eos_id]
            self.buffer[0].extend(ids[:-1])
            self.buffer[1].extend(ids[1:])
            self.buffer[2].extend(i % self.seq_len for i in range(len(ids) - 1))
        batch = {}
        for key, values in zip(("input", "labels", "positions"), self.buffer):
            batch[key] = torch.tensor(values[:needed]).view(self.batch_size, self.seq_len)
            del values[:needed]
        return batch

    def state_dict(self):
        return copy.deepcopy({"file_index": self.file_index, "doc_index": self.doc_index, "buffer": self.buffer})

    def load_state_dict(self, sd):
        self.file_index, self.doc_index = int(sd["file_index"]), int(sd["doc_index"])
        self.buffer = tuple(list(v) for v in sd["buffer"])
        self._docs = None
