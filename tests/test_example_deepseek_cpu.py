"""The DeepSeek-V3 example end to end on two gloo ranks (``--small``): a run interrupted by a checkpoint and
resumed prints the same losses as the uninterrupted run, for AdamW and for Muon (whose momentum buffers are
part of the checkpoint).  Behaviour restated from ``src/flex_shard/tests/test_example_deepseek_v3.py:448-503``."""
import json
import os
import shutil
import subprocess
import sys

import pytest

from tests.common import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(ckpt_dir, extra):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "examples", "deepseek_v3", "train.py"),
           "--small", "--steps", "4", "--seq-len", "32", "--local-batch-size", "2", "--ep", "2", "--checkpoint-dir",
           ckpt_dir, "--checkpoint-interval", "2", *extra]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    recs = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{") and '"step"' in l]
    return {r["step"]: r for r in recs}


@pytest.mark.parametrize("optimizer", ["adamw", "muon"])
def test_resume_equals_uninterrupted_run(tmp_path, optimizer):
    full_dir, part_dir = str(tmp_path / "full"), str(tmp_path / "part")
    full = _run(full_dir, ["--optimizer", optimizer])
    assert sorted(full) == [0, 1, 2, 3]
    os.makedirs(part_dir)
    shutil.copytree(os.path.join(full_dir, "step00000002"), os.path.join(part_dir, "step00000002"))
    resumed = _run(part_dir, ["--optimizer", optimizer])
    assert sorted(resumed) == [2, 3], resumed
    for s in (2, 3):
        assert resumed[s]["loss"] == full[s]["loss"], (s, resumed[s], full[s])
        assert resumed[s]["grad_norm"] == full[s]["grad_norm"]
        assert resumed[s]["lr"] == full[s]["lr"]


def test_init_checkpoint_document_mask_and_balance_loss_flags(tmp_path):
    """``--init-checkpoint`` starts from saved weights with fresh optimizers and data position; the document
    mask, the balance loss and explicit prefetch lists run end to end (activation checkpointing is on by default)."""
    first = _run(str(tmp_path / "a"), ["--optimizer", "adamw"])
    warm = _run(str(tmp_path / "b"), ["--optimizer", "adamw", "--init-checkpoint", str(tmp_path / "a" / "step00000002"),
                                      "--document-length", "8", "--aux-loss-coeff", "0.01"])
    assert sorted(warm) == [0, 1, 2, 3]
    assert warm[0]["loss"] != first[0]["loss"]          # not the random initial weights
    plain = _run(str(tmp_path / "c"), ["--optimizer", "adamw", "--no-activation-checkpointing", "--no-explicit-prefetch"])
    assert [plain[s]["loss"] for s in range(4)] == [first[s]["loss"] for s in range(4)]   # recompute and prefetch lists change no value


def test_packed_document_batches_pack_label_and_resume(tmp_path):
    import numpy as np
    import torch

    sys.path.insert(0, os.path.join(ROOT, "examples", "deepseek_v3"))
    from data import PackedDocumentBatches

    docs = [np.arange(10, 15), np.arange(20, 23), np.arange(30, 41)]
    np.save(tmp_path / "a.npy", np.array(docs, dtype=object), allow_pickle=True)
    torch.save([torch.arange(50, 54)], tmp_path / "b.pt")
    ds = PackedDocumentBatches(str(tmp_path), batch_size=1, seq_len=8, bos_id=0, eos_id=1, loop=False)
    b0 = next(ds)
    # [BOS 10..14 EOS] [BOS 20..22 EOS]: inputs drop each document's last token, labels its first
    assert b0["input"].tolist() == [[0, 10, 11, 12, 13, 14, 0, 20]]
    assert b0["labels"].tolist() == [[10, 11, 12, 13, 14, 1, 20, 21]]
    assert b0["positions"].tolist() == [[0, 1, 2, 3, 4, 5, 0, 1]]
    state = ds.state_dict()
    b1 = next(ds)
    assert b1["positions"].tolist()[0][:2] == [2, 3] and b1["positions"].tolist()[0][2] == 0   # the document continues, then a new one
    again = PackedDocumentBatches(str(tmp_path), batch_size=1, seq_len=8, bos_id=0, eos_id=1, loop=False)
    again.load_state_dict(state)
    resumed = next(again)
    assert all(torch.equal(resumed[k], b1[k]) for k in b1)
    # files are split across ranks
    r1 = PackedDocumentBatches(str(tmp_path), batch_size=1, seq_len=4, rank=1, world_size=2, loop=True)
    assert next(r1)["input"].tolist() == [[0, 50, 51, 52]]


@pytest.mark.parametrize("split", ["head", "role"])
def test_muon_head_block_storage_trains_like_owner_storage(tmp_path, split):
    """Per-head matrices stored in head blocks over the ranks (BlockShard by attention head) or whole on owners:
    the same per-head Newton-Schulz either way, so the same losses; also with every head cut into its roles
    (no-position / rotary / value rows as matrices of their own)."""
    # clipping off: the global gradient norm is summed in storage order, its last bit differs between the two
    # layouts, and Newton-Schulz rounds its input to bf16, which turns that bit into visible differences
    common = ["--optimizer", "muon", "--max-norm", "1e9", "--muon-split", split]
    owners = _run(str(tmp_path / "o"), common)
    heads = _run(str(tmp_path / "h"), [*common, "--muon-storage", "heads"])
    assert [heads[s]["loss"] for s in range(4)] == [owners[s]["loss"] for s in range(4)]


def test_training_on_packed_document_files_resumes_bitwise(tmp_path):
    """``--data files``: documents from local token files, packed with per-document positions (document-masked
    attention) and split across ranks file by file; a run resumed from its checkpoint continues with the same
    batches and prints the same losses."""
    import numpy as np

    rng = np.random.default_rng(0)
    files = tmp_path / "tokens"
    files.mkdir()
    for f in range(4):                                   # two files per rank, ragged documents
        docs = np.empty(12, dtype=object)
        for i in range(12):
            docs[i] = rng.integers(2, 256, size=int(rng.integers(5, 40)))
        np.save(files / f"part{f}.npy", docs, allow_pickle=True)
    extra = ["--optimizer", "adamw", "--data", "files", "--data-files", str(files)]
    full_dir, part_dir = str(tmp_path / "full"), str(tmp_path / "part")
    full = _run(full_dir, extra)
    assert sorted(full) == [0, 1, 2, 3]
    os.makedirs(part_dir)
    shutil.copytree(os.path.join(full_dir, "step00000002"), os.path.join(part_dir, "step00000002"))
    resumed = _run(part_dir, extra)
    assert sorted(resumed) == [2, 3]
    for s in (2, 3):
        assert resumed[s]["loss"] == full[s]["loss"] and resumed[s]["grad_norm"] == full[s]["grad_norm"]
