"""``Shard`` buckets against PyTorch FSDP2 ``fully_shard`` on gloo ranks: losses, gradients, parameters
and the bytes handed to every collective, bit for bit, over the 24-configuration matrix (4 dtype
policies x 2 divide factors x 3 accumulation modes) at 2 and 4 ranks, plus the chunked-loss and
head-called-twice variants.  4 ranks make the summation order observable; because both sides hand the
same bytes to the same collective, the results agree whatever order the backend sums in."""
import pytest
import torch

from tests import fsdp2_parity_common as pc
from tests.common import run_ranks


def _matrix(rank, world, variant, only):
    from torch.distributed.device_mesh import init_device_mesh

    mesh = init_device_mesh("cpu", (world,))
    bad = []
    cfgs = pc.configs()
    if only is not None:
        cfgs = [cfgs[i] for i in only]
    for cfg in cfgs:
        # The head variants compare values only. Chunked: the library follows the reference's documented
        # schedule (the head reduces its weight after the last chunk, the norm's gradient goes with the
        # trunk's backward) while the installed FSDP2 reduces the two in one later collective. Head called
        # twice: the installed FSDP2 reshards the group after each call's backward and gathers it again
        # for the other call; here the group stays gathered until both calls are done. Same sums either way.
        bad += pc.run_pair(torch.device("cpu"), mesh, rank, cfg, steps=2, variant=variant,
                           record=variant == "plain")
    return bad


@pytest.mark.parametrize("world", [2, 4])
def test_matrix_bitwise_equal_to_fsdp2(world):
    res = run_ranks(_matrix, world, "plain", None, timeout=900)
    bad = [m for r in res for m in r]
    assert not bad, "\n".join(bad[:40])


# Indices into ``configs()``: 6 per dtype policy = 2 factors x 3 accumulation modes.
# head_twice: every dtype policy with one microbatch, and bf16/fp32 with no-sync microbatches.
# chunked: the head's chunks accumulate without reduction while the norm's gradient only arrives with
# the trunk's backward; with a reduce dtype wider than the compute dtype the installed FSDP2 then
# refuses the group's mixed gradient dtypes, so that policy is left to the library's own chunked test.
_VARIANTS = {"head_twice": [0, 6, 12, 18, 8], "chunked": [0, 3, 12, 13, 18]}


@pytest.mark.parametrize("variant", ["chunked", "head_twice"])
def test_head_variants_bitwise_equal_to_fsdp2(variant):
    res = run_ranks(_matrix, 4, variant, _VARIANTS[variant], timeout=900)
    bad = [m for r in res for m in r]
    assert not bad, "\n".join(bad[:40])
