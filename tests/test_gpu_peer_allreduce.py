"""The peer-memory all-reduce as an operator on ONE GPU: a second region on the same device stands in for a peer. The
peer is either staged by hand as if it had arrived (its flags and buffers pre-set; nothing waits for another launch), or
left silent so that the bounded wait runs out: the launch must then give up with a status the host reads, and the runtime
must keep working. No launch here waits for another launch."""
import numpy as np
import pytest
import torch

import effect_torch_b200 as et
from tests.gpu_util import dev, host, runtime

pytestmark = pytest.mark.gpu

HEADER, FLAG_STRIDE = 4096, 8  # region layout: flag arrays of 8 words from byte 0, partial buffers from byte 4096


def region(capacity):
    t = torch.zeros(et.peer_region_bytes(capacity), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    return t


def partial_view(reg, capacity, buffer):
    stride = (capacity * 4 + 255) // 256 * 256
    return reg[HEADER + buffer * stride:HEADER + buffer * stride + capacity * 4].view(torch.float32)


def flags(reg):
    return reg[:96].view(torch.int32)


def test_a_single_rank_adds_its_own_partial_sum():
    rt = runtime()
    n = 4096
    rng = np.random.default_rng(0)
    h, p = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    hidden, partial, mine = dev(h), dev(p), region(n)
    rt.peer_allreduce_into(0, 1, [mine], n, 0, hidden, n, partial=partial)
    np.testing.assert_array_equal(host(hidden), h + p)


@pytest.mark.parametrize("two_shot", [False, True])
def test_two_ranks_with_the_peer_staged_by_hand(two_shot):
    """Rank 0 of 2. The peer's region holds its partial sum, and (two shot) the total of the peer's slice where its own
    reduction would have left it; its arrival epochs are written into rank 0's flag arrays before the launch."""
    rt = runtime()
    n = 8192
    rng = np.random.default_rng(1)
    h, p0, p1 = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    hidden, mine, peer = dev(h), region(n), region(n)
    total = p0 + p1
    staged = p1.copy()
    if two_shot:
        staged[n // 2:] = total[n // 2:]  # the peer owns the second half of the message
    partial_view(peer, n, 1).copy_(torch.from_numpy(staged).cuda())
    f = flags(mine)
    f[0 * FLAG_STRIDE + 1] = 1  # "rank 1's partial of epoch 1 is complete"
    f[1 * FLAG_STRIDE + 1] = 1  # "rank 1's slice total of epoch 1 is complete"
    torch.cuda.synchronize()
    own = dev(p0)
    rt.peer_allreduce_into(0, 2, [mine, peer], n, 1, hidden, n, partial=own, two_shot=two_shot)
    np.testing.assert_array_equal(host(hidden), h + total)
    if two_shot:  # rank 0 left the total of its own slice where the peer would read it
        np.testing.assert_array_equal(partial_view(mine, n, 1)[:n // 2].cpu().numpy(), total[:n // 2])
    # rank 0 told the peer about both of its phases
    assert int(flags(peer)[0 * FLAG_STRIDE + 0]) == 1
    assert int(flags(peer)[1 * FLAG_STRIDE + 0]) == (1 if two_shot else 0)


@pytest.mark.parametrize("two_shot", [False, True])
def test_a_peer_that_never_arrives_turns_into_an_execution_error_and_the_runtime_stays_usable(two_shot):
    rt = runtime()
    n = 4096
    h = np.arange(n, dtype=np.float32)
    hidden, mine, silent, ones = dev(h), region(n), region(n), dev(np.ones(n, np.float32))
    rt.peer_allreduce_into(0, 2, [mine, silent], n, 0, hidden, n, partial=ones, two_shot=two_shot,
                           wait_cycles=4_000_000)  # about two milliseconds
    with pytest.raises(et.BackendError) as err:
        rt.synchronize()
    assert err.value.reason == "execution-failed" and "peer never arrived" in str(err.value)
    np.testing.assert_array_equal(hidden.cpu().numpy(), h)  # nothing was added
    # the context is intact: the same operator on a fresh region, and an unrelated operator, both work
    again = region(n)
    rt.peer_allreduce_into(0, 1, [again], n, 0, hidden, n, partial=ones)
    np.testing.assert_array_equal(host(hidden), h + 1)
    out = torch.zeros(n, device="cuda")
    rt.add_into(hidden, hidden, n, out)
    np.testing.assert_array_equal(host(out), 2 * (h + 1))
