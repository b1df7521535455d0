"""The peer-memory all-reduce as an operator on ONE GPU: a second region on the same device stands in for a peer. The
peer is either staged by hand as if it had arrived (what it would have stored into this rank's region, and its arrival
epochs, are written before the launch; nothing waits for another launch), or left silent so that the bounded wait runs out:
the launch must then give up with a status the host reads, and the runtime must keep working."""
import numpy as np
import pytest
import torch

import effect_torch_b200 as et
from tests.gpu_util import dev, host, runtime

pytestmark = pytest.mark.gpu

HEADER, FLAG_STRIDE = 4096, 8  # region layout: flag arrays of 8 words from byte 0, exchange buffers from byte 4096


class Region:
    """One rank's exchange region: per buffer an inbox of `world` slots and a table of totals, `capacity` floats each."""

    def __init__(self, capacity, world):
        self.capacity, self.world = capacity, world
        self.slot = (capacity * 4 + 255) // 256 * 256
        self.bytes = torch.zeros(et.peer_region_bytes(capacity, world), dtype=torch.uint8, device="cuda")
        assert self.bytes.numel() == HEADER + 2 * (world + 1) * self.slot
        torch.cuda.synchronize()

    def _floats(self, buffer, slot_index):
        start = HEADER + (buffer * (self.world + 1) + slot_index) * self.slot
        return self.bytes[start:start + self.capacity * 4].view(torch.float32)

    def inbox(self, buffer, sender, slot_floats=None):
        """Slot `sender` of the inbox: `capacity` floats apart for whole messages, packed `slot_floats` apart for slices."""
        if slot_floats is None:
            return self._floats(buffer, sender)
        start = HEADER + buffer * (self.world + 1) * self.slot + sender * slot_floats * 4
        return self.bytes[start:start + slot_floats * 4].view(torch.float32)

    def totals(self, buffer):
        return self._floats(buffer, self.world)

    @property
    def flags(self):
        return self.bytes[:96].view(torch.int32)


def test_a_single_rank_adds_its_own_partial_sum():
    rt = runtime()
    n = 4096
    rng = np.random.default_rng(0)
    h, p = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    hidden, partial, mine = dev(h), dev(p), Region(n, 1)
    rt.peer_allreduce_into(0, 1, [mine.bytes], n, 0, hidden, n, partial)
    np.testing.assert_array_equal(host(hidden), h + p)


@pytest.mark.parametrize("two_shot", [False, True])
def test_two_ranks_with_the_peer_staged_by_hand(two_shot):
    """Rank 0 of 2, buffer 1. Staged: what rank 1 stores into rank 0's inbox (its whole partial sum, or the first half of it
    when the message is cut in slices), the total of rank 1's slice in rank 0's table of totals, and rank 1's epochs."""
    rt = runtime()
    n = 8192
    rng = np.random.default_rng(1)
    h, p0, p1 = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    hidden, own, mine, peer = dev(h), dev(p0), Region(n, 2), Region(n, 2)
    total = p0 + p1
    half = n // 2
    if two_shot:
        mine.inbox(1, 1, half).copy_(torch.from_numpy(p1[:half]).cuda())
        mine.totals(1)[half:].copy_(torch.from_numpy(total[half:]).cuda())
    else:
        mine.inbox(1, 1).copy_(torch.from_numpy(p1).cuda())
    mine.flags[0 * FLAG_STRIDE + 1] = 1  # "rank 1 has stored its partial sums of epoch 1"
    mine.flags[1 * FLAG_STRIDE + 1] = 1  # "rank 1 has stored the total of its slice of epoch 1"
    torch.cuda.synchronize()
    rt.peer_allreduce_into(0, 2, [mine.bytes, peer.bytes], n, 1, hidden, n, own, two_shot=two_shot)
    np.testing.assert_array_equal(host(hidden), h + total)
    # what rank 0 stored into the peer's region, and the epochs it published there
    if two_shot:
        np.testing.assert_array_equal(peer.inbox(1, 0, half).cpu().numpy(), p0[half:])
        np.testing.assert_array_equal(peer.totals(1)[:half].cpu().numpy(), total[:half])
    else:
        np.testing.assert_array_equal(peer.inbox(1, 0).cpu().numpy(), p0)
    assert int(peer.flags[0 * FLAG_STRIDE + 0]) == 1
    assert int(peer.flags[1 * FLAG_STRIDE + 0]) == (1 if two_shot else 0)


@pytest.mark.parametrize("two_shot", [False, True])
def test_a_peer_that_never_arrives_turns_into_an_execution_error_and_the_runtime_stays_usable(two_shot):
    rt = runtime()
    n = 4096
    h = np.arange(n, dtype=np.float32)
    hidden, mine, silent, ones = dev(h), Region(n, 2), Region(n, 2), dev(np.ones(n, np.float32))
    rt.peer_allreduce_into(0, 2, [mine.bytes, silent.bytes], n, 0, hidden, n, ones, two_shot=two_shot,
                           wait_cycles=4_000_000)  # about two milliseconds
    with pytest.raises(et.BackendError) as err:
        rt.synchronize()
    assert err.value.reason == "execution-failed" and "peer never arrived" in str(err.value)
    np.testing.assert_array_equal(hidden.cpu().numpy(), h)  # nothing was added
    # the context is intact: the same operator on a fresh region, and an unrelated operator, both work
    again = Region(n, 1)
    rt.peer_allreduce_into(0, 1, [again.bytes], n, 0, hidden, n, ones)
    np.testing.assert_array_equal(host(hidden), h + 1)
    out = torch.zeros(n, device="cuda")
    torch.cuda.synchronize()
    rt.add_into(hidden, hidden, n, out)
    np.testing.assert_array_equal(host(out), 2 * (h + 1))


def test_a_decoder_step_whose_peer_never_arrives_is_rolled_back():
    """Rank 0 of a two-rank decoder on one GPU; the peer's region is a zeroed buffer nobody drives. The first all-reduce of
    the step runs out of its (shortened) wait, execute raises execution-failed, and the transaction is undone: the cursor
    has not moved, the pages went back to the pool, and the runtime serves an ordinary decoder afterwards."""
    import oracle as orc
    from effect_torch_b200 import tensor_parallel as tp
    from tests import helpers

    rt = runtime()
    cfg = helpers.TINY_Q
    weights = helpers.make_weights(cfg, seed=5, codec=orc.Q4_0)
    local = tp.local_config(cfg, 2)

    def build(c, w):
        dec = et.Executable(rt, layers=c["layers"], d_model=c["d_model"], q_heads=c["q_heads"], kv_heads=c["kv_heads"],
                            head_dim=c["head_dim"], ffn=c["ffn"], vocab=c["vocab"], rms_eps=c["rms_eps"], rope_theta=c["rope_theta"],
                            batch=2, max_tokens=256, block_size=16, kv_dtype=et.KV_F16, exact=False, max_advance=4)
        helpers.load_into(dec, w)
        dec.finalize()
        return dec

    dec = build(local, tp.shard_weights(weights, cfg, 0, 2))
    dec.set_tensor_parallel(0, 2, None)  # no communicator: peer regions only
    _, size = dec.peer_region()
    silent = torch.zeros(size, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    dec.attach_peer_regions([None, silent])
    dec.set_wait_limit(2_000_000)  # about a millisecond per all-reduce
    pool = et.NativeKvPool(rt, local["layers"], local["kv_heads"], local["head_dim"], 256, 16, et.KV_F16)
    seqs = [pool.makeSequence() for _ in range(2)]
    free_before = pool._stats()
    toks = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.uint32)
    for _ in range(2):  # the failure repeats and leaves the same state behind
        with pytest.raises(et.BackendError) as err:
            dec.executeSampled(pool, seqs, toks)
        assert err.value.reason == "execution-failed" and "peer never arrived" in str(err.value)
        assert [s.cursor for s in seqs] == [0, 0]
        assert pool._stats() == free_before
    dec.close()
    # the runtime is intact: the whole model on this device decodes as usual
    whole = build(cfg, weights)
    pool2 = et.NativeKvPool(rt, cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 256, 16, et.KV_F16)
    seqs2 = [pool2.makeSequence() for _ in range(2)]
    out = whole.executeSampled(pool2, seqs2, toks)
    assert out.shape == (2,) and [s.cursor for s in seqs2] == [3, 3]
