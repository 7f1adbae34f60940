"""The one-shot peer-memory all-reduce (tq_comm_enable_peer / tq_comm_peer_local) on ONE GPU, with the test playing
the peer: it writes the other rank's partial and flag into rank 0's buffer from the host, so the kernel's arithmetic,
slot addressing, sequence numbers and parity are checked without a second GPU, and a peer that never arrives is
shown to end in TQ_ETIMEOUT (a bounded wait running out: nothing hangs, nothing traps).  The real two-GPU path runs in
tests/test_tp.py."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture()
def dev():
    import tang_b200

    d = tang_b200.QuantComputeDevice(0)
    yield d
    d.close()


def _setup(dev, world, max_elems):
    import tang_b200 as tb

    nbytes = dev._L.tq_comm_peer_bytes(world, max_elems)
    assert nbytes == (2 * world * max_elems + 2 * world) * 4
    bufs = [dev.alloc(nbytes // 4, tb.F32) for _ in range(world)]
    for b in bufs:
        dev.memset(b)
    dev.sync()
    return bufs


def _poke(dev, buf, float_offset, array):
    a = np.ascontiguousarray(array)
    dev._check(dev._L.tq_upload(dev._ctx, buf.ptr + 4 * float_offset, a.ctypes.data, a.nbytes))


def test_sum_with_the_host_playing_rank_one(dev):
    import tang_b200 as tb

    world, max_elems, n = 2, 1024, 1000
    bufs = _setup(dev, world, max_elems)
    comm = tb.Comm.peer_local(dev, 0, world, bufs, max_elems)
    rng = np.random.default_rng(0)
    flags0 = 2 * world * max_elems
    for call in (1, 2, 3):                    # sequence numbers 1, 2, 3 -> parities 1, 0, 1
        parity = call & 1
        mine = rng.standard_normal(n).astype(np.float32)
        theirs = rng.standard_normal(n).astype(np.float32)
        _poke(dev, bufs[0], (parity * world + 1) * max_elems, theirs)          # rank 1's partial, in rank 0's buffer
        _poke(dev, bufs[0], flags0 + parity * world + 1, np.array([call], np.int32))   # ... and its flag
        x = dev.upload(mine)
        comm.all_reduce(x)
        dev.sync()
        assert np.array_equal(x.to_vec(), mine + theirs)                       # rank order: 0 then 1, one f32 addition
        # what rank 0 stored for its peer: its partial in slot (parity, 0) of rank 1's buffer, and the flag
        peer_view = bufs[1].to_vec()
        assert np.array_equal(peer_view[(parity * world) * max_elems:(parity * world) * max_elems + n], mine)
        assert peer_view.view(np.int32)[flags0 + parity * world + 0] == call
    comm.destroy()


def test_a_peer_that_never_arrives_times_out(dev):
    import tang_b200 as tb

    world, max_elems, n = 2, 256, 256
    bufs = _setup(dev, world, max_elems)
    comm = tb.Comm.peer_local(dev, 0, world, bufs, max_elems)
    comm.set_wait_limit(2000)                 # a few milliseconds instead of seconds
    mine = np.arange(n, dtype=np.float32)
    x = dev.upload(mine)
    comm.all_reduce(x)                        # rank 1's flag is never raised
    with pytest.raises(tb.TangqError) as e:
        dev.sync()
    assert e.value.status == tb._lib.TQ_ETIMEOUT
    assert np.array_equal(x.to_vec(), mine)   # the output keeps this rank's own partial
    # the context is usable afterwards
    y = dev.upload(np.ones(8, np.float32))
    dev.sync()
    assert y.to_vec().sum() == 8
    comm.destroy()


def test_argument_errors(dev):
    import tang_b200 as tb

    bufs = _setup(dev, 2, 64)
    with pytest.raises(tb.TangqError):
        tb.Comm.peer_local(dev, 2, 2, bufs, 64)          # rank outside the world
    with pytest.raises(tb.TangqError):
        tb.Comm.peer_local(dev, 0, 2, bufs, 63)          # max_elems not a multiple of 4
    assert dev._L.tq_comm_peer_bytes(9, 64) == 0          # more ranks than the path supports
