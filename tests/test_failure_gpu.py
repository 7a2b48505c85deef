"""GPU (one GPU is enough): what the library does when something is wrong, without faulting, trapping or hanging.

* a peer GPU that never publishes its flag: the exchange kernel's bounded wait runs out after the limit set with
  lb_set_wait_limit, the kernel RETURNS, the status word reads 0x1003 and the host gets LB_ERR_DEVICE_WAIT; the next
  exchange returns at once; after the status is cleared and the peer answers, an exchange succeeds.  The silent peer is
  a local buffer standing in for rank 1 (lb_comm_set_peer): no second process, nothing removed while in use.
  The reference's bounded wait traps the GPU (runtime/sync.ls:50-60); this one reports.
* the same through the decode step of a 2-way tensor-parallel shard whose peer is silent;
* a replay that would run past the KV cache is refused on the host before anything is launched."""
import ctypes as C
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
LIMIT_NS = 5_000_000   # 5 ms


def silent_pair(ctx, lb, n_max):
    from lithos_b200 import tp
    comm = tp.Comm(ctx, 0, 2, n_max)
    peer = ctx.alloc(comm.nbytes + 256)
    peer.zero()
    base = (peer.ptr + 255) & ~255
    comm.set_peer(1, base)
    return comm, peer, base


def test_silent_peer_times_out_reports_and_recovers(ctx, lb):
    n = 5120
    comm, peer, base = silent_pair(ctx, lb, n)
    x = ctx.to_device(np.ones(n, np.float32))
    mine = np.full(n, 2.0, np.float32)
    lb.lib().lb_memcpy_h2d(ctx.h, comm.buffer + comm.partial_offset(0, 0), mine.ctypes.data_as(C.c_void_p), mine.nbytes)   # rank 0's partial, slot 0
    theirs = np.full(n, 3.0, np.float32)
    lb.lib().lb_memcpy_h2d(ctx.h, base + comm.partial_offset(0, 1), theirs.ctypes.data_as(C.c_void_p), theirs.nbytes)      # "rank 1"'s partial, slot 0
    ctx.sync()
    ctx.set_wait_limit(LIMIT_NS)
    t0 = time.perf_counter()
    comm.allreduce(x, n, 0)
    with pytest.raises(lb.LithosError) as e:
        ctx.device_status()
    first = time.perf_counter() - t0
    assert e.value.status == lb.LB_ERR_DEVICE_WAIT and "0x1003" in str(e.value)
    assert first < 1.0                                              # the 5 ms limit, not the built-in 2 s
    assert np.array_equal(x.download(np.float32, n), np.ones(n, np.float32))   # nothing was added
    # the status word was cleared by the read above; a second silent exchange fails the same way ...
    comm.allreduce(x, n, 1)
    ctx.sync()
    # ... and while the word is still set, a third one does not wait at all
    t0 = time.perf_counter()
    comm.allreduce(x, n, 0)
    ctx.sync()
    assert time.perf_counter() - t0 < 0.004
    with pytest.raises(lb.LithosError):
        ctx.device_status()
    # recovery: the peer "answers" (its generation word reaches ours), the status is clear
    ctx.reset_status()
    gen = np.array([1 << 20], np.uint32)                            # far ahead of any generation used so far
    lb.lib().lb_memcpy_h2d(ctx.h, comm.buffer + comm.flags_offset + 4, gen.ctypes.data_as(C.c_void_p), 4)   # my_flags[1]
    ctx.sync()
    comm.allreduce(x, n, 0)
    assert ctx.device_status() == 0
    assert np.array_equal(x.download(np.float32, n), np.full(n, 6.0, np.float32))   # 1 + 2 + 3, rank order
    ctx.set_wait_limit(0)
    comm.close()
    peer.free()
    x.free()


def test_decode_step_with_a_silent_peer_reports(ctx, lb):
    from lithos_b200 import model as M, tp
    cfg = M.tiny(max_ctx=16)
    comm, peer, _ = silent_pair(ctx, lb, cfg.hidden)
    m = M.Model(ctx, cfg, 0, 2)
    tp.attach(m, comm)
    m.fill_synthetic(5)
    ctx.set_wait_limit(LIMIT_NS)
    t0 = time.perf_counter()
    with pytest.raises(lb.LithosError) as e:
        m.decode(3, 0)
    assert e.value.status == lb.LB_ERR_DEVICE_WAIT and "0x1003" in str(e.value)
    assert time.perf_counter() - t0 < 2.0          # one limit, not one per exchange of the step
    ctx.set_wait_limit(0)
    ctx.reset_status()
    ctx.sync()
    m.close()
    comm.close()
    peer.free()
    # the context is still usable: a single-GPU model decodes normally afterwards
    m1 = M.Model(ctx, cfg)
    m1.fill_synthetic(5)
    assert 0 <= m1.decode(3, 0) < cfg.vocab
    assert ctx.device_status() == 0
    m1.close()


def test_replay_past_the_context_is_refused_before_launch(ctx, lb):
    from lithos_b200 import model as M
    cfg = M.tiny(max_ctx=8)
    m = M.Model(ctx, cfg)
    m.fill_synthetic(5)
    m.capture()
    m.set_input(1, 5)
    ctx.reset_launches()
    with pytest.raises(lb.LithosError) as e:
        m.replay(4)                                  # positions 5, 6, 7, 8: the last one has no cache row
    assert e.value.status == lb.LB_ERR_INVALID and ctx.launches == 0
    m.replay(3)                                      # 5, 6, 7 fit
    assert 0 <= m.read_next() < cfg.vocab
    with pytest.raises(lb.LithosError):
        m.replay(1)
    with pytest.raises(lb.LithosError):
        m.set_input(1, 8)
    m.close()
