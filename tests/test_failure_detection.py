"""Failure detection without faulting a GPU: heartbeats over a store, a rank that leaves between
steps (gloo ranks on CPU), collective deadlines, and — on a GPU — a device-side wait that runs out and
reports through the status word while the context stays usable."""
import multiprocessing as mp
import socket
import time

import pytest
import torch

from axon_b200.utils.failure import CollectiveTimeout, Heartbeat, PeerLostError, guarded_collective


class DictStore(dict):
    def set(self, k, v):
        self[k] = v

    def get(self, k):
        return self[k]


def test_heartbeat_detects_silent_peer_with_fake_store():
    store = DictStore()
    a = Heartbeat(store, 0, 3, interval=0.05, timeout=0.4).start()
    b = Heartbeat(store, 1, 3, interval=0.05, timeout=0.4).start()
    c = Heartbeat(store, 2, 3, interval=0.05, timeout=0.4).start()
    time.sleep(0.2)
    a.check()
    c.stop()                                    # rank 2 goes silent
    deadline = time.time() + 3
    while time.time() < deadline and not a.lost_peers():
        time.sleep(0.05)
    with pytest.raises(PeerLostError) as ei:
        a.check()
    assert ei.value.ranks == [2]
    b.check() if not b.lost_peers() else None
    a.stop(), b.stop()


def test_guarded_collective_deadline():
    assert guarded_collective(lambda: 7, 1.0) == 7
    with pytest.raises(CollectiveTimeout):
        guarded_collective(lambda: time.sleep(5), 0.2, "sleepy")
    with pytest.raises(ValueError):
        guarded_collective(lambda: (_ for _ in ()).throw(ValueError("boom")), 1.0)


def _rank(rank, world, port, leave_after, q):
    import torch.distributed as dist
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), wait_for_workers=False)
    import datetime
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=3))
    hb = Heartbeat(dist.PrefixStore("hb", store), rank, world, interval=0.1, timeout=1.0).start()
    steps = 0
    try:
        for step in range(6):
            if rank == 1 and step == leave_after:      # leaves BETWEEN steps, nothing in flight
                hb.stop()
                q.put((rank, "left", steps))
                return
            time.sleep(0.5)
            hb.check()                                 # learn of a lost peer on the host, before the collective
            t = torch.ones(1)
            dist.all_reduce(t)
            steps += 1
        q.put((rank, "finished", steps))
    except PeerLostError as e:
        q.put((rank, "peer_lost", steps, e.ranks))
    except Exception as e:   # noqa: BLE001 - a short process-group timeout is the other legitimate outcome
        q.put((rank, "collective_error", steps, type(e).__name__))
    finally:
        hb.stop()


@pytest.mark.timeout(120)
def test_rank_leaving_between_steps_is_noticed_on_the_host():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, 2, q)) for r in range(2)]
    [p.start() for p in procs]
    out = {}
    for _ in range(2):
        item = q.get(timeout=60)
        out[item[0]] = item
    [p.join(20) for p in procs]
    assert out[1][1] == "left" and out[1][2] == 2
    assert out[0][1] in ("peer_lost", "collective_error") and out[0][2] == 2     # two steps together, then rank 0 stops cleanly
    if out[0][1] == "peer_lost":
        assert out[0][3] == [1]


@pytest.mark.gpu
def test_device_wait_times_out_and_context_survives():
    """A barrier kernel waits for a peer slot that nothing ever writes: after its bounded wait it
    records AXB_ERR_WAIT_PEER; the next kernels run normally."""
    import ctypes
    from axon_b200.ops import _common as C
    from axon_b200.ops import gemm as G
    dev = torch.device("cuda", 0)
    pads = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]     # "rank 1" never arrives
    arr = (ctypes.c_ulonglong * 2)(pads[0].data_ptr(), pads[1].data_ptr())
    C.check_status(dev)
    t0 = time.time()
    rc = C.lib().axb_peer_barrier(arr, 0, 2, ctypes.c_uint(1), C.ptr(C.status(dev)), C.stream())
    assert rc == 0
    with pytest.raises(C.NativeKernelError) as ei:
        C.check_status(dev)
    assert "5" in str(ei.value) and time.time() - t0 < 30
    assert int(pads[1][0]) == 1                                                  # our own arrival was published
    a = torch.randn(256, 256, device=dev).to(torch.bfloat16)
    out = G.gemm_nt(a, a)
    torch.cuda.synchronize()
    C.check_status(dev)
    assert (out.float() - a.float() @ a.float().t()).abs().max() < 1.0
