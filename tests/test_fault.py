"""Failure detection with host-made failures only: a rank that stops beating, dropped control messages, a device wait
on a flag that nobody sets (bounded: the kernel returns a status), corrupt / truncated files."""
import os

import pytest
import torch

from transformers_fusion_b200.parallel import fault


def test_heartbeat_detects_silent_rank_and_recovery():
    store = fault.DictStore()
    now = [100.0]
    events = []
    hbs = [fault.Heartbeat(store, r, 3, 1.0, 5.0, on_failure=lambda r_, me=r: events.append(("fail", me, r_)),
                           on_recovery=lambda r_, me=r: events.append(("rec", me, r_)), clock=lambda: now[0]) for r in range(3)]
    for h in hbs:
        h.beat()
    assert hbs[0].check_peers() == []
    hbs[2].paused = True                        # injected fault: rank 2 stops beating
    for _ in range(7):
        now[0] += 1.0
        for h in hbs:
            h.beat()
    assert hbs[0].check_peers() == [2] and hbs[1].check_peers() == [2]
    assert ("fail", 0, 2) in events and ("fail", 1, 2) in events
    hbs[2].paused = False
    hbs[2].beat()
    assert hbs[0].check_peers() == [] and ("rec", 0, 2) in events


def test_heartbeat_thread_and_lossy_store():
    inj = fault.FaultInjector(seed=1)
    inj.drop_prob = 1.0                          # every beat of rank 1 is lost in transit
    store = fault.DictStore()
    a = fault.Heartbeat(store, 0, 2, 0.05, 0.3).start()
    b = fault.Heartbeat(inj.wrap_store(store), 1, 2, 0.05, 0.3).start()
    import time
    time.sleep(0.7)
    a.stop(), b.stop()
    assert 1 in a.failed and inj.dropped > 3 and 0 not in b.failed


def test_manager_checkpoint_and_redistribution(tmp_path):
    m = fault.FaultToleranceManager()
    for i in range(4):
        m.add_node(fault.NodeInfo(i, "10.0.0.%d" % i, 9000 + i, 4))
    seen = []
    m.failure_cbs.append(seen.append)
    m.on_node_failure(2)
    m.on_node_failure(2)                          # idempotent
    m.stats["routed"] = 77
    assert seen == [2] and m.alive_nodes() == [0, 1, 3] and not m.check_node_health(2)
    text = m.checkpoint_state()
    assert text.startswith("nodes:4;failed:1;failed_node{2};node{0,10.0.0.0,9000,4}") and text.endswith("stats{routed=77,dropped=0,failures=1}")
    m.save(str(tmp_path / "ft.state"))
    m2 = fault.FaultToleranceManager()
    assert m2.load(str(tmp_path / "ft.state")) and m2.checkpoint_state() == text and m2.alive_nodes() == [0, 1, 3]
    assert not m2.restore_state("nodes:9;failed:0;stats{routed=0,dropped=0,failures=0}")
    fault.FaultInjector.truncate_file(str(tmp_path / "ft.state"), 0.4)
    assert not fault.FaultToleranceManager().load(str(tmp_path / "ft.state"))
    old = fault.redistribute_experts(16, [0, 1, 2, 3])
    new = fault.redistribute_experts(16, m.alive_nodes())
    assert [len(v) for v in new.values()] == [6, 5, 5] and sorted(sum(new.values(), [])) == list(range(16))
    moves = fault.compute_redistribution(old, new)
    assert all(src is None for e, src, dst in moves if e in old[2]) and len({e for e, _, _ in moves}) == len(moves)
    with pytest.raises(RuntimeError):
        fault.redistribute_experts(4, [])


def test_elastic_reshard():
    full = torch.arange(10000, dtype=torch.float32)
    old = list(torch.cat([full, torch.zeros(240)]).chunk(4))        # world 4, padded to 10240
    new = fault.reshard_flat(old, 3, pad_multiple=1024)
    assert len(new) == 3 and all(s.numel() == new[0].numel() for s in new) and new[0].numel() % 1024 == 0
    assert torch.equal(torch.cat(new)[:10000], full) and float(torch.cat(new)[10000:].abs().sum()) == 0


def test_corrupt_quant_block_detected(tmp_path):
    from transformers_fusion_b200.quant import codec
    w = codec.QuantWriter(tmp_path / "m.quant")
    w.add_tensor("a", torch.randn(4096))
    w.close()
    fault.FaultInjector.truncate_file(str(tmp_path / "m.quant"), 0.5)
    with pytest.raises((ValueError, KeyError)):
        codec.QuantReader(tmp_path / "m.quant").read_tensor("a")


@pytest.mark.gpu
def test_device_wait_times_out_with_status():
    """A device-side barrier whose peer never arrives: the kernel gives up after its bounded wait and reports it."""
    from transformers_fusion_b200.ops import _lib
    dev = torch.device("cuda")
    _lib.register("tfb_comm_barrier", [_lib.c_p, _lib.c_p, _lib.c_i, _lib.c_i, _lib.c_p, _lib.c_p])
    flags = torch.zeros(32, dtype=torch.int32, device=dev)           # world of 2, rank 1 is imaginary: its flag never moves
    ptrs = torch.tensor([flags.data_ptr(), flags.data_ptr()], dtype=torch.int64, device=dev)
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    fault.device_wait_status(dev)
    _lib.check(_lib.lib().tfb_comm_barrier(ptrs.data_ptr(), epoch.data_ptr(), 0, 2, _lib.status_word(dev).data_ptr(), _lib.stream()), "barrier")
    torch.cuda.synchronize()
    code, name = fault.device_wait_status(dev)
    assert name == "timeout_flag", (code, name)
    assert fault.device_wait_status(dev) == (0, "ok")
    x = torch.ones(8, device=dev) * 2                                  # the context is still usable
    assert float(x.sum()) == 16.0


@pytest.mark.gpu
def test_heap_reset_after_timed_out_wait():
    """After a bounded wait ran out, SymmetricHeap.reset() clears the status, tickets and accumulators, moves the epoch
    past anything in flight and leaves the heap usable (the failure is a flag that nothing sets; no GPU fault)."""
    from transformers_fusion_b200.ops import _lib
    from transformers_fusion_b200.parallel.symm import SymmetricHeap
    dev = torch.device("cuda", 0)
    heap = SymmetricHeap(0, 1, dev)
    ticket = torch.full((1,), 7, dtype=torch.int32, device=dev)        # a last-CTA counter left at a partial count
    heap.on_reset(ticket.zero_)
    fault.device_wait_status(dev)
    ptrs = torch.tensor([heap.flags.local_ptr, heap.flags.local_ptr], dtype=torch.int64, device=dev)   # imaginary rank 1
    _lib.check(_lib.lib().tfb_comm_barrier(ptrs.data_ptr(), heap.epoch.data_ptr(), 0, 2, _lib.status_word(dev).data_ptr(),
                                           _lib.stream()), "barrier")
    torch.cuda.synchronize()
    with pytest.raises(_lib.KernelError):
        _lib.check_status(dev, reset=False)
    e0 = int(heap.epoch.item())
    heap.reset()
    assert int(ticket.item()) == 0 and int(heap.epoch.item()) > e0 + 1000
    assert fault.device_wait_status(dev) == (0, "ok")
    heap.barrier()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    heap.close()
