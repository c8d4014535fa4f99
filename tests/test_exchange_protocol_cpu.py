"""A model of the peer exchange's protocol (alignedkv_b200/csrc/akv_exchange.cuh) with threads for ranks: every rank
stores (value, epoch) words into slot `rank` of every rank's buffer and then reads the words of all ranks from its own
buffer until each carries the step's epoch.  Buffers are two epochs deep (index = epoch & 1).  The model checks what
the kernel relies on: with ranks that run at random, different speeds, a word of step k+1 never replaces a word of
step k-1 that somebody still waits for (no reader ever runs into its time limit, every value read is the one its
writer published for that step), also across the wrap of the epoch counter."""
import random
import threading
import time

import pytest


def next_epoch(e):
    return e % 0x7FFFFFFE + 1          # sharded.PeerExchange.next_epoch


@pytest.mark.parametrize("world,start_epoch", [(2, 0), (4, 0), (8, 0), (3, 0x7FFFFFFE - 5)])
def test_two_epochs_deep_is_enough(world, start_epoch):
    steps, limit_s = 60, 5.0
    bufs = [[[(None, 0)] * world for _ in range(2)] for _ in range(world)]     # bufs[rank][parity][source]
    failures = []

    def rank_main(r):
        rng = random.Random(1000 + r)
        epoch = start_epoch
        for k in range(steps):
            epoch = next_epoch(epoch)
            par = epoch & 1
            time.sleep(rng.random() * 0.002)                    # the step's own work, a different time on every rank
            for g in rng.sample(range(world), world):           # publish: one atomic word per destination
                bufs[g][par][r] = ((r, k), epoch)
                if rng.random() < 0.2:
                    time.sleep(rng.random() * 0.001)
            t0 = time.time()
            for g in range(world):                              # collect from the own buffer
                while True:
                    value, e = bufs[r][par][g]
                    if e == epoch:
                        break
                    if time.time() - t0 > limit_s:
                        failures.append(f"rank {r} step {k}: word of rank {g} carries epoch {e}, not {epoch}")
                        return
                    time.sleep(0)
                if value != (g, k):
                    failures.append(f"rank {r} step {k}: read {value} from rank {g}")
                    return

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not failures, failures[:3]


def test_epoch_sequence_never_zero_and_alternates():
    from alignedkv_b200.sharded import PeerExchange

    class Counter:
        epoch = 0x7FFFFFFE - 3

    c, e, seen = Counter(), 0x7FFFFFFE - 3, []
    for _ in range(8):
        e = next_epoch(e)
        assert PeerExchange.next_epoch(c) == e          # the model's counter is the library's
        seen.append(e)
    assert all(x != 0 for x in seen)
    assert all((a & 1) != (b & 1) for a, b in zip(seen, seen[1:]))
