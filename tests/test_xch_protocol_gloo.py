"""The peer-store exchange protocol, stepped through on CPU by two gloo ranks.

The device code (csrc/kernels.cuh: XchPeers, xch_number, xch_wait_flags, xch_sum4, the EPI_PEERS
epilogue) keeps, per rank, one buffer of ``slots[2 parities][ranks][row]``, ``flags[ranks][tiles]``
and a token counter.  A producer stores its tile's partial sums into slot (e & 1, its rank) of every
rank's buffer and then sets flags[its rank][tile] = e there; a consumer waits, with a budget, until
all flags of its own buffer have reached e and adds the slots in rank order.  Exchanges are numbered
e = (token - 1) * exchanges_per_token + index + 1 on every rank alike.

Here each rank's buffer lives in shared memory that the other process maps, like a peer mapping,
and the same steps run in Python.  What is pinned: the numbering, that two parities suffice, the
rank-ordered sum, that a rank which arrives late is simply waited for, and that a rank which skips
one contribution makes its peer's wait run out (an error is reported, nothing blocks for good)
while the following token is healthy again because every rank still runs every later exchange.
No GPU is involved and nothing here is on the product path.
"""
import os
import socket
import time
from multiprocessing import shared_memory

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

TILES, TILE, WORLD = 4, 128, 2
ROW = TILES * TILE
PER_TOKEN = 4  # two layers: wo and down each


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class Buf:
    """One rank's exchange buffer: slots, flags, token counter."""

    def __init__(self, name, create):
        n = 2 * WORLD * ROW * 4 + WORLD * TILES * 4 + 4
        self.shm = shared_memory.SharedMemory(name=name, create=create, size=n)
        if create:
            self.shm.buf[:n] = bytes(n)
        self.slots = np.ndarray((2, WORLD, ROW), np.float32, self.shm.buf, 0)
        self.flags = np.ndarray((WORLD, TILES), np.uint32, self.shm.buf, 2 * WORLD * ROW * 4)
        self.tok = np.ndarray((1,), np.uint32, self.shm.buf, 2 * WORLD * ROW * 4 + WORLD * TILES * 4)

    def close(self, unlink):
        del self.slots, self.flags, self.tok
        self.shm.close()
        if unlink:
            self.shm.unlink()


def number(tok, index):
    return np.uint32((int(tok) - 1) * PER_TOKEN + index + 1)


def produce(bufs, rank, e, part, skip=False):
    """EPI_PEERS: per tile, rows into every rank's slot, then the flag (release order)."""
    if skip:
        return
    for t in range(TILES):
        for b in bufs:
            b.slots[int(e) & 1, rank, t * TILE:(t + 1) * TILE] = part[t * TILE:(t + 1) * TILE]
        for b in bufs:
            b.flags[rank, t] = e


def consume(mine, e, resid, budget_s):
    """xch_wait_flags + xch_sum4: bounded wait, then residual + (slot 0 + slot 1 + ...) in rank order."""
    t0 = time.perf_counter()
    ok = True
    while True:
        if np.all((mine.flags.astype(np.int64) - int(e)).astype(np.int32) >= 0):
            break
        if time.perf_counter() - t0 > budget_s:
            ok = False
            break
        time.sleep(0.0005)
    s = np.zeros(ROW, np.float32)
    for r in range(WORLD):
        s = (s + mine.slots[int(e) & 1, r]).astype(np.float32)
    return (resid + s).astype(np.float32), ok


def _worker(rank, port, tag, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    mine = Buf(f"apkx{tag}r{rank}", True)
    dist.barrier()
    bufs = [mine if r == rank else Buf(f"apkx{tag}r{r}", False) for r in range(WORLD)]
    dist.barrier()
    results = []
    rng = np.random.default_rng(5)
    parts = rng.standard_normal((6, PER_TOKEN, WORLD, ROW)).astype(np.float32)  # [token][exchange][rank]
    x = np.zeros(ROW, np.float32)
    for tok_i in range(6):
        mine.tok[0] += 1  # the token's first launch
        for idx in range(PER_TOKEN):
            e = number(mine.tok[0], idx)
            late = tok_i == 1 and idx == 2 and rank == 1       # a rank that is merely slow
            skip = tok_i == 3 and idx == 1 and rank == 1       # a rank that never delivers this one
            if late:
                time.sleep(0.15)
            produce(bufs, rank, e, parts[tok_i, idx, rank], skip=skip)
            # (the rank that skipped keeps waiting a little longer than its peer, so that the peer's
            # wait really runs out before the next exchange's flags overtake this one's)
            budget = 2.0 if not (tok_i == 3 and idx == 1) else (0.1 if rank == 0 else 0.4)
            x_new, ok = consume(mine, e, x, budget_s=budget)
            want = (x + ((np.zeros(ROW, np.float32) + parts[tok_i, idx, 0]) + parts[tok_i, idx, 1])).astype(np.float32)
            results.append((tok_i, idx, bool(ok), bool(np.array_equal(x_new, want))))
            x = want  # carry the right row on, so later exchanges are judged on their own
        dist.barrier()  # tokens are host calls: every rank returns from one before the next starts
    if rank == 0:
        out_q.put(results)
    dist.barrier()
    for r, b in enumerate(bufs):
        if r != rank:
            b.close(False)
    dist.barrier()
    mine.close(True)
    dist.destroy_process_group()


def test_exchange_protocol_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, port, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    res = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert len(res) == 6 * PER_TOKEN
    for tok_i, idx, ok, equal in res:
        if tok_i == 3 and idx == 1:
            assert not ok and not equal   # rank 1 skipped: rank 0's wait ran out and it says so
        else:
            assert ok and equal, (tok_i, idx)  # including the late rank (waited for) and every token after the timeout


def test_exchange_numbers_wrap_safely():
    # flags and numbers are u32; the comparison is on the signed difference
    a, b = np.uint32(0xFFFFFFFE), np.uint32(2)
    assert np.int32(np.uint32(b - a)) >= 0 and np.int32(np.uint32(a - b)) < 0
    assert number(1, 0) == 1 and number(2, 0) == PER_TOKEN + 1 and number(3, 3) == 3 * PER_TOKEN
