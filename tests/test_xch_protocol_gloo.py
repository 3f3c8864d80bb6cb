"""The peer-store exchange protocol, stepped through on CPU by two gloo ranks.

The device code (csrc/kernels.cuh: XchPeers, xch_number, xch_gather4, the EPI_PEERS epilogue)
keeps, per rank, one buffer of ``slots[2 parities][ranks][row]`` 64-bit words and a token counter.
A producer stores its tile's partial sums into slot (e & 1, its rank) of every rank's buffer, each
value as one word {e, f32}; a consumer polls, with a budget, until every word of its own buffer
carries tag e and adds the slots in rank order.  Nothing is ever cleared: old words carry older
tags.  Exchanges are numbered e = (token - 1) * exchanges_per_token + index + 1 on every rank alike.

Here each rank's buffer lives in shared memory that the other process maps, like a peer mapping,
and the same steps run in Python.  What is pinned: the numbering, that two parities suffice, the
rank-ordered sum, that a rank which arrives late is simply waited for, and that a rank which skips
one contribution makes the waits for it run out (an error is reported, nothing blocks for good)
while the following exchanges are healthy again because every rank still runs every later one.
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
        n = 2 * WORLD * ROW * 8 + 8
        self.shm = shared_memory.SharedMemory(name=name, create=create, size=n)
        if create:
            self.shm.buf[:n] = bytes(n)
        self.slots = np.ndarray((2, WORLD, ROW), np.uint64, self.shm.buf, 0)
        self.tok = np.ndarray((1,), np.uint32, self.shm.buf, 2 * WORLD * ROW * 8)

    def close(self, unlink):
        del self.slots, self.tok
        self.shm.close()
        if unlink:
            self.shm.unlink()


def number(tok, index):
    return np.uint32((int(tok) - 1) * PER_TOKEN + index + 1)


def produce(bufs, rank, e, part, skip=False):
    """EPI_PEERS: per tile, every value as a word {e, f32} into every rank's slot.  No flag follows."""
    if skip:
        return
    words = (np.uint64(int(e)) << np.uint64(32)) | part.view(np.uint32).astype(np.uint64)
    for t in range(TILES):
        for b in bufs:
            b.slots[int(e) & 1, rank, t * TILE:(t + 1) * TILE] = words[t * TILE:(t + 1) * TILE]


def consume(mine, e, resid, budget_s):
    """xch_gather4: poll (bounded) until all words carry tag e, then residual + (slot 0 + slot 1 + ...) in rank order."""
    t0 = time.perf_counter()
    ok = True
    while True:
        w = mine.slots[int(e) & 1].copy()
        if np.all((w >> np.uint64(32)) == np.uint64(int(e))):
            break
        if time.perf_counter() - t0 > budget_s:
            ok = False
            break
        time.sleep(0.0005)
    s = np.zeros(ROW, np.float32)
    for r in range(WORLD):
        s = (s + (w[r] & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.float32)).astype(np.float32)
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
            budget = 2.0 if not (tok_i == 3 and idx == 1) else 0.2
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


def test_exchange_numbers():
    # tags are compared for equality with the exchange number; the same parity comes round again two
    # exchanges later, with a different tag
    assert number(1, 0) == 1 and number(2, 0) == PER_TOKEN + 1 and number(3, 3) == 3 * PER_TOKEN
    assert (int(number(5, 1)) & 1) == (int(number(5, 3)) & 1) and number(5, 1) != number(5, 3)
