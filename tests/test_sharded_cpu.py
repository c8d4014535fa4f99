"""Host-side logic of the sharded decoders on CPU: shard arithmetic, the sequence-sharded protocol
(local record -> all-gather -> log-sum-exp merge) run as two gloo ranks with the numpy oracle standing in for the
CUDA kernels, and the exchanges of the decision-exact protocol run as two gloo ranks with an engine that checks what
each phase receives."""
import os
import socket

import numpy as np
import pytest

from helpers import make_kvq

torch = pytest.importorskip("torch")


def test_shard_bounds_and_batch():
    from alignedkv_b200.sharded import shard_batch, shard_bounds
    b = shard_bounds(131072, 8)
    assert b[0] == (0, 16384) and b[-1] == (114688, 131072) and all(hi - lo == 16384 for lo, hi in b)
    b = shard_bounds(1000, 4)                     # 15 whole blocks + 40 tokens: 4,4,4,3 blocks, tail on the last
    assert [hi - lo for lo, hi in b] == [256, 256, 256, 232] and b[-1][1] == 1000
    assert all(lo % 64 == 0 for lo, _ in b)
    b = shard_bounds(100, 4)                      # fewer blocks than ranks: empty shards are allowed
    assert [hi - lo for lo, hi in b] == [64, 0, 0, 36]
    rows = [shard_batch(10, 4, r) for r in range(4)]
    assert rows == [(0, 3), (3, 6), (6, 8), (8, 10)]


class NumpyBackend:
    """The oracle pipeline as the per-shard engine (torch CPU tensors in and out)."""

    def __init__(self, bsz, max_local, heads, head_dim):
        from oracle.pipeline import OracleLayerCache
        self.cache = OracleLayerCache(bsz, max_local, heads, head_dim)

    def prefill(self, k, v):
        self.cache.save(k.numpy(), v.numpy(), 0, k.shape[1])

    def record(self, q, k, v, append):
        rec = self.cache.decode_record(q.numpy(), k.numpy() if append else None, v.numpy() if append else None,
                                       append=append, order_free=True)[1]
        return torch.from_numpy(rec)

    def merge(self, gathered, rows, head_dim):
        from oracle.pipeline import lse_merge_np
        return torch.from_numpy(lse_merge_np(gathered.numpy()))


def _worker(rank, world, port, results):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from alignedkv_b200.sharded import SequenceShardedDecoder, shard_bounds
        from oracle.pipeline import dense_attention_fp32
        B, H, D, S, steps = 1, 4, 128, 256 + 20, 3      # (the oracle, like the reference kernel, serves heads in fours)
        k, v, _ = make_kvq(81, B, S + steps, H, D)
        rng = np.random.default_rng(82)
        qs = rng.standard_normal((steps, B, 1, H, D), dtype=np.float32).astype(np.float16)
        lo, hi = shard_bounds(S, world)[rank]
        max_local = -(-(hi - lo + (steps if rank == world - 1 else 0)) // 64) * 64
        dec = SequenceShardedDecoder(B, S, steps, H, D, "cpu", backend=NumpyBackend(B, max(64, max_local), H, D))
        # (a backend of the caller's and CPU tensors: the records meet through the process group's all-gather, never
        # through peer memory)
        assert dec.exchange == "collective" and dec.peer is None
        dec.prefill(torch.from_numpy(k[:, lo:hi].copy()), torch.from_numpy(v[:, lo:hi].copy()))
        errs = []
        for i in range(steps):
            out = dec.decode(torch.from_numpy(qs[i]), torch.from_numpy(k[:, S + i:S + i + 1].copy()),
                             torch.from_numpy(v[:, S + i:S + i + 1].copy())).numpy()
            truth = dense_attention_fp32(qs[i], k[:, :S + i + 1], v[:, :S + i + 1])
            errs.append(float(np.abs(out.astype(np.float32) - truth).max() / np.abs(truth).max()))
        results[rank] = errs
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_protocol_two_gloo_ranks():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        errs = dict(results)
    assert set(errs) == {0, 1}
    assert errs[0] == errs[1], "every rank must hold the same merged output"
    # against fp32 dense attention the aligned path itself is 1e-2 .. 4e-2 off (skipped nibble planes, fp16 scores); the
    # bound only guards the protocol (a wrong merge is off by order 1)
    assert max(errs[0]) <= 6e-2, errs[0]


def test_chunk_bounds_and_exchange_layout():
    from alignedkv_b200.sharded import chunk_bounds, local_chunks, pad_chunks, pad_stats, sequence_order
    b = chunk_bounds(131071, 8)
    assert b[0] == (0, 16384) and b[-1] == (114688, 131071) and all(lo % 4096 == 0 for lo, _ in b)
    assert chunk_bounds(20470, 3) == [(0, 8192), (8192, 12288), (12288, 20470)]
    assert chunk_bounds(5000, 4) == [(0, 4096), (4096, 4096), (4096, 4096), (4096, 5000)]   # empty shards are allowed
    assert local_chunks(0) == 1 and local_chunks(4032) == 1 and local_chunks(4096) == 2 and local_chunks(8192) == 3
    x = torch.arange(2 * 1 * 2, dtype=torch.float32).view(2, 1, 2)
    p = pad_stats(x, 3)
    assert p.shape == (2, 3, 2) and torch.isinf(p[:, 1:, 0]).all() and (p[:, 1:, 0] < 0).all() and (p[:, 1:, 1] == 0).all()
    g = torch.stack([torch.full((2, 3, 1), float(r)) for r in range(4)])      # [world, rows, cmax, 1]
    s = sequence_order(g)
    assert s.shape == (2, 12, 1) and s[0, :, 0].tolist() == [0, 0, 0, 1, 1, 1, 2, 2, 2, 3, 3, 3]
    assert pad_chunks(torch.ones(2, 3, 5), 3, 0).shape == (2, 3, 5)


class CheckingEngine:
    """Stands in for the CUDA kernels: every phase returns a buffer that encodes (rank, chunk) and checks that what it
    receives is every rank's buffer in sequence order."""

    def __init__(self, rank, world, rows, D, chunks_of):
        self.rank, self.world, self.rows, self.D, self.chunks_of = rank, world, rows, D, chunks_of
        self.maxima = None
        self.steps = 0

    def prefill(self, k, v):
        pass

    def set_maxima(self, k_exp, v_exp):
        self.maxima = (k_exp.clone(), v_exp.clone())

    def phase(self, i, exch_in, q, k_new, v_new, chunks, chunks_total, token_base, n_ranks=1, out=None, out_chunks=0):
        cmax = max(self.chunks_of)
        assert chunks == self.chunks_of[self.rank] and out is not None
        if i == 1:
            assert out.shape == (self.rows, cmax, 2) and out_chunks == cmax
            for c in range(chunks):
                out[:, c, 0] = 100.0 * self.rank + c
                out[:, c, 1] = self.rank + 1.0
            return out
        assert chunks_total == self.world * cmax and n_ranks == self.world
        if i == 2:
            assert exch_in.shape == (self.world, self.rows, cmax, 2)
            for r in range(self.world):
                for c in range(cmax):
                    m, l = exch_in[r, 0, c].tolist()
                    if c < self.chunks_of[r]:
                        assert (m, l) == (100.0 * r + c, r + 1.0)
                    else:
                        assert m == float("-inf") and l == 0.0          # padding chunk of a shorter shard
            assert out.shape == (2, self.rows, cmax, 32) and out_chunks == cmax
            out[0, :, :chunks] = 1000 * (self.rank + 1)
            out[1, :, :chunks] = token_base // 32
            return out
        if i == 3:
            assert exch_in.shape == (self.world, 2, self.rows, cmax, 32) and exch_in.dtype == torch.int32
            for r in range(self.world):
                assert int(exch_in[r, 0, 0, 0, 0]) == 1000 * (r + 1)
                if self.chunks_of[r] < cmax:
                    assert int(exch_in[r, 0, 0, cmax - 1, 0]) == 0      # padding candidates
            out.zero_()
            out[:, self.rank::self.world] = self.rank + 1           # "the winners this rank holds"
            return out
        assert exch_in.dtype == torch.uint8
        for j in range(32):
            assert int(exch_in[0, j, 0]) == j % self.world + 1
        out.zero_()
        out[:, 2:] = self.rank + 1.0
        return out

    def finish_step(self):
        self.steps += 1

    def snapshot(self):
        return self.steps

    def restore(self, snap):
        self.steps = snap


def _exact_worker(rank, world, port, results):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from alignedkv_b200.sharded import DecisionExactShardedDecoder, chunk_bounds, local_chunks
        B, H, D, prompt = 1, 4, 128, 12288 + 200
        bounds = chunk_bounds(prompt, world)
        chunks_of = [local_chunks(((hi - lo + (1 if r == world - 1 else 0)) // 64) * 64) for r, (lo, hi) in enumerate(bounds)]
        eng = CheckingEngine(rank, world, B * H, D, chunks_of)
        dec = DecisionExactShardedDecoder(B, prompt, 4, H, D, "cpu", engine=eng)
        lo, hi = bounds[rank]
        k = torch.full((B, hi - lo, H, D), 1.0 + rank).half()
        k[:, 0, 0, 0] = -3.0 if rank == 0 else 0.5
        dec.prefill(k, k.clone())
        # signed maximum over BOTH ranks' tokens: 2.0 (exponent 16) everywhere
        assert int(eng.maxima[0].min()) == 16 and int(eng.maxima[0].max()) == 16
        z = torch.zeros(B, 1, H, D).half()
        out = dec.decode(z, z, z)
        assert eng.steps == 1 and dec.appended == 1
        results[rank] = out.float().flatten()[:4].tolist()
    finally:
        dist.destroy_process_group()


def test_decision_exact_exchanges_two_gloo_ranks():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_exact_worker, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        res = dict(results)
    assert res[0] == res[1] == [3.0, 3.0, 3.0, 3.0]      # the parts (1 and 2) added up, the same on every rank
