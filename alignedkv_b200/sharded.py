"""Decode attention over a cache that is sharded across the GPUs of one node (one process per GPU).

Two ways to shard, neither of which exists in the reference (it is single-device):

* (batch, KV head) sharding - every (batch, KV head) pair is independent in all operators, so each rank simply owns
  a `DecodeLayer` over its slice of the batch and no collective is on the data path (`shard_batch`).
* sequence sharding for long contexts - `SequenceShardedDecoder`: the cached tokens are split into contiguous,
  64-aligned shards, one per rank.  Every rank receives the query, runs the aligned q.K^T / softmax / P.V over its
  own shard and produces, per (batch, query head), the record (m, l, o): maximum score, sum of exponentials and
  locally normalised output.  The records ((D+2) floats per row and rank) are exchanged and merged (log-sum-exp) by
  ONE kernel per rank that stores its record into every rank's exchange buffer over NVLink, publishes a flag and
  waits, time-bounded, for the others' (`PeerExchange`, `akv_exchange_merge`); where peer memory cannot be set up
  (or on request) an NCCL all-gather followed by the merge kernel does the same.  Every rank ends up with the full
  attention output.  New tokens are appended on the last rank.
  Read decisions are taken from each shard's own softmax and magnitude probe, so they can differ from a
  single-device run over the whole sequence; the merged output is compared against fp32 dense attention.
* the same split, decision-exact - `DecisionExactShardedDecoder`: the step is cut into four phases
  (`akv_shard_step`) with a small exchange after each - chunk statistics of the softmax, residue-class candidates
  of the magnitude probe, the winners' high-byte rows, the partial outputs - so that probabilities, thresholds and
  with them every plane-read decision are those of one device holding the whole sequence.
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["shard_bounds", "shard_batch", "chunk_bounds", "SequenceShardedDecoder", "DecisionExactShardedDecoder"]

BLOCK = 64


def shard_bounds(n_tokens: int, world: int, block: int = BLOCK):
    """Contiguous token ranges [lo, hi) per rank: whole blocks, as even as possible, the remainder on the last."""
    nblk = n_tokens // block
    per, extra = divmod(nblk, world)
    bounds, lo = [], 0
    for r in range(world):
        hi = lo + (per + (1 if r < extra else 0)) * block
        bounds.append((lo, hi))
        lo = hi
    bounds[-1] = (bounds[-1][0], n_tokens)
    return bounds


def shard_batch(bsz: int, world: int, rank: int):
    """Rows [lo, hi) of the batch owned by `rank` under (batch, KV head) sharding."""
    per, extra = divmod(bsz, world)
    lo = rank * per + min(rank, extra)
    return lo, lo + per + (1 if rank < extra else 0)


class _CudaBackend:
    """Local step and merge through the C ABI."""

    def __init__(self, bsz, max_local_len, n_kv_heads, head_dim, device, n_q_heads, v_mode):
        from .decode import DecodeLayer
        self.layer = DecodeLayer(bsz, max_local_len, n_kv_heads, head_dim, device, n_q_heads=n_q_heads, v_mode=v_mode)
        self.lib = _lib.load()
        self.device = torch.device(device)

    def prefill(self, k, v):
        self.layer.prefill(k, v)

    def record(self, q, k, v, append):
        return self.layer.decode(q, k, v, append=append, packed=True)

    def decode_exchange(self, q, k, v, append, peer):
        """The local step with the exchange and the merge inside its last kernel: the merged output [B,1,Hq,D]."""
        return self.layer.decode(q, k, v, append=append, exchange=peer)

    def merge(self, gathered, rows, head_dim):
        out = torch.empty((rows, head_dim), dtype=torch.half, device=self.device)
        with torch.cuda.device(self.device):
            rc = self.lib.akv_lse_merge(gathered.data_ptr(), out.data_ptr(), gathered.shape[0], rows, head_dim,
                                        torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check("lse_merge", rc)
        return out


class PeerExchange:
    """Exchange buffers of the ranks of `group` for `akv_exchange_merge`: every rank allocates one, the 64-byte IPC
    handles travel through one all-gather, every rank maps the others' buffers.  All ranks must sit on GPUs of one
    node with peer access to each other.  The constructor raises on EVERY rank when the set-up failed on any of them."""

    MAX_RANKS = 8

    def __init__(self, rows: int, head_dim: int, device, group=None, timeout_ms: int = 2000):
        import ctypes
        import torch.distributed as dist
        self.lib = _lib.load()
        self.device = torch.device(device)
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.rows, self.D, self.timeout_ms = rows, head_dim, timeout_ms
        self.epoch = 0
        self.own = None
        self.mapped = []
        if self.world > self.MAX_RANKS:
            raise ValueError(f"peer exchange covers at most {self.MAX_RANKS} ranks, the group has {self.world}")
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        if rows > 2 * sms or head_dim > 256:
            # (every row's CTA must be resident at once, and the collected row lives in shared memory; the same on
            # every rank, so all of them take the other path together)
            raise RuntimeError(f"peer exchange serves at most {2 * sms} rows of head_dim <= 256, not {rows} x {head_dim}")
        nbytes = self.lib.akv_exchange_bytes(self.world, rows, head_dim)
        handle = (ctypes.c_ubyte * 64)()
        own = ctypes.c_void_p()
        err = None
        with torch.cuda.device(self.device):
            rc = self.lib.akv_peer_alloc(nbytes, ctypes.byref(own), handle)
            if rc != 0:
                err = self.lib.akv_last_error().decode("utf-8", "replace")
            else:
                self.own = own.value
            mine = torch.tensor(list(handle) + [0 if err is None else 1, torch.cuda.current_device()],
                                dtype=torch.uint8, device=self.device)
            every = torch.empty((self.world, 66), dtype=torch.uint8, device=self.device)
            dist.all_gather_into_tensor(every, mine, group=group)
            every = every.cpu()
            ptrs = [None] * self.world
            if len(set(every[:, 65].tolist())) != self.world:
                # two ranks on one GPU: their exchange kernels would wait for each other on the same device
                err = "two ranks of the group run on the same GPU"
            elif err is None and int(every[:, 64].sum()) == 0:
                for g in range(self.world):
                    if g == self.rank:
                        ptrs[g] = self.own
                        continue
                    h = (ctypes.c_ubyte * 64)(*every[g, :64].tolist())
                    p = ctypes.c_void_p()
                    rc = self.lib.akv_peer_open(h, ctypes.byref(p))
                    if rc != 0:
                        err = self.lib.akv_last_error().decode("utf-8", "replace")
                        break
                    self.mapped.append(p.value)
                    ptrs[g] = p.value
            elif err is None:
                err = "another rank could not allocate its exchange buffer"
            ok = torch.tensor([0 if err is None else 1], dtype=torch.int32, device=self.device)
            dist.all_reduce(ok, group=group)          # (also: nobody stores into a buffer before every rank mapped it)
        if int(ok.item()) != 0:
            self.close()
            raise RuntimeError("peer exchange set-up failed" + (f": {err}" if err else " on another rank"))
        self.bufs = (ctypes.c_void_p * self.world)(*ptrs)

    def next_epoch(self) -> int:
        """The epoch of the next exchange (every rank calls this once per step): never 0, and its parity alternates,
        also across the wrap."""
        self.epoch = self.epoch % 0x7FFFFFFE + 1
        return self.epoch

    def merge(self, rec: torch.Tensor) -> torch.Tensor:
        """rec: this rank's packed fp32 [rows, D+2] -> merged fp16 [rows, D] (one launch on the current stream)."""
        self.next_epoch()
        out = torch.empty((self.rows, self.D), dtype=torch.half, device=self.device)
        rec = rec.contiguous()
        with torch.cuda.device(self.device):
            rc = self.lib.akv_exchange_merge(self.bufs, self.rank, self.world, rec.data_ptr(), out.data_ptr(), self.rows,
                                             self.D, self.epoch, self.timeout_ms,
                                             torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check("exchange_merge", rc)
        return out

    def close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's (call it on every rank, after a barrier: nobody may still
        store into a buffer that is being freed)."""
        with torch.cuda.device(self.device):
            for p in self.mapped:
                self.lib.akv_peer_close(p)
            self.mapped = []
            if self.own is not None:
                torch.cuda.synchronize(self.device)
                self.lib.akv_peer_free(self.own)
                self.own = None


class SequenceShardedDecoder:
    """One layer's cache with the sequence split across the ranks of `group` (see the module docstring).

    backend: object with prefill(k, v), record(q, k, v, append) -> fp32 [B*Hq, D+2] and merge(gathered, rows, D);
    the default drives the CUDA kernels.  Tests substitute a CPU implementation to exercise the protocol with gloo.
    exchange: "peer" (records exchanged through peer memory and merged at the end of the step's last kernel),
    "peer_unfused" (the same exchange as a kernel of its own after the step), "collective" (all-gather + merge
    kernel) or "auto": peer memory with the CUDA backend on 2..8 ranks when it can be set up on all of them, else the
    collective; `self.exchange` says which one runs.  With peer memory a rank's step waits inside its last kernel for
    the other ranks' results for at most `exchange_timeout_ms` (then: zeros, and bit 2 of `akv_device_error_flag()`):
    the ranks have to reach every step within that time of each other."""

    def __init__(self, bsz: int, prompt_len: int, max_new_tokens: int, n_kv_heads: int, head_dim: int, device,
                 n_q_heads: int | None = None, v_mode: str = "order_free", group=None, backend=None,
                 exchange: str = "auto", exchange_timeout_ms: int = 2000):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.B, self.D = bsz, head_dim
        self.Hq = n_kv_heads if n_q_heads is None else n_q_heads
        self.bounds = shard_bounds(prompt_len, self.world)
        lo, hi = self.bounds[self.rank]
        self.is_last = self.rank == self.world - 1
        self.local_len = hi - lo
        max_local = self.local_len + (max_new_tokens if self.is_last else 0)
        max_local = max(BLOCK, -(-max_local // BLOCK) * BLOCK)
        self.backend = backend if backend is not None else _CudaBackend(bsz, max_local, n_kv_heads, head_dim, device,
                                                                        self.Hq, v_mode)
        if exchange not in ("auto", "peer", "peer_unfused", "collective"):
            raise ValueError(f"exchange must be 'auto', 'peer', 'peer_unfused' or 'collective', not {exchange!r}")
        self.peer = None
        self.exchange_note = ""
        wants_peer = exchange in ("peer", "peer_unfused") or (
            exchange == "auto" and backend is None and 2 <= self.world <= PeerExchange.MAX_RANKS and
            torch.device(device).type == "cuda")
        if wants_peer and self.world > 1:
            try:
                self.peer = PeerExchange(bsz * self.Hq, head_dim, device, group, exchange_timeout_ms)
            except RuntimeError as e:                 # (raised on every rank alike)
                if exchange != "auto":
                    raise
                self.exchange_note = str(e)
        self.exchange = "collective" if self.peer is None else ("peer_unfused" if exchange == "peer_unfused" else "peer")
        self.fused = self.exchange == "peer" and hasattr(self.backend, "decode_exchange")

    def prefill(self, k_shard, v_shard) -> None:
        """k_shard, v_shard: this rank's tokens [B, hi-lo, H, D] of the prompt (ranks load their own shard)."""
        if k_shard.shape[1] != self.local_len:
            raise ValueError(f"rank {self.rank} owns {self.local_len} tokens, got {k_shard.shape[1]}")
        if self.local_len:
            self.backend.prefill(k_shard, v_shard)

    def decode(self, q, k_new, v_new):
        """q [B,1,Hq,D], k_new / v_new [B,1,H,D] (used on the last rank only) -> merged output [B,1,Hq,D] on every
        rank."""
        if self.peer is not None and self.fused:
            return self.backend.decode_exchange(q, k_new if self.is_last else None, v_new if self.is_last else None,
                                                self.is_last, self.peer)
        rec = self.backend.record(q, k_new if self.is_last else None, v_new if self.is_last else None, self.is_last)
        rows = self.B * self.Hq
        if self.peer is not None:
            return self.peer.merge(rec.reshape(rows, self.D + 2)).reshape(self.B, 1, self.Hq, self.D)
        if self.world == 1:
            gathered = rec.reshape(1, rows, self.D + 2)
        else:
            flat = torch.empty((self.world * rows, self.D + 2), dtype=rec.dtype, device=rec.device)
            self.dist.all_gather_into_tensor(flat, rec.contiguous(), group=self.group)   # rank-major concatenation
            gathered = flat.view(self.world, rows, self.D + 2)
        return self.backend.merge(gathered, rows, self.D).reshape(self.B, 1, self.Hq, self.D)


SM_CHUNK = 4096     # scores per chunk of the split softmax (the granularity of decision-exact shards)


def chunk_bounds(n_tokens: int, world: int, chunk: int = SM_CHUNK):
    """Contiguous token ranges [lo, hi) per rank whose starts are multiples of `chunk`: whole chunks, as even as
    possible, everything that is left (a partial chunk included) on the last rank."""
    nchunk = n_tokens // chunk
    per, extra = divmod(nchunk, world)
    bounds, lo = [], 0
    for r in range(world):
        hi = lo + (per + (1 if r < extra else 0)) * chunk
        bounds.append((lo, hi))
        lo = hi
    bounds[-1] = (bounds[-1][0], n_tokens)
    return bounds


def local_chunks(quantized_tokens: int, chunk: int = SM_CHUNK) -> int:
    """Chunks of a shard's score row: the row holds the quantized tokens plus one block for the residual tokens."""
    return -(-((quantized_tokens // BLOCK + 1) * BLOCK) // chunk)


def pad_chunks(x: torch.Tensor, cmax: int, fill: float):
    """[rows, chunks, ...] -> [rows, cmax, ...], the missing chunks filled with `fill` (an empty chunk)."""
    if x.shape[1] == cmax:
        return x.contiguous()
    pad = torch.full((x.shape[0], cmax - x.shape[1]) + tuple(x.shape[2:]), fill, dtype=x.dtype, device=x.device)
    return torch.cat([x, pad], dim=1).contiguous()


def pad_stats(x: torch.Tensor, cmax: int) -> torch.Tensor:
    """Chunk statistics [rows, chunks, 2] -> [rows, cmax, 2]; an empty chunk is (maximum -inf, sum 0)."""
    return torch.cat([pad_chunks(x[:, :, 0:1], cmax, float("-inf")), pad_chunks(x[:, :, 1:2], cmax, 0.0)], dim=2).contiguous()


def sequence_order(gathered: torch.Tensor) -> torch.Tensor:
    """[world, rows, cmax, ...] as gathered rank by rank -> [rows, world * cmax, ...]: every row's chunks in the order
    of the sequence (padding chunks stay where they are; they are empty and take no part in any reduction)."""
    w, rows, cmax = gathered.shape[:3]
    return gathered.transpose(0, 1).reshape((rows, w * cmax) + tuple(gathered.shape[3:])).contiguous()


class TorchComm:
    """The collectives the protocol needs, over torch.distributed (NCCL on GPUs, gloo on CPU tensors)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def all_gather_into(self, out: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """out [world, *x.shape] <- every rank's x, rank-major."""
        if self.world == 1:
            out[0].copy_(x)
        else:
            self.dist.all_gather_into_tensor(out.view((self.world * x.shape[0],) + tuple(x.shape[1:])), x,
                                             group=self.group)
        return out

    def all_reduce(self, x: torch.Tensor, op: str) -> torch.Tensor:
        if self.world > 1:
            self.dist.all_reduce(x, op=self.dist.ReduceOp.SUM if op == "sum" else self.dist.ReduceOp.MAX,
                                 group=self.group)
        return x


class _CudaShardEngine:
    """A DecodeLayer over the local tokens, stepped through akv_shard_step."""

    def __init__(self, bsz, max_local, n_kv_heads, head_dim, device, n_q_heads, is_last):
        from .decode import DecodeLayer, AKV_STEP_ORDER_FREE, AKV_STEP_NO_APPEND, AKV_STEP_TRACK_MAXIMA
        self.layer = DecodeLayer(bsz, max_local, n_kv_heads, head_dim, device, n_q_heads=n_q_heads, v_mode="order_free")
        self.lib, self.device = self.layer.lib, self.layer.device
        self.is_last = is_last
        self.flags = AKV_STEP_ORDER_FREE | (0 if is_last else (AKV_STEP_NO_APPEND | AKV_STEP_TRACK_MAXIMA))

    def prefill(self, k, v):
        self.layer.prefill(k, v)

    def set_maxima(self, k_exp, v_exp):
        self.layer.k_exp_max.copy_(k_exp)
        self.layer.v_exp_max.copy_(v_exp)

    def phase(self, i, exch_in, q, k_new, v_new, chunks, chunks_total, token_base, n_ranks=1, out=None, out_chunks=0):
        """out: buffer to write (phase 1 / 2: rows of out_chunks chunks, padding left untouched); default: a new tensor
        over the local chunks.  n_ranks: rank blocks in exch_in (see akv_shard_step)."""
        lay = self.layer
        rows, D = lay.B * lay.Hq, lay.D
        if out is None:
            shape, dtype = {1: ((rows, chunks, 2), torch.float32), 2: ((2, rows, chunks, 32), torch.int32),
                            3: ((rows, 32, D), torch.uint8), 4: ((rows, D + 2), torch.float32)}[i]
            out = torch.empty(shape, dtype=dtype, device=self.device)
            out_chunks = 0
        with torch.cuda.device(self.device):
            rc = self.lib.akv_shard_step(
                lay.k_first_8.data_ptr(), lay.k_mid_4.data_ptr(), lay.k_last_4.data_ptr(),
                lay.v_first_8.data_ptr(), lay.v_mid_4.data_ptr(), lay.v_last_4.data_ptr(),
                lay.k_exp_max.data_ptr(), lay.v_exp_max.data_ptr(), lay.restk.data_ptr(), lay.restv.data_ptr(),
                q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), exch_in.data_ptr() if exch_in is not None else None,
                out.data_ptr(), lay.scratch.data_ptr(), lay.scratch.numel(), lay.B, lay.H, lay.G, D,
                lay.L, lay.rest_len, lay.rest_start, token_base, chunks_total, n_ranks, out_chunks, self.flags, i,
                torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check("shard_step", rc)
        return out

    def finish_step(self):
        """Advance the residual state after phase 4 (as DecodeLayer.decode does)."""
        lay = self.layer
        if self.is_last:
            if lay.rest_len + 1 == BLOCK:
                lay.rest_start += BLOCK
                lay.rest_len = 0
            else:
                lay.rest_len += 1
            lay.cache_len += 1

    def snapshot(self):
        return self.layer.snapshot()

    def restore(self, snap):
        self.layer.restore(snap)


class DecisionExactShardedDecoder:
    """One layer's cache with the sequence split across ranks at multiples of 4096 tokens, decoded with the read
    decisions of a single device (see the module docstring; `akv_shard_step` documents the four phases).

    The exponent maxima every decision starts from are those of the whole sequence on every rank: after the prompt
    they are reduced across ranks, and every rank takes each new token into them (the token is stored on the last
    rank only).  `decode` runs the phases with the exchanges of `comm`; a test may also call `phase(i, exch_in, ...)`
    on several instances in turn and do the exchanges itself.  engine: object with prefill / set_maxima / phase /
    finish_step / snapshot / restore (default: the CUDA kernels); tests substitute one to exercise the exchanges with
    gloo on CPU."""

    def __init__(self, bsz: int, prompt_len: int, max_new_tokens: int, n_kv_heads: int, head_dim: int, device,
                 n_q_heads: int | None = None, comm=None, rank: int | None = None, world: int | None = None,
                 engine=None):
        self.comm = comm if comm is not None else TorchComm()
        self.world = world if world is not None else self.comm.world
        if rank is None:
            rank = self.comm.dist.get_rank(self.comm.group) if self.world > 1 else 0
        self.rank = rank
        self.B, self.D, self.H = bsz, head_dim, n_kv_heads
        self.Hq = n_kv_heads if n_q_heads is None else n_q_heads
        self.rows = bsz * self.Hq
        self.bounds = chunk_bounds(prompt_len, self.world)
        lo, hi = self.bounds[rank]
        self.token_base, self.local_len = lo, hi - lo
        self.is_last = rank == self.world - 1
        max_local = self.local_len + (max_new_tokens if self.is_last else 0)
        max_local = max(BLOCK, -(-max_local // BLOCK) * BLOCK)
        self.engine = engine if engine is not None else _CudaShardEngine(bsz, max_local, n_kv_heads, head_dim, device,
                                                                         self.Hq, self.is_last)
        self.device = torch.device(device)
        self.appended = 0                     # tokens decoded so far (every rank counts them)

    @property
    def layer(self):
        return self.engine.layer

    # ---- geometry every rank can compute for every other rank
    def _chunks_of(self, r: int, appended: int) -> int:
        lo, hi = self.bounds[r]
        n = hi - lo + (appended if r == self.world - 1 else 0)
        return local_chunks((n // BLOCK) * BLOCK)

    def prefill(self, k_shard, v_shard) -> None:
        """k_shard, v_shard: this rank's tokens [B, hi-lo, H, D] of the prompt."""
        from .extension._planes import exponent_field
        if k_shard.shape[1] != self.local_len:
            raise ValueError(f"rank {self.rank} owns {self.local_len} tokens, got {k_shard.shape[1]}")
        if self.local_len:
            self.engine.prefill(k_shard, v_shard)
        # maxima of the whole prompt: the reference takes the exponent of the SIGNED maximum (k_cache_file.py:77-78)
        exps = []
        for x in (k_shard, v_shard):
            if self.local_len:
                mx = torch.max(x, dim=1, keepdim=True).values.float()
            else:
                mx = torch.full((self.B, 1, self.H, self.D), float("-inf"), device=x.device)
            exps.append(exponent_field(self.comm.all_reduce(mx.contiguous(), "max").half()))
        self.engine.set_maxima(*exps)

    def phase(self, i: int, exch_in, q, k_new, v_new, chunks_total: int = 0, n_ranks: int = 1, out=None,
              out_chunks: int = 0):
        """Run phase i (1..4) of the step in progress and return its exchange buffer (see akv_shard_step)."""
        return self.engine.phase(i, exch_in, q, k_new, v_new, self._chunks_of(self.rank, self.appended + 1),
                                 chunks_total, self.token_base, n_ranks=n_ranks, out=out, out_chunks=out_chunks)

    def _buffers(self, cmax: int, like):
        """Exchange buffers for a common chunk count of cmax (kept between steps; the padding chunks of the phase 1 / 2
        outputs are filled once: the kernels only write the local chunks)."""
        if getattr(self, "_buf_cmax", None) != cmax or self._buf["st"].device != like.device:
            dev, W, rows, D = like.device, self.world, self.rows, self.D
            st = torch.empty((rows, cmax, 2), dtype=torch.float32, device=dev)
            st[:, :, 0] = float("-inf")
            st[:, :, 1] = 0.0
            self._buf = dict(
                st=st, st_all=torch.empty((W, rows, cmax, 2), dtype=torch.float32, device=dev),
                cand=torch.zeros((2, rows, cmax, 32), dtype=torch.int32, device=dev),
                cand_all=torch.empty((W, 2, rows, cmax, 32), dtype=torch.int32, device=dev),
                win=torch.empty((rows, 32, D), dtype=torch.uint8, device=dev),
                part=torch.empty((rows, D + 2), dtype=torch.float32, device=dev),
                parts=torch.empty((W, rows, D + 2), dtype=torch.float32, device=dev))
            self._buf_cmax = cmax
        return self._buf

    def finish_step(self) -> None:
        self.engine.finish_step()
        self.appended += 1

    def snapshot(self):
        """State to come back to with `restore` (see DecodeLayer.snapshot)."""
        return dict(engine=self.engine.snapshot(), appended=self.appended)

    def restore(self, snap) -> None:
        before = self._chunks_of(self.rank, self.appended + 1)
        self.engine.restore(snap["engine"])
        self.appended = snap["appended"]
        if self._chunks_of(self.rank, self.appended + 1) < before:
            self._buf_cmax = None       # a chunk written earlier is padding again: rebuild the exchange buffers

    def decode(self, q, k_new, v_new):
        """q [B,1,Hq,D], k_new / v_new [B,1,H,D] (needed on every rank: they feed the exponent maxima) -> output
        [B,1,Hq,D], the same on every rank."""
        W = self.world
        cmax = max(self._chunks_of(r, self.appended + 1) for r in range(W))
        total = W * cmax
        buf = self._buffers(cmax, q)
        # every phase writes straight into the buffer that is exchanged, and reads the gathered buffer as it arrives
        self.phase(1, None, q, k_new, v_new, out=buf["st"], out_chunks=cmax)
        self.comm.all_gather_into(buf["st_all"], buf["st"])
        self.phase(2, buf["st_all"], q, k_new, v_new, total, n_ranks=W, out=buf["cand"], out_chunks=cmax)
        self.comm.all_gather_into(buf["cand_all"], buf["cand"])
        self.phase(3, buf["cand_all"], q, k_new, v_new, total, n_ranks=W, out=buf["win"])
        self.comm.all_reduce(buf["win"], "sum")                # every byte is non-zero on at most one rank
        self.phase(4, buf["win"], q, k_new, v_new, total, n_ranks=W, out=buf["part"])
        self.comm.all_gather_into(buf["parts"], buf["part"])
        out = buf["parts"][:, :, 2:].sum(dim=0)                # the ranks' parts add up (fp32)
        self.finish_step()
        return out.half().reshape(self.B, 1, self.Hq, self.D)
