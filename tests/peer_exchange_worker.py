"""One rank of tests/test_gpu_peer_exchange.py (launched with torch.distributed.run, one process per GPU).

Three sequence-sharded decoders over the same shard of the same seeded prompt - one exchanging through peer memory at
the end of the step's last kernel (`akv_decode_step_exchange`), one with the exchange kernel by itself
(`akv_exchange_merge`), one through the NCCL all-gather and `akv_lse_merge`: their outputs must be bit-identical on
every rank for every step (a run that crosses a 64-token block boundary), and no bounded wait may have given up.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    from helpers import make_kvq
    from alignedkv_b200 import _lib
    from alignedkv_b200.sharded import SequenceShardedDecoder, shard_bounds
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    B, H, D, S, steps = 2, 4, 128, 4096 + 40, 30
    k, v, _ = make_kvq(123, B, S + steps, H, D)
    qs = np.random.default_rng(124).standard_normal((steps, B, 1, H, D), dtype=np.float32).astype(np.float16)
    lo, hi = shard_bounds(S, world)[rank]
    decs = [SequenceShardedDecoder(B, S, steps, H, D, dev, exchange=e) for e in ("peer", "peer_unfused", "collective")]
    assert [d.exchange for d in decs] == ["peer", "peer_unfused", "collective"] and decs[0].fused
    for d in decs:
        d.prefill(torch.from_numpy(k[:, lo:hi]).to(dev), torch.from_numpy(v[:, lo:hi]).to(dev))
    for t in range(steps):
        q = torch.from_numpy(qs[t]).to(dev)
        kt, vt = torch.from_numpy(k[:, S + t:S + t + 1]).to(dev), torch.from_numpy(v[:, S + t:S + t + 1]).to(dev)
        a, a2, b = (d.decode(q, kt, vt) for d in decs)
        torch.cuda.synchronize()
        for name, x in (("fused", a), ("stand-alone", a2)):
            if not torch.equal(x, b):
                raise SystemExit(f"rank {rank} step {t}: {name} peer exchange and all-gather differ "
                                 f"(max {float((x.float() - b.float()).abs().max()):.3e})")
        if not bool(torch.isfinite(a.float()).all()) or float(a.float().abs().max()) == 0.0:
            raise SystemExit(f"rank {rank} step {t}: output is not a finite non-zero attention result")
    flag = _lib.load().akv_device_error_flag()
    if flag != 0:
        raise SystemExit(f"rank {rank}: device error flag {flag}")
    dist.barrier()                       # nobody frees a buffer that a peer may still store into
    torch.cuda.synchronize()
    decs[0].peer.close()
    decs[1].peer.close()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: {steps} steps identical", flush=True)


if __name__ == "__main__":
    main()
