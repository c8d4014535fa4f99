"""Generate tests/golden/wrappers.npz by running the REFERENCE's own Python wrappers on CPU.

The reference's extension/k_cache_file.py, extension/v_cache_file.py and model/KVCache_AlignedKV.py are imported
unchanged from a reference checkout (argument, else $AKV_REFERENCE_ROOT); only two things around them are substituted:
  * `extension.KV_cache_cpp_extention.cuda_module` (the reference builds CUDA at import time) becomes the
    oracle-backed stand-in of tests/fake_cuda_module.py, so the kernels' arithmetic comes from oracle/akv_oracle.c;
  * `transformers.cache_utils.Cache` becomes a plain base class (the installed transformers release changed it).
What the fixture pins is therefore the reference's HOST logic: residual buffering, exponent maxima, alignment
inputs, probe inputs, the threshold arithmetic with its [B,H,H,D] broadcast, residual matmuls, -inf padding and
the softmax/decode orchestration.  Run:  python tests/golden/make_golden_wrappers.py [/path/to/reference]
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

CASES = [
    # name, B, H, D, prompt, steps, max_len, reference flag
    ("flush", 2, 4, 128, 190, 4, 256, False),          # third decode token completes block 3
    ("example", 1, 4, 128, 29, 1, 30, False),          # the reference example's size: nothing quantized
    ("blocks", 1, 4, 128, 128, 2, 192, False),
    ("allplanes", 1, 4, 128, 130, 2, 192, True),
]


def run_reference(ref_root: str):
    from fake_cuda_module import OracleCudaModule
    from helpers import make_kvq
    fake = OracleCudaModule()
    stub = types.ModuleType("extension.KV_cache_cpp_extention")
    stub.cuda_module = fake
    sys.modules["extension.KV_cache_cpp_extention"] = stub
    sys.path.insert(0, ref_root)
    import transformers.cache_utils as cu

    class _PlainCache:
        def __init__(self, *a, **k):
            pass

    real = cu.Cache
    cu.Cache = _PlainCache
    try:
        from model.KVCache_AlignedKV import QuantizedCache_AlignedKV   # noqa: E402  (the reference's class)
    finally:
        cu.Cache = real
    out = {}
    for name, B, H, D, prompt, steps, max_len, reference in CASES:
        cfg = types.SimpleNamespace(num_hidden_layers=1, num_attention_heads=H, num_key_value_heads=H,
                                    hidden_size=H * D, max_position_embeddings=max_len)
        cache = QuantizedCache_AlignedKV(cfg, B, max_len, "cpu", torch.float16)
        cache.reference = reference
        k, v, _ = make_kvq(77, B, prompt + steps, H, D)
        qs = np.random.default_rng(78).standard_normal((steps + 1, B, 1, H, D), dtype=np.float32).astype(np.float16)
        qp = torch.from_numpy(np.repeat(qs[0], prompt, axis=1))
        pre = cache.auto_compute(qp, torch.from_numpy(k[:, :prompt]), torch.from_numpy(v[:, :prompt]), 0)
        out[f"{name}.prefill_out"] = pre.numpy().view(np.uint16)
        for i in range(steps):
            pos = prompt + i
            o = cache.auto_compute(torch.from_numpy(qs[i + 1]), torch.from_numpy(k[:, pos:pos + 1]),
                                   torch.from_numpy(v[:, pos:pos + 1]), 0)
            out[f"{name}.out{i}"] = o.numpy().view(np.uint16)
        kc, vc = cache.key_cache[0], cache.value_cache[0]
        out[f"{name}.k_exp"] = kc.k_cache_exp_column_max.numpy()
        out[f"{name}.v_exp"] = vc.v_cache_exp_column_max.numpy()
        out[f"{name}.state"] = np.array([kc.restklen, kc.reststartpos, kc.current_cache_len, vc.restvlen,
                                         vc.reststartpos, vc.current_cache_len], np.int64)
        out[f"{name}.k_mid_4_sum"] = np.array([int(kc.k_cache_mid_4.numpy().astype(np.int64).sum()),
                                               int(kc.k_cache_first_8.numpy().astype(np.int64).sum()),
                                               int(vc.v_cache_first_8.numpy().astype(np.int64).sum()),
                                               int(vc.v_cache_last_4.numpy().astype(np.int64).sum())], np.int64)
        # one more decode step, op by op, to pin the intermediate tensors
        pos = prompt + steps
    return out


if __name__ == "__main__":
    from helpers import reference_root
    ref = sys.argv[1] if len(sys.argv) > 1 else reference_root()
    if ref is None:
        raise SystemExit("no reference checkout: pass its path or set AKV_REFERENCE_ROOT")
    data = run_reference(ref)
    path = os.path.join(HERE, "wrappers.npz")
    np.savez_compressed(path, **data)
    print(f"wrote {path}: {len(data)} arrays, {os.path.getsize(path)} bytes")
