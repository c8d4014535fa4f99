"""Generate tests/golden/ref_kernels.npz from the REFERENCE's own CUDA kernels.

Needs a CUDA device and oracle/_ref/kv_cache_cuda.so (the unmodified reference extension, built by
oracle/build_ref.py).  Inputs are regenerated from seeds by tests/helpers.py, so the fixture only stores what
the reference kernels returned.  Run on a GPU box:  python tests/golden/make_golden_gpu.py <output-dir>
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import (exponent_field, k_planes_np, load_reference_extension, make_kvq, softmax_probs,  # noqa: E402
                     v_planes_np)

B, H, D, L, MAXLEN = 1, 4, 128, 128, 192


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def u8(a):
    return np.ascontiguousarray(a).view(np.uint8)


def main(out_dir):
    ref = load_reference_extension()
    assert ref is not None, "oracle/_ref/kv_cache_cuda.so is missing"
    out = {}
    nmb = -(-MAXLEN // 64)
    # ---- K planes: prefill of 2 blocks, flush of a third block, one single-token append
    k, v, q = make_kvq(101, B, L + 64 + 1, H, D)
    kp = [dev(p) for p in k_planes_np(B, H, nmb, D)]
    ref.k_cache_save(*kp, dev(u8(k[:, :L])), B, H, L // 64, nmb, D, 64, 0, L)
    ref.k_cache_save(*kp, dev(u8(k[:, L:L + 64])), B, H, 1, nmb, D, 64, L, 64)
    out["k_planes_after_flush"] = np.concatenate([p.cpu().numpy().reshape(-1) for p in kp])
    kp2 = [p.clone() for p in kp]
    ref.k_cache_save(*kp2, dev(u8(k[:, L + 64:L + 65])), B, H, 0, nmb, D, 64, 70, 1)   # token into block 1, slot 6
    out["k_planes_after_token"] = np.concatenate([p.cpu().numpy().reshape(-1) for p in kp2])
    # ---- q.K^T over the 3 quantized blocks
    kexp = exponent_field(k[:, :L + 64].max(axis=1, keepdims=True))
    kq = (exponent_field(q) + kexp).astype(np.uint8)
    kqmax = kq.max(axis=3, keepdims=True)
    for reference in (False, True):
        s = ref.k_cache_compute(*kp, dev(kq), dev(kqmax), dev(u8(q)), B, H, 3, nmb, D, 64, L + 64,
                                1.0 / math.sqrt(D), reference)
        out[f"k_scores_ref{int(reference)}"] = s.cpu().numpy().view(np.uint16)[..., :3 * 64].copy()
    # ---- V planes
    vp = [dev(p) for p in v_planes_np(B, H, MAXLEN, D)]
    ref.v_cache_save(*vp, dev(u8(v[:, :L])), B, H, MAXLEN, D, 0, L)
    ref.v_cache_save(*vp, dev(u8(v[:, L:L + 64])), B, H, MAXLEN, D, L, 64)
    out["v_planes"] = np.concatenate([p.cpu().numpy().reshape(-1) for p in vp])
    # ---- probe and aligned P.V over 192 tokens
    n = L + 64
    p = softmax_probs(102, B, H, n, pad=64)
    grp = p[..., :n].reshape(B, H, n // 32, 32)
    val = np.ascontiguousarray(grp.max(axis=2, keepdims=True))
    idx = grp.argmax(axis=2).astype(np.int32)[:, :, None, :]
    o = ref.v_cache_test_compute(*vp, dev(u8(val)), dev(u8(idx)), B, H, MAXLEN, D, 32)
    out["v_probe"] = o.cpu().numpy().view(np.uint16).copy()
    pe = int(exponent_field(p[..., :n]).max())
    for shift in (0, 2, 5):
        amin = np.full((B, H, H, 1), max(pe - shift, 0), np.uint8)
        for reference in (False, True):
            o = ref.v_cache_compute(*vp, dev(u8(p)), dev(amin), B, H, MAXLEN, D, p.shape[-1], n, reference)
            out[f"v_out_shift{shift}_ref{int(reference)}"] = o.cpu().numpy().view(np.uint16).copy()
    torch.cuda.synchronize()
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "ref_kernels.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    # output directory: argument, else $AKV_GOLDEN_OUT, else beside this script (where the committed fixture lives)
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AKV_GOLDEN_OUT", HERE))
