"""Pipeline-level parity on the GPU: the reference's own caller (model/KVCache_AlignedKV.py, imported unchanged) over
the host-side mirror of the reference's cache classes, and the one-call decode step, against the numpy restatement
of the reference pipeline (oracle/pipeline.py) and against each other.

Planes, exponent maxima and residual buffers must be bit-exact.  Attention outputs are compared with the
max-norm relative error max|a-b| / max|b| <= 1e-3 (the tolerance the parity target states); the softmax and the
residual-token dot products run in fp32 in all three implementations but are not bit-pinned to each other."""
from types import SimpleNamespace

import numpy as np
import pytest

from helpers import load_reference_caller, make_kvq

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
TOL = 1e-3


def rel_err(a, b):
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    return float(np.abs(a - b).max() / np.abs(b).max())


def t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.fixture(scope="module")
def built(akv_lib):
    return akv_lib


@pytest.mark.parametrize("B,H,D,prompt,steps,max_len", [
    (2, 4, 128, 200, 70, 320),     # crosses a block boundary (flush at 256) and keeps decoding
    (1, 4, 128, 29, 1, 30),        # the reference example's size: nothing is ever quantized
    (1, 8, 128, 255, 2, 512),      # first decode token flushes
    (2, 4, 128, 128, 3, 192),      # prompt of whole blocks: empty residual at the start
])
@pytest.mark.parametrize("reference", [False, True])
def test_decode_paths_agree(built, B, H, D, prompt, steps, max_len, reference):
    QuantizedCache_AlignedKV = load_reference_caller()     # the reference's own caller, imported unchanged
    if QuantizedCache_AlignedKV is None:
        pytest.skip("no reference checkout (baseline/_ref, $AKV_REFERENCE_ROOT or ../reference)")
    from alignedkv_b200.decode import DecodeLayer
    from oracle.pipeline import OracleLayerCache, dense_attention_fp32
    L = prompt + steps
    k, v, _ = make_kvq(21, B, L, H, D)
    rng = np.random.default_rng(5)
    qs = rng.standard_normal((steps, B, 1, H, D), dtype=np.float32).astype(np.float16)

    cfg = SimpleNamespace(num_hidden_layers=1, num_attention_heads=H, num_key_value_heads=H, hidden_size=H * D,
                          max_position_embeddings=max_len)
    mirror = QuantizedCache_AlignedKV(cfg, B, max_len, "cuda:0", torch.float16)
    mirror.reference = reference
    fused = DecodeLayer(B, max_len, H, D, "cuda:0")
    fused.reference = reference
    orc = OracleLayerCache(B, max_len, H, D)

    qp = t(np.repeat(qs[0], prompt, axis=1))
    mirror.auto_compute(qp, t(k[:, :prompt]), t(v[:, :prompt]), 0)
    fused.prefill(t(k[:, :prompt]), t(v[:, :prompt]))
    orc.save(k[:, :prompt], v[:, :prompt], 0, prompt)

    worst = dict(mirror=0.0, fused=0.0, fused_vs_mirror=0.0)
    for i in range(steps):
        pos = prompt + i
        kq_, vq_ = k[:, pos:pos + 1], v[:, pos:pos + 1]
        want = orc.decode(qs[i], kq_, vq_, reference)
        got_m = mirror.auto_compute(t(qs[i]), t(kq_), t(vq_), 0).cpu().numpy()
        got_f = fused.decode(t(qs[i]), t(kq_), t(vq_)).cpu().numpy()
        assert got_m.shape == (B, 1, H, D) and got_f.shape == (B, 1, H, D)
        worst["mirror"] = max(worst["mirror"], rel_err(got_m, want))
        worst["fused"] = max(worst["fused"], rel_err(got_f, want))
        worst["fused_vs_mirror"] = max(worst["fused_vs_mirror"], rel_err(got_f, got_m))
    torch.cuda.synchronize()
    kc, vc = mirror.key_cache[0], mirror.value_cache[0]
    exact = [("k_first_8", kc.k_cache_first_8, fused.k_first_8, orc.k_first_8),
             ("k_mid_4", kc.k_cache_mid_4, fused.k_mid_4, orc.k_mid_4),
             ("k_last_4", kc.k_cache_last_4, fused.k_last_4, orc.k_last_4),
             ("v_first_8", vc.v_cache_first_8, fused.v_first_8, orc.v_first_8),
             ("v_mid_4", vc.v_cache_mid_4, fused.v_mid_4, orc.v_mid_4),
             ("v_last_4", vc.v_cache_last_4, fused.v_last_4, orc.v_last_4),
             ("k_exp_max", kc.k_cache_exp_column_max, fused.k_exp_max, orc.k_exp_max),
             ("v_exp_max", vc.v_cache_exp_column_max, fused.v_exp_max, orc.v_exp_max)]
    for name, a, b, c in exact:
        assert np.array_equal(a.cpu().numpy(), c), f"mirror {name} differs from the oracle"
        assert np.array_equal(b.cpu().numpy(), c), f"fused {name} differs from the oracle"
    assert (kc.restklen, kc.reststartpos, kc.current_cache_len) == (orc.rest_len, orc.rest_start, orc.cache_len)
    assert (fused.rest_len, fused.rest_start, fused.cache_len) == (orc.rest_len, orc.rest_start, orc.cache_len)
    n = orc.rest_len
    assert np.array_equal(fused.restk[:, :n].cpu().numpy(), orc.restk[:, :n])
    assert np.array_equal(kc.restk[:, :n].cpu().numpy(), orc.restk[:, :n])
    for name, e in worst.items():
        assert e <= TOL, f"{name}: max-norm relative error {e:.2e} > {TOL}"
    # context: distance of the aligned result from fp32 dense attention over the original fp16 tensors
    truth = dense_attention_fp32(qs[-1], k[:, :L], v[:, :L])
    assert rel_err(got_f, truth) < 0.1


def test_decode_step_rejects_bad_state(built):
    from alignedkv_b200._lib import AlignedKVError
    from alignedkv_b200.decode import DecodeLayer
    layer = DecodeLayer(1, 64, 4, 128, "cuda:0")
    x = torch.zeros((1, 1, 4, 128), dtype=torch.half, device="cuda")
    layer.rest_len = 64          # impossible residual fill
    with pytest.raises(AlignedKVError, match="residual state"):
        layer.decode(x, x, x)
    layer.rest_len = 0
    with pytest.raises(RuntimeError, match="contiguous CUDA fp16"):
        layer.decode(x.float(), x, x)
    torch.cuda.synchronize()


def test_no_kernel_wait_gave_up(built):
    """Every in-kernel wait is bounded; the flag that a wait ran out must still be clear after the tests above."""
    assert built.akv_device_error_flag() == 0


def test_smoke_entry(built):
    import __graft_entry__
    __graft_entry__.smoke()
