"""CPU tests of the host side: the mirror of the reference's cache classes driven by an oracle-backed `cuda_module`
against golden vectors produced by the REFERENCE's own Python wrappers (tests/golden/wrappers.npz, made by
make_golden_wrappers.py), the numpy pipeline restatement, the C-ABI surface, and the bench's CPU leg."""
import ctypes
import os
import re
import types

import numpy as np
import pytest

from helpers import ROOT, load_reference_caller, make_kvq

torch = pytest.importorskip("torch")
GOLD = os.path.join(ROOT, "tests", "golden", "wrappers.npz")
CASES = [("flush", 2, 4, 128, 190, 4, 256, False), ("example", 1, 4, 128, 29, 1, 30, False),
         ("blocks", 1, 4, 128, 128, 2, 192, False), ("allplanes", 1, 4, 128, 130, 2, 192, True)]


@pytest.fixture()
def cpu_mirror(akv_lib, monkeypatch):
    """The mirror classes with their `cuda_module` replaced by the oracle-backed stand-in (CPU tensors)."""
    from fake_cuda_module import OracleCudaModule
    from alignedkv_b200.extension import k_cache_file, v_cache_file
    fake = OracleCudaModule()
    monkeypatch.setattr(k_cache_file, "cuda_module", fake)
    monkeypatch.setattr(v_cache_file, "cuda_module", fake)
    return fake


@pytest.mark.parametrize("name,B,H,D,prompt,steps,max_len,reference", CASES)
def test_mirror_matches_reference_wrappers(cpu_mirror, name, B, H, D, prompt, steps, max_len, reference):
    """The reference's own caller (model/KVCache_AlignedKV.py, imported unchanged) over the mirror classes reproduces
    what it produced over the reference's own wrapper classes when the fixture was made."""
    QuantizedCache_AlignedKV = load_reference_caller()
    if QuantizedCache_AlignedKV is None:
        pytest.skip("no reference checkout (baseline/_ref, $AKV_REFERENCE_ROOT or ../reference)")
    from oracle.pipeline import OracleLayerCache
    gold = np.load(GOLD)
    cfg = types.SimpleNamespace(num_hidden_layers=1, num_attention_heads=H, num_key_value_heads=H,
                                hidden_size=H * D, max_position_embeddings=max_len)
    cache = QuantizedCache_AlignedKV(cfg, B, max_len, "cpu", torch.float16)
    cache.reference = reference
    orc = OracleLayerCache(B, max_len, H, D)
    k, v, _ = make_kvq(77, B, prompt + steps, H, D)
    qs = np.random.default_rng(78).standard_normal((steps + 1, B, 1, H, D), dtype=np.float32).astype(np.float16)
    qp = torch.from_numpy(np.repeat(qs[0], prompt, axis=1))
    pre = cache.auto_compute(qp, torch.from_numpy(k[:, :prompt]), torch.from_numpy(v[:, :prompt]), 0)
    assert np.array_equal(pre.numpy().view(np.uint16), gold[f"{name}.prefill_out"])
    orc.save(k[:, :prompt], v[:, :prompt], 0, prompt)
    for i in range(steps):
        pos = prompt + i
        o = cache.auto_compute(torch.from_numpy(qs[i + 1]), torch.from_numpy(k[:, pos:pos + 1]),
                               torch.from_numpy(v[:, pos:pos + 1]), 0)
        assert np.array_equal(o.numpy().view(np.uint16), gold[f"{name}.out{i}"]), f"decode output {i}"
        want = orc.decode(qs[i + 1], k[:, pos:pos + 1], v[:, pos:pos + 1], reference)
        err = np.abs(o.numpy().astype(np.float32) - want.astype(np.float32)).max() / np.abs(want.astype(np.float32)).max()
        assert err <= 1e-3, f"numpy pipeline restatement differs: {err:.2e}"
    kc, vc = cache.key_cache[0], cache.value_cache[0]
    assert np.array_equal(kc.k_cache_exp_column_max.numpy(), gold[f"{name}.k_exp"])
    assert np.array_equal(vc.v_cache_exp_column_max.numpy(), gold[f"{name}.v_exp"])
    state = [kc.restklen, kc.reststartpos, kc.current_cache_len, vc.restvlen, vc.reststartpos, vc.current_cache_len]
    assert state == list(gold[f"{name}.state"])
    sums = [int(kc.k_cache_mid_4.numpy().astype(np.int64).sum()), int(kc.k_cache_first_8.numpy().astype(np.int64).sum()),
            int(vc.v_cache_first_8.numpy().astype(np.int64).sum()), int(vc.v_cache_last_4.numpy().astype(np.int64).sum())]
    assert sums == list(gold[f"{name}.k_mid_4_sum"])
    assert np.array_equal(kc.k_cache_first_8.numpy(), orc.k_first_8) and np.array_equal(vc.v_cache_mid_4.numpy(), orc.v_mid_4)
    assert cache.get_seq_length(0) == prompt + steps and cache.get_max_length() == max_len


def test_threshold_broadcast_quirk(cpu_mirror):
    """The threshold of (b, h) is built from probe row (b // H, b % H) and exponent row (b // H, h): the reference
    subtracts a [B,1,H,D] tensor from a [B,H,1,D] one (extension/v_cache_file.py:157) and the kernel reads the
    [B,H,H,1] result flat at b*H+h.  Checked here through the shape and values handed to v_cache_compute."""
    from alignedkv_b200.extension.v_cache_file import V_Cache_Class
    B, H, D, L = 2, 4, 128, 128
    seen = {}
    real = cpu_mirror.v_cache_compute

    def spy(f8, m4, l4, s, amin, *rest):
        seen["amin"] = amin.clone()
        return real(f8, m4, l4, s, amin, *rest)

    cpu_mirror.v_cache_compute = spy
    vc = V_Cache_Class(B, L, H, D, 0, "cpu")
    _, v, _ = make_kvq(5, B, L, H, D)
    vc.save(torch.from_numpy(v), 0, L)
    p = torch.softmax(torch.randn(B, H, 1, L + 64), -1).half()
    p[..., L:] = 0
    # the wrapper asserts start_pos + seqlen bookkeeping, so emulate the state right after a flush
    vc.decoding_compute(p, L - 1, 1)
    amin = seen["amin"]
    assert tuple(amin.shape) == (B, H, H, 1)
    teo = vc.test_compute(p[..., :L], L - 1, 1, 32)                       # [B,H,1,D]
    full = (teo.to(torch.int32) + 15 - vc.v_cache_exp_column_max.to(torch.int32)) & 0xFF   # [B,H,H,D]
    assert torch.equal(amin.to(torch.int32), full.min(dim=-1, keepdim=True).values)
    flat = amin.reshape(-1)
    for b in range(B):
        for h in range(H):
            i = b * H + h
            assert int(flat[i]) == int(full[i // (H * H), (i // H) % H, i % H].min())


def test_mirror_asserts_like_the_reference(cpu_mirror):
    from alignedkv_b200.extension.k_cache_file import K_Cache_Class
    kc = K_Cache_Class(1, 64, 4, 128, 0, "cpu")
    x = torch.zeros((1, 8, 4, 128), dtype=torch.half)
    with pytest.raises(AssertionError, match="new_k.shape"):
        kc.save(x[:, :4], 0, 8)
    kc.save(x, 0, 8)
    with pytest.raises(AssertionError, match="start pos != current KV-Cache len"):
        kc.save(x[:, :1], 3, 1)
    with pytest.raises(AssertionError, match="start_pos: 8, seqlen: 2"):
        kc.save(x[:, :2], 8, 2)
    with pytest.raises(AssertionError, match="> 64"):
        K_Cache_Class(1, 64, 4, 128, 0, "cpu").save(torch.zeros((1, 65, 4, 128), dtype=torch.half), 0, 65)
    with pytest.raises(AssertionError, match="only support MHA"):
        kc.decoding_compute(torch.zeros((1, 1, 8, 128), dtype=torch.half), 8, 1)
    kc.zerolize()
    assert kc.current_cache_len == 0 and not kc.k_cache_first_8.any()


def test_install_as_extension_aliases(akv_lib):
    import sys
    import alignedkv_b200
    saved = {k: sys.modules.get(k) for k in ("extension", "extension.k_cache_file", "extension.v_cache_file",
                                             "extension.KV_cache_cpp_extention")}
    try:
        alignedkv_b200.install_as_extension()
        from extension.k_cache_file import K_Cache_Class          # the reference's import path
        from extension.KV_cache_cpp_extention import cuda_module
        assert K_Cache_Class.__module__ == "alignedkv_b200.extension.k_cache_file"
        for op in ("k_cache_save", "k_cache_compute", "v_cache_save", "v_cache_test_compute", "v_cache_compute"):
            assert callable(getattr(cuda_module, op))
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


# ------------------------------------------------------------------ C ABI
def test_library_exports_every_declared_symbol(akv_lib):
    from alignedkv_b200 import _lib
    header = open(os.path.join(ROOT, "include", "alignedkv_b200.h")).read()
    declared = set(re.findall(r"\b(akv_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SIGNATURES), "header and ctypes binding disagree"
    for name in declared:
        assert hasattr(akv_lib, name), f"{name} is not exported"
    assert akv_lib.akv_abi_version() == 1


def test_argument_validation_happens_before_any_launch(akv_lib):
    """Bad arguments come back as error codes (no CUDA call is made, so this runs without a GPU)."""
    from alignedkv_b200 import _lib
    L = akv_lib
    assert L.akv_v_cache_save(None, None, None, None, 1, 4, 64, 128, 0, 64, 64, None) == -1
    assert b"null pointer" in L.akv_last_error()
    one = ctypes.c_void_p(16)
    assert L.akv_v_cache_save(one, one, one, one, 1, 4, 64, 128, 32, 64, 64, None) == -2
    assert b"exceed max_seq_len" in L.akv_last_error()
    assert L.akv_v_cache_save(one, one, one, one, 1, 4, 64, 127, 0, 64, 64, None) == -2
    assert L.akv_k_cache_save(one, one, one, one, 1, 4, 2, 1, 128, 64, 0, 128, None) == -2
    assert L.akv_k_cache_save(one, one, one, one, 1, 4, 1, 1, 128, 63, 0, 63, None) == -2
    assert L.akv_k_cache_save(one, one, one, one, 1 << 30, 1 << 30, 1, 1 << 30, 1 << 30, 64, 0, 64, None) == -4
    assert L.akv_k_cache_compute(one, one, one, one, one, ctypes.c_void_p(17), one, 1, 4, 1, 1, 128, 64, 64, 0.1, 0,
                                 None) == -3
    assert L.akv_k_cache_compute(None, None, None, None, None, None, None, 1, 4, 0, 1, 128, 64, 0, 0.1, 0, None) == 0
    assert L.akv_v_cache_compute(one, one, one, one, one, one, 1, 4, 64, 128, 64, 65, 0, None) == -2
    assert L.akv_v_cache_save(one, one, one, one, 1, 4, 64, 128, 0, 0, 0, None) == 0       # seq_len 0: no-op
    assert L.akv_set_tuning(b"no_such_knob", 1) == -2 and L.akv_set_tuning(None, 1) == -1
    assert L.akv_decode_scratch_bytes(8, 32, 128, 4096) > 0 and L.akv_decode_scratch_bytes(0, 1, 1, 1) == -1
    assert L.akv_decode_step(*([one] * 15), 1 << 40, 1, 4, 128, 64, 64, 0, 0, None) == -2
    assert b"residual state" in L.akv_last_error()
    assert L.akv_decode_step(*([one] * 15), 16, 1, 4, 128, 64, 0, 0, 0, None) == -2
    assert b"scratch" in L.akv_last_error()
    # the sharded step: 16 pointers, scratch bytes, bsz, kv heads, group, head_dim, max_seq_len, rest_len, rest_start,
    # token_base, chunks_total, n_ranks, out_chunks, flags, phase, stream
    big = 1 << 40
    assert L.akv_shard_step(*([None] * 16), big, 1, 4, 1, 128, 64, 0, 0, 0, 1, 1, 0, 2, 1, None) == -1
    assert L.akv_shard_step(*([one] * 16), big, 1, 4, 1, 128, 64, 0, 0, 0, 1, 1, 0, 2, 5, None) == -2       # phase 5
    assert L.akv_shard_step(*([one] * 16), big, 1, 4, 1, 128, 64, 0, 0, 100, 1, 1, 0, 2, 1, None) == -2     # token_base
    assert b"token_base" in L.akv_last_error()
    assert L.akv_shard_step(*([one] * 16), big, 1, 4, 1, 64, 64, 0, 0, 0, 1, 1, 0, 2, 1, None) == -2        # head_dim
    assert L.akv_shard_step(*([one] * 16), big, 1, 4, 1, 128, 64, 0, 0, 0, 3, 2, 0, 2, 2, None) == -2       # 3 chunks, 2 ranks
    assert b"rank blocks" in L.akv_last_error()
    assert L.akv_shard_step(*([one] * 16), 16, 1, 4, 1, 128, 64, 0, 0, 0, 1, 1, 0, 2, 1, None) == -2
    assert b"scratch" in L.akv_last_error()
    with pytest.raises(_lib.AlignedKVError):
        _lib.check("x", -2)


def test_product_has_no_cpu_fallback_and_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "alignedkv_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} refers to the oracle: product code must not use it"


def test_cpu_baseline_leg_runs():
    """The dense CPU path the bench times (restated from the reference's torch code) agrees with fp32 attention."""
    from oracle.pipeline import dense_attention_fp32, dense_attention_torch_cpu
    k, v, q = make_kvq(1, 1, 96, 4, 64)
    got = dense_attention_torch_cpu(torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v)).numpy()
    want = dense_attention_fp32(q, k, v)
    assert got.shape == (1, 1, 4, 64)
    assert np.abs(got.astype(np.float32) - want).max() / np.abs(want).max() < 5e-3
