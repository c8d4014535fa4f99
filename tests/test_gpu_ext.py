"""GPU parity of the entry points that extend the reference's surface: grouped-query attention, the order-free
(split-sequence, fp32) P.V kernel, the packed per-shard record and the log-sum-exp merge.

Specification used for each:
  grouped-query   the reference (which asserts multi-head attention) run on a cache whose KV heads are repeated
                  `group` times; with the exact P.V kernel results must be BIT-EXACT against that oracle.
  order-free P.V  same read decisions; the sum is compared with the exact (float64) sum of probability x
                  dequantized value rounded once to fp16: max-norm relative error <= 1e-3.
  merge           numpy restatement of the weighted sum; max-norm relative error <= 1e-3.
"""
import ctypes
import math

import numpy as np
import pytest

from helpers import exponent_field, make_kvq, softmax_probs, v_planes_np, k_planes_np

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
TOL = 1e-3
ORDER_FREE = 2


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def u8(a):
    return np.ascontiguousarray(a).view(np.uint8)


def rel_err(a, b):
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def stream():
    return torch.cuda.current_stream().cuda_stream


def check(lib, rc):
    assert rc == 0, lib.akv_last_error().decode()


def v_state(seed, B, H, L, max_len, D=128):
    from oracle import akv_oracle as orc
    _, v, _ = make_kvq(seed, B, L, H, D)
    planes = v_planes_np(B, H, max_len, D)
    orc.v_cache_save(*planes, u8(v), B, H, max_len, D, 0, L)
    return v, planes


@pytest.mark.parametrize("B,H,G,n,max_len,amin_val", [
    (2, 4, 1, 512, 512, 13),
    (1, 2, 1, 1000, 1024, 14),      # ragged token count (not a multiple of 8, 32 or 64)
    (1, 3, 1, 4500, 4608, 13),      # several chunks per head, ragged last stage (order-free: streaming form)
    (1, 2, 1, 2048, 2048, 3),       # a low threshold: many tokens read the nibble planes, several per lane
    (2, 2, 4, 640, 768, 13),        # grouped-query: 4 query heads per KV head, different probabilities each
    (1, 2, 2, 256, 256, 15),
    (1, 1, 8, 320, 320, 13),
])
@pytest.mark.parametrize("reference", [False, True])
def test_v_compute_gqa_and_order_free(akv_lib, B, H, G, n, max_len, amin_val, reference):
    """Exact kernel with a group: bit-exact against the oracle on repeated heads.  Order-free kernel: <= 1e-3."""
    from oracle import akv_oracle as orc
    lib = akv_lib
    D, Hq = 128, H * G
    _, planes = v_state(31, B, H, n, max_len)
    pad = (-n) % 8
    p = softmax_probs(32, B, Hq, n, pad=pad)
    amin = np.full((B, Hq, 1, 1), amin_val, np.uint8)
    amin[0, 0] = amin_val - 1
    exp_planes = [np.ascontiguousarray(np.repeat(x, G, axis=1)) for x in planes]
    want_u8, codes = orc.v_cache_compute(*exp_planes, u8(p), amin, B, Hq, max_len, D, n + pad, n, reference)
    want = want_u8.view(np.float16).reshape(B, Hq, D)

    dp = [dev(x) for x in planes]
    ds, da = dev(u8(p)), dev(amin)
    out = torch.empty((B, Hq, 1, D), dtype=torch.half, device="cuda")
    flags = 1 if reference else 0
    check(lib, lib.akv_v_cache_compute_gqa(dp[0].data_ptr(), dp[1].data_ptr(), dp[2].data_ptr(), ds.data_ptr(),
                                           da.data_ptr(), out.data_ptr(), None, 0, B, H, G, max_len, D, n + pad, n,
                                           flags, stream()))
    got = out.cpu().numpy().reshape(B, Hq, D)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), "exact grouped P.V differs from the oracle"

    # order-free: exact sum under the same decisions
    c = codes[..., None]
    f = exp_planes[0][:, :, :n].astype(np.uint16)
    mid = np.where(c < 2, exp_planes[1][:, :, :n].astype(np.uint16), 0x88)
    low = np.where(c == 0, exp_planes[2][:, :, :n].astype(np.uint16), np.where(c == 1, 0x88, 0))
    bits = np.empty(f.shape, np.uint16)
    bits[..., 0::2] = (f[..., 0::2] << 8) | (mid & 0xF0) | (low >> 4)
    bits[..., 1::2] = (f[..., 1::2] << 8) | ((mid << 4) & 0xF0) | (low & 0x0F)
    exact = np.einsum("bht,bhtd->bhd", p[:, :, 0, :n].astype(np.float64), bits.view(np.float16).astype(np.float64))
    nbytes = lib.akv_v_cache_compute_scratch_bytes(B, H, G, n)
    assert nbytes > 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out2 = torch.empty((B, Hq, 1, D), dtype=torch.half, device="cuda")
    check(lib, lib.akv_v_cache_compute_gqa(dp[0].data_ptr(), dp[1].data_ptr(), dp[2].data_ptr(), ds.data_ptr(),
                                           da.data_ptr(), out2.data_ptr(), ws.data_ptr(), nbytes, B, H, G, max_len, D,
                                           n + pad, n, flags | ORDER_FREE, stream()))
    got2 = out2.cpu().numpy().reshape(B, Hq, D)
    assert rel_err(got2, exact) <= TOL, f"order-free P.V: {rel_err(got2, exact):.2e}"
    assert lib.akv_device_error_flag() == 0


@pytest.mark.parametrize("form", [1, 2])
@pytest.mark.parametrize("B,H,G,n,max_len,amin_val", [
    (2, 3, 4, 1100, 1152, 13),      # ragged token count, several stages, four query heads per KV head
    (1, 2, 2, 640, 640, 14),
    (1, 2, 4, 2048, 2048, 11),      # a low threshold: many stages hold flagged tokens (the tables are handed around)
])
def test_v_chain_grouped_forms(akv_lib, form, B, H, G, n, max_len, amin_val):
    """Exact P.V with grouped queries through both forms of the chain kernel - a ring per query head (1) and one ring
    shared by the heads of a KV head (2) - bit-exact against the oracle on repeated heads."""
    from oracle import akv_oracle as orc
    lib = akv_lib
    D, Hq = 128, H * G
    _, planes = v_state(33, B, H, n, max_len)
    pad = (-n) % 8
    p = softmax_probs(34, B, Hq, n, pad=pad)
    amin = np.full((B, Hq, 1, 1), amin_val, np.uint8)
    amin[0, 1] = amin_val - 1
    exp_planes = [np.ascontiguousarray(np.repeat(x, G, axis=1)) for x in planes]
    want_u8, _ = orc.v_cache_compute(*exp_planes, u8(p), amin, B, Hq, max_len, D, n + pad, n, False)
    want = want_u8.view(np.float16).reshape(B, Hq, D)
    dp = [dev(x) for x in planes]
    ds, da = dev(u8(p)), dev(amin)
    out = torch.empty((B, Hq, 1, D), dtype=torch.half, device="cuda")
    assert lib.akv_set_tuning(b"v_gqa_form", form) == 0
    try:
        check(lib, lib.akv_v_cache_compute_gqa(dp[0].data_ptr(), dp[1].data_ptr(), dp[2].data_ptr(), ds.data_ptr(),
                                               da.data_ptr(), out.data_ptr(), None, 0, B, H, G, max_len, D, n + pad, n,
                                               0, stream()))
        torch.cuda.synchronize()
    finally:
        lib.akv_set_tuning(b"v_gqa_form", 0)
    got = out.cpu().numpy().reshape(B, Hq, D)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), "grouped P.V (chain kernel) differs from the oracle"
    assert lib.akv_device_error_flag() == 0


@pytest.mark.parametrize("B,H,G,nb,nmb", [(2, 2, 4, 6, 8), (1, 4, 2, 3, 3), (1, 1, 8, 9, 12)])
@pytest.mark.parametrize("reference", [False, True])
def test_k_compute_gqa(akv_lib, B, H, G, nb, nmb, reference):
    """Grouped q.K^T: bit-exact scores against the oracle on repeated heads."""
    from oracle import akv_oracle as orc
    lib = akv_lib
    D, Hq, L = 128, H * G, nb * 64
    k, _, _ = make_kvq(41, B, L, H, D)
    _, _, q = make_kvq(42, B, 1, Hq, D)
    planes = k_planes_np(B, H, nmb, D)
    orc.k_cache_save(*planes, u8(k), B, H, nb, nmb, D, 64, 0, L)
    kexp = exponent_field(np.abs(k).max(axis=1, keepdims=True))                     # B,1,H,D
    kq = (exponent_field(q) + np.repeat(kexp, G, axis=2)).astype(np.uint8)          # B,1,Hq,D
    kqmax = kq.max(axis=3, keepdims=True)
    exp_planes = [np.ascontiguousarray(np.repeat(x, G, axis=1)) for x in planes]
    want_u8, _ = orc.k_cache_compute(*exp_planes, kq, kqmax, u8(q), B, Hq, nb, nmb, D, 64, L, 1 / math.sqrt(D),
                                     reference)
    want = want_u8.view(np.uint16).reshape(B, Hq, -1)[..., :L]
    dp = [dev(x) for x in planes]
    dkq, dkm, dq = dev(kq), dev(kqmax), dev(u8(q))
    s = torch.zeros((B, Hq, 1, (nb + 1) * 64), dtype=torch.half, device="cuda")
    check(lib, lib.akv_k_cache_compute_gqa(dp[0].data_ptr(), dp[1].data_ptr(), dp[2].data_ptr(), dkq.data_ptr(),
                                           dkm.data_ptr(), dq.data_ptr(), s.data_ptr(), B, H, G, nb, nmb, D, 64, L,
                                           1 / math.sqrt(D), int(reference), stream()))
    got = s.cpu().numpy().view(np.uint16).reshape(B, Hq, -1)[..., :L]
    assert np.array_equal(got, want), "grouped q.K^T differs from the oracle"


@pytest.mark.parametrize("B,H,G,prompt,steps,max_len,v_mode", [
    (2, 2, 4, 200, 70, 320, "exact"),          # grouped-query, crosses a block boundary
    (1, 4, 1, 255, 3, 512, "order_free"),      # multi-head, order-free P.V, first token flushes
    (2, 2, 2, 128, 3, 256, "order_free"),
    (1, 2, 4, 29, 2, 64, "exact"),             # nothing quantized yet
    (1, 4, 1, 12400, 3, 12480, "exact"),       # few long rows: the softmax is split across CTAs (4 chunks)
    (1, 2, 2, 12350, 2, 12416, "order_free"),  # a row of 12416 scores: the 512-thread softmax with the probe fused in
    (1, 2, 2, 19990, 2, 20032, "order_free"),  # split softmax (rows too long for one CTA), residual tail in the last chunk
                                               # (heads in multiples of four: the reference's kernels, and with them
                                               # the oracle, cover heads in groups of four)
    (1, 4, 1, 9000, 2, 9088, "exact"),         # rows too long for the register-cached softmax, too short to split:
                                               # plain softmax + separate probe and threshold launches
    (10, 8, 8, 100, 2, 128, "exact"),          # many rows (640): the probe is not fused into the softmax CTAs
])
def test_decode_step_ex(akv_lib, B, H, G, prompt, steps, max_len, v_mode):
    """DecodeLayer (akv_decode_step_ex) with a group and either P.V kernel against the oracle pipeline: planes
    bit-exact, outputs and packed records within 1e-3."""
    from alignedkv_b200.decode import DecodeLayer
    from oracle.pipeline import OracleGQACache
    D, Hq, L = 128, H * G, prompt + steps
    k, v, _ = make_kvq(51, B, L, H, D)
    rng = np.random.default_rng(52)
    qs = rng.standard_normal((steps, B, 1, Hq, D), dtype=np.float32).astype(np.float16)
    layer = DecodeLayer(B, max_len, H, D, "cuda:0", n_q_heads=Hq, v_mode=v_mode)
    orc = OracleGQACache(B, max_len, H, G, D)
    layer.prefill(dev(k[:, :prompt]), dev(v[:, :prompt]))
    orc.save(k[:, :prompt], v[:, :prompt], 0, prompt)
    for i in range(steps):
        kt, vt = k[:, prompt + i:prompt + i + 1], v[:, prompt + i:prompt + i + 1]
        want, want_rec = orc.decode_record(qs[i], kt, vt, order_free=(v_mode == "order_free"))
        if i % 2 == 0:
            got = layer.decode(dev(qs[i]), dev(kt), dev(vt)).cpu().numpy()
            assert rel_err(got, want) <= TOL, f"step {i}: {rel_err(got, want):.2e}"
        else:
            rec = layer.decode(dev(qs[i]), dev(kt), dev(vt), packed=True).cpu().numpy()
            assert np.allclose(rec[:, 0], want_rec[:, 0], rtol=0, atol=1e-6), "maximum score"
            assert np.allclose(rec[:, 1], want_rec[:, 1], rtol=1e-4), "sum of exponentials"
            assert rel_err(rec[:, 2:], want_rec[:, 2:]) <= TOL, f"step {i}: {rel_err(rec[:, 2:], want_rec[:, 2:]):.2e}"
    torch.cuda.synchronize()
    # exponent maxima (signed maximum over the prompt, then magnitudes of the decode tokens) per KV head
    assert np.array_equal(layer.k_exp_max.cpu().numpy(), orc.inner.k_exp_max[:, :, ::G]), "k exponent maxima"
    assert np.array_equal(layer.v_exp_max.cpu().numpy(), orc.inner.v_exp_max[:, :, ::G]), "v exponent maxima"
    got_planes = [x.cpu().numpy() for x in (layer.k_first_8, layer.k_mid_4, layer.k_last_4, layer.v_first_8,
                                            layer.v_mid_4, layer.v_last_4)]
    for g_, w_, name in zip(got_planes, orc.kv_planes(), ("k_first_8", "k_mid_4", "k_last_4", "v_first_8", "v_mid_4",
                                                          "v_last_4")):
        assert np.array_equal(g_, w_), f"plane {name} differs from the oracle"
    assert akv_lib.akv_device_error_flag() == 0


def test_device_error_flag_clear(akv_lib):
    """The device error flag is zero after healthy runs, and akv_device_error_clear leaves it zero and returns 0."""
    assert akv_lib.akv_device_error_flag() == 0
    assert akv_lib.akv_device_error_clear() == 0
    assert akv_lib.akv_device_error_flag() == 0


def test_launch_count(akv_lib):
    """The library counts its own kernel launches: a decode step with one quantized block, no flush and a residual
    tail is append, q.K^T, softmax (+ probe + the residual tokens' part of the output), P.V (+ threshold) = 4 launches."""
    from alignedkv_b200.decode import DecodeLayer
    B, H, D = 1, 2, 128
    k, v, q = make_kvq(97, B, 80, H, D)
    layer = DecodeLayer(B, 128, H, D, "cuda:0")
    layer.prefill(dev(k[:, :70]), dev(v[:, :70]))
    before = akv_lib.akv_launch_count()
    layer.launches = 0
    layer.decode(dev(q), dev(k[:, 70:71]), dev(v[:, 70:71]))
    torch.cuda.synchronize()
    assert layer.launches == 4 and akv_lib.akv_launch_count() - before == 4


@pytest.mark.parametrize("B,H,D,S,max_len", [(2, 4, 128, 200, 256), (1, 8, 128, 640, 640), (2, 2, 64, 70, 128),
                                              (1, 4, 256, 130, 192), (3, 4, 128, 63, 64)])
def test_prefill_one_pass(akv_lib, B, H, D, S, max_len):
    """akv_prefill (planes + residual tail + exponent maxima in one pass) against the oracle's prompt save:
    everything bit-exact, including the SIGNED maximum the reference uses for a prompt."""
    from alignedkv_b200.decode import DecodeLayer
    from oracle.pipeline import OracleLayerCache
    k, v, _ = make_kvq(91, B, S, H, D)
    k[:, :, 0, 5] = -np.abs(k[:, :, 0, 5])          # an all-negative channel: signed max != max magnitude
    layer = DecodeLayer(B, max_len, H, D, "cuda:0")
    orc = OracleLayerCache(B, max_len, H, D)
    layer.prefill(dev(k), dev(v))
    orc.save(k, v, 0, S)
    torch.cuda.synchronize()
    for name, got, want in (("k_first_8", layer.k_first_8, orc.k_first_8), ("k_mid_4", layer.k_mid_4, orc.k_mid_4),
                            ("k_last_4", layer.k_last_4, orc.k_last_4), ("v_first_8", layer.v_first_8, orc.v_first_8),
                            ("v_mid_4", layer.v_mid_4, orc.v_mid_4), ("v_last_4", layer.v_last_4, orc.v_last_4),
                            ("k_exp_max", layer.k_exp_max, orc.k_exp_max), ("v_exp_max", layer.v_exp_max, orc.v_exp_max)):
        assert np.array_equal(got.cpu().numpy(), want), f"{name} differs from the oracle"
    r = S % 64
    assert (layer.rest_len, layer.rest_start) == (r, S - r)
    assert np.array_equal(layer.restk[:, :r].cpu().numpy().view(np.uint16), orc.restk[:, :r].view(np.uint16))
    assert np.array_equal(layer.restv[:, :r].cpu().numpy().view(np.uint16), orc.restv[:, :r].view(np.uint16))


@pytest.mark.parametrize("prompt,steps", [(255, 1), (200, 5), (192, 70)])
def test_rollback_replays_bit_exactly(akv_lib, prompt, steps):
    """snapshot -> decode some tokens (with or without a block flush) -> restore -> the same tokens again: outputs and
    planes are bit-identical to the first pass (akv_rollback clears the K nibble blocks written since, which the
    accumulating K writer needs)."""
    from alignedkv_b200.decode import DecodeLayer
    B, H, D, max_len = 2, 4, 128, 320
    k, v, _ = make_kvq(95, B, prompt + steps, H, D)
    rng = np.random.default_rng(96)
    qs = rng.standard_normal((steps, B, 1, H, D), dtype=np.float32).astype(np.float16)
    layer = DecodeLayer(B, max_len, H, D, "cuda:0")
    layer.prefill(dev(k[:, :prompt]), dev(v[:, :prompt]))
    snap = layer.snapshot()

    def run():
        outs = [layer.decode(dev(qs[i]), dev(k[:, prompt + i:prompt + i + 1]), dev(v[:, prompt + i:prompt + i + 1]))
                for i in range(steps)]
        planes = [x.clone() for x in (layer.k_first_8, layer.k_mid_4, layer.k_last_4, layer.v_first_8, layer.v_mid_4,
                                      layer.v_last_4, layer.k_exp_max, layer.v_exp_max)]
        return outs, planes
    o1, p1 = run()
    layer.restore(snap)
    assert (layer.cache_len, layer.rest_len) == (prompt, prompt % 64)
    o2, p2 = run()
    for a, b in zip(o1 + p1, o2 + p2):
        assert torch.equal(a, b)
    future = layer.snapshot()
    future["cache_len"] = layer.cache_len + 1          # a snapshot from the future cannot be restored
    with pytest.raises(RuntimeError):
        layer.restore(future)


def test_lse_merge(akv_lib):
    from oracle.pipeline import lse_merge_np
    lib = akv_lib
    rng = np.random.default_rng(61)
    R, rows, D = 5, 37, 128
    packed = np.empty((R, rows, D + 2), np.float32)
    packed[..., 0] = rng.standard_normal((R, rows)) * 8
    packed[..., 1] = rng.uniform(1, 4000, (R, rows))
    packed[..., 2:] = rng.standard_normal((R, rows, D))
    packed[3, :, 1] = 0                      # a shard without tokens
    packed[3, :, 0] = -np.inf
    packed[3, :, 2:] = np.nan
    out = torch.empty((rows, D), dtype=torch.half, device="cuda")
    dp = dev(packed)
    check(lib, lib.akv_lse_merge(dp.data_ptr(), out.data_ptr(), R, rows, D, stream()))
    want = lse_merge_np(packed)
    assert rel_err(out.cpu().numpy(), want) <= TOL


def test_sequence_shards_merge_to_dense_attention(akv_lib):
    """The shards of a sequence-sharded cache, emulated as independent layers on one GPU: packed records merged by
    akv_lse_merge against (i) the same protocol in numpy on oracle shards (<= 1e-3) and (ii) fp32 dense attention
    over the whole sequence (error reported; bounded by 6e-2: the aligned path itself is 1e-2 .. 4e-2 off fp32 because of
    the skipped nibble planes and fp16 scores, a wrong merge would be off by order 1)."""
    from alignedkv_b200.decode import DecodeLayer
    from alignedkv_b200.sharded import shard_bounds
    from oracle.pipeline import OracleLayerCache, dense_attention_fp32, lse_merge_np
    lib = akv_lib
    B, H, D, S, R = 1, 4, 128, 1024 + 40, 4
    k, v, q = make_kvq(71, B, S + 1, H, D)
    bounds = shard_bounds(S, R)
    assert bounds[0][0] == 0 and bounds[-1][1] == S and all(lo % 64 == 0 for lo, _ in bounds)
    recs, want_recs = [], []
    for r, (lo, hi) in enumerate(bounds):
        last = r == R - 1
        max_local = -(-(hi - lo + (1 if last else 0)) // 64) * 64
        layer = DecodeLayer(B, max_local, H, D, "cuda:0", v_mode="order_free")
        orc = OracleLayerCache(B, max_local, H, D)
        layer.prefill(dev(k[:, lo:hi]), dev(v[:, lo:hi]))
        orc.save(k[:, lo:hi], v[:, lo:hi], 0, hi - lo)
        kt, vt = (dev(k[:, S:]), dev(v[:, S:])) if last else (None, None)
        recs.append(layer.decode(dev(q), kt, vt, append=last, packed=True))
        want_recs.append(orc.decode_record(q, k[:, S:] if last else None, v[:, S:] if last else None, append=last,
                                           order_free=True)[1])
    gathered = torch.stack(recs).contiguous()
    out = torch.empty((B * H, D), dtype=torch.half, device="cuda")
    check(lib, lib.akv_lse_merge(gathered.data_ptr(), out.data_ptr(), R, B * H, D, stream()))
    got = out.cpu().numpy()
    want = lse_merge_np(np.stack(want_recs))
    assert rel_err(got, want) <= TOL, f"vs numpy protocol: {rel_err(got, want):.2e}"
    truth = dense_attention_fp32(q, k, v).reshape(B * H, D)
    err = rel_err(got, truth)
    print(f"sequence-sharded merge vs fp32 dense attention: {err:.2e}")
    assert err <= 6e-2


def _exchange_buffers(lib, R, rows, D):
    """R exchange buffers of one process (stand-ins for the ranks' buffers): words [2][R][rows][D+2] of (float bits,
    epoch), with a float view (values at [..., 0]) and an int view (epochs at [..., 1]) of each."""
    W = D + 2
    nbytes = lib.akv_exchange_bytes(R, rows, D)
    assert nbytes == 2 * R * rows * W * 8
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(R)]
    data = [b.view(torch.float32).view(2, R, rows, W, 2) for b in bufs]
    flags = [b.view(torch.int32).view(2, R, rows, W, 2) for b in bufs]
    ptrs = (ctypes.c_void_p * R)(*[b.data_ptr() for b in bufs])
    return bufs, data, flags, ptrs


def _place(data, flags, r, par, g, rec, epoch):
    """Puts rank g's record and its epoch into rank r's buffer, as rank g's kernel would have."""
    data[r][par, g, :, :, 0] = rec
    flags[r][par, g, :, :, 1] = epoch


@pytest.mark.parametrize("R", [2, 3, 8])
def test_exchange_merge_matches_lse_merge(akv_lib, R):
    """akv_exchange_merge (publish to every rank's buffer, collect, merge) on one GPU: the other ranks' records (every
    float with its epoch) are put into the buffers beforehand from the host side, so the launch never waits for another kernel.  The merged
    rows equal akv_lse_merge over the same records bit for bit; this rank's record and flags reach every buffer; two
    consecutive epochs use the two halves of the buffers."""
    lib = akv_lib
    rows, D = 12, 128
    W = D + 2
    gen = torch.Generator(device="cuda").manual_seed(5 + R)
    bufs, data, flags, ptrs = _exchange_buffers(lib, R, rows, D)
    for epoch in (1, 2, 3):
        par = epoch & 1
        rec = torch.randn(R, rows, W, device="cuda", generator=gen)
        rec[:, :, 1] = rec[:, :, 1].abs() + 0.1
        rec[R - 1, ::3, 1] = 0.0                                # shards without tokens in some rows
        want = torch.empty((rows, D), dtype=torch.half, device="cuda")
        check(lib, lib.akv_lse_merge(rec.data_ptr(), want.data_ptr(), R, rows, D, stream()))
        for r in range(R):
            for g in range(R):
                if g != r:
                    _place(data, flags, r, par, g, rec[g], epoch)
            out = torch.full((rows, D), 7.0, dtype=torch.half, device="cuda")
            check(lib, lib.akv_exchange_merge(ptrs, r, R, rec[r].contiguous().data_ptr(), out.data_ptr(), rows, D, epoch,
                                              1000, stream()))
            torch.cuda.synchronize()
            assert torch.equal(out, want), f"rank {r} of {R}, epoch {epoch}"
            for g in range(R):
                assert torch.equal(data[g][par, r, :, :, 0], rec[r]) and bool((flags[g][par, r, :, :, 1] == epoch).all())
    assert lib.akv_device_error_flag() == 0


def test_exchange_wait_runs_out(akv_lib):
    """A rank whose peer never publishes: the bounded wait of akv_exchange_merge runs out after the given time, the
    kernel raises the device error flag, writes zeros and returns; the context stays usable and the flag clears."""
    lib = akv_lib
    R, rows, D = 2, 4, 128
    bufs, data, flags, ptrs = _exchange_buffers(lib, R, rows, D)
    rec = torch.ones(rows, D + 2, device="cuda")
    out = torch.full((rows, D), 7.0, dtype=torch.half, device="cuda")
    check(lib, lib.akv_exchange_merge(ptrs, 0, R, rec.data_ptr(), out.data_ptr(), rows, D, 1, 20, stream()))
    torch.cuda.synchronize()
    assert lib.akv_device_error_flag() & 4
    assert bool((out == 0).all())
    assert lib.akv_device_error_clear() == 0 and lib.akv_device_error_flag() == 0
    _place(data, flags, 0, 1, 1, rec, 1)                         # now the peer's record is there
    check(lib, lib.akv_exchange_merge(ptrs, 0, R, rec.data_ptr(), out.data_ptr(), rows, D, 1, 20, stream()))
    torch.cuda.synchronize()
    assert lib.akv_device_error_flag() == 0 and bool((out == 1).all())


class _LocalPeers:
    """Stands in for `sharded.PeerExchange` when all the "ranks'" buffers live in this process."""

    def __init__(self, ptrs, rank, world):
        self.bufs, self.rank, self.world, self.timeout_ms, self.epoch = ptrs, rank, world, 1000, 0

    def next_epoch(self):
        self.epoch += 1
        return self.epoch


def test_decode_step_exchange_matches_merge(akv_lib):
    """akv_decode_step_exchange (the exchange and the merge at the end of the step's last kernel) for every shard of a
    sequence in turn, the other shards' records and flags put into the buffers beforehand: the merged output equals
    akv_lse_merge over the records of plain packed steps bit for bit, and the shard's own record is returned as before."""
    from alignedkv_b200.decode import DecodeLayer
    from alignedkv_b200.sharded import shard_bounds
    lib = akv_lib
    B, H, D, S, R = 1, 4, 128, 2048 + 40, 3
    rows = B * H
    k, v, q = make_kvq(73, B, S + 1, H, D)
    bounds = shard_bounds(S, R)

    def shard(r):
        lo, hi = bounds[r]
        last = r == R - 1
        layer = DecodeLayer(B, -(-(hi - lo + (1 if last else 0)) // 64) * 64, H, D, "cuda:0", v_mode="order_free")
        layer.prefill(dev(k[:, lo:hi]), dev(v[:, lo:hi]))
        return layer, ((dev(k[:, S:]), dev(v[:, S:])) if last else (None, None)), last

    recs = []
    for r in range(R):
        layer, (kt, vt), last = shard(r)
        recs.append(layer.decode(dev(q), kt, vt, append=last, packed=True))
    gathered = torch.stack(recs).contiguous()
    want = torch.empty((rows, D), dtype=torch.half, device="cuda")
    check(lib, lib.akv_lse_merge(gathered.data_ptr(), want.data_ptr(), R, rows, D, stream()))
    for r in range(R):
        bufs, data, flags, ptrs = _exchange_buffers(lib, R, rows, D)
        for g in range(R):
            if g != r:
                _place(data, flags, r, 1, g, recs[g], 1)
        layer, (kt, vt), last = shard(r)
        out = layer.decode(dev(q), kt, vt, append=last, exchange=_LocalPeers(ptrs, r, R))
        torch.cuda.synchronize()
        assert out.shape == (B, 1, H, D) and torch.equal(out.view(rows, D), want), f"shard {r}"
        assert torch.equal(data[(r + 1) % R][1, r, :, :, 0], recs[r])        # its record reached the other buffers
    assert lib.akv_device_error_flag() == 0


class _LoneComm:
    """Stands in for the collectives when several shards are driven phase by phase inside one process."""
    world = 1

    def all_reduce(self, x, op):
        return x


@pytest.mark.parametrize("prompt,steps,world", [(16500, 3, 2), (20470, 4, 3)])
def test_decision_exact_shards(akv_lib, prompt, steps, world):
    """Sequence shards decoded with akv_shard_step (exchanges done by hand, all shards on this GPU) against one
    DecodeLayer over the whole sequence that takes the split-softmax path: probabilities and threshold bytes - hence
    every plane-read decision - bit-identical, outputs equal up to the grouping of the fp32 partial sums."""
    from alignedkv_b200.decode import DecodeLayer
    from alignedkv_b200.extension._planes import exponent_field
    from alignedkv_b200.sharded import (DecisionExactShardedDecoder, chunk_bounds, pad_chunks, pad_stats,
                                        sequence_order)
    B, H, G, D = 1, 4, 1, 128
    Hq, L = H * G, prompt + steps
    k, v, _ = make_kvq(71, B, L, H, D)
    rng = np.random.default_rng(72)
    qs = rng.standard_normal((steps, B, 1, Hq, D), dtype=np.float32).astype(np.float16)
    max_len = -(-L // 64) * 64
    whole = DecodeLayer(B, max_len, H, D, "cuda:0", n_q_heads=Hq, v_mode="order_free")
    whole.prefill(dev(k[:, :prompt]), dev(v[:, :prompt]))
    bounds = chunk_bounds(prompt, world)
    decs = [DecisionExactShardedDecoder(B, prompt, steps, H, D, "cuda:0", n_q_heads=Hq, comm=_LoneComm(), rank=r,
                                        world=world) for r in range(world)]
    for r, dec in enumerate(decs):
        lo, hi = bounds[r]
        dec.prefill(dev(np.ascontiguousarray(k[:, lo:hi])), dev(np.ascontiguousarray(v[:, lo:hi])))
        # the exponent maxima of the whole prompt (what the all-reduce gives every rank)
        dec.layer.k_exp_max.copy_(exponent_field(dev(k[:, :prompt]).max(dim=1, keepdim=True).values))
        dec.layer.v_exp_max.copy_(exponent_field(dev(v[:, :prompt]).max(dim=1, keepdim=True).values))
    assert torch.equal(decs[0].layer.k_exp_max, whole.k_exp_max) and torch.equal(decs[0].layer.v_exp_max, whole.v_exp_max)
    rows = B * Hq
    for i in range(steps):
        q, kt, vt = dev(qs[i]), dev(k[:, prompt + i:prompt + i + 1]), dev(v[:, prompt + i:prompt + i + 1])
        want = whole.decode(q, kt, vt)
        cmax = max(d_._chunks_of(r, d_.appended + 1) for r, d_ in enumerate(decs))
        total = world * cmax
        st = [pad_stats(d_.phase(1, None, q, kt, vt), cmax) for d_ in decs]
        st_all = sequence_order(torch.stack(st))
        cand = [d_.phase(2, st_all, q, kt, vt, total) for d_ in decs]
        g = torch.stack([torch.stack([pad_chunks(c[0], cmax, 0), pad_chunks(c[1], cmax, 0)]) for c in cand])
        cand_all = torch.stack([sequence_order(g[:, 0]), sequence_order(g[:, 1])]).contiguous()
        win = [d_.phase(3, cand_all, q, kt, vt, total) for d_ in decs]
        win_all = win[0].clone()
        for w_ in win[1:]:
            assert int(((win_all != 0) & (w_ != 0)).sum()) == 0, "a winner's row came from two shards"
            win_all += w_
        parts = [d_.phase(4, win_all, q, kt, vt, total)[:, 2:] for d_ in decs]
        got = parts[0].clone()
        for p_ in parts[1:]:
            got += p_
        torch.cuda.synchronize()
        # decisions: threshold bytes and probabilities of every shard against the whole-sequence run
        a_off = whole._scratch_offset("amin")
        amin_whole = whole.scratch[a_off:a_off + rows].cpu()
        qn_whole = whole.rest_start
        R_whole = (qn_whole // 64 + 1) * 64
        p_whole = whole.scratch[:rows * R_whole * 2].view(torch.int16).view(rows, R_whole).cpu()
        for r, d_ in enumerate(decs):
            lay = d_.layer
            o = lay._scratch_offset("amin")
            assert torch.equal(lay.scratch[o:o + rows].cpu(), amin_whole), f"step {i}: threshold bytes of shard {r}"
            d_.finish_step()
            qn = lay.rest_start
            R_loc = (qn // 64 + 1) * 64
            p_loc = lay.scratch[:rows * R_loc * 2].view(torch.int16).view(rows, R_loc).cpu()
            n_loc = qn + lay.rest_len
            assert torch.equal(p_loc[:, :n_loc], p_whole[:, d_.token_base:d_.token_base + n_loc]), \
                f"step {i}: probabilities of shard {r}"
        assert rel_err(got.cpu().numpy(), want.float().cpu().numpy().reshape(rows, D)) <= TOL
    assert akv_lib.akv_device_error_flag() == 0
