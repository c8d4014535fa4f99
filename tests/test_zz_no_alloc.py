"""The allocation-free decode step (akv_decode_step_noalloc), called through the C ABI.

Who needs it: a host that may not allocate device memory when it calls in - an inference server whose GPU memory
was partitioned once at start-up, or a plugin invoked from a context where cudaMalloc is off limits because it
synchronises the device.  Such a caller still passes every input and output buffer; only the step's workspace comes
from a fixed array inside the library.  The test runs two decode steps in a row through the new entry point and
through akv_decode_step (caller-provided workspace) on identical cache states and requires identical bytes: the two
entry points launch the same kernels, so the tolerance of the other pipeline tests (1e-3) is met with zero error.
This file sorts last so that a run that stops at the first failure has already run everything else; it also passes
when run alone in a fresh process."""
import numpy as np
import pytest

from helpers import make_kvq

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _args(layer, q, k, v, out):
    return [layer.k_first_8.data_ptr(), layer.k_mid_4.data_ptr(), layer.k_last_4.data_ptr(),
            layer.v_first_8.data_ptr(), layer.v_mid_4.data_ptr(), layer.v_last_4.data_ptr(),
            layer.k_exp_max.data_ptr(), layer.v_exp_max.data_ptr(), layer.restk.data_ptr(), layer.restv.data_ptr(),
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()]


def test_noalloc_decode_step_matches_decode_step(akv_lib):
    from alignedkv_b200 import _lib
    from alignedkv_b200.decode import DecodeLayer
    lib = akv_lib
    assert lib.akv_set_tuning(b"timing", 0) == 0
    B, H, D, prompt, max_len = 2, 4, 128, 254, 320      # the second step completes block 3 and flushes it
    dev = torch.device("cuda:0")
    kk, vv, _ = make_kvq(31, B, prompt + 2, H, D)
    qs = np.random.default_rng(32).standard_normal((2, B, 1, H, D), dtype=np.float32).astype(np.float16)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    a, b = DecodeLayer(B, max_len, H, D, dev), DecodeLayer(B, max_len, H, D, dev)
    for layer in (a, b):
        layer.prefill(t(kk[:, :prompt]), t(vv[:, :prompt]))
    stream = torch.cuda.current_stream(dev).cuda_stream
    for i in range(2):
        pos = prompt + i
        q, k, v = t(qs[i]), t(kk[:, pos:pos + 1]), t(vv[:, pos:pos + 1])
        out_a = torch.full((B, 1, H, D), float("nan"), dtype=torch.half, device=dev)
        out_b = torch.full((B, 1, H, D), float("nan"), dtype=torch.half, device=dev)
        rc = lib.akv_decode_step(*_args(a, q, k, v, out_a), a.scratch.data_ptr(), a.scratch.numel(), B, H, D, max_len,
                                 a.rest_len, a.rest_start, 0, stream)
        _lib.check("decode_step", rc)
        torch.cuda.synchronize(dev)
        free_before, torch_before = torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev)
        rc = lib.akv_decode_step_noalloc(*_args(b, q, k, v, out_b), B, H, D, max_len, b.rest_len, b.rest_start, 0,
                                         stream)
        _lib.check("decode_step_noalloc", rc)
        torch.cuda.synchronize(dev)
        if i == 1:
            # the second call (every kernel of the step, block writers included, was loaded by the first two library
            # steps above) takes no device memory: neither from the driver nor from torch's allocator
            assert torch.cuda.mem_get_info(dev)[0] == free_before, "the allocation-free step took device memory"
            assert torch.cuda.memory_allocated(dev) == torch_before
        for layer in (a, b):      # advance the host-side residual state as the caller of the C ABI must
            if layer.rest_len + 1 == 64:
                layer.rest_len, layer.rest_start = 0, layer.rest_start + 64
            else:
                layer.rest_len += 1
            layer.cache_len += 1
        assert not torch.isnan(out_b.float()).any()
        assert torch.equal(out_a, out_b), f"step {i}: outputs differ"
    assert (b.rest_len, b.rest_start) == (0, 256)
    for name in ("k_first_8", "k_mid_4", "k_last_4", "v_first_8", "v_mid_4", "v_last_4", "k_exp_max", "v_exp_max"):
        assert torch.equal(getattr(a, name), getattr(b, name)), name


def test_noalloc_rejects_what_does_not_fit(akv_lib):
    from alignedkv_b200 import _lib
    lib = akv_lib
    one = 16
    # a workspace far beyond the built-in 8 MiB: refused before anything is launched
    assert lib.akv_decode_scratch_bytes(64, 32, 128, 8192) > (8 << 20)
    rc = lib.akv_decode_step_noalloc(*([one] * 14), 64, 32, 128, 8192, 0, 0, 0, None)
    assert rc == -2 and b"built-in one holds" in lib.akv_last_error()
    with pytest.raises(_lib.AlignedKVError):
        _lib.check("decode_step_noalloc", rc)
