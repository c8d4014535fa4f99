"""The Llama-shaped decoder driver (full-decoder configuration) on a small shape: the AlignedKV cache on every layer
against the same weights with dense fp16 torch attention.  The aligned path is an approximation (skipped nibble planes,
fp16 accumulation in the reference's order), so logits are compared with a max-norm relative tolerance of 5e-2 and the
greedy tokens must agree for a clear majority of steps."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv_heads,v_mode", [(4, "exact"), (2, "order_free")])
def test_decoder_matches_dense_attention(akv_lib, kv_heads, v_mode):
    from alignedkv_b200.llama import LlamaConfig, LlamaDecoder
    cfg = LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=kv_heads, vocab_size=1000)
    B, S, new = 2, 150, 6
    ids = torch.randint(0, cfg.vocab_size, (B, S), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    a = LlamaDecoder(cfg, B, S + new + 1, "cuda:0", seed=1, v_mode=v_mode)
    d = LlamaDecoder(cfg, B, S + new + 1, "cuda:0", seed=1, attention="dense")
    la, ld = a.prefill(ids), d.prefill(ids)
    assert torch.equal(la, ld), "the prompt path is the same dense attention in both"
    agree, worst = 0, 0.0
    tok = ld.argmax(-1)
    for _ in range(new):
        la, ld = a.step(tok), d.step(tok)
        err = float((la.float() - ld.float()).abs().max() / ld.float().abs().max())
        worst = max(worst, err)
        agree += int(torch.equal(la.argmax(-1), ld.argmax(-1)))
        tok = ld.argmax(-1)
    print(f"decoder logits: worst max-norm relative error {worst:.2e}; greedy tokens agree in {agree}/{new} steps")
    assert worst <= 5e-2
    assert agree >= new - 2
    assert akv_lib.akv_device_error_flag() == 0


def test_decoder_graph_replay_matches_eager(akv_lib):
    """The decode step with its dense parts replayed from CUDA graphs gives the logits of the eager step."""
    from alignedkv_b200.llama import LlamaConfig, LlamaDecoder
    cfg = LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=4, vocab_size=1000)
    B, S, new = 2, 100, 5
    ids = torch.randint(0, cfg.vocab_size, (B, S), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    a = LlamaDecoder(cfg, B, S + new + 1, "cuda:0", seed=2)
    b = LlamaDecoder(cfg, B, S + new + 1, "cuda:0", seed=2)
    tok = a.prefill(ids).argmax(-1)
    assert torch.equal(tok, b.prefill(ids).argmax(-1))
    b.capture_graphs()
    for _ in range(new):
        la, lb = a.step(tok), b.step(tok).clone()
        err = float((la.float() - lb.float()).abs().max() / la.float().abs().max())
        assert err <= 1e-3, err
        tok = la.argmax(-1)
    assert a.pos == b.pos and akv_lib.akv_device_error_flag() == 0
