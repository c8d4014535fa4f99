"""Minimal Llama-shaped decoder that drives the AlignedKV cache on every layer.

Stands in for the reference's model glue (model/Llama_AlignedKV.py, a transformers 4.44 subclass that cannot run under
the installed transformers) for the full-decoder configuration: RMSNorm, rotary embeddings, grouped-query attention and
SwiGLU exactly as in Llama; the projections are plain fp16 matmuls (cuBLAS through torch); attention follows the
reference's cache: the prompt uses dense causal attention and fills the cache (model/KVCache_AlignedKV.py:92-99), every
later token goes through `DecodeLayer.decode` - append, aligned q.K^T, softmax, aligned P.V
(model/KVCache_AlignedKV.py:116-124; call site model/Llama_AlignedKV.py:111-113).  Weights are random-initialised
(N(0, 0.02), the configuration's stated stand-in for the checkpoint that is not available offline).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .decode import DecodeLayer

__all__ = ["LlamaConfig", "LlamaDecoder"]


@dataclass
class LlamaConfig:
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    vocab_size: int = 32000
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


def _rms_norm(x, w, eps):
    return F.rms_norm(x, (x.shape[-1],), w, eps)


def _rope_tables(pos, D, theta):
    """cos / signed sin tables [1,S,1,D] (fp32) of the rotate_half form of the rotary embedding (as HF Llama)."""
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=pos.device, dtype=torch.float32) / D))
    ang = pos.float()[:, None] * inv[None, :]                       # S, D/2
    cos = torch.cat([ang.cos(), ang.cos()], -1)[None, :, None, :]
    sin = torch.cat([-ang.sin(), ang.sin()], -1)[None, :, None, :]  # sign of rotate_half folded in
    return cos, sin


def _rope(x, tables):
    """x [B,S,H,D] -> x * cos + rotate_half(x) * sin."""
    cos, sin = tables
    D = x.shape[-1]
    swapped = torch.cat([x[..., D // 2:], x[..., :D // 2]], -1)
    return torch.addcmul(x.float() * cos, swapped.float(), sin).to(x.dtype)


class LlamaDecoder:
    """Random-init Llama decoder with one AlignedKV `DecodeLayer` per transformer layer."""

    def __init__(self, cfg: LlamaConfig, bsz: int, max_seq_len: int, device, seed: int = 0, v_mode: str = "exact",
                 attention: str = "alignedkv"):
        self.cfg, self.B, self.L = cfg, bsz, max_seq_len
        self.device = torch.device(device)
        self.attention = attention                  # "alignedkv" or "dense" (fp16 torch attention over a plain cache)
        g = torch.Generator(device=self.device).manual_seed(seed)
        H, Hkv, D, E, Fi = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.hidden_size, \
            cfg.intermediate_size

        def w(*shape):
            return (torch.randn(*shape, device=self.device, generator=g) * 0.02).half()

        self.embed = w(cfg.vocab_size, E)
        self.lm_head = w(cfg.vocab_size, E)
        self.final_norm = torch.ones(E, dtype=torch.half, device=self.device)
        self.layers = []
        for _ in range(cfg.num_hidden_layers):
            self.layers.append(dict(
                wqkv=w((H + 2 * Hkv) * D, E), wo=w(E, H * D), w_gate_up=w(2 * Fi, E), w_down=w(E, Fi),
                norm1=torch.ones(E, dtype=torch.half, device=self.device),
                norm2=torch.ones(E, dtype=torch.half, device=self.device)))
        if attention == "alignedkv":
            self.caches = [DecodeLayer(bsz, max_seq_len, Hkv, D, self.device, n_q_heads=H, v_mode=v_mode)
                           for _ in range(cfg.num_hidden_layers)]
        else:
            self.kcache = [torch.zeros(bsz, max_seq_len, Hkv, D, dtype=torch.half, device=self.device)
                           for _ in range(cfg.num_hidden_layers)]
            self.vcache = [torch.zeros_like(t) for t in self.kcache]
        self.pos = 0

    # ------------------------------------------------------------------ one transformer layer
    def _layer(self, i: int, x: torch.Tensor, pos: torch.Tensor, prompt: bool) -> torch.Tensor:
        cfg, p = self.cfg, self.layers[i]
        H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        B, S, _ = x.shape
        h = _rms_norm(x, p["norm1"], cfg.rms_norm_eps)
        qkv = F.linear(h, p["wqkv"]).view(B, S, H + 2 * Hkv, D)
        qk = _rope(qkv[:, :, :H + Hkv], pos)             # queries and keys rotate together
        q, k = qk[:, :, :H].contiguous(), qk[:, :, H:].contiguous()
        v = qkv[:, :, H + Hkv:].contiguous()
        if prompt:
            # dense causal attention over the prompt, then the cache takes the keys and values
            kk, vv = (t.repeat_interleave(H // Hkv, dim=2) if Hkv != H else t for t in (k, v))
            o = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                               is_causal=True).transpose(1, 2)
            if self.attention == "alignedkv":
                self.caches[i].prefill(k, v)
            else:
                self.kcache[i][:, :S] = k
                self.vcache[i][:, :S] = v
        elif self.attention == "alignedkv":
            o = self.caches[i].decode(q, k, v)                                   # [B,1,H,D]
        else:
            n = self.pos + 1
            self.kcache[i][:, self.pos:n] = k
            self.vcache[i][:, self.pos:n] = v
            kk, vv = self.kcache[i][:, :n], self.vcache[i][:, :n]
            if Hkv != H:
                kk, vv = kk.repeat_interleave(H // Hkv, dim=2), vv.repeat_interleave(H // Hkv, dim=2)
            s = torch.matmul(q.transpose(1, 2), kk.permute(0, 2, 3, 1)) / math.sqrt(D)
            o = torch.matmul(F.softmax(s.float(), dim=-1).to(q.dtype), vv.transpose(1, 2)).transpose(1, 2)
        x = torch.addmm(x.view(B * S, -1), o.reshape(B * S, H * D), p["wo"].t()).view(B, S, -1)
        h = _rms_norm(x, p["norm2"], cfg.rms_norm_eps)
        gate, up = F.linear(h, p["w_gate_up"]).chunk(2, dim=-1)
        return torch.addmm(x.view(B * S, -1), F.silu(gate).mul_(up).view(B * S, -1), p["w_down"].t()).view(B, S, -1)

    # ------------------------------------------------------------------ decode step with the dense parts as CUDA graphs
    def _pre(self, i: int, x: torch.Tensor, tables):
        """Everything of layer i before its attention: norm, q/k/v projection, rotary embedding."""
        cfg, p = self.cfg, self.layers[i]
        H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        B = x.shape[0]
        qkv = F.linear(_rms_norm(x, p["norm1"], cfg.rms_norm_eps), p["wqkv"]).view(B, 1, H + 2 * Hkv, D)
        qk = _rope(qkv[:, :, :H + Hkv], tables)
        return qk[:, :, :H].contiguous(), qk[:, :, H:].contiguous(), qkv[:, :, H + Hkv:].contiguous()

    def _post(self, i: int, x: torch.Tensor, o: torch.Tensor) -> torch.Tensor:
        """Everything of layer i after its attention: output projection, residual, SwiGLU MLP, residual."""
        cfg, p = self.cfg, self.layers[i]
        B = x.shape[0]
        x = torch.addmm(x.view(B, -1), o.reshape(B, -1), p["wo"].t()).view(B, 1, -1)
        gate, up = F.linear(_rms_norm(x, p["norm2"], cfg.rms_norm_eps), p["w_gate_up"]).chunk(2, dim=-1)
        return torch.addmm(x.view(B, -1), F.silu(gate).mul_(up).view(B, -1), p["w_down"].t()).view(B, 1, -1)

    @torch.no_grad()
    def capture_graphs(self) -> None:
        """Capture the dense parts of a decode step as CUDA graphs: one graph per stretch between two attention calls
        (embedding + layer 0 up to its attention; the rest of layer i + layer i+1 up to its attention; the rest of the
        last layer + final norm + logits).  The attention calls stay ordinary launches between the replays - the
        cache's state (residual length, block count) changes from token to token and is passed by value.  After this,
        `step` replays: ~35 torch launches per layer become one graph launch, which is what the step was bound by."""
        assert self.attention == "alignedkv", "only the AlignedKV path is split into graphs"
        cfg, B, dev = self.cfg, self.B, self.device
        H, D, n = cfg.num_attention_heads, cfg.head_dim, cfg.num_hidden_layers
        self._g_ids = torch.zeros(B, dtype=torch.long, device=dev)
        self._g_pos = torch.zeros(1, dtype=torch.long, device=dev)
        self._g_o = torch.zeros(B, 1, H, D, dtype=torch.half, device=dev)
        segs = []          # (graph, outputs) per stretch

        def run(j, x_prev):
            tables = _rope_tables(self._g_pos, D, cfg.rope_theta)
            if j == 0:
                x = self.embed[self._g_ids].view(B, 1, -1)
            else:
                x = self._post(j - 1, x_prev, self._g_o)
            if j == n:
                x = _rms_norm(x, self.final_norm, cfg.rms_norm_eps)
                return (F.linear(x, self.lm_head)[:, 0],)
            return (x,) + self._pre(j, x, tables)

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        x_prev = None
        with torch.cuda.stream(side):
            for j in range(n + 1):              # warm-up outside capture (library workspaces, lazy initialisation)
                outs = run(j, x_prev)
                x_prev = outs[0]
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        x_prev = None
        for j in range(n + 1):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                outs = run(j, x_prev)
            segs.append((g, outs))
            x_prev = outs[0]
        self._segs = segs

    def _step_graphs(self, ids: torch.Tensor) -> torch.Tensor:
        n = self.cfg.num_hidden_layers
        self._g_ids.copy_(ids.view(-1))
        self._g_pos.fill_(self.pos)
        for j in range(n):
            g, (x, q, k, v) = self._segs[j]
            g.replay()
            self.caches[j].decode(q, k, v, out=self._g_o)
        g, (logits,) = self._segs[n]
        g.replay()
        self.pos += 1
        return logits

    def _forward(self, ids: torch.Tensor, prompt: bool) -> torch.Tensor:
        B, S = ids.shape
        pos = _rope_tables(torch.arange(self.pos, self.pos + S, device=self.device), self.cfg.head_dim,
                           self.cfg.rope_theta)
        x = self.embed[ids]
        for i in range(self.cfg.num_hidden_layers):
            x = self._layer(i, x, pos, prompt)
        self.pos += S
        x = _rms_norm(x[:, -1:], self.final_norm, self.cfg.rms_norm_eps)
        return F.linear(x, self.lm_head)[:, 0]                                   # logits of the last position [B,V]

    # ------------------------------------------------------------------ public
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B,S] -> logits [B,V] of the last prompt position; fills every layer's cache."""
        assert self.pos == 0 and ids.shape[0] == self.B and ids.shape[1] <= self.L
        return self._forward(ids, True)

    @torch.no_grad()
    def step(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B] (one token per sequence) -> logits [B,V]; appends to every layer's cache."""
        assert self.pos + 1 <= self.L
        if getattr(self, "_segs", None) is not None:
            return self._step_graphs(ids)       # (the returned logits are overwritten by the next step)
        return self._forward(ids.view(self.B, 1), False)

    @torch.no_grad()
    def generate(self, ids: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Greedy decoding: returns [B, new_tokens]."""
        out = []
        tok = self.prefill(ids).argmax(-1)
        for _ in range(new_tokens):
            out.append(tok)
            tok = self.step(tok).argmax(-1)
        return torch.stack(out, 1)
