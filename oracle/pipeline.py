"""numpy restatement of the reference's per-layer decode pipeline around the five operators.  TEST
INFRASTRUCTURE ONLY (see oracle/akv_oracle.py).

Follows extension/k_cache_file.py:69-159 (K store: residual buffering, exponent maxima, alignment inputs, residual
scores, -inf padding), extension/v_cache_file.py:72-190 (V store: probe inputs, threshold arithmetic with its
[B,H,H,D] broadcast, residual P.V) and model/KVCache_AlignedKV.py:72-135 (prefill = dense attention, decode =
append -> q.K^T -> fp32 softmax -> P.V).  Operators are the C restatements in oracle/akv_oracle.c.
Also holds the two dense baselines: fp32 "truth" attention and the reference's fp16 torch path on CPU.
"""
from __future__ import annotations

import math

import numpy as np

from . import akv_oracle as orc

COLUMN_BLOCK = 64
TOP_MAX_K = 32


def exponent_field(x16: np.ndarray) -> np.ndarray:
    """(x.view(int16) >> 10).to(uint8) & 0x1F of the reference."""
    return ((np.ascontiguousarray(x16).view(np.uint16) >> 10) & 0x1F).astype(np.uint8)


def softmax_fp32_to_half(scores16: np.ndarray) -> np.ndarray:
    """F.softmax(scores.float(), dim=-1).type_as(q) (model/KVCache_AlignedKV.py:121)."""
    x = scores16.astype(np.float32)
    m = x.max(axis=-1, keepdims=True)
    e = np.exp(x - m, dtype=np.float32)
    return (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float16)


def dense_attention_fp32(q16, k16, v16) -> np.ndarray:
    """fp32 truth: softmax(q K^T / sqrt(D)) V from the original fp16 tensors.  q [B,1,H,D]; k, v [B,L,H,D]."""
    q = q16.astype(np.float32).transpose(0, 2, 1, 3)          # B,H,1,D
    k = k16.astype(np.float32).transpose(0, 2, 1, 3)          # B,H,L,D
    v = v16.astype(np.float32).transpose(0, 2, 1, 3)
    s = np.matmul(q, k.transpose(0, 1, 3, 2)) / math.sqrt(q.shape[-1])
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    return np.matmul(p, v).transpose(0, 2, 1, 3)               # B,1,H,D


def dense_attention_torch_cpu(q, k, v):
    """The reference's dense path on the host: matmul(q,k^T)/sqrt(D) -> softmax(float) -> matmul(.,v) on fp16
    torch tensors (model/KVCache_AlignedKV.py:77-79,97,87-88).  q [B,1,H,D]; k, v [B,L,H,D] (torch, CPU)."""
    import torch
    import torch.nn.functional as F
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    scores = torch.matmul(qt, kt.transpose(2, 3)) / math.sqrt(q.shape[-1])
    scores = F.softmax(scores.float(), dim=-1).type_as(q)
    return torch.matmul(scores, vt).transpose(1, 2).contiguous()


class OracleLayerCache:
    """One layer's K and V plane stores plus the decode arithmetic, all in numpy."""

    def __init__(self, bsz: int, max_seq_len: int, heads: int, head_dim: int, top_max_k: int = TOP_MAX_K):
        self.B, self.L, self.H, self.D = bsz, max_seq_len, heads, head_dim
        self.nmb = -(-max_seq_len // COLUMN_BLOCK)
        B, H, D, nmb = bsz, heads, head_dim, self.nmb
        self.k_first_8 = np.zeros((B, H, nmb, D, COLUMN_BLOCK), np.uint8)
        self.k_mid_4 = np.zeros((B, H, nmb, D, COLUMN_BLOCK // 2), np.uint8)
        self.k_last_4 = np.zeros((B, H, nmb, D, COLUMN_BLOCK // 2), np.uint8)
        self.v_first_8 = np.zeros((B, H, max_seq_len, D), np.uint8)
        self.v_mid_4 = np.zeros((B, H, max_seq_len, D // 2), np.uint8)
        self.v_last_4 = np.zeros((B, H, max_seq_len, D // 2), np.uint8)
        self.k_exp_max = np.zeros((B, 1, H, D), np.uint8)
        self.v_exp_max = np.zeros((B, 1, H, D), np.uint8)
        self.restk = np.zeros((B, COLUMN_BLOCK, H, D), np.float16)
        self.restv = np.zeros((B, COLUMN_BLOCK, H, D), np.float16)
        self.rest_len = 0
        self.rest_start = 0
        self.cache_len = 0
        self.top_max_k = top_max_k
        self.last = {}   # decision codes and intermediates of the latest decode step

    # ------------------------------------------------------------------ save
    def save(self, k16: np.ndarray, v16: np.ndarray, start_pos: int, seqlen: int) -> None:
        B, H, D = self.B, self.H, self.D
        assert k16.shape == (B, seqlen, H, D) and v16.shape == (B, seqlen, H, D)
        assert start_pos == self.cache_len and (start_pos == 0 or seqlen == 1)
        assert start_pos + seqlen <= self.L
        self.cache_len += seqlen
        if start_pos == 0:
            # exponent of the signed maximum over the prompt (k_cache_file.py:77-78, v_cache_file.py:80-81)
            self.k_exp_max = exponent_field(k16.max(axis=1, keepdims=True))
            self.v_exp_max = exponent_field(v16.max(axis=1, keepdims=True))
            full = seqlen - seqlen % COLUMN_BLOCK
            orc.k_cache_save(self.k_first_8, self.k_mid_4, self.k_last_4, k16.view(np.uint8), B, H,
                             seqlen // COLUMN_BLOCK, self.nmb, D, COLUMN_BLOCK, 0, seqlen)
            orc.v_cache_save(self.v_first_8, self.v_mid_4, self.v_last_4, v16.view(np.uint8), B, H, self.L, D, 0,
                             full)
            self.restk[:] = 0
            self.restv[:] = 0
            self.rest_len = seqlen % COLUMN_BLOCK
            self.restk[:, :self.rest_len] = k16[:, full:]
            self.restv[:, :self.rest_len] = v16[:, full:]
            self.rest_start = full
        else:
            self.k_exp_max = np.maximum(self.k_exp_max, exponent_field(k16))
            self.v_exp_max = np.maximum(self.v_exp_max, exponent_field(v16))
            self.restk[:, self.rest_len:self.rest_len + 1] = k16
            self.restv[:, self.rest_len:self.rest_len + 1] = v16
            self.rest_len += 1
            if self.rest_len == COLUMN_BLOCK:
                orc.k_cache_save(self.k_first_8, self.k_mid_4, self.k_last_4, self.restk.view(np.uint8), B, H, 1,
                                 self.nmb, D, COLUMN_BLOCK, self.rest_start, COLUMN_BLOCK)
                orc.v_cache_save(self.v_first_8, self.v_mid_4, self.v_last_4, self.restv.view(np.uint8), B, H,
                                 self.L, D, self.rest_start, COLUMN_BLOCK)
                self.rest_len = 0
                self.rest_start += COLUMN_BLOCK
                self.restk[:] = 0
                self.restv[:] = 0

    # ------------------------------------------------------------------ decode pieces
    def scores(self, q16: np.ndarray, reference: bool = False) -> np.ndarray:
        """k_cache_file.py:132-159 -> fp16 [B,H,1,(nb+1)*64] with -inf past the cached tokens."""
        B, H, D = self.B, self.H, self.D
        nb = self.rest_start // COLUMN_BLOCK
        kq = (exponent_field(q16) + self.k_exp_max).astype(np.uint8)
        kqmax = kq.max(axis=3, keepdims=True)
        s_u8, codes = orc.k_cache_compute(self.k_first_8, self.k_mid_4, self.k_last_4, kq, kqmax, q16.view(np.uint8),
                                          B, H, nb, self.nmb, D, COLUMN_BLOCK, self.rest_start,
                                          1.0 / math.sqrt(D), reference)
        s = s_u8.view(np.float16).copy()
        qf = q16.astype(np.float32).transpose(0, 2, 1, 3)                       # B,H,1,D
        kr = self.restk[:, :self.rest_len].astype(np.float32).transpose(0, 2, 3, 1)  # B,H,D,r
        rest = np.matmul(qf, kr).astype(np.float16)                              # fp16 matmul result
        rest = (rest.astype(np.float32) / np.float32(math.sqrt(D))).astype(np.float16)
        s[..., self.rest_start:self.rest_start + self.rest_len] = rest
        s[..., self.cache_len:] = -np.inf
        self.last.update(k_codes=codes, kq=kq, kqmax=kqmax)
        return s

    def probe_exponent(self, p16: np.ndarray) -> np.ndarray:
        """v_cache_file.py:119-143 on the score tensor handed to it."""
        B, H, D, K = self.B, self.H, self.D, self.top_max_k
        length = p16.shape[-1]
        if self.cache_len == length:
            groups = -(-length // K)
            p16 = np.concatenate([p16, np.zeros((B, H, 1, groups * K - length), np.float16)], -1)
        else:
            groups = length // K
        g = np.ascontiguousarray(p16[..., :groups * K]).reshape(B, H, groups, K)
        val = g.max(axis=2, keepdims=True)
        idx = g.argmax(axis=2).astype(np.int32)[:, :, None, :]          # first maximal index, like torch.max
        rows = idx.astype(np.int64) * K + np.arange(K)
        if rows.max() >= self.L:            # the reference would read out of bounds here (v_cache_file.py:151)
            raise ValueError("probe row outside the cache")
        o = orc.v_cache_test_compute(self.v_first_8, self.v_mid_4, self.v_last_4, val.view(np.uint8),
                                     idx.view(np.uint8), B, H, self.L, D, K)
        self.last.update(probe_val=val, probe_idx=idx, probe_o=o.view(np.float16))
        return exponent_field(o.view(np.float16)) & 0x1E

    def output(self, p16: np.ndarray, reference: bool = False) -> np.ndarray:
        """v_cache_file.py:145-190 -> fp16 [B,H,1,D]."""
        B, H, D = self.B, self.H, self.D
        qn = self.rest_start
        stride = p16.shape[-1]
        if qn:
            test_o_exp = self.probe_exponent(np.ascontiguousarray(p16[..., :qn]))
            # [B,H,1,D] + 15 - [B,1,H,D] -> [B,H,H,D] in uint8 arithmetic; min over D; read flat at b*H+h
            align = (test_o_exp.astype(np.uint8) + np.uint8(15) - self.v_exp_max.astype(np.uint8)).astype(np.uint8)
            amin = align.min(axis=-1, keepdims=True)
        else:
            amin = np.zeros((B, H, H, 1), np.uint8)      # nothing quantized: the aligned kernel runs 0 tokens
        o_u8, codes = orc.v_cache_compute(self.v_first_8, self.v_mid_4, self.v_last_4, p16.view(np.uint8), amin, B, H,
                                          self.L, D, stride, qn, reference)
        o = o_u8.view(np.float16).copy()
        pr = p16[..., qn:self.cache_len].astype(np.float32)                         # B,H,1,r
        vr = self.restv[:, :self.rest_len].astype(np.float32).transpose(0, 2, 1, 3)  # B,H,r,D
        o = (o.astype(np.float32) + np.matmul(pr, vr).astype(np.float16).astype(np.float32)).astype(np.float16)
        self.last.update(v_codes=codes, amin=amin)
        return o

    def decode(self, q16, k16, v16, reference: bool = False, mask16=None) -> np.ndarray:
        """One decode step (model/KVCache_AlignedKV.py:116-124) -> fp16 [B,1,H,D].  mask16 (optional): additive fp16
        mask broadcastable to [B,H,1,cache length after the step], added to the fp16 scores in fp16 before the
        softmax (model/KVCache_AlignedKV.py:119-120)."""
        start = self.cache_len
        self.save(k16, v16, start, 1)
        s = self.scores(q16, reference)
        if mask16 is not None:
            n = start + 1
            s = s.copy()
            s[..., :n] = (s[..., :n] + np.broadcast_to(np.asarray(mask16, np.float16)[..., :n], s[..., :n].shape)
                          ).astype(np.float16)      # one fp16 addition, as the in-place += on fp16 tensors
        p = softmax_fp32_to_half(s)
        self.last.update(s=s, p=p)
        return self.output(p, reference).reshape(self.B, 1, self.H, self.D)

    def bytes_read(self) -> dict:
        """Plane bytes the latest decode step had to read under its decisions, and the dense fp16 equivalent."""
        B, H, D = self.B, self.H, self.D
        qn = self.rest_start
        kc, vc = self.last["k_codes"], self.last["v_codes"]
        k_bytes = qn * ((kc >= 0).sum() + 0.5 * (kc < 2).sum() + 0.5 * (kc < 1).sum())
        v_bytes = D * ((vc >= 0).sum() + 0.5 * (vc < 2).sum() + 0.5 * (vc < 1).sum())
        rest = 4 * (self.cache_len - qn) * D * B * H
        return {"k": float(k_bytes), "v": float(v_bytes), "rest": float(rest),
                "dense": float(4 * B * H * self.cache_len * D)}

    # ------------------------------------------------------------------ variants used by the extended entry points
    def dequantized_v(self) -> np.ndarray:
        """fp16 values [B,H,qn,D] the latest decode step's P.V saw: planes reassembled under its read codes with
        the reference's substitute constants (V_cache.cu:198-202,250-253)."""
        qn = self.rest_start
        codes = np.asarray(self.last["v_codes"]).reshape(self.B, self.H, -1)[..., :qn]          # B,H,qn
        f = self.v_first_8[:, :, :qn].astype(np.uint16)                                          # B,H,qn,D
        mid = self.v_mid_4[:, :, :qn].astype(np.uint16)
        low = self.v_last_4[:, :, :qn].astype(np.uint16)
        c = codes[..., None]
        mid = np.where(c < 2, mid, 0x88)
        low = np.where(c == 0, low, np.where(c == 1, 0x88, 0x00))
        lo_e = (mid & 0xF0) | (low >> 4)
        lo_o = ((mid << 4) & 0xF0) | (low & 0x0F)
        bits = np.empty(f.shape, np.uint16)
        bits[..., 0::2] = (f[..., 0::2] << 8) | lo_e
        bits[..., 1::2] = (f[..., 1::2] << 8) | lo_o
        return bits.view(np.float16)

    def decode_record(self, q16, k16=None, v16=None, *, append: bool = True, reference: bool = False,
                      order_free: bool = False):
        """One decode step returning (out fp16 [B,1,H,D], record fp32 [B*H, D+2] = (max score, sum of exponentials,
        output)).  append=False leaves the cache untouched.  order_free: P.V as an exact sum (float64) of
        probability x dequantized value under the same read decisions, rounded once - the arithmetic the order-free
        kernel approximates in fp32."""
        if append:
            self.save(k16, v16, self.cache_len, 1)
        s = self.scores(q16, reference)
        p = softmax_fp32_to_half(s)
        self.last.update(s=s, p=p)
        x = s.astype(np.float32)[..., :self.cache_len]
        m = x.max(axis=-1)
        l = np.exp(x - m[..., None], dtype=np.float32).sum(axis=-1, dtype=np.float32)
        o16 = self.output(p, reference)                                   # B,H,1,D (also fills last["v_codes"])
        if order_free:
            qn = self.rest_start
            o = np.zeros((self.B, self.H, self.D), np.float64)
            if qn:
                vq = self.dequantized_v().astype(np.float64)              # B,H,qn,D
                o += np.einsum("bht,bhtd->bhd", p[:, :, 0, :qn].astype(np.float64), vq)
            pr = p[:, :, 0, qn:self.cache_len].astype(np.float64)
            vr = self.restv[:, :self.rest_len].astype(np.float64).transpose(0, 2, 1, 3)
            o += np.einsum("bhr,bhrd->bhd", pr, vr)
            o32 = o.astype(np.float32)
            o16 = o32.astype(np.float16)[:, :, None, :]
        else:
            o32 = o16[:, :, 0, :].astype(np.float32)
        rec = np.concatenate([m.reshape(-1, 1), l.reshape(-1, 1), o32.reshape(-1, self.D)], axis=1).astype(np.float32)
        return o16.reshape(self.B, 1, self.H, self.D), rec


class OracleGQACache:
    """Grouped-query attention through the multi-head oracle: the reference asserts MHA
    (model/KVCache_AlignedKV.py:32), so the specification of a G-way group is the reference run on a cache whose
    KV heads are repeated G times (HF's repeat_kv).  KV head h is expanded head h*G."""

    def __init__(self, bsz: int, max_seq_len: int, kv_heads: int, group: int, head_dim: int):
        self.G = group
        self.inner = OracleLayerCache(bsz, max_seq_len, kv_heads * group, head_dim)

    def _expand(self, x16):
        return np.ascontiguousarray(np.repeat(x16, self.G, axis=2))

    def save(self, k16, v16, start_pos, seqlen):
        self.inner.save(self._expand(k16), self._expand(v16), start_pos, seqlen)

    def decode_record(self, q16, k16=None, v16=None, **kw):
        if k16 is not None:
            k16, v16 = self._expand(k16), self._expand(v16)
        return self.inner.decode_record(q16, k16, v16, **kw)

    def kv_planes(self):
        """The six planes restricted to the real KV heads (every G-th expanded head)."""
        i = self.inner
        return tuple(x[:, ::self.G] for x in (i.k_first_8, i.k_mid_4, i.k_last_4, i.v_first_8, i.v_mid_4, i.v_last_4))


def lse_merge_np(packed: np.ndarray) -> np.ndarray:
    """Merge per-shard records [R, rows, D+2] = (m, l, o) -> fp16 [rows, D]:
    out = sum_g w_g o_g, w_g = l_g exp(m_g - M) / sum_g' l_g' exp(m_g' - M).  Shards with l = 0 are ignored."""
    packed = np.asarray(packed, np.float64)
    m, l, o = packed[..., 0], packed[..., 1], packed[..., 2:]
    m = np.where(l > 0, m, -np.inf)
    M = m.max(axis=0, keepdims=True)
    w = np.where(l > 0, l * np.exp(m - M), 0.0)
    den = w.sum(axis=0, keepdims=True)
    w = np.where(den > 0, w / np.where(den > 0, den, 1.0), 0.0)
    return np.where(w[..., None] > 0, w[..., None] * o, 0.0).sum(axis=0).astype(np.float32).astype(np.float16)
