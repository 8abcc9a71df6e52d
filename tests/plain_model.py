"""Plain, slow implementation of the Qwen3 dense decoder: the oracle of the test-suite.

Whole sequences, no cache, no batching, one function for each part, torch on the CPU.
It shares no code with ``dinfer_b200``: weights arrive as a plain ``{name: tensor}``
dictionary and the configuration as the raw ``config.json`` dictionary.

The reference engine (rayze-ai/dinfer) can be neither compiled nor run on a machine
without a Rust toolchain and a GPU, so the whole-model path rests on its formulas;
each function cites the file and line of the reference it restates.  The per-part
functions are compared once with the reference's own torch-CPU formulas
(``scripts/verify/ops_parity_ref.py``), see ``tests/golden/make_golden.py``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """``x0[t, :] = E[ids[t], :]``  (models/qwen3/src/model.rs:699,
    crates/kernels/cuda/activation.cu:121-129)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w`` over the last axis
    (crates/kernels/cuda/norm.cu:54-115, scripts/verify/ops_parity_ref.py:59-61)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def rope_cos_sin(positions: torch.Tensor, rotary_dim: int, theta: float):
    """Angles ``p * theta^(-2i/rotary_dim)`` for ``i < rotary_dim/2``, computed in 64-bit
    (crates/layers/src/nn.rs:157-173)."""
    half = rotary_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    inv_freq = 1.0 / (float(theta) ** (2.0 * i / rotary_dim))
    ang = positions.to(torch.float64)[:, None] * inv_freq[None, :]
    return ang.cos(), ang.sin()


def rope_neox(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotation of the pairs ``(i, i + D/2)`` of every head: ``x[..., T, heads, D]`` with
    ``cos``/``sin`` of shape ``[T, D/2]``  (crates/kernels/cuda/qkv_post.cu:65-76,
    scripts/verify/ops_parity_ref.py:123-128)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                         window: Optional[int] = None) -> torch.Tensor:
    """Causal softmax attention, query head ``h`` reading key/value head ``h // group``.

    ``q [T, H, D]``, ``k``/``v`` ``[T, Hkv, D]`` -> ``[T, H, D]``.  Row ``i`` sees keys
    ``[0, i]`` (crates/kernels/cuda/gqa.cu:183-189,300-348; scripts/verify/ops_parity_ref.py:208-222);
    with ``window`` it sees the last ``window`` of them, itself included.
    """
    T, H, D = q.shape
    Hkv = k.shape[1]
    group = H // Hkv
    out = torch.empty_like(q)
    pos = torch.arange(T)
    hidden = pos[None, :] > pos[:, None]
    if window is not None:
        hidden = hidden | (pos[None, :] <= pos[:, None] - window)
    for h in range(H):
        kh, vh = k[:, h // group], v[:, h // group]
        s = (q[:, h] @ kh.T) * scale
        s = s.masked_fill(hidden, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ vh
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """``x / (1 + exp(-x))`` (crates/kernels/cuda/common.cuh:55)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(x, w_gate, w_up, w_down):
    """``(silu(x Wg^T) * (x Wu^T)) Wd^T`` (crates/layers/src/nn.rs:373-381,
    crates/kernels/cuda/activation.cu:80-99)."""
    return gate(torch.cat([x @ w_gate.T, x @ w_up.T], dim=-1)) @ w_down.T


def attention_block(x, W: Dict[str, torch.Tensor], prefix: str, cfg: dict, positions,
                    window: Optional[int] = None):
    """q/k/v projections, per-head RMSNorm of q and k, neox RoPE over the whole head,
    causal attention at scale ``D^-0.5``, output projection
    (models/qwen3/src/model.rs:141-172,212-313)."""
    T = x.shape[0]
    H, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    qkv = torch.cat([x @ W[prefix + "q_proj.weight"].T, x @ W[prefix + "k_proj.weight"].T,
                     x @ W[prefix + "v_proj.weight"].T], dim=1)
    rows, _ = qk_post(qkv, positions, H, Hkv, D, W[prefix + "q_norm.weight"], W[prefix + "k_norm.weight"], eps,
                      cfg["rope_theta"])
    q = rows[:, :H * D].reshape(T, H, D)
    k = rows[:, H * D:(H + Hkv) * D].reshape(T, Hkv, D)
    v = rows[:, (H + Hkv) * D:].reshape(T, Hkv, D)
    o = causal_gqa_attention(q, k, v, 1.0 / math.sqrt(D), window)
    return o.reshape(T, H * D) @ W[prefix + "o_proj.weight"].T


def decoder_layer(x, W, l: int, cfg: dict, positions, window: Optional[int] = None):
    """Pre-norm residual block: ``x += attn(norm1(x)); x += mlp(norm2(x))``
    (models/qwen3/src/model.rs:709-813)."""
    p = f"model.layers.{l}."
    eps = cfg["rms_norm_eps"]
    h = rms_norm(x, W[p + "input_layernorm.weight"], eps)
    x, h = add_and_norm(x, attention_block(h, W, p + "self_attn.", cfg, positions, window),
                        W[p + "post_attention_layernorm.weight"], eps)
    x = x + swiglu_mlp(h, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                       W[p + "mlp.down_proj.weight"])
    return x


def qwen3_logits(W: Dict[str, torch.Tensor], cfg: dict, ids: List[int],
                 dtype: torch.dtype = torch.float64,
                 schedule: Optional[List[int]] = None,
                 window: Optional[int] = None) -> torch.Tensor:
    """Logits ``[T, V]`` of every position of one whole sequence.

    ``lm_head.weight`` when the file has it, else the embedding table if the configuration
    ties them (models/qwen3/src/model.rs:487-496); final norm before the head
    (models/qwen3/src/model.rs:821-853).  ``schedule`` lists the layers in the order they run
    (default: each once, in order).
    """
    raw = W
    W = _Converted(raw, dtype)                    # each tensor is widened when it is used (a large table never whole)
    ids_t = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(len(ids))
    x = embedding(ids_t, raw["model.embed_tokens.weight"]).to(dtype)
    order = list(range(cfg["num_hidden_layers"])) if schedule is None else schedule
    for l in order:
        x = decoder_layer(x, W, l, cfg, positions, window)
    x = rms_norm(x, W["model.norm.weight"], cfg["rms_norm_eps"])
    if "lm_head.weight" in raw:
        head = raw["lm_head.weight"]
    else:
        assert cfg.get("tie_word_embeddings", False), "no lm_head.weight and embeddings not tied"
        head = raw["model.embed_tokens.weight"]
    return lm_head(x, head)


def lm_head(x: torch.Tensor, head: torch.Tensor, rows: int = 32768) -> torch.Tensor:
    """``logits = x head^T`` (models/qwen3/src/model.rs:852-853), the table widened a slice of rows at a time."""
    return torch.cat([x @ head[i:i + rows].to(x.dtype).T for i in range(0, head.shape[0], rows)], dim=1)


class _Converted:
    """``{name: tensor}`` whose tensors come out in ``dtype``."""

    def __init__(self, raw: Dict[str, torch.Tensor], dtype: torch.dtype):
        self.raw, self.dtype = raw, dtype

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.raw[name].to(self.dtype)

    def __contains__(self, name: str) -> bool:
        return name in self.raw


def greedy_generate(W, cfg, prompt: List[int], n: int, dtype=torch.float64) -> List[int]:
    """``n`` tokens by argmax (ties to the lowest index: crates/kernels/cuda/sampling.cu:13-56),
    each from a whole forward pass over the sequence so far."""
    seq = list(prompt)
    out = []
    for _ in range(n):
        logits = qwen3_logits(W, cfg, seq, dtype)[-1]
        tok = int(torch.argmax(logits))
        out.append(tok)
        seq.append(tok)
    return out


# ---- sampling, restated from crates/kernels/cuda/sampling.cu ----

def philox_uniform(seed: int, offset: int) -> float:
    """One Philox4x32-10 call: counter ``(offset_lo, offset_hi, 0, 0)``, key ``(seed_lo, seed_hi)``,
    ``u = (c0 >> 8) / 2^24`` (crates/kernels/cuda/sampling.cu:143-157)."""
    M = 0xFFFFFFFF
    c = [offset & M, (offset >> 32) & M, 0, 0]
    k = [seed & M, (seed >> 32) & M]
    for _ in range(10):
        p0 = 0xD2511F53 * c[0]
        p1 = 0xCD9E8D57 * c[2]
        hi0, lo0 = p0 >> 32, p0 & M
        hi1, lo1 = p1 >> 32, p1 & M
        c = [(hi1 ^ c[1] ^ k[0]) & M, lo1, (hi0 ^ c[3] ^ k[1]) & M, lo0]
        k = [(k[0] + 0x9E3779B9) & M, (k[1] + 0xBB67AE85) & M]
    return (c[0] >> 8) / 16777216.0


def add_and_norm(x: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float):
    """The fused residual add and norm: ``x <- x + delta``, then ``rms_norm(x)``; returns both
    (crates/kernels/cuda/norm.cu:60-95; scripts/verify/ops_parity_ref.py:70-76, where the sum is rounded to
    the storage type before it is normed)."""
    x = x + delta
    return x, rms_norm(x, weight, eps)


def qk_post(qkv: torch.Tensor, positions: torch.Tensor, H: int, Hkv: int, D: int, wq, wk, eps: float, theta: float):
    """What happens to a step's q/k/v rows between the projection and attention: per-head RMSNorm of q and k,
    THEN the rotation, v untouched; returns the rows ``[T, (H + 2 Hkv) D]`` and what goes into the cache per token,
    ``[T, Hkv, 2 (k, v), D]`` (crates/kernels/cuda/qkv_post.cu:54-90; scripts/verify/ops_parity_ref.py:131-152)."""
    T = qkv.shape[0]
    q = qkv[:, :H * D].reshape(T, H, D)
    k = qkv[:, H * D:(H + Hkv) * D].reshape(T, Hkv, D)
    v = qkv[:, (H + Hkv) * D:].reshape(T, Hkv, D)
    cos, sin = rope_cos_sin(positions, D, theta)
    qn = rope_neox(rms_norm(q, wq, eps), cos, sin)
    kn = rope_neox(rms_norm(k, wk, eps), cos, sin)
    rows = torch.cat([qn.reshape(T, -1), kn.reshape(T, -1), v.reshape(T, -1)], dim=1)
    return rows, torch.stack([kn, v], dim=2)


def gate(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(first half) * second half`` of the fused gate/up product's rows: the gate comes first
    (crates/kernels/cuda/activation.cu:80-99; scripts/verify/ops_parity_ref.py:84-89)."""
    i = gate_up.shape[-1] // 2
    return silu(gate_up[..., :i]) * gate_up[..., i:]


def penalties(logits: torch.Tensor, prompt: List[int], output: List[int], repetition: float = 1.0,
              frequency: float = 0.0, presence: float = 0.0) -> torch.Tensor:
    """Every token of the prompt or the output, once: a positive logit is divided by the repetition penalty, any
    other multiplied; tokens of the OUTPUT lose ``frequency * count + presence``
    (crates/kernels/cuda/sampling.cu:322-349; scripts/verify/ops_parity_ref.py:285-299)."""
    out = logits.clone()
    for tok in set(prompt) | set(output):
        x = float(out[tok])
        if repetition != 1.0:
            x = x / repetition if x > 0 else x * repetition
        cnt = output.count(tok)
        if cnt > 0:
            x -= frequency * cnt + presence
        out[tok] = x
    return out


def filter_logits(x: torch.Tensor, top_k: int = -1, top_p: float = 1.0, min_p: float = 0.0) -> torch.Tensor:
    """min_p -> top-k -> top-p on the scaled logits: what is filtered out becomes -inf
    (crates/kernels/cuda/sampling.cu:196-256,353-367; scripts/verify/ops_parity_ref.py:301-312,347-352)."""
    neg = torch.full_like(x, float("-inf"))
    if min_p > 0.0:
        probs = torch.softmax(x, dim=-1)
        x = torch.where(probs >= min_p * probs.max(), x, neg)
    if 0 < top_k < x.numel():
        kth = torch.topk(x, top_k).values[-1]
        x = torch.where(x >= kth, x, neg)
    if top_p < 1.0:
        probs = torch.softmax(x, dim=-1)          # over what min_p and top-k left
        sp, si = torch.sort(probs, descending=True)
        before = torch.cumsum(sp, 0) - sp
        keep = torch.zeros_like(x, dtype=torch.bool)
        keep[si[before < top_p]] = True
        x = torch.where(keep, x, neg)
    return x


def sample_token(logits: torch.Tensor, temperature: float, seed: int, offset: int,
                 top_k: int = -1, top_p: float = 1.0, min_p: float = 0.0) -> int:
    """temperature -> min_p -> top-k/top-p -> inverse CDF in vocabulary order
    (crates/kernels/cuda/sampling.cu:196-283; models/qwen3/src/executor.rs:552-605).
    Greedy when ``temperature <= 1e-5`` (crates/core/src/sample.rs:143-145)."""
    x = logits.to(torch.float64)
    if temperature <= 1e-5:
        return int(torch.argmax(x))
    x = filter_logits(x / temperature, top_k, top_p, min_p)
    w = torch.exp(x - x.max())
    target = philox_uniform(seed, offset) * float(w.sum())
    cum = torch.cumsum(w, 0)
    hit = torch.nonzero((cum >= target) & (w > 0))
    return int(hit[0]) if hit.numel() else int(torch.nonzero(w > 0)[-1])
