"""Plain, slow, whole-sequence Qwen2 decoder used as the oracle of the test suite.

Written from the formulas of the reference project's own model file
(engine/model.py, engine/attention.py); every function cites the lines it
restates. It takes a whole token sequence, keeps no cache, has one function for
each part and shares no code with the engine package: it reads config.json and
model.safetensors by itself.

Everything runs in the dtype given (float32 by default, float64 for a tighter
oracle, bfloat16 to see what the reference's rounding points cost), on the CPU
or on any torch device.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path

import torch


# --------------------------------------------------------------------------- #
# configuration and weights (a reader of its own)
# --------------------------------------------------------------------------- #

@dataclass(frozen=True)
class PlainConfig:
    """The sizes the formulas need (engine/model.py:43-80 reads the same keys)."""

    num_layers: int
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    # Window of each layer: 0 means every earlier key.
    layer_windows: tuple[int, ...]

    @property
    def groups(self) -> int:
        return self.num_heads // self.num_kv_heads


def read_config(folder: str | Path) -> PlainConfig:
    """Reads config.json. head_dim falls back to hidden // heads (engine/model.py:67-69)."""
    raw = json.loads((Path(folder) / "config.json").read_text())
    heads = int(raw["num_attention_heads"])
    hidden = int(raw["hidden_size"])
    head_dim = int(raw.get("head_dim") or hidden // heads)
    if "rope_theta" in raw:
        theta = float(raw["rope_theta"])
    else:
        theta = float(raw["rope_parameters"]["rope_theta"])  # engine/model.py:79
    layers = int(raw["num_hidden_layers"])
    windows = [0] * layers
    if raw.get("use_sliding_window", False):
        first_windowed = int(raw.get("max_window_layers", layers))
        for i in range(first_windowed, layers):
            windows[i] = int(raw["sliding_window"])
    return PlainConfig(
        num_layers=layers,
        hidden_size=hidden,
        num_heads=heads,
        num_kv_heads=int(raw["num_key_value_heads"]),
        head_dim=head_dim,
        intermediate_size=int(raw["intermediate_size"]),
        vocab_size=int(raw["vocab_size"]),
        rms_norm_eps=float(raw["rms_norm_eps"]),
        rope_theta=theta,
        tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
        layer_windows=tuple(windows),
    )


def read_weights(folder: str | Path) -> dict[str, torch.Tensor]:
    """All tensors of model.safetensors by name (names as in engine/model.py:200-227)."""
    from safetensors import safe_open

    out: dict[str, torch.Tensor] = {}
    with safe_open(str(Path(folder) / "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            out[name] = f.get_tensor(name)
    return out


# --------------------------------------------------------------------------- #
# one function for each part
# --------------------------------------------------------------------------- #

def embed(token_ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather, no scaling (engine/model.py:401)."""
    return table[token_ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Variance in float32 (or wider), cast back, then the weight (engine/model.py:117-123)."""
    dtype = x.dtype
    wide = x.to(torch.float64 if dtype == torch.float64 else torch.float32)
    variance = wide.pow(2).mean(-1, keepdim=True)
    wide = wide * torch.rsqrt(variance + eps)
    return weight * wide.to(dtype)


def rotary_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """1 / theta^(2i/d) in float32 from an integer range (engine/model.py:132-135)."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.int64).to(torch.float32)
    return 1.0 / (theta ** (exponent / head_dim))


def rotary_tables(inv_freq: torch.Tensor, positions: torch.Tensor, dtype: torch.dtype):
    """cos and sin of position x inv_freq, both halves alike (engine/model.py:138-152).

    The angle is a float32 product, as in the reference; for a float64 run the
    tables are widened after the float32 angle so that only the angle's own
    rounding is shared with the engine.
    """
    angle = positions.to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)
    both = torch.cat((angle, angle), dim=-1)
    if dtype == torch.float64:
        both = both.to(torch.float64)
    return both.cos().to(dtype), both.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """(-second half, first half) (engine/model.py:126-129)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin for x of [tokens, heads, head_dim] (engine/model.py:155-161)."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0
) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.

    q is [tokens, heads, d]; k and v are [tokens, kv_heads, d]. Query head h reads
    kv head h // (heads / kv_heads) (engine/attention.py:46-74). The query at
    position p sees keys j <= p (engine/attention.py:581-586), and with a window
    w > 0 only those with p - j < w. Scores are scaled by head_dim**-0.5
    (engine/model.py:60-62); softmax over the keys; dropout none.
    """
    tokens, heads, _ = q.shape
    groups = heads // k.shape[1]
    k_full = k.repeat_interleave(groups, dim=1)
    v_full = v.repeat_interleave(groups, dim=1)
    wide = torch.float64 if q.dtype == torch.float64 else torch.float32
    scores = torch.einsum("qhd,khd->hqk", q.to(wide), k_full.to(wide)) * scale
    pos = torch.arange(tokens, device=q.device)
    allowed = pos[None, :] <= pos[:, None]
    if window > 0:
        allowed = allowed & (pos[:, None] - pos[None, :] < window)
    scores = scores.masked_fill(~allowed[None, :, :], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("hqk,khd->qhd", probs, v_full.to(wide))
    return out.to(q.dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """x . W^T (+ b) with W stored [out, in] (engine/model.py:303-305)."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def swiglu(x: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), no biases (engine/model.py:317-320)."""
    gate = linear(x, gate_w)
    up = linear(x, up_w)
    return linear(torch.nn.functional.silu(gate) * up, down_w)


def attention_layer(
    x: torch.Tensor,
    w: dict[str, torch.Tensor],
    prefix: str,
    cfg: PlainConfig,
    cos: torch.Tensor,
    sin: torch.Tensor,
    window: int,
) -> torch.Tensor:
    """Projections with bias, rotary on q and k, attention, output projection
    (engine/model.py:284-315)."""
    tokens = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"], w[prefix + "q_proj.bias"])
    k = linear(x, w[prefix + "k_proj.weight"], w[prefix + "k_proj.bias"])
    v = linear(x, w[prefix + "v_proj.weight"], w[prefix + "v_proj.bias"])
    q = q.view(tokens, cfg.num_heads, cfg.head_dim)
    k = k.view(tokens, cfg.num_kv_heads, cfg.head_dim)
    v = v.view(tokens, cfg.num_kv_heads, cfg.head_dim)
    q = apply_rotary(q, cos, sin)
    k = apply_rotary(k, cos, sin)
    out = attention(q, k, v, cfg.head_dim ** -0.5, window)
    return linear(out.reshape(tokens, cfg.num_heads * cfg.head_dim), w[prefix + "o_proj.weight"])


def forward_hidden(
    token_ids: torch.Tensor, weights: dict[str, torch.Tensor], cfg: PlainConfig, dtype=torch.float32
) -> torch.Tensor:
    """The residual stream after the final norm for every position (engine/model.py:322-351)."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    x = embed(token_ids, w["model.embed_tokens.weight"])
    positions = torch.arange(token_ids.shape[0], device=token_ids.device)
    cos, sin = rotary_tables(
        rotary_inv_freq(cfg.head_dim, cfg.rope_theta).to(token_ids.device), positions, dtype
    )
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        normed = rms_norm(x, w[p + "input_layernorm.weight"], cfg.rms_norm_eps)
        x = x + attention_layer(normed, w, p + "self_attn.", cfg, cos, sin, cfg.layer_windows[i])
        normed = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        x = x + swiglu(
            normed,
            w[p + "mlp.gate_proj.weight"],
            w[p + "mlp.up_proj.weight"],
            w[p + "mlp.down_proj.weight"],
        )
    return rms_norm(x, w["model.norm.weight"], cfg.rms_norm_eps)


def lm_head_weight(weights: dict[str, torch.Tensor]) -> torch.Tensor:
    """The head is the embedding table when the file has no head (engine/model.py:220-222)."""
    return weights.get("lm_head.weight", weights["model.embed_tokens.weight"])


def forward_logits(
    token_ids, weights: dict[str, torch.Tensor], cfg: PlainConfig, dtype=torch.float32
) -> torch.Tensor:
    """Logits at EVERY position of one whole sequence, [tokens, vocab], as float32.

    The reference emits only the last position (engine/model.py:406); the row for
    position p here is what it would emit for the prefix ending at p.
    """
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    hidden = forward_hidden(ids, weights, cfg, dtype)
    logits = linear(hidden, lm_head_weight(weights).to(dtype))
    return logits.to(torch.float32)


def generate_greedy(prompt, new_tokens: int, weights, cfg: PlainConfig, dtype=torch.float32):
    """Greedy decoding without a cache: argmax of the last row, exactly `new_tokens`
    of them, end-of-sequence ignored (engine/model.py:459-503)."""
    ids = list(prompt)
    rows = []
    for _ in range(new_tokens):
        logits = forward_logits(ids, weights, cfg, dtype)[-1]
        rows.append(logits)
        ids.append(int(torch.argmax(logits)))
    return ids[len(prompt):], torch.stack(rows)


# --------------------------------------------------------------------------- #
# sampling restated (the reference samples greedily only: engine/scheduler.py:610;
# temperature sampling rests on the formula below, not on reference code)
# --------------------------------------------------------------------------- #

_M32 = 0xFFFFFFFF


def _mix32(x: int) -> int:
    x &= _M32
    x ^= x >> 16
    x = (x * 0x85EBCA6B) & _M32
    x ^= x >> 13
    x = (x * 0xC2B2AE35) & _M32
    x ^= x >> 16
    return x


def gumbel_uniform(seed: int, request_key: int, output_index: int, vocab_index: int) -> float:
    """The uniform number in (0, 1) that belongs to one (request, output, vocabulary entry)."""
    h = _mix32((seed & _M32) ^ 0x9E3779B9)
    h = _mix32(h ^ ((seed >> 32) & _M32))
    h = _mix32(h + (request_key & _M32) * 0x7FEB352D)
    h = _mix32(h + (output_index & _M32) * 0x846CA68B)
    h = _mix32(h + (vocab_index & _M32) * 0x9E3779B1)
    return ((h >> 9) + 0.5) * (1.0 / 8388608.0)


def sample_scores(logits: torch.Tensor, temperature: float, seed: int, request_key: int, output_index: int):
    """logits / T + Gumbel noise; the sampled token is the argmax of the result."""
    vocab = logits.shape[0]
    noise = torch.tensor(
        [-math.log(-math.log(gumbel_uniform(seed, request_key, output_index, j))) for j in range(vocab)],
        dtype=torch.float64,
    )
    return logits.to(torch.float64) / temperature + noise


def sample(logits: torch.Tensor, temperature: float, seed: int = 0, request_key: int = 0, output_index: int = 0) -> int:
    """Greedy for T == 0 (lowest index wins a tie), else Gumbel-max at temperature T."""
    if temperature == 0.0:
        return int(torch.argmax(logits))
    return int(torch.argmax(sample_scores(logits, temperature, seed, request_key, output_index)))
