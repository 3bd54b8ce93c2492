"""A stand-in for the kernel library, written with plain torch indexing, for tests only.

The engine has no CPU path: its parts call hand-written CUDA kernels through
`kernels.ops`. These functions have the same names and arguments and do the same
work slowly, so that everything ABOVE the kernels (batch flattening, block tables,
slots, the cache manager, the schedule, the scheduler) can be tested without a GPU,
and so that each kernel has a plain reference to be compared with on the GPU.
"""

from __future__ import annotations

import math

import torch


def materialized(x):
    return x


def embedding(ids, table, feedback=None):
    ids = ids.long()
    if feedback is not None:
        last_token, state_slot, seq_index = feedback
        fed = last_token[state_slot[seq_index.long()].long()].long()
        ids = torch.where(ids < 0, fed, ids)
    return table[ids]


def scatter_tokens(last_token, tokens, logit_rows, seq_index, state_slot):
    last_token[state_slot[seq_index[logit_rows.long()].long()].long()] = tokens.to(last_token.dtype)


def rms_norm(x, weight, eps):
    wide = x.float()
    scaled = wide * torch.rsqrt(wide.pow(2).mean(-1, keepdim=True) + eps)
    return (scaled * weight.float()).to(x.dtype)


def linear(x, weight, bias=None, residual=None, out_dtype=None):
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def rotary_table(positions, inv_freq):
    angle = positions.float()[:, None] * inv_freq.float()[None, :]
    return torch.cat((angle.cos(), angle.sin()), dim=-1)


def rotary_qk_cache_write(qkv, table, slots, keys, values, num_heads, num_kv_heads, head_dim, page_size):
    tokens = qkv.shape[0]
    view = qkv.view(tokens, num_heads + 2 * num_kv_heads, head_dim)
    half = head_dim // 2
    if table is not None:
        cos = table[:, None, :half]
        sin = table[:, None, half:]
        rot = view[:, : num_heads + num_kv_heads].float()
        lo, hi = rot[..., :half], rot[..., half:]
        out = torch.cat((lo * cos - hi * sin, hi * cos + lo * sin), dim=-1)
        view[:, : num_heads + num_kv_heads] = out.to(qkv.dtype)
    if slots is not None:
        page = (slots // page_size).long()
        offset = (slots % page_size).long()
        keys[page, :, offset, :] = view[:, num_heads : num_heads + num_kv_heads]
        values[page, :, offset, :] = view[:, num_heads + num_kv_heads :]
    return qkv


def paged_attention(
    qkv, keys, values, block_table, q_start, q_pos0, kv_len,
    num_heads, num_kv_heads, head_dim, page_size, max_q_len, max_kv_len, scale, window, num_single=None, multi_index=None,
):
    tokens = qkv.shape[0]
    q_all = qkv.view(tokens, num_heads + 2 * num_kv_heads, head_dim)[:, :num_heads]
    out = torch.zeros(tokens, num_heads, head_dim, dtype=torch.float32, device=qkv.device)
    groups = num_heads // num_kv_heads
    for b in range(block_table.shape[0]):
        start, end = int(q_start[b]), int(q_start[b + 1])
        n_kv, p0 = int(kv_len[b]), int(q_pos0[b])
        lowest = 0 if window <= 0 else max(0, p0 - window + 1)
        pos = torch.arange(lowest, n_kv, device=qkv.device)
        pages = block_table[b, (pos // page_size).long()].long()
        assert (pages >= 0).all(), "a key that is still visible lies in a released page"
        k = keys[pages, :, (pos % page_size).long(), :].float()      # [kv, kv_heads, d]
        v = values[pages, :, (pos % page_size).long(), :].float()
        q = q_all[start:end].float()                                   # [q, heads, d]
        q_pos = torch.arange(p0, p0 + (end - start), device=qkv.device)
        allowed = pos[None, :] <= q_pos[:, None]
        if window > 0:
            allowed &= (q_pos[:, None] - pos[None, :]) < window
        k = k.repeat_interleave(groups, dim=1)
        v = v.repeat_interleave(groups, dim=1)
        scores = torch.einsum("qhd,khd->hqk", q, k) * scale
        scores = scores.masked_fill(~allowed[None], float("-inf"))
        out[start:end] = torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), v)
    return out.view(tokens, num_heads * head_dim).to(qkv.dtype)


def silu_mul(gate_up):
    half = gate_up.shape[-1] // 2
    gate, up = gate_up[..., :half].float(), gate_up[..., half:].float()
    return (torch.nn.functional.silu(gate) * up).to(gate_up.dtype)


def gather_rows(x, rows):
    return x[rows.long()]


_M32 = 0xFFFFFFFF


def _mix32(x):
    x = x & _M32
    x = x ^ (x >> 16)
    x = (x * 0x85EBCA6B) & _M32
    x = x ^ (x >> 13)
    x = (x * 0xC2B2AE35) & _M32
    x = x ^ (x >> 16)
    return x


def gumbel_scores(row, t, seed_lo, seed_hi, request_key, output_index):
    """float64 [vocab]: logits / t + Gumbel noise of the row's counters, every entry at once."""
    vocab = torch.arange(row.shape[0], dtype=torch.int64)
    h = _mix32((int(seed_lo) & _M32) ^ 0x9E3779B9)
    h = _mix32(h ^ (int(seed_hi) & _M32))
    h = _mix32(h + (int(request_key) & _M32) * 0x7FEB352D)
    h = _mix32(h + (int(output_index) & _M32) * 0x846CA68B)
    hv = _mix32((h + ((vocab * 0x9E3779B1) & _M32)) & _M32)
    u = ((hv >> 9).double() + 0.5) / 8388608.0
    return row.double().cpu() / t - torch.log(-torch.log(u))


def sample(logits, temperature, seed_lo, seed_hi, request_key, output_index, keep=None):
    """Per row: argmax for temperature 0, else Gumbel-max with the engine's counter-based noise."""
    out = torch.empty(logits.shape[0], dtype=torch.int32)
    for r in range(logits.shape[0]):
        t = float(temperature[r])
        row = logits[r].double().cpu()
        if t > 0.0:
            row = gumbel_scores(logits[r], t, seed_lo[r], seed_hi[r], request_key[r], output_index[r])
        out[r] = int(torch.argmax(row))
    if keep is not None:
        scatter_tokens(keep[0], out, keep[1], keep[2], keep[3])
    return out
