"""The kernels with a fault put in on purpose, for the negative controls.

`FaultyOps(real, layers, layer, fault)` hands every call through to the real kernels,
except that the attention of ONE layer sees a damaged block table or a shortened context.
A test that compares the engine with the plain model must leave its tolerance under each
of these faults; if it does not, the tolerance is too wide to mean anything. (The
reference does the same to its own tests: a backend that ignores the block table must
diverge, tests/test_parity.py:333-380.)

  swap_pages   the first two pages of the first request change places in the table
  wrong_page   the first request's first page becomes its second page (two entries alike)
  drop_tile    the first request's context is `drop` keys shorter (decode-only steps)
"""

from __future__ import annotations


class FaultyOps:
    def __init__(self, real, layers: int, layer: int, fault: str, drop: int = 16) -> None:
        self.real = real
        self.layers = layers
        self.layer = layer
        self.fault = fault
        self.drop = drop
        self.calls = 0
        self.faults_made = 0

    def __getattr__(self, name):
        return getattr(self.real, name)

    def paged_attention(self, qkv, keys, values, block_table, q_start, q_pos0, kv_len, num_heads, num_kv_heads,
                        head_dim, page_size, max_q_len, max_kv_len, scale, window, num_single=None, multi_index=None):
        layer = self.calls % self.layers
        self.calls += 1
        if layer == self.layer:
            if self.fault == "swap_pages" and block_table.shape[1] >= 2:
                block_table = block_table.clone()
                block_table[0, 0], block_table[0, 1] = block_table[0, 1].clone(), block_table[0, 0].clone()
                self.faults_made += 1
            elif self.fault == "wrong_page" and block_table.shape[1] >= 2:
                block_table = block_table.clone()
                block_table[0, 0] = block_table[0, 1]
                self.faults_made += 1
            elif self.fault == "drop_tile" and max_q_len == 1 and max_kv_len > self.drop + 1:
                kv_len = kv_len.clone()
                kv_len[0] = kv_len[0] - self.drop
                self.faults_made += 1
        return self.real.paged_attention(qkv, keys, values, block_table, q_start, q_pos0, kv_len, num_heads,
                                         num_kv_heads, head_dim, page_size, max_q_len, max_kv_len, scale, window,
                                         num_single=num_single, multi_index=multi_index)


class RecordingOps:
    """Hands every call through to the real kernels and keeps what `paged_attention` reports
    about each of its calls (which kernel ran, how a query tile's keys were shared out), so that
    a test at model level can tell which form of the attention a step took."""

    def __init__(self, real) -> None:
        self.real = real
        self.attention_calls: list[dict] = []

    def __getattr__(self, name):
        return getattr(self.real, name)

    def paged_attention(self, *args, **kwargs):
        info: dict = {}
        out = self.real.paged_attention(*args, **kwargs, info=info)
        self.attention_calls.append(info)
        return out
