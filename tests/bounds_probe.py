"""Run with PAE_BOUNDS=1 (tests/test_bounds_gpu.py does): the engine on the checked build of
its kernels, in which every slot, block-table index and page id is compared with the pool on
the device before it is used.

1. Mixed replays (portions beside decoded tokens, few pages, windows whose pages have been
   given back) must match the plain model AND leave the error word at 0: no kernel reads or
   writes through an index that is out of range, a released table entry (-1) included.
2. An index that IS out of range must be caught: the error word names the kind, and the access
   is not made. The "pool" that the kernels are told about is the first half of a larger
   tensor, so even an unchecked access would stay inside allocated memory; that the second
   half is untouched shows that the write was skipped.
"""

import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
for extra in (ROOT, ROOT / "tests"):
    sys.path.insert(0, str(extra))

import torch

torch.backends.cuda.matmul.allow_tf32 = False
torch.set_float32_matmul_precision("highest")

import helpers
from paged_attention_engine_b200.kernels import build, ops

WINDOWED_128 = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=256, num_attention_heads=2,
    num_key_value_heads=1, head_dim=128, intermediate_size=512, vocab_size=1000, rope_theta=1e6,
    rms_norm_eps=1e-6, max_position_embeddings=1024, tie_word_embeddings=True, use_sliding_window=True,
    sliding_window=96, max_window_layers=0,
)


def replays() -> None:
    cases = [(helpers.TINY_B, 16, 1, (33, 47, 64, 90, 17, 70)), (helpers.TINY_C, 8, 2, (33, 47, 64, 90, 17, 70)),
             (helpers.TINY_D, 16, 3, (150, 80, 200, 31)), (WINDOWED_128, 16, 4, (260, 150, 330, 97))]
    for raw, page, seed, lengths in cases:
        for dtype_name, dtype in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            with tempfile.TemporaryDirectory() as tmp:
                folder = helpers.write_model(Path(tmp) / "m", raw, seed, dtype, sharpen=3.0)
                requests = {f"r{i}": helpers.random_tokens(raw["vocab_size"], n, seed * 100 + i) for i, n in enumerate(lengths)}
                trace = helpers.trace_mixed(requests, seed=11 + seed, live_limit=3)
                # long prompts come in portions of up to 34 tokens; add one whole prompt so that the
                # kernels for long portions run too
                big = max(requests, key=lambda k: len(requests[k]))
                trace = helpers.trace_whole({big: requests[big]}, first_step=10_000) + trace
                budget = helpers.max_live_tokens(trace)
                outputs, replayer = helpers.run_in_process(folder, dtype_name, trace, budget, page)
                assert not replayer.runner.use_graphs
                ops.check_device_errors()
                got = helpers.collect(trace[1:], outputs, requests)
                for key, ids in requests.items():
                    want = helpers.plain_logits(folder, ids)
                    gap = (got[key] - want).abs().max().item()
                    assert gap <= helpers.tolerance(dtype, want), f"{raw['hidden_size']}/{dtype_name}/{key}: {gap}"
        print(f"replayed hidden {raw['hidden_size']} under the checked build: no index out of range", flush=True)


def caught(code: int) -> None:
    try:
        ops.check_device_errors()
    except ops.KernelError as exc:
        assert f"bounds code {code}" in str(exc), str(exc)
        return
    raise AssertionError(f"bounds code {code} was not raised")


def violations() -> None:
    heads, kv_heads, d, page = 4, 2, 64, 16
    for dtype in (torch.float32, torch.bfloat16):
        whole_k = torch.zeros(8, kv_heads, page, d, dtype=dtype, device="cuda")
        whole_v = torch.zeros_like(whole_k)
        keys, values = whole_k[:4], whole_v[:4]                      # the pool the kernels are told about: 4 pages
        qkv = torch.randn(3, (heads + 2 * kv_heads) * d, device="cuda").to(dtype)
        table = ops.rotary_table(torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda"),
                                 torch.ones(d // 2, device="cuda"))
        slots = torch.tensor([2 * page + 1, 6 * page + 3, 3 * page], dtype=torch.int32, device="cuda")   # the second lies in page 6
        ops.rotary_qk_cache_write(qkv.clone(), table, slots, keys, values, heads, kv_heads, d, page)
        torch.cuda.synchronize()
        caught(101)
        assert whole_k[4:].abs().sum().item() == 0 and whole_v[4:].abs().sum().item() == 0, "the write beyond the pool was made"
        assert whole_k[2, :, 1].abs().sum().item() > 0 and whole_k[3, :, 0].abs().sum().item() > 0, "the other tokens' writes were lost"
        # attention through a table that names page 6 of a pool of 4, and, separately, a context
        # longer than the table is wide
        whole_k.normal_()
        whole_v.normal_()
        block_table = torch.tensor([[1, 6], [0, 2]], dtype=torch.int32, device="cuda")
        q_start = torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda")
        kv_len = torch.tensor([20, 30], dtype=torch.int32, device="cuda")
        args = (qkv[:2].contiguous(), keys, values, block_table, q_start, kv_len - 1, kv_len, heads, kv_heads, d, page, 1, 30, 0.125, 0)
        ops.paged_attention(*args)
        torch.cuda.synchronize()
        caught(103)
        # the table is the head of a longer buffer of valid page ids: were the index not checked,
        # the read past the table's width would still find a page that exists
        good = torch.tensor([1, 3, 0, 2, 0, 0, 0, 0], dtype=torch.int32, device="cuda")[:4].view(2, 2)
        long_kv = torch.tensor([20, 40], dtype=torch.int32, device="cuda")     # 40 keys need 3 table entries, the table has 2
        ops.paged_attention(qkv[:2].contiguous(), keys, values, good, q_start, long_kv - 1, long_kv, heads, kv_heads, d, page, 1, 40, 0.125, 0)
        torch.cuda.synchronize()
        caught(102)
        ops.paged_attention(qkv[:2].contiguous(), keys, values, good, q_start, kv_len - 1, kv_len, heads, kv_heads, d, page, 1, 30, 0.125, 0)
        ops.check_device_errors()          # and a call that is in range leaves the word at 0
    print("indices out of range were caught and skipped", flush=True)


if __name__ == "__main__":
    assert build.BOUNDS and ops.bounds_checked, "run with PAE_BOUNDS=1"
    violations()
    replays()
    print("BOUNDS PROBE OK")
