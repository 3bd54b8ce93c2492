"""Makes the golden logits under tests/golden/ from the reference project's own model code.

    python tests/golden/make_golden.py --reference <checkout of paged-attention-engine>

The reference's engine/model.py imports and runs on the CPU without network once
its weights are handed over as tensors (ModelDims / LayerWeights / Qwen2Weights /
Qwen2Engine, engine/model.py:43-106,164-186), so the plain implementation under
tests/plain/ is compared with it once, on two tiny random models, and the outputs
are committed beside this script:

    tiny_a.safetensors, tiny_b.safetensors
        ids_<r>      the whole token sequence of request r (prompt + greedy tokens)
        rows_<r>     the positions whose logits are kept
        logits_<r>   [len(rows), vocab] float32: the reference's logits for the
                     prefix ending at each kept position (engine/model.py:362-384)
        greedy_<r>   the tokens the reference's generate_greedy produced
                     (engine/model.py:459-503)
        checksum     sum of |w| over all weights, to notice a change of the
                     random generator between torch versions

The weights are not stored: `make_weights` rebuilds them from the seed, and the
test that reads the golden files calls the same function.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent

# The two tiny configurations: they differ in every size and option.
TINY_A = dict(
    name="tiny_a", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, intermediate_size=176, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
    max_position_embeddings=128, tie_word_embeddings=True, seed=0, prompts=(5, 11, 17), new_tokens=8,
)
TINY_B = dict(
    name="tiny_b", num_hidden_layers=3, hidden_size=96, num_attention_heads=3, num_key_value_heads=1,
    head_dim=32, intermediate_size=256, vocab_size=509, rope_theta=1e6, rms_norm_eps=1e-5,
    max_position_embeddings=256, tie_word_embeddings=False, seed=1, prompts=(1, 7, 23, 40, 64), new_tokens=12,
)


def tensor_shapes(cfg: dict) -> list[tuple[str, tuple[int, ...], str]]:
    """(name, shape, kind) of every tensor of the checkpoint, in a fixed order."""
    h, d = cfg["hidden_size"], cfg["head_dim"]
    nh, nkv, inter, vocab = (
        cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"],
    )
    out = [("model.embed_tokens.weight", (vocab, h), "weight")]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out += [
            (p + "input_layernorm.weight", (h,), "norm"),
            (p + "self_attn.q_proj.weight", (nh * d, h), "weight"),
            (p + "self_attn.q_proj.bias", (nh * d,), "bias"),
            (p + "self_attn.k_proj.weight", (nkv * d, h), "weight"),
            (p + "self_attn.k_proj.bias", (nkv * d,), "bias"),
            (p + "self_attn.v_proj.weight", (nkv * d, h), "weight"),
            (p + "self_attn.v_proj.bias", (nkv * d,), "bias"),
            (p + "self_attn.o_proj.weight", (h, nh * d), "weight"),
            (p + "post_attention_layernorm.weight", (h,), "norm"),
            (p + "mlp.gate_proj.weight", (inter, h), "weight"),
            (p + "mlp.up_proj.weight", (inter, h), "weight"),
            (p + "mlp.down_proj.weight", (h, inter), "weight"),
        ]
    out.append(("model.norm.weight", (h,), "norm"))
    if not cfg["tie_word_embeddings"]:
        out.append(("lm_head.weight", (vocab, h), "weight"))
    return out


def make_weights(cfg: dict) -> dict[str, torch.Tensor]:
    """Weights N(0, 0.02), norm weights 1 + N(0, 0.02), biases N(0, 0.02), float32."""
    gen = torch.Generator(device="cpu").manual_seed(int(cfg["seed"]))
    out = {}
    for name, shape, kind in tensor_shapes(cfg):
        t = torch.randn(shape, generator=gen, dtype=torch.float32) * 0.02
        out[name] = t + 1.0 if kind == "norm" else t
    return out


def make_prompts(cfg: dict) -> list[list[int]]:
    gen = torch.Generator(device="cpu").manual_seed(1000 + int(cfg["seed"]))
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in cfg["prompts"]]


def checksum(weights: dict[str, torch.Tensor]) -> torch.Tensor:
    return torch.tensor([float(sum(w.double().abs().sum() for w in weights.values()))], dtype=torch.float64)


def kept_rows(total: int) -> list[int]:
    """Every position of a short sequence; the first 20 and the last 20 of a long one."""
    if total <= 40:
        return list(range(total))
    return list(range(20)) + list(range(total - 20, total))


def build_reference_engine(cfg: dict, weights: dict[str, torch.Tensor]):
    from engine.model import LayerWeights, ModelDims, Qwen2Engine, Qwen2Weights

    dims = ModelDims(
        num_layers=cfg["num_hidden_layers"], num_heads=cfg["num_attention_heads"],
        num_kv_heads=cfg["num_key_value_heads"], head_dim=cfg["head_dim"], hidden_size=cfg["hidden_size"],
        rms_norm_eps=cfg["rms_norm_eps"], vocab_size=cfg["vocab_size"], rope_theta=cfg["rope_theta"],
    )
    layers = []
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        layers.append(LayerWeights(
            q_proj_weight=weights[p + "self_attn.q_proj.weight"], q_proj_bias=weights[p + "self_attn.q_proj.bias"],
            k_proj_weight=weights[p + "self_attn.k_proj.weight"], k_proj_bias=weights[p + "self_attn.k_proj.bias"],
            v_proj_weight=weights[p + "self_attn.v_proj.weight"], v_proj_bias=weights[p + "self_attn.v_proj.bias"],
            o_proj_weight=weights[p + "self_attn.o_proj.weight"],
            gate_proj_weight=weights[p + "mlp.gate_proj.weight"], up_proj_weight=weights[p + "mlp.up_proj.weight"],
            down_proj_weight=weights[p + "mlp.down_proj.weight"],
            input_layernorm_weight=weights[p + "input_layernorm.weight"],
            post_attention_layernorm_weight=weights[p + "post_attention_layernorm.weight"],
        ))
    embed = weights["model.embed_tokens.weight"]
    head = weights.get("lm_head.weight", embed)
    return Qwen2Engine(
        Qwen2Weights(embed, tuple(layers), weights["model.norm.weight"], head),
        dims, torch.device("cpu"), torch.float32,
    )


def main() -> int:
    from safetensors.torch import save_file

    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of the reference project")
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_num_threads(1)

    for cfg in (TINY_A, TINY_B):
        weights = make_weights(cfg)
        engine = build_reference_engine(cfg, weights)
        out = {"checksum": checksum(weights)}
        for r, prompt in enumerate(make_prompts(cfg)):
            result = engine.generate_greedy(prompt, cfg["new_tokens"])
            ids = prompt + list(result.token_ids)
            rows = kept_rows(len(ids))
            logits = []
            for p in rows:
                prefix = torch.tensor(ids[: p + 1], dtype=torch.long)
                backend = engine.new_contiguous_backend(p + 1)
                logits.append(engine.forward(prefix, torch.arange(p + 1), backend).to(torch.float32))
            out[f"ids_{r}"] = torch.tensor(ids, dtype=torch.int64)
            out[f"rows_{r}"] = torch.tensor(rows, dtype=torch.int64)
            out[f"logits_{r}"] = torch.stack(logits).contiguous()
            out[f"greedy_{r}"] = torch.tensor(result.token_ids, dtype=torch.int64)
        save_file(out, str(HERE / f"{cfg['name']}.safetensors"))
        print(cfg["name"], {k: tuple(v.shape) for k, v in out.items()})
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
